// Linear recurrences with one matrix state S [dk, dv] per head and request, and what surrounds them.
//
//     S <- diag(w_t) S                       (w_t: a decay per key channel, or one number per head)
//     u  = beta_t (v_t - S^T k_t)            (`delta`: the delta rule's correction; else u = v_t)
//     S <- S + k_t u^T
//     o_t = S^T q_t                          (the read-out sees the token's own write)
//
// `matrix_state_scan` walks each request's tokens in order.  Columns of S do not talk to one another:
// a CTA holds a block of columns of one (request, head), a column's rows spread over LANES lanes of a
// warp (ROWS rows each, in registers), dot products over the rows finished by shuffles.  The inputs of
// every token (q, k, v, w, beta) are 32-bit rows of an `aux` buffer that a prep kernel writes:
//   * `conv_delta_prep`: q, k, v through a short causal convolution over time and silu, q and k scaled
//     to unit length per head, beta = sigmoid(.), w = exp(-exp(A) softplus(. + dt)) per head; the last
//     taps - 1 inputs of the convolutions are part of the request's state (`conv_state_update`);
//   * `decay_gate_prep`: q scaled, k, v, and w = sigmoid(z)^(1 / tau) per key channel with z a
//     low-rank product plus bias.
// `head_norm_gate` norms each head's read-out over dv, applies the weight and silu(gate).
// `head_talk_mix` and `pair_norm_mean` belong to attention whose heads exchange their weights and to
// two mixers side by side.
// The state lives in 32-bit in the request's slot, in the order the scan's threads hold it:
// [head][row / LANES][column][row % LANES]; a request whose first token is in the step starts from zero.
#include <type_traits>

#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ------------------------------------------------------ convolution + delta-rule inputs
// proj row: [q (G d) | k (G d) | v (H dv) | gate (H dv) | b (H) | a (H)].  aux row: [q (G d) | k (G d) |
// v (H dv) | w (H) | beta (H)].  conv_w [2 G d + H dv][taps] float.  conv_state: inside the slot's state
// at `conv_off`, [taps - 1][C].  Grid (tokens, blocks of heads); a warp per head of q, k or v (2 G + H of
// them): a q or k head is written as the convolution left it, then scaled by the same lanes once its
// sum of squares is known.
template <typename T>
__global__ void __launch_bounds__(256)
conv_delta_prep_kernel(GemmOut<T> proj, int cols, const int* __restrict__ tok_entry,
                       const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                       const int* __restrict__ slots, int n_slots, const float* __restrict__ state,
                       long long slot_stride, long long conv_off, const float* __restrict__ conv_w, int taps,
                       const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                       float* __restrict__ aux, int aux_cols, int H, int G, int d, int dv, float key_eps,
                       float q_scale, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int e = tok_entry[t];
    if (e < 0) return;
    const int C = 2 * G * d + H * dv;
    const int first = cu_q[e];
    const int i = t - first;                                         // the token's place in its portion
    const int start = kv_len[e] - (cu_q[e + 1] - first);             // tokens of the request before the step
    const int slot = slots[e];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, CRANE_ERR_SLOT_RANGE);
        return;
    }
    const float* cs = state + (long long)slot * slot_stride + conv_off;
    float* out = aux + (long long)t * aux_cols;
    const int lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int unit = blockIdx.y * nw + (threadIdx.x >> 5); unit < 2 * G + H; unit += gridDim.y * nw) {
        const bool qk = unit < 2 * G;
        const int width = qk ? d : dv;
        const int c_first = qk ? unit * d : 2 * G * d + (unit - 2 * G) * dv;
        float ss = 0.f;
        for (int cc = lane; cc < width; cc += 32) {
            const int c = c_first + cc;
            float acc = 0.f;
            for (int j = 0; j < taps; ++j) {
                const int back = taps - 1 - j;
                float x = 0.f;
                if (i - back >= 0) x = proj.load((long long)(t - back) * cols + c);
                else if (start + i - back >= 0) x = cs[(long long)(taps - 1 + i - back) * C + c];
                acc = fmaf(conv_w[(long long)c * taps + j], x, acc);
            }
            const float v = silu_f(acc);
            out[c] = v;
            ss = fmaf(v, v, ss);
        }
        if (qk) {
            ss = warp_sum(ss);
            const float r = rsqrtf(ss + key_eps) * (unit < G ? q_scale : 1.f);
            for (int cc = lane; cc < width; cc += 32) out[c_first + cc] *= r;      // each lane its own elements
        }
    }
    if (blockIdx.y == 0) {
        for (int h = threadIdx.x; h < H; h += blockDim.x) {
            const long long row = (long long)t * cols + C + H * dv;
            const float b = proj.load(row + h), a = proj.load(row + H + h);
            out[C + h] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
            out[C + H + h] = 1.f / (1.f + expf(-b));
        }
    }
}

// One thread per (entry, channel): the last taps - 1 inputs of the channel after this step.
constexpr int MAX_TAPS = 16;
template <typename T>
__global__ void __launch_bounds__(128)
conv_state_update_kernel(GemmOut<T> proj, int cols, const int* __restrict__ cu_q,
                         const int* __restrict__ kv_len, const int* __restrict__ slots, int n_slots,
                         float* __restrict__ state, long long slot_stride, long long conv_off, int taps, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int first = cu_q[e], q_len = cu_q[e + 1] - first;
    if (q_len <= 0 || c >= C) return;
    const int slot = slots[e];
    if (slot < 0 || slot >= n_slots) return;
    const int end = kv_len[e], start = end - q_len;
    float* cs = state + (long long)slot * slot_stride + conv_off;
    float old[MAX_TAPS];
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) old[j] = (j < taps - 1) ? cs[(long long)j * C + c] : 0.f;
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) {
        if (j < taps - 1) {
            const int p = end - (taps - 1) + j;
            float v = 0.f;
            if (p >= start) v = proj.load((long long)(first + p - start) * cols + c);
            else if (p >= 0) {
                const int k = taps - 1 + p - start;
                float o = 0.f;
#pragma unroll
                for (int m = 0; m < MAX_TAPS; ++m) if (m == k) o = old[m];
                v = o;
            }
            cs[(long long)j * C + c] = v;
        }
    }
}

// ------------------------------------------------------ inputs of the recurrence with a decay per channel
// proj row: [q (H d) | k (H d) | v (H dv) | gate (H dv) | low (rank)].  aux row: [q (H d) | k (H d) |
// v (H dv) | w (H d)].  a2t [rank][H d] float, bias [H d].
template <typename T>
__global__ void __launch_bounds__(256)
decay_gate_prep_kernel(GemmOut<T> proj, int cols, const int* __restrict__ tok_entry,
                       const float* __restrict__ a2t, const float* __restrict__ bias, int rank,
                       float inv_tau, float q_scale, float* __restrict__ aux, int aux_cols, int H, int d, int dv) {
    extern __shared__ float low[];                    // [rank]
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (tok_entry[t] < 0) return;
    const int hd = H * d, hv = H * dv;
    const long long row = (long long)t * cols;
    for (int r = threadIdx.x; r < rank; r += blockDim.x) low[r] = proj.load(row + 2 * hd + 2 * hv + r);
    __syncthreads();
    float* out = aux + (long long)t * aux_cols;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < hd; c += gridDim.y * blockDim.x) {
        out[c] = proj.load(row + c) * q_scale;
        out[hd + c] = proj.load(row + hd + c);
        float z = bias[c];
#pragma unroll 8
        for (int r = 0; r < rank; ++r) z = fmaf(low[r], a2t[(long long)r * hd + c], z);
        // sigmoid(z)^(1 / tau) = exp(-softplus(-z) / tau)
        out[2 * hd + hv + c] = expf(-softplus_f(-z) * inv_tau);
    }
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < hv; c += gridDim.y * blockDim.x)
        out[2 * hd + c] = proj.load(row + 2 * hd + c);
}

// ------------------------------------------------------ the recurrence
// grid (entries, heads, column blocks); block = COLS columns x LANES lanes.  aux offsets: q_off, k_off,
// v_off, w_off, beta_off (beta only with `delta`); q/k head of head h is h / qk_rep; w is [Hqk d]
// (w_vec) or [H].  o_raw float [n][H dv].
// Tokens come in tiles of `tile_tokens` whose vectors all threads copy into shared memory with 4-byte
// asynchronous copies, the next tile while the current one is walked: a tile's fetch from DRAM is as
// long as walking several tokens, and the walk must not wait for it.
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}
constexpr int SCAN_TOKENS = 16;
// The sum over the LANES (a power of two, aligned in the warp) that share a column; LANES 0: `lanes` at run
// time.
template <int LANES>
__device__ __forceinline__ float lanes_sum(float x, int lanes) {
    if (LANES > 0) {
#pragma unroll
        for (int o = LANES >> 1; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
        return x;
    }
    if (lanes > 16) x += __shfl_xor_sync(0xffffffffu, x, 16);
    if (lanes > 8) x += __shfl_xor_sync(0xffffffffu, x, 8);
    if (lanes > 4) x += __shfl_xor_sync(0xffffffffu, x, 4);
    if (lanes > 2) x += __shfl_xor_sync(0xffffffffu, x, 2);
    if (lanes > 1) x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x;
}
// A lane holds ROWS neighbouring rows of its column.  FULL: the lanes' rows are exactly the dk rows; no row
// is tested and a lane reads its part of a vector 16 bytes at a time.  WVEC: a decay per row (else one per
// head).  DELTA: the delta rule's correction.  LANES: the lanes of a column when the kernel is compiled for
// them (0: any).  The first `walkers` threads walk the tokens; one more warp does nothing but copy the next
// tile of tokens into shared memory meanwhile, since a walking warp's time is its instructions per token.
template <int ROWS, bool FULL, bool DELTA, bool WVEC, int LANES>
__global__ void __launch_bounds__(288)
matrix_state_scan_kernel(const float* __restrict__ aux, int aux_cols, int q_off, int k_off, int v_off, int w_off,
                         int beta_off, int qk_rep, const int* __restrict__ cu_q,
                         const int* __restrict__ kv_len, const int* __restrict__ slots, int n_slots,
                         float* __restrict__ state, long long slot_stride, float* __restrict__ o_raw,
                         int H, int dk, int dv, int lanes_rt, int cols_per_block, int tile_tokens, int vec4,
                         int walkers, int* err) {
    extern __shared__ __align__(16) float tile[];     // two tiles of [tile_tokens][3 dk + cols + 2, to a multiple of 4]
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x, h = blockIdx.y;
    const int first = cu_q[e], q_len = cu_q[e + 1] - first;
    if (q_len <= 0) return;
    const int slot = slots[e];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_SLOT_RANGE);
        return;
    }
    const int lanes = LANES > 0 ? LANES : lanes_rt;
    const int start = kv_len[e] - q_len;
    const int hq = h / qk_rep;
    const int stride = (3 * dk + cols_per_block + 2 + 3) & ~3;       // rows start on 16 bytes
    const int c0 = blockIdx.z * cols_per_block;
    const int tile_floats = tile_tokens * stride;
    const int n_tiles = (q_len + tile_tokens - 1) / tile_tokens;
    const bool producer = (int)threadIdx.x >= walkers;

    // ---- the copying warp: a token's vectors are runs of its row; units of 16 bytes (`vec4`: every run starts
    // on 16 bytes and is a multiple of them) or of 4
    const int wl = threadIdx.x & 31;
    const int unit = vec4 ? 4 : 1;
    const int nq = dk / unit, nvu = min(cols_per_block, dv - c0) / unit;
    const int n_units = (WVEC ? 3 : 2) * nq + nvu;
    auto place = [&](int x, int& so, int& dofs) {                    // unit x of a token: where from, where to
        if (x < nq) so = q_off + hq * dk + x * unit, dofs = x * unit;
        else if (x < 2 * nq) so = k_off + hq * dk + (x - nq) * unit, dofs = dk + (x - nq) * unit;
        else if (WVEC && x < 3 * nq) so = w_off + hq * dk + (x - 2 * nq) * unit, dofs = 2 * dk + (x - 2 * nq) * unit;
        else {
            const int y = x - (WVEC ? 3 : 2) * nq;
            so = v_off + h * dv + c0 + y * unit, dofs = 3 * dk + y * unit;
        }
    };
    auto copy = [&](float* dst, const float* src) {
        if (vec4) cp_async16(dst, src);
        else cp_async4(dst, src);
    };
    int so0 = -1, do0 = 0, so1 = -1, do1 = 0;                         // the lane's first two units, the same for every token
    if (producer) {
        if (wl < n_units) place(wl, so0, do0);
        if (wl + 32 < n_units) place(wl + 32, so1, do1);
    }
    auto fetch = [&](int t0, float* buf) {
        const int nt = min(tile_tokens, q_len - t0);
        const float* a = aux + (long long)(first + t0) * aux_cols;
        float* b = buf;
        for (int tt = 0; tt < nt; ++tt, a += aux_cols, b += stride) {
            if (so0 >= 0) copy(b + do0, a + so0);
            if (so1 >= 0) copy(b + do1, a + so1);
            for (int x = wl + 64; x < n_units; x += 32) {
                int so, dofs;
                place(x, so, dofs);
                copy(b + dofs, a + so);
            }
            if (wl == 0) {
                if (WVEC) b[3 * dk + cols_per_block] = 1.f;
                else cp_async4(b + 3 * dk + cols_per_block, a + w_off + h);
            } else if (wl == 1) {
                if (DELTA) cp_async4(b + 3 * dk + cols_per_block + 1, a + beta_off + h);
                else b[3 * dk + cols_per_block + 1] = 1.f;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    };
    if (producer) fetch(0, tile);

    // ---- the walkers
    const int lane = threadIdx.x % lanes, cl = threadIdx.x / lanes;
    const int r0 = lane * ROWS;                       // the lane's rows: r0 .. r0 + ROWS - 1
    const int col = c0 + cl;
    const bool live = !producer && cl < cols_per_block && col < dv;
    const int vcol = live ? cl : 0;
    // state [H][ROWS][dv][lanes]
    float* sp = state + (long long)slot * slot_stride + (long long)h * ROWS * dv * lanes;
    float s[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
        s[i] = (live && start > 0 && (FULL || r0 + i < dk)) ? sp[((long long)i * dv + col) * lanes + lane] : 0.f;
    __syncthreads();                                  // the first tile is there
    const long long o_step = (long long)H * dv;
    for (int it = 0; it < n_tiles; ++it) {
        const int t0 = it * tile_tokens;
        const int nt = min(tile_tokens, q_len - t0);
        if (producer) {
            if (it + 1 < n_tiles) fetch(t0 + tile_tokens, tile + ((it + 1) & 1) * tile_floats);
        } else {
            const float* tp = tile + (it & 1) * tile_floats;
            float* op = o_raw + (long long)(first + t0) * o_step + h * dv + (live ? col : 0);
#pragma unroll(ROWS == 8 ? 2 : 1)
            for (int tt = 0; tt < nt; ++tt, tp += stride, op += o_step) {
                float qv[ROWS], kv[ROWS], wv[ROWS];
                if (FULL) {                            // lane's rows are one aligned run of each vector
#pragma unroll
                    for (int i = 0; i < ROWS; i += 4) {
                        const float4 a4 = *reinterpret_cast<const float4*>(tp + r0 + i);
                        const float4 b4 = *reinterpret_cast<const float4*>(tp + dk + r0 + i);
                        qv[i] = a4.x, qv[i + 1] = a4.y, qv[i + 2] = a4.z, qv[i + 3] = a4.w;
                        kv[i] = b4.x, kv[i + 1] = b4.y, kv[i + 2] = b4.z, kv[i + 3] = b4.w;
                        if (WVEC) {
                            const float4 c4 = *reinterpret_cast<const float4*>(tp + 2 * dk + r0 + i);
                            wv[i] = c4.x, wv[i + 1] = c4.y, wv[i + 2] = c4.z, wv[i + 3] = c4.w;
                        }
                    }
                } else {                               // rows past dk: zeros, and their state stays zero
#pragma unroll
                    for (int i = 0; i < ROWS; ++i) {
                        const bool in = r0 + i < dk;
                        qv[i] = in ? tp[r0 + i] : 0.f;
                        kv[i] = in ? tp[dk + r0 + i] : 0.f;
                        if (WVEC) wv[i] = in ? tp[2 * dk + r0 + i] : 0.f;
                    }
                }
                const float vv = tp[3 * dk + vcol];    // a column that is not live reads a neighbour's and writes nothing
                const float ws = WVEC ? 1.f : tp[3 * dk + cols_per_block];
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < ROWS; ++i) {
                    s[i] *= WVEC ? wv[i] : ws;
                    if (DELTA) dot = fmaf(s[i], kv[i], dot);
                }
                float u = vv;
                if (DELTA) {
                    dot = lanes_sum<LANES>(dot, lanes);
                    u = tp[3 * dk + cols_per_block + 1] * (vv - dot);
                }
                float rd = 0.f;
#pragma unroll
                for (int i = 0; i < ROWS; ++i) {
                    s[i] = fmaf(kv[i], u, s[i]);
                    rd = fmaf(s[i], qv[i], rd);
                }
                rd = lanes_sum<LANES>(rd, lanes);
                if (live && lane == 0) *op = rd;
            }
        }
        __syncthreads();              // the next tile is there for all; all have left this one
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) sp[((long long)i * dv + col) * lanes + lane] = s[i];
    }
}

// ------------------------------------------------------ head norm and gate
// out[t][h dv + c] = o_raw / rms_over_dv(o_raw) * norm_w[c] * silu(gate[t][gate_off + h dv + c]); a warp per
// (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o_raw, GemmOut<T> proj, int cols, int gate_off,
                      const int* __restrict__ tok_entry, const float* __restrict__ norm_w, float eps,
                      T* __restrict__ out, int n, int H, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)n * H) return;
    const int t = (int)(wid / H), h = (int)(wid % H);
    if (tok_entry[t] < 0) return;
    const float* o = o_raw + ((long long)t * H + h) * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) { const float v = o[c]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        const float g = proj.load((long long)t * cols + gate_off + h * dv + c);
        out[((long long)t * H + h) * dv + c] = from_f32<T>(o[c] * rstd * norm_w[c] * silu_f(g));
    }
}

// ------------------------------------------------------ heads that exchange their weights
// cross [n][H][G][dv] float: query head g's softmax weights applied to the values of every key/value
// head.  out[t][h] = sum_g talk[h][g] cross[t][g][h / (H / G)].  Grid (tokens, heads).
template <typename T>
__global__ void __launch_bounds__(128)
head_talk_mix_kernel(const float* __restrict__ cross, const float* __restrict__ talk,
                     const int* __restrict__ tok_entry, T* __restrict__ out, int H, int G, int dv, int out_head) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    if (tok_entry[t] < 0) return;
    const int rep = H / G;
    for (int c = threadIdx.x; c < out_head; c += blockDim.x) {               // out_head <= dv columns are kept
        const float* src = cross + ((long long)t * H * G + h / rep) * dv + c;
        float acc = 0.f;
        for (int g = 0; g < H; ++g) acc = fmaf(talk[h * H + g], src[(long long)g * G * dv], acc);
        out[((long long)t * H + h) * out_head + c] = from_f32<T>(acc);
    }
}

// ------------------------------------------------------ two mixers side by side
// out = (a / rms(a) * wa + b / rms(b) * wb) / 2 over the width; a CTA per row.
template <typename T>
__global__ void __launch_bounds__(256)
pair_norm_mean_kernel(GemmOut<T> a, GemmOut<T> b, const float* __restrict__ wa, const float* __restrict__ wb,
                      float eps, T* __restrict__ out, int hidden) {
    extern __shared__ float row2[];                   // [2 hidden]
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const long long base = (long long)blockIdx.x * hidden;
    float sa = 0.f, sb = 0.f;
    const bool pairs = (hidden & 1) == 0;             // rows of even length: two neighbours a load and a store
    if (pairs) {
        for (int c = 2 * threadIdx.x; c < hidden; c += 2 * blockDim.x) {
            const float2 x = a.load2(base + c), y = b.load2(base + c);
            row2[c] = x.x, row2[c + 1] = x.y;
            row2[hidden + c] = y.x, row2[hidden + c + 1] = y.y;
            sa = fmaf(x.x, x.x, fmaf(x.y, x.y, sa));
            sb = fmaf(y.x, y.x, fmaf(y.y, y.y, sb));
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float x = a.load(base + c), y = b.load(base + c);
            row2[c] = x;
            row2[hidden + c] = y;
            sa = fmaf(x, x, sa);
            sb = fmaf(y, y, sb);
        }
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ra = rsqrtf(sa / (float)hidden + eps), rb = rsqrtf(sb / (float)hidden + eps);
    if (pairs) {
        for (int c = 2 * threadIdx.x; c < hidden; c += 2 * blockDim.x)
            st2(out + base + c, 0.5f * (row2[c] * ra * wa[c] + row2[hidden + c] * rb * wb[c]),
                0.5f * (row2[c + 1] * ra * wa[c + 1] + row2[hidden + c + 1] * rb * wb[c + 1]));
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x)
            out[base + c] = from_f32<T>(0.5f * (row2[c] * ra * wa[c] + row2[hidden + c] * rb * wb[c]));
    }
}

}  // namespace

CRANE_API int crane_conv_delta_prep(int dtype, const void* proj, const float* proj_parts, int n_parts,
                                    long long part_stride, int cols, const int* tok_entry, const int* cu_q,
                                    const int* kv_len, const int* slots, int n_slots, float* state,
                                    long long slot_stride, long long conv_off, const float* conv_w, int taps,
                                    const float* a_log, const float* dt_bias, float* aux, int aux_cols,
                                    int n_tokens, int n_entries, int H, int G, int d, int dv, float key_eps,
                                    float q_scale, int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    const int C = 2 * G * d + H * dv;
    if (taps < 1 || taps > MAX_TAPS) return (int)cudaErrorInvalidValue;
    // a warp per head; with few tokens the heads spread over more CTAs
    const int units = 2 * G + H;
    int by = (units + 7) / 8;
    while (by > 1 && (long long)n_tokens * by > 4 * 148) by = (by + 1) / 2;
    DISPATCH_T(dtype, {
        GemmOut<T> p{(const T*)proj, proj_parts, n_parts, part_stride};
        int rc = crane_launch(conv_delta_prep_kernel<T>, dim3(n_tokens, by), dim3(256), 0, st, p, cols, tok_entry,
                              cu_q, kv_len, slots, n_slots, (const float*)state, slot_stride, conv_off, conv_w,
                              taps, a_log, dt_bias, aux, aux_cols, H, G, d, dv, key_eps, q_scale, err);
        if (rc != 0 || taps == 1) return rc;
        return crane_launch(conv_state_update_kernel<T>, dim3((C + 127) / 128, n_entries), dim3(128), 0, st, p,
                            cols, cu_q, kv_len, slots, n_slots, state, slot_stride, conv_off, taps, C);
    });
}

CRANE_API int crane_decay_gate_prep(int dtype, const void* proj, const float* proj_parts, int n_parts,
                                    long long part_stride, int cols, const int* tok_entry, const float* a2t,
                                    const float* bias, int rank, float inv_tau, float q_scale, float* aux,
                                    int aux_cols, int n_tokens, int H, int d, int dv, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (rank < 0 || rank > 8192) return (int)cudaErrorInvalidValue;
    DISPATCH_T(dtype, {
        GemmOut<T> p{(const T*)proj, proj_parts, n_parts, part_stride};
        int by = (H * (d > dv ? d : dv) + 255) / 256;            // with few tokens the channels spread over more CTAs
        while (by > 1 && (long long)n_tokens * by > 4 * 148) by = (by + 1) / 2;
        return crane_launch(decay_gate_prep_kernel<T>, dim3(n_tokens, by), dim3(256), (size_t)(rank > 0 ? rank : 1) * 4,
                            st, p, cols, tok_entry, a2t, bias, rank, inv_tau, q_scale, aux, aux_cols, H, d, dv);
    });
}

// The scan's geometry for a key size: (rows per lane, lanes per column); 0 rows: too wide.
CRANE_API int crane_matrix_state_plan(int dk, int* rows, int* lanes) {
    int r = dk <= 256 ? 8 : 16, l = 1;
    while (l * r < dk && l < 32) l *= 2;
    if (l * r < dk) { *rows = 0; *lanes = 0; return 1; }
    *rows = r;
    *lanes = l;
    return 0;
}

CRANE_API int crane_matrix_state_scan(const float* aux, int aux_cols, int q_off, int k_off, int v_off, int w_off,
                                      int beta_off, int w_vec, int delta, int qk_rep, const int* cu_q,
                                      const int* kv_len, const int* slots, int n_slots, float* state,
                                      long long slot_stride, float* o_raw, int n_entries, int H, int dk, int dv,
                                      int* err, cudaStream_t st) {
    if (n_entries <= 0) return 0;
    int rows, lanes;
    if (crane_matrix_state_plan(dk, &rows, &lanes) || dv <= 0 || qk_rep <= 0) return (int)cudaErrorInvalidValue;
    int cpb = 256 / lanes;
    if (cpb > dv) cpb = dv;
    // few entries and heads: narrower blocks of columns, so that more SMs walk (a column's result does not
    // depend on the block it is in)
    while ((long long)n_entries * H * ((dv + cpb - 1) / cpb) < 148 && cpb > 8) cpb /= 2;
    const int blocks = (dv + cpb - 1) / cpb;
    const int walkers = ((cpb * lanes + 31) / 32) * 32;        // and a warp that copies
    const size_t per_token = (size_t)((3 * dk + cpb + 2 + 3) & ~3) * sizeof(float);
    const int vec4 = (dk % 4 == 0 && dv % 4 == 0 && cpb % 4 == 0 && aux_cols % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 &&
                      v_off % 4 == 0 && (!w_vec || w_off % 4 == 0) && (uintptr_t)aux % 16 == 0) ? 1 : 0;
    int tile_tokens = (int)((48 * 1024) / (2 * per_token));
    if (tile_tokens > SCAN_TOKENS) tile_tokens = SCAN_TOKENS;
    if (tile_tokens < 1) return (int)cudaErrorInvalidValue;
    const size_t smem = 2 * (size_t)tile_tokens * per_token;
    const bool full = rows * lanes == dk;
    using Kern = decltype(&matrix_state_scan_kernel<8, true, true, true, 0>);
    auto pick = [&](auto rows_c, auto lanes_c) -> Kern {
        constexpr int R = decltype(rows_c)::value, L = decltype(lanes_c)::value;
        if (full) return delta ? (w_vec ? matrix_state_scan_kernel<R, true, true, true, L> : matrix_state_scan_kernel<R, true, true, false, L>)
                               : (w_vec ? matrix_state_scan_kernel<R, true, false, true, L> : matrix_state_scan_kernel<R, true, false, false, L>);
        return delta ? (w_vec ? matrix_state_scan_kernel<R, false, true, true, 0> : matrix_state_scan_kernel<R, false, true, false, 0>)
                     : (w_vec ? matrix_state_scan_kernel<R, false, false, true, 0> : matrix_state_scan_kernel<R, false, false, false, 0>);
    };
    using std::integral_constant;
    Kern kern;
    if (rows != 8) kern = pick(integral_constant<int, 16>{}, integral_constant<int, 0>{});
    else if (full && lanes == 4) kern = pick(integral_constant<int, 8>{}, integral_constant<int, 4>{});      // heads of 32,
    else if (full && lanes == 8) kern = pick(integral_constant<int, 8>{}, integral_constant<int, 8>{});      // 64
    else if (full && lanes == 16) kern = pick(integral_constant<int, 8>{}, integral_constant<int, 16>{});    // and 128
    else kern = pick(integral_constant<int, 8>{}, integral_constant<int, 0>{});
    return crane_launch(kern, dim3(n_entries, H, blocks), dim3(walkers + 32), smem, st, aux, aux_cols, q_off, k_off,
                        v_off, w_off, beta_off, qk_rep, cu_q, kv_len, slots, n_slots, state, slot_stride,
                        o_raw, H, dk, dv, lanes, cpb, tile_tokens, vec4, walkers, err);
}

CRANE_API int crane_head_norm_gate(int dtype, const float* o_raw, const void* proj, const float* proj_parts,
                                   int n_parts, long long part_stride, int cols, int gate_off,
                                   const int* tok_entry, const float* norm_w, float eps, void* out, int n_tokens,
                                   int H, int dv, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    const long long warps = (long long)n_tokens * H;
    DISPATCH_T(dtype, {
        GemmOut<T> p{(const T*)proj, proj_parts, n_parts, part_stride};
        return crane_launch(head_norm_gate_kernel<T>, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, st, o_raw, p,
                            cols, gate_off, tok_entry, norm_w, eps, (T*)out, n_tokens, H, dv);
    });
}

CRANE_API int crane_head_talk_mix(int dtype, const float* cross, const float* talk, const int* tok_entry, void* out,
                                  int n_tokens, int H, int G, int dv, int out_head, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (G <= 0 || H % G || out_head > dv) return (int)cudaErrorInvalidValue;
    DISPATCH_T(dtype, return crane_launch(head_talk_mix_kernel<T>, dim3(n_tokens, H), dim3(out_head > 64 ? 128 : 64), 0, st, cross, talk,
                                          tok_entry, (T*)out, H, G, dv, out_head));
}

CRANE_API int crane_pair_norm_mean(int dtype, const void* a, const float* a_parts, int an, long long astr,
                                   const void* b, const float* b_parts, int bn, long long bstr, const float* wa,
                                   const float* wb, float eps, void* out, int n_rows, int hidden, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)2 * hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    DISPATCH_T(dtype, {
        GemmOut<T> ga{(const T*)a, a_parts, an, astr};
        GemmOut<T> gb{(const T*)b, b_parts, bn, bstr};
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(pair_norm_mean_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return crane_launch(pair_norm_mean_kernel<T>, dim3(n_rows), dim3(256), smem, st, ga, gb, wa, wb, eps, (T*)out,
                            hidden);
    });
}
