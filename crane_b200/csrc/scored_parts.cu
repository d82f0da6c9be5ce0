// Kernels around attention whose scores are worked on before they become weights, and of the block
// that holds it.
//
// 1. `add_group_rmsnorm`: x += (a + f), the two results of a block whose sublayers read the same norm,
//    then RMS norm in groups: the row in `groups` equal consecutive parts, each over the root of its own
//    mean square (+ eps), the whole times w.
// 2. `poly_norm`: act(z) = a N(z) + b N(z^2) + c N(z^3) + e over a token's row of a feed-forward, N dividing
//    by the root of the mean square of what it is given.
// 3. `scored_prep`: a token's row [q | k | v | gate] of the merged projection -> the query rows for the
//    attention kernel, the token's key and value rows in the pages, sigmoid(gate) per head.  On the way:
//    a causal convolution of a few taps over time on every channel (weights [taps][channels]; the inputs of the taps - 1 positions
//    before the step come from the request's state slot), RMS norm of q and of k over their whole rows,
//    rotation of the leading `rot_dims` elements of every head (element i with i + rot_dims / 2).  A head
//    may hold several maps of `dim` elements (differential attention: two); each map turns like a head of
//    its own.  Stored heads may be wider than they are (zero-filled), so that kernels compiled for one
//    head size serve.  `conv_tail_update` then replaces the slot's last taps - 1 inputs.
// 4. `head_finish`: what follows the weighted sums of a head: o = a1 - lambda a2 for two maps, o over the
//    root of its mean square times a constant, times the head's gate.
#include "common.cuh"

namespace {

// ------------------------------------------------------ residual + norm in groups
template <typename T>
__global__ void __launch_bounds__(1024)
add_group_rmsnorm_kernel(float* __restrict__ x, GemmOut<T> a, int has_a, GemmOut<T> f, int has_f,
                         const float* __restrict__ w, const int* __restrict__ rows, T* __restrict__ out,
                         int width, int groups, float eps) {
    extern __shared__ float row[];                    // [width]
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const long long base = (long long)(rows != nullptr ? rows[r] : r) * width;
    const int gsize = width / groups;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    T* o = out + (long long)r * width;
    // The row in 32 equal runs, where it splits so and a group is made of whole runs: a warp fetches, adds
    // and squares a run at a time, the runs of a group are added up in order, and the warp that fetched a
    // run writes it.  One barrier, all warps busy throughout, and the same sums whatever the number of warps.
    constexpr int RUNS = 32;
    const int seg = width / RUNS;
    if (width % RUNS == 0 && seg > 0 && gsize % seg == 0) {
        const bool pairs = (seg & 63) == 0;           // two neighbours a lane: loads and stores of pairs
        for (int run = warp; run < RUNS; run += nwarps) {
            const int c0 = run * seg;
            float ss = 0.f;
            if (pairs) {
                for (int c = c0 + 2 * lane; c < c0 + seg; c += 64) {
                    float2 v = ld2(x + base + c);
                    if (has_a || has_f) {
                        const float2 da = has_a ? a.load2(base + c) : make_float2(0.f, 0.f);
                        const float2 df = has_f ? f.load2(base + c) : make_float2(0.f, 0.f);
                        v.x += da.x + df.x;
                        v.y += da.y + df.y;
                        if (rows == nullptr) st2(x + base + c, v.x, v.y);
                    }
                    *(float2*)(row + c) = v;
                    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, ss));
                }
            } else {
                for (int c = c0 + lane; c < c0 + seg; c += 32) {
                    float v = x[base + c];
                    if (has_a || has_f) {
                        v += (has_a ? a.load(base + c) : 0.f) + (has_f ? f.load(base + c) : 0.f);
                        if (rows == nullptr) x[base + c] = v;
                    }
                    row[c] = v;
                    ss = fmaf(v, v, ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) scratch[run] = ss;
        }
        __syncthreads();
        const int per = gsize / seg;
        for (int run = warp; run < RUNS; run += nwarps) {
            const int c0 = run * seg, first = run / per * per;
            float total = 0.f;
            for (int i = 0; i < per; ++i) total += scratch[first + i];
            const float rstd = rsqrtf(total / (float)gsize + eps);
            if (pairs) {
                for (int c = c0 + 2 * lane; c < c0 + seg; c += 64) {
                    const float2 v = *(const float2*)(row + c), wv = ld2(w + c);
                    st2(o + c, v.x * rstd * wv.x, v.y * rstd * wv.y);
                }
            } else {
                for (int c = c0 + lane; c < c0 + seg; c += 32) o[c] = from_f32<T>(row[c] * rstd * w[c]);
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = x[base + c];
        if (has_a || has_f) {
            // the two results are added to one another first, then to the stream
            const float d = (has_a ? a.load(base + c) : 0.f) + (has_f ? f.load(base + c) : 0.f);
            v += d;
            if (rows == nullptr) x[base + c] = v;
        }
        row[c] = v;
    }
    __syncthreads();
    if (groups >= nwarps) {
        for (int g = warp; g < groups; g += nwarps) {
            const float* p = row + g * gsize;
            float ss = 0.f;
            for (int c = lane; c < gsize; c += 32) ss = fmaf(p[c], p[c], ss);
            const float rstd = rsqrtf(warp_sum(ss) / (float)gsize + eps);
            for (int c = lane; c < gsize; c += 32) o[g * gsize + c] = from_f32<T>(p[c] * rstd * w[g * gsize + c]);
        }
        return;
    }
    for (int g = 0; g < groups; ++g) {
        const float* p = row + g * gsize;
        float ss = 0.f;
        for (int c = threadIdx.x; c < gsize; c += blockDim.x) ss = fmaf(p[c], p[c], ss);
        const float rstd = rsqrtf(block_sum(ss, scratch) / (float)gsize + eps);
        for (int c = threadIdx.x; c < gsize; c += blockDim.x)
            o[g * gsize + c] = from_f32<T>(p[c] * rstd * w[g * gsize + c]);
    }
}

// ------------------------------------------------------ PolyNorm
// The row is read once (partial sums are added up once) and kept in shared memory between the pass that
// forms the three mean squares and the pass that writes; CACHED false: rows too long for that are read twice.
template <typename T, bool CACHED>
__global__ void __launch_bounds__(1024)
poly_norm_kernel(GemmOut<T> up, const float* __restrict__ coef, T* __restrict__ out, int F, float eps) {
    extern __shared__ float zrow[];                   // [F] when CACHED
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const long long base = (long long)blockIdx.x * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    if ((F & 1) == 0) {
        for (int c = 2 * threadIdx.x; c < F; c += 2 * blockDim.x) {
            const float2 z = up.load2(base + c);
            if (CACHED) *(float2*)(zrow + c) = z;
            const float a = z.x * z.x, b = z.y * z.y;
            s2 += a + b;
            s4 += a * a + b * b;
            s6 += a * a * a + b * b * b;
        }
    } else {
        for (int c = threadIdx.x; c < F; c += blockDim.x) {
            const float z = up.load(base + c), a = z * z;
            if (CACHED) zrow[c] = z;
            s2 += a;
            s4 += a * a;
            s6 += a * a * a;
        }
    }
    s2 = block_sum(s2, scratch);
    s4 = block_sum(s4, scratch);
    s6 = block_sum(s6, scratch);
    const float inv = 1.f / (float)F;
    const float r1 = coef[0] * rsqrtf(s2 * inv + eps), r2 = coef[1] * rsqrtf(s4 * inv + eps),
                r3 = coef[2] * rsqrtf(s6 * inv + eps), e = coef[3];
    // each thread reads back what it wrote itself
    if ((F & 1) == 0) {
        for (int c = 2 * threadIdx.x; c < F; c += 2 * blockDim.x) {
            const float2 z = CACHED ? *(const float2*)(zrow + c) : up.load2(base + c);
            st2(out + base + c, fmaf(z.x, fmaf(z.x, fmaf(z.x, r3, r2), r1), e),
                fmaf(z.y, fmaf(z.y, fmaf(z.y, r3, r2), r1), e));
        }
    } else {
        for (int c = threadIdx.x; c < F; c += blockDim.x) {
            const float z = CACHED ? zrow[c] : up.load(base + c);
            out[base + c] = from_f32<T>(fmaf(z, fmaf(z, fmaf(z, r3, r2), r1), e));
        }
    }
}

// Many rows of bf16 that come whole: every thread keeps its share of the row in registers, 16 bytes a load
// (NV loads a thread, all in flight together), one round of block sums for the three mean squares.
template <int NV>
__global__ void __launch_bounds__(256)
poly_norm_bf16_rows_kernel(const __nv_bfloat16* __restrict__ up, const float* __restrict__ coef,
                           __nv_bfloat16* __restrict__ out, int F, float eps) {
    __shared__ float red[3][8];
    pdl_launch_dependents();
    pdl_wait();
    const uint4* src = (const uint4*)(up + (long long)blockIdx.x * F);
    uint4* dst = (uint4*)(out + (long long)blockIdx.x * F);
    const int nvec = F >> 3;
    uint4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int idx = threadIdx.x + k * 256;
        v[k] = idx < nvec ? src[idx] : make_uint4(0u, 0u, 0u, 0u);
    }
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const __nv_bfloat162* h = (const __nv_bfloat162*)&v[k];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 z = __bfloat1622float2(h[i]);
            const float a = z.x * z.x, b = z.y * z.y;
            s2 += a + b;
            s4 += a * a + b * b;
            s6 += a * a * a + b * b * b;
        }
    }
    s2 = warp_sum(s2);
    s4 = warp_sum(s4);
    s6 = warp_sum(s6);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { red[0][warp] = s2; red[1][warp] = s4; red[2][warp] = s6; }
    __syncthreads();
    s2 = s4 = s6 = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { s2 += red[0][w]; s4 += red[1][w]; s6 += red[2][w]; }
    const float inv = 1.f / (float)F;
    const float r1 = coef[0] * rsqrtf(s2 * inv + eps), r2 = coef[1] * rsqrtf(s4 * inv + eps),
                r3 = coef[2] * rsqrtf(s6 * inv + eps), e = coef[3];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int idx = threadIdx.x + k * 256;
        if (idx < nvec) {
            uint4 o;
            const __nv_bfloat162* h = (const __nv_bfloat162*)&v[k];
            __nv_bfloat162* q = (__nv_bfloat162*)&o;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 z = __bfloat1622float2(h[i]);
                q[i] = __floats2bfloat162_rn(fmaf(z.x, fmaf(z.x, fmaf(z.x, r3, r2), r1), e),
                                             fmaf(z.y, fmaf(z.y, fmaf(z.y, r3, r2), r1), e));
            }
            dst[idx] = o;
        }
    }
}

// ------------------------------------------------------ projection -> queries, pages
struct PrepArgs {
    int cols;                       // columns of a row of the merged projection
    const int* positions;
    const int* tok_entry;
    const int* cu_q;
    const int* kv_len;
    const int* slots;
    int n_slots;
    const float* tails;             // [slots][taps - 1][C]: the convolutions' last inputs (taps > 1)
    long long slot_stride;
    const float* conv_w;            // [taps][C] (a tap's weights of neighbouring channels side by side), or null
    int taps;
    const int* block_table;
    int max_blocks, num_pages, page_size;
    const float* qw;                // norm weights over the whole q / k rows, or null
    const float* kw;
    float eps;
    void* q_out;                    // [n][H][dk_store]
    void* k_pool;                   // [pages][G][page_size][dk_store]
    void* v_pool;                   // [pages][G][page_size][dv_store]
    int H, G, maps, dim, dv;        // a query / key head holds `maps` maps of `dim` elements, a value head dv
    int dk_store, dpad, dv_store;   // stored widths; map i of a head starts at i * dpad
    const float* cos_tab;
    const float* sin_tab;
    int n_positions, rot_dims;
    float* gate_out;                // [n][H] sigmoid of the gate columns, or null
    int gate_col;                   // where they start in the row
    int* err;
};

// One stored head row of queries or keys: norm factor and weight, rotation.  sm: the token's channels
// after the convolution; ch0: the first channel of the head's map; i: element within the map.
__device__ __forceinline__ float prep_element(const float* sm, const float* nw, float rn, int ch0, int i, int half,
                                              const float* ct, const float* sn) {
    float v = sm[ch0 + i] * rn * (nw != nullptr ? nw[ch0 + i] : 1.f);
    if (i < 2 * half) {
        const int j = i < half ? i + half : i - half, a = i < half ? i : i - half;
        const float o = sm[ch0 + j] * rn * (nw != nullptr ? nw[ch0 + j] : 1.f);
        v = i < half ? v * ct[a] - o * sn[a] : v * ct[a] + o * sn[a];
    }
    return v;
}

// TAPS: the convolution's taps when they are 2, 3 or 4 (the loads of a channel's taps are then in flight
// together), 0: any number, or no convolution.  VEC: two neighbouring channels a thread (every width even,
// the rotated half even): loads and stores of pairs.
template <typename T, int TAPS, bool VEC>
__global__ void __launch_bounds__(1024)
scored_prep_kernel(GemmOut<T> proj, const PrepArgs a) {
    extern __shared__ float sm[];                     // [C] the token's q, k, v after the convolution
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int e = a.tok_entry[t];
    if (e < 0) return;
    const int Cq = a.H * a.maps * a.dim, Ck = a.G * a.maps * a.dim, Cv = a.G * a.dv, C = Cq + Ck + Cv;
    const int pos = a.positions[t];
    const int half = a.cos_tab != nullptr ? a.rot_dims >> 1 : 0;
    if (half > 0 && (pos < 0 || pos >= a.n_positions)) {
        if (threadIdx.x == 0) atomicOr(a.err, CRANE_ERR_POSITION_RANGE);
        return;
    }
    constexpr int W = VEC ? 2 : 1;
    const long long base = (long long)t * a.cols;
    float sq = 0.f, sk = 0.f;
    if (a.conv_w != nullptr) {
        const int first = a.cu_q[e];
        const int i = t - first;                                      // the token's place in its portion
        const int start = a.kv_len[e] - (a.cu_q[e + 1] - first);      // tokens of the request before the step
        const int taps = TAPS ? TAPS : a.taps;
        const float* tail = nullptr;                                  // (a single tap reads no earlier position)
        if (taps > 1) {
            const int slot = a.slots[e];
            if (slot < 0 || slot >= a.n_slots) {
                if (threadIdx.x == 0) atomicOr(a.err, CRANE_ERR_SLOT_RANGE);
                return;
            }
            tail = a.tails + (long long)slot * a.slot_stride;
        }
        for (int c = W * threadIdx.x; c < C; c += W * blockDim.x) {
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int j = 0; j < (TAPS ? TAPS : taps); ++j) {
                const int back = taps - 1 - j;
                float u0 = 0.f, u1 = 0.f;
                if (i - back >= 0) {
                    if (VEC) { const float2 u = proj.load2(base - (long long)back * a.cols + c); u0 = u.x; u1 = u.y; }
                    else u0 = proj.load(base - (long long)back * a.cols + c);
                } else if (start + i - back >= 0) {
                    const float* p = tail + (long long)(taps - 1 + i - back) * C + c;
                    if (VEC) { const float2 u = *(const float2*)p; u0 = u.x; u1 = u.y; }
                    else u0 = *p;
                }
                if (VEC) {
                    const float2 w = *(const float2*)(a.conv_w + (long long)j * C + c);
                    acc0 = fmaf(w.x, u0, acc0);
                    acc1 = fmaf(w.y, u1, acc1);
                } else {
                    acc0 = fmaf(a.conv_w[(long long)j * C + c], u0, acc0);
                }
            }
            sm[c] = acc0;
            if (VEC) sm[c + 1] = acc1;
            const float ss = VEC ? fmaf(acc0, acc0, acc1 * acc1) : acc0 * acc0;
            if (c < Cq) sq += ss;
            else if (c < Cq + Ck) sk += ss;
        }
    } else {
        for (int c = W * threadIdx.x; c < C; c += W * blockDim.x) {
            float v0, v1 = 0.f;
            if (VEC) { const float2 u = proj.load2(base + c); v0 = u.x; v1 = u.y; sm[c + 1] = v1; }
            else v0 = proj.load(base + c);
            sm[c] = v0;
            const float ss = fmaf(v0, v0, v1 * v1);
            if (c < Cq) sq += ss;
            else if (c < Cq + Ck) sk += ss;
        }
    }
    float rq = 1.f, rk = 1.f;
    if (a.qw != nullptr) rq = rsqrtf(block_sum(sq, scratch) / (float)Cq + a.eps);
    if (a.kw != nullptr) rk = rsqrtf(block_sum(sk, scratch) / (float)Ck + a.eps);
    __syncthreads();
    const float* ct = a.cos_tab + (long long)pos * half;
    const float* sn = a.sin_tab + (long long)pos * half;
    if (a.gate_out != nullptr)
        for (int h = threadIdx.x; h < a.H; h += blockDim.x)
            a.gate_out[(long long)t * a.H + h] = 1.f / (1.f + expf(-proj.load(base + a.gate_col + h)));
    const int blk = pos / a.page_size;
    const int page = (pos >= 0 && blk < a.max_blocks) ? a.block_table[(long long)e * a.max_blocks + blk] : -1;
    const bool page_ok = page >= 0 && page < a.num_pages;
    if (!page_ok && threadIdx.x == 0) atomicOr(a.err, CRANE_ERR_PAGE_RANGE);
    const long long place = ((long long)page * a.G) * a.page_size + pos % a.page_size;   // of key/value head 0
    // a warp per stored head: H of queries, then G of keys, then G of values
    const int lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int u = threadIdx.x >> 5; u < a.H + 2 * a.G; u += nwarps) {
        if (u >= a.H && !page_ok) break;
        if (u < a.H + a.G) {
            const bool is_q = u < a.H;
            const int hd = is_q ? u : u - a.H;
            T* dst = is_q ? (T*)a.q_out + ((long long)t * a.H + hd) * a.dk_store
                          : (T*)a.k_pool + (place + (long long)hd * a.page_size) * a.dk_store;
            const float* src = is_q ? sm : sm + Cq;
            const float* nw = is_q ? a.qw : a.kw;
            const float rn = is_q ? rq : rk;
            for (int mp = 0; mp < a.maps; ++mp) {
                const int ch0 = (hd * a.maps + mp) * a.dim;
                for (int i = W * lane; i < a.dpad; i += W * 32) {
                    float v0 = 0.f, v1 = 0.f;
                    if (i < a.dim) {
                        v0 = prep_element(src, nw, rn, ch0, i, half, ct, sn);
                        if (VEC) v1 = prep_element(src, nw, rn, ch0, i + 1, half, ct, sn);
                    }
                    if (VEC) st2(dst + mp * a.dpad + i, v0, v1);
                    else dst[mp * a.dpad + i] = from_f32<T>(v0);
                }
            }
            for (int i = a.maps * a.dpad + W * lane; i < a.dk_store; i += W * 32) {
                if (VEC) st2(dst + i, 0.f, 0.f);
                else dst[i] = from_f32<T>(0.f);
            }
        } else {
            const int g = u - a.H - a.G;
            T* dst = (T*)a.v_pool + (place + (long long)g * a.page_size) * a.dv_store;
            const float* src = sm + Cq + Ck + g * a.dv;
            for (int i = W * lane; i < a.dv_store; i += W * 32) {
                const float v0 = i < a.dv ? src[i] : 0.f;
                if (VEC) st2(dst + i, v0, i + 1 < a.dv ? src[i + 1] : 0.f);
                else dst[i] = from_f32<T>(v0);
            }
        }
    }
}

// The slot's last taps - 1 inputs after the step.  One thread per (entry, channel) walks the places in
// order: place j takes what lay q_len places further on (or a row of this step), which no earlier
// write of the walk has touched.
template <typename T>
__global__ void __launch_bounds__(128)
conv_tail_update_kernel(GemmOut<T> proj, int cols, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                        const int* __restrict__ slots, int n_slots, float* __restrict__ tails, long long slot_stride,
                        int taps, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int first = cu_q[e], q_len = cu_q[e + 1] - first;
    if (q_len <= 0 || c >= C) return;
    const int slot = slots[e];
    if (slot < 0 || slot >= n_slots) return;
    const int end = kv_len[e], start = end - q_len;
    float* tail = tails + (long long)slot * slot_stride;
    for (int j = 0; j < taps - 1; ++j) {
        const int p = end - (taps - 1) + j;            // the position whose input place j holds afterwards
        float v = 0.f;
        if (p >= start) v = proj.load((long long)(first + p - start) * cols + c);
        else if (p >= 0) v = tail[(long long)(j + q_len) * C + c];
        tail[(long long)j * C + c] = v;
    }
}

// ------------------------------------------------------ after the weighted sums
// a: float [n][H][maps][dv_in] (the maps' normalised results).  One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(256)
head_finish_kernel(const float* __restrict__ a, const int* __restrict__ tok_entry, const float* __restrict__ gate,
                   T* __restrict__ out, int n, int H, int maps, int dv, int dv_in, int dv_out, float lambda,
                   int norm, float norm_scale, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)n * H) return;
    const int t = (int)(unit / H);
    if (tok_entry[t] < 0) return;
    const float* p = a + unit * maps * dv_in;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) {
        const float o = maps == 2 ? p[c] - lambda * p[dv_in + c] : p[c];
        ss = fmaf(o, o, ss);
    }
    float f = 1.f;
    if (norm) f = rsqrtf(warp_sum(ss) / (float)dv + eps) * norm_scale;
    if (gate != nullptr) f *= gate[unit];
    T* op = out + unit * dv_out;
    for (int c = lane; c < dv_out; c += 32) {
        float o = 0.f;
        if (c < dv) o = (maps == 2 ? p[c] - lambda * p[dv_in + c] : p[c]) * f;
        op[c] = from_f32<T>(o);
    }
}

}  // namespace

CRANE_API int crane_add_group_rmsnorm(int dtype, float* x, const void* a, const float* a_parts, int a_n,
                                      long long a_stride, const void* f, const float* f_parts, int f_n,
                                      long long f_stride, const float* w, const int* rows, void* out, int n_rows,
                                      int width, int groups, float eps, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (groups <= 0 || width % groups != 0 || (size_t)width * sizeof(float) > 200 * 1024) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)width * sizeof(float);
    DISPATCH_T(dtype, {
        GemmOut<T> ga{(const T*)a, a_parts, a_n, a_stride}, gf{(const T*)f, f_parts, f_n, f_stride};
        auto kern = add_group_rmsnorm_kernel<T>;
        if (smem > 48 * 1024) {
            static size_t configured = 0;
            if (configured < smem) {
                if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                    return (int)cudaGetLastError();
                configured = smem;
            }
        }
        // few rows: more threads a row (what bounds them is the chain of loads a thread waits for), where the
        // row goes in runs whose sums do not depend on the number of warps
        const bool runs = width % 32 == 0 && (width / groups) % (width / 32) == 0;
        return crane_launch(kern, dim3(n_rows), dim3(runs && n_rows <= 64 ? 1024 : 256), smem, st, x, ga,
                            (a != nullptr || a_parts != nullptr) ? 1 : 0, gf,
                            (f != nullptr || f_parts != nullptr) ? 1 : 0, w, rows, (T*)out, width, groups, eps);
    });
}

CRANE_API int crane_poly_norm(int dtype, const void* up, const float* up_parts, int n_parts, long long part_stride,
                              const float* coef, void* out, int n_rows, int F, float eps, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)F * sizeof(float);
    const bool cached = smem <= 96 * 1024;
    // few rows: more threads a row (what bounds them is the chain of loads a thread waits for)
    // (bfloat16 only: in true 32-bit the sums keep one order whatever the step's size, so that a position's
    // logits do not depend on how its request was cut, to the bit)
    const int threads = (dtype == 1 && n_rows <= 64) ? 1024 : 256;
    if (dtype == 1 && up != nullptr && n_rows > 64 && F % 8 == 0 && F <= 16384 && ((uintptr_t)up & 15) == 0 &&
        ((uintptr_t)out & 15) == 0) {
        const __nv_bfloat16* u = (const __nv_bfloat16*)up;
        __nv_bfloat16* o = (__nv_bfloat16*)out;
        if (F <= 4096) return crane_launch(poly_norm_bf16_rows_kernel<2>, dim3(n_rows), dim3(256), 0, st, u, coef, o, F, eps);
        if (F <= 8192) return crane_launch(poly_norm_bf16_rows_kernel<4>, dim3(n_rows), dim3(256), 0, st, u, coef, o, F, eps);
        if (F <= 12288) return crane_launch(poly_norm_bf16_rows_kernel<6>, dim3(n_rows), dim3(256), 0, st, u, coef, o, F, eps);
        return crane_launch(poly_norm_bf16_rows_kernel<8>, dim3(n_rows), dim3(256), 0, st, u, coef, o, F, eps);
    }
    DISPATCH_T(dtype, {
        GemmOut<T> g{(const T*)up, up_parts, n_parts, part_stride};
        if (!cached)
            return crane_launch(poly_norm_kernel<T, false>, dim3(n_rows), dim3(threads), 0, st, g, coef, (T*)out, F, eps);
        auto kern = poly_norm_kernel<T, true>;
        if (smem > 48 * 1024) {
            static size_t configured = 0;
            if (configured < smem) {
                if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                    return (int)cudaGetLastError();
                configured = smem;
            }
        }
        return crane_launch(kern, dim3(n_rows), dim3(threads), smem, st, g, coef, (T*)out, F, eps);
    });
}

// Every pointer and size of the preparation in one block of arguments (see PrepArgs); then, with a
// convolution, the slot's last inputs are replaced by a second kernel.
CRANE_API int crane_scored_prep(int dtype, const void* proj, const float* proj_parts, int n_parts, long long part_stride,
                                int cols, const int* positions, const int* tok_entry, const int* cu_q,
                                const int* kv_len, const int* slots, int n_slots, float* tails, long long slot_stride,
                                const float* conv_w, int taps, const int* block_table, int max_blocks, int num_pages,
                                int page_size, const float* qw, const float* kw, float eps, void* q_out, void* k_pool,
                                void* v_pool, int n_tokens, int n_entries, int H, int G, int maps, int dim, int dv,
                                int dk_store, int dpad, int dv_store, const float* cos_tab, const float* sin_tab,
                                int n_positions, int rot_dims, float* gate_out, int gate_col, int* err,
                                cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    const int C = (H + G) * maps * dim + G * dv;
    if (maps < 1 || dpad < dim || dk_store < maps * dpad || dv_store < dv || taps < 1 || rot_dims > dim || (conv_w != nullptr && taps > 1 && tails == nullptr) ||
        (size_t)C * sizeof(float) > 200 * 1024)
        return (int)cudaErrorInvalidValue;
    PrepArgs a;
    a.cols = cols; a.positions = positions; a.tok_entry = tok_entry; a.cu_q = cu_q; a.kv_len = kv_len;
    a.slots = slots; a.n_slots = n_slots; a.tails = taps > 1 ? tails : nullptr; a.slot_stride = slot_stride;
    a.conv_w = conv_w; a.taps = taps; a.block_table = block_table; a.max_blocks = max_blocks;
    a.num_pages = num_pages; a.page_size = page_size; a.qw = qw; a.kw = kw; a.eps = eps; a.q_out = q_out;
    a.k_pool = k_pool; a.v_pool = v_pool; a.H = H; a.G = G; a.maps = maps; a.dim = dim; a.dv = dv;
    a.dk_store = dk_store; a.dpad = dpad; a.dv_store = dv_store; a.cos_tab = cos_tab; a.sin_tab = sin_tab;
    a.n_positions = n_positions; a.rot_dims = cos_tab != nullptr ? rot_dims : 0; a.gate_out = gate_out;
    a.gate_col = gate_col; a.err = err;
    const size_t smem = (size_t)C * sizeof(float);
    DISPATCH_T(dtype, {
        GemmOut<T> g{(const T*)proj, proj_parts, n_parts, part_stride};
        // pairs of channels where every width is even and a rotated half is too; the taps known at compile
        // time where they are few
        const bool vec = !(dim & 1) && !(dv & 1) && !(dpad & 1) && !(dk_store & 1) && !(dv_store & 1) && !(cols & 1) &&
                         !(a.rot_dims & 3) && !(slot_stride & 1) && !(C & 1);
        const int known = (conv_w != nullptr && taps >= 2 && taps <= 4) ? taps : 0;
        void (*kern)(GemmOut<T>, const PrepArgs) = nullptr;
        if (vec) kern = known == 2 ? scored_prep_kernel<T, 2, true> : known == 3 ? scored_prep_kernel<T, 3, true>
                      : known == 4 ? scored_prep_kernel<T, 4, true> : scored_prep_kernel<T, 0, true>;
        else kern = known == 2 ? scored_prep_kernel<T, 2, false> : known == 3 ? scored_prep_kernel<T, 3, false>
                  : known == 4 ? scored_prep_kernel<T, 4, false> : scored_prep_kernel<T, 0, false>;
        if (smem > 48 * 1024) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                return (int)cudaGetLastError();
        }
        // few tokens: more threads a token (what bounds them is the chain of loads a thread waits for)
        // (bfloat16 only: in true 32-bit the sums keep one order whatever the step's size)
        // (many tokens: CTAs of 128 threads, of which more are in different phases at once: 33 against 37 us at
        // 2,048 tokens, 46 us with 512)
        int rc = crane_launch(kern, dim3(n_tokens), dim3((dtype == 1 && n_tokens <= 64) ? 1024 : 128), smem, st, g, a);
        if (rc != 0 || taps <= 1 || tails == nullptr) return rc;
        return crane_launch(conv_tail_update_kernel<T>, dim3((C + 127) / 128, n_entries), dim3(128), 0, st, g, cols,
                            cu_q, kv_len, slots, n_slots, tails, slot_stride, taps, C);
    });
}

CRANE_API int crane_head_finish(int dtype, const float* a, const int* tok_entry, const float* gate, void* out, int n,
                                int H, int maps, int dv, int dv_in, int dv_out, float lambda, int norm,
                                float norm_scale, float eps, cudaStream_t st) {
    if (n <= 0) return 0;
    if (maps < 1 || maps > 2 || dv_in < dv || dv_out < dv) return (int)cudaErrorInvalidValue;
    const long long units = (long long)n * H;
    DISPATCH_T(dtype, {
        return crane_launch(head_finish_kernel<T>, dim3((unsigned)((units + 7) / 8)), dim3(256), 0, st, a, tok_entry,
                            gate, (T*)out, n, H, maps, dv, dv_in, dv_out, lambda, norm, norm_scale, eps);
    });
}
