// Kernels of two mixers.
//
// 1. Attention whose queries and keys are RMS-normed over their whole projections (all heads at
//    once) and not rotated: `projection_norm_cache` norms q and k, writes q for the attention kernel
//    and the token's key and value rows into the pages.  Key and value rows may be stored wider than
//    they are (zero-filled), so that kernels written for one head size serve both.
//
// 2. The generalized delta rule, a linear recurrence with one matrix state S [dk, dv] per head:
//        S <- diag(w) S - (a * u) (u^T S) + k v^T,     o = S^T r
//    w the decay per key channel, a the removal rate, u the key scaled to unit length; both
//    corrections read the state before the token.  `delta_rule_prep` forms w, a * u and u of every
//    token in 32-bit; `delta_rule_scan` walks each request's tokens in order with the state of a head
//    spread over the threads of a CTA (columns of S do not talk to one another; a column's rows are
//    spread over a few lanes), then norms each head's read-out, gates it and writes it for the output
//    projection.
//    The state lives in 32-bit in the request's slot between steps.
#include "common.cuh"

namespace {

// ------------------------------------------------------ projection norm + cache write
// qkv row: [q (nq * d) | k (nkv * d) | v (nkv * dv)].  One CTA per token.
template <typename T>
__global__ void __launch_bounds__(256)
projection_norm_cache_kernel(GemmOut<T> qkv, int cols, const int* __restrict__ positions,
                             const int* __restrict__ tok_entry, const int* __restrict__ block_table,
                             int max_blocks, int num_pages, int page_size, const float* __restrict__ qw,
                             const float* __restrict__ kw, float eps, T* __restrict__ q_out,
                             T* __restrict__ k_pool, T* __restrict__ v_pool, int nq, int nkv, int d, int dv,
                             int d_store, int dv_store, const float* __restrict__ cos_tab,
                             const float* __restrict__ sin_tab, int n_positions, int rot_dims,
                             const float* __restrict__ q_head_scale, int* err) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int e = tok_entry[t];
    if (e < 0) return;
    // Rotary positions (after the norms): the leading rot_dims elements of every query and key head,
    // element i paired with i + rot_dims / 2, by the angles of the token's row of the tables.
    const int half = cos_tab != nullptr ? rot_dims >> 1 : 0;
    const int rpos = positions[t];
    if (half > 0 && (rpos < 0 || rpos >= n_positions)) {
        if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_POSITION_RANGE);
        return;
    }
    const float* ct = cos_tab + (long long)rpos * half;
    const float* sn = sin_tab + (long long)rpos * half;
    const long long base = (long long)t * cols;
    const int nqd = nq * d, nkd = nkv * d, nvd = nkv * dv;
    float sq = 0.f, sk = 0.f;
#pragma unroll 4
    for (int c = threadIdx.x; c < nqd; c += blockDim.x) { const float v = qkv.load(base + c); sq += v * v; }
#pragma unroll 4
    for (int c = threadIdx.x; c < nkd; c += blockDim.x) { const float v = qkv.load(base + nqd + c); sk += v * v; }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    const float rq = qw != nullptr ? rsqrtf(sq / (float)nqd + eps) : 1.f;
    const float rk = kw != nullptr ? rsqrtf(sk / (float)nkd + eps) : 1.f;
    // queries, heads d_store apart
#pragma unroll 4
    for (int c = threadIdx.x; c < nq * d_store; c += blockDim.x) {
        const int h = c / d_store, i = c % d_store;
        float v = 0.f;
        if (i < d) v = qkv.load(base + h * d + i) * rq * (qw != nullptr ? qw[h * d + i] : 1.f);
        if (i < 2 * half) {
            const int j = i < half ? i + half : i - half, a = i < half ? i : i - half;
            const float o = qkv.load(base + h * d + j) * rq * (qw != nullptr ? qw[h * d + j] : 1.f);
            v = i < half ? v * ct[a] - o * sn[a] : v * ct[a] + o * sn[a];
        }
        if (q_head_scale != nullptr) v *= q_head_scale[h];
        q_out[(long long)t * nq * d_store + c] = from_f32<T>(v);
    }
    const int pos = positions[t];
    const int blk = pos / page_size;
    const int page = blk < max_blocks ? block_table[(long long)e * max_blocks + blk] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
        return;
    }
    const int slot = pos % page_size;
#pragma unroll 4
    for (int c = threadIdx.x; c < nkv * d_store; c += blockDim.x) {
        const int g = c / d_store, i = c % d_store;
        float v = 0.f;
        if (i < d) v = qkv.load(base + nqd + g * d + i) * rk * (kw != nullptr ? kw[g * d + i] : 1.f);
        if (i < 2 * half) {
            const int j = i < half ? i + half : i - half, a = i < half ? i : i - half;
            const float o = qkv.load(base + nqd + g * d + j) * rk * (kw != nullptr ? kw[g * d + j] : 1.f);
            v = i < half ? v * ct[a] - o * sn[a] : v * ct[a] + o * sn[a];
        }
        k_pool[(((long long)page * nkv + g) * page_size + slot) * d_store + i] = from_f32<T>(v);
    }
#pragma unroll 4
    for (int c = threadIdx.x; c < nkv * dv_store; c += blockDim.x) {
        const int g = c / dv_store, i = c % dv_store;
        const float v = i < dv ? qkv.load(base + nqd + nkd + g * dv + i) : 0.f;
        v_pool[(((long long)page * nkv + g) * page_size + slot) * dv_store + i] = from_f32<T>(v);
    }
    (void)nvd;
}

// ------------------------------------------------------ delta rule: per-token inputs
// proj row: [r | k | v | g | a | low] with r, k, v, g, a of heads * d columns and `rank` columns of
// the decay's inner product.  aux row (float): [w | a * u | u], each heads * d.
//   w = exp(-decay_scale * sigmoid(sum_j w2[c][j] tanh(low[j]) + w0[c]))
//   a = sigmoid(a_pre + ab[c]);  u = k / sqrt(sum over the head of k^2 + key_eps)
// `w2t` is w2 turned over, [rank][heads * d], so that neighbouring threads (channels) read neighbouring
// weights.  A CTA takes PREP_TOKENS tokens and a block of whole heads: every weight it reads serves
// all its tokens: PREP_TOKENS = 8 for many tokens.  For the few tokens of a step of single tokens a CTA
// takes one token: what bounds it there is the chain of loads a thread waits for one after the other.
template <typename T, int PREP_TOKENS>
__global__ void __launch_bounds__(256)
delta_rule_prep_kernel(GemmOut<T> proj, int cols, const int* __restrict__ tok_entry, const T* __restrict__ w2t,
                       const float* __restrict__ w0, const float* __restrict__ ab, float* __restrict__ aux,
                       int n_tokens, int heads, int d, int rank, int heads_per_cta, float decay_scale,
                       float key_eps) {
    extern __shared__ float sm[];          // [PREP_TOKENS][rank] tanh(low), [PREP_TOKENS][heads_per_cta] 1 / |k|
    float* th = sm;
    float* inv_len = sm + PREP_TOKENS * rank;
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * PREP_TOKENS;
    const int nt = min(PREP_TOKENS, n_tokens - t0);
    const int h0 = blockIdx.y * heads_per_cta;
    const int nh = min(heads_per_cta, heads - h0);
    const int hd = heads * d;
    for (int idx = threadIdx.x; idx < PREP_TOKENS * rank; idx += blockDim.x) {
        const int tt = idx / rank, j = idx % rank;
        th[idx] = tt < nt ? tanhf(proj.load((long long)(t0 + tt) * cols + 5 * hd + j)) : 0.f;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int idx = warp; idx < nt * nh; idx += nwarps) {
        const int tt = idx / nh, h = idx % nh;
        const long long kb = (long long)(t0 + tt) * cols + hd + (h0 + h) * d;
        float ss = 0.f;
#pragma unroll 4
        for (int i = lane; i < d; i += 32) { const float kv = proj.load(kb + i); ss += kv * kv; }
        ss = warp_sum(ss);
        if (lane == 0) inv_len[tt * heads_per_cta + h] = rsqrtf(ss + key_eps);
    }
    __syncthreads();
    for (int cc = threadIdx.x; cc < nh * d; cc += blockDim.x) {
        const int c = h0 * d + cc;
        float low[PREP_TOKENS], a_pre[PREP_TOKENS], key[PREP_TOKENS];
        const float b0 = w0[c];
        // (what the end of the loop needs of the product is asked for now, so that it arrives meanwhile)
#pragma unroll
        for (int tt = 0; tt < PREP_TOKENS; ++tt) {
            low[tt] = b0;
            const long long base = (long long)(t0 + (tt < nt ? tt : 0)) * cols;
            a_pre[tt] = proj.load(base + 4 * hd + c);
            key[tt] = proj.load(base + hd + c);
        }
#pragma unroll 8
        for (int j = 0; j < rank; ++j) {
            const float wv = to_f32(w2t[(long long)j * hd + c]);
#pragma unroll
            for (int tt = 0; tt < PREP_TOKENS; ++tt) low[tt] = fmaf(wv, th[tt * rank + j], low[tt]);
        }
        const float bias = ab[c];
#pragma unroll
        for (int tt = 0; tt < PREP_TOKENS; ++tt) {
            if (tt >= nt || tok_entry[t0 + tt] < 0) continue;
            const float w = expf(-decay_scale / (1.f + expf(-low[tt])));
            const float a = 1.f / (1.f + expf(-(a_pre[tt] + bias)));
            const float u = key[tt] * inv_len[tt * heads_per_cta + cc / d];
            float* out = aux + (long long)(t0 + tt) * 3 * hd;
            out[c] = w;
            out[hd + c] = a * u;
            out[2 * hd + c] = u;
        }
    }
}

// ------------------------------------------------------ delta rule: the recurrence
// grid (entries, heads); thread j < d owns column j of the head's state.  DK > 0: the column lives in
// registers (d == DK); DK == 0: in shared memory (any d that fits).  Tokens come in tiles of TT whose
// per-token vectors (r, k, w, a u, u over the key channels, v and the gate over the columns) all threads
// load together.  After a tile, a warp per token norms the head's read-out (RMS over the columns),
// multiplies by the norm's weight and sigmoid(gate) and writes T for the output projection.
constexpr int TT = 16;

template <typename T, int DK>
__global__ void __launch_bounds__(256)
delta_rule_scan_kernel(GemmOut<T> proj, int cols, const float* __restrict__ aux, const int* __restrict__ cu_q,
                       const int* __restrict__ kv_len, const int* __restrict__ slots, int n_slots,
                       float* __restrict__ state, const float* __restrict__ norm_w, float norm_eps,
                       T* __restrict__ out, int heads, int d, int* err) {
    extern __shared__ float sm[];
    // layout: vec [TT][5][d] (r, k, w, au, u), val [TT][d] (v), gate [TT][d], o [TT][d], then the state (DK == 0)
    float* vec = sm;
    float* val = vec + TT * 5 * d;
    float* gat = val + TT * d;
    float* o_s = gat + TT * d;
    float* S_s = o_s + TT * d;
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x, h = blockIdx.y;
    const int first = cu_q[e], n = cu_q[e + 1] - first;
    if (n <= 0) return;                                  // an entry that pads the step: no slot is touched
    int slot = slots[e];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_SLOT_RANGE);
        return;
    }
    const int j = threadIdx.x;
    const bool own = j < d;
    const int hd = heads * d;
    float* S_g = state + ((long long)slot * heads + h) * d * d;
    const bool fresh = kv_len[e] - n == 0;               // the request's first tokens: the state starts at zero
    float S[DK > 0 ? DK : 1];
    if (own) {
        if (DK > 0) {
#pragma unroll
            for (int i = 0; i < DK; ++i) S[i] = fresh ? 0.f : S_g[i * d + j];
        } else {
            for (int i = 0; i < d; ++i) S_s[i * d + j] = fresh ? 0.f : S_g[i * d + j];
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int t0 = 0; t0 < n; t0 += TT) {
        const int nt = min(TT, n - t0);
        __syncthreads();                                 // the tile before has been read out
        for (int idx = threadIdx.x; idx < nt * d; idx += blockDim.x) {
            const int tt = idx / d, c = idx % d;
            const long long row = (long long)(first + t0 + tt);
            const long long pb = row * cols + h * d + c;
            const float* ax = aux + row * 3 * hd + h * d + c;
            float* v5 = vec + (tt * 5) * d + c;
            v5[0] = proj.load(pb);                       // r
            v5[d] = proj.load(pb + hd);                  // k
            v5[2 * d] = ax[0];                           // w
            v5[3 * d] = ax[hd];                          // a u
            v5[4 * d] = ax[2 * hd];                      // u
            val[tt * d + c] = proj.load(pb + 2 * hd);    // v
            gat[tt * d + c] = proj.load(pb + 3 * hd);    // gate, before its sigmoid
        }
        __syncthreads();
        if (own) {
            for (int tt = 0; tt < nt; ++tt) {
                const float* r = vec + (tt * 5) * d;
                const float *k = r + d, *w = r + 2 * d, *au = r + 3 * d, *u = r + 4 * d;
                const float v = val[tt * d + j];
                float dot0 = 0.f, dot1 = 0.f, dot2 = 0.f, dot3 = 0.f;
                if (DK > 0) {
#pragma unroll
                    for (int i = 0; i < DK; i += 4) {
                        dot0 = fmaf(u[i], S[i], dot0);
                        dot1 = fmaf(u[i + 1], S[i + 1], dot1);
                        dot2 = fmaf(u[i + 2], S[i + 2], dot2);
                        dot3 = fmaf(u[i + 3], S[i + 3], dot3);
                    }
                } else {
                    for (int i = 0; i < d; ++i) dot0 = fmaf(u[i], S_s[i * d + j], dot0);
                }
                const float dot = (dot0 + dot1) + (dot2 + dot3);
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
                if (DK > 0) {
#pragma unroll
                    for (int i = 0; i < DK; i += 4) {
                        S[i] = fmaf(w[i], S[i], fmaf(-au[i], dot, k[i] * v));
                        S[i + 1] = fmaf(w[i + 1], S[i + 1], fmaf(-au[i + 1], dot, k[i + 1] * v));
                        S[i + 2] = fmaf(w[i + 2], S[i + 2], fmaf(-au[i + 2], dot, k[i + 2] * v));
                        S[i + 3] = fmaf(w[i + 3], S[i + 3], fmaf(-au[i + 3], dot, k[i + 3] * v));
                        o0 = fmaf(r[i], S[i], o0);
                        o1 = fmaf(r[i + 1], S[i + 1], o1);
                        o2 = fmaf(r[i + 2], S[i + 2], o2);
                        o3 = fmaf(r[i + 3], S[i + 3], o3);
                    }
                } else {
                    for (int i = 0; i < d; ++i) {
                        const float s = fmaf(w[i], S_s[i * d + j], fmaf(-au[i], dot, k[i] * v));
                        S_s[i * d + j] = s;
                        o0 = fmaf(r[i], s, o0);
                    }
                }
                o_s[tt * d + j] = (o0 + o1) + (o2 + o3);
            }
        }
        __syncthreads();
        for (int tt = warp; tt < nt; tt += nwarps) {
            float ss = 0.f;
            for (int c = lane; c < d; c += 32) { const float v = o_s[tt * d + c]; ss += v * v; }
            ss = warp_sum(ss);
            const float rs = rsqrtf(ss / (float)d + norm_eps);
            T* op = out + (long long)(first + t0 + tt) * hd + h * d;
            for (int c = lane; c < d; c += 32) {
                const float g = 1.f / (1.f + expf(-gat[tt * d + c]));
                op[c] = from_f32<T>(o_s[tt * d + c] * rs * norm_w[h * d + c] * g);
            }
        }
    }
    if (own) {
        if (DK > 0) {
#pragma unroll
            for (int i = 0; i < DK; ++i) S_g[i * d + j] = S[i];
        } else {
            for (int i = 0; i < d; ++i) S_g[i * d + j] = S_s[i * d + j];
        }
    }
}

// The same recurrence for heads of at most 128 elements as a register tile: a lane holds SPLIT_ROWS
// rows of COLS columns of S.  A column's rows are spread over P = 1, 2 or 4 lanes of a warp (part p
// has rows p * rows_pp ...), so the chain of multiply-adds per token is SPLIT_ROWS long instead of d and
// the partial sums of u^T S and of the read-out go round by shuffles; there is no block barrier inside
// a tile.  What a lane reads of the per-token vectors (its part's rows of r, k, w, a u, u) serves all
// its columns.  Lane = part * (32 / P) + i, and its
// c-th column is warp * COLS * (32 / P) + c * (32 / P) + i: at a given c neighbouring lanes hold
// neighbouring columns.  In shared memory every per-token vector lies in P segments SPLIT_ROWS + 8
// apart (the rows of a part, zero-filled to SPLIT_ROWS), read as 16-byte words.
// (SPLIT_ROWS, COLS) = (16, 1) serves heads of up to 64, (32, 2) up to 128.
template <typename T, int SPLIT_ROWS, int COLS, int MAX_THREADS, int MIN_CTAS>
__global__ void __launch_bounds__(MAX_THREADS, MIN_CTAS)
delta_rule_scan_split_kernel(GemmOut<T> proj, int cols, const float* __restrict__ aux,
                             const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                             const int* __restrict__ slots, int n_slots, float* __restrict__ state,
                             const float* __restrict__ norm_w, float norm_eps, T* __restrict__ out,
                             float* __restrict__ o_raw, int heads, int d, int P, int rows_pp, int* err) {
    // gridDim.z > 1: a head's columns are cut into that many blocks, a CTA each (columns do not talk to one
    // another, so a long prompt's heads spread over more SMs); the read-out then goes unnormed to `o_raw`
    // [rows, heads * d] (float), and `delta_rule_finish` norms and gates it.
    constexpr int SEG = SPLIT_ROWS + 8;
    extern __shared__ __align__(16) float sm[];
    const int VS = P * SEG;                               // floats of one vector
    float* vec = sm;                                      // [TT][5][VS]  r, k, w, a u, u
    float* val = vec + TT * 5 * VS;                       // [TT][d]  v
    float* gat = val + TT * d;                            // [TT][d]  gate, before its sigmoid
    float* o_s = gat + TT * d;                            // [TT][d]
    pdl_launch_dependents();
    if (rows_pp < SPLIT_ROWS)                             // the rows that pad a part stay zero
        for (int i = threadIdx.x; i < TT * 5 * VS; i += blockDim.x) vec[i] = 0.f;
    pdl_wait();
    const int e = blockIdx.x, h = blockIdx.y;
    const int first = cu_q[e], n = cu_q[e + 1] - first;
    if (n <= 0) return;                                  // an entry that pads the step: no slot is touched
    const int slot = slots[e];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_SLOT_RANGE);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int cpw = 32 / P;
    const int part = lane / cpw;
    const int col_end = (d / (int)gridDim.z) * ((int)blockIdx.z + 1);                // (d is a multiple of gridDim.z)
    const int j0 = (d / (int)gridDim.z) * (int)blockIdx.z + warp * COLS * cpw + lane % cpw;   // column c of this lane is j0 + c * cpw
    const int row0 = part * rows_pp;
    const int hd = heads * d;
    float* S_g = state + ((long long)slot * heads + h) * d * d;
    const bool fresh = kv_len[e] - n == 0;               // the request's first tokens: the state starts at zero
    float S[COLS][SPLIT_ROWS];
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
        for (int r = 0; r < SPLIT_ROWS; ++r)
            S[c][r] = (!fresh && j0 + c * cpw < col_end && r < rows_pp && row0 + r < d) ? S_g[(row0 + r) * d + j0 + c * cpw] : 0.f;
    for (int t0 = 0; t0 < n; t0 += TT) {
        const int nt = min(TT, n - t0);
        __syncthreads();                                 // the tile before has been read out
        for (int tt = warp; tt < nt; tt += nwarps) {
            const long long row = (long long)(first + t0 + tt);
            const long long pb = row * cols + h * d;
            const float* ax = aux + row * 3 * hd + h * d;
            float* v5 = vec + tt * 5 * VS;
            // (d <= 128: at most four columns a lane.  Every load goes out before the first value is stored:
            // the loads are unconditional, from a column that exists, and without the branch on the
            // product's form between them, or each would wait for the one before.)
            float t[4][7];
            if (proj.parts == nullptr) {
                const T* pw = proj.whole + pb;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = lane + 32 * i < d ? lane + 32 * i : 0;
                    t[i][0] = to_f32(pw[c]);
                    t[i][1] = to_f32(pw[hd + c]);
                    t[i][2] = ax[c];
                    t[i][3] = ax[hd + c];
                    t[i][4] = ax[2 * hd + c];
                    t[i][5] = to_f32(pw[2 * hd + c]);
                    t[i][6] = to_f32(pw[3 * hd + c]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = lane + 32 * i < d ? lane + 32 * i : 0;
                    t[i][0] = proj.load(pb + c);
                    t[i][1] = proj.load(pb + hd + c);
                    t[i][2] = ax[c];
                    t[i][3] = ax[hd + c];
                    t[i][4] = ax[2 * hd + c];
                    t[i][5] = proj.load(pb + 2 * hd + c);
                    t[i][6] = proj.load(pb + 3 * hd + c);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = lane + 32 * i;
                if (c < d) {
                    const int at = (c / rows_pp) * SEG + c % rows_pp;
                    v5[at] = t[i][0];                             // r
                    v5[VS + at] = t[i][1];                        // k
                    v5[2 * VS + at] = t[i][2];                    // w
                    v5[3 * VS + at] = t[i][3];                    // a u
                    v5[4 * VS + at] = t[i][4];                    // u
                    val[tt * d + c] = t[i][5];
                    gat[tt * d + c] = t[i][6];
                }
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float* base = vec + tt * 5 * VS + part * SEG;
            float v[COLS], dot[COLS], po[COLS];
#pragma unroll
            for (int c = 0; c < COLS; ++c) {
                v[c] = j0 + c * cpw < col_end ? val[tt * d + j0 + c * cpw] : 0.f;
                dot[c] = 0.f;
                po[c] = 0.f;
            }
#pragma unroll
            for (int q4 = 0; q4 < SPLIT_ROWS / 4; ++q4) {
                const float4 uu = *(const float4*)(base + 4 * VS + 4 * q4);
#pragma unroll
                for (int c = 0; c < COLS; ++c)
                    dot[c] += (uu.x * S[c][4 * q4] + uu.y * S[c][4 * q4 + 1]) + (uu.z * S[c][4 * q4 + 2] + uu.w * S[c][4 * q4 + 3]);
            }
            for (int o = cpw; o < 32; o <<= 1)
#pragma unroll
                for (int c = 0; c < COLS; ++c) dot[c] += __shfl_xor_sync(0xffffffffu, dot[c], o);
#pragma unroll
            for (int q4 = 0; q4 < SPLIT_ROWS / 4; ++q4) {
                const float4 rr = *(const float4*)(base + 4 * q4);
                const float4 kk = *(const float4*)(base + VS + 4 * q4);
                const float4 ww = *(const float4*)(base + 2 * VS + 4 * q4);
                const float4 aa = *(const float4*)(base + 3 * VS + 4 * q4);
                const int r = 4 * q4;
#pragma unroll
                for (int c = 0; c < COLS; ++c) {
                    S[c][r] = fmaf(ww.x, S[c][r], fmaf(-aa.x, dot[c], kk.x * v[c]));
                    S[c][r + 1] = fmaf(ww.y, S[c][r + 1], fmaf(-aa.y, dot[c], kk.y * v[c]));
                    S[c][r + 2] = fmaf(ww.z, S[c][r + 2], fmaf(-aa.z, dot[c], kk.z * v[c]));
                    S[c][r + 3] = fmaf(ww.w, S[c][r + 3], fmaf(-aa.w, dot[c], kk.w * v[c]));
                    po[c] += (rr.x * S[c][r] + rr.y * S[c][r + 1]) + (rr.z * S[c][r + 2] + rr.w * S[c][r + 3]);
                }
            }
            for (int o = cpw; o < 32; o <<= 1)
#pragma unroll
                for (int c = 0; c < COLS; ++c) po[c] += __shfl_xor_sync(0xffffffffu, po[c], o);
            if (part == 0) {
#pragma unroll
                for (int c = 0; c < COLS; ++c)
                    if (j0 + c * cpw < col_end) {
                        if (o_raw != nullptr) o_raw[(long long)(first + t0 + tt) * hd + h * d + j0 + c * cpw] = po[c];
                        else o_s[tt * d + j0 + c * cpw] = po[c];
                    }
            }
        }
        __syncthreads();
        if (o_raw != nullptr) continue;
        for (int tt = warp; tt < nt; tt += nwarps) {
            float ss = 0.f;
            for (int c = lane; c < d; c += 32) { const float x = o_s[tt * d + c]; ss += x * x; }
            ss = warp_sum(ss);
            const float rs = rsqrtf(ss / (float)d + norm_eps);
            T* op = out + (long long)(first + t0 + tt) * hd + h * d;
            for (int c = lane; c < d; c += 32) {
                const float g = 1.f / (1.f + expf(-gat[tt * d + c]));
                op[c] = from_f32<T>(o_s[tt * d + c] * rs * norm_w[h * d + c] * g);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
        for (int r = 0; r < SPLIT_ROWS; ++r)
            if (j0 + c * cpw < col_end && r < rows_pp && row0 + r < d) S_g[(row0 + r) * d + j0 + c * cpw] = S[c][r];
}

template <typename T, int SPLIT_ROWS, int COLS, int MAX_THREADS, int MIN_CTAS>
int launch_scan_split(GemmOut<T> proj, int cols, const float* aux, const int* cu_q, const int* kv_len,
                      const int* slots, int n_slots, float* state, const float* norm_w, float norm_eps, T* out,
                      float* o_raw, int col_blocks, int n_entries, int heads, int d, int* err, cudaStream_t st) {
    constexpr int SEG = SPLIT_ROWS + 8;
    int P = 1;
    while (P * SPLIT_ROWS < d) P *= 2;                   // 1, 2 or 4 (up to 16 with 4 rows a lane)
    const int rows_pp = (d + P - 1) / P, cpw = 32 / P;
    const int warps = (d / col_blocks + COLS * cpw - 1) / (COLS * cpw);
    const size_t smem = (size_t)(TT * 5 * P * SEG + 3 * TT * d) * sizeof(float);
    auto kern = delta_rule_scan_split_kernel<T, SPLIT_ROWS, COLS, MAX_THREADS, MIN_CTAS>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return crane_launch(kern, dim3(n_entries, heads, col_blocks), dim3(warps * 32), smem, st, proj, cols, aux, cu_q,
                        kv_len, slots, n_slots, state, norm_w, norm_eps, out, col_blocks > 1 ? o_raw : nullptr, heads, d,
                        P, rows_pp, err);
}

// out = o_raw / rms over the head * norm_w * sigmoid(gate): a warp per (row, head); the gate is column
// block 3 of the row's merged product.  Rows of no entry are skipped.
template <typename T>
__global__ void __launch_bounds__(256)
delta_rule_finish_kernel(const float* __restrict__ o_raw, GemmOut<T> proj, int cols, const int* __restrict__ tok_entry,
                         const float* __restrict__ norm_w, float norm_eps, T* __restrict__ out, int n_rows, int heads,
                         int d) {
    pdl_launch_dependents();
    pdl_wait();
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (long long)n_rows * heads) return;
    const int t = (int)(w / heads), h = (int)(w % heads);
    if (tok_entry[t] < 0) return;
    const int hd = heads * d;
    const float* o = o_raw + (long long)t * hd + h * d;
    float ss = 0.f;
    for (int c = lane; c < d; c += 32) ss += o[c] * o[c];
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / (float)d + norm_eps);
    for (int c = lane; c < d; c += 32) {
        const float g = 1.f / (1.f + expf(-proj.load((long long)t * cols + 3 * hd + h * d + c)));
        out[(long long)t * hd + h * d + c] = from_f32<T>(o[c] * rs * norm_w[h * d + c] * g);
    }
}

template <typename T, int DK>
int launch_scan(GemmOut<T> proj, int cols, const float* aux, const int* cu_q, const int* kv_len, const int* slots,
                int n_slots, float* state, const float* norm_w, float norm_eps, T* out, int n_entries, int heads,
                int d, int* err, cudaStream_t st) {
    size_t smem = (size_t)(TT * 8 * d) * sizeof(float);
    if (DK == 0) smem += (size_t)d * d * sizeof(float);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(delta_rule_scan_kernel<T, DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int threads = (d + 31) / 32 * 32;
    return crane_launch(delta_rule_scan_kernel<T, DK>, dim3(n_entries, heads), dim3(threads < 64 ? 64 : threads), smem,
                        st, proj, cols, aux, cu_q, kv_len, slots, n_slots, state, norm_w, norm_eps, out, heads, d, err);
}

template <typename T>
int scan_dispatch(GemmOut<T> g, int cols, const float* aux, const int* cu_q, const int* kv_len, const int* slots,
                  int n_slots, float* state, const float* norm_w, float norm_eps, T* out, float* o_raw,
                  const int* tok_entry, int n_rows, int col_blocks, int n_entries, int heads, int d, int* err,
                  cudaStream_t st) {
#define SPLIT(ROWS, COLS, THREADS, CTAS, BLOCKS)                                                                   \
    return launch_scan_split<T, ROWS, COLS, THREADS, CTAS>(g, cols, aux, cu_q, kv_len, slots, n_slots, state, norm_w, \
                                                          norm_eps, out, o_raw, BLOCKS, n_entries, heads, d, err, st)
    int lanes4 = 1;                                      // lanes a column takes with 4 rows a lane
    while (lanes4 * 4 < d) lanes4 *= 2;
    const bool fits = lanes4 <= 32 && (d / (col_blocks > 0 ? col_blocks : 1) + 32 / lanes4 - 1) / (32 / lanes4) <= 8;
    if (col_blocks > 1 && o_raw != nullptr && d <= 64 && d % col_blocks == 0 && fits) {
        // Few, long entries: a head's columns over `col_blocks` CTAs with 4 rows of a column a lane (the chain of
        // instructions per token is the shortest that way, and the CTAs are small enough to share an SM's
        // schedulers with little waiting), then the norm and the gate in a kernel of their own.
        const int rc = [&]() -> int { SPLIT(4, 1, 256, 2, col_blocks); }();
        if (rc != 0) return rc;
        const long long warps = (long long)n_rows * heads;
        return crane_launch(delta_rule_finish_kernel<T>, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, st,
                            (const float*)o_raw, g, cols, tok_entry, norm_w, norm_eps, out, n_rows, heads, d);
    }
    if (d <= 32) SPLIT(16, 1, 64, 8, 1);
    // (measured on one prompt of 2,048 tokens, 32 heads of 64, a CTA a head: 8 or 4 rows a lane, two or four
    // columns a lane and further warps that fetch the next tile while this one runs all took as long or longer)
    if (d <= 64) SPLIT(16, 1, 256, 2, 1);
    if (d <= 128) SPLIT(32, 2, 256, 1, 1);
#undef SPLIT
    return launch_scan<T, 0>(g, cols, aux, cu_q, kv_len, slots, n_slots, state, norm_w, norm_eps, out, n_entries,
                             heads, d, err, st);
}

}  // namespace

CRANE_API int crane_projection_norm_cache(int dtype, const void* qkv, const float* qkv_parts, int n_parts,
                                          long long part_stride, int cols, const int* positions,
                                          const int* tok_entry, const int* block_table, int max_blocks,
                                          int num_pages, int page_size, const float* qw, const float* kw,
                                          float eps, void* q_out, void* k_pool, void* v_pool, int n_tokens,
                                          int nq, int nkv, int d, int dv, int d_store, int dv_store,
                                          const float* cos_tab, const float* sin_tab, int n_positions,
                                          int rot_dims, const float* q_head_scale, int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (d_store < d || dv_store < dv) return (int)cudaErrorInvalidValue;
    if (cos_tab != nullptr && (rot_dims < 0 || rot_dims > d || rot_dims % 2 || sin_tab == nullptr))
        return (int)cudaErrorInvalidValue;
    DISPATCH_T(dtype, {
        GemmOut<T> g{(const T*)qkv, qkv_parts, n_parts, part_stride};
        return crane_launch(projection_norm_cache_kernel<T>, dim3(n_tokens), dim3(256), 0, st, g, cols, positions,
                            tok_entry, block_table, max_blocks, num_pages, page_size, qw, kw, eps, (T*)q_out,
                            (T*)k_pool, (T*)v_pool, nq, nkv, d, dv, d_store, dv_store, cos_tab, sin_tab,
                            n_positions, rot_dims, q_head_scale, err);
    });
}

CRANE_API int crane_delta_rule_prep(int dtype, const void* proj, const float* proj_parts, int n_parts,
                                    long long part_stride, int cols, const int* tok_entry, const void* w2t,
                                    const float* w0, const float* ab, float* aux, int n_tokens, int heads,
                                    int d, int rank, float decay_scale, float key_eps, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    const int hpc = d >= 256 ? 1 : (256 / d < heads ? 256 / d : heads);
    const int group = n_tokens <= 64 ? 1 : 8;
    const size_t smem = (size_t)(group * (rank + hpc)) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const dim3 grid((n_tokens + group - 1) / group, (heads + hpc - 1) / hpc);
    DISPATCH_T(dtype, {
        GemmOut<T> g{(const T*)proj, proj_parts, n_parts, part_stride};
        if (group == 1)
            return crane_launch(delta_rule_prep_kernel<T, 1>, grid, dim3(256), smem, st, g, cols, tok_entry,
                                (const T*)w2t, w0, ab, aux, n_tokens, heads, d, rank, hpc, decay_scale, key_eps);
        return crane_launch(delta_rule_prep_kernel<T, 8>, grid, dim3(256), smem, st, g, cols, tok_entry,
                            (const T*)w2t, w0, ab, aux, n_tokens, heads, d, rank, hpc, decay_scale, key_eps);
    });
}

// The widest head the recurrence takes: its state and a tile of vectors must fit shared memory.
CRANE_API int crane_delta_rule_max_dim() {
    int d = 16;
    while ((size_t)(TT * 8 * (d + 1) + (d + 1) * (d + 1)) * sizeof(float) <= 227 * 1024) ++d;
    return d;
}

CRANE_API int crane_delta_rule_scan(int dtype, const void* proj, const float* proj_parts, int n_parts,
                                    long long part_stride, int cols, const float* aux, const int* cu_q,
                                    const int* kv_len, const int* slots, int n_slots, float* state,
                                    const float* norm_w, float norm_eps, void* out, float* o_raw,
                                    const int* tok_entry, int n_rows, int col_blocks, int n_entries, int heads,
                                    int d, int* err, cudaStream_t st) {
    if (n_entries <= 0) return 0;
    if (d <= 0 || d > 1024) return (int)cudaErrorInvalidValue;
    DISPATCH_T(dtype, {
        GemmOut<T> g{(const T*)proj, proj_parts, n_parts, part_stride};
        return scan_dispatch<T>(g, cols, aux, cu_q, kv_len, slots, n_slots, state, norm_w, norm_eps, (T*)out, o_raw,
                                tok_entry, n_rows, col_blocks, n_entries, heads, d, err, st);
    });
}
