// Attention over the paged cache in bf16 whose scores are worked on before they become weights, on
// the warp-level tensor-core tiles of attention_mma.cuh.  What can happen to a score s = q . k * scale:
//   * squashed: s <- cap * tanh(s / cap);
//   * visibility: key j is seen from position p when j <= p, j > p - window (window > 0), and j lies in
//     p's own block of `chunk` positions (chunk > 0; blocks are counted from position 0 of the request);
//   * weights: softmax over the visible keys, or sigmoid(s + bias of the head) for every visible key with
//     no normalisation over the keys at all;
//   * MAPS == 2 (differential attention): a head's query and key rows hold two maps, the leading and the
//     trailing D / 2 elements; each is a softmax attention of its own over the same values, and the head's
//     result is o = a1 - lambda a2.
// Behind the weighted sums, in the same kernel: o over the root of its mean square over the head's
// `dv` values times a constant, and times a gate per (token, head).
//
// Two kernels.  `scored_prefill_attn`: one CTA per tile of 64 query rows of one request and one query
// head, four warps of 16 rows, keys and values in tiles of 64 through shared memory (two stages);
// portions cut anywhere, whole prompts and single tokens are the same case.  `scored_decode_attn`: the
// entries of exactly one token, split along the keys: one CTA per (slice of the keys, key/value head,
// request), the query heads that share the key/value head in the rows of one MMA tile, each warp with its
// own ring of three 32-key tiles (two with two maps); every slice leaves (max, sum, unnormalised sums) per head and map in
// scratch memory, and `scored_decode_merge` merges the slices and finishes the head.
#include "attention_mma.cuh"

namespace {
using namespace attn;

struct ScoreArgs {
    float softcap, inv_softcap;     // 0: the score is not squashed
    int chunk;                      // 0: no blocks
    int sigmoid;                    // weights sigmoid(s + head_bias[h]) without normalisation
    const float* head_bias;         // [nq] or null
    float lam;                      // MAPS == 2: o = a1 - lam a2
    int head_norm;                  // o over the root of its mean square over dv values, times norm_scale
    float norm_scale, eps;
    const float* gate;              // float [rows][nq] or null
    int dv;                         // the width of a value row that is real (the rest of D is zero)
    int compact;                    // out rows are [nq][dv] instead of [nq][D]
};

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float squash(float s, const ScoreArgs& a) {
    if (a.softcap <= 0.f) return s;
    // cap * tanh(s / cap), tanh(x) = 1 - 2 / (exp(2x) + 1)
    const float e = __expf(2.f * s * a.inv_softcap);
    return a.softcap * (1.f - __fdividef(2.f, e + 1.f));
}
// the first key position that position p sees
__device__ __forceinline__ int first_visible(int p, int window, int chunk) {
    int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    if (chunk > 0) lo = max(lo, p / chunk * chunk);
    return lo;
}

// ------------------------------------------------------------------ portions
constexpr int BQ = 64, BKV = 64, PWARPS = 4, PTHREADS = PWARPS * 32;

template <int D, int MAPS>
__global__ void __launch_bounds__(PTHREADS, MAPS == 2 ? (D > 64 ? 1 : 2) : 3)
scored_prefill_attn_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                           const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                           const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                           const int* __restrict__ block_table, int max_blocks, int num_pages, int page_size,
                           int n_entries, int nq, int nkv, int window, float scale, int skip_single,
                           const ScoreArgs sa, int* err) {
    constexpr int RB = Tile<D>::ROW_BYTES;
    constexpr int TILE_BYTES = BKV * RB;
    constexpr int KS = D / 16, DN = D / 8, KSM = KS / MAPS;
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_launch_dependents();
    pdl_wait();

    // which request and which of its query tiles: a request's last tiles (the longest) come first
    int e = 0, tile = blockIdx.y;
    for (; e < n_entries; ++e) {
        const int rows = cu_q[e + 1] - cu_q[e];
        const int tiles = (skip_single && rows == 1) ? 0 : (rows + BQ - 1) / BQ;
        if (tile < tiles) {
            tile = tiles - 1 - tile;
            break;
        }
        tile -= tiles;
    }
    if (e >= n_entries) return;
    const int h = blockIdx.x, g = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = cu_q[e], q_len = cu_q[e + 1] - row0;
    const int pos0 = kv_len[e] - q_len;
    const int r_begin = tile * BQ, r_end = min(q_len, r_begin + BQ);
    const int* table = block_table + (long long)e * max_blocks;

    const int ra = r_begin + warp * 16 + (lane >> 2), rb = ra + 8;
    const int pa = pos0 + ra, pb = pos0 + rb;
    const int la = first_visible(pa, window, sa.chunk), lb = first_visible(pb, window, sa.chunk);
    uint32_t qf[KS][4];
    {
        const int c0 = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = (i & 1) ? rb : ra, c = ks * 16 + c0 + (i >> 1) * 8;
                qf[ks][i] = r < r_end ? *(const uint32_t*)(q + ((long long)(row0 + r) * nq + h) * D + c) : 0u;
            }
    }
    float o[MAPS][DN][4];
    float m[MAPS][2], l[MAPS][2];
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
#pragma unroll
        for (int i = 0; i < DN; ++i) o[mp][i][0] = o[mp][i][1] = o[mp][i][2] = o[mp][i][3] = 0.f;
        m[mp][0] = m[mp][1] = -INFINITY;
        l[mp][0] = l[mp][1] = 0.f;
    }
    bool bad_page = false;
    const float bias = (sa.sigmoid && sa.head_bias != nullptr) ? sa.head_bias[h] : 0.f;

    // keys that any row of the CTA reads (the first visible key does not fall as the position grows)
    const int p_first = pos0 + r_begin, p_last = pos0 + r_end - 1;
    const int lo = first_visible(p_first, window, sa.chunk);
    const int t_begin = lo / BKV, t_end = p_last / BKV + 1;
    const int wp_first = pos0 + r_begin + warp * 16;
    const int wp_last = min(p_last, wp_first + 15);
    const int w_lo = first_visible(min(wp_first, p_last), window, sa.chunk);

    const uint32_t sbase = smem_u32(smem);
    load_tile_async<D, BKV, PTHREADS>(sbase, k_pool, table, num_pages, page_size, nkv, g, t_begin * BKV, lo, p_last,
                                      threadIdx.x, bad_page);
    load_tile_async<D, BKV, PTHREADS>(sbase + TILE_BYTES, v_pool, table, num_pages, page_size, nkv, g, t_begin * BKV,
                                      lo, p_last, threadIdx.x, bad_page);
    cp_async_commit();
    for (int ti = t_begin, it = 0; ti < t_end; ++ti, ++it) {
        const uint32_t kt = sbase + (it & 1) * 2 * TILE_BYTES, vt = kt + TILE_BYTES;
        if (ti + 1 < t_end) {
            const uint32_t nk = sbase + ((it + 1) & 1) * 2 * TILE_BYTES;
            load_tile_async<D, BKV, PTHREADS>(nk, k_pool, table, num_pages, page_size, nkv, g, (ti + 1) * BKV, lo,
                                              p_last, threadIdx.x, bad_page);
            load_tile_async<D, BKV, PTHREADS>(nk + TILE_BYTES, v_pool, table, num_pages, page_size, nkv, g,
                                              (ti + 1) * BKV, lo, p_last, threadIdx.x, bad_page);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const int key_base = ti * BKV;
        // a warp skips tiles that lie wholly behind its last row or before what its first row sees
        const bool skip = key_base > wp_last || key_base + BKV - 1 < w_lo || wp_first > p_last;
        if (!skip) {
            const int mi = lane >> 3, mr = lane & 7;
            const int key0 = key_base + (lane & 3) * 2;
#pragma unroll
            for (int mp = 0; mp < MAPS; ++mp) {
                float s[8][4];
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
                for (int ks = mp * KSM; ks < (mp + 1) * KSM; ++ks) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const int key = q4 * 16 + (mi >> 1) * 8 + mr;
                        const int chunk = ks * 2 + (mi & 1);
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(kt + key * RB + chunk * 16, b0, b1, b2, b3);
                        mma_bf16(s[q4 * 2], qf[ks], b0, b1);
                        mma_bf16(s[q4 * 2 + 1], qf[ks], b2, b3);
                    }
                }
                if (sa.sigmoid) {
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int j = key0 + nt * 8 + (c & 1);
                            const bool ok = (c >> 1) ? (j <= pb && j >= lb) : (j <= pa && j >= la);
                            const float v = squash(s[nt][c] * scale, sa) + bias;
                            s[nt][c] = ok ? __fdividef(1.f, 1.f + exp2f(-v * LOG2E)) : 0.f;
                        }
                } else {
                    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int j = key0 + nt * 8 + (c & 1);
                            const bool ok = (c >> 1) ? (j <= pb && j >= lb) : (j <= pa && j >= la);
                            const float v = ok ? squash(s[nt][c] * scale, sa) * LOG2E : -INFINITY;
                            s[nt][c] = v;
                            mx[c >> 1] = fmaxf(mx[c >> 1], v);
                        }
                    float corr[2], base[2];
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const float m_new = fmaxf(m[mp][hh], quad_max(mx[hh]));
                        base[hh] = (m_new == -INFINITY) ? 0.f : m_new;
                        corr[hh] = exp2f(m[mp][hh] - base[hh]);
                        m[mp][hh] = m_new;
                    }
                    float rs[2] = {0.f, 0.f};
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float p = exp2f(s[nt][c] - base[c >> 1]);
                            s[nt][c] = p;
                            rs[c >> 1] += p;
                        }
                    l[mp][0] = l[mp][0] * corr[0] + rs[0];
                    l[mp][1] = l[mp][1] * corr[1] + rs[1];
#pragma unroll
                    for (int i = 0; i < DN; ++i) {
                        o[mp][i][0] *= corr[0]; o[mp][i][1] *= corr[0];
                        o[mp][i][2] *= corr[1]; o[mp][i][3] *= corr[1];
                    }
                }
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    uint32_t pf[4];
                    pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                    pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                    pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                    pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                    for (int dn = 0; dn < DN; dn += 2) {
                        const int key = kk * 16 + (mi & 1) * 8 + mr;
                        const int chunk = dn + (mi >> 1);
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4_trans(vt + key * RB + chunk * 16, b0, b1, b2, b3);
                        mma_bf16(o[mp][dn], pf, b0, b1);
                        mma_bf16(o[mp][dn + 1], pf, b2, b3);
                    }
                }
            }
        }
        __syncthreads();                             // the stage may be overwritten now
    }
    cp_async_wait<0>();
    if (__any_sync(0xffffffffu, bad_page) && lane == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
    float inv[MAPS][2];
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const float L = quad_sum(l[mp][hh]);
            inv[mp][hh] = sa.sigmoid ? 1.f : L > 0.f ? 1.f / L : 0.f;
        }
    // the head's result in o[0]: a1 - lam a2 for two maps
    float ss[2] = {0.f, 0.f};
#pragma unroll
    for (int dn = 0; dn < DN; ++dn)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float v = o[0][dn][c] * inv[0][c >> 1];
            if (MAPS == 2) v -= sa.lam * (o[MAPS - 1][dn][c] * inv[MAPS - 1][c >> 1]);
            o[0][dn][c] = v;
            ss[c >> 1] = fmaf(v, v, ss[c >> 1]);
        }
    float fa = 1.f, fb = 1.f;
    if (sa.head_norm) {
        fa = rsqrtf(quad_sum(ss[0]) / (float)sa.dv + sa.eps) * sa.norm_scale;
        fb = rsqrtf(quad_sum(ss[1]) / (float)sa.dv + sa.eps) * sa.norm_scale;
    }
    if (sa.gate != nullptr) {
        if (ra < r_end) fa *= sa.gate[(long long)(row0 + ra) * nq + h];
        if (rb < r_end) fb *= sa.gate[(long long)(row0 + rb) * nq + h];
    }
    const int c0 = (lane & 3) * 2;
    if (sa.compact) {
        const int dv = sa.dv;
#pragma unroll
        for (int dn = 0; dn < DN; ++dn)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int r = (c >> 1) ? rb : ra, col = dn * 8 + c0 + (c & 1);
                if (r < r_end && col < dv)
                    out[((long long)(row0 + r) * nq + h) * dv + col] = __float2bfloat16_rn(o[0][dn][c] * ((c >> 1) ? fb : fa));
            }
        return;
    }
#pragma unroll
    for (int dn = 0; dn < DN; ++dn) {
        if (ra < r_end)
            *(uint32_t*)(out + ((long long)(row0 + ra) * nq + h) * D + dn * 8 + c0) =
                pack_bf16(o[0][dn][0] * fa, o[0][dn][1] * fa);
        if (rb < r_end)
            *(uint32_t*)(out + ((long long)(row0 + rb) * nq + h) * D + dn * 8 + c0) =
                pack_bf16(o[0][dn][2] * fb, o[0][dn][3] * fb);
    }
}

// ------------------------------------------------------------------ single tokens, split along the keys
constexpr int TILE = 32, DWARPS = 2;
// tile stages per warp: with two maps a tile costs half as much again to work through, and two stages let a
// third CTA move in on the SM
template <int MAPS> constexpr int stages_of() { return MAPS == 2 ? 2 : 3; }

// part_o [entry][head][map][slice][D], part_ml [entry][head][map][slice][2] (max in base 2, sum)
template <int D, int MAPS>
__global__ void __launch_bounds__(DWARPS * 32)
scored_decode_attn_kernel(const __nv_bfloat16* __restrict__ q, float* __restrict__ part_o,
                          float* __restrict__ part_ml, const __nv_bfloat16* __restrict__ k_pool,
                          const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ cu_q,
                          const int* __restrict__ kv_len, const int* __restrict__ block_table, int max_blocks,
                          int num_pages, int page_size, int nq, int nkv, int window, float scale, int n_splits,
                          const ScoreArgs sa, int* err) {
    constexpr int RB = Tile<D>::ROW_BYTES;
    constexpr int TILE_BYTES = TILE * RB;
    constexpr int KS = D / 16, DN = D / 8, KSM = KS / MAPS;
    constexpr int NSTAGE = stages_of<MAPS>();
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int split = blockIdx.x, g = blockIdx.y, e = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_rep = nq / nkv;
    const int t = cu_q[e];
    if (cu_q[e + 1] - t != 1) return;               // a portion, or an entry without rows: not this kernel's
    const int pos = kv_len[e] - 1;
    const int lo = first_visible(pos, window, sa.chunk);
    const int* table = block_table + (long long)e * max_blocks;

    const int first_tile = lo / TILE;
    const int n_tiles = pos / TILE - first_tile + 1;
    const int per_split = (n_tiles + n_splits - 1) / n_splits;
    const int tile_begin = first_tile + split * per_split;
    const int tile_end = min(first_tile + n_tiles, tile_begin + per_split);
    const uint32_t wbase = smem_u32(smem) + warp * NSTAGE * 2 * TILE_BYTES;
    bool bad_page = false;

    int ti = tile_begin + warp;
#pragma unroll
    for (int s = 0; s < NSTAGE - 1; ++s) {
        const int tj = ti + s * DWARPS;
        if (tj < tile_end) {
            const uint32_t st = wbase + s * 2 * TILE_BYTES;
            load_tile_async<D, TILE>(st, k_pool, table, num_pages, page_size, nkv, g, tj * TILE, lo, pos, lane, bad_page);
            load_tile_async<D, TILE>(st + TILE_BYTES, v_pool, table, num_pages, page_size, nkv, g, tj * TILE, lo, pos,
                                     lane, bad_page);
        }
        cp_async_commit();
    }
    // query rows: row r of the MMA tile is query head g * n_rep + r
    uint32_t qf[KS][4];
    float bias[2] = {0.f, 0.f};
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = r0 + (i & 1) * 8, c = ks * 16 + c0 + (i >> 1) * 8;
                qf[ks][i] = r < n_rep ? *(const uint32_t*)(q + ((long long)t * nq + g * n_rep + r) * D + c) : 0u;
            }
        if (sa.sigmoid && sa.head_bias != nullptr) {
            if (r0 < n_rep) bias[0] = sa.head_bias[g * n_rep + r0];
            if (r0 + 8 < n_rep) bias[1] = sa.head_bias[g * n_rep + r0 + 8];
        }
    }
    float o[MAPS][DN][4];
    float m[MAPS][2], l[MAPS][2];
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
#pragma unroll
        for (int i = 0; i < DN; ++i) o[mp][i][0] = o[mp][i][1] = o[mp][i][2] = o[mp][i][3] = 0.f;
        m[mp][0] = m[mp][1] = -INFINITY;
        l[mp][0] = l[mp][1] = 0.f;
    }
    for (int it = 0; ti < tile_end; ti += DWARPS, ++it) {
        const uint32_t kt = wbase + (it % NSTAGE) * 2 * TILE_BYTES, vt = kt + TILE_BYTES;
        const int nxt = ti + (NSTAGE - 1) * DWARPS;
        if (nxt < tile_end) {
            const uint32_t nk = wbase + ((it + NSTAGE - 1) % NSTAGE) * 2 * TILE_BYTES;
            load_tile_async<D, TILE>(nk, k_pool, table, num_pages, page_size, nkv, g, nxt * TILE, lo, pos, lane, bad_page);
            load_tile_async<D, TILE>(nk + TILE_BYTES, v_pool, table, num_pages, page_size, nkv, g, nxt * TILE, lo, pos,
                                     lane, bad_page);
        }
        cp_async_commit();
        cp_async_wait<NSTAGE - 1>();
        __syncwarp();
        const int mi = lane >> 3, mr = lane & 7;
        const int key0 = ti * TILE + (lane & 3) * 2;
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            float s[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int ks = mp * KSM; ks < (mp + 1) * KSM; ++ks) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int key = half * 16 + (mi >> 1) * 8 + mr;
                    const int chunk = ks * 2 + (mi & 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(kt + key * RB + chunk * 16, b0, b1, b2, b3);
                    mma_bf16(s[half * 2], qf[ks], b0, b1);
                    mma_bf16(s[half * 2 + 1], qf[ks], b2, b3);
                }
            }
            if (sa.sigmoid) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = key0 + nt * 8 + (c & 1);
                        const float v = squash(s[nt][c] * scale, sa) + bias[c >> 1];
                        s[nt][c] = (j >= lo && j <= pos) ? __fdividef(1.f, 1.f + exp2f(-v * LOG2E)) : 0.f;
                    }
            } else {
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = key0 + nt * 8 + (c & 1);
                        const float v = (j >= lo && j <= pos) ? squash(s[nt][c] * scale, sa) * LOG2E : -INFINITY;
                        s[nt][c] = v;
                        mx[c >> 1] = fmaxf(mx[c >> 1], v);
                    }
                float corr[2], base[2];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const float m_new = fmaxf(m[mp][hh], quad_max(mx[hh]));
                    base[hh] = (m_new == -INFINITY) ? 0.f : m_new;
                    corr[hh] = exp2f(m[mp][hh] - base[hh]);
                    m[mp][hh] = m_new;
                }
                float rs[2] = {0.f, 0.f};
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float p = exp2f(s[nt][c] - base[c >> 1]);
                        s[nt][c] = p;
                        rs[c >> 1] += p;
                    }
                l[mp][0] = l[mp][0] * corr[0] + rs[0];
                l[mp][1] = l[mp][1] * corr[1] + rs[1];
#pragma unroll
                for (int i = 0; i < DN; ++i) {
                    o[mp][i][0] *= corr[0]; o[mp][i][1] *= corr[0];
                    o[mp][i][2] *= corr[1]; o[mp][i][3] *= corr[1];
                }
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                uint32_t pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dn = 0; dn < DN; dn += 2) {
                    const int key = kk * 16 + (mi & 1) * 8 + mr;
                    const int chunk = dn + (mi >> 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(vt + key * RB + chunk * 16, b0, b1, b2, b3);
                    mma_bf16(o[mp][dn], pf, b0, b1);
                    mma_bf16(o[mp][dn + 1], pf, b2, b3);
                }
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    if (__any_sync(0xffffffffu, bad_page) && lane == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);

    // ---- merge the warps, leave the slice's sums in scratch ----
    __syncthreads();
    float* sm_o = (float*)smem;                              // [DWARPS][MAPS][16][D]
    float* sm_ml = sm_o + DWARPS * MAPS * 16 * D;            // [DWARPS][MAPS][16][2]
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            const int wb = (warp * MAPS + mp) * 16;
#pragma unroll
            for (int dn = 0; dn < DN; ++dn) {
                float* p0 = sm_o + (wb + r0) * D + dn * 8 + c0;
                float* p1 = sm_o + (wb + r0 + 8) * D + dn * 8 + c0;
                p0[0] = o[mp][dn][0]; p0[1] = o[mp][dn][1];
                p1[0] = o[mp][dn][2]; p1[1] = o[mp][dn][3];
            }
            const float l0 = quad_sum(l[mp][0]), l1 = quad_sum(l[mp][1]);
            if ((lane & 3) == 0) {
                sm_ml[(wb + r0) * 2] = m[mp][0];      sm_ml[(wb + r0) * 2 + 1] = l0;
                sm_ml[(wb + r0 + 8) * 2] = m[mp][1];  sm_ml[(wb + r0 + 8) * 2 + 1] = l1;
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < MAPS * n_rep * D; idx += DWARPS * 32) {
        const int c = idx % D, r = (idx / D) % n_rep, mp = idx / (D * n_rep);
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DWARPS; ++w) M = fmaxf(M, sm_ml[((w * MAPS + mp) * 16 + r) * 2]);
        const float mb = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < DWARPS; ++w) {
            const int row = (w * MAPS + mp) * 16 + r;
            const float f = sa.sigmoid ? 1.f : exp2f(sm_ml[row * 2] - mb);
            L += f * sm_ml[row * 2 + 1];
            O += f * sm_o[row * D + c];
        }
        const long long pi = ((((long long)e * nq + g * n_rep + r) * MAPS + mp) * n_splits + split);
        part_o[pi * D + c] = O;
        if (c == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
    }
}

// One warp per (entry, query head): the slices of each map merged in slice order, then the head finished
// as in the kernel for portions.
template <int MAPS>
__global__ void __launch_bounds__(128)
scored_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                           __nv_bfloat16* __restrict__ out, const int* __restrict__ cu_q, int n_entries, int nq, int D,
                           int n_splits, const ScoreArgs sa) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int MAXC = 8;                                   // columns per lane: D <= 256
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)n_entries * nq) return;
    const int e = (int)(unit / nq), h = (int)(unit % nq);
    const int t = cu_q[e];
    if (cu_q[e + 1] - t != 1) return;
    float res[MAXC];
#pragma unroll
    for (int i = 0; i < MAXC; ++i) res[i] = 0.f;
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
        const long long p0 = (unit * MAPS + mp) * n_splits;
        float M = -INFINITY;
        for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(p0 + s) * 2]);
        const float mb = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, acc[MAXC];
#pragma unroll
        for (int i = 0; i < MAXC; ++i) acc[i] = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float f = sa.sigmoid ? 1.f : exp2f(part_ml[(p0 + s) * 2] - mb);
            L += f * part_ml[(p0 + s) * 2 + 1];
#pragma unroll
            for (int i = 0; i < MAXC; ++i) {
                const int c = lane + 32 * i;
                if (c < D) acc[i] = fmaf(f, part_o[(p0 + s) * D + c], acc[i]);
            }
        }
        const float inv = sa.sigmoid ? 1.f : L > 0.f ? 1.f / L : 0.f;
        const float sign = mp == 0 ? 1.f : -sa.lam;
#pragma unroll
        for (int i = 0; i < MAXC; ++i) res[i] = fmaf(sign, acc[i] * inv, res[i]);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) ss = fmaf(res[i], res[i], ss);      // columns beyond dv hold zeros
    float f = 1.f;
    if (sa.head_norm) f = rsqrtf(warp_sum(ss) / (float)sa.dv + sa.eps) * sa.norm_scale;
    if (sa.gate != nullptr) f *= sa.gate[(long long)t * nq + h];
    const int width = sa.compact ? sa.dv : D;
    __nv_bfloat16* op = out + ((long long)t * nq + h) * width;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
        const int c = lane + 32 * i;
        if (c < width) op[c] = __float2bfloat16_rn(res[i] * f);
    }
}

template <int D, int MAPS>
int launch_scored_prefill(const void* q, void* out, const void* k_pool, const void* v_pool, const int* cu_q,
                          const int* kv_len, const int* block_table, int max_blocks, int num_pages, int page_size,
                          int n_entries, int total_q_tiles, int nq, int nkv, int window, float scale, int skip_single,
                          const ScoreArgs& sa, int* err, cudaStream_t st) {
    constexpr int smem = 4 * BKV * Tile<D>::ROW_BYTES;
    auto kern = scored_prefill_attn_kernel<D, MAPS>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    return crane_launch(kern, dim3(nq, total_q_tiles), dim3(PTHREADS), smem, st, (const __nv_bfloat16*)q,
                        (__nv_bfloat16*)out, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, cu_q, kv_len,
                        block_table, max_blocks, num_pages, page_size, n_entries, nq, nkv, window, scale, skip_single,
                        sa, err);
}

template <int D, int MAPS>
int launch_scored_decode(const void* q, void* out, float* part_o, float* part_ml, const void* k_pool,
                         const void* v_pool, const int* cu_q, const int* kv_len, const int* block_table,
                         int max_blocks, int num_pages, int page_size, int n_entries, int nq, int nkv, int window,
                         float scale, int n_splits, const ScoreArgs& sa, int* err, cudaStream_t st) {
    constexpr int ring = DWARPS * stages_of<MAPS>() * 2 * TILE * Tile<D>::ROW_BYTES;
    constexpr int merge = DWARPS * MAPS * 16 * (D + 2) * (int)sizeof(float);
    constexpr int smem = ring > merge ? ring : merge;
    auto kern = scored_decode_attn_kernel<D, MAPS>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    int rc = crane_launch(kern, dim3(n_splits, nkv, n_entries), dim3(DWARPS * 32), smem, st, (const __nv_bfloat16*)q,
                          part_o, part_ml, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, cu_q, kv_len,
                          block_table, max_blocks, num_pages, page_size, nq, nkv, window, scale, n_splits, sa, err);
    if (rc != 0) return rc;
    const long long units = (long long)n_entries * nq;
    return crane_launch(scored_decode_merge_kernel<MAPS>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, st,
                        (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, cu_q, n_entries, nq, D,
                        n_splits, sa);
}
}  // namespace

// Every head size is compiled as an object of its own from this file (the build passes CRANE_HEAD_SIZE),
// side by side; the object without it holds the entry points.  Two maps need a head size whose halves
// are whole MMA steps (a multiple of 32) and, for the registers of two sets of sums, at most 128.
#define CRANE_CAT2(a, b) a##b
#define CRANE_CAT(a, b) CRANE_CAT2(a, b)
#define CRANE_SCORED_ARGS                                                                                  \
    int decode, int maps, const void *q, void *out, float *part_o, float *part_ml, const void *k_pool,       \
        const void *v_pool, const int *cu_q, const int *kv_len, const int *block_table, int max_blocks,      \
        int num_pages, int page_size, int n_entries, int total_q_tiles, int nq, int nkv, int window,         \
        float scale, int n_splits, int skip_single, const void *score_args, int *err, cudaStream_t st
#ifdef CRANE_HEAD_SIZE
template <int D>
int scored_launch(CRANE_SCORED_ARGS) {
    const ScoreArgs& sa = *(const ScoreArgs*)score_args;
    if (maps == 1) {
        if (decode)
            return launch_scored_decode<D, 1>(q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len, block_table,
                                              max_blocks, num_pages, page_size, n_entries, nq, nkv, window, scale,
                                              n_splits, sa, err, st);
        return launch_scored_prefill<D, 1>(q, out, k_pool, v_pool, cu_q, kv_len, block_table, max_blocks, num_pages,
                                           page_size, n_entries, total_q_tiles, nq, nkv, window, scale, skip_single,
                                           sa, err, st);
    }
    if constexpr (D % 32 == 0 && D <= 128) {
        if (decode)
            return launch_scored_decode<D, 2>(q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len, block_table,
                                              max_blocks, num_pages, page_size, n_entries, nq, nkv, window, scale,
                                              n_splits, sa, err, st);
        return launch_scored_prefill<D, 2>(q, out, k_pool, v_pool, cu_q, kv_len, block_table, max_blocks, num_pages,
                                           page_size, n_entries, total_q_tiles, nq, nkv, window, scale, skip_single,
                                           sa, err, st);
    }
    return (int)cudaErrorInvalidValue;
}
extern "C" int CRANE_CAT(crane_scored_launch_d, CRANE_HEAD_SIZE)(CRANE_SCORED_ARGS) {
    return scored_launch<CRANE_HEAD_SIZE>(decode, maps, q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len,
                                          block_table, max_blocks, num_pages, page_size, n_entries, total_q_tiles, nq,
                                          nkv, window, scale, n_splits, skip_single, score_args, err, st);
}
#else
#ifdef CRANE_HEAD_SIZE_LIST          // the head sizes linked into this library
#define CRANE_SCORED_HEAD_SIZES(X) CRANE_HEAD_SIZE_LIST(X)
#else
#define CRANE_SCORED_HEAD_SIZES(X) X(16) X(32) X(48) X(64) X(80) X(96) X(112) X(128) X(160) X(192) X(256)
#endif
#define DECLARE(DD) extern "C" int crane_scored_launch_d##DD(CRANE_SCORED_ARGS);
CRANE_SCORED_HEAD_SIZES(DECLARE)
#undef DECLARE

CRANE_API int crane_scored_attention_supports(int d, int nq, int nkv, int maps) {
    if (nkv <= 0 || nq % nkv != 0 || maps < 1 || maps > 2) return 0;
    if (maps == 2 && (d % 32 != 0 || d > 128)) return 0;
#define IS(DD) if (d == DD) return 1;
    CRANE_SCORED_HEAD_SIZES(IS)
#undef IS
    return 0;
}

// decode == 0: every entry (but, with skip_single, those of exactly one token) through the kernel for
// portions; total_q_tiles: sum over the entries of ceil(q_len / 64), or an upper bound.  decode != 0: the
// entries of exactly one token through the split-KV kernel and the merge; part_o holds
// entries * nq * maps * n_splits rows of d floats, part_ml as many pairs; at most 16 query heads per
// key/value head.  `out`: bf16 [rows][nq][d], or [rows][nq][dv] with `compact`.
CRANE_API int crane_scored_attention(int decode, int maps, const void* q, void* out, float* part_o, float* part_ml,
                                     const void* k_pool, const void* v_pool, const int* cu_q, const int* kv_len,
                                     const int* block_table, int max_blocks, int num_pages, int page_size,
                                     int n_entries, int total_q_tiles, int nq, int nkv, int d, int window, float scale,
                                     int n_splits, int skip_single, float softcap, int chunk, int sigmoid,
                                     const float* head_bias, float lam, int head_norm, float norm_scale, float eps,
                                     const float* gate, int dv, int compact, int* err, cudaStream_t st) {
    if (n_entries <= 0 || (!decode && total_q_tiles <= 0)) return 0;
    if (!crane_scored_attention_supports(d, nq, nkv, maps) || dv <= 0 || dv > d) return (int)cudaErrorInvalidValue;
    if (decode && (nq / nkv > 16 || part_o == nullptr || part_ml == nullptr || n_splits < 1))
        return (int)cudaErrorInvalidValue;
    ScoreArgs sa;
    sa.softcap = softcap; sa.inv_softcap = softcap > 0.f ? 1.f / softcap : 0.f; sa.chunk = chunk; sa.sigmoid = sigmoid;
    sa.head_bias = head_bias; sa.lam = lam; sa.head_norm = head_norm; sa.norm_scale = norm_scale; sa.eps = eps;
    sa.gate = gate; sa.dv = dv; sa.compact = compact;
#define CASE(DD)                                                                                              \
    case DD:                                                                                                  \
        return crane_scored_launch_d##DD(decode, maps, q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len,   \
                                         block_table, max_blocks, num_pages, page_size, n_entries,              \
                                         total_q_tiles, nq, nkv, window, scale, n_splits, skip_single, &sa, err, st);
    switch (d) { CRANE_SCORED_HEAD_SIZES(CASE) }
#undef CASE
    return (int)cudaErrorInvalidValue;
}
#endif  // CRANE_HEAD_SIZE
