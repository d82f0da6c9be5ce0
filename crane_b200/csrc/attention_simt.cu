// Attention over the paged cache on the FP32 cores, for any batch of prompt
// portions and single decoded tokens, any key width up to 1024 and any value
// width up to 512.  Values are rows of `dv` elements, `v_stride` elements apart,
// in `v_pool`: a pool of their own, or (v_pool == k_pool, v_stride == d) the
// leading dv columns of the key rows, which is how latent attention keeps them.
// One warp per (token, query head): the token at position p of
// request e attends the keys of positions max(0, p - window + 1) .. p of the
// same request, found through the request's block table.  Scores, softmax
// statistics and the weighted sum are float whatever the storage type.  `sink`: the
// softmax has one more candidate of score 0 and no value (p_j = exp(s_j) / (1 + sum exp(s))).
// `ScoreMod` says what happens to a score before it becomes a weight: squashed to cap * tanh(s / cap);
// keys seen only within the query's own block of `chunk` positions (blocks counted from position 0);
// weights sigmoid(s + bias of the head) that are not normalised over the keys instead of a softmax; a
// head of `maps` maps of d elements side by side in its query and key rows (rows of `d_row` elements, map
// i at i * d_map), each map an attention of its own over the same values; results in float
// [token][head][map][dv].
//
// scores = q k^T / sqrt(d), causal j <= p, softmax over the last dimension,
// query head h reads kv head h / (nq / nkv):
// crane-core/src/models/hunyuan_dense/modeling.rs:572-636, 1012-1033.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAXD = 1024;     // widest key row
constexpr int MAXDV = 512;     // widest value row

struct ScoreMod {
    float softcap;              // 0: none
    int chunk;                  // 0: none
    int sigmoid;                // weights sigmoid(s + head_bias[h]), not normalised
    const float* head_bias;     // [nq] or null
    int maps;                   // maps per head (1: a plain head)
    int d_row;                  // elements of a query / key row of a head (>= maps * d_map)
    int d_map;                  // elements from one map's start to the next
    float* out_f32;             // float [token][head][map][dv] instead of `out`, or null
};

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_simt_kernel(const T* __restrict__ q, T* __restrict__ out,
                            const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                            const int* __restrict__ positions, const int* __restrict__ tok_entry,
                            const int* __restrict__ block_table, int max_blocks, int num_pages,
                            int page_size, int n_tokens, int nq, int nkv, int d, int dv,
                            int v_stride, int window, float scale, int sink, float* __restrict__ out_cross,
                            const ScoreMod sm, int* err) {
    extern __shared__ float q_all[];              // [WARPS][d]
    float* q_s = q_all + (threadIdx.x >> 5) * d;
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * WARPS + wib;
    // `out_cross`: every query head is paired with every key/value head's values (its keys stay its own
    // group's): nq * nkv warps a token, results float [token][query head][value head][dv]
    const int pairs = out_cross != nullptr ? nq * nkv : nq * sm.maps;
    if (warp >= (long long)n_tokens * pairs) return;
    const int t = (int)(warp / pairs), hv = (int)(warp % pairs);
    const int h = out_cross != nullptr ? hv / nkv : hv / sm.maps;
    const int map_off = out_cross != nullptr ? 0 : (hv % sm.maps) * sm.d_map;
    const int g = h / (nq / nkv);
    const int gv = out_cross != nullptr ? hv % nkv : g;
    const int pos = positions[t];
    if (tok_entry[t] < 0) return;                 // a row that pads the step: it attends to nothing
    const int* table = block_table + (long long)tok_entry[t] * max_blocks;
    const T* qp = q + ((long long)t * nq + h) * sm.d_row + map_off;
    for (int c = lane; c < d; c += 32) q_s[c] = to_f32(qp[c]);
    __syncwarp();

    int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (sm.chunk > 0) lo = max(lo, pos / sm.chunk * sm.chunk);
    const float bias = sm.head_bias != nullptr ? sm.head_bias[h] : 0.f;
    constexpr int NACC = MAXDV / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool bad = false;
    const long long v_shift = (long long)(gv - g) * page_size;      // from a key row to the value row read with it

    for (int base = lo; base <= pos; base += 32) {
        const int j = base + lane;
        float s = -INFINITY;
        long long row = -1;                       // this lane's key/value row in the pools
        if (j <= pos) {
            const int page = table[j / page_size];
            if (page < 0 || page >= num_pages) {
                bad = true;
            } else {
                row = ((long long)page * nkv + g) * page_size + j % page_size;
                const T* kp = k_pool + row * sm.d_row + map_off;
                float dot = 0.f;
                for (int c = 0; c < d; ++c) dot = fmaf(q_s[c], to_f32(kp[c]), dot);
                s = dot * scale;
                if (sm.softcap > 0.f) s = sm.softcap * tanhf(s / sm.softcap);
            }
        }
        float p;
        if (sm.sigmoid) {
            p = (s == -INFINITY) ? 0.f : 1.f / (1.f + expf(-(s + bias)));
        } else {
            const float m_new = fmaxf(m, warp_max(s));
            if (m_new == -INFINITY) continue;         // every key of this chunk was unreadable
            p = (s == -INFINITY) ? 0.f : expf(s - m_new);
            const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
            l = l * corr + warp_sum(p);
            m = m_new;
#pragma unroll
            for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        }
        const int cnt = min(32, pos - base + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long rj = __shfl_sync(0xffffffffu, row, jj);
            if (rj < 0) continue;
            const T* vp = v_pool + (rj + v_shift) * v_stride;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int c = lane + 32 * i;
                if (c < dv) acc[i] = fmaf(pj, to_f32(vp[c]), acc[i]);
            }
        }
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
    // a sink: one more candidate of score 0 that has no value, so it only adds exp(0 - m) to the sum
    if (sink) l += expf(-m);
    const float inv = sm.sigmoid ? 1.f : l > 0.f ? 1.f / l : 0.f;
    if (sm.out_f32 != nullptr) {
        float* op = sm.out_f32 + ((long long)t * pairs + hv) * dv;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
            const int c = lane + 32 * i;
            if (c < dv) op[c] = acc[i] * inv;
        }
        return;
    }
    if (out_cross != nullptr) {
        float* op = out_cross + ((long long)t * pairs + hv) * dv;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
            const int c = lane + 32 * i;
            if (c < dv) op[c] = acc[i] * inv;
        }
        return;
    }
    T* op = out + ((long long)t * nq + h) * dv;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) op[c] = from_f32<T>(acc[i] * inv);
    }
}
}  // namespace

static int launch_simt(int dtype, const void* q, void* out, const void* k_pool, const void* v_pool,
                       const int* positions, const int* tok_entry, const int* block_table, int max_blocks,
                       int num_pages, int page_size, int n_tokens, int nq, int nkv, int d, int dv, int v_stride,
                       int window, float scale, int sink, float* out_cross, ScoreMod sm, int* err,
                       cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (d > MAXD || d <= 0 || dv > MAXDV || dv <= 0 || v_stride < dv || nkv <= 0 || nq % nkv != 0 ||
        sm.maps < 1 || sm.d_row < (sm.maps - 1) * sm.d_map + d || (out_cross != nullptr && sm.maps != 1))
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)WARPS * d * sizeof(float);
    const long long warps = (long long)n_tokens * nq * (out_cross != nullptr ? nkv : sm.maps);
    const int blocks = (int)((warps + WARPS - 1) / WARPS);
    if (dtype == 0)
        paged_attention_simt_kernel<float><<<blocks, WARPS * 32, smem, st>>>(
            (const float*)q, (float*)out, (const float*)k_pool, (const float*)v_pool, positions,
            tok_entry, block_table, max_blocks, num_pages, page_size, n_tokens, nq, nkv, d, dv,
            v_stride, window, scale, sink, out_cross, sm, err);
    else
        paged_attention_simt_kernel<__nv_bfloat16><<<blocks, WARPS * 32, smem, st>>>(
            (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_pool,
            (const __nv_bfloat16*)v_pool, positions, tok_entry, block_table, max_blocks, num_pages,
            page_size, n_tokens, nq, nkv, d, dv, v_stride, window, scale, sink, out_cross, sm, err);
    return crane_launch_status();
}

CRANE_API int crane_paged_attention_simt(int dtype, const void* q, void* out, const void* k_pool,
                                         const void* v_pool, const int* positions,
                                         const int* tok_entry, const int* block_table,
                                         int max_blocks, int num_pages, int page_size,
                                         int n_tokens, int nq, int nkv, int d, int dv,
                                         int v_stride, int window, float scale, int sink, float* out_cross,
                                         int* err, cudaStream_t st) {
    const ScoreMod plain{0.f, 0, 0, nullptr, 1, d, d, nullptr};
    return launch_simt(dtype, q, out, k_pool, v_pool, positions, tok_entry, block_table, max_blocks, num_pages,
                       page_size, n_tokens, nq, nkv, d, dv, v_stride, window, scale, sink, out_cross, plain, err, st);
}

// The same with the scores worked on (see ScoreMod): d is the width of one map.
CRANE_API int crane_scored_attention_simt(int dtype, const void* q, void* out, const void* k_pool,
                                          const void* v_pool, const int* positions, const int* tok_entry,
                                          const int* block_table, int max_blocks, int num_pages, int page_size,
                                          int n_tokens, int nq, int nkv, int d, int dv, int v_stride, int window,
                                          float scale, float softcap, int chunk, int sigmoid,
                                          const float* head_bias, int maps, int d_row, int d_map, float* out_f32,
                                          int* err, cudaStream_t st) {
    const ScoreMod sm{softcap, chunk, sigmoid, head_bias, maps, d_row, d_map, out_f32};
    return launch_simt(dtype, q, out, k_pool, v_pool, positions, tok_entry, block_table, max_blocks, num_pages,
                       page_size, n_tokens, nq, nkv, d, dv, v_stride, window, scale, 0, nullptr, sm, err, st);
}
