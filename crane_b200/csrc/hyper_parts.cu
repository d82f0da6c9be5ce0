// Memory-bound kernels of layers that keep several residual streams, and of routed feed-forwards
// whose experts are gated and whose router chooses within groups of experts.
//
// 1. `streams_norm`: R float streams x_1 .. x_R per token.  A sublayer's result y joins them as
//        x_t <- sum_s mix[s][t] x_s + out[t] y        (all t at once, from the old streams)
//    and what the next sublayer reads is u = sum_t in[t] x_t, RMS-normed and multiplied by ONE number
//    g.  Both happen in one kernel, a row in shared memory between its passes; either half may be
//    absent (no pending result: the streams stay; `first`: all streams start as the embedding output).
//    R = 1 with mix = out = in = 1 is the plain residual sum.
// 2. `route_grouped`: softmax over all experts, a correction added for the choice only, experts in
//    equal groups of neighbours of which the best few groups stay eligible, the `top` largest choice
//    scores chosen, weighted by their uncorrected scores; an optional further logit becomes the
//    sigmoid gate of a shared expert.
// 3. `gated_activation`: silu(gate) * up per feed-forward column, times the column's routing weight.
// All arithmetic in 32-bit; T is the storage type of activations (float or bf16).
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;

template <typename T>
__global__ void __launch_bounds__(256)
streams_norm_kernel(float* __restrict__ streams, long long stream_stride, int R,
                    const float* __restrict__ x_first, GemmOut<T> y, int has_y,
                    const float* __restrict__ mix, const float* __restrict__ outw,
                    const float* __restrict__ inw, const float* __restrict__ g,
                    const int* __restrict__ rows, T* __restrict__ out, int hidden, float eps) {
    extern __shared__ float u_row[];                  // [hidden]
    __shared__ float scratch[32];
    __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_out[MAX_STREAMS], s_in[MAX_STREAMS];
    pdl_launch_dependents();
    if (threadIdx.x < R * R) s_mix[threadIdx.x] = has_y ? mix[threadIdx.x] : (threadIdx.x / R == threadIdx.x % R ? 1.f : 0.f);
    if (threadIdx.x < R) {
        s_out[threadIdx.x] = has_y ? outw[threadIdx.x] : 0.f;
        s_in[threadIdx.x] = inw != nullptr ? inw[threadIdx.x] : 1.f;
    }
    const float gain = g[0];
    pdl_wait();
    __syncthreads();
    const int r = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
    const long long base = (long long)r * hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float old[MAX_STREAMS], nw[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s)
            if (s < R) old[s] = x_first != nullptr ? x_first[base + c] : streams[s * stream_stride + base + c];
        const float yv = has_y ? y.load(base + c) : 0.f;
        float u = 0.f;
#pragma unroll
        for (int t = 0; t < MAX_STREAMS; ++t) {
            if (t < R) {
                float v = s_out[t] * yv;
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s)
                    if (s < R) v = fmaf(s_mix[s * R + t], old[s], v);
                nw[t] = v;
                u = fmaf(s_in[t], v, u);
            }
        }
        if (rows == nullptr && (has_y || x_first != nullptr)) {
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t)
                if (t < R) streams[t * stream_stride + base + c] = nw[t];
        }
        u_row[c] = u;
        ss = fmaf(u, u, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)hidden + eps) * gain;
    T* o = out + (long long)blockIdx.x * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = from_f32<T>(u_row[c] * rstd);
}

// One warp per token.  z: float logits [n][ld], the first `experts` of a row the router's, column
// `experts` (if `shared_gate`) the shared expert's gate.  route [n][experts + shared_gate].
__global__ void __launch_bounds__(128)
route_grouped_kernel(const float* __restrict__ z, int ld, const float* __restrict__ correction,
                     float* __restrict__ route, int n, int experts, int top, int groups, int keep,
                     int shared_gate) {
    extern __shared__ float sm[];                     // per warp: score [E], choice [E], group score [groups]
    pdl_launch_dependents();
    pdl_wait();
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + wib;
    if (t >= n) return;
    float* score = sm + (size_t)wib * (2 * experts + groups);
    float* choice = score + experts;
    float* gscore = choice + experts;
    const float* zr = z + (long long)t * ld;
    float* r = route + (long long)t * (experts + shared_gate);
    float zmax = -INFINITY;
    for (int e = lane; e < experts; e += 32) zmax = fmaxf(zmax, zr[e]);
    zmax = warp_max(zmax);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) {
        const float p = expf(zr[e] - zmax);
        score[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < experts; e += 32) {
        const float s = score[e] * inv;
        score[e] = s;
        choice[e] = s + (correction != nullptr ? correction[e] : 0.f);
        r[e] = 0.f;
    }
    __syncwarp();
    const int per = experts / groups;
    if (keep < groups) {
        for (int gi = lane; gi < groups; gi += 32) {
            float best = -INFINITY;
            for (int j = 0; j < per; ++j) best = fmaxf(best, choice[gi * per + j]);
            gscore[gi] = best;
        }
        __syncwarp();
        // the `keep` best groups are marked (their score becomes NaN-free +inf); the others' experts leave
        for (int j = 0; j < keep; ++j) {
            float best = -INFINITY;
            int bi = 0x7fffffff;
            for (int gi = lane; gi < groups; gi += 32) {
                const float v = gscore[gi];
                if (v == INFINITY) continue;          // taken
                if (bi == 0x7fffffff || v > best) { best = v; bi = gi; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
            }
            if (bi == 0x7fffffff) break;
            if (lane == 0) gscore[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32)
            if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = choice[e];
            if (v == -INFINITY) continue;             // not eligible, or taken
            if (bi == 0x7fffffff || v > best) { best = v; bi = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
        }
        if (bi == 0x7fffffff) break;                  // fewer eligible experts than `top`
        if (lane == 0) {
            r[bi] = score[bi];
            choice[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (shared_gate && lane == 0) r[experts] = 1.f / (1.f + expf(-zr[experts]));
}

// gu rows: [gate (cols) | up (cols)].  out[t][c] = silu(gate) * up * weight(c): route[t][c / per_expert]
// for c < routed_cols, behind them route[t][experts] (`shared_gate`) or 1.
template <typename T>
__global__ void __launch_bounds__(256)
gated_activation_kernel(GemmOut<T> gu, T* __restrict__ out, long long n, int cols,
                        const float* __restrict__ route, int experts, int per_expert, int routed_cols,
                        int shared_gate) {
    pdl_launch_dependents();
    pdl_wait();
    const int rl = experts + shared_gate;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / cols;
        const int c = (int)(i % cols);
        float w = 1.f;
        if (route != nullptr) {
            if (c < routed_cols) w = route[row * rl + c / per_expert];
            else if (shared_gate) w = route[row * rl + experts];
        }
        float v = 0.f;
        if (w != 0.f) {
            const float a = gu.load(row * 2 * cols + c), b = gu.load(row * 2 * cols + cols + c);
            v = a / (1.f + expf(-a)) * b * w;
        }
        out[i] = from_f32<T>(v);
    }
}

}  // namespace

CRANE_API int crane_streams_norm(int dtype, float* streams, long long stream_stride, int n_streams,
                                 const float* x_first, const void* y, const float* y_parts, int n_parts,
                                 long long part_stride, const float* mix, const float* outw, const float* inw,
                                 const float* g, const int* rows, void* out, int n_rows, int hidden, float eps,
                                 cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (n_streams < 1 || n_streams > MAX_STREAMS) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const int has_y = (y != nullptr || y_parts != nullptr) ? 1 : 0;
    DISPATCH_T(dtype, {
        GemmOut<T> d{(const T*)y, y_parts, n_parts, part_stride};
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(streams_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return crane_launch(streams_norm_kernel<T>, dim3(n_rows), dim3(256), smem, st, streams, stream_stride,
                            n_streams, x_first, d, has_y, mix, outw, inw, g, rows, (T*)out, hidden, eps);
    });
}

CRANE_API int crane_route_grouped(const float* z, int ld, const float* correction, float* route, int n,
                                  int experts, int top, int groups, int keep, int shared_gate, cudaStream_t st) {
    if (n <= 0) return 0;
    if (experts <= 0 || top <= 0 || groups <= 0 || experts % groups || keep <= 0 || keep > groups)
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)4 * (2 * experts + groups) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return crane_launch(route_grouped_kernel, dim3((n + 3) / 4), dim3(128), smem, st, z, ld, correction, route, n,
                        experts, top, groups, keep, shared_gate ? 1 : 0);
}

CRANE_API int crane_gated_activation(int dtype, const void* gu, const float* gu_parts, int n_parts,
                                     long long part_stride, void* out, int n_rows, int cols, const float* route,
                                     int experts, int per_expert, int routed_cols, int shared_gate,
                                     cudaStream_t st) {
    if (n_rows <= 0 || cols <= 0) return 0;
    const long long n = (long long)n_rows * cols;
    const int blocks = (int)((n + 255) / 256 < 16384 ? (n + 255) / 256 : 16384);
    DISPATCH_T(dtype, {
        GemmOut<T> u{(const T*)gu, gu_parts, n_parts, part_stride};
        return crane_launch(gated_activation_kernel<T>, dim3(blocks), dim3(256), 0, st, u, (T*)out, n, cols, route,
                            experts, per_expert > 0 ? per_expert : 1, routed_cols, shared_gate ? 1 : 0);
    });
}
