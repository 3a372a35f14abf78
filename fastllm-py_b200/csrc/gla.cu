// Gated linear attention: a matrix state per head whose rows decay by numbers made from the token.
//
// Per token, from one product proj = [q | k | v | gate | low] (heads x dim, heads x dim, heads x vdim, heads x vdim,
// rank):
//     q' = q * q_scale,   z = W_2 low + b_2 (heads x dim),   alpha = sigmoid(z)^(1 / tau) = exp(logsigmoid(z) / tau)
//     S <- diag(alpha) S + k v^T      (S: dim x vdim per head; alpha acts on the rows, one per key channel)
//     o = S^T q'
// then each head's o is divided by its root mean square over vdim, multiplied by a weight [vdim] shared by the heads and
// by silu(gate).  A request's state row is S for every head, [heads][vdim][dim] float; it is read unless the request
// starts (context 0) and written at the end of the step.
//
//   gla_prep         per token: q', k, alpha, v widened to float in one work row; the small product W_2 low on the CUDA
//                    cores in float
//   gla_scan         per (request, head, 16 value columns): the recurrence over the request's tokens in order; a column
//                    of S lives in the registers of eight lanes, the tokens' rows pass through two stages of shared
//                    memory, one copied ahead while the other is walked
//   gla_gated_norm   per (token, head): norm, weight, gate
//
// Everything after the product is float.  Every sum's order depends on the token alone.
#include "common.cuh"

// work row: q' (heads x dim) | k (heads x dim) | alpha (heads x dim) | v (heads x vdim), float.
template <typename T>
__global__ void __launch_bounds__(256) gla_prep_kernel(const T* __restrict__ proj, long ld, const float* __restrict__ w2,
                                                       const float* __restrict__ b2, float* __restrict__ work, long w_ld,
                                                       int heads, int dim, int vdim, int rank, float q_scale, float tau) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float low_s[];                    // [rank]
    const long t = blockIdx.x;
    const T* row = proj + t * ld;
    const int hd = heads * dim, hv = heads * vdim;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) low_s[i] = to_f32<T>(row[2 * hd + 2 * hv + i]);
    __syncthreads();
    float* w = work + t * w_ld;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        w[i] = to_f32<T>(row[i]) * q_scale;
        w[hd + i] = to_f32<T>(row[hd + i]);
        float z = b2[i];
        const float* wr = w2 + (long)i * rank;
        for (int k = 0; k < rank; ++k) z += wr[k] * low_s[k];
        const float logsig = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
        w[2 * hd + i] = expf(logsig / tau);
    }
    for (int i = threadIdx.x; i < hv; i += blockDim.x) w[3 * hd + i] = to_f32<T>(row[2 * hd + i]);
}

#define GLA_COLS 16              // value columns of a block
#define GLA_LANES 8              // lanes that share a column: lane l holds the rows l R .. l R + R - 1

__device__ __forceinline__ void gla_cp4(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void gla_cp16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void gla_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void gla_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

// R: rows of a column that a lane holds (dim <= 8 R; the rows beyond dim stay zero).  A stage of shared memory holds
// `chunk` tokens: [chunk][3][8 R] q', k, alpha, then [chunk][COLS] v; two stages, the next chunk copied (cp.async) while
// this one is walked.  Per token a lane does S <- alpha S + k v and sums S q over its rows, then the eight lanes of a
// column add up in a fixed order; only the state's multiply-add is a chain from token to token.
template <int R>
__global__ void __launch_bounds__(GLA_COLS * GLA_LANES) gla_scan_kernel(
    const float* __restrict__ work, long w_ld, float* __restrict__ o, long o_ld, float* __restrict__ state,
    long state_stride, const int* __restrict__ req_start, const int* __restrict__ req_ctx,
    const int* __restrict__ req_qlen, const int* __restrict__ req_slot, int heads, int dim, int vdim, int chunk, int vec4) {
    pdl_wait();
    pdl_trigger();
    constexpr int DP = R * GLA_LANES;
    extern __shared__ __align__(16) float gla_s[];
    const int stage_floats = chunk * (3 * DP + GLA_COLS);
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * GLA_COLS;
    const int tid = threadIdx.x, lane = tid & (GLA_LANES - 1), cl = tid / GLA_LANES;
    const int col = col0 + cl;
    const bool live = col < vdim;
    const int start = req_start[r], ctx = req_ctx[r], qlen = req_qlen[r];
    const int hd = heads * dim;
    for (int i = tid; i < 2 * stage_floats; i += blockDim.x) gla_s[i] = 0.0f;      // the padding stays zero
    float* srow = state + (long)req_slot[r] * state_stride + ((long)h * vdim + (live ? col : 0)) * dim;
    float S[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = lane * R + i;
        S[i] = (ctx > 0 && live && d < dim) ? srow[d] : 0.0f;
    }
    __syncthreads();
    auto load = [&](int stage, int c0) {
        float* st = gla_s + stage * stage_floats;
        float* vs = st + chunk * 3 * DP;
        const int n_here = min(chunk, qlen - c0);
        if (vec4) {
            const int d4 = dim / 4;
            for (int i = tid; i < n_here * 3 * d4; i += blockDim.x) {
                const int tt = i / (3 * d4), k = i - tt * 3 * d4;
                const int part = k / d4, d = (k - part * d4) * 4;
                gla_cp16(st + (tt * 3 + part) * DP + d, work + (long)(start + c0 + tt) * w_ld + (long)part * hd + (long)h * dim + d);
            }
            const int cols4 = min(GLA_COLS, vdim - col0) / 4;
            for (int i = tid; i < n_here * cols4; i += blockDim.x) {
                const int tt = i / cols4, cc = (i - tt * cols4) * 4;
                gla_cp16(vs + tt * GLA_COLS + cc, work + (long)(start + c0 + tt) * w_ld + 3L * hd + (long)h * vdim + col0 + cc);
            }
        } else {
            for (int i = tid; i < n_here * 3 * dim; i += blockDim.x) {
                const int tt = i / (3 * dim), k = i - tt * 3 * dim;
                const int part = k / dim, d = k - part * dim;
                gla_cp4(st + (tt * 3 + part) * DP + d, work + (long)(start + c0 + tt) * w_ld + (long)part * hd + (long)h * dim + d);
            }
            const int cols = min(GLA_COLS, vdim - col0);
            for (int i = tid; i < n_here * cols; i += blockDim.x) {
                const int tt = i / cols, cc = i - tt * cols;
                gla_cp4(vs + tt * GLA_COLS + cc, work + (long)(start + c0 + tt) * w_ld + 3L * hd + (long)h * vdim + col0 + cc);
            }
        }
        gla_commit();
    };
    load(0, 0);
    int stage = 0;
    for (int c0 = 0; c0 < qlen; c0 += chunk, stage ^= 1) {
        const int n_here = min(chunk, qlen - c0);
        if (c0 + chunk < qlen) {
            load(stage ^ 1, c0 + chunk);
            gla_wait<1>();
        } else {
            gla_wait<0>();
        }
        __syncthreads();                                // this chunk has landed
        const float* st = gla_s + stage * stage_floats;
        const float* vs = st + chunk * 3 * DP;
        float* orow = o + (long)(start + c0) * o_ld + (long)h * vdim + col;
#pragma unroll 4
        for (int tt = 0; tt < n_here; ++tt) {
            const float4* q4 = reinterpret_cast<const float4*>(st + tt * 3 * DP + lane * R);
            const float4* k4 = reinterpret_cast<const float4*>(st + tt * 3 * DP + DP + lane * R);
            const float4* a4 = reinterpret_cast<const float4*>(st + tt * 3 * DP + 2 * DP + lane * R);
            const float v = vs[tt * GLA_COLS + cl];
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const float4 q = q4[i], k = k4[i], a = a4[i];
                S[4 * i] = fmaf(a.x, S[4 * i], k.x * v);
                acc = fmaf(S[4 * i], q.x, acc);
                S[4 * i + 1] = fmaf(a.y, S[4 * i + 1], k.y * v);
                acc = fmaf(S[4 * i + 1], q.y, acc);
                S[4 * i + 2] = fmaf(a.z, S[4 * i + 2], k.z * v);
                acc = fmaf(S[4 * i + 2], q.z, acc);
                S[4 * i + 3] = fmaf(a.w, S[4 * i + 3], k.w * v);
                acc = fmaf(S[4 * i + 3], q.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (lane == 0 && live) orow[(long)tt * o_ld] = acc;
        }
        __syncthreads();                                // the stage is rewritten two chunks on
    }
    if (live)
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int d = lane * R + i;
            if (d < dim) srow[d] = S[i];
        }
}

template <typename T, typename TW>
__global__ void __launch_bounds__(128) gla_gated_norm_kernel(const float* __restrict__ o, long o_ld, const T* __restrict__ gate,
                                                             long g_ld, const TW* __restrict__ weight, T* __restrict__ out,
                                                             long out_ld, int n_tokens, int heads, int vdim, float eps) {
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long pair = (long)blockIdx.x * 4 + warp;
    if (pair >= (long)n_tokens * heads) return;
    const long t = pair / heads;
    const int h = (int)(pair - t * heads);
    const float* orow = o + t * o_ld + (long)h * vdim;
    float ss = 0.0f;
    for (int d = lane; d < vdim; d += 32) ss += orow[d] * orow[d];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    for (int d = lane; d < vdim; d += 32) {
        const float g = to_f32<T>(gate[t * g_ld + (long)h * vdim + d]);
        const float w = weight != nullptr ? to_f32<TW>(weight[d]) : 1.0f;
        out[t * out_ld + (long)h * vdim + d] = from_f32<T>(orow[d] * inv * w * (g / (1.0f + expf(-g))));
    }
}

FL_API int fl_gla_prep(const void* proj, int dtype, long ld, const float* w2, const float* b2, float* work, long w_ld,
                       int n_tokens, int heads, int dim, int vdim, int rank, float q_scale, float tau, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank < 1 || (size_t)rank * sizeof(float) > 48 * 1024 || !(tau > 0.0f)) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, return fl_launch(gla_prep_kernel<T>, dim3(n_tokens), dim3(256), (size_t)rank * sizeof(float), stream,
                                           (const T*)proj, ld, w2, b2, work, w_ld, heads, dim, vdim, rank, q_scale,
                                           tau));
    return 0;
}

FL_API int fl_gla_scan(const float* work, long w_ld, float* o, long o_ld, float* state, long state_stride,
                       const int* req_start, const int* req_ctx, const int* req_qlen, const int* req_slot, int n_requests,
                       int heads, int dim, int vdim, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (dim < 1 || dim > 32 * GLA_LANES || heads > 65535 || (vdim + GLA_COLS - 1) / GLA_COLS > 65535)
        return (int)cudaErrorInvalidValue;
    const int rows = dim <= 4 * GLA_LANES ? 4 : dim <= 8 * GLA_LANES ? 8 : dim <= 16 * GLA_LANES ? 16 : 32;
    const int chunk = rows <= 8 ? 16 : rows == 16 ? 8 : 4;               // tokens of a stage: two stages within 48 KB
    const size_t smem = 2 * (size_t)chunk * (3 * rows * GLA_LANES + GLA_COLS) * sizeof(float);
    // 16-byte copies where every source address is a multiple of 16 bytes
    const int vec4 = dim % 4 == 0 && vdim % 4 == 0 && w_ld % 4 == 0 && ((uintptr_t)work % 16) == 0;
    dim3 grid(n_requests, heads, (vdim + GLA_COLS - 1) / GLA_COLS);
#define FL_GLA_SCAN(R)                                                                                                  \
    return fl_launch(gla_scan_kernel<R>, grid, dim3(GLA_COLS * GLA_LANES), smem, stream, work, w_ld, o, o_ld, state,    \
                     state_stride, req_start, req_ctx, req_qlen, req_slot, heads, dim, vdim, chunk, vec4)
    if (rows == 4) { FL_GLA_SCAN(4); }
    if (rows == 8) { FL_GLA_SCAN(8); }
    if (rows == 16) { FL_GLA_SCAN(16); }
    FL_GLA_SCAN(32);
#undef FL_GLA_SCAN
}

FL_API int fl_gla_gated_norm(const float* o, long o_ld, const void* gate, int dtype, long g_ld, const void* weight,
                             int w_dtype, void* out, long out_ld, int n_tokens, int heads, int vdim, float eps,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const long pairs = (long)n_tokens * heads;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        return fl_launch(gla_gated_norm_kernel<T, TW>, dim3((unsigned)((pairs + 3) / 4)), dim3(128), 0, stream, o, o_ld,
                         (const T*)gate, g_ld, (const TW*)weight, (T*)out, out_ld, n_tokens, heads, vdim, eps)));
    return 0;
}
