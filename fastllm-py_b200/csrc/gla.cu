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
// w2: the decay's second matrix transposed, [rank][heads x dim], so that neighbouring threads read neighbouring floats.
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
    // (blockIdx.y shares a token's columns out over blocks: a handful of tokens alone would leave the GPU idle)
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hd; i += gridDim.y * blockDim.x) {
        w[i] = to_f32<T>(row[i]) * q_scale;
        w[hd + i] = to_f32<T>(row[hd + i]);
        float z = b2[i];
        for (int k = 0; k < rank; ++k) z += w2[(long)k * hd + i] * low_s[k];       // w2 is stored [rank][heads x dim]
        const float logsig = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
        w[2 * hd + i] = expf(logsig / tau);
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hv; i += gridDim.y * blockDim.x) w[3 * hd + i] = to_f32<T>(row[2 * hd + i]);
}

#define GLA_COLS 16              // value columns of a block
#define GLA_STAGES 4             // stages of shared memory: chunks copied ahead of the one being walked

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

// LANES lanes share a column of S; a lane holds R of its rows (dim <= LANES R; the rows beyond dim stay zero): the
// groups of four rows g = lane + LANES i, so that the lanes of a column read consecutive 16 bytes of a staged row.  A
// stage of shared memory holds `chunk` tokens: [chunk][3][LANES R] q', k, alpha, then [chunk][COLS] v; four stages, three
// chunks being copied (cp.async) while one is walked, so that a copy's latency is hidden behind three chunks' arithmetic.
// Per token a lane does S <- alpha S + k v and sums S q over its rows, then the lanes of a column add up in a fixed
// order; only the state's multiply-add is a chain from token to token.  Eight lanes a column in the 32-bit path whatever
// the step's shape (so that its sums keep one order); sixteen where the launch would otherwise leave the GPU idle.
template <int R, int LANES>
__global__ void __launch_bounds__(GLA_COLS * LANES) gla_scan_kernel(
    const float* __restrict__ work, long w_ld, float* __restrict__ o, long o_ld, float* __restrict__ state,
    long state_stride, const int* __restrict__ req_start, const int* __restrict__ req_ctx,
    const int* __restrict__ req_qlen, const int* __restrict__ req_slot, int heads, int dim, int vdim, int chunk, int vec4) {
    pdl_wait();
    pdl_trigger();
    constexpr int DP = R * LANES;
    extern __shared__ __align__(16) float gla_s[];
    const int stage_floats = chunk * (3 * DP + GLA_COLS);
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * GLA_COLS;
    const int tid = threadIdx.x, lane = tid & (LANES - 1), cl = tid / LANES;
    const int col = col0 + cl;
    const bool live = col < vdim;
    const int start = req_start[r], ctx = req_ctx[r], qlen = req_qlen[r];
    const int hd = heads * dim;
    for (int i = tid; i < GLA_STAGES * stage_floats; i += blockDim.x) gla_s[i] = 0.0f;      // the padding stays zero
    float* srow = state + (long)req_slot[r] * state_stride + ((long)h * vdim + (live ? col : 0)) * dim;
    float S[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = 4 * (lane + LANES * (i / 4)) + (i & 3);
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
    // one group of copies per chunk, also for chunks beyond the end (empty groups), so that waiting for all but the
    // last STAGES - 1 groups always means: this chunk has landed
#pragma unroll
    for (int p = 0; p < GLA_STAGES - 1; ++p) {
        if (p * chunk < qlen) load(p, p * chunk); else gla_commit();
    }
    int stage = 0;
    float* op = o + (long)start * o_ld + (long)h * vdim + col;
    for (int c0 = 0; c0 < qlen; c0 += chunk, stage = (stage + 1) % GLA_STAGES) {
        const int n_here = min(chunk, qlen - c0);
        const int ahead = c0 + (GLA_STAGES - 1) * chunk;
        // (the stage copied into now was walked in the last round, behind that round's closing barrier)
        if (ahead < qlen) load((stage + GLA_STAGES - 1) % GLA_STAGES, ahead); else gla_commit();
        gla_wait<GLA_STAGES - 1>();
        __syncthreads();                                // this chunk has landed
        const float4* row4 = reinterpret_cast<const float4*>(gla_s + stage * stage_floats) + lane;
        const float* vp = gla_s + stage * stage_floats + chunk * 3 * DP + cl;
#pragma unroll 4
        for (int tt = 0; tt < n_here; ++tt) {
            const float v = *vp;
            float acc = 0.0f, acc1 = 0.0f;                  // two partial sums: half as long a chain
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const float4 q = row4[i * LANES], k = row4[DP / 4 + i * LANES], a = row4[2 * (DP / 4) + i * LANES];
                S[4 * i] = fmaf(a.x, S[4 * i], k.x * v);
                acc = fmaf(S[4 * i], q.x, acc);
                S[4 * i + 1] = fmaf(a.y, S[4 * i + 1], k.y * v);
                acc1 = fmaf(S[4 * i + 1], q.y, acc1);
                S[4 * i + 2] = fmaf(a.z, S[4 * i + 2], k.z * v);
                acc = fmaf(S[4 * i + 2], q.z, acc);
                S[4 * i + 3] = fmaf(a.w, S[4 * i + 3], k.w * v);
                acc1 = fmaf(S[4 * i + 3], q.w, acc1);
            }
            acc += acc1;
#pragma unroll
            for (int off = 1; off < LANES; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (lane == 0 && live) *op = acc;
            row4 += 3 * (DP / 4);
            vp += GLA_COLS;
            op += o_ld;
        }
        __syncthreads();                                // the stage is copied into again in the next round
    }
    if (live)
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int d = 4 * (lane + LANES * (i / 4)) + (i & 3);
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
    int share = n_tokens >= 256 ? 1 : (heads * dim + 255) / 256;
    if (share > 16) share = 16;
    FL_DISPATCH(dtype, T, return fl_launch(gla_prep_kernel<T>, dim3(n_tokens, share), dim3(256), (size_t)rank * sizeof(float), stream,
                                           (const T*)proj, ld, w2, b2, work, w_ld, heads, dim, vdim, rank, q_scale,
                                           tau));
    return 0;
}

template <int R, int LANES>
static int gla_scan_launch(dim3 grid, size_t smem, cudaStream_t stream, const float* work, long w_ld, float* o, long o_ld,
                           float* state, long state_stride, const int* req_start, const int* req_ctx, const int* req_qlen,
                           const int* req_slot, int heads, int dim, int vdim, int chunk, int vec4) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gla_scan_kernel<R, LANES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 104 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return fl_launch(gla_scan_kernel<R, LANES>, grid, dim3(GLA_COLS * LANES), smem, stream, work, w_ld, o, o_ld, state,
                     state_stride, req_start, req_ctx, req_qlen, req_slot, heads, dim, vdim, chunk, vec4);
}

// fixed_order: eight lanes a column whatever the step's shape (the sums of the read-out then keep one order).
FL_API int fl_gla_scan(const float* work, long w_ld, float* o, long o_ld, float* state, long state_stride,
                       const int* req_start, const int* req_ctx, const int* req_qlen, const int* req_slot, int n_requests,
                       int heads, int dim, int vdim, int sms, int fixed_order, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (dim < 1 || dim > 256 || heads > 65535 || (vdim + GLA_COLS - 1) / GLA_COLS > 65535)
        return (int)cudaErrorInvalidValue;
    const int padded = dim <= 32 ? 32 : dim <= 64 ? 64 : dim <= 128 ? 128 : 256;      // rows of a column, padded
    const int chunk = padded <= 128 ? 16 : 8;                            // tokens of a stage
    const size_t smem = GLA_STAGES * (size_t)chunk * (3 * padded + GLA_COLS) * sizeof(float);   // <= 103 KB
    // 16-byte copies where every source address is a multiple of 16 bytes
    const int vec4 = dim % 4 == 0 && vdim % 4 == 0 && w_ld % 4 == 0 && ((uintptr_t)work % 16) == 0;
    dim3 grid(n_requests, heads, (vdim + GLA_COLS - 1) / GLA_COLS);
    const bool wide = !fixed_order && padded >= 64 && (long)grid.x * grid.y * grid.z < 2L * sms;
#define FL_GLA_SCAN(R, L)                                                                                               \
    return gla_scan_launch<R, L>(grid, smem, stream, work, w_ld, o, o_ld, state, state_stride, req_start, req_ctx,      \
                                 req_qlen, req_slot, heads, dim, vdim, chunk, vec4)
    if (wide) {
        if (padded == 64) { FL_GLA_SCAN(4, 16); }
        if (padded == 128) { FL_GLA_SCAN(8, 16); }
        FL_GLA_SCAN(16, 16);
    }
    if (padded == 32) { FL_GLA_SCAN(4, 8); }
    if (padded == 64) { FL_GLA_SCAN(8, 8); }
    if (padded == 128) { FL_GLA_SCAN(16, 8); }
    FL_GLA_SCAN(32, 8);
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
