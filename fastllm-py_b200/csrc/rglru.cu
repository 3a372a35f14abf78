// A gated linear recurrence per channel (the real-gated linear recurrent unit) between two branches.
//
// Per token, from one product proj = [y_pre | x_pre] (each `width` wide; biases added here):
//     y = gelu_tanh(y_pre)                                   the gate branch
//     u = conv(x_pre)                                        causal, per channel, `taps` taps, the last tap the token's own;
//                                                            zeros before the sequence's start
//     r = sigmoid(A_b u_b + a_b),  i = sigmoid(I_b u_b + i_b)   per block b of width / blocks channels (square matrices)
//     a = exp(rate * r)            rate[c] = -c softplus(lam[c]), made by the caller
//     S <- a S + sqrt(1 - a^2) * i * u;     out = S * y
// A request's state row is [S (width) | the last taps - 1 rows of x_pre (width each)], float; it is read unless the
// request starts (context 0) and written at the end of the step.
//
//   rglru_conv    per (token, channel): u, from the step's rows of the same request and the kept rows before them; four
//                 channels a thread where the pitches allow 16-byte accesses
//   rglru_gates   per (16 tokens, block): both block products on the CUDA cores in float, one thread an output channel,
//                 then a and the input term
//   rglru_scan    per (request, channel): the recurrence over the request's tokens in order, the gate branch, the new
//                 state and the new kept rows; for prompt portions outside the 32-bit path a form that runs 32 segments
//                 of the tokens side by side
//
// Everything after the product is float.  Every sum's order depends on the token alone.
#include "common.cuh"

#define RG_MAX_TAPS 16

template <typename T>
__global__ void __launch_bounds__(256) rglru_conv_kernel(
    const T* __restrict__ proj, long ld, const float* __restrict__ bias, const float* __restrict__ conv_w,
    const float* __restrict__ conv_b, const float* __restrict__ state, long state_stride, const int* __restrict__ tok_req,
    const int* __restrict__ positions, const int* __restrict__ req_start, const int* __restrict__ req_ctx,
    const int* __restrict__ req_slot, float* __restrict__ u, long u_ld, int width, int taps) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int r = tok_req[t], pos = positions[t];
    const int start = req_start[r], ctx = req_ctx[r];
    const float* tail = state + (long)req_slot[r] * state_stride + width;      // row k: position ctx - (taps - 1) + k
    const float xb = bias[width + c];
    float acc = conv_b[c];
    for (int j = 0; j < taps; ++j) {
        const int p = pos - (taps - 1) + j;
        if (p < 0) continue;
        float x;
        if (p >= ctx) x = to_f32<T>(proj[(long)(start + p - ctx) * ld + width + c]) + xb;
        else x = tail[(long)(p - ctx + taps - 1) * width + c];
        acc += conv_w[(long)c * taps + j] * x;
    }
    u[(long)t * u_ld + c] = acc;
}

// Four channels a thread (width a multiple of 4, rows 8-byte aligned): the same sums, each channel's taps in order.
__device__ __forceinline__ void rg_load4(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void rg_load4(const bf16* p, float* v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

template <typename T>
__global__ void __launch_bounds__(256) rglru_conv4_kernel(
    const T* __restrict__ proj, long ld, const float* __restrict__ bias, const float* __restrict__ conv_w,
    const float* __restrict__ conv_b, const float* __restrict__ state, long state_stride, const int* __restrict__ tok_req,
    const int* __restrict__ positions, const int* __restrict__ req_start, const int* __restrict__ req_ctx,
    const int* __restrict__ req_slot, float* __restrict__ u, long u_ld, int width, int taps) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= width) return;
    const int r = tok_req[t], pos = positions[t];
    const int start = req_start[r], ctx = req_ctx[r];
    const float* tail = state + (long)req_slot[r] * state_stride + width;
    float xb[4], acc[4];
    rg_load4(bias + width + c, xb);
    rg_load4(conv_b + c, acc);
    for (int j = 0; j < taps; ++j) {
        const int p = pos - (taps - 1) + j;
        if (p < 0) continue;
        float x[4];
        if (p >= ctx) {
            rg_load4(proj + (long)(start + p - ctx) * ld + width + c, x);
#pragma unroll
            for (int e = 0; e < 4; ++e) x[e] += xb[e];
        } else {
            rg_load4(tail + (long)(p - ctx + taps - 1) * width + c, x);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] += conv_w[(long)(c + e) * taps + j] * x[e];
    }
    *reinterpret_cast<float4*>(u + (long)t * u_ld + c) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

#define RG_TT 16                 // tokens of a block of rglru_gates

__device__ __forceinline__ void rg_load8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void rg_load8(const bf16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

// w_a, w_i: [blocks][bw][bw] (out, in); b_a, b_i: [blocks][bw] float.  a_out, b_out: [n, width] float.
// One thread per output channel of the block: it walks its two weight rows once (eight elements a load where the rows
// are 16-byte aligned: VEC) against the 16 tokens' inputs in shared memory, so every sum runs over k in order and
// nothing crosses lanes.
template <typename TW, bool VEC>
__global__ void __launch_bounds__(256) rglru_gates_kernel(const float* __restrict__ u, long u_ld, const TW* __restrict__ w_a,
                                                          const TW* __restrict__ w_i, const float* __restrict__ b_a,
                                                          const float* __restrict__ b_i, const float* __restrict__ rate,
                                                          float* __restrict__ a_out, float* __restrict__ b_out, long o_ld,
                                                          int n_tokens, int width, int bw) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) float u_s[];        // [RG_TT][bw]
    const int t0 = blockIdx.x * RG_TT, b = blockIdx.y;
    const int n_here = min(RG_TT, n_tokens - t0);
    for (int i = threadIdx.x; i < RG_TT * bw; i += blockDim.x) {
        const int tt = i / bw, k = i - tt * bw;
        u_s[i] = tt < n_here ? u[(long)(t0 + tt) * u_ld + b * bw + k] : 0.0f;
    }
    __syncthreads();
    const int o = blockIdx.z * blockDim.x + threadIdx.x;
    if (o >= bw) return;
    const TW* ra = w_a + ((long)b * bw + o) * bw;
    const TW* ri = w_i + ((long)b * bw + o) * bw;
    float sa[RG_TT], si[RG_TT];
#pragma unroll
    for (int tt = 0; tt < RG_TT; ++tt) sa[tt] = si[tt] = 0.0f;
    if (VEC) {
        for (int k = 0; k < bw; k += 8) {
            float wa[8], wi[8];
            rg_load8(ra + k, wa);
            rg_load8(ri + k, wi);
#pragma unroll
            for (int tt = 0; tt < RG_TT; ++tt) {
                float uu[8];
                rg_load8(u_s + tt * bw + k, uu);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    sa[tt] = fmaf(wa[e], uu[e], sa[tt]);
                    si[tt] = fmaf(wi[e], uu[e], si[tt]);
                }
            }
        }
    } else {
        for (int k = 0; k < bw; ++k) {
            const float wa = to_f32<TW>(ra[k]), wi = to_f32<TW>(ri[k]);
#pragma unroll
            for (int tt = 0; tt < RG_TT; ++tt) {
                sa[tt] = fmaf(wa, u_s[tt * bw + k], sa[tt]);
                si[tt] = fmaf(wi, u_s[tt * bw + k], si[tt]);
            }
        }
    }
    const int c = b * bw + o;
    const float ba = b_a[c], bi = b_i[c], rt = rate[c];
#pragma unroll
    for (int tt = 0; tt < RG_TT; ++tt)
        if (tt < n_here) {
            const float r = 1.0f / (1.0f + expf(-(sa[tt] + ba)));
            const float g = 1.0f / (1.0f + expf(-(si[tt] + bi)));
            const float log_a = rt * r;
            const long at = (long)(t0 + tt) * o_ld + c;
            a_out[at] = expf(log_a);
            b_out[at] = sqrtf(-expm1f(2.0f * log_a)) * g * u_s[tt * bw + o];
        }
}

// The same for a handful of tokens (single tokens of a few requests), where a thread an output would leave the GPU
// idle behind a few long walks: one warp per output channel, the lanes sharing the row, eight tokens a block.  Its sums
// run in another order than the kernel's above, so the 32-bit path, whose results must not depend on what else is in the
// step, never takes it.
#define RG_FEW 8
template <typename TW>
__global__ void __launch_bounds__(256) rglru_gates_few_kernel(const float* __restrict__ u, long u_ld, const TW* __restrict__ w_a,
                                                              const TW* __restrict__ w_i, const float* __restrict__ b_a,
                                                              const float* __restrict__ b_i, const float* __restrict__ rate,
                                                              float* __restrict__ a_out, float* __restrict__ b_out, long o_ld,
                                                              int n_tokens, int width, int bw) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) float u_s[];        // [RG_FEW][bw]
    const int t0 = blockIdx.x * RG_FEW, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_here = min(RG_FEW, n_tokens - t0);
    for (int i = threadIdx.x; i < RG_FEW * bw; i += blockDim.x) {
        const int tt = i / bw, k = i - tt * bw;
        u_s[i] = tt < n_here ? u[(long)(t0 + tt) * u_ld + b * bw + k] : 0.0f;
    }
    __syncthreads();
    for (int o = blockIdx.z * 8 + warp; o < bw; o += gridDim.z * 8) {
        const TW* ra = w_a + ((long)b * bw + o) * bw;
        const TW* ri = w_i + ((long)b * bw + o) * bw;
        float sa[RG_FEW], si[RG_FEW];
#pragma unroll
        for (int tt = 0; tt < RG_FEW; ++tt) sa[tt] = si[tt] = 0.0f;
        for (int k = lane; k < bw; k += 32) {
            const float wa = to_f32<TW>(ra[k]), wi = to_f32<TW>(ri[k]);
#pragma unroll
            for (int tt = 0; tt < RG_FEW; ++tt) {
                sa[tt] = fmaf(wa, u_s[tt * bw + k], sa[tt]);
                si[tt] = fmaf(wi, u_s[tt * bw + k], si[tt]);
            }
        }
        float mine_a = 0.0f, mine_i = 0.0f;
#pragma unroll
        for (int tt = 0; tt < RG_FEW; ++tt) {
            const float ta = warp_sum(sa[tt]), ti = warp_sum(si[tt]);
            if (lane == tt) { mine_a = ta; mine_i = ti; }
        }
        if (lane < n_here) {
            const int c = b * bw + o;
            const float r = 1.0f / (1.0f + expf(-(mine_a + b_a[c])));
            const float g = 1.0f / (1.0f + expf(-(mine_i + b_i[c])));
            const float log_a = rate[c] * r;
            const long at = (long)(t0 + lane) * o_ld + c;
            a_out[at] = expf(log_a);
            b_out[at] = sqrtf(-expm1f(2.0f * log_a)) * g * u_s[lane * bw + o];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128) rglru_scan_kernel(
    const float* __restrict__ a, const float* __restrict__ bx, long ab_ld, const T* __restrict__ proj, long ld,
    const float* __restrict__ bias, float* __restrict__ state, long state_stride, const int* __restrict__ req_start,
    const int* __restrict__ req_ctx, const int* __restrict__ req_qlen, const int* __restrict__ req_slot,
    T* __restrict__ out, long out_ld, int width, int taps) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int start = req_start[r], ctx = req_ctx[r], qlen = req_qlen[r];
    float* row = state + (long)req_slot[r] * state_stride;
    float S = ctx > 0 ? row[c] : 0.0f;
    const float yb = bias[c], xb = bias[width + c];
#pragma unroll 4
    for (int i = 0; i < qlen; ++i) {
        const long t = start + i;
        S = a[t * ab_ld + c] * S + bx[t * ab_ld + c];
        const float z = to_f32<T>(proj[t * ld + c]) + yb;
        const float y = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        out[t * out_ld + c] = from_f32<T>(S * y);
    }
    row[c] = S;
    // the kept rows: row k is position ctx + qlen - (taps - 1) + k, from this step's rows or from the rows kept before
    // (old row k + qlen: read at or ahead of the place being written, so the shift works in place)
    float* tail = row + width;
    for (int k = 0; k < taps - 1; ++k) {
        const int p = ctx + qlen - (taps - 1) + k;
        float x = 0.0f;
        if (p >= ctx) x = to_f32<T>(proj[(long)(start + p - ctx) * ld + width + c]) + xb;
        else if (p >= 0) x = tail[(long)(k + qlen) * width + c];
        tail[(long)k * width + c] = x;
    }
}

// The same recurrence with a request's tokens cut into 32 segments that run side by side: each (segment, channel)
// thread first folds its segment into (product of a, result from zero), the carries are chained through shared memory,
// and a second walk from the carry writes the outputs.  The sums' order depends on the cut, so the 32-bit path, whose
// results must not, keeps the kernel above.
#define RG_SEGS 32
template <typename T>
__global__ void __launch_bounds__(32 * RG_SEGS) rglru_scan_split_kernel(
    const float* __restrict__ a, const float* __restrict__ bx, long ab_ld, const T* __restrict__ proj, long ld,
    const float* __restrict__ bias, float* __restrict__ state, long state_stride, const int* __restrict__ req_start,
    const int* __restrict__ req_ctx, const int* __restrict__ req_qlen, const int* __restrict__ req_slot,
    T* __restrict__ out, long out_ld, int width, int taps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float A_s[RG_SEGS][33], B_s[RG_SEGS][33];
    const int r = blockIdx.x, cl = threadIdx.x & 31, seg = threadIdx.x >> 5;
    const int c = blockIdx.y * 32 + cl;
    const bool live = c < width;
    const int start = req_start[r], ctx = req_ctx[r], qlen = req_qlen[r];
    const int len = (qlen + RG_SEGS - 1) / RG_SEGS;
    const int t0 = min(qlen, seg * len), t1 = min(qlen, t0 + len);
    float A = 1.0f, B = 0.0f;
    if (live) {
#pragma unroll 4
        for (int i = t0; i < t1; ++i) {
            const long t = start + i;
            const float av = a[t * ab_ld + c];
            B = fmaf(av, B, bx[t * ab_ld + c]);
            A *= av;
        }
    }
    A_s[seg][cl] = A;
    B_s[seg][cl] = B;
    __syncthreads();
    if (!live) return;
    float* row = state + (long)req_slot[r] * state_stride;
    float S = ctx > 0 ? row[c] : 0.0f;
    for (int k = 0; k < seg; ++k) S = fmaf(A_s[k][cl], S, B_s[k][cl]);
    const float yb = bias[c];
#pragma unroll 4
    for (int i = t0; i < t1; ++i) {
        const long t = start + i;
        S = fmaf(a[t * ab_ld + c], S, bx[t * ab_ld + c]);
        const float z = to_f32<T>(proj[t * ld + c]) + yb;
        const float y = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        out[t * out_ld + c] = from_f32<T>(S * y);
    }
    if (seg != RG_SEGS - 1) return;                     // the last segment ends with the request's new state
    row[c] = S;
    const float xb = bias[width + c];
    float* tail = row + width;
    for (int k = 0; k < taps - 1; ++k) {
        const int p = ctx + qlen - (taps - 1) + k;
        float x = 0.0f;
        if (p >= ctx) x = to_f32<T>(proj[(long)(start + p - ctx) * ld + width + c]) + xb;
        else if (p >= 0) x = tail[(long)(k + qlen) * width + c];
        tail[(long)k * width + c] = x;
    }
}

// proj: [n, 2 width] = y_pre | x_pre; bias: [2 width] float; conv_w: [width][taps] float; state rows:
// width * taps floats.  u, a, bx: float [n, width] scratch.  out: [n, width] = S * y in the activations' type.
FL_API int fl_rglru(const void* proj, int dtype, long ld, const float* bias, const float* conv_w, const float* conv_b,
                    const void* w_a, const void* w_i, int w_dtype, const float* b_a, const float* b_i, const float* rate,
                    float* state, long state_stride, const int* tok_req, const int* positions, const int* req_start,
                    const int* req_ctx, const int* req_qlen, const int* req_slot, int n_tokens, int n_requests,
                    float* u, float* a, float* bx, long s_ld, void* out, long out_ld, int width, int blocks, int taps,
                    int fixed_order, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (blocks < 1 || width % blocks || taps < 1 || taps > RG_MAX_TAPS) return (int)cudaErrorInvalidValue;
    const int bw = width / blocks;
    const size_t smem = (size_t)RG_TT * bw * sizeof(float);
    if (smem > 48 * 1024 || blocks > 65535) return (int)cudaErrorInvalidValue;
    int rc = 0;
    const bool four = width % 4 == 0 && ld % 4 == 0 && s_ld % 4 == 0 && state_stride % 4 == 0 && ((uintptr_t)proj % 16) == 0 &&
                      ((uintptr_t)u % 16) == 0 && ((uintptr_t)state % 16) == 0 && ((uintptr_t)bias % 16) == 0 &&
                      ((uintptr_t)conv_b % 16) == 0;
    if (four) {
        FL_DISPATCH(dtype, T, rc = fl_launch(rglru_conv4_kernel<T>, dim3(n_tokens, (width / 4 + 255) / 256), dim3(256), 0,
                                             stream, (const T*)proj, ld, bias, conv_w, conv_b, (const float*)state,
                                             state_stride, tok_req, positions, req_start, req_ctx, req_slot, u, s_ld, width,
                                             taps));
    } else {
        FL_DISPATCH(dtype, T, rc = fl_launch(rglru_conv_kernel<T>, dim3(n_tokens, (width + 255) / 256), dim3(256), 0, stream,
                                             (const T*)proj, ld, bias, conv_w, conv_b, (const float*)state, state_stride,
                                             tok_req, positions, req_start, req_ctx, req_slot, u, s_ld, width, taps));
    }
    if (rc) return rc;
    const int tiles = (n_tokens + RG_TT - 1) / RG_TT;
    const int threads = bw >= 256 ? 256 : ((bw + 31) / 32) * 32;
    const int vec = bw % 8 == 0 && ((uintptr_t)w_a % 16) == 0 && ((uintptr_t)w_i % 16) == 0;
    dim3 ggrid(tiles, blocks, (bw + threads - 1) / threads);
#define FL_RG_GATES(VEC)                                                                                               \
    FL_DISPATCH(w_dtype, TW, rc = fl_launch(rglru_gates_kernel<TW, VEC>, ggrid, dim3(threads), smem, stream,           \
                                            (const float*)u, s_ld, (const TW*)w_a, (const TW*)w_i, b_a, b_i, rate, a, bx, \
                                            s_ld, n_tokens, width, bw))
    if (!fixed_order && n_tokens < 64) {                // a handful of tokens: a warp an output
        int z = (bw + 7) / 8;
        const int few_tiles = (n_tokens + RG_FEW - 1) / RG_FEW;
        while (z > 1 && (long)few_tiles * blocks * z > 1024) z = (z + 1) / 2;
        FL_DISPATCH(w_dtype, TW, rc = fl_launch(rglru_gates_few_kernel<TW>, dim3(few_tiles, blocks, z), dim3(256),
                                                (size_t)RG_FEW * bw * sizeof(float), stream, (const float*)u, s_ld,
                                                (const TW*)w_a, (const TW*)w_i, b_a, b_i, rate, a, bx, s_ld, n_tokens,
                                                width, bw));
    } else if (vec) { FL_RG_GATES(true); } else { FL_RG_GATES(false); }
#undef FL_RG_GATES
    if (rc) return rc;
    if (!fixed_order && n_tokens > 32 * n_requests) {   // prompt portions: the tokens of a request side by side
        FL_DISPATCH(dtype, T, return fl_launch(rglru_scan_split_kernel<T>, dim3(n_requests, (width + 31) / 32),
                                               dim3(32 * RG_SEGS), 0, stream, (const float*)a, (const float*)bx, s_ld,
                                               (const T*)proj, ld, bias, state, state_stride, req_start, req_ctx, req_qlen,
                                               req_slot, (T*)out, out_ld, width, taps));
    }
    FL_DISPATCH(dtype, T, return fl_launch(rglru_scan_kernel<T>, dim3(n_requests, (width + 127) / 128), dim3(128), 0, stream,
                                           (const float*)a, (const float*)bx, s_ld, (const T*)proj, ld, bias, state,
                                           state_stride, req_start, req_ctx, req_qlen, req_slot, (T*)out, out_ld, width,
                                           taps));
    return 0;
}
