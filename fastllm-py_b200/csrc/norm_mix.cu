// Layer norm over the residual stream, the average of two normed rows, a scaled residual add and a
// one-argument activation.
//
//   add_layernorm   x += scale * delta (when there is a pending sum), out = (x - mean) / sqrt(var + eps) * w + b with
//                   the variance as the mean of the squared deviations (two passes over the row, which waits in shared
//                   memory); with `rows` only those rows are normed and x is not written back
//   rms_mix         out = weight * (a / rms(a) * wa + b / rms(b) * wb): two mixers' results, each normed over the
//                   width, averaged
//   scaled_add      x += scale * delta
//   activation      out = f(x, 1) for the gated units' f (relu squared among them): a feed-forward without a gate
//
// All arithmetic is float; a row's sums depend on the row alone.
#include "common.cuh"

template <typename TD, typename TW, typename TO>
__global__ void __launch_bounds__(256) add_layernorm_kernel(float* __restrict__ x, long x_ld, const TD* __restrict__ delta,
                                                            long d_ld, float scale, const TW* __restrict__ w,
                                                            const TW* __restrict__ b, TO* __restrict__ out, long out_ld,
                                                            int dim, float eps, const int* __restrict__ rows,
                                                            int write_back) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float ln_row[];                   // [dim]
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const long src = rows ? rows[r] : r;
    float* xr = x + src * x_ld;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = xr[i];
        if (delta != nullptr) {
            v += scale * to_f32<TD>(delta[src * d_ld + i]);
            if (write_back) xr[i] = v;
        }
        ln_row[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)dim;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float d = ln_row[i] - mean;
        sq += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        out[(long)r * out_ld + i] = from_f32<TO>((ln_row[i] - mean) * inv * to_f32<TW>(w[i]) + (b ? to_f32<TW>(b[i]) : 0.0f));
}

FL_API int fl_add_layernorm(float* x, long x_ld, const void* delta, int d_dtype, long d_ld, float scale, const void* w,
                            const void* b, int w_dtype, void* out, int out_dtype, long out_ld, int n_rows, int dim,
                            float eps, const int* rows, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if ((size_t)dim * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    const int write_back = rows ? 0 : 1;
    FL_DISPATCH(d_dtype, TD, FL_DISPATCH(w_dtype, TW, FL_DISPATCH(out_dtype, TO,
        return fl_launch(add_layernorm_kernel<TD, TW, TO>, dim3(n_rows), dim3(256), (size_t)dim * sizeof(float), stream, x,
                         x_ld, (const TD*)delta, d_ld, scale, (const TW*)w, (const TW*)b, (TO*)out, out_ld, dim, eps, rows,
                         write_back))));
    return 0;
}

template <typename T, typename TW>
__global__ void __launch_bounds__(256) rms_mix_kernel(const T* __restrict__ a, long a_ld, const T* __restrict__ b, long b_ld,
                                                      const TW* __restrict__ wa, const TW* __restrict__ wb, T* __restrict__ out,
                                                      long out_ld, int dim, float eps, float weight) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const long r = blockIdx.x;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float va = to_f32<T>(a[r * a_ld + i]), vb = to_f32<T>(b[r * b_ld + i]);
        sa += va * va;
        sb += vb * vb;
    }
    const float ia = 1.0f / sqrtf(block_sum(sa, scratch) / (float)dim + eps);
    const float ib = 1.0f / sqrtf(block_sum(sb, scratch) / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float va = to_f32<T>(a[r * a_ld + i]) * ia * to_f32<TW>(wa[i]);
        const float vb = to_f32<T>(b[r * b_ld + i]) * ib * to_f32<TW>(wb[i]);
        out[r * out_ld + i] = from_f32<T>(weight * (va + vb));
    }
}

FL_API int fl_rms_mix(const void* a, long a_ld, const void* b, long b_ld, int dtype, const void* wa, const void* wb,
                      int w_dtype, void* out, long out_ld, int n_rows, int dim, float eps, float weight,
                      cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        return fl_launch(rms_mix_kernel<T, TW>, dim3(n_rows), dim3(256), 0, stream, (const T*)a, a_ld, (const T*)b, b_ld,
                         (const TW*)wa, (const TW*)wb, (T*)out, out_ld, dim, eps, weight)));
    return 0;
}

template <typename TD>
__global__ void __launch_bounds__(256) scaled_add_kernel(float* __restrict__ x, long x_ld, const TD* __restrict__ delta,
                                                         long d_ld, int dim, float scale) {
    pdl_wait();
    pdl_trigger();
    const long r = blockIdx.x;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) x[r * x_ld + i] += scale * to_f32<TD>(delta[r * d_ld + i]);
}

FL_API int fl_scaled_add(float* x, long x_ld, const void* delta, int d_dtype, long d_ld, int n_rows, int dim, float scale,
                         cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    FL_DISPATCH(d_dtype, TD, return fl_launch(scaled_add_kernel<TD>, dim3(n_rows), dim3(256), 0, stream, x, x_ld,
                                              (const TD*)delta, d_ld, dim, scale));
    return 0;
}

template <typename T>
__global__ void __launch_bounds__(256) activation_kernel(const T* __restrict__ x, long x_ld, T* __restrict__ out, long out_ld,
                                                         int cols, FlGate act) {
    pdl_wait();
    pdl_trigger();
    const long r = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < cols; i += gridDim.y * blockDim.x)
        out[r * out_ld + i] = from_f32<T>(fl_gated(to_f32<T>(x[r * x_ld + i]), 1.0f, act));
}

FL_API int fl_activation(const void* x, int dtype, long x_ld, void* out, long out_ld, int n_rows, int cols, int act,
                         float p0, float p1, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (act < 0 || act >= FL_ACT_COUNT) return (int)cudaErrorInvalidValue;
    int col_blocks = (cols + 1023) / 1024;
    if (col_blocks > 16) col_blocks = 16;
    FL_DISPATCH(dtype, T, return fl_launch(activation_kernel<T>, dim3(n_rows, col_blocks), dim3(256), 0, stream,
                                           (const T*)x, x_ld, (T*)out, out_ld, cols, FlGate{act, p0, p1}));
    return 0;
}
