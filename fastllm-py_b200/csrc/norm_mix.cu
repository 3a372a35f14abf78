// Layer norm over the residual stream, the average of two normed rows, a scaled residual add and a
// one-argument activation.
//
//   add_layernorm   x += scale * delta (when there is a pending sum), out = (x - mean) / sqrt(var + eps) * w + b with
//                   the variance as the mean of the squared deviations (two passes over the row, which waits in shared
//                   memory); with `rows` only those rows are normed and x is not written back
//   rms_mix         out = weight * (a / rms(a) * wa + b / rms(b) * wb): two mixers' results, each normed over the
//                   width, averaged (`dtype` is the type of out and of whichever of a and b is a tensor)
//   scaled_add      x += scale * delta
//   activation      out = f(x, 1) for the gated units' f (relu squared among them): a feed-forward without a gate
//
// A sum that waits as the split-K partial sums of the product that made it (`splits` float slabs, `split_stride`
// floats apart, rows `ld` apart) is added up in slab order while it is read, in float, without a kernel of its own.
//
// All arithmetic is float; a row's sums depend on the row alone.
#include "common.cuh"

// Element `idx` of a tensor of T, or (splits > 0) of the float slabs behind the same pointer, added in slab order.
template <typename T>
__device__ __forceinline__ float nm_read(const T* p, long idx, int splits, long split_stride) {
    if (splits > 0) {
        const float* f = reinterpret_cast<const float*>(p);
        float sum = f[idx];
        for (int k = 1; k < splits; ++k) sum += f[(long)k * split_stride + idx];
        return sum;
    }
    return to_f32<T>(p[idx]);
}

template <typename TD, typename TW, typename TO>
__global__ void __launch_bounds__(256) add_layernorm_kernel(float* __restrict__ x, long x_ld, const TD* __restrict__ delta,
                                                            long d_ld, float scale, const TW* __restrict__ w,
                                                            const TW* __restrict__ b, TO* __restrict__ out, long out_ld,
                                                            int dim, float eps, const int* __restrict__ rows,
                                                            int write_back, int splits, long split_stride) {
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
            v += scale * nm_read<TD>(delta, src * d_ld + i, splits, split_stride);
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
                            float eps, const int* rows, int splits, long split_stride, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if ((size_t)dim * sizeof(float) > 48 * 1024 || (splits > 0 && d_dtype != FL_F32)) return (int)cudaErrorInvalidValue;
    const int write_back = rows ? 0 : 1;
    FL_DISPATCH(d_dtype, TD, FL_DISPATCH(w_dtype, TW, FL_DISPATCH(out_dtype, TO,
        return fl_launch(add_layernorm_kernel<TD, TW, TO>, dim3(n_rows), dim3(256), (size_t)dim * sizeof(float), stream, x,
                         x_ld, (const TD*)delta, d_ld, scale, (const TW*)w, (const TW*)b, (TO*)out, out_ld, dim, eps, rows,
                         write_back, splits, split_stride))));
    return 0;
}

template <typename T, typename TW>
__global__ void __launch_bounds__(256) rms_mix_kernel(const T* __restrict__ a, long a_ld, const T* __restrict__ b, long b_ld,
                                                      const TW* __restrict__ wa, const TW* __restrict__ wb, T* __restrict__ out,
                                                      long out_ld, int dim, float eps, float weight, int a_splits,
                                                      long a_stride, int b_splits, long b_stride) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float mix_row[];                  // [2][dim]: both rows, read (and added up) once
    __shared__ float scratch[32];
    const long r = blockIdx.x;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float va = nm_read<T>(a, r * a_ld + i, a_splits, a_stride), vb = nm_read<T>(b, r * b_ld + i, b_splits, b_stride);
        mix_row[i] = va;
        mix_row[dim + i] = vb;
        sa += va * va;
        sb += vb * vb;
    }
    const float ia = 1.0f / sqrtf(block_sum(sa, scratch) / (float)dim + eps);
    const float ib = 1.0f / sqrtf(block_sum(sb, scratch) / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float va = mix_row[i] * ia * to_f32<TW>(wa[i]);
        const float vb = mix_row[dim + i] * ib * to_f32<TW>(wb[i]);
        out[r * out_ld + i] = from_f32<T>(weight * (va + vb));
    }
}

FL_API int fl_rms_mix(const void* a, long a_ld, const void* b, long b_ld, int dtype, const void* wa, const void* wb,
                      int w_dtype, void* out, long out_ld, int n_rows, int dim, float eps, float weight, int a_splits,
                      long a_stride, int b_splits, long b_stride, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if ((size_t)dim * 2 * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        return fl_launch(rms_mix_kernel<T, TW>, dim3(n_rows), dim3(256), (size_t)dim * 2 * sizeof(float), stream, (const T*)a,
                         a_ld, (const T*)b, b_ld, (const TW*)wa, (const TW*)wb, (T*)out, out_ld, dim, eps, weight, a_splits,
                         a_stride, b_splits, b_stride)));
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
