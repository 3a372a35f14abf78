// Kernels of the post-norm block with a short input convolution and a gated residual, and of the
// embedding with a hashed table of token pairs.
//
// The block: a sublayer reads the residual stream x itself (no norm in front), through a causal
// convolution over time on every channel; its result is gated, normed and added:
//     h  = x                       hc_t = h_t + sum_j w[:, j] h_(t - taps + 1 + j)      (zeros before position 0)
//     y  = sublayer(hc) * sigmoid(W_g h + b_g)
//     x <- x + y / sqrt(mean(y^2) + eps) * w_out
// The last taps - 1 rows h of a request are its state, kept by position: ring[(position) mod (taps - 1)].
//
//   input_conv       per token: h (x in the activation type) and hc; rows before the step's first come from the ring
//   gated_norm_add   per token: the gate, the norm and the add; also files the row's x (as it was before the add:
//                    the input the sublayer's convolution saw) into the ring when it is among the request's last
//                    taps - 1 rows of the step.  It runs after every reader of the ring in this step, so the ring is
//                    never read and written by one launch
//   sigmoid_gate     a[t, i] *= sigmoid(g[t, i])  (an output gate inside a mixer)
//   pair_embed       x[t] = table[id_t] * scale + pairs[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets], row
//                    `buckets` for a request's first token; the token before a step's first is per-request state,
//                    read and rewritten by the block of the request's first row only
//
// All arithmetic is float; the residual stream is float in both precisions.
#include "common.cuh"

// V consecutive channels a thread (4 where width, the row pitches and the bases allow 16-byte accesses, else 1): a row
// is spread over gridDim.y blocks, so a step of a few rows still has its loads in flight side by side.  Every element
// is the same chain of fused multiply-adds whichever form runs.
template <int V> struct ConvRow { float v[V]; };

template <int V> __device__ __forceinline__ ConvRow<V> conv_load(const float* p) {
    ConvRow<V> r;
    if constexpr (V == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        r.v[0] = q.x; r.v[1] = q.y; r.v[2] = q.z; r.v[3] = q.w;
    } else {
        r.v[0] = *p;
    }
    return r;
}

template <typename TO, int V> __device__ __forceinline__ void conv_store(TO* p, const ConvRow<V>& r) {
    if constexpr (V == 4 && sizeof(TO) == 2) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(r.v[0], r.v[1]), hi = __floats2bfloat162_rn(r.v[2], r.v[3]);
        uint2 q;
        q.x = *reinterpret_cast<unsigned*>(&lo);
        q.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(p) = q;
    } else if constexpr (V == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    } else {
        p[0] = from_f32<TO>(r.v[0]);
    }
}

template <typename TO, int V>
__global__ void __launch_bounds__(256) input_conv_kernel(
    const float* __restrict__ x, long x_ld, const float* __restrict__ w, int taps, const float* __restrict__ ring,
    long ring_slot_stride, const int* __restrict__ positions, const int* __restrict__ tok_req,
    const int* __restrict__ req_start, const int* __restrict__ req_slot, TO* __restrict__ h, long h_ld,
    TO* __restrict__ hc, long hc_ld, int width) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int i = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (i >= width) return;
    const int r = tok_req[t];
    const int pos = positions[t], start = req_start[r];
    const int back = taps - 1;
    const float* ring_r = ring != nullptr ? ring + (long)req_slot[r] * ring_slot_stride : nullptr;
    const ConvRow<V> xi = conv_load<V>(x + (long)t * x_ld + i);
    ConvRow<V> acc;
#pragma unroll
    for (int c = 0; c < V; ++c) acc.v[c] = 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int k = back - j;                            // rows back in time
        ConvRow<V> v;
        if (k == 0) v = xi;
        else if (pos - k < 0) continue;                    // zeros before the sequence's start (acc + w * 0 == acc)
        else if (t - k >= start) v = conv_load<V>(x + (long)(t - k) * x_ld + i);
        else v = conv_load<V>(ring_r + (long)((pos - k) % back) * width + i);
#pragma unroll
        for (int c = 0; c < V; ++c) acc.v[c] = __fmaf_rn(w[(long)(i + c) * taps + j], v.v[c], acc.v[c]);
    }
    if (h != nullptr) conv_store<TO, V>(h + (long)t * h_ld + i, xi);
#pragma unroll
    for (int c = 0; c < V; ++c) acc.v[c] = xi.v[c] + acc.v[c];
    conv_store<TO, V>(hc + (long)t * hc_ld + i, acc);
}

static inline bool fl_rows_take_vectors(const void* p, long ld, int elem_bytes) {
    return p == nullptr || (((uintptr_t)p % (4 * elem_bytes)) == 0 && ld % 4 == 0);
}

// w: [width, taps] float; ring: [slots, >= (taps - 1) * width] float (may be null when taps == 1).
FL_API int fl_input_conv(const float* x, long x_ld, const float* w, int taps, const float* ring, long ring_slot_stride,
                         const int* positions, const int* tok_req, const int* req_start, const int* req_slot, void* h,
                         long h_ld, void* hc, long hc_ld, int out_dtype, int n_tokens, int width, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (taps < 1 || (taps > 1 && ring == nullptr)) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(out_dtype, TO, {
        const bool vec = width % 4 == 0 && fl_rows_take_vectors(x, x_ld, 4) && fl_rows_take_vectors(ring, ring_slot_stride, 4) &&
                         fl_rows_take_vectors(h, h_ld, sizeof(TO)) && fl_rows_take_vectors(hc, hc_ld, sizeof(TO));
        if (vec)
            return fl_launch(input_conv_kernel<TO, 4>, dim3(n_tokens, (width / 4 + 255) / 256), dim3(256), 0, stream, x, x_ld,
                             w, taps, ring, ring_slot_stride, positions, tok_req, req_start, req_slot, (TO*)h, h_ld,
                             (TO*)hc, hc_ld, width);
        return fl_launch(input_conv_kernel<TO, 1>, dim3(n_tokens, (width + 255) / 256), dim3(256), 0, stream, x, x_ld, w,
                         taps, ring, ring_slot_stride, positions, tok_req, req_start, req_slot, (TO*)h, h_ld, (TO*)hc,
                         hc_ld, width);
    });
    return 0;
}

// One block a row, blockDim a function of the width alone (so equal rows give equal sums wherever they sit).  y is
// either a matrix of TD or, with y_splits > 0, the float partial sums of a product whose K was split: y_splits slabs
// of [rows, y_ld] floats y_split_stride apart, added here in slab order and rounded to TD first (what the reduce
// kernel would have written).  The gate likewise, with g_splits.
template <typename TD, int V> __device__ __forceinline__ ConvRow<V> td_load(const TD* p) {
    ConvRow<V> r;
    if constexpr (V == 4 && sizeof(TD) == 2) {
        const uint2 q = *reinterpret_cast<const uint2*>(p);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
        r.v[0] = lo.x; r.v[1] = lo.y; r.v[2] = hi.x; r.v[3] = hi.y;
    } else if constexpr (V == 4) {
        r = conv_load<4>(reinterpret_cast<const float*>(p));
    } else {
        r.v[0] = to_f32<TD>(p[0]);
    }
    return r;
}

template <typename TD, int V>
__global__ void __launch_bounds__(1024) gated_norm_add_kernel(
    float* __restrict__ x, long x_ld, const void* __restrict__ y, long y_ld, int y_splits, long y_split_stride,
    const void* __restrict__ gate, long gate_ld, int g_splits, long g_split_stride, const float* __restrict__ gate_bias,
    const float* __restrict__ w, float eps, int width, float* __restrict__ ring, long ring_slot_stride, int taps, const int* __restrict__ positions,
    const int* __restrict__ tok_req, const int* __restrict__ req_start, const int* __restrict__ req_qlen,
    const int* __restrict__ req_slot) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) float gated_row[];     // [width]
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const TD* yr = y_splits > 0 ? nullptr : (const TD*)y + (long)t * y_ld;
    const float* yp = y_splits > 0 ? (const float*)y + (long)t * y_ld : nullptr;
    const TD* gr = (gate != nullptr && g_splits == 0) ? (const TD*)gate + (long)t * gate_ld : nullptr;
    const float* gp = (gate != nullptr && g_splits > 0) ? (const float*)gate + (long)t * gate_ld : nullptr;
    float* xr = x + (long)t * x_ld;
    // a row that one pass of the block covers (the usual case): x and the weight are asked for before the sum's
    // barrier, so the row's loads are all in flight together; the arithmetic is the same either way
    const bool one_pass = (int)blockDim.x * V >= width;
    const int i0 = threadIdx.x * V;
    ConvRow<V> x0, w0;
    if (one_pass && i0 < width) {
        x0 = conv_load<V>(xr + i0);
        w0 = conv_load<V>(w + i0);
    }
    float ss = 0.0f;
    for (int i = threadIdx.x * V; i < width; i += blockDim.x * V) {
        ConvRow<V> v;
        if (yp != nullptr) {
            v = conv_load<V>(yp + i);
            for (int s = 1; s < y_splits; ++s) {
                const ConvRow<V> p = conv_load<V>(yp + (long)s * y_split_stride + i);
#pragma unroll
                for (int c = 0; c < V; ++c) v.v[c] += p.v[c];
            }
#pragma unroll
            for (int c = 0; c < V; ++c) v.v[c] = to_f32<TD>(from_f32<TD>(v.v[c]));
        } else {
            v = td_load<TD, V>(yr + i);
        }
        if (gr != nullptr || gp != nullptr) {
            ConvRow<V> g;
            if (gp != nullptr) {
                g = conv_load<V>(gp + i);
                for (int s = 1; s < g_splits; ++s) {
                    const ConvRow<V> p = conv_load<V>(gp + (long)s * g_split_stride + i);
#pragma unroll
                    for (int c = 0; c < V; ++c) g.v[c] += p.v[c];
                }
#pragma unroll
                for (int c = 0; c < V; ++c) g.v[c] = to_f32<TD>(from_f32<TD>(g.v[c]));
            } else {
                g = td_load<TD, V>(gr + i);
            }
#pragma unroll
            for (int c = 0; c < V; ++c) {
                const float z = g.v[c] + (gate_bias != nullptr ? gate_bias[i + c] : 0.0f);
                v.v[c] = v.v[c] / (1.0f + expf(-z));
            }
        }
#pragma unroll
        for (int c = 0; c < V; ++c) {
            gated_row[i + c] = v.v[c];
            ss += v.v[c] * v.v[c];
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    float* file = nullptr;
    if (ring != nullptr && taps > 1) {
        const int r = tok_req[t];
        if (t >= req_start[r] + req_qlen[r] - (taps - 1))
            file = ring + (long)req_slot[r] * ring_slot_stride + (long)(positions[t] % (taps - 1)) * width;
    }
    for (int i = threadIdx.x * V; i < width; i += blockDim.x * V) {
        ConvRow<V> xi = one_pass ? x0 : conv_load<V>(xr + i);
        const ConvRow<V> wi = one_pass ? w0 : conv_load<V>(w + i);
        if (file != nullptr) conv_store<float, V>(file + i, xi);
#pragma unroll
        for (int c = 0; c < V; ++c) xi.v[c] = xi.v[c] + gated_row[i + c] * inv * wi.v[c];
        conv_store<float, V>(xr + i, xi);
    }
}

// gate may be null (no gate); ring may be null (nothing to file).  y_splits 0: y is [n_tokens, width] of `dtype`;
// the gate likewise with g_splits.
FL_API int fl_gated_norm_add(float* x, long x_ld, const void* y, long y_ld, int y_splits, long y_split_stride,
                             const void* gate, long gate_ld, int g_splits, long g_split_stride, int dtype,
                             const float* gate_bias, const float* w, float eps,
                             int n_tokens, int width, float* ring, long ring_slot_stride, int taps, const int* positions,
                             const int* tok_req, const int* req_start, const int* req_qlen, const int* req_slot,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, TD, {
        // four channels a thread where every row takes 16-byte (8-byte for bfloat16) accesses; which form runs, and
        // with how many threads, depends on the layer's width and buffers only, never on the step
        const int y_bytes = y_splits > 0 ? 4 : (int)sizeof(TD), g_bytes = g_splits > 0 ? 4 : (int)sizeof(TD);
        const bool vec = width % 4 == 0 && fl_rows_take_vectors(x, x_ld, 4) && fl_rows_take_vectors(y, y_ld, y_bytes) &&
                         y_split_stride % 4 == 0 && g_split_stride % 4 == 0 && fl_rows_take_vectors(gate, gate_ld, g_bytes) &&
                         fl_rows_take_vectors(ring, ring_slot_stride, 4) && fl_rows_take_vectors(w, 4, 4) &&
                         fl_rows_take_vectors(gate_bias, 4, 4);
        const int per_thread = vec ? 4 : 2;
        int threads = 64;
        while (threads < 1024 && threads * per_thread < width) threads *= 2;
        auto kernel = vec ? gated_norm_add_kernel<TD, 4> : gated_norm_add_kernel<TD, 1>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return fl_launch(kernel, dim3(n_tokens), dim3(threads), smem, stream, x, x_ld, y, y_ld, y_splits, y_split_stride,
                         gate, gate_ld, g_splits, g_split_stride, gate_bias, w, eps, width, ring, ring_slot_stride, taps,
                         positions, tok_req, req_start, req_qlen, req_slot);
    });
    return 0;
}

template <typename T>
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(T* __restrict__ a, long a_ld, const T* __restrict__ g, long g_ld,
                                                           int cols) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    T* ar = a + (long)t * a_ld;
    const T* gr = g + (long)t * g_ld;
    for (int i = threadIdx.x; i < cols; i += blockDim.x)
        ar[i] = from_f32<T>(to_f32<T>(ar[i]) / (1.0f + expf(-to_f32<T>(gr[i]))));
}

FL_API int fl_sigmoid_gate(void* a, long a_ld, const void* g, long g_ld, int dtype, int n_rows, int cols,
                           cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    FL_DISPATCH(dtype, T, return fl_launch(sigmoid_gate_kernel<T>, dim3(n_rows), dim3(256), 0, stream, (T*)a, a_ld,
                                           (const T*)g, g_ld, cols));
    return 0;
}

__device__ __forceinline__ int fed_token(int id, const int* fed, int n_fed) {
    return (id < 0 && fed != nullptr && -1 - id < n_fed) ? fed[-1 - id] : id;
}

template <typename TT>
__global__ void __launch_bounds__(256) pair_embed_kernel(
    const TT* __restrict__ table, long table_ld, const TT* __restrict__ pairs, long pairs_ld, const int* __restrict__ ids,
    float* __restrict__ out, long out_ld, int hidden, int vocab, int buckets, long mul_prev, long mul_cur, float scale,
    const int* __restrict__ tok_req, const int* __restrict__ req_start, const int* __restrict__ req_ctx,
    const int* __restrict__ req_qlen, const int* __restrict__ req_slot, int* __restrict__ last_token,
    int* __restrict__ status, const int* __restrict__ fed, int n_fed) {
    pdl_wait();
    pdl_trigger();
    __shared__ int before;
    const int t = blockIdx.x;
    const int r = tok_req[t], start = req_start[r];
    const int id = fed_token(ids[t], fed, n_fed);
    if (threadIdx.x == 0) {
        if (t > start) {
            before = fed_token(ids[t - 1], fed, n_fed);
        } else {                                           // the request's first row of the step: the state is this block's
            int* kept = last_token + req_slot[r];
            before = req_ctx[r] > 0 ? *kept : -1;
            *kept = fed_token(ids[start + req_qlen[r] - 1], fed, n_fed);
        }
    }
    __syncthreads();
    float* o = out + (long)t * out_ld;
    const int prev = before;
    if (id < 0 || id >= vocab || prev >= vocab) {
        if (threadIdx.x == 0) atomicCAS(status, 0, t + 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const long pair_row = prev < 0 ? (long)buckets : ((long)prev * mul_prev + (long)id * mul_cur) % (long)buckets;
    const TT* row = table + (long)id * table_ld;
    const TT* prow = pairs + pair_row * pairs_ld;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        o[i] = to_f32<TT>(row[i]) * scale + to_f32<TT>(prow[i]);
}

// pairs: [buckets + 1, hidden]; last_token: [slots] int.
FL_API int fl_pair_embed(const void* table, long table_ld, const void* pairs, long pairs_ld, int dtype, const int* ids,
                         float* out, long out_ld, int n_tokens, int hidden, int vocab, int buckets, long mul_prev,
                         long mul_cur, float scale, const int* tok_req, const int* req_start, const int* req_ctx,
                         const int* req_qlen, const int* req_slot, int* last_token, int* status, const int* fed, int n_fed,
                         cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (buckets < 1) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, TT, return fl_launch(pair_embed_kernel<TT>, dim3(n_tokens), dim3(256), 0, stream, (const TT*)table,
                                            table_ld, (const TT*)pairs, pairs_ld, ids, out, out_ld, hidden, vocab, buckets,
                                            mul_prev, mul_cur, scale, tok_req, req_start, req_ctx, req_qlen, req_slot,
                                            last_token, status, fed, n_fed));
    return 0;
}
