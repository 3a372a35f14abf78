// Grouped-query attention without rotation, whose scores pass a soft cap and take a learned bias by distance, over a
// sliding window that also keeps a sequence's first tokens, with a sink in the softmax's denominator.
//
// Per token: q, k, v come from one product (biases added here); q and k are each divided by the root mean square of
// the WHOLE projection (all heads at once) and multiplied by a weight per coordinate; v may be blended with the values
// that an earlier layer of the model made for the same token, v <- (1 - lambda) v + lambda v_first.  Query i sees key j
// when j <= i and (i - j < window or j < keep_first).  With c the cap and b the bias table,
//     s_ij = c tanh(q_i . k_j * scale / c) + b[bucket(i - j), head]          (no cap when c <= 0; no bias without a table)
//     p_ij = exp(s_ij) / (exp(sink_head) + sum_j' exp(s_ij'))                (the sink has no key and no value)
// bucket() is a table by distance made by the caller; distances beyond its end take its last entry.
//
// A cache page is [kv_heads, page_size, dim + vdim]: a token's key, then its value (the blended one).
//
//   sink_prep             per token: biases, both norms, the blend; q to its buffer, k and v to the token's cache rows
//   sink_attention_simt   per (token, query head): CUDA cores, any sizes, bfloat16 or true 32-bit; key tiles start at
//                         multiples of 128 of the absolute position and tiles without a visible key are skipped, so
//                         every sum's order depends on the token's own position only
//
// Scores, softmax, norms and the blend are float.
#include "common.cuh"

#define SINK_TILE 128

// proj row: heads x dim queries, kv_heads x dim keys, kv_heads x vdim values.  bias: the same layout, float, or null.
// v_mode 0: values as they are; 1: also kept in v_first (float, [n, kv_heads x vdim]); 2: blended with v_first.
template <typename T, typename TQ>
__global__ void __launch_bounds__(256) sink_prep_kernel(
    const T* __restrict__ proj, long ld, const float* __restrict__ bias, const float* __restrict__ q_w,
    const float* __restrict__ k_w, float eps, TQ* __restrict__ q_out, long q_ld, int heads, int kv_heads, int dim, int vdim,
    int v_mode, float lambda, float* __restrict__ v_first, long vf_ld, const int* __restrict__ slots,
    T* __restrict__ cache, long page_stride, int page_size) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const T* row = proj + (long)t * ld;
    const int nq = heads * dim, nk = kv_heads * dim, nv = kv_heads * vdim;
    float ssq = 0.0f, ssk = 0.0f;
    for (int i = tid; i < nq; i += blockDim.x) {
        const float a = to_f32<T>(row[i]) + (bias ? bias[i] : 0.0f);
        ssq += a * a;
    }
    for (int i = tid; i < nk; i += blockDim.x) {
        const float a = to_f32<T>(row[nq + i]) + (bias ? bias[nq + i] : 0.0f);
        ssk += a * a;
    }
    ssq = block_sum(ssq, scratch);
    ssk = block_sum(ssk, scratch);
    const float inv_q = q_w != nullptr ? 1.0f / sqrtf(ssq / (float)nq + eps) : 1.0f;
    const float inv_k = k_w != nullptr ? 1.0f / sqrtf(ssk / (float)nk + eps) : 1.0f;
    TQ* qo = q_out + (long)t * q_ld;
    for (int i = tid; i < nq; i += blockDim.x) {
        const float a = to_f32<T>(row[i]) + (bias ? bias[i] : 0.0f);
        qo[i] = from_f32<TQ>(q_w != nullptr ? a * inv_q * q_w[i] : a);
    }
    if (cache == nullptr) return;
    const int slot = slots[t];
    const long page = slot / page_size;
    const int off = slot - (int)page * page_size;
    const int row_w = dim + vdim;
    T* dst = cache + page * page_stride + (long)off * row_w;                  // head g's row: + g * page_size * row_w
    const long head_stride = (long)page_size * row_w;
    for (int i = tid; i < nk; i += blockDim.x) {
        const int g = i / dim, d = i - g * dim;
        const float a = to_f32<T>(row[nq + i]) + (bias ? bias[nq + i] : 0.0f);
        dst[g * head_stride + d] = from_f32<T>(k_w != nullptr ? a * inv_k * k_w[i] : a);
    }
    for (int i = tid; i < nv; i += blockDim.x) {
        const int g = i / vdim, d = i - g * vdim;
        float a = to_f32<T>(row[nq + nk + i]) + (bias ? bias[nq + nk + i] : 0.0f);
        if (v_mode == 1) v_first[(long)t * vf_ld + i] = a;
        else if (v_mode == 2) a = (1.0f - lambda) * a + lambda * v_first[(long)t * vf_ld + i];
        dst[g * head_stride + dim + d] = from_f32<T>(a);
    }
}

FL_API int fl_sink_prep(const void* proj, int dtype, long ld, const float* bias, const float* q_w, const float* k_w, float eps,
                        void* q_out, int q_dtype, long q_ld, int n_tokens, int heads, int kv_heads, int dim, int vdim,
                        int v_mode, float lambda, float* v_first, long vf_ld, const int* slots, void* cache,
                        long page_stride, int page_size, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (v_mode < 0 || v_mode > 2 || (v_mode != 0 && v_first == nullptr)) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, FL_DISPATCH(q_dtype, TQ,
        return fl_launch(sink_prep_kernel<T, TQ>, dim3(n_tokens), dim3(256), 0, stream, (const T*)proj, ld, bias, q_w, k_w,
                         eps, (TQ*)q_out, q_ld, heads, kv_heads, dim, vdim, v_mode, lambda, v_first, vf_ld, slots, (T*)cache,
                         page_stride, page_size)));
    return 0;
}

// The score of key j for a query at `pos` from the dot product.
__device__ __forceinline__ float sink_score(float dot, float scale, float cap, const int* bucket_of, int n_dist,
                                            const float* rel, int heads, int h, int dist) {
    float s = dot * scale;
    if (cap > 0.0f) s = cap * tanhf(s / cap);
    if (rel != nullptr) s += rel[(long)bucket_of[min(dist, n_dist - 1)] * heads + h];
    return s;
}

template <typename T, typename TQ>
__global__ void __launch_bounds__(SINK_TILE) sink_attention_simt_kernel(
    const TQ* __restrict__ q, long q_ld, T* __restrict__ out, long out_ld, const T* __restrict__ cache, long page_stride,
    int page_size, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req,
    const int* __restrict__ positions, int heads, int kv_heads, int dim, int vdim, int window, int keep_first, float scale,
    float cap, const int* __restrict__ bucket_of, int n_dist, const float* __restrict__ rel,
    const float* __restrict__ sink) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char sink_smem[];
    long* off_s = reinterpret_cast<long*>(sink_smem);                 // [TILE] element offset of each key row's value part
    float* p_s = reinterpret_cast<float*>(off_s + SINK_TILE);         // [TILE] numerators
    float* q_s = p_s + SINK_TILE;                                     // [dim]
    __shared__ float scratch[32];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int g = h / (heads / kv_heads);
    const int pos = positions[t];
    const int* bt = block_table + (long)tok_req[t] * bt_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int kept = min(keep_first, lo);                             // keys [0, kept) are seen beside [lo, pos]
    const int row_w = dim + vdim;

    const TQ* qr = q + (long)t * q_ld + (long)h * dim;
    for (int d = tid; d < dim; d += SINK_TILE) q_s[d] = to_f32<TQ>(qr[d]);
    __syncthreads();

    // the sink is a term exp(sink) of the denominator without a value: the running maximum and sum start from it
    float m = sink != nullptr ? sink[h] : -CUDART_INF_F;
    float l = sink != nullptr ? 1.0f : 0.0f;
    float acc[2] = {0.0f, 0.0f};                                      // value columns tid and tid + TILE
    for (int tile = 0; tile <= pos; tile += SINK_TILE) {
        if (tile >= kept && tile + SINK_TILE <= lo) continue;         // no visible key in this tile
        const int j = tile + tid;
        const bool valid = j <= pos && (j >= lo || j < kept);
        float s = -CUDART_INF_F;
        long off = 0;
        if (valid) {
            const long page = bt[j / page_size];
            off = page * page_stride + ((long)g * page_size + j % page_size) * row_w;
            const T* kp = cache + off;
            float dot = 0.0f;
            for (int d = 0; d < dim; ++d) dot += q_s[d] * to_f32<T>(kp[d]);
            s = sink_score(dot, scale, cap, bucket_of, n_dist, rel, heads, h, pos - j);
        }
        off_s[tid] = off + dim;
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float p = valid ? expf(s - m_new) : 0.0f;
        p_s[tid] = p;
        const float tile_sum = block_sum(p, scratch);     // its barriers also publish p_s / off_s
        const float corr = expf(m - m_new);               // 0 at the first tile without a sink (m = -inf)
        l = l * corr + tile_sum;
        const int j_end = min(SINK_TILE, pos - tile + 1);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int d = tid + c * SINK_TILE;
            if (d < vdim) {
                float a = acc[c] * corr;
                for (int jj = 0; jj < j_end; ++jj) {
                    const int jk = tile + jj;
                    if (jk >= lo || jk < kept) a += p_s[jj] * to_f32<T>(cache[off_s[jj] + d]);
                }
                acc[c] = a;
            }
        }
        m = m_new;
        __syncthreads();                                  // p_s / off_s are rewritten by the next tile
    }
    T* dst = out + (long)t * out_ld + (long)h * vdim;
#pragma unroll
    for (int c = 0; c < 2; ++c)
        if (tid + c * SINK_TILE < vdim) dst[tid + c * SINK_TILE] = from_f32<T>(acc[c] / l);
}

// q: [n_tokens, q_ld], head h at columns [h * dim, (h + 1) * dim); out: [n_tokens, out_ld], head h at columns
// [h * vdim, (h + 1) * vdim).  window <= 0: all keys.  bucket_of: [n_dist] rows of rel ([rows, heads] float) by distance.
FL_API int fl_sink_attention_simt(const void* q, int q_dtype, long q_ld, void* out, long out_ld, const void* cache, int dtype,
                                  long page_stride, int page_size, const int* block_table, int bt_stride,
                                  const int* tok_req, const int* positions, int n_tokens, int heads, int kv_heads, int dim,
                                  int vdim, int window, int keep_first, float scale, float cap, const int* bucket_of,
                                  int n_dist, const float* rel, const float* sink, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (vdim < 1 || vdim > 2 * SINK_TILE || dim < 1 || dim > 4096 || heads > 65535 || heads % kv_heads ||
        (rel != nullptr && (bucket_of == nullptr || n_dist < 1)))
        return (int)cudaErrorInvalidValue;
    const size_t smem = SINK_TILE * (sizeof(long) + sizeof(float)) + (size_t)dim * sizeof(float);
    dim3 grid(n_tokens, heads);
    FL_DISPATCH(dtype, T, FL_DISPATCH(q_dtype, TQ,
        return fl_launch(sink_attention_simt_kernel<T, TQ>, grid, dim3(SINK_TILE), smem, stream, (const TQ*)q, q_ld, (T*)out,
                         out_ld, (const T*)cache, page_stride, page_size, block_table, bt_stride, tok_req, positions, heads,
                         kv_heads, dim, vdim, window, keep_first, scale, cap, bucket_of, n_dist, rel, sink)));
    return 0;
}
