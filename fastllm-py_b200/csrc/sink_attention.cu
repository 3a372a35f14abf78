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
//   head_prep             the per-head form of the preparation, for attention whose q and k are normed head by head and
//                         rotated (see there); head_gate multiplies a head's result by a sigmoid
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

// ------------------------------------------------------------------ preparation head by head
// proj row: heads x dim queries, kv_heads x dim keys and (unless the keys serve as values) kv_heads x vdim values; bias:
// the same layout, float, or null.  Each query and key head passes, in this order:
//   norm_mode 1: an RMS norm over its dim elements, times q_w / k_w ([dim], shared by the heads; null: no weight)
//   rot > 0:     the rotation of its first `rot` dimensions by the row `position` of cos / sin ([positions, rot / 2]);
//                pair i is (2i, 2i + 1) with `interleaved`, else (i, i + rot / 2)
//   norm_mode 2: an RMS norm without weight, after the rotation
//   queries:     times 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1)      (temp_every <= 0: not)
// q goes to q_out, k to the token's cache row.  The value beside it is the projected value with its bias, or, with
// v_from_k, the key as projected (with its bias, before norm and rotation); vdim = dim then.
template <typename T, typename TQ>
__global__ void __launch_bounds__(256) head_prep_kernel(
    const T* __restrict__ proj, long ld, const float* __restrict__ bias, const float* __restrict__ q_w,
    const float* __restrict__ k_w, int norm_mode, float eps, int rot, int interleaved, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, const int* __restrict__ positions, float temp_coef, int temp_every, int v_from_k,
    TQ* __restrict__ q_out, long q_ld, int heads, int kv_heads, int dim, int vdim, const int* __restrict__ slots,
    T* __restrict__ cache, long page_stride, int page_size) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float prep_s[];                                 // [8 warps][dim]
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* row = proj + (long)t * ld;
    const int nq = heads * dim, nk = kv_heads * dim;
    const int pos = positions[t];
    const int half = rot / 2;
    const int slot = slots[t];
    const long page = slot / page_size;
    const int off = slot - (int)page * page_size;
    const int row_w = dim + vdim;
    T* dst = cache + page * page_stride + (long)off * row_w;          // head g's row: + g * page_size * row_w
    const long head_stride = (long)page_size * row_w;
    float* buf = prep_s + warp * dim;
    float factor = 1.0f;
    if (temp_every > 0) factor = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
    // (a block's eight warps take eight of the token's heads; blockIdx.y counts the eights)
    for (int idx = blockIdx.y * 8 + warp; idx < heads + kv_heads; idx += gridDim.y * 8) {
        const bool is_q = idx < heads;
        const int col0 = is_q ? idx * dim : nq + (idx - heads) * dim;
        T* krow = dst + (long)(idx - heads) * head_stride;
        float ss = 0.0f;
        for (int d = lane; d < dim; d += 32) {
            const float a = to_f32<T>(row[col0 + d]) + (bias ? bias[col0 + d] : 0.0f);
            buf[d] = a;
            ss += a * a;
            if (!is_q && v_from_k) krow[dim + d] = from_f32<T>(a);
        }
        __syncwarp();
        if (norm_mode == 1) {
            const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
            const float* w = is_q ? q_w : k_w;
            for (int d = lane; d < dim; d += 32) buf[d] = buf[d] * inv * (w ? w[d] : 1.0f);
            __syncwarp();
        }
        for (int i = lane; i < half; i += 32) {
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            const float c = cos_t[(long)pos * half + i], sn = sin_t[(long)pos * half + i];
            const float a = buf[ia], b = buf[ib];
            buf[ia] = a * c - b * sn;
            buf[ib] = b * c + a * sn;
        }
        __syncwarp();
        float inv = 1.0f;
        if (norm_mode == 2) {
            float s2 = 0.0f;
            for (int d = lane; d < dim; d += 32) s2 += buf[d] * buf[d];
            inv = 1.0f / sqrtf(warp_sum(s2) / (float)dim + eps);
        }
        if (is_q) {
            TQ* qo = q_out + (long)t * q_ld + (long)idx * dim;
            for (int d = lane; d < dim; d += 32) qo[d] = from_f32<TQ>(buf[d] * inv * factor);
        } else {
            for (int d = lane; d < dim; d += 32) krow[d] = from_f32<T>(buf[d] * inv);
        }
        __syncwarp();                                                 // buf is rewritten for the next head
    }
    if (!v_from_k) {
        const int nv = kv_heads * vdim;
        for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < nv; i += gridDim.y * blockDim.x) {
            const int g = i / vdim, d = i - g * vdim;
            dst[g * head_stride + dim + d] = from_f32<T>(to_f32<T>(row[nq + nk + i]) + (bias ? bias[nq + nk + i] : 0.0f));
        }
    }
}

FL_API int fl_head_prep(const void* proj, int dtype, long ld, const float* bias, const float* q_w, const float* k_w,
                        int norm_mode, float eps, int rot, int interleaved, const float* cos_t, const float* sin_t,
                        const int* positions, float temp_coef, int temp_every, int v_from_k, void* q_out, int q_dtype,
                        long q_ld, int n_tokens, int heads, int kv_heads, int dim, int vdim, const int* slots, void* cache,
                        long page_stride, int page_size, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (norm_mode < 0 || norm_mode > 2 || rot < 0 || rot > dim || (rot & 1) || (rot > 0 && (cos_t == nullptr || sin_t == nullptr)) ||
        (v_from_k && vdim != dim) || (size_t)dim * 8 * sizeof(float) > 48 * 1024 || cache == nullptr ||
        (heads + kv_heads + 7) / 8 > 65535)
        return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, FL_DISPATCH(q_dtype, TQ,
        return fl_launch(head_prep_kernel<T, TQ>, dim3(n_tokens, (heads + kv_heads + 7) / 8), dim3(256), (size_t)dim * 8 * sizeof(float), stream,
                         (const T*)proj, ld, bias, q_w, k_w, norm_mode, eps, rot, interleaved, cos_t, sin_t, positions,
                         temp_coef, temp_every, v_from_k, (TQ*)q_out, q_ld, heads, kv_heads, dim, vdim, slots, (T*)cache,
                         page_stride, page_size)));
    return 0;
}

// x[t, h * vdim + d] *= sigmoid(gate[t, h]): one number per token and head on the head's whole result.
template <typename T>
__global__ void __launch_bounds__(256) head_gate_kernel(T* __restrict__ x, long x_ld, const T* __restrict__ gate, long g_ld,
                                                        int heads, int vdim) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < heads * vdim; i += blockDim.x) {
        const float g = to_f32<T>(gate[(long)t * g_ld + i / vdim]);
        x[(long)t * x_ld + i] = from_f32<T>(to_f32<T>(x[(long)t * x_ld + i]) / (1.0f + expf(-g)));
    }
}

FL_API int fl_head_gate(void* x, int dtype, long x_ld, const void* gate, long g_ld, int n_tokens, int heads, int vdim,
                        cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    FL_DISPATCH(dtype, T, return fl_launch(head_gate_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (T*)x, x_ld,
                                           (const T*)gate, g_ld, heads, vdim));
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
    const int* __restrict__ positions, int heads, int kv_heads, int dim, int vdim, int window, int keep_first, int chunk,
    float scale, float cap, const int* __restrict__ bucket_of, int n_dist, const float* __restrict__ rel,
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
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);                 // a query sees its own chunk of positions only
    const int kept = window > 0 ? min(keep_first, lo) : 0;            // keys [0, kept) are seen beside [lo, pos]
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
// [h * vdim, (h + 1) * vdim).  window <= 0: all keys.  chunk > 0: only keys at or after the last multiple of `chunk`
// at or below the query's position.  bucket_of: [n_dist] rows of rel ([rows, heads] float) by distance.
FL_API int fl_sink_attention_simt(const void* q, int q_dtype, long q_ld, void* out, long out_ld, const void* cache, int dtype,
                                  long page_stride, int page_size, const int* block_table, int bt_stride,
                                  const int* tok_req, const int* positions, int n_tokens, int heads, int kv_heads, int dim,
                                  int vdim, int window, int keep_first, int chunk, float scale, float cap,
                                  const int* bucket_of, int n_dist, const float* rel, const float* sink,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (vdim < 1 || vdim > 2 * SINK_TILE || dim < 1 || dim > 4096 || heads > 65535 || heads % kv_heads ||
        (rel != nullptr && (bucket_of == nullptr || n_dist < 1)))
        return (int)cudaErrorInvalidValue;
    const size_t smem = SINK_TILE * (sizeof(long) + sizeof(float)) + (size_t)dim * sizeof(float);
    dim3 grid(n_tokens, heads);
    FL_DISPATCH(dtype, T, FL_DISPATCH(q_dtype, TQ,
        return fl_launch(sink_attention_simt_kernel<T, TQ>, grid, dim3(SINK_TILE), smem, stream, (const TQ*)q, q_ld, (T*)out,
                         out_ld, (const T*)cache, page_stride, page_size, block_table, bt_stride, tok_req, positions, heads,
                         kv_heads, dim, vdim, window, keep_first, chunk, scale, cap, bucket_of, n_dist, rel, sink)));
    return 0;
}

// ------------------------------------------------------------------ single tokens, keys split over blocks
//   sink_decode         per (token, key/value head, split): the maxima, sums and weighted values of every query head
//                       of the group over one split of 128 keys, so that a cache row is read once for the group.
//                       The first `kept_splits` splits walk the kept first tokens (those the window has left behind),
//                       the others the window from the multiple of 128 at or below its first key
//   sink_decode_merge   per (token, query head): the splits and the sink added up
#define SINK_SPLIT 128           // keys of a split: one per thread

__device__ __forceinline__ void sink_load8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void sink_load8(const bf16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

// GROUP: query heads per key/value head, rounded up to a power of two (at most 8).
// partial: [n_decode][heads][n_splits][vdim + 2] floats: maximum, sum, weighted values.
template <typename T, int GROUP>
__global__ void __launch_bounds__(SINK_SPLIT) sink_decode_kernel(
    const T* __restrict__ q, long q_ld, const T* __restrict__ cache, long page_stride, int page_size,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req, const int* __restrict__ positions,
    const int* __restrict__ decode_tokens, float* __restrict__ partial, int n_splits, int kept_splits, int heads,
    int kv_heads, int dim, int vdim, int window, int keep_first, int chunk, float scale, float cap,
    const int* __restrict__ bucket_of, int n_dist, const float* __restrict__ rel, int vec8) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char dec_smem[];
    long* off_s = reinterpret_cast<long*>(dec_smem);                  // [SPLIT] element offset of each row's value part
    float* p_s = reinterpret_cast<float*>(off_s + SINK_SPLIT);        // [SPLIT][GROUP] numerators
    float* red_s = p_s + SINK_SPLIT * GROUP;                          // [4 warps][GROUP]
    float* q_s = red_s + 4 * GROUP;                                   // [GROUP][dim]
    const int t = decode_tokens[blockIdx.x], g = blockIdx.y, split = blockIdx.z, tid = threadIdx.x;
    const int group = heads / kv_heads;
    const int pos = positions[t];
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    const int kept = window > 0 ? min(keep_first, lo) : 0;
    // the split's keys: [first, first + 128) cut to [from, to)
    int first, from, to;
    if (split < kept_splits) {
        first = split * SINK_SPLIT;
        from = first;
        to = min(first + SINK_SPLIT, kept);
    } else {
        first = (lo / SINK_SPLIT + (split - kept_splits)) * SINK_SPLIT;
        from = max(first, lo);
        to = min(first + SINK_SPLIT, pos + 1);
    }
    const int row_w = dim + vdim;
    float* out = partial + (((long)blockIdx.x * heads + (long)g * group) * n_splits + split) * (vdim + 2);
    const long h_stride = (long)n_splits * (vdim + 2);                // from one head to the next
    if (from >= to) {                                                 // nothing of this token in the split
        for (int hh = tid; hh < group; hh += SINK_SPLIT) {
            out[hh * h_stride] = -CUDART_INF_F;
            out[hh * h_stride + 1] = 0.0f;
        }
        return;
    }
    for (int i = tid; i < group * dim; i += SINK_SPLIT) q_s[i] = to_f32<T>(q[(long)t * q_ld + (long)g * group * dim + i]);
    __syncthreads();
    const int* bt = block_table + (long)tok_req[t] * bt_stride;
    const int j = first + tid;
    const bool valid = j >= from && j < to;
    float s[GROUP];
#pragma unroll
    for (int hh = 0; hh < GROUP; ++hh) s[hh] = 0.0f;
    if (valid) {
        const long off = (long)bt[j / page_size] * page_stride + ((long)g * page_size + j % page_size) * row_w;
        off_s[tid] = off + dim;
        const T* kp = cache + off;
        if (vec8) {
            int d = 0;
            for (; d + 32 <= dim; d += 32) {                          // four loads in flight before the first is used
                float k[4][8];
#pragma unroll
                for (int u = 0; u < 4; ++u) sink_load8(kp + d + u * 8, k[u]);
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int e = 0; e < 8; ++e)
#pragma unroll
                        for (int hh = 0; hh < GROUP; ++hh)
                            if (hh < group) s[hh] += q_s[hh * dim + d + u * 8 + e] * k[u][e];
            }
            for (; d < dim; d += 8) {
                float k[8];
                sink_load8(kp + d, k);
#pragma unroll
                for (int e = 0; e < 8; ++e)
#pragma unroll
                    for (int hh = 0; hh < GROUP; ++hh)
                        if (hh < group) s[hh] += q_s[hh * dim + d + e] * k[e];
            }
        } else {
            for (int d = 0; d < dim; ++d) {
                const float k = to_f32<T>(kp[d]);
#pragma unroll
                for (int hh = 0; hh < GROUP; ++hh)
                    if (hh < group) s[hh] += q_s[hh * dim + d] * k;
            }
        }
    }
    const int warp = tid >> 5, lane = tid & 31;
    float m[GROUP];
#pragma unroll
    for (int hh = 0; hh < GROUP; ++hh) {
        s[hh] = (valid && hh < group) ? sink_score(s[hh], scale, cap, bucket_of, n_dist, rel, heads, g * group + hh, pos - j)
                                      : -CUDART_INF_F;
        const float w = warp_max(s[hh]);
        if (lane == 0) red_s[warp * GROUP + hh] = w;
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < GROUP; ++hh) {
        m[hh] = fmaxf(fmaxf(red_s[hh], red_s[GROUP + hh]), fmaxf(red_s[2 * GROUP + hh], red_s[3 * GROUP + hh]));
        const float p = (valid && hh < group) ? expf(s[hh] - m[hh]) : 0.0f;      // (some key of the split is valid: m is finite)
        p_s[tid * GROUP + hh] = p;
        s[hh] = warp_sum(p);
    }
    __syncthreads();                                                  // red_s was read; p_s and off_s are written
#pragma unroll
    for (int hh = 0; hh < GROUP; ++hh)
        if (lane == 0) red_s[warp * GROUP + hh] = s[hh];
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < GROUP; ++hh)
        if (tid == hh && hh < group) {                                // (m is the same in every thread)
            out[hh * h_stride] = m[hh];
            out[hh * h_stride + 1] = red_s[hh] + red_s[GROUP + hh] + red_s[2 * GROUP + hh] + red_s[3 * GROUP + hh];
        }
    const int j_begin = from - first, j_end = to - first;
    for (int d = tid; d < vdim; d += SINK_SPLIT) {
        float acc[GROUP];
#pragma unroll
        for (int hh = 0; hh < GROUP; ++hh) acc[hh] = 0.0f;
        int jj = j_begin;
        for (; jj + 16 <= j_end; jj += 16) {                          // sixteen rows' loads in flight together
            T raw[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) raw[u] = cache[off_s[jj + u] + d];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const float v = to_f32<T>(raw[u]);
#pragma unroll
                for (int hh = 0; hh < GROUP; ++hh) acc[hh] += p_s[(jj + u) * GROUP + hh] * v;
            }
        }
        for (; jj < j_end; ++jj) {
            const float v = to_f32<T>(cache[off_s[jj] + d]);
#pragma unroll
            for (int hh = 0; hh < GROUP; ++hh) acc[hh] += p_s[jj * GROUP + hh] * v;
        }
#pragma unroll
        for (int hh = 0; hh < GROUP; ++hh)
            if (hh < group) out[hh * h_stride + 2 + d] = acc[hh];
    }
}

// One block per (token, query head): the splits and the sink added up.
template <typename T>
__global__ void __launch_bounds__(128) sink_decode_merge_kernel(const float* __restrict__ partial, int n_splits,
                                                                const int* __restrict__ decode_tokens, T* __restrict__ out,
                                                                long out_ld, int heads, int vdim,
                                                                const float* __restrict__ sink) {
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.y, tid = threadIdx.x;
    const float* base = partial + ((long)blockIdx.x * heads + h) * n_splits * (vdim + 2);
    float top = sink != nullptr ? sink[h] : -CUDART_INF_F;
    for (int s = 0; s < n_splits; ++s) top = fmaxf(top, base[(long)s * (vdim + 2)]);
    float sum = sink != nullptr ? expf(sink[h] - top) : 0.0f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = base[(long)s * (vdim + 2)];
        if (ms != -CUDART_INF_F) sum += base[(long)s * (vdim + 2) + 1] * expf(ms - top);
    }
    T* dst = out + (long)decode_tokens[blockIdx.x] * out_ld + (long)h * vdim;
    for (int d = tid; d < vdim; d += 128) {
        float a = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = base[(long)s * (vdim + 2)];
            if (ms != -CUDART_INF_F) a += base[(long)s * (vdim + 2) + 2 + d] * expf(ms - top);
        }
        dst[d] = from_f32<T>(a / sum);
    }
}

// Whether the split-key kernels take a layer of these sizes.
FL_API int fl_sink_decode_takes(int heads, int kv_heads, int dim, int vdim) {
    const int group = kv_heads > 0 && heads % kv_heads == 0 ? heads / kv_heads : 0;
    return group >= 1 && group <= 8 && vdim >= 1 && vdim <= 4096 && dim >= 1 &&
           (size_t)SINK_SPLIT * (sizeof(long) + 8 * sizeof(float)) + (size_t)(32 + 8 * dim) * sizeof(float) <= 48 * 1024;
}

// The rows `decode_tokens` (n_decode of them, each the single token of its request) of q get attention over their
// requests' cache rows.  kept_splits = ceil(keep_first / 128) (0 without a window); n_splits = kept_splits + enough
// window splits to reach every token's last key: (longest visible span - 1) / 128 + 2 does.
// partial: n_decode * heads * n_splits * (vdim + 2) floats.
FL_API int fl_sink_decode(const void* q, int dtype, long q_ld, void* out, long out_ld, const void* cache, long page_stride,
                          int page_size, const int* block_table, int bt_stride, const int* tok_req, const int* positions,
                          const int* decode_tokens, int n_decode, float* partial, int n_splits, int kept_splits, int heads,
                          int kv_heads, int dim, int vdim, int window, int keep_first, int chunk, float scale, float cap,
                          const int* bucket_of, int n_dist, const float* rel, const float* sink, cudaStream_t stream) {
    if (n_decode <= 0) return 0;
    if (!fl_sink_decode_takes(heads, kv_heads, dim, vdim) || n_splits < 1 || n_splits > 65535 || kv_heads > 65535 ||
        kept_splits < 0 || kept_splits >= n_splits || (rel != nullptr && (bucket_of == nullptr || n_dist < 1)))
        return (int)cudaErrorInvalidValue;
    const int group = heads / kv_heads;
    const int gp = group <= 1 ? 1 : group <= 2 ? 2 : group <= 4 ? 4 : 8;
    const size_t smem = (size_t)SINK_SPLIT * (sizeof(long) + gp * sizeof(float)) + (size_t)(4 * gp + gp * dim) * sizeof(float);
    dim3 grid(n_decode, kv_heads, n_splits);
    // (rows start 16 bytes aligned when the row and page sizes are multiples of 8 elements and the pool is aligned)
    const int vec8 = dim % 8 == 0 && vdim % 8 == 0 && page_stride % 8 == 0 && ((uintptr_t)cache % 32) == 0;
    int rc = 0;
#define FL_SINK_DECODE(G)                                                                                            \
    FL_DISPATCH(dtype, T, rc = fl_launch(sink_decode_kernel<T, G>, grid, dim3(SINK_SPLIT), smem, stream, (const T*)q, \
                                         q_ld, (const T*)cache, page_stride, page_size, block_table, bt_stride,      \
                                         tok_req, positions, decode_tokens, partial, n_splits, kept_splits, heads,   \
                                         kv_heads, dim, vdim, window, keep_first, chunk, scale, cap, bucket_of, n_dist, rel, vec8))
    if (gp == 1) { FL_SINK_DECODE(1); }
    else if (gp == 2) { FL_SINK_DECODE(2); }
    else if (gp == 4) { FL_SINK_DECODE(4); }
    else { FL_SINK_DECODE(8); }
#undef FL_SINK_DECODE
    if (rc) return rc;
    FL_DISPATCH(dtype, T, return fl_launch(sink_decode_merge_kernel<T>, dim3(n_decode, heads), dim3(128), 0, stream,
                                           (const float*)partial, n_splits, decode_tokens, (T*)out, out_ld, heads, vdim,
                                           sink));
    return 0;
}
