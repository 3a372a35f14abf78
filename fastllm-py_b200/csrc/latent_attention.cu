// Latent attention: causal attention whose cache holds, per token, one compressed vector c (`rank`
// elements, RMS-normed) and one rotated key part (`rot` elements) that all heads share.
//
// A head's key is [W_uk c | rotated part] and its value W_uv c.  Neither is ever made: with
//     q~ = [W_uk^T q_plain | q_rotated]          (rank + rot elements per head)
// the score is q~ . [c | rotated part] * scale, and the weighted sum of values is W_uv (sum_j p_j c_j).
// So attention runs over the cache rows themselves, all heads on the one row per token, and two small
// per-head products (q_plain -> q~ before, latent sum -> value after) stand on either side of it.
//
//   latent_prep       per token: rotary encoding of the queries' rotated parts, written behind where q~'s
//                     first part will go; the latent normed and, with the rotated key part, written into
//                     the token's cache row.  Rotary pairs are (i, i + rot/2), or with `interleaved`
//                     (2i, 2i + 1); pair i turns by the table's column i either way
//   latent_attention  per (token, head): softmax over the visible rows (a window, if the layer has one),
//                     keys walked in tiles of 128 aligned to absolute positions
//
// Cache: [pages][page_size][rank + rot] in the activation type.  Scores, softmax and sums are float.
#include "common.cuh"

#define LAT_TILE 128
#define LAT_MAX_ACC 8            // value elements per thread: rank <= LAT_TILE * LAT_MAX_ACC

// proj row: heads x [dim plain | rot rotated] queries; kv row (has_kv): rank latent + rot key elements.
template <typename T, typename TW, typename TQ>
__global__ void __launch_bounds__(256) latent_prep_kernel(
    const T* __restrict__ proj, long ld, const T* __restrict__ kv_src, long kv_ld, int interleaved,
    TQ* __restrict__ q_out, long q_ld, int heads, int dim, int rot, int rank,
    const TW* __restrict__ norm_w, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ positions,
    const int* __restrict__ slots, T* __restrict__ cache, int has_kv) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int half = rot / 2;
    const long pos = positions[t];
    const T* row = proj + (long)t * ld;
    TQ* q_row = q_out + (long)t * q_ld;
    const float* cs = cos_t + pos * half;
    const float* sn = sin_t + pos * half;
    for (int idx = tid; idx < heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        const T* p = row + (long)h * (dim + rot) + dim;
        TQ* o = q_row + (long)h * (rank + rot) + rank;
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        const float u = to_f32<T>(p[a]), v = to_f32<T>(p[b]);
        o[a] = from_f32<TQ>(u * cs[i] - v * sn[i]);
        o[b] = from_f32<TQ>(v * cs[i] + u * sn[i]);
    }
    if (!has_kv) return;
    const T* kv = kv_src + (long)t * kv_ld;
    T* dst = cache + (long)slots[t] * (rank + rot);
    float ss = 0.0f;
    for (int i = tid; i < rank; i += blockDim.x) {
        const float x = to_f32<T>(kv[i]);
        ss += x * x;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int i = tid; i < rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32<T>(kv[i]) * inv * to_f32<TW>(norm_w[i]));
    for (int i = tid; i < half; i += blockDim.x) {
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        const float u = to_f32<T>(kv[rank + a]), v = to_f32<T>(kv[rank + b]);
        dst[rank + a] = from_f32<T>(u * cs[i] - v * sn[i]);
        dst[rank + b] = from_f32<T>(v * cs[i] + u * sn[i]);
    }
}

// q: [n_tokens, heads x (rank + rot)]; out: [n_tokens, heads x rank] float.
template <typename T, typename TQ>
__global__ void __launch_bounds__(LAT_TILE) latent_attention_kernel(
    const TQ* __restrict__ q, long q_ld, float* __restrict__ out, long out_ld, const T* __restrict__ cache,
    int page_size, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req,
    const int* __restrict__ positions, int rank, int rot, int window, float scale) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    long* off_s = reinterpret_cast<long*>(smem_raw);                  // [LAT_TILE] element offset of each row
    float* p_s = reinterpret_cast<float*>(off_s + LAT_TILE);          // [LAT_TILE] softmax numerators of the tile
    float* q_s = p_s + LAT_TILE;                                      // [rank + rot]
    __shared__ float scratch[32];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int width = rank + rot;
    const int pos = positions[t];
    const int* bt = block_table + (long)tok_req[t] * bt_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const TQ* qr = q + (long)t * q_ld + (long)h * width;
    for (int d = tid; d < width; d += LAT_TILE) q_s[d] = to_f32<TQ>(qr[d]);
    __syncthreads();
    float m = -CUDART_INF_F, l = 0.0f, acc[LAT_MAX_ACC];
#pragma unroll
    for (int a = 0; a < LAT_MAX_ACC; ++a) acc[a] = 0.0f;
    for (int tile = (lo / LAT_TILE) * LAT_TILE; tile <= pos; tile += LAT_TILE) {
        const int j = tile + tid;
        const bool valid = j >= lo && j <= pos;
        float s = -CUDART_INF_F;
        long off = 0;
        if (valid) {
            off = ((long)bt[j / page_size] * page_size + j % page_size) * width;
            const T* kp = cache + off;
            float dot = 0.0f;
            for (int d = 0; d < width; ++d) dot += q_s[d] * to_f32<T>(kp[d]);
            s = dot * scale;
        }
        off_s[tid] = off;
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float p = valid ? expf(s - m_new) : 0.0f;
        p_s[tid] = p;
        const float tile_sum = block_sum(p, scratch);     // its barriers also publish p_s / off_s
        const float corr = expf(m - m_new);               // 0 at the first tile (m = -inf)
        l = l * corr + tile_sum;
        const int j_begin = max(0, lo - tile), j_end = min(LAT_TILE, pos - tile + 1);
#pragma unroll
        for (int a = 0; a < LAT_MAX_ACC; ++a) {
            const int d = tid + a * LAT_TILE;
            if (d < rank) {
                float v = acc[a] * corr;
                for (int jj = j_begin; jj < j_end; ++jj) v += p_s[jj] * to_f32<T>(cache[off_s[jj] + d]);
                acc[a] = v;
            }
        }
        m = m_new;
        __syncthreads();                                  // p_s / off_s are rewritten by the next tile
    }
    float* o = out + (long)t * out_ld + (long)h * rank;
#pragma unroll
    for (int a = 0; a < LAT_MAX_ACC; ++a) {
        const int d = tid + a * LAT_TILE;
        if (d < rank) o[d] = acc[a] / l;
    }
}

// q_out: [n_tokens, q_ld] (float or bfloat16), heads x [rank | rot]: the rot columns of every head are written here.
// kv: [n_tokens, kv_ld] rows of rank latent + rot key elements (null: they follow the queries in `proj`'s rows).
FL_API int fl_latent_prep(const void* proj, int dtype, long ld, const void* kv, long kv_ld, int interleaved, void* q_out, int q_dtype, long q_ld, int n_tokens, int heads, int dim,
                          int rot, int rank,
                          const void* norm_w, int w_dtype, float eps, const float* cos_t, const float* sin_t,
                          const int* positions, const int* slots, void* cache, int has_kv, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot % 2) return (int)cudaErrorInvalidValue;
    const long esize = dtype == FL_F32 ? 4 : 2;
    if (kv == nullptr) {
        kv = (const char*)proj + (long)heads * (dim + rot) * esize;
        kv_ld = ld;
    }
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW, FL_DISPATCH(q_dtype, TQ,
        return fl_launch(latent_prep_kernel<T, TW, TQ>, dim3(n_tokens), dim3(256), 0, stream, (const T*)proj, ld, (const T*)kv, kv_ld, interleaved, (TQ*)q_out,
                         q_ld, heads, dim, rot, rank, (const TW*)norm_w, eps, cos_t, sin_t, positions, slots, (T*)cache,
                         has_kv))));
    return 0;
}

// window <= 0: all earlier tokens.
FL_API int fl_latent_attention(const void* q, int q_dtype, long q_ld, float* out, long out_ld, const void* cache, int cache_dtype,
                               int page_size, const int* block_table, int bt_stride, const int* tok_req,
                               const int* positions, int n_tokens, int heads, int rank, int rot, int window,
                               float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank < 1 || rank > LAT_TILE * LAT_MAX_ACC || heads > 65535) return (int)cudaErrorInvalidValue;
    const size_t smem = LAT_TILE * (sizeof(long) + sizeof(float)) + (size_t)(rank + rot) * sizeof(float);
    FL_DISPATCH(cache_dtype, T, FL_DISPATCH(q_dtype, TQ,
        return fl_launch(latent_attention_kernel<T, TQ>, dim3(n_tokens, heads), dim3(LAT_TILE), smem, stream, (const TQ*)q,
                         q_ld, out, out_ld, (const T*)cache, page_size, block_table, bt_stride, tok_req, positions, rank, rot,
                         window, scale)));
    return 0;
}
