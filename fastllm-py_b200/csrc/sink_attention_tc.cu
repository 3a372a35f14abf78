// Sink attention over a paged cache on the tensor cores (bfloat16, mma.sync m16n8k16): grouped-query attention whose
// scores pass a soft cap and take a bias by distance, over a sliding window that also keeps a sequence's first
// tokens, with a sink in the softmax's denominator.  Softmax in float.
//
// A cache row holds a token's key and its value (k | v, SINK_DIM and SINK_VDIM elements).  With c the cap,
//     s_ij = c tanh(q_i . k_j scale / c) + bias[row_of[i - j], head]
//     p_ij = exp(s_ij) / (exp(sink_head) + sum_j' exp(s_ij')),   j seen when j <= i and (i - j < window or j < keep_first)
//
// A CTA of four warps (16 rows each) takes 64 consecutive query rows of one request and one query head and walks the
// request's keys in blocks of 64 through the block table: first the blocks that hold kept first tokens, then from the
// first key any of its rows' windows may see to the last; blocks in between are never touched (their pages may have
// gone back).  Rows cached by earlier steps and the rows this step wrote are read alike, so a portion of a prompt
// is the same as a whole prompt, and a single decoded token is a tile of one row (warps without rows only help to
// load; steps of single tokens have a kernel of their own that splits the keys, sink_attention.cu, and the launcher
// can leave such requests out).  Key blocks start at multiples of 64 of the absolute position, so the partial maxima and sums a row goes
// through depend on the row's position only.  A block's rows (key and value: one piece of memory per token) come by
// cp.async into a two-stage ring while the block before is multiplied.  The bias of this head by distance is staged
// in shared memory for the first SINK_NEAR distances; farther ones (kept tokens far behind) are looked up in global
// memory.  The sink enters as the softmax's starting state: running maximum = sink, running sum = 1, no value.
// Probabilities are rounded to bfloat16 only as the operand of P V.
//
// SINK_DIM and SINK_VDIM are compile-time constants, multiples of 16 up to 128.
#include "common.cuh"

#ifndef SINK_DIM
#define SINK_DIM 64
#endif
#ifndef SINK_VDIM
#define SINK_VDIM 64
#endif
#define STC_BM 64
#define STC_BN 64
#define STC_THREADS 128
#define STC_ROW (SINK_DIM + SINK_VDIM)        // elements of a cache row
#define STC_KP (STC_ROW + 8)                  // padded pitches in shared memory: ldmatrix without bank conflicts
#define STC_QP (SINK_DIM + 8)
#define SINK_NEAR 1024                        // distances whose bias is staged in shared memory

static_assert(SINK_DIM % 16 == 0 && SINK_DIM >= 16 && SINK_DIM <= 128, "SINK_DIM: multiple of 16, at most 128");
static_assert(SINK_VDIM % 16 == 0 && SINK_VDIM >= 16 && SINK_VDIM <= 128, "SINK_VDIM: multiple of 16, at most 128");

__device__ __forceinline__ uint32_t stc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void stc_cp16(void* dst, const void* src, bool real) {
    const int bytes = real ? 16 : 0;                       // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(stc_smem(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void stc_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void stc_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void stc_ldm(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(stc_smem(p)));
}
__device__ __forceinline__ void stc_ldm_t(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(stc_smem(p)));
}
__device__ __forceinline__ void stc_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t stc_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float stc_weight(float a, float b) { return (a == -CUDART_INF_F) ? 0.0f : exp2f(a - b); }


#define STC_LOG2E 1.4426950408889634f

__global__ void __launch_bounds__(STC_THREADS, 3) sink_attention_tc_kernel(
    const bf16* __restrict__ q, long q_ld, bf16* __restrict__ out, long out_ld, const bf16* __restrict__ cache,
    long page_stride, int page_size, int page_shift, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ req_start, const int* __restrict__ req_ctx, const int* __restrict__ req_qlen,
    int n_requests, int include_single, int heads, int kv_heads, int window, int keep_first, int chunk, float scale, float cap,
    const int* __restrict__ row_of, int n_dist, const float* __restrict__ rel, const float* __restrict__ sink) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char stc_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(stc_raw);                       // [64][QP]
    bf16* Rs = Qs + STC_BM * STC_QP;                                   // [2 stages][64][KP]
    float* near_bias = reinterpret_cast<float*>(Rs + 2 * STC_BN * STC_KP);   // [SINK_NEAR], in units of log2

    // which request and which 64-row tile of it this CTA serves (heaviest tiles first)
    int req = -1, tile = 0;
    {
        int acc = 0;
        for (int r = 0; r < n_requests; ++r) {
            const int ql = req_qlen[r];
            const int nt = (ql > 1 || include_single) ? (ql + STC_BM - 1) / STC_BM : 0;
            if ((int)blockIdx.x < acc + nt) { req = r; tile = nt - 1 - ((int)blockIdx.x - acc); break; }
            acc += nt;
        }
    }
    if (req < 0) return;
    const int h = blockIdx.y;
    const int kvh = h / (heads / kv_heads);
    const int q_len = req_qlen[req], ctx = req_ctx[req], row0 = tile * STC_BM;
    const int tok0 = req_start[req] + row0;
    const int rows_here = min(STC_BM, q_len - row0);
    const int pos_first = ctx + row0, pos_last = ctx + row0 + rows_here - 1;
    int lo_tile = window > 0 ? max(0, pos_first - window + 1) : 0;
    if (chunk > 0) lo_tile = max(lo_tile, pos_first / chunk * chunk);        // a row sees its own chunk of positions only
    const int keep = window > 0 ? keep_first : 0;
    const int kb_begin = lo_tile / STC_BN, kb_end = pos_last / STC_BN + 1;
    const int n_kept = min((min(keep, pos_last + 1) + STC_BN - 1) / STC_BN, kb_begin);   // blocks of kept tokens before the window's
    const int n_iters = n_kept + kb_end - kb_begin;
    const int* bt = block_table + (long)req * bt_stride;
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = tid >> 5;                                         // which 16 rows of the tile
    const bool has_rows = warp * 16 < rows_here;                       // a warp without rows only loads

    if (rel != nullptr)
        for (int d = tid; d < SINK_NEAR; d += STC_THREADS)
            near_bias[d] = rel[(long)row_of[min(d, n_dist - 1)] * heads + h] * STC_LOG2E;

    constexpr int Q_CHUNKS = SINK_DIM / 8, R_CHUNKS = STC_ROW / 8;
    auto load_q = [&]() {
        for (int c = tid; c < STC_BM * Q_CHUNKS; c += STC_THREADS) {
            const int r = c / Q_CHUNKS, ch = c - r * Q_CHUNKS;
            const bool real = r < rows_here;
            const bf16* src = q + (long)(tok0 + (real ? r : 0)) * q_ld + (long)h * SINK_DIM + ch * 8;
            stc_cp16(Qs + r * STC_QP + ch * 8, src, real);
        }
    };
    // Two threads per token row, half of the row's chunks each: one page lookup per thread and block.
    auto load_rows = [&](int kb, int stage) {
        bf16* dst = Rs + stage * STC_BN * STC_KP;
        const int r = tid >> 1;
        const int j = kb * STC_BN + r;
        const bool real = j <= pos_last && (j >= lo_tile || j < keep);
        long a = 0;
        if (real) {
            const int pg = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
            const int off = page_shift >= 0 ? (j & (page_size - 1)) : (j - pg * page_size);
            a = (long)bt[pg] * page_stride + ((long)kvh * page_size + off) * STC_ROW;
        }
        for (int ch = (tid & 1); ch < R_CHUNKS; ch += 2) stc_cp16(dst + r * STC_KP + ch * 8, cache + a + ch * 8, real);
    };
    auto block_of = [&](int it) { return it < n_kept ? it : kb_begin + (it - n_kept); };

    float o_acc[SINK_VDIM / 8][4];
#pragma unroll
    for (int i = 0; i < SINK_VDIM / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.0f;
    const int g = lane >> 2, tq = lane & 3;
    // the sink: a term exp(sink) of the denominator without a value (counted once per row: by the lane with tq == 0)
    float m_run[2], l_run[2];
    m_run[0] = m_run[1] = sink != nullptr ? sink[h] * STC_LOG2E : -CUDART_INF_F;
    l_run[0] = l_run[1] = (sink != nullptr && tq == 0) ? 1.0f : 0.0f;
    const int pos_row[2] = {ctx + row0 + warp * 16 + g, ctx + row0 + warp * 16 + g + 8};
    const int chunk_row[2] = {chunk > 0 ? pos_row[0] / chunk * chunk : 0, chunk > 0 ? pos_row[1] / chunk * chunk : 0};
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;

    load_q();
    load_rows(block_of(0), 0);
    stc_commit();

    for (int it = 0; it < n_iters; ++it) {
        const int kb = block_of(it);
        const int stage = it & 1;
        if (it + 1 < n_iters) {
            load_rows(block_of(it + 1), stage ^ 1);
            stc_commit();
            stc_wait<1>();
        } else {
            stc_wait<0>();
        }
        __syncthreads();
        const bf16* rt = Rs + stage * STC_BN * STC_KP;
        const int warp_pos_lo = ctx + row0 + warp * 16, warp_pos_hi = warp_pos_lo + 15;
        const int b_lo = kb * STC_BN, b_hi = b_lo + STC_BN - 1;
        const bool all_seen = b_hi <= warp_pos_lo && (window <= 0 || b_lo > warp_pos_hi - window || b_hi < keep) &&
                              (chunk <= 0 || b_lo >= warp_pos_hi / chunk * chunk);
        const bool none_seen = b_lo > warp_pos_hi || (window > 0 && b_hi <= warp_pos_lo - window && b_lo >= keep) ||
                               (chunk > 0 && b_hi < warp_pos_lo / chunk * chunk);
        if (has_rows && !none_seen) {
            // ---- S = Q K^T for this warp's 16 rows and the block's 64 keys
            float s[STC_BN / 8][4];
#pragma unroll
            for (int i = 0; i < STC_BN / 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < SINK_DIM / 16; ++ks) {
                uint32_t a[4];
                stc_ldm(a, Qs + (warp * 16 + (lane & 15)) * STC_QP + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < STC_BN / 16; ++np) {
                    uint32_t b[4];
                    stc_ldm(b, rt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * STC_KP + ks * 16 + ((lane >> 3) & 1) * 8);
                    stc_mma(s[2 * np], a, b[0], b[1]);
                    stc_mma(s[2 * np + 1], a, b[2], b[3]);
                }
            }
            // ---- scale, cap, bias, mask, running softmax (maxima and sums in units of log2)
            float corr[2];
            float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int nt = 0; nt < STC_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = b_lo + nt * 8 + 2 * tq + (e & 1);
                    const int pr = pos_row[e >> 1];
                    const bool seen = all_seen || (j <= pr && (window <= 0 || j > pr - window || j < keep) && j >= chunk_row[e >> 1]);
                    float v = -CUDART_INF_F;
                    if (seen) {
                        v = s[nt][e] * scale;
                        // tanh(y) = 1 - 2 / (exp(2 y) + 1): absolute error about 1e-7, two fast instructions
                        if (cap > 0.0f) v = cap * (1.0f - __fdividef(2.0f, __expf(2.0f * v * inv_cap) + 1.0f));
                        v *= STC_LOG2E;
                        if (rel != nullptr) {
                            const int d = pr - j;
                            v += d < SINK_NEAR ? near_bias[d] : rel[(long)row_of[min(d, n_dist - 1)] * heads + h] * STC_LOG2E;
                        }
                    }
                    s[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                corr[r] = stc_weight(m_run[r], m_new);
                m_run[r] = m_new;
                l_run[r] *= corr[r];
            }
#pragma unroll
            for (int nt = 0; nt < STC_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = stc_weight(s[nt][e], m_run[e >> 1]);
                    s[nt][e] = p;
                    l_run[e >> 1] += p;
                }
            }
#pragma unroll
            for (int i = 0; i < SINK_VDIM / 8; ++i) {
                o_acc[i][0] *= corr[0];
                o_acc[i][1] *= corr[0];
                o_acc[i][2] *= corr[1];
                o_acc[i][3] *= corr[1];
            }
            // ---- O += P V
#pragma unroll
            for (int kk = 0; kk < STC_BN / 16; ++kk) {
                uint32_t a[4];
                a[0] = stc_pack(s[2 * kk][0], s[2 * kk][1]);
                a[1] = stc_pack(s[2 * kk][2], s[2 * kk][3]);
                a[2] = stc_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                a[3] = stc_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < SINK_VDIM / 16; ++dp) {
                    uint32_t b[4];
                    stc_ldm_t(b, rt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STC_KP + SINK_DIM + dp * 16 +
                                     (lane >> 4) * 8);
                    stc_mma(o_acc[2 * dp], a, b[0], b[1]);
                    stc_mma(o_acc[2 * dp + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                    // the stage is refilled two iterations on
    }
    if (!has_rows) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        const int row = warp * 16 + g + r * 8;
        if (row >= rows_here) continue;
        const float inv = 1.0f / l_run[r];
        bf16* dst = out + (long)(tok0 + row) * out_ld + (long)h * SINK_VDIM + 2 * tq;
#pragma unroll
        for (int i = 0; i < SINK_VDIM / 8; ++i) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = v;
        }
    }
}

FL_API int fl_sink_attention_tc_dim() { return SINK_DIM; }
FL_API int fl_sink_attention_tc_vdim() { return SINK_VDIM; }

// Every request r of the step with req_qlen[r] > 1 (or >= 1 with include_single) gets attention for its rows req_start[r] .. req_start[r] + req_qlen[r] - 1 at positions
// req_ctx[r] + i over its cached rows.  n_tokens bounds the number of 64-row tiles.  cap <= 0: no cap; rel null: no
// bias; sink null: no sink; window <= 0: every earlier key; chunk > 0: only keys at or after the last multiple of
// `chunk` at or below the query's position.
FL_API int fl_sink_attention_tc(const void* q, long q_ld, void* out, long out_ld, const void* cache, long page_stride,
                                int page_size, const int* block_table, int bt_stride, const int* req_start,
                                const int* req_ctx, const int* req_qlen, int n_requests, int n_tokens,
                                int include_single, int heads,
                                int kv_heads, int window, int keep_first, int chunk, float scale, float cap, const int* row_of,
                                int n_dist, const float* rel, const float* sink, cudaStream_t stream) {
    if (n_requests <= 0 || n_tokens <= 0) return 0;
    if (heads > 65535 || heads % kv_heads || (rel != nullptr && (row_of == nullptr || n_dist < 1)))
        return (int)cudaErrorInvalidValue;
    if ((q_ld % 8) || (out_ld % 2) || (page_stride % 8) || ((uintptr_t)q % 16) || ((uintptr_t)cache % 16) || ((uintptr_t)out % 4))
        return (int)cudaErrorMisalignedAddress;
    const size_t smem = ((size_t)STC_BM * STC_QP + 2 * (size_t)STC_BN * STC_KP) * sizeof(bf16) + SINK_NEAR * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sink_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int page_shift = -1;
    if ((page_size & (page_size - 1)) == 0) {
        page_shift = 0;
        while ((1 << page_shift) < page_size) ++page_shift;
    }
    const int max_tiles = n_tokens / STC_BM + n_requests;   // the sum of ceil(q_len / 64) is at most this
    dim3 grid(max_tiles, heads);
    return fl_launch(sink_attention_tc_kernel, grid, dim3(STC_THREADS), smem, stream, (const bf16*)q, q_ld, (bf16*)out,
                     out_ld, (const bf16*)cache, page_stride, page_size, page_shift, block_table, bt_stride, req_start,
                     req_ctx, req_qlen, n_requests, include_single, heads, kv_heads, window, keep_first, chunk, scale, cap, row_of, n_dist, rel,
                     sink);
}
