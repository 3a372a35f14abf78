// Batched bfloat16 product on tensor cores (mma.sync m16n8k16, float accumulation):
//     C_b[M, N] = A_b[M, K] * W_b[N, K]^T   for b = 0 .. batch - 1
// where A_b and C_b are column blocks of wider row-major buffers (A + b * a_batch, C + b * c_batch, in
// elements) and W is [batch][N][K].  This is the product per head that stands on either side of latent
// attention (a head's query block through its own small matrix), for steps of any size: a block takes 64
// rows x 128 columns of one batch entry, K in steps of 32 through a two-stage cp.async ring.
// With `gate` (laid out like C: gate + b * g_batch, ldg between rows) the epilogue writes C * sigmoid(gate): the
// product is rounded to C's type first, as a gate applied by a kernel of its own would have read it.
// K must be a multiple of 32 and every A row 16-byte aligned; other shapes go to gemm_simt's batched form.
#include "common.cuh"

#define GM_BM 64
#define GM_BN 128
#define GM_BK 32
#define GM_PITCH 40              // bfloat16 elements between staged rows: ldmatrix without bank conflicts

__device__ __forceinline__ void gm_cp16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}

template <typename TC>
__global__ void __launch_bounds__(256) gemm_mma_batched_kernel(const bf16* __restrict__ A, long lda, long a_batch,
                                                               const bf16* __restrict__ W, TC* __restrict__ C, long ldc,
                                                               long c_batch, int M, int N, int K,
                                                               const TC* __restrict__ gate, long ldg, long g_batch) {
    pdl_wait();
    pdl_trigger();
    __shared__ __align__(16) bf16 a_s[2][GM_BM][GM_PITCH];
    __shared__ __align__(16) bf16 w_s[2][GM_BN][GM_PITCH];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3;                    // 2 x 4 warps, 32 rows x 32 columns each
    const int m0 = blockIdx.x * GM_BM, n0 = blockIdx.y * GM_BN, b = blockIdx.z;
    const int ar = tid >> 2, ac = (tid & 3) * 8;                // this thread's 16-byte pieces of a stage
    const bf16* a_src = A + b * a_batch + (long)min(m0 + ar, M - 1) * lda + ac;
    const bf16* w_src[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) w_src[i] = W + ((long)b * N + min(n0 + ar + i * 64, N - 1)) * K + ac;
    auto stage = [&](int buf, int k0) {
        gm_cp16(&a_s[buf][ar][ac], a_src + k0);
#pragma unroll
        for (int i = 0; i < 2; ++i) gm_cp16(&w_s[buf][ar + i * 64][ac], w_src[i] + k0);
        asm volatile("cp.async.commit_group;");
    };
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;
    const int n_k = K / GM_BK;
    stage(0, 0);
    for (int kb = 0; kb < n_k; ++kb) {
        const int buf = kb & 1;
        if (kb + 1 < n_k) {
            stage(buf ^ 1, (kb + 1) * GM_BK);
            asm volatile("cp.async.wait_group 1;");
        } else {
            asm volatile("cp.async.wait_group 0;");
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < GM_BK; ks += 16) {
            unsigned af[2][4], bfr[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const unsigned s = (unsigned)__cvta_generic_to_shared(&a_s[buf][wm * 32 + i * 16 + (lane & 15)][ks + (lane >> 4) * 8]);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(af[i][0]), "=r"(af[i][1]), "=r"(af[i][2]), "=r"(af[i][3]) : "r"(s));
            }
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
                const unsigned s = (unsigned)__cvta_generic_to_shared(
                    &w_s[buf][wn * 32 + j2 * 16 + (lane & 7) + (lane >> 4) * 8][ks + ((lane >> 3) & 1) * 8]);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(bfr[j2 * 2][0]), "=r"(bfr[j2 * 2][1]), "=r"(bfr[j2 * 2 + 1][0]), "=r"(bfr[j2 * 2 + 1][1])
                             : "r"(s));
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(acc[i][j][0]), "+f"(acc[i][j][1]), "+f"(acc[i][j][2]), "+f"(acc[i][j][3])
                                 : "r"(af[i][0]), "r"(af[i][1]), "r"(af[i][2]), "r"(af[i][3]), "r"(bfr[j][0]), "r"(bfr[j][1]));
        }
        __syncthreads();
    }
    TC* c_base = C + b * c_batch;
    const TC* g_base = gate != nullptr ? gate + b * g_batch : nullptr;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = m0 + wm * 32 + i * 16 + (lane >> 2) + half * 8;
            if (m >= M) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int n = n0 + wn * 32 + j * 8 + (lane & 3) * 2 + c;
                    if (n >= N) continue;
                    TC v = from_f32<TC>(acc[i][j][half * 2 + c]);
                    if (g_base != nullptr) v = from_f32<TC>(to_f32<TC>(v) / (1.0f + expf(-to_f32<TC>(g_base[(long)m * ldg + n]))));
                    c_base[(long)m * ldc + n] = v;
                }
        }
}

FL_API int fl_gemm_mma_batched_takes(long lda, long a_batch, int K, const void* A) {
    return K % GM_BK == 0 && lda % 8 == 0 && a_batch % 8 == 0 && ((uintptr_t)A % 16) == 0;
}

FL_API int fl_gemm_mma_batched(const void* A, long lda, long a_batch, const void* W, void* C, int c_dtype, long ldc,
                               long c_batch, int M, int N, int K, int batch, const void* gate, long ldg, long g_batch,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (!fl_gemm_mma_batched_takes(lda, a_batch, K, A) || ((uintptr_t)W % 16) || batch > 65535 || (N + GM_BN - 1) / GM_BN > 65535)
        return (int)cudaErrorInvalidValue;
    dim3 grid((M + GM_BM - 1) / GM_BM, (N + GM_BN - 1) / GM_BN, batch);
    FL_DISPATCH(c_dtype, TC,
        return fl_launch(gemm_mma_batched_kernel<TC>, grid, dim3(256), 0, stream, (const bf16*)A, lda, a_batch,
                         (const bf16*)W, (TC*)C, ldc, c_batch, M, N, K, (const TC*)gate, ldg, g_batch));
    return 0;
}
