// Routed experts: each token's feed-forward is a weighted sum of a few small gated feed-forwards
// chosen by a router.
//
//   moe_pick      per token, from the router's float logits z (a product the caller makes): score
//                 s = sigmoid(z) (or a softmax over the experts); the `top` experts with the largest
//                 s + bias are chosen (the bias steers the choice only), ties to the lower index; the
//                 weights are the chosen s, optionally renormalised to sum 1 (divided by their sum + an
//                 epsilon) and multiplied by `weight_scale`.  With groups, the experts form `n_groups`
//                 equal groups of neighbours, a group's score is the sum of the `group_top` largest
//                 s + bias in it (1: the largest), and only experts of the `keep` best groups (ties to
//                 the lower index) can be chosen
//   moe_gate_up   per (token, choice): act(W_gate[e] h) * (W_up[e] h), one warp per feature; experts
//                 without a gate: act(W_up[e] h), the unit's f(x, 1)
//   moe_down      per token: sum over its choices, in order of choice, of weight * W_down[e] a (with
//                 `accumulate` added to what `out` holds: a shared unit's result)
//
// The last two read an expert's matrices once per token that chose it: the right shape for decode
// steps, where tokens are few and the matrices stream from memory.  All sums are float and depend only
// on the token itself.
#include "common.cuh"

// One warp per token; z: float logits [n_tokens, experts] (the router's product, made by the caller).
template <typename TW>
__global__ void __launch_bounds__(128) moe_pick_kernel(const float* __restrict__ z, long z_ld, const TW* __restrict__ bias,
                                                       int* __restrict__ chosen, float* __restrict__ weights, int n_tokens,
                                                       int experts, int top, int softmax_scores, int renormalise,
                                                       int n_groups, int keep, float renorm_eps, int group_top,
                                                       float weight_scale) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float route_s[];                  // per warp: [experts] scores, [experts] scores + bias, [n_groups]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= n_tokens) return;
    float* score = route_s + (long)warp * (2 * experts + n_groups);
    float* pick = score + experts;
    const float* zr = z + (long)t * z_ld;
    if (softmax_scores) {
        float mx = -CUDART_INF_F;
        for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, zr[e]);
        mx = warp_max(mx);
        float sum = 0.0f;
        for (int e = lane; e < experts; e += 32) sum += expf(zr[e] - mx);
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) score[e] = expf(zr[e] - mx) / sum;
    } else {
        for (int e = lane; e < experts; e += 32) score[e] = 1.0f / (1.0f + expf(-zr[e]));
    }
    for (int e = lane; e < experts; e += 32) pick[e] = score[e] + (bias ? to_f32<TW>(bias[e]) : 0.0f);
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        const int per = experts / n_groups;
        float* group = pick + experts;
        for (int g = lane; g < n_groups; g += 32) {
            float b = 0.0f, last = CUDART_INF_F;        // the sum of the group's `group_top` largest, in falling order
            int last_at = -1;
            for (int n = 0; n < group_top && n < per; ++n) {
                float best = -CUDART_INF_F;
                int at = per;
                for (int i = 0; i < per; ++i) {
                    const float v = pick[g * per + i];
                    if ((v < last || (v == last && i > last_at)) && v > best) { best = v; at = i; }
                }
                if (at == per) break;
                b += best;
                last = best;
                last_at = at;
            }
            group[g] = b;
        }
        __syncwarp();
        for (int g = lane; g < n_groups; g += 32) {
            const float mine = group[g];
            int ahead = 0;                              // groups that come before this one
            for (int o = 0; o < n_groups; ++o) ahead += (group[o] > mine) || (group[o] == mine && o < g);
            if (ahead >= keep)
                for (int i = 0; i < per; ++i) pick[g * per + i] = -CUDART_INF_F;
        }
        __syncwarp();
    }
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -CUDART_INF_F;
        int at = experts;
        for (int e = lane; e < experts; e += 32)
            if (pick[e] > best) { best = pick[e]; at = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= experts) at = 0;                      // every remaining score is NaN or -inf
        if (lane == 0) {
            chosen[(long)t * top + k] = at;
            weights[(long)t * top + k] = score[at];
            pick[at] = -CUDART_INF_F;
        }
        total += score[at];
        __syncwarp();
    }
    if (lane == 0)
        for (int k = 0; k < top; ++k) {
            float w = weights[(long)t * top + k];
            if (renormalise) w /= total + renorm_eps;
            weights[(long)t * top + k] = w * weight_scale;
        }
}

// w_gu: [experts][2 ff][width] (gate rows, then up rows), or [experts][ff][width] without a gate;
// a: [tokens x top][ff] float
template <typename T, typename TW>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const T* __restrict__ h, long h_ld, const TW* __restrict__ w_gu,
                                                          const int* __restrict__ chosen, float* __restrict__ a,
                                                          int width, int ff, int top, FlGate act, int gated) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float moe_x[];                    // [width]
    const int pair = blockIdx.x, t = pair / top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < width; i += blockDim.x) moe_x[i] = to_f32<T>(h[(long)t * h_ld + i]);
    __syncthreads();
    const int f = blockIdx.y * 8 + warp;
    if (f >= ff) return;
    if (!gated) {
        const TW* wx = w_gu + ((long)chosen[pair] * ff + f) * width;
        float x = 0.0f;
        for (int i = lane; i < width; i += 32) x += moe_x[i] * to_f32<TW>(wx[i]);
        x = warp_sum(x);
        if (lane == 0) a[(long)pair * ff + f] = fl_gated(x, 1.0f, act);
        return;
    }
    const TW* wg = w_gu + ((long)chosen[pair] * 2 * ff + f) * width;
    const TW* wu = wg + (long)ff * width;
    float g = 0.0f, u = 0.0f;
    for (int i = lane; i < width; i += 32) {
        g += moe_x[i] * to_f32<TW>(wg[i]);
        u += moe_x[i] * to_f32<TW>(wu[i]);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) a[(long)pair * ff + f] = fl_gated(g, u, act);
}

// w_down: [experts][width][ff]
template <typename T, typename TW>
__global__ void __launch_bounds__(256) moe_down_kernel(const float* __restrict__ a, const TW* __restrict__ w_down,
                                                       const int* __restrict__ chosen, const float* __restrict__ weights,
                                                       T* __restrict__ out, long out_ld, int width, int ff, int top,
                                                       int accumulate) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.y * 8 + warp;
    if (c >= width) return;
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
        const long pair = (long)t * top + k;
        const TW* wd = w_down + ((long)chosen[pair] * width + c) * ff;
        const float* ar = a + pair * ff;
        float y = 0.0f;
        for (int i = lane; i < ff; i += 32) y += ar[i] * to_f32<TW>(wd[i]);
        sum += weights[pair] * warp_sum(y);
    }
    if (lane == 0) out[(long)t * out_ld + c] = from_f32<T>(accumulate ? to_f32<T>(out[(long)t * out_ld + c]) + sum : sum);
}

FL_API int fl_moe_pick(const float* z, long z_ld, const void* bias, int bias_dtype, int* chosen, float* weights,
                       int n_tokens, int experts, int top, int softmax_scores, int renormalise, int n_groups, int keep,
                       float renorm_eps, int group_top, float weight_scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_groups < 1) n_groups = keep = 1;
    const size_t smem = (size_t)(2 * experts + n_groups) * 4 * sizeof(float);
    if (top < 1 || top > experts || smem > 48 * 1024 || experts % n_groups || keep < 1 || keep > n_groups ||
        (long)keep * (experts / n_groups) < top || group_top < 1)
        return (int)cudaErrorInvalidValue;
    FL_DISPATCH(bias_dtype, TW,
        return fl_launch(moe_pick_kernel<TW>, dim3((n_tokens + 3) / 4), dim3(128), smem, stream,
                         z, z_ld, (const TW*)bias, chosen, weights, n_tokens, experts, top, softmax_scores, renormalise,
                         n_groups, keep, renorm_eps, group_top, weight_scale));
    return 0;
}

FL_API int fl_moe_experts(const void* h, int dtype, long h_ld, const void* w_gu, const void* w_down, int w_dtype,
                          const int* chosen, const float* weights, float* a, void* out, long out_ld, int n_tokens,
                          int width, int ff, int top, int act, float act_p0, float act_p1, int gated,
                          int accumulate, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if ((size_t)width * sizeof(float) > 48 * 1024 || (ff + 7) / 8 > 65535 || (width + 7) / 8 > 65535 || act < 0 || act >= FL_ACT_COUNT)
        return (int)cudaErrorInvalidValue;
    int rc = 0;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        rc = fl_launch(moe_gate_up_kernel<T, TW>, dim3(n_tokens * top, (ff + 7) / 8), dim3(256),
                       (size_t)width * sizeof(float), stream, (const T*)h, h_ld, (const TW*)w_gu, chosen, a, width, ff,
                       top, FlGate{act, act_p0, act_p1}, gated)));
    if (rc) return rc;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        return fl_launch(moe_down_kernel<T, TW>, dim3(n_tokens, (width + 7) / 8), dim3(256), 0, stream, (const float*)a,
                         (const TW*)w_down, chosen, weights, (T*)out, out_ld, width, ff, top, accumulate)));
    return 0;
}

// ----------------------------------------------------------------- many tokens: grouped products
// With many tokens the per-token kernels above would read each expert's matrices once per token.  Here
// the (token, choice) pairs are ordered by expert, each expert's rows padded to whole tiles of 64, and
// two tensor-core products run over the tiles: a tile's rows share one expert's matrix.
//
//   moe_sort        one block: counts per expert, padded offsets, row -> pair, pair -> row, tile -> expert
//   moe_group_mma   bfloat16 mma.sync m16n8k16, 64 rows x 128 weight rows per block, K in steps of 32 through
//                   a three-stage cp.async ring.  GATED: the 128 weight rows are 64 gate rows and the 64 up rows
//                   of the same features, A rows are gathered token rows, the epilogue writes act(g) * u
//                   (bfloat16, in row order); UP: experts without a gate, A gathered, 128 up rows, the epilogue
//                   writes the unit's f(x, 1); DOWN: A is that buffer and the output float [rows, width]
//   moe_combine     out[t] = sum_k weight[t, k] * y[row of pair (t, k)], in order of choice
//
// A row's sums do not depend on the other rows of its tile, so the order of rows within an expert (it
// comes from atomics) does not show in the results.
#define MOE_TM 64

__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ chosen, int n_pairs, int experts,
                                                       int* __restrict__ row_pair, int* __restrict__ pair_row,
                                                       int* __restrict__ tile_expert, int* __restrict__ n_tiles_out,
                                                       int max_tiles) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ int sort_s[];                      // [experts] counts -> cursors, [experts + 1] first rows
    int* count = sort_s;
    int* first = sort_s + experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&count[chosen[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = at;
            const int tiles = (count[e] + MOE_TM - 1) / MOE_TM;
            for (int i = 0; i < tiles; ++i) tile_expert[at / MOE_TM + i] = e;
            at += tiles * MOE_TM;
            count[e] = 0;
        }
        first[experts] = at;
        *n_tiles_out = at / MOE_TM;
    }
    __syncthreads();
    const int total = first[experts];
    for (int r = threadIdx.x; r < max_tiles * MOE_TM; r += blockDim.x) row_pair[r] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = chosen[p];
        const int r = first[e] + atomicAdd(&count[e], 1);
        row_pair[r] = p;
        pair_row[p] = r;
    }
    (void)total;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

#define MOE_BK 32
#define MOE_STAGES 3
#define MOE_PITCH (MOE_BK + 8)   // bfloat16 elements between rows of a staged tile: ldmatrix without bank conflicts
#define MOE_PIECES (MOE_BK / 32) // 16-byte pieces of a row that a thread copies per stage
#define MOE_SMEM (MOE_STAGES * (MOE_TM + 128) * MOE_PITCH * 2)

// grid: (tiles of rows, blocks of 64 features (GATED) or 128 columns).  K % 32 == 0, rows 16-byte aligned.
enum { MOE_DOWN = 0, MOE_GATED = 1, MOE_UP = 2 };
template <int MODE>
__global__ void __launch_bounds__(256) moe_group_mma_kernel(
    const bf16* __restrict__ a, long a_ld, const bf16* __restrict__ w, int n_out, int K, const int* __restrict__ row_pair,
    const int* __restrict__ tile_expert, const int* __restrict__ n_tiles, int top, bf16* __restrict__ act_out,
    float* __restrict__ y_out, long out_ld, FlGate act) {
    pdl_wait();
    pdl_trigger();
    constexpr bool GATED = MODE == MOE_GATED;
    extern __shared__ __align__(16) unsigned char moe_smem[];
    bf16 (*a_s)[MOE_TM][MOE_PITCH] = reinterpret_cast<bf16 (*)[MOE_TM][MOE_PITCH]>(moe_smem);
    bf16 (*w_s)[128][MOE_PITCH] = reinterpret_cast<bf16 (*)[128][MOE_PITCH]>(moe_smem + MOE_STAGES * MOE_TM * MOE_PITCH * 2);
    __shared__ int pair_s[MOE_TM];
    const int tile = blockIdx.x;
    if (tile >= *n_tiles) return;
    const int e = tile_expert[tile];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3;                    // 2 x 4 warps: 32 rows x (GATED: 16 + 16, else 32) columns
    if (tid < MOE_TM) pair_s[tid] = row_pair[tile * MOE_TM + tid];
    __syncthreads();
    // sources of this thread's 16-byte pieces of a stage: its part of one row of A and of two rows of W
    const int ar = tid >> 2, ac = (tid & 3) * 8 * MOE_PIECES;
    const bf16* a_src;
    if (MODE != MOE_DOWN) {
        const int pair = pair_s[ar];
        a_src = a + (long)(pair < 0 ? 0 : pair / top) * a_ld + ac;
    } else {
        a_src = a + ((long)tile * MOE_TM + ar) * a_ld + ac;
    }
    const bf16* w_src[2];
    bool w_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int wr = (tid >> 2) + i * 64;
        long row;                                               // row of this expert's matrix
        if (GATED) {
            const int f = blockIdx.y * 64 + (wr & 63);          // rows 0..63 gate features, 64..127 their up rows
            w_ok[i] = f < n_out;
            row = (long)e * 2 * n_out + (wr < 64 ? 0 : n_out) + (w_ok[i] ? f : 0);
        } else {
            const int c = blockIdx.y * 128 + wr;
            w_ok[i] = c < n_out;
            row = (long)e * n_out + (w_ok[i] ? c : 0);
        }
        w_src[i] = w + row * K + ac;
    }
    auto stage = [&](int buf, int k0) {
#pragma unroll
        for (int half = 0; half < MOE_PIECES; ++half) {
            cp_async16(&a_s[buf][ar][ac + half * 8], a_src + k0 + half * 8);
#pragma unroll
            for (int i = 0; i < 2; ++i) cp_async16(&w_s[buf][(tid >> 2) + i * 64][ac + half * 8], w_src[i] + k0 + half * 8);
        }
        cp_async_commit();
    };
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.0f;
    const int n_k = K / MOE_BK;
    stage(0, 0);
    if (n_k > 1) stage(1, MOE_BK);
    for (int kb = 0; kb < n_k; ++kb) {
        const int buf = kb % MOE_STAGES;
        if (kb + 1 < n_k) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();                                            // stage kb has landed; stage kb - 1 is read by no one
        if (kb + 2 < n_k) stage((kb + 2) % MOE_STAGES, (kb + 2) * MOE_BK);
#pragma unroll
        for (int ks = 0; ks < MOE_BK; ks += 16) {
            unsigned af[2][4], bfr[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const bf16* p = &a_s[buf][wm * 32 + i * 16 + (lane & 15)][ks + (lane >> 4) * 8];
                const unsigned s = (unsigned)__cvta_generic_to_shared(p);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(af[i][0]), "=r"(af[i][1]), "=r"(af[i][2]), "=r"(af[i][3]) : "r"(s));
            }
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
                // GATED: column blocks 0, 1 are 16 gate features, 2, 3 the same features' up rows
                const int n0 = GATED ? (j2 * 64 + wn * 16) : (wn * 32 + j2 * 16);
                const bf16* p = &w_s[buf][n0 + (lane & 7) + (lane >> 4) * 8][ks + ((lane >> 3) & 1) * 8];
                const unsigned s = (unsigned)__cvta_generic_to_shared(p);
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
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * 32 + i * 16 + (lane >> 2) + half * 8;
            const long row = (long)tile * MOE_TM + r;
            if (GATED) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int f = blockIdx.y * 64 + wn * 16 + j * 8 + (lane & 3) * 2 + c;
                        if (f < n_out)
                            act_out[row * out_ld + f] = __float2bfloat16_rn(fl_gated(acc[i][j][half * 2 + c],
                                                                                     acc[i][j + 2][half * 2 + c], act));
                    }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int col = blockIdx.y * 128 + wn * 32 + j * 8 + (lane & 3) * 2 + c;
                        if (col >= n_out) continue;
                        if (MODE == MOE_UP) act_out[row * out_ld + col] = __float2bfloat16_rn(fl_gated(acc[i][j][half * 2 + c], 1.0f, act));
                        else y_out[row * out_ld + col] = acc[i][j][half * 2 + c];
                    }
            }
        }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, long y_ld, const int* __restrict__ pair_row,
                                                          const float* __restrict__ weights, T* __restrict__ out, long out_ld,
                                                          int width, int top, int accumulate) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) sum += weights[(long)t * top + k] * y[(long)pair_row[(long)t * top + k] * y_ld + c];
        out[(long)t * out_ld + c] = from_f32<T>(accumulate ? to_f32<T>(out[(long)t * out_ld + c]) + sum : sum);
    }
}

// Rows of the ordered buffers a step of n_tokens needs: every expert may end with a partly filled tile.
FL_API long fl_moe_group_rows(int n_tokens, int top, int experts) {
    return (((long)n_tokens * top + MOE_TM - 1) / MOE_TM + experts) * MOE_TM;
}

// Does the grouped path take this problem?  (bfloat16 everywhere, K of both products a multiple of 32.)
FL_API int fl_moe_group_takes(int dtype, int w_dtype, int width, int ff) {
    return dtype == FL_BF16 && w_dtype == FL_BF16 && width % MOE_BK == 0 && ff % MOE_BK == 0;
}

static int moe_group_smem_ready() {
    static int rc = -1;
    if (rc < 0) {
        rc = (int)cudaFuncSetAttribute(moe_group_mma_kernel<MOE_GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, MOE_SMEM);
        if (rc == 0)
            rc = (int)cudaFuncSetAttribute(moe_group_mma_kernel<MOE_DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, MOE_SMEM);
        if (rc == 0)
            rc = (int)cudaFuncSetAttribute(moe_group_mma_kernel<MOE_UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, MOE_SMEM);
    }
    return rc;
}

// ints: row_pair [rows] | pair_row [n_tokens * top] | tile_expert [rows / 64] | n_tiles [1];
// act: bfloat16 [rows, ff]; y: float [rows, width].
FL_API int fl_moe_experts_grouped(const void* h, long h_ld, const void* w_gu, const void* w_down, const int* chosen,
                                  const float* weights, int* ints, void* act, float* y, void* out, long out_ld,
                                  int n_tokens, int width, int ff, int top, int experts, int act_code, float act_p0, float act_p1,
                                  int gated, int accumulate, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (act_code < 0 || act_code >= FL_ACT_COUNT) return (int)cudaErrorInvalidValue;
    const FlGate gate{act_code, act_p0, act_p1};
    const long rows = fl_moe_group_rows(n_tokens, top, experts);
    const int max_tiles = (int)(rows / MOE_TM);
    int* row_pair = ints;
    int* pair_row = row_pair + rows;
    int* tile_expert = pair_row + (long)n_tokens * top;
    int* n_tiles = tile_expert + max_tiles;
    if ((size_t)(2 * experts + 1) * sizeof(int) > 48 * 1024 || ((uintptr_t)h % 16) || (h_ld % 8)) return (int)cudaErrorInvalidValue;
    int rc = moe_group_smem_ready();
    if (rc) return rc;
    rc = fl_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)(2 * experts + 1) * sizeof(int), stream, chosen,
                       n_tokens * top, experts, row_pair, pair_row, tile_expert, n_tiles, max_tiles);
    if (rc) return rc;
    if (gated)
        rc = fl_launch(moe_group_mma_kernel<MOE_GATED>, dim3(max_tiles, (ff + 63) / 64), dim3(256), MOE_SMEM, stream, (const bf16*)h, h_ld,
                       (const bf16*)w_gu, ff, width, (const int*)row_pair, (const int*)tile_expert, (const int*)n_tiles, top,
                       (bf16*)act, (float*)nullptr, (long)ff, gate);
    else
        rc = fl_launch(moe_group_mma_kernel<MOE_UP>, dim3(max_tiles, (ff + 127) / 128), dim3(256), MOE_SMEM, stream, (const bf16*)h, h_ld,
                       (const bf16*)w_gu, ff, width, (const int*)row_pair, (const int*)tile_expert, (const int*)n_tiles, top,
                       (bf16*)act, (float*)nullptr, (long)ff, gate);
    if (rc) return rc;
    rc = fl_launch(moe_group_mma_kernel<MOE_DOWN>, dim3(max_tiles, (width + 127) / 128), dim3(256), MOE_SMEM, stream,
                   (const bf16*)act, (long)ff, (const bf16*)w_down, width, ff, (const int*)row_pair,
                   (const int*)tile_expert, (const int*)n_tiles, top, (bf16*)nullptr, y, (long)width, gate);
    if (rc) return rc;
    int col_blocks = (width + 255) / 256;
    if (col_blocks > 8) col_blocks = 8;
    return fl_launch(moe_combine_kernel<bf16>, dim3(n_tokens, col_blocks), dim3(256), 0, stream, (const float*)y,
                     (long)width, (const int*)pair_row, weights, (bf16*)out, out_ld, width, top, accumulate);
}
