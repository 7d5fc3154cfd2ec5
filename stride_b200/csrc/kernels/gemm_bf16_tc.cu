// bfloat16 matrix product on the fifth-generation tensor cores:
//   D[M, N] = A[M, K] * B[N, K]^T     (both operands row-major with K innermost)
//
// One CTA computes a 128 x BLOCK_N tile. A producer thread streams 128x64 and
// BLOCK_N x 64 tiles of A and B into a ring of shared-memory stages with TMA
// (cp.async.bulk.tensor, 128-byte swizzle, completion on an mbarrier); one thread
// issues tcgen05.mma (M = 128, N = BLOCK_N, K = 16 per instruction) with the
// accumulator in tensor memory and frees each stage with tcgen05.commit; four
// epilogue warps read the accumulator back with tcgen05.ld and store it.
//
// The decode step uses it "swapped": A is the weight matrix [out, in] (so the
// 128 rows of a tile are output features and the weights stream through the
// deep TMA ring once), B is the activation [tokens, in] with BLOCK_N >= tokens,
// and the epilogue stores the tile transposed into out[tokens, out]. With few
// output tiles the K range is split over several CTAs (grid.z); each writes a
// float32 partial tile to scratch, takes a ticket, and the CTA that takes the
// last ticket adds the partials in split order and stores the result. Nobody
// waits for another CTA.
//
// For 17 to 64 tokens (decode steps of many requests) the CTAs that share an output
// tile form a thread-block cluster instead (CLUSTER): when all of them have finished
// their part of K, the others write their accumulators into the first one's shared
// memory (the ring, no longer in use) over the cluster's network, and the first adds
// them in split order and stores the tile. No partial tile touches global memory;
// the cluster's barrier, which every CTA of it passes twice, is the only wait, and
// CTAs of a cluster are guaranteed to run together.
//
// Every wait on an mbarrier is bounded by a clock; a wait that runs out sets
// *status and the CTA winds down (tensor memory is freed on every path).
#include <cstdio>

#include "tcgen05.cuh"

namespace stride {
namespace tc {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;              // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;            // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue

// kind::f16 instruction descriptor: float32 accumulator, bf16 x bf16, both K-major, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
}

template <typename OutT>
__device__ __forceinline__ void store_value(OutT* p, float v);
template <>
__device__ __forceinline__ void store_value<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_value<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// D tile rows are rows of A, columns are rows of B. TRANSPOSED: out[col * ldo + row]
// (swapped use: rows are output features, columns tokens); else out[row * ldo + col].
// GATED (swapped use, one split, bfloat16 out): the rows of A alternate in blocks of 64 between the gate and the
// up matrix of a gated feed-forward; the tile's rows 0-63 and 64-127 then belong together, and the epilogue writes
// silu(gate) * up, 64 columns of the inner activation per tile, instead of the 128 products.
template <int BLOCK_N, int STAGES, bool TRANSPOSED, bool A_INDEPENDENT, typename OutT, bool GATED = false, bool CLUSTER = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tn_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, OutT* __restrict__ out,
                    int ldo, int M, int N, int K, int k_blocks_per_split, float* __restrict__ partials,
                    int* __restrict__ tickets, int* __restrict__ status, const float* __restrict__ norm_partials, int norm_count,
                    float norm_eps) {
    constexpr int A_BYTES = kBlockM * kBlockK * 2;
    constexpr int B_BYTES = BLOCK_N * kBlockK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = BLOCK_N < 32 ? 32 : BLOCK_N;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int last_flag;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * kBlockM, n0 = blockIdx.y * BLOCK_N;
    const int total_k_blocks = (K + kBlockK - 1) / kBlockK;
    const int kb_begin = blockIdx.z * k_blocks_per_split;
    const int kb_end = min(total_k_blocks, kb_begin + k_blocks_per_split);
    const int num_kb = max(0, kb_end - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&done_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: one thread feeds the ring. The A operand (the weights, when the
            // product is used swapped) is written by no kernel of the step, so its first
            // ring of tiles is requested before waiting for the kernel that produces B.
            const int early = A_INDEPENDENT ? min(num_kb, STAGES) : 0;
            for (int i = 0; i < early; ++i) {
                const uint32_t bar = smem_u32(&full_bar[i]);
                mbar_expect_tx(bar, STAGE_BYTES);
                tma_load_2d(smem_u32(smem + i * STAGE_BYTES), &map_a, bar, (kb_begin + i) * kBlockK, m0);
            }
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(smem_u32(smem + i * STAGE_BYTES) + A_BYTES, &map_b, smem_u32(&full_bar[i]), (kb_begin + i) * kBlockK, n0);
            for (int i = early; i < num_kb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(smem_u32(&empty_bar[s]), ((i / STAGES) & 1) ^ 1, status, 1)) break;
                const uint32_t bar = smem_u32(&full_bar[s]);
                mbar_expect_tx(bar, STAGE_BYTES);
                const uint32_t a_dst = smem_u32(smem + s * STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, bar, (kb_begin + i) * kBlockK, m0);
                tma_load_2d(a_dst + A_BYTES, &map_b, bar, (kb_begin + i) * kBlockK, n0);
            }
        }
        __syncwarp();
        if constexpr (CLUSTER) {       // take part in the cluster's two barriers (see the epilogue)
            cluster_arrive();
            cluster_wait();
            cluster_arrive();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issuer
            constexpr uint32_t idesc = instr_desc(BLOCK_N);
            bool ok = true;
            for (int i = 0; i < num_kb && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(smem_u32(&full_bar[s]), (i / STAGES) & 1, status, 2);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
                const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                    // advancing 16 elements along K inside the swizzled row: +32 bytes = +2 in the address field
                    umma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(smem_u32(&empty_bar[s]));      // the stage is free once these products have read it
            }
            umma_commit(smem_u32(&done_bar));              // the accumulator is complete
        }
        __syncwarp();
        if constexpr (CLUSTER) {
            cluster_arrive();
            cluster_wait();
            cluster_arrive();
        }
    } else {
        // ---- epilogue: warps 2..5 own the lane quadrants 2, 3, 0, 1 of tensor memory
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                  // row of the tile this thread holds
        float norm_part = 0.f;                             // GATED with a folded norm: this thread's share of a token's sum of squares
        if constexpr (GATED) {
            if (norm_partials != nullptr) {
                pdl_wait();                                // the sums are written by the kernel before this one
                for (int c = row >> 4; c < norm_count; c += 8) norm_part += norm_partials[c * 16 + (row & 15)];
            }
        }
        const bool ok = mbar_wait(smem_u32(&done_bar), 0, status, 3);
        tc_fence_after();
        pdl_wait();        // returns at once here (the producer passed it long ago); keeps this thread's stores ordered too
        if constexpr (CLUSTER) {
            // The CTAs of the cluster hold the same output tile for different parts of K (blockIdx.z = rank in the
            // cluster). First barrier: every CTA's products are complete, so every ring is free and every CTA runs.
            // Then the others send their accumulators into the first CTA's ring, [rank - 1][row][BLOCK_N] float32 with
            // the 16-byte chunks of a row permuted by the row's low bits (a thread owns a row: without that all lanes
            // of a warp would hit one bank). Second barrier: the partial tiles have landed; the first CTA adds them in
            // the order of the ranks and stores.
            static_assert(!CLUSTER || !GATED, "the gated epilogue is not written for clusters");
            constexpr int CHUNKS = BLOCK_N / 4, MASK = CHUNKS >= 8 ? 7 : CHUNKS - 1;
            const uint32_t rank = cluster_rank();
            float* part = reinterpret_cast<float*>(smem);
            cluster_arrive();
            cluster_wait();
            if (rank != 0) {
#pragma unroll
                for (int c0 = 0; c0 < BLOCK_N; c0 += 16) {
                    float v[16];
                    if (ok && num_kb > 0) {
                        tmem_ld16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + c0, v);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const int chunk = ((c0 + j) / 4) ^ (row & MASK);
                        store_cluster_f4(smem_u32(part + (static_cast<size_t>(rank - 1) * kBlockM + row) * BLOCK_N + chunk * 4), 0, v[j], v[j + 1],
                                         v[j + 2], v[j + 3]);
                    }
                }
                cluster_arrive();
            } else {
                cluster_arrive();
                cluster_wait();
                const int r = m0 + row;
#pragma unroll
                for (int c0 = 0; c0 < BLOCK_N; c0 += 16) {
                    float v[16];
                    if (ok && num_kb > 0) {
                        tmem_ld16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + c0, v);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
                    }
                    for (int z = 1; z < static_cast<int>(gridDim.z); ++z) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            const int chunk = ((c0 + j) / 4) ^ (row & MASK);
                            const float4 p = *reinterpret_cast<const float4*>(part + (static_cast<size_t>(z - 1) * kBlockM + row) * BLOCK_N + chunk * 4);
                            v[j] += p.x; v[j + 1] += p.y; v[j + 2] += p.z; v[j + 3] += p.w;
                        }
                    }
                    if (ok) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int c = n0 + c0 + j;
                            if (r < M && c < N) {
                                if (TRANSPOSED) store_value<OutT>(out + static_cast<size_t>(c) * ldo + r, v[j]);
                                else store_value<OutT>(out + static_cast<size_t>(r) * ldo + c, v[j]);
                            }
                        }
                    }
                }
            }
        } else {
        const bool split = gridDim.z > 1;
        const int tile = blockIdx.y * gridDim.x + blockIdx.x;
        float* my_partial = split ? partials + ((static_cast<size_t>(blockIdx.z) * gridDim.x * gridDim.y + tile) * kBlockM + row) * BLOCK_N
                                  : nullptr;
        if constexpr (GATED) {
            static_assert(!GATED || (BLOCK_N == 16 && TRANSPOSED), "the gated epilogue is written for one 16-token column block");
            // The activations may be the x~ of an RMS norm folded into the products around it (gemm_bf16_stream.cu,
            // RowNorm): then the accumulators still lack the factor 1/rms of their token, which is formed here from
            // the producer's sums of squares (norm_partials [norm_count][16], width K), eight threads per token,
            // added in a fixed order.
            float* fold = reinterpret_cast<float*>(smem) + 64 * 17;         // [8][16] partial sums, then [16] factors
            {
                fold[(row >> 4) * 16 + (row & 15)] = norm_part;      // summed while the products were still running
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (row < 16) {
                    float all = 0.f;
#pragma unroll
                    for (int p8 = 0; p8 < 8; ++p8) all += fold[p8 * 16 + row];
                    fold[128 + row] = norm_partials != nullptr ? rsqrtf(all / static_cast<float>(K) + norm_eps) : 1.f;
                }
            }
            float v[16];
            if (ok && num_kb > 0) {
                tmem_ld16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16), v);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.f;
            }
            // The up half of the tile is handed to the gate half through the first stage of the ring, which
            // nothing reads any more (static shared memory of its own would cost the second CTA per SM).
            float (*up_rows)[17] = reinterpret_cast<float (*)[17]>(smem);
            if (row >= 64) {
#pragma unroll
                for (int j = 0; j < 16; ++j) up_rows[row - 64][j] = v[j];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");          // the four epilogue warps, on every path
            if (ok) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] *= fold[128 + j];
            }
            if (ok && row < 64) {
                const int col = m0 / 2 + row;                        // column of the inner activation
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int c = n0 + j;
                    if (c < N) {
                        // as the unfused path: both products rounded to bfloat16, the activation in float32
                        const float g = __bfloat162float(__float2bfloat16_rn(v[j]));
                        const float u = __bfloat162float(__float2bfloat16_rn(up_rows[row][j] * fold[128 + j]));
                        out[static_cast<size_t>(c) * ldo + col] = __float2bfloat16_rn(g / (1.f + __expf(-g)) * u);
                    }
                }
            }
        } else if (ok) {
#pragma unroll
            for (int c0 = 0; c0 < BLOCK_N; c0 += 16) {
                float v[16];
                if (num_kb > 0) {
                    tmem_ld16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + c0, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.f;
                }
                if (split) {
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        *reinterpret_cast<float4*>(my_partial + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                } else {
                    const int r = m0 + row;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int c = n0 + c0 + j;
                        if (r < M && c < N) {
                            if (TRANSPOSED) store_value<OutT>(out + static_cast<size_t>(c) * ldo + r, v[j]);
                            else store_value<OutT>(out + static_cast<size_t>(r) * ldo + c, v[j]);
                        }
                    }
                }
            }
        }
        if (split) {
            // Publish the partial tile, take a ticket; the last CTA of the tile adds all partials in split order.
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");          // the four epilogue warps only
            if (threadIdx.x == 64) last_flag = atomicAdd(&tickets[tile], 1) == static_cast<int>(gridDim.z) - 1;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (last_flag) {
                __threadfence();
                const int r = m0 + row;
#pragma unroll
                for (int c0 = 0; c0 < BLOCK_N; c0 += 4) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int z = 0; z < static_cast<int>(gridDim.z); ++z) {
                        const float4 p = __ldcg(reinterpret_cast<const float4*>(
                            partials + ((static_cast<size_t>(z) * gridDim.x * gridDim.y + tile) * kBlockM + row) * BLOCK_N + c0));
                        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
                    }
                    const float vv[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int c = n0 + c0 + j;
                        if (r < M && c < N) {
                            if (TRANSPOSED) store_value<OutT>(out + static_cast<size_t>(c) * ldo + r, vv[j]);
                            else store_value<OutT>(out + static_cast<size_t>(r) * ldo + c, vv[j]);
                        }
                    }
                }
                if (threadIdx.x == 64) tickets[tile] = 0;            // ready for the next launch
            }
        }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int BLOCK_N, int STAGES, bool TRANSPOSED, typename OutT, bool GATED = false>
int launch(const CUtensorMap* map_a, const CUtensorMap* map_b, OutT* out, int ldo, int M, int N, int K, int splits,
           float* partials, int* tickets, int* status, cudaStream_t stream, const float* norm_partials = nullptr, int norm_count = 0,
           float norm_eps = 0.f) {
    constexpr int smem = STAGES * (kBlockM * kBlockK * 2 + BLOCK_N * kBlockK * 2) + 1024;
    static bool configured = false;
    auto kernel = gemm_tn_bf16_kernel<BLOCK_N, STAGES, TRANSPOSED, TRANSPOSED, OutT, GATED>;   // swapped use: A holds weights
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    const int k_blocks = (K + kBlockK - 1) / kBlockK;
    const int per_split = (k_blocks + splits - 1) / splits;
    dim3 grid((M + kBlockM - 1) / kBlockM, (N + BLOCK_N - 1) / BLOCK_N, splits);
    stride::launch(kernel, dim3(grid), dim3(kThreads), smem, stream, *map_a, *map_b, out, ldo, M, N, K, per_split, partials, tickets, status,
                   norm_partials, norm_count, norm_eps);
    return STRIDE_LAUNCH_STATUS();
}

// The product with the CTAs of an output tile in a cluster of `splits` (1 to 8): no scratch in global memory.
template <int BLOCK_N, int STAGES, typename OutT>
int launch_clustered(const CUtensorMap* map_a, const CUtensorMap* map_b, OutT* out, int ldo, int M, int N, int K, int splits,
                     int* status, cudaStream_t stream) {
    constexpr int smem = STAGES * (kBlockM * kBlockK * 2 + BLOCK_N * kBlockK * 2) + 1024;
    static bool configured[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return STRIDE_BAD_ARGUMENT;
    auto kernel = gemm_tn_bf16_kernel<BLOCK_N, STAGES, true, true, OutT, false, true>;
    if (!configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured[device] = true;
    }
    // the partial tiles of the other CTAs must fit the first one's ring
    if (static_cast<long long>(splits - 1) * kBlockM * BLOCK_N * 4 > smem - 1024) return STRIDE_UNSUPPORTED;
    const int k_blocks = (K + kBlockK - 1) / kBlockK;
    const int per_split = (k_blocks + splits - 1) / splits;
    dim3 grid((M + kBlockM - 1) / kBlockM, (N + BLOCK_N - 1) / BLOCK_N, splits);
    stride::launch_clusters(kernel, grid, dim3(kThreads), smem, stream, splits, *map_a, *map_b, out, ldo, M, N, K, per_split,
                            static_cast<float*>(nullptr), static_cast<int*>(nullptr), status, static_cast<const float*>(nullptr), 0, 0.f);
    return STRIDE_LAUNCH_STATUS();
}

}  // namespace tc
}  // namespace stride

using namespace stride;

extern "C" {

// CTAs per output tile for the clustered product: as many as it takes to put a CTA on every SM, each with at least
// four 64-wide blocks of K, at most four (what the ring holds of partial tiles at 64 tokens).
int stride_gemm_tc_cluster_splits(int rows_a, int k) {
    const int tiles = (rows_a + tc::kBlockM - 1) / tc::kBlockM;
    const int k_blocks = (k + tc::kBlockK - 1) / tc::kBlockK;
    int splits = 148 / (tiles > 0 ? tiles : 1);
    if (splits > 4) splits = 4;
    if (splits > k_blocks / 4) splits = k_blocks / 4;
    return splits < 1 ? 1 : splits;
}

// out = x @ w^T for 17 to 64 tokens (it takes fewer too), computed swapped with the CTAs of an output tile in a
// cluster; see the kernel. Needs no scratch. Returns -2 for shapes it does not take (k % 8 != 0, more than 64
// tokens, unaligned pointers); the caller then uses the library product.
int stride_gemm_tc_clustered(const void* x, const void* w, void* out, int tokens, int n_out, int k, int out_is_f32, int* status,
                             cudaStream_t stream) {
    if (tokens < 0 || n_out <= 0 || k <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (tokens > 64 || k % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return STRIDE_UNSUPPORTED;
    if (status == nullptr) return STRIDE_BAD_ARGUMENT;
    const int block_n = tokens <= 16 ? 16 : (tokens <= 32 ? 32 : 64);
    const int splits = stride_gemm_tc_cluster_splits(n_out, k);
    const CUtensorMap* map_a = tc::cached_map(w, n_out, k, k, tc::kBlockM);
    const CUtensorMap* map_b = tc::cached_map(x, tokens, k, k, block_n);
    if (!map_a || !map_b) return STRIDE_UNSUPPORTED;
#define STRIDE_TC_CLUSTERED(BN, ST)                                                                                              \
    (out_is_f32 ? tc::launch_clustered<BN, ST, float>(map_a, map_b, static_cast<float*>(out), n_out, n_out, tokens, k, splits,   \
                                                      status, stream)                                                           \
                : tc::launch_clustered<BN, ST, __nv_bfloat16>(map_a, map_b, static_cast<__nv_bfloat16*>(out), n_out, n_out,      \
                                                              tokens, k, splits, status, stream))
    switch (block_n) {
        // stages sized so that two CTAs fit one SM (a ring as deep as shared memory allows, one CTA per SM, measured
        // 7 % slower over a decode step of 32 tokens: the widest matrix has 224 tiles for 148 SMs)
        case 16: return STRIDE_TC_CLUSTERED(16, 6);
        case 32: return STRIDE_TC_CLUSTERED(32, 5);
        default: return STRIDE_TC_CLUSTERED(64, 4);
    }
#undef STRIDE_TC_CLUSTERED
}

// How many CTAs split the K range for these sizes (also sizes the scratch): enough
// to give every SM about two CTAs, each with at least eight 64-wide K blocks.
int stride_gemm_tc_splits(int rows_a, int rows_b, int k) {
    const int tiles = ((rows_a + tc::kBlockM - 1) / tc::kBlockM) * ((rows_b + 255) / 256);
    const int k_blocks = (k + tc::kBlockK - 1) / tc::kBlockK;
    int splits = 296 / (tiles > 0 ? tiles : 1);
    if (splits > 8) splits = 8;
    if (splits > k_blocks / 8) splits = k_blocks / 8;
    return splits < 1 ? 1 : splits;
}

// float32 elements of scratch for the partial tiles, and int32 ticket counters (zeroed once by the caller).
long long stride_gemm_tc_scratch_floats(int rows_a, int rows_b, int k) {
    const int splits = stride_gemm_tc_splits(rows_a, rows_b, k);
    if (splits == 1) return 0;
    const int block_n = rows_b <= 16 ? 16 : (rows_b <= 32 ? 32 : (rows_b <= 64 ? 64 : (rows_b <= 128 ? 128 : 256)));
    const long long tiles = static_cast<long long>((rows_a + tc::kBlockM - 1) / tc::kBlockM) * ((rows_b + block_n - 1) / block_n);
    return static_cast<long long>(splits) * tiles * tc::kBlockM * block_n;
}
int stride_gemm_tc_tickets(int rows_a, int rows_b) {
    return ((rows_a + tc::kBlockM - 1) / tc::kBlockM) * ((rows_b + 15) / 16);
}

// out = x @ w^T for few tokens, computed swapped: the weight rows are the 128-row
// tile dimension. x: [tokens, k] bf16, w: [n_out, k] bf16, out: [tokens, n_out]
// (bf16 when out_is_f32 == 0, float32 otherwise). Returns -2 for shapes it does
// not take (k % 8 != 0, tokens > 256, unaligned pointers), after which the
// caller uses the library product.
int stride_gemm_tc_skinny(const void* x, const void* w, void* out, int tokens, int n_out, int k, int out_is_f32,
                          float* partials, long long partial_floats, int* tickets, int ticket_count, int* status,
                          cudaStream_t stream) {
    if (tokens < 0 || n_out <= 0 || k <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (tokens > 256 || k % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return STRIDE_UNSUPPORTED;
    if (status == nullptr) return STRIDE_BAD_ARGUMENT;
    const int block_n = tokens <= 16 ? 16 : (tokens <= 32 ? 32 : (tokens <= 64 ? 64 : (tokens <= 128 ? 128 : 256)));
    const int splits = stride_gemm_tc_splits(n_out, tokens, k);
    if (splits > 1) {
        if (partials == nullptr || tickets == nullptr || partial_floats < stride_gemm_tc_scratch_floats(n_out, tokens, k) ||
            ticket_count < stride_gemm_tc_tickets(n_out, tokens))
            return STRIDE_BAD_ARGUMENT;
    }
    const CUtensorMap* map_a = tc::cached_map(w, n_out, k, k, tc::kBlockM);
    const CUtensorMap* map_b = tc::cached_map(x, tokens, k, k, block_n);
    if (!map_a || !map_b) return STRIDE_UNSUPPORTED;
#define STRIDE_TC_LAUNCH(BN, ST)                                                                                          \
    (out_is_f32 ? tc::launch<BN, ST, true, float>(map_a, map_b, static_cast<float*>(out), n_out, n_out, tokens, k, splits, \
                                                  partials, tickets, status, stream)                                      \
                : tc::launch<BN, ST, true, __nv_bfloat16>(map_a, map_b, static_cast<__nv_bfloat16*>(out), n_out, n_out,   \
                                                          tokens, k, splits, partials, tickets, status, stream))
    switch (block_n) {
        // stages sized so that two CTAs fit one SM (except the widest tile)
        case 16: return STRIDE_TC_LAUNCH(16, 6);
        case 32: return STRIDE_TC_LAUNCH(32, 5);
        case 64: return STRIDE_TC_LAUNCH(64, 4);
        case 128: return STRIDE_TC_LAUNCH(128, 3);
        default: return STRIDE_TC_LAUNCH(256, 4);
    }
#undef STRIDE_TC_LAUNCH
}

// out = silu(x @ gate^T) * (x @ up^T) for at most 16 tokens. w: [2 * inner, k] bf16 with the rows of gate and up
// alternating in blocks of 64 (gate 0-63, up 0-63, gate 64-127, ...); out: [tokens, inner] bf16. Returns -2 for
// what it does not take (inner % 64 != 0, more than 16 tokens, sizes for which K would be split, unaligned
// operands); the caller then runs the product and the activation separately. With norm_partials, x is the x~ of a
// folded RMS norm (see the kernel) and the factor 1/rms per token is applied here.
int stride_gemm_tc_gated(const void* x, const void* w, void* out, int tokens, int inner, int k, int* status,
                         const float* norm_partials, int norm_count, float norm_eps, cudaStream_t stream) {
    if (tokens < 0 || inner <= 0 || k <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (status == nullptr) return STRIDE_BAD_ARGUMENT;
    if (tokens > 16 || inner % 64 || k % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return STRIDE_UNSUPPORTED;
    if (stride_gemm_tc_splits(2 * inner, tokens, k) != 1) return STRIDE_UNSUPPORTED;
    const CUtensorMap* map_a = tc::cached_map(w, 2 * inner, k, k, tc::kBlockM);
    const CUtensorMap* map_b = tc::cached_map(x, tokens, k, k, 16);
    if (!map_a || !map_b) return STRIDE_UNSUPPORTED;
    return tc::launch<16, 6, true, __nv_bfloat16, true>(map_a, map_b, static_cast<__nv_bfloat16*>(out), inner, 2 * inner, tokens, k, 1,
                                                        nullptr, nullptr, status, stream, norm_partials, norm_count, norm_eps);
}

}  // extern "C"
