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
// Every wait on an mbarrier is bounded by a clock; a wait that runs out sets
// *status and the CTA winds down (tensor memory is freed on every path).
#include <cuda.h>

#include <cstdio>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace stride {
namespace tc {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;              // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;            // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr long long kWaitCycles = 4000000000LL;   // about two seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Returns false (and records `code`) when the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
    const long long start = clock64();
    while (true) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if (clock64() - start > kWaitCycles) {
            atomicCAS(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive columns: thread i of the warp gets lane (base + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes,
// stored with the 128-byte swizzle: 8-row groups 1024 bytes apart (stride byte
// offset 64 in 16-byte units), leading byte offset 1, descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | (1u << 16);
    const uint32_t hi = 64u | (1u << 14) | (2u << 29);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}
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
template <int BLOCK_N, int STAGES, bool TRANSPOSED, bool A_INDEPENDENT, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tn_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, OutT* __restrict__ out,
                    int ldo, int M, int N, int K, int k_blocks_per_split, float* __restrict__ partials,
                    int* __restrict__ tickets, int* __restrict__ status) {
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
    } else {
        // ---- epilogue: warps 2..5 own the lane quadrants 2, 3, 0, 1 of tensor memory
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                  // row of the tile this thread holds
        const bool ok = mbar_wait(smem_u32(&done_bar), 0, status, 3);
        tc_fence_after();
        pdl_wait();        // returns at once here (the producer passed it long ago); keeps this thread's stores ordered too
        const bool split = gridDim.z > 1;
        const int tile = blockIdx.y * gridDim.x + blockIdx.x;
        float* my_partial = split ? partials + ((static_cast<size_t>(blockIdx.z) * gridDim.x * gridDim.y + tile) * kBlockM + row) * BLOCK_N
                                  : nullptr;
        if (ok) {
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
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------------- host
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

// A [rows, cols] bf16 row-major matrix viewed in boxes of box_rows x 64 with the 128-byte swizzle.
// Rows and columns past the end read as zero.
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    const cuuint32_t box[2] = {kBlockK, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapKey {
    const void* base;
    long long rows, cols, ld;
    int box_rows;
    bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.base);
        h = h * 1000003u ^ static_cast<size_t>(k.rows);
        h = h * 1000003u ^ static_cast<size_t>(k.cols);
        h = h * 1000003u ^ static_cast<size_t>(k.ld * 31 + k.box_rows);
        return h;
    }
};

static const CUtensorMap* cached_map(const void* base, long long rows, long long cols, long long ld, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    MapKey key{base, rows, cols, ld, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) return &it->second;
    CUtensorMap m;
    if (!make_map(&m, base, rows, cols, ld, box_rows)) return nullptr;
    return &cache.emplace(key, m).first->second;
}

template <int BLOCK_N, int STAGES, bool TRANSPOSED, typename OutT>
int launch(const CUtensorMap* map_a, const CUtensorMap* map_b, OutT* out, int ldo, int M, int N, int K, int splits,
           float* partials, int* tickets, int* status, cudaStream_t stream) {
    constexpr int smem = STAGES * (kBlockM * kBlockK * 2 + BLOCK_N * kBlockK * 2) + 1024;
    static bool configured = false;
    auto kernel = gemm_tn_bf16_kernel<BLOCK_N, STAGES, TRANSPOSED, TRANSPOSED, OutT>;   // swapped use: A holds weights
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    const int k_blocks = (K + kBlockK - 1) / kBlockK;
    const int per_split = (k_blocks + splits - 1) / splits;
    dim3 grid((M + kBlockM - 1) / kBlockM, (N + BLOCK_N - 1) / BLOCK_N, splits);
    stride::launch(kernel, dim3(grid), dim3(kThreads), smem, stream, *map_a, *map_b, out, ldo, M, N, K, per_split, partials, tickets, status);
    return STRIDE_LAUNCH_STATUS();
}

}  // namespace tc
}  // namespace stride

using namespace stride;

extern "C" {

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

}  // extern "C"
