// out = x @ w^T in bfloat16 for 17 to 128 tokens (decode steps of many requests) on the fifth-generation tensor
// cores, with what follows the product in its epilogue.
//
// The product is bound by reading the weights once, and the norm, rotation and activation around it are launches of
// their own when a library computes it. Here the tokens are the rows of the tile: A is the activation [tokens, k],
// B is a block of BLOCK_N output features [BLOCK_N, k] of the weight matrix, and the accumulator [128 tokens x
// BLOCK_N features] lives in tensor memory. One CTA owns its BLOCK_N features for all of K: nothing is split across
// CTAs and nothing is reduced through memory, and BLOCK_N is chosen so that every SM gets a CTA (32 features for a
// 4096-row matrix). A token is a lane of tensor memory, so an epilogue thread holds all BLOCK_N results of its
// token: storing them, adding them to the residual stream, the two halves of an RMS norm, rotating query and key
// pairs and writing the cache, or SiLU(gate) * up are a few lines each, with contiguous 16-byte stores. The price:
// every CTA reads all of the activations (from L2), which is more than its weights once there are more tokens than
// BLOCK_N. Measured against the library product with separate elementwise kernels it is level at 17 to 32 tokens on
// 4096-row matrices and slower otherwise, so the callers use it only when asked to.
//
// A tcgen05.mma costs its issuing thread 60 to 70 cycles whatever its size (measured in attention_prefill_tc.cu), and
// a block of 64 columns of K takes four: ISSUERS warps issue, warp j the blocks j, j + ISSUERS, ... of K, each into
// an accumulator of its own, and the epilogue adds them. Two more warps feed the ring with TMA (one the activation
// tiles, one the weight tiles; the weights do not depend on the kernel before this one, so their first ring is
// requested before the dependency wait). The ring is as deep as shared memory allows, because the bytes in flight
// decide the bandwidth: the activation box has only as many rows as there are tokens (rounded up to 8), the rows of
// the 128-row operand past it are whatever lies behind in shared memory, and so are the accumulator rows that
// nobody reads. Every wait on an mbarrier is bounded; a wait that runs out sets *status.
#include "mma.cuh"
#include "tcgen05.cuh"

namespace stride {
namespace rows_gemm {

constexpr int kRows = 128;               // token rows of the tile (the M of the product)
constexpr int kBlockK = 64;              // 64 bf16 = one 128-byte swizzle row
constexpr int kMaxStages = 32;
// warps 0-1: TMA (activations, weights), 2 .. 2 + ISSUERS - 1: tensor-core issuers (warp 2 owns tensor memory), then four epilogue warps
__host__ __device__ constexpr int threads_of(int issuers) { return (2 + issuers + 4) * 32; }

enum Mode { kStore = 0, kStoreF32 = 1, kAddResidual = 2, kQkvRope = 3, kGated = 4, kAddResidualNorm = 5 };

// What the projection of queries, keys and values does with its result instead of storing it (kQkvRope): bias,
// rotation of queries and keys by the token's position (pairs (i, i + hd/2), float32 tables [position][hd/2]:
// python/stride_worker/layers.py:85-106), queries into `out`, keys and values into the token's slot of the paged
// cache (python/stride_worker/cache.py:58-90, pages [page][kv head][slot][hd]). The CTA's BLOCK_N features are
// BLOCK_N / 2 rotation pairs of one head: the pairs' first halves in columns [0, BLOCK_N / 2), their second halves
// after them (two boxes of weight rows per stage).
struct QkvEpilogue {
    const float* bias;                 // [(nq + 2 nkv) * hd] or null
    const int32_t* positions;          // [tokens]
    const int32_t* slot_mapping;       // [tokens], page * page_size + offset, negative: store nothing; null: store nothing
    const float* cos_table;
    const float* sin_table;
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    int nq, nkv, hd, page_size, rotate;
};

// An RMS norm folded into the products around it (python/stride_worker/layers.py:20-36 gives the norm:
// x * rsqrt(mean(x^2) + eps) * weight, in float32). The product before the norm (kAddResidualNorm) adds itself to the
// residual stream, writes x~ = residual * norm_weight in bfloat16 and, per CTA and token, the sum of squares of its
// columns of the residual: partials_out[cta][128]. The product after the norm reads x~ as its activations and
// multiplies its accumulators by rsqrt(sum over `count` CTAs of partials / k + eps): a token is an epilogue thread,
// so the factor is one scalar per thread.
struct NormFold {
    const float* partials;             // consumer: [count][128], or null
    int count;
    float eps;
    const float* norm_weight;          // producer: [n_out]
    __nv_bfloat16* xt;                 // producer: [tokens, n_out]
    float* partials_out;               // producer: [ctas][128]
};

__host__ __device__ constexpr uint32_t instr_desc(int n) {       // float32 accumulator, bf16 x bf16, both K-major, M = 128
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kRows >> 4) << 24);
}

// `stages` is a multiple of ISSUERS: an issuer sees every phase of the barriers it waits on only if its blocks of K
// always fall on the same stages (a wait by parity that skips a phase can mistake an older phase for its own).
// Shared memory: the ring of activation boxes [stages][x_rows x 64], then the ring of weight boxes [stages][BLOCK_N x 64].
template <int BLOCK_N, int ISSUERS, int MODE>
__global__ void __launch_bounds__(threads_of(ISSUERS), 1)
gemm_rows_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, void* __restrict__ out, int ldo,
                 int tokens, int n_out, int k, int x_rows, int stages, float* __restrict__ residual, const QkvEpilogue qkv,
                 const NormFold fold, int* __restrict__ status) {
    constexpr int W_BYTES = BLOCK_N * kBlockK * 2;
    constexpr int ACC_COLS = ISSUERS * BLOCK_N;
    static_assert(ACC_COLS <= 512, "the accumulators do not fit tensor memory");
    constexpr uint32_t TMEM_COLS = ACC_COLS <= 32 ? 32 : (ACC_COLS <= 64 ? 64 : (ACC_COLS <= 128 ? 128 : (ACC_COLS <= 256 ? 256 : 512)));
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int x_bytes = x_rows * kBlockK * 2;
    unsigned char* w_ring = smem + stages * x_bytes;
    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_base_slot;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (k + kBlockK - 1) / kBlockK;
    // The CTA's features: rows [n0, n0 + BLOCK_N) of the weight matrix, or for kQkvRope BLOCK_N / 2 rotation pairs of
    // one head (rows w0 .. and w0 + hd/2 ..).
    int n0 = blockIdx.x * BLOCK_N, w0 = n0, w1 = 0;
    if (MODE == kQkvRope) {
        const int per_head = qkv.hd / BLOCK_N;                  // CTAs per head
        const int head = blockIdx.x / per_head, part = blockIdx.x - head * per_head;
        w0 = head * qkv.hd + part * (BLOCK_N / 2);
        w1 = w0 + qkv.hd / 2;
        n0 = w0;
    }

    if (threadIdx.x == 32) tc::prefetch_map(&map_w);
    if (threadIdx.x == 64) tc::prefetch_map(&map_x);
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            tc::mbar_init(tc::smem_u32(&full_bar[s]), 2);        // the two copying threads each announce their bytes
            tc::mbar_init(tc::smem_u32(&empty_bar[s]), 1);
        }
        tc::mbar_init(tc::smem_u32(&done_bar), ISSUERS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) tc::tmem_alloc(tc::smem_u32(&tmem_base_slot), TMEM_COLS);
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    // One thread needs about 300 cycles per TMA instruction, far more than a block of K may take; the same instruction
    // executed by several lanes at once, each with its own block of K and stage, costs the warp no more. So a copying
    // warp works in batches of `batch` blocks: lane j waits for the stage of block i0 + j, then all issue together.
    // A batch is a quarter of the ring at most, so that copies are requested while the other stages are worked on.
    const int batch = stages >= 32 ? 8 : (stages >= 4 ? stages / 4 : 1);
    if (warp == 0) {
        // ---- activations: one box of x_rows rows x 64 columns per block of K (written by the kernel before this one)
        pdl_wait();
        for (int i0 = 0; i0 < num_kb; i0 += batch) {
            const int i = i0 + lane;
            const bool mine = lane < batch && i < num_kb;
            const int s = i % stages, turn = i / stages;
            bool ok = true;
            if (mine && turn > 0) ok = tc::mbar_wait(tc::smem_u32(&empty_bar[s]), (turn & 1) ^ 1, status, 51);
            if (__any_sync(0xffffffffu, !ok)) break;
            if (mine) {
                const uint32_t bar = tc::smem_u32(&full_bar[s]);
                tc::mbar_expect_tx(bar, x_bytes);
                tc::tma_load_2d(tc::smem_u32(smem + s * x_bytes), &map_x, bar, i * kBlockK, 0);
            }
        }
    } else if (warp == 1) {
        // ---- weights: they are written by no kernel of the step, so the first ring is requested at once
        for (int i0 = 0; i0 < num_kb; i0 += batch) {
            const int i = i0 + lane;
            const bool mine = lane < batch && i < num_kb;
            const int s = i % stages, turn = i / stages;
            bool ok = true;
            if (mine && turn > 0) ok = tc::mbar_wait(tc::smem_u32(&empty_bar[s]), (turn & 1) ^ 1, status, 52);
            if (__any_sync(0xffffffffu, !ok)) break;
            if (mine) {
                const uint32_t bar = tc::smem_u32(&full_bar[s]);
                const uint32_t dst = tc::smem_u32(w_ring + s * W_BYTES);
                tc::mbar_expect_tx(bar, W_BYTES);
                if (MODE == kQkvRope) {
                    tc::tma_load_2d(dst, &map_w, bar, i * kBlockK, w0);
                    tc::tma_load_2d(dst + W_BYTES / 2, &map_w, bar, i * kBlockK, w1);
                } else {
                    tc::tma_load_2d(dst, &map_w, bar, i * kBlockK, w0);
                }
            }
        }
    } else if (warp < 2 + ISSUERS) {
        // ---- tensor-core issuers: warp 2 + j takes the blocks j, j + ISSUERS, ... of K into accumulator j. The whole
        // warp walks the loop and the waits, one lane issues.
        const int which = warp - 2;
        const bool issuer = tc::elect_one();
        constexpr uint32_t idesc = instr_desc(BLOCK_N);
        const uint32_t acc = tmem_base + which * BLOCK_N;
        bool ok = true;
        for (int i = which, s = which, turn = 0; i < num_kb && ok; i += ISSUERS) {
            ok = tc::mbar_wait(tc::smem_u32(&full_bar[s]), turn & 1, status, 53);
            if (!ok) break;
            tc::tc_fence_after();
            const uint64_t a_desc = tc::smem_desc_sw128(tc::smem_u32(smem + s * x_bytes));
            const uint64_t b_desc = tc::smem_desc_sw128(tc::smem_u32(w_ring + s * W_BYTES));
#pragma unroll
            for (int kk = 0; kk < kBlockK / 16; ++kk) {
                // advancing 16 elements along K inside the swizzled row: +32 bytes = +2 in the address field
                if (issuer) tc::umma_bf16(acc, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (i >= ISSUERS || kk > 0) ? 1u : 0u);
            }
            if (issuer) tc::umma_commit(tc::smem_u32(&empty_bar[s]));      // the stage is free once these products have read it
            s += ISSUERS;
            if (s >= stages) { s -= stages; ++turn; }
        }
        if (issuer) tc::umma_commit(tc::smem_u32(&done_bar));              // this accumulator is complete
    } else {
        // ---- epilogue: warp w may read the lanes 32 (w % 4) .. of tensor memory; a lane is a token
        const int quad = warp & 3;
        const int token = quad * 32 + lane;
        // What the epilogue reads besides the accumulators is asked for before the wait for them: the token's row of
        // the residual stream, or its position, slot and rows of the rotation tables.
        pdl_wait();        // orders this thread's reads and writes of what other kernels wrote
        constexpr bool kSums = MODE == kAddResidual || MODE == kAddResidualNorm;
        constexpr bool kResidualAhead = kSums && BLOCK_N <= 64;
        float scale = 1.f;
        if (fold.partials != nullptr && token < tokens) {       // the factor of the norm before this product
            float total = 0.f;
#pragma unroll 8
            for (int c = 0; c < fold.count; ++c) total += fold.partials[c * kRows + token];
            scale = rsqrtf(total / static_cast<float>(k) + fold.eps);
        }
        float squares = 0.f;
        constexpr int kAhead = kResidualAhead ? BLOCK_N : (MODE == kQkvRope ? BLOCK_N / 2 : 1);
        float ahead[kAhead], ahead_sin[MODE == kQkvRope ? BLOCK_N / 2 : 1];
        int pos = 0, slot = -1;
        const bool full_block = n0 + BLOCK_N <= n_out && (ldo % 4) == 0;
        if (kResidualAhead && token < tokens && full_block) {
            const float4* src = reinterpret_cast<const float4*>(residual + static_cast<size_t>(token) * ldo + n0);
#pragma unroll
            for (int j = 0; j < BLOCK_N / 4; ++j) {
                const float4 r = src[j];
                ahead[4 * j] = r.x; ahead[4 * j + 1] = r.y; ahead[4 * j + 2] = r.z; ahead[4 * j + 3] = r.w;
            }
        }
        if (MODE == kQkvRope && token < tokens) {
            pos = qkv.positions[token];
            const int head = w0 / qkv.hd, in_head = w0 - head * qkv.hd, half = qkv.hd / 2;
            if (head >= qkv.nq && qkv.slot_mapping) slot = qkv.slot_mapping[token];
            if (head < qkv.nq + qkv.nkv && qkv.rotate) {
                const float4* cs = reinterpret_cast<const float4*>(qkv.cos_table + static_cast<size_t>(pos) * half + in_head);
                const float4* sn = reinterpret_cast<const float4*>(qkv.sin_table + static_cast<size_t>(pos) * half + in_head);
#pragma unroll
                for (int j = 0; j < BLOCK_N / 8; ++j) {
                    const float4 c = cs[j], z = sn[j];
                    ahead[4 * j] = c.x; ahead[4 * j + 1] = c.y; ahead[4 * j + 2] = c.z; ahead[4 * j + 3] = c.w;
                    ahead_sin[4 * j] = z.x; ahead_sin[4 * j + 1] = z.y; ahead_sin[4 * j + 2] = z.z; ahead_sin[4 * j + 3] = z.w;
                }
            }
        }
        const bool ok = tc::mbar_wait(tc::smem_u32(&done_bar), 0, status, 54);
        tc::tc_fence_after();
        const int parts = num_kb < ISSUERS ? num_kb : ISSUERS;      // accumulators that were written
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        if (quad * 32 < tokens) {                            // a warp whose 32 tokens all lie past the end has nothing to do
#pragma unroll
            for (int c0 = 0; c0 < BLOCK_N; c0 += 16) {
                if (MODE == kQkvRope && c0 >= BLOCK_N / 2) break;        // the second halves are read with the first
                if (MODE == kGated && c0 >= BLOCK_N / 2) break;          // the up columns are read with the gate columns
                float v[16], u[16];
                tc::tmem_ld16(tmem_base + lane_base + c0, v);
#pragma unroll
                for (int a = 1; a < ISSUERS; ++a) {
                    if (a < parts) {
                        float p[16];
                        tc::tmem_ld16(tmem_base + lane_base + a * BLOCK_N + c0, p);
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] += p[j];
                    }
                }
                if (MODE == kQkvRope || MODE == kGated) {        // the partner columns: second halves of the pairs, or up
                    tc::tmem_ld16(tmem_base + lane_base + BLOCK_N / 2 + c0, u);
#pragma unroll
                    for (int a = 1; a < ISSUERS; ++a) {
                        if (a < parts) {
                            float p[16];
                            tc::tmem_ld16(tmem_base + lane_base + a * BLOCK_N + BLOCK_N / 2 + c0, p);
#pragma unroll
                            for (int j = 0; j < 16; ++j) u[j] += p[j];
                        }
                    }
                }
                if (!ok || token >= tokens) continue;
                if (fold.partials != nullptr) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] *= scale;
                    if (MODE == kQkvRope || MODE == kGated) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) u[j] *= scale;
                    }
                }
                if (MODE == kStore) {
                    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(token) * ldo + n0 + c0;
                    if (n0 + c0 + 16 <= n_out && (ldo % 8) == 0) {
                        uint32_t w[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) w[j] = pack_bf16(v[2 * j], v[2 * j + 1]);
                        *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                        *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (n0 + c0 + j < n_out) dst[j] = __float2bfloat16_rn(v[j]);
                    }
                } else if (MODE == kStoreF32) {
                    float* dst = static_cast<float*>(out) + static_cast<size_t>(token) * ldo + n0 + c0;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (n0 + c0 + j < n_out) dst[j] = v[j];
                } else if (MODE == kAddResidualNorm) {
                    // only launched with whole blocks of at most 64 features: the residual row was read ahead
                    float* dst = residual + static_cast<size_t>(token) * ldo + n0 + c0;
                    __nv_bfloat16* xt = fold.xt + static_cast<size_t>(token) * ldo + n0 + c0;
                    const float4* nw = reinterpret_cast<const float4*>(fold.norm_weight + n0 + c0);
                    float r[16];
                    uint32_t w[8];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        r[j] = __fadd_rn(ahead[(kResidualAhead ? c0 : 0) + j], __bfloat162float(__float2bfloat16_rn(v[j])));
                        squares = fmaf(r[j], r[j], squares);
                    }
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const float4 g = nw[j / 4];
                        *reinterpret_cast<float4*>(dst + j) = make_float4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                        w[j / 2] = pack_bf16(r[j] * g.x, r[j + 1] * g.y);
                        w[j / 2 + 1] = pack_bf16(r[j + 2] * g.z, r[j + 3] * g.w);
                    }
                    *reinterpret_cast<uint4*>(xt) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(xt + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                } else if (MODE == kAddResidual) {
                    // as the unfused path: the product rounded to bfloat16, the sum in float32
                    float* dst = residual + static_cast<size_t>(token) * ldo + n0 + c0;
                    if (kResidualAhead && full_block) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            *reinterpret_cast<float4*>(dst + j) = make_float4(
                                __fadd_rn(ahead[(kResidualAhead ? c0 : 0) + j], __bfloat162float(__float2bfloat16_rn(v[j]))),
                                __fadd_rn(ahead[(kResidualAhead ? c0 : 0) + j + 1], __bfloat162float(__float2bfloat16_rn(v[j + 1]))),
                                __fadd_rn(ahead[(kResidualAhead ? c0 : 0) + j + 2], __bfloat162float(__float2bfloat16_rn(v[j + 2]))),
                                __fadd_rn(ahead[(kResidualAhead ? c0 : 0) + j + 3], __bfloat162float(__float2bfloat16_rn(v[j + 3]))));
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (n0 + c0 + j < n_out) dst[j] = __fadd_rn(dst[j], __bfloat162float(__float2bfloat16_rn(v[j])));
                    }
                } else if (MODE == kGated) {
                    // columns [0, 64) of the tile are gate features, [64, 128) the up features of the same inner columns
                    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(token) * ldo + n0 / 2 + c0;
                    uint32_t w[8];
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        // as the unfused path: both products rounded to bfloat16, the activation in float32
                        const float g0 = __bfloat162float(__float2bfloat16_rn(v[j])), g1 = __bfloat162float(__float2bfloat16_rn(v[j + 1]));
                        const float u0 = __bfloat162float(__float2bfloat16_rn(u[j])), u1 = __bfloat162float(__float2bfloat16_rn(u[j + 1]));
                        w[j / 2] = pack_bf16(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
                    }
                    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                } else {       // kQkvRope: v holds the pairs' first halves (features w0 + c0 ..), u their second halves
                    const int head = w0 / qkv.hd, in_head = w0 - head * qkv.hd + c0;      // index of the first half inside the head
                    const int half = qkv.hd / 2;
                    if (qkv.bias) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            // as the unfused path: the product rounded to bfloat16, then the bias in float32
                            v[j] = __fadd_rn(__bfloat162float(__float2bfloat16_rn(v[j])), qkv.bias[head * qkv.hd + in_head + j]);
                            u[j] = __fadd_rn(__bfloat162float(__float2bfloat16_rn(u[j])), qkv.bias[head * qkv.hd + in_head + half + j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
                            u[j] = __bfloat162float(__float2bfloat16_rn(u[j]));
                        }
                    }
                    if (head < qkv.nq + qkv.nkv && qkv.rotate) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float c = ahead[(MODE == kQkvRope ? c0 : 0) + j], s = ahead_sin[(MODE == kQkvRope ? c0 : 0) + j];
                            const float ra = __fadd_rn(__fmul_rn(v[j], c), __fmul_rn(-u[j], s));
                            const float rb = __fadd_rn(__fmul_rn(u[j], c), __fmul_rn(v[j], s));
                            v[j] = ra;
                            u[j] = rb;
                        }
                    }
                    __nv_bfloat16* lo = nullptr;
                    if (head < qkv.nq) {
                        lo = static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(token) * ldo + head * qkv.hd + in_head;
                    } else {
                        if (slot >= 0) {
                            const bool is_key = head < qkv.nq + qkv.nkv;
                            const int kvh = is_key ? head - qkv.nq : head - qkv.nq - qkv.nkv;
                            lo = (is_key ? qkv.k_pages : qkv.v_pages) +
                                 ((static_cast<size_t>(slot / qkv.page_size) * qkv.nkv + kvh) * qkv.page_size + slot % qkv.page_size) * qkv.hd + in_head;
                        }
                    }
                    if (lo != nullptr) {
                        uint32_t a[8], b[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            a[j] = pack_bf16(v[2 * j], v[2 * j + 1]);
                            b[j] = pack_bf16(u[2 * j], u[2 * j + 1]);
                        }
                        *reinterpret_cast<uint4*>(lo) = make_uint4(a[0], a[1], a[2], a[3]);
                        *reinterpret_cast<uint4*>(lo + 8) = make_uint4(a[4], a[5], a[6], a[7]);
                        *reinterpret_cast<uint4*>(lo + half) = make_uint4(b[0], b[1], b[2], b[3]);
                        *reinterpret_cast<uint4*>(lo + half + 8) = make_uint4(b[4], b[5], b[6], b[7]);
                    }
                }
            }
        }
        if (MODE == kAddResidualNorm && ok && token < tokens) fold.partials_out[blockIdx.x * kRows + token] = squares;
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 2) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

struct Plan {
    int block_n, ctas, x_rows, stages, smem;
};

// Features per CTA: the widest block of 32, 64 or 128 that still gives every SM a CTA (at least 120 of them), 32 at
// the least. The ring: when the grid has more CTAs than SMs, two of them share an SM, so that one's epilogue runs
// under the other's stream and no second wave of few CTAs is left over; each then gets half the shared memory.
inline int choose_block_n(int n_out) {
    if (n_out >= 120 * 128) return 128;
    if (n_out >= 120 * 64) return 64;
    return 32;
}
constexpr int issuers_of(int block_n) { return block_n == 128 ? 2 : 4; }

inline Plan plan_for(int block_n, int ctas, int tokens, int k) {
    Plan p;
    p.block_n = block_n;
    p.ctas = ctas;
    p.x_rows = (tokens + 7) / 8 * 8;
    const int issuers = issuers_of(block_n);
    const int stage = (p.x_rows + block_n) * kBlockK * 2;
    const int num_kb = (k + kBlockK - 1) / kBlockK;
    int sms = 148;
    int budget = ctas > sms ? 110 * 1024 : 220 * 1024;
    if (budget / stage < 2 * issuers) budget = 220 * 1024;
    int stages = budget / stage;
    stages = stages / issuers * issuers;
    const int useful = (num_kb + issuers - 1) / issuers * issuers;
    if (stages > useful) stages = useful;
    if (stages > kMaxStages) stages = kMaxStages / issuers * issuers;
    if (stages < issuers) stages = issuers;
    // the 128-row operand of the last stage's activation box must end inside the allocation
    while (stages * block_n * kBlockK * 2 + p.x_rows * kBlockK * 2 < kRows * kBlockK * 2) stages += issuers;
    p.stages = stages;
    p.smem = stages * stage + 1024;
    return p;
}

template <int BLOCK_N, int MODE>
int launch(const Plan& p, const CUtensorMap* map_x, const CUtensorMap* map_w, void* out, int ldo, int tokens, int n_out, int k,
           float* residual, const QkvEpilogue& qkv, const NormFold& fold, int* status, cudaStream_t stream) {
    constexpr int ISSUERS = issuers_of(BLOCK_N);
    constexpr int kMaxSmem = 226 * 1024;
    if (p.smem > kMaxSmem || p.stages % ISSUERS || p.stages > kMaxStages) return STRIDE_UNSUPPORTED;
    static bool configured[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return STRIDE_BAD_ARGUMENT;
    auto kernel = gemm_rows_kernel<BLOCK_N, ISSUERS, MODE>;
    if (!configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured[device] = true;
    }
    stride::launch(kernel, dim3(p.ctas), dim3(threads_of(ISSUERS)), p.smem, stream, *map_x, *map_w, out, ldo, tokens, n_out, k,
                   p.x_rows, p.stages, residual, qkv, fold, status);
    return STRIDE_LAUNCH_STATUS();
}

inline bool operands_ok(const void* x, const void* w, int tokens, int k) {
    return tokens <= kRows && k % 8 == 0 && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16 == 0;
}

template <int MODE>
int launch_any(const Plan& p, const CUtensorMap* map_x, const CUtensorMap* map_w, void* out, int ldo, int tokens, int n_out, int k,
               float* residual, const QkvEpilogue& qkv, const NormFold& fold, int* status, cudaStream_t stream) {
    switch (p.block_n) {
        case 128: return launch<128, MODE>(p, map_x, map_w, out, ldo, tokens, n_out, k, residual, qkv, fold, status, stream);
        case 64: return launch<64, MODE>(p, map_x, map_w, out, ldo, tokens, n_out, k, residual, qkv, fold, status, stream);
        case 32: return launch<32, MODE>(p, map_x, map_w, out, ldo, tokens, n_out, k, residual, qkv, fold, status, stream);
    }
    return STRIDE_UNSUPPORTED;
}

}  // namespace rows_gemm
}  // namespace stride

using namespace stride;

extern "C" {

// out = x @ w^T for up to 128 tokens. x: [tokens, k] bf16, w: [n_out, k] bf16, out: [tokens, n_out] (bf16 when
// out_is_f32 == 0, float32 otherwise). Returns -2 for what it does not take (k % 8 != 0, more than 128 tokens,
// unaligned pointers); the caller then uses the library product.
int stride_gemm_rows(const void* x, const void* w, void* out, int tokens, int n_out, int k, int out_is_f32, int* status,
                     cudaStream_t stream) {
    if (tokens < 0 || n_out <= 0 || k <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (status == nullptr) return STRIDE_BAD_ARGUMENT;
    if (!rows_gemm::operands_ok(x, w, tokens, k)) return STRIDE_UNSUPPORTED;
    const int bn = rows_gemm::choose_block_n(n_out);
    const rows_gemm::Plan p = rows_gemm::plan_for(bn, (n_out + bn - 1) / bn, tokens, k);
    const CUtensorMap* map_x = tc::cached_map(x, tokens, k, k, p.x_rows);
    const CUtensorMap* map_w = tc::cached_map(w, n_out, k, k, bn);
    if (!map_x || !map_w) return STRIDE_UNSUPPORTED;
    const rows_gemm::QkvEpilogue none = {};
    const rows_gemm::NormFold no_fold = {};
    if (out_is_f32) return rows_gemm::launch_any<rows_gemm::kStoreF32>(p, map_x, map_w, out, n_out, tokens, n_out, k, nullptr, none, no_fold, status, stream);
    return rows_gemm::launch_any<rows_gemm::kStore>(p, map_x, map_w, out, n_out, tokens, n_out, k, nullptr, none, no_fold, status, stream);
}

// residual[tokens, n_out] (float32) += bf16(x @ w^T): the product before a norm, with the residual sum in its epilogue.
int stride_gemm_rows_add(const void* x, const void* w, float* residual, int tokens, int n_out, int k, int* status,
                         cudaStream_t stream) {
    if (tokens < 0 || n_out <= 0 || k <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (status == nullptr || residual == nullptr) return STRIDE_BAD_ARGUMENT;
    if (!rows_gemm::operands_ok(x, w, tokens, k) || reinterpret_cast<uintptr_t>(residual) % 16) return STRIDE_UNSUPPORTED;
    const int bn = rows_gemm::choose_block_n(n_out);
    const rows_gemm::Plan p = rows_gemm::plan_for(bn, (n_out + bn - 1) / bn, tokens, k);
    const CUtensorMap* map_x = tc::cached_map(x, tokens, k, k, p.x_rows);
    const CUtensorMap* map_w = tc::cached_map(w, n_out, k, k, bn);
    if (!map_x || !map_w) return STRIDE_UNSUPPORTED;
    const rows_gemm::QkvEpilogue none = {};
    const rows_gemm::NormFold no_fold = {};
    return rows_gemm::launch_any<rows_gemm::kAddResidual>(p, map_x, map_w, nullptr, n_out, tokens, n_out, k, residual, none, no_fold, status, stream);
}

// The product before an RMS norm with the norm's first half in its epilogue (see NormFold): residual += bf16(x @ w^T),
// xt = residual * norm_weight in bfloat16, partials[cta][128] the sums of squares of the CTA's columns. *count_out is
// the number of CTAs that a consumer has to add up. Returns -2 for what it does not take (n_out no multiple of the
// block of 32 or 64 features, partials too small, more than 128 tokens, unaligned operands).
int stride_gemm_rows_add_norm(const void* x, const void* w, void* xt, float* residual, const float* norm_weight, float* partials,
                              long long partials_capacity, int tokens, int n_out, int k, int* count_out, int* status, cudaStream_t stream) {
    if (tokens < 0 || n_out <= 0 || k <= 0) return STRIDE_BAD_ARGUMENT;
    if (status == nullptr || residual == nullptr || xt == nullptr || norm_weight == nullptr || partials == nullptr || count_out == nullptr)
        return STRIDE_BAD_ARGUMENT;
    *count_out = 0;
    if (tokens == 0) return 0;
    int bn = rows_gemm::choose_block_n(n_out);
    if (bn > 64) bn = 64;
    if (!rows_gemm::operands_ok(x, w, tokens, k) || n_out % bn || n_out % 8 ||
        (reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(xt) | reinterpret_cast<uintptr_t>(norm_weight)) % 16)
        return STRIDE_UNSUPPORTED;
    const int ctas = n_out / bn;
    if (static_cast<long long>(ctas) * rows_gemm::kRows > partials_capacity) return STRIDE_UNSUPPORTED;
    const rows_gemm::Plan p = rows_gemm::plan_for(bn, ctas, tokens, k);
    const CUtensorMap* map_x = tc::cached_map(x, tokens, k, k, p.x_rows);
    const CUtensorMap* map_w = tc::cached_map(w, n_out, k, k, bn);
    if (!map_x || !map_w) return STRIDE_UNSUPPORTED;
    const rows_gemm::QkvEpilogue none = {};
    const rows_gemm::NormFold fold = {nullptr, 0, 0.f, norm_weight, static_cast<__nv_bfloat16*>(xt), partials};
    *count_out = ctas;
    if (bn == 64) return rows_gemm::launch<64, rows_gemm::kAddResidualNorm>(p, map_x, map_w, nullptr, n_out, tokens, n_out, k, residual, none, fold, status, stream);
    return rows_gemm::launch<32, rows_gemm::kAddResidualNorm>(p, map_x, map_w, nullptr, n_out, tokens, n_out, k, residual, none, fold, status, stream);
}

// out = silu(x @ gate^T) * (x @ up^T). w: [2 * inner, k] bf16 with the rows of gate and up alternating in blocks of 64
// (gate 0-63, up 0-63, gate 64-127, ...); out: [tokens, inner] bf16. Returns -2 for what it does not take
// (inner % 64 != 0, more than 128 tokens, unaligned operands).
// With fold_partials (a NormFold consumer: [fold_count][128]) x is x~ and the accumulators get the norm's factor.
int stride_gemm_rows_gated(const void* x, const void* w, void* out, int tokens, int inner, int k, const float* fold_partials,
                           int fold_count, float fold_eps, int* status, cudaStream_t stream) {
    if (tokens < 0 || inner <= 0 || k <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (status == nullptr) return STRIDE_BAD_ARGUMENT;
    if (!rows_gemm::operands_ok(x, w, tokens, k) || inner % 64 || reinterpret_cast<uintptr_t>(out) % 16) return STRIDE_UNSUPPORTED;
    const rows_gemm::Plan p = rows_gemm::plan_for(128, inner / 64, tokens, k);
    const CUtensorMap* map_x = tc::cached_map(x, tokens, k, k, p.x_rows);
    const CUtensorMap* map_w = tc::cached_map(w, 2 * inner, k, k, 128);
    if (!map_x || !map_w) return STRIDE_UNSUPPORTED;
    const rows_gemm::QkvEpilogue none = {};
    const rows_gemm::NormFold fold = {fold_count > 0 ? fold_partials : nullptr, fold_count, fold_eps, nullptr, nullptr, nullptr};
    return rows_gemm::launch<128, rows_gemm::kGated>(p, map_x, map_w, out, inner, tokens, 2 * inner, k, nullptr, none, fold, status, stream);
}

// The projection of queries, keys and values with bias, rotation and the cache write in its epilogue (see
// QkvEpilogue): afterwards qkv [tokens, (nq + 2 nkv) * hd] holds the rotated queries (its key and value columns are
// not written) and the cache the rotated keys and the values. Returns -2 for what it does not take (head sizes
// other than multiples of 64, more than 128 tokens, unaligned operands). fold_partials: as for stride_gemm_rows_gated.
int stride_gemm_rows_qkv_rope(const void* x, const void* w, void* qkv_out, const float* bias, const int32_t* positions,
                              const int32_t* slot_mapping, const float* cos_table, const float* sin_table, void* k_pages, void* v_pages,
                              int tokens, int nq, int nkv, int hd, int page_size, int k, int rotate, const float* fold_partials,
                              int fold_count, float fold_eps, int* status, cudaStream_t stream) {
    if (tokens < 0 || nq <= 0 || nkv <= 0 || hd <= 0 || k <= 0 || page_size <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (status == nullptr || positions == nullptr) return STRIDE_BAD_ARGUMENT;
    if (!rows_gemm::operands_ok(x, w, tokens, k) || hd % 64 ||
        (reinterpret_cast<uintptr_t>(qkv_out) | reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages) |
         reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table)) % 16)
        return STRIDE_UNSUPPORTED;
    const int heads = nq + 2 * nkv, n_out = heads * hd;
    // 32 pairs (64 features) a CTA where that gives 90 CTAs or more, else 16 pairs: a CTA's weight tile comes as two
    // boxes (first and second halves of the pairs), and boxes of 16 rows cost the copying warp as much as boxes of 32
    const int bn = n_out >= 90 * 64 ? 64 : 32;
    const rows_gemm::Plan p = rows_gemm::plan_for(bn, heads * (hd / bn), tokens, k);
    const CUtensorMap* map_x = tc::cached_map(x, tokens, k, k, p.x_rows);
    const CUtensorMap* map_w = tc::cached_map(w, n_out, k, k, bn / 2);
    if (!map_x || !map_w) return STRIDE_UNSUPPORTED;
    const rows_gemm::QkvEpilogue e = {bias, positions, slot_mapping, cos_table, sin_table, static_cast<__nv_bfloat16*>(k_pages),
                                      static_cast<__nv_bfloat16*>(v_pages), nq, nkv, hd, page_size, rotate};
    const rows_gemm::NormFold fold = {fold_count > 0 ? fold_partials : nullptr, fold_count, fold_eps, nullptr, nullptr, nullptr};
    if (bn == 64) return rows_gemm::launch<64, rows_gemm::kQkvRope>(p, map_x, map_w, qkv_out, n_out, tokens, n_out, k, nullptr, e, fold, status, stream);
    return rows_gemm::launch<32, rows_gemm::kQkvRope>(p, map_x, map_w, qkv_out, n_out, tokens, n_out, k, nullptr, e, fold, status, stream);
}

}  // extern "C"
