// Prefill attention in bfloat16 on the fifth-generation tensor cores.
//
// One CTA owns 128 consecutive query rows of one request and one query head; two CTAs share
// an SM. Keys and values are walked in tiles of 64. For each tile
//   S = Q K^T        tcgen05.mma, M = 128 queries, N = 64 keys, accumulator in tensor memory
//   P = softmax part four warps, one thread per query row, read S with tcgen05.ld, keep the
//                    running maximum and sum in float32, write P (bfloat16 pairs) back into
//                    tensor memory over S with tcgen05.st
//   O += P V         tcgen05.mma with A = P from tensor memory, N = head size, V taken MN-major
//                    straight from the cache layout
// There are two score buffers in tensor memory and the scores run two tiles ahead: S of tile
// j+2 is issued right after the output product of tile j, so the softmax warps go from one
// tile to the next without waiting for the tensor cores, and the products hide behind them.
// Q, K and V arrive by TMA: Q as a 128-row box of the projection output, K and V page by page
// through the request's block table (a page's keys of one head are contiguous in the cache, so
// a page is one box per 64 columns). The output accumulator is rescaled only when a row's
// maximum has grown by more than 2^8 since the value in use, which keeps tensor-memory traffic
// low and the exponentials bounded. The mask is that of python/stride_worker/layers.py:109-149
// (key <= query position) plus an optional window.
//
// Roles: warp 0 issues TMA, warp 1 issues the products and owns tensor memory, warps 2-5 do the
// softmax and the final store. Every mbarrier wait is bounded; a wait that runs out sets *status.
#include "tcgen05.cuh"

namespace stride {
namespace tc {

constexpr int kQRows = 128;
constexpr int kKeys = 64;
constexpr int kAttnThreads = 192;
constexpr float kRescaleThreshold = 8.f;      // in log2 units

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                       const int32_t* __restrict__ block_table, int table_width, const int32_t* __restrict__ q_start,
                       const int32_t* __restrict__ q_len, const int32_t* __restrict__ ctx_len, int num_seqs, int nq, int nkv,
                       int page_size, float scale_log2e, int window, int* __restrict__ status) {
    constexpr int HALVES = HD / 64;                       // 64-column boxes per row
    constexpr int HALF_BYTES = kQRows * 128;              // a [128 rows x 64 columns] bf16 box of Q
    constexpr int KV_HALF_BYTES = kKeys * 128;            // a [64 keys x 64 columns] box of K or V
    constexpr int Q_BYTES = HALVES * HALF_BYTES;
    constexpr int KV_BYTES = HALVES * KV_HALF_BYTES;      // one K tile or one V tile
    constexpr uint32_t TMEM_COLS = 256;                   // two score buffers (P over S) of 64 columns, O: HD columns
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = smem;
    unsigned char* k_s = q_s + Q_BYTES;                   // two key tiles, then two value tiles
    unsigned char* v_s = k_s + 2 * KV_BYTES;
    __shared__ __align__(8) uint64_t q_full, pv_done;
    __shared__ __align__(8) uint64_t s_full[2], p_full[2], k_full[2], k_empty[2], v_full[2], v_empty[2];
    __shared__ uint32_t tmem_base_slot;

    pdl_trigger();
    // Which request and which of its query tiles is this CTA? Within a request the last tile, which
    // has the most keys to walk, comes first in the grid, so that the long CTAs do not form the tail.
    int seq = -1, tile = 0;
    {
        int acc = 0;
        for (int s = 0; s < num_seqs; ++s) {
            const int tiles = (q_len[s] + kQRows - 1) / kQRows;
            if (static_cast<int>(blockIdx.x) < acc + tiles) {
                seq = s;
                tile = tiles - 1 - (blockIdx.x - acc);
                break;
            }
            acc += tiles;
        }
    }
    if (seq < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y, kvh = head / (nq / nkv);
    const int n_q = q_len[seq];
    const int row0 = tile * kQRows;
    const int rows = min(kQRows, n_q - row0);
    const int pos0 = ctx_len[seq] - n_q + row0;
    const int last_pos = pos0 + rows - 1;
    const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kt_first = first_key / kKeys;
    const int n_tiles = last_pos / kKeys - kt_first + 1;
    const int q_row0 = q_start[seq] + row0;                // row of the projection output that holds query 0 of this tile
    const int32_t* table = block_table + static_cast<size_t>(seq) * table_width;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), 1);
        mbar_init(smem_u32(&pv_done), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&p_full[s]), 4);
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = tmem_base_slot, tmem_o = tmem_base_slot + 2 * kKeys;     // score buffer b at tmem_s + b * kKeys
    pdl_wait();       // queries, keys and values were written by the kernels before this one

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer. Keys of tile j go to k_s[j & 1] once the scores of tile j-2 are done, values of
            // tile j to v_s[j & 1] once the output product of tile j-2 is done; keys run two tiles ahead.
            const uint32_t qb = smem_u32(&q_full);
            mbar_expect_tx(qb, Q_BYTES);
            for (int h = 0; h < HALVES; ++h) tma_load_2d(smem_u32(q_s + h * HALF_BYTES), &map_q, qb, head * HD + h * 64, q_row0);
            const int pages_per_tile = kKeys / page_size;
            const uint32_t page_bytes = static_cast<uint32_t>(page_size) * 128;       // one page, one 64-column box
            auto load_tile = [&](const CUtensorMap* map, unsigned char* ring, uint64_t* full, uint64_t* empty, int j, int code) {
                const int st = j & 1;
                if (!mbar_wait(smem_u32(&empty[st]), (static_cast<uint32_t>(j >> 1) & 1u) ^ 1u, status, code)) return false;
                const int k0 = (kt_first + j) * kKeys;
                int needed = 0;
                for (int i = 0; i < pages_per_tile; ++i) {
                    const int lo = k0 + i * page_size;
                    needed += (lo <= last_pos && lo + page_size > first_key);
                }
                const uint32_t bar = smem_u32(&full[st]);
                mbar_expect_tx(bar, static_cast<uint32_t>(needed) * HALVES * page_bytes);
                unsigned char* dst = ring + st * KV_BYTES;
                for (int i = 0; i < pages_per_tile; ++i) {
                    const int lo = k0 + i * page_size;
                    if (!(lo <= last_pos && lo + page_size > first_key)) continue;
                    const int y = (table[lo / page_size] * nkv + kvh) * page_size;
                    for (int h = 0; h < HALVES; ++h) tma_load_2d(smem_u32(dst + h * KV_HALF_BYTES) + i * page_bytes, map, bar, h * 64, y);
                }
                return true;
            };
            bool ok = load_tile(&map_k, k_s, k_full, k_empty, 0, 11);
            if (ok && n_tiles > 1) ok = load_tile(&map_k, k_s, k_full, k_empty, 1, 11);
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = load_tile(&map_v, v_s, v_full, v_empty, j, 18);
                if (ok && j + 2 < n_tiles) ok = load_tile(&map_k, k_s, k_full, k_empty, j + 2, 11);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issuer. The scores of tile j+2 are issued right after the output product of
            // tile j, so the softmax of tile j+1 always finds its scores ready and overlaps both.
            constexpr uint32_t idesc_qk = instr_desc_bf16(kQRows, kKeys, false);
            constexpr uint32_t idesc_pv = instr_desc_bf16(kQRows, HD, true);
            auto scores = [&](int j) {
                const int st = j & 1;
                if (!mbar_wait(smem_u32(&k_full[st]), static_cast<uint32_t>(j >> 1) & 1u, status, 13)) return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(k_s + st * KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {      // S = Q K^T, 16 head columns per product
                    umma_bf16(tmem_s + st * kKeys, smem_desc(smem_u32(q_s) + (kk / 4) * HALF_BYTES + (kk % 4) * 32, 16, 1024),
                              smem_desc(k_addr + (kk / 4) * KV_HALF_BYTES + (kk % 4) * 32, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
                }
                umma_commit(smem_u32(&k_empty[st]));         // these keys may be replaced
                umma_commit(smem_u32(&s_full[st]));
                return true;
            };
            bool ok = mbar_wait(smem_u32(&q_full), 0, status, 12);
            if (ok) ok = scores(0);
            if (ok && n_tiles > 1) ok = scores(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
                ok = mbar_wait(smem_u32(&v_full[st]), ph, status, 19) && mbar_wait(smem_u32(&p_full[st]), ph, status, 14);
                if (!ok) break;
                tc_fence_after();
                const uint32_t v_addr = smem_u32(v_s + st * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < kKeys / 16; ++ks) {   // O += P V, 16 keys per product: P from tensor memory
                    // (16 bfloat16 = 8 columns per step), V MN-major: 64-column chunks KV_HALF_BYTES apart
                    umma_bf16_tmem_a(tmem_o, tmem_s + st * kKeys + ks * 8, smem_desc(v_addr + ks * 2048, KV_HALF_BYTES, 1024),
                                     idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(smem_u32(&v_empty[st]));         // these values may be replaced
                umma_commit(smem_u32(&pv_done));             // O holds this tile
                // the products run in order, so these scores overwrite P of tile j only after it has been read
                if (j + 2 < n_tiles) ok = scores(j + 2);
            }
        }
    } else {
        // ---- softmax and output: warps 2..5 own tensor-memory lanes 64-95, 96-127, 0-31, 32-63
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                    // query row of the tile, also the key row this thread may clear
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const int pos_r = pos0 + min(row, rows - 1);
        float m_ref = -INFINITY, l = 0.f;                    // m_ref in log2 units (scaled scores)
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j & 1;
            const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
            const int k0 = (kt_first + j) * kKeys;
            const uint32_t tmem_sj = tmem_s + st * kKeys + lane_base;
            ok = mbar_wait(smem_u32(&s_full[st]), ph, status, 15);
            if (!ok) break;
            tc_fence_after();
            const bool edge = k0 + kKeys - 1 > pos0 || (window > 0 && k0 <= last_pos - window);   // some (row, key) is masked
            float sv[kKeys];                                 // raw scores; a masked one is -inf
            float mx = -INFINITY;
            tmem_ld64(tmem_sj, sv);
            if (edge) {
#pragma unroll
                for (int i = 0; i < kKeys; ++i) {
                    const int key = k0 + i;
                    if (!(key <= pos_r && (window <= 0 || key > pos_r - window))) sv[i] = -INFINITY;
                }
            }
#pragma unroll
            for (int i = 0; i < kKeys; ++i) mx = fmaxf(mx, sv[i]);
            mx *= scale_log2e;                               // the scale is positive: the maximum of the scaled scores
            const bool grow = mx > m_ref + kRescaleThreshold;      // also true for the first finite maximum
            // Every warp waits for every phase of pv_done exactly once (a parity wait cannot skip a phase):
            // before a rescale if there is one, else at the end of the iteration, where it costs nothing.
            bool waited = j == 0;
            if (__any_sync(0xffffffffu, grow)) {
                const float factor = grow ? (m_ref == -INFINITY ? 0.f : ex2_approx(m_ref - mx)) : 1.f;
                if (grow) m_ref = mx;
                l *= factor;
                if (j > 0) {
                    // O belongs to the output product of the tile before until that has finished
                    ok = mbar_wait(smem_u32(&pv_done), static_cast<uint32_t>(j - 1) & 1u, status, 16);
                    if (!ok) break;
                    waited = true;
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < HD / 32; ++c) {
                        float v[32];
                        tmem_ld32(tmem_o + lane_base + c * 32, v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] *= factor;
                        tmem_st32(tmem_o + lane_base + c * 32, v);
                    }
                }
            }
            {
                // A masked score is -inf and gives exactly 0. A row that has seen no key yet has m_ref = -inf and
                // only masked scores: subtract 0 there, or -inf - -inf would make a NaN.
                const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
                float packed[kKeys / 2];       // bfloat16 pairs, carried as 32-bit words
#pragma unroll
                for (int i = 0; i < kKeys; i += 2) {
                    const float p0 = ex2_approx(fmaf(sv[i], scale_log2e, neg_m));
                    const float p1 = ex2_approx(fmaf(sv[i + 1], scale_log2e, neg_m));
                    l += p0 + p1;
                    __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                    packed[i / 2] = __uint_as_float(*reinterpret_cast<uint32_t*>(&b));
                }
                tmem_st32(tmem_sj, packed);
            }
            // Key rows that no query of this tile may see can hold anything (a page never written, the
            // rest of a page): clear their values, or 0 * garbage would poison the product.
            if (k0 + kKeys - 1 > last_pos || k0 < first_key) {
                ok = mbar_wait(smem_u32(&v_full[st]), ph, status, 20);
                if (!ok) break;
                const int key = k0 + row;
                if (row < kKeys && (key > last_pos || key < first_key)) {
                    unsigned char* v_row = v_s + st * KV_BYTES + row * 128;
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
#pragma unroll
                        for (int ch = 0; ch < 8; ++ch)
                            *reinterpret_cast<uint4*>(v_row + h * KV_HALF_BYTES + ch * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[st]));
            if (!waited) ok = mbar_wait(smem_u32(&pv_done), static_cast<uint32_t>(j - 1) & 1u, status, 21);
        }
        if (ok) ok = mbar_wait(smem_u32(&pv_done), static_cast<uint32_t>(n_tiles - 1) & 1u, status, 17);
        tc_fence_after();
        if (ok) {
            // tcgen05.ld is a warp-wide instruction: rows past the portion's end take part and store nothing
            const float inv = 1.f / l;
            __nv_bfloat16* dst = out + (static_cast<size_t>(q_row0 + row) * nq + head) * HD;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                float v[32];
                tmem_ld32(tmem_o + lane_base + c * 32, v);
                if (row < rows) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 b = __floats2bfloat162_rn(v[q4 * 8 + 2 * e] * inv, v[q4 * 8 + 2 * e + 1] * inv);
                            w[e] = *reinterpret_cast<uint32_t*>(&b);
                        }
                        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base_slot, TMEM_COLS);
}

template <int HD>
int launch_attn(const CUtensorMap* map_q, const CUtensorMap* map_k, const CUtensorMap* map_v, __nv_bfloat16* out,
                const int32_t* block_table, int table_width, const int32_t* q_start, const int32_t* q_len, const int32_t* ctx_len,
                int num_seqs, int max_tiles, int nq, int nkv, int page_size, float scale, int window, int* status,
                cudaStream_t stream) {
    constexpr int smem = (HD / 64) * (kQRows * 128 + 4 * kKeys * 128) + 1024;      // Q, two key tiles, two value tiles
    static bool configured = false;
    auto kernel = attn_prefill_tc_kernel<HD>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    stride::launch(kernel, dim3(max_tiles, nq), dim3(kAttnThreads), smem, stream, *map_q, *map_k, *map_v, out, block_table,
                   table_width, q_start, q_len, ctx_len, num_seqs, nq, nkv, page_size, scale * 1.4426950408889634f, window, status);
    return STRIDE_LAUNCH_STATUS();
}

}  // namespace tc
}  // namespace stride

using namespace stride;

// Attention for the first `num_seqs` requests of the step, which own the first `tokens` rows of
// the flat batch. q: [tokens, q_stride] bf16 (head h at columns h*hd); out: [tokens, nq*hd];
// pages: [num_pages, nkv, page_size, hd]. Returns -2 for what it does not take (head sizes other
// than 64 and 128, page sizes that are not 8, 16, 32 or 64, unaligned strides); the caller
// then uses the mma.sync kernel.
extern "C" int stride_paged_prefill_attention_tc(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                                 int num_pages, const int32_t* block_table, int table_width,
                                                 const int32_t* q_start, const int32_t* q_len, const int32_t* ctx_len,
                                                 int num_seqs, int tokens, int nq, int nkv, int hd, int page_size, float scale,
                                                 int window, int* status, cudaStream_t stream) {
    if (tokens < 0 || num_seqs < 0 || nq <= 0 || nkv <= 0 || page_size <= 0 || table_width <= 0 || window < 0 || num_pages <= 0)
        return STRIDE_BAD_ARGUMENT;
    if (nq % nkv || status == nullptr) return STRIDE_BAD_ARGUMENT;
    if ((hd != 64 && hd != 128) || page_size % 8 || tc::kKeys % page_size || q_stride % 8 || nq > 65535) return STRIDE_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(k_pages) |
         reinterpret_cast<uintptr_t>(v_pages)) % 16)
        return STRIDE_UNSUPPORTED;
    if (tokens == 0 || num_seqs == 0) return 0;
    const long long cache_rows = static_cast<long long>(num_pages) * nkv * page_size;
    const CUtensorMap* map_q = tc::cached_map(q, tokens, q_stride, q_stride, tc::kQRows);
    const CUtensorMap* map_k = tc::cached_map(k_pages, cache_rows, hd, hd, page_size);
    const CUtensorMap* map_v = tc::cached_map(v_pages, cache_rows, hd, hd, page_size);
    if (!map_q || !map_k || !map_v) return STRIDE_UNSUPPORTED;
    const int max_tiles = (tokens + tc::kQRows - 1) / tc::kQRows + num_seqs;
    auto op = static_cast<__nv_bfloat16*>(out);
    if (hd == 64)
        return tc::launch_attn<64>(map_q, map_k, map_v, op, block_table, table_width, q_start, q_len, ctx_len, num_seqs, max_tiles,
                                   nq, nkv, page_size, scale, window, status, stream);
    return tc::launch_attn<128>(map_q, map_k, map_v, op, block_table, table_width, q_start, q_len, ctx_len, num_seqs, max_tiles, nq,
                                nkv, page_size, scale, window, status, stream);
}
