// Prefill attention in bfloat16 on the fifth-generation tensor cores.
//
// One CTA owns 128 consecutive query rows of one request and two query heads that share a key head (one
// head, and then two CTAs per SM, when the group is odd): both heads use every key and value tile that is
// loaded. Keys and values are walked in tiles of 64. For each tile and head
//   S = Q K^T        tcgen05.mma, M = 128 queries, N = 64 keys, accumulator in tensor memory
//   P = softmax part four warps, one thread per query row, read S with tcgen05.ld, keep the
//                    running maximum and sum in float32, write P (bfloat16 pairs) back into
//                    tensor memory over S with tcgen05.st
//   O += P V         tcgen05.mma with A = P from tensor memory, N = head size, V taken MN-major
//                    straight from the cache layout
// There are two score buffers in tensor memory and the scores run two tiles ahead: S of tile
// j+2 is issued right after the output product of tile j, so the softmax warps go from one
// tile to the next without waiting for the tensor cores, and the products hide behind them.
//
// Q arrives by TMA as one 128-row box of the projection output. Keys and values come through
// the request's block table with cp.async, 16 bytes per thread, written in the 128-byte-swizzle
// layout the products expect: a page is small (16 keys of one head are 4 KB) and a TMA copy per
// page and 64-column half cost more to issue than the softmax of the tile takes (measured: 16
// copies of 2 KB per tile held the tile at 3300 cycles, the softmax needs 1400), while
// cp.async by a few warps works the same for any page size. The output accumulator is
// rescaled only when a row's maximum has grown by more than 2^8 since the value in use, which
// keeps tensor-memory traffic low and the exponentials bounded. The mask is that of
// python/stride_worker/layers.py:109-149 (key <= query position) plus an optional window.
//
// Roles (two heads, 512 threads): warps 0-2 copy keys, warp 3 issues the products and owns tensor memory,
// warps 4-6 copy values, warp 7 fetches Q, warps 8-15 do the softmax and the final store, four per head.
// CTAs are dispatched longest first (the grid's fast dimension is the head, the slow one the query tile,
// last tile first). Every mbarrier wait is bounded; a wait that runs out sets *status.
#include "tcgen05.cuh"
#include "mma.cuh"

namespace stride {
namespace tc {

constexpr int kQRows = 128;
constexpr int kKeys = 64;
constexpr float kRescaleThreshold = 8.f;      // in log2 units

// HEADS query heads of one key head per CTA (1 or 2). One head: 4 service warps (keys, products, values, Q) and 4
// softmax warps, two CTAs per SM. Two heads: 8 service warps (three for keys, products, three for values, Q) and
// 8 softmax warps, one CTA per SM: a single warp cannot issue a tile's copies as fast as two heads consume them.
template <int HD, int HEADS>
__global__ void __launch_bounds__(HEADS == 1 ? 256 : 512, HEADS == 1 ? 2 : 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __nv_bfloat16* __restrict__ k_pages,
                       const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                       const int32_t* __restrict__ block_table, int table_width, const int32_t* __restrict__ q_start,
                       const int32_t* __restrict__ q_len, const int32_t* __restrict__ ctx_len, int num_seqs, int nq, int nkv,
                       int page_shift, float scale_log2e, int window, int* __restrict__ status) {
    constexpr int HALVES = HD / 64;                       // 64-column boxes per row
    constexpr int HALF_BYTES = kQRows * 128;              // a [128 rows x 64 columns] bf16 box of Q
    constexpr int KV_HALF_BYTES = kKeys * 128;            // [64 keys x 64 columns] of K or V
    constexpr int Q_BYTES = HALVES * HALF_BYTES;
    constexpr int KV_BYTES = HALVES * KV_HALF_BYTES;      // one K tile or one V tile
    constexpr uint32_t HEAD_COLS = 256;                   // per head: two score buffers (P over S) of 64 columns, O: HD columns
    constexpr uint32_t TMEM_COLS = HEAD_COLS * HEADS;
    constexpr int KS = HEADS == 1 ? 2 : 4;                // stages of the key ring and of the value ring
    constexpr int LOADERS = HEADS == 1 ? 1 : 3;           // warps per copy stream
    constexpr int MMA_WARP = LOADERS, Q_WARP = 2 * LOADERS + 1, SERVICE_WARPS = 2 * LOADERS + 2;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = smem;                            // HEADS query tiles
    unsigned char* k_s = q_s + HEADS * Q_BYTES;           // KS key tiles, then KS value tiles
    unsigned char* v_s = k_s + KS * KV_BYTES;
    __shared__ __align__(8) uint64_t q_full, pv_done[HEADS];
    __shared__ __align__(8) uint64_t s_full[HEADS][2], p_full[HEADS][2], k_full[KS], k_empty[KS], v_full[KS], v_empty[KS];
    __shared__ uint32_t tmem_base_slot;

    pdl_trigger();
    // Which request and which of its query tiles is this CTA? blockIdx.y counts the tiles, blockIdx.x the heads:
    // CTAs are handed out x first, so all heads of a tile start together, and within a request the last tile,
    // which has the most keys to walk, comes first: the long CTAs start first and do not form the tail.
    int seq = -1, tile = 0;
    {
        int acc = 0;
        for (int s = 0; s < num_seqs; ++s) {
            const int tiles = (q_len[s] + kQRows - 1) / kQRows;
            if (static_cast<int>(blockIdx.y) < acc + tiles) {
                seq = s;
                tile = tiles - 1 - (blockIdx.y - acc);
                break;
            }
            acc += tiles;
        }
    }
    if (seq < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head0 = blockIdx.x * HEADS, kvh = head0 / (nq / nkv);      // heads head0 .. head0 + HEADS - 1 share the key head
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
        for (int h = 0; h < HEADS; ++h) {
            mbar_init(smem_u32(&pv_done[h]), 1);
            for (int s = 0; s < 2; ++s) {
                mbar_init(smem_u32(&s_full[h][s]), 1);
                mbar_init(smem_u32(&p_full[h][s]), 4);
            }
        }
        for (int s = 0; s < KS; ++s) {
            mbar_init(smem_u32(&k_full[s]), 32 * LOADERS);       // one arrival per lane of the copying warps
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 32 * LOADERS);
            mbar_init(smem_u32(&v_empty[s]), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // head h: score buffer b at tmem_base + h * HEAD_COLS + b * kKeys, output at + 2 * kKeys
    const uint32_t tmem_base = tmem_base_slot;
    pdl_wait();       // queries, keys and values were written by the kernels before this one

    if (warp < SERVICE_WARPS && warp != MMA_WARP && warp != Q_WARP) {
        // ---- copying warps: the first LOADERS warps walk the key tiles, the LOADERS after the issuer the value
        // tiles, each taking every LOADERS-th group of rows. A lane owns one 16-byte chunk position of the row
        // (cc) and every (32 / chunks per row)-th key; the block table is read 32 pages at a time, one entry
        // per lane, and handed round by shuffle.
        const bool is_k = warp < MMA_WARP;
        const int part = is_k ? warp : warp - MMA_WARP - 1;
        const __nv_bfloat16* pages = is_k ? k_pages : v_pages;
        unsigned char* ring = is_k ? k_s : v_s;
        uint64_t* full = is_k ? k_full : v_full;
        uint64_t* empty = is_k ? k_empty : v_empty;
        constexpr int CPR = HD / 8;                         // 16-byte chunks per row
        constexpr int RPI = 32 / CPR;                       // rows per iteration of the warp
        const int cc = lane % CPR, sub = lane / CPR;
        const int page_size = 1 << page_shift;
        const int first_page = (kt_first * kKeys) >> page_shift;
        const uint32_t dst_lane = static_cast<uint32_t>((cc >> 3) * KV_HALF_BYTES);
        int win_at = -1, win_entry = 0;
        for (int j = 0; j < n_tiles; ++j) {
            const int st = j % KS;
            if (!mbar_wait(smem_u32(&empty[st]), (static_cast<uint32_t>(j / KS) & 1u) ^ 1u, status, is_k ? 11 : 18)) break;
            const int k0 = (kt_first + j) * kKeys;
            {   // a tile never straddles a window of 32 pages (tiles and windows are aligned)
                const int at = ((k0 >> page_shift) - first_page) >> 5;
                if (at != win_at) {
                    const int idx = first_page + at * 32 + lane;
                    win_entry = idx < table_width ? table[idx] : 0;
                    win_at = at;
                }
            }
            unsigned char* dst_tile = ring + st * KV_BYTES + dst_lane;
#pragma unroll 4
            for (int it = part; it < kKeys / RPI; it += LOADERS) {
                const int r = it * RPI + sub;
                const int key = k0 + r;
                const bool valid = key >= first_key && key <= last_pos;      // other rows keep what they held: masked (K) or cleared (V) later
                const int page_rel = (min(key, last_pos) >> page_shift) - first_page;
                const int entry = __shfl_sync(0xffffffffu, win_entry, page_rel & 31);
                if (valid) {
                    const size_t src_row = (static_cast<size_t>(entry) * nkv + kvh) * page_size + (key & (page_size - 1));
                    cp_async_16(dst_tile + r * 128 + (((cc & 7) ^ (r & 7)) << 4), pages + src_row * HD + cc * 8);
                }
            }
            cp_async_arrive_noinc(smem_u32(&full[st]));
        }
        cp_async_wait<0>();
    } else if (warp == Q_WARP) {
        if (lane == 0) {       // ---- Q: one box per 64 columns
            const uint32_t qb = smem_u32(&q_full);
            mbar_expect_tx(qb, HEADS * Q_BYTES);
            for (int hh = 0; hh < HEADS; ++hh)
                for (int h = 0; h < HALVES; ++h)
                    tma_load_2d(smem_u32(q_s + hh * Q_BYTES + h * HALF_BYTES), &map_q, qb, (head0 + hh) * HD + h * 64, q_row0);
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            // ---- tensor-core issuer. The scores of tile j+2 are issued right after the output product of
            // tile j, so the softmax of tile j+1 always finds its scores ready and overlaps both.
            constexpr uint32_t idesc_qk = instr_desc_bf16(kQRows, kKeys, false);
            constexpr uint32_t idesc_pv = instr_desc_bf16(kQRows, HD, true);
            auto scores = [&](int j) {      // S = Q K^T of tile j for every head of the CTA
                const int st = j % KS;
                if (!mbar_wait(smem_u32(&k_full[st]), static_cast<uint32_t>(j / KS) & 1u, status, 13)) return false;
                // (cp.async data whose arrival the mbarrier has reported needs no proxy fence before tcgen05.mma reads it)
                tc_fence_after();
                const uint32_t k_addr = smem_u32(k_s + st * KV_BYTES);
#pragma unroll
                for (int h = 0; h < HEADS; ++h) {
                    const uint32_t q_addr = smem_u32(q_s + h * Q_BYTES);
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {      // 16 head columns per product
                        umma_bf16(tmem_base + h * HEAD_COLS + (j & 1) * kKeys,
                                  smem_desc(q_addr + (kk / 4) * HALF_BYTES + (kk % 4) * 32, 16, 1024),
                                  smem_desc(k_addr + (kk / 4) * KV_HALF_BYTES + (kk % 4) * 32, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&s_full[h][j & 1]));
                }
                umma_commit(smem_u32(&k_empty[st]));         // these keys may be replaced
                return true;
            };
            bool ok = mbar_wait(smem_u32(&q_full), 0, status, 12);
            if (ok) ok = scores(0);
            if (ok && n_tiles > 1) ok = scores(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int st = j % KS;
                const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
                ok = mbar_wait(smem_u32(&v_full[st]), static_cast<uint32_t>(j / KS) & 1u, status, 19);
                const uint32_t v_addr = smem_u32(v_s + st * KV_BYTES);
#pragma unroll
                for (int h = 0; h < HEADS; ++h) {
                    ok = ok && mbar_wait(smem_u32(&p_full[h][j & 1]), ph, status, 14);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t tmem_h = tmem_base + h * HEAD_COLS;
#pragma unroll
                    for (int ks = 0; ks < kKeys / 16; ++ks) {   // O += P V, 16 keys per product: P from tensor memory
                        // (16 bfloat16 = 8 columns per step), V MN-major: 64-column chunks KV_HALF_BYTES apart
                        umma_bf16_tmem_a(tmem_h + 2 * kKeys, tmem_h + (j & 1) * kKeys + ks * 8,
                                         smem_desc(v_addr + ks * 2048, KV_HALF_BYTES, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&pv_done[h]));      // this head's O holds the tile
                }
                if (!ok) break;
                umma_commit(smem_u32(&v_empty[st]));         // these values may be replaced
                // the products run in order, so these scores overwrite P of tile j only after it has been read
                if (j + 2 < n_tiles) ok = scores(j + 2);
            }
        }
    } else {
        // ---- softmax and output: four warps per head, which own tensor-memory lanes 0-31, 32-63, 64-95 and
        // 96-127 of their head's columns
        const int hh = (warp - SERVICE_WARPS) >> 2;          // which head of the CTA
        const int head = head0 + hh;
        const uint32_t tmem_s = tmem_base + hh * HEAD_COLS, tmem_o = tmem_s + 2 * kKeys;
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
            ok = mbar_wait(smem_u32(&s_full[hh][st]), ph, status, 15);
            if (!ok) break;
            tc_fence_after();
            const bool edge = k0 + kKeys - 1 > pos0 || (window > 0 && k0 <= last_pos - window);   // some (row, key) is masked
            // The 64 scores are taken in two halves of 32 to stay within the registers that two CTAs per SM leave:
            // first the maximum over both (the second half stays in registers), then P for the second half, then
            // the first half again from tensor memory.
            float sv[32];                                    // raw scores of one half; a masked one is -inf
            auto load_half = [&](int half) {
                tmem_ld32(tmem_sj + half * 32, sv);
                if (edge) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = k0 + half * 32 + i;
                        if (!(key <= pos_r && (window <= 0 || key > pos_r - window))) sv[i] = -INFINITY;
                    }
                }
            };
            auto half_max = [&]() {       // four independent chains of three-input maxima
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) m4[c] = max3(m4[c], sv[i + 2 * c], sv[i + 2 * c + 1]);
                }
                return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            };
            load_half(0);
            float mx = half_max();
            load_half(1);
            mx = fmaxf(mx, half_max()) * scale_log2e;        // the scale is positive: the maximum of the scaled scores
            const bool grow = mx > m_ref + kRescaleThreshold;      // also true for the first finite maximum
            // Every warp waits for every phase of pv_done exactly once (a parity wait cannot skip a phase):
            // before a rescale if there is one, else at the end of the iteration, by when it has long completed.
            bool waited = j == 0;
            if (__any_sync(0xffffffffu, grow)) {
                const float factor = grow ? (m_ref == -INFINITY ? 0.f : ex2_approx(m_ref - mx)) : 1.f;
                if (grow) m_ref = mx;
                l *= factor;
                if (j > 0) {
                    // O belongs to the output product of the tile before until that has finished
                    ok = mbar_wait(smem_u32(&pv_done[hh]), static_cast<uint32_t>(j - 1) & 1u, status, 16);
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
                float l4[4] = {0.f, 0.f, 0.f, 0.f};       // independent partial sums
                float packed[32];             // bfloat16 pairs, carried as 32-bit words: P's columns hold two keys each
                auto pack_half = [&](int half) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = ex2_approx(fmaf(sv[i], scale_log2e, neg_m));
                        const float p1 = ex2_approx(fmaf(sv[i + 1], scale_log2e, neg_m));
                        l4[(i / 2) & 3] += p0 + p1;
                        packed[half * 16 + i / 2] = __uint_as_float(pack_bf16(p0, p1));
                    }
                };
                pack_half(1);                 // the second half is still in registers
                load_half(0);
                pack_half(0);
                tmem_st32(tmem_sj, packed);   // over S columns 0-31, all of which have been read
                l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            }
            // Key rows that no query of this tile may see can hold anything (a page never written, the
            // rest of a page): clear their values, or 0 * garbage would poison the product.
            if (k0 + kKeys - 1 > last_pos || k0 < first_key) {
                // (with two heads both groups of warps clear the same rows with the same zeros: each must be
                // sure of them before it lets its own product go)
                const int vst = j % KS;
                ok = mbar_wait(smem_u32(&v_full[vst]), static_cast<uint32_t>(j / KS) & 1u, status, 20);
                if (!ok) break;
                const int key = k0 + row;
                if (row < kKeys && (key > last_pos || key < first_key)) {
                    unsigned char* v_row = v_s + vst * KV_BYTES + row * 128;
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
#pragma unroll
                        for (int ch = 0; ch < 8; ++ch)
                            *reinterpret_cast<uint4*>(v_row + h * KV_HALF_BYTES + ch * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            // Before this warp lets the output product of tile j go: once that one can finish, pv_done may be
            // two phases on and its parity says nothing any more.
            if (!waited) ok = mbar_wait(smem_u32(&pv_done[hh]), static_cast<uint32_t>(j - 1) & 1u, status, 21);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[hh][st]));
        }
        if (ok) ok = mbar_wait(smem_u32(&pv_done[hh]), static_cast<uint32_t>(n_tiles - 1) & 1u, status, 17);
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
                        for (int e = 0; e < 4; ++e) w[e] = pack_bf16(v[q4 * 8 + 2 * e] * inv, v[q4 * 8 + 2 * e + 1] * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base_slot, TMEM_COLS);
}

template <int HD, int HEADS>
int launch_attn(const CUtensorMap* map_q, const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages, __nv_bfloat16* out,
                const int32_t* block_table, int table_width, const int32_t* q_start, const int32_t* q_len, const int32_t* ctx_len,
                int num_seqs, int max_tiles, int nq, int nkv, int page_shift, float scale, int window, int* status,
                cudaStream_t stream) {
    constexpr int stages = HEADS == 1 ? 2 : 4;
    constexpr int smem = (HD / 64) * (HEADS * kQRows * 128 + 2 * stages * kKeys * 128) + 1024;      // Q tiles, key ring, value ring
    static bool configured = false;
    auto kernel = attn_prefill_tc_kernel<HD, HEADS>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    stride::launch(kernel, dim3(nq / HEADS, max_tiles), dim3(HEADS == 1 ? 256 : 512), smem, stream, *map_q, k_pages, v_pages, out,
                   block_table, table_width, q_start, q_len, ctx_len, num_seqs, nq, nkv, page_shift, scale * 1.4426950408889634f,
                   window, status);
    return STRIDE_LAUNCH_STATUS();
}

}  // namespace tc
}  // namespace stride

using namespace stride;

// STRIDE_ATTN_PAIR_HEADS=0 keeps one head per CTA (for comparisons).
static bool pair_heads() {
    static const bool on = [] {
        const char* e = getenv("STRIDE_ATTN_PAIR_HEADS");
        return !(e && e[0] == '0');
    }();
    return on;
}

// Attention for the first `num_seqs` requests of the step, which own the first `tokens` rows of
// the flat batch. q: [tokens, q_stride] bf16 (head h at columns h*hd); out: [tokens, nq*hd];
// pages: [num_pages, nkv, page_size, hd]. Returns -2 for what it does not take (head sizes other
// than 64 and 128, page sizes that are no power of two from 4 to 64, unaligned strides); the caller
// then uses the mma.sync kernel.
extern "C" int stride_paged_prefill_attention_tc(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                                 int num_pages, const int32_t* block_table, int table_width,
                                                 const int32_t* q_start, const int32_t* q_len, const int32_t* ctx_len,
                                                 int num_seqs, int tokens, int nq, int nkv, int hd, int page_size, float scale,
                                                 int window, int* status, cudaStream_t stream) {
    if (tokens < 0 || num_seqs < 0 || nq <= 0 || nkv <= 0 || page_size <= 0 || table_width <= 0 || window < 0 || num_pages <= 0)
        return STRIDE_BAD_ARGUMENT;
    if (nq % nkv || status == nullptr) return STRIDE_BAD_ARGUMENT;
    if ((hd != 64 && hd != 128) || page_size > tc::kKeys || page_size < 4 || q_stride % 8 || nq > 65535) return STRIDE_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(k_pages) |
         reinterpret_cast<uintptr_t>(v_pages)) % 16)
        return STRIDE_UNSUPPORTED;
    if (tokens == 0 || num_seqs == 0) return 0;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    if ((1 << page_shift) != page_size) return STRIDE_UNSUPPORTED;
    const CUtensorMap* map_q = tc::cached_map(q, tokens, q_stride, q_stride, tc::kQRows);
    if (!map_q) return STRIDE_UNSUPPORTED;
    const int max_tiles = (tokens + tc::kQRows - 1) / tc::kQRows + num_seqs;
    if (max_tiles > 65535) return STRIDE_UNSUPPORTED;
    auto op = static_cast<__nv_bfloat16*>(out);
    auto kp = static_cast<const __nv_bfloat16*>(k_pages);
    auto vp = static_cast<const __nv_bfloat16*>(v_pages);
    // Two heads of a key head per CTA share every key and value tile they load; with an odd group one head per CTA.
    const bool pair = (nq / nkv) % 2 == 0 && pair_heads();
#define STRIDE_ATTN_LAUNCH(HD_, HEADS_)                                                                                          \
    tc::launch_attn<HD_, HEADS_>(map_q, kp, vp, op, block_table, table_width, q_start, q_len, ctx_len, num_seqs, max_tiles, nq, \
                                 nkv, page_shift, scale, window, status, stream)
    if (hd == 64) return pair ? STRIDE_ATTN_LAUNCH(64, 2) : STRIDE_ATTN_LAUNCH(64, 1);
    return pair ? STRIDE_ATTN_LAUNCH(128, 2) : STRIDE_ATTN_LAUNCH(128, 1);
#undef STRIDE_ATTN_LAUNCH
}
