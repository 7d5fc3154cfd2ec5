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
// j+2 is issued as soon as the output product of tile j has read P of tile j out of the buffer,
// so the softmax warps go from one tile to the next without waiting for the tensor cores, and
// the products hide behind them. A softmax thread holds the 64 scores of its row in registers
// (the warps that only copy or issue give registers up for that, setmaxnreg) and asks for the
// next tile's scores before it hands the current tile over.
//
// Q arrives by TMA as one 128-row box of the projection output. Keys and values come through the
// request's block table: with pages of 16 keys and more as TMA boxes of one page (or 64 keys) by
// 64 columns, every box issued by a lane of its own in one instruction (one thread issuing them
// one after the other held a tile at 3300 cycles; side by side they cost the issuing warp 1000
// and leave the instruction slots to the softmax); with smaller pages by cp.async, 16 bytes per
// thread, written in the same 128-byte-swizzle layout. The output accumulator is rescaled only
// when a row's maximum has grown by more than 2^8 since the value in use, which keeps
// tensor-memory traffic low and the exponentials bounded. The mask is that of
// python/stride_worker/layers.py:109-149 (key <= query position) plus an optional window.
//
// What the time goes to (cycle stamps on a B200, 2,048 tokens, 32 heads of 128): one tcgen05.mma
// costs its issuing thread some 60 to 70 cycles whatever its size, and a tile of 64 keys needs 12
// per head, so one issuing thread (about 2,300 cycles a tile for two heads) held everything up;
// with a thread per head for the scores and another for the output products the softmax is what
// is left: about 2,000 cycles per tile and warp (load 350, 64 exponentials 900, hand-over 500).
// Evaluating a share of the exponentials as a polynomial on the FMA pipe made it slower (the
// warps are short of instruction slots, not of the special-function unit), starting the second
// head half a tile late made it 12 % faster (see kStaggerCycles).
//
// Roles (two heads, 512 threads): warps 0-1 copy keys (one of them with TMA), warps 2-3 issue the scores of head 1
// and head 0 (warp 3 owns tensor memory), warps 4-5 copy values, warps 6-7 issue the output products of head 1 and
// head 0 (warp 7 fetches Q first), warps 8-15 do the softmax and the final store, four per head.
// CTAs are dispatched longest first (the grid's fast dimension is the head, the slow one the query tile,
// last tile first). Every mbarrier wait is bounded; a wait that runs out sets *status.
#include "tcgen05.cuh"
#include "mma.cuh"

namespace stride {
namespace tc {

constexpr int kQRows = 128;
constexpr int kKeys = 64;
constexpr float kRescaleThreshold = 8.f;      // in log2 units
constexpr int kServiceRegs = 48, kSoftmaxRegs = 208;     // per thread, after the warps have sorted themselves into roles
// With two heads per CTA the softmax warps of the second head start this many cycles after those of the first (half
// of what a tile takes them), so that one head's exponentials, which queue for the special-function unit, fall into
// the other head's loads, maxima and hand-over. Left to themselves both heads run in step and the unit is contended
// for in one half of the time and idle in the other (measured: 56 us against 50 us for 2,048 tokens).
constexpr long long kStaggerCycles = 1000;

// HEADS query heads of one key head per CTA (1 or 2). One head: 4 service warps (keys, products, values, Q) and 4
// softmax warps, two CTAs per SM. Two heads: 8 service warps (three for keys, products, three for values, Q) and
// 8 softmax warps, one CTA per SM: a single warp cannot issue a tile's copies as fast as two heads consume them.
template <int HD, int HEADS, bool TMA_KV>
__global__ void __launch_bounds__(HEADS == 1 ? 256 : 512, HEADS == 1 ? 2 : 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __nv_bfloat16* __restrict__ k_pages,
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
    // Service warps, in this order: LOADERS for the keys, one per head that issues the scores (the last of them, for
    // head 0, owns tensor memory), LOADERS for the values, one per head that issues the output products (the last of
    // them, for head 0, fetches Q first).
    constexpr int LOADERS = HEADS == 1 ? 1 : 2;           // warps per copy stream
    constexpr int MMA_WARP = LOADERS + HEADS - 1, SERVICE_WARPS = 2 * LOADERS + 2 * HEADS, Q_WARP = SERVICE_WARPS - 1;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = smem;                            // HEADS query tiles
    unsigned char* k_s = q_s + HEADS * Q_BYTES;           // KS key tiles, then KS value tiles
    unsigned char* v_s = k_s + KS * KV_BYTES;
    __shared__ __align__(8) uint64_t q_full;
    __shared__ __align__(8) uint64_t s_full[HEADS][2], p_full[HEADS][2], s_free[HEADS][2], k_full[KS], k_empty[KS], v_full[KS], v_empty[KS];
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
            for (int s = 0; s < 2; ++s) {
                mbar_init(smem_u32(&s_full[h][s]), 1);
                mbar_init(smem_u32(&p_full[h][s]), 4);
                mbar_init(smem_u32(&s_free[h][s]), 1);
            }
        }
        for (int s = 0; s < KS; ++s) {
            // cp.async: one arrival per lane of the copying warps; TMA: the one that announces the tile's bytes
            mbar_init(smem_u32(&k_full[s]), TMA_KV ? 1 : 32 * LOADERS);
            mbar_init(smem_u32(&k_empty[s]), HEADS);             // one arrival per issuing warp
            mbar_init(smem_u32(&v_full[s]), TMA_KV ? 1 : 32 * LOADERS);
            mbar_init(smem_u32(&v_empty[s]), HEADS);
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
    // The softmax warps keep a whole tile of scores in registers; the warps that copy and issue need few. Registers
    // move from the one kind to the other (whole warpgroups of four warps each, every warp of a group through the
    // same instruction).

    if (warp < SERVICE_WARPS) {
    reg_release<kServiceRegs>();
    if (warp < LOADERS || (warp > MMA_WARP && warp <= MMA_WARP + LOADERS)) {
        // ---- copying warps: the first LOADERS warps walk the key tiles, the LOADERS after the issuer the value
        // tiles, each taking every LOADERS-th group of rows. A lane owns one 16-byte chunk position of the row
        // (cc) and every (32 / chunks per row)-th key; the block table is read 32 pages at a time, one entry
        // per lane, and handed round by shuffle.
        const bool is_k = warp < LOADERS;
        const int part = is_k ? warp : warp - MMA_WARP - 1;
        const __nv_bfloat16* pages = is_k ? k_pages : v_pages;
        unsigned char* ring = is_k ? k_s : v_s;
        uint64_t* full = is_k ? k_full : v_full;
        uint64_t* empty = is_k ? k_empty : v_empty;
        if constexpr (TMA_KV) {
            // Pages of 16 keys and more: a tile is 64 / page_size boxes of [page_size keys x 64 columns] per half
            // (one box of 64 keys when the page is larger), each issued by a lane of its own in the same
            // instruction, so that the copy engine sees them together; one warp per stream is enough. A page that
            // the table does not hold (entry -1: beyond the request's end, or given back by a window) makes a row
            // coordinate below zero, which the copy fills with zeros; keys past the step's end inside a page are
            // masked (K) or cleared (V) by the softmax warps, as with cp.async.
            if (part == 0) {
                const CUtensorMap* map = is_k ? &map_k : &map_v;
                const int page_size = 1 << page_shift;
                const int box_rows = min(page_size, kKeys);
                const int boxes = kKeys / box_rows;
                for (int j = 0; j < n_tiles; ++j) {
                    const int st = j % KS;
                    if (!mbar_wait(smem_u32(&empty[st]), (static_cast<uint32_t>(j / KS) & 1u) ^ 1u, status, is_k ? 11 : 18)) break;
                    const uint32_t bar = smem_u32(&full[st]);
                    if (lane == 0) mbar_expect_tx(bar, KV_BYTES);
                    __syncwarp();
                    if (lane < boxes) {
                        const int key0 = (kt_first + j) * kKeys + lane * box_rows;
                        const int page = key0 >> page_shift;
                        const int entry = page < table_width ? table[page] : -1;
                        const int y = entry < 0 ? -box_rows : (entry * nkv + kvh) * page_size + (key0 & (page_size - 1));
                        const uint32_t dst = smem_u32(ring + st * KV_BYTES + lane * box_rows * 128);
#pragma unroll
                        for (int h = 0; h < HALVES; ++h) tma_load_2d(dst + h * KV_HALF_BYTES, map, bar, h * 64, y);
                    }
                }
            }
        } else {
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
        }
    } else if (warp > MMA_WARP) {
        // ---- the output products O += P V of one head. One tcgen05.mma costs its issuing thread some 60 cycles
        // whatever its size, and a tile needs 12 of them per head: every head has a warp for its scores and a warp
        // for its output products, so that four threads issue side by side. The whole warp walks the loop and the
        // waits, one lane issues.
        const int h = Q_WARP - warp;
        if (warp == Q_WARP && lane == 0) {       // Q first: one box per head and 64 columns
            const uint32_t qb = smem_u32(&q_full);
            mbar_expect_tx(qb, HEADS * Q_BYTES);
            for (int hh = 0; hh < HEADS; ++hh)
                for (int c = 0; c < HALVES; ++c)
                    tma_load_2d(smem_u32(q_s + hh * Q_BYTES + c * HALF_BYTES), &map_q, qb, (head0 + hh) * HD + c * 64, q_row0);
        }
        __syncwarp();
        const bool issuer = elect_one();
        constexpr uint32_t idesc_pv = instr_desc_bf16(kQRows, HD, true);
        const uint32_t tmem_h = tmem_base + h * HEAD_COLS;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j % KS;
            ok = mbar_wait(smem_u32(&v_full[st]), static_cast<uint32_t>(j / KS) & 1u, status, 19);
            ok = ok && mbar_wait(smem_u32(&p_full[h][j & 1]), static_cast<uint32_t>(j >> 1) & 1u, status, 14);
            if (!ok) break;
            tc_fence_after();
            const uint32_t v_addr = smem_u32(v_s + st * KV_BYTES);
#pragma unroll
            for (int ks = 0; ks < kKeys / 16; ++ks) {   // 16 keys per product: P from tensor memory (16 bfloat16 =
                // 8 columns per step), V MN-major: 64-column chunks KV_HALF_BYTES apart
                const uint64_t b = smem_desc(v_addr + ks * 2048, KV_HALF_BYTES, 1024);
                if (issuer) umma_bf16_tmem_a(tmem_h + 2 * kKeys, tmem_h + (j & 1) * kKeys + ks * 8, b, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
            }
            if (issuer) {
                umma_commit(smem_u32(&s_free[h][j & 1]));     // O holds the tile and P has been read: the score buffer may be written again
                umma_commit(smem_u32(&v_empty[st]));          // this head is done with these values
            }
        }
    } else {
        // ---- the scores S = Q K^T of one head. They run two tiles ahead of the softmax: the scores of tile j+2 go
        // into the buffer that held P of tile j as soon as the output product of tile j has read it.
        const int h = MMA_WARP - warp;
        const bool issuer = elect_one();
        constexpr uint32_t idesc_qk = instr_desc_bf16(kQRows, kKeys, false);
        const uint32_t q_addr = smem_u32(q_s + h * Q_BYTES);
        bool ok = mbar_wait(smem_u32(&q_full), 0, status, 12);
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j % KS;
            if (j >= 2) ok = mbar_wait(smem_u32(&s_free[h][j & 1]), static_cast<uint32_t>((j - 2) >> 1) & 1u, status, 22);
            ok = ok && mbar_wait(smem_u32(&k_full[st]), static_cast<uint32_t>(j / KS) & 1u, status, 13);
            if (!ok) break;
            // (data whose arrival the mbarrier has reported needs no proxy fence before tcgen05.mma reads it)
            tc_fence_after();
            const uint32_t k_addr = smem_u32(k_s + st * KV_BYTES);
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {      // 16 head columns per product
                const uint64_t a = smem_desc(q_addr + (kk / 4) * HALF_BYTES + (kk % 4) * 32, 16, 1024);
                const uint64_t b = smem_desc(k_addr + (kk / 4) * KV_HALF_BYTES + (kk % 4) * 32, 16, 1024);
                if (issuer) umma_bf16(tmem_base + h * HEAD_COLS + (j & 1) * kKeys, a, b, idesc_qk, kk > 0 ? 1u : 0u);
            }
            if (issuer) {
                umma_commit(smem_u32(&s_full[h][j & 1]));
                umma_commit(smem_u32(&k_empty[st]));          // this head is done with these keys
            }
        }
    }
    } else {
        reg_acquire<kSoftmaxRegs>();
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
        // The output product of tile x has finished when phase x / 2 of s_free[x & 1] has: the phase before it
        // (tile x - 2) is known to be over whenever this is asked, because the scores of tile x could only be issued
        // after it, so the parity cannot be mistaken.
        auto output_done = [&](int x, int code) {
            return mbar_wait(smem_u32(&s_free[hh][x & 1]), static_cast<uint32_t>(x >> 1) & 1u, status, code);
        };
        uint32_t sr[64];                                     // the scores of the row, requested one tile ahead
        bool ok = mbar_wait(smem_u32(&s_full[hh][0]), 0, status, 15);
        tc_fence_after();
        if (ok) tmem_ld64_issue(tmem_s + lane_base, sr);
        if (hh == 1) {
            const long long t0 = clock64();
            while (clock64() - t0 < kStaggerCycles) {}
        }
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j & 1;
            const int k0 = (kt_first + j) * kKeys;
            const uint32_t tmem_sj = tmem_s + st * kKeys + lane_base;
            tmem_ld64_wait(sr);
            const bool edge = k0 + kKeys - 1 > pos0 || (window > 0 && k0 <= last_pos - window);   // some (row, key) is masked
            float sv[64];                                    // raw scores; a masked one is -inf
#pragma unroll
            for (int i = 0; i < 64; ++i) sv[i] = __uint_as_float(sr[i]);
            if (edge) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int key = k0 + i;
                    if (!(key <= pos_r && (window <= 0 || key > pos_r - window))) sv[i] = -INFINITY;
                }
            }
            float mx;
            {       // four independent chains of three-input maxima
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < 64; i += 8) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) m4[c] = max3(m4[c], sv[i + 2 * c], sv[i + 2 * c + 1]);
                }
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale_log2e;   // the scale is positive
            }
            const bool grow = mx > m_ref + kRescaleThreshold;      // also true for the first finite maximum
            if (__any_sync(0xffffffffu, grow)) {
                const float factor = grow ? (m_ref == -INFINITY ? 0.f : ex2_approx(m_ref - mx)) : 1.f;
                if (grow) m_ref = mx;
                l *= factor;
                if (j > 0) {
                    // O belongs to the output product of the tile before until that has finished
                    ok = output_done(j - 1, 16);
                    if (!ok) break;
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
#pragma unroll
                for (int i = 0; i < 64; i += 2) {
                    const float p0 = ex2_approx(fmaf(sv[i], scale_log2e, neg_m));
                    const float p1 = ex2_approx(fmaf(sv[i + 1], scale_log2e, neg_m));
                    l4[(i / 2) & 3] += p0 + p1;
                    packed[i / 2] = __uint_as_float(pack_bf16(p0, p1));
                }
                tmem_st32(tmem_sj, packed);   // over S columns 0-31, all of which have been read
                l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            }
            // The scores of the next tile were issued two tiles ago: ask for them now, so that they travel while this
            // tile is handed over.
            if (j + 1 < n_tiles) {
                ok = mbar_wait(smem_u32(&s_full[hh][st ^ 1]), static_cast<uint32_t>((j + 1) >> 1) & 1u, status, 15);
                if (!ok) break;
                tc_fence_after();
                tmem_ld64_issue(tmem_s + (st ^ 1) * kKeys + lane_base, sr);
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[hh][st]));
        }
        if (ok) ok = output_done(n_tiles - 1, 17);
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
int launch_attn(const CUtensorMap* map_q, const CUtensorMap* map_k, const CUtensorMap* map_v, const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages, __nv_bfloat16* out,
                const int32_t* block_table, int table_width, const int32_t* q_start, const int32_t* q_len, const int32_t* ctx_len,
                int num_seqs, int max_tiles, int nq, int nkv, int page_shift, float scale, int window, int* status,
                cudaStream_t stream) {
    constexpr int stages = HEADS == 1 ? 2 : 4;
    constexpr int smem = (HD / 64) * (HEADS * kQRows * 128 + 2 * stages * kKeys * 128) + 1024;      // Q tiles, key ring, value ring
    static bool configured[64] = {};        // the shared-memory limit is set per kernel and device
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return STRIDE_BAD_ARGUMENT;
    if (!configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, HEADS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, HEADS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured[device] = true;
    }
    const dim3 grid(nq / HEADS, max_tiles), block(HEADS == 1 ? 256 : 512);
    if (map_k != nullptr && map_v != nullptr)
        stride::launch(attn_prefill_tc_kernel<HD, HEADS, true>, grid, block, smem, stream, *map_q, *map_k, *map_v, k_pages, v_pages, out,
                       block_table, table_width, q_start, q_len, ctx_len, num_seqs, nq, nkv, page_shift, scale * 1.4426950408889634f,
                       window, status);
    else
        stride::launch(attn_prefill_tc_kernel<HD, HEADS, false>, grid, block, smem, stream, *map_q, *map_q, *map_q, k_pages, v_pages, out,
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

// STRIDE_ATTN_KV_TMA=0 keeps the cp.async copies of keys and values for every page size (for comparisons).
static bool kv_tma() {
    static const bool on = [] {
        const char* e = getenv("STRIDE_ATTN_KV_TMA");
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
    // keys and values by TMA where a page holds at least 16 keys (boxes of min(page, 64) rows); smaller pages by cp.async
    const CUtensorMap* map_k = nullptr;
    const CUtensorMap* map_v = nullptr;
    if (page_size >= 16 && kv_tma()) {
        const long long cache_rows = static_cast<long long>(num_pages) * nkv * page_size;
        const int box_rows = page_size < tc::kKeys ? page_size : tc::kKeys;
        map_k = tc::cached_map(k_pages, cache_rows, hd, hd, box_rows);
        map_v = tc::cached_map(v_pages, cache_rows, hd, hd, box_rows);
        if (!map_k || !map_v) map_k = map_v = nullptr;
    }
#define STRIDE_ATTN_LAUNCH(HD_, HEADS_)                                                                                          \
    tc::launch_attn<HD_, HEADS_>(map_q, map_k, map_v, kp, vp, op, block_table, table_width, q_start, q_len, ctx_len, num_seqs, max_tiles, nq, \
                                 nkv, page_shift, scale, window, status, stream)
    if (hd == 64) return pair ? STRIDE_ATTN_LAUNCH(64, 2) : STRIDE_ATTN_LAUNCH(64, 1);
    return pair ? STRIDE_ATTN_LAUNCH(128, 2) : STRIDE_ATTN_LAUNCH(128, 1);
#undef STRIDE_ATTN_LAUNCH
}
