// Decode attention in bfloat16 over the paged cache, split over the keys.
//
// A decoded token reads every key of its request, so the step is bound by the
// memory bandwidth; with few requests there are too few (request, head) pairs to
// fill 148 SMs. The keys are therefore cut into splits (a multiple of 64 keys,
// chosen from the launch's sizes): one CTA handles
// (split, key head, token), multiplies the whole query group of that key head
// (nq / nkv heads, padded to the 16 rows of an m16n8k16 tile) with its keys on
// the tensor cores, keeps an online softmax in float32, and writes an
// unnormalised partial result. The CTAs of one (token, key head) count themselves
// off on a ticket; the one that arrives last merges the splits of the group's
// query heads and writes the output, so there is no second kernel. Each warp walks
// its own 16-key tiles through a private two-stage cp.async ring (no block-wide
// barrier inside the loop), so every resident CTA always has copies in flight
// while it computes. A CTA whose keys do not include the token's own position
// starts its first copies before it waits for the kernel before it: those keys
// were written by earlier steps, only the query and the newest key are new.
//
// The rule is that of python/stride_worker/layers.py:109-149 for a single query
// at position p: keys j <= p (and j > p - window), softmax(q k^T * scale) v, query
// head h reading key head h / (nq / nkv). Scratch: kTicketInts ticket counters (zero
// before the first launch; every launch leaves them zero), part_o[token][head][split][hd]
// and part_ml[token][head][split][2] (running maximum in the log2 domain, sum).
#include <cstdlib>

#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"      // TMA and mbarrier helpers, tensor-map cache

namespace stride {

constexpr int kTileKeys = 16;     // keys one warp works on at a time
constexpr int kGroupKeys = 64;    // keys the four warps of a CTA cover per pipeline stage
constexpr int kStages = 2;        // three stages (two CTAs per SM) measured 1 % slower at batch 8, 1 % faster at batch 1
constexpr int kTicketInts = 65536;   // ticket counters at the start of the scratch, one per (token, key head)
constexpr int kCodeBeyondBound = 32; // status code: a token's position is not below the launch's max_context

// TMA: the 16-key tiles (16 keys of one head never straddle a page when the page size is a multiple of 16) come as
// boxes of 16 rows x 64 columns, issued by lane 0 of the warp that owns the tile and awaited on an mbarrier of that
// warp; otherwise every lane copies its pieces with cp.async. Many warps issuing small boxes stream faster than
// cp.async does (measured on a B200: 6.7 to 7.0 TB/s from twelve to twenty-four issuing warps per SM, against
// 5.7 TB/s), and the lanes are free of the address arithmetic.
template <int HD, bool TMA>
__global__ void __launch_bounds__(128)
paged_decode_split_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                          const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_pages,
                          const __nv_bfloat16* __restrict__ v_pages, const int32_t* __restrict__ block_table,
                          int table_width, const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ positions,
                          float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ tickets,
                          __nv_bfloat16* __restrict__ out, int nq, int nkv, int page_size, float scale_log2e, int window,
                          int split_keys, int num_splits, int* __restrict__ status) {
    pdl_trigger();
    // The step's index arrays and the keys of earlier steps are not written by the kernels before this one.
    constexpr int ROW_BYTES = HD * 2;
    constexpr int CHUNKS = HD / 8;           // 16-byte chunks per row
    constexpr int KSTEPS = HD / 16;
    constexpr int TILE_BYTES = kTileKeys * ROW_BYTES;
    constexpr int HALVES = HD / 64;          // TMA: 64-column boxes per tile
    constexpr int BOX_BYTES = kTileKeys * 128;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t tile_bar[4][kStages];       // TMA: one barrier per warp and stage

    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int seq = seq_of_token[t];
    const int group = nq / nkv;
    if (seq < 0) {        // a padded row: zeros
        if (split == 0) {
            pdl_wait();
            for (int i = threadIdx.x; i < group * HD; i += blockDim.x)
                out[(static_cast<size_t>(t) * nq + kvh * group) * HD + i] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int pos = positions[t];
    if (pos >= num_splits * split_keys) {
        // The token lies beyond the context bound that this launch was sized for (the caller's max_context): the
        // splits that would hold its newest keys do not exist, and the merge below would wait for tickets that
        // nobody draws. Treated like a padded row: zeros, no ticket (the counters stay zero for the next launch),
        // and a code for the caller where it gave a status word.
        if (split == 0) {
            pdl_wait();
            for (int i = threadIdx.x; i < group * HD; i += blockDim.x)
                out[(static_cast<size_t>(t) * nq + kvh * group) * HD + i] = __float2bfloat16_rn(0.f);
            if (status != nullptr && threadIdx.x == 0) atomicCAS(status, 0, kCodeBeyondBound);
        }
        return;
    }
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int lo = split * split_keys;
    if (lo > pos || lo + split_keys <= first) return;   // uniform for the CTA

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tg = lane & 3;
    const int32_t* table = block_table + static_cast<size_t>(seq) * table_width;
    const int n_tiles = split_keys / kGroupKeys;          // tiles this warp walks: tile j holds keys base(j) .. +15
    auto tile_base = [&](int j) { return lo + j * kGroupKeys + warp * kTileKeys; };
    auto tile_live = [&](int j) { const int b = tile_base(j); return j < n_tiles && b <= pos && b + kTileKeys > first; };
    // Each warp owns a ring of kStages (keys, values) tiles; no other warp touches it.
    auto k_stage = [&](int stage) { return smem + (stage * 4 + warp) * 2 * TILE_BYTES; };

    bool alive = true;       // false once a bounded wait has run out: the warp then copies and computes nothing more
    uint32_t stage_uses = 0; // TMA: bit s is the parity of the number of tiles awaited in stage s so far
    // Byte offset of 16-byte chunk `chunk` of key row `row` inside a tile. cp.async: rows of HD elements, chunks
    // permuted by the row's low bits. TMA: one box of 16 rows x 128 bytes per 64 columns, the 128-byte swizzle.
    auto tile_off = [&](int row, int chunk) -> uint32_t {
        if (TMA) return static_cast<uint32_t>((chunk >> 3) * BOX_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
        return swizzled<ROW_BYTES>(row, chunk);
    };
    if (TMA) {
        if (lane == 0)
            for (int st = 0; st < kStages; ++st) tc::mbar_init(tc::smem_u32(&tile_bar[warp][st]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        __syncwarp();
    }

    // Starts the copies of tile j into its stage. cp.async: always commits one group, so that
    // "all but the newest group have landed" means the same thing in every iteration.
    auto issue = [&](int j) {
        if (TMA) {
            // One thread needs 100 to 300 cycles per TMA instruction; executed by several lanes at once, each with
            // its own box, the instruction costs the warp no more. Lane b < 2 HALVES copies box b: keys or values
            // (b & 1), columns 64 (b >> 1) .. of the head. The barrier's pending arrival (lane 0's, with the byte
            // count) keeps the phase open whichever lane's copy lands first.
            if (tile_live(j) && alive && lane < 2 * HALVES) {
                const int key0 = tile_base(j);                        // a multiple of 16: the tile lies inside one page
                const int y = (table[key0 / page_size] * nkv + kvh) * page_size + key0 % page_size;
                const uint32_t bar = tc::smem_u32(&tile_bar[warp][j % kStages]);
                const uint32_t ks = tc::smem_u32(k_stage(j % kStages));
                if (lane == 0) tc::mbar_expect_tx(bar, 2 * TILE_BYTES);
                const int h = lane >> 1;
                tc::tma_load_2d(ks + (lane & 1) * TILE_BYTES + h * BOX_BYTES, (lane & 1) ? &map_v : &map_k, bar, h * 64, y);
            }
            return;
        }
        if (tile_live(j)) {
            unsigned char* ks = k_stage(j % kStages);
            unsigned char* vs = ks + TILE_BYTES;
            int my_row = -1;   // lane r < 16 looks up where key base + r lives: one division per key, not per chunk
            {
                const int key = tile_base(j) + lane;
                if (lane < kTileKeys && key >= first && key <= pos)
                    my_row = (table[key / page_size] * nkv + kvh) * page_size + key % page_size;
            }
#pragma unroll
            for (int i = 0; i < kTileKeys * CHUNKS / 32; ++i) {
                const int idx = i * 32 + lane;
                const int row = idx / CHUNKS, c = idx % CHUNKS;
                const int src_row = __shfl_sync(0xffffffffu, my_row, row);
                const uint32_t off = swizzled<ROW_BYTES>(row, c);
                if (src_row >= 0) {
                    const size_t src = static_cast<size_t>(src_row) * HD + c * 8;
                    cp_async_16(ks + off, k_pages + src);
                    cp_async_16(vs + off, v_pages + src);
                } else {   // masked keys: zeros, so that 0 * value stays 0
                    *reinterpret_cast<uint4*>(ks + off) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(vs + off) = make_uint4(0, 0, 0, 0);
                }
            }
        }
        cp_async_commit();
    };
    const bool holds_newest = pos < lo + split_keys;      // the key written by the kernel before this one is in this split
    if (!holds_newest) {
#pragma unroll
        for (int st = 0; st < kStages; ++st) issue(st);
    }
    pdl_wait();
    if (holds_newest) {
#pragma unroll
        for (int st = 0; st < kStages; ++st) issue(st);
    }

    // The query group as the A operand: row r is query head kvh * group + r.
    uint32_t qa[KSTEPS][4];
    {
        const __nv_bfloat16* q_tok = q + static_cast<size_t>(t) * q_stride + static_cast<size_t>(kvh) * group * HD;
        const bool r0 = g < group, r1 = g + 8 < group;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            const int d = kk * 16 + 2 * tg;
            qa[kk][0] = r0 ? *reinterpret_cast<const uint32_t*>(q_tok + g * HD + d) : 0u;
            qa[kk][1] = r1 ? *reinterpret_cast<const uint32_t*>(q_tok + (g + 8) * HD + d) : 0u;
            qa[kk][2] = r0 ? *reinterpret_cast<const uint32_t*>(q_tok + g * HD + d + 8) : 0u;
            qa[kk][3] = r1 ? *reinterpret_cast<const uint32_t*>(q_tok + (g + 8) * HD + d + 8) : 0u;
        }
    }

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    const int lm = lane >> 3, lr = lane & 7;     // ldmatrix: matrix index and row within it
    for (int j = 0; j < n_tiles; ++j) {
        if (TMA) {
            // a stage's barrier completes once per tile that was copied into it: tiles outside the window are
            // skipped, so the phase is counted per stage, not taken from j
            if (tile_live(j) && alive) {
                alive = tc::mbar_wait(tc::smem_u32(&tile_bar[warp][j % kStages]), (stage_uses >> (j % kStages)) & 1u, status, 31);
                stage_uses ^= 1u << (j % kStages);
            }
        } else {
            cp_async_wait<kStages - 1>();          // tile j has landed (only the newest group may be pending)
        }
        __syncwarp();
        if (tile_live(j) && alive) {
            const int tlo = tile_base(j);
            const uint32_t ks_addr = smem_addr(k_stage(j % kStages)), vs_addr = ks_addr + TILE_BYTES;
            if (TMA && (tlo + kTileKeys - 1 > pos || tlo < first)) {
                // the box brought whole rows of the page: clear the values of keys this token may not see, or
                // 0 * whatever they hold would poison the product (their scores are masked below)
                unsigned char* vs = k_stage(j % kStages) + TILE_BYTES;
#pragma unroll
                for (int i = 0; i < kTileKeys * CHUNKS / 32; ++i) {
                    const int idx = i * 32 + lane;
                    const int row = idx / CHUNKS, c = idx % CHUNKS;
                    const int key = tlo + row;
                    if (key > pos || key < first) *reinterpret_cast<uint4*>(vs + tile_off(row, c)) = make_uint4(0, 0, 0, 0);
                }
                tc::fence_proxy_async();      // these stores must be ordered before the TMA copy that refills the stage
                __syncwarp();
            }
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                uint32_t b[4];
                ldmatrix_x4(b, ks_addr + tile_off((lm >> 1) * 8 + lr, kk * 2 + (lm & 1)));
                mma_bf16_16816(s[0], qa[kk], b[0], b[1]);
                mma_bf16_16816(s[1], qa[kk], b[2], b[3]);
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = tlo + nt * 8 + 2 * tg + (e & 1);
                    const bool ok = key >= first && key <= pos;
                    s[nt][e] = ok ? s[nt][e] * scale_log2e : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
                }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m[r], mx[r]);     // finite: the tile holds at least one allowed key
                corr[r] = exp2f(m[r] - m_new);
                m[r] = m_new;
                l[r] *= corr[r];
            }
            uint32_t pa[4];
            {
                float p[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        p[nt][e] = exp2f(s[nt][e] - m[e >> 1]);
                        l[e >> 1] += p[nt][e];
                    }
                pa[0] = pack_bf16(p[0][0], p[0][1]);
                pa[1] = pack_bf16(p[0][2], p[0][3]);
                pa[2] = pack_bf16(p[1][0], p[1][1]);
                pa[3] = pack_bf16(p[1][2], p[1][3]);
            }
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                o[i][0] *= corr[0];
                o[i][1] *= corr[0];
                o[i][2] *= corr[1];
                o[i][3] *= corr[1];
            }
#pragma unroll
            for (int dn = 0; dn < HD / 16; ++dn) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vs_addr + tile_off((lm & 1) * 8 + lr, dn * 2 + (lm >> 1)));
                mma_bf16_16816(o[2 * dn], pa, b[0], b[1]);
                mma_bf16_16816(o[2 * dn + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();                              // every lane is done with the stage before it is refilled
        issue(j + kStages);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }

    // Merge the four warps through shared memory (the key and value tiles are no longer needed).
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem);
    constexpr int RS = HD + 2;          // per row: hd accumulators, maximum, sum
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
        if (row < group) {
            float* dst = red + (warp * group + row) * RS;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                dst[i * 8 + 2 * tg] = o[i][2 * r];
                dst[i * 8 + 2 * tg + 1] = o[i][2 * r + 1];
            }
            if (tg == 0) {
                dst[HD] = m[r];
                dst[HD + 1] = l[r];
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * HD; idx += blockDim.x) {
        const int row = idx / HD, d = idx - row * HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[(w * group + row) * RS + HD]);
        float acc = 0.f, sum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = red + (w * group + row) * RS;
            const float f = exp2f(src[HD] - mm);     // a warp without keys has maximum -inf and weight 0
            acc += f * src[d];
            sum += f * src[HD + 1];
        }
        const size_t slot = (static_cast<size_t>(t) * nq + kvh * group + row) * num_splits + split;
        part_o[slot * HD + d] = acc;
        if (d == 0) {
            part_ml[slot * 2] = mm;
            part_ml[slot * 2 + 1] = sum;
        }
    }

    // ---- the CTA that finishes last for this (token, key head) merges the splits
    const int s_lo = first / split_keys, n = pos / split_keys - s_lo + 1;      // live splits
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* ticket = tickets + static_cast<size_t>(t) * nkv + kvh;
        is_last = atomicAdd(ticket, 1) == n - 1;
        if (is_last) *ticket = 0;       // ready for the next launch; nobody else touches it before then
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // out[head, :] = sum_s w_s * part_o[s] / sum_s w_s * part_l[s], w_s = 2^(m_s - max m), summed in the order of the
    // splits whichever CTA happens to do it. A warp per head computes the weights, then a thread per column sums.
    float* wts = red;                       // [group][n]
    float* total = red + group * n;         // [group]
    for (int row = warp; row < group; row += 4) {
        const size_t base = (static_cast<size_t>(t) * nq + kvh * group + row) * num_splits + s_lo;
        float mx = -INFINITY;
        for (int sp = lane; sp < n; sp += 32) {
            const float v = __ldcg(part_ml + (base + sp) * 2);
            wts[row * n + sp] = v;
            mx = fmaxf(mx, v);
        }
        mx = warp_max(mx);
        float lsum = 0.f;
        for (int sp = lane; sp < n; sp += 32) {
            const float w = exp2f(wts[row * n + sp] - mx);
            wts[row * n + sp] = w;
            lsum += w * __ldcg(part_ml + (base + sp) * 2 + 1);
        }
        lsum = warp_sum(lsum);
        if (lane == 0) total[row] = lsum;
    }
    __syncthreads();
    // four columns per thread, eight splits in flight
    for (int idx = threadIdx.x; idx < group * (HD / 4); idx += blockDim.x) {
        const int row = idx / (HD / 4), d = (idx - row * (HD / 4)) * 4;
        const size_t base = (static_cast<size_t>(t) * nq + kvh * group + row) * num_splits + s_lo;
        const float4* col = reinterpret_cast<const float4*>(part_o + base * HD + d);
        const float* w = wts + row * n;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int sp = 0;
        for (; sp + 7 < n; sp += 8) {
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __ldcg(col + static_cast<size_t>(sp + j) * (HD / 4));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc.x = fmaf(w[sp + j], v[j].x, acc.x);
                acc.y = fmaf(w[sp + j], v[j].y, acc.y);
                acc.z = fmaf(w[sp + j], v[j].z, acc.z);
                acc.w = fmaf(w[sp + j], v[j].w, acc.w);
            }
        }
        for (; sp < n; ++sp) {
            const float4 v = __ldcg(col + static_cast<size_t>(sp) * (HD / 4));
            acc.x = fmaf(w[sp], v.x, acc.x);
            acc.y = fmaf(w[sp], v.y, acc.y);
            acc.z = fmaf(w[sp], v.z, acc.z);
            acc.w = fmaf(w[sp], v.w, acc.w);
        }
        const float inv = 1.f / total[row];
        uint2 packed;
        packed.x = pack_bf16(acc.x * inv, acc.y * inv);
        packed.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(out + (static_cast<size_t>(t) * nq + kvh * group + row) * HD + d) = packed;
    }
}

// Keys per CTA: a multiple of 64 between 128 and 1024. Measured on a B200 (8 key heads, context 8192, inside
// the captured decode step): every CTA pays a fixed start-up of dependent loads, so fewer, longer CTAs win as
// long as the SMs stay filled, and a last wave that is nearly full beats one more wave. With enough work the
// grid is therefore sized to about 1.85 waves of the 444 CTAs that fit (batch 8: 640 keys, 832 CTAs, 3 us a
// layer faster than 448 keys); with little work to about 1.4 CTAs per SM (batch 1: 320 keys instead of 128,
// 4 us a layer). The choice depends only on the launch's sizes (not on the contexts of the moment), so a
// captured graph stays valid.
inline int choose_split_keys(int tokens, int nkv, int max_context) {
    static const int forced = [] {      // tuning hook: STRIDE_DECODE_SPLIT_KEYS=<multiple of 64>
        const char* e = getenv("STRIDE_DECODE_SPLIT_KEYS");
        const int v = e ? atoi(e) : 0;
        return v > 0 ? (v + kGroupKeys - 1) / kGroupKeys * kGroupKeys : 0;
    }();
    if (forced) return forced;
    const long long groups = static_cast<long long>(tokens) * nkv * ((max_context + kGroupKeys - 1) / kGroupKeys);
    long long u = (groups + 820) / 821;                 // 1.85 waves of 148 SMs x 3 CTAs
    if (u < 4) u = (groups + 206) / 207;                // too little work for that: 1.4 CTAs per SM
    u = u < 2 ? 2 : (u > 16 ? 16 : u);
    return static_cast<int>(u) * kGroupKeys;
}

// STRIDE_DECODE_TMA=0 keeps the cp.async copies (for comparisons).
inline bool decode_tma_enabled() {
    static const bool on = [] {
        const char* e = getenv("STRIDE_DECODE_TMA");
        return !(e && e[0] == '0');
    }();
    return on;
}

template <int HD>
int launch_decode(const __nv_bfloat16* q, int q_stride, __nv_bfloat16* out, const __nv_bfloat16* k_pages,
                  const __nv_bfloat16* v_pages, long long cache_rows, const int32_t* block_table, int table_width,
                  const int32_t* seq_of_token, const int32_t* positions, float* part_o, float* part_ml, int* tickets, int tokens,
                  int nq, int nkv, int page_size, float scale, int window, int split_keys, int num_splits, int* status,
                  cudaStream_t stream) {
    constexpr int smem = kStages * 4 * 2 * kTileKeys * HD * 2 + 1024;      // the rings, and room to align them to 1024 bytes
    // the merge keeps one weight per (head of the group, split) and one sum per head in the tile ring's memory
    if (static_cast<long long>(nq / nkv) * (num_splits + 1) * 4 > smem - 1024) return STRIDE_UNSUPPORTED;
    // TMA needs whole tiles inside pages, a place to report a wait that ran out, and the extent of the cache
    const CUtensorMap* map_k = nullptr;
    const CUtensorMap* map_v = nullptr;
    if (decode_tma_enabled() && page_size % kTileKeys == 0 && status != nullptr && cache_rows > 0 &&
        (reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) % 16 == 0) {
        map_k = tc::cached_map(k_pages, cache_rows, HD, HD, kTileKeys);
        map_v = tc::cached_map(v_pages, cache_rows, HD, HD, kTileKeys);
    }
    const bool tma = map_k != nullptr && map_v != nullptr;
    // the shared-memory limit is an attribute of the kernel on one device: raised once on every device that launches
    static bool configured[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return STRIDE_BAD_ARGUMENT;
    if (!configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(paged_decode_split_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(paged_decode_split_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured[device] = true;
    }
    static const CUtensorMap no_map = {};
    const dim3 grid(num_splits, nkv, tokens);
    if (tma)
        stride::launch(paged_decode_split_kernel<HD, true>, grid, dim3(128), smem, stream, *map_k, *map_v, q, q_stride, k_pages, v_pages,
                       block_table, table_width, seq_of_token, positions, part_o, part_ml, tickets, out, nq, nkv, page_size,
                       scale * 1.4426950408889634f, window, split_keys, num_splits, status);
    else
        stride::launch(paged_decode_split_kernel<HD, false>, grid, dim3(128), smem, stream, no_map, no_map, q, q_stride, k_pages, v_pages,
                       block_table, table_width, seq_of_token, positions, part_o, part_ml, tickets, out, nq, nkv, page_size,
                       scale * 1.4426950408889634f, window, split_keys, num_splits, status);
    return STRIDE_LAUNCH_STATUS();
}

}  // namespace stride

using namespace stride;

extern "C" {

// Number of float32 scratch elements the launcher needs for these sizes.
long long stride_paged_decode_scratch_floats(int tokens, int nq, int nkv, int hd, int max_context) {
    if (tokens <= 0 || nq <= 0 || nkv <= 0 || max_context <= 0) return 0;
    const int split_keys = choose_split_keys(tokens, nkv, max_context);
    const long long splits = (max_context + split_keys - 1) / split_keys;
    return kTicketInts + static_cast<long long>(tokens) * nq * splits * (hd + 2);
}

// One query token per entry of the flat batch (decode). `scratch` must be zero when it is
// first used (the ticket counters at its start; every launch leaves them zero again) and
// belongs to one stream at a time. `max_context` must exceed every token's position: a row
// whose position does not lie below it gets zeros (and code 32 in the status word, where one
// is given), and the scratch stays usable. Returns -2 for sizes it does not run (head sizes
// other than 64 and 128, groups above 16, more than 65535 tokens, more than 65536 (token,
// key head) pairs); the caller then uses the generic kernel.
int stride_paged_decode_attention_tma(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                      int num_pages, const int32_t* block_table, int table_width, const int32_t* seq_of_token,
                                      const int32_t* positions, float* scratch, long long scratch_floats, int tokens, int nq,
                                      int nkv, int hd, int page_size, float scale, int window, int max_context, int* status,
                                      cudaStream_t stream);

// The same without the two things the TMA copies need (the number of pages and a status word): cp.async copies.
int stride_paged_decode_attention(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                  const int32_t* block_table, int table_width, const int32_t* seq_of_token,
                                  const int32_t* positions, float* scratch, long long scratch_floats, int tokens, int nq,
                                  int nkv, int hd, int page_size, float scale, int window, int max_context,
                                  cudaStream_t stream) {
    return stride_paged_decode_attention_tma(q, q_stride, out, k_pages, v_pages, 0, block_table, table_width, seq_of_token, positions,
                                             scratch, scratch_floats, tokens, nq, nkv, hd, page_size, scale, window, max_context,
                                             nullptr, stream);
}

// With num_pages (the cache tensors are [num_pages, nkv, page_size, hd]) and status (a device word that receives a
// code when a bounded wait runs out) the tiles are copied by TMA where the page size allows it.
int stride_paged_decode_attention_tma(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                      int num_pages, const int32_t* block_table, int table_width, const int32_t* seq_of_token,
                                      const int32_t* positions, float* scratch, long long scratch_floats, int tokens, int nq,
                                      int nkv, int hd, int page_size, float scale, int window, int max_context, int* status,
                                      cudaStream_t stream) {
    if (tokens < 0 || nq <= 0 || nkv <= 0 || page_size <= 0 || table_width <= 0 || window < 0 || max_context <= 0)
        return STRIDE_BAD_ARGUMENT;
    if (nq % nkv) return STRIDE_BAD_ARGUMENT;
    if ((hd != 64 && hd != 128) || nq / nkv > 16 || tokens > 65535 || nkv > 65535 || q_stride % 2) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    const int split_keys = choose_split_keys(tokens, nkv, max_context);
    const int num_splits = (max_context + split_keys - 1) / split_keys;
    if (num_splits > 8192 || static_cast<long long>(tokens) * nkv > kTicketInts) return STRIDE_UNSUPPORTED;
    const long long need = stride_paged_decode_scratch_floats(tokens, nq, nkv, hd, max_context);
    if (scratch == nullptr || scratch_floats < need) return STRIDE_BAD_ARGUMENT;
    static_assert(sizeof(int) == sizeof(float), "the tickets live in the float scratch");
    int* tickets = reinterpret_cast<int*>(scratch);
    float* part_o = scratch + kTicketInts;
    float* part_ml = part_o + static_cast<long long>(tokens) * nq * num_splits * hd;
    auto qp = static_cast<const __nv_bfloat16*>(q);
    auto op = static_cast<__nv_bfloat16*>(out);
    auto kp = static_cast<const __nv_bfloat16*>(k_pages);
    auto vp = static_cast<const __nv_bfloat16*>(v_pages);
    const long long cache_rows = static_cast<long long>(num_pages) * nkv * page_size;
    if (hd == 64)
        return launch_decode<64>(qp, q_stride, op, kp, vp, cache_rows, block_table, table_width, seq_of_token, positions, part_o,
                                 part_ml, tickets, tokens, nq, nkv, page_size, scale, window, split_keys, num_splits, status, stream);
    return launch_decode<128>(qp, q_stride, op, kp, vp, cache_rows, block_table, table_width, seq_of_token, positions, part_o,
                              part_ml, tickets, tokens, nq, nkv, page_size, scale, window, split_keys, num_splits, status, stream);
}

}  // extern "C"
