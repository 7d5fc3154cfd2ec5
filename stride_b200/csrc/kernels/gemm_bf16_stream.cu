// out = x @ w^T in bfloat16 for a handful of tokens (decode steps): the product is bound by
// reading the weights once, so the kernel is built around that stream and nothing else.
//
// A CTA owns a run of weight rows (MT tiles of 16) and all of K; its warps take interleaved
// batches of 32-column steps of K. mma.sync.m16n8k16 does not care which physical column sits
// in which k slot as long as both operands agree, so thread (g, t) of a quad fetches the eight
// consecutive columns 8t..8t+7 of rows g and g+8 of each tile and the same eight columns of
// token g of x, as 16-byte pieces, and feeds them to two products (columns 0-3, then 4-7):
// every thread consumes exactly the pieces it fetched itself. The pieces travel by cp.async
// into a ring in shared memory that is private to the thread (no barrier, only
// cp.async.wait_group), several batches ahead. (That is the path for short K and the fallback;
// for the matrices of a real model the operands come as TMA boxes into rings private to the
// warps and the fragments are read with ldmatrix: see the TMA note at the kernel.) Shared memory rather than registers as the
// landing zone on purpose: plain loads in flight live in the L1 part of the SM's memory, and
// when this kernel shares an SM with kernels that have configured it for shared memory (which
// programmatic dependent launch makes the normal case), almost no L1 is left and a load-based
// stream starves; a ring in shared memory does not care.
// The rows are dealt out so that every SM gets one CTA with the same number of rows (28 of a
// 4096-row matrix on 148 SMs): with whole 16-row tiles some SMs would stream twice as much as
// others, and the kernel is as slow as its busiest SM. Nothing is split across CTAs and nothing
// is reduced through global memory: the warps of a CTA add their partial sums in shared memory
// in warp order. The first batches of weights are requested before the kernel waits for its
// predecessor (the weights do not depend on it).
#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"      // TMA and mbarrier helpers, tensor-map cache

namespace stride {
namespace stream_gemm {

constexpr int kStepCols = 32;    // columns of K per warp step (a quad's four 16-byte pieces)
constexpr int kUnroll = 2;       // steps per batch (one cp.async group)
constexpr int kMaxTiles = 4;     // 16-row tiles per CTA at most

__device__ __forceinline__ void cp_async_16_or_zero(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;        // 0 source bytes: the 16 destination bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(smem)), "l"(gmem), "r"(bytes));
}

// Ring depth in batches: what fits into about STRIDE_STREAM_RING_KB for 256 threads, four at most (deeper measured
// the same), two at least.
#ifndef STRIDE_STREAM_RING_KB
#define STRIDE_STREAM_RING_KB 200
#endif
__host__ __device__ constexpr int ring_stages(int nt, int mt, int warps) {
    const int per_stage = kUnroll * (2 * mt + nt) * warps * 32 * 16;
    const int fit = (STRIDE_STREAM_RING_KB * 1024) / per_stage;
    return fit > 4 ? 4 : (fit < 2 ? 2 : fit);
}

// What the projection of queries, keys and values does with its result instead of storing it (MODE 2): bias,
// rotation of queries and keys by the token's position (pairs (i, i + hd/2), float32 tables
// [position][hd/2]: python/stride_worker/layers.py:85-106), queries back into `out`, keys and values into
// the token's slot of the paged cache (python/stride_worker/cache.py:58-90, pages [page][kv head][slot][hd]).
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

// An RMS norm taken apart and folded into the products around it. The product before the norm (MODE 3) adds its
// result to the residual stream, writes x~ = residual * norm_weight in bfloat16 (without the 1/rms factor) and, per
// CTA and token, the sum of squares of the residual values it produced. The product after the norm reads x~ as its
// activations, adds the partial sums up in CTA order, and multiplies its accumulators by rsqrt(sum / width + eps):
// W (x~ / rms) = (W x~) / rms, with the norm's statistics and scaling in float32 as before and no kernel of its own.
struct RowNorm {
    const float* in_partials;          // consumer: [in_count][16] sums of squares per producer CTA and token, or null
    int in_count;
    float inv_width, eps;
    float* residual;                   // producer (MODE 3): [tokens, n] float32, updated in place
    const float* norm_weight;          // producer: [n]
    float* out_partials;               // producer: [gridDim.x][16]
};

// NT: token tiles of eight, MT: row tiles of 16 per CTA. MODE 0: bfloat16 output, 1: float32 output, 3: RowNorm
// producer (out receives x~); the CTA owns
// rows [blockIdx.x * per_cta, + per_cta). MODE 2: the QKV projection with QkvEpilogue; the CTA owns per_cta rotation
// pairs (pair p of head h is rows h * hd + p and h * hd + p + hd/2), eight per tile, rows 0-7 of the tile holding
// the pairs' first halves and rows 8-15 their second halves, so that both halves of a pair meet in its epilogue.
// TMA: the operands come as boxes instead (64 columns of the CTA's rows, and of the tokens), one stage of a ring
// per box pair, the rings private to the warps as before; the warp's lane 0 issues the copies, all lanes wait on the
// stage's mbarrier and read their fragments with ldmatrix. Many warps issuing small boxes stream faster than
// cp.async does on this GPU (see attention_decode.cu). MODE 2 then keeps a CTA's pairs inside one head (two boxes per
// stage: the pairs' first halves and their second halves), `per_cta` pairs at `ctas_per_head` CTAs a head.
template <int NT, int MT, int WARPS, int MODE, bool TMA>
__global__ void __launch_bounds__(WARPS * 32)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, void* __restrict__ out, int m, int n,
                   int k, int per_cta, int ctas_per_head, const QkvEpilogue qkv, const RowNorm norm, int* __restrict__ status) {
    constexpr int STAGES = ring_stages(NT, MT, WARPS);
    constexpr int THREADS = WARPS * 32;
    constexpr int PIECES = 2 * MT + NT;      // per step: rows g and g + 8 of every tile, then one piece of x per token tile
    constexpr int W_BYTES = MT * 2048, X_BYTES = NT * 1024, STAGE_BYTES = W_BYTES + X_BYTES;      // TMA: a stage of one warp
    extern __shared__ __align__(1024) unsigned char ring_raw[];
    unsigned char* ring_bytes = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ring_raw) + 1023) & ~uintptr_t(1023));
    uint4* ring = reinterpret_cast<uint4*>(ring_bytes);  // cp.async: [STAGES][kUnroll][PIECES][THREADS]
    __shared__ __align__(8) uint64_t stage_bar[TMA ? WARPS : 1][TMA ? STAGES : 1];
    __shared__ float red[WARPS][MT][NT][16][8];
    __shared__ float rstd_s[16];                          // per token: 1/rms of the norm folded into this product (1 without one)
    __shared__ float share_s[WARPS * 2][16];              // its sums of squares, one share per 16 threads
    __shared__ float sq_s[MODE == 3 ? NT * 8 : 1][MODE == 3 ? MT * 16 : 1];
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int half = qkv.hd / 2;
    const int units = MODE == 2 ? n / 2 : n;              // rows, or rotation pairs
    int first = blockIdx.x * per_cta, last = min(first + per_cta, units);       // this CTA's rows or pairs
    if (TMA && MODE == 2) {                               // pairs of one head
        const int head = blockIdx.x / ctas_per_head, in_head = (blockIdx.x - head * ctas_per_head) * per_cta;
        first = head * half + in_head;
        last = head * half + min(in_head + per_cta, half);
    }
    // the weight row behind fragment row g (lo) and g + 8 (hi) of tile mt, or -1
    const __nv_bfloat16* w_lo[MT];
    const __nv_bfloat16* w_hi[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        int lo = -1, hi = -1;
        if (MODE == 2) {
            const int pair = first + mt * 8 + g;
            if (pair < last) {
                lo = (pair / half) * qkv.hd + pair % half;
                hi = lo + half;
            }
        } else {
            lo = first + mt * 16 + g < last ? first + mt * 16 + g : -1;
            hi = first + mt * 16 + 8 + g < last ? first + mt * 16 + 8 + g : -1;
        }
        w_lo[mt] = lo >= 0 ? w + static_cast<size_t>(lo) * k + 8 * t : nullptr;
        w_hi[mt] = hi >= 0 ? w + static_cast<size_t>(hi) * k + 8 * t : nullptr;
    }
    const int steps = (k + kStepCols - 1) / kStepCols;
    // K is dealt out in batches of kUnroll consecutive steps, batch b to warp b % WARPS
    const int batches = (steps + kUnroll - 1) / kUnroll;
    const int my_batches = batches > warp ? (batches - warp + WARPS - 1) / WARPS : 0;
    auto slot = [&](int batch, int u, int piece) { return ring + (((batch % STAGES) * kUnroll + u) * PIECES + piece) * THREADS + threadIdx.x; };
    auto column = [&](int batch, int u) { return ((batch * WARPS + warp) * kUnroll + u) * kStepCols; };
    auto request_weights = [&](int batch) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int col = column(batch, u);
            const bool in = batch < my_batches && col + 8 * t < k;      // k % 8 == 0: a thread's eight columns are all inside or all outside
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                cp_async_16_or_zero(slot(batch, u, 2 * mt), w_lo[mt] ? w_lo[mt] + (in ? col : 0) : w, in && w_lo[mt]);
                cp_async_16_or_zero(slot(batch, u, 2 * mt + 1), w_hi[mt] ? w_hi[mt] + (in ? col : 0) : w, in && w_hi[mt]);
            }
        }
    };
    auto request_x = [&](int batch) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int col = column(batch, u) + 8 * t;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int token = nt * 8 + g;
                const bool in = batch < my_batches && col < k && token < m;
                cp_async_16_or_zero(slot(batch, u, 2 * MT + nt), x + (in ? static_cast<size_t>(token) * k + col : 0), in);
            }
        }
    };

    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;

    // ---- TMA: stage i of this warp holds columns (i * WARPS + warp) * 64 .. + 63
    const int k_stages = (k + 63) / 64;
    const int my_stages = k_stages > warp ? (k_stages - warp + WARPS - 1) / WARPS : 0;
    unsigned char* my_ring = ring_bytes + warp * STAGES * STAGE_BYTES;
    bool alive = true;                                      // false once a bounded wait has run out
    auto request_stage = [&](int i, bool weights, bool tokens) {
        if (lane != 0 || i >= my_stages || !alive) return;
        const int st = i % STAGES, col = (i * WARPS + warp) * 64;
        const uint32_t bar = tc::smem_u32(&stage_bar[warp][st]), dst = tc::smem_u32(my_ring + st * STAGE_BYTES);
        if (weights) {
            // one arrival per stage use: the bytes of every box of the stage are announced with the first copies
            if (MODE == 2) {
                tc::mbar_expect_tx(bar, 2 * per_cta * 128 + NT * 8 * 128);
                const int head = first / half, i0 = first - head * half;
                tc::tma_load_2d(dst, &map_w, bar, col, head * qkv.hd + i0);
                tc::tma_load_2d(dst + MT * 1024, &map_w, bar, col, head * qkv.hd + half + i0);
            } else {
                tc::mbar_expect_tx(bar, per_cta * 128 + NT * 8 * 128);
                tc::tma_load_2d(dst, &map_w, bar, col, first);
            }
        }
        if (tokens) tc::tma_load_2d(dst + W_BYTES, &map_x, bar, col, 0);
    };
    if (TMA) {
        if (lane == 0)
            for (int st = 0; st < STAGES; ++st) tc::mbar_init(tc::smem_u32(&stage_bar[warp][st]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int i = 0; i < STAGES - 1; ++i) request_stage(i, true, false);
        pdl_wait();       // x is written by the kernel before this one
#pragma unroll
        for (int i = 0; i < STAGES - 1; ++i) request_stage(i, false, true);
    } else {
    #pragma unroll
        for (int b = 0; b < STAGES - 1; ++b) request_weights(b);
        pdl_wait();       // x is written by the kernel before this one
#pragma unroll
        for (int b = 0; b < STAGES - 1; ++b) {
            request_x(b);
            cp_async_commit();      // group b: x of batch b (and, in group 0, the weights requested above)
        }
    }
    // The folded norm's sums of squares, while the ring fills: every thread adds up a share of the producer CTAs for
    // one token (loads first, then the sums, so that no load waits for another); the shares meet after the main loop.
    constexpr int SHARES = THREADS / 16;
    {
        float share = 0.f;
        if (norm.in_partials != nullptr) {
            const int token = threadIdx.x & 15, part = threadIdx.x >> 4;
            for (int c0 = part; c0 < norm.in_count; c0 += SHARES * 4) {
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = c0 + j * SHARES < norm.in_count ? norm.in_partials[(c0 + j * SHARES) * 16 + token] : 0.f;
                share += (v[0] + v[1]) + (v[2] + v[3]);
            }
        }
        share_s[threadIdx.x >> 4][threadIdx.x & 15] = share;
    }
    // The producer's epilogue reads the residual and the norm's weight; ask for them now.
    constexpr int ITEMS = (NT * 8 * MT * 16 + THREADS - 1) / THREADS;
    float res_pre[MODE == 3 ? ITEMS : 1], w_pre[MODE == 3 ? ITEMS : 1];
    if (MODE == 3) {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int i = threadIdx.x + it * THREADS;
            const int local = i % (MT * 16), token = i / (MT * 16), row = first + local;
            const bool live = i < NT * 8 * MT * 16 && token < m && row < last;
            res_pre[it] = live ? norm.residual[static_cast<size_t>(token) * n + row] : 0.f;
            w_pre[it] = live ? norm.norm_weight[row] : 0.f;
        }
    }

    if (TMA) {
        const int lm = lane >> 3, lr = lane & 7;            // ldmatrix: matrix index and row within it
        for (int i = 0; i < my_stages; ++i) {
            const int st = i % STAGES;
            if (alive) alive = tc::mbar_wait(tc::smem_u32(&stage_bar[warp][st]), static_cast<uint32_t>(i / STAGES) & 1u, status, 41);
            __syncwarp();
            if (alive) {
                const uint32_t ws = smem_addr(my_ring + st * STAGE_BYTES), xs = ws + W_BYTES;
#pragma unroll
                for (int kp = 0; kp < 2; ++kp) {            // two 16-column steps per ldmatrix of x
                    uint32_t bx[NT][4];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {       // tokens nt*8 + lr, chunks 4 kp + lm: b0, b1 of step 2 kp, then of 2 kp + 1
                        const int row = nt * 8 + lr, chunk = 4 * kp + lm;
                        ldmatrix_x4(bx[nt], xs + row * 128 + ((chunk ^ (row & 7)) << 4));
                    }
#pragma unroll
                    for (int kk = 2 * kp; kk < 2 * kp + 2; ++kk) {
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            // A fragment: rows 0-7 / 8-15 of the tile, columns 16 kk .. + 15
                            int row;
                            uint32_t base = ws;
                            if (MODE == 2) {                // rows 0-7: the pairs' first halves (first box), rows 8-15: their second halves
                                row = mt * 8 + lr;
                                base += (lm & 1) * (MT * 1024);
                            } else {
                                row = mt * 16 + (lm & 1) * 8 + lr;
                            }
                            const int chunk = 2 * kk + (lm >> 1);
                            uint32_t a[4];
                            ldmatrix_x4(a, base + row * 128 + ((chunk ^ (row & 7)) << 4));
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(acc[mt][nt], a, bx[nt][2 * (kk & 1)], bx[nt][2 * (kk & 1) + 1]);
                        }
                    }
                }
            }
            __syncwarp();                                   // every lane is done with the stage before it is refilled
            request_stage(i + STAGES - 1, true, true);
        }
    } else {
        for (int b = 0; b < my_batches; ++b) {
            cp_async_wait<STAGES - 2>();       // batch b has landed; the pieces are this thread's own, so no barrier
            uint4 wl[kUnroll][MT], wh[kUnroll][MT], xv[kUnroll][NT];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    wl[u][mt] = *slot(b, u, 2 * mt);
                    wh[u][mt] = *slot(b, u, 2 * mt + 1);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) xv[u][nt] = *slot(b, u, 2 * MT + nt);
            }
            // the stage read in the iteration before this one is free again
            request_weights(b + STAGES - 1);
            request_x(b + STAGES - 1);
            cp_async_commit();
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint32_t f0[4] = {wl[u][mt].x, wh[u][mt].x, wl[u][mt].y, wh[u][mt].y};
                    const uint32_t f1[4] = {wl[u][mt].z, wh[u][mt].z, wl[u][mt].w, wh[u][mt].w};
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        mma_bf16_16816(acc[mt][nt], f0, xv[u][nt].x, xv[u][nt].y);
                        mma_bf16_16816(acc[mt][nt], f1, xv[u][nt].z, xv[u][nt].w);
                    }
                }
            }
        }
        cp_async_wait<0>();
    }

#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            red[warp][mt][nt][g][2 * t] = acc[mt][nt][0];
            red[warp][mt][nt][g][2 * t + 1] = acc[mt][nt][1];
            red[warp][mt][nt][g + 8][2 * t] = acc[mt][nt][2];
            red[warp][mt][nt][g + 8][2 * t + 1] = acc[mt][nt][3];
        }
    __syncthreads();
    if (threadIdx.x < 16) {
        float scale = 1.f;
        if (norm.in_partials != nullptr) {
            float total = 0.f;
#pragma unroll
            for (int p = 0; p < SHARES; ++p) total += share_s[p][threadIdx.x];
            scale = rsqrtf(total * norm.inv_width + norm.eps);
        }
        rstd_s[threadIdx.x] = scale;
    }
    __syncthreads();
    if (MODE == 2) {
        // one thread per (token, pair): same arithmetic as rope_kv_write_kernel on the product rounded to bfloat16
        for (int i = threadIdx.x; i < NT * 8 * MT * 8; i += THREADS) {
            const int local = i % (MT * 8), token = i / (MT * 8);
            const int pair = first + local;
            if (token >= m || pair >= last) continue;
            const int mt = local >> 3, c = local & 7, nt = token >> 3, tk = token & 7;
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int wp = 0; wp < WARPS; ++wp) {
                a += red[wp][mt][nt][c][tk];
                b += red[wp][mt][nt][c + 8][tk];
            }
            a = __bfloat162float(__float2bfloat16_rn(a * rstd_s[token]));
            b = __bfloat162float(__float2bfloat16_rn(b * rstd_s[token]));
            const int head = pair / half, idx = pair - head * half;        // index of the pair's first half inside the head
            if (qkv.bias) {
                a = __fadd_rn(a, qkv.bias[head * qkv.hd + idx]);
                b = __fadd_rn(b, qkv.bias[head * qkv.hd + idx + half]);
            }
            if (head < qkv.nq + qkv.nkv && qkv.rotate) {
                const size_t at = static_cast<size_t>(qkv.positions[token]) * half + idx;
                const float cs = qkv.cos_table[at], sn = qkv.sin_table[at];
                const float ra = __fadd_rn(__fmul_rn(a, cs), __fmul_rn(-b, sn));
                const float rb = __fadd_rn(__fmul_rn(b, cs), __fmul_rn(a, sn));
                a = ra;
                b = rb;
            }
            __nv_bfloat16* dst = nullptr;
            if (head < qkv.nq) {
                dst = static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(token) * n + head * qkv.hd;
            } else {
                const int slot_of_token = qkv.slot_mapping ? qkv.slot_mapping[token] : -1;
                if (slot_of_token >= 0) {
                    const bool is_key = head < qkv.nq + qkv.nkv;
                    const int kvh = is_key ? head - qkv.nq : head - qkv.nq - qkv.nkv;
                    const int page = slot_of_token / qkv.page_size, offset = slot_of_token - page * qkv.page_size;
                    dst = (is_key ? qkv.k_pages : qkv.v_pages) +
                          ((static_cast<size_t>(page) * qkv.nkv + kvh) * qkv.page_size + offset) * qkv.hd;
                }
            }
            if (dst) {
                dst[idx] = __float2bfloat16_rn(a);
                dst[idx + half] = __float2bfloat16_rn(b);
            }
        }
    } else {
        // one thread per (token, row): the warps' partial sums are added in warp order
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int i = threadIdx.x + it * THREADS;
            const int local = i % (MT * 16), token = i / (MT * 16);
            const int row = first + local;
            if (i >= NT * 8 * MT * 16 || token >= m || row >= last) continue;
            const int mt = local >> 4, r = local & 15, nt = token >> 3, tk = token & 7;
            float sum = 0.f;
#pragma unroll
            for (int wp = 0; wp < WARPS; ++wp) sum += red[wp][mt][nt][r][tk];
            sum *= rstd_s[token];
            const size_t at = static_cast<size_t>(token) * n + row;
            if (MODE == 1) {
                static_cast<float*>(out)[at] = sum;
            } else if (MODE == 3) {
                // as the unfused path: the product rounded to bfloat16, added to the stream in float32
                const float r_new = __fadd_rn(res_pre[MODE == 3 ? it : 0], __bfloat162float(__float2bfloat16_rn(sum)));
                norm.residual[at] = r_new;
                static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(__fmul_rn(r_new, w_pre[MODE == 3 ? it : 0]));
                sq_s[token][local] = r_new * r_new;
            } else {
                static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(sum);
            }
        }
        if (MODE == 3) {
            __syncthreads();
            if (threadIdx.x < 16) {     // this CTA's sum of squares per token, in row order
                float total = 0.f;
                if (static_cast<int>(threadIdx.x) < m)
                    for (int r = 0; r < last - first; ++r) total += sq_s[threadIdx.x][r];
                norm.out_partials[blockIdx.x * 16 + threadIdx.x] = total;
            }
        }
    }
}

template <int NT, int MT, int WARPS, int MODE, bool TMA>
int launch_warps(const CUtensorMap* map_w, const CUtensorMap* map_x, const __nv_bfloat16* x, const __nv_bfloat16* w, void* out, int m,
                 int n, int k, int per_cta, int ctas_per_head, int ctas, const QkvEpilogue& qkv, const RowNorm& norm, int* status,
                 cudaStream_t stream) {
    constexpr int smem = (TMA ? ring_stages(NT, MT, WARPS) * WARPS * (MT * 2048 + NT * 1024)
                              : ring_stages(NT, MT, WARPS) * kUnroll * (2 * MT + NT) * WARPS * 32 * 16) + 1024;
    auto kernel = gemm_stream_kernel<NT, MT, WARPS, MODE, TMA>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    static const CUtensorMap no_map = {};
    stride::launch(kernel, dim3(static_cast<unsigned>(ctas)), dim3(WARPS * 32), smem, stream, TMA ? *map_w : no_map, TMA ? *map_x : no_map,
                   x, w, out, m, n, k, per_cta, ctas_per_head, qkv, norm, status);
    return STRIDE_LAUNCH_STATUS();
}

inline int sm_count() {
    static const int count = [] {
        int device = 0, sms = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 0;
        return sms > 0 ? sms : 148;
    }();
    return count;
}

// STRIDE_STREAM_TMA=0 keeps the cp.async copies (for comparisons).
inline bool stream_tma_enabled() {
    static const bool on = [] {
        const char* e = getenv("STRIDE_STREAM_TMA");
        return !(e && e[0] == '0');
    }();
    return on;
}

// Rows (MODE 2: rotation pairs) per CTA and the number of CTAs: one CTA per SM with equal shares when a CTA's
// kMaxTiles tiles can hold such a share, else full CTAs of kMaxTiles tiles; a short K (small models) gets one tile
// per CTA and fewer warps. With TMA copies a MODE 2 CTA stays inside one head: `ctas_per_head` CTAs of `per_cta`
// pairs each (the last one of a head may hold fewer).
struct Shape {
    int per_cta, ctas, tiles, warps, ctas_per_head;
    bool tma;
};
inline Shape shape_for(int n, int k, int mode, int hd, bool tma_possible) {
    const int batches = ((k + kStepCols - 1) / kStepCols + kUnroll - 1) / kUnroll;
    const int units = mode == 2 ? n / 2 : n, per_tile = mode == 2 ? 8 : 16;
    Shape s{};
    s.ctas_per_head = 1;
    if (batches < 8 * 4) {
        s.per_cta = per_tile;
        s.tiles = 1;
        s.warps = batches >= 4 * 4 ? 4 : 2;
        s.ctas = (units + s.per_cta - 1) / s.per_cta;
        return s;
    }
    s.warps = 8;
    s.per_cta = (units + sm_count() - 1) / sm_count();
    if (s.per_cta > kMaxTiles * per_tile) s.per_cta = kMaxTiles * per_tile;
    s.tma = tma_possible && stream_tma_enabled();
    if (s.tma && mode == 2) {
        const int half = hd / 2;
        int per_head = (half + s.per_cta / 2) / s.per_cta;          // rounded: CTAs a head is cut into
        if (per_head < 1) per_head = 1;
        const int pairs = (half + per_head - 1) / per_head;
        if (pairs > kMaxTiles * per_tile) {
            s.tma = false;
        } else {
            s.ctas_per_head = per_head;
            s.per_cta = pairs;
            s.tiles = (pairs + per_tile - 1) / per_tile;
            s.ctas = (units / half) * per_head;
            return s;
        }
    }
    s.tiles = (s.per_cta + per_tile - 1) / per_tile;
    s.ctas = (units + s.per_cta - 1) / s.per_cta;
    return s;
}

template <int NT, int MODE>
int launch_stream(const __nv_bfloat16* x, const __nv_bfloat16* w, void* out, int m, int n, int k, cudaStream_t stream, int* status,
                  const QkvEpilogue& qkv = QkvEpilogue{}, const RowNorm& norm = RowNorm{}) {
    Shape s = shape_for(n, k, MODE, qkv.hd, status != nullptr);
    const CUtensorMap* map_w = nullptr;
    const CUtensorMap* map_x = nullptr;
    if (s.tma) {
        map_w = tc::cached_map(w, n, k, k, s.per_cta);
        map_x = tc::cached_map(x, m, k, k, NT * 8);
        if (map_w == nullptr || map_x == nullptr) s = shape_for(n, k, MODE, qkv.hd, false);
    }
#define STRIDE_STREAM_LAUNCH(MT_, WARPS_, TMA_)                                                                                 \
    launch_warps<NT, MT_, WARPS_, MODE, TMA_>(map_w, map_x, x, w, out, m, n, k, s.per_cta, s.ctas_per_head, s.ctas, qkv, norm, status, \
                                              stream)
    if (s.warps == 4) return STRIDE_STREAM_LAUNCH(1, 4, false);
    if (s.warps == 2) return STRIDE_STREAM_LAUNCH(1, 2, false);
    if (s.tma) {
        switch (s.tiles) {
            case 1: return STRIDE_STREAM_LAUNCH(1, 8, true);
            case 2: return STRIDE_STREAM_LAUNCH(2, 8, true);
            case 3: return STRIDE_STREAM_LAUNCH(3, 8, true);
            default: return STRIDE_STREAM_LAUNCH(4, 8, true);
        }
    }
    switch (s.tiles) {
        case 1: return STRIDE_STREAM_LAUNCH(1, 8, false);
        case 2: return STRIDE_STREAM_LAUNCH(2, 8, false);
        case 3: return STRIDE_STREAM_LAUNCH(3, 8, false);
        default: return STRIDE_STREAM_LAUNCH(4, 8, false);
    }
#undef STRIDE_STREAM_LAUNCH
}

}  // namespace stream_gemm
}  // namespace stride

using namespace stride;

// out = x @ w^T. x: [tokens, k] bf16, w: [n_out, k] bf16, both 16-byte aligned with k % 8 == 0.
// out: [tokens, n_out], bf16 (out_is_f32 == 0) or float32. Returns -2 for what it does not take
// (more than 16 tokens, unaligned operands); the caller then uses another product.
extern "C" int stride_gemm_stream_bf16(const void* x, const void* w, void* out, int tokens, int n_out, int k, int out_is_f32,
                                       int* status, cudaStream_t stream) {
    if (tokens < 0 || n_out <= 0 || k <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens > 16 || k % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    auto xp = static_cast<const __nv_bfloat16*>(x);
    auto wp = static_cast<const __nv_bfloat16*>(w);
    if (tokens <= 8)
        return out_is_f32 ? stream_gemm::launch_stream<1, 1>(xp, wp, out, tokens, n_out, k, stream, status)
                          : stream_gemm::launch_stream<1, 0>(xp, wp, out, tokens, n_out, k, stream, status);
    return out_is_f32 ? stream_gemm::launch_stream<2, 1>(xp, wp, out, tokens, n_out, k, stream, status)
                      : stream_gemm::launch_stream<2, 0>(xp, wp, out, tokens, n_out, k, stream, status);
}

// The projection of queries, keys and values for at most 16 tokens with rotation and cache write in its
// epilogue: qkv_out [tokens, (nq + 2 nkv) * hd] receives the rotated queries (its key and value columns are
// not written), the rotated keys and the values go to the page slots of slot_mapping. Arguments as
// stride_rope_kv_write. Returns -2 for what it does not take (hd % 16 != 0, more than 16 tokens, unaligned
// operands); the caller then runs the product and stride_rope_kv_write.
extern "C" int stride_gemm_stream_qkv_rope(const void* x, const void* w, void* qkv_out, const float* bias, const int32_t* positions,
                                           const int32_t* slot_mapping, const float* cos_table, const float* sin_table,
                                           void* k_pages, void* v_pages, int tokens, int nq, int nkv, int hd, int page_size,
                                           int k, int rotate, const float* norm_partials, int norm_count, float norm_eps,
                                           int* status, cudaStream_t stream) {
    if (tokens < 0 || nq <= 0 || nkv <= 0 || hd <= 0 || page_size <= 0 || k <= 0 || positions == nullptr) return STRIDE_BAD_ARGUMENT;
    if (tokens > 16 || hd % 16 || k % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    stream_gemm::QkvEpilogue e{bias, positions, slot_mapping, cos_table, sin_table, static_cast<__nv_bfloat16*>(k_pages),
                               static_cast<__nv_bfloat16*>(v_pages), nq, nkv, hd, page_size, rotate};
    auto xp = static_cast<const __nv_bfloat16*>(x);
    auto wp = static_cast<const __nv_bfloat16*>(w);
    const int n_out = (nq + 2 * nkv) * hd;
    stream_gemm::RowNorm norm{};       // x may be the x~ of a folded norm: norm_partials [norm_count][16], width k
    if (norm_partials != nullptr) {
        if (norm_count <= 0) return STRIDE_BAD_ARGUMENT;
        norm.in_partials = norm_partials;
        norm.in_count = norm_count;
        norm.inv_width = 1.f / static_cast<float>(k);
        norm.eps = norm_eps;
    }
    if (tokens <= 8) return stream_gemm::launch_stream<1, 2>(xp, wp, qkv_out, tokens, n_out, k, stream, status, e, norm);
    return stream_gemm::launch_stream<2, 2>(xp, wp, qkv_out, tokens, n_out, k, stream, status, e, norm);
}

// The product before an RMS norm, for at most 16 tokens: residual [tokens, n_out] float32 += bf16(x @ w^T),
// xtilde [tokens, n_out] bf16 = residual * norm_weight, partials [ctas][16] = sums of squares of the new residual
// per CTA and token; *ctas_out receives the number of CTAs (what the consumer has to add up). Returns -2 for
// what it does not take, -1 if `partials_capacity` (floats) is too small.
extern "C" int stride_gemm_stream_add_norm(const void* x, const void* w, void* xtilde, float* residual, const float* norm_weight,
                                           float* partials, long long partials_capacity, int tokens, int n_out, int k,
                                           int* ctas_out, int* status, cudaStream_t stream) {
    if (tokens < 0 || n_out <= 0 || k <= 0 || residual == nullptr || norm_weight == nullptr || partials == nullptr || ctas_out == nullptr)
        return STRIDE_BAD_ARGUMENT;
    if (tokens > 16 || k % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return STRIDE_UNSUPPORTED;
    const stream_gemm::Shape shape = stream_gemm::shape_for(n_out, k, 3, 0, status != nullptr);
    if (partials_capacity < static_cast<long long>(shape.ctas) * 16) return STRIDE_BAD_ARGUMENT;
    *ctas_out = shape.ctas;
    if (tokens == 0) return 0;
    stream_gemm::RowNorm norm{};
    norm.residual = residual;
    norm.norm_weight = norm_weight;
    norm.out_partials = partials;
    auto xp = static_cast<const __nv_bfloat16*>(x);
    auto wp = static_cast<const __nv_bfloat16*>(w);
    if (tokens <= 8) return stream_gemm::launch_stream<1, 3>(xp, wp, xtilde, tokens, n_out, k, stream, status, stream_gemm::QkvEpilogue{}, norm);
    return stream_gemm::launch_stream<2, 3>(xp, wp, xtilde, tokens, n_out, k, stream, status, stream_gemm::QkvEpilogue{}, norm);
}
