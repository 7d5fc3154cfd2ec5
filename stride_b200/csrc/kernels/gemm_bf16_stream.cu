// out = x @ w^T in bfloat16 for a handful of tokens (decode steps): the product is bound by
// reading the weights once, so the kernel is built around that stream and nothing else.
//
// A CTA owns 16 weight rows and all of K; its warps take interleaved batches of 32-column steps
// of K. mma.sync.m16n8k16 does not care which physical column sits in which k slot as long as
// both operands agree, so thread (g, t) of a quad fetches the eight consecutive columns
// 8t..8t+7 of rows g and g+8 and the same eight columns of token g of x, as 16-byte pieces, and
// feeds them to two products (columns 0-3, then 4-7): every thread consumes exactly the pieces
// it fetched itself. The pieces travel by cp.async into a ring in shared memory that is private
// to the thread (no barrier, only cp.async.wait_group), several batches ahead. Shared memory
// rather than registers as the landing zone on purpose: plain loads in flight live in the L1
// part of the SM's memory, and when this kernel shares an SM with kernels that have configured
// it for shared memory (which programmatic dependent launch makes the normal case), almost no
// L1 is left and a load-based stream starves; a ring in shared memory does not care.
// With 16 rows per CTA even a 4096 x 4096 matrix gives 256 CTAs, all resident at once, so
// nothing is split across CTAs and nothing is reduced through global memory: the warps of a CTA
// add their partial sums in shared memory in warp order. The first batches of weights are
// requested before the kernel waits for its predecessor (the weights do not depend on it).
#include "common.cuh"
#include "mma.cuh"

namespace stride {
namespace stream_gemm {

constexpr int kRows = 16;        // weight rows per CTA
constexpr int kStepCols = 32;    // columns of K per warp step (a quad's four 16-byte pieces)
constexpr int kUnroll = 2;       // steps per batch (one cp.async group)

__device__ __forceinline__ void cp_async_16_or_zero(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;        // 0 source bytes: the 16 destination bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(smem)), "l"(gmem), "r"(bytes));
}

template <int NT>
struct Ring {
    static constexpr int kStages = NT == 1 ? 4 : 3;      // 96 KB of ring per 256-thread CTA either way (deeper or shallower rings measured the same)
};

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

// NT: token tiles of eight. MODE 0: bfloat16 output, 1: float32 output, 2: the QKV projection with QkvEpilogue:
// a CTA then owns eight rotation pairs of one head, rows p..p+7 and p + hd/2..p + hd/2 + 7, so that both
// halves of a pair meet in its epilogue.
template <int NT, int WARPS, int MODE>
__global__ void __launch_bounds__(WARPS * 32)
gemm_stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, void* __restrict__ out, int m, int n,
                   int k, const QkvEpilogue qkv) {
    constexpr int STAGES = Ring<NT>::kStages;
    constexpr int THREADS = WARPS * 32;
    constexpr int PIECES = 2 + NT;           // per step: rows g and g + 8 of the weights, then one piece of x per token tile
    extern __shared__ __align__(16) uint4 ring[];        // [STAGES][kUnroll][PIECES][THREADS]
    __shared__ float red[WARPS][NT][kRows][8];
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * kRows;
    int row_lo = r0, row_hi = r0 + 8;                      // first weight row of fragment rows 0-7 and of rows 8-15
    if (MODE == 2) {
        const int per_head = qkv.hd / kRows;               // CTAs per head
        const int head = blockIdx.x / per_head;
        row_lo = head * qkv.hd + (blockIdx.x - head * per_head) * 8;
        row_hi = row_lo + qkv.hd / 2;
    }
    const __nv_bfloat16* w_lo = w + static_cast<size_t>(min(row_lo + g, n - 1)) * k + 8 * t;
    const __nv_bfloat16* w_hi = w + static_cast<size_t>(min(row_hi + g, n - 1)) * k + 8 * t;
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
            cp_async_16_or_zero(slot(batch, u, 0), w_lo + (in ? col : 0), in);
            cp_async_16_or_zero(slot(batch, u, 1), w_hi + (in ? col : 0), in);
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
                cp_async_16_or_zero(slot(batch, u, 2 + nt), x + (in ? static_cast<size_t>(token) * k + col : 0), in);
            }
        }
    };

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;

#pragma unroll
    for (int b = 0; b < STAGES - 1; ++b) request_weights(b);
    pdl_wait();       // x is written by the kernel before this one
#pragma unroll
    for (int b = 0; b < STAGES - 1; ++b) {
        request_x(b);
        cp_async_commit();      // group b: x of batch b (and, in group 0, the weights requested above)
    }

    for (int b = 0; b < my_batches; ++b) {
        cp_async_wait<STAGES - 2>();       // batch b has landed; the pieces are this thread's own, so no barrier
        uint4 wl[kUnroll], wh[kUnroll], xv[kUnroll][NT];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            wl[u] = *slot(b, u, 0);
            wh[u] = *slot(b, u, 1);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) xv[u][nt] = *slot(b, u, 2 + nt);
        }
        // the stage read in the iteration before this one is free again
        request_weights(b + STAGES - 1);
        request_x(b + STAGES - 1);
        cp_async_commit();
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t f0[4] = {wl[u].x, wh[u].x, wl[u].y, wh[u].y};
            const uint32_t f1[4] = {wl[u].z, wh[u].z, wl[u].w, wh[u].w};
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                mma_bf16_16816(acc[nt], f0, xv[u][nt].x, xv[u][nt].y);
                mma_bf16_16816(acc[nt], f1, xv[u][nt].z, xv[u][nt].w);
            }
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][nt][g][2 * t] = acc[nt][0];
        red[warp][nt][g][2 * t + 1] = acc[nt][1];
        red[warp][nt][g + 8][2 * t] = acc[nt][2];
        red[warp][nt][g + 8][2 * t + 1] = acc[nt][3];
    }
    __syncthreads();
    if (MODE == 2) {
        // one thread per (token, pair): same arithmetic as rope_kv_write_kernel on the product rounded to bfloat16
        const int head = row_lo / qkv.hd, i0 = row_lo - head * qkv.hd, half = qkv.hd / 2;
        for (int i = threadIdx.x; i < NT * 8 * 8; i += THREADS) {
            const int c = i & 7, token = i >> 3;
            if (token >= m) continue;
            const int nt = token >> 3, tk = token & 7;
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int wp = 0; wp < WARPS; ++wp) {
                a += red[wp][nt][c][tk];
                b += red[wp][nt][c + 8][tk];
            }
            a = __bfloat162float(__float2bfloat16_rn(a));
            b = __bfloat162float(__float2bfloat16_rn(b));
            const int idx = i0 + c;                        // index of the pair's first half inside the head
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
                const int slot = qkv.slot_mapping ? qkv.slot_mapping[token] : -1;
                if (slot >= 0) {
                    const bool is_key = head < qkv.nq + qkv.nkv;
                    const int kvh = is_key ? head - qkv.nq : head - qkv.nq - qkv.nkv;
                    const int page = slot / qkv.page_size, offset = slot - page * qkv.page_size;
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
        for (int i = threadIdx.x; i < NT * 8 * kRows; i += THREADS) {
            const int row = i & (kRows - 1), token = i / kRows;
            const int nt = token >> 3, tk = token & 7;
            float sum = 0.f;
#pragma unroll
            for (int wp = 0; wp < WARPS; ++wp) sum += red[wp][nt][row][tk];
            if (token < m && r0 + row < n) {
                const size_t at = static_cast<size_t>(token) * n + r0 + row;
                if (MODE == 1) static_cast<float*>(out)[at] = sum;
                else static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(sum);
            }
        }
    }
}

template <int NT, int WARPS, int MODE>
int launch_warps(const __nv_bfloat16* x, const __nv_bfloat16* w, void* out, int m, int n, int k, const QkvEpilogue& qkv, cudaStream_t stream) {
    constexpr int smem = Ring<NT>::kStages * kUnroll * (2 + NT) * WARPS * 32 * 16;
    auto kernel = gemm_stream_kernel<NT, WARPS, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    stride::launch(kernel, dim3(static_cast<unsigned>((n + kRows - 1) / kRows)), dim3(WARPS * 32), smem, stream, x, w, out, m, n, k, qkv);
    return STRIDE_LAUNCH_STATUS();
}

template <int NT, int MODE>
int launch_stream(const __nv_bfloat16* x, const __nv_bfloat16* w, void* out, int m, int n, int k, cudaStream_t stream,
                  const QkvEpilogue& qkv = QkvEpilogue{}) {
    const int batches = ((k + kStepCols - 1) / kStepCols + kUnroll - 1) / kUnroll;
    if (batches >= 8 * 4) return launch_warps<NT, 8, MODE>(x, w, out, m, n, k, qkv, stream);
    if (batches >= 4 * 4) return launch_warps<NT, 4, MODE>(x, w, out, m, n, k, qkv, stream);
    return launch_warps<NT, 2, MODE>(x, w, out, m, n, k, qkv, stream);
}

}  // namespace stream_gemm
}  // namespace stride

using namespace stride;

// out = x @ w^T. x: [tokens, k] bf16, w: [n_out, k] bf16, both 16-byte aligned with k % 8 == 0.
// out: [tokens, n_out], bf16 (out_is_f32 == 0) or float32. Returns -2 for what it does not take
// (more than 16 tokens, unaligned operands); the caller then uses another product.
extern "C" int stride_gemm_stream_bf16(const void* x, const void* w, void* out, int tokens, int n_out, int k, int out_is_f32,
                                       cudaStream_t stream) {
    if (tokens < 0 || n_out <= 0 || k <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens > 16 || k % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    auto xp = static_cast<const __nv_bfloat16*>(x);
    auto wp = static_cast<const __nv_bfloat16*>(w);
    if (tokens <= 8)
        return out_is_f32 ? stream_gemm::launch_stream<1, 1>(xp, wp, out, tokens, n_out, k, stream)
                          : stream_gemm::launch_stream<1, 0>(xp, wp, out, tokens, n_out, k, stream);
    return out_is_f32 ? stream_gemm::launch_stream<2, 1>(xp, wp, out, tokens, n_out, k, stream)
                      : stream_gemm::launch_stream<2, 0>(xp, wp, out, tokens, n_out, k, stream);
}

// The projection of queries, keys and values for at most 16 tokens with rotation and cache write in its
// epilogue: qkv_out [tokens, (nq + 2 nkv) * hd] receives the rotated queries (its key and value columns are
// not written), the rotated keys and the values go to the page slots of slot_mapping. Arguments as
// stride_rope_kv_write. Returns -2 for what it does not take (hd % 16 != 0, more than 16 tokens, unaligned
// operands); the caller then runs the product and stride_rope_kv_write.
extern "C" int stride_gemm_stream_qkv_rope(const void* x, const void* w, void* qkv_out, const float* bias, const int32_t* positions,
                                           const int32_t* slot_mapping, const float* cos_table, const float* sin_table,
                                           void* k_pages, void* v_pages, int tokens, int nq, int nkv, int hd, int page_size,
                                           int k, int rotate, cudaStream_t stream) {
    if (tokens < 0 || nq <= 0 || nkv <= 0 || hd <= 0 || page_size <= 0 || k <= 0 || positions == nullptr) return STRIDE_BAD_ARGUMENT;
    if (tokens > 16 || hd % 16 || k % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    stream_gemm::QkvEpilogue e{bias, positions, slot_mapping, cos_table, sin_table, static_cast<__nv_bfloat16*>(k_pages),
                               static_cast<__nv_bfloat16*>(v_pages), nq, nkv, hd, page_size, rotate};
    auto xp = static_cast<const __nv_bfloat16*>(x);
    auto wp = static_cast<const __nv_bfloat16*>(w);
    const int n_out = (nq + 2 * nkv) * hd;
    if (tokens <= 8) return stream_gemm::launch_stream<1, 2>(xp, wp, qkv_out, tokens, n_out, k, stream, e);
    return stream_gemm::launch_stream<2, 2>(xp, wp, qkv_out, tokens, n_out, k, stream, e);
}
