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

// NT: token tiles of eight. MODE 0: bfloat16 output, 1: float32 output.
template <int NT, int WARPS, int MODE>
__global__ void __launch_bounds__(WARPS * 32)
gemm_stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, void* __restrict__ out, int m, int n,
                   int k) {
    constexpr int STAGES = Ring<NT>::kStages;
    constexpr int THREADS = WARPS * 32;
    constexpr int PIECES = 2 + NT;           // per step: rows g and g + 8 of the weights, then one piece of x per token tile
    extern __shared__ __align__(16) uint4 ring[];        // [STAGES][kUnroll][PIECES][THREADS]
    __shared__ float red[WARPS][NT][kRows][8];
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * kRows;
    const __nv_bfloat16* w_lo = w + static_cast<size_t>(min(r0 + g, n - 1)) * k + 8 * t;
    const __nv_bfloat16* w_hi = w + static_cast<size_t>(min(r0 + g + 8, n - 1)) * k + 8 * t;
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
    {
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
int launch_warps(const __nv_bfloat16* x, const __nv_bfloat16* w, void* out, int m, int n, int k, cudaStream_t stream) {
    constexpr int smem = Ring<NT>::kStages * kUnroll * (2 + NT) * WARPS * 32 * 16;
    auto kernel = gemm_stream_kernel<NT, WARPS, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    stride::launch(kernel, dim3(static_cast<unsigned>((n + kRows - 1) / kRows)), dim3(WARPS * 32), smem, stream, x, w, out, m, n, k);
    return STRIDE_LAUNCH_STATUS();
}

template <int NT, int MODE>
int launch_stream(const __nv_bfloat16* x, const __nv_bfloat16* w, void* out, int m, int n, int k, cudaStream_t stream) {
    const int batches = ((k + kStepCols - 1) / kStepCols + kUnroll - 1) / kUnroll;
    if (batches >= 8 * 4) return launch_warps<NT, 8, MODE>(x, w, out, m, n, k, stream);
    if (batches >= 4 * 4) return launch_warps<NT, 4, MODE>(x, w, out, m, n, k, stream);
    return launch_warps<NT, 2, MODE>(x, w, out, m, n, k, stream);
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
