// Paged attention for any mix of prompt portions and decoded tokens, in float32
// or bfloat16 storage with float32 arithmetic. This is the exact, slower kernel:
// the whole 32-bit path runs on it, and the bfloat16 path falls back to it for
// head sizes or windows that the tensor-core kernels refuse.
//
// One warp owns one (token, query head). The token at absolute position p of its
// request reads the keys j <= p (and j > p - window when a window is set) through
// the request's block table: softmax(q k^T * scale) v with the causal rule of
// python/stride_worker/layers.py:109-149; query head h reads key head
// h / (nq / nkv). Keys are walked in groups of 32 aligned to absolute position 0,
// with an online softmax, so the order of every sum depends only on p: the result
// for a token is bitwise the same in a whole prompt, in a portion or as a single
// decoded token, whatever pages hold the keys.
#include "common.cuh"

namespace stride {

constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int hd) {
    float acc = 0.f;
    for (int d = 0; d < hd; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + d);
        acc = fmaf(q[d], kv.x, acc);
        acc = fmaf(q[d + 1], kv.y, acc);
        acc = fmaf(q[d + 2], kv.z, acc);
        acc = fmaf(q[d + 3], kv.w, acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int hd) {
    float acc = 0.f;
    for (int d = 0; d < hd; d += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(pairs[i]);
            acc = fmaf(q[d + 2 * i], f.x, acc);
            acc = fmaf(q[d + 2 * i + 1], f.y, acc);
        }
    }
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, const T* __restrict__ k_pages,
                               const T* __restrict__ v_pages, const int32_t* __restrict__ block_table, int table_width,
                               const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ positions, int nq,
                               int nkv, int hd, int page_size, float scale, int window) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float q_smem[kWarps][kMaxHeadDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * kWarps + warp;
    if (head >= nq) return;
    T* out_row = out + (static_cast<size_t>(t) * nq + head) * hd;
    const int seq = seq_of_token[t];
    if (seq < 0) {  // a padded token of a fixed-size batch
        for (int d = lane; d < hd; d += 32) out_row[d] = from_f32<T>(0.f);
        return;
    }
    const int pos = positions[t];
    const int kvh = head / (nq / nkv);
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int32_t* table = block_table + static_cast<size_t>(seq) * table_width;

    float* qs = q_smem[warp];
    const T* q_row = q + static_cast<size_t>(t) * q_stride + static_cast<size_t>(head) * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32(q_row[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[kMaxHeadDim / 32];
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.f;

    for (int base = (first / 32) * 32; base <= pos; base += 32) {
        const int key = base + lane;
        const bool ok = key >= first && key <= pos;
        float s = -INFINITY;
        if (ok) {
            const int page = table[key / page_size];
            const T* k_row = k_pages + ((static_cast<size_t>(page) * nkv + kvh) * page_size + key % page_size) * hd;
            s = dot_row<T>(qs, k_row, hd) * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = ok ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= corr;
        unsigned valid = __ballot_sync(0xffffffffu, ok);
        while (valid) {
            const int j = __ffs(valid) - 1;
            valid &= valid - 1;
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const int kj = base + j;
            const int page = table[kj / page_size];
            const T* v_row = v_pages + ((static_cast<size_t>(page) * nkv + kvh) * page_size + kj % page_size) * hd;
#pragma unroll
            for (int i = 0; i < kMaxHeadDim / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pj, to_f32(v_row[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) out_row[d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace stride

using namespace stride;

// q: [tokens, q_stride] with head h at columns [h*hd, (h+1)*hd); out: [tokens, nq, hd];
// pages: [num_pages, nkv, page_size, hd]; block_table: [seqs, table_width].
extern "C" int stride_paged_attention_generic(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                              const int32_t* block_table, int table_width, const int32_t* seq_of_token,
                                              const int32_t* positions, int tokens, int nq, int nkv, int hd, int page_size,
                                              float scale, int window, int dtype, cudaStream_t stream) {
    if (tokens < 0 || nq <= 0 || nkv <= 0 || hd <= 0 || page_size <= 0 || table_width <= 0 || window < 0) return STRIDE_BAD_ARGUMENT;
    if (nq % nkv) return STRIDE_BAD_ARGUMENT;
    if (hd % 16 || hd > kMaxHeadDim) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    dim3 grid(tokens, (nq + kWarps - 1) / kWarps);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(paged_attention_generic_kernel<float>, dim3(grid), dim3(kWarps * 32), 0, stream, 
            static_cast<const float*>(q), q_stride, static_cast<float*>(out), static_cast<const float*>(k_pages),
            static_cast<const float*>(v_pages), block_table, table_width, seq_of_token, positions, nq, nkv, hd, page_size, scale, window);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(paged_attention_generic_kernel<__nv_bfloat16>, dim3(grid), dim3(kWarps * 32), 0, stream, 
            static_cast<const __nv_bfloat16*>(q), q_stride, static_cast<__nv_bfloat16*>(out),
            static_cast<const __nv_bfloat16*>(k_pages), static_cast<const __nv_bfloat16*>(v_pages), block_table, table_width,
            seq_of_token, positions, nq, nkv, hd, page_size, scale, window);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}
