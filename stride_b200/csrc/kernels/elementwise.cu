// Memory-bound kernels of the decoder step: embedding gather, residual add fused
// with RMSNorm, rotary position encoding fused with the write of keys and values
// into cache pages, and SiLU(gate) * up.
//
// Reductions, rotation angles and the residual sum are float32 in every mode.
// The residual stream itself is float32 in both modes; activations between the
// matrix products have the model's element type T (float or bfloat16).
#include "common.cuh"

namespace stride {

// ----------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] as float32 (python/stride_worker/model.py:252).
// Padded tokens (seq_of_token < 0) get zeros.
template <typename T>
__global__ void embed_gather_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ seq_of_token,
                                    const T* __restrict__ table, float* __restrict__ out, int hidden, int vocab) {
    const int t = blockIdx.x;
    const bool live = seq_of_token == nullptr || seq_of_token[t] >= 0;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // ids are validated on the host; never read outside the table
    const T* row = table + static_cast<size_t>(id) * hidden;
    float* dst = out + static_cast<size_t>(t) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = live ? to_f32(row[i]) : 0.f;
}

// ------------------------------------------------------- residual add + RMSNorm
// For row r (source row s = rows ? rows[r] : r):
//   x = residual[s] + delta[s]            (float32 sum; delta may be absent)
//   residual[s] = x                       (only when rows == nullptr)
//   out[r] = x * rsqrt(mean(x^2) + eps) * w
// The weight multiplies after the normalisation, all in float32, one rounding
// at the end (python/stride_worker/layers.py:24-35; sums model.py:300,310).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int32_t* __restrict__ rows, int hidden, float eps) {
    extern __shared__ float row_buf[];  // hidden floats, then 32 for the reduction
    float* scratch = row_buf + hidden;
    const int r = blockIdx.x;
    const size_t s = rows ? static_cast<size_t>(rows[r]) : static_cast<size_t>(r);
    float* res = residual + s * hidden;
    const T* del = delta ? delta + s * hidden : nullptr;
    float sq = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float x = res[i];
        if (del) x = __fadd_rn(x, to_f32(del[i]));
        row_buf[i] = x;
        sq = fmaf(x, x, sq);
    }
    const float total = block_sum(sq, scratch);
    const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
    T* dst = out + static_cast<size_t>(r) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float x = row_buf[i];
        if (del && !rows) res[i] = x;
        dst[i] = from_f32<T>(__fmul_rn(__fmul_rn(x, inv), weight[i]));
    }
}

// Writes residual += delta without a norm (the last sum of a model that wants
// its hidden state, or a part that asks for the materialised stream).
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ residual, const T* __restrict__ delta, size_t n) {
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (i < n) residual[i] = __fadd_rn(residual[i], to_f32(delta[i]));
}

// ------------------------------------------------- rotary encoding + cache write
// qkv is [tokens, (nq + 2 nkv) * hd]: query heads, key heads, value heads. For a
// query or key head, with c = cos[pos, i] and s = sin[pos, i] for i < hd/2:
//   out[i]        = x[i] * c - x[i + hd/2] * s
//   out[i + hd/2] = x[i + hd/2] * c + x[i] * s
// (x*cos + rotate_half(x)*sin with the half-split layout,
// python/stride_worker/layers.py:85-106). Queries are rotated in place; rotated
// keys and plain values go to the page slot of the token
// (python/stride_worker/cache.py:58-90). Pages are [page, kv_head, slot, hd].
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ bias,
                                     const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping,
                                     const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv, int hd,
                                     int page_size, int rotate) {
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int heads = nq + 2 * nkv;
    const int pos = positions[t];
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    T* row = qkv + static_cast<size_t>(t) * heads * hd;
    const float* cs = cos_table + static_cast<size_t>(pos) * half;
    const float* sn = sin_table + static_cast<size_t>(pos) * half;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int offset = slot >= 0 ? slot % page_size : 0;
    for (int w = threadIdx.x; w < heads * half; w += blockDim.x) {
        const int head = w / half, i = w - head * half;
        T* x = row + head * hd;
        float a = to_f32(x[i]), b = to_f32(x[i + half]);
        if (bias) {
            a = __fadd_rn(a, bias[head * hd + i]);
            b = __fadd_rn(b, bias[head * hd + i + half]);
        }
        if (head < nq + nkv && rotate) {
            const float c = cs[i], s = sn[i];
            const float ra = __fadd_rn(__fmul_rn(a, c), __fmul_rn(-b, s));
            const float rb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
            a = ra;
            b = rb;
        }
        if (head < nq) {
            x[i] = from_f32<T>(a);
            x[i + half] = from_f32<T>(b);
        } else if (slot >= 0) {
            const bool is_key = head < nq + nkv;
            const int kvh = is_key ? head - nq : head - nq - nkv;
            T* dst = (is_key ? k_pages : v_pages) +
                     ((static_cast<size_t>(page) * nkv + kvh) * page_size + offset) * hd;
            dst[i] = from_f32<T>(a);
            dst[i + half] = from_f32<T>(b);
        }
    }
}

// ---------------------------------------------------------------- SiLU(gate) * up
// in is [tokens, 2 * inter] (gate columns, then up columns); out is [tokens, inter].
// silu(z) = z * sigmoid(z) (python/stride_worker/layers.py:161), in float32.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, size_t total) {
    size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int i = static_cast<int>(idx - t * inter);
    const float g = to_f32(in[t * 2 * inter + i]);
    const float u = to_f32(in[t * 2 * inter + inter + i]);
    const float silu = g / (1.f + expf(-g));
    out[idx] = from_f32<T>(silu * u);
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_embed_gather(const int32_t* ids, const int32_t* seq_of_token, const void* table, float* out, int tokens,
                        int hidden, int vocab, int dtype, cudaStream_t stream) {
    if (tokens < 0 || hidden <= 0 || vocab <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == STRIDE_DTYPE_F32)
        embed_gather_kernel<float><<<tokens, threads, 0, stream>>>(ids, seq_of_token, static_cast<const float*>(table), out, hidden, vocab);
    else if (dtype == STRIDE_DTYPE_BF16)
        embed_gather_kernel<__nv_bfloat16><<<tokens, threads, 0, stream>>>(ids, seq_of_token, static_cast<const __nv_bfloat16*>(table), out, hidden, vocab);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_add_rmsnorm(float* residual, const void* delta, const float* weight, void* out, const int32_t* rows,
                       int num_rows, int hidden, float eps, int dtype, cudaStream_t stream) {
    if (num_rows < 0 || hidden <= 0) return STRIDE_BAD_ARGUMENT;
    if (num_rows == 0) return 0;
    const size_t smem = (static_cast<size_t>(hidden) + 32) * sizeof(float);
    if (smem > 200 * 1024) return STRIDE_UNSUPPORTED;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (dtype == STRIDE_DTYPE_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        add_rmsnorm_kernel<float><<<num_rows, threads, smem, stream>>>(residual, static_cast<const float*>(delta), weight, static_cast<float*>(out), rows, hidden, eps);
    } else if (dtype == STRIDE_DTYPE_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        add_rmsnorm_kernel<__nv_bfloat16><<<num_rows, threads, smem, stream>>>(residual, static_cast<const __nv_bfloat16*>(delta), weight, static_cast<__nv_bfloat16*>(out), rows, hidden, eps);
    } else {
        return STRIDE_BAD_ARGUMENT;
    }
    return STRIDE_LAUNCH_STATUS();
}

int stride_add_residual(float* residual, const void* delta, long long n, int dtype, cudaStream_t stream) {
    if (n < 0) return STRIDE_BAD_ARGUMENT;
    if (n == 0) return 0;
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
    if (dtype == STRIDE_DTYPE_F32)
        add_residual_kernel<float><<<blocks, 256, 0, stream>>>(residual, static_cast<const float*>(delta), static_cast<size_t>(n));
    else if (dtype == STRIDE_DTYPE_BF16)
        add_residual_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(residual, static_cast<const __nv_bfloat16*>(delta), static_cast<size_t>(n));
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_rope_kv_write(void* qkv, const float* bias, const int32_t* positions, const int32_t* slot_mapping,
                         const float* cos_table, const float* sin_table, void* k_pages, void* v_pages, int tokens,
                         int nq, int nkv, int hd, int page_size, int rotate, int dtype, cudaStream_t stream) {
    if (tokens < 0 || nq <= 0 || nkv <= 0 || hd <= 0 || page_size <= 0) return STRIDE_BAD_ARGUMENT;
    if (hd % 2) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    const int work = (nq + 2 * nkv) * (hd / 2);
    const int threads = work >= 1024 ? 256 : 128;
    if (dtype == STRIDE_DTYPE_F32)
        rope_kv_write_kernel<float><<<tokens, threads, 0, stream>>>(static_cast<float*>(qkv), bias, positions, slot_mapping, cos_table, sin_table, static_cast<float*>(k_pages), static_cast<float*>(v_pages), nq, nkv, hd, page_size, rotate);
    else if (dtype == STRIDE_DTYPE_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<tokens, threads, 0, stream>>>(static_cast<__nv_bfloat16*>(qkv), bias, positions, slot_mapping, cos_table, sin_table, static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), nq, nkv, hd, page_size, rotate);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_silu_mul(const void* in, void* out, int tokens, int inter, int dtype, cudaStream_t stream) {
    if (tokens < 0 || inter <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const size_t total = static_cast<size_t>(tokens) * inter;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    if (dtype == STRIDE_DTYPE_F32)
        silu_mul_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(in), static_cast<float*>(out), inter, total);
    else if (dtype == STRIDE_DTYPE_BF16)
        silu_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), inter, total);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
