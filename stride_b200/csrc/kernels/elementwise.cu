// Memory-bound kernels of the decoder step: embedding gather, residual add fused
// with RMSNorm, rotary position encoding fused with the write of keys and values
// into cache pages, and SiLU(gate) * up.
//
// Reductions, rotation angles and the residual sum are float32 in every mode.
// The residual stream itself is float32 in both modes; activations between the
// matrix products have the model's element type T (float or bfloat16).
#include <algorithm>

#include "common.cuh"

namespace stride {

// ----------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] as float32 (python/stride_worker/model.py:252).
// Padded tokens (seq_of_token < 0) get zeros.
template <typename T>
__global__ void embed_gather_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ seq_of_token,
                                    const T* __restrict__ table, float* __restrict__ out, int hidden, int vocab) {
    pdl_trigger();
    pdl_wait();
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
    pdl_trigger();
    pdl_wait();
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
    pdl_trigger();
    pdl_wait();
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
    pdl_trigger();
    pdl_wait();
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
// in is [tokens, 2 * inter], out is [tokens, inter]. The gate and up columns alternate in blocks of `block`
// columns (gate 0..block-1, up 0..block-1, gate block.., ...); block == inter is the plain layout, all gate
// columns and then all up columns. silu(z) = z * sigmoid(z) (python/stride_worker/layers.py:161), in float32.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, int block, size_t total) {
    pdl_trigger();
    pdl_wait();
    size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int i = static_cast<int>(idx - t * inter);
    const size_t at = t * 2 * inter + static_cast<size_t>(i / block) * 2 * block + i % block;
    const float g = to_f32(in[at]);
    const float u = to_f32(in[at + block]);
    const float silu = g / (1.f + expf(-g));
    out[idx] = from_f32<T>(silu * u);
}

// ------------------------------------------------------------------ 16-byte vectors
// A pack of V consecutive elements that is loaded and stored with one 16-byte
// access (4 floats or 8 bfloat16).
template <typename T>
struct Pack;
template <>
struct Pack<float> {
    static constexpr int V = 4;
    float v[4];
    __device__ __forceinline__ void load(const float* p) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct Pack<__nv_bfloat16> {
    static constexpr int V = 8;
    float v[8];
    __device__ __forceinline__ void load(const __nv_bfloat16* p) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

// Same arithmetic as add_rmsnorm_kernel, four columns per thread and the row
// kept in registers (hidden <= 4 * ITERS * blockDim.x, hidden % 4 == 0).
template <typename T, int ITERS>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                       const float* __restrict__ weight, T* __restrict__ out,
                                       const int32_t* __restrict__ rows, int hidden, float eps) {
    pdl_trigger();
    __shared__ float scratch[32];
    // the norm's weight does not depend on the kernel before this one: fetch it while that one finishes
    float4 wv[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        wv[it] = c < hidden ? *reinterpret_cast<const float4*>(weight + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    const int r = blockIdx.x;
    const size_t s = rows ? static_cast<size_t>(rows[r]) : static_cast<size_t>(r);
    float* res = residual + s * hidden;
    const T* del = delta ? delta + s * hidden : nullptr;
    float4 x[ITERS];
    float sq = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < hidden) {
            x[it] = *reinterpret_cast<const float4*>(res + c);
            if (del) {
                float d[4];
                if constexpr (sizeof(T) == 2) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(del + c);
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
                    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
                    d[0] = a.x; d[1] = a.y; d[2] = b.x; d[3] = b.y;
                } else {
                    const float4 t = *reinterpret_cast<const float4*>(del + c);
                    d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
                }
                x[it].x = __fadd_rn(x[it].x, d[0]);
                x[it].y = __fadd_rn(x[it].y, d[1]);
                x[it].z = __fadd_rn(x[it].z, d[2]);
                x[it].w = __fadd_rn(x[it].w, d[3]);
                if (!rows) *reinterpret_cast<float4*>(res + c) = x[it];
            }
            sq = fmaf(x[it].x, x[it].x, sq);
            sq = fmaf(x[it].y, x[it].y, sq);
            sq = fmaf(x[it].z, x[it].z, sq);
            sq = fmaf(x[it].w, x[it].w, sq);
        }
    }
    const float total = block_sum(sq, scratch);
    const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
    T* dst = out + static_cast<size_t>(r) * hidden;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < hidden) {
            const float4 w = wv[it];
            const float y0 = __fmul_rn(__fmul_rn(x[it].x, inv), w.x), y1 = __fmul_rn(__fmul_rn(x[it].y, inv), w.y);
            const float y2 = __fmul_rn(__fmul_rn(x[it].z, inv), w.z), y3 = __fmul_rn(__fmul_rn(x[it].w, inv), w.w);
            if constexpr (sizeof(T) == 2) {
                uint2 raw;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
                h[0] = __floats2bfloat162_rn(y0, y1);
                h[1] = __floats2bfloat162_rn(y2, y3);
                *reinterpret_cast<uint2*>(dst + c) = raw;
            } else {
                *reinterpret_cast<float4*>(dst + c) = make_float4(y0, y1, y2, y3);
            }
        }
    }
}

// The same arithmetic once more in the form that streams fastest: one pack of V consecutive columns per thread
// (8 for bfloat16, 4 for float32; hidden <= V * blockDim.x), every load issued before anything is computed or
// stored, so that a store to the residual never stands between two loads. One CTA per row.
template <typename T>
__global__ void add_rmsnorm_pack_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                        const float* __restrict__ weight, T* __restrict__ out,
                                        const int32_t* __restrict__ rows, int hidden, float eps) {
    pdl_trigger();
    constexpr int V = Pack<T>::V;
    __shared__ float scratch[32];
    const int c = threadIdx.x * V;
    const bool live = c < hidden;
    // the norm's weight does not depend on the kernel before this one: fetch it while that one finishes
    float w[V];
#pragma unroll
    for (int j = 0; j < V; j += 4) {
        const float4 t = live ? *reinterpret_cast<const float4*>(weight + c + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        w[j] = t.x; w[j + 1] = t.y; w[j + 2] = t.z; w[j + 3] = t.w;
    }
    pdl_wait();
    const int r = blockIdx.x;
    const size_t s = rows ? static_cast<size_t>(rows[r]) : static_cast<size_t>(r);
    float* res = residual + s * hidden;
    float x[V];
    Pack<T> d;
    if (live) {
#pragma unroll
        for (int j = 0; j < V; j += 4) {
            const float4 t = *reinterpret_cast<const float4*>(res + c + j);
            x[j] = t.x; x[j + 1] = t.y; x[j + 2] = t.z; x[j + 3] = t.w;
        }
        if (delta) d.load(delta + s * hidden + c);
    }
    float sq = 0.f;
    if (live) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
            if (delta) x[j] = __fadd_rn(x[j], d.v[j]);
            sq = fmaf(x[j], x[j], sq);
        }
        if (delta && !rows) {
#pragma unroll
            for (int j = 0; j < V; j += 4) *reinterpret_cast<float4*>(res + c + j) = make_float4(x[j], x[j + 1], x[j + 2], x[j + 3]);
        }
    }
    const float total = block_sum(sq, scratch);
    const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
    if (live) {
        Pack<T> y;
#pragma unroll
        for (int j = 0; j < V; ++j) y.v[j] = __fmul_rn(__fmul_rn(x[j], inv), w[j]);
        y.store(out + static_cast<size_t>(r) * hidden + c);
    }
}

// rope_kv_write_kernel with 16-byte accesses: one unit of work is V consecutive
// pair indices of one head (needs hd / 2 to be a multiple of V).
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, const float* __restrict__ bias,
                                         const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping,
                                         const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                         T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv, int hd,
                                         int page_size, int rotate) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Pack<T>::V;
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int per_head = half / V;
    const int heads = nq + 2 * nkv;
    const int pos = positions[t];
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    T* row = qkv + static_cast<size_t>(t) * heads * hd;
    const float* cs = cos_table + static_cast<size_t>(pos) * half;
    const float* sn = sin_table + static_cast<size_t>(pos) * half;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int offset = slot >= 0 ? slot % page_size : 0;
    for (int w = threadIdx.x; w < heads * per_head; w += blockDim.x) {
        const int head = w / per_head, i = (w - head * per_head) * V;
        T* x = row + head * hd;
        Pack<T> a, b;
        a.load(x + i);
        b.load(x + i + half);
        if (bias) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                a.v[j] = __fadd_rn(a.v[j], bias[head * hd + i + j]);
                b.v[j] = __fadd_rn(b.v[j], bias[head * hd + i + half + j]);
            }
        }
        if (head < nq + nkv && rotate) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const float c = cs[i + j], s = sn[i + j];
                const float ra = __fadd_rn(__fmul_rn(a.v[j], c), __fmul_rn(-b.v[j], s));
                const float rb = __fadd_rn(__fmul_rn(b.v[j], c), __fmul_rn(a.v[j], s));
                a.v[j] = ra;
                b.v[j] = rb;
            }
        }
        if (head < nq) {
            a.store(x + i);
            b.store(x + i + half);
        } else if (slot >= 0) {
            const bool is_key = head < nq + nkv;
            const int kvh = is_key ? head - nq : head - nq - nkv;
            T* dst = (is_key ? k_pages : v_pages) + ((static_cast<size_t>(page) * nkv + kvh) * page_size + offset) * hd;
            a.store(dst + i);
            b.store(dst + i + half);
        }
    }
}

// The same with one unit of work per thread and no loop (a unit: V consecutive pair indices of one head, i.e. one
// pack from each half of the head), loads before stores: blockIdx.x is the token, blockIdx.y a chunk of the units.
template <typename T>
__global__ void rope_kv_write_pack_kernel(T* __restrict__ qkv, const float* __restrict__ bias,
                                          const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping,
                                          const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                          T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv, int hd,
                                          int page_size, int rotate) {
    pdl_trigger();
    constexpr int V = Pack<T>::V;
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int per_head = half / V;
    const int heads = nq + 2 * nkv;
    const int w = blockIdx.y * blockDim.x + threadIdx.x;
    if (w >= heads * per_head) return;
    const int head = w / per_head, i = (w - head * per_head) * V;
    const int pos = positions[t];                  // the step's index arrays are not written by the kernel before
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    const bool turns = head < nq + nkv && rotate;
    float c[V], sn[V];
    if (turns) {
#pragma unroll
        for (int j = 0; j < V; j += 4) {
            const float4 a = *reinterpret_cast<const float4*>(cos_table + static_cast<size_t>(pos) * half + i + j);
            const float4 b = *reinterpret_cast<const float4*>(sin_table + static_cast<size_t>(pos) * half + i + j);
            c[j] = a.x; c[j + 1] = a.y; c[j + 2] = a.z; c[j + 3] = a.w;
            sn[j] = b.x; sn[j + 1] = b.y; sn[j + 2] = b.z; sn[j + 3] = b.w;
        }
    }
    pdl_wait();
    T* x = qkv + (static_cast<size_t>(t) * heads + head) * hd;
    Pack<T> a, b;
    a.load(x + i);
    b.load(x + i + half);
    if (bias) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
            a.v[j] = __fadd_rn(a.v[j], bias[head * hd + i + j]);
            b.v[j] = __fadd_rn(b.v[j], bias[head * hd + i + half + j]);
        }
    }
    if (turns) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float ra = __fadd_rn(__fmul_rn(a.v[j], c[j]), __fmul_rn(-b.v[j], sn[j]));
            const float rb = __fadd_rn(__fmul_rn(b.v[j], c[j]), __fmul_rn(a.v[j], sn[j]));
            a.v[j] = ra;
            b.v[j] = rb;
        }
    }
    if (head < nq) {
        a.store(x + i);
        b.store(x + i + half);
    } else if (slot >= 0) {
        const int page = slot / page_size, offset = slot % page_size;
        const bool is_key = head < nq + nkv;
        const int kvh = is_key ? head - nq : head - nq - nkv;
        T* dst = (is_key ? k_pages : v_pages) + ((static_cast<size_t>(page) * nkv + kvh) * page_size + offset) * hd;
        a.store(dst + i);
        b.store(dst + i + half);
    }
}

// silu_mul_kernel with 16-byte accesses (block % V == 0): one pack per thread and no loop, the form that streams
// fastest here (several packs per thread, a grid-stride apart, measured 25 to 80 % slower).
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, int block, size_t packs) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Pack<T>::V;
    const int per_row = inter / V;
    const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= packs) return;
    const size_t t = idx / per_row;
    const int i = static_cast<int>(idx - t * per_row) * V;
    Pack<T> g, u;
    const size_t at = t * 2 * inter + static_cast<size_t>(i / block) * 2 * block + i % block;
    g.load(in + at);
    u.load(in + at + block);
#pragma unroll
    for (int j = 0; j < V; ++j) {
        if constexpr (sizeof(T) == 2) {
            // bfloat16: the hardware exponential and reciprocal (a few units in the last place of float32, far below
            // the rounding of the result to bfloat16) take a tenth off the kernel; float32 stays exact
            g.v[j] = __fmul_rn(__fmul_rn(g.v[j], __frcp_rn(1.f + __expf(-g.v[j]))), u.v[j]);
        } else {
            g.v[j] = (g.v[j] / (1.f + expf(-g.v[j]))) * u.v[j];
        }
    }
    g.store(out + t * inter + i);
}

// embed_gather_kernel with 16-byte reads of the table (hidden % V == 0).
template <typename T>
__global__ void embed_gather_vec_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ seq_of_token,
                                        const T* __restrict__ table, float* __restrict__ out, int hidden, int vocab) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Pack<T>::V;
    const int t = blockIdx.x;
    const bool live = seq_of_token == nullptr || seq_of_token[t] >= 0;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const T* row = table + static_cast<size_t>(id) * hidden;
    float* dst = out + static_cast<size_t>(t) * hidden;
    for (int i = threadIdx.x * V; i < hidden; i += blockDim.x * V) {
        Pack<T> p;
        if (live) p.load(row + i);
#pragma unroll
        for (int j = 0; j < V; j += 4)
            *reinterpret_cast<float4*>(dst + i + j) =
                live ? make_float4(p.v[j], p.v[j + 1], p.v[j + 2], p.v[j + 3]) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// The second half of an RMS norm that was folded into the product before it (gemm_bf16_stream.cu, RowNorm): x~
// holds residual * weight in bfloat16, `partials` [count][token_stride] the sums of squares of the residual per producer CTA
// and token. out = x~ * rsqrt(sum / width + eps). Only needed when what consumes the norm cannot apply the factor
// itself.
__global__ void scale_rows_kernel(const __nv_bfloat16* __restrict__ xt, const float* __restrict__ partials, int count, float eps,
                                  __nv_bfloat16* __restrict__ out, int width, int token_stride) {
    pdl_trigger();
    pdl_wait();
    __shared__ float factor;
    const int t = blockIdx.x;
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int c = 0; c < count; ++c) total += partials[c * token_stride + t];
        factor = rsqrtf(total / static_cast<float>(width) + eps);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        out[static_cast<size_t>(t) * width + c] = __float2bfloat16_rn(__bfloat162float(xt[static_cast<size_t>(t) * width + c]) * factor);
}

// --------------------------------------------------------------------------- state slots
// A request's state slot starts at zero: a sequence whose first token of this step sits at position 0 is at its
// beginning (a new request, or one that is recomputed after it was preempted), so the row of its slot is cleared
// before any layer runs. Reads only the step's index arrays, so it can sit in a captured graph. One row of CTAs
// per sequence of the layout (padded ones have q_len 0), 4-byte words.
__global__ void zero_fresh_state_kernel(uint32_t* __restrict__ state, long long row_words, const int32_t* __restrict__ state_slot,
                                        const int32_t* __restrict__ q_start, const int32_t* __restrict__ q_len,
                                        const int32_t* __restrict__ positions, int num_slots) {
    pdl_trigger();
    const int s = blockIdx.y;
    if (q_len[s] <= 0 || positions[q_start[s]] != 0) return;
    const int slot = state_slot[s];
    if (slot < 0 || slot >= num_slots) return;
    pdl_wait();
    uint32_t* row = state + static_cast<size_t>(slot) * row_words;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < row_words;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        row[i] = 0u;
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_embed_gather(const int32_t* ids, const int32_t* seq_of_token, const void* table, float* out, int tokens,
                        int hidden, int vocab, int dtype, cudaStream_t stream) {
    if (tokens < 0 || hidden <= 0 || vocab <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    const bool aligned = (reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
    if (dtype == STRIDE_DTYPE_F32) {
        if (aligned && hidden % 4 == 0)
            stride::launch(embed_gather_vec_kernel<float>, dim3(tokens), dim3(128), 0, stream, ids, seq_of_token, static_cast<const float*>(table), out, hidden, vocab);
        else
            stride::launch(embed_gather_kernel<float>, dim3(tokens), dim3(threads), 0, stream, ids, seq_of_token, static_cast<const float*>(table), out, hidden, vocab);
    } else if (dtype == STRIDE_DTYPE_BF16) {
        if (aligned && hidden % 8 == 0)
            stride::launch(embed_gather_vec_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, ids, seq_of_token, static_cast<const __nv_bfloat16*>(table), out, hidden, vocab);
        else
            stride::launch(embed_gather_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, ids, seq_of_token, static_cast<const __nv_bfloat16*>(table), out, hidden, vocab);
    } else {
        return STRIDE_BAD_ARGUMENT;
    }
    return STRIDE_LAUNCH_STATUS();
}

int stride_add_rmsnorm(float* residual, const void* delta, const float* weight, void* out, const int32_t* rows,
                       int num_rows, int hidden, float eps, int dtype, cudaStream_t stream) {
    if (num_rows < 0 || hidden <= 0) return STRIDE_BAD_ARGUMENT;
    if (num_rows == 0) return 0;
    {
        // Vector path: the row stays in registers, four columns per thread.
        const uintptr_t bits = reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(delta) |
                               reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out);
        const int quads = hidden / 4;
        // one pack per thread where a row fits one CTA that way (the choice depends on the width alone, never on the
        // number of rows, so a row's bits do not depend on what else is in the batch)
        const int pack = dtype == STRIDE_DTYPE_F32 ? 4 : 8;
        if (hidden % pack == 0 && bits % 16 == 0 && hidden / pack <= 1024 && (dtype == STRIDE_DTYPE_F32 || dtype == STRIDE_DTYPE_BF16)) {
            const int pthreads = (hidden / pack + 31) / 32 * 32;
            if (dtype == STRIDE_DTYPE_F32)
                stride::launch(add_rmsnorm_pack_kernel<float>, dim3(num_rows), dim3(pthreads), 0, stream, residual, static_cast<const float*>(delta), weight, static_cast<float*>(out), rows, hidden, eps);
            else
                stride::launch(add_rmsnorm_pack_kernel<__nv_bfloat16>, dim3(num_rows), dim3(pthreads), 0, stream, residual, static_cast<const __nv_bfloat16*>(delta), weight, static_cast<__nv_bfloat16*>(out), rows, hidden, eps);
            return STRIDE_LAUNCH_STATUS();
        }
        if (hidden % 4 == 0 && bits % 16 == 0 && quads <= 8 * 256 && (dtype == STRIDE_DTYPE_F32 || dtype == STRIDE_DTYPE_BF16)) {
            const int threads = quads <= 32 ? 32 : (quads <= 64 ? 64 : (quads <= 128 ? 128 : 256));
            const int iters = (quads + threads - 1) / threads;
#define STRIDE_NORM_LAUNCH(T, I)                                                                                            \
    stride::launch(add_rmsnorm_vec_kernel<T, I>, dim3(num_rows), dim3(threads), 0, stream, residual, static_cast<const T*>(delta), weight,         \
                                                                   static_cast<T*>(out), rows, hidden, eps)
#define STRIDE_NORM_DISPATCH(T)                                                                                             \
    do {                                                                                                                   \
        if (iters <= 1) STRIDE_NORM_LAUNCH(T, 1);                                                                          \
        else if (iters <= 2) STRIDE_NORM_LAUNCH(T, 2);                                                                     \
        else if (iters <= 4) STRIDE_NORM_LAUNCH(T, 4);                                                                     \
        else STRIDE_NORM_LAUNCH(T, 8);                                                                                     \
    } while (0)
            if (dtype == STRIDE_DTYPE_F32) STRIDE_NORM_DISPATCH(float);
            else STRIDE_NORM_DISPATCH(__nv_bfloat16);
#undef STRIDE_NORM_DISPATCH
#undef STRIDE_NORM_LAUNCH
            return STRIDE_LAUNCH_STATUS();
        }
    }
    const size_t smem = (static_cast<size_t>(hidden) + 32) * sizeof(float);
    if (smem > 200 * 1024) return STRIDE_UNSUPPORTED;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (dtype == STRIDE_DTYPE_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        stride::launch(add_rmsnorm_kernel<float>, dim3(num_rows), dim3(threads), smem, stream, residual, static_cast<const float*>(delta), weight, static_cast<float*>(out), rows, hidden, eps);
    } else if (dtype == STRIDE_DTYPE_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        stride::launch(add_rmsnorm_kernel<__nv_bfloat16>, dim3(num_rows), dim3(threads), smem, stream, residual, static_cast<const __nv_bfloat16*>(delta), weight, static_cast<__nv_bfloat16*>(out), rows, hidden, eps);
    } else {
        return STRIDE_BAD_ARGUMENT;
    }
    return STRIDE_LAUNCH_STATUS();
}

// Clears the state rows [num_slots, row_bytes] of the sequences that start at position 0 in this step.
// `seq_cap`: entries of state_slot / q_start / q_len (the layout's capacity; padded sequences have q_len 0).
int stride_zero_fresh_state(void* state, long long row_bytes, int num_slots, const int32_t* state_slot, const int32_t* q_start,
                            const int32_t* q_len, const int32_t* positions, int seq_cap, cudaStream_t stream) {
    if (row_bytes <= 0 || row_bytes % 4 || num_slots <= 0 || seq_cap < 0 || seq_cap > 65535) return STRIDE_BAD_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(state) % 4) return STRIDE_BAD_ARGUMENT;
    if (seq_cap == 0) return 0;
    const long long words = row_bytes / 4;
    const unsigned blocks = static_cast<unsigned>(words >= 65536 ? 64 : (words + 255) / 256 > 0 ? (words + 255) / 256 : 1);
    stride::launch(zero_fresh_state_kernel, dim3(blocks, seq_cap), dim3(256), 0, stream, static_cast<uint32_t*>(state), words, state_slot,
                   q_start, q_len, positions, num_slots);
    return STRIDE_LAUNCH_STATUS();
}

int stride_add_residual(float* residual, const void* delta, long long n, int dtype, cudaStream_t stream) {
    if (n < 0) return STRIDE_BAD_ARGUMENT;
    if (n == 0) return 0;
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(add_residual_kernel<float>, dim3(blocks), dim3(256), 0, stream, residual, static_cast<const float*>(delta), static_cast<size_t>(n));
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(add_residual_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, residual, static_cast<const __nv_bfloat16*>(delta), static_cast<size_t>(n));
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
    {
        const uintptr_t bits = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages);
        const int vec = dtype == STRIDE_DTYPE_F32 ? 4 : 8;
        if (bits % 16 == 0 && (hd / 2) % vec == 0 && (dtype == STRIDE_DTYPE_F32 || dtype == STRIDE_DTYPE_BF16)) {
            const int units = work / vec;
            if (reinterpret_cast<uintptr_t>(cos_table) % 16 == 0 && reinterpret_cast<uintptr_t>(sin_table) % 16 == 0 && (hd / 2) % 4 == 0) {
                // one unit per thread, no loop
                const int pthreads = units >= 512 ? 256 : (units + 31) / 32 * 32;
                const dim3 grid(tokens, (units + pthreads - 1) / pthreads);
                if (dtype == STRIDE_DTYPE_F32)
                    stride::launch(rope_kv_write_pack_kernel<float>, grid, dim3(pthreads), 0, stream, static_cast<float*>(qkv), bias, positions, slot_mapping, cos_table, sin_table, static_cast<float*>(k_pages), static_cast<float*>(v_pages), nq, nkv, hd, page_size, rotate);
                else
                    stride::launch(rope_kv_write_pack_kernel<__nv_bfloat16>, grid, dim3(pthreads), 0, stream, static_cast<__nv_bfloat16*>(qkv), bias, positions, slot_mapping, cos_table, sin_table, static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), nq, nkv, hd, page_size, rotate);
                return STRIDE_LAUNCH_STATUS();
            }
            const int vthreads = units >= 256 ? 256 : (units >= 128 ? 128 : 64);
            if (dtype == STRIDE_DTYPE_F32)
                stride::launch(rope_kv_write_vec_kernel<float>, dim3(tokens), dim3(vthreads), 0, stream, static_cast<float*>(qkv), bias, positions, slot_mapping, cos_table, sin_table, static_cast<float*>(k_pages), static_cast<float*>(v_pages), nq, nkv, hd, page_size, rotate);
            else
                stride::launch(rope_kv_write_vec_kernel<__nv_bfloat16>, dim3(tokens), dim3(vthreads), 0, stream, static_cast<__nv_bfloat16*>(qkv), bias, positions, slot_mapping, cos_table, sin_table, static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), nq, nkv, hd, page_size, rotate);
            return STRIDE_LAUNCH_STATUS();
        }
    }
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(rope_kv_write_kernel<float>, dim3(tokens), dim3(threads), 0, stream, static_cast<float*>(qkv), bias, positions, slot_mapping, cos_table, sin_table, static_cast<float*>(k_pages), static_cast<float*>(v_pages), nq, nkv, hd, page_size, rotate);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(rope_kv_write_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, static_cast<__nv_bfloat16*>(qkv), bias, positions, slot_mapping, cos_table, sin_table, static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), nq, nkv, hd, page_size, rotate);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_silu_mul(const void* in, void* out, int tokens, int inter, int block, int dtype, cudaStream_t stream) {
    if (tokens < 0 || inter <= 0 || block <= 0 || inter % block) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const size_t total = static_cast<size_t>(tokens) * inter;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    {
        const uintptr_t bits = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out);
        const int vec = dtype == STRIDE_DTYPE_F32 ? 4 : 8;
        if (bits % 16 == 0 && block % vec == 0 && (dtype == STRIDE_DTYPE_F32 || dtype == STRIDE_DTYPE_BF16)) {
            const size_t packs = total / vec;
            if ((packs + 127) / 128 > 0x7fffffffull) return STRIDE_UNSUPPORTED;
            const unsigned vblocks = static_cast<unsigned>((packs + 127) / 128);
            if (dtype == STRIDE_DTYPE_F32)
                stride::launch(silu_mul_vec_kernel<float>, dim3(vblocks), dim3(128), 0, stream, static_cast<const float*>(in), static_cast<float*>(out), inter, block, packs);
            else
                stride::launch(silu_mul_vec_kernel<__nv_bfloat16>, dim3(vblocks), dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), inter, block, packs);
            return STRIDE_LAUNCH_STATUS();
        }
    }
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, static_cast<const float*>(in), static_cast<float*>(out), inter, block, total);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), inter, block, total);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_scale_rows(const void* xtilde, const float* partials, int count, float eps, void* out, int tokens, int width,
                      int token_stride, cudaStream_t stream) {
    if (tokens < 0 || tokens > token_stride || width <= 0 || count <= 0 || partials == nullptr) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    stride::launch(scale_rows_kernel, dim3(tokens), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(xtilde), partials, count, eps,
                   static_cast<__nv_bfloat16*>(out), width, token_stride);
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
