// Prefill attention in bfloat16 over the paged cache: portions of prompts of any
// length, each attending to the keys its request already holds plus its own.
//
// One CTA owns 64 consecutive query rows of one request and one query head; each
// of its four warps owns 16 rows. Keys and values are walked in tiles of 64,
// fetched through the request's block table with cp.async into two shared-memory
// stages (rows XOR-swizzled for ldmatrix), multiplied on the tensor cores
// (mma.sync m16n8k16, float32 accumulators) with an online softmax in float32.
// The query at absolute position p sees keys j <= p and, with a window, j > p -
// window (python/stride_worker/layers.py:109-149: the mask is
// k_pos <= query_start + i, the scale hd^-0.5, query head h reads key head
// h / (nq / nkv)). The keys of the portion itself are read from the cache, where
// the rotary kernel has just written them.
#include "common.cuh"
#include "mma.cuh"

namespace stride {

constexpr int kQTile = 64;    // query rows per CTA
constexpr int kKTile = 64;    // keys per step

template <int HD>
__global__ void __launch_bounds__(128)
paged_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                     const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                     const int32_t* __restrict__ block_table, int table_width, const int32_t* __restrict__ q_start,
                     const int32_t* __restrict__ q_len, const int32_t* __restrict__ ctx_len, int num_seqs, int nq, int nkv,
                     int page_size, float scale_log2e, int window) {
    pdl_trigger();
    pdl_wait();
    constexpr int ROW_BYTES = HD * 2;
    constexpr int CHUNKS = HD / 8;
    constexpr int KSTEPS = HD / 16;
    constexpr int STAGE_BYTES = 2 * kKTile * ROW_BYTES;     // keys, then values
    extern __shared__ __align__(128) unsigned char smem[];

    // Which request and which of its query tiles is this CTA?
    int seq = -1, tile = 0;
    {
        int acc = 0;
        for (int s = 0; s < num_seqs; ++s) {
            const int tiles = (q_len[s] + kQTile - 1) / kQTile;
            if (static_cast<int>(blockIdx.x) < acc + tiles) {
                seq = s;
                tile = blockIdx.x - acc;
                break;
            }
            acc += tiles;
        }
    }
    if (seq < 0) return;
    const int head = blockIdx.y;
    const int kvh = head / (nq / nkv);
    const int n_q = q_len[seq];
    const int row0 = tile * kQTile;                          // first query of this CTA within the portion
    const int rows = min(kQTile, n_q - row0);
    const int pos0 = ctx_len[seq] - n_q + row0;              // absolute position of that query
    const int last_pos = pos0 + rows - 1;
    const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int32_t* table = block_table + static_cast<size_t>(seq) * table_width;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tg = lane & 3;
    const int lm = lane >> 3, lr = lane & 7;

    auto load_tile = [&](int kt, int stage) {
        unsigned char* ks = smem + stage * STAGE_BYTES;
        unsigned char* vs = ks + kKTile * ROW_BYTES;
        const int k0 = kt * kKTile;
#pragma unroll
        for (int i = 0; i < kKTile * CHUNKS / 128; ++i) {
            const int idx = i * 128 + threadIdx.x;
            const int row = idx / CHUNKS, c = idx % CHUNKS;
            const int key = k0 + row;
            const uint32_t off = swizzled<ROW_BYTES>(row, c);
            if (key >= first_key && key <= last_pos) {
                const int page = table[key / page_size];
                const size_t src = ((static_cast<size_t>(page) * nkv + kvh) * page_size + key % page_size) * HD + c * 8;
                cp_async_16(ks + off, k_pages + src);
                cp_async_16(vs + off, v_pages + src);
            } else {
                *reinterpret_cast<uint4*>(ks + off) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vs + off) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    };

    const int kt_first = first_key / kKTile, kt_last = last_pos / kKTile;
    load_tile(kt_first, 0);

    // This warp's 16 query rows as A fragments. Rows past the portion's end repeat its last row.
    const int wr0 = warp * 16;
    const int ra = min(wr0 + g, rows - 1), rb = min(wr0 + g + 8, rows - 1);
    const int pos_a = pos0 + ra, pos_b = pos0 + rb;
    uint32_t qa[KSTEPS][4];
    {
        const __nv_bfloat16* base = q + static_cast<size_t>(q_start[seq] + row0) * q_stride + static_cast<size_t>(head) * HD;
        const __nv_bfloat16* pa = base + static_cast<size_t>(ra) * q_stride;
        const __nv_bfloat16* pb = base + static_cast<size_t>(rb) * q_stride;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            const int d = kk * 16 + 2 * tg;
            qa[kk][0] = *reinterpret_cast<const uint32_t*>(pa + d);
            qa[kk][1] = *reinterpret_cast<const uint32_t*>(pb + d);
            qa[kk][2] = *reinterpret_cast<const uint32_t*>(pa + d + 8);
            qa[kk][3] = *reinterpret_cast<const uint32_t*>(pb + d + 8);
        }
    }
    const bool warp_active = wr0 < rows;
    const int warp_last_pos = pos0 + min(wr0 + 15, rows - 1);
    const int warp_first_key = window > 0 ? max(0, pos0 + wr0 - window + 1) : 0;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int kt = kt_first; kt <= kt_last; ++kt) {
        const int stage = (kt - kt_first) & 1;
        cp_async_wait<0>();
        __syncthreads();                                  // tile kt is visible; everyone is done with the other stage
        if (kt < kt_last) load_tile(kt + 1, stage ^ 1);
        const int k0 = kt * kKTile;
        // A warp skips tiles that lie wholly after its last query or before its first query's window.
        if (!warp_active || k0 > warp_last_pos || k0 + kKTile <= warp_first_key) continue;
        const uint32_t ks_addr = smem_addr(smem + stage * STAGE_BYTES);
        const uint32_t vs_addr = ks_addr + kKTile * ROW_BYTES;

        float s[kKTile / 8][4];
#pragma unroll
        for (int nt = 0; nt < kKTile / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
            for (int kb = 0; kb < kKTile / 16; ++kb) {
                uint32_t b[4];
                ldmatrix_x4(b, ks_addr + swizzled<ROW_BYTES>(kb * 16 + (lm >> 1) * 8 + lr, kk * 2 + (lm & 1)));
                mma_bf16_16816(s[2 * kb], qa[kk], b[0], b[1]);
                mma_bf16_16816(s[2 * kb + 1], qa[kk], b[2], b[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
        // Only tiles that touch the diagonal or the window's edge need the mask.
        const int warp_first_pos = pos0 + min(wr0, rows - 1);
        const bool needs_mask = k0 + kKTile - 1 > warp_first_pos || (window > 0 && k0 <= warp_last_pos - window);
        if (needs_mask) {
#pragma unroll
            for (int nt = 0; nt < kKTile / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = k0 + nt * 8 + 2 * tg + (e & 1);
                    const int p = (e >> 1) ? pos_b : pos_a;
                    const bool ok = key <= p && (window <= 0 || key > p - window);
                    s[nt][e] = ok ? s[nt][e] * scale_log2e : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < kKTile / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[nt][e] *= scale_log2e;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
                }
        }
        float corr[2], base[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m[r], mx[r]);
            base[r] = m_new == -INFINITY ? 0.f : m_new;    // a row that has seen no key yet
            corr[r] = exp2f(m[r] - base[r]);
            m[r] = m_new;
            l[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
#pragma unroll
        for (int kb = 0; kb < kKTile / 16; ++kb) {
            uint32_t pa[4];
            float p[2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[h][e] = exp2f(s[2 * kb + h][e] - base[e >> 1]);
                    l[e >> 1] += p[h][e];
                }
            pa[0] = pack_bf16(p[0][0], p[0][1]);
            pa[1] = pack_bf16(p[0][2], p[0][3]);
            pa[2] = pack_bf16(p[1][0], p[1][1]);
            pa[3] = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
            for (int dn = 0; dn < HD / 16; ++dn) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vs_addr + swizzled<ROW_BYTES>(kb * 16 + (lm & 1) * 8 + lr, dn * 2 + (lm >> 1)));
                mma_bf16_16816(o[2 * dn], pa, b[0], b[1]);
                mma_bf16_16816(o[2 * dn + 1], pa, b[2], b[3]);
            }
        }
    }

    if (!warp_active) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    __nv_bfloat16* out_base = out + static_cast<size_t>(q_start[seq] + row0) * nq * HD + static_cast<size_t>(head) * HD;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = wr0 + g + 8 * r;
        if (row >= rows) continue;
        const float inv = 1.f / l[r];
        __nv_bfloat16* dst = out_base + static_cast<size_t>(row) * nq * HD;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * tg) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
}

template <int HD>
int launch_prefill(const __nv_bfloat16* q, int q_stride, __nv_bfloat16* out, const __nv_bfloat16* k_pages,
                   const __nv_bfloat16* v_pages, const int32_t* block_table, int table_width, const int32_t* q_start,
                   const int32_t* q_len, const int32_t* ctx_len, int num_seqs, int max_tiles, int nq, int nkv, int page_size,
                   float scale, int window, cudaStream_t stream) {
    const int smem = 2 * 2 * kKTile * HD * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(paged_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    dim3 grid(max_tiles, nq);
    stride::launch(paged_prefill_kernel<HD>, dim3(grid), dim3(128), smem, stream, q, q_stride, out, k_pages, v_pages, block_table, table_width, q_start,
                                                          q_len, ctx_len, num_seqs, nq, nkv, page_size,
                                                          scale * 1.4426950408889634f, window);
    return STRIDE_LAUNCH_STATUS();
}

}  // namespace stride

using namespace stride;

// Attention for the first `num_seqs` requests of the step, which own the first
// `tokens` rows of the flat batch. q: [tokens, q_stride]; out: [tokens, nq * hd].
// Returns -2 for sizes it does not run (head sizes other than 64 and 128); the
// caller then uses the generic kernel.
extern "C" int stride_paged_prefill_attention(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                              const int32_t* block_table, int table_width, const int32_t* q_start,
                                              const int32_t* q_len, const int32_t* ctx_len, int num_seqs, int tokens, int nq,
                                              int nkv, int hd, int page_size, float scale, int window, cudaStream_t stream) {
    if (tokens < 0 || num_seqs < 0 || nq <= 0 || nkv <= 0 || page_size <= 0 || table_width <= 0 || window < 0) return STRIDE_BAD_ARGUMENT;
    if (nq % nkv) return STRIDE_BAD_ARGUMENT;
    if ((hd != 64 && hd != 128) || nq > 65535 || q_stride % 2) return STRIDE_UNSUPPORTED;
    if (tokens == 0 || num_seqs == 0) return 0;
    const int max_tiles = (tokens + kQTile - 1) / kQTile + num_seqs;   // every request may end with a partial tile
    auto qp = static_cast<const __nv_bfloat16*>(q);
    auto op = static_cast<__nv_bfloat16*>(out);
    auto kp = static_cast<const __nv_bfloat16*>(k_pages);
    auto vp = static_cast<const __nv_bfloat16*>(v_pages);
    if (hd == 64)
        return launch_prefill<64>(qp, q_stride, op, kp, vp, block_table, table_width, q_start, q_len, ctx_len, num_seqs, max_tiles,
                                  nq, nkv, page_size, scale, window, stream);
    return launch_prefill<128>(qp, q_stride, op, kp, vp, block_table, table_width, q_start, q_len, ctx_len, num_seqs, max_tiles,
                               nq, nkv, page_size, scale, window, stream);
}
