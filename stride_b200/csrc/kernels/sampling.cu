// Token selection on the device from float32 logits [rows, vocab].
//
// A row with temperature 0 takes the first maximum (crates/stride-backend/src/sampler.rs:157-165).
// Otherwise the logits are divided by the temperature, a max-subtracted softmax is formed in
// float32 (sampler.rs:169-183) and the token is drawn by inverse CDF with the uniform number
// that the host's generator supplies: the first index, in vocabulary order, at which the
// running sum of probabilities reaches u * total. A suppressed token (EOS below min_tokens,
// sampler.rs:81-86) counts as -inf. Rows with a top-k or nucleus cut are drawn by
// sampling_ranked.cu (or, when the engine is told so, by the host sampler from their logits).
//
// The vocabulary is cut into segments of 4096 columns, one CTA per (segment, row), so that a
// step of a few rows still reads its logits with many SMs. A CTA keeps its segment in shared
// memory, finds the segment's first maximum and, for temperature rows, the sum of
// exp(x - segment maximum); the CTAs of a row count themselves off on a ticket and the last one
// combines the segments in vocabulary order, finds the segment in which the running sum reaches
// the target, and walks that segment in order. Every sum is taken in an order fixed by the sizes
// alone, so a draw does not depend on which CTA happens to come last.
#include "common.cuh"

namespace stride {

constexpr int kSampleThreads = 256;
constexpr int kSegment = 4096;                            // columns per CTA
constexpr int kChunk = kSegment / kSampleThreads;         // columns a thread walks in order when the pick is made
constexpr int kTicketWords = 65536;                       // one ticket per row at the start of the scratch, whatever the launch's sizes

struct BestOf {
    float v;
    int i;                                                // 0x7fffffff: nothing seen yet
};
// the larger value wins; on a tie (or when one side has seen nothing) the lower index
__device__ __forceinline__ BestOf better(BestOf a, BestOf b) {
    if (b.i == 0x7fffffff) return a;
    if (a.i == 0x7fffffff) return b;
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ BestOf block_best(BestOf mine, float* s_val, int* s_idx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        BestOf other{__shfl_xor_sync(0xffffffffu, mine.v, o), __shfl_xor_sync(0xffffffffu, mine.i, o)};
        mine = better(mine, other);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) {
        s_val[warp] = mine.v;
        s_idx[warp] = mine.i;
    }
    __syncthreads();
    BestOf all{s_val[0], s_idx[0]};
    for (int w = 1; w < kSampleThreads / 32; ++w) all = better(all, BestOf{s_val[w], s_idx[w]});
    return all;
}

// Sum over the block in a fixed order: a shuffle tree inside each warp, then the warps in order.
__device__ __forceinline__ float block_sum_ordered(float v, float* s_val) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) s_val[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < kSampleThreads / 32; ++w) total += s_val[w];
    return total;
}

// scratch: kTicketWords tickets (zero between launches; always the same words, so that launches of different sizes
// never find another launch's results where they expect zeros), then per (row, segment) the maximum, the sum and
// the index of the maximum
__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, int vocab, long long row_stride, const float* __restrict__ temperature,
                   const float* __restrict__ uniform, const int32_t* __restrict__ suppress, int32_t* __restrict__ out,
                   int* __restrict__ tickets, float* __restrict__ seg_max, float* __restrict__ seg_sum, int* __restrict__ seg_arg) {
    pdl_trigger();
    pdl_wait();
    __shared__ float buf[kSegment];
    __shared__ float s_val[kSampleThreads];
    __shared__ int s_idx[kSampleThreads];
    __shared__ int s_flag;
    const int seg = blockIdx.x, segments = gridDim.x, r = blockIdx.y, tid = threadIdx.x;
    const float* row = logits + static_cast<size_t>(r) * row_stride;
    const int banned = suppress ? suppress[r] : -1;
    const float t = temperature ? temperature[r] : 0.f;
    const bool draw = t > 0.f;
    const float inv_t = draw ? 1.f / t : 1.f;

    auto load_segment = [&](int which) {          // columns of segment `which`, scaled and masked, into buf; returns the thread's best
        const int lo = which * kSegment, n = min(kSegment, vocab - lo);
        BestOf mine{-INFINITY, 0x7fffffff};
        for (int i = tid; i < n; i += kSampleThreads) {
            const int col = lo + i;
            const float v = col == banned ? -INFINITY : row[col] * inv_t;
            buf[i] = v;
            mine = better(mine, BestOf{v, col});
        }
        return mine;
    };

    const int n_here = min(kSegment, vocab - seg * kSegment);
    const BestOf best = block_best(load_segment(seg), s_val, s_idx);
    float sum = 0.f;
    if (draw && best.v > -INFINITY) {
        float part = 0.f;
        for (int i = tid; i < n_here; i += kSampleThreads) part += expf(buf[i] - best.v);
        sum = block_sum_ordered(part, s_val);
    }
    const size_t slot = static_cast<size_t>(r) * segments + seg;
    if (tid == 0) {
        seg_max[slot] = best.v;
        seg_sum[slot] = sum;
        seg_arg[slot] = best.i;
        __threadfence();
        const int last = atomicAdd(&tickets[r], 1) == segments - 1;
        if (last) tickets[r] = 0;                 // ready for the next launch
        s_flag = last;
    }
    __syncthreads();
    if (!s_flag) return;
    __threadfence();

    // ---- the last CTA of the row: combine the segments in vocabulary order
    const size_t base = static_cast<size_t>(r) * segments;
    BestOf mine{-INFINITY, 0x7fffffff};
    for (int sgm = tid; sgm < segments; sgm += kSampleThreads) mine = better(mine, BestOf{__ldcg(seg_max + base + sgm), __ldcg(seg_arg + base + sgm)});
    const BestOf top = block_best(mine, s_val, s_idx);
    if (!draw) {
        if (tid == 0) out[r] = top.i;
        return;
    }
    if (!(top.v > -INFINITY)) {      // every logit is -inf: uniform over the vocabulary
        if (tid == 0) out[r] = min(static_cast<int>(uniform[r] * vocab), vocab - 1);
        return;
    }
    __syncthreads();
    if (tid == 0) {                  // one thread walks the segments: in order, deterministic
        float total = 0.f;
        for (int sgm = 0; sgm < segments; ++sgm) {
            const float m = __ldcg(seg_max + base + sgm);
            total += m > -INFINITY ? __ldcg(seg_sum + base + sgm) * expf(m - top.v) : 0.f;
        }
        const float target = uniform[r] * total;
        float run = 0.f;
        int owner = -1;
        for (int sgm = 0; sgm < segments; ++sgm) {
            const float m = __ldcg(seg_max + base + sgm);
            const float w = m > -INFINITY ? __ldcg(seg_sum + base + sgm) * expf(m - top.v) : 0.f;
            if (w > 0.f) {
                owner = sgm;                      // the sums are the ones of `total`, in the same order: the last one reaches the target
                if (run + w >= target) break;
                run += w;
            }
        }
        s_idx[0] = owner;
        s_val[0] = target - run;
    }
    __syncthreads();
    const int owner = s_idx[0];
    const float remaining_in_segment = s_val[0];
    __syncthreads();
    load_segment(owner);                          // its scaled logits into buf (the CTA's own segment is no longer needed)
    __syncthreads();
    const int n_owner = min(kSegment, vocab - owner * kSegment);
    // every thread sums a chunk of consecutive columns; one thread finds the chunk, its owner the column
    float chunk = 0.f;
    for (int i = tid * kChunk; i < min((tid + 1) * kChunk, n_owner); ++i) chunk += expf(buf[i] - top.v);
    s_val[tid] = chunk;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        int who = -1;
        for (int c = 0; c < kSampleThreads; ++c) {
            if (s_val[c] > 0.f) {
                who = c;
                if (run + s_val[c] >= remaining_in_segment) break;
                run += s_val[c];
            }
        }
        s_idx[0] = who;
        s_idx[1] = __float_as_int(remaining_in_segment - run);
        // every chunk's sum underflowed to zero (a target of zero among denormal weights): no thread below would
        // write the row, which would then keep the token of an earlier step; the first maximum stands in
        if (who < 0) out[r] = top.i;
    }
    __syncthreads();
    if (tid == s_idx[0]) {
        float remaining = __int_as_float(s_idx[1]);
        int pick = -1, last_positive = -1;
        for (int i = tid * kChunk; i < min((tid + 1) * kChunk, n_owner); ++i) {
            const float p = expf(buf[i] - top.v);
            if (p > 0.f) last_positive = i;
            remaining -= p;
            if (remaining <= 0.f && p > 0.f) { pick = i; break; }
        }
        if (pick < 0) pick = last_positive;
        out[r] = pick >= 0 ? owner * kSegment + pick : top.i;
    }
}

}  // namespace stride

extern "C" {

// int32 words of scratch for `rows` rows of `vocab` columns; zero when first used (the tickets at its start).
long long stride_sample_scratch_words(int rows, int vocab) {
    if (rows <= 0 || vocab <= 0) return 0;
    const long long segments = (vocab + stride::kSegment - 1) / stride::kSegment;
    return stride::kTicketWords + 3 * segments * rows;
}

int stride_sample_rows(const float* logits, int rows, int vocab, long long row_stride, const float* temperature,
                       const float* uniform, const int32_t* suppress, int32_t* out, int32_t* scratch, long long scratch_words,
                       cudaStream_t stream) {
    if (rows < 0 || vocab <= 0 || row_stride < vocab) return STRIDE_BAD_ARGUMENT;
    if (temperature != nullptr && uniform == nullptr) return STRIDE_BAD_ARGUMENT;
    if (rows == 0) return 0;
    if (rows > 65535) return STRIDE_UNSUPPORTED;
    if (scratch == nullptr || scratch_words < stride_sample_scratch_words(rows, vocab)) return STRIDE_BAD_ARGUMENT;
    const int segments = (vocab + stride::kSegment - 1) / stride::kSegment;
    int* tickets = scratch;
    float* seg_max = reinterpret_cast<float*>(scratch + stride::kTicketWords);
    float* seg_sum = seg_max + static_cast<size_t>(segments) * rows;
    int* seg_arg = scratch + stride::kTicketWords + 2 * static_cast<size_t>(segments) * rows;
    stride::launch(stride::sample_rows_kernel, dim3(segments, rows), dim3(stride::kSampleThreads), 0, stream, logits, vocab, row_stride,
                   temperature, uniform, suppress, out, tickets, seg_max, seg_sum, seg_arg);
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
