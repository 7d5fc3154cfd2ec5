// Top-k and nucleus draws on the device, for the rows of a step that ask for them.
//
// The rule is the reference sampler's (crates/stride-backend/src/sampler.rs:88-146): logits divided by the
// temperature, a max-subtracted softmax in float32, one ranking by probability (descending, equal probabilities in
// vocabulary order), the first top_k entries, cut where the cumulated probability reaches top_p (at least one entry),
// and a walk down the kept ranking until u * kept mass is used up. A suppressed token counts as -inf.
//
// Nothing is sorted. Probabilities are not negative, so their float32 bit patterns order like the numbers, and the
// kept set is "everything above a value b, and the first r entries equal to b": b is found by a search over bit
// patterns, seven thresholds a pass (three bits of the pattern per pass over the row, eleven passes), each pass
// counting and summing what lies above every threshold. A second search of the same kind finds the value at which
// the walk ends, and a last pass the entry among equals, by vocabulary order. One CTA per row; the row's
// probabilities are written once to scratch and read from L2 afterwards. Sums are taken in an order fixed by the
// sizes alone (a thread's columns in order, a shuffle tree, the warps in order), so a draw is reproducible; they
// are not the sequential sums of a host that walks a sorted list, so a draw whose target falls within rounding of a
// boundary may differ from the host sampler's by one entry of the ranking.
#include "common.cuh"

namespace stride {
namespace ranked {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kWays = 7;                 // thresholds per pass

// Reduces kWays (count, sum) pairs over the block in a fixed order; every thread gets the result.
__device__ __forceinline__ void block_reduce(int (&count)[kWays], float (&sum)[kWays], int* s_count, float* s_sum) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            count[w] += __shfl_xor_sync(0xffffffffu, count[w], o);
            sum[w] += __shfl_xor_sync(0xffffffffu, sum[w], o);
        }
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
            s_count[warp * kWays + w] = count[w];
            s_sum[warp * kWays + w] = sum[w];
        }
    }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
        int c = 0;
        float s = 0.f;
        for (int k = 0; k < kWarps; ++k) {
            c += s_count[k * kWays + w];
            s += s_sum[k * kWays + w];
        }
        count[w] = c;
        sum[w] = s;
    }
}

__device__ __forceinline__ float block_max(float v, float* s_val) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_val[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = s_val[0];
    for (int k = 1; k < kWarps; ++k) m = fmaxf(m, s_val[k]);
    return m;
}

__device__ __forceinline__ float block_sum(float v, float* s_val) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_val[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
    for (int k = 0; k < kWarps; ++k) s += s_val[k];
    return s;
}

// Count and sum of the probabilities whose bit pattern lies strictly above each of kWays thresholds (ascending).
__device__ __forceinline__ void above(const float* __restrict__ p, int vocab, const int (&threshold)[kWays], int (&count)[kWays],
                                      float (&sum)[kWays], int* s_count, float* s_sum) {
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
        count[w] = 0;
        sum[w] = 0.f;
    }
    for (int i = threadIdx.x; i < vocab; i += kThreads) {
        const float v = __ldcg(p + i);
        const int bits = __float_as_int(v);
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
            if (bits > threshold[w]) {
                ++count[w];
                sum[w] += v;
            }
        }
    }
    block_reduce(count, sum, s_count, s_sum);
}

// The smallest bit pattern b in (lo, hi] for which `holds(count above b, sum above b)` is true, given that it is true
// at hi and false at lo (lo may be -1: every probability lies above it) and true for every pattern above the first
// that makes it true. On return count_b / sum_b are what lies above b, and count_lo what lies above b - 1.
template <typename Holds>
__device__ __forceinline__ int search(const float* __restrict__ p, int vocab, int lo, int hi, int count_lo, int count_hi, float sum_hi,
                                      Holds holds, int& count_b, float& sum_b, int& count_below, int* s_count, float* s_sum) {
    while (hi - lo > 1) {
        const long long span = static_cast<long long>(hi) - lo;
        const long long step = span / (kWays + 1) > 0 ? span / (kWays + 1) : 1;
        int threshold[kWays], count[kWays];
        float sum[kWays];
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
            const long long t = lo + step * (w + 1);
            threshold[w] = static_cast<int>(t < hi ? t : hi - 1);
        }
        above(p, vocab, threshold, count, sum, s_count, s_sum);
        int first = kWays;                    // the first threshold at which it holds
#pragma unroll
        for (int w = kWays - 1; w >= 0; --w)
            if (holds(count[w], sum[w])) first = w;
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
            if (w == first) {
                hi = threshold[w];
                count_hi = count[w];
                sum_hi = sum[w];
            }
            if (w == first - 1) {
                lo = threshold[w];
                count_lo = count[w];
            }
        }
    }
    count_b = count_hi;
    sum_b = sum_hi;
    count_below = count_lo;
    return hi;
}

__global__ void __launch_bounds__(kThreads)
sample_ranked_kernel(const float* __restrict__ logits, int vocab, long long row_stride, const float* __restrict__ temperature,
                     const float* __restrict__ uniform, const int32_t* __restrict__ suppress, const int32_t* __restrict__ top_k,
                     const float* __restrict__ top_p, int32_t* __restrict__ out, float* __restrict__ probs) {
    pdl_trigger();
    pdl_wait();
    __shared__ int s_count[kWarps * kWays];
    __shared__ float s_sum[kWarps * kWays];
    __shared__ float s_val[kWarps];
    __shared__ int s_scan[kThreads];
    const int r = blockIdx.x, tid = threadIdx.x;
    const float t = temperature[r];
    const int k_limit = top_k[r] > 0 ? top_k[r] : 0x7fffffff;
    const float p_limit = top_p[r];
    const bool nucleus = p_limit < 1.f;
    if (!(t > 0.f) || (top_k[r] <= 0 && !nucleus)) return;       // not a ranked row: the other kernel has drawn it
    const float* row = logits + static_cast<size_t>(r) * row_stride;
    float* p = probs + static_cast<size_t>(r) * vocab;
    const int banned = suppress ? suppress[r] : -1;
    const bool scaled = fabsf(t - 1.f) > 1.1920929e-07f;

    // ---- the probabilities, once
    float mine = -INFINITY;
    for (int i = tid; i < vocab; i += kThreads) {
        float v = i == banned ? -INFINITY : row[i];
        if (scaled) v = v / t;
        p[i] = v;
        mine = fmaxf(mine, v);
    }
    const float mx = block_max(mine, s_val);
    float pmax;
    if (!(mx > -INFINITY)) {                 // every logit is -inf: the uniform distribution
        pmax = 1.f / static_cast<float>(vocab);
        for (int i = tid; i < vocab; i += kThreads) p[i] = pmax;
    } else {
        float part = 0.f;
        for (int i = tid; i < vocab; i += kThreads) {
            const float e = expf(p[i] - mx);
            p[i] = e;
            part += e;
        }
        const float sum = block_sum(part, s_val);
        float top = 0.f;
        for (int i = tid; i < vocab; i += kThreads) {
            const float q = sum > 0.f ? p[i] / sum : p[i];
            p[i] = q;
            top = fmaxf(top, q);
        }
        pmax = block_max(top, s_val);
    }
    __syncthreads();                         // every thread reads other threads' columns from here on
    const int top_bits = __float_as_int(pmax);

    // ---- the value of the last kept entries: the smallest b such that what lies above b fills neither the top-k
    // budget nor the nucleus
    auto open_budget = [&](int count, float sum) { return count < k_limit && (!nucleus || sum < p_limit); };
    int b, count_b, count_below;
    float sum_b;
    {
        int threshold[kWays], count[kWays];
        float sum[kWays];
#pragma unroll
        for (int w = 0; w < kWays; ++w) threshold[w] = -1;
        above(p, vocab, threshold, count, sum, s_count, s_sum);          // everything: the whole mass in this order of summing
        if (open_budget(count[0], sum[0])) {                               // the whole vocabulary is kept
            b = -1;
            count_b = count[0];
            sum_b = sum[0];
            count_below = count[0];
        } else {
            b = search(p, vocab, -1, top_bits, vocab, 0, 0.f, open_budget, count_b, sum_b, count_below, s_count, s_sum);
        }
    }
    const float v_b = b >= 0 ? __int_as_float(b) : 0.f;
    int kept_equals = 0;                     // how many of the entries equal to v_b are kept (in vocabulary order)
    float total = sum_b;
    if (b >= 0) {
        const int equals = count_below - count_b;
        kept_equals = min(equals, k_limit - count_b);
        if (nucleus && v_b > 0.f) {
            const float need = ceilf((p_limit - sum_b) / v_b);
            if (need < static_cast<float>(kept_equals)) kept_equals = static_cast<int>(need);
        }
        kept_equals = max(kept_equals, 1);
        total = sum_b + static_cast<float>(kept_equals) * v_b;
    }

    // ---- the walk: the value at which the cumulated probability, from the top, reaches the target
    const float target = uniform[r] * total;
    int w_bits = top_bits, index_among_equals = 1;
    if (target > 0.f && isfinite(total)) {
        auto short_of_target = [&](int, float sum) { return sum < target; };
        int count_w, count_below_w;
        float sum_w;
        w_bits = search(p, vocab, b >= 0 ? b - 1 : -1, top_bits, count_below, 0, 0.f, short_of_target, count_w, sum_w, count_below_w,
                        s_count, s_sum);
        const float v_w = __int_as_float(w_bits);
        const int equals = w_bits == b ? kept_equals : count_below_w - count_w;
        const float steps = v_w > 0.f ? ceilf((target - sum_w) / v_w) : 1.f;
        index_among_equals = steps < 1.f ? 1 : (steps > static_cast<float>(equals) ? equals : static_cast<int>(steps));
        index_among_equals = max(index_among_equals, 1);
    }

    // ---- the entry: the index_among_equals-th column, in vocabulary order, whose probability is v_w
    const int chunk = (vocab + kThreads - 1) / kThreads;
    const int begin = min(tid * chunk, vocab), end = min(begin + chunk, vocab);
    int here = 0;
    for (int i = begin; i < end; ++i) here += __float_as_int(__ldcg(p + i)) == w_bits;
    s_scan[tid] = here;
    __syncthreads();
    if (tid == 0) {
        int before = 0, owner = -1, last = -1;
        for (int k = 0; k < kThreads; ++k) {
            if (s_scan[k] > 0) last = k;
            if (owner < 0 && before + s_scan[k] >= index_among_equals) {
                owner = k;
                s_count[1] = index_among_equals - before;
            }
            before += s_scan[k];
        }
        if (owner < 0) {                     // fewer equals than counted (cannot happen): the last of them
            owner = last;
            s_count[1] = last >= 0 ? s_scan[last] : 0;
        }
        s_count[0] = owner;
    }
    __syncthreads();
    if (tid == s_count[0]) {
        int left = s_count[1], pick = -1;
        for (int i = begin; i < end; ++i) {
            if (__float_as_int(__ldcg(p + i)) == w_bits) {
                pick = i;
                if (--left <= 0) break;
            }
        }
        if (pick >= 0) out[r] = pick;
    }
}

}  // namespace ranked
}  // namespace stride

extern "C" {

// Draws the rows that ask for top-k (top_k[r] > 0) or a nucleus (top_p[r] < 1) with a temperature above 0; other
// rows are left as they are (stride_sample_rows draws them). probs: [rows, vocab] float32 scratch.
int stride_sample_ranked(const float* logits, int rows, int vocab, long long row_stride, const float* temperature,
                         const float* uniform, const int32_t* suppress, const int32_t* top_k, const float* top_p, int32_t* out,
                         float* probs, long long probs_floats, cudaStream_t stream) {
    if (rows < 0 || vocab <= 0 || row_stride < vocab) return STRIDE_BAD_ARGUMENT;
    if (temperature == nullptr || uniform == nullptr || top_k == nullptr || top_p == nullptr || out == nullptr) return STRIDE_BAD_ARGUMENT;
    if (rows == 0) return 0;
    if (probs == nullptr || probs_floats < static_cast<long long>(rows) * vocab) return STRIDE_BAD_ARGUMENT;
    stride::launch(stride::ranked::sample_ranked_kernel, dim3(rows), dim3(stride::ranked::kThreads), 0, stream, logits, vocab, row_stride,
                   temperature, uniform, suppress, top_k, top_p, out, probs);
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
