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
// probabilities are written once to scratch and read from L2 afterwards. Sums of probabilities are integers (fixed
// point), so a draw is reproducible and does not depend on how the columns are spread over threads; they are not
// the sequential float32 sums of a host that walks a sorted list, so a draw whose target falls within rounding of a
// boundary may differ from the host sampler's by one entry of the ranking.
#include "common.cuh"

namespace stride {
namespace ranked {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kWays = 7;                 // thresholds per pass

// Sums of probabilities are taken in fixed point (40 binary places): integer sums do not depend on the order of the
// additions, so the sum above a threshold is the same number however the columns were grouped when it was formed, and
// two thresholds with no probability between them always give the same answer. (Sums in float32 that were put together
// from different pieces differ in the last place, and a search led by them can settle between two probabilities.)
typedef unsigned long long Mass;
__device__ __forceinline__ Mass mass_of(float v) { return __float2ull_rz(v * 1099511627776.f); }

// Reduces kWays (count, sum) pairs over the block in a fixed order; every thread gets the result.
__device__ __forceinline__ void block_reduce(int (&count)[kWays], Mass (&sum)[kWays], int* s_count, Mass* s_sum) {
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
        Mass s = 0;
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

// Count and sum of the probabilities whose bit pattern lies strictly above each of kWays thresholds (ascending, all
// in [lo, hi)). What lies above hi lies above every threshold and is known (count_hi, sum_hi); what does not lie above
// lo lies above none: only the columns in between are compared with the thresholds.
__device__ __forceinline__ void above(const float* __restrict__ p, int vocab, int lo, int hi, int count_hi, Mass sum_hi,
                                      const int (&threshold)[kWays], int (&count)[kWays], Mass (&sum)[kWays], int* s_count, Mass* s_sum) {
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
        count[w] = 0;
        sum[w] = 0;
    }
    auto take = [&](float v) {
        const int bits = __float_as_int(v);
        if (bits > lo && bits <= hi) {
            const Mass m = mass_of(v);
#pragma unroll
            for (int w = 0; w < kWays; ++w) {
                if (bits > threshold[w]) {
                    ++count[w];
                    sum[w] += m;
                }
            }
        }
    };
    // The order in which a thread adds its columns is fixed by the sizes alone. Rows of a vocabulary that is a multiple
    // of 4 start on 16 bytes (the scratch does): 16-byte loads, eight in flight.
    if ((vocab & 3) == 0) {
        const float4* p4 = reinterpret_cast<const float4*>(p);
        const int n4 = vocab >> 2;
        constexpr int kInFlight = 8;
        int i = threadIdx.x;
        for (; i + (kInFlight - 1) * kThreads < n4; i += kInFlight * kThreads) {
            float4 v[kInFlight];
#pragma unroll
            for (int k = 0; k < kInFlight; ++k) v[k] = __ldcg(p4 + i + k * kThreads);
#pragma unroll
            for (int k = 0; k < kInFlight; ++k) {
                take(v[k].x); take(v[k].y); take(v[k].z); take(v[k].w);
            }
        }
        for (; i < n4; i += kThreads) {
            const float4 a = __ldcg(p4 + i);
            take(a.x); take(a.y); take(a.z); take(a.w);
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += kThreads) take(__ldcg(p + i));
    }
    block_reduce(count, sum, s_count, s_sum);
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
        count[w] += count_hi;
        sum[w] = sum_hi + sum[w];
    }
}

// The smallest bit pattern b in (lo, hi] for which `holds(count above b, sum above b)` is true, given that it is true
// at hi and false at lo (lo may be -1: every probability lies above it) and true for every pattern above the first
// that makes it true. On return count_b / sum_b are what lies above b, and count_lo what lies above b - 1.
template <typename Holds>
__device__ __forceinline__ int search(const float* __restrict__ p, int vocab, int lo, int hi, int count_lo, int count_hi, Mass sum_hi,
                                      Holds holds, int& count_b, Mass& sum_b, int& count_below, int* s_count, Mass* s_sum) {
    while (hi - lo > 1) {
        const long long span = static_cast<long long>(hi) - lo;
        const long long step = span / (kWays + 1) > 0 ? span / (kWays + 1) : 1;
        int threshold[kWays], count[kWays];
        Mass sum[kWays];
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
            const long long t = lo + step * (w + 1);
            threshold[w] = static_cast<int>(t < hi ? t : hi - 1);
        }
        above(p, vocab, lo, hi, count_hi, sum_hi, threshold, count, sum, s_count, s_sum);
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
    __shared__ Mass s_sum[kWarps * kWays];
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

    // ---- the probabilities, once. Each thread owns the same columns in every pass (groups of four where the row and
    // the scratch allow 16-byte accesses).
    const bool wide = (vocab & 3) == 0 && (row_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
    const int groups = wide ? vocab >> 2 : vocab;
    auto scaled_logit = [&](int i, float v) {
        v = i == banned ? -INFINITY : v;
        return scaled ? v / t : v;
    };
    float mine = -INFINITY;
    for (int gi = tid; gi < groups; gi += kThreads) {
        if (wide) {
            float4 v = reinterpret_cast<const float4*>(row)[gi];
            v.x = scaled_logit(4 * gi, v.x); v.y = scaled_logit(4 * gi + 1, v.y); v.z = scaled_logit(4 * gi + 2, v.z); v.w = scaled_logit(4 * gi + 3, v.w);
            reinterpret_cast<float4*>(p)[gi] = v;
            mine = fmaxf(fmaxf(mine, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
        } else {
            const float v = scaled_logit(gi, row[gi]);
            p[gi] = v;
            mine = fmaxf(mine, v);
        }
    }
    const float mx = block_max(mine, s_val);
    float pmax;
    if (!(mx > -INFINITY)) {                 // every logit is -inf: the uniform distribution
        pmax = 1.f / static_cast<float>(vocab);
        for (int i = tid; i < vocab; i += kThreads) p[i] = pmax;
    } else {
        float part = 0.f;
        for (int gi = tid; gi < groups; gi += kThreads) {
            if (wide) {
                float4 v = reinterpret_cast<float4*>(p)[gi];
                v.x = expf(v.x - mx); v.y = expf(v.y - mx); v.z = expf(v.z - mx); v.w = expf(v.w - mx);
                reinterpret_cast<float4*>(p)[gi] = v;
                part += (v.x + v.y) + (v.z + v.w);
            } else {
                const float e = expf(p[gi] - mx);
                p[gi] = e;
                part += e;
            }
        }
        const float sum = block_sum(part, s_val);
        float top = 0.f;
        for (int gi = tid; gi < groups; gi += kThreads) {
            if (wide) {
                float4 v = reinterpret_cast<float4*>(p)[gi];
                if (sum > 0.f) { v.x /= sum; v.y /= sum; v.z /= sum; v.w /= sum; }
                reinterpret_cast<float4*>(p)[gi] = v;
                top = fmaxf(fmaxf(top, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
            } else {
                const float q = sum > 0.f ? p[gi] / sum : p[gi];
                p[gi] = q;
                top = fmaxf(top, q);
            }
        }
        pmax = block_max(top, s_val);
    }
    __syncthreads();                         // every thread reads other threads' columns from here on
    const int top_bits = __float_as_int(pmax);

    // ---- the value of the last kept entries: the smallest b such that what lies above b fills neither the top-k
    // budget nor the nucleus
    const Mass p_mass = nucleus ? mass_of(p_limit) : ~Mass(0);
    auto open_budget = [&](int count, Mass sum) { return count < k_limit && sum < p_mass; };
    int b, count_b, count_below;
    Mass sum_b;
    {
        int threshold[kWays], count[kWays];
        Mass sum[kWays];
#pragma unroll
        for (int w = 0; w < kWays; ++w) threshold[w] = -1;
        above(p, vocab, -1, 0x7fffffff, 0, 0, threshold, count, sum, s_count, s_sum);      // everything: the whole mass
        if (open_budget(count[0], sum[0])) {                               // the whole vocabulary is kept
            b = -1;
            count_b = count[0];
            sum_b = sum[0];
            count_below = count[0];
        } else {
            b = search(p, vocab, -1, top_bits, vocab, 0, 0, open_budget, count_b, sum_b, count_below, s_count, s_sum);
        }
    }
    const Mass m_b = b >= 0 ? mass_of(__int_as_float(b)) : 0;
    int kept_equals = 0;                     // how many of the entries equal to b's value are kept (in vocabulary order)
    Mass total = sum_b;
    if (b >= 0) {
        const int equals = count_below - count_b;
        kept_equals = min(equals, k_limit - count_b);
        if (nucleus && m_b > 0) {            // the fewest that bring the cumulated mass to top_p
            const Mass need = (p_mass - sum_b + m_b - 1) / m_b;
            if (need < static_cast<Mass>(kept_equals)) kept_equals = static_cast<int>(need);
        }
        kept_equals = max(kept_equals, 1);
        total = sum_b + static_cast<Mass>(kept_equals) * m_b;
    }

    // ---- the walk: the value at which the cumulated probability, from the top, reaches the target u * total
    const Mass target = static_cast<Mass>(static_cast<double>(uniform[r]) * static_cast<double>(total));
    int w_bits = top_bits, index_among_equals = 1;
    if (target > 0) {
        auto short_of_target = [&](int, Mass sum) { return sum < target; };
        int count_w, count_below_w;
        Mass sum_w;
        w_bits = search(p, vocab, b >= 0 ? b - 1 : -1, top_bits, count_below, 0, 0, short_of_target, count_w, sum_w, count_below_w,
                        s_count, s_sum);
        const Mass m_w = mass_of(__int_as_float(w_bits));
        const int equals = w_bits == b ? kept_equals : count_below_w - count_w;
        const Mass steps = m_w > 0 ? (target - sum_w + m_w - 1) / m_w : 1;
        index_among_equals = steps < 1 ? 1 : (steps > static_cast<Mass>(equals) ? equals : static_cast<int>(steps));
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
