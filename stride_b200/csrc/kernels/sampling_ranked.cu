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
// the walk ends, and a last pass the entry among equals, by vocabulary order. A row belongs to a thread-block cluster
// of 1 to 8 CTAs (more CTAs a row when the step has few rows), each with its share of the columns; what a pass
// counts is added up over the cluster through distributed shared memory. The row's probabilities are written once to scratch and read from L2 afterwards. Sums of probabilities are integers (fixed
// point), so a draw is reproducible and does not depend on how the columns are spread over threads; they are not
// the sequential float32 sums of a host that walks a sorted list, so a draw whose target falls within rounding of a
// boundary may differ from the host sampler's by one entry of the ranking.
#include "common.cuh"

namespace stride {
namespace ranked {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kWays = 7;                 // thresholds per pass
constexpr int kMaxCluster = 8;

// Sums of probabilities are taken in fixed point (40 binary places): integer sums do not depend on the order of the
// additions, so the sum above a threshold is the same number however the columns were grouped when it was formed, and
// two thresholds with no probability between them always give the same answer. (Sums in float32 that were put together
// from different pieces differ in the last place, and a search led by them can settle between two probabilities.)
typedef unsigned long long Mass;
__device__ __forceinline__ Mass mass_of(float v) { return __float2ull_rz(v * 1099511627776.f); }

// What the CTAs of a cluster tell one another: per parity of the exchange, per CTA, kWays words of 16 bytes.
struct Exchange {
    float4 slot[2][kMaxCluster][kWays];
};

// Every CTA of the cluster puts `mine` into its slot of every CTA's exchange area; after the cluster's barrier
// x.slot[parity][rank] holds what CTA `rank` sent. Returns the parity to read and flips `turn` (every thread keeps
// its own copy, they all take the same path). The areas take turns, so a CTA that runs ahead into the next exchange
// does not overwrite what a slower one still reads (it cannot be two ahead: the barrier in between needs everyone).
template <int C>
__device__ __forceinline__ int exchange(Exchange& x, int& turn, const float4 (&mine)[kWays], int used) {
    const int parity = turn;
    turn ^= 1;
    const uint32_t me = cluster_rank();
    if (threadIdx.x < C) {
        for (int w = 0; w < used; ++w)
            store_cluster_f4(static_cast<uint32_t>(__cvta_generic_to_shared(&x.slot[parity][me][w])), threadIdx.x, mine[w].x, mine[w].y,
                             mine[w].z, mine[w].w);
    }
    cluster_arrive();
    cluster_wait();
    return parity;
}

// Reduces kWays (count, sum) pairs over the block, then over the cluster; every thread gets the result.
template <int C>
__device__ __forceinline__ void reduce_all(int (&count)[kWays], Mass (&sum)[kWays], int* s_count, Mass* s_sum, Exchange& x, int& turn) {
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
    if (C > 1) {
        float4 mine[kWays];
#pragma unroll
        for (int w = 0; w < kWays; ++w)
            mine[w] = make_float4(__int_as_float(count[w]), __uint_as_float(static_cast<uint32_t>(sum[w])),
                                  __uint_as_float(static_cast<uint32_t>(sum[w] >> 32)), 0.f);
        const int parity = exchange<C>(x, turn, mine, kWays);
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
            int c = 0;
            Mass s = 0;
            for (int k = 0; k < C; ++k) {
                const float4 v = x.slot[parity][k][w];
                c += __float_as_int(v.x);
                s += static_cast<Mass>(__float_as_uint(v.y)) | (static_cast<Mass>(__float_as_uint(v.z)) << 32);
            }
            count[w] = c;
            sum[w] = s;
        }
    }
}

// Maximum (or, with `add`, sum in the order warps, then CTAs) of one float per thread over the cluster.
template <int C>
__device__ __forceinline__ float reduce_float(float v, bool add, float* s_val, Exchange& x, int& turn) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, v, o);
        v = add ? v + other : fmaxf(v, other);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_val[threadIdx.x >> 5] = v;
    __syncthreads();
    float all = s_val[0];
    for (int k = 1; k < kWarps; ++k) all = add ? all + s_val[k] : fmaxf(all, s_val[k]);
    if (C > 1) {
        float4 mine[kWays];
        mine[0] = make_float4(all, 0.f, 0.f, 0.f);
        const int parity = exchange<C>(x, turn, mine, 1);
        all = x.slot[parity][0][0].x;
        for (int k = 1; k < C; ++k) all = add ? all + x.slot[parity][k][0].x : fmaxf(all, x.slot[parity][k][0].x);
    }
    return all;
}

// Shared state of a CTA that the helpers below use.
struct Shared {
    int count[kWarps * kWays];
    Mass sum[kWarps * kWays];
    float val[kWarps];
    int scan[kThreads];
    int pick[2];
    Exchange x;
};

// Count and sum of the probabilities whose bit pattern lies strictly above each of kWays thresholds (ascending, all
// in [lo, hi)). What lies above hi lies above every threshold and is known (count_hi, sum_hi); what does not lie above
// lo lies above none: only the columns in between are compared with the thresholds. A CTA of the cluster takes every
// C-th group of kThreads columns (or of kThreads packs of four).
template <int C>
__device__ __forceinline__ void above(const float* __restrict__ p, int vocab, int lo, int hi, int count_hi, Mass sum_hi,
                                      const int (&threshold)[kWays], int (&count)[kWays], Mass (&sum)[kWays], Shared& sh, int& turn) {
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
    const int first = (C > 1 ? cluster_rank() : 0) * kThreads + threadIdx.x;
    constexpr int kStride = C * kThreads;
    if ((vocab & 3) == 0) {          // rows of such a vocabulary start on 16 bytes in the scratch: 16-byte loads, several in flight
        const float4* p4 = reinterpret_cast<const float4*>(p);
        const int n4 = vocab >> 2;
        constexpr int kInFlight = C >= 4 ? 4 : 8;
        int i = first;
        for (; i + (kInFlight - 1) * kStride < n4; i += kInFlight * kStride) {
            float4 v[kInFlight];
#pragma unroll
            for (int k = 0; k < kInFlight; ++k) v[k] = __ldcg(p4 + i + k * kStride);
#pragma unroll
            for (int k = 0; k < kInFlight; ++k) {
                take(v[k].x); take(v[k].y); take(v[k].z); take(v[k].w);
            }
        }
        for (; i < n4; i += kStride) {
            const float4 a = __ldcg(p4 + i);
            take(a.x); take(a.y); take(a.z); take(a.w);
        }
    } else {
        for (int i = first; i < vocab; i += kStride) take(__ldcg(p + i));
    }
    reduce_all<C>(count, sum, sh.count, sh.sum, sh.x, turn);
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
        count[w] += count_hi;
        sum[w] = sum_hi + sum[w];
    }
}

// The smallest bit pattern b in (lo, hi] for which `holds(count above b, sum above b)` is true, given that it is true
// at hi and false at lo (lo may be -1: every probability lies above it) and true for every pattern above the first
// that makes it true. On return count_b / sum_b are what lies above b, and count_below what lies above b - 1.
template <int C, typename Holds>
__device__ __forceinline__ int search(const float* __restrict__ p, int vocab, int lo, int hi, int count_lo, int count_hi, Mass sum_hi,
                                      Holds holds, int& count_b, Mass& sum_b, int& count_below, Shared& sh, int& turn) {
    // The first pass puts its thresholds a factor of 16 apart below hi (the largest probability): what a draw keeps
    // mostly lies within a few such factors of the top, and every later pass then compares only the few columns between
    // the new bounds with its thresholds. The passes after it cut the range of bit patterns into equal parts.
    bool by_factors = true;
    while (hi - lo > 1) {
        const long long span = static_cast<long long>(hi) - lo;
        const long long step = span / (kWays + 1) > 0 ? span / (kWays + 1) : 1;
        int threshold[kWays], count[kWays];
        Mass sum[kWays];
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
            long long t = lo + step * (w + 1);
            if (by_factors) {
                t = static_cast<long long>(hi) - (static_cast<long long>(kWays - w) << 25);      // 4 steps of the exponent
                if (t < lo) t = lo;
            }
            threshold[w] = static_cast<int>(t < hi ? t : hi - 1);
        }
        by_factors = false;
        above<C>(p, vocab, lo, hi, count_hi, sum_hi, threshold, count, sum, sh, turn);
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

template <int C>
__global__ void __launch_bounds__(kThreads)
sample_ranked_kernel(const float* __restrict__ logits, int vocab, long long row_stride, const float* __restrict__ temperature,
                     const float* __restrict__ uniform, const int32_t* __restrict__ suppress, const int32_t* __restrict__ top_k,
                     const float* __restrict__ top_p, int32_t* __restrict__ out, float* __restrict__ probs) {
    pdl_trigger();
    pdl_wait();
    __shared__ Shared sh;
    const int r = blockIdx.x, tid = threadIdx.x;
    const int rank = C > 1 ? static_cast<int>(cluster_rank()) : 0;
    int turn = 0;
    const float t = temperature[r];
    const int k_limit = top_k[r] > 0 ? top_k[r] : 0x7fffffff;
    const float p_limit = top_p[r];
    const bool nucleus = p_limit < 1.f;
    if (!(t > 0.f) || (top_k[r] <= 0 && !nucleus)) return;       // not a ranked row (the whole cluster leaves): the other kernel has drawn it
    const float* row = logits + static_cast<size_t>(r) * row_stride;
    float* p = probs + static_cast<size_t>(r) * vocab;
    const int banned = suppress ? suppress[r] : -1;
    const bool scaled = fabsf(t - 1.f) > 1.1920929e-07f;

    // ---- the probabilities, once. Each thread owns the same columns in every pass (packs of four where the row and
    // the scratch allow 16-byte accesses).
    const bool wide = (vocab & 3) == 0 && (row_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
    const int groups = wide ? vocab >> 2 : vocab;
    const int first = rank * kThreads + tid;
    constexpr int kStride = C * kThreads;
    auto scaled_logit = [&](int i, float v) {
        v = i == banned ? -INFINITY : v;
        return scaled ? v / t : v;
    };
    float mine = -INFINITY;
    for (int gi = first; gi < groups; gi += kStride) {
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
    const float mx = reduce_float<C>(mine, false, sh.val, sh.x, turn);
    float pmax;
    if (!(mx > -INFINITY)) {                 // every logit is -inf: the uniform distribution
        pmax = 1.f / static_cast<float>(vocab);
        for (int i = first; i < vocab; i += kStride) p[i] = pmax;
    } else {
        // the sum of the exponentials in fixed point too (they are at most 1 each): it does not depend on how the
        // columns are spread over threads and CTAs, so neither do the probabilities
        int none[kWays];
        Mass part[kWays];
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
            none[w] = 0;
            part[w] = 0;
        }
        for (int gi = first; gi < groups; gi += kStride) {
            if (wide) {
                float4 v = reinterpret_cast<float4*>(p)[gi];
                v.x = expf(v.x - mx); v.y = expf(v.y - mx); v.z = expf(v.z - mx); v.w = expf(v.w - mx);
                reinterpret_cast<float4*>(p)[gi] = v;
                part[0] += (mass_of(v.x) + mass_of(v.y)) + (mass_of(v.z) + mass_of(v.w));
            } else {
                const float e = expf(p[gi] - mx);
                p[gi] = e;
                part[0] += mass_of(e);
            }
        }
        reduce_all<C>(none, part, sh.count, sh.sum, sh.x, turn);
        const float sum = __ull2float_rn(part[0]) * (1.f / 1099511627776.f);
        float top = 0.f;
        for (int gi = first; gi < groups; gi += kStride) {
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
        pmax = reduce_float<C>(top, false, sh.val, sh.x, turn);
    }
    // Threads read other threads' columns from here on (the last pass also other CTAs'); the reductions above and the
    // barrier below order the writes before those reads.
    if (C > 1) {
        cluster_arrive();
        cluster_wait();
    } else {
        __syncthreads();
    }
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
        above<C>(p, vocab, -1, 0x7fffffff, 0, 0, threshold, count, sum, sh, turn);      // everything: the whole mass
        if (open_budget(count[0], sum[0])) {                               // the whole vocabulary is kept
            b = -1;
            count_b = count[0];
            sum_b = sum[0];
            count_below = count[0];
        } else {
            b = search<C>(p, vocab, -1, top_bits, vocab, 0, 0, open_budget, count_b, sum_b, count_below, sh, turn);
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
        w_bits = search<C>(p, vocab, b >= 0 ? b - 1 : -1, top_bits, count_below, 0, 0, short_of_target, count_w, sum_w, count_below_w, sh, turn);
        const Mass m_w = mass_of(__int_as_float(w_bits));
        const int equals = w_bits == b ? kept_equals : count_below_w - count_w;
        const Mass steps = m_w > 0 ? (target - sum_w + m_w - 1) / m_w : 1;
        index_among_equals = steps < 1 ? 1 : (steps > static_cast<Mass>(equals) ? equals : static_cast<int>(steps));
        index_among_equals = max(index_among_equals, 1);
    }

    // ---- the entry: the index_among_equals-th column, in vocabulary order, whose probability has the pattern w_bits.
    // Here a thread takes consecutive columns (thread `rank * kThreads + tid` of C * kThreads the chunk of that number).
    const int chunk = (vocab + kStride - 1) / kStride;
    const int begin = min(first * chunk, vocab), end = min(begin + chunk, vocab);
    int here = 0;
    for (int i = begin; i < end; ++i) here += __float_as_int(__ldcg(p + i)) == w_bits;
    sh.scan[tid] = here;
    __syncthreads();
    int wanted = index_among_equals;         // counted from this CTA's first column on
    if (C > 1) {
        if (tid == 0) {
            int mine_total = 0;
            for (int k = 0; k < kThreads; ++k) mine_total += sh.scan[k];
            sh.pick[0] = mine_total;
        }
        __syncthreads();
        float4 tell[kWays];
        tell[0] = make_float4(__int_as_float(sh.pick[0]), 0.f, 0.f, 0.f);
        const int parity = exchange<C>(sh.x, turn, tell, 1);
        for (int k = 0; k < rank; ++k) wanted -= __float_as_int(sh.x.slot[parity][k][0].x);
    }
    if (tid == 0) {
        int before = 0, owner = -1;
        for (int k = 0; k < kThreads && wanted >= 1; ++k) {
            if (before + sh.scan[k] >= wanted) {
                owner = k;
                sh.pick[1] = wanted - before;
                break;
            }
            before += sh.scan[k];
        }
        sh.pick[0] = owner;                  // -1: the entry lies in another CTA's columns
    }
    __syncthreads();
    if (tid == sh.pick[0]) {
        int left = sh.pick[1];
        for (int i = begin; i < end; ++i) {
            if (__float_as_int(__ldcg(p + i)) == w_bits && --left == 0) {
                out[r] = i;
                break;
            }
        }
    }
}

}  // namespace ranked
}  // namespace stride

extern "C" {

// Draws the rows that ask for top-k (top_k[r] > 0) or a nucleus (top_p[r] < 1) with a temperature above 0; other
// rows are left as they are (stride_sample_rows draws them). probs: [rows, vocab] float32 scratch. A row gets a
// cluster of 8, 4, 2 or 1 CTAs, the more the fewer rows there are.
int stride_sample_ranked(const float* logits, int rows, int vocab, long long row_stride, const float* temperature,
                         const float* uniform, const int32_t* suppress, const int32_t* top_k, const float* top_p, int32_t* out,
                         float* probs, long long probs_floats, cudaStream_t stream) {
    using namespace stride::ranked;
    if (rows < 0 || vocab <= 0 || row_stride < vocab) return STRIDE_BAD_ARGUMENT;
    if (temperature == nullptr || uniform == nullptr || top_k == nullptr || top_p == nullptr || out == nullptr) return STRIDE_BAD_ARGUMENT;
    if (rows == 0) return 0;
    if (probs == nullptr || probs_floats < static_cast<long long>(rows) * vocab) return STRIDE_BAD_ARGUMENT;
    const dim3 block(kThreads);
#define STRIDE_RANKED(C)                                                                                                          \
    stride::launch_clusters(sample_ranked_kernel<C>, dim3(rows, 1, C), block, 0, stream, C, logits, vocab, row_stride, temperature, uniform, \
                            suppress, top_k, top_p, out, probs)
    if (rows <= 18) STRIDE_RANKED(8);
    else if (rows <= 37) STRIDE_RANKED(4);
    else if (rows <= 74) STRIDE_RANKED(2);
    else stride::launch(sample_ranked_kernel<1>, dim3(rows), block, 0, stream, logits, vocab, row_stride, temperature, uniform, suppress, top_k,
                        top_p, out, probs);
#undef STRIDE_RANKED
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
