// Top-k and nucleus draws on the device, for the rows of a step that ask for them.
//
// The rule is the reference sampler's (crates/stride-backend/src/sampler.rs:88-146): logits divided by the
// temperature, a max-subtracted softmax in float32, one ranking by probability (descending, equal probabilities in
// vocabulary order), the first top_k entries, cut where the cumulated probability reaches top_p (at least one entry),
// and a walk down the kept ranking until u * kept mass is used up. A suppressed token counts as -inf.
//
// Nothing is sorted. Probabilities are not negative, so their float32 bit patterns order like the numbers, and the
// kept set is "everything above a value b, and the first r entries equal to b": b is found by a search over bit
// patterns, seven thresholds a pass (count and mass of what lies above each): the first pass puts them a factor of 16
// apart below the largest probability, the later ones cut the remaining range of patterns into eight parts. A second
// search of the same kind finds the value at which the walk ends, and a last step the entry among equals, by
// vocabulary order. A row belongs to a thread-block cluster of 1 to 8 CTAs (more CTAs a row when the step has few
// rows), each with its share of the columns; what a pass counts is added up over the cluster through distributed
// shared memory. The row's probabilities are written once to scratch and read from L2 afterwards; the first pass of
// the search also collects the columns within 2^-16 of the largest probability in shared memory, and when the last
// kept value lies among them (peaked rows), every later pass reads that list instead of the row (and when the lists of
// a cluster fit into one, its first CTA takes them all and finishes the draw alone). Sums of probabilities
// are integers (fixed point), so a draw is reproducible and does not depend on how the columns are spread over threads
// and CTAs; they are not the sequential float32 sums of a host that walks a sorted list, so a draw whose target
// falls within rounding of a boundary may differ from the host sampler's by one entry of the ranking.
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

// A column that may matter to the draw: its probability and its number in the vocabulary.
struct Candidate {
    float v;
    int i;
};

// Shared state of a CTA that the helpers below use.
struct Shared {
    int count[kWarps * kWays];
    Mass sum[kWarps * kWays];
    float val[kWarps];
    int scan[kThreads];
    int pick[2];
    int listed;                          // candidates that asked for a place in the list (more than its capacity: the list is not used)
    Exchange x;
};

// Where a pass finds the row: in global memory (this CTA takes every C-th group of kThreads columns, or of kThreads
// packs of four), or, once the columns that can still matter were collected, in the CTA's list in shared memory.
struct Row {
    const float* p;                      // [vocab] probabilities
    int vocab;
    const Candidate* list;               // the CTA's candidates, or null
    int listed;
};

// Calls take(probability, column) for every column of the row that this CTA is in charge of.
template <int C, typename Take>
__device__ __forceinline__ void for_columns(const Row& row, Take take) {
    if (row.list != nullptr) {
        for (int k = threadIdx.x; k < row.listed; k += kThreads) take(row.list[k].v, row.list[k].i);
        return;
    }
    const int first = (C > 1 ? cluster_rank() : 0) * kThreads + threadIdx.x;
    constexpr int kStride = C * kThreads;
    if ((row.vocab & 3) == 0) {          // rows of such a vocabulary start on 16 bytes in the scratch: 16-byte loads, several in flight
        const float4* p4 = reinterpret_cast<const float4*>(row.p);
        const int n4 = row.vocab >> 2;
        constexpr int kInFlight = C >= 4 ? 4 : 8;
        int i = first;
        for (; i + (kInFlight - 1) * kStride < n4; i += kInFlight * kStride) {
            float4 v[kInFlight];
#pragma unroll
            for (int k = 0; k < kInFlight; ++k) v[k] = __ldcg(p4 + i + k * kStride);
#pragma unroll
            for (int k = 0; k < kInFlight; ++k) {
                const int col = 4 * (i + k * kStride);
                take(v[k].x, col); take(v[k].y, col + 1); take(v[k].z, col + 2); take(v[k].w, col + 3);
            }
        }
        for (; i < n4; i += kStride) {
            const float4 a = __ldcg(p4 + i);
            take(a.x, 4 * i); take(a.y, 4 * i + 1); take(a.z, 4 * i + 2); take(a.w, 4 * i + 3);
        }
    } else {
        for (int i = first; i < row.vocab; i += kStride) take(__ldcg(row.p + i), i);
    }
}

// Count and sum of the probabilities whose bit pattern lies strictly above each of kWays thresholds (ascending, all
// in [lo, hi)). What lies above hi lies above every threshold and is known (count_hi, sum_hi); what does not lie above
// lo lies above none: only the columns in between are compared with the thresholds. With `collect_above` >= -1 the
// pass also puts every column above that pattern into `collect` (as far as it has room; sh.listed counts them all).
template <int C>
__device__ __forceinline__ void above(const Row& row, int lo, int hi, int count_hi, Mass sum_hi, const int (&threshold)[kWays],
                                      int (&count)[kWays], Mass (&sum)[kWays], Shared& sh, int& turn, Candidate* collect = nullptr,
                                      int capacity = 0, int collect_above = 0x7fffffff) {
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
        count[w] = 0;
        sum[w] = 0;
    }
    for_columns<C>(row, [&](float v, int col) {
        const int bits = __float_as_int(v);
        if (collect != nullptr && bits > collect_above) {
            const int place = atomicAdd(&sh.listed, 1);
            if (place < capacity) collect[place] = Candidate{v, col};
        }
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
    });
    reduce_all<C>(count, sum, sh.count, sh.sum, sh.x, turn);
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
        count[w] += count_hi;
        sum[w] = sum_hi + sum[w];
    }
}

// One step of a search: given what lies above each threshold, the first threshold at which `holds` is true becomes
// the new hi and the one before it the new lo.
template <typename Holds>
__device__ __forceinline__ void narrow(const int (&threshold)[kWays], const int (&count)[kWays], const Mass (&sum)[kWays], Holds holds,
                                       int& lo, int& hi, int& count_lo, int& count_hi, Mass& sum_hi) {
    int first = kWays;
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

// Thresholds a factor of 16 apart below hi (4 steps of the exponent each), none below lo: the first pass of a
// search. What a draw keeps mostly lies within a few such factors of the largest probability.
__device__ __forceinline__ void thresholds_by_factors(int lo, int hi, int (&threshold)[kWays]) {
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
        long long t = static_cast<long long>(hi) - (static_cast<long long>(kWays - w) << 25);
        if (t < lo) t = lo;
        threshold[w] = static_cast<int>(t < hi ? t : hi - 1);
    }
}

// The smallest bit pattern b in (lo, hi] for which `holds(count above b, sum above b)` is true, given that it is true
// at hi and false at lo (lo may be -1: every probability lies above it) and true for every pattern above the first
// that makes it true. On return count_b / sum_b are what lies above b, and count_below what lies above b - 1. The
// first pass goes by factors (unless the caller has made it already), the others cut the range of bit patterns into
// equal parts.
template <int C, typename Holds>
__device__ __forceinline__ int search(const Row& row, int lo, int hi, int count_lo, int count_hi, Mass sum_hi, bool by_factors, Holds holds,
                                      int& count_b, Mass& sum_b, int& count_below, Shared& sh, int& turn) {
    while (hi - lo > 1) {
        int threshold[kWays], count[kWays];
        Mass sum[kWays];
        if (by_factors) {
            thresholds_by_factors(lo, hi, threshold);
        } else {
            const long long span = static_cast<long long>(hi) - lo;
            const long long step = span / (kWays + 1) > 0 ? span / (kWays + 1) : 1;
#pragma unroll
            for (int w = 0; w < kWays; ++w) {
                const long long t = lo + step * (w + 1);
                threshold[w] = static_cast<int>(t < hi ? t : hi - 1);
            }
        }
        by_factors = false;
        above<C>(row, lo, hi, count_hi, sum_hi, threshold, count, sum, sh, turn);
        narrow(threshold, count, sum, holds, lo, hi, count_lo, count_hi, sum_hi);
    }
    count_b = count_hi;
    sum_b = sum_hi;
    count_below = count_lo;
    return hi;
}

// What a draw needs besides the row.
struct Draw {
    int vocab, k_limit, top_bits;
    bool nucleus;
    Mass p_mass;
    float u;
    int32_t* out;
    const float* p;
};

// The rest of a draw once the first pass has narrowed the last kept value to (lo, hi] (or found that the whole
// vocabulary is kept): by the CC CTAs that still take part (`rank` among them).
template <int CC, typename Budget>
__device__ __forceinline__ void finish(const Row& row, const Draw& d, bool keep_all, int lo, int hi, int count_lo, int count_hi, Mass sum_hi,
                                       Mass whole, Budget open_budget, int rank, Shared& sh, int& turn) {
    const int tid = threadIdx.x;
    const float* p = d.p;
    int b = -1, count_b = d.vocab, count_below = d.vocab;
    Mass sum_b = whole;
    if (!keep_all) b = search<CC>(row, lo, hi, count_lo, count_hi, sum_hi, false, open_budget, count_b, sum_b, count_below, sh, turn);
    const Mass m_b = b >= 0 ? mass_of(__int_as_float(b)) : 0;
    int kept_equals = 0;                     // how many of the entries equal to b's value are kept (in vocabulary order)
    Mass total = sum_b;
    if (b >= 0) {
        const int equals = count_below - count_b;
        kept_equals = min(equals, d.k_limit - count_b);
        if (d.nucleus && m_b > 0) {            // the fewest that bring the cumulated mass to top_p
            const Mass need = (d.p_mass - sum_b + m_b - 1) / m_b;
            if (need < static_cast<Mass>(kept_equals)) kept_equals = static_cast<int>(need);
        }
        kept_equals = max(kept_equals, 1);
        total = sum_b + static_cast<Mass>(kept_equals) * m_b;
    }

    // ---- the walk: the value at which the cumulated probability, from the top, reaches the target u * total
    const Mass target = static_cast<Mass>(static_cast<double>(d.u) * static_cast<double>(total));
    int w_bits = d.top_bits, index_among_equals = 1;
    if (target > 0) {
        auto short_of_target = [&](int, Mass sum_above) { return sum_above < target; };
        int count_w, count_below_w;
        Mass sum_w;
        w_bits = search<CC>(row, b >= 0 ? b - 1 : -1, d.top_bits, count_below, 0, 0, true, short_of_target, count_w, sum_w, count_below_w, sh, turn);
        const Mass m_w = mass_of(__int_as_float(w_bits));
        const int equals = w_bits == b ? kept_equals : count_below_w - count_w;
        const Mass steps = m_w > 0 ? (target - sum_w + m_w - 1) / m_w : 1;
        index_among_equals = steps < 1 ? 1 : (steps > static_cast<Mass>(equals) ? equals : static_cast<int>(steps));
        index_among_equals = max(index_among_equals, 1);
    }

    // ---- the entry: the index_among_equals-th column, in vocabulary order, whose probability has the pattern w_bits
    if (row.list != nullptr) {
        // from the lists: the smallest column number that has index_among_equals such columns at or below it
        int lo = -1, hi = d.vocab - 1;
        while (hi - lo > 1) {
            const int step = (hi - lo) / (kWays + 1) > 0 ? (hi - lo) / (kWays + 1) : 1;
            int threshold[kWays], count[kWays];
            Mass unused[kWays];
#pragma unroll
            for (int w = 0; w < kWays; ++w) {
                threshold[w] = min(lo + step * (w + 1), hi - 1);
                count[w] = 0;
                unused[w] = 0;
            }
            for_columns<CC>(row, [&](float v, int col) {
                if (__float_as_int(v) == w_bits) {
#pragma unroll
                    for (int w = 0; w < kWays; ++w) count[w] += col <= threshold[w];
                }
            });
            reduce_all<CC>(count, unused, sh.count, sh.sum, sh.x, turn);
            int first_enough = kWays;
#pragma unroll
            for (int w = kWays - 1; w >= 0; --w)
                if (count[w] >= index_among_equals) first_enough = w;
            if (first_enough < kWays) hi = threshold[first_enough];
            if (first_enough > 0) lo = threshold[first_enough - 1];
        }
        if (rank == 0 && tid == 0) *d.out = hi;
        return;
    }
    // from the row: here a thread takes consecutive columns (thread `rank * kThreads + tid` of CC * kThreads the chunk of that number)
    constexpr int kStride = CC * kThreads;
    const int first = rank * kThreads + tid;
    const int chunk = (d.vocab + kStride - 1) / kStride;
    const int begin = min(first * chunk, d.vocab), end = min(begin + chunk, d.vocab);
    int here = 0;
    for (int i = begin; i < end; ++i) here += __float_as_int(__ldcg(p + i)) == w_bits;
    sh.scan[tid] = here;
    __syncthreads();
    int wanted = index_among_equals;         // counted from this CTA's first column on
    if (CC > 1) {
        if (tid == 0) {
            int mine_total = 0;
            for (int k = 0; k < kThreads; ++k) mine_total += sh.scan[k];
            sh.pick[0] = mine_total;
        }
        __syncthreads();
        float4 tell[kWays];
        tell[0] = make_float4(__int_as_float(sh.pick[0]), 0.f, 0.f, 0.f);
        const int parity = exchange<CC>(sh.x, turn, tell, 1);
        for (int k = 0; k < rank; ++k) wanted -= __float_as_int(sh.x.slot[parity][k][0].x);
        __syncthreads();
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
                *d.out = i;
                break;
            }
        }
    }
}

template <int C>
__global__ void __launch_bounds__(kThreads)
sample_ranked_kernel(const float* __restrict__ logits, int vocab, long long row_stride, const float* __restrict__ temperature,
                     const float* __restrict__ uniform, const int32_t* __restrict__ suppress, const int32_t* __restrict__ top_k,
                     const float* __restrict__ top_p, int32_t* __restrict__ out, float* __restrict__ probs, int capacity) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char dynamic[];
    Candidate* list = reinterpret_cast<Candidate*>(dynamic);
    __shared__ Shared sh;
    const int r = blockIdx.x, tid = threadIdx.x;
    const int rank = C > 1 ? static_cast<int>(cluster_rank()) : 0;
    int turn = 0;
    const float t = temperature[r];
    const int k_limit = top_k[r] > 0 ? top_k[r] : 0x7fffffff;
    const float p_limit = top_p[r];
    const bool nucleus = p_limit < 1.f;
    if (!(t > 0.f) || (top_k[r] <= 0 && !nucleus)) return;       // not a ranked row (the whole cluster leaves): the other kernel has drawn it
    const float* logit_row = logits + static_cast<size_t>(r) * row_stride;
    float* p = probs + static_cast<size_t>(r) * vocab;
    const int banned = suppress ? suppress[r] : -1;
    const bool scaled = fabsf(t - 1.f) > 1.1920929e-07f;

    // ---- the probabilities: the maximum, the sum of the exponentials, then each probability, written once. Each pass
    // reads the logits (packs of four where they allow 16-byte accesses); a thread has the same columns in every pass.
    const bool wide = (vocab & 3) == 0 && (row_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
    const int groups = wide ? vocab >> 2 : vocab;
    const int first = rank * kThreads + tid;
    constexpr int kStride = C * kThreads;
    auto scaled_logit = [&](int i, float v) {
        v = i == banned ? -INFINITY : v;
        return scaled ? v / t : v;
    };
    auto for_logits = [&](auto&& each) {         // each(column, scaled logit) -> what to write to p[column] (only the last pass writes)
        for (int gi = first; gi < groups; gi += kStride) {
            if (wide) {
                const float4 v = reinterpret_cast<const float4*>(logit_row)[gi];
                each(4 * gi, scaled_logit(4 * gi, v.x)); each(4 * gi + 1, scaled_logit(4 * gi + 1, v.y));
                each(4 * gi + 2, scaled_logit(4 * gi + 2, v.z)); each(4 * gi + 3, scaled_logit(4 * gi + 3, v.w));
            } else {
                each(gi, scaled_logit(gi, logit_row[gi]));
            }
        }
    };
    float mine = -INFINITY;
    for_logits([&](int, float x) { mine = fmaxf(mine, x); });
    const float mx = reduce_float<C>(mine, false, sh.val, sh.x, turn);
    const bool flat = !(mx > -INFINITY);         // every logit is -inf: the uniform distribution
    int none[kWays];
    Mass part[kWays];
    auto clear = [&]() {
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
            none[w] = 0;
            part[w] = 0;
        }
    };
    // the sum of the exponentials in fixed point too (they are at most 1 each): it does not depend on how the columns
    // are spread over threads and CTAs, so neither do the probabilities
    float sum = static_cast<float>(vocab);
    if (!flat) {
        clear();
        for_logits([&](int, float x) { part[0] += mass_of(expf(x - mx)); });
        reduce_all<C>(none, part, sh.count, sh.sum, sh.x, turn);
        sum = __ull2float_rn(part[0]) * (1.f / 1099511627776.f);
    }
    const float pmax = sum > 0.f ? 1.f / sum : 1.f;           // the probability of a column that holds the maximum: exp(0) / sum
    clear();
    for_logits([&](int col, float x) {
        const float e = flat ? 1.f : expf(x - mx);
        const float q = sum > 0.f ? e / sum : e;
        p[col] = q;
        part[0] += mass_of(q);
    });
    reduce_all<C>(none, part, sh.count, sh.sum, sh.x, turn);    // also orders the writes above before what reads them below
    const Mass whole = part[0];
    if (tid == 0) sh.listed = 0;
    __syncthreads();
    const int top_bits = __float_as_int(pmax);

    // ---- the value of the last kept entries: the smallest b such that what lies above b fills neither the top-k
    // budget nor the nucleus
    const Mass p_mass = nucleus ? mass_of(p_limit) : ~Mass(0);
    auto open_budget = [&](int count, Mass sum_above) { return count < k_limit && sum_above < p_mass; };
    Row row{p, vocab, nullptr, 0};
    const Draw d{vocab, k_limit, top_bits, nucleus, p_mass, uniform[r], out + r, p};
    if (open_budget(vocab, whole)) {             // the whole vocabulary is kept
        finish<C>(row, d, true, -1, top_bits, vocab, 0, 0, whole, open_budget, rank, sh, turn);
        return;
    }
    // The first pass, by factors below the top, also collects what lies within 2^-16 of the top in shared memory:
    // when the last kept value lies in there (it mostly does), every later pass reads that list instead of the row.
    int threshold[kWays], count[kWays];
    Mass above_sum[kWays];
    thresholds_by_factors(-1, top_bits, threshold);
    const int collect_above = threshold[3];
    above<C>(row, -1, top_bits, 0, 0, threshold, count, above_sum, sh, turn, list, capacity, collect_above);
    int lo = -1, hi = top_bits, count_lo = vocab, count_hi = 0;
    Mass sum_hi = 0;
    narrow(threshold, count, above_sum, open_budget, lo, hi, count_lo, count_hi, sum_hi);
    // Every CTA of the cluster must take the same way from here on (they meet at the same barriers). The lists are used
    // when the value lies within them and none of them ran over; when they fit into one list together, CTA 0 takes them
    // all and finishes the draw alone, with no more than a block's reduction per pass.
    int listed_by[kMaxCluster];
    int listed_total = sh.listed;
    bool over = sh.listed > capacity;
    if (C > 1) {
        float4 tell[kWays];
        tell[0] = make_float4(__int_as_float(sh.listed), 0.f, 0.f, 0.f);
        const int parity = exchange<C>(sh.x, turn, tell, 1);
        listed_total = 0;
        over = false;
        for (int k = 0; k < C; ++k) {
            listed_by[k] = __float_as_int(sh.x.slot[parity][k][0].x);
            over = over || listed_by[k] > capacity;
            listed_total += min(listed_by[k], capacity);
        }
    }
    if (lo < collect_above || over) {            // from the row in global memory
        finish<C>(row, d, false, lo, hi, count_lo, count_hi, sum_hi, whole, open_budget, rank, sh, turn);
        return;
    }
    row.list = list;
    row.listed = sh.listed;
    if (C > 1 && listed_total <= capacity) {
        int offset = 0;
        for (int k = 0; k < rank; ++k) offset += listed_by[k];
        if (rank != 0) {
            for (int k = tid; k < row.listed; k += kThreads)
                store_cluster_f2(static_cast<uint32_t>(__cvta_generic_to_shared(list + offset + k)), 0, list[k].v, __int_as_float(list[k].i));
        }
        cluster_arrive();
        cluster_wait();
        if (rank != 0) return;
        row.listed = listed_total;
        finish<1>(row, d, false, lo, hi, count_lo, count_hi, sum_hi, whole, open_budget, 0, sh, turn);
        return;
    }
    finish<C>(row, d, false, lo, hi, count_lo, count_hi, sum_hi, whole, open_budget, rank, sh, turn);
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
    constexpr int kCapacity = 20480;                                   // candidates a CTA's list holds: 160 KB
    constexpr int smem = kCapacity * static_cast<int>(sizeof(Candidate));
    static bool configured[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return STRIDE_BAD_ARGUMENT;
    if (!configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(sample_ranked_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(sample_ranked_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(sample_ranked_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(sample_ranked_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured[device] = true;
    }
    const dim3 block(kThreads);
#define STRIDE_RANKED(C)                                                                                                             \
    stride::launch_clusters(sample_ranked_kernel<C>, dim3(rows, 1, C), block, smem, stream, C, logits, vocab, row_stride, temperature, uniform, \
                            suppress, top_k, top_p, out, probs, kCapacity)
    if (rows <= 18) STRIDE_RANKED(8);
    else if (rows <= 37) STRIDE_RANKED(4);
    else if (rows <= 74) STRIDE_RANKED(2);
    else stride::launch(sample_ranked_kernel<1>, dim3(rows), block, smem, stream, logits, vocab, row_stride, temperature, uniform, suppress, top_k,
                        top_p, out, probs, kCapacity);
#undef STRIDE_RANKED
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
