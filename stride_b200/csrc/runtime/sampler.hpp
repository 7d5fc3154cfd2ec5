// Sampling parameters and the host-side sampler.
//
// Names, defaults, validation and the order of operations are those of the
// reference (crates/stride-core/src/sampling.rs:5-80,
// crates/stride-backend/src/sampler.rs:18-165): EOS is suppressed until
// min_tokens are out; temperature 0 or top_k 1 is greedy (first maximum);
// otherwise logits / temperature, one softmax, one descending ranking, top-k
// then nucleus cut, and an inverse-CDF walk down the kept ranking with a
// uniform number from a xorshift64* generator seeded through splitmix64.
//
// The engine draws greedy and plain-temperature tokens on the GPU and only
// brings logits to this class when top-k or top-p is set; the generator here
// supplies the uniform number in both cases, so a seed fixes the stream.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <numeric>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace stride {

struct SamplingParams {
    float temperature = 1.0f;
    float top_p = 1.0f;
    std::optional<uint32_t> top_k;
    size_t max_tokens = 128;
    size_t min_tokens = 0;
    std::vector<int32_t> stop_tokens;
    std::optional<uint64_t> seed;
    bool ignore_eos = false;

    bool is_greedy() const { return temperature == 0.0f || (top_k && *top_k == 1); }
    bool needs_ranking() const { return !is_greedy() && (top_k.has_value() || top_p < 1.0f); }

    void validate() const {
        if (!(temperature >= 0.0f && temperature <= 2.0f))
            throw std::invalid_argument("temperature must be in [0, 2], got " + std::to_string(temperature));
        if (!(top_p >= 0.0f && top_p <= 1.0f))
            throw std::invalid_argument("top_p must be in (0, 1], got " + std::to_string(top_p));
        if (top_p == 0.0f) throw std::invalid_argument("top_p must be > 0");
        if (top_k && *top_k == 0) throw std::invalid_argument("top_k must be >= 1, or None to disable");
        if (max_tokens == 0) throw std::invalid_argument("max_tokens must be >= 1");
        if (min_tokens > max_tokens)
            throw std::invalid_argument("min_tokens (" + std::to_string(min_tokens) + ") exceeds max_tokens (" +
                                        std::to_string(max_tokens) + ")");
    }
};

class Rng {
public:
    explicit Rng(uint64_t seed) {
        uint64_t z = seed + 0x9E3779B97F4A7C15ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        state_ = std::max<uint64_t>(z ^ (z >> 31), 1);
    }
    uint64_t next_u64() {
        uint64_t x = state_;
        x ^= x >> 12;
        x ^= x << 25;
        x ^= x >> 27;
        state_ = x;
        return x * 0x2545F4914F6CDD1Dull;
    }
    // Uniform in [0, 1) with 24 bits.
    float next_f32() { return float(next_u64() >> 40) / float(1u << 24); }

private:
    uint64_t state_;
};

inline int32_t argmax_first(const float* logits, size_t n) {
    size_t best = 0;
    for (size_t i = 1; i < n; ++i)
        if (logits[i] > logits[best]) best = i;
    return static_cast<int32_t>(best);
}

// The head of the ranking of `work` (weights that sum to 1): by weight, descending, equal weights in vocabulary order
// (what a stable sort of 0 .. n-1 gives). Returns how many entries the draw keeps (the first top_k, cut where the
// cumulated weight reaches top_p, at least one); order[0 .. keep) is sorted, the rest of `order` is in no order.
// Only the head is ever read, so it is selected and sorted `head` entries at a time instead of all n: a vocabulary of
// 128k sorts in about 10 ms, a head of a few hundred is found in a fraction of one.
inline size_t rank_head(const std::vector<float>& work, const std::optional<uint32_t>& top_k, float top_p, std::vector<uint32_t>& order) {
    const size_t n = work.size();
    order.resize(n);
    std::iota(order.begin(), order.end(), 0u);
    auto before = [&](uint32_t a, uint32_t b) { return work[a] > work[b] || (work[a] == work[b] && a < b); };
    const size_t limit = top_k ? std::min<size_t>(n, *top_k) : n;
    size_t keep = limit;
    size_t head = top_p < 1.0f ? std::min<size_t>(limit, 256) : limit;
    for (;;) {
        if (head < n) std::nth_element(order.begin(), order.begin() + head, order.end(), before);
        std::sort(order.begin(), order.begin() + head, before);
        if (!(top_p < 1.0f)) break;
        float cumulative = 0.0f;
        size_t nucleus = 0;
        bool reached = false;
        for (size_t rank = 0; rank < head; ++rank) {
            cumulative += work[order[rank]];
            nucleus = rank + 1;
            if (cumulative >= top_p) {
                reached = true;
                break;
            }
        }
        if (reached || head == limit) {      // the nucleus ends inside the head, or top_k (or the vocabulary) ends first
            keep = std::min(limit, std::max<size_t>(nucleus, 1));
            break;
        }
        head = std::min(limit, head * 8);
    }
    return keep;
}

class Sampler {
public:
    Sampler(SamplingParams params, int32_t eos, uint64_t fallback_seed)
        : params_(std::move(params)), rng_(params_.seed.value_or(fallback_seed)), eos_(eos),
          seed_(params_.seed.value_or(fallback_seed)) {}

    const SamplingParams& params() const { return params_; }
    uint64_t effective_seed() const { return seed_; }
    float next_uniform() { return rng_.next_f32(); }

    // Token to suppress at this point of the generation, or -1.
    int32_t suppressed_token(size_t generated) const { return generated < params_.min_tokens ? eos_ : -1; }

    bool is_stop(int32_t token) const {
        if (token == eos_ && eos_ >= 0 && !params_.ignore_eos) return true;
        return std::find(params_.stop_tokens.begin(), params_.stop_tokens.end(), token) != params_.stop_tokens.end();
    }

    int32_t sample(const float* logits, size_t n, size_t generated) {
        if (n == 0) throw std::invalid_argument("cannot sample from an empty distribution");
        std::vector<float> work(logits, logits + n);
        int32_t banned = suppressed_token(generated);
        if (banned >= 0 && size_t(banned) < n) work[banned] = -std::numeric_limits<float>::infinity();
        if (params_.is_greedy()) return argmax_first(work.data(), n);

        float t = params_.temperature;
        if (t > 0.0f && std::fabs(t - 1.0f) > std::numeric_limits<float>::epsilon())
            for (auto& l : work) l /= t;

        // softmax with the maximum subtracted; all -inf gives the uniform distribution
        float mx = -std::numeric_limits<float>::infinity();
        for (float l : work) mx = std::max(mx, l);
        if (!std::isfinite(mx)) {
            std::fill(work.begin(), work.end(), 1.0f / float(n));
        } else {
            float sum = 0.0f;
            for (auto& l : work) {
                l = std::exp(l - mx);
                sum += l;
            }
            if (sum > 0.0f)
                for (auto& l : work) l /= sum;
        }

        std::vector<uint32_t> order;
        const size_t keep = rank_head(work, params_.top_k, params_.top_p, order);
        float total = 0.0f;
        for (size_t i = 0; i < keep; ++i) total += work[order[i]];
        if (!(total > 0.0f) || !std::isfinite(total)) return static_cast<int32_t>(order[0]);
        float target = rng_.next_f32() * total;
        for (size_t i = 0; i < keep; ++i) {
            target -= work[order[i]];
            if (target <= 0.0f) return static_cast<int32_t>(order[i]);
        }
        return static_cast<int32_t>(order[keep - 1]);
    }

private:
    SamplingParams params_;
    Rng rng_;
    int32_t eos_;
    uint64_t seed_;
};

}  // namespace stride
