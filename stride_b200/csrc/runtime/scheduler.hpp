// Continuous-batching scheduler over the cache manager.
//
// The rules are those of the reference (crates/stride-sched/src/lib.rs:188-538):
// every step places decodes first, then prefills that already hold pages, then
// waiting requests ranked by the time left to their deadline; prompts are cut
// into portions inside one token budget; when a decode cannot get a page, the
// running request with the most slack (ties: fewest generated tokens, then the
// highest id) gives up its pages and is later resumed by recomputing its whole
// context. Differences, each on purpose:
//   * a request preempted in this step is taken out of the batch being built;
//   * pages are published by the number of tokens whose keys are written, not by
//     the number of tokens sampled, and also at preemption;
//   * a decode reserves pages for the tokens it has, not for one more;
//   * prefills that block one another are resolved by the same preemption rule;
//   * ranking ties are broken by id, so that a trace replays.
// Time is a logical tick in microseconds that the caller advances.
#pragma once

#include <deque>
#include <map>

#include "cache_manager.hpp"
#include "sampler.hpp"
#include "step_batch.hpp"

namespace stride {

using Tick = uint64_t;
using SeqId = int64_t;

enum class ServiceClass { Interactive = 0, Batch = 1, Background = 2 };

// Budgets in microseconds (crates/stride-core/src/request.rs:18-36).
inline Tick ttft_budget_us(ServiceClass c) {
    switch (c) {
        case ServiceClass::Interactive: return 500000;
        case ServiceClass::Batch: return 10000000;
        default: return 120000000;
    }
}
inline Tick itl_budget_us(ServiceClass c) {
    switch (c) {
        case ServiceClass::Interactive: return 50000;
        case ServiceClass::Batch: return 200000;
        default: return 1000000;
    }
}

enum class SeqState { Waiting, Prefilling, Decoding, Swapped, Finished };
enum class FinishReason { None, Length, Stop, Cancelled, Preempted };

struct Sequence {
    SeqId id = 0;
    int64_t request = 0;
    std::string tenant;
    ServiceClass klass = ServiceClass::Interactive;
    SeqState state = SeqState::Waiting;
    FinishReason reason = FinishReason::None;
    std::vector<TokenId> tokens;  // prompt, then every generated token
    size_t prompt_len = 0;
    size_t kv_len = 0;            // leading tokens whose keys and values are in the cache
    size_t cached_prefix_len = 0;
    size_t max_tokens = 0;
    Tick arrived_at = 0;
    std::optional<Tick> first_token_at, last_token_at;
    uint64_t preemptions = 0;

    size_t total_len() const { return tokens.size(); }
    size_t output_len() const { return tokens.size() - prompt_len; }
    bool at_limit() const { return output_len() >= max_tokens; }
    std::optional<Tick> ttft_us() const {
        if (!first_token_at) return std::nullopt;
        return *first_token_at >= arrived_at ? *first_token_at - arrived_at : 0;
    }
    std::optional<double> mean_itl_us() const {
        if (!first_token_at || !last_token_at || output_len() < 2) return std::nullopt;
        return double(*last_token_at - *first_token_at) / double(output_len() - 1);
    }
};

struct SchedulerConfig {
    size_t max_batch_seqs = 256;
    size_t max_batch_tokens = 2048;
    size_t max_model_len = 8192;
    double watermark = 0.01;
    bool chunked_prefill = true;
};

struct PrefillChunk {
    SeqId seq;
    size_t start, len, cached;
};

struct ScheduledBatch {
    std::vector<PrefillChunk> prefill;
    std::vector<SeqId> decode;
    std::vector<SeqId> preempted;
    bool empty() const { return prefill.empty() && decode.empty(); }
    size_t num_tokens() const {
        size_t n = decode.size();
        for (auto& c : prefill) n += c.len;
        return n;
    }
    size_t num_seqs() const { return decode.size() + prefill.size(); }
};

struct Finished {
    SeqId seq;
    int64_t request;
    FinishReason reason;
    std::vector<TokenId> output;
    std::optional<Tick> ttft_us;
    std::optional<double> mean_itl_us;
    size_t cached_prefix_len;
};

struct SchedulerMetrics {
    uint64_t admitted = 0, finished = 0, preemptions = 0, ttft_deadline_misses = 0, steps = 0;
    uint64_t prefill_tokens_computed = 0, prefill_tokens_reused = 0;
    double prefill_reuse_rate() const {
        uint64_t total = prefill_tokens_computed + prefill_tokens_reused;
        return total ? double(prefill_tokens_reused) / double(total) : 0.0;
    }
};

struct AdmissionError : std::invalid_argument {
    using std::invalid_argument::invalid_argument;
};

class Scheduler {
public:
    Scheduler(SchedulerConfig cfg, CacheManager* cache) : cfg_(cfg), cache_(cache) {
        if (cfg_.max_batch_tokens == 0 || cfg_.max_batch_seqs == 0)
            throw std::invalid_argument("the step budgets must be positive");
    }

    const SchedulerConfig& config() const { return cfg_; }
    const SchedulerMetrics& metrics() const { return metrics_; }
    CacheManager& cache() { return *cache_; }
    size_t num_waiting() const { return waiting_.size(); }
    size_t num_running() const { return running_.size(); }
    const std::vector<SeqId>& running_ids() const { return running_; }
    const std::vector<SeqId>& waiting_ids() const { return waiting_; }
    bool idle() const { return waiting_.empty() && running_.empty(); }

    const Sequence* sequence(SeqId id) const {
        auto it = seqs_.find(id);
        return it == seqs_.end() ? nullptr : &it->second;
    }

    size_t reserved_pages() const {
        size_t r = static_cast<size_t>(std::ceil(double(cache_->min_capacity()) * cfg_.watermark));
        return std::max<size_t>(r, 1);
    }

    // Accepts a request: one sequence, state Waiting, no pages yet.
    SeqId admit(int64_t request, const std::string& tenant, std::vector<TokenId> prompt, const SamplingParams& params,
                ServiceClass klass, Tick arrived_at) {
        params.validate();
        if (prompt.empty()) throw AdmissionError("prompt must not be empty");
        if (prompt.size() >= cfg_.max_model_len)
            throw AdmissionError("prompt of " + std::to_string(prompt.size()) + " tokens does not fit max_model_len " +
                                 std::to_string(cfg_.max_model_len));
        // A request that could never be held, even alone, is refused here
        // rather than left waiting for ever.
        size_t worst = std::min(prompt.size() + params.max_tokens, cfg_.max_model_len);
        if (!cfg_.chunked_prefill && prompt.size() > cfg_.max_batch_tokens)
            throw AdmissionError("prompt exceeds max_batch_tokens and chunked prefill is off");
        bool windowed = false;
        for (size_t g = 0; g < cache_->num_groups(); ++g) windowed = windowed || cache_->group(g).window != 0;
        if (!windowed && cache_->pages_for(worst) + reserved_pages() > cache_->min_capacity())
            throw AdmissionError("request needs " + std::to_string(cache_->pages_for(worst)) + " pages plus a reserve of " +
                                 std::to_string(reserved_pages()) + "; the pool has " +
                                 std::to_string(cache_->min_capacity()));
        Sequence s;
        s.id = next_seq_++;
        s.request = request;
        s.tenant = tenant;
        s.klass = klass;
        s.prompt_len = prompt.size();
        s.tokens = std::move(prompt);
        s.max_tokens = params.max_tokens;
        s.arrived_at = arrived_at;
        SeqId id = s.id;
        seqs_.emplace(id, std::move(s));
        waiting_.push_back(id);
        ++metrics_.admitted;
        return id;
    }

    // Time left before the sequence breaches its budget; lower is more urgent.
    int64_t slack_us(SeqId id, Tick now) const {
        auto it = seqs_.find(id);
        if (it == seqs_.end()) return INT64_MAX;
        const Sequence& s = it->second;
        Tick deadline = s.last_token_at ? *s.last_token_at + itl_budget_us(s.klass) : s.arrived_at + ttft_budget_us(s.klass);
        return int64_t(deadline) - int64_t(now);
    }

    // Chooses the work of one step.
    ScheduledBatch step(Tick now) {
        ++metrics_.steps;
        ScheduledBatch batch;
        size_t reserve = reserved_pages();
        std::vector<SeqId> running = running_;

        // 1. decodes, which may use the reserve and may preempt
        for (SeqId id : running) {
            if (batch.decode.size() >= cfg_.max_batch_seqs || batch.num_tokens() >= cfg_.max_batch_tokens) break;
            auto it = seqs_.find(id);
            if (it == seqs_.end() || it->second.state != SeqState::Decoding) continue;
            if (it->second.kv_len + 1 != it->second.total_len()) continue;  // no new token was fed back: nothing to run
            size_t need = it->second.total_len();
            bool ok = cache_->ensure(id, need, 0);
            while (!ok) {
                auto victim = preemption_victim(now, id);
                if (!victim) break;
                preempt(*victim);
                batch.preempted.push_back(*victim);
                batch.decode.erase(std::remove(batch.decode.begin(), batch.decode.end(), *victim), batch.decode.end());
                ok = cache_->ensure(id, need, 0);
            }
            if (ok) batch.decode.push_back(id);
        }
        for (SeqId id : batch.decode) seqs_.at(id).kv_len = seqs_.at(id).total_len();

        // 2. prefills that already hold pages
        for (SeqId id : running) {
            size_t used = batch.num_tokens();
            if (used >= cfg_.max_batch_tokens || batch.num_seqs() >= cfg_.max_batch_seqs) break;
            auto it = seqs_.find(id);
            if (it == seqs_.end() || it->second.state != SeqState::Prefilling) continue;
            auto c = try_prefill(id, cfg_.max_batch_tokens - used, reserve);
            // Prefills that hold pages can block one another with no decode left
            // to preempt for them. When nothing at all is placed yet, the first of
            // them takes pages from the others, so that every step makes progress.
            while (!c && batch.empty()) {
                auto victim = preemption_victim(now, id);
                if (!victim) break;
                preempt(*victim);
                batch.preempted.push_back(*victim);
                c = try_prefill(id, cfg_.max_batch_tokens - used, 0);
            }
            if (c) batch.prefill.push_back(*c);
        }

        // 3. waiting requests, most urgent first
        std::vector<std::pair<int64_t, SeqId>> ranked;
        for (SeqId id : waiting_) ranked.emplace_back(slack_us(id, now), id);
        std::sort(ranked.begin(), ranked.end());
        std::vector<SeqId> deferred;
        for (auto& r : ranked) {
            size_t used = batch.num_tokens();
            if (used >= cfg_.max_batch_tokens || batch.num_seqs() >= cfg_.max_batch_seqs) {
                deferred.push_back(r.second);
                continue;
            }
            if (auto c = try_prefill(r.second, cfg_.max_batch_tokens - used, reserve))
                batch.prefill.push_back(*c);
            else
                deferred.push_back(r.second);
        }
        waiting_ = deferred;
        if (batch.num_tokens() > cfg_.max_batch_tokens) throw InvariantError("the token budget was exceeded");
        return batch;
    }

    // ---- a step launched before the tokens of the step before it are known.
    // After a step of decodes only has been scheduled (and launched), the same requests can be launched one
    // position further right away, their next tokens travelling on the device, if nothing else could change the
    // batch: nobody waits for admission, every running request is in the batch, none reaches max_tokens or
    // max_model_len with the token to come, and a page for one more token each is there without taking one from
    // anybody. What cannot be known in advance is a stop token; such a request's row in the chained step is
    // dropped by the caller when its tokens arrive. Returns false, and reserves nothing that matters, otherwise.
    bool reserve_chain(const ScheduledBatch& batch) {
        if (!batch.prefill.empty() || batch.decode.empty() || !waiting_.empty()) return false;
        if (batch.decode.size() != running_.size()) return false;
        for (SeqId id : batch.decode) {
            const Sequence& s = seqs_.at(id);
            if (s.state != SeqState::Decoding || s.kv_len != s.total_len()) return false;
            if (s.output_len() + 1 >= s.max_tokens || s.total_len() + 1 >= cfg_.max_model_len) return false;
        }
        for (SeqId id : batch.decode)       // pages a request gets here and does not use go back when it ends
            if (!cache_->ensure(id, seqs_.at(id).total_len() + 1, 0)) return false;
        return true;
    }

    // The chained step's work, once the tokens of the step before it have been fed back (on_tokens) and requests
    // that stopped have been retired: the survivors of `chained`, each with its newest token at the next position.
    // Counts as a step if anybody is left; the scheduler's own step() is not called for it.
    ScheduledBatch adopt_chain(const std::vector<SeqId>& chained) {
        ScheduledBatch batch;
        for (SeqId id : chained) {
            auto it = seqs_.find(id);
            if (it == seqs_.end() || it->second.state != SeqState::Decoding) continue;
            Sequence& s = it->second;
            if (s.kv_len + 1 != s.total_len()) throw InvariantError("a chained request did not receive its token");
            s.kv_len = s.total_len();
            batch.decode.push_back(id);
        }
        if (!batch.decode.empty()) ++metrics_.steps;
        return batch;
    }

    // The step's work items: portions first, then decodes; logits are wanted
    // where a portion reaches the end of the context and at every decode
    // (crates/stride-engine/src/lib.rs:314-369).
    std::vector<WorkItem> work_items(const ScheduledBatch& batch) const {
        std::vector<WorkItem> out;
        for (auto& c : batch.prefill) {
            const Sequence& s = seqs_.at(c.seq);
            size_t end = std::min(c.start + c.len, s.total_len());
            WorkItem w;
            w.request = c.seq;
            w.tokens.assign(s.tokens.begin() + c.start, s.tokens.begin() + end);
            w.position = c.start;
            if (end >= s.total_len()) w.want.push_back(static_cast<int32_t>(end - c.start - 1));
            out.push_back(std::move(w));
        }
        for (SeqId id : batch.decode) {
            const Sequence& s = seqs_.at(id);
            WorkItem w;
            w.request = id;
            w.tokens = {s.tokens.back()};
            w.position = s.total_len() - 1;
            w.want = {0};
            out.push_back(std::move(w));
        }
        return out;
    }

    // Called after the step ran: window groups give back the pages they have passed.
    void after_step(const ScheduledBatch& batch) {
        for (auto& c : batch.prefill) cache_->trim(c.seq, seqs_.at(c.seq).kv_len);
        for (SeqId id : batch.decode) cache_->trim(id, seqs_.at(id).kv_len);
    }

    // Feeds sampled tokens back. Returns the sequences that reached max_tokens.
    std::vector<Finished> on_tokens(const std::vector<std::pair<SeqId, TokenId>>& outputs, Tick now) {
        std::vector<Finished> done;
        for (auto& o : outputs) {
            auto it = seqs_.find(o.first);
            if (it == seqs_.end() || it->second.state != SeqState::Decoding) continue;
            Sequence& s = it->second;
            bool first = !s.first_token_at.has_value();
            s.tokens.push_back(o.second);
            if (first) s.first_token_at = now;
            s.last_token_at = now;
            if (first && *s.ttft_us() > ttft_budget_us(s.klass)) ++metrics_.ttft_deadline_misses;
            if (s.at_limit() || s.total_len() >= cfg_.max_model_len)
                if (auto f = retire(o.first, FinishReason::Length)) done.push_back(std::move(*f));
        }
        return done;
    }

    std::optional<Finished> stop(SeqId id) { return retire(id, FinishReason::Stop); }

    // `publish` false: the request's pages go back without being indexed for sharing (what they hold is not to
    // be trusted, e.g. after a step that the device reported as failed).
    std::vector<Finished> cancel(int64_t request, bool publish = true) {
        std::vector<SeqId> ids;
        for (auto& kv : seqs_)
            if (kv.second.request == request && kv.second.state != SeqState::Finished) ids.push_back(kv.first);
        std::vector<Finished> out;
        for (SeqId id : ids)
            if (auto f = retire(id, FinishReason::Cancelled, publish)) out.push_back(std::move(*f));
        return out;
    }

    // Forget a finished sequence's record.
    void forget(SeqId id) {
        auto it = seqs_.find(id);
        if (it != seqs_.end() && it->second.state == SeqState::Finished) seqs_.erase(it);
    }

private:
    std::optional<SeqId> preemption_victim(Tick now, SeqId protect) const {
        std::optional<SeqId> best;
        int64_t best_slack = 0;
        size_t best_lost = 0;
        for (SeqId id : running_) {
            if (id == protect) continue;
            int64_t slack = slack_us(id, now);
            size_t lost = seqs_.at(id).output_len();
            bool better = !best || slack > best_slack || (slack == best_slack && lost < best_lost) ||
                          (slack == best_slack && lost == best_lost && id > *best);
            if (better) {
                best = id;
                best_slack = slack;
                best_lost = lost;
            }
        }
        return best;
    }

    void preempt(SeqId id) {
        Sequence& s = seqs_.at(id);
        if (cache_->has(id)) {
            cache_->publish(id, s.tokens, s.kv_len);
            cache_->close(id);
        }
        s.kv_len = 0;
        s.cached_prefix_len = 0;
        s.state = SeqState::Swapped;
        ++s.preemptions;
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        waiting_.push_back(id);
        ++metrics_.preemptions;
    }

    // One portion of a context: the prompt, or after a preemption the prompt
    // and what was generated so far.
    std::optional<PrefillChunk> try_prefill(SeqId id, size_t budget, size_t reserve) {
        Sequence& s = seqs_.at(id);
        bool fresh = !cache_->has(id);
        if (fresh) {
            if (cache_->free_slots() == 0) return std::nullopt;
            cache_->open(id, s.tenant);
            size_t hit = cache_->adopt_prefix(id, s.tokens);
            s.cached_prefix_len = hit;
            s.kv_len = hit;
        }
        size_t start = s.kv_len;
        size_t remaining = s.total_len() - start;
        size_t len = cfg_.chunked_prefill ? std::min(remaining, budget) : (remaining <= budget ? remaining : 0);
        if (len == 0 || !cache_->ensure(id, start + len, reserve)) {
            if (fresh) {  // leave nothing behind: a deferred request holds no pages and no slot
                cache_->close(id);
                s.cached_prefix_len = 0;
                s.kv_len = 0;
            }
            return std::nullopt;
        }
        if (fresh) metrics_.prefill_tokens_reused += s.cached_prefix_len;
        s.kv_len = start + len;
        s.state = s.kv_len >= s.total_len() ? SeqState::Decoding : SeqState::Prefilling;
        if (std::find(running_.begin(), running_.end(), id) == running_.end()) running_.push_back(id);
        metrics_.prefill_tokens_computed += len;
        return PrefillChunk{id, start, len, s.cached_prefix_len};
    }

    std::optional<Finished> retire(SeqId id, FinishReason reason, bool publish = true) {
        auto it = seqs_.find(id);
        if (it == seqs_.end() || it->second.state == SeqState::Finished) return std::nullopt;
        Sequence& s = it->second;
        s.state = SeqState::Finished;
        s.reason = reason;
        Finished f{id, s.request, reason, std::vector<TokenId>(s.tokens.begin() + s.prompt_len, s.tokens.end()),
                   s.ttft_us(), s.mean_itl_us(), s.cached_prefix_len};
        if (cache_->has(id)) {
            if (publish) cache_->publish(id, s.tokens, s.kv_len);
            cache_->close(id);
        }
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
        ++metrics_.finished;
        return f;
    }

    SchedulerConfig cfg_;
    CacheManager* cache_;
    std::map<SeqId, Sequence> seqs_;
    std::vector<SeqId> waiting_, running_;
    SchedulerMetrics metrics_;
    SeqId next_seq_ = 1;
};

}  // namespace stride
