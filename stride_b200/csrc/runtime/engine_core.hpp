// The host side of one engine step, without the device: what runs before the
// kernels are launched (scheduling, the step's batch, the parameters of the
// device sampler) and what runs after the sampled tokens are back (stop rules,
// feeding tokens to the scheduler, retiring). The reference's engine loop does
// the same between its scheduler and its executor
// (crates/stride-engine/src/lib.rs:263-297 admit, :299-414 step, :433-457
// retire); here the executor is the caller, who launches the step function and
// the sampling kernel between begin_step() and finish_step().
//
// Per request the core keeps its sampler (seeded base + request id when the
// request brings no seed, lib.rs:278-287), the tokens it has produced and, once
// it has ended, why. Greedy and plain-temperature rows are drawn on the device
// from the arrays that prepare_sampling() fills; rows that need a ranking
// (top-k, top-p) are drawn here from their logits, which the caller brings.
#pragma once

#include <map>

#include "scheduler.hpp"

namespace stride {

struct EngineBusy : std::runtime_error {
    using std::runtime_error::runtime_error;
};

struct StepEvent {
    int64_t request = 0;
    bool has_token = false;
    TokenId token = 0;
    FinishReason reason = FinishReason::None;      // None: the request goes on
};

struct RequestRecord {
    int64_t request = 0;
    SeqId seq = 0;
    size_t prompt_len = 0;
    uint64_t seed = 0;
    std::vector<TokenId> tokens;
    bool finished = false;
    FinishReason reason = FinishReason::None;
    size_t cached_prefix_len = 0;
    std::optional<Tick> ttft_us;
    std::optional<double> mean_itl_us;
};

class EngineCore {
public:
    EngineCore(Scheduler* scheduler, int32_t eos, std::vector<int32_t> extra_stops, uint64_t base_seed, size_t max_queued,
               size_t vocab)
        : sched_(scheduler), eos_(eos), extra_stops_(std::move(extra_stops)), base_seed_(base_seed), max_queued_(max_queued),
          vocab_(vocab) {
        if (max_queued_ == 0) throw std::invalid_argument("max_queued must be positive");
    }

    // Admits a request and returns its id. Throws EngineBusy when too many requests wait already, AdmissionError
    // (from the scheduler) for a request that can never run, std::invalid_argument for bad parameters or tokens.
    int64_t add_request(std::vector<TokenId> prompt, SamplingParams params, const std::string& tenant, ServiceClass klass,
                        Tick now) {
        if (sched_->num_waiting() >= max_queued_)
            throw EngineBusy(std::to_string(sched_->num_waiting()) + " requests are waiting for admission (max_queued " +
                             std::to_string(max_queued_) + ")");
        for (TokenId t : prompt)
            if (t < 0 || size_t(t) >= vocab_)
                throw std::invalid_argument("token " + std::to_string(t) + " lies outside the vocabulary of " + std::to_string(vocab_));
        for (int32_t s : extra_stops_)
            if (std::find(params.stop_tokens.begin(), params.stop_tokens.end(), s) == params.stop_tokens.end())
                params.stop_tokens.push_back(s);
        int64_t rid = next_request_;
        SeqId seq = sched_->admit(rid, tenant, prompt, params, klass, now);
        ++next_request_;
        Live live{rid, Sampler(params, eos_, base_seed_ + uint64_t(rid))};
        RequestRecord rec;
        rec.request = rid;
        rec.seq = seq;
        rec.prompt_len = prompt.size();
        rec.seed = live.sampler.effective_seed();
        records_.emplace(rid, std::move(rec));
        live_.emplace(seq, std::move(live));
        return rid;
    }

    bool has_unfinished() const { return !live_.empty(); }
    size_t num_live() const { return live_.size(); }

    const RequestRecord& record(int64_t request) const {
        auto it = records_.find(request);
        if (it == records_.end()) throw std::out_of_range("unknown request " + std::to_string(request));
        return it->second;
    }
    // Drops the record of a finished request (its output has been handed over).
    void forget(int64_t request) {
        auto it = records_.find(request);
        if (it != records_.end() && it->second.finished) records_.erase(it);
    }

    std::vector<StepEvent> cancel(int64_t request, bool publish = true) {
        std::vector<StepEvent> events;
        for (auto& f : sched_->cancel(request, publish)) {
            events.push_back(StepEvent{f.request, false, 0, FinishReason::Cancelled});
            retire(f.seq, FinishReason::Cancelled, &f);
        }
        return events;
    }

    // ---- before the launch. False: nothing can run at this tick (the caller advances its clock).
    bool begin_step(Tick now) {
        if (in_step_) throw std::logic_error("begin_step while a step is open");
        launched_ = false;
        if (next_batch_) {
            // The step was launched ahead (chain_step): take it over instead of scheduling. Requests of it that
            // have ended since keep their rows, which finish_step passes over. If all of them have ended, the
            // launched step is of no use to anybody: it is dropped (its results are never read) and the step is
            // scheduled in the ordinary way.
            ScheduledBatch adopted = sched_->adopt_chain(next_rows_);
            if (!adopted.decode.empty()) {
                scheduled_ = std::move(adopted);
                batch_ = std::move(next_batch_);
                rows_ = std::move(next_rows_);
                next_rows_.clear();
                ++chained_steps_;
                launched_ = true;
                in_step_ = true;
                return true;
            }
            next_batch_.reset();
            next_rows_.clear();
            ++dropped_chains_;
        }
        scheduled_ = sched_->step(now);
        if (scheduled_.empty()) return false;
        batch_ = std::make_unique<StepBatch>(sched_->cache());
        for (auto& item : sched_->work_items(scheduled_)) batch_->add(item);
        rows_ = batch_->row_requests();
        in_step_ = true;
        return true;
    }

    // True when the open step was launched ahead by chain_step(): the caller only waits for its tokens.
    bool launched_ahead() const { return in_step_ && launched_; }
    uint64_t chained_steps() const { return chained_steps_; }
    // Whether the device half draws the rows that need a ranking (it then passes top_k / top_p arrays to
    // prepare_sampling); otherwise finish_step draws them on the host from their logits.
    void set_device_ranks(bool on) { device_ranks_ = on; }
    bool device_ranks() const { return device_ranks_; }
    uint64_t dropped_chains() const { return dropped_chains_; }

    // ---- between the launch of the open step and the arrival of its tokens: the step after it, launched ahead.
    // Possible when the open step holds single decoded tokens only, every one of its rows is drawn on the device
    // (so that the tokens can travel to the next step without the host), and the scheduler can promise the same
    // requests one position further (Scheduler::reserve_chain). On success next_batch() holds the chained step: the
    // same requests in the same order, one position on, with token ids that the caller overwrites on the device
    // with the open step's sampled tokens (row r of the open step feeds token r of the chained one);
    // prepare_next_sampling() fills its sampler arrays. The chained step becomes the open step at the next
    // begin_step(). False: nothing was changed and the next step is scheduled in the ordinary way.
    bool chain_step() {
        if (!in_step_) throw std::logic_error("no step is open");
        if (next_batch_) throw std::logic_error("a chained step is pending already");
        if (!batch_->decode_only() || rows_.size() != batch_->num_seqs()) return false;
        for (RequestKey seq : rows_) {
            auto it = live_.find(seq);
            if (it == live_.end() || (!device_ranks_ && it->second.sampler.params().needs_ranking())) return false;
        }
        if (scheduled_.decode != rows_) return false;      // rows of ended requests (a chained step being chained again)
        if (!sched_->reserve_chain(scheduled_)) return false;
        auto next = std::make_unique<StepBatch>(sched_->cache());
        for (auto& item : batch_->items()) next->add(WorkItem{item.request, {0}, item.position + 1, {0}});
        next_batch_ = std::move(next);
        next_rows_ = rows_;
        return true;
    }

    bool has_next() const { return bool(next_batch_); }
    const StepBatch& next_batch() const {
        if (!next_batch_) throw std::logic_error("no chained step is pending");
        return *next_batch_;
    }

    // prepare_sampling for the chained step: every request is one token further than its record says.
    void prepare_next_sampling(float* temperature, float* uniform, int32_t* suppress, size_t capacity, int32_t* top_k = nullptr,
                               float* top_p = nullptr) {
        if (!next_batch_) throw std::logic_error("no chained step is pending");
        if (next_rows_.size() > capacity) throw std::invalid_argument("more rows than the sampling arrays hold");
        if (!fill_sampling(next_rows_, 1, temperature, uniform, suppress, top_k, top_p).empty())
            throw std::logic_error("a chained step holds a row that the host would have to rank");
    }

    const StepBatch& batch() const {
        if (!batch_) throw std::logic_error("no step is open");
        return *batch_;
    }
    const std::vector<RequestKey>& rows() const { return rows_; }

    // Fills, per wanted row, what the device sampler reads: the temperature (0: first maximum), a uniform number
    // from the request's generator (0 for greedy rows, which draw none) and the token to suppress (-1: none).
    // Returns the rows that need a ranking and are therefore drawn by finish_step from their logits; their
    // device parameters are those of a greedy row.
    std::vector<int32_t> prepare_sampling(float* temperature, float* uniform, int32_t* suppress, size_t capacity, int32_t* top_k = nullptr,
                                          float* top_p = nullptr) {
        if (!in_step_) throw std::logic_error("no step is open");
        if (rows_.size() > capacity) throw std::invalid_argument("more rows than the sampling arrays hold");
        if (launched_) throw std::logic_error("the open step was launched ahead with its sampler arrays");
        return fill_sampling(rows_, 0, temperature, uniform, suppress, top_k, top_p);
    }

    // ---- after the launch. `tokens`: one per wanted row, from the device. `ranked_logits`: [ranked rows][vocab]
    // in the order that prepare_sampling returned. The window groups give back passed pages, every token goes
    // through the stop rules and on to the scheduler, and requests that end are retired.
    std::vector<StepEvent> finish_step(const int32_t* tokens, size_t count, const std::vector<int32_t>& ranked,
                                       const float* ranked_logits, size_t vocab, Tick now) {
        if (!in_step_) throw std::logic_error("no step is open");
        if (count != rows_.size()) throw std::invalid_argument("one token per wanted row is needed");
        in_step_ = false;
        sched_->after_step(scheduled_);
        std::vector<TokenId> drawn(tokens, tokens + count);
        for (size_t i = 0; i < ranked.size(); ++i) {
            size_t r = size_t(ranked[i]);
            if (r >= count || ranked_logits == nullptr) throw std::invalid_argument("ranked rows without their logits");
            Live& live = live_.at(rows_[r]);
            drawn[r] = live.sampler.sample(ranked_logits + i * vocab, vocab, records_.at(live.request).tokens.size());
        }
        std::vector<StepEvent> events;
        std::vector<std::pair<SeqId, TokenId>> sampled;
        std::vector<SeqId> stopped;
        for (size_t r = 0; r < count; ++r) {
            auto it = live_.find(rows_[r]);
            if (it == live_.end()) continue;
            Live& live = it->second;
            if (live.sampler.is_stop(drawn[r])) {
                stopped.push_back(rows_[r]);        // the stop token itself is not appended (lib.rs:393-397)
            } else {
                sampled.emplace_back(rows_[r], drawn[r]);
                records_.at(live.request).tokens.push_back(drawn[r]);
                events.push_back(StepEvent{live.request, true, drawn[r], FinishReason::None});
            }
        }
        std::vector<Finished> at_limit = sched_->on_tokens(sampled, now);
        for (SeqId seq : stopped) {
            auto f = sched_->stop(seq);
            events.push_back(StepEvent{live_.at(seq).request, false, 0, FinishReason::Stop});
            retire(seq, FinishReason::Stop, f ? &*f : nullptr);
        }
        for (auto& f : at_limit) {
            events.push_back(StepEvent{f.request, false, 0, FinishReason::Length});
            retire(f.seq, FinishReason::Length, &f);
        }
        batch_.reset();
        return events;
    }

    // Gives up the open step (and a step chained after it) because the device reported a failure: nothing was
    // sampled. Returns the requests that had work in those steps. The scheduler has already advanced them, as in
    // the reference (crates/stride-sched/src/lib.rs:431-440), so they cannot go on; the caller cancels them and
    // keeps serving the others.
    std::vector<int64_t> abandon_step() {
        std::vector<int64_t> requests;
        auto collect = [&](const StepBatch* b) {
            if (!b) return;
            for (auto& item : b->items()) {
                auto it = live_.find(item.request);
                if (it != live_.end() && std::find(requests.begin(), requests.end(), it->second.request) == requests.end())
                    requests.push_back(it->second.request);
            }
        };
        collect(batch_.get());
        collect(next_batch_.get());
        in_step_ = false;
        launched_ = false;
        batch_.reset();
        next_batch_.reset();
        next_rows_.clear();
        return requests;
    }

private:
    struct Live {
        int64_t request;
        Sampler sampler;
    };

    // `ahead`: tokens that the requests will have produced by then beyond what their records hold. With `top_k` and
    // `top_p` (arrays for a device that ranks: 0 and 1 mean "no cut") a row that needs a ranking gets its temperature,
    // a uniform number and its cuts like any other; without them it is returned for the host to draw.
    std::vector<int32_t> fill_sampling(const std::vector<RequestKey>& rows, size_t ahead, float* temperature, float* uniform,
                                       int32_t* suppress, int32_t* top_k = nullptr, float* top_p = nullptr) {
        std::vector<int32_t> ranked;
        const bool device_ranks = top_k != nullptr && top_p != nullptr;
        for (size_t r = 0; r < rows.size(); ++r) {
            Live& live = live_.at(rows[r]);
            const SamplingParams& p = live.sampler.params();
            size_t generated = records_.at(live.request).tokens.size() + ahead;
            suppress[r] = live.sampler.suppressed_token(generated);
            if (device_ranks) {
                top_k[r] = 0;
                top_p[r] = 1.f;
            }
            if (p.needs_ranking() && !device_ranks) {
                ranked.push_back(int32_t(r));
                temperature[r] = 0.f;
                uniform[r] = 0.f;
            } else if (p.is_greedy()) {
                temperature[r] = 0.f;
                uniform[r] = 0.f;
            } else {
                temperature[r] = p.temperature;
                uniform[r] = live.sampler.next_uniform();
                if (p.needs_ranking()) {
                    top_k[r] = p.top_k ? int32_t(std::min<uint32_t>(*p.top_k, 0x7fffffffu)) : 0;
                    top_p[r] = p.top_p;
                }
            }
        }
        return ranked;
    }

    void retire(SeqId seq, FinishReason reason, const Finished* f) {
        auto it = live_.find(seq);
        if (it == live_.end()) return;
        RequestRecord& rec = records_.at(it->second.request);
        rec.finished = true;
        rec.reason = reason;
        if (f) {
            rec.cached_prefix_len = f->cached_prefix_len;
            rec.ttft_us = f->ttft_us;
            rec.mean_itl_us = f->mean_itl_us;
        }
        live_.erase(it);
        sched_->forget(seq);
    }

    Scheduler* sched_;
    int32_t eos_;
    std::vector<int32_t> extra_stops_;
    uint64_t base_seed_;
    size_t max_queued_, vocab_;
    int64_t next_request_ = 1;
    std::map<SeqId, Live> live_;
    std::map<int64_t, RequestRecord> records_;
    ScheduledBatch scheduled_;
    std::unique_ptr<StepBatch> batch_, next_batch_;
    std::vector<RequestKey> rows_, next_rows_;
    bool in_step_ = false, launched_ = false;
    bool device_ranks_ = false;      // the device draws top-k and nucleus rows too: such rows do not keep a step from being chained
    uint64_t chained_steps_ = 0, dropped_chains_ = 0;
};

}  // namespace stride
