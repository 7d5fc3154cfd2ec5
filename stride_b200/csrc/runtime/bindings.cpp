// Python bindings of the host runtime: page pools, cache manager, step batches,
// sampler, scheduler and the host side of the engine's step. No CUDA here: this module builds and runs without a GPU.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "engine_core.hpp"
#include "scheduler.hpp"

namespace py = pybind11;
using namespace stride;

static py::dict pool_stats(const PagePool& p) {
    auto s = p.stats();
    py::dict d;
    d["capacity"] = s.capacity;
    d["live"] = s.live;
    d["cached"] = s.cached;
    d["free"] = s.free;
    d["hits"] = s.hits;
    d["misses"] = s.misses;
    d["block_hit_rate"] = s.hit_rate();
    d["evictions"] = p.evictions();
    return d;
}

static py::dict layout_dict(const PackedLayout& l) {
    py::dict d;
    d["token_ids"] = l.token_ids;
    d["positions"] = l.positions;
    d["seq_of_token"] = l.seq_of_token;
    d["logit_rows"] = l.logit_rows;
    d["q_start"] = l.q_start;
    d["q_len"] = l.q_len;
    d["ctx_len"] = l.ctx_len;
    d["state_slot"] = l.state_slot;
    d["slot_mapping"] = l.slot_mapping;
    d["block_table"] = l.block_table;
    d["total"] = l.total;
    d["token_cap"] = l.token_cap;
    d["seq_cap"] = l.seq_cap;
    d["row_cap"] = l.row_cap;
    d["table_width"] = l.table_width;
    return d;
}

PYBIND11_MODULE(_runtime, m) {
    m.doc() = "stride_b200 host runtime";

    py::register_exception<InvariantError>(m, "InvariantError");
    py::register_exception<OutOfPages>(m, "OutOfPages");
    py::register_exception<AdmissionError>(m, "AdmissionError", PyExc_ValueError);
    py::register_exception<EngineBusy>(m, "EngineBusy", PyExc_RuntimeError);

    m.def("tenant_root", &prefix_hash::tenant_root);
    m.def("prefix_chain", [](const std::string& tenant, const std::vector<TokenId>& tokens, size_t page_size) {
        return prefix_hash::chain(tenant, tokens, page_size, tokens.size());
    });

    py::class_<PagePool>(m, "PagePool")
        .def(py::init<size_t, size_t>(), py::arg("num_pages"), py::arg("page_size"))
        .def_property_readonly("page_size", &PagePool::page_size)
        .def_property_readonly("capacity", &PagePool::capacity)
        .def_property_readonly("num_allocatable", &PagePool::num_allocatable)
        .def("pages_for", &PagePool::pages_for)
        .def("refcount", &PagePool::refcount)
        .def("acquire_prefix", &PagePool::acquire_prefix)
        .def("allocate", &PagePool::allocate)
        .def("publish", &PagePool::publish, py::arg("tenant"), py::arg("tokens"), py::arg("written_tokens"), py::arg("pages"))
        .def("release", &PagePool::release)
        .def("stats", &pool_stats)
        .def("check_invariants", &PagePool::check_invariants)
        .def("corrupt_for_test", &PagePool::corrupt_for_test);

    py::class_<CacheManager>(m, "CacheManager")
        .def(py::init([](size_t page_size, const std::vector<std::pair<size_t, size_t>>& groups, size_t slots, bool prefix) {
                 std::vector<GroupConfig> g;
                 for (auto& x : groups) g.push_back(GroupConfig{x.first, x.second});
                 return new CacheManager(page_size, g, slots, prefix);
             }),
             py::arg("page_size"), py::arg("groups"), py::arg("num_state_slots"), py::arg("prefix_caching") = true)
        .def_property_readonly("page_size", &CacheManager::page_size)
        .def_property_readonly("num_groups", &CacheManager::num_groups)
        .def_property_readonly("prefix_caching", &CacheManager::prefix_caching)
        .def_property_readonly("num_requests", &CacheManager::num_requests)
        .def_property_readonly("free_slots", &CacheManager::free_slots)
        .def_property_readonly("slot_capacity", &CacheManager::slot_capacity)
        .def_property_readonly("num_allocatable", &CacheManager::num_allocatable)
        .def("group", [](const CacheManager& c, size_t g) { return std::make_pair(c.group(g).num_pages, c.group(g).window); })
        .def("pages_for", &CacheManager::pages_for)
        .def("has", &CacheManager::has)
        .def("open", &CacheManager::open, py::arg("request"), py::arg("tenant") = "default")
        .def("adopt_prefix", &CacheManager::adopt_prefix)
        .def("ensure", &CacheManager::ensure, py::arg("request"), py::arg("num_tokens"), py::arg("reserve") = 0)
        .def("pages_missing", &CacheManager::pages_missing)
        .def("trim", &CacheManager::trim)
        .def("publish", &CacheManager::publish)
        .def("close", &CacheManager::close)
        .def("table", [](const CacheManager& c, RequestKey r, size_t g) { return c.table(r, g); }, py::arg("request"), py::arg("group") = 0)
        .def("state_slot", &CacheManager::state_slot)
        .def("stats", [](const CacheManager& c, size_t g) { return pool_stats(c.pool(g)); }, py::arg("group") = 0)
        .def("check_invariants", &CacheManager::check_invariants)
        .def("corrupt_for_test", [](CacheManager& c, size_t g, int what) { c.pool_mut(g).corrupt_for_test(what); });

    py::class_<StepBatch>(m, "StepBatch")
        .def(py::init<const CacheManager&>(), py::keep_alive<1, 2>())
        .def("add",
             [](StepBatch& b, RequestKey request, std::vector<TokenId> tokens, size_t position, std::vector<int32_t> want) {
                 b.add(WorkItem{request, std::move(tokens), position, std::move(want)});
             },
             py::arg("request"), py::arg("tokens"), py::arg("position"), py::arg("want"))
        .def_property_readonly("num_tokens", &StepBatch::num_tokens)
        .def_property_readonly("num_seqs", &StepBatch::num_seqs)
        .def_property_readonly("num_rows", &StepBatch::num_rows)
        .def_property_readonly("max_q_len", &StepBatch::max_q_len)
        .def_property_readonly("max_ctx", &StepBatch::max_ctx)
        .def_property_readonly("max_pages", &StepBatch::max_pages)
        .def_property_readonly("decode_only", &StepBatch::decode_only)
        .def("row_requests", &StepBatch::row_requests)
        .def("items",
             [](const StepBatch& b) {
                 py::list out;
                 for (auto& it : b.items()) out.append(py::make_tuple(it.request, it.tokens, it.position, it.want));
                 return out;
             })
        .def("pack",
             [](const StepBatch& b, size_t groups, size_t token_cap, size_t seq_cap, size_t row_cap, size_t table_width,
                py::object out, size_t row_offset, py::object row_count) -> py::tuple {
                 PackedLayout l = make_layout(groups, token_cap, seq_cap, row_cap, table_width);
                 size_t count = row_count.is_none() ? SIZE_MAX : row_count.cast<size_t>();
                 if (out.is_none()) {
                     py::array_t<int32_t> arr(l.total);
                     b.pack(l, arr.mutable_data(), row_offset, count);
                     return py::make_tuple(arr, layout_dict(l));
                 }
                 auto arr = out.cast<py::array_t<int32_t, py::array::c_style>>();
                 if (size_t(arr.size()) < l.total) throw std::invalid_argument("the output buffer is too small");
                 b.pack(l, arr.mutable_data(), row_offset, count);
                 return py::make_tuple(py::object(arr), layout_dict(l));
             },
             py::arg("groups"), py::arg("token_cap"), py::arg("seq_cap"), py::arg("row_cap"), py::arg("table_width"),
             py::arg("out") = py::none(), py::arg("row_offset") = 0, py::arg("row_count") = py::none());

    m.def("packed_layout", [](size_t groups, size_t token_cap, size_t seq_cap, size_t row_cap, size_t table_width) {
        return layout_dict(make_layout(groups, token_cap, seq_cap, row_cap, table_width));
    });

    py::class_<SamplingParams>(m, "SamplingParams")
        .def(py::init([](float temperature, float top_p, std::optional<uint32_t> top_k, size_t max_tokens, size_t min_tokens,
                         std::vector<int32_t> stop_tokens, std::optional<uint64_t> seed, bool ignore_eos) {
                 SamplingParams p;
                 p.temperature = temperature;
                 p.top_p = top_p;
                 p.top_k = top_k;
                 p.max_tokens = max_tokens;
                 p.min_tokens = min_tokens;
                 p.stop_tokens = std::move(stop_tokens);
                 p.seed = seed;
                 p.ignore_eos = ignore_eos;
                 return p;
             }),
             py::arg("temperature") = 1.0f, py::arg("top_p") = 1.0f, py::arg("top_k") = py::none(),
             py::arg("max_tokens") = 128, py::arg("min_tokens") = 0, py::arg("stop_tokens") = std::vector<int32_t>{},
             py::arg("seed") = py::none(), py::arg("ignore_eos") = false)
        .def_static("greedy",
                    [](size_t max_tokens) {
                        SamplingParams p;
                        p.temperature = 0.0f;
                        p.max_tokens = max_tokens;
                        return p;
                    },
                    py::arg("max_tokens") = 128)
        .def_readwrite("temperature", &SamplingParams::temperature)
        .def_readwrite("top_p", &SamplingParams::top_p)
        .def_readwrite("top_k", &SamplingParams::top_k)
        .def_readwrite("max_tokens", &SamplingParams::max_tokens)
        .def_readwrite("min_tokens", &SamplingParams::min_tokens)
        .def_readwrite("stop_tokens", &SamplingParams::stop_tokens)
        .def_readwrite("seed", &SamplingParams::seed)
        .def_readwrite("ignore_eos", &SamplingParams::ignore_eos)
        .def("is_greedy", &SamplingParams::is_greedy)
        .def("needs_ranking", &SamplingParams::needs_ranking)
        .def("validate", &SamplingParams::validate);

    py::class_<Rng>(m, "Rng")
        .def(py::init<uint64_t>())
        .def("next_u64", &Rng::next_u64)
        .def("next_f32", &Rng::next_f32);

    m.def("rank_head",
          [](py::array_t<float, py::array::c_style | py::array::forcecast> weights, std::optional<uint32_t> top_k, float top_p) {
              std::vector<float> work(weights.data(), weights.data() + weights.size());
              std::vector<uint32_t> order;
              const size_t keep = rank_head(work, top_k, top_p, order);
              order.resize(keep);
              return order;
          },
          py::arg("weights"), py::arg("top_k") = py::none(), py::arg("top_p") = 1.0f,
          "The tokens a draw keeps, in the order in which it walks them (see sampler.hpp).");
    py::class_<Sampler>(m, "Sampler")
        .def(py::init<SamplingParams, int32_t, uint64_t>(), py::arg("params"), py::arg("eos"), py::arg("fallback_seed"))
        .def_property_readonly("params", &Sampler::params)
        .def_property_readonly("effective_seed", &Sampler::effective_seed)
        .def("next_uniform", &Sampler::next_uniform)
        .def("suppressed_token", &Sampler::suppressed_token)
        .def("is_stop", &Sampler::is_stop)
        .def("sample",
             [](Sampler& s, py::array_t<float, py::array::c_style | py::array::forcecast> logits, size_t generated) {
                 return s.sample(logits.data(), size_t(logits.size()), generated);
             },
             py::arg("logits"), py::arg("generated") = 0);

    m.def("argmax_first", [](py::array_t<float, py::array::c_style | py::array::forcecast> logits) {
        return argmax_first(logits.data(), size_t(logits.size()));
    });

    py::enum_<ServiceClass>(m, "ServiceClass")
        .value("Interactive", ServiceClass::Interactive)
        .value("Batch", ServiceClass::Batch)
        .value("Background", ServiceClass::Background);
    m.def("ttft_budget_us", &ttft_budget_us);
    m.def("itl_budget_us", &itl_budget_us);

    py::enum_<SeqState>(m, "SeqState")
        .value("Waiting", SeqState::Waiting)
        .value("Prefilling", SeqState::Prefilling)
        .value("Decoding", SeqState::Decoding)
        .value("Swapped", SeqState::Swapped)
        .value("Finished", SeqState::Finished);

    py::enum_<FinishReason>(m, "FinishReason")
        .value("NotFinished", FinishReason::None)
        .value("Length", FinishReason::Length)
        .value("Stop", FinishReason::Stop)
        .value("Cancelled", FinishReason::Cancelled)
        .value("Preempted", FinishReason::Preempted);

    py::class_<SchedulerConfig>(m, "SchedulerConfig")
        .def(py::init([](size_t seqs, size_t tokens, size_t model_len, double watermark, bool chunked) {
                 return SchedulerConfig{seqs, tokens, model_len, watermark, chunked};
             }),
             py::arg("max_batch_seqs") = 256, py::arg("max_batch_tokens") = 2048, py::arg("max_model_len") = 8192,
             py::arg("watermark") = 0.01, py::arg("chunked_prefill") = true)
        .def_readwrite("max_batch_seqs", &SchedulerConfig::max_batch_seqs)
        .def_readwrite("max_batch_tokens", &SchedulerConfig::max_batch_tokens)
        .def_readwrite("max_model_len", &SchedulerConfig::max_model_len)
        .def_readwrite("watermark", &SchedulerConfig::watermark)
        .def_readwrite("chunked_prefill", &SchedulerConfig::chunked_prefill);

    py::class_<PrefillChunk>(m, "PrefillChunk")
        .def_readonly("seq", &PrefillChunk::seq)
        .def_readonly("start", &PrefillChunk::start)
        .def_readonly("len", &PrefillChunk::len)
        .def_readonly("cached", &PrefillChunk::cached);

    py::class_<ScheduledBatch>(m, "ScheduledBatch")
        .def_readonly("prefill", &ScheduledBatch::prefill)
        .def_readonly("decode", &ScheduledBatch::decode)
        .def_readonly("preempted", &ScheduledBatch::preempted)
        .def("is_empty", &ScheduledBatch::empty)
        .def_property_readonly("num_tokens", &ScheduledBatch::num_tokens)
        .def_property_readonly("num_seqs", &ScheduledBatch::num_seqs);

    py::class_<Finished>(m, "Finished")
        .def_readonly("seq", &Finished::seq)
        .def_readonly("request", &Finished::request)
        .def_readonly("reason", &Finished::reason)
        .def_readonly("output", &Finished::output)
        .def_readonly("ttft_us", &Finished::ttft_us)
        .def_readonly("mean_itl_us", &Finished::mean_itl_us)
        .def_readonly("cached_prefix_len", &Finished::cached_prefix_len);

    py::class_<Sequence>(m, "Sequence")
        .def_readonly("id", &Sequence::id)
        .def_readonly("request", &Sequence::request)
        .def_readonly("tenant", &Sequence::tenant)
        .def_readonly("klass", &Sequence::klass)
        .def_readonly("state", &Sequence::state)
        .def_readonly("reason", &Sequence::reason)
        .def_readonly("tokens", &Sequence::tokens)
        .def_readonly("prompt_len", &Sequence::prompt_len)
        .def_readonly("kv_len", &Sequence::kv_len)
        .def_readonly("cached_prefix_len", &Sequence::cached_prefix_len)
        .def_readonly("max_tokens", &Sequence::max_tokens)
        .def_readonly("arrived_at", &Sequence::arrived_at)
        .def_readonly("first_token_at", &Sequence::first_token_at)
        .def_readonly("last_token_at", &Sequence::last_token_at)
        .def_readonly("preemptions", &Sequence::preemptions)
        .def_property_readonly("total_len", &Sequence::total_len)
        .def_property_readonly("output_len", &Sequence::output_len)
        .def_property_readonly("output", [](const Sequence& s) {
            return std::vector<TokenId>(s.tokens.begin() + s.prompt_len, s.tokens.end());
        });

    py::class_<Scheduler>(m, "Scheduler")
        .def(py::init<SchedulerConfig, CacheManager*>(), py::arg("config"), py::arg("cache"), py::keep_alive<1, 3>())
        .def_property_readonly("config", &Scheduler::config)
        .def_property_readonly("num_waiting", &Scheduler::num_waiting)
        .def_property_readonly("num_running", &Scheduler::num_running)
        .def_property_readonly("running_ids", &Scheduler::running_ids)
        .def_property_readonly("waiting_ids", &Scheduler::waiting_ids)
        .def_property_readonly("idle", &Scheduler::idle)
        .def_property_readonly("reserved_pages", &Scheduler::reserved_pages)
        .def("admit", &Scheduler::admit, py::arg("request"), py::arg("tenant"), py::arg("prompt"), py::arg("params"),
             py::arg("klass") = ServiceClass::Interactive, py::arg("arrived_at") = 0)
        .def("slack_us", &Scheduler::slack_us)
        .def("step", &Scheduler::step, py::arg("now"))
        .def("work_items",
             [](const Scheduler& s, const ScheduledBatch& b) {
                 py::list out;
                 for (auto& it : s.work_items(b)) out.append(py::make_tuple(it.request, it.tokens, it.position, it.want));
                 return out;
             })
        .def("build_batch",
             [](Scheduler& s, const ScheduledBatch& b) {
                 auto batch = std::make_unique<StepBatch>(s.cache());
                 for (auto& it : s.work_items(b)) batch->add(it);
                 return batch;
             },
             py::keep_alive<0, 1>())
        .def("after_step", &Scheduler::after_step)
        .def("reserve_chain", &Scheduler::reserve_chain)
        .def("adopt_chain", &Scheduler::adopt_chain)
        .def("on_tokens", &Scheduler::on_tokens, py::arg("outputs"), py::arg("now"))
        .def("stop", &Scheduler::stop)
        .def("cancel", &Scheduler::cancel, py::arg("request"), py::arg("publish") = true)
        .def("forget", &Scheduler::forget)
        .def("sequence", &Scheduler::sequence, py::return_value_policy::copy)
        .def("metrics", [](const Scheduler& s) {
            auto& mt = s.metrics();
            py::dict d;
            d["admitted"] = mt.admitted;
            d["finished"] = mt.finished;
            d["preemptions"] = mt.preemptions;
            d["ttft_deadline_misses"] = mt.ttft_deadline_misses;
            d["steps"] = mt.steps;
            d["prefill_tokens_computed"] = mt.prefill_tokens_computed;
            d["prefill_tokens_reused"] = mt.prefill_tokens_reused;
            d["prefill_reuse_rate"] = mt.prefill_reuse_rate();
            return d;
        });

    py::class_<StepEvent>(m, "StepEvent")
        .def_readonly("request", &StepEvent::request)
        .def_property_readonly("token", [](const StepEvent& e) -> py::object { return e.has_token ? py::cast(e.token) : py::none(); })
        .def_readonly("reason", &StepEvent::reason);

    py::class_<RequestRecord>(m, "RequestRecord")
        .def_readonly("request", &RequestRecord::request)
        .def_readonly("seq", &RequestRecord::seq)
        .def_readonly("prompt_len", &RequestRecord::prompt_len)
        .def_readonly("seed", &RequestRecord::seed)
        .def_readonly("tokens", &RequestRecord::tokens)
        .def_readonly("finished", &RequestRecord::finished)
        .def_readonly("reason", &RequestRecord::reason)
        .def_readonly("cached_prefix_len", &RequestRecord::cached_prefix_len)
        .def_readonly("ttft_us", &RequestRecord::ttft_us)
        .def_readonly("mean_itl_us", &RequestRecord::mean_itl_us);

    py::class_<EngineCore>(m, "EngineCore")
        .def(py::init<Scheduler*, int32_t, std::vector<int32_t>, uint64_t, size_t, size_t>(), py::arg("scheduler"), py::arg("eos"),
             py::arg("extra_stops"), py::arg("base_seed"), py::arg("max_queued"), py::arg("vocab"), py::keep_alive<1, 2>())
        .def("add_request", &EngineCore::add_request, py::arg("prompt"), py::arg("params"), py::arg("tenant") = "default",
             py::arg("klass") = ServiceClass::Interactive, py::arg("now") = 0)
        .def("has_unfinished", &EngineCore::has_unfinished)
        .def_property_readonly("num_live", &EngineCore::num_live)
        .def("record", &EngineCore::record, py::return_value_policy::copy)
        .def("forget", &EngineCore::forget)
        .def("cancel", &EngineCore::cancel, py::arg("request"), py::arg("publish") = true)
        .def("begin_step", &EngineCore::begin_step, py::arg("now"))
        .def("batch", [](EngineCore& c) { return &c.batch(); }, py::return_value_policy::reference_internal)
        .def("rows", &EngineCore::rows)
        .def("prepare_sampling",
             [](EngineCore& c, py::array_t<float, py::array::c_style> temperature, py::array_t<float, py::array::c_style> uniform,
                py::array_t<int32_t, py::array::c_style> suppress, py::object top_k, py::object top_p) {
                 size_t cap = std::min({size_t(temperature.size()), size_t(uniform.size()), size_t(suppress.size())});
                 if (top_k.is_none() || top_p.is_none())
                     return c.prepare_sampling(temperature.mutable_data(), uniform.mutable_data(), suppress.mutable_data(), cap);
                 auto k = top_k.cast<py::array_t<int32_t, py::array::c_style>>();
                 auto p = top_p.cast<py::array_t<float, py::array::c_style>>();
                 cap = std::min({cap, size_t(k.size()), size_t(p.size())});
                 return c.prepare_sampling(temperature.mutable_data(), uniform.mutable_data(), suppress.mutable_data(), cap,
                                           k.mutable_data(), p.mutable_data());
             },
             py::arg("temperature"), py::arg("uniform"), py::arg("suppress"), py::arg("top_k") = py::none(), py::arg("top_p") = py::none())
        .def("set_device_ranks", &EngineCore::set_device_ranks)
        .def_property_readonly("device_ranks", &EngineCore::device_ranks)
        .def("finish_step",
             [](EngineCore& c, py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens, std::vector<int32_t> ranked,
                py::object ranked_logits, Tick now) {
                 if (ranked.empty()) return c.finish_step(tokens.data(), size_t(tokens.size()), ranked, nullptr, 0, now);
                 auto rows = ranked_logits.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>();
                 if (rows.ndim() != 2 || size_t(rows.shape(0)) != ranked.size())
                     throw std::invalid_argument("ranked_logits must be [ranked rows, vocab]");
                 return c.finish_step(tokens.data(), size_t(tokens.size()), ranked, rows.data(), size_t(rows.shape(1)), now);
             },
             py::arg("tokens"), py::arg("ranked") = std::vector<int32_t>{}, py::arg("ranked_logits") = py::none(), py::arg("now") = 0)
        .def("abandon_step", &EngineCore::abandon_step)
        .def("launched_ahead", &EngineCore::launched_ahead)
        .def_property_readonly("chained_steps", &EngineCore::chained_steps)
        .def_property_readonly("dropped_chains", &EngineCore::dropped_chains)
        .def("chain_step", &EngineCore::chain_step)
        .def("has_next", &EngineCore::has_next)
        .def("next_batch", [](EngineCore& c) { return &c.next_batch(); }, py::return_value_policy::reference_internal)
        .def("prepare_next_sampling",
             [](EngineCore& c, py::array_t<float, py::array::c_style> temperature, py::array_t<float, py::array::c_style> uniform,
                py::array_t<int32_t, py::array::c_style> suppress, py::object top_k, py::object top_p) {
                 size_t cap = std::min({size_t(temperature.size()), size_t(uniform.size()), size_t(suppress.size())});
                 if (top_k.is_none() || top_p.is_none()) {
                     c.prepare_next_sampling(temperature.mutable_data(), uniform.mutable_data(), suppress.mutable_data(), cap);
                     return;
                 }
                 auto k = top_k.cast<py::array_t<int32_t, py::array::c_style>>();
                 auto p = top_p.cast<py::array_t<float, py::array::c_style>>();
                 cap = std::min({cap, size_t(k.size()), size_t(p.size())});
                 c.prepare_next_sampling(temperature.mutable_data(), uniform.mutable_data(), suppress.mutable_data(), cap, k.mutable_data(),
                                         p.mutable_data());
             },
             py::arg("temperature"), py::arg("uniform"), py::arg("suppress"), py::arg("top_k") = py::none(), py::arg("top_p") = py::none());
}
