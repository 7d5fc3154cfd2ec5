"""Measures decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Llama-3.1-8B with random bfloat16 weights,
a batch of 8 requests at a context of 8192 tokens. It prints ONE JSON line:

* ``value``: decoded tokens a second, K decode steps replayed from the captured
  CUDA graph and timed on the device with CUDA events (the step reads every
  weight and the whole cache of the live requests, far more than the L2 holds);
* ``e2e``: the same through the Python entry point (``Engine.step``): host token
  ids in through pinned memory, scheduling, the step, sampling on the device,
  token ids back to the host, every step (``top_k_top_p``: the same with every row drawn at a
  temperature with a top-k and a nucleus cut);
* ``prefill``: one 2,048-token prompt, tokens a second and the fraction of the
  bf16 matrix peak;
* ``roofline``: bytes the decode step has to read divided by its time, against
  the measured copy bandwidth;
* ``points``: decode at batch 1 and 64 at the run's context, and at batch 1, 8 and
  64 at a context of 2,048 (``--points`` chooses other batches; the page pool is
  sized for what the run holds at once); also two more prefill steps of 2,048
  tokens (tokens a second): the first 256 tokens of eight prompts in one step,
  and 2,048 tokens of a prompt over 6,144 tokens that are already cached;
* ``breakdown``: device time per class of kernel of one decode step and of the
  prefill, from CUDA events around every launch of an eagerly run step.

Peaks come from MEASURED_PEAKS.json when the file exists, else from an earlier
measurement on the same pool (6.65 TB/s, 1.59 PFLOP/s). ``--impl reference``
runs the unmodified reference (``baseline/_ref``) on the same shapes.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_burst": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            # The prefill is a long step of several hundred kernels under the power cap, so its fraction is taken
            # of the library product's sustained rate; the burst rate is reported beside it.
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops_sustained") or d["bf16_tflops"]),
                    "bf16_tflops_burst": float(d["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    @staticmethod
    def _device_id() -> str:
        """What ``nvidia-smi -i`` should be given for the GPU this process computes on: its UUID, since on a
        machine with several GPUs the process may have been handed any of them (index 0 of torch is then not
        index 0 of nvidia-smi)."""
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
            return uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:  # noqa: BLE001
            first = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0].strip()
            return first or "0"

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i",
                                          self._device_id(), "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            self.summary = {"sm_mhz": statistics.median(clocks), "sm_max_mhz": mx, "reasons": sorted(reasons)}


# ------------------------------------------------------------------------ shapes
SHAPES = {"llama3.1-8b": "Llama-3.1-8B", "llama3.2-3b": "Llama-3.2-3B", "llama3.1-70b": "Llama-3.1-70B"}


def bench_config(layers: int | None, shape: str = "llama3.1-8b"):
    from stride_b200.config import config_from_dict, preset

    d = preset(shape)
    full_layers = d["num_hidden_layers"]
    if layers:
        d["num_hidden_layers"] = layers
    return config_from_dict(d), full_layers


def decode_bytes(cfg, batch: int, context: int, itemsize: int = 2) -> int:
    """Bytes a decode step has to read: every matrix once (the embedding table
    is only gathered from) and the keys and values of the live requests."""
    matrices = cfg.params_per_layer() * cfg.num_hidden_layers + cfg.vocab_size * cfg.hidden_size
    return matrices * itemsize + batch * context * cfg.kv_bytes_per_token(itemsize)


def prefill_flops(cfg, tokens: int, rows: int = 1) -> float:
    linear = 2.0 * tokens * cfg.params_per_layer() * cfg.num_hidden_layers + 2.0 * rows * cfg.hidden_size * cfg.vocab_size
    attention = cfg.num_hidden_layers * 4.0 * cfg.num_attention_heads * cfg.head_dim * tokens * (tokens + 1) / 2
    return linear + attention


# -------------------------------------------------------------------------- ours
def _synthetic_decode_batch(engine, batch: int, context: int, first_key: int):
    """``batch`` requests that hold ``context - 1`` tokens in the cache (pages
    allocated through the cache manager; contents are whatever the pool holds)
    and bring their next token."""
    import torch

    rt = engine._rt
    g = torch.Generator().manual_seed(batch)
    step = rt.StepBatch(engine.cache)
    keys = []
    for i in range(batch):
        key = first_key + i
        engine.cache.open(key, "bench")
        if not engine.cache.ensure(key, context, 0):
            raise RuntimeError("the page pool is too small for the benchmark batch")
        step.add(key, [int(torch.randint(0, engine.model.vocab, (1,), generator=g))], context - 1, [0])
        keys.append(key)
    return step, keys


def _time_graph(engine, step_batch, steps: int, warmup: int):
    """Device time of ``steps`` replays of the decode graph for this batch."""
    import torch

    runner = engine.runner
    for _ in range(max(warmup, 3)):
        runner.step(step_batch)
    torch.cuda.synchronize()
    launches_before = runner.replayed_launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler() as clocks:
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            runner.step(step_batch)
        end.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    return ms / steps, clocks.summary, runner.replayed_launches - launches_before


def _rounded(milliseconds: dict, keep: int = 14) -> dict:
    """The largest classes in microseconds, the rest summed up."""
    items = list(milliseconds.items())
    out = {k: round(v * 1e3) for k, v in items[:keep]}
    if len(items) > keep:
        out["other"] = round(sum(v for _k, v in items[keep:]) * 1e3)
    return out


def _end_to_end(engine, cfg, batch: int, context: int, steps: int, warmup: int, g, cuts: bool = False) -> dict:
    """``steps`` decode steps of ``batch`` requests at ``context`` through ``Engine.step``: the prompts go in as
    host token ids, are prefilled in portions, and every timed step brings host token ids back."""
    import torch

    from stride_b200 import SamplingParams
    prompts = [torch.randint(0, cfg.vocab_size, (context - 1,), generator=g).tolist() for _ in range(batch)]
    # requests that finish their prompt early keep decoding while the others are still prefilled in portions
    spare = batch * (-(-context // 2048)) + 16
    params = SamplingParams(temperature=0.0, max_tokens=warmup + steps + spare, ignore_eos=True)
    if cuts:        # every row drawn with a temperature, a top-k and a nucleus cut
        params = SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=7, max_tokens=warmup + steps + spare, ignore_eos=True)
    ids = [engine.add_request(p, params) for p in prompts]
    while engine.scheduler.num_waiting or any(engine.scheduler.sequence(engine._seq_of_request[i]).state != engine._rt.SeqState.Decoding
                                              for i in ids):
        engine.step()
    for _ in range(warmup):
        engine.step()
    h2d0, d2h0 = engine.h2d_bytes, engine.d2h_bytes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced, step_ms = 0, []
    for _ in range(steps):
        t_step = time.perf_counter()
        produced += sum(1 for _rid, tok, _why in engine.step() if tok is not None)
        step_ms.append((time.perf_counter() - t_step) * 1e3)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    if os.environ.get("STRIDE_BENCH_DEBUG"):
        print("e2e step ms:", [round(x, 2) for x in step_ms], file=sys.stderr)
        print("metrics:", engine.metrics(), file=sys.stderr)
    if produced != batch * steps:
        raise RuntimeError(f"the end-to-end loop produced {produced} tokens, expected {batch * steps}")
    for i in ids:
        engine.cancel(i)
    while engine.step():        # a step launched ahead for the cancelled requests is dropped here
        pass
    return {"value": round(produced / elapsed, 1), "unit": "tokens/s", "h2d_bytes_per_step": (engine.h2d_bytes - h2d0) // steps,
            "d2h_bytes_per_step": (engine.d2h_bytes - d2h0) // steps}


def run_ours(args) -> dict:
    import torch

    from stride_b200 import Engine, SamplingParams
    from stride_b200.csrc import ops

    pk = peaks()
    cfg, full_layers = bench_config(args.layers, args.shape)
    batch, context, prompt_len = args.batch, args.context, 2048
    page = 16
    point_batches = sorted({int(b) for b in args.points.split(",") if b.strip()})
    short_context = 2048 if context > 2048 else 0
    # the pool holds the largest batch that is live at any one time (the points run one after the other), and the
    # end-to-end requests, which decode past the context
    most = max(point_batches + [batch])
    need_tokens = max(most * (context + page), batch * (context + 1024), prompt_len) + 4096
    engine = Engine(config=cfg, random_weights=0, dtype="bfloat16", block_size=page, num_blocks=need_tokens // page + 64,
                    max_batch_tokens=2048, max_batch_seqs=max(most, 8), max_model_len=context + 1024, prefix_caching=False,
                    check_invariants=False)
    for pages in engine.device_cache.pages:      # synthetic cache contents: small random keys and values
        pages.normal_(0.0, 0.5)
    torch.cuda.synchronize()

    # ---- prefill: one 2,048-token prompt, device-timed
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist()
    times = []
    for i in range(3 + 5):
        key = 900000 + i
        engine.cache.open(key, "bench")
        engine.cache.ensure(key, prompt_len, 0)
        sb = engine._rt.StepBatch(engine.cache)
        sb.add(key, prompt, 0, [prompt_len - 1])
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.runner.step(sb)
        end.record()
        torch.cuda.synchronize()
        engine.cache.close(key)
        if i >= 3:
            times.append(start.elapsed_time(end))
    prefill_ms = statistics.median(times)
    prefill = {"value": round(prompt_len / prefill_ms * 1e3, 1), "tokens": prompt_len, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops(cfg, prompt_len) / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "frac_of_burst_peak": round(prefill_flops(cfg, prompt_len) / (prefill_ms * 1e-3) / (pk["bf16_tflops_burst"] * 1e12), 4)}

    # ---- two more prefill steps of 2,048 tokens: eight prompts' portions of 256 tokens in one step, and the last portion
    # of an 8,192-token prompt (2,048 tokens over 6,144 cached ones), when the run's context has room for it
    def portion_step(requests):
        """Median device time (ms) of one step with the given (cached tokens, new tokens) per request."""
        took = []
        for i in range(2 + 3):
            sb, keys = engine._rt.StepBatch(engine.cache), []
            for j, (cached, new) in enumerate(requests):
                key = 700000 + 100 * i + j
                engine.cache.open(key, "bench")
                engine.cache.ensure(key, cached + new, 0)
                sb.add(key, prompt[:new], cached, [new - 1])
                keys.append(key)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            engine.runner.step(sb)
            end.record()
            torch.cuda.synchronize()
            for key in keys:
                engine.cache.close(key)
            if i >= 2:
                took.append(start.elapsed_time(end))
        return statistics.median(took)

    prefill_points = {"prefill_8x256": round(prompt_len / portion_step([(0, prompt_len // 8)] * 8) * 1e3, 1)}
    if context >= 8192:
        prefill_points["prefill_2048_after_6144"] = round(prompt_len / portion_step([(6144, prompt_len)]) * 1e3, 1)

    # ---- decode points, device-timed graph replays on synthetic caches
    points, key_base = dict(prefill_points), 1000
    main = None
    runs = [(b, context) for b in point_batches if b != batch] + [(batch, context)]
    if short_context:
        runs = [(b, short_context) for b in sorted(set(point_batches + [batch]))] + runs
    breakdown = {}
    for b, c in runs:
        sb, keys = _synthetic_decode_batch(engine, b, c, key_base)
        key_base += 1000
        ms, clocks, launches = _time_graph(engine, sb, args.steps, args.warmup)
        if (b, c) == (batch, context):
            main = (ms, clocks, launches)
            if not args.no_breakdown:
                engine.runner.timed_step(sb)                                    # once untimed: lazily loaded kernels
                breakdown["decode"] = _rounded(engine.runner.timed_step(sb)[1])
        else:
            points[f"decode_b{b}" + ("" if c == context else f"_ctx{c}")] = round(b / ms * 1e3, 1)
        for k in keys:
            engine.cache.close(k)
    ms_per_step, clocks, launches = main
    value = batch / ms_per_step * 1e3
    achieved = decode_bytes(cfg, batch, context) / (ms_per_step * 1e-3) / 1e9
    if not args.no_breakdown:
        engine.cache.open(800000, "bench")
        engine.cache.ensure(800000, prompt_len, 0)
        sb = engine._rt.StepBatch(engine.cache)
        sb.add(800000, prompt, 0, [prompt_len - 1])
        breakdown["prefill"] = _rounded(engine.runner.timed_step(sb)[1])
        engine.cache.close(800000)

    # ---- end to end through the entry point: real prompts, scheduling, sampling, host tokens in and out
    e2e = None
    if not args.no_e2e:
        e2e = _end_to_end(engine, cfg, batch, context, args.steps, max(args.warmup, 3), g)
        if batch != 1 and 1 in point_batches:
            e2e["decode_b1"] = _end_to_end(engine, cfg, 1, context, args.steps, max(args.warmup, 3), g)["value"]
        # the same with every row drawn at a temperature with a top-k and a nucleus cut (on the device)
        e2e["top_k_top_p"] = _end_to_end(engine, cfg, batch, context, args.steps, max(args.warmup, 3), g, cuts=True)["value"]

    return {
        "metric": f"{SHAPES[args.shape]} decode tok/s at batch {batch}, context {context} (bf16, one B200)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), uniform token ids, random cache contents)",
        "impl": "ours",
        "config": {"model": f"{SHAPES[args.shape].lower()}-shape", "layers": cfg.num_hidden_layers, "layers_of_named_config": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": batch, "seq_len": context, "page_size": page, "prefill_tokens": prompt_len,
                   "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights + cache read every step)",
                   "peaks": pk["source"], "hbm_peak_gbs": pk["hbm_gbs"], "bf16_peak_tflops": pk["bf16_tflops"]},
        "e2e": e2e, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "breakdown": breakdown, "clocks": clocks, "gpu_launches": launches,
    }


def run_profile(args) -> dict:
    """A few eager steps (no CUDA graph) of one kind, small enough to sit under a
    profiler: ``--profile decode`` (batch x context synthetic cache) or
    ``--profile prefill`` (one 2,048-token prompt)."""
    import torch

    from stride_b200 import Engine

    cfg, full_layers = bench_config(args.layers, args.shape)
    batch, context = args.batch, args.context
    engine = Engine(config=cfg, random_weights=0, dtype="bfloat16", block_size=16,
                    num_blocks=(batch * (context + 64) + 4096) // 16, max_batch_tokens=2048, max_batch_seqs=64,
                    max_model_len=context + 512, prefix_caching=False, cuda_graphs=False)
    for pages in engine.device_cache.pages:
        pages.normal_(0.0, 0.5)
    if args.profile == "decode":
        step_batch, _ = _synthetic_decode_batch(engine, batch, context, 1000)
    else:
        g = torch.Generator().manual_seed(1)
        engine.cache.open(1, "bench")
        engine.cache.ensure(1, 2048, 0)
        step_batch = engine._rt.StepBatch(engine.cache)
        step_batch.add(1, torch.randint(0, cfg.vocab_size, (2048,), generator=g).tolist(), 0, [2047])
    for _ in range(args.warmup + args.steps):
        engine.runner.step(step_batch)
    torch.cuda.synchronize()
    return {"profiled": args.profile, "layers": cfg.num_hidden_layers, "layers_of_named_config": full_layers, "batch": batch,
            "context": context, "steps": args.warmup + args.steps}


# --------------------------------------------------------------------- reference
def run_reference(args) -> dict:
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "stride_worker")):
        return {"impl": "reference", "unavailable": "baseline/_ref holds no stride_worker package (the offline install was not done here)"}
    sys.path.insert(0, ref)
    try:
        import torch
        from stride_worker.cache import PagedKVCache
        from stride_worker.model import StrideModel
        from stride_worker.protocol import SequenceWork
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"the reference does not import: {type(e).__name__}: {e}"[:300]}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}

    from stride_b200.config import preset
    d = preset("llama3.1-8b")
    if args.layers:
        d["num_hidden_layers"] = args.layers
    dev, dt = torch.device("cuda"), torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(0)
    H, I, V, L = d["hidden_size"], d["intermediate_size"], d["vocab_size"], d["num_hidden_layers"]
    q, kv = d["num_attention_heads"] * d["head_dim"], d["num_key_value_heads"] * d["head_dim"]

    def mat(r, c):
        return (torch.randn(r, c, generator=g, device=dev, dtype=torch.float32) * 0.02).to(dt)

    state = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": torch.ones(H, device=dev, dtype=dt),
             "lm_head.weight": mat(V, H)}
    for i in range(L):
        p = f"model.layers.{i}"
        state.update({f"{p}.input_layernorm.weight": torch.ones(H, device=dev, dtype=dt),
                      f"{p}.post_attention_layernorm.weight": torch.ones(H, device=dev, dtype=dt),
                      f"{p}.self_attn.q_proj.weight": mat(q, H), f"{p}.self_attn.k_proj.weight": mat(kv, H),
                      f"{p}.self_attn.v_proj.weight": mat(kv, H), f"{p}.self_attn.o_proj.weight": mat(H, q),
                      f"{p}.mlp.gate_proj.weight": mat(I, H), f"{p}.mlp.up_proj.weight": mat(I, H),
                      f"{p}.mlp.down_proj.weight": mat(H, I)})
    model = StrideModel(d, state, dev, dt)
    batch, context, page = args.batch, args.context, 16
    pages_per_seq = (context + page - 1) // page + 1
    cache = PagedKVCache(model.cache_spec(batch * pages_per_seq + 4, page))
    tokens = torch.randint(0, V, (batch,), generator=torch.Generator().manual_seed(1)).tolist()
    work = [SequenceWork(seq=i, tokens=[tokens[i]], position=context - 1,
                         blocks=list(range(i * pages_per_seq, (i + 1) * pages_per_seq)), needs_logits=True) for i in range(batch)]
    for _ in range(max(args.warmup, 3)):
        model.forward(work, cache)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler() as clocks:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        start.record()
        produced = 0
        for _ in range(args.steps):
            _, logits, _ = model.forward(work, cache)
            produced += len(logits.to("cpu", torch.float32).argmax(-1).tolist())   # host tokens out, as its worker returns logits
        end.record()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    ms = start.elapsed_time(end) / args.steps
    prompt = torch.randint(0, V, (2048,), generator=torch.Generator().manual_seed(2)).tolist()
    pw = [SequenceWork(seq=0, tokens=prompt, position=0, blocks=list(range(2048 // page)), needs_logits=True)]
    model.forward(pw, cache)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    model.forward(pw, cache)
    torch.cuda.synchronize()
    prefill_ms = (time.perf_counter() - t1) * 1e3
    return {"metric": "Llama-3.1-8B decode tok/s at batch 8, context 8192 (bf16, one B200)", "impl": "reference",
            "value": round(batch / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, zeroed cache)",
            "config": {"model": "llama-3.1-8b-shape", "layers": L, "global_batch": batch, "seq_len": context,
                       "page_size": page, "parallelism": "single-gpu"},
            "e2e": {"value": round(produced / elapsed, 1), "unit": "tokens/s", "h2d_bytes_per_step": batch * 16,
                    "d2h_bytes_per_step": batch * V * 4},
            "prefill": {"value": round(2048 / prefill_ms * 1e3, 1), "tokens": 2048, "ms": round(prefill_ms, 2)},
            "clocks": clocks.summary, "gpu_launches": 0}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=8192)
    p.add_argument("--shape", default="llama3.1-8b", choices=sorted(SHAPES),
                   help="layer sizes of another named model (the headline is the default)")
    p.add_argument("--layers", type=int, default=None, help="fewer layers than the named configuration (reported in config)")
    p.add_argument("--no-e2e", action="store_true", help="skip the end-to-end measurement")
    p.add_argument("--points", default="1,64", help="batch sizes of the extra decode points (comma-separated)")
    p.add_argument("--no-breakdown", action="store_true", help="skip the per-class times of one decode step and the prefill")
    p.add_argument("--profile", choices=["decode", "prefill"], default=None,
                   help="run a few eager steps of one kind for a profiler instead of measuring")
    args = p.parse_args(argv)
    if args.gpus != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"unsupported": f"this engine runs on one GPU; --gpus {args.gpus} is not measured"}))
        return 2
    if args.profile:
        print(json.dumps(run_profile(args)))
        return 0
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
