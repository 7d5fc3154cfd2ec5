"""Command line of the engine.

    stride-b200 generate --model DIR --prompt-tokens 1,2,3 --max-tokens 16 --temperature 0
    stride-b200 random-model --preset tiny-a --seed 1 --out DIR
    stride-b200 replay --model DIR --dtype float32 --out DIR --max-tokens 1024 < trace.jsonl

Option names and defaults follow the reference where it has them: ``--model``,
``--dtype`` (bfloat16), ``--block-size`` (16), ``--num-blocks`` (sized from free
memory), ``--activation-reserve`` (0.15) from its worker
(python/stride_worker/worker.py:252-280); ``--max-batch-tokens`` (2048),
``--max-batch-seqs`` (256), ``--max-model-len`` (8192) from its server
(crates/stride-server/src/main.rs:86-107); sampling options from
crates/stride-core/src/sampling.rs:5-31. Prompts are token ids; there is no
tokenizer in this package.
"""

from __future__ import annotations

import argparse
import json
import sys


def _add_engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", help="folder with config.json and *.safetensors")
    p.add_argument("--preset", help="a built-in shape instead of --model (needs --random-weights)")
    p.add_argument("--config", help="a config.json instead of --model (needs --random-weights)")
    p.add_argument("--random-weights", type=int, metavar="SEED", help="seeded random weights for --preset/--config")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--block-size", type=int, default=16, help="tokens per KV page")
    p.add_argument("--num-blocks", type=int, default=None, help="override the page count; by default sized from free device memory")
    p.add_argument("--activation-reserve", type=float, default=0.15, help="share of free memory held back for activations")
    p.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget per step")
    p.add_argument("--max-batch-seqs", type=int, default=256, help="sequence budget per step")
    p.add_argument("--max-model-len", type=int, default=8192, help="longest prompt plus completion accepted")
    p.add_argument("--max-queued", type=int, default=1024, help="requests that may wait for admission before more are refused")
    p.add_argument("--watermark", type=float, default=0.01, help="share of pages held back from admission")
    p.add_argument("--no-chunked-prefill", action="store_true")
    p.add_argument("--no-prefix-caching", action="store_true")
    p.add_argument("--no-cuda-graphs", action="store_true")
    p.add_argument("--no-chain-steps", action="store_true",
                   help="wait for every decode step's tokens before the next step is launched")
    p.add_argument("--host-ranking", action="store_true",
                   help="draw top-k and nucleus rows on the host from their logits instead of on the device")
    p.add_argument("--check-invariants", action="store_true", help="verify the cache manager after every step")


def _add_sampling_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--max-tokens", type=int, default=128)
    p.add_argument("--min-tokens", type=int, default=0)
    p.add_argument("--stop-token", type=int, action="append", default=[])
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--ignore-eos", action="store_true")


def _engine(args):
    from .config import preset
    from .engine import Engine

    options = dict(dtype=args.dtype, block_size=args.block_size, num_blocks=args.num_blocks,
                   activation_reserve=args.activation_reserve, max_batch_tokens=args.max_batch_tokens,
                   max_batch_seqs=args.max_batch_seqs, max_model_len=args.max_model_len, max_queued=args.max_queued,
                   watermark=args.watermark,
                   chunked_prefill=not args.no_chunked_prefill, prefix_caching=not args.no_prefix_caching,
                   cuda_graphs=not args.no_cuda_graphs, chain_steps=not args.no_chain_steps, device_ranking=not args.host_ranking,
                   check_invariants=args.check_invariants)
    if args.model:
        return Engine(args.model, **options)
    if args.preset or args.config:
        if args.random_weights is None:
            raise SystemExit("--preset/--config needs --random-weights SEED")
        cfg = preset(args.preset) if args.preset else json.load(open(args.config))
        return Engine(config=cfg, random_weights=args.random_weights, **options)
    raise SystemExit("give --model DIR, or --preset/--config with --random-weights SEED")


def _prompts(args) -> list:
    prompts = []
    for text in args.prompt_tokens or []:
        prompts.append([int(t) for t in text.replace(",", " ").split()])
    if args.prompt_file:
        with open(args.prompt_file) as f:
            data = json.load(f)
        prompts += [list(map(int, p)) for p in (data if data and isinstance(data[0], list) else [data])]
    if not prompts:
        raise SystemExit("give --prompt-tokens 1,2,3 (repeatable) or --prompt-file FILE.json")
    return prompts


def cmd_generate(args) -> int:
    from .sampling import SamplingParams

    params = SamplingParams(args.temperature, args.top_p, args.top_k, args.max_tokens, args.min_tokens, args.stop_token,
                            args.seed, args.ignore_eos)
    engine = _engine(args)
    for out in engine.generate(_prompts(args), params):
        print(json.dumps({"request": out.request_id, "tokens": out.tokens, "finish_reason": out.finish_reason,
                          "prompt_tokens": out.prompt_len, "cached_prompt_tokens": out.cached_prompt_tokens,
                          "seed": out.seed}))
    if args.metrics:
        print(json.dumps(engine.metrics()), file=sys.stderr)
    return 0


def cmd_random_model(args) -> int:
    from .config import config_from_dict, preset
    from .engine import write_random_model

    cfg = preset(args.preset) if args.preset else json.load(open(args.config))
    path = write_random_model(config_from_dict(cfg), args.seed, args.out, stored_dtype=args.dtype,
                              vector_jitter=args.norm_jitter)
    print(path)
    return 0


def add_replay_options(p: argparse.ArgumentParser) -> None:
    """The options of trace replay; ``bin/trace_run`` and the ``replay`` command share them."""
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens that live requests hold at any time (each rounded up to a multiple of 64)")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--max-requests", type=int, default=8, help="most requests live at a time")


def cmd_replay(args) -> int:
    """Reads steps from standard input, one JSON object a line, runs each through a ``TraceSession`` and writes
    ``<out>/<step>.f32`` (little-endian float32 [wanted, vocab]) for every step that wants logits; prints
    ``done <step>`` after every step."""
    import os

    print("[trace_run] loading the engine", file=sys.stderr, flush=True)
    import numpy as np

    from .engine.trace import TraceSession

    os.makedirs(args.out, exist_ok=True)
    session = TraceSession(args.model, dtype=args.dtype, max_tokens=args.max_tokens, block_size=args.block_size,
                           max_requests=args.max_requests)
    print("[trace_run] ready", file=sys.stderr, flush=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        logits = session.run_step(step)
        if logits is not None:
            np.ascontiguousarray(logits.numpy(), dtype="<f4").tofile(os.path.join(args.out, f"{step['step']}.f32"))
        print(f"done {step['step']}", flush=True)
    return 0


def cmd_plan(args) -> int:
    """Weights, activation reserve and cache pages for a model on one device, without loading anything
    (the reference's planner, crates/stride-model/examples/plan.rs, and its server's ``--dry-run``)."""
    from .config import PlanError, config_from_dict, load_config, plan_memory, preset

    if args.model:
        config = load_config(args.model)
    else:
        config = config_from_dict(preset(args.preset) if args.preset else json.load(open(args.config)))
    try:
        plan = plan_memory(config, args.dtype, int(args.memory_gib * (1 << 30)), args.block_size, args.activation_reserve,
                           name=args.preset or args.model or args.config)
    except PlanError as e:
        print(f"does not fit: {e}", file=sys.stderr)
        return 1
    print(plan.describe())
    for context in args.context:
        print(f"  requests of {context:<7} {plan.concurrent_sequences(context):9d}      at once")
    return 0


def cmd_diagnose_prefill(args) -> int:
    """Portions against the whole prompt, logits of the last token (the reference's ``stride-diagnose prefill``,
    python/stride_worker/diagnose/cli.py:44-73)."""
    from .diagnose import report
    from .diagnose.prefill import PrefillProbe, seeded_prompt
    from .engine.trace import TraceSession

    session = TraceSession(args.model, dtype=args.dtype, max_tokens=-(-args.tokens // 64) * 64, block_size=args.block_size,
                           max_requests=2)
    tokens = seeded_prompt(session.model.vocab, args.tokens, args.seed)
    sizes = [int(s) for s in args.chunk.split(",") if s.strip()]
    print(f"prompt: {len(tokens)} tokens, chunk sizes {sizes}\n")
    all_ok = True
    for size, agreement in PrefillProbe(session).sweep(tokens, sizes).items():
        ok, _ = agreement.verdict(args.dtype)
        all_ok &= ok
        print(report(f"chunk={size}", agreement, args.dtype))
        print()
    print("Portions match the whole prompt." if all_ok else
          "Portions do not match the whole prompt: look at the mask and the position arithmetic at a portion's first token.")
    return 0 if all_ok else 1


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="stride-b200", description="LLM inference engine for one B200 (Llama 3 dense decoder)")
    sub = parser.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    _add_engine_options(g)
    _add_sampling_options(g)
    g.add_argument("--prompt-tokens", action="append", help="comma- or space-separated token ids; repeatable")
    g.add_argument("--prompt-file", help="JSON: a list of token ids or a list of such lists")
    g.add_argument("--metrics", action="store_true", help="print engine counters to stderr at the end")
    g.set_defaults(run=cmd_generate)

    r = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    r.add_argument("--preset")
    r.add_argument("--config")
    r.add_argument("--seed", type=int, required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="element type stored in the file")
    r.add_argument("--norm-jitter", type=float, default=0.0, help="norm weights are 1 + N(0, this)")
    r.set_defaults(run=cmd_random_model)

    t = sub.add_parser("replay", help="feed a trace of token ids step by step and write logits (see bin/trace_run)")
    add_replay_options(t)
    t.set_defaults(run=cmd_replay)

    pl = sub.add_parser("plan", help="what fits: weights, activation reserve and cache pages on one device (no GPU needed)")
    pl.add_argument("--model", help="folder with config.json")
    pl.add_argument("--preset")
    pl.add_argument("--config")
    pl.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    pl.add_argument("--memory-gib", type=float, default=183359 / 1024, help="device memory (default: a B200)")
    pl.add_argument("--block-size", type=int, default=16)
    pl.add_argument("--activation-reserve", type=float, default=0.15)
    pl.add_argument("--context", type=int, action="append", default=[], help="also print how many requests of this length fit; repeatable")
    pl.set_defaults(run=cmd_plan)

    d = sub.add_parser("diagnose", help="probes of the engine's numerics")
    dsub = d.add_subparsers(dest="probe", required=True)
    dp = dsub.add_parser("prefill", help="a prompt in portions against the prompt whole")
    dp.add_argument("--model", required=True)
    dp.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    dp.add_argument("--tokens", type=int, default=5000)
    dp.add_argument("--chunk", default="512,1024,2048", help="comma-separated portion sizes")
    dp.add_argument("--seed", type=int, default=0)
    dp.add_argument("--block-size", type=int, default=16)
    dp.set_defaults(run=cmd_diagnose_prefill)

    args = parser.parse_args(argv)
    if args.command == "random-model" and not (args.preset or args.config):
        parser.error("random-model needs --preset or --config")
    if args.command == "plan" and not (args.model or args.preset or args.config):
        parser.error("plan needs --model, --preset or --config")
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())
