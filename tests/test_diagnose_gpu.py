"""The prefill probe on the GPU: a prompt in portions against the prompt whole through the engine's own trace
replay, the capture hook against the plain implementation's hidden states, and the command line."""

import os
import subprocess
import sys

import pytest
import torch

import plain_llama as plain
from helpers import TINY, read_model_dir, seeded_state, write_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", params=[("A", "float32"), ("B", "float32"), ("D", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def probe_case(request, tmp_models):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    name, dtype = request.param
    cfg = TINY[name]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_model_dir(str(tmp_models / f"diagnose_{name}_{dtype}"), cfg, seeded_state(cfg, 77, std=0.05), stored)
    return name, dtype, cfg, folder


def test_portions_match_the_whole_prompt(probe_case):
    from stride_b200.diagnose import first_divergence
    from stride_b200.diagnose.prefill import PrefillProbe, seeded_prompt
    from stride_b200.engine.trace import TraceSession

    name, dtype, cfg, folder = probe_case
    n = 150
    session = TraceSession(folder, dtype, max_tokens=192, block_size=16, max_requests=2)
    tokens = seeded_prompt(cfg["vocab_size"], n, 3)
    probe = PrefillProbe(session)
    results = probe.sweep(tokens, [2, 16, 33, 149])
    for size, agreement in results.items():
        ok, why = agreement.verdict(dtype)
        assert ok, f"{name} {dtype} chunk={size}: {why}"
        if dtype == "float32":
            assert agreement.max_abs_diff == 0.0, f"float32 logits must not depend on the cutting (chunk={size})"
    assert probe.check(tokens, 7).verdict(dtype)[0]
    # the capture hook: hidden states after every layer, against the plain implementation
    logits, states = probe.run_prompt(tokens, capture=True)
    _, stored = read_model_dir(folder)
    want_states: list = []
    want = plain.forward(cfg, stored, tokens, torch.float64, want_states)
    assert len(states) == cfg["num_hidden_layers"] and states[0].shape == (n, cfg["hidden_size"])
    floor = 0.9999999 if dtype == "float32" else 0.999
    assert first_divergence(states, want_states, cosine_floor=floor) is None
    from stride_b200.diagnose import compare_logits
    ok, why = compare_logits(logits, want[-1:]).verdict(dtype)
    assert ok, why
    assert session.model.capture is None and session.runner.cuda_graphs, "the probe leaves the session as it found it"


def test_the_diagnose_command_line(probe_case):
    name, dtype, cfg, folder = probe_case
    proc = subprocess.run([sys.executable, "-m", "stride_b200", "diagnose", "prefill", "--model", folder, "--dtype", dtype,
                           "--tokens", "100", "--chunk", "5,64"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "chunk=5 [same]" in proc.stdout and "chunk=64 [same]" in proc.stdout
    assert "Portions match the whole prompt." in proc.stdout
