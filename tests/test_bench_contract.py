"""What bench.py promises without a GPU: more than one GPU is refused with one line and exit code 2; the arithmetic
behind its fractions (bytes of a decode step, FLOPs of a prefill) matches the sizes of the named shapes."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_more_than_one_gpu_is_refused_with_one_line():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 2
    lines = [l for l in proc.stdout.strip().splitlines() if l.strip()]
    assert len(lines) == 1, proc.stdout


def test_bytes_and_flops_of_the_named_shape():
    sys.path.insert(0, ROOT)
    import bench
    cfg, layers = bench.bench_config(None, "llama3.1-8b")
    assert layers == 32
    # every matrix once (15.01 GB) and 131,072 bytes of keys and values a token
    assert abs(bench.decode_bytes(cfg, 8, 8192) / 1e9 - 23.60) < 0.01
    assert abs(bench.decode_bytes(cfg, 1, 2048) / 1e9 - 15.28) < 0.01
    assert abs(bench.decode_bytes(cfg, 64, 8192) / 1e9 - 83.73) < 0.01
    # 28.59 TFLOP of products, 1.10 of causal attention and the head for one row
    assert abs(bench.prefill_flops(cfg, 2048) / 1e12 - 29.7) < 0.05
    few, full = bench.bench_config(4, "llama3.1-8b")
    assert few.num_hidden_layers == 4 and full == 32


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    sys.path.insert(0, ROOT)
    import bench
    pk = bench.peaks()
    assert pk["hbm_gbs"] > 1000 and pk["bf16_tflops"] > 100 and pk["bf16_tflops_burst"] >= pk["bf16_tflops"]
    measured = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(measured):
        d = json.load(open(measured))
        assert abs(pk["hbm_gbs"] - float(d["hbm_gbs"])) < 1e-6
