"""Python faces of the CUDA kernels.

Each function checks its tensors (device, dtype, contiguity, sizes) and calls
one ``extern "C"`` launcher through ctypes on the current torch stream. There is
no CPU path and no fallback: a tensor that is not on a CUDA device, a missing
compiler or a size that a kernel refuses raises an error.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

_ERRORS = {-1: "bad argument", -2: "size not supported by this kernel"}


class KernelError(RuntimeError):
    pass


_bound: dict[str, ctypes._CFuncPtr] = {}

_SIGNATURES = {
    # name: (library, argtypes)
    "stride_embed_gather": ("elementwise", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_add_rmsnorm": ("elementwise", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]),
    "stride_add_residual": ("elementwise", [c_void_p, c_void_p, c_longlong, c_int, c_void_p]),
    "stride_zero_fresh_state": ("elementwise", [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "stride_rope_kv_write": ("elementwise", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_silu_mul": ("elementwise", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_gemm_tc_gated": ("gemm_bf16_tc", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float,
                                              c_void_p]),
    "stride_gemm_nt_f32": ("gemm_f32", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "stride_paged_attention_generic": ("attention_generic", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                                             c_int, c_int, c_void_p]),
    "stride_gemm_tc_skinny": ("gemm_bf16_tc", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_longlong,
                                               c_void_p, c_int, c_void_p, c_void_p]),
    "stride_gemm_tc_clustered": ("gemm_bf16_tc", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "stride_gemm_rows": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "stride_gemm_rows_add": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "stride_gemm_rows_gated": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_float,
                                                  c_void_p, c_void_p]),
    "stride_gemm_rows_qkv_rope": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                     c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                     c_int, c_float, c_void_p, c_void_p]),
    "stride_gemm_rows_add_norm": ("gemm_bf16_rows", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int,
                                                     c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "stride_gemm_stream_bf16": ("gemm_bf16_stream", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "stride_gemm_stream_qkv_rope": ("gemm_bf16_stream", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                         c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                         c_void_p, c_int, c_float, c_void_p, c_void_p]),
    "stride_gemm_stream_add_norm": ("gemm_bf16_stream", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong,
                                                         c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "stride_scale_rows": ("elementwise", [c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p]),
    "stride_paged_decode_attention": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                           c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int,
                                                           c_float, c_int, c_int, c_void_p]),
    "stride_paged_decode_attention_tma": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                                               c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                                                               c_int, c_float, c_int, c_int, c_void_p, c_void_p]),
    "stride_paged_prefill_attention": ("attention_prefill", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                             c_int, c_float, c_int, c_void_p]),
    "stride_paged_prefill_attention_tc": ("attention_prefill_tc", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                                   c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                                   c_int, c_int, c_float, c_int, c_void_p, c_void_p]),
    "stride_sample_ranked": ("sampling_ranked", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_longlong, c_void_p]),
    "stride_sample_rows": ("sampling", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_longlong, c_void_p]),
}


def _fn(name: str, what: str | None = None):
    f = _bound.get(name)
    if f is None:
        library, argtypes = _SIGNATURES[name]
        f = getattr(build.load_kernel_library(library), name)
        f.argtypes = argtypes
        f.restype = c_int
        _bound[name] = f
    if _timer is not None:
        return _timer.timed(what or _CLASS_OF.get(name, name), f)
    return f


# ---------------------------------------------------------------- time per class of kernel
# What a launcher counts as when the time of a step is split up. Matrix products say more (their shape) at the call.
_CLASS_OF = {
    "stride_embed_gather": "embedding", "stride_add_rmsnorm": "norm", "stride_add_residual": "residual sum",
    "stride_scale_rows": "norm", "stride_zero_fresh_state": "state slots", "stride_rope_kv_write": "rotation + cache write",
    "stride_silu_mul": "silu * up", "stride_paged_attention_generic": "attention (exact kernel)",
    "stride_paged_decode_attention_tma": "attention (decode)", "stride_paged_prefill_attention": "attention (prefill, mma.sync)",
    "stride_paged_prefill_attention_tc": "attention (prefill, tcgen05)", "stride_sample_rows": "sampling", "stride_sample_ranked": "sampling",
}


class KernelTimer:
    """Device time per class of kernel inside a step, from CUDA events around every launch (the reference records
    one duration per pass, python/stride_worker/model.py:238-240,343-345; this splits it up). Use::

        with ops.KernelTimer() as timer:
            model.forward(ctx)              # eagerly: a captured graph has no place for events
        timer.milliseconds()                # {"attention (decode)": 1.52, "product 6144x4096 (qkv + rotation)": 1.18, ...}

    The events stand between the kernels, so launches do not overlap their predecessors' tails as they do in a
    real step: the classes' shares are right, their sum is somewhat above the step's own time."""

    def __init__(self):
        self.spans: list = []       # (class, start event, end event)

    def __enter__(self):
        global _timer
        if _timer is not None:
            raise KernelError("a KernelTimer is active already")
        _timer = self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = None

    def timed(self, what: str, call):
        def run(*args):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            code = call(*args)
            end.record()
            self.spans.append((what, start, end))
            return code
        return run

    def milliseconds(self) -> dict:
        """Synchronises; class -> summed device time, largest first."""
        torch.cuda.synchronize()
        out: dict = {}
        for what, start, end in self.spans:
            out[what] = out.get(what, 0.0) + start.elapsed_time(end)
        return dict(sorted(out.items(), key=lambda kv: -kv[1]))


_timer: KernelTimer | None = None


# How many of the package's own kernels were launched (library matrix products
# are not counted). A captured graph counts its launches once, at capture.
counters = {"launches": 0}


def _check(code: int, name: str) -> None:
    if code == 0:
        counters["launches"] += 1
        return
    if code in _ERRORS:
        raise KernelError(f"{name}: {_ERRORS[code]}")
    raise KernelError(f"{name}: CUDA error {code} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle. Asked for on every launch, so through the one C call when torch has it
    (``torch.cuda.current_stream()`` builds a Python object every time)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device; stride_b200 has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t, name: str, dtype=None) -> int | None:
    return None if t is None else _dev(t, name, dtype)


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not supported (float32 and bfloat16 are)") from None


def require_device() -> None:
    """Fails loudly when the product path cannot run."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: stride_b200 runs its models on the GPU only")


# ------------------------------------------------------------------ elementwise
def embed_gather(ids, seq_of_token, table, out) -> None:
    tokens, hidden = out.shape
    _check(_fn("stride_embed_gather")(_dev(ids, "ids", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
                                      _dev(table, "table"), _dev(out, "out", torch.float32), tokens, hidden,
                                      table.shape[0], _code(table.dtype), _stream()), "embed_gather")


def add_rmsnorm(residual, delta, weight, out, eps: float, rows=None) -> None:
    """``x = residual (+ delta)``; writes x back to ``residual`` (unless ``rows``
    selects source rows) and ``rmsnorm(x) * weight`` to ``out``."""
    num_rows, hidden = out.shape
    if delta is not None and delta.dtype != out.dtype:
        raise KernelError("delta and out must have the same element type")
    _check(_fn("stride_add_rmsnorm")(_dev(residual, "residual", torch.float32), _opt(delta, "delta"),
                                     _dev(weight, "weight", torch.float32), _dev(out, "out"),
                                     _opt(rows, "rows", torch.int32), num_rows, hidden, float(eps), _code(out.dtype),
                                     _stream()), "add_rmsnorm")


def add_residual(residual, delta) -> None:
    _check(_fn("stride_add_residual")(_dev(residual, "residual", torch.float32), _dev(delta, "delta"), delta.numel(),
                                      _code(delta.dtype), _stream()), "add_residual")


def zero_fresh_state(state, state_slot, q_start, q_len, positions) -> None:
    """Clears ``state[slot]`` for every sequence of the step whose first token sits at position 0 (``state``:
    [num_slots, ...] of a 4-byte element type; the index arrays are the step's, at their layout's capacity)."""
    if state.element_size() != 4:
        raise KernelError("state rows must have a 4-byte element type")
    row_bytes = (state.numel() // state.shape[0]) * 4
    _check(_fn("stride_zero_fresh_state")(_dev(state, "state"), row_bytes, state.shape[0], _dev(state_slot, "state_slot", torch.int32),
                                          _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32),
                                          _dev(positions, "positions", torch.int32), q_len.shape[0], _stream()), "zero_fresh_state")


def rope_kv_write(qkv, bias, positions, slot_mapping, cos, sin, k_pages, v_pages, nq: int, nkv: int, hd: int,
                  page_size: int, rotate: bool = True) -> None:
    tokens = qkv.shape[0]
    if qkv.shape[1] != (nq + 2 * nkv) * hd:
        raise KernelError("qkv has the wrong width")
    if k_pages.dtype != qkv.dtype or v_pages.dtype != qkv.dtype:
        raise KernelError("cache pages and activations must have the same element type")
    _check(_fn("stride_rope_kv_write")(_dev(qkv, "qkv"), _opt(bias, "bias", torch.float32),
                                       _dev(positions, "positions", torch.int32),
                                       _opt(slot_mapping, "slot_mapping", torch.int32), _dev(cos, "cos", torch.float32),
                                       _dev(sin, "sin", torch.float32), _dev(k_pages, "k_pages"), _dev(v_pages, "v_pages"),
                                       tokens, nq, nkv, hd, page_size, int(rotate), _code(qkv.dtype), _stream()),
           "rope_kv_write")


def silu_mul(inp, out, block: int | None = None) -> None:
    """``out = silu(gate) * up`` for ``inp`` = [tokens, 2 * inter] whose gate and up columns alternate in
    blocks of ``block`` columns (default: all gate columns, then all up columns)."""
    tokens, inter = out.shape
    if inp.shape != (tokens, 2 * inter) or inp.dtype != out.dtype:
        raise KernelError("silu_mul wants [tokens, 2*inter] in and [tokens, inter] out of one element type")
    _check(_fn("stride_silu_mul")(_dev(inp, "in"), _dev(out, "out"), tokens, inter, inter if block is None else int(block),
                                  _code(out.dtype), _stream()), "silu_mul")


# ----------------------------------------------------------------------- matmul
# Up to this many rows (tokens: a decode step) the bfloat16 products run on the package's own kernels, which
# stream the weights once; above it the library product is called, as the reference's engine does.
# STRIDE_B200_TC_GEMM=0 switches both off, STRIDE_TC_MAX_TOKENS moves the limit (the tcgen05 kernel takes up to
# 256 rows, the weight-streaming kernel 16; measured at 32 and 64 rows the library is level or faster).
import os as _os

TC_GEMM_MAX_TOKENS = 0 if _os.environ.get("STRIDE_B200_TC_GEMM", "1") == "0" else int(_os.environ.get("STRIDE_TC_MAX_TOKENS", "16"))
# The tcgen05 kernel (TMA ring, weight rows as the 128-row tile side) takes the weight matrices with at least this
# many 128-row tiles (gate/up, the head): with fewer, K has to be split over several CTAs and the partial tiles go
# through global memory. STRIDE_TC_MIN_TILES=0 sends every product to it.
TC_GEMM_MIN_TILES = int(_os.environ.get("STRIDE_TC_MIN_TILES", "100"))
# The smaller matrices (QKV, O, down) go to the weight-streaming kernel, which gives a CTA 16 rows and all of K.
# STRIDE_B200_STREAM_GEMM=0 sends them to the library product instead.
STREAM_GEMM = _os.environ.get("STRIDE_B200_STREAM_GEMM", "1") != "0"
_TC_TICKETS = 8192
_tc_state: dict = {}


def _device_key(device) -> torch.device:
    """``cuda`` and ``cuda:<current>`` are one device: state kept per device must not be kept twice."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
    return device


def _tc_buffers(device, partial_floats: int):
    device = _device_key(device)
    st = _tc_state.get(device)
    if st is None:
        st = {"tickets": torch.zeros(_TC_TICKETS, dtype=torch.int32, device=device),
              "status": torch.zeros(64, dtype=torch.int32, device=device), "partials": None, "retired": []}
        _tc_state[device] = st
    if partial_floats and (st["partials"] is None or st["partials"].numel() < partial_floats):
        if st["partials"] is not None:
            st["retired"].append(st["partials"])      # a captured graph may still use it
        st["partials"] = torch.empty(max(partial_floats, 1 << 20), dtype=torch.float32, device=device)
    return st


def _tc_scratch_floats(n_out: int, tokens: int, k: int) -> int:
    f = _bound.get("stride_gemm_tc_scratch_floats")
    if f is None:
        f = build.load_kernel_library("gemm_bf16_tc").stride_gemm_tc_scratch_floats
        f.argtypes = [c_int, c_int, c_int]
        f.restype = c_longlong
        _bound["stride_gemm_tc_scratch_floats"] = f
    return int(f(n_out, tokens, k))


def tc_status(device=None) -> int:
    """0, or the code of the first bounded wait that ran out inside the tcgen05
    kernels (1 producer, 2 tensor-core issuer, 3 epilogue). Synchronises."""
    codes = [int(st["status"][0].item()) for dev, st in _tc_state.items() if device is None or dev == _device_key(device)]
    return next((c for c in codes if c), 0)


_WAIT_CODES = {1: "matrix product: producer", 2: "matrix product: tensor-core issuer", 3: "matrix product: epilogue",
               31: "decode attention: a tile copy", 41: "weight-streaming product: a tile copy",
               51: "tokens-as-rows product: activation copies", 52: "tokens-as-rows product: weight copies",
               53: "tokens-as-rows product: tensor-core issuer", 54: "tokens-as-rows product: epilogue"}
_WAIT_CODES.update({c: "prefill attention (attention_prefill_tc.cu)" for c in range(11, 22)})
_OTHER_CODES = {32: "decode attention was given a token whose position is not below the context bound of its launch"}


def reset_kernel_status(device=None) -> None:
    """Sets the status word back to 0 (on ``device``, or wherever one exists), so that later steps are judged on
    their own: the kernels only ever write the first code into a word that is still 0."""
    for dev, st in _tc_state.items():
        if device is None or dev == _device_key(device):
            st["status"].zero_()


def raise_on_kernel_status(code: int, device=None) -> None:
    """Raises when ``code`` (the status word, read back by the caller) is not 0: a bounded wait inside a kernel ran
    out, or a kernel refused a row, so what the step wrote is not to be trusted. With ``device`` the word there is
    cleared first, so that the failure is reported once and the next step starts clean (the reference's worker
    reports a failed pass and keeps serving, python/stride_worker/worker.py:156-165)."""
    if not code:
        return
    if device is not None:
        reset_kernel_status(device)
    if code in _OTHER_CODES:
        raise KernelError(f"kernel status {code}: {_OTHER_CODES[code]}; the step's results are invalid")
    raise KernelError(f"a bounded wait inside a kernel ran out (code {code}: {_WAIT_CODES.get(code, 'unknown place')}); "
                      "the step's results are invalid")


def check_kernel_status(device=None) -> None:
    """Reads the status word (synchronises), clears it if it is set, and raises if a kernel recorded a failure."""
    code = tc_status(device)
    if code:
        reset_kernel_status(device)
    raise_on_kernel_status(code)


def status_tensor(device):
    """The device word that the tcgen05 kernels set on a timed-out wait (for callers that copy it with their own results)."""
    return _tc_buffers(device, 0)["status"]


def linear_tc(x, weight, out) -> bool:
    """``out = x @ weight.T`` on the tcgen05 kernel. Returns False when the kernel
    does not take the shape (the caller then uses the library product)."""
    m, k = x.shape
    n = weight.shape[0]
    st = _tc_buffers(x.device, _tc_scratch_floats(n, m, k))
    partials = st["partials"]
    code = _fn("stride_gemm_tc_skinny", f"product {n}x{k} (tcgen05)")(_dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out"),
                                        m, n, k, int(out.dtype == torch.float32),
                                        None if partials is None else partials.data_ptr(),
                                        0 if partials is None else partials.numel(), st["tickets"].data_ptr(), _TC_TICKETS,
                                        st["status"].data_ptr(), _stream())
    if code == -2:
        return False
    _check(code, "gemm_tc_skinny")
    return True


# The tcgen05 kernel with the CTAs of an output tile in a cluster (the parts of K meet in the first CTA's shared
# memory, nothing goes through global memory) takes up to 64 tokens. Measured over whole decode steps of the 8B shape
# at a context of 2,048 it is level with the library product at 17 and 32 tokens (4.51 against 4.44 ms, 5.11 against
# 5.02) and slower at 64 (7.3 against 6.3: there the library streams the small matrices in 48- and 64-row tiles
# through a 15-stage ring at about 0.6 of the memory bandwidth, this kernel's 128-row tiles with K split four ways at
# 0.35), so it is off by default: STRIDE_TC_CLUSTER_MAX_TOKENS=64 switches it on.
TC_CLUSTER_MAX_TOKENS = int(_os.environ.get("STRIDE_TC_CLUSTER_MAX_TOKENS", "0"))


def linear_tc_clustered(x, weight, out) -> bool:
    """``out = x @ weight.T`` for up to 64 rows of ``x`` on the clustered tcgen05 kernel. Returns False when the
    kernel does not take the shape."""
    m, k = x.shape
    n = weight.shape[0]
    code = _fn("stride_gemm_tc_clustered", f"product {n}x{k} (tcgen05, clusters)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out"), m, n, k,
        int(out.dtype == torch.float32), _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_tc_clustered")
    return True


# Decode steps of 17 to this many tokens (128 at the most) run the package's tcgen05 product with the tokens as the
# rows of the tile (gemm_bf16_rows.cu: one CTA per block of output features and all of K; residual sum and the
# statistics of the norm that follows, the norm's factor, rotation with cache write and SiLU * up in its epilogues).
# Off by default: it is level with the library product plus separate elementwise kernels where a 4096-row matrix
# gives every SM a CTA, and slower elsewhere. Whole decode steps from a graph, this kernel / library: 8B sizes at a
# context of 2,048, 17 tokens 4.43 / 4.44 ms, 24: 4.70 / 4.63, 32: 4.92 / 4.97, 40: 5.60 / 5.28, 64: 6.57 / 6.29,
# 128: 10.0 / 9.1; at a context of 1,024, 32 tokens 4.33 / 4.42; 3B sizes (3072-row matrices: 96 CTAs), 32 tokens at
# a context of 4,096 4.50 / 4.28. Every CTA reads all of the activations, which is more than its weights once there
# are more tokens than features in its block; the library shares them between the CTAs of a cluster.
ROWS_GEMM_MAX_TOKENS = min(128, int(_os.environ.get("STRIDE_ROWS_GEMM_MAX_TOKENS", "0")))


def rows_wanted(tokens: int) -> bool:
    """Whether a step of this many tokens runs its products on the tokens-as-rows kernel (the callers' policy; the
    ``linear_rows*`` functions themselves take up to 128 rows)."""
    return TC_GEMM_MAX_TOKENS < tokens <= ROWS_GEMM_MAX_TOKENS


def _rows_ok(x, m: int) -> bool:
    return m <= 128 and x.dtype == torch.bfloat16 and TC_GEMM_MAX_TOKENS > 0


def linear_rows(x, weight, out) -> bool:
    """``out = x @ weight.T`` (bfloat16 or float32 out) for up to 128 rows of ``x`` on the tokens-as-rows tcgen05 kernel.
    Returns False when the kernel does not take the shape."""
    m, k = x.shape
    n = weight.shape[0]
    code = _fn("stride_gemm_rows", f"product {n}x{k} (tcgen05, tokens as rows)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out"), m, n, k,
        int(out.dtype == torch.float32), _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_rows")
    return True


def linear_rows_add(x, weight, residual) -> bool:
    """``residual += bf16(x @ weight.T)`` (float32 residual) in one kernel, for 17 to 128 rows. False: not done."""
    m, k = x.shape
    n = weight.shape[0]
    if not _rows_ok(x, m) or residual.shape != (m, n):
        return False
    code = _fn("stride_gemm_rows_add", f"product {n}x{k} (tcgen05, tokens as rows, + residual)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(residual, "residual", torch.float32), m, n, k,
        _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_rows_add")
    return True


def linear_rows_add_norm(x, weight, residual, norm_weight, xt, partials) -> int:
    """``linear_add_norm`` for 17 to 128 rows: ``partials[cta, token]`` has 128 tokens a CTA. Returns the number of
    producer CTAs, or 0 when the kernel does not take the sizes."""
    m, k = x.shape
    n = weight.shape[0]
    if not (FOLD_NORMS and _rows_ok(x, m)) or residual.shape != (m, n):
        return 0
    count = c_int(0)
    code = _fn("stride_gemm_rows_add_norm", f"product {n}x{k} (tcgen05, tokens as rows, + residual, norm statistics)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(xt, "xt", torch.bfloat16),
        _dev(residual, "residual", torch.float32), _dev(norm_weight, "norm_weight", torch.float32),
        _dev(partials, "partials", torch.float32), partials.numel(), m, n, k, ctypes.byref(count), _status_ptr(x.device), _stream())
    if code == -2:
        return 0
    _check(code, "gemm_rows_add_norm")
    return count.value


ROWS_FOLD_STRIDE = 128      # tokens a CTA in the partials that ``linear_rows_add_norm`` writes


def linear_rows_gated(x, weight, out, folded=None) -> bool:
    """``out = silu(x @ gate.T) * (x @ up.T)`` for 17 to 128 rows; ``weight`` as for ``linear_gated_tc``; ``folded``: a
    FoldedNorm from ``linear_rows_add_norm`` whose ``xt`` is ``x``. False: not done."""
    m, k = x.shape
    inter = weight.shape[0] // 2
    if not _rows_ok(x, m) or out.shape != (m, inter) or (folded is not None and folded.stride != ROWS_FOLD_STRIDE):
        return False
    partials, count, eps = _fold_args(folded, ROWS_FOLD_STRIDE)
    code = _fn("stride_gemm_rows_gated", f"product 2x{inter}x{k} (tcgen05, tokens as rows, silu * up)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out", torch.bfloat16), m, inter, k,
        partials, count, eps, _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_rows_gated")
    return True


def linear_rows_qkv_rope(x, weight, qkv, bias, positions, slot_mapping, cos, sin, k_pages, v_pages, nq: int, nkv: int, hd: int,
                         page_size: int, rotate: bool, folded=None) -> bool:
    """``linear_qkv_rope`` for 17 to 128 rows of ``x`` (``folded``: from ``linear_rows_add_norm``). False: not done."""
    m, k = x.shape
    if not _rows_ok(x, m) or qkv.shape != (m, (nq + 2 * nkv) * hd) or (folded is not None and folded.stride != ROWS_FOLD_STRIDE):
        return False
    partials, count, eps = _fold_args(folded, ROWS_FOLD_STRIDE)
    code = _fn("stride_gemm_rows_qkv_rope", f"product {weight.shape[0]}x{k} (tcgen05, tokens as rows, qkv + rotation + cache write)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(qkv, "qkv", torch.bfloat16),
        _opt(bias, "bias", torch.float32), _dev(positions, "positions", torch.int32), _opt(slot_mapping, "slot_mapping", torch.int32),
        _dev(cos, "cos", torch.float32), _dev(sin, "sin", torch.float32), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), m, nq, nkv, hd, page_size, k, int(rotate), partials, count, eps,
        _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_rows_qkv_rope")
    return True


GATED_BLOCK = 64      # rows of gate and up alternate in blocks of this many in a weight laid out for ``linear_gated_tc``


FOLD_NORMS = _os.environ.get("STRIDE_B200_FOLD_NORMS", "1") != "0"


class FoldedNorm:
    """The output of an RMS norm whose two halves were folded into the products around it: ``xt`` holds
    ``residual * weight`` in bfloat16 (no 1/rms yet), ``partials`` [count, 16] the sums of squares of the
    residual per producer CTA and token (``stride`` tokens a CTA: 16 from the kernels for at most 16 tokens, 128 from
    the tokens-as-rows kernel). A product that takes it applies ``rsqrt(sum / width + eps)`` to its
    accumulators; anything else asks for ``tensor()``, which runs the small kernel that finishes the norm."""

    def __init__(self, xt, partials, count: int, eps: float, make_buffer, stride: int = 16):
        self.xt, self.partials, self.count, self.eps, self.stride = xt, partials, int(count), float(eps), int(stride)
        self.shape, self.dtype, self.device = xt.shape, xt.dtype, xt.device
        self._make_buffer = make_buffer
        self._tensor = None

    def tensor(self):
        if self._tensor is None:
            out = self._make_buffer()
            _check(_fn("stride_scale_rows")(self.xt.data_ptr(), self.partials.data_ptr(), self.count, self.eps, out.data_ptr(),
                                            self.shape[0], self.shape[1], self.stride, _stream()), "scale_rows")
            self._tensor = out
        return self._tensor


def _fold_args(folded, stride: int = 16):
    if folded is None:
        return None, 0, 0.0
    if folded.stride != stride:
        raise ValueError(f"a folded norm with {folded.stride} tokens a CTA was given to a kernel that reads {stride}")
    return folded.partials.data_ptr(), folded.count, folded.eps


def linear_add_norm(x, weight, residual, norm_weight, xt, partials) -> int:
    """The product before an RMS norm, for at most 16 rows: ``residual += bf16(x @ weight.T)`` (float32),
    ``xt = residual * norm_weight`` in bfloat16, ``partials[cta, token]`` the sums of squares. Returns the number
    of producer CTAs (what a consumer has to add up), or 0 when the kernel does not take the sizes."""
    m, k = x.shape
    n = weight.shape[0]
    if not (FOLD_NORMS and STREAM_GEMM) or m > TC_GEMM_MAX_TOKENS or x.dtype != torch.bfloat16 or residual.shape != (m, n):
        return 0
    count = c_int(0)
    code = _fn("stride_gemm_stream_add_norm", f"product {n}x{k} (+ residual, norm statistics)")(_dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16),
                                              _dev(xt, "xt", torch.bfloat16), _dev(residual, "residual", torch.float32),
                                              _dev(norm_weight, "norm_weight", torch.float32), _dev(partials, "partials", torch.float32),
                                              partials.numel(), m, n, k, ctypes.byref(count), _status_ptr(x.device), _stream())
    if code == -2:
        return 0
    _check(code, "gemm_stream_add_norm")
    return count.value


def linear_gated_tc(x, weight, out, folded=None) -> bool:
    """``out = silu(x @ gate.T) * (x @ up.T)`` in one tcgen05 kernel for at most 16 rows of ``x``; ``weight`` is
    [2 * inter, k] with gate and up rows alternating in blocks of ``GATED_BLOCK``. With ``folded`` (a FoldedNorm
    whose ``xt`` is ``x``) the kernel applies the norm's 1/rms itself. Returns False when the kernel does not take
    the sizes (the caller then runs the product and ``silu_mul`` with the same block)."""
    m, k = x.shape
    inter = weight.shape[0] // 2
    if m > TC_GEMM_MAX_TOKENS or out.shape != (m, inter):
        return False
    st = _tc_buffers(x.device, 0)
    partials, count, eps = _fold_args(folded)
    code = _fn("stride_gemm_tc_gated", f"product 2x{inter}x{k} (tcgen05, silu * up)")(_dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16),
                                       _dev(out, "out", torch.bfloat16), m, inter, k, st["status"].data_ptr(), partials, count, eps,
                                       _stream())
    if code == -2:
        return False
    _check(code, "gemm_tc_gated")
    return True


def _status_ptr(device) -> int:
    return _tc_buffers(device, 0)["status"].data_ptr()


def linear_stream(x, weight, out) -> bool:
    """``out = x @ weight.T`` on the weight-streaming kernel (at most 16 rows of ``x``).
    Returns False when the kernel does not take the shape."""
    m, k = x.shape
    n = weight.shape[0]
    code = _fn("stride_gemm_stream_bf16", f"product {n}x{k} (weight streaming)")(_dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out"),
                                          m, n, k, int(out.dtype == torch.float32), _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_stream_bf16")
    return True


def linear_qkv_rope(x, weight, qkv, bias, positions, slot_mapping, cos, sin, k_pages, v_pages, nq: int, nkv: int, hd: int,
                    page_size: int, rotate: bool, folded=None) -> bool:
    """The projection of queries, keys and values with ``rope_kv_write`` in its epilogue, for at most 16 rows of
    ``x``: afterwards ``qkv`` holds the rotated queries (its key and value columns are not written) and the cache
    the rotated keys and the values. With ``folded`` (a FoldedNorm whose ``xt`` is ``x``) the kernel applies the
    norm's 1/rms itself. Returns False when the kernel does not take the sizes; the caller then runs ``linear`` and
    ``rope_kv_write``."""
    m, k = x.shape
    if not STREAM_GEMM or m > TC_GEMM_MAX_TOKENS or x.dtype != torch.bfloat16 or qkv.shape != (m, (nq + 2 * nkv) * hd):
        return False
    partials, count, eps = _fold_args(folded)
    code = _fn("stride_gemm_stream_qkv_rope", f"product {weight.shape[0]}x{k} (qkv + rotation + cache write)")(
        _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(qkv, "qkv", torch.bfloat16),
        _opt(bias, "bias", torch.float32), _dev(positions, "positions", torch.int32), _opt(slot_mapping, "slot_mapping", torch.int32),
        _dev(cos, "cos", torch.float32), _dev(sin, "sin", torch.float32), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), m, nq, nkv, hd, page_size, k, int(rotate), partials, count, eps,
        _status_ptr(x.device), _stream())
    if code == -2:
        return False
    _check(code, "gemm_stream_qkv_rope")
    return True


def linear(x, weight, out) -> None:
    """``out = x @ weight.T`` for row-major ``weight`` [out_features, in_features].

    float32 runs the package's own FMA kernel (true 32-bit, order of the sum
    fixed). bfloat16 with few rows (decode steps) runs the package's own kernels:
    the tcgen05 kernel for large matrices, the weight-streaming kernel for the
    others; with many rows it calls the library matrix product, as the
    reference's engine does (python/stride_worker/model.py:258-260). ``out`` may
    be float32 for bfloat16 inputs to keep the accumulator's precision (the
    output head).
    """
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"linear: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> {tuple(out.shape)} do not agree")
    if x.dtype == torch.float32:
        _check(_fn("stride_gemm_nt_f32", f"product {n}x{k} (float32)")(_dev(x, "x", torch.float32), _dev(weight, "weight", torch.float32),
                                         _dev(out, "out", torch.float32), m, n, k, k, k, n, _stream()), "gemm_nt_f32")
        return
    _dev(x, "x", torch.bfloat16), _dev(weight, "weight", torch.bfloat16), _dev(out, "out")
    if m == 0:
        return
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("linear: the output must be bfloat16 or float32")
    if m <= TC_GEMM_MAX_TOKENS:
        if -(-n // 128) >= TC_GEMM_MIN_TILES:
            if linear_tc(x, weight, out):
                return
        elif STREAM_GEMM and linear_stream(x, weight, out):
            return
    elif m <= TC_CLUSTER_MAX_TOKENS and TC_GEMM_MAX_TOKENS > 0 and linear_tc_clustered(x, weight, out):
        return
    def library(*_):
        if out.dtype == torch.float32:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        else:
            torch.mm(x, weight.t(), out=out)
        return 0
    (_timer.timed(f"product {n}x{k} (library)", library) if _timer is not None else library)()


# -------------------------------------------------------------------- attention
def paged_attention(q, q_stride: int, out, k_pages, v_pages, block_table, seq_of_token, positions, nq: int, nkv: int,
                    hd: int, page_size: int, scale: float, window: int = 0) -> None:
    """Attention of every token in the flat batch over its request's pages.
    ``q`` holds head h of token t at ``q[t * q_stride + h * hd]``."""
    tokens = out.shape[0]
    if out.shape[1] != nq * hd:
        raise KernelError("attention output has the wrong width")
    _check(_fn("stride_paged_attention_generic")(
        _dev(q, "q"), q_stride, _dev(out, "out"), _dev(k_pages, "k_pages"), _dev(v_pages, "v_pages"),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1], _dev(seq_of_token, "seq_of_token", torch.int32),
        _dev(positions, "positions", torch.int32), tokens, nq, nkv, hd, page_size, float(scale), int(window),
        _code(q.dtype), _stream()), "paged_attention")


def fast_attention_supported(dtype, nq: int, nkv: int, hd: int) -> bool:
    """Sizes that the tensor-core attention kernels run; others use the generic kernel."""
    return dtype == torch.bfloat16 and hd in (64, 128) and nq % nkv == 0 and nq // nkv <= 16


def decode_scratch_floats(tokens: int, nq: int, nkv: int, hd: int, max_context: int) -> int:
    """float32 elements of scratch that ``paged_attention_decode`` needs for these sizes."""
    f = _bound.get("stride_paged_decode_scratch_floats")
    if f is None:
        f = build.load_kernel_library("attention_decode").stride_paged_decode_scratch_floats
        f.argtypes = [c_int, c_int, c_int, c_int, c_int]
        f.restype = c_longlong
        _bound["stride_paged_decode_scratch_floats"] = f
    return int(f(tokens, nq, nkv, hd, max_context))


def paged_attention_decode(q, q_stride: int, out, k_pages, v_pages, block_table, seq_of_token, positions, scratch, nq: int,
                           nkv: int, hd: int, page_size: int, scale: float, window: int, max_context: int) -> None:
    """Attention for single decoded tokens (one query per row), split over the keys;
    ``scratch`` (float32, zero when first used) holds the ticket counters and the
    partial results of the splits."""
    tokens = out.shape[0]
    if out.shape[1] != nq * hd:
        raise KernelError("attention output has the wrong width")
    _check(_fn("stride_paged_decode_attention_tma")(
        _dev(q, "q", torch.bfloat16), q_stride, _dev(out, "out", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), k_pages.shape[0], _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], _dev(seq_of_token, "seq_of_token", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(scratch, "scratch", torch.float32), scratch.numel(), tokens, nq, nkv, hd, page_size, float(scale), int(window),
        int(max_context), _tc_buffers(q.device, 0)["status"].data_ptr(), _stream()), "paged_attention_decode")


TC_ATTENTION = _os.environ.get("STRIDE_B200_TC_ATTENTION", "1") != "0"


def paged_attention_prefill_tc(q, q_stride: int, out, k_pages, v_pages, block_table, q_start, q_len, ctx_len, num_seqs: int,
                               nq: int, nkv: int, hd: int, page_size: int, scale: float, window: int) -> bool:
    """The tcgen05 version of ``paged_attention_prefill`` (same arguments). Returns False
    when it does not take the sizes; the caller then uses the mma.sync kernel."""
    tokens = out.shape[0]
    if out.shape[1] != nq * hd:
        raise KernelError("attention output has the wrong width")
    st = _tc_buffers(q.device, 0)
    code = _fn("stride_paged_prefill_attention_tc")(
        _dev(q, "q", torch.bfloat16), q_stride, _dev(out, "out", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), k_pages.shape[0], _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32),
        _dev(ctx_len, "ctx_len", torch.int32), num_seqs, tokens, nq, nkv, hd, page_size, float(scale), int(window),
        st["status"].data_ptr(), _stream())
    if code == -2:
        return False
    _check(code, "paged_attention_prefill_tc")
    return True


def paged_attention_prefill(q, q_stride: int, out, k_pages, v_pages, block_table, q_start, q_len, ctx_len, num_seqs: int,
                            nq: int, nkv: int, hd: int, page_size: int, scale: float, window: int) -> None:
    """Attention for the first ``num_seqs`` requests of the step (portions of any
    length), which own the rows of ``out``."""
    tokens = out.shape[0]
    if out.shape[1] != nq * hd:
        raise KernelError("attention output has the wrong width")
    _check(_fn("stride_paged_prefill_attention")(
        _dev(q, "q", torch.bfloat16), q_stride, _dev(out, "out", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        _dev(q_start, "q_start", torch.int32), _dev(q_len, "q_len", torch.int32), _dev(ctx_len, "ctx_len", torch.int32),
        num_seqs, tokens, nq, nkv, hd, page_size, float(scale), int(window), _stream()), "paged_attention_prefill")


# --------------------------------------------------------------------- sampling
_sample_scratch: dict = {}


def _sampling_scratch(device, rows: int, vocab: int):
    """Zeroed int32 words for the segment results and tickets of ``sample_rows`` (it leaves the tickets zero)."""
    f = _bound.get("stride_sample_scratch_words")
    if f is None:
        f = build.load_kernel_library("sampling").stride_sample_scratch_words
        f.argtypes = [c_int, c_int]
        f.restype = c_longlong
        _bound["stride_sample_scratch_words"] = f
    need = int(f(rows, vocab))
    st = _sample_scratch.setdefault(device, {"buf": None, "retired": []})
    if st["buf"] is None or st["buf"].numel() < need:
        if st["buf"] is not None:
            st["retired"].append(st["buf"])          # a captured graph may still use it
        st["buf"] = torch.zeros(max(need, 1 << 18), dtype=torch.int32, device=device)
    return st["buf"]


def sample_rows(logits, out, temperature=None, uniform=None, suppress=None) -> None:
    """Greedy (no ``temperature``, or 0) or temperature sampling per row."""
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("logits rows must be dense")
    if not logits.is_cuda:
        raise KernelError("logits must live on a CUDA device; stride_b200 has no CPU path")
    scratch = _sampling_scratch(logits.device, rows, vocab)
    _check(_fn("stride_sample_rows")(logits.data_ptr(), rows, vocab, logits.stride(0),
                                     _opt(temperature, "temperature", torch.float32),
                                     _opt(uniform, "uniform", torch.float32), _opt(suppress, "suppress", torch.int32),
                                     _dev(out, "out", torch.int32), scratch.data_ptr(), scratch.numel(), _stream()), "sample_rows")


_ranked_probs: dict = {}


def sample_ranked(logits, out, temperature, uniform, suppress, top_k, top_p) -> None:
    """Draws the rows with a temperature above 0 that ask for top-k (``top_k[r] > 0``) or a nucleus (``top_p[r] < 1``)
    by the reference sampler's rule and writes their tokens to ``out``; the other rows of ``out`` are left as they
    are (``sample_rows`` draws those). One [rows, vocab] float32 scratch per device, grown when a step needs more."""
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("logits rows must be dense")
    if not logits.is_cuda:
        raise KernelError("logits must live on a CUDA device; stride_b200 has no CPU path")
    key = _device_key(logits.device)
    probs = _ranked_probs.get(key)
    if probs is None or probs.numel() < rows * vocab:
        probs = torch.empty(rows * vocab, dtype=torch.float32, device=logits.device)
        _ranked_probs[key] = probs
    _check(_fn("stride_sample_ranked")(logits.data_ptr(), rows, vocab, logits.stride(0), _dev(temperature, "temperature", torch.float32),
                                       _dev(uniform, "uniform", torch.float32), _opt(suppress, "suppress", torch.int32),
                                       _dev(top_k, "top_k", torch.int32), _dev(top_p, "top_p", torch.float32),
                                       _dev(out, "out", torch.int32), probs.data_ptr(), probs.numel(), _stream()), "sample_ranked")
