"""The allocation-free decode attention entry point, called through its exported
C symbol, against the ordinary entry point (bit for bit: both run the same
kernel with the same splits) and against the one-row attention formula in
float64.

Collected last on purpose (see the file name): a run that stops at the first
failure has then already run every other test. Who needs this entry point: hosts
that cannot allocate device memory when they call into the library — code inside
a stream capture, runtimes whose memory is handed out once and then locked,
plugins restricted to the buffers their host passes in. It keeps the partial
results of the key splits in an 8 MiB array inside the library instead of asking
the caller for scratch."""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

CAPACITY = 2 * 1024 * 1024          # STRIDE_DECODE_STATIC_SCRATCH_FLOATS
TOO_SMALL = -3                      # STRIDE_STATIC_SCRATCH_TOO_SMALL


def _case(seed, nq, nkv, hd, page, contexts):
    g = torch.Generator().manual_seed(seed)
    pages_per_seq = [-(-c // page) for c in contexts]
    num_pages = sum(pages_per_seq) + 3
    order = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((len(contexts), max(pages_per_seq)), -1, dtype=torch.int32)
    for s, n in enumerate(pages_per_seq):
        for p in range(n):
            table[s, p] = order.pop()
    dev = lambda t: t.cuda().contiguous()
    k_pages = dev((torch.randn(num_pages, nkv, page, hd, generator=g) * 0.5).bfloat16())
    v_pages = dev((torch.randn(num_pages, nkv, page, hd, generator=g) * 0.5).bfloat16())
    q = dev(torch.randn(len(contexts) + 1, nq * hd, generator=g).bfloat16())
    seq_of = dev(torch.tensor(list(range(len(contexts))) + [-1], dtype=torch.int32))       # the last row is padding
    positions = dev(torch.tensor([c - 1 for c in contexts] + [0], dtype=torch.int32))
    return q, k_pages, v_pages, dev(table), seq_of, positions


def _plain(q, k_pages, v_pages, table, seq_of, positions, nq, nkv, hd, page):
    """softmax(q K^T / sqrt(hd)) V per row in float64, keys gathered through the block table
    (python/stride_worker/layers.py:128-149 for one query); padded rows give zeros."""
    q, k_pages, v_pages, table = q.cpu().double(), k_pages.cpu().double(), v_pages.cpu().double(), table.cpu()
    out = torch.zeros(q.shape[0], nq * hd, dtype=torch.float64)
    for t, (s, pos) in enumerate(zip(seq_of.cpu().tolist(), positions.cpu().tolist())):
        if s < 0:
            continue
        n = pos + 1
        pages = table[s, : -(-n // page)].long()
        k = k_pages[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n]
        v = v_pages[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n]
        for h in range(nq):
            qh = q[t, h * hd:(h + 1) * hd]
            w = torch.softmax(k[h // (nq // nkv)] @ qh * hd ** -0.5, dim=0)
            out[t, h * hd:(h + 1) * hd] = w @ v[h // (nq // nkv)]
    return out


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200.csrc import build, ops

    lib = build.load_kernel_library("attention_decode_static")
    fn = lib.stride_paged_decode_attention_static
    fn.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                   c_int, c_float, c_int, c_int, c_void_p]
    fn.restype = c_int
    floats = lib.stride_paged_decode_attention_static_floats
    floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
    floats.restype = c_longlong
    # the ordinary entry point in the form that copies with cp.async, as the static one does: caller's scratch
    ordinary = build.load_kernel_library("attention_decode").stride_paged_decode_attention
    ordinary.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong,
                         c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    ordinary.restype = c_int

    nq, nkv, hd, page = 8, 2, 128, 16
    stream = torch.cuda.current_stream().cuda_stream
    first_call = True
    # the third case gives one row a position that is not below the bound: zeros for that row, no ticket left behind
    # (the fourth, an ordinary call again, would otherwise merge wrongly)
    for seed, contexts, bound, beyond in ((1, [700, 1, 129, 2000], 2048, None), (2, [33, 1500, 640, 64], 4096, None),
                                          (3, [300, 2500, 77, 1024], 2048, 1), (4, [1999, 5, 512, 90], 2048, None)):
        q, k_pages, v_pages, table, seq_of, positions = _case(seed, nq, nkv, hd, page, contexts)
        tokens = q.shape[0]
        assert 0 < floats(tokens, nq, nkv, hd, bound) <= CAPACITY
        want = torch.full((tokens, nq * hd), 3.0, dtype=torch.bfloat16, device="cuda")
        scratch = torch.zeros(ops.decode_scratch_floats(tokens, nq, nkv, hd, bound), device="cuda")
        rc = ordinary(q.data_ptr(), nq * hd, want.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), table.data_ptr(), table.shape[1],
                      seq_of.data_ptr(), positions.data_ptr(), scratch.data_ptr(), scratch.numel(), tokens, nq, nkv, hd, page,
                      hd ** -0.5, 0, bound, stream)
        assert rc == 0
        got = torch.full_like(want, 5.0)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(q.data_ptr(), nq * hd, got.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), table.data_ptr(), table.shape[1],
                seq_of.data_ptr(), positions.data_ptr(), tokens, nq, nkv, hd, page, hd ** -0.5, 0, bound, stream)
        assert rc == 0, f"the entry point returned {rc}"
        torch.cuda.synchronize()
        if not first_call:       # the first call on a device may load the module lazily; later calls must not take memory
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
        first_call = False
        assert torch.equal(got, want), "the static entry point and the ordinary one run the same kernel: the bits must agree"
        plain = _plain(q, k_pages, v_pages, table, seq_of, positions, nq, nkv, hd, page)
        if beyond is not None:
            assert int(positions[beyond]) >= bound
            assert float(got[beyond].float().abs().max()) == 0.0, "a row beyond the bound must be zero"
            plain[beyond] = 0
        scale = float(plain.abs().max())
        err = float((got.double().cpu() - plain).abs().max())
        assert err <= 1.2e-2 * scale, f"max abs difference {err:.3e} from the float64 formula against scale {scale:.3e}"
        assert float(got[-1].float().abs().max()) == 0.0, "the padded row must be zero"
        assert int(scratch[:65536].view(torch.int32).abs().max()) == 0, "the ordinary call left a ticket behind"

    # a size that the static array cannot hold is refused, and nothing is launched
    big_tokens, big_bound = 64, 131072
    assert floats(big_tokens, 32, 8, 128, big_bound) > CAPACITY
    untouched = torch.full((big_tokens, 32 * 128), 9.0, dtype=torch.bfloat16, device="cuda")
    z = torch.zeros(big_tokens, dtype=torch.int32, device="cuda")
    rc = fn(untouched.data_ptr(), 32 * 128, untouched.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), table.data_ptr(),
            table.shape[1], z.data_ptr(), z.data_ptr(), big_tokens, 32, 8, 128, page, 0.1, 0, big_bound, stream)
    assert rc == TOO_SMALL
    torch.cuda.synchronize()
    assert float(untouched.float().min()) == 9.0
