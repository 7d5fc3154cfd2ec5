"""The allocation-free decode attention entry point, called through its exported
C symbol, against the ordinary entry point.

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

    nq, nkv, hd, page = 8, 2, 128, 16
    stream = torch.cuda.current_stream().cuda_stream
    first_call = True
    for seed, contexts, bound in ((1, [700, 1, 129, 2000], 2048), (2, [33, 1500, 640, 64], 4096)):
        q, k_pages, v_pages, table, seq_of, positions = _case(seed, nq, nkv, hd, page, contexts)
        tokens = q.shape[0]
        assert 0 < floats(tokens, nq, nkv, hd, bound) <= CAPACITY
        want = torch.full((tokens, nq * hd), 3.0, dtype=torch.bfloat16, device="cuda")
        scratch = torch.zeros(ops.decode_scratch_floats(tokens, nq, nkv, hd, bound), device="cuda")
        ops.paged_attention_decode(q, nq * hd, want, k_pages, v_pages, table, seq_of, positions, scratch, nq, nkv, hd, page,
                                   hd ** -0.5, 0, bound)
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
        scale = float(want.float().abs().max())
        err = float((got.float() - want.float()).abs().max())
        assert err <= 1.2e-2 * scale, f"max abs difference {err:.3e} against scale {scale:.3e}"
        assert float(got[-1].float().abs().max()) == 0.0, "the padded row must be zero"

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
