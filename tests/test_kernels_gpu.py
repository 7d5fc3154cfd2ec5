"""Each CUDA kernel alone against a plain float64 reference of the same
operation, at sizes other than the engine's test models (odd widths, a prime
vocabulary, several head sizes and groupings)."""

import math

import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-6, torch.bfloat16: 1.2e-2}


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from stride_b200.csrc import ops as _ops
    return _ops


def dev(t, dtype=None):
    return t.to(device="cuda", dtype=dtype or t.dtype).contiguous()


def close(got, want, dtype, scale=None):
    got, want = got.double().cpu(), want.double().cpu()
    scale = scale if scale is not None else float(want.abs().max().clamp_min(1e-6))
    err = float((got - want).abs().max())
    assert err <= TOL[dtype] * scale, f"max abs error {err:.3e} against scale {scale:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(ops, dtype):
    g = torch.Generator().manual_seed(1)
    table = torch.randn(251, 88, generator=g).to(dtype)
    ids = torch.tensor([0, 250, 17, 17, 3], dtype=torch.int32)
    seq = torch.tensor([0, 0, 1, -1, 2], dtype=torch.int32)
    out = torch.full((5, 88), 7.0, device="cuda")
    ops.embed_gather(dev(ids), dev(seq), dev(table), out)
    want = table[ids.long()].float()
    want[3] = 0
    assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,eps", [(88, 3e-5), (4104, 1e-6), (64, 1e-5)])
def test_add_rmsnorm(ops, dtype, hidden, eps):
    g = torch.Generator().manual_seed(2)
    res = torch.randn(9, hidden, generator=g) * 3
    delta = (torch.randn(9, hidden, generator=g)).to(dtype)
    w = 1 + 0.2 * torch.randn(hidden, generator=g)
    # with delta: residual updated, norm of the sum
    r = dev(res.clone())
    out = torch.empty(9, hidden, dtype=dtype, device="cuda")
    ops.add_rmsnorm(r, dev(delta), dev(w), out, eps)
    x = res.double() + delta.double()
    close(r, x, torch.float32)
    close(out, plain.rms_norm(x, w.double(), eps), dtype)
    # without delta: residual untouched
    r = dev(res.clone())
    ops.add_rmsnorm(r, None, dev(w), out, eps)
    assert torch.equal(r.cpu(), res)
    close(out, plain.rms_norm(res.double(), w.double(), eps), dtype)
    # gathered rows: residual untouched, only those rows produced
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    r = dev(res.clone())
    out3 = torch.empty(3, hidden, dtype=dtype, device="cuda")
    ops.add_rmsnorm(r, dev(delta), dev(w), out3, eps, rows=dev(rows))
    assert torch.equal(r.cpu(), res)
    close(out3, plain.rms_norm(x[rows.long()], w.double(), eps), dtype)


def test_rmsnorm_is_not_fooled_by_a_missing_eps_or_a_mean_over_the_wrong_axis(ops):
    # negative controls in the manner of python/stride_worker/autotune/negative_control.py
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, 96, generator=g) * 1e-3
    w = torch.ones(96)
    out = torch.empty(4, 96, device="cuda")
    ops.add_rmsnorm(dev(x.clone()), None, dev(w), out, 1e-5)
    good = plain.rms_norm(x.double(), w.double(), 1e-5)
    no_eps = plain.rms_norm(x.double(), w.double(), 0.0)
    wrong_axis = x.double() * torch.rsqrt((x.double() ** 2).mean(0, keepdim=True) + 1e-5)
    err = lambda ref: float((out.cpu().double() - ref).abs().max())
    assert err(good) < 1e-6 < min(err(no_eps), err(wrong_axis))


@pytest.mark.parametrize("m", [1, 7, 65, 130])
def test_gemm_f32_matches_float64_and_does_not_depend_on_the_batch(ops, m):
    g = torch.Generator().manual_seed(4)
    a = torch.randn(130, 137, generator=g)
    w = torch.randn(251, 137, generator=g)
    out = torch.empty(m, 251, device="cuda")
    ops.linear(dev(a[:m]), dev(w), out)
    close(out, a[:m].double() @ w.double().T, torch.float32)
    full = torch.empty(130, 251, device="cuda")
    ops.linear(dev(a), dev(w), full)
    assert torch.equal(full[:m], out), "a row's result changed with the number of rows"


def test_linear_bf16(ops):
    g = torch.Generator().manual_seed(5)
    a = torch.randn(33, 96, generator=g).bfloat16()
    w = torch.randn(251, 96, generator=g).bfloat16()
    want = a.double() @ w.double().T
    out = torch.empty(33, 251, dtype=torch.bfloat16, device="cuda")
    ops.linear(dev(a), dev(w), out)
    close(out, want, torch.bfloat16)
    out32 = torch.empty(33, 251, dtype=torch.float32, device="cuda")
    ops.linear(dev(a), dev(w), out32)
    close(out32, want, torch.float32, scale=float(want.abs().max()) * 10)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,page,bias", [(5, 5, 48, 16, False), (6, 2, 16, 8, True), (8, 1, 128, 16, False)])
def test_rope_kv_write(ops, dtype, nq, nkv, hd, page, bias):
    g = torch.Generator().manual_seed(6)
    tokens, num_pages, max_pos = 11, 9, 700
    heads = nq + 2 * nkv
    qkv = torch.randn(tokens, heads * hd, generator=g).to(dtype)
    b = torch.randn(heads * hd, generator=g) * 0.1 if bias else None
    positions = torch.tensor([0, 1, 2, 3, 650, 651, 15, 16, 17, 699, 5], dtype=torch.int32)
    slots = torch.randperm(num_pages * page, generator=g)[:tokens].to(torch.int32)
    slots[10] = -1  # a padded token writes nothing
    scaling = {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 2.0,
               "original_max_position_embeddings": 32}
    inv = plain.rope_inv_freq(hd, 25000.0, scaling)
    angles = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    k_pages = torch.zeros(num_pages, nkv, page, hd, dtype=dtype, device="cuda")
    v_pages = torch.zeros_like(k_pages)
    q_dev = dev(qkv.clone())
    ops.rope_kv_write(q_dev, None if b is None else dev(b), dev(positions), dev(slots), dev(angles.cos()), dev(angles.sin()),
                      k_pages, v_pages, nq, nkv, hd, page)
    x = qkv.double().view(tokens, heads, hd)
    if b is not None:
        x = x + b.double().view(1, heads, hd)
    cos, sin = plain.rope_tables(hd, positions, 25000.0, scaling)
    q_want = plain.apply_rope(x[:, :nq], cos.double(), sin.double())
    k_want = plain.apply_rope(x[:, nq:nq + nkv], cos.double(), sin.double())
    v_want = x[:, nq + nkv:]
    close(q_dev.view(tokens, heads, hd)[:, :nq], q_want, dtype)
    # values and keys in the pool: only the addressed slots changed
    k_ref = torch.zeros(num_pages, nkv, page, hd, dtype=torch.float64)
    v_ref = torch.zeros_like(k_ref)
    for t in range(tokens):
        s = int(slots[t])
        if s >= 0:
            k_ref[s // page, :, s % page] = k_want[t]
            v_ref[s // page, :, s % page] = v_want[t]
    close(k_pages, k_ref, dtype)
    close(v_pages, v_ref, dtype)
    # the q part of a padded token is still rotated; untouched columns (k, v in qkv) are not required to change
    # negative control: the interleaved rotation is a different function
    inter = x[:, :nq].clone()
    a, c = inter[..., 0::2], inter[..., 1::2]
    ch, sh = cos.double()[:, None, :hd // 2], sin.double()[:, None, :hd // 2]
    wrong = torch.stack([a * ch - c * sh, c * ch + a * sh], -1).flatten(-2)
    assert float((q_dev.view(tokens, heads, hd)[:, :nq].double().cpu() - wrong).abs().max()) > 1e-2


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(ops, dtype):
    g = torch.Generator().manual_seed(7)
    x = (torch.randn(13, 2 * 136, generator=g) * 4).to(dtype)
    out = torch.empty(13, 136, dtype=dtype, device="cuda")
    ops.silu_mul(dev(x), out)
    gate, up = x[:, :136].double(), x[:, 136:].double()
    close(out, gate * torch.sigmoid(gate) * up, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter,block", [(192, 64), (136, 4), (320, 5)])
def test_silu_mul_with_gate_and_up_in_alternating_blocks(ops, dtype, inter, block):
    g = torch.Generator().manual_seed(8)
    gate = (torch.randn(7, inter, generator=g) * 4).to(dtype)
    up = (torch.randn(7, inter, generator=g) * 4).to(dtype)
    x = torch.stack([gate.view(7, inter // block, block), up.view(7, inter // block, block)], dim=2).reshape(7, 2 * inter)
    out = torch.empty(7, inter, dtype=dtype, device="cuda")
    ops.silu_mul(dev(x.contiguous()), out, block)
    close(out, gate.double() * torch.sigmoid(gate.double()) * up.double(), dtype)


@pytest.mark.parametrize("tokens,inter,k", [(8, 14336, 4096), (3, 9472, 192), (16, 14336, 1000), (1, 14336, 4096)])
def test_tcgen05_product_with_gate_epilogue(ops, tokens, inter, k):
    from stride_b200.parts.swiglu import interleave_gate_up

    g = torch.Generator().manual_seed(33)
    x = torch.randn(tokens, k, generator=g).bfloat16()
    gate = (torch.randn(inter, k, generator=g) * 0.05).bfloat16()
    up = (torch.randn(inter, k, generator=g) * 0.05).bfloat16()
    # the unfused path: each product rounded to bfloat16, then the activation (python/stride_worker/layers.py:152-161)
    gx = (x.double() @ gate.double().T).bfloat16().double()
    ux = (x.double() @ up.double().T).bfloat16().double()
    want = torch.nn.functional.silu(gx) * ux
    w = dev(interleave_gate_up(gate, up, ops.GATED_BLOCK))
    out = torch.full((tokens, inter), 7.0, dtype=torch.bfloat16, device="cuda")
    assert ops.linear_gated_tc(dev(x), w, out), "the kernel refused sizes it should take"
    torch.cuda.synchronize()
    assert ops.tc_status() == 0
    close(out, want, torch.bfloat16)
    # the same weight through the product and the blocked silu_mul gives the same within rounding
    both = torch.empty(tokens, 2 * inter, dtype=torch.bfloat16, device="cuda")
    ops.linear(dev(x), w, both)
    unfused = torch.empty_like(out)
    ops.silu_mul(both, unfused, ops.GATED_BLOCK)
    close(out, unfused.double(), torch.bfloat16)


def test_tcgen05_product_with_gate_epilogue_refuses_what_it_cannot_run(ops):
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    assert not ops.linear_gated_tc(x, torch.zeros(2 * 96, 64, dtype=torch.bfloat16, device="cuda"),
                                   torch.zeros(4, 96, dtype=torch.bfloat16, device="cuda"))          # inner % 64 != 0
    x = torch.zeros(4, 1024, dtype=torch.bfloat16, device="cuda")
    assert not ops.linear_gated_tc(x, torch.zeros(2 * 128, 1024, dtype=torch.bfloat16, device="cuda"),
                                   torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda"))         # so few tiles that K would be split


def _paged_case(g, dtype, seqs, nq, nkv, hd, page, window=None, spike=None):
    """seqs: list of (context_before, new_tokens). Builds scattered pages that hold
    the keys and values of every token and returns what the kernel needs together
    with the plain result for the new tokens."""
    total_pages = sum(-(-(c + n) // page) for c, n in seqs) + 5
    perm = torch.randperm(total_pages, generator=g).tolist()
    k_pages = torch.zeros(total_pages, nkv, page, hd)
    v_pages = torch.zeros_like(k_pages)
    width = max(-(-(c + n) // page) for c, n in seqs) + 1
    table = torch.full((len(seqs), width), -1, dtype=torch.int32)
    q_rows, pos_rows, seq_rows, want_rows = [], [], [], []
    for s, (ctx, new) in enumerate(seqs):
        n = ctx + new
        q = torch.randn(n, nq, hd, generator=g)
        k = torch.randn(n, nkv, hd, generator=g)
        v = torch.randn(n, nkv, hd, generator=g)
        if spike is not None and n > spike[1]:
            # one far key gets a score that stands out for one query
            qi, kj = n - 1, spike[1]
            k[kj, :] = q[qi].view(nkv, nq // nkv, hd)[:, 0] * 3.0
        q, k, v = q.to(dtype).float(), k.to(dtype).float(), v.to(dtype).float()
        for p in range(-(-n // page)):
            page_id = perm.pop()
            table[s, p] = page_id
            lo, hi = p * page, min(n, (p + 1) * page)
            k_pages[page_id, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            v_pages[page_id, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        if ctx > 8192 and window is None:
            # a long context: the plain formula (python/stride_worker/layers.py:109-149) for the new rows only, on the GPU
            qn, kd, vd = q[ctx:].double().cuda(), k.double().cuda(), v.double().cuda()
            group = nq // nkv
            scores = torch.einsum("tkgd,skd->kgts", qn.view(new, nkv, group, hd), kd) * hd ** -0.5
            allowed = torch.arange(n, device="cuda")[None, :] <= torch.arange(ctx, n, device="cuda")[:, None]
            scores = scores.masked_fill(~allowed[None, None], float("-inf"))
            rows = torch.einsum("kgts,skd->tkgd", torch.softmax(scores, -1), vd).reshape(new, nq, hd).cpu()
            want_rows.append(rows)
        else:
            want_rows.append(plain.causal_attention(q.double(), k.double(), v.double(), hd ** -0.5, window)[ctx:])
        q_rows.append(q[ctx:])
        pos_rows += list(range(ctx, n))
        seq_rows += [s] * new
    q_flat = torch.cat(q_rows).reshape(-1, nq * hd)
    return (q_flat.to(dtype), k_pages.to(dtype), v_pages.to(dtype), table, torch.tensor(seq_rows, dtype=torch.int32),
            torch.tensor(pos_rows, dtype=torch.int32), torch.cat(want_rows).reshape(-1, nq * hd))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,page,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (5, 5, 48, 16, None), (8, 2, 128, 16, None), (2, 1, 256, 16, None),
    (4, 2, 64, 8, 5), (4, 4, 32, 16, 40),
])
def test_paged_attention(ops, dtype, nq, nkv, hd, page, window):
    g = torch.Generator().manual_seed(8)
    # a whole prompt, a portion that starts at a page edge, one in the middle of a page, single decoded tokens
    seqs = [(0, 37), (32, 9), (45, 2), (130, 1), (16, 1), (0, 1), (63, 1), (64, 1)]
    q, k_pages, v_pages, table, seq_of, pos, want = _paged_case(g, dtype, seqs, nq, nkv, hd, page, window)
    # padding rows
    q = torch.cat([q, torch.zeros(2, nq * hd, dtype=dtype)])
    seq_of = torch.cat([seq_of, torch.tensor([-1, -1], dtype=torch.int32)])
    pos = torch.cat([pos, torch.zeros(2, dtype=torch.int32)])
    out = torch.full((q.shape[0], nq * hd), 5.0, dtype=dtype, device="cuda")
    ops.paged_attention(dev(q), nq * hd, out, dev(k_pages), dev(v_pages), dev(table), dev(seq_of), dev(pos), nq, nkv, hd,
                        page, hd ** -0.5, window or 0)
    close(out[:-2], want, dtype)
    assert float(out[-2:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(ops, dtype):
    g = torch.Generator().manual_seed(9)
    nq, nkv, hd, page = 4, 2, 64, 16
    seqs = [(699, 1), (0, 700)]
    q, k_pages, v_pages, table, seq_of, pos, want = _paged_case(g, dtype, seqs, nq, nkv, hd, page, spike=(None, 17))
    out = torch.empty(q.shape[0], nq * hd, dtype=dtype, device="cuda")
    ops.paged_attention(dev(q), nq * hd, out, dev(k_pages), dev(v_pages), dev(table), dev(seq_of), dev(pos), nq, nkv, hd,
                        page, hd ** -0.5, 0)
    close(out, want, dtype)
    # the spiked key dominates the first head of each group for the last query: a kernel that skipped key 17 would be far off
    assert float(want[0].abs().max()) > 0.5


def test_attention_f32_is_bitwise_the_same_for_a_token_alone_and_in_a_portion(ops):
    g = torch.Generator().manual_seed(10)
    nq, nkv, hd, page = 4, 2, 32, 8
    q, k_pages, v_pages, table, seq_of, pos, _ = _paged_case(g, torch.float32, [(0, 100)], nq, nkv, hd, page)
    out = torch.empty(100, nq * hd, device="cuda")
    args = (dev(k_pages), dev(v_pages), dev(table))
    ops.paged_attention(dev(q), nq * hd, out, *args, dev(seq_of), dev(pos), nq, nkv, hd, page, hd ** -0.5, 0)
    for t in (0, 7, 8, 31, 32, 99):
        one = torch.empty(1, nq * hd, device="cuda")
        ops.paged_attention(dev(q[t:t + 1]), nq * hd, one, *args, dev(seq_of[t:t + 1]), dev(pos[t:t + 1]), nq, nkv, hd,
                            page, hd ** -0.5, 0)
        assert torch.equal(one[0], out[t])


def test_kernels_refuse_sizes_they_cannot_run(ops):
    q = torch.zeros(1, 24, device="cuda")
    pages = torch.zeros(1, 1, 16, 24, device="cuda")
    table = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="not supported"):
        ops.paged_attention(q, 24, torch.empty(1, 24, device="cuda"), pages, pages, table, z, z, 1, 1, 24, 16, 1.0, 0)
    with pytest.raises(ops.KernelError, match="CUDA device"):
        ops.silu_mul(torch.zeros(1, 4), torch.zeros(1, 2))


def test_sample_rows_greedy_takes_the_first_maximum_and_honours_suppression(ops):
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(6, 1003, generator=g)
    logits[0, 5] = logits[0, 900] = 9.0          # a tie: the lower index wins
    logits[1, 1002] = 9.0                        # the last column
    logits[2, 0] = 9.0
    logits[3, 77] = 9.0                          # suppressed below
    logits[3, 78] = 8.0
    logits[4] = float("-inf")
    logits[4, 400] = -3.0
    suppress = torch.tensor([-1, -1, -1, 77, -1, -1], dtype=torch.int32)
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.sample_rows(dev(logits), out, suppress=dev(suppress))
    want = [plain.sample(logits[r], plain.XorShiftRng(0), temperature=0.0, eos=int(suppress[r]) if suppress[r] >= 0 else None,
                         min_tokens=1, generated=0) for r in range(6)]
    assert out.tolist() == want == [5, 1002, 0, 78, 400, int(logits[5].argmax())]


def _ranked_reference(logits_row, t, top_k, top_p, banned):
    """The reference sampler's rule in float64 on the float32 scaled logits: (ranking, cumulated kept mass)."""
    x = logits_row.clone().float()
    if banned >= 0:
        x[banned] = float("-inf")
    if abs(t - 1.0) > 1.1920929e-07:
        x = x / t
    if torch.isinf(x).all():
        probs = torch.full_like(x, 1.0 / x.numel(), dtype=torch.float64)
    else:
        probs = torch.softmax(x.double(), 0)
    order = torch.argsort(-probs, stable=True)
    keep = x.numel() if not top_k else min(x.numel(), top_k)
    sorted_p = probs[order]
    if top_p < 1.0:
        cum_all = torch.cumsum(sorted_p, 0)
        reached = torch.nonzero(cum_all >= top_p)
        nucleus = int(reached[0]) + 1 if len(reached) else x.numel()
        keep = min(keep, max(nucleus, 1))
    return order[:keep], torch.cumsum(sorted_p[:keep], 0)


@pytest.mark.parametrize("vocab,t,top_k,top_p", [(30011, 1.0, 0, 0.9), (30011, 0.7, 50, 1.0), (30011, 1.3, 700, 0.95), (30011, 1.0, 1, 1.0),
                                                 (1003, 0.8, 5, 0.5), (128256, 0.9, 0, 0.999), (128256, 1.0, 40000, 1.0), (97, 1.0, 200, 0.3)])
def test_sample_ranked_follows_the_reference_rule(ops, vocab, t, top_k, top_p):
    """Top-k and nucleus draws on the device against the rule in float64: flat rows (a nucleus of most of the vocabulary),
    peaked rows, coarse logits with many equal probabilities, every logit -inf, a suppressed maximum. A draw may differ
    only where the target lies within rounding of a boundary of the cumulated mass, and then by a neighbour."""
    g = torch.Generator().manual_seed(vocab + top_k)
    rows = [torch.randn(vocab, generator=g) * 0.3, torch.randn(vocab, generator=g) * 6, torch.round(torch.randn(vocab, generator=g) * 2) / 2,
            torch.full((vocab,), float("-inf")), torch.randn(vocab, generator=g) * 3]
    banned = [-1, -1, -1, -1, int(rows[4].argmax())]
    draws = 256
    for row, ban in zip(rows, banned):
        u = torch.rand(draws, generator=g)
        u[0], u[1] = 0.0, 1.0 - 2.0 ** -24
        logits = dev(row.expand(draws, vocab).contiguous())
        out = torch.full((draws,), -7, dtype=torch.int32, device="cuda")
        ops.sample_ranked(logits, out, dev(torch.full((draws,), t)), dev(u), dev(torch.full((draws,), ban, dtype=torch.int32)),
                          dev(torch.full((draws,), top_k, dtype=torch.int32)), dev(torch.full((draws,), top_p)))
        got = out.cpu().long()
        # fewer rows in a launch: clusters of 2, 4 and 8 CTAs a row share the columns; sums are integers, so the draws are the same
        for fewer in (60, 30, 7):
            again = torch.full((fewer,), -7, dtype=torch.int32, device="cuda")
            ops.sample_ranked(logits[:fewer], again, dev(torch.full((fewer,), t)), dev(u[:fewer]), dev(torch.full((fewer,), ban, dtype=torch.int32)),
                              dev(torch.full((fewer,), top_k, dtype=torch.int32)), dev(torch.full((fewer,), top_p)))
            assert torch.equal(again.cpu().long(), got[:fewer]), f"{fewer} rows in a launch draw other tokens than 256"
        kept, cum = _ranked_reference(row, t, top_k, top_p, ban)
        target = u.double() * cum[-1]
        where = torch.searchsorted(cum, target).clamp(max=len(kept) - 1)
        want = kept[where]
        assert int((got < 0).sum()) == 0 and int((got >= vocab).sum()) == 0, "a row was not drawn"
        if ban >= 0:
            assert int((got == ban).sum()) == 0, "the suppressed token was drawn"
        # Where the cumulated mass passes top_p within rounding of it, the cut may fall one entry earlier or later; the
        # kept mass, and with it every target, then moves by a share of that entry's probability.
        shift = 0.0
        if top_p < 1.0 and len(kept) > 1:
            slack = min(float(cum[-1]) - top_p, top_p - float(cum[-2]))
            if slack < 1e-5:
                shift = float(cum[-1] - cum[-2])
        rank_of = torch.full((vocab,), -1, dtype=torch.long)
        rank_of[kept] = torch.arange(len(kept))
        wrong = torch.nonzero(got != want).flatten()
        assert shift > 0.0 or len(wrong) <= max(2, draws // 50), f"{len(wrong)} of {draws} draws differ from the rule"
        sorted_p = torch.cat([cum[:1], cum[1:] - cum[:-1]])
        for i in wrong.tolist():
            pos = int(rank_of[got[i]])
            if pos >= 0 and abs(float(sorted_p[pos] - sorted_p[int(where[i])])) <= 1e-6 * float(sorted_p[pos]):
                continue         # a run of entries that are equal in float32 (the ranking is sorted, so everything between the two
                                 # is): such entries go by vocabulary order, not by what float64 still tells apart
            if pos < 0:          # just past the kept set: only where the cut itself lies within rounding
                assert abs(float(cum[-1]) - top_p) < 1e-5 or int(where[i]) == len(kept) - 1, f"draw {i}: token outside the kept set"
                continue
            assert abs(pos - int(where[i])) <= 1 or float(cum[max(pos, int(where[i]))] - cum[min(pos, int(where[i]))]) < 1e-5, \
                f"draw {i}: rank {pos} instead of {int(where[i])}"
            edge = min(abs(float(cum[pos] - target[i])), abs(float(cum[max(pos - 1, 0)] - target[i])))
            assert edge < 1e-5 + shift, f"draw {i}: rank {pos} instead of {int(where[i])}, {edge:.2e} from a boundary (cut slack allows {shift:.2e})"


def test_sample_ranked_leaves_other_rows_alone_and_is_exact_on_a_small_distribution(ops):
    logits = torch.log(torch.tensor([[0.05, 0.4, 0.05, 0.3, 0.2]] * 6))
    t = torch.tensor([1.0, 1.0, 1.0, 0.0, 1.0, 1.0])
    top_k = torch.tensor([2, 2, 0, 2, 0, 3], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.6, 1.0, 1.0, 0.95])
    u = torch.tensor([0.2, 0.8, 0.9, 0.5, 0.5, 0.99])
    out = torch.full((6,), -7, dtype=torch.int32, device="cuda")
    ops.sample_ranked(dev(logits), out, dev(t), dev(u), None, dev(top_k), dev(top_p))
    # rows 0, 1: {1: 0.4, 3: 0.3}, targets 0.14 and 0.56; row 2: nucleus 0.6 keeps {1, 3}, target 0.63; row 3 is greedy and row 4
    # plain temperature (left alone); row 5: top 3 = {1, 3, 4} = 0.9 < 0.95, target 0.891
    assert out.tolist() == [1, 3, 3, -7, -7, 4]


def test_sample_rows_draws_from_the_softmax(ops):
    g = torch.Generator().manual_seed(12)
    vocab = 1003
    logits = torch.randn(1, vocab, generator=g) * 2
    t = 0.7
    probs = torch.softmax(logits[0].double() / t, 0)
    cdf = torch.cumsum(probs, 0)
    n = 4096
    u = torch.rand(n, generator=g)
    rows = logits.expand(n, vocab).contiguous()
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample_rows(dev(rows), out, temperature=dev(torch.full((n,), t)), uniform=dev(u))
    got = out.cpu().long()
    want = torch.searchsorted(cdf, u.double()).clamp(max=vocab - 1)
    # the same inverse-CDF rule; rounding may move a draw that falls within 1e-5 of a boundary
    boundary_gap = (cdf[want] - u.double()).abs().minimum((cdf[(want - 1).clamp(min=0)] - u.double()).abs())
    differs = got != want
    assert int((differs & (boundary_gap > 1e-5)).sum()) == 0
    assert float(differs.float().mean()) < 0.01
    # and the frequencies follow the distribution
    top = int(probs.argmax())
    assert abs(float((got == top).float().mean()) - float(probs[top])) < 0.03
    # temperature 0 inside the same call is greedy; a suppressed token is never drawn
    mixed_t = torch.tensor([0.0, 1.0], dtype=torch.float32)
    two = logits.expand(2, vocab).contiguous()
    out2 = torch.empty(2, dtype=torch.int32, device="cuda")
    ops.sample_rows(dev(two), out2, temperature=dev(mixed_t), uniform=dev(torch.tensor([0.5, 0.5])),
                    suppress=dev(torch.tensor([-1, top], dtype=torch.int32)))
    assert out2[0].item() == top and out2[1].item() != top
    uniform_logits = torch.full((1, 10), float("-inf"))
    out1 = torch.empty(1, dtype=torch.int32, device="cuda")
    ops.sample_rows(dev(uniform_logits), out1, temperature=dev(torch.ones(1)), uniform=dev(torch.tensor([0.35])))
    assert out1.item() == 3


# ----------------------------------------------------------- tensor-core attention (bfloat16)
def _seq_arrays(seqs):
    q_start, q_len, ctx_len, at = [], [], [], 0
    for ctx, new in seqs:
        q_start.append(at)
        q_len.append(new)
        ctx_len.append(ctx + new)
        at += new
    mk = lambda v: torch.tensor(v, dtype=torch.int32)
    return mk(q_start), mk(q_len), mk(ctx_len)


@pytest.mark.parametrize("nq,nkv,hd,page,window", [
    (8, 2, 128, 16, None), (3, 1, 64, 8, None), (16, 1, 64, 16, None), (4, 4, 128, 32, None), (8, 2, 128, 16, 200),
    (6, 2, 64, 16, 5),
])
def test_decode_attention_split_over_the_keys(ops, nq, nkv, hd, page, window):
    g = torch.Generator().manual_seed(20)
    dtype = torch.bfloat16
    # contexts around the split size of 128 keys, a first token, and long ones
    seqs = [(0, 1), (126, 1), (127, 1), (128, 1), (255, 1), (256, 1), (700, 1), (1500, 1), (31, 1)]
    q, k_pages, v_pages, table, seq_of, pos, want = _paged_case(g, dtype, seqs, nq, nkv, hd, page, window, spike=(None, 3))
    q = torch.cat([q, torch.zeros(1, nq * hd, dtype=dtype)])
    seq_of = torch.cat([seq_of, torch.tensor([-1], dtype=torch.int32)])
    pos = torch.cat([pos, torch.zeros(1, dtype=torch.int32)])
    for bound in (1501, 4096, 200000):
        # the scratch starts with the ticket counters (zero before the first launch); what follows is poisoned
        scratch = torch.full((ops.decode_scratch_floats(q.shape[0], nq, nkv, hd, bound),), float("nan"), device="cuda")
        scratch[:65536] = 0
        for _ in range(2):      # twice on the same scratch: the tickets must be ready again
            out = torch.full((q.shape[0], nq * hd), 5.0, dtype=dtype, device="cuda")
            ops.paged_attention_decode(dev(q), nq * hd, out, dev(k_pages), dev(v_pages), dev(table), dev(seq_of), dev(pos), scratch,
                                       nq, nkv, hd, page, hd ** -0.5, window or 0, bound)
            close(out[:-1], want, dtype)
            assert float(out[-1].abs().max()) == 0.0
        assert int(scratch[:65536].view(torch.int32).abs().max()) == 0, "a launch left a ticket behind"
    assert ops.fast_attention_supported(dtype, nq, nkv, hd)
    assert not ops.fast_attention_supported(dtype, 34, 2, 128) and not ops.fast_attention_supported(dtype, 4, 2, 48)
    assert not ops.fast_attention_supported(torch.float32, 4, 2, 128)


@pytest.mark.parametrize("tokens,n,k", [(17, 4096, 4096), (33, 6144, 4096), (64, 4096, 14336), (64, 28672, 4096), (40, 1000, 520),
                                        (64, 384, 256), (20, 128256, 1024), (5, 4096, 2048)])
def test_the_clustered_product_for_17_to_64_tokens(ops, tokens, n, k):
    """The tcgen05 product whose CTAs of an output tile form a cluster and add their parts of K through shared
    memory: matrices of one to a thousand 128-row tiles, K split over one to four CTAs, rows and widths that fill no
    whole tile, float32 and bfloat16 results; twice in a row on other data (nothing is left behind)."""
    g = torch.Generator().manual_seed(tokens + n)
    for turn in range(2):
        x = (torch.randn(tokens, k, generator=g) * 0.5).bfloat16()
        w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
        w[min(n - 1, 130), :] = w[min(n - 1, 130), :] * 8       # one row stands out: a tile or a split that is dropped shows
        want = x.double() @ w.double().T
        scale = float(want.abs().max())
        for out_dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):       # as for the product of few tokens
            out = torch.full((tokens, n), 7.0, dtype=out_dtype, device="cuda")
            assert ops.linear_tc_clustered(dev(x), dev(w), out), "the kernel refused the shape"
            ops.check_kernel_status()
            err = float((out.double().cpu() - want).abs().max())
            assert err <= tol * scale, f"{out_dtype}: max abs error {err:.3e} against scale {scale:.3e}"


@pytest.mark.parametrize("tokens,n,k", [(17, 4096, 4096), (33, 6144, 4096), (64, 4096, 14336), (100, 28672, 1024), (128, 1000, 520),
                                        (40, 384, 64), (20, 128256, 1024), (64, 8192, 8192)])
def test_the_tokens_as_rows_product(ops, tokens, n, k):
    """The tcgen05 product whose tile rows are the tokens (17 to 128 of them), one CTA per block of 32, 64 or 128 output
    features and all of K, two issuing warps with an accumulator each: feature counts that fill no whole block, one
    block of K and hundreds, float32 and bfloat16 results, the residual sum in the epilogue; nothing is written past
    the last token."""
    g = torch.Generator().manual_seed(tokens + n)
    x = (torch.randn(tokens, k, generator=g) * 0.5).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    w[min(n - 1, 130), :] = w[min(n - 1, 130), :] * 8       # one feature stands out: a block that is dropped shows
    want = x.double() @ w.double().T
    scale = float(want.abs().max())
    for out_dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((tokens + 3, n), 7.0, dtype=out_dtype, device="cuda")
        assert ops.linear_rows(dev(x), dev(w), out[:tokens]), "the kernel refused the shape"
        ops.check_kernel_status()
        err = float((out[:tokens].double().cpu() - want).abs().max())
        assert err <= tol * scale, f"{out_dtype}: max abs error {err:.3e} against scale {scale:.3e}"
        assert float(out[tokens:].min()) == 7.0 and float(out[tokens:].max()) == 7.0, "the kernel wrote past the last token"
    # residual += bf16(product), in float32
    residual = torch.randn(tokens, n, generator=g)
    got = dev(residual.clone())
    assert ops.linear_rows_add(dev(x), dev(w), got)
    ops.check_kernel_status()
    plain_sum = residual.double() + want.bfloat16().double()
    assert float((got.double().cpu() - plain_sum).abs().max()) <= 1e-2 * scale
    bf = torch.empty(tokens, n, dtype=torch.bfloat16, device="cuda")
    assert ops.linear_rows(dev(x), dev(w), bf)
    assert torch.equal(got, dev(residual) + bf.float()), "the fused residual sum differs from product, then sum"


@pytest.mark.parametrize("tokens,inter,k", [(17, 14336, 4096), (64, 8192, 3072), (128, 320, 192), (33, 64, 64)])
def test_the_tokens_as_rows_product_with_gate_epilogue(ops, tokens, inter, k):
    from stride_b200.parts.swiglu import interleave_gate_up
    g = torch.Generator().manual_seed(35)
    x = (torch.randn(tokens, k, generator=g) * 0.5).bfloat16()
    gate = (torch.randn(inter, k, generator=g) * 0.05).bfloat16()
    up = (torch.randn(inter, k, generator=g) * 0.05).bfloat16()
    w = dev(interleave_gate_up(gate, up, ops.GATED_BLOCK))
    out = torch.full((tokens, inter), 7.0, dtype=torch.bfloat16, device="cuda")
    assert ops.linear_rows_gated(dev(x), w, out)
    ops.check_kernel_status()
    gu = torch.empty(tokens, 2 * inter, dtype=torch.bfloat16, device="cuda")
    assert ops.linear_rows(dev(x), w, gu)
    unfused = torch.empty_like(out)
    ops.silu_mul(gu, unfused, ops.GATED_BLOCK)
    gd, ud = (x.double() @ gate.double().T), (x.double() @ up.double().T)
    want = gd * torch.sigmoid(gd) * ud
    close(out, want, torch.bfloat16)
    close(out, unfused.double(), torch.bfloat16)


@pytest.mark.parametrize("tokens,nq,nkv,hd,k,page,bias,rotate", [
    (64, 32, 8, 128, 4096, 16, False, True), (17, 4, 4, 64, 256, 16, True, True), (100, 6, 2, 128, 200, 8, False, True),
    (33, 4, 1, 128, 192, 32, True, False), (128, 3, 1, 64, 96, 16, False, True),
])
def test_the_tokens_as_rows_projection_with_rotation_and_cache_write(ops, tokens, nq, nkv, hd, k, page, bias, rotate):
    """The fused kernel against the same product followed by ``rope_kv_write`` (itself tested against float64): bit for bit."""
    g = torch.Generator().manual_seed(36)
    heads = nq + 2 * nkv
    x = dev((torch.randn(tokens, k, generator=g) * 0.5).bfloat16())
    w = dev((torch.randn(heads * hd, k, generator=g) * 0.05).bfloat16())
    b = dev(torch.randn(heads * hd, generator=g) * 0.1) if bias else None
    num_pages, max_pos = 40, 700
    positions = dev(torch.randint(0, max_pos, (tokens,), generator=g).to(torch.int32))
    slots = torch.randperm(num_pages * page, generator=g)[:tokens].to(torch.int32)
    slots[tokens - 1] = -1                       # a padded token stores nothing
    slots = dev(slots)
    inv = plain.rope_inv_freq(hd, 25000.0, None)
    angles = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    cos, sin = dev(angles.cos()), dev(angles.sin())

    def run(fused):
        k_pages = torch.full((num_pages, nkv, page, hd), 3.0, dtype=torch.bfloat16, device="cuda")
        v_pages = torch.full_like(k_pages, 3.0)
        qkv = torch.full((tokens, heads * hd), 7.0, dtype=torch.bfloat16, device="cuda")
        if fused:
            assert ops.linear_rows_qkv_rope(x, w, qkv, b, positions, slots, cos, sin, k_pages, v_pages, nq, nkv, hd, page, rotate)
        else:
            assert ops.linear_rows(x, w, qkv)
            ops.rope_kv_write(qkv, b, positions, slots, cos, sin, k_pages, v_pages, nq, nkv, hd, page, rotate=rotate)
        ops.check_kernel_status()
        return qkv[:, :nq * hd].clone(), k_pages, v_pages

    q1, k1, v1 = run(True)
    q0, k0, v0 = run(False)
    assert torch.equal(q1, q0) and torch.equal(k1, k0) and torch.equal(v1, v0), "the fused projection differs from product + rope_kv_write"
    assert float(k1.float().sub(3.0).abs().max()) > 0.0     # something was stored


@pytest.mark.parametrize("tokens,hidden,k,inter", [(17, 4096, 4096, 14336), (64, 1024, 2048, 1024), (128, 192, 512, 320), (40, 8192, 1024, 128)])
def test_rms_norm_folded_into_the_tokens_as_rows_products(ops, tokens, hidden, k, inter):
    """As for at most 16 tokens: the product before the norm adds to the residual and leaves x~ and the sums of
    squares of its columns per CTA (128 tokens a CTA), the products after it apply 1/rms to their accumulators."""
    from stride_b200.parts.swiglu import interleave_gate_up
    g = torch.Generator().manual_seed(37)
    x = dev(torch.randn(tokens, k, generator=g).bfloat16())
    w = dev((torch.randn(hidden, k, generator=g) * 0.05).bfloat16())
    residual0 = torch.randn(tokens, hidden, generator=g) * 3
    residual0[tokens - 1] *= 40                   # one token far larger than the others: a factor taken from another row shows
    norm_w = dev(1 + 0.1 * torch.randn(hidden, generator=g))
    eps = 1e-5
    delta = torch.empty(tokens, hidden, dtype=torch.bfloat16, device="cuda")
    assert ops.linear_rows(x, w, delta)
    res_a = dev(residual0.clone())
    normed = torch.empty_like(delta)
    ops.add_rmsnorm(res_a, delta, norm_w, normed, eps)
    res_b = dev(residual0.clone())
    xt = torch.empty_like(delta)
    partials = torch.full((max(16 * 1024, hidden // 32 * 128),), float("nan"), device="cuda")
    count = ops.linear_rows_add_norm(x, w, res_b, norm_w, xt, partials)
    assert count > 0, "the kernel refused sizes it should take"
    ops.check_kernel_status()
    assert torch.equal(res_a, res_b), "the residual stream differs"
    folded = ops.FoldedNorm(xt, partials, count, eps, lambda: torch.empty_like(delta), ops.ROWS_FOLD_STRIDE)
    want = res_a.double() * torch.rsqrt((res_a.double() ** 2).mean(-1, keepdim=True) + eps) * norm_w.double()
    for t in range(tokens):     # row by row: the rows differ in size by a factor of 40
        close(folded.tensor()[t], want[t], torch.bfloat16)
    if inter % 64 == 0:
        gate = (torch.randn(inter, hidden, generator=g) * 0.05).bfloat16()
        up = (torch.randn(inter, hidden, generator=g) * 0.05).bfloat16()
        wgu = dev(interleave_gate_up(gate, up, ops.GATED_BLOCK))
        plain_out = torch.empty(tokens, inter, dtype=torch.bfloat16, device="cuda")
        fold_out = torch.empty_like(plain_out)
        assert ops.linear_rows_gated(normed, wgu, plain_out)
        assert ops.linear_rows_gated(xt, wgu, fold_out, folded)
        ops.check_kernel_status()
        gd, ud = want @ dev(gate).double().T, want @ dev(up).double().T       # from the norm in float64
        truth = gd * torch.sigmoid(gd) * ud
        for t in range(tokens):
            close(plain_out[t], truth[t], torch.bfloat16)
            close(fold_out[t], truth[t], torch.bfloat16)
    if hidden % 128 == 0:
        nq, nkv, hd, page = max(1, hidden // 256), 1, 128, 16
        heads = nq + 2 * nkv
        wqkv = dev((torch.randn(heads * hd, hidden, generator=g) * 0.05).bfloat16())
        positions = dev(torch.arange(tokens, dtype=torch.int32) * 3)
        slots = dev(torch.arange(tokens, dtype=torch.int32))
        inv = plain.rope_inv_freq(hd, 10000.0, None)
        angles = torch.outer(torch.arange(3 * tokens + 1, dtype=torch.float32), inv)
        cos, sin = dev(angles.cos()), dev(angles.sin())
        results = []
        for source, fold in ((normed, None), (xt, folded)):
            k_pages = torch.zeros(tokens // page + 1, nkv, page, hd, dtype=torch.bfloat16, device="cuda")
            v_pages = torch.zeros_like(k_pages)
            qkv = torch.zeros(tokens, heads * hd, dtype=torch.bfloat16, device="cuda")
            assert ops.linear_rows_qkv_rope(source, wqkv, qkv, None, positions, slots, cos, sin, k_pages, v_pages, nq, nkv, hd, page, True, fold)
            ops.check_kernel_status()
            results.append((qkv[:, :nq * hd].clone(), k_pages, v_pages))
        for a, b in zip(results[0], results[1]):
            close(b, a.double(), torch.bfloat16, scale=float(results[0][0].double().abs().max()))


def test_the_tokens_as_rows_product_refuses_what_it_cannot_run(ops):
    x = torch.zeros(129, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    assert not ops.linear_rows(x, w, torch.zeros(129, 128, dtype=torch.bfloat16, device="cuda"))              # more than 128 tokens
    assert not ops.linear_rows(x[:20, :60].contiguous(), w[:, :60].contiguous(), torch.zeros(20, 128, dtype=torch.bfloat16, device="cuda"))   # k % 8
    assert not ops.linear_rows_gated(x[:20], torch.zeros(2 * 96, 64, dtype=torch.bfloat16, device="cuda"),
                                     torch.zeros(20, 96, dtype=torch.bfloat16, device="cuda"))                # inner % 64
    assert not ops.rows_wanted(8) and not ops.rows_wanted(129)       # the callers' policy: other kernels take few tokens, the library many


def test_decode_attention_refuses_a_position_beyond_the_bound_of_its_launch(ops):
    """A launch is sized for positions below ``max_context``. A row beyond it would wait for splits that were never
    launched; it gets zeros and a code in the status word instead, and leaves no ticket behind: the next launch on
    the same scratch is right."""
    g = torch.Generator().manual_seed(21)
    dtype, nq, nkv, hd, page = torch.bfloat16, 8, 2, 128, 16
    seqs = [(300, 1), (1100, 1), (40, 1)]
    q, k_pages, v_pages, table, seq_of, pos, want = _paged_case(g, dtype, seqs, nq, nkv, hd, page)
    scratch = torch.zeros(ops.decode_scratch_floats(q.shape[0], nq, nkv, hd, 2048), device="cuda")
    args = (dev(k_pages), dev(v_pages), dev(table), dev(seq_of), dev(pos), scratch, nq, nkv, hd, page, hd ** -0.5, 0)
    ops.check_kernel_status()
    out = torch.full((3, nq * hd), 5.0, dtype=dtype, device="cuda")
    ops.paged_attention_decode(dev(q), nq * hd, out, *args, 1024)          # the second row sits at position 1100
    with pytest.raises(ops.KernelError, match="context bound"):
        ops.check_kernel_status()
    ops.check_kernel_status()                                              # reported once, then cleared
    assert float(out[1].abs().max()) == 0.0
    close(out[[0, 2]], want[[0, 2]], dtype)
    assert int(scratch[:65536].view(torch.int32).abs().max()) == 0, "the refused row left a ticket behind"
    ops.paged_attention_decode(dev(q), nq * hd, out, *args, 1024 + 128)
    close(out, want, dtype)
    ops.check_kernel_status()


@pytest.mark.parametrize("nq,nkv,hd,page,window", [(8, 2, 128, 16, None), (4, 1, 64, 32, None), (8, 2, 128, 16, 3000)])
def test_decode_attention_long_contexts(ops, nq, nkv, hd, page, window):
    """Tens of splits of up to 1,024 keys, each walked in many tiles; one far key per request carries nearly all
    of the weight, so a split that is dropped, merged twice or read from the wrong page shows. The plain result
    is the one-row formula softmax(q K^T * scale) V in float64 (python/stride_worker/layers.py:128-149)."""
    g = torch.Generator().manual_seed(31)
    dtype = torch.bfloat16
    contexts, far = [20000, 9001, 33000, 1], [1234, 8000, 31999, 0]
    pages_of = [-(-n // page) for n in contexts]
    perm = torch.randperm(sum(pages_of) + 3, generator=g).tolist()
    k_pages = torch.zeros(sum(pages_of) + 3, nkv, page, hd)
    v_pages = torch.zeros_like(k_pages)
    table = torch.full((len(contexts), max(pages_of) + 1), -1, dtype=torch.int32)
    qs, wants = [], []
    for s, (n, kj) in enumerate(zip(contexts, far)):
        q = torch.randn(nq, hd, generator=g)
        k = torch.randn(n, nkv, hd, generator=g)
        v = torch.randn(n, nkv, hd, generator=g)
        if window is None or n - 1 - kj < window:
            k[kj] = q.view(nkv, nq // nkv, hd)[:, 0] * 2.0
        q, k, v = q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double()
        for p in range(pages_of[s]):
            table[s, p] = perm.pop()
            lo, hi = p * page, min(n, (p + 1) * page)
            k_pages[table[s, p], :, :hi - lo] = k[lo:hi].transpose(0, 1).float()
            v_pages[table[s, p], :, :hi - lo] = v[lo:hi].transpose(0, 1).float()
        first = 0 if window is None else max(0, n - window)
        rows = []
        for h in range(nq):
            kh = h // (nq // nkv)
            w = torch.softmax(k[first:, kh] @ q[h] * hd ** -0.5, 0)
            rows.append(w @ v[first:, kh])
        qs.append(q.reshape(-1))
        wants.append(torch.cat(rows))
    q = torch.stack(qs).to(dtype)
    want = torch.stack(wants).float()
    seq_of = torch.arange(len(contexts), dtype=torch.int32)
    pos = torch.tensor([n - 1 for n in contexts], dtype=torch.int32)
    for bound in (33000, 131072):
        scratch = torch.full((ops.decode_scratch_floats(q.shape[0], nq, nkv, hd, bound),), float("nan"), device="cuda")
        scratch[:65536] = 0
        out = torch.full((q.shape[0], nq * hd), 5.0, dtype=dtype, device="cuda")
        ops.paged_attention_decode(dev(q), nq * hd, out, dev(k_pages.to(dtype)), dev(v_pages.to(dtype)), dev(table), dev(seq_of),
                                   dev(pos), scratch, nq, nkv, hd, page, hd ** -0.5, window or 0, bound)
        close(out, want, dtype)


@pytest.mark.parametrize("nq,nkv,hd,page,window", [
    (8, 2, 128, 16, None), (3, 1, 64, 8, None), (4, 4, 128, 32, None), (8, 2, 128, 16, 70), (6, 2, 64, 16, 5), (4, 1, 128, 16, 64),
])
def test_prefill_attention_over_portions(ops, nq, nkv, hd, page, window):
    g = torch.Generator().manual_seed(21)
    dtype = torch.bfloat16
    # whole prompts (one longer than several tiles), portions that start inside a page or a tile, tiny portions, one token
    seqs = [(0, 200), (0, 64), (0, 65), (100, 37), (64, 2), (333, 130), (5, 1), (0, 1), (128, 63)]
    q, k_pages, v_pages, table, _seq_of, _pos, want = _paged_case(g, dtype, seqs, nq, nkv, hd, page, window, spike=(None, 2))
    q_start, q_len, ctx_len = _seq_arrays(seqs)
    out = torch.full((q.shape[0], nq * hd), 5.0, dtype=dtype, device="cuda")
    ops.paged_attention_prefill(dev(q), nq * hd, out, dev(k_pages), dev(v_pages), dev(table), dev(q_start), dev(q_len),
                                dev(ctx_len), len(seqs), nq, nkv, hd, page, hd ** -0.5, window or 0)
    close(out, want, dtype)
    # only the first requests: the rows of the others are left alone
    first = 3
    rows = int(q_start[first])
    out2 = torch.full((rows, nq * hd), 5.0, dtype=dtype, device="cuda")
    ops.paged_attention_prefill(dev(q[:rows]), nq * hd, out2, dev(k_pages), dev(v_pages), dev(table), dev(q_start), dev(q_len),
                                dev(ctx_len), first, nq, nkv, hd, page, hd ** -0.5, window or 0)
    assert torch.equal(out2, out[:rows])


def test_prefill_attention_masks_the_future_and_the_far_past(ops):
    """Negative control in the manner of the reference's off-by-one mask: keys after a
    query, or before its window, must not leak, even with huge values behind the mask."""
    g = torch.Generator().manual_seed(22)
    nq, nkv, hd, page, window = 4, 2, 64, 16, 20
    seqs = [(40, 90)]
    q, k_pages, v_pages, table, _s, _p, want = _paged_case(g, torch.bfloat16, seqs, nq, nkv, hd, page, window)
    q_start, q_len, ctx_len = _seq_arrays(seqs)
    out = torch.empty(q.shape[0], nq * hd, dtype=torch.bfloat16, device="cuda")
    args = (dev(table), dev(q_start), dev(q_len), dev(ctx_len), 1, nq, nkv, hd, page, hd ** -0.5)
    ops.paged_attention_prefill(dev(q), nq * hd, out, dev(k_pages), dev(v_pages), *args, window)
    close(out, want, torch.bfloat16)
    no_window = torch.empty_like(out)
    ops.paged_attention_prefill(dev(q), nq * hd, no_window, dev(k_pages), dev(v_pages), *args, 0)
    assert float((no_window.float() - out.float()).abs().max()) > 0.05, "the window changed nothing"


# ------------------------------------------------- weight-streaming product (decode)
@pytest.mark.parametrize("tokens,n_out,k", [
    (1, 16, 8), (8, 4096, 4096), (7, 4096, 14336), (16, 136, 4104), (9, 251, 88), (3, 515, 192), (12, 6144, 1000), (5, 33, 2056),
])
def test_streaming_product_for_few_tokens(ops, tokens, n_out, k):
    g = torch.Generator().manual_seed(31)
    x = torch.randn(tokens, k, generator=g).bfloat16()
    w = (torch.randn(n_out, k, generator=g) * 0.05).bfloat16()
    want = x.double() @ w.double().T
    scale = float(want.abs().max())
    for out_dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((tokens + 1, n_out), 7.0, dtype=out_dtype, device="cuda")
        assert ops.linear_stream(dev(x), dev(w), out[:tokens]), "the kernel refused a shape it should take"
        torch.cuda.synchronize()
        err = float((out[:tokens].double().cpu() - want).abs().max())
        assert err <= tol * scale, f"{out_dtype}: max abs error {err:.3e} against scale {scale:.3e}"
        assert float(out[tokens].min()) == 7.0, "the kernel wrote past the last token"


@pytest.mark.parametrize("tokens,nq,nkv,hd,k,page,bias,rotate", [
    (8, 32, 8, 128, 4096, 16, False, True), (3, 5, 5, 48, 88, 16, True, True), (16, 6, 2, 16, 200, 8, False, True),
    (11, 4, 1, 128, 192, 16, True, False), (1, 3, 1, 64, 96, 32, False, True),
])
def test_streaming_projection_with_rotation_and_cache_write(ops, tokens, nq, nkv, hd, k, page, bias, rotate):
    """The fused kernel against the product followed by ``rope_kv_write`` (itself tested against float64)."""
    g = torch.Generator().manual_seed(34)
    heads = nq + 2 * nkv
    x = dev(torch.randn(tokens, k, generator=g).bfloat16())
    w = dev((torch.randn(heads * hd, k, generator=g) * 0.05).bfloat16())
    b = dev(torch.randn(heads * hd, generator=g) * 0.1) if bias else None
    num_pages, max_pos = 9, 700
    positions = dev(torch.randint(0, max_pos, (tokens,), generator=g).to(torch.int32))
    slots = torch.randperm(num_pages * page, generator=g)[:tokens].to(torch.int32)
    if tokens > 2:
        slots[tokens - 1] = -1                       # a padded token stores nothing
    slots = dev(slots)
    inv = plain.rope_inv_freq(hd, 25000.0, None)
    angles = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    cos, sin = dev(angles.cos()), dev(angles.sin())

    def run(fused):
        k_pages = torch.full((num_pages, nkv, page, hd), 3.0, dtype=torch.bfloat16, device="cuda")
        v_pages = torch.full_like(k_pages, 3.0)
        qkv = torch.full((tokens, heads * hd), 7.0, dtype=torch.bfloat16, device="cuda")
        if fused:
            assert ops.linear_qkv_rope(x, w, qkv, b, positions, slots, cos, sin, k_pages, v_pages, nq, nkv, hd, page, rotate)
        else:
            ops.linear_stream(x, w, qkv)
            ops.rope_kv_write(qkv, b, positions, slots, cos, sin, k_pages, v_pages, nq, nkv, hd, page, rotate=rotate)
        torch.cuda.synchronize()
        return qkv[:, :nq * hd].clone(), k_pages, v_pages

    q1, k1, v1 = run(True)
    q0, k0, v0 = run(False)
    assert torch.equal(q1, q0) and torch.equal(k1, k0) and torch.equal(v1, v0), "the fused projection differs from product + rope_kv_write"
    assert float(k1.float().sub(3.0).abs().max()) > 0.0     # something was stored


@pytest.mark.parametrize("tokens,hidden,k,inter", [(8, 4096, 4096, 14336), (3, 192, 512, 320), (16, 1024, 2048, 1024), (1, 4096, 14336, 14336)])
def test_rms_norm_folded_into_the_products_around_it(ops, tokens, hidden, k, inter):
    """product -> sum -> norm -> product as three kernels and as two: the product before the norm adds to the
    residual and leaves x~ and sums of squares, the product after it applies 1/rms to its accumulators."""
    from stride_b200.parts.swiglu import interleave_gate_up
    g = torch.Generator().manual_seed(35)
    x = dev(torch.randn(tokens, k, generator=g).bfloat16())
    w = dev((torch.randn(hidden, k, generator=g) * 0.05).bfloat16())
    residual0 = torch.randn(tokens, hidden, generator=g) * 3
    norm_w = dev(1 + 0.1 * torch.randn(hidden, generator=g))
    eps = 1e-5
    # in steps: product, then sum and norm in one kernel
    delta = torch.empty(tokens, hidden, dtype=torch.bfloat16, device="cuda")
    ops.linear_stream(x, w, delta)
    res_a = dev(residual0.clone())
    normed = torch.empty_like(delta)
    ops.add_rmsnorm(res_a, delta, norm_w, normed, eps)
    # folded
    res_b = dev(residual0.clone())
    xt = torch.empty_like(delta)
    partials = torch.full((16 * 1024,), float("nan"), device="cuda")
    count = ops.linear_add_norm(x, w, res_b, norm_w, xt, partials)
    assert count > 0, "the kernel refused sizes it should take"
    torch.cuda.synchronize()
    assert torch.equal(res_a, res_b), "the residual stream differs"
    folded = ops.FoldedNorm(xt, partials, count, eps, lambda: torch.empty_like(delta))
    close(folded.tensor(), normed.double(), torch.bfloat16)
    want = res_a.double() * torch.rsqrt((res_a.double() ** 2).mean(-1, keepdim=True) + eps) * norm_w.double().cpu().to(res_a.device)
    close(folded.tensor(), want, torch.bfloat16)
    # the consumer applies 1/rms itself: gated feed-forward product
    if inter % 64 == 0 and tokens <= 16:
        gate = (torch.randn(inter, hidden, generator=g) * 0.05).bfloat16()
        up = (torch.randn(inter, hidden, generator=g) * 0.05).bfloat16()
        wgu = dev(interleave_gate_up(gate, up, ops.GATED_BLOCK))
        plain_out = torch.empty(tokens, inter, dtype=torch.bfloat16, device="cuda")
        fold_out = torch.empty_like(plain_out)
        if ops.linear_gated_tc(normed, wgu, plain_out):
            assert ops.linear_gated_tc(xt, wgu, fold_out, folded)
            torch.cuda.synchronize()
            assert ops.tc_status() == 0
            close(fold_out, plain_out.double(), torch.bfloat16)
    # ... and the projection of queries, keys and values
    if hidden % 128 == 0:
        nq, nkv, hd, page = hidden // 128, 1, 128, 16
        heads = nq + 2 * nkv
        wqkv = dev((torch.randn(heads * hd, hidden, generator=g) * 0.05).bfloat16())
        positions = dev(torch.arange(tokens, dtype=torch.int32) * 3)
        slots = dev(torch.arange(tokens, dtype=torch.int32))
        inv = plain.rope_inv_freq(hd, 10000.0, None)
        angles = torch.outer(torch.arange(64, dtype=torch.float32), inv)
        cos, sin = dev(angles.cos()), dev(angles.sin())
        results = []
        for source, fold in ((normed, None), (xt, folded)):
            k_pages = torch.zeros(2, nkv, page, hd, dtype=torch.bfloat16, device="cuda")
            v_pages = torch.zeros_like(k_pages)
            qkv = torch.zeros(tokens, heads * hd, dtype=torch.bfloat16, device="cuda")
            assert ops.linear_qkv_rope(source, wqkv, qkv, None, positions, slots, cos, sin, k_pages, v_pages, nq, nkv, hd, page, True, fold)
            torch.cuda.synchronize()
            results.append((qkv[:, :nq * hd].clone(), k_pages, v_pages))
        for a, b in zip(results[0], results[1]):
            close(b, a.double(), torch.bfloat16, scale=float(results[0][0].double().abs().max()))


def test_streaming_product_refuses_what_it_cannot_run(ops):
    w = torch.zeros(128, 100, dtype=torch.bfloat16, device="cuda")
    assert not ops.linear_stream(torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda"), w,
                                 torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda"))                 # k % 8 != 0
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    assert not ops.linear_stream(torch.zeros(17, 64, dtype=torch.bfloat16, device="cuda"), w,
                                 torch.zeros(17, 128, dtype=torch.bfloat16, device="cuda"))                # more than 16 tokens


# ------------------------------------------------------------- tcgen05 matrix product
@pytest.mark.parametrize("tokens,n_out,k", [
    (1, 128, 64), (8, 6144, 4096), (8, 4096, 14336), (16, 136, 4104), (17, 256, 512), (33, 384, 1024), (64, 1000, 4096),
    (5, 251, 88), (200, 512, 256), (3, 128256, 256),
])
def test_tcgen05_product_for_few_tokens(ops, tokens, n_out, k):
    g = torch.Generator().manual_seed(30)
    x = torch.randn(tokens, k, generator=g).bfloat16()
    w = (torch.randn(n_out, k, generator=g) * 0.05).bfloat16()
    want = x.double() @ w.double().T
    scale = float(want.abs().max())
    for out_dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((tokens, n_out), 7.0, dtype=out_dtype, device="cuda")
        for _ in range(2):      # twice: the tickets of a split product must be ready again
            out.fill_(7.0)
            assert ops.linear_tc(dev(x), dev(w), out), "the kernel refused a shape it should take"
            torch.cuda.synchronize()
            err = float((out.double().cpu() - want).abs().max())
            assert err <= tol * scale, f"{out_dtype}: max abs error {err:.3e} against scale {scale:.3e}"
    assert ops.tc_status() == 0


def test_tcgen05_product_refuses_what_it_cannot_run(ops):
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda")        # k % 8 != 0
    w = torch.zeros(128, 100, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
    assert not ops.linear_tc(x, w, out)
    ops.linear(x, w, out)                                                # falls back to the library product
    big = torch.zeros(300, 64, dtype=torch.bfloat16, device="cuda")
    assert not ops.linear_tc(big, torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda"),
                             torch.zeros(300, 128, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("nq,nkv,hd,page,window", [
    (8, 2, 128, 16, None), (3, 1, 64, 8, None), (4, 4, 128, 32, None), (8, 2, 128, 16, 70), (6, 2, 64, 16, 5), (4, 1, 128, 16, 64),
    (2, 1, 128, 8, None), (4, 2, 128, 64, 300),
])
def test_prefill_attention_on_tcgen05(ops, nq, nkv, hd, page, window):
    g = torch.Generator().manual_seed(23)
    dtype = torch.bfloat16
    # whole prompts across several 128-key tiles, portions that start inside a page or a tile, tiny portions, one token
    seqs = [(0, 300), (0, 128), (0, 129), (100, 37), (64, 2), (333, 260), (5, 1), (0, 1), (128, 127), (250, 10)]
    q, k_pages, v_pages, table, _seq_of, _pos, want = _paged_case(g, dtype, seqs, nq, nkv, hd, page, window, spike=(None, 2))
    # poison every key and value slot that no request owns: stale contents must never reach a result
    used = torch.zeros(k_pages.shape[0], page, dtype=torch.bool)
    for s, (ctx, new) in enumerate(seqs):
        for p in range(-(-(ctx + new) // page)):
            n = min(page, ctx + new - p * page)
            used[int(table[s, p]), :n] = True
    k_pages = k_pages.clone()
    v_pages = v_pages.clone()
    k_pages.transpose(1, 2)[~used] = float("nan")
    v_pages.transpose(1, 2)[~used] = float("nan")
    q_start, q_len, ctx_len = _seq_arrays(seqs)
    out = torch.full((q.shape[0], nq * hd), 5.0, dtype=dtype, device="cuda")
    took = ops.paged_attention_prefill_tc(dev(q), nq * hd, out, dev(k_pages), dev(v_pages), dev(table), dev(q_start), dev(q_len),
                                          dev(ctx_len), len(seqs), nq, nkv, hd, page, hd ** -0.5, window or 0)
    assert took, "the kernel refused sizes it should take"
    torch.cuda.synchronize()
    assert ops.tc_status() == 0
    close(out, want, dtype)
    mma = torch.empty_like(out)
    ops.paged_attention_prefill(dev(q), nq * hd, mma, dev(k_pages), dev(v_pages), dev(table), dev(q_start), dev(q_len),
                                dev(ctx_len), len(seqs), nq, nkv, hd, page, hd ** -0.5, window or 0)
    close(out, mma.float(), dtype)


def test_prefill_attention_on_tcgen05_walks_long_contexts(ops):
    """Portions deep inside long contexts: a hundred and more key tiles per query tile, so every ring and
    barrier of the kernel wraps many times; none of its bounded waits may run out."""
    g = torch.Generator().manual_seed(24)
    dtype = torch.bfloat16
    nq, nkv, hd, page = 8, 2, 128, 16
    for seqs, repeats in (([(6100, 1024), (3333, 515), (0, 700)], 3), ([(70000, 300), (0, 130)], 1)):       # the second: a thousand key tiles
        q, k_pages, v_pages, table, _seq_of, _pos, want = _paged_case(g, dtype, seqs, nq, nkv, hd, page, None, spike=(None, 2))
        q_start, q_len, ctx_len = _seq_arrays(seqs)
        for _ in range(repeats):
            out = torch.full((q.shape[0], nq * hd), 5.0, dtype=dtype, device="cuda")
            assert ops.paged_attention_prefill_tc(dev(q), nq * hd, out, dev(k_pages), dev(v_pages), dev(table), dev(q_start), dev(q_len),
                                                  dev(ctx_len), len(seqs), nq, nkv, hd, page, hd ** -0.5, 0)
            torch.cuda.synchronize()
            assert ops.tc_status() == 0
            close(out, want, dtype)


def test_prefill_attention_on_tcgen05_refuses_odd_page_sizes(ops):
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
    pages = torch.zeros(2, 1, 24, 128, dtype=torch.bfloat16, device="cuda")
    table = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    assert not ops.paged_attention_prefill_tc(q, 128, torch.empty_like(q), pages, pages, table, z, z + 4, z + 4, 1, 1, 1, 128, 24,
                                              0.1, 0)
