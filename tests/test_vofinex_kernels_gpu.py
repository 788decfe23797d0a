"""Each Vofinex mechanism's kernels alone on the GPU against the plain functions of ``tests/plain_vofinex.py``:
sizes that are no powers of two, constants that a real configuration may make 1 or equal made different, and
inputs built so that one wrong key, block edge, sink, correction or identity output shows."""

from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch

from tests import plain_vofinex as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture()
def ops():
    from turingserve_b200 import kernels
    kernels.use(None)
    return kernels.ops()


def tol(dtype):
    return dict(rtol=3e-5, atol=3e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# -- the stream's layer norm -------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,h", [(1, 72), (5, 131), (33, 192), (3, 2048), (2, 5000), (70, 48)])
def test_stream_layer_norm_takes_two_branches_a_constant_and_a_common_row(ops, dtype, T, h):
    """stream += alpha (a + b) + row, then (stream - mean) / sqrt(var + eps) w + bias: the stream stays 32-bit and is
    updated in place; every operand may be missing; ``first`` starts the stream from the operands."""
    g = torch.Generator(device=DEV).manual_seed(T * h)
    w = 1.0 + 0.3 * torch.randn(h, generator=g, device=DEV)
    bias = 0.2 * torch.randn(h, generator=g, device=DEV)
    row = torch.randn(h, generator=g, device=DEV)
    for alpha, with_b, with_row, first in ((0.7, True, True, False), (1.0, False, False, False), (0.25, True, False, False),
                                           (3.0, False, True, True), (13.5, False, False, True)):
        stream = 5.0 * torch.randn(T, h, generator=g, device=DEV) + 2.0             # a mean that is not zero
        a = torch.randn(T, h, generator=g, device=DEV).to(dtype)
        b = torch.randn(T, h, generator=g, device=DEV).to(dtype) if with_b else None
        want = (0.0 if first else stream.double()) + alpha * (a.double() + (b.double() if with_b else 0.0))
        if with_row:
            want = want + row.double()
        out = torch.empty(T, h, dtype=dtype, device=DEV)
        ops.rmsnorm_stream(out, stream, a, b, w, 1e-5, first, alpha=alpha, row=row if with_row else None, norm_bias=bias)
        assert torch.allclose(stream.double(), want, rtol=1e-6, atol=1e-6), (alpha, with_b, with_row, first)
        y = plain.layer_norm(want.cpu(), w.double().cpu(), bias.double().cpu(), 1e-5)
        assert torch.allclose(out.double().cpu(), y, **tol(dtype)), (alpha, with_b, with_row, first)


def test_stream_layer_norm_of_a_constant_row_is_the_bias_and_eps_sits_inside_the_root(ops):
    h = 40
    stream = torch.full((2, h), 7.0, device=DEV)
    w, bias = torch.full((h,), 2.0, device=DEV), torch.arange(h, dtype=torch.float32, device=DEV)
    out = torch.empty(2, h, device=DEV)
    ops.rmsnorm_stream(out, stream, None, None, w, 1e-6, False, norm_bias=bias)
    assert torch.allclose(out[0], bias) and torch.allclose(out[1], bias)
    # deviations of +-1 and eps = 3: (x - mean) / sqrt(1 + 3)
    stream = torch.tensor([[1.0, -1.0] * 8], device=DEV)
    out = torch.empty(1, 16, device=DEV)
    ops.rmsnorm_stream(out, stream, None, None, torch.ones(16, device=DEV), 3.0, False, norm_bias=torch.zeros(16, device=DEV))
    assert torch.allclose(out, stream / 2.0, atol=1e-6)


# -- rotation, per-head norm, cache write ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,V,rot,page", [(4, 2, 16, 8, 8, 16), (3, 3, 24, 40, 24, 8), (7, 1, 128, 72, 48, 64),
                                              (2, 1, 12, 20, 0, 4), (5, 5, 10, 6, 6, 16), (2, 2, 40, 24, 2, 8),
                                              (8, 2, 64, 64, 64, 32), (1, 1, 200, 3, 100, 16), (2, 1, 256, 64, 128, 16),
                                              (3, 1, 192, 40, 64, 8), (5, 2, 32, 16, 16, 8), (9, 3, 128, 128, 0, 16)])
def test_rotation_by_halves_then_unit_heads_into_the_cache(ops, dtype, H, G, D, V, rot, page):
    """q in place; rotated, normed keys and untouched values at slots of a shuffled pool; positions far from 0 (the
    angle is computed in 32-bit from the position itself); rot = 0: no rotation; dims behind ``rot`` pass."""
    g = torch.Generator(device=DEV).manual_seed(H * D + V)
    T = 23
    eps = 1e-3
    positions = [0, 1, 2, 63, 64, 65, 999, 4095, 4096, 70001] + list(range(300, 313))
    width = H * D + G * D + G * V
    proj = (torch.randn(T, width + 8, generator=g, device=DEV) * 2).to(dtype)[:, :width]       # rows with a stride
    before = proj.clone()
    base = 500.0
    freq = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(DEV) if rot else None
    n_pages = 9
    k_cache = torch.full((n_pages, G, page, D), 9.0, dtype=dtype, device=DEV)
    v_cache = torch.full((n_pages, G, page, V), 9.0, dtype=dtype, device=DEV)
    slots = torch.randperm(n_pages * page - page, generator=torch.Generator().manual_seed(1))[:T] + page
    ops.rope_headnorm_write(proj, H * D, H * D + G * D, i32(positions), freq, rot, eps, k_cache, v_cache,
                            slots.to(torch.int32).to(DEV), H, G, D, V, page)
    b = before.double().cpu()
    pos = torch.tensor(positions)
    q = plain.unit_rms(plain.rotate_half(b[:, :H * D].view(T, H, D), pos, rot, base), eps)
    k = plain.unit_rms(plain.rotate_half(b[:, H * D:H * D + G * D].view(T, G, D), pos, rot, base), eps)
    # (a 32-bit angle at position p is off by about p 2^-23 radians, frequency and product rounded once each: the
    # tolerance of a row follows its position)
    for t in range(T):
        slack = 1.0 + positions[t] / 50.0
        lim = {k_: v_ * slack for k_, v_ in tol(dtype).items()}
        assert torch.allclose(proj[t, :H * D].double().cpu().view(H, D), q[t], **lim), t
        page_i, at = int(slots[t]) // page, int(slots[t]) % page
        assert torch.allclose(k_cache[page_i, :, at].double().cpu(), k[t], **lim), t
        assert torch.equal(v_cache[page_i, :, at].cpu(), before[t, H * D + G * D:].view(G, V).cpu()), t
    assert torch.equal(proj[:, H * D:], before[:, H * D:])                          # k and v columns of the input stay
    written = torch.zeros(n_pages * page, dtype=torch.bool)
    written[slots] = True
    untouched = k_cache.permute(0, 2, 1, 3).reshape(n_pages * page, G, D)[~written.to(DEV)]
    assert float((untouched.float() - 9.0).abs().max()) == 0.0
    # without a cache (slots None) only q changes
    again = before.clone()
    ops.rope_headnorm_write(again, H * D, H * D + G * D, i32(positions), freq, rot, eps, k_cache, v_cache, None, H, G, D, V, page)
    assert torch.equal(again[:, :H * D], proj[:, :H * D])


@pytest.mark.parametrize("T", [1, 5, 8, 33, 100])
@pytest.mark.parametrize("H,G,D,V,rot", [(6, 2, 128, 72, 32), (12, 2, 128, 128, 64), (4, 2, 64, 64, 64), (3, 3, 24, 40, 24)])
def test_a_projection_left_unreduced_is_finished_by_the_rotation_kernel(ops, T, H, G, D, V, rot):
    """bfloat16, a few tokens: the q/k/v product leaves the partial sums of its cuts along K and the kernel that rotates
    sums them on the way: the same bits in q and in the cache as the finished product followed by the kernel."""
    from turingserve_b200 import kernels
    g = torch.Generator(device=DEV).manual_seed(T + D)
    K, page = 1536, 16
    N = (H + G) * D + G * V
    x = torch.randn(T, K, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device=DEV) * 0.05).to(torch.bfloat16)
    freq = (500000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(DEV)
    pos = i32([700 + 3 * t for t in range(T)])
    slots = i32([page + 2 * t for t in range(T)])
    results = []
    for defer in (False, True):
        out = torch.zeros(T, N, dtype=torch.bfloat16, device=DEV)
        k_cache = torch.zeros(2 + 2 * T // page + 1, G, page, D, dtype=torch.bfloat16, device=DEV)
        v_cache = torch.zeros(2 + 2 * T // page + 1, G, page, V, dtype=torch.bfloat16, device=DEV)
        proj = ops.linear(out, x, w, may_defer=defer, lazy=False)
        if defer and N % 8 == 0:
            assert isinstance(proj, kernels.Deferred)
        proj = ops.rope_headnorm_write(proj, H * D, (H + G) * D, pos, freq, rot, 1e-6, k_cache, v_cache, slots, H, G, D, V, page)
        results.append((proj[:, :H * D].clone(), k_cache, v_cache))
    for a, b in zip(*results):
        assert torch.equal(a, b)
    want = plain.unit_rms(plain.rotate_half((x.double() @ w.double().T).cpu()[:, :H * D].view(T, H, D),
                                            pos.cpu(), rot, 500000.0), 1e-6)
    assert torch.allclose(results[1][0].double().cpu().view(T, H, D), want, rtol=3e-2, atol=3e-2)


def test_rotation_keeps_scores_a_function_of_distance(ops):
    """The same q and k rows at positions (p + 7, p) for p = 0, 50, 3000: equal scores after rotation (no norm)."""
    H = G = 1
    D, rot = 32, 16
    g = torch.Generator(device=DEV).manual_seed(3)
    row = torch.randn(1, 3 * D, generator=g, device=DEV)
    freq = (100.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(DEV)
    scores = []
    for p in (0, 50, 3000):
        two = row.repeat(2, 1)
        k_cache = torch.zeros(2, 1, 4, D, device=DEV)
        v_cache = torch.zeros(2, 1, 4, D, device=DEV)
        ops.rope_headnorm_write(two, D, 2 * D, i32([p + 7, p]), freq, rot, None, k_cache, v_cache, i32([4, 5]), H, G, D, D, 4)
        scores.append(float((two[0, :D] * k_cache[1, 0, 1]).sum()))
    assert max(scores) - min(scores) < 2e-3 * abs(scores[0]) + 2e-4, scores


# -- attention in blocks of positions with a sink ----------------------------------------------------------------
def paged(rows, page, order=None):
    """rows [T, KVH, D] -> (cache [pages + 1, KVH, page, D], block table row): pages in ``order`` (shuffled pool)."""
    T, KVH, D = rows.shape
    n = -(-T // page)
    order = order or list(range(1, n + 1))
    cache = torch.zeros(max(order) + 1, KVH, page, D, dtype=rows.dtype, device=DEV)
    for j in range(T):
        cache[order[j // page], :, j % page] = rows[j]
    return cache, order


def attention_step(q_lens, seq_lens):
    starts = [0]
    for n in q_lens:
        starts.append(starts[-1] + n)
    return SimpleNamespace(q_start=i32(starts), seq_lens=i32(seq_lens), num_requests=len(q_lens),
                           num_decode=sum(1 for n in q_lens if n == 1), max_q_len=max(q_lens), max_seq_len=max(seq_lens))


def plain_sink_attention(q, k, v, KVH, scale, size, sink, first_pos):
    """q [Tq, H, Dk] at positions first_pos.., k [Tk, KVH, Dk], v [Tk, KVH, Dv] -> [Tq, H, Dv] in 64-bit."""
    Tq, H, _ = q.shape
    Tk = k.shape[0]
    per = H // KVH
    kk = k.double().cpu().repeat_interleave(per, dim=1)
    vv = v.double().cpu().repeat_interleave(per, dim=1)
    s = torch.einsum("ihd,jhd->hij", q.double().cpu(), kk) * scale
    ok = plain.visible(Tk, size)[first_pos:first_pos + Tq]
    s = s.masked_fill(~ok[None], -math.inf)
    p = plain.sink_softmax(s, None if sink is None else sink.double().cpu())
    return torch.einsum("hij,jhd->ihd", p, vv).float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KVH,Dk,Dv,page,size,sinks", [
    (4, 2, 16, 8, 16, 9, True), (3, 3, 24, 40, 8, 33, True), (6, 2, 128, 96, 64, 50, True), (4, 1, 16, 16, 4, 20, False),
    (6, 1, 8, 12, 8, None, True), (4, 2, 64, 64, 64, 64, True), (2, 1, 128, 128, 16, 100, True), (5, 5, 10, 6, 16, 7, True),
    (20, 1, 64, 64, 8, 40, True), (8, 2, 128, 128, 32, None, True), (40, 1, 128, 128, 16, 24, True)])
def test_blocks_and_sinks_in_batches_of_unequal_requests(ops, dtype, H, KVH, Dk, Dv, page, size, sinks):
    """A prompt from position 0, a portion that starts in the middle of a block and crosses two block edges, a single
    token that opens a block (it sees itself only: the sink takes most of its weight), a single token deep in a block,
    one with a context of one key; one launch, pages in a shuffled pool; against each request alone in the plain
    functions.  Key rows of 64 and 128 with values as wide go to the tensor cores in bfloat16."""
    g = torch.Generator(device=DEV).manual_seed(H * Dk + Dv)
    c = size or 1000
    opener = 3 * c + 1                                  # contexts whose last position is the first of a block
    q_lens, seq_lens = [1, 1, 1, 2 * c + 3, c + 5], [1, opener if size else 77, 2 * c + c // 2 + 2 if size else 130,
                                                      2 * c + 3 if size else 90, 4 * c + 2 if size else 300]
    if not size:
        q_lens[3], q_lens[4] = 90, 40
    sink = torch.randn(H, generator=g, device=DEV) * 1.5 if sinks else None
    ks, vs, tables = [], [], []
    base = 1
    for T in seq_lens:
        ks.append((torch.randn(T, KVH, Dk, generator=g, device=DEV) * 1.5).to(dtype))
        vs.append(torch.randn(T, KVH, Dv, generator=g, device=DEV).to(dtype))
        n = -(-T // page)
        tables.append(list(range(base, base + n))[::-1])
        base += n
    k_cache = torch.zeros(base, KVH, page, Dk, dtype=dtype, device=DEV)
    v_cache = torch.zeros(base, KVH, page, Dv, dtype=dtype, device=DEV)
    for k, v, order in zip(ks, vs, tables):
        for j in range(k.shape[0]):
            k_cache[order[j // page], :, j % page] = k[j]
            v_cache[order[j // page], :, j % page] = v[j]
    width = max(len(t) for t in tables)
    bt = i32([t + [0] * (width - len(t)) for t in tables])
    pad = 8 if Dk % 64 == 0 else 3
    q = (torch.randn(sum(q_lens), H, Dk + pad, generator=g, device=DEV) * 1.5).to(dtype)[:, :, pad:]
    out = torch.zeros(sum(q_lens), H, Dv + 2, dtype=dtype, device=DEV)[:, :, :Dv]
    step = attention_step(q_lens, seq_lens)
    for splits in (0, 1, 3):
        ops.biased_decode_splits = splits
        out.zero_()
        ops.attention_biased(out, q, k_cache, v_cache, bt, step, KVH, page, 0.3, 0.0, None, None, chunk=size, sinks=sink)
        at = 0
        for n, T, k, v in zip(q_lens, seq_lens, ks, vs):
            want = plain_sink_attention(q[at:at + n], k, v, KVH, 0.3, size, sink, T - n)
            loose = {k_: v_ * max(1.0, Dk / 64) for k_, v_ in tol(dtype).items()} if dtype == torch.float32 else tol(dtype)
            assert torch.allclose(out[at:at + n].float().cpu(), want, **loose), (splits, n, T)
            at += n
    ops.biased_decode_splits = 0


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("size,page", [(48, 16), (64, 64), (5, 8), (120, 64), (None, 16)])
@pytest.mark.parametrize("dtype,D", [(torch.float32, 12), (torch.bfloat16, 64), (torch.bfloat16, 128), (torch.bfloat16, 40)])
def test_one_loud_key_at_the_blocks_edges_at_page_edges_and_far_away(ops, size, page, decode, dtype, D):
    """Built inputs: all keys are silent but one, whose value is marked, and a sink far below.  The query finds it at
    the first place of its own block and does not find it one place before (the last place of the block before);
    at a page's last and first place; hundreds of tokens back when there are no blocks; never one place ahead of
    itself.  The query is the block's last position, a position in the middle of it, and the block's first position.
    ``decode``: the query comes alone (keys cut over several launch blocks) or at the end of a portion of 30."""
    H, KVH = 2, 1
    sink = torch.full((H,), -30.0, device=DEV)
    c = size or 10 ** 6
    for T in ((700 // c) * c if size else 700, (700 // c) * c + c // 2 + 1 if size else 650, (700 // c) * c + 1 if size else 601):
        n_q = 1 if decode else min(30, T)
        i = T - 1
        start = (i // c) * c
        cases = {i, start, start - 1, i - (i % page), i - (i % page) - 1, 0, 1, start + 1, start - c}
        if not size:
            cases |= {i - 500, 3 * page - 1, 3 * page}
        for j in sorted(x for x in cases if 0 <= x <= i):
            k = torch.zeros(T + 1, KVH, D, dtype=dtype, device=DEV)
            v = torch.zeros(T + 1, KVH, D, dtype=dtype, device=DEV)
            k[j, 0, 3] = 60.0
            v[j, 0, 7] = 1.0
            k[T, 0, 3] = 90.0                                  # one place ahead of the query: in the cache's page, unseen
            v[T, 0, 5] = 1.0
            k_cache, order = paged(k, page, order=list(range(-(-(T + 1) // page), 0, -1)))
            v_cache, _ = paged(v, page, order=order)
            q = torch.zeros(n_q, H, D, dtype=dtype, device=DEV)
            q[:, :, 3] = 1.0
            out = torch.empty(n_q, H, D, dtype=dtype, device=DEV)
            ops.attention_biased(out, q, k_cache, v_cache, i32([order]), attention_step([n_q], [T]), KVH, page, 1.0, 0.0,
                                 None, None, chunk=size, sinks=sink)
            seen = j >= start
            assert abs(float(out[-1, 0, 7]) - (1.0 if seen else 0.0)) < 1e-6, (T, j, seen)
            assert float(out[-1, :, 5].abs().max()) == 0.0, (T, j)


@pytest.mark.parametrize("dtype,D", [(torch.float32, 20), (torch.bfloat16, 64), (torch.bfloat16, 24)])
def test_the_sink_counts_once_unscaled_and_has_no_value(ops, dtype, D):
    """Built inputs: n equal keys with score 0 and a sink s_h give every key the weight 1 / (n + e^{s_h}), whatever the
    score scale is; the sink adds no value, so the output's sum is n / (n + e^{s_h}); a sink far above every score
    leaves nearly nothing, one far below is a plain softmax; heads have sinks of their own.  The first position of a
    block (n = 1), a position inside (n = 7), a single token and a portion, keys over two pages."""
    H, page, size = 3, 4, 9
    sink = torch.tensor([0.0, math.log(3.0), -40.0], device=DEV)
    for T, n_q in ((10, 1), (16, 1), (16, 5), (30, 30)):
        k = torch.zeros(T, 1, D, dtype=dtype, device=DEV)
        v = torch.ones(T, 1, D, dtype=dtype, device=DEV)
        k_cache, order = paged(k, page)
        v_cache, _ = paged(v, page)
        q = torch.ones(n_q, H, D, dtype=dtype, device=DEV)
        out = torch.empty(n_q, H, D, dtype=dtype, device=DEV)
        ops.attention_biased(out, q, k_cache, v_cache, i32([order]), attention_step([n_q], [T]), 1, page, 0.37, 0.0, None,
                             None, chunk=size, sinks=sink)
        for r in range(n_q):
            n = (T - n_q + r) % size + 1
            for h, extra in enumerate((1.0, 3.0, 0.0)):
                assert abs(float(out[r, h, 0]) - n / (n + extra)) < (1e-6 if dtype == torch.float32 else 4e-3), (T, r, h)
    # a loud sink: the keys keep e^{-20} of the weight
    sink = torch.tensor([20.0, 20.0, 20.0], device=DEV)
    ops.attention_biased(out, q, k_cache, v_cache, i32([order]), attention_step([n_q], [T]), 1, page, 0.37, 0.0, None, None,
                         chunk=size, sinks=sink)
    assert float(out.float().abs().max()) < 1e-7


# -- the router with a correction, gated experts, identity outputs -----------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("outputs,top,K", [(5, 3, 72), (11, 4, 160), (4, 4, 48), (7, 1, 33), (2, 2, 32), (64, 6, 100)])
def test_the_correction_enters_the_choice_and_not_the_weights(ops, dtype, outputs, top, K):
    """Softmax over all router outputs; the choice by score + correction; the weights are the scores themselves, not
    renormalised.  A correction as large as the scores: the choice differs from the uncorrected one."""
    g = torch.Generator(device=DEV).manual_seed(outputs * K)
    T = 40
    x = torch.randn(T, K, generator=g, device=DEV).to(dtype)
    wr = torch.randn(outputs, K, generator=g, device=DEV) * 0.3
    corr = torch.randn(outputs, generator=g, device=DEV) * 0.3
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    changed = 0
    for c in (corr, None):
        ops.router_topk(idx, wts, x, wr, True, False, c)
        want_idx, want_w = plain.route(x.double().cpu(), wr.double().cpu(), None if c is None else c.double().cpu(), top)
        s = torch.softmax(x.double().cpu() @ wr.double().cpu().T, -1)
        for t in range(T):
            got = idx[t].cpu().tolist()
            assert len(set(got)) == top and all(0 <= e < outputs for e in got), (t, got)
            if sorted(got) != sorted(want_idx[t].tolist()):
                # a close call between two outputs: the choice scores of the two differ by rounding only
                pick = s[t] + (0.0 if c is None else c.double().cpu())
                odd = set(got) ^ set(want_idx[t].tolist())
                assert max(pick[list(odd)]) - min(pick[list(odd)]) < 1e-5, (t, got, want_idx[t].tolist())
            assert torch.allclose(wts[t].double().cpu(), s[t][got], rtol=1e-4, atol=1e-6), t
        if c is not None and top < outputs:
            plain_idx, _ = plain.route(x.double().cpu(), wr.double().cpu(), None, top)
            changed = sum(sorted(a) != sorted(b) for a, b in zip(plain_idx.tolist(), want_idx.tolist()))
            assert changed > 0
    if top == outputs:
        assert torch.allclose(wts.sum(-1), torch.ones(T, device=DEV), atol=1e-5)           # all chosen: the whole softmax


def test_a_built_correction_turns_the_choice_round(ops):
    """Scores (0.6, 0.3, 0.1) whatever the token; corrections (0, 0, 1): top 1 is output 2 with weight 0.1."""
    K = 8
    x = torch.zeros(3, K, device=DEV)
    x[:, 0] = 1.0
    wr = torch.zeros(3, K, device=DEV)
    wr[:, 0] = torch.log(torch.tensor([0.6, 0.3, 0.1]))
    idx = torch.empty(3, 1, dtype=torch.int32, device=DEV)
    wts = torch.empty(3, 1, device=DEV)
    ops.router_topk(idx, wts, x, wr, True, False, torch.tensor([0.0, 0.0, 1.0], device=DEV))
    assert idx.flatten().tolist() == [2, 2, 2] and torch.allclose(wts, torch.full((3, 1), 0.1, device=DEV), atol=1e-6)
    ops.router_topk(idx, wts, x, wr, True, False, None)
    assert idx.flatten().tolist() == [0, 0, 0] and torch.allclose(wts, torch.full((3, 1), 0.6, device=DEV), atol=1e-6)


def routed_part(dtype, W, ff, E, identity, top, g, monkeypatch=None):
    from turingserve_b200.config.model_config import RoutedMLPSpec
    from turingserve_b200.parts.base import BuildContext
    from turingserve_b200.parts.routed_mlp import RoutedMLP
    spec = RoutedMLPSpec(num_experts=E, top_k=top, intermediate_size=ff, activation="silu", scoring="softmax",
                         renormalize=False, weight_on="output", gated=True, correction=True, identity=identity)
    part = RoutedMLP(spec, BuildContext(W, dtype, torch.device(DEV), 0))
    t = {"router": torch.randn(E + identity, W, generator=g, device=DEV) * 0.4,
         "correction": torch.randn(E + identity, generator=g, device=DEV) * 0.2}
    for e in range(E):
        for n, shape in (("gate", (ff, W)), ("up", (ff, W)), ("down", (W, ff))):
            t[f"e{e}.{n}"] = (torch.randn(*shape, generator=g, device=DEV) * 0.3).to(dtype)
    part.load(t)
    return part, {k: v.double().cpu() for k, v in t.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,ff,E,identity,top,T", [(72, 24, 3, 2, 3, 50), (48, 20, 1, 3, 4, 33), (64, 16, 4, 0, 1, 90),
                                                    (128, 64, 8, 4, 4, 1), (32, 12, 2, 2, 2, 7), (160, 48, 8, 3, 5, 400),
                                                    (40, 8, 0, 3, 2, 9)])
def test_gated_experts_with_identity_outputs_against_the_plain_sum(ops, dtype, W, ff, E, identity, top, T, monkeypatch):
    """The routed feed-forward as a part, with the grouped kernels and with every expert's rows as a product of their
    own: experts with tensors beside outputs that return the token's own row times its weight; one expert with tensors
    among three identity outputs with top = all; no identity outputs; no expert with tensors at all; a single token."""
    from turingserve_b200.parts.routed_mlp import RoutedMLP
    g = torch.Generator(device=DEV).manual_seed(W + ff + T)
    part, w = routed_part(dtype, W, ff, E, identity, top, g)
    x = torch.randn(T, W, generator=g, device=DEV).to(dtype)
    f = {"router": {"experts": E, "identity": identity, "top": top}}
    want = plain.routed_ff(x.double().cpu(), w, f)
    if identity and top < E + identity:
        idx, _ = plain.route(x.double().cpu(), w["router"], w["correction"], top)
        assert bool((idx >= E).any()) and (E == 0 or bool((idx < E).any()))       # both kinds are chosen
    lim = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2 * float(want.abs().max()))
    for rows in (10 ** 9, 1):
        monkeypatch.setattr(RoutedMLP, "LIBRARY_ROWS", rows)
        got = part.forward(x).double().cpu()
        assert torch.allclose(got, want, **lim), rows


def test_identity_outputs_alone_return_the_input_times_the_weights(ops):
    """Every router output an identity one and top = all: ff(h) = h (the softmax sums to one); top 1 of built scores
    (0.7, 0.2, 0.1) with a correction for the last: 0.1 h."""
    g = torch.Generator(device=DEV).manual_seed(2)
    part, _ = routed_part(torch.float32, 40, 8, 0, 3, 3, g)
    x = torch.randn(11, 40, generator=g, device=DEV)
    assert torch.allclose(part.forward(x), x, rtol=1e-5, atol=1e-6)
    part, _ = routed_part(torch.float32, 40, 8, 0, 3, 1, g)
    wr = torch.zeros(3, 40, device=DEV)
    wr[:, 0] = torch.log(torch.tensor([0.7, 0.2, 0.1]))
    part.load({"router": wr, "correction": torch.tensor([0.0, 0.0, 2.0], device=DEV)})
    x[:, 0] = 1.0
    assert torch.allclose(part.forward(x), 0.1 * x, rtol=1e-5, atol=1e-6)
