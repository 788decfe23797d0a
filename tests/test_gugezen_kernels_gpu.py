"""Each Gugezen mechanism's kernels alone on the GPU against the plain functions of ``tests/plain_gugezen.py``: sizes
that are no powers of two, values that a real configuration makes equal or 1 made different, and inputs built so that
one wrong key, state row, stream copy or expert shows."""

from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch
import torch.nn.functional as F

from tests import plain_gugezen as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture()
def ops():
    from turingserve_b200 import kernels
    kernels.use(None)
    return kernels.ops()


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# -- the stream in several copies --------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,hidden", [(1, 48), (2, 256), (3, 72), (5, 1030), (8, 200)])
def test_stream_copies_start_write_back_read_and_norm(ops, dtype, S, hidden):
    g = torch.Generator(device=DEV).manual_seed(S * hidden)
    T, eps = 7, 1e-5
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=DEV)
    rows, y = (rnd(T, hidden) * 2).to(dtype), (rnd(T, hidden) * 3).to(dtype)
    w = 1 + 0.3 * rnd(hidden)
    w_in, w_out, mix = 1.0 / S + 0.3 * rnd(S), 1 + 0.3 * rnd(S), torch.eye(S, device=DEV) + 0.2 * rnd(S, S)
    streams = torch.full((T, S, hidden), 99.0, device=DEV)
    out = torch.empty(T, hidden, dtype=dtype, device=DEV)
    # the start: every copy is the rows times the constant; 99 is never read
    ops.hyper_norm(out, streams, rows, None, None, w_in, w, eps, first=True, alpha=2.5)
    x0 = 2.5 * rows.float()
    assert torch.equal(streams, x0[:, None, :].expand(T, S, hidden))
    u = w_in.sum() * x0
    assert torch.allclose(out.float(), plain.unit_rms(u, eps) * w, **tol(dtype))
    # a pending output comes back through mix ([from, to]) and out, all copies at once from the old ones
    xs = streams.clone()
    ops.hyper_norm(out, streams, y, mix, w_out, w_in, w, eps)
    want = torch.einsum("st,bsh->bth", mix, xs) + w_out[None, :, None] * y.float()[:, None, :]
    assert torch.allclose(streams, want, rtol=1e-5, atol=1e-5)
    u = torch.einsum("s,bsh->bh", w_in, want)
    assert torch.allclose(out.float(), plain.unit_rms(u, eps) * w, **tol(dtype))
    # the model's last norm reads the plain sum of the copies; nothing pending changes nothing
    before = streams.clone()
    ops.hyper_norm(out, streams, None, None, None, None, w, eps)
    assert torch.equal(streams, before)
    assert torch.allclose(out.float(), plain.unit_rms(before.sum(1), eps) * w, **tol(dtype))
    # without link tensors a copy is the ordinary residual sum
    ops.hyper_norm(out, streams, y, None, None, None, w, eps)
    assert torch.allclose(streams, before + y.float()[:, None, :], rtol=1e-6, atol=1e-6)
    # eps sits inside the root
    tiny = torch.full((T, hidden), 1e-4, device=DEV).to(dtype)
    ops.hyper_norm(out, streams, tiny, None, None, None, w, 1e-2, first=True)
    v = S * float(tiny[0, 0])
    assert torch.allclose(out.float(), torch.full((T, hidden), v / math.sqrt(v * v + 1e-2), device=DEV) * w, rtol=2e-2, atol=1e-7)


@pytest.mark.parametrize("T", [1, 5, 40])
def test_a_product_put_off_is_finished_by_the_stream_norm(ops, T):
    """bfloat16, few tokens: the output projection's split sums arrive unreduced and are summed, rounded as the product's
    own epilogue rounds, on their way into the copies."""
    g = torch.Generator(device=DEV).manual_seed(T)
    S, hidden, K = 2, 256, 1536
    x = (torch.randn(T, K, generator=g, device=DEV) * 0.5).bfloat16()
    wo = (torch.randn(hidden, K, generator=g, device=DEV) * 0.05).bfloat16()
    lazy = ops.linear(torch.empty(T, hidden, dtype=torch.bfloat16, device=DEV), x, wo, may_defer=True)
    from turingserve_b200.kernels import Deferred, LazyProduct
    assert isinstance(lazy, (LazyProduct, Deferred))
    mix, w_out = torch.tensor([[0.9, 0.2], [-0.1, 1.1]], device=DEV), torch.tensor([1.2, 0.7], device=DEV)
    streams = torch.randn(T, S, hidden, generator=g, device=DEV)
    xs = streams.clone()
    out = torch.empty(T, hidden, dtype=torch.bfloat16, device=DEV)
    w = torch.ones(hidden, device=DEV)
    ops.hyper_norm(out, streams, lazy, mix, w_out, None, w, 1e-6)
    y = (x.float() @ wo.float().T).bfloat16().float()
    want = torch.einsum("st,bsh->bth", mix, xs) + w_out[None, :, None] * y[:, None, :]
    assert torch.allclose(streams, want, rtol=1e-2, atol=2e-2)
    assert torch.allclose(out.float(), plain.unit_rms(streams.sum(1), 1e-6), **tol(torch.bfloat16))


# -- gates, grouped norms, activations ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,groups", [(72, 1), (72, 3), (256, 2), (1030, 5), (60, 60)])
def test_gated_norm_in_parts(ops, dtype, n, groups):
    g = torch.Generator(device=DEV).manual_seed(n + groups)
    T = 5
    x = torch.randn(T, n, generator=g, device=DEV) * 4
    wide = torch.randn(T, 3 * n, generator=g, device=DEV).to(dtype)
    gate = wide[:, n:2 * n]
    w = 1 + 0.3 * torch.randn(n, generator=g, device=DEV)
    room = torch.zeros(T, 2 * n + 8, dtype=dtype, device=DEV)
    out = room[:, 8:8 + n]                                            # a column slice of a wider tensor
    parts = lambda v: plain.unit_rms(v.view(T, groups, n // groups), 1e-5).reshape(T, n)
    ops.gated_group_rmsnorm(out, x, gate, w, 1e-5, groups, "silu", True)            # the gate comes before the norm
    assert torch.allclose(out.float(), parts(x * F.silu(gate.float())) * w, **tol(dtype))
    ops.gated_group_rmsnorm(out, x, gate, w, 1e-5, groups, "sigmoid", False, 0.7)   # the gate and a constant behind it
    assert torch.allclose(out.float(), parts(x) * w * torch.sigmoid(gate.float()) * 0.7, **tol(dtype))
    assert float(room[:, :8].abs().max()) == 0.0 and float(room[:, 8 + n:].abs().max()) == 0.0
    a = torch.randn(T, n + 4, generator=g, device=DEV).to(dtype)[:, 4:]
    ops.gate_mul(out, a, gate, "sigmoid", 1.3)
    assert torch.allclose(out.float(), a.float() * torch.sigmoid(gate.float()) * 1.3, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations_and_gated_products(ops, dtype):
    z = torch.linspace(-6, 6, 1001, device=DEV).to(dtype)
    for kind, f in (("gelu", plain.gelu_erf), ("gelu_tanh", plain.gelu_tanh)):
        y = torch.empty_like(z)
        ops.activation(y, z, kind)
        assert torch.allclose(y.float(), f(z.float()), **tol(dtype)), kind
    g = torch.Generator(device=DEV).manual_seed(1)
    for T, inter, group in ((3, 40, 0), (5, 384, 64), (2, 128, 64), (4, 21, 0)):
        gate, up = (torch.randn(T, inter, generator=g, device=DEV) * 2).to(dtype), torch.randn(T, inter, generator=g, device=DEV).to(dtype)
        if group:
            gu = torch.cat([gate.view(T, -1, 1, group), up.view(T, -1, 1, group)], 2).reshape(T, 2 * inter)
        else:
            gu = torch.cat([gate, up], 1)
        for kind, f in (("gelu_tanh", plain.gelu_tanh), ("gelu", plain.gelu_erf), ("silu", F.silu)):
            out = torch.empty(T, inter, dtype=dtype, device=DEV)
            ops.act_mul(out, gu.contiguous(), kind, group)
            assert torch.allclose(out.float(), f(gate.float()) * up.float(), **tol(dtype)), (kind, inter, group)


# -- rotation of neighbouring pairs with the cache write ----------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,V,rot,page", [(4, 2, 16, 8, 8, 16), (3, 3, 24, 40, 24, 8), (8, 4, 64, 64, 64, 64),
                                              (2, 1, 128, 128, 32, 16), (5, 5, 10, 6, 0, 4), (6, 1, 8, 12, 2, 8)])
def test_neighbouring_pairs_turn_and_keys_and_values_reach_their_slots(ops, dtype, H, G, D, V, rot, page):
    g = torch.Generator(device=DEV).manual_seed(H * D + V)
    T = 23
    n_in = (H + G) * D + G * V
    wide = (torch.randn(T, n_in + 24, generator=g, device=DEV) * 2).to(dtype)
    proj = wide[:, 8:8 + n_in + 8]                                    # rows inside a wider tensor; gate columns behind
    before = proj.clone()
    positions = i32([0, 1, 2, 3, 500, 70001] + list(range(40, 40 + T - 6)))
    freq = torch.tensor(plain.scaled_frequencies(300.0, rot, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64.0}),
                        dtype=torch.float32, device=DEV) if rot else None
    pages = 7
    slots = torch.randperm(pages * page, generator=torch.Generator().manual_seed(3))[:T].to(torch.int32)
    slots[5] = -1                                                     # a row that caches nothing
    slots = slots.to(DEV)
    k_cache = torch.zeros(pages, G, page, D, dtype=dtype, device=DEV)
    v_cache = torch.zeros(pages, G, page, V, dtype=dtype, device=DEV)
    ops.rope_pairs_write(proj, H * D, (H + G) * D, positions, freq, 1.0, rot, k_cache, v_cache, slots, H, G, D, V, page)
    f = freq.double().cpu().tolist() if rot else []
    pos = positions.cpu()
    q_want = plain.rotate_neighbours(before[:, :H * D].double().cpu().view(T, H, D), pos, f)
    k_want = plain.rotate_neighbours(before[:, H * D:(H + G) * D].double().cpu().view(T, G, D), pos, f)
    # angles up to 70,001 radians in 32-bit: an absolute error of a few 1e-3 there, 3e-5 at position 500, nothing below 100
    loose = dict(rtol=2e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=2e-2)
    tight = tol(dtype) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)      # (32-bit frequencies times 60)
    got_q = proj[:, :H * D].double().cpu().view(T, H, D)
    far = pos > 1000
    assert torch.allclose(got_q[~far], q_want[~far], **{k_: float(v_) for k_, v_ in tight.items()})
    assert torch.allclose(got_q[far], q_want[far], **loose)
    assert torch.equal(proj[:, H * D:], before[:, H * D:])            # k, v and what lies behind stay as projected
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        kk = k_cache[s // page, :, s % page].double().cpu()
        assert torch.allclose(kk, k_want[t], **(loose if far[t] else {k_: float(v_) for k_, v_ in tight.items()}))
        assert torch.equal(v_cache[s // page, :, s % page].reshape(-1), before[t, (H + G) * D:(H + G) * D + G * V])
    assert int((k_cache.abs().sum((1, 3)) > 0).sum()) <= T - 1        # nothing written anywhere else
    # without slots nothing is cached and q still turns
    again = before.clone()
    ops.rope_pairs_write(again, H * D, (H + G) * D, positions, freq, 1.0, rot, None, None, None, H, G, D, V, page)
    assert torch.equal(again[:, :H * D], proj[:, :H * D])


def test_rotated_scores_depend_on_the_distance_only(ops):
    H, G, D, page = 1, 1, 32, 16
    freq = torch.tensor(plain.scaled_frequencies(10000.0, D, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128.0}),
                        dtype=torch.float32, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(0)
    q0, k0 = torch.randn(D, generator=g, device=DEV), torch.randn(D, generator=g, device=DEV)
    scores = []
    for p in (0, 9, 300, 2000):
        proj = torch.cat([q0, k0, torch.zeros(4, device=DEV)])[None].repeat(2, 1).contiguous()
        k_cache = torch.zeros(2, G, page, D, device=DEV)
        v_cache = torch.zeros(2, G, page, 4, device=DEV)
        ops.rope_pairs_write(proj, D, 2 * D, i32([p + 7, p]), freq, 1.0, D, k_cache, v_cache, i32([16, 17]), H, G, D, 4, page)
        scores.append(float(proj[0, :D] @ k_cache[1, 0, 1]))
    assert max(scores) - min(scores) < 2e-3 * abs(scores[0]) + 2e-4, scores


def paged(rows, page, order):
    T, KVH, D = rows.shape
    cache = torch.zeros(max(order) + 1, KVH, page, D, dtype=rows.dtype, device=DEV)
    for j in range(T):
        cache[order[j // page], :, j % page] = rows[j]
    return cache


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype,D,page", [(torch.float32, 12, 16), (torch.bfloat16, 64, 64), (torch.bfloat16, 128, 16), (torch.bfloat16, 40, 8)])
def test_one_loud_key_far_away_and_at_page_edges_through_rotation_cache_and_attention(ops, decode, dtype, D, page):
    """Built inputs: every key is silent but one, marked in dimensions the rotation does not touch, whose value is marked
    too, and a sink far below.  The query finds it hundreds of tokens back, at a page's last and first place, at position
    0 and at its own place; never one place ahead of itself.  The query comes alone or at the end of a portion of 30."""
    H, G, rot = 2, 1, 8
    freq = torch.tensor(plain.scaled_frequencies(100.0, rot, None), dtype=torch.float32, device=DEV)
    sink = torch.full((H,), -30.0, device=DEV)
    for T in (700, 641, 1):
        n_q = 1 if decode else min(30, T)
        i = T - 1
        for j in sorted({x for x in (i, 0, 1, i - 500, i - (i % page), i - (i % page) - 1, 3 * page - 1, 3 * page) if 0 <= x <= i}):
            k = torch.zeros(T + 1, G, D, dtype=dtype, device=DEV)
            v = torch.zeros(T + 1, G, D, dtype=dtype, device=DEV)
            k[j, 0, rot + 1] = 60.0
            v[j, 0, 7] = 1.0
            k[T, 0, rot + 1] = 90.0                            # one place ahead of the query: in the cache's page, unseen
            v[T, 0, 5] = 1.0
            order = list(range(-(-(T + 1) // page), 0, -1))
            k_cache, v_cache = paged(k, page, order), paged(v, page, order)
            # the step's own rows go through the rotation kernel into their slots (the rest is there already)
            proj = torch.zeros(n_q, (H + 2 * G) * D, dtype=dtype, device=DEV)
            proj[:, rot + 1] = 1.0
            proj[:, D + rot + 1] = 1.0
            first = T - n_q
            proj[:, H * D:(H + G) * D] = k[first:T, 0]
            proj[:, (H + G) * D:] = v[first:T, 0]
            slots = i32([order[p // page] * page + p % page for p in range(first, T)])
            ops.rope_pairs_write(proj, H * D, (H + G) * D, i32(list(range(first, T))), freq, 1.0, rot, k_cache, v_cache,
                                 slots, H, G, D, D, page)
            out = torch.empty(n_q, H, D, dtype=dtype, device=DEV)
            step = SimpleNamespace(q_start=i32([0, n_q]), seq_lens=i32([T]), num_requests=1, num_decode=1 if n_q == 1 else 0,
                                   max_q_len=n_q, max_seq_len=T)
            ops.attention_biased(out, proj[:, :H * D].view(n_q, H, D), k_cache, v_cache, i32([order]), step, G, page, 1.0,
                                 0.0, None, None, chunk=None, sinks=sink)
            assert abs(float(out[-1, 0, 7]) - 1.0) < 1e-6, (T, j)
            assert float(out[-1, :, 5].abs().max()) == 0.0, (T, j)


# -- the state-space mixer ---------------------------------------------------------------------------------------------
def ssm_sizes(H, P, N, G):
    inner, channels = H * P, H * P + 2 * G * N
    return inner, channels, 2 * inner + 2 * G * N + H


def run_ssm(ops, proj, state, consts, cuts, slots, H, P, N, G, taps):
    """The rows of ``proj`` belong to len(slots) requests of equal length; ``cuts`` are the step sizes."""
    conv_w, conv_b, a_log, dt_bias, skip = consts
    inner, channels, _ = ssm_sizes(H, P, N, G)
    n_req, T = len(slots), proj.shape[0] // len(slots)
    out = torch.empty(proj.shape[0], inner, device=DEV)
    at = 0
    for c in cuts:
        rows = torch.cat([torch.arange(r * T + at, r * T + at + c) for r in range(n_req)]).to(DEV)
        step = SimpleNamespace(q_start=i32([i * c for i in range(n_req + 1)]), state_slots=i32(slots), num_requests=n_req,
                               token_request=i32([r for r in range(n_req) for _ in range(c)]))
        p = proj[rows].contiguous()
        ready = torch.empty(len(rows), channels + 2 * H, device=DEV)
        ops.ssm_prepare(ready, p, inner, inner + channels, conv_w, conv_b, a_log, dt_bias, state, H * N * P, step, H, channels, taps)
        o = torch.empty(len(rows), inner, device=DEV)
        ops.ssm_scan(o, ready, p, inner, state, skip, step, H, G, N, P, taps)
        out[rows] = o
        at += c
    assert at == T
    return out


def plain_ssm(proj, consts, H, P, N, G):
    """One request's rows [T, n_in] -> (y [T, H P], final state [H, N, P]) in 64-bit."""
    conv_w, conv_b, a_log, dt_bias, skip = (c.double().cpu() for c in consts)
    inner, channels, _ = ssm_sizes(H, P, N, G)
    u = proj.double().cpu()
    T = u.shape[0]
    xbc = plain.silu(plain.causal_filter(u[:, inner:inner + channels], conv_w, conv_b))
    x, B, C = xbc[:, :inner].view(T, H, P), xbc[:, inner:inner + G * N].view(T, G, N), xbc[:, inner + G * N:].view(T, G, N)
    dt = plain.softplus(u[:, inner + channels:] + dt_bias)
    y = plain.state_space_scan(x, dt, a_log, B, C, skip).reshape(T, inner)
    S = torch.zeros(H, N, P, dtype=torch.float64)
    for h in range(H):
        for t in range(T):
            S[h] = torch.exp(-torch.exp(a_log[h]) * dt[t, h]) * S[h] + dt[t, h] * torch.outer(B[t, h // (H // G)], x[t, h])
    return y.float(), S.float()


def ssm_consts(g, H, channels, taps):
    rnd = lambda *s: torch.randn(*s, generator=g, device=DEV)
    return (rnd(channels, taps) * 0.5, rnd(channels) * 0.2, 2 * torch.rand(H, generator=g, device=DEV) - 1.5, rnd(H) * 0.7,
            1 + 0.3 * rnd(H))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,P,N,G,taps", [(4, 6, 10, 2, 4), (2, 16, 7, 1, 2), (3, 8, 16, 3, 1), (4, 32, 64, 1, 4),
                                          (2, 64, 128, 2, 3), (6, 4, 9, 2, 3), (2, 40, 256, 1, 8)])
def test_state_space_whole_in_portions_and_token_by_token(ops, dtype, H, P, N, G, taps):
    """The same tokens as one portion, as portions down to two tokens and one (shorter than the filter's memory), and
    one by one: the same outputs, the same state and the same filter memory; two requests in one launch with slots that
    are not their batch rows.  Sizes in multiples of 4 (rows fetched by 16-byte copies) and others; states of 7 to 256
    rows; value columns that do not fill a block; filters of 1 to 8 taps."""
    g = torch.Generator(device=DEV).manual_seed(H * P + N)
    inner, channels, n_in = ssm_sizes(H, P, N, G)
    T = 37
    consts = ssm_consts(g, H, channels, taps)
    proj = (torch.randn(2 * T, n_in, generator=g, device=DEV)).to(dtype)
    wants = [plain_ssm(proj[r * T:(r + 1) * T], consts, H, P, N, G) for r in range(2)]
    width = H * N * P + (taps - 1) * channels
    results = []
    for cuts in ([T], [16, 2, 1, 1, 5, 2, 10], [1] * T):
        state = torch.zeros(6, width, device=DEV)
        state[0] = 7.0                                         # rows of other requests: never touched
        out = run_ssm(ops, proj, state, consts, cuts, [4, 2], H, P, N, G, taps)
        for r, slot in enumerate((4, 2)):
            assert torch.allclose(out[r * T:(r + 1) * T].cpu(), wants[r][0], rtol=2e-4, atol=2e-4), (cuts[:3], r)
            assert torch.allclose(state[slot, :H * N * P].cpu().view(H, N, P), wants[r][1], rtol=2e-4, atol=2e-4)
            if taps > 1:
                tail = state[slot, H * N * P:].view(taps - 1, channels)
                assert torch.equal(tail, proj[r * T:(r + 1) * T][-(taps - 1):, inner:inner + channels].float())
        assert float((state[0] - 7.0).abs().max()) == 0.0 and float(state[[1, 3, 5]].abs().max()) == 0.0
        results.append((out.clone(), state.clone()))
    for out, state in results[1:]:                             # cutting a prompt changes no bit
        assert torch.equal(out, results[0][0]) and torch.equal(state, results[0][1])


def test_state_space_memory_kept_and_forgotten_and_long_decoding(ops):
    """Built inputs: a head whose decay is almost 1 still reads, 400 tokens later, what one early token wrote; a head that
    decays fast has forgotten it.  Then 600 single steps against the plain scan."""
    H, P, N, G, taps = 2, 8, 8, 1, 1
    inner, channels, n_in = ssm_sizes(H, P, N, G)
    T = 420
    conv_w, conv_b = torch.ones(channels, 1, device=DEV), torch.zeros(channels, device=DEV)
    a_log = torch.tensor([-12.0, 1.0], device=DEV)             # exp(-exp(A) dt): 0.999996 and 0.15 a token at dt = 0.69
    consts = (conv_w, conv_b, a_log, torch.zeros(H, device=DEV), torch.zeros(H, device=DEV))
    proj = torch.zeros(T, n_in, device=DEV)
    proj[:, inner + inner:] = -20.0                            # B and C: silu(-20) = 0
    proj[:, inner:2 * inner] = -20.0
    proj[:, inner + channels:] = 0.0                           # dt = softplus(0)
    proj[3, inner:2 * inner] = 5.0                             # token 3 writes x = silu(5) through B
    proj[3, 2 * inner + 2] = 5.0
    proj[T - 1, 2 * inner + N + 2] = 5.0                       # the last token reads through C, row 2
    state = torch.zeros(2, H * N * P, device=DEV)
    out = run_ssm(ops, proj, state, consts, [200, 1, 1, 218], [1], H, P, N, G, taps)
    s5 = float(F.silu(torch.tensor(5.0)))
    dt = math.log(2.0)
    keep = math.exp(-math.exp(-12.0) * dt) ** (T - 1 - 3)
    assert abs(float(out[-1, 0]) - dt * s5 * s5 * s5 * keep) < 1e-3 * s5 ** 3
    assert abs(float(out[-1, P])) < 1e-10                      # the fast head forgot (silu(-20) is -4e-8, not 0)
    g = torch.Generator(device=DEV).manual_seed(5)
    H, P, N, G, taps = 3, 12, 20, 3, 3
    inner, channels, n_in = ssm_sizes(H, P, N, G)
    consts = ssm_consts(g, H, channels, taps)
    proj = torch.randn(600, n_in, generator=g, device=DEV)
    state = torch.zeros(3, H * N * P + (taps - 1) * channels, device=DEV)
    out = run_ssm(ops, proj, state, consts, [1] * 600, [2], H, P, N, G, taps)
    want, S = plain_ssm(proj, consts, H, P, N, G)
    assert torch.allclose(out.cpu(), want, rtol=5e-4, atol=5e-4)
    assert torch.allclose(state[2, :H * N * P].cpu().view(H, N, P), S, rtol=5e-4, atol=5e-4)


# -- the routed feed-forward with its shared expert, the gated dense one ---------------------------------------------------
def build_part(family, spec, hidden, dtype):
    from turingserve_b200.parts.base import BuildContext, build
    return build(family, spec, BuildContext(hidden_size=hidden, dtype=dtype, device=torch.device(DEV), max_positions=64))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,ff,E,top,shared,T", [(72, 24, 5, 2, 16, 9), (48, 8, 3, 1, 24, 5), (128, 32, 8, 8, None, 4),
                                                 (256, 64, 16, 3, 128, 700), (64, 16, 1, 1, 8, 3)])
def test_routed_experts_renormalised_with_a_shared_expert(ops, dtype, W, ff, E, top, shared, T):
    """Through the part (both product paths: grouped kernels, and one product an expert from 1,024 pairs on) against the
    plain sum.  bfloat16 is compared where the plain router's choice is no close call."""
    from turingserve_b200.config.model_config import RoutedMLPSpec
    g = torch.Generator(device=DEV).manual_seed(W + E)
    spec = RoutedMLPSpec(num_experts=E, top_k=top, intermediate_size=ff, activation="gelu", scoring="softmax",
                         renormalize=True, weight_on="output", shared_intermediate_size=shared)
    part = build_part("feed_forward", spec, W, dtype)
    tensors = {}
    for name, p in part.parameters().items():
        t = torch.randn(p.shape, generator=g, device=DEV) * (0.6 if name == "router" else 0.15)
        tensors[name] = t if not p.compute_dtype else t.to(dtype)
    part.load(tensors)
    x = torch.randn(T, W, generator=g, device=DEV).to(dtype)
    got = part.forward(x).float().cpu()
    Wd = {"p." + k: v.double().cpu() for k, v in tensors.items()}
    f = {"router": {"experts": E, "top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.routed_ff(x.double().cpu(), Wd, "p.", f).float()
    if dtype == torch.float32:
        assert torch.allclose(got, want, rtol=1e-4, atol=1e-4)
    else:
        s = torch.softmax(x.double().cpu() @ Wd["p.router"].T, -1).sort(-1, descending=True).values
        clear = (s[:, top - 1] - s[:, top] > 0.15 * s[:, top - 1]) if top < E else torch.ones(T, dtype=torch.bool)
        assert int(clear.sum()) >= T // 5
        assert float((got[clear] - want[clear]).abs().max()) <= 2e-2 * float(want.abs().max())


def test_router_weights_sum_to_one_and_the_largest_scores_win(ops):
    g = torch.Generator(device=DEV).manual_seed(2)
    T, E, K, top = 6, 7, 40, 3
    x, wr = torch.randn(T, K, generator=g, device=DEV), torch.randn(E, K, generator=g, device=DEV)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wt = torch.empty(T, top, device=DEV)
    ops.router_topk(idx, wt, x, wr, True, True)
    want_idx, want_w = plain.route(x.double().cpu(), wr.double().cpu(), top)
    assert torch.equal(idx.long().cpu(), want_idx) and torch.allclose(wt.cpu().double(), want_w, rtol=1e-5, atol=1e-6)
    assert torch.allclose(wt.sum(-1), torch.ones(T, device=DEV), atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,ff,T", [(72, 40, 5), (256, 384, 3), (256, 384, 300), (48, 56, 17)])
def test_dense_feed_forward_with_a_gelu_gate(ops, dtype, W, ff, T):
    from turingserve_b200.config.model_config import GatedMLPSpec
    g = torch.Generator(device=DEV).manual_seed(W + ff)
    part = build_part("feed_forward", GatedMLPSpec(intermediate_size=ff, activation="gelu_tanh", names=("gate", "up", "down")), W, dtype)
    tensors = {n: (torch.randn(p.shape, generator=g, device=DEV) * 0.15).to(dtype) for n, p in part.parameters().items()}
    part.load(tensors)
    x = torch.randn(T, W, generator=g, device=DEV).to(dtype)
    got = ops.materialize(part.forward(x)).float().cpu()
    want = plain.dense_ff(x.double().cpu(), {"p." + k: v.double().cpu() for k, v in tensors.items()}, "p.").float()
    # (sums over hundreds of rounded terms: the bound goes by the largest output)
    assert float((got - want).abs().max()) <= (1e-5 if dtype == torch.float32 else 1.5e-2) * float(want.abs().max())
