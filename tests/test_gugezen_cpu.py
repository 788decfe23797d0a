"""Gugezen without a GPU: the parser and its refusals, layers that borrow tensors, checkpoint names, the memory the two
mixers declare (pages for the attention half, one flat state slot for the linear-attention half and for the state-space
mixer), the engine's host logic (portions down to two tokens, mixed batches, pages and slots used again) through the
kernel twins against the plain model, and the plain model's mechanisms against closed forms."""

from __future__ import annotations

import json
import math

import pytest
import torch

from tests import gugezen_tiny as gt
from tests import plain_gugezen as plain
from tests import schedules
from turingserve_b200.cache.manager import CacheManager
from turingserve_b200.config.model_config import (
    BandScaledRotarySpec, GatedMLPSpec, LightningSpec, Mamba2Spec, PairedMixerSpec, RoutedMLPSpec, SinkAttentionSpec)
from turingserve_b200.config.registry import get_architecture, load_model_config
from turingserve_b200.parts.base import CacheNeed, StateNeed


def test_parser_reads_every_size_and_option():
    cfg = gt.tiny_config("A")
    assert cfg.architecture == "Gugezen" and cfg.hidden_size == 72 and cfg.vocab_size == 131 and cfg.tie_word_embeddings
    assert cfg.extra("embedding_scale") == 3.0 and cfg.extra("logit_scale") == 0.5 and cfg.extra("streams") == 3
    assert [r.layer for r in cfg.schedule] == [0, 1, 0, 1, 2] and cfg.extra("layer_ids") == (0, 1, 4)
    m0, m1, m2 = (cfg.layers[i].mixer for i in range(3))
    assert m0 == Mamba2Spec(num_heads=4, head_dim=6, state_size=10, num_groups=2, conv_taps=4, norm_groups=3, norm_eps=1e-5)
    assert isinstance(m1, PairedMixerSpec) and (m1.left_scale, m1.right_scale) == (0.7, 1.3)
    a, b = m1.left, m1.right
    assert isinstance(a, SinkAttentionSpec) and (a.num_heads, a.num_kv_heads, a.key_dim, a.value_dim) == (4, 2, 16, 8)
    assert a.scale == 0.4 and a.sinks and a.qkv_bias and a.out_gate and a.qk_norm_eps is None and a.chunk is None
    assert a.position == BandScaledRotarySpec(base=100.0, dims=8, factor=8.0, low=1.0, high=4.0, original=40.0)
    assert b == LightningSpec(num_heads=3, key_dim=12, value_dim=20, decays=(0.5, 0.9, 1.0), norm_eps=1e-5)
    assert (m2.num_heads, m2.num_groups, m2.conv_taps, m2.norm_groups) == (2, 1, 2, 1)
    n = cfg.layers[0].mixer_norm
    assert (n.eps, n.streams, n.weight_offset) == (1e-5, 3, 1.0) and cfg.final_norm == n
    assert cfg.layers[0].mixer_link.streams == 3 and cfg.layers[0].mixer_link.learned
    f0, f1 = cfg.layers[0].feed_forward, cfg.layers[1].feed_forward
    assert isinstance(f0, GatedMLPSpec) and f0.intermediate_size == 40 and f0.activation == "gelu_tanh"
    assert isinstance(f1, RoutedMLPSpec) and (f1.num_experts, f1.top_k, f1.intermediate_size) == (5, 2, 24)
    assert f1.scoring == "softmax" and f1.renormalize and f1.weight_on == "output" and f1.activation == "gelu"
    assert f1.shared_intermediate_size == 16 and not f1.gated
    assert "feed_forward" not in cfg.layers[2].roles and "ffn_link" not in cfg.layers[2].roles
    b_cfg = gt.tiny_config("B")
    assert b_cfg.extra("streams") is None and not b_cfg.layers[0].mixer_link.learned and b_cfg.layers[0].mixer_norm.streams == 1
    assert b_cfg.layers[0].mixer.left.position == BandScaledRotarySpec(base=500.0, dims=4)
    assert b_cfg.layers[2].mixer.left.position is None and b_cfg.layers[0].feed_forward.shared_intermediate_size is None
    d = gt.tiny_config("D")
    assert [r.layer for r in d.schedule] == [0, 0] and d.layers[0].mixer_link.learned and d.extra("streams") == 1


def test_names_round_trip_and_registry(tmp_path):
    arch = get_architecture("Gugezen")
    cfg = gt.tiny_config("A")
    names = arch.tensor_names(cfg)
    assert names.embedding == "embed" and names.lm_head == "embed" and names.final_norm == "final.norm"
    assert [n.mixer for n in names.layers] == ["l0.mix.", "l1.mix.", "l4.mix."]          # borrowing layers have no names
    assert names.layers[1]["ffn_link"] == "l1.hc2." and names.layers[0]["mixer_norm"] == "l0.norm1"
    assert "feed_forward" not in names.layers[2].roles()
    for name in gt.TINY:
        c = gt.tiny_config(name)
        again = arch.parse_config(json.loads(json.dumps(arch.to_config_json(c))))
        assert again.layers == c.layers and again.schedule == c.schedule and again.extras == c.extras
    folder = gt.make_tiny_folder("A", tmp_path)
    assert load_model_config(folder).architecture == "Gugezen"
    _, w = plain.read_folder(folder)
    assert w["l0.mix.in"].shape == (2 * 24 + 2 * 2 * 10 + 4, 72) and w["l0.mix.conv"].shape == (24 + 40, 4)
    assert w["l1.hc2.mix"].shape == (3, 3) and w["l1.mix.left.sink"].shape == (4,) and w["l1.mix.left.k.b"].shape == (32,)
    assert w["l1.mix.left.g"].shape == (32, 72) and w["l1.mix.right.norm"].shape == (60,) and w["l1.mlp.shared.up"].shape == (16, 72)
    assert not any(n.startswith(("l2.", "l3.")) for n in w) and "l4.norm2" not in w and "l4.norm1" in w
    _, wb = plain.read_folder(gt.make_tiny_folder("B", tmp_path))
    assert not any(".hc" in n for n in wb) and "l0.mlp.shared.up" not in wb                # no copies: no link tensors


def test_parser_refusals():
    arch = get_architecture("Gugezen")
    good = arch.to_config_json(gt.tiny_config("A"))
    for edit, match in ((lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
                        (lambda c: c["layers"][0]["mlp"].update(kind="wide"), "unknown feed-forward kind"),
                        (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
                        (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "decays"),
                        (lambda c: c["layers"][0]["mixer"].pop("state"), "state"),
                        (lambda c: c["layers"][1]["mlp"]["router"].pop("top"), "top"),
                        (lambda c: c["layers"][2].update(weights_of=1), "another type"),
                        (lambda c: c["layers"][2].update(weights_of=3), "earlier layer"),
                        (lambda c: c.update(streams=0), "streams"),
                        (lambda c: c.pop("width"), "width"),
                        (lambda c: c.pop("norm"), "norm")):
        bad = json.loads(json.dumps(good))
        edit(bad)
        with pytest.raises(ValueError, match=match):
            arch.parse_config(bad)


def test_memory_of_every_run(tmp_path):
    """The paired mixer declares its attention half's pages AND its linear half's state; a borrowing layer has memory of
    its own; the state-space mixer's slot holds the state and the filter's last inputs."""
    from turingserve_b200.engine.runner import run_needs
    from turingserve_b200.weights.loader import load_model
    model, cfg = load_model(gt.make_tiny_folder("A", tmp_path), torch.float32, "cpu")
    needs = run_needs(model)
    assert len(needs) == 5
    assert needs[0].cache is None and needs[0].state == StateNeed((4 * 10 * 6 + 3 * (24 + 40),), torch.float32)
    assert needs[1].cache == CacheNeed(2, 16, None, value_dim=8, chunk=None) and needs[1].state == StateNeed((3, 12, 20), torch.float32)
    assert needs[3] == needs[1] and needs[2] == needs[0]
    assert needs[4].state == StateNeed((2 * 7 * 16 + 1 * (32 + 14),), torch.float32)
    cm = CacheManager(needs, 16, 12, 3, torch.float32, "cpu")
    assert len(cm.groups) == 1 and cm.view(1).k.data_ptr() != cm.view(3).k.data_ptr()
    assert cm.states[1].data_ptr() != cm.states[3].data_ptr() and cm.states[0].shape == (4, 432)
    # a filter of one tap keeps nothing
    model, _ = load_model(gt.make_tiny_folder("B", tmp_path), torch.float32, "cpu")
    assert run_needs(model)[1].state == StateNeed((3 * 16 * 8,), torch.float32)


def test_the_frequencies_of_the_product_are_the_plain_ones():
    from turingserve_b200.parts.base import BuildContext, build
    ctx = BuildContext(hidden_size=8, dtype=torch.float32, device=torch.device("cpu"), max_positions=16)
    for base, dims, sc in ((100.0, 8, (8.0, 1.0, 4.0, 40.0)), (300000.0, 48, (3.0, 1.0, 3.0, 900.0)), (10000.0, 6, None),
                           (50.0, 16, (3.0, 2.0, 8.0, 100.0))):
        spec = BandScaledRotarySpec(base=base, dims=dims, **(dict(zip(("factor", "low", "high", "original"), sc)) if sc else {}))
        want = plain.scaled_frequencies(base, dims, dict(zip(("factor", "low", "high", "original"), sc)) if sc else None)
        got = build("position", spec, ctx).freq
        assert torch.allclose(got.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-7, atol=0)


def _replay_cpu(folder, name, steps, page=None):
    from turingserve_b200 import kernels
    from turingserve_b200.engine.replay import Replayer
    from tests.twin_ops import TwinOps
    kernels.use(TwinOps())
    try:
        rp = Replayer(folder, torch.float32, schedules.peak_tokens(steps), "cpu", page_size=page or gt.page_size(name))
        outs = {}
        with torch.inference_mode():
            for s in steps:
                o = rp.step(s)
                if o is not None:
                    outs[s["step"]] = o
                rp.cache.check()
        assert not rp.cache.live
    finally:
        kernels.use(None)
    return schedules.collect(steps, outs)


@pytest.mark.parametrize("name", ["A", "B", "D"])
@pytest.mark.parametrize("schedule", ["decode_tail", "portions", "mixed"])
def test_host_logic_against_plain(tmp_path, name, schedule):
    """More requests than live slots, a pool that makes pages go round, state slots handed on from request to request,
    portions down to two tokens (shorter than the filter's memory) that end in the middle of pages."""
    folder = gt.make_tiny_folder(name, tmp_path)
    cfg, w = plain.read_folder(folder)
    reqs = {f"r{i}": gt.random_ids(n, cfg["vocab"], 50 + i) for i, n in enumerate([1, 9, 34, 21, 17, 40])}
    steps = getattr(schedules, schedule)(reqs, tail=5) if schedule != "portions" else schedules.portions(reqs)
    got = _replay_cpu(folder, name, steps)
    expected = {rid: plain.forward(cfg, w, toks)[0].numpy() for rid, toks in reqs.items()}
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    bad = schedules.first_bad(got, expected, 2e-4)
    assert bad is None, f"first wrong place (request, position, error): {bad}"


def test_the_plain_functions_agree_with_closed_forms():
    f64 = torch.float64
    g = torch.Generator().manual_seed(0)
    # the norm: eps inside the root, a stored weight of zero is a scale of one
    x = torch.tensor([[3.0, 4.0]], dtype=f64)
    assert torch.allclose(plain.zero_centred_norm(x, torch.tensor([0.0, 1.0], dtype=f64), 3.5), torch.tensor([[0.75, 2.0]], dtype=f64))
    # activations at known points
    z = torch.tensor([0.0, 1.0, -2.0], dtype=f64)
    assert torch.allclose(plain.gelu_erf(z), z * 0.5 * (1 + torch.erf(z / math.sqrt(2))))
    assert abs(float(plain.gelu_erf(torch.tensor(1.0, dtype=f64))) - 0.8413447460685429) < 1e-12
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=f64))) - 0.8411919906082768) < 1e-12
    assert abs(float(plain.softplus(torch.tensor(0.0, dtype=f64))) - math.log(2)) < 1e-15
    assert float(plain.softplus(torch.tensor(50.0, dtype=f64))) == 50.0
    # frequency bands: short wavelengths stay, long ones are divided, the middle is blended; the edges belong to the blend
    base, dims, sc = 100.0, 8, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 40.0}
    f = plain.scaled_frequencies(base, dims, sc)
    raw = [base ** (-2 * i / dims) for i in range(4)]
    assert f[0] == raw[0] and 2 * math.pi / raw[0] < 10                          # wavelength 6.3 < 40 / 4
    assert 10 < 2 * math.pi / raw[1] < 40 and raw[1] / 8 < f[1] < raw[1]
    s1 = (40 / (2 * math.pi / raw[1]) - 1.0) / 3.0
    assert abs(f[1] - ((1 - s1) * raw[1] / 8 + s1 * raw[1])) < 1e-15
    assert f[2] == raw[2] / 8 and f[3] == raw[3] / 8                             # wavelengths 63 and 199 > 40 / 1
    assert plain.scaled_frequencies(base, dims, None) == raw
    # rotation of neighbours: (2i, 2i + 1) turn by position * f_i; the rest passes; a score depends on the distance only
    v = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 7.0, 9.0]]], dtype=f64)
    r = plain.rotate_neighbours(v, torch.tensor([3]), [1.0, 0.1])[0, 0]
    assert torch.allclose(r, torch.tensor([math.cos(3.0), math.sin(3.0), -2 * math.sin(0.3), 2 * math.cos(0.3), 7.0, 9.0], dtype=f64))
    q = torch.randn(1, 1, 8, generator=g, dtype=f64)
    k = torch.randn(1, 1, 8, generator=g, dtype=f64)
    dots = [float((plain.rotate_neighbours(q, torch.tensor([p + 5]), f) * plain.rotate_neighbours(k, torch.tensor([p]), f)).sum())
            for p in (0, 11, 400)]
    assert max(dots) - min(dots) < 1e-9
    # the sink: n equal keys and a sink s give each key 1 / (n + e^(s - score)), whatever the scale; causal
    n, s = 5, 0.7
    q = torch.zeros(n, 1, 4, dtype=f64)
    vals = torch.eye(n, dtype=f64)[:, None, :]
    out = plain.sink_attention(q, torch.randn(n, 1, 4, generator=g, dtype=f64), vals, 0.3, torch.tensor([s], dtype=f64))
    for i in range(n):
        want = torch.zeros(n, dtype=f64)
        want[:i + 1] = 1.0 / (i + 1 + math.exp(s))
        assert torch.allclose(out[i, 0], want)
    # the decaying state: with constant q = k = v = 1 (one dimension) o_t = 1 + d + ... + d^t
    one = torch.ones(6, 1, 1, dtype=f64)
    o = plain.decayed_state_scan(one, one, one, [0.5])[:, 0, 0]
    assert torch.allclose(o, torch.tensor([2 - 0.5 ** t for t in range(6)], dtype=f64))
    # the causal filter: the last column is the present token's, zeros before the start
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=f64)
    y = plain.causal_filter(x, torch.tensor([[100.0, 10.0, 1.0]], dtype=f64), torch.tensor([0.5], dtype=f64))[:, 0]
    assert y.tolist() == [1.5, 12.5, 124.5]
    # the state-space scan: one head, one state row: S_t = a S + dt B x, y = C S + D x with a = exp(-exp(A) dt)
    T = 5
    x = torch.ones(T, 1, 1, dtype=f64)
    dt = torch.full((T, 1), 0.5, dtype=f64)
    B = torch.full((T, 1, 1), 2.0, dtype=f64)
    C = torch.full((T, 1, 1), 3.0, dtype=f64)
    y = plain.state_space_scan(x, dt, torch.tensor([0.0], dtype=f64), B, C, torch.tensor([0.25], dtype=f64))[:, 0, 0]
    a, S, want = math.exp(-0.5), 0.0, []
    for _ in range(T):
        S = a * S + 0.5 * 2.0
        want.append(3.0 * S + 0.25)
    assert torch.allclose(y, torch.tensor(want, dtype=f64))
    # the router: the largest scores, renormalised to one
    h = torch.tensor([[1.0, 0.0]], dtype=f64)
    router = torch.tensor([[2.0, 0.0], [0.0, 0.0], [1.0, 0.0]], dtype=f64)
    idx, wt = plain.route(h, router, 2)
    sm = torch.softmax(torch.tensor([2.0, 0.0, 1.0], dtype=f64), 0)
    assert idx.tolist() == [[0, 2]] and torch.allclose(wt[0], sm[[0, 2]] / (sm[0] + sm[2])) and abs(float(wt.sum()) - 1) < 1e-12
    # streams: with in = (1, 0), out = (1, 1), mix = identity, two copies behave as one residual stream in copy 0
    cfg = {"norm": {"eps": 1e-6}, "streams": 2, "layers": [{"type": "mamba2", "mlp": None, "mixer":
           {"heads": 1, "vdim": 2, "state": 2, "groups": 1, "conv": 2, "norm_groups": 1}}]}
    W = {"embed": torch.randn(5, 4, generator=g), "final.norm": torch.zeros(4), "l0.norm1": torch.zeros(4),
         "l0.mix.in": torch.randn(2 * 2 + 2 * 2 + 1, 4, generator=g), "l0.mix.conv": torch.randn(6, 2, generator=g),
         "l0.mix.conv.b": torch.zeros(6), "l0.mix.dt_bias": torch.zeros(1), "l0.mix.A_log": torch.zeros(1),
         "l0.mix.D": torch.ones(1), "l0.mix.norm": torch.ones(2), "l0.mix.o": torch.randn(4, 2, generator=g),
         "l0.hc1.in": torch.tensor([1.0, 0.0]), "l0.hc1.out": torch.tensor([1.0, 0.0]), "l0.hc1.mix": torch.eye(2)}
    _, after2 = plain.forward(cfg, W, [1, 3, 2])
    one = {k: v for k, v in W.items() if ".hc" not in k}
    _, after1 = plain.forward({k: v for k, v in cfg.items() if k != "streams"}, one, [1, 3, 2])
    x0 = W["embed"].double()[torch.tensor([1, 3, 2])]
    assert torch.allclose(after2[0], after1[0] + x0)             # copy 1 keeps the embedding; the sum holds both


def test_a_pair_takes_one_cache_and_one_state_and_mixers_that_expose_their_products():
    from turingserve_b200.parts.base import BuildContext, build
    ctx = BuildContext(hidden_size=24, dtype=torch.float32, device=torch.device("cpu"), max_positions=16)
    lin = LightningSpec(num_heads=2, key_dim=4, value_dim=6, decays=(0.5, 0.9), norm_eps=1e-6)
    att = SinkAttentionSpec(num_heads=2, num_kv_heads=1, key_dim=8, value_dim=4, scale=0.3, qkv_bias=True, out_gate=True)
    pair = build("mixer", PairedMixerSpec(left=att, right=lin, left_scale=0.5, right_scale=2.0), ctx)
    assert pair.cache_need() == CacheNeed(1, 8, None, value_dim=4, chunk=None) and pair.state_need() == StateNeed((2, 4, 6), torch.float32)
    names = set(pair.parameters())
    assert {"left.q", "left.q.b", "left.g", "left.sink", "right.norm", "right.o"} <= names and len(names) == 9 + 6
    # either order of the halves
    assert build("mixer", PairedMixerSpec(left=lin, right=att), ctx).cache_need() is not None
    with pytest.raises(ValueError, match="at most one"):
        build("mixer", PairedMixerSpec(left=lin, right=lin), ctx)
    with pytest.raises(ValueError, match="at most one"):
        build("mixer", PairedMixerSpec(left=att, right=att), ctx)
    # a mixer that does not expose its products is refused when the pair is loaded, by name
    ssm = Mamba2Spec(num_heads=2, head_dim=4, state_size=4, num_groups=1, conv_taps=2, norm_groups=1, norm_eps=1e-6)
    odd = build("mixer", PairedMixerSpec(left=att, right=ssm), ctx)
    tensors = {n: torch.zeros(p.shape) for n, p in odd.parameters().items()}
    with pytest.raises(NotImplementedError, match="Mamba2 does not expose"):
        odd.load(tensors)
