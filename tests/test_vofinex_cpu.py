"""Vofinex without a GPU: the parser and its refusals, the order of runs of a repeated span, checkpoint names, the
cache need of attention in blocks (pages before the present block go back to the pool), the engine's host logic
(portions down to two tokens, mixed batches, pages and slots used again) through the kernel twins against the
plain model, and the plain model's mechanisms against closed forms."""

from __future__ import annotations

import json
import math

import pytest
import torch

from tests import plain_vofinex as plain
from tests import schedules
from tests import vofinex_tiny as vt
from turingserve_b200.cache.manager import CacheManager
from turingserve_b200.config.model_config import GatedMLPSpec, HalfRotarySpec, RoutedMLPSpec, SinkAttentionSpec
from turingserve_b200.config.registry import get_architecture, load_model_config
from turingserve_b200.parts.base import CacheNeed


def test_parser_reads_every_size_and_option():
    cfg = vt.tiny_config("A")
    assert cfg.architecture == "Vofinex" and cfg.hidden_size == 72 and cfg.vocab_size == 131
    assert cfg.extra("embedding_scale") == 3.0 and cfg.extra("logit_scale") == 0.5
    assert [(r.layer, r.opens_pass) for r in cfg.schedule] == [
        (0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    a0, a1, a2, _ = (cfg.layers[i].mixer for i in range(4))
    assert isinstance(a0, SinkAttentionSpec) and (a0.num_heads, a0.num_kv_heads, a0.key_dim, a0.value_dim) == (4, 2, 16, 8)
    assert a0.chunk == 9 and a0.scale == 0.4 and a0.sinks and a0.qk_norm_eps == 1e-5 and a0.window is None
    assert a0.position == HalfRotarySpec(base=100.0, dims=8) and a1.position.dims == 24 and a2.position.dims == 2
    assert cfg.layers[0].roles["join"].scale == 0.7 and cfg.layers[0].norm.eps == 1e-5 and cfg.final_norm.bias_name == ".b"
    f0, f1 = cfg.layers[0].feed_forward, cfg.layers[1].feed_forward
    assert isinstance(f0, GatedMLPSpec) and f0.intermediate_size == 40 and f0.activation == "silu"
    assert isinstance(f1, RoutedMLPSpec) and (f1.num_experts, f1.identity, f1.top_k, f1.intermediate_size) == (3, 2, 3, 24)
    assert f1.correction and not f1.renormalize and f1.scoring == "softmax"
    assert "feed_forward" not in cfg.layers[2].roles
    b = vt.tiny_config("B")
    assert b.layers[0].mixer.chunk is None and b.layers[1].mixer.position is None and b.extra("loop") is None
    assert [(r.layer, r.opens_pass) for r in b.schedule] == [(i, None) for i in range(4)]
    c, d = vt.tiny_config("C"), vt.tiny_config("D")
    assert [(r.layer, r.opens_pass) for r in c.schedule] == [(0, 0), (1, None), (2, None)]     # one pass: still opened
    assert [(r.layer, r.opens_pass) for r in d.schedule] == [(0, 0), (0, 1)]


def test_names_round_trip_and_registry(tmp_path):
    arch = get_architecture("Vofinex")
    cfg = vt.tiny_config("A")
    names = arch.tensor_names(cfg)
    assert names.embedding == "embed" and names.lm_head == "embed" and names.final_norm == "final.norm"
    assert [n.mixer for n in names.layers] == [f"l{i}.mix." for i in range(4)]
    assert names.layers[0]["feed_forward"] == "l0.mlp." and "feed_forward" not in names.layers[2].roles()
    for name in vt.TINY:
        c = vt.tiny_config(name)
        again = arch.parse_config(json.loads(json.dumps(arch.to_config_json(c))))
        assert again.layers == c.layers and again.schedule == c.schedule and again.extras == c.extras
    folder = vt.make_tiny_folder("D", tmp_path)
    assert load_model_config(folder).architecture == "Vofinex"
    _, w = plain.read_folder(folder)
    assert w["loop.step"].shape == (2, 32) and w["l0.mlp.router"].shape == (4, 32) and w["l0.mlp.correction"].shape == (4,)
    assert "l0.mlp.e1.down" in w and "l0.mlp.e2.down" not in w and w["l0.mix.sink"].shape == (2,)


def test_parser_refusals():
    arch = get_architecture("Vofinex")
    good = arch.to_config_json(vt.tiny_config("A"))
    for edit, match in ((lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
                        (lambda c: c["layers"][0]["mlp"].update(kind="wide"), "unknown feed-forward kind"),
                        (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
                        (lambda c: c["layers"][1]["mixer"].pop("heads"), "heads"),
                        (lambda c: c["layers"][1]["mlp"]["router"].pop("top"), "top"),
                        (lambda c: c["loop"].update(stop=9), "does not fit"),
                        (lambda c: c.pop("width"), "width"),
                        (lambda c: c.pop("norm"), "norm")):
        bad = json.loads(json.dumps(good))
        edit(bad)
        with pytest.raises(ValueError, match=match):
            arch.parse_config(bad)


def test_every_pass_has_memory_of_its_own_and_blocks_give_pages_back(tmp_path):
    from turingserve_b200.engine.runner import run_needs
    from turingserve_b200.weights.loader import load_model
    model, cfg = load_model(vt.make_tiny_folder("A", tmp_path), torch.float32, "cpu")
    needs = run_needs(model)
    assert len(needs) == 8 and all(n.state is None for n in needs)
    assert needs[0].cache == CacheNeed(2, 16, None, value_dim=8, chunk=9)
    assert needs[1].cache == needs[3].cache == needs[5].cache == CacheNeed(3, 24, None, value_dim=40, chunk=33)
    cm = CacheManager(needs, 16, 12, 3, torch.float32, "cpu")
    views = [cm.view(i) for i in range(8)]
    assert len({v.k.data_ptr() for v in views}) == 8                       # a layer run three times: three memories
    assert views[1].k.shape[1:] == (3, 16, 24) and views[1].v.shape[1:] == (3, 16, 40)
    rc = cm.admit("a")
    cm.grow(rc, 40)
    cm.advance(rc, 40)
    # the next position, 40, lies in the block of 9 that starts at 36: pages 0 and 1 (positions 0..31) are free again;
    # in blocks of 33 it lies in the block that starts at 33: pages 0 and 1 as well; blocks of 20: the block starts at 40
    t9, t33, t20 = (rc.tables[views[i].group] for i in (0, 1, 2))
    assert t9[0] == 0 and t9[1] == 0 and t9[2] != 0
    assert t33[0] == 0 and t33[1] == 0 and t33[2] != 0
    assert t20[0] == 0 and t20[1] == 0 and t20[2] != 0
    cm.release(rc)
    cm.check()
    # without blocks nothing goes back before the request ends
    model, _ = load_model(vt.make_tiny_folder("B", tmp_path), torch.float32, "cpu")
    cm = CacheManager(run_needs(model), 8, 12, 3, torch.float32, "cpu")
    rc = cm.admit("a")
    cm.grow(rc, 40)
    cm.advance(rc, 40)
    assert all(p != 0 for p in rc.tables[cm.view(0).group][:5])
    cm.release(rc)
    cm.check()


def _replay_cpu(folder, name, steps, page=None):
    from turingserve_b200 import kernels
    from turingserve_b200.engine.replay import Replayer
    from tests.twin_ops import TwinOps
    kernels.use(TwinOps())
    try:
        rp = Replayer(folder, torch.float32, schedules.peak_tokens(steps), "cpu", page_size=page or vt.page_size(name))
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
    """More requests than live slots, a pool that makes pages go round, portions down to two tokens that end in
    the middle of pages and of blocks."""
    folder = vt.make_tiny_folder(name, tmp_path)
    cfg, w = plain.read_folder(folder)
    reqs = {f"r{i}": vt.random_ids(n, cfg["vocab"], 50 + i) for i, n in enumerate([1, 9, 34, 21, 17, 40])}
    steps = getattr(schedules, schedule)(reqs, tail=5) if schedule != "portions" else schedules.portions(reqs)
    got = _replay_cpu(folder, name, steps)
    expected = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    bad = schedules.first_bad(got, expected, 2e-4)
    assert bad is None, f"first wrong place (request, position, error): {bad}"


def test_the_plain_functions_agree_with_closed_forms():
    f64 = torch.float64
    g = torch.Generator().manual_seed(0)
    # layer norm: zero mean and unit variance before weight and bias; a constant row gives the bias
    x = torch.randn(3, 11, generator=g, dtype=f64)
    y = plain.layer_norm(x, torch.ones(11, dtype=f64), torch.zeros(11, dtype=f64), 0.0)
    assert torch.allclose(y.mean(-1), torch.zeros(3, dtype=f64), atol=1e-12)
    assert torch.allclose((y * y).mean(-1), torch.ones(3, dtype=f64))
    b = torch.arange(11, dtype=f64)
    assert torch.allclose(plain.layer_norm(torch.full((1, 11), 4.0, dtype=f64), 2 * torch.ones(11, dtype=f64), b, 1e-6)[0], b)
    # unit norm: eps inside the root
    assert torch.allclose(plain.unit_rms(torch.tensor([[3.0, 4.0]], dtype=f64), 3.5), torch.tensor([[0.75, 1.0]], dtype=f64))
    # rotation: dimension i with i + dims / 2, angle position * base^(-2 i / dims); the rest passes
    v = torch.tensor([[[1.0, 2.0, 0.0, 0.0, 7.0, 9.0]]], dtype=f64)
    r = plain.rotate_half(v, torch.tensor([3]), 4, 100.0)[0, 0]
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert torch.allclose(r, torch.tensor([math.cos(a0), 2 * math.cos(a1), math.sin(a0), 2 * math.sin(a1), 7.0, 9.0], dtype=f64))
    assert torch.equal(plain.rotate_half(v, torch.tensor([3]), 0, 100.0), v)
    q = torch.randn(1, 1, 8, generator=g, dtype=f64)
    k = torch.randn(1, 1, 8, generator=g, dtype=f64)
    dots = [float((plain.rotate_half(q, torch.tensor([p + 5]), 8, 50.0) * plain.rotate_half(k, torch.tensor([p]), 8, 50.0)).sum())
            for p in (0, 11, 400)]
    assert max(dots) - min(dots) < 1e-9                                      # a score depends on the distance only
    # blocks: counted from position 0; the first position of a block sees itself only
    ok = plain.visible(12, 5)
    assert ok[4, 0] and not ok[5, 4] and ok[5, 5] and ok[9, 5] and not ok[10, 9] and not ok[3, 4]
    assert plain.visible(12, None)[11, 0]
    # the sink: a row alone with a sink of the same score keeps half its weight; a very negative sink is a softmax
    s = torch.zeros(2, 1, 1, dtype=f64)
    p = plain.sink_softmax(s, torch.tensor([0.0, -50.0], dtype=f64))
    assert abs(float(p[0, 0, 0]) - 0.5) < 1e-12 and abs(float(p[1, 0, 0]) - 1.0) < 1e-12
    s = torch.randn(2, 3, 3, generator=g, dtype=f64)
    p = plain.sink_softmax(s, torch.tensor([0.3, -0.7], dtype=f64))
    den = torch.exp(s).sum(-1) + torch.exp(torch.tensor([0.3, -0.7], dtype=f64))[:, None]
    assert torch.allclose(p, torch.exp(s) / den[..., None])
    # the router: the correction changes the choice, never the weight; weights are not renormalised
    h = torch.tensor([[1.0, 0.0]], dtype=f64)
    router = torch.tensor([[2.0, 0.0], [1.0, 0.0], [0.0, 0.0]], dtype=f64)
    idx, wt = plain.route(h, router, None, 2)
    sm = torch.softmax(torch.tensor([2.0, 1.0, 0.0], dtype=f64), 0)
    assert idx.tolist() == [[0, 1]] and torch.allclose(wt[0], sm[:2]) and float(wt.sum()) < 1.0
    idx, wt = plain.route(h, router, torch.tensor([0.0, -1.0, 1.0], dtype=f64), 2)
    assert sorted(idx[0].tolist()) == [0, 2] and torch.allclose(wt[0].sort().values, sm[[2, 0]])
    # identity outputs return the input times the weight: with every output an identity one, ff(h) = sum(w) h
    f = {"router": {"experts": 0, "identity": 3, "top": 3}}
    out = plain.routed_ff(h, {"router": router}, f)
    assert torch.allclose(out, h)
    f = {"router": {"experts": 0, "identity": 3, "top": 1}}
    assert torch.allclose(plain.routed_ff(h, {"router": router}, f), sm[0] * h)
    # the order of runs
    assert plain.order(4, {"start": 1, "stop": 3, "times": 2}) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert plain.order(2, None) == [(0, None), (1, None)]
