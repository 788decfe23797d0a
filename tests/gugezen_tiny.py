"""Tiny Gugezen configurations of the test-suite and their random weights.  They differ in every size and option:
width, vocabulary (no multiples of anything), eps, the embedding and logit constants, the number of stream copies
(three, two, one with learned links, and no ``streams`` key at all: the ordinary residual sum), the order of the two
mixers, layers that borrow another layer's tensors, heads and kv heads, key and value widths that differ, rotation over
part of a head, over all of it and none, frequency bands that leave, blend and slow frequencies, and none; decays of
exactly 1 and well below; state-space heads in one, two and three groups, states of 7 to 64 rows, filters of 1 to 4
taps, output norms in one to three parts; dense, routed and no feed-forward; routers with top 1, top = all, with and
without the shared expert; page size."""

from __future__ import annotations

import json
import os

import numpy as np
import torch
from safetensors.torch import save_file

from turingserve_b200.models.gugezen import make_config
from turingserve_b200.weights.random_init import random_tensors


def pair(heads, kv, dim, vdim, scale, rot, rheads, rdim, rvdim, decay, ls, rs):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        left["rot"] = {"base": rot[0], "dims": rot[1]}
        if len(rot) > 2:
            left["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), rot[2]))
    right = {"heads": rheads, "dim": rdim, "vdim": rvdim, "decay": list(decay)}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}}


def ssm(heads, vdim, state, groups, conv, parts):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": parts}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


# name -> (config arguments, seed, cache page size)
TINY = {
    # three copies of the stream; both mixers run twice with borrowed tensors; bands that keep the first frequencies,
    # blend the middle ones and slow the last; a head that never decays; a state of 10 rows in 2 groups, 4 taps
    "A": (dict(width=72, vocab=131, eps=1e-5, streams=3, embedding_scale=3.0, logit_scale=0.5, layers=[
        {**ssm(4, 6, 10, 2, 4, 3), "mlp": dense(40)},
        {**pair(4, 2, 16, 8, 0.4, (100.0, 8, (8.0, 1.0, 4.0, 40.0)), 3, 12, 20, (0.5, 0.9, 1.0), 0.7, 1.3), "mlp": moe(5, 2, 24, 16)},
        {**ssm(4, 6, 10, 2, 4, 3), "mlp": dense(40), "weights_of": 0},
        {**pair(4, 2, 16, 8, 0.4, (100.0, 8, (8.0, 1.0, 4.0, 40.0)), 3, 12, 20, (0.5, 0.9, 1.0), 0.7, 1.3), "mlp": moe(5, 2, 24, 16),
         "weights_of": 1},
        {**ssm(2, 16, 7, 1, 2, 1), "mlp": None},
    ]), 41, 16),
    # no ``streams`` key: the ordinary residual; six heads on one kv head; a rotation without bands and a layer without
    # rotation; a filter of one tap (nothing of it in the state); top = all experts, no shared expert; pages of 8
    "B": (dict(width=48, vocab=257, eps=1e-6, embedding_scale=1.0, logit_scale=2.0, layers=[
        {**pair(6, 1, 8, 12, 0.5, (500.0, 4), 2, 8, 8, (0.8, 0.95), 1.0, 0.5), "mlp": moe(4, 4, 20)},
        {**ssm(3, 8, 16, 3, 1, 1), "mlp": dense(56)},
        {**pair(5, 5, 10, 6, 0.45, None, 1, 20, 12, (0.97,), 1.5, 1.0), "mlp": None},
        {**ssm(6, 4, 9, 2, 3, 2), "mlp": moe(3, 1, 8, 24)},
    ]), 42, 8),
    # sizes in multiples of 16 and pages of 64: heads of 64 and of 128 with values as wide (the tensor-core attention in
    # bfloat16), two copies of the stream
    "C": (dict(width=128, vocab=300, eps=1e-6, streams=2, embedding_scale=11.3, logit_scale=0.4, layers=[
        {**pair(4, 2, 64, 64, 0.13, (300000.0, 32, (3.0, 1.0, 3.0, 200.0)), 2, 64, 64, (0.9, 0.9995), 0.75, 1.2), "mlp": dense(256)},
        {**ssm(4, 32, 64, 1, 4, 2), "mlp": moe(8, 2, 32, 64)},
        {**pair(2, 1, 128, 128, 0.09, (10000.0, 128), 4, 32, 16, (0.6, 0.8, 0.9, 0.99), 1.0, 1.0), "mlp": moe(6, 3, 64)},
        {**ssm(4, 32, 64, 1, 4, 2), "mlp": moe(8, 2, 32, 64), "weights_of": 1},
    ]), 43, 64),
    # one copy of the stream with learned links; one layer, run twice
    "D": (dict(width=32, vocab=50, eps=1e-5, streams=1, embedding_scale=5.0, logit_scale=1.0, layers=[
        {**pair(2, 1, 12, 20, 0.4, (30.0, 12, (2.0, 1.0, 2.0, 16.0)), 2, 6, 10, (0.7, 0.99), 0.9, 1.1), "mlp": dense(24)},
        {**pair(2, 1, 12, 20, 0.4, (30.0, 12, (2.0, 1.0, 2.0, 16.0)), 2, 6, 10, (0.7, 0.99), 0.9, 1.1), "mlp": dense(24),
         "weights_of": 0},
    ]), 44, 16),
}

# how much larger than the base deviation a tensor's entries are (by the end of its name)
BOOST = {".router": 8.0, "embed": 4.0, ".in": 3.0, ".left.q": 2.0, ".left.k": 2.0}


def tiny_config(name: str):
    return make_config(**TINY[name][0])


def page_size(name: str) -> int:
    return TINY[name][2]


def tiny_tensors(cfg, seed: int, std: float = 0.05) -> dict[str, torch.Tensor]:
    tensors = random_tensors(cfg, seed, std)
    g = torch.Generator().manual_seed(seed + 1000)
    rnd = lambda t, s: s * torch.randn(t.shape, generator=g)
    for n, t in tensors.items():
        last = n.rsplit(".", 1)[-1]
        if n.endswith((".norm1", ".norm2")) or n == "final.norm":     # stored around zero: the scale is 1 + w
            new = rnd(t, 0.3)
        elif n.endswith(".norm"):                    # the mixers' own norms: plain scales around one
            new = 1.0 + rnd(t, 0.3)
        elif n.endswith(".sink"):                    # sinks that take between a tenth and most of a row's weight
            new = rnd(t, 1.5)
        elif n.endswith(".b"):                       # projection and filter biases
            new = rnd(t, 0.2)
        elif ".hc" in n:
            S = t.shape[0]
            new = {"in": 1.0 / S + rnd(t, 0.3), "out": 1.0 + rnd(t, 0.3)}.get(last)
            if new is None:
                new = torch.eye(S) + rnd(t, 0.2)
        elif n.endswith(".conv"):
            new = rnd(t, 0.5)
        elif n.endswith(".dt_bias"):
            new = rnd(t, 0.7)
        elif n.endswith(".A_log"):                   # decays exp(-exp(A) dt) from slow to fast
            new = 2.0 * torch.rand(t.shape, generator=g) - 1.5
        elif n.endswith(".D"):
            new = 1.0 + rnd(t, 0.3)
        else:
            new = t.float()
            for end, f in BOOST.items():
                if n.endswith(end):
                    new = new * f
        tensors[n] = new.to(t.dtype)
    return tensors


def make_tiny_folder(name: str, base, std: float = 0.05) -> str:
    kw, seed, _ = TINY[name]
    folder = os.path.join(str(base), f"gugezen_{name}")
    if os.path.exists(os.path.join(folder, "model.safetensors")):
        return folder
    cfg = make_config(**kw)
    from turingserve_b200.config.registry import get_architecture
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(get_architecture(cfg.architecture).to_config_json(cfg), f, indent=1)
    save_file(tiny_tensors(cfg, seed, std), os.path.join(folder, "model.safetensors"))
    return folder


def random_ids(n: int, vocab: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
