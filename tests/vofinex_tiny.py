"""Tiny Vofinex configurations of the test-suite and their random weights.  They differ in every size and option:
width, vocabulary (no multiples of anything), eps, the three constants (stream multiplier, embedding and logit
scale), the span that repeats (at the start, in the middle, one pass only, none), heads and kv heads, key and
value widths that differ, rotation over part of a head, over all of it and none, blocks of positions smaller and
larger than a page and no multiple of it, a layer without blocks, dense and routed feed-forwards and none, routers
with and without identity outputs, one expert with tensors among identity outputs, top 1 and top = all, page size."""

from __future__ import annotations

import json
import os

import numpy as np
import torch
from safetensors.torch import save_file

from turingserve_b200.models.vofinex import make_config
from turingserve_b200.weights.random_init import random_tensors


def attn(heads, kv, dim, vdim, scale, size=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


# name -> (config arguments, seed, cache page size)
TINY = {
    # the span in the middle, three passes; blocks of 9 positions in pages of 16 and blocks of 33; a rotation over
    # half a head and over the whole head; two of five router outputs are identity experts
    "A": (dict(width=72, vocab=131, eps=1e-5, residual_mult=0.7, embedding_scale=3.0, logit_scale=0.5,
               loop={"start": 1, "stop": 3, "times": 3}, layers=[
        {**attn(4, 2, 16, 8, 0.4, size=9, rot=(100.0, 8)), "mlp": dense(40)},
        {**attn(3, 3, 24, 40, 0.3, size=33, rot=(10000.0, 24)), "mlp": moe(3, 2, 3, 24)},
        {**attn(4, 1, 16, 16, 0.35, size=20, rot=(50.0, 2)), "mlp": None},
        {**attn(4, 2, 16, 8, 0.4, size=9, rot=(100.0, 8)), "mlp": moe(4, 0, 1, 16)},
    ]), 31, 16),
    # no span at all; pages of 8; a layer without blocks (every earlier key is seen: far keys) and one without
    # rotation; one expert with tensors beside three identity outputs, top = all four; six heads on one kv head
    "B": (dict(width=48, vocab=257, eps=1e-6, residual_mult=1.0, embedding_scale=1.0, logit_scale=2.0, layers=[
        {**attn(6, 1, 8, 12, 0.5, rot=(500.0, 4)), "mlp": moe(1, 3, 4, 20)},
        {**attn(2, 2, 40, 24, 0.2, size=20), "mlp": dense(56)},
        {**attn(6, 1, 8, 12, 0.5, size=5, rot=(500.0, 8)), "mlp": moe(6, 1, 2, 8)},
        {**attn(5, 5, 10, 6, 0.45, size=64, rot=(20.0, 6)), "mlp": None},
    ]), 32, 8),
    # sizes in multiples of 16 and pages of 64: heads of 64 and of 128 with values as wide (the tensor-core attention
    # in bfloat16) and of 128 with values of 48; the span at the start, one pass (its vector is still added);
    # blocks of a page, of two and of 100 positions
    "C": (dict(width=128, vocab=300, eps=1e-6, residual_mult=0.5, embedding_scale=11.3, logit_scale=1.5,
               loop={"start": 0, "stop": 2, "times": 1}, layers=[
        {**attn(4, 2, 64, 64, 0.19, size=64, rot=(500000.0, 32)), "mlp": dense(256)},
        {**attn(4, 1, 128, 48, 0.13, size=100, rot=(500000.0, 64)), "mlp": moe(7, 4, 5, 64)},
        {**attn(2, 1, 128, 128, 0.13, size=128, rot=(10000.0, 128)), "mlp": moe(8, 2, 2, 32)},
    ]), 33, 64),
    # the span is the whole model, twice; a single layer
    "D": (dict(width=32, vocab=50, eps=1e-5, residual_mult=0.25, embedding_scale=5.0, logit_scale=1.0,
               loop={"start": 0, "stop": 1, "times": 2}, layers=[
        {**attn(2, 1, 12, 20, 0.4, size=7, rot=(30.0, 12)), "mlp": moe(2, 2, 2, 12)},
    ]), 34, 16),
}

# how much larger than the base deviation a tensor's entries are (by the end of its name): routers for scores that
# tell experts apart (q and k are normed head by head, so their scale is the configuration's)
BOOST = {".router": 8.0, "embed": 10.0, ".v": 3.0}


def tiny_config(name: str):
    return make_config(**TINY[name][0])


def page_size(name: str) -> int:
    return TINY[name][2]


def make_tiny_folder(name: str, base, std: float = 0.05) -> str:
    kw, seed, _ = TINY[name]
    folder = os.path.join(str(base), f"vofinex_{name}")
    if os.path.exists(os.path.join(folder, "model.safetensors")):
        return folder
    cfg = make_config(**kw)
    from turingserve_b200.config.registry import get_architecture
    tensors = random_tensors(cfg, seed, std)
    g = torch.Generator().manual_seed(seed + 1000)
    for n, t in tensors.items():
        if n.endswith(".b"):                         # norm biases
            tensors[n] = (0.2 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif "norm" in n:                            # scales around one, not all equal
            tensors[n] = (1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n.endswith(".sink"):                    # sinks that take between a tenth and most of a row's weight
            tensors[n] = (1.5 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n.endswith(".correction"):              # as large as the scores themselves: the choice changes
            tensors[n] = (0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n == "loop.step":
            tensors[n] = (0.5 * torch.randn(t.shape, generator=g)).to(t.dtype)
        for end, f in BOOST.items():
            if n.endswith(end):
                tensors[n] = (t.float() * f).to(t.dtype)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(get_architecture(cfg.architecture).to_config_json(cfg), f, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder


def random_ids(n: int, vocab: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
