"""A plain, slow implementation of the Vofinex design: whole sequences, no cache, no batching, one function per
mechanism, in the precision of the tensors it is given (float32 or float64).  It shares nothing with the
package: the tests compare the engine with it.

The design: a decoder over a residual stream x.  x = scale_e * E[token].  A layer is PARALLEL: with
h = LN(x) (mean and variance over the width, learned weight and bias) x <- x + m * (mixer(h) + ff(h)); the
feed-forward may be missing.  The mixer is grouped-query attention: q, k rotated over their first R dimensions
(dimension i with i + R/2), then each head's q and k divided by its root mean square (no weight); a query sees
the keys of its own block of `size` positions up to itself; the softmax's denominator also holds exp(sink_h).
The feed-forward is a gated SiLU one, dense or routed (softmax router; a learned correction enters the choice
only; the last router outputs are identity experts that return their input).  A span of layers may run several
times with the same weights; every pass is opened by adding a vector of its own to x.  Output: LN, then the
embedding table again, times a constant.
"""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors.torch import load_file


def read_folder(folder: str, dtype=torch.float32):
    with open(os.path.join(folder, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    return cfg, {k: (v.to(dtype) if v.dtype.is_floating_point else v) for k, v in tensors.items()}


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last dimension (eps inside the root), no weight."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, D]: dimension i < dims/2 and dimension i + dims/2 turn by positions * base^(-2i/dims);
    dimensions from ``dims`` on pass."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    f = torch.as_tensor(base, dtype=x.dtype) ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * f[None, :]                       # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T: int, size: int | None) -> torch.Tensor:
    """[T, T] bool: query i sees key j when j <= i and both lie in the same block of ``size`` positions
    counted from 0 (``size`` None: every j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size:
        ok = ok & (i // size == j // size)
    return ok


def sink_softmax(scores: torch.Tensor, sink: torch.Tensor | None) -> torch.Tensor:
    """Softmax along the last dimension of scores [H, T, T] (masked entries -inf) whose denominator also
    holds exp(sink[h]); the weights of a row then sum to less than one."""
    if sink is None:
        return torch.softmax(scores, dim=-1)
    extra = sink.to(scores.dtype)[:, None, None].expand(scores.shape[0], scores.shape[1], 1)
    return torch.softmax(torch.cat([scores, extra], dim=-1), dim=-1)[..., :-1]


def attention(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor | None = None) -> torch.Tensor:
    """h [T, width]; w: 'q', 'k', 'v', 'o' and optionally 'sink'; m: the mixer's sizes and constants."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    pos = torch.arange(T) if positions is None else positions
    q = (h @ w["q"].T).view(T, H, D)
    k = (h @ w["k"].T).view(T, G, D)
    v = (h @ w["v"].T).view(T, G, V)
    rot = m.get("rot") or None
    if rot:
        q = rotate_half(q, pos, rot["dims"], rot["base"])
        k = rotate_half(k, pos, rot["dims"], rot["base"])
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    per = H // G
    k = k.repeat_interleave(per, dim=1)
    v = v.repeat_interleave(per, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    mask = m.get("mask") or None
    s = s.masked_fill(~visible(T, mask["size"] if mask else None)[None], -math.inf)
    p = sink_softmax(s, w.get("sink"))
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * V)
    return o @ w["o"].T


def gated_ff(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    g = h @ gate.T
    return ((g * torch.sigmoid(g)) * (h @ up.T)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor | None, top: int):
    """Chosen outputs [T, top] of the router and their weights: softmax over all outputs; the choice is by
    score + correction, the weight is the score itself."""
    s = torch.softmax(h @ router.T, dim=-1)
    pick = s if correction is None else s + correction
    idx = torch.topk(pick, top, dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def routed_ff(h: torch.Tensor, w: dict, f: dict) -> torch.Tensor:
    """w: 'router', optionally 'correction', and 'e<i>.gate' / '.up' / '.down' of the experts that have tensors;
    router outputs from ``experts`` on are identity experts."""
    r = f["router"]
    E, top = r["experts"], r["top"]
    idx, weight = route(h, w["router"], w.get("correction"), top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            if e < E:
                y = gated_ff(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
            else:
                y = h[t]
            out[t] += weight[t, c] * y
    return out


def order(n_layers: int, loop: dict | None) -> list[tuple[int, int | None]]:
    """(layer, number of the pass this run opens or None) in execution order."""
    if not loop:
        return [(i, None) for i in range(n_layers)]
    a, b, times = loop["start"], loop["stop"], loop.get("times", 1)
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n_layers)]


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(c: dict, weights: dict, ids, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence ``ids``.  ``streams``: a list that receives x after every run."""
    eps = c["norm"]["eps"]
    m = c.get("residual_mult", 1.0)
    E = weights["embed"]
    x = E[torch.as_tensor(ids, dtype=torch.long)] * (c.get("embedding") or {}).get("scale", 1.0)
    for layer, opens in order(len(c["layers"]), c.get("loop") or None):
        entry = c["layers"][layer]
        p = f"l{layer}."
        if opens is not None:
            x = x + weights["loop.step"][opens]
        h = layer_norm(x, weights[p + "norm1"], weights[p + "norm1.b"], eps)
        y = attention(h, sub(weights, p + "mix."), entry["mixer"], eps)
        f = entry.get("mlp")
        if f:
            fw = sub(weights, p + "mlp.")
            y = y + (gated_ff(h, fw["gate"], fw["up"], fw["down"]) if f["kind"] == "dense" else routed_ff(h, fw, f))
        x = x + m * y
        if streams is not None:
            streams.append(x.clone())
    x = layer_norm(x, weights["final.norm"], weights["final.norm.b"], eps)
    return (x @ E.T) * c.get("logit_scale", 1.0)
