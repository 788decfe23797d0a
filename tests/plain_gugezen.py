"""Plain, slow Gugezen: one function per mechanism, whole sequences, no cache, nothing shared with the product.

Everything runs in the type of the tensors it is given (the tests hand it float64 or float32).  ``forward`` takes
the configuration as config.json spells it and the tensors by their checkpoint names.
"""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors.torch import load_file


def read_folder(folder: str, dtype=torch.float64):
    with open(os.path.join(folder, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    return cfg, {k: (v.to(dtype) if v.dtype.is_floating_point else v) for k, v in tensors.items()}


# -- norms and activations -------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last dimension, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight lies around zero: the scale is 1 + w."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# -- rotation ----------------------------------------------------------------------------------------------------------
def scaled_frequencies(base: float, dims: int, scaling: dict | None) -> list[float]:
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` (factor, low, high, original) a frequency whose wavelength
    is below original/high stays, one above original/low is divided by factor, and between them the two are blended
    linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            original = float(scaling["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_neighbours(x: torch.Tensor, positions: torch.Tensor, freqs: list[float]) -> torch.Tensor:
    """x [T, heads, D]: dimensions (2i, 2i+1), i < len(freqs), turned by position * f_i; the rest pass."""
    out = x.clone()
    f = torch.tensor(freqs, dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]                   # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    n = 2 * len(freqs)
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


# -- the left half of the 'parallel' mixer ----------------------------------------------------------------------------
def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, sink: torch.Tensor) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V]; causal; the denominator of head h also holds exp(sink_h)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        m = torch.maximum(s.max(-1).values, sink[h].expand(T))
        e = torch.exp(s - m[:, None])
        out[:, h] = (e @ v[:, g]) / (e.sum(-1) + torch.exp(sink[h] - m))[:, None]
    return out


def left_branch(h: torch.Tensor, W: dict, p: str, m: dict, positions: torch.Tensor) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, V)
    rot = m.get("rot")
    if rot and rot.get("dims", 0):
        f = scaled_frequencies(float(rot["base"]), int(rot["dims"]), rot.get("scaling"))
        q, k = rotate_neighbours(q, positions, f), rotate_neighbours(k, positions, f)
    a = sink_attention(q, k, v, float(m["scale"]), W[p + "sink"])
    a = a.reshape(T, H * V) * torch.sigmoid(h @ W[p + "g"].T)
    return a @ W[p + "o"].T


# -- the right half ----------------------------------------------------------------------------------------------------
def decayed_state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: list[float]) -> torch.Tensor:
    """q, k [T, H, D], v [T, H, V]: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, D = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        S = torch.zeros(D, v.shape[2], dtype=q.dtype)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def right_branch(h: torch.Tensor, W: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).view(T, H, D)
    k = silu(h @ W[p + "k"].T).view(T, H, D)
    v = silu(h @ W[p + "v"].T).view(T, H, V)
    o = decayed_state_scan(q, k, v, [float(d) for d in m["decay"]]).reshape(T, H * V)
    o = unit_rms(o, eps) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def parallel_mixer(h: torch.Tensor, W: dict, p: str, m: dict, eps: float, positions: torch.Tensor) -> torch.Tensor:
    return (float(m["left_scale"]) * left_branch(h, W, p + "left.", m["left"], positions)
            + float(m["right_scale"]) * right_branch(h, W, p + "right.", m["right"], eps))


# -- the state-space mixer ----------------------------------------------------------------------------------------------
def causal_filter(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps] (the last column is the present token's), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    out = b.expand(T, C).clone()
    for j in range(taps):
        out = out + padded[j:j + T] * w[:, j]
    return out


def state_space_scan(x, dt, a_log, B, C, D):
    """x [T, H, P], dt [T, H], B and C [T, G, N]: S_t = exp(-exp(a_log_h) dt) S_(t-1) + dt B_t x_t^T (S is N x P),
    y_t = S_t^T C_t + D_h x_t; head h reads group h // (H / G)."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros(T, H, P, dtype=x.dtype)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros(N, P, dtype=x.dtype)
        for t in range(T):
            S = torch.exp(-torch.exp(a_log[h]) * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return y


def mamba2_mixer(h: torch.Tensor, W: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ W[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_filter(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])
    y = state_space_scan(x, dt, W[p + "A_log"], B, C, W[p + "D"]).reshape(T, inner)
    y = y * silu(z)
    parts = int(m["norm_groups"])
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


# -- feed-forwards ------------------------------------------------------------------------------------------------------
def dense_ff(h: torch.Tensor, W: dict, p: str) -> torch.Tensor:
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def small_ff(h: torch.Tensor, W: dict, p: str) -> torch.Tensor:
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


def route(h: torch.Tensor, w_router: torch.Tensor, top: int):
    """The ``top`` experts with the largest softmax scores, and the scores over their sum."""
    s = torch.softmax(h @ w_router.T, -1)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20)


def routed_ff(h: torch.Tensor, W: dict, p: str, f: dict) -> torch.Tensor:
    idx, wt = route(h, W[p + "router"], int(f["router"]["top"]))
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for r in range(idx.shape[1]):
            out[t] += wt[t, r] * small_ff(h[t:t + 1], W, f"{p}e{int(idx[t, r])}.")[0]
    if f.get("shared"):
        out = out + small_ff(h, W, p + "shared.")
    return out


def feed_forward(h: torch.Tensor, W: dict, p: str, f: dict) -> torch.Tensor:
    return dense_ff(h, W, p) if f["kind"] == "dense" else routed_ff(h, W, p, f)


# -- the model ------------------------------------------------------------------------------------------------------------
def forward(config: dict, W: dict, tokens: list[int], dtype=torch.float64):
    """(logits [T, vocab], the sum of the streams after every layer run [runs, T, width])."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x0 = W["embed"][torch.tensor(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    S = config.get("streams")
    xs = [x0.clone() for _ in range(S or 1)]
    after = []
    for i, entry in enumerate(config["layers"]):
        src = entry.get("weights_of", i)
        pre = f"l{src}."
        subs = [(1, lambda u: parallel_mixer(u, W, pre + "mix.", entry["mixer"], eps, positions)
                 if entry["type"] == "parallel" else mamba2_mixer(u, W, pre + "mix.", entry["mixer"], eps))]
        if entry.get("mlp"):
            subs.append((2, lambda u: feed_forward(u, W, pre + "mlp.", entry["mlp"])))
        for q, fn in subs:
            if S:
                w_in, w_out, w_mix = W[f"{pre}hc{q}.in"], W[f"{pre}hc{q}.out"], W[f"{pre}hc{q}.mix"]
                u = sum(w_in[s] * xs[s] for s in range(S))
                y = fn(zero_centred_norm(u, W[f"{pre}norm{q}"], eps))
                xs = [sum(w_mix[s, t] * xs[s] for s in range(S)) + w_out[t] * y for t in range(S)]
            else:
                xs = [xs[0] + fn(zero_centred_norm(xs[0], W[f"{pre}norm{q}"], eps))]
        after.append(sum(xs))
    x = zero_centred_norm(sum(xs), W["final.norm"], eps)
    logits = (x @ W["embed"].T) * float(config.get("logit_scale", 1.0))
    return logits, torch.stack(after)
