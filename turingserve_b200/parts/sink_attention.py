"""Grouped-query attention in blocks of positions with a sink in the softmax, over the paged cache.

One fused projection gives, per token, [q (H D) | k (G D) | v (G V)]; no biases.  q and k are rotated over
their first dimensions (the position encoding named in the spec: pairs (i, i + dims / 2), angle = position *
frequency in 32-bit) and then, head by head, divided by their root mean square (no learned weight); the new key
and value rows go to the cache, whose key rows are D wide and value rows V wide.  score = q.k scale; position i
sees j <= i with floor(i / c) = floor(j / c) when a block size c is given (blocks are counted from the
sequence's position 0, wherever a prompt was cut), and with a window w only i - w < j; the softmax's denominator
also holds exp(sink_h), a learned number per head ('sink') without key or value.  Output projection on the
heads side by side.  Rotation, norm, block size, window and sink are each optional in the spec; so are biases on
q, k and v ('q.b', ...) and an output gate: the heads side by side times sigmoid(W_g h) ('g', a fourth block of
the fused projection) before the output projection.  The rotation pairs dimension i with i + dims / 2 or, with a
position encoding of neighbouring pairs (``pairing == "neighbours"``), dimension 2i with 2i + 1.

Pages: every key before the start of the block the next position lies in can never be seen again; the mixer
declares that as its cache need (``CacheNeed.chunk``) and the manager gives such pages back.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, CacheNeed, Mixer, ParamSpec, build, register


class SinkAttention(Mixer):
    MAX_KEY, MAX_VALUE = 1024, 512          # the any-size attention kernel's limits

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.H, self.G = int(spec.num_heads), int(spec.num_kv_heads)
        self.D, self.V = int(spec.key_dim), int(spec.value_dim)
        if self.G < 1 or self.H % self.G:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not (0 < self.D <= self.MAX_KEY and 0 < self.V <= self.MAX_VALUE):
            raise ValueError(f"sink_attention: keys of {self.D}, values of {self.V}: the kernels take up to "
                             f"{self.MAX_KEY} and {self.MAX_VALUE}")
        self.scale = float(spec.scale)
        self.norm_eps = None if spec.qk_norm_eps is None else float(spec.qk_norm_eps)
        self.chunk = int(spec.chunk) if spec.chunk else None
        self.window = int(spec.window) if spec.window else None
        self.has_sinks = bool(spec.sinks)
        self.position = build("position", spec.position, ctx) if spec.position is not None else None
        self.rot_dims = 0
        if self.position is not None:
            if not hasattr(self.position, "freq") or not hasattr(self.position, "dims"):
                raise ValueError("sink_attention takes a position encoding given by frequencies (kinds rope_half, "
                                 "rope_pairs_banded, yarn_pairs)")
            self.rot_dims = int(self.position.dims)
            if self.rot_dims > self.D:
                raise ValueError(f"sink_attention: {self.rot_dims} rotated dimensions of {self.D}")
        self.neighbours = self.position is not None and getattr(self.position, "pairing", "halves") == "neighbours"
        if self.neighbours and self.norm_eps is not None:
            raise ValueError("sink_attention: the per-head norm comes with the rotation by halves")
        self.has_bias, self.has_gate = bool(getattr(spec, "qkv_bias", False)), bool(getattr(spec, "out_gate", False))
        self.q_dim, self.k_dim, self.v_dim = self.H * self.D, self.G * self.D, self.G * self.V
        self.g_dim = self.H * self.V if self.has_gate else 0
        self.dtype = ctx.dtype
        self.w_qkv = self.w_o = self.sinks = self.b_qkv = None

    def parameters(self) -> dict[str, ParamSpec]:
        p = {"q": ParamSpec((self.q_dim, self.hidden)), "k": ParamSpec((self.k_dim, self.hidden)),
             "v": ParamSpec((self.v_dim, self.hidden)), "o": ParamSpec((self.hidden, self.H * self.V))}
        if self.has_sinks:
            p["sink"] = ParamSpec((self.H,), compute_dtype=False, init="zeros")
        if self.has_bias:
            p.update({"q.b": ParamSpec((self.q_dim,)), "k.b": ParamSpec((self.k_dim,)), "v.b": ParamSpec((self.v_dim,))})
        if self.has_gate:
            p["g"] = ParamSpec((self.g_dim, self.hidden))
        return p

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([t["q"], t["k"], t["v"]] + ([t["g"]] if self.has_gate else []), dim=0).contiguous()
        self.w_o = t["o"].contiguous()
        if self.has_sinks:
            self.sinks = t["sink"].float().contiguous()
        if self.has_bias:
            gate0 = [torch.zeros(self.g_dim, dtype=t["q.b"].dtype, device=t["q.b"].device)] if self.has_gate else []
            self.b_qkv = torch.cat([t["q.b"], t["k.b"], t["v.b"]] + gate0).contiguous()

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.G, self.D, self.window, value_dim=self.V, chunk=self.chunk)

    # -- the two products apart (a mixer made of several runs them fused with its other halves') -------------------
    def in_projection(self):
        return self.w_qkv, self.b_qkv

    def out_projection(self):
        return self.w_o

    def heads_forward(self, proj, step, cache, state, out, scale: float = 1.0) -> None:
        """``proj`` [T, q | k | v | gate]: rotation and cache write, attention, gate; the heads side by side, times
        ``scale``, into ``out`` [T, H V].  Both may be column slices of wider tensors."""
        ops = kernels.ops()
        T = proj.shape[0]
        H, G, D, V = self.H, self.G, self.D, self.V
        grp = step.groups[cache.group]
        slots = grp.slot_mapping if cache.writable else None
        k_off, v_off = self.q_dim, self.q_dim + self.k_dim
        if self.neighbours or (not self.rot_dims and self.norm_eps is None):
            # (without a rotation the same kernel is the plain cache write)
            ops.rope_pairs_write(proj, k_off, v_off, step.positions, self.position.freq if self.rot_dims else None,
                                 float(getattr(self.position, "magnitude", 1.0)), self.rot_dims, cache.k, cache.v, slots,
                                 H, G, D, V, cache.page_size)
        else:
            ops.rope_headnorm_write(proj, k_off, v_off, step.positions, self.position.freq if self.rot_dims else None,
                                    self.rot_dims, self.norm_eps, cache.k, cache.v, slots, H, G, D, V, cache.page_size)
        q = proj[:, :self.q_dim].view(T, H, D)
        plain = not self.has_gate and scale == 1.0
        attn = out.view(T, H, V) if plain else torch.empty((T, H, V), dtype=proj.dtype, device=proj.device)
        ops.attention_biased(attn, q, cache.k, cache.v, grp.block_tables, step, G, cache.page_size, self.scale, 0.0, None,
                             self.window, chunk=self.chunk, sinks=self.sinks)
        if self.has_gate:
            ops.gate_mul(out, attn.view(T, H * V), proj[:, v_off + self.v_dim:], "sigmoid", scale)
        elif not plain:
            raise ValueError("sink_attention: an output scale needs the output gate's kernel")

    def forward(self, x: torch.Tensor, step, cache, state=None) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        H, G, D, V = self.H, self.G, self.D, self.V
        if self.has_bias or self.has_gate or self.neighbours:
            proj = torch.empty((T, self.w_qkv.shape[0]), dtype=x.dtype, device=x.device)
            ops.linear(proj, x, self.w_qkv, self.b_qkv)
            heads = torch.empty((T, H * V), dtype=x.dtype, device=x.device)
            self.heads_forward(proj, step, cache, state, heads)
            out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
            return ops.linear(out, heads, self.w_o, may_defer=True)
        grp = step.groups[cache.group]
        proj = torch.empty((T, self.q_dim + self.k_dim + self.v_dim), dtype=x.dtype, device=x.device)
        # (a few tokens: the product's partial sums are summed by the kernel that rotates them)
        proj = ops.linear(proj, x, self.w_qkv, may_defer=True, lazy=False)
        # q rotated and normed in place; rotated, normed keys and the values into the cache
        proj = ops.rope_headnorm_write(proj, self.q_dim, self.q_dim + self.k_dim, step.positions,
                                self.position.freq if self.rot_dims else None, self.rot_dims, self.norm_eps,
                                cache.k, cache.v, grp.slot_mapping if cache.writable else None, H, G, D, V,
                                cache.page_size)
        attn = torch.empty((T, H, V), dtype=x.dtype, device=x.device)
        ops.attention_biased(attn, proj[:, :self.q_dim].view(T, H, D), cache.k, cache.v, grp.block_tables, step, G,
                             cache.page_size, self.scale, 0.0, None, self.window, chunk=self.chunk, sinks=self.sinks)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, attn.view(T, H * V), self.w_o, may_defer=True)


register("mixer", "sink_attention", SinkAttention)
