"""Two mixers side by side: left_scale * left(h) + right_scale * right(h), both reading the same input.

Both halves are mixers of the form W_out f(W_in h + b) that expose their two products (``Mixer.in_projection`` /
``heads_forward`` / ``out_projection``).  The pair then runs ONE input product for both (the weights stacked by rows)
and ONE output product (the weights side by side along the inner dimension, each half writing its heads, already
multiplied by its scale in 32-bit before the one rounding, into its columns of a common tensor); the sum of the two
halves is the output product's own accumulation.  At most one half may want the paged cache and at most one a state
slot; the pair declares them as its own.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, CacheNeed, Mixer, ParamSpec, StateNeed, build, register


class PairedMixer(Mixer):
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.left = build("mixer", spec.left, ctx)
        self.right = build("mixer", spec.right, ctx)
        self.scales = (float(spec.left_scale), float(spec.right_scale))
        self.prefixes = tuple(spec.names)
        if len(set(self.prefixes)) != 2:
            raise ValueError("paired_mixer: the halves need two tensor prefixes")
        halves = (self.left, self.right)
        if sum(m.cache_need() is not None for m in halves) > 1 or sum(m.state_need() is not None for m in halves) > 1:
            raise ValueError("paired_mixer: at most one half may use the paged cache and at most one a state slot")
        self.w_in = self.b_in = self.w_out = None
        self.n_in = self.n_heads = (0, 0)

    def parameters(self) -> dict[str, ParamSpec]:
        out = {}
        for prefix, m in zip(self.prefixes, (self.left, self.right)):
            out.update({prefix + k: v for k, v in m.parameters().items()})
        return out

    def load(self, t: dict[str, torch.Tensor]) -> None:
        for prefix, m in zip(self.prefixes, (self.left, self.right)):
            m.load({k: t[prefix + k] for k in m.parameters()})
        (wl, bl), (wr, br) = self.left.in_projection(), self.right.in_projection()
        self.n_in = (wl.shape[0], wr.shape[0])
        self.w_in = torch.cat([wl, wr], dim=0).contiguous()
        if bl is not None or br is not None:
            zeros = lambda w: torch.zeros(w.shape[0], dtype=w.dtype, device=w.device)
            self.b_in = torch.cat([zeros(wl) if bl is None else bl, zeros(wr) if br is None else br]).contiguous()
        ol, orr = self.left.out_projection(), self.right.out_projection()
        self.n_heads = (ol.shape[1], orr.shape[1])
        self.w_out = torch.cat([ol, orr], dim=1).contiguous()

    def cache_need(self) -> CacheNeed | None:
        return self.left.cache_need() or self.right.cache_need()

    def state_need(self) -> StateNeed | None:
        return self.left.state_need() or self.right.state_need()

    def forward(self, x: torch.Tensor, step, cache, state) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        (nl, nr), (hl, hr) = self.n_in, self.n_heads
        proj = torch.empty((T, nl + nr), dtype=x.dtype, device=x.device)
        ops.linear(proj, x, self.w_in, self.b_in)
        heads = torch.empty((T, hl + hr), dtype=x.dtype, device=x.device)
        self.left.heads_forward(proj[:, :nl], step, cache, state, heads[:, :hl], self.scales[0])
        self.right.heads_forward(proj[:, nl:], step, cache, state, heads[:, hl:], self.scales[1])
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, heads, self.w_out, may_defer=True)


register("mixer", "paired_mixer", PairedMixer)
