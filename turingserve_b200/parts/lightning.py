"""Linear attention with a decaying matrix state per head ("lightning attention").

q, k, v = silu of one fused projection; per head S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, the
state in 32-bit in the request's state slot; the heads' outputs side by side get one RMS norm with a
learned scale, a sigmoid gate from a fourth projection of the same input, and the output projection.
Nothing is cached per token: the mixer declares a ``StateNeed`` and no ``CacheNeed``.  A request's slot
is zeroed when it is admitted, so the first portion needs no branch, and a captured step's padding rows
update the null slot.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, Mixer, ParamSpec, StateNeed, register


class Lightning(Mixer):
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.H, self.D, self.V = int(spec.num_heads), int(spec.key_dim), int(spec.value_dim)
        if len(spec.decays) != self.H:
            raise ValueError(f"lightning: {len(spec.decays)} decays for {self.H} heads")
        if spec.activation != "silu":
            raise ValueError(f"lightning: activation {spec.activation!r} has no kernel")
        self.decays = tuple(float(d) for d in spec.decays)
        self.eps = float(spec.norm_eps)
        self.device = ctx.device
        self.w_in = self.w_o = self.norm_w = self.norm_w32 = self.decay = None

    def parameters(self) -> dict[str, ParamSpec]:
        hd, hv = self.H * self.D, self.H * self.V
        return {"q": ParamSpec((hd, self.hidden)), "k": ParamSpec((hd, self.hidden)),
                "v": ParamSpec((hv, self.hidden)), "g": ParamSpec((hv, self.hidden)),
                "o": ParamSpec((self.hidden, hv)),
                "norm": ParamSpec((hv,), compute_dtype=False, init="ones")}

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([t["q"], t["k"], t["v"], t["g"]], dim=0).contiguous()
        self.w_o = t["o"].contiguous()
        self.norm_w = t["norm"].contiguous()
        self.norm_w32 = self.norm_w.float().contiguous()
        self.decay = torch.tensor(self.decays, dtype=torch.float32, device=self.w_o.device)

    def state_need(self) -> StateNeed:
        return StateNeed((self.H, self.D, self.V), torch.float32)

    # -- the two products apart (a mixer made of several runs them fused with its other halves') -------------------
    def in_projection(self):
        return self.w_in, None

    def out_projection(self):
        return self.w_o

    def heads_forward(self, proj, step, cache, state, out, scale: float = 1.0) -> None:
        """``proj`` [T, q | k | v | gate]: the scan, then the norm over all heads times sigmoid(gate) and ``scale`` into
        ``out`` [T, H V].  Both may be column slices of wider tensors."""
        ops = kernels.ops()
        hd, hv = self.H * self.D, self.H * self.V
        o = torch.empty((proj.shape[0], hv), dtype=torch.float32, device=proj.device)
        ops.lightning(o, proj, state, self.decay, step, self.H, self.D, self.V)
        ops.gated_group_rmsnorm(out, o, proj[:, 2 * hd + hv:], self.norm_w32, self.eps, 1, "sigmoid", False, scale)

    def forward(self, x: torch.Tensor, step, cache, state: torch.Tensor) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        hd, hv = self.H * self.D, self.H * self.V
        proj = torch.empty((T, 2 * hd + 2 * hv), dtype=x.dtype, device=x.device)
        ops.linear(proj, x, self.w_in)
        o = torch.empty((T, hv), dtype=torch.float32, device=x.device)
        ops.lightning(o, proj, state, self.decay, step, self.H, self.D, self.V)
        y = torch.empty((T, hv), dtype=x.dtype, device=x.device)
        ops.gated_rmsnorm(y, o, proj[:, 2 * hd + hv:], self.norm_w, self.eps)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, y, self.w_o, may_defer=True)


register("mixer", "lightning", Lightning)
