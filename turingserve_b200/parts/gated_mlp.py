"""Dense gated feed-forward: down(act(gate(x)) * up(x)), gate and up fused into one product
(turingserve/model/qwen2.py:35-36, turingserve/model/loader.py:84, turingserve/ops/reference.py:26-28).
act is SiLU (the activation may then sit in the product's epilogue) or another one-input activation the kernels
have (the two GELUs, squared ReLU: product, then the activation kernel).
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, FeedForward, ParamSpec, register


class GatedMLP(FeedForward):
    def __init__(self, spec, ctx: BuildContext) -> None:
        if spec.activation not in ("silu", "gelu_tanh", "gelu", "relu2"):
            raise ValueError(f"gated_mlp: activation {spec.activation!r} has no kernel")
        self.activation = spec.activation
        self.hidden = ctx.hidden_size
        self.inter = int(spec.intermediate_size)
        self.bias = bool(spec.bias)
        self.names = tuple(getattr(spec, "names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        if self.bias and any(not n.endswith(".weight") for n in self.names):
            raise ValueError("gated_mlp: biases are named after weights that end in '.weight'")
        self.w_gate_up = self.b_gate_up = self.w_down = self.b_down = None
        self.group = 0

    def parameters(self) -> dict[str, ParamSpec]:
        g, u, d = self.names
        p = {g: ParamSpec((self.inter, self.hidden)), u: ParamSpec((self.inter, self.hidden)),
             d: ParamSpec((self.hidden, self.inter))}
        if self.bias:
            p[self._bias_of(g)] = ParamSpec((self.inter,))
            p[self._bias_of(u)] = ParamSpec((self.inter,))
            p[self._bias_of(d)] = ParamSpec((self.hidden,))
        return p

    @staticmethod
    def _bias_of(weight_name: str) -> str:
        return weight_name[: -len("weight")] + "bias"

    # Gate and up rows are interleaved in blocks of GROUP when the width allows: a 128-row tile of the
    # fused product then holds 64 gates and their 64 ups, and a kernel that computes such a tile can
    # apply the activation before anything leaves the chip.
    GROUP = 64

    def _pack(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        if not self.group:
            return torch.cat([gate, up], dim=0).contiguous()
        g = gate.reshape(self.inter // self.group, self.group, *gate.shape[1:])
        u = up.reshape(self.inter // self.group, self.group, *up.shape[1:])
        return torch.cat([g, u], dim=1).reshape(2 * self.inter, *gate.shape[1:]).contiguous()

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.group = self.GROUP if self.inter % self.GROUP == 0 else 0
        g, u, d = self.names
        self.w_gate_up = self._pack(t[g], t[u])
        self.w_down = t[d].contiguous()
        if self.bias:
            self.b_gate_up = self._pack(t[self._bias_of(g)], t[self._bias_of(u)])
            self.b_down = t[self._bias_of(d)].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        act = torch.empty((T, self.inter), dtype=x.dtype, device=x.device)
        if self.activation == "silu":
            ops.gated_linear(act, x, self.w_gate_up, self.b_gate_up, self.group)
        else:
            gu = torch.empty((T, 2 * self.inter), dtype=x.dtype, device=x.device)
            ops.linear(gu, x, self.w_gate_up, self.b_gate_up)
            ops.act_mul(act, gu, self.activation, self.group)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, act, self.w_down, self.b_down, may_defer=True)


register("feed_forward", "gated_mlp", GatedMLP)
