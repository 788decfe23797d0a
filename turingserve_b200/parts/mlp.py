"""Dense feed-forward without a gate: down(act(up(x))), act one of the one-input activations the kernels
have (the tanh form of GELU, the GELU with the error function, squared ReLU, SiLU).  No biases.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, FeedForward, ParamSpec, register

ACTIVATIONS = ("gelu_tanh", "relu2", "silu", "gelu")


class MLP(FeedForward):
    def __init__(self, spec, ctx: BuildContext) -> None:
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"mlp: activation {spec.activation!r} has no kernel (known: {', '.join(ACTIVATIONS)})")
        self.hidden, self.inter, self.activation = ctx.hidden_size, int(spec.intermediate_size), spec.activation
        self.w_up = self.w_down = None

    def parameters(self) -> dict[str, ParamSpec]:
        return {"up": ParamSpec((self.inter, self.hidden)), "down": ParamSpec((self.hidden, self.inter))}

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_up, self.w_down = t["up"].contiguous(), t["down"].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        a = torch.empty((T, self.inter), dtype=x.dtype, device=x.device)
        ops.activation(a, ops.linear(a, x, self.w_up, may_defer=True), self.activation)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, a, self.w_down, may_defer=True)


register("feed_forward", "mlp", MLP)
