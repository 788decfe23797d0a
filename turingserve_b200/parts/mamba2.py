"""Selective state-space mixer with a scalar decay per head (the state-space-duality form).

One fused projection gives, per token, [z (H P) | x (H P) | B (G N) | C (G N) | dt (H)].  x, B and C pass a causal
filter of a few taps per channel ('conv' [channels, taps], the last column the present token's, with bias 'conv.b')
and SiLU.  dt <- softplus(dt + dt_bias).  Per head, in 32-bit, with S the head's state [N, P] and head h reading
group h // (H / G):   S <- exp(-exp(A_log_h) dt) S + dt B x^T;   y = S^T C + D_h x.  The heads side by side are
multiplied by silu(z), RMS-normed in ``norm_groups`` equal parts (each by its own root mean square) times 'norm',
and projected.

Nothing is cached per token.  The mixer declares one flat 32-bit state per request:
[H N P values of S | (taps - 1) x (H P + 2 G N) last filter inputs], zeroed when the request is admitted, so the first
portion needs no branch and a captured step's padding rows update the null slot.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, Mixer, ParamSpec, StateNeed, register


class Mamba2(Mixer):
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.H, self.P, self.N, self.G = int(spec.num_heads), int(spec.head_dim), int(spec.state_size), int(spec.num_groups)
        self.taps, self.norm_groups, self.eps = int(spec.conv_taps), int(spec.norm_groups), float(spec.norm_eps)
        if self.G < 1 or self.H % self.G:
            raise ValueError("mamba2: num_heads must be a multiple of num_groups")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"mamba2: a filter of {self.taps} taps (the kernels take 1 to 8)")
        self.inner = self.H * self.P
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.inner} columns do not fall into {self.norm_groups} equal parts")
        if self.N > 256:
            raise ValueError(f"mamba2: a state of {self.N} rows (the scan takes up to 256)")
        self.channels = self.inner + 2 * self.G * self.N                 # what passes the filter
        self.n_in = 2 * self.inner + 2 * self.G * self.N + self.H
        self.w_in = self.w_o = self.conv = self.conv_b = self.a_log = self.dt_bias = self.skip = self.norm_w = None

    def parameters(self) -> dict[str, ParamSpec]:
        return {"in": ParamSpec((self.n_in, self.hidden)),
                "conv": ParamSpec((self.channels, self.taps), compute_dtype=False),
                "conv.b": ParamSpec((self.channels,), compute_dtype=False, init="zeros"),
                "dt_bias": ParamSpec((self.H,), compute_dtype=False, init="zeros"),
                "A_log": ParamSpec((self.H,), compute_dtype=False, init="zeros"),
                "D": ParamSpec((self.H,), compute_dtype=False, init="ones"),
                "norm": ParamSpec((self.inner,), compute_dtype=False, init="ones"),
                "o": ParamSpec((self.hidden, self.inner))}

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_in, self.w_o = t["in"].contiguous(), t["o"].contiguous()
        self.conv, self.conv_b = t["conv"].float().contiguous(), t["conv.b"].float().contiguous()
        self.a_log, self.dt_bias = t["A_log"].float().contiguous(), t["dt_bias"].float().contiguous()
        self.skip, self.norm_w = t["D"].float().contiguous(), t["norm"].float().contiguous()

    def state_need(self) -> StateNeed:
        return StateNeed((self.H * self.N * self.P + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x: torch.Tensor, step, cache, state: torch.Tensor) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        H, P, N, G = self.H, self.P, self.N, self.G
        proj = torch.empty((T, self.n_in), dtype=x.dtype, device=x.device)
        ops.linear(proj, x, self.w_in)
        # 32-bit rows [x | B | C | dt | a] for the scan
        ready = torch.empty((T, self.channels + 2 * H), dtype=torch.float32, device=x.device)
        ops.ssm_prepare(ready, proj, self.inner, self.inner + self.channels, self.conv, self.conv_b, self.a_log,
                        self.dt_bias, state, H * N * P, step, H, self.channels, self.taps)
        y = torch.empty((T, self.inner), dtype=torch.float32, device=x.device)
        ops.ssm_scan(y, ready, proj, self.inner, state, self.skip, step, H, G, N, P, self.taps)
        g = torch.empty((T, self.inner), dtype=x.dtype, device=x.device)
        ops.gated_group_rmsnorm(g, y, proj[:, :self.inner], self.norm_w, self.eps, self.norm_groups, "silu", True)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, g, self.w_o, may_defer=True)


register("mixer", "mamba2", Mamba2)
