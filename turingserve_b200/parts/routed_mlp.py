"""Routed feed-forward: every token goes through the ``top_k`` of ``num_experts`` small feed-forwards
down_e(act(up_e(.))), or gated ones down_e(act(gate_e(.)) * up_e(.)), whose router scores are largest.
A learned correction may enter the choice (score + correction) without entering the weights.  The router may have
more outputs than there are experts with tensors: the outputs behind them are experts that return their input,
which cost no product (their pairs are sorted behind the others and the sum takes the token's own row for them).

A shared expert (``shared_intermediate_size``: one more feed-forward of the experts' form under 'shared.') runs for every
token and is added, unweighted, in the kernel that sums a token's choices.

Router logits and scores are 32-bit.  The (token, choice) pairs are sorted by expert on the device and the
two products run over the sorted groups; the chosen score multiplies the expert's input (``weight_on``
"input", the product reads score * x rounded to the engine's type) or its output; a token's choices are
summed in 32-bit in the order of their rank.  No count comes back to the host, so the chain may sit in a
captured step.  The experts' weights are stacked [E, ff, hidden] and [E, hidden, ff] when they arrive.

Many rows (``LIBRARY_ROWS`` pairs or more, outside a capture): the group sizes are read back once, the input
rows are gathered in sorted order, and every expert's rows go through ``ops().linear`` as a product of their own,
i.e. to the many-row kernels and the vendor library that the dense products of such steps use.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, FeedForward, ParamSpec, register
from turingserve_b200.parts.mlp import ACTIVATIONS


class RoutedMLP(FeedForward):
    # from this many (token, choice) pairs in a step the experts' products are launched one by one (2,048 tokens of
    # width 3,584 through 8 experts of 7,104: 2.7 ms for the two grouped products, 0.5 ms this way)
    LIBRARY_ROWS = 1024

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.E, self.top, self.inter = int(spec.num_experts), int(spec.top_k), int(spec.intermediate_size)
        if self.top < 1 or self.E < 0:
            raise ValueError(f"routed_mlp: top {self.top} of {self.E} experts")
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"routed_mlp: activation {spec.activation!r} has no kernel")
        if spec.scoring not in ("sigmoid", "softmax") or spec.weight_on not in ("input", "output"):
            raise ValueError(f"routed_mlp: scoring {spec.scoring!r} / weight_on {spec.weight_on!r}")
        self.activation, self.softmax = spec.activation, spec.scoring == "softmax"
        self.renormalize, self.on_input = bool(spec.renormalize), spec.weight_on == "input"
        self.gated, self.has_correction = bool(getattr(spec, "gated", False)), bool(getattr(spec, "correction", False))
        self.identity = int(getattr(spec, "identity", 0))
        if self.identity < 0:
            raise ValueError(f"routed_mlp: {self.identity} identity experts")
        if self.gated and self.activation != "silu":
            raise ValueError(f"routed_mlp: gated experts with activation {self.activation!r} have no kernel")
        if self.identity and self.on_input:
            raise ValueError("routed_mlp: experts that return their input are weighted on the output")
        self.outputs = self.E + self.identity           # what the router scores
        if self.top > self.outputs:
            raise ValueError(f"routed_mlp: top {self.top} of {self.outputs} router outputs")
        shared = getattr(spec, "shared_intermediate_size", None)
        self.shared_inter = int(shared) if shared else 0
        self.w_router = self.w_up = self.w_down = self.correction = self.w_shared_up = self.w_shared_down = None

    def parameters(self) -> dict[str, ParamSpec]:
        p = {"router": ParamSpec((self.outputs, self.hidden), compute_dtype=False)}
        if self.has_correction:
            p["correction"] = ParamSpec((self.outputs,), compute_dtype=False, init="zeros")
        for e in range(self.E):
            if self.gated:
                p[f"e{e}.gate"] = ParamSpec((self.inter, self.hidden))
            p[f"e{e}.up"] = ParamSpec((self.inter, self.hidden))
            p[f"e{e}.down"] = ParamSpec((self.hidden, self.inter))
        if self.shared_inter:
            if self.gated:
                p["shared.gate"] = ParamSpec((self.shared_inter, self.hidden))
            p["shared.up"] = ParamSpec((self.shared_inter, self.hidden))
            p["shared.down"] = ParamSpec((self.hidden, self.shared_inter))
        return p

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_router = t["router"].float().contiguous()
        if self.has_correction:
            self.correction = t["correction"].float().contiguous()
        if self.shared_inter:
            self.w_shared_up = (torch.cat([t["shared.gate"], t["shared.up"]], dim=0) if self.gated else t["shared.up"]).contiguous()
            self.w_shared_down = t["shared.down"].contiguous()
        if self.E == 0:
            return
        # gated experts: an expert's gate rows, then its up rows, in one product
        ups = [torch.cat([t[f"e{e}.gate"], t[f"e{e}.up"]], dim=0) if self.gated else t[f"e{e}.up"] for e in range(self.E)]
        self.w_up = torch.stack(ups).contiguous()
        self.w_down = torch.stack([t[f"e{e}.down"] for e in range(self.E)]).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = kernels.ops()
        T, top = x.shape[0], self.top
        idx = torch.empty((T, top), dtype=torch.int32, device=x.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=x.device)
        ops.router_topk(idx, weights, x, self.w_router, self.softmax, self.renormalize, self.correction)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        if self.identity:
            # the pairs of the experts with tensors are sorted first; the others' output is the token's own row
            offsets, order, place, tiles = ops.moe_align(idx, self.outputs, self.E)
            passing = dict(x=x, pass_from=offsets[self.E:self.E + 1])
        else:
            offsets, order, place, tiles = ops.moe_align(idx, self.E)
            passing = {}
        if self.shared_inter:
            passing["add"] = self._shared(x)
        y = torch.empty((T * top, self.hidden), dtype=torch.float32, device=x.device)
        if self.E == 0:
            ops.moe_combine(out, y, place, weights, top, **passing)
            return out
        up_width = (2 if self.gated else 1) * self.inter
        a = torch.empty((T * top, up_width), dtype=x.dtype, device=x.device)
        scale = weights if self.on_input else None
        if T * top >= self.LIBRARY_ROWS and x.is_cuda and not torch.cuda.is_current_stream_capturing():
            # the experts' input rows in sorted order, weighted and rounded once (the products then read plain rows)
            xs = torch.empty((T * top, self.hidden), dtype=x.dtype, device=x.device)
            ops.moe_gather(xs, x, order, scale, top)
            bounds = offsets[: self.E + 1].tolist()                      # the one read-back of this path
            for e in range(self.E):
                lo, hi = bounds[e], bounds[e + 1]
                if hi > lo:
                    ops.linear(a[lo:hi], xs[lo:hi], self.w_up[e])
            a = self._activate(a, bounds[self.E])
            for e in range(self.E):
                lo, hi = bounds[e], bounds[e + 1]
                if hi > lo:
                    ops.linear(y[lo:hi], a[lo:hi], self.w_down[e])
        elif self.gated:
            # (the first product fetches a pair's token row itself, weighted and rounded as the gather would)
            ops.grouped_linear(a, x, self.w_up, order, scale, offsets, tiles, top)
            a = self._activate(a, T * top)
            ops.grouped_linear(y, a, self.w_down, None, None, offsets, tiles, 1)
        else:
            ops.grouped_linear(a, x, self.w_up, order, scale, offsets, tiles, top, self.activation)
            ops.grouped_linear(y, a, self.w_down, None, None, offsets, tiles, 1)
        ops.moe_combine(out, y, place, None if self.on_input else weights, top, **passing)
        return out

    def _shared(self, x: torch.Tensor) -> torch.Tensor:
        """The expert that every token uses: down(act(up(x))), or the gated form."""
        ops = kernels.ops()
        T = x.shape[0]
        a = torch.empty((T, self.shared_inter), dtype=x.dtype, device=x.device)
        if self.gated:
            gu = torch.empty((T, 2 * self.shared_inter), dtype=x.dtype, device=x.device)
            ops.linear(gu, x, self.w_shared_up)
            ops.silu_mul(a, gu, 0)
        else:
            ops.activation(a, ops.linear(a, x, self.w_shared_up, may_defer=True), self.activation)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, a, self.w_shared_down)

    def _activate(self, a: torch.Tensor, rows: int) -> torch.Tensor:
        """The first ``rows`` rows of the experts' first product through the activation (the rows behind them belong
        to experts without tensors and hold nothing); gated experts: act(gate) * up, half as wide."""
        ops = kernels.ops()
        if not self.gated:
            if rows:
                ops.activation(a[:rows], a[:rows], self.activation)
            return a
        g = torch.empty((a.shape[0], self.inter), dtype=a.dtype, device=a.device)
        if rows:
            ops.silu_mul(g[:rows], a[:rows], 0)
        return g


register("feed_forward", "routed_mlp", RoutedMLP)
