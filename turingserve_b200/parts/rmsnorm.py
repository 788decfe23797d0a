"""RMSNorm with the residual add fused in.

y = w * dtype(x32 * rsqrt(mean(x32^2) + eps)); with a residual, first residual = x + residual
(rounded to the model dtype) and the norm is taken of that sum
(turingserve/ops/reference.py:13-23, turingserve/ops/triton_rmsnorm.py:10-27).
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BranchSum, BuildContext, Norm, ParamSpec, StreamUpdate, register


class RMSNorm(Norm):
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.eps = float(spec.eps)
        self.size = ctx.hidden_size
        self.weight: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), compute_dtype=False, init="ones")}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``x`` is a tensor, or a product that its kernel left unreduced (it has shape, dtype and
        device; the norm kernel finishes the sum)."""
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        kernels.ops().rmsnorm(out, x, self.weight, self.eps, residual)
        return out


class StreamRMSNorm(Norm):
    """The norm of a residual stream kept in 32-bit whatever the engine's type: ``forward(x, stream)``
    first adds the pending branch output ``x`` (and ``extra``, when given) to ``stream`` in place, then
    returns stream / sqrt(mean(stream^2) + eps) * weight in the engine's type (32-bit arithmetic, one
    rounding).  ``first``: ``stream`` is started from ``x`` instead of added to.  The spec's
    ``weight_name`` is the scale's local tensor name ('' where the checkpoint names the scale by the
    norm's own prefix)."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.eps = float(spec.eps)
        self.size = ctx.hidden_size
        self.dtype = ctx.dtype
        self.weight_name = str(getattr(spec, "weight_name", "weight"))
        self.weight: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.size,), compute_dtype=False, init="ones")}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, x, residual: torch.Tensor | None = None, extra=None, first: bool = False) -> torch.Tensor:
        if residual is None:
            raise ValueError("the stream norm needs the 32-bit stream it adds to")
        out = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
        kernels.ops().rmsnorm_stream(out, residual, x, extra, self.weight, self.eps, first)
        return out


class StreamLayerNorm(Norm):
    """The layer norm of a residual stream kept in 32-bit whatever the engine's type.  ``forward(x, stream)`` first
    takes what is pending into ``stream`` in place, stream += scale * (a + b) + row, where ``x`` is a tensor (scale 1)
    or a ``BranchSum`` (the outputs of a layer's branches and the constant they are multiplied by) and ``row`` a
    float32 vector common to all tokens; then returns (stream - mean) / sqrt(variance + eps) * weight + bias in the
    engine's type (32-bit arithmetic, one rounding).  ``first``: ``stream`` is started instead of added to."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.eps = float(spec.eps)
        self.size = ctx.hidden_size
        self.dtype = ctx.dtype
        self.weight_name, self.bias_name = str(spec.weight_name), str(spec.bias_name)
        if self.weight_name == self.bias_name:
            raise ValueError("layernorm_stream: weight and bias need two tensor names")
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.size,), compute_dtype=False, init="ones"),
                self.bias_name: ParamSpec((self.size,), compute_dtype=False, init="zeros")}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        # both in 32-bit: the kernel reads them as one type, and the norm's arithmetic is 32-bit anyway
        self.weight = tensors[self.weight_name].float().contiguous()
        self.bias = tensors[self.bias_name].float().contiguous()

    def forward(self, x, residual: torch.Tensor | None = None, row=None, first: bool = False) -> torch.Tensor:
        if residual is None:
            raise ValueError("the stream norm needs the 32-bit stream it adds to")
        a, b, scale = (x.first, x.second, x.scale) if isinstance(x, BranchSum) else (x, None, 1.0)
        out = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
        kernels.ops().rmsnorm_stream(out, residual, a, b, self.weight, self.eps, first, alpha=scale, row=row,
                                     norm_bias=self.bias)
        return out


class HyperRMSNorm(Norm):
    """The norm a sublayer reads a residual stream of several 32-bit copies through.  ``forward(pending, streams,
    link)``: first the write-back of what the sublayer before left pending (a ``StreamUpdate``; a ``BranchSum`` with
    ``first``: the embedding rows times a constant start every copy), then u = sum_s in[s] x_s with the weights of
    ``link`` (None: the plain sum of the copies, which is what a model's last norm reads), then
    u / sqrt(mean(u^2) + eps) * (weight_offset + weight) in the engine's type (32-bit arithmetic, one rounding)."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.eps = float(spec.eps)
        self.size = ctx.hidden_size
        self.dtype = ctx.dtype
        self.S = int(spec.streams)
        self.offset = float(spec.weight_offset)
        self.weight_name = str(spec.weight_name)
        self.weight: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.size,), compute_dtype=False, init="zeros" if self.offset else "ones")}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        # in 32-bit, the offset added once: the kernel multiplies by one vector
        self.weight = (tensors[self.weight_name].float() + self.offset).contiguous()

    def forward(self, pending, streams: torch.Tensor | None = None, link=None, first: bool = False) -> torch.Tensor:
        if streams is None:
            raise ValueError("the stream norm needs the 32-bit copies it reads")
        T = streams.shape[0]
        out = torch.empty((T, self.size), dtype=self.dtype, device=streams.device)
        in_w = None if link is None else link.w_in
        ops = kernels.ops()
        if first:
            rows, alpha = (pending.first, pending.scale) if isinstance(pending, BranchSum) else (pending, 1.0)
            ops.hyper_norm(out, streams, rows, None, None, in_w, self.weight, self.eps, first=True, alpha=alpha)
        elif isinstance(pending, StreamUpdate):
            ops.hyper_norm(out, streams, pending.y, pending.link.mix, pending.link.w_out, in_w, self.weight, self.eps)
        elif pending is None:
            ops.hyper_norm(out, streams, None, None, None, in_w, self.weight, self.eps)
        else:
            raise TypeError(f"rmsnorm_hyper: what is pending must be a StreamUpdate, not {type(pending).__name__}")
        return out


register("norm", "rmsnorm", RMSNorm)
register("norm", "rmsnorm_hyper", HyperRMSNorm)
register("norm", "layernorm_stream", StreamLayerNorm)
register("norm", "rmsnorm_stream", StreamRMSNorm)
