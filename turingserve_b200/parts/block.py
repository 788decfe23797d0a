"""How a mixer, a feed-forward and their norms are wired into one layer.

"pre_norm" carries (h, residual) and defers each residual add into the next norm: the first
block takes residual = h; afterwards every norm first does residual = h + residual in the model
dtype (turingserve/model/qwen2.py:42-57).
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BranchSum, BuildContext, StreamUpdate, build, register


class PreNormBlock:
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.mixer_norm = build("norm", spec.mixer_norm, ctx)
        self.mixer = build("mixer", spec.mixer, ctx)
        self.ffn_norm = build("norm", spec.ffn_norm, ctx)
        self.feed_forward = build("feed_forward", spec.feed_forward, ctx)

    def parts(self) -> dict[str, object]:
        """Sub-parts by the role names used in ``LayerTensorNames``."""
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "ffn_norm": self.ffn_norm, "feed_forward": self.feed_forward}

    def forward(self, h, residual, step, cache, state, inject=None):
        """``inject``: a tensor added to the stream before this layer (a model that re-injects its input)."""
        if inject is not None:
            h = kernels.ops().materialize(h) + inject
        if residual is None:
            residual = h
            x = self.mixer_norm.forward(h)
        else:
            x = self.mixer_norm.forward(h, residual)
        a = self.mixer.forward(x, step, cache, state)
        x = self.ffn_norm.forward(a, residual)
        h = self.feed_forward.forward(x)
        return h, residual


def _build_block(spec, ctx: BuildContext):
    return PreNormBlock(spec, ctx)


class StreamBlock:
    """Pre-norm wiring over a residual stream in 32-bit: x += mixer(norm(x)); x += ff(norm(x)), where
    x is a float32 tensor whatever the engine's type and the branch outputs are in the engine's type.
    Each add is deferred into the norm that follows (``StreamRMSNorm``): the block carries
    (pending branch output, stream).  The feed-forward role may be missing (a layer that is only a mixer)."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.mixer_norm = build("norm", spec.mixer_norm, ctx)
        self.mixer = build("mixer", spec.mixer, ctx)
        self.has_ff = "feed_forward" in spec.roles
        self.ffn_norm = build("norm", spec.ffn_norm, ctx) if self.has_ff else None
        self.feed_forward = build("feed_forward", spec.feed_forward, ctx) if self.has_ff else None

    def parts(self) -> dict[str, object]:
        p = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.has_ff:
            p.update(ffn_norm=self.ffn_norm, feed_forward=self.feed_forward)
        return p

    def forward(self, h, residual, step, cache, state, inject=None):
        first = residual is None
        if first:
            residual = torch.empty(h.shape, dtype=torch.float32, device=h.device)
        x = self.mixer_norm.forward(h, residual, extra=inject, first=first)
        h = self.mixer.forward(x, step, cache, state)
        if self.has_ff:
            x = self.ffn_norm.forward(h, residual)
            h = self.feed_forward.forward(x)
        return h, residual


class ParallelBlock:
    """One norm, whose output every branch reads, over a residual stream in 32-bit:
    h = norm(x); x <- x + scale * (mixer(h) + ff(h)).  The add is put off into the norm that follows (the next
    layer's, or the model's last): the block returns the branches' outputs as a ``BranchSum``.  Roles: ``norm``,
    ``mixer``, ``feed_forward`` (may be missing) and ``join`` (a ``BranchJoinSpec``: the constant ``scale``).
    ``inject``: a float32 vector added to every row of the stream before the norm."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.norm = build("norm", spec.norm, ctx)
        self.mixer = build("mixer", spec.mixer, ctx)
        self.has_ff = "feed_forward" in spec.roles
        self.feed_forward = build("feed_forward", spec.feed_forward, ctx) if self.has_ff else None
        self.scale = float(spec.roles["join"].scale) if "join" in spec.roles else 1.0

    def parts(self) -> dict[str, object]:
        p = {"norm": self.norm, "mixer": self.mixer}
        if self.has_ff:
            p["feed_forward"] = self.feed_forward
        return p

    def forward(self, h, residual, step, cache, state, inject=None):
        first = residual is None
        if first:
            rows = h.first if isinstance(h, BranchSum) else h
            residual = torch.empty(rows.shape, dtype=torch.float32, device=rows.device)
        x = self.norm.forward(h, residual, row=inject, first=first)
        a = self.mixer.forward(x, step, cache, state)
        if self.has_ff and isinstance(a, kernels.Deferred):
            # a product whose partial sums already sit in the work buffer that all such products share: the
            # feed-forward's last product would write over them, so this one is finished first
            a = kernels.ops().materialize(a)
        b = self.feed_forward.forward(x) if self.has_ff else None
        return BranchSum(a, b, self.scale), residual


class HyperBlock:
    """Pre-norm wiring over a residual stream kept as several copies in 32-bit (hyper-connections): every sublayer
    reads a weighted sum of the copies through its norm and its output comes back into all copies through its link
    (``parts.stream_link``).  Each write-back is put off into the norm that follows, so the block carries (what is
    pending, the copies [T, S, hidden]).  Roles: ``mixer_norm``, ``mixer``, ``mixer_link`` and, where the layer has a
    feed-forward, ``ffn_norm``, ``feed_forward``, ``ffn_link``."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.mixer_norm = build("norm", spec.mixer_norm, ctx)
        self.mixer = build("mixer", spec.mixer, ctx)
        self.mixer_link = build("link", spec.mixer_link, ctx)
        self.S = self.mixer_link.S
        self.has_ff = "feed_forward" in spec.roles
        self.ffn_norm = build("norm", spec.ffn_norm, ctx) if self.has_ff else None
        self.feed_forward = build("feed_forward", spec.feed_forward, ctx) if self.has_ff else None
        self.ffn_link = build("link", spec.ffn_link, ctx) if self.has_ff else None
        if self.has_ff and self.ffn_link.S != self.S:
            raise ValueError("a layer's sublayers hang on the same number of stream copies")

    def parts(self) -> dict[str, object]:
        p = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_link": self.mixer_link}
        if self.has_ff:
            p.update(ffn_norm=self.ffn_norm, feed_forward=self.feed_forward, ffn_link=self.ffn_link)
        return p

    def forward(self, h, residual, step, cache, state, inject=None):
        if inject is not None:
            raise ValueError("hyper_streams: nothing is injected into the copies of the stream")
        first = residual is None
        if first:
            rows = h.first if isinstance(h, BranchSum) else h
            residual = torch.empty((rows.shape[0], self.S, self.hidden), dtype=torch.float32, device=rows.device)
        x = self.mixer_norm.forward(h, residual, self.mixer_link, first=first)
        pending = StreamUpdate(self.mixer.forward(x, step, cache, state), self.mixer_link)
        if self.has_ff:
            x = self.ffn_norm.forward(pending, residual, self.ffn_link)
            pending = StreamUpdate(self.feed_forward.forward(x), self.ffn_link)
        return pending, residual


register("block", "pre_norm", _build_block)
register("block", "hyper_streams", lambda spec, ctx: HyperBlock(spec, ctx))
register("block", "parallel", lambda spec, ctx: ParallelBlock(spec, ctx))
register("block", "pre_norm_stream", lambda spec, ctx: StreamBlock(spec, ctx))
