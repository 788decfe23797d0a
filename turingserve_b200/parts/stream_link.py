"""How a sublayer hangs on a residual stream kept as several copies (hyper-connections).

The sublayer reads u = sum_s in[s] x_s; its output y comes back into all copies at once,
x_t <- sum_s mix[s, t] x_s + out[t] y (mix indexed [from, to]).  The part holds the three small tensors in
32-bit; the arithmetic happens in the norm kernel of the NEXT sublayer (``ops().hyper_norm``).  Without learned
tensors (``learned`` False) in = out = 1 and mix is the identity: with one copy that is the ordinary residual sum.
"""

from __future__ import annotations

import torch

from turingserve_b200.parts.base import BuildContext, ParamSpec, Part, register


class StreamLink(Part):
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.S = int(spec.streams)
        self.learned = bool(spec.learned)
        self.names = tuple(spec.names)
        if self.S < 1:
            raise ValueError(f"stream_link: {self.S} copies of the stream")
        self.w_in = self.w_out = self.mix = None        # None: ones / ones / identity

    def parameters(self) -> dict[str, ParamSpec]:
        if not self.learned:
            return {}
        n_in, n_out, n_mix = self.names
        return {n_in: ParamSpec((self.S,), compute_dtype=False, init="ones"),
                n_out: ParamSpec((self.S,), compute_dtype=False, init="ones"),
                n_mix: ParamSpec((self.S, self.S), compute_dtype=False, init="identity")}

    def load(self, t: dict[str, torch.Tensor]) -> None:
        if not self.learned:
            return
        n_in, n_out, n_mix = self.names
        self.w_in = t[n_in].float().contiguous()
        self.w_out = t[n_out].float().contiguous()
        self.mix = t[n_mix].float().contiguous()


register("link", "stream_link", StreamLink)
