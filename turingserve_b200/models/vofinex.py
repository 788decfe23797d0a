"""Vofinex: config.json keys -> ``ModelConfig``, checkpoint tensor names, and the model class.

A decoder of PARALLEL layers over a residual stream kept in 32-bit: one layer norm (weight and bias) whose
output both the mixer and the feed-forward read, x <- x + residual_mult * (mixer(h) + ff(h)).  The mixer is
grouped-query attention with keys and values of widths of their own, a rotation of q and k over their first
dimensions (pairs (i, i + dims / 2)), a per-head RMS norm of q and k without weights after it, visibility in
blocks of ``mask.size`` positions and a learned sink per head in the softmax's denominator.  The feed-forward is
a gated SiLU one, dense or routed (softmax over all router outputs, a correction that enters the choice only,
weights not renormalised, the last ``router.identity`` outputs experts that return their input), or none.
The embedding rows are multiplied by ``embedding.scale``; a span of layers (``loop``: start, stop, times) runs
several times with the same weights, every pass with memory of its own and opened by adding that pass's row of
the tensor 'loop.step' to the stream; the output head is the embedding table itself after the model's layer
norm, times ``logit_scale``.  Every size and constant comes from config.json.
"""

from __future__ import annotations

import torch

from turingserve_b200.config.model_config import (
    BranchJoinSpec, GatedMLPSpec, HalfRotarySpec, LayerRun, LayerSpec, ModelConfig, RoutedMLPSpec, SinkAttentionSpec,
    StreamLayerNormSpec)
from turingserve_b200.config.registry import (
    Architecture, LayerTensorNames, TensorNames, register_architecture)
from turingserve_b200.parts.base import BranchSum, ParamSpec
from turingserve_b200.parts.model import DecoderModel

NAME = "Vofinex"
# the rotation's angles are computed from the position itself: nothing in the design bounds a sequence
NO_POSITION_LIMIT = 1 << 30
PASS_VECTORS = "loop.step"


def _require(c: dict, key: str, where: str = "config.json"):
    if key not in c:
        raise ValueError(f"{where} is missing required key {key!r}")
    return c[key]


def _mixer(kind: str, m: dict, eps: float, where: str) -> SinkAttentionSpec:
    if kind != "attention":
        raise ValueError(f"{where}: unknown layer type {kind!r} (known: attention)")
    heads = int(_require(m, "heads", where))
    dim = int(_require(m, "dim", where))
    rot = m.get("rot") or None
    position = None
    if rot and int(rot.get("dims", 0)) > 0:
        position = HalfRotarySpec(base=float(_require(rot, "base", where)), dims=int(rot["dims"]))
    mask = m.get("mask") or None
    return SinkAttentionSpec(
        num_heads=heads, num_kv_heads=int(m.get("kv_heads", heads)), key_dim=dim, value_dim=int(m.get("vdim", dim)),
        scale=float(_require(m, "scale", where)), position=position, qk_norm_eps=eps,
        chunk=int(_require(mask, "size", where)) if mask else None, sinks=True)


FF_NAMES = ("gate", "up", "down")


def _feed_forward(f: dict | None, where: str):
    if f is None:
        return None
    kind = _require(f, "kind", where)
    if kind == "dense":
        return GatedMLPSpec(intermediate_size=int(_require(f, "ff", where)), activation="silu", names=FF_NAMES)
    if kind == "moe":
        router = _require(f, "router", where)
        return RoutedMLPSpec(
            num_experts=int(_require(router, "experts", where)), top_k=int(_require(router, "top", where)),
            intermediate_size=int(_require(_require(f, "expert", where), "ff", where)), activation="silu",
            scoring="softmax", renormalize=False, weight_on="output", gated=True, correction=True,
            identity=int(router.get("identity", 0)))
    raise ValueError(f"{where}: unknown feed-forward kind {kind!r} (known: dense, moe)")


def run_order(n_layers: int, loop: dict | None) -> tuple[LayerRun, ...]:
    """Layers before ``start`` once, layers start..stop-1 ``times`` times, the rest once; the first run of
    every pass, the first pass too, opens it (the model adds the pass's vector before it)."""
    if not loop:
        return tuple(LayerRun(i) for i in range(n_layers))
    a, b, times = int(_require(loop, "start", "loop")), int(_require(loop, "stop", "loop")), int(loop.get("times", 1))
    if not (0 <= a <= b <= n_layers) or times < 1:
        raise ValueError(f"loop {loop!r} does not fit {n_layers} layers")
    runs = [LayerRun(i) for i in range(a)]
    for p in range(times):
        runs += [LayerRun(i, opens_pass=p if i == a else None) for i in range(a, b)]
    return tuple(runs + [LayerRun(i) for i in range(b, n_layers)])


def parse_config(c: dict, gen: dict | None = None) -> ModelConfig:
    eps = float(_require(_require(c, "norm"), "eps", "norm"))
    norm = StreamLayerNormSpec(eps=eps, weight_name="", bias_name=".b")
    join = BranchJoinSpec(scale=float(c.get("residual_mult", 1.0)))
    layers = []
    for i, entry in enumerate(_require(c, "layers")):
        where = f"layers[{i}]"
        roles = dict(norm=norm, mixer=_mixer(_require(entry, "type", where), _require(entry, "mixer", where), eps, where),
                     join=join)
        ff = _feed_forward(entry.get("mlp"), where)
        if ff is not None:
            roles["feed_forward"] = ff
        layers.append(LayerSpec("parallel", **roles))
    eos = (gen or {}).get("eos_token_id", c.get("eos_token_id"))
    eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(x) for x in eos))
    loop = c.get("loop") or None
    extras = [("embedding_scale", float((c.get("embedding") or {}).get("scale", 1.0))),
              ("logit_scale", float(c.get("logit_scale", 1.0)))]
    if loop:
        extras.append(("loop", tuple(sorted(loop.items()))))
    return ModelConfig(
        architecture=NAME, hidden_size=int(_require(c, "width")), vocab_size=int(_require(c, "vocab")),
        layers=tuple(layers), schedule=run_order(len(layers), loop), final_norm=norm, tie_word_embeddings=True,
        max_position_embeddings=int(c.get("max_positions", NO_POSITION_LIMIT)), eos_token_ids=eos_ids,
        bos_token_id=c.get("bos_token_id"), extras=tuple(extras))


def tensor_names(cfg: ModelConfig) -> TensorNames:
    """'l<i>.norm1' (+ '.b'), 'l<i>.mix.<name>', 'l<i>.mlp.<name>'; 'embed', 'final.norm' (+ '.b'), 'loop.step'.
    A norm's weight is named by the prefix itself, its bias by the prefix and '.b'."""
    layers = []
    for i, spec in enumerate(cfg.layers):
        names = dict(norm=f"l{i}.norm1", mixer=f"l{i}.mix.")
        if "feed_forward" in spec.roles:
            names["feed_forward"] = f"l{i}.mlp."
        layers.append(LayerTensorNames(**names))
    return TensorNames(embedding="embed", lm_head="embed", final_norm="final.norm", layers=tuple(layers))


def to_config_json(cfg: ModelConfig) -> dict:
    layers = []
    for spec in cfg.layers:
        m = spec.mixer
        mixer = {"heads": m.num_heads, "kv_heads": m.num_kv_heads, "dim": m.key_dim, "vdim": m.value_dim, "scale": m.scale}
        if m.position is not None:
            mixer["rot"] = {"base": m.position.base, "dims": m.position.dims}
        if m.chunk:
            mixer["mask"] = {"size": m.chunk}
        entry = {"type": "attention", "mixer": mixer}
        f = spec.roles.get("feed_forward")
        if f is None:
            entry["mlp"] = None
        elif isinstance(f, GatedMLPSpec):
            entry["mlp"] = {"kind": "dense", "ff": f.intermediate_size}
        else:
            entry["mlp"] = {"kind": "moe", "expert": {"ff": f.intermediate_size},
                            "router": {"experts": f.num_experts, "top": f.top_k, "identity": f.identity}}
        layers.append(entry)
    out = {"architecture": NAME, "width": cfg.hidden_size, "vocab": cfg.vocab_size, "layers": layers,
           "norm": {"eps": cfg.final_norm.eps}, "residual_mult": cfg.layers[0].roles["join"].scale,
           "embedding": {"scale": cfg.extra("embedding_scale", 1.0)}, "logit_scale": cfg.extra("logit_scale", 1.0)}
    loop = cfg.extra("loop")
    if loop:
        out["loop"] = dict(loop)
    if cfg.max_position_embeddings != NO_POSITION_LIMIT:
        out["max_positions"] = cfg.max_position_embeddings
    if cfg.eos_token_ids:
        out["eos_token_id"] = list(cfg.eos_token_ids) if len(cfg.eos_token_ids) > 1 else cfg.eos_token_ids[0]
    return out


def make_config(*, width: int, vocab: int, layers: list[dict], eps: float = 1e-6, loop: dict | None = None,
                residual_mult: float = 1.0, embedding_scale: float = 1.0, logit_scale: float = 1.0,
                eos_token_id: int | None = None) -> ModelConfig:
    """A Vofinex ``ModelConfig`` from sizes (through the same parser as config.json); ``layers`` as the
    configuration file lists them."""
    c = {"architecture": NAME, "width": width, "vocab": vocab, "layers": layers, "norm": {"eps": eps},
         "residual_mult": residual_mult, "embedding": {"scale": embedding_scale}, "logit_scale": logit_scale}
    if loop:
        c["loop"] = loop
    if eos_token_id is not None:
        c["eos_token_id"] = eos_token_id
    return parse_config(c)


class VofinexModel(DecoderModel):
    """The decoder with what this family adds around the layers: the embedding rows enter the 32-bit stream times a
    constant (the multiplication happens in 32-bit, inside the first layer's norm kernel); every pass of the
    repeated span is opened by its own row of 'loop.step'; the logits are multiplied by a constant (folded into the final
    norm's weight and bias when they are loaded)."""

    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device, max_positions: int) -> None:
        super().__init__(cfg, dtype, device, max_positions)
        self.embedding_scale = float(cfg.extra("embedding_scale", 1.0))
        self.logit_scale = float(cfg.extra("logit_scale", 1.0))
        loop = dict(cfg.extra("loop") or ())
        # (a span without layers has no pass to open)
        self.passes = int(loop.get("times", 1)) if loop and int(loop["stop"]) > int(loop["start"]) else 0
        self.pass_vectors: torch.Tensor | None = None

    def extra_parameters(self) -> dict[str, ParamSpec]:
        if not dict(self.cfg.extra("loop") or ()):
            return {}
        times = int(dict(self.cfg.extra("loop")).get("times", 1))
        return {PASS_VECTORS: ParamSpec((times, self.cfg.hidden_size), compute_dtype=False, init="normal")}

    def load_extras(self, tensors: dict[str, torch.Tensor]) -> None:
        if PASS_VECTORS in tensors:
            self.pass_vectors = tensors[PASS_VECTORS].float().contiguous()

    def embed(self, step):
        return BranchSum(super().embed(step), None, self.embedding_scale)

    def injection(self, run, h0):
        if run.opens_pass is None or self.pass_vectors is None:
            return None
        return self.pass_vectors[run.opens_pass]

    def load(self, names, tensors) -> None:
        super().load(names, tensors)
        # the head has no bias, so the constant that multiplies the logits multiplies the final norm's output instead:
        # its 32-bit weight and bias take it once, here, and no step spends a kernel on it
        if self.logit_scale != 1.0:
            self.final_norm.weight = (self.final_norm.weight * self.logit_scale).contiguous()
            self.final_norm.bias = (self.final_norm.bias * self.logit_scale).contiguous()


register_architecture(Architecture(NAME, parse_config, tensor_names, to_config_json, build_model=VofinexModel))
