"""Gugezen: config.json keys -> ``ModelConfig``, checkpoint tensor names, and the model class.

A decoder whose layers are, in the order the configuration lists them, one of two mixers and a feed-forward or none,
pre-norm over a residual stream in 32-bit that may be kept as several copies (``streams``: hyper-connections, every
sublayer with a read vector, a write vector and a mix matrix of its own; without the key the ordinary residual sum).
``parallel``: two mixers side by side on the same input, left_scale * left + right_scale * right: grouped-query
softmax attention (biases on q, k, v; neighbouring pairs rotated with frequencies rescaled by wavelength bands; a
learned sink per head in the softmax's denominator; the heads gated by sigmoid(W_g h)) beside linear attention with a
fixed decay per head.  ``mamba2``: the selective state-space mixer with short causal filters.  Feed-forwards: dense
gated with the tanh form of GELU, or routed (softmax over all experts, the top scores renormalised, small experts
down(gelu(up(.))) with the error-function GELU, plus an expert every token uses).  Norms are RMS norms whose weights
are stored around zero (scale 1 + w).  A layer may use another layer's tensors (``weights_of``) while keeping memory
of its own.  The embedding rows are multiplied by ``embedding.scale``; the output head is the embedding table itself
after the model's norm, times ``logit_scale``.  Every size and constant comes from config.json.
"""

from __future__ import annotations

import torch

from turingserve_b200.config.model_config import (
    BandScaledRotarySpec, GatedMLPSpec, HyperRMSNormSpec, LayerRun, LayerSpec, LightningSpec, Mamba2Spec, ModelConfig,
    PairedMixerSpec, RoutedMLPSpec, SinkAttentionSpec, StreamLinkSpec)
from turingserve_b200.config.registry import (
    Architecture, LayerTensorNames, TensorNames, register_architecture)
from turingserve_b200.parts.base import BranchSum
from turingserve_b200.parts.model import DecoderModel

NAME = "Gugezen"
# the rotation's angles are computed from the position itself: nothing in the design bounds a sequence
NO_POSITION_LIMIT = 1 << 30
FF_NAMES = ("gate", "up", "down")


def _require(c: dict, key: str, where: str = "config.json"):
    if key not in c:
        raise ValueError(f"{where} is missing required key {key!r}")
    return c[key]


def _rotation(rot: dict | None, where: str):
    if not rot or int(rot.get("dims", 0)) <= 0:
        return None
    sc = rot.get("scaling") or None
    kw = {}
    if sc:
        kw = dict(factor=float(_require(sc, "factor", where)), low=float(_require(sc, "low", where)),
                  high=float(_require(sc, "high", where)), original=float(_require(sc, "original", where)))
    return BandScaledRotarySpec(base=float(_require(rot, "base", where)), dims=int(rot["dims"]), **kw)


def _mixer(kind: str, m: dict, eps: float, where: str):
    if kind == "parallel":
        a, b = _require(m, "left", where), _require(m, "right", where)
        heads, dim = int(_require(a, "heads", where)), int(_require(a, "dim", where))
        left = SinkAttentionSpec(
            num_heads=heads, num_kv_heads=int(a.get("kv_heads", heads)), key_dim=dim, value_dim=int(a.get("vdim", dim)),
            scale=float(_require(a, "scale", where)), position=_rotation(a.get("rot"), where), qk_norm_eps=None,
            sinks=True, qkv_bias=True, out_gate=True)
        rh = int(_require(b, "heads", where))
        decay = tuple(float(d) for d in _require(b, "decay", where))
        if len(decay) != rh:
            raise ValueError(f"{where}: {len(decay)} decays for {rh} heads")
        rd = int(_require(b, "dim", where))
        right = LightningSpec(num_heads=rh, key_dim=rd, value_dim=int(b.get("vdim", rd)), decays=decay, norm_eps=eps)
        return PairedMixerSpec(left=left, right=right, left_scale=float(m.get("left_scale", 1.0)),
                               right_scale=float(m.get("right_scale", 1.0)))
    if kind == "mamba2":
        heads = int(_require(m, "heads", where))
        return Mamba2Spec(num_heads=heads, head_dim=int(_require(m, "vdim", where)), state_size=int(_require(m, "state", where)),
                          num_groups=int(m.get("groups", 1)), conv_taps=int(_require(m, "conv", where)),
                          norm_groups=int(m.get("norm_groups", 1)), norm_eps=eps)
    raise ValueError(f"{where}: unknown layer type {kind!r} (known: parallel, mamba2)")


def _feed_forward(f: dict | None, where: str):
    if f is None:
        return None
    kind = _require(f, "kind", where)
    if kind == "dense":
        return GatedMLPSpec(intermediate_size=int(_require(f, "ff", where)), activation="gelu_tanh", names=FF_NAMES)
    if kind == "moe":
        router = _require(f, "router", where)
        shared = f.get("shared") or None
        return RoutedMLPSpec(
            num_experts=int(_require(router, "experts", where)), top_k=int(_require(router, "top", where)),
            intermediate_size=int(_require(_require(f, "expert", where), "ff", where)), activation="gelu",
            scoring="softmax", renormalize=True, weight_on="output",
            shared_intermediate_size=int(_require(shared, "ff", where)) if shared else None)
    raise ValueError(f"{where}: unknown feed-forward kind {kind!r} (known: dense, moe)")


def parse_config(c: dict, gen: dict | None = None) -> ModelConfig:
    eps = float(_require(_require(c, "norm"), "eps", "norm"))
    streams = c.get("streams")
    S = int(streams) if streams is not None else 1
    if S < 1:
        raise ValueError(f"streams = {S}")
    norm = HyperRMSNormSpec(eps=eps, streams=S, weight_offset=1.0, weight_name="")
    link = StreamLinkSpec(streams=S, learned=streams is not None)
    entries = _require(c, "layers")
    layers, ids, place, runs = [], [], {}, []
    for i, entry in enumerate(entries):
        where = f"layers[{i}]"
        src = entry.get("weights_of")
        if src is not None:
            src = int(src)
            if src not in place:
                raise ValueError(f"{where}: weights_of {src} must name an earlier layer with tensors of its own")
            if entry.get("type") != entries[src].get("type"):
                raise ValueError(f"{where}: uses the tensors of layer {src}, which is of another type")
            runs.append(LayerRun(place[src]))
            continue
        mixer = _mixer(_require(entry, "type", where), _require(entry, "mixer", where), eps, where)
        ff = _feed_forward(entry.get("mlp"), where)
        roles = dict(mixer=mixer, mixer_norm=norm, mixer_link=link)
        if ff is not None:
            roles.update(feed_forward=ff, ffn_norm=norm, ffn_link=link)
        place[i] = len(layers)
        ids.append(i)
        layers.append(LayerSpec("hyper_streams", **roles))
        runs.append(LayerRun(place[i]))
    eos = (gen or {}).get("eos_token_id", c.get("eos_token_id"))
    eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(x) for x in eos))
    # which entry of config.json every set of weights belongs to (its tensors are named 'l<entry>.')
    extras = (("layer_ids", tuple(ids)), ("embedding_scale", float((c.get("embedding") or {}).get("scale", 1.0))),
              ("logit_scale", float(c.get("logit_scale", 1.0))), ("streams", None if streams is None else S))
    return ModelConfig(
        architecture=NAME, hidden_size=int(_require(c, "width")), vocab_size=int(_require(c, "vocab")),
        layers=tuple(layers), schedule=tuple(runs), final_norm=norm, tie_word_embeddings=True,
        max_position_embeddings=int(c.get("max_positions", NO_POSITION_LIMIT)), eos_token_ids=eos_ids,
        bos_token_id=c.get("bos_token_id"), extras=extras)


def tensor_names(cfg: ModelConfig) -> TensorNames:
    """'l<i>.norm1', 'l<i>.mix.<name>', 'l<i>.hc1.<name>', 'l<i>.norm2', 'l<i>.mlp.<name>', 'l<i>.hc2.<name>'; 'embed',
    'final.norm'; i counts the entries of config.json's layer list, so the numbers of layers that borrow their tensors
    are skipped.  A norm's weight is named by the prefix itself."""
    ids = cfg.extra("layer_ids") or tuple(range(len(cfg.layers)))
    layers = []
    for i, spec in zip(ids, cfg.layers):
        names = dict(mixer=f"l{i}.mix.", mixer_norm=f"l{i}.norm1", mixer_link=f"l{i}.hc1.")
        if "feed_forward" in spec.roles:
            names.update(feed_forward=f"l{i}.mlp.", ffn_norm=f"l{i}.norm2", ffn_link=f"l{i}.hc2.")
        layers.append(LayerTensorNames(**names))
    return TensorNames(embedding="embed", lm_head="embed", final_norm="final.norm", layers=tuple(layers))


def _entry(spec: LayerSpec) -> dict:
    m = spec.mixer
    if isinstance(m, PairedMixerSpec):
        a, b = m.left, m.right
        left = {"heads": a.num_heads, "kv_heads": a.num_kv_heads, "dim": a.key_dim, "vdim": a.value_dim, "scale": a.scale}
        if a.position is not None:
            r = a.position
            left["rot"] = {"base": r.base, "dims": r.dims}
            if r.factor:
                left["rot"]["scaling"] = {"factor": r.factor, "low": r.low, "high": r.high, "original": r.original}
        right = {"heads": b.num_heads, "dim": b.key_dim, "vdim": b.value_dim, "decay": list(b.decays)}
        entry = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": m.left_scale,
                                               "right_scale": m.right_scale}}
    else:
        entry = {"type": "mamba2", "mixer": {"heads": m.num_heads, "vdim": m.head_dim, "state": m.state_size,
                                             "groups": m.num_groups, "conv": m.conv_taps, "norm_groups": m.norm_groups}}
    f = spec.roles.get("feed_forward")
    if f is None:
        entry["mlp"] = None
    elif isinstance(f, GatedMLPSpec):
        entry["mlp"] = {"kind": "dense", "ff": f.intermediate_size}
    else:
        entry["mlp"] = {"kind": "moe", "expert": {"ff": f.intermediate_size},
                        "router": {"experts": f.num_experts, "top": f.top_k}}
        if f.shared_intermediate_size:
            entry["mlp"]["shared"] = {"ff": f.shared_intermediate_size}
    return entry


def to_config_json(cfg: ModelConfig) -> dict:
    """The layer list in schedule order: a run of a layer that ran before borrows its tensors."""
    first_run: dict[int, int] = {}
    layers = []
    for r, run in enumerate(cfg.schedule):
        entry = _entry(cfg.layers[run.layer])
        if run.layer in first_run:
            entry["weights_of"] = first_run[run.layer]
        else:
            first_run[run.layer] = r
        layers.append(entry)
    out = {"architecture": NAME, "width": cfg.hidden_size, "vocab": cfg.vocab_size, "layers": layers,
           "norm": {"eps": cfg.final_norm.eps}, "embedding": {"scale": cfg.extra("embedding_scale", 1.0)},
           "logit_scale": cfg.extra("logit_scale", 1.0)}
    if cfg.extra("streams") is not None:
        out["streams"] = cfg.extra("streams")
    if cfg.max_position_embeddings != NO_POSITION_LIMIT:
        out["max_positions"] = cfg.max_position_embeddings
    if cfg.eos_token_ids:
        out["eos_token_id"] = list(cfg.eos_token_ids) if len(cfg.eos_token_ids) > 1 else cfg.eos_token_ids[0]
    return out


def make_config(*, width: int, vocab: int, layers: list[dict], eps: float = 1e-6, streams: int | None = None,
                embedding_scale: float = 1.0, logit_scale: float = 1.0, eos_token_id: int | None = None) -> ModelConfig:
    """A Gugezen ``ModelConfig`` from sizes (through the same parser as config.json); ``layers`` as the configuration
    file lists them."""
    c = {"architecture": NAME, "width": width, "vocab": vocab, "layers": layers, "norm": {"eps": eps},
         "embedding": {"scale": embedding_scale}, "logit_scale": logit_scale}
    if streams is not None:
        c["streams"] = streams
    if eos_token_id is not None:
        c["eos_token_id"] = eos_token_id
    return parse_config(c)


class GugezenModel(DecoderModel):
    """The decoder with what this family adds around the layers: the embedding rows, times a constant, start every copy
    of the 32-bit stream (inside the first layer's norm kernel); the model's last norm reads the sum of the copies; the
    logits are multiplied by a constant (folded into the last norm's 32-bit weight when it is loaded: the head has no
    bias)."""

    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device, max_positions: int) -> None:
        super().__init__(cfg, dtype, device, max_positions)
        self.embedding_scale = float(cfg.extra("embedding_scale", 1.0))
        self.logit_scale = float(cfg.extra("logit_scale", 1.0))

    def embed(self, step):
        return BranchSum(super().embed(step), None, self.embedding_scale)

    def finish(self, h, residual):
        return self.final_norm.forward(h, residual, None)

    def load(self, names, tensors) -> None:
        super().load(names, tensors)
        if self.logit_scale != 1.0:
            self.final_norm.weight = (self.final_norm.weight * self.logit_scale).contiguous()


register_architecture(Architecture(NAME, parse_config, tensor_names, to_config_json, build_model=GugezenModel))
