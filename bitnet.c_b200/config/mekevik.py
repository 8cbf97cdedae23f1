"""Mekevik: a decoder whose layers are listed one by one in ``config.json``.

Every layer is a parallel block with two norms of the same stream, x <- x + (mixer(norm1(x)) + ffn(norm2(x))).
The mixer is attention without a softmax (a visible key weighs sigmoid(score + bias); the heads' weights are
mixed by a matrix; RMS norms over the whole query and key projections; a learned bias by log-bucketed
distance; a sliding window; values blended with those of the first blending layer; an element-wise logistic
gate on the output).  The feed-forward is a dense clamped gated unit, a mixture of SiLU-gated experts with
softmax router scores, or absent.  The keys of ``config.json``:

    architecture            "Mekevik"
    vocab, width            sizes of the embedding and the residual stream
    embedding.scale         factor on the embedding rows
    logit_scale             factor on the logits
    norm.eps                eps of every norm (also of the norms inside the mixers)
    layers[i].type          "attention"
    layers[i].mixer         heads, kv_heads, dim, vdim, scale, bias_max, mask.size, v_mix
    layers[i].mlp           null; kind "dense" with ff, limit; or kind "moe" with router.experts, router.top,
                            router.scale and expert.ff
    max_positions           (optional) the longest sequence; the design itself has no limit

Sizes that the file's tensors fix (the number of distance buckets) are read from them when the model is
loaded from a folder; a configuration without a folder names them under ``bias_buckets``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict

from .fesorax import _int, _need, _num
from .spec import (ConfigError, LimitedMlpSpec, LinearHeadSpec, ModelSpec, MoeSpec, ParallelBlockSpec, RmsNormSpec,
                   ScheduleEntry, SigmoidAttentionSpec)

ARCHITECTURE = "Mekevik"
DEFAULT_MAX_POSITIONS = 1 << 20
DEFAULT_BIAS_BUCKETS = 32  # for configurations without a folder (random weights); a folder's tables say their own
GATE_SLOPE = 1.702  # of the dense feed-forward's clamped unit
WEIGHT_EPS = 1e-20  # added to the sum the chosen experts' scores are divided by


@dataclass(frozen=True)
class MekevikConfig:
    """The file as it was read (``text``: canonical JSON, so that the record is hashable and can be
    written back unchanged) plus the checked top-level numbers."""

    text: str
    vocab: int
    width: int
    n_layers: int
    max_positions: int

    @property
    def data(self) -> Dict[str, Any]:
        return json.loads(self.text)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MekevikConfig":
        layers = _need(d, "layers", "the file")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        _num(_need(d, "embedding", "the file"), "scale", "embedding")
        if not _num(_need(d, "norm", "the file"), "eps", "norm") > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        _num(d, "logit_scale", "the file")
        mp = d.get("max_positions") or DEFAULT_MAX_POSITIONS
        cfg = cls(text=json.dumps(d, sort_keys=True), vocab=_int(d, "vocab", "the file"), width=_int(d, "width", "the file"),
                  n_layers=len(layers), max_positions=int(mp))
        cfg.to_spec()  # every layer is checked by building its spec
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return self.data

    def with_max_positions(self, max_seq: int) -> "MekevikConfig":
        if max_seq and 0 < max_seq < self.max_positions:
            d = self.data
            d["max_positions"] = int(max_seq)
            return MekevikConfig.from_dict(d)
        return self

    # ---- translation into parts ------------------------------------------------------------
    def _mixer(self, i: int, layer: Dict[str, Any], eps: float, source: Dict[str, Any]) -> SigmoidAttentionSpec:
        where = f"layers[{i}].mixer"
        m = _need(layer, "mixer", f"layers[{i}]")
        kind = _need(layer, "type", f"layers[{i}]")
        if kind != "attention":
            raise ConfigError(f"config.json: layers[{i}].type is 'attention', not {kind!r}")
        heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        dim, vdim = _int(m, "dim", where), _int(m, "vdim", where)
        mask = m.get("mask") or {}
        window = int(mask.get("size") or 0)
        if window < 0:
            raise ConfigError(f"config.json: {where}.mask.size={window} must not be negative")
        bias_max = _int(m, "bias_max", where)
        # without tables to read the number of rows from: the default, or fewer where the bias reaches less far
        buckets = int(m.get("bias_buckets") or max(2, min(DEFAULT_BIAS_BUCKETS, 2 * (bias_max - 1))))
        if buckets < 2 or bias_max <= buckets // 2:
            raise ConfigError(f"config.json: {where}.bias_max={bias_max} must exceed half the {buckets} distance buckets")
        value_mix = "none"
        if m.get("v_mix"):
            # the first layer that blends is the source of the others, whose tokens must have as many value numbers
            if not source:
                source.update(layer=i, size=kv_heads * vdim)
                value_mix = "source"
            else:
                if source["size"] != kv_heads * vdim:
                    raise ConfigError(f"config.json: {where}.v_mix: kv_heads x vdim = {kv_heads} x {vdim} = {kv_heads * vdim} numbers "
                                      f"per token, but layer {source['layer']}, whose values it blends in, has {source['size']}")
                value_mix = "blend"
        return SigmoidAttentionSpec(width=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim, v_head_dim=vdim,
                                    scale=_num(m, "scale", where), window=window, whole_norm=True, norm_eps=eps,
                                    bias_buckets=buckets, bias_max_distance=bias_max, head_bias=True, head_mix=True,
                                    value_mix=value_mix, output_gate=True)

    def _ffn(self, i: int, layer: Dict[str, Any]) -> Any:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        where = f"layers[{i}].mlp"
        kind = _need(mlp, "kind", where)
        if kind == "dense":
            limit = _num(mlp, "limit", where)
            if not limit > 0:
                raise ConfigError(f"config.json: {where}.limit={limit} must be positive")
            return LimitedMlpSpec(width=self.width, intermediate=_int(mlp, "ff", where), limit=limit, slope=GATE_SLOPE)
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind is 'dense' or 'moe', not {kind!r}")
        router, expert = _need(mlp, "router", where), _need(mlp, "expert", where)
        experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router.top={top} exceeds its {experts} experts")
        return MoeSpec(width=self.width, n_experts=experts, top=top, expert_ff=_int(expert, "ff", where + ".expert"),
                       expert_limit=0.0, weight_on_input=False, renormalise=True, scores="softmax",
                       weight_scale=_num(router, "scale", where + ".router"), renormalise_eps=WEIGHT_EPS, activation="silu")

    def to_spec(self) -> ModelSpec:
        d = self.data
        eps = float(d["norm"]["eps"])
        norm = RmsNormSpec(width=self.width, eps=eps)
        blocks, schedule = [], []
        source: Dict[str, Any] = {}
        for i, layer in enumerate(d["layers"]):
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            ffn = self._ffn(i, layer)
            blocks.append(ParallelBlockSpec(mixer=self._mixer(i, layer, eps, source), ffn=ffn, norm=norm,
                                            # without a feed-forward the second norm's gain may or may not be in the file
                                            ffn_norm=norm if ffn is not None else RmsNormSpec(width=self.width, eps=eps, optional=True)))
            schedule.append(ScheduleEntry(block=i))
        spec = ModelSpec(vocab_size=self.vocab, width=self.width, blocks=tuple(blocks), schedule=tuple(schedule),
                         final_norm=norm, max_positions=self.max_positions, embedding_scale=float(d["embedding"]["scale"]),
                         head=LinearHeadSpec(scale=float(d["logit_scale"])))
        spec.validate()
        return spec


def with_sizes_of(config: Dict[str, Any], shapes: Dict[str, Any]) -> Dict[str, Any]:
    """``config`` with the sizes that only the file's tensors fix filled in: the rows of each layer's
    distance-bias table."""
    out = json.loads(json.dumps(config))
    for i, layer in enumerate(out.get("layers") or []):
        shape = shapes.get(f"l{i}.mix.rel")
        if shape is not None and isinstance(layer, dict) and isinstance(layer.get("mixer"), dict):
            layer["mixer"]["bias_buckets"] = int(shape[0])
    return out


def tensor_name(path: str) -> str:
    """Checkpoint name of the parameter at ``path``: ``blocks.3.mixer.q`` is ``l3.mix.q``."""
    fixed = {"embedding.table": "embed", "final_norm.weight": "final.norm", "head.weight": "head"}
    if path in fixed:
        return fixed[path]
    parts = path.split(".")
    if parts[0] == "blocks" and len(parts) >= 4:
        i, role, rest = parts[1], parts[2], ".".join(parts[3:])
        if role == "norm" and rest == "weight":
            return f"l{i}.norm1"
        if role == "ffn_norm" and rest == "weight":
            return f"l{i}.norm2"
        if role == "mixer":
            return f"l{i}.mix.{rest}"
        if role == "ffn":
            return f"l{i}.mlp.{rest}"
    raise KeyError(f"the Mekevik architecture has no tensor for parameter '{path}'")
