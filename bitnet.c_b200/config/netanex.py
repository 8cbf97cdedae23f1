"""Netanex: a decoder whose layers are listed one by one in ``config.json``.

The embedding row of a token is normed; every layer is a block with a norm before and after each sublayer,
x <- x + n1b(mixer(n1(x))), x <- x + n2b(ffn(n2(x))), all four RMS norms with a gain kept as its offset from one
(the factor is 1 + w).  Three mixers: ``attention`` (grouped-query attention with two maps of scores per
head over the same values, the second subtracted with a learned factor; queries and keys normed per head and
map; queries that grow with the logarithm of the position; biases on all four projections), ``attention_2``
(grouped-query attention with norms over the whole query and key projections, a one in the softmax's
denominator, a logistic gate per head, biases on the query, key and value projections) and
``latent_attention`` (keys and values of all heads from one cached normed latent per token plus one rotated
key part shared by all heads, rotary positions with blended frequencies in the halves pairing, a sliding
window, a learned sink per head in the softmax's denominator, a logistic gate on every output number).  The
feed-forward is a mixture of SiLU-gated experts that a table chooses by token id, each with weight 1 / top,
or absent.  A layer may run with the weights of an earlier one and a cache of its own.  The output head is
the embedding table.  The keys of ``config.json``:

    architecture            "Netanex"
    vocab, width            sizes of the embedding and the residual stream
    norm.eps                eps of every norm (also of the norms inside the mixers)
    layers[i].type          "attention" | "attention_2" | "latent_attention"
    layers[i].mixer         attention: heads, kv_heads, dim, vdim, scale, diff, q_temp.coef / every, mask.size
                            attention_2: heads, kv_heads, dim, vdim, scale, mask.size
                            latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, mask.size,
                            rot.base / dims / scaling.factor / original / fast / slow
    layers[i].mlp           null, or kind "moe" with router.experts, router.top and expert.ff
    layers[i].weights_of    (optional) the layer whose tensors this one uses
    max_positions           (optional) the longest sequence; the design itself has no limit
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict

from .fesorax import _int, _need, _num
from .spec import (ConfigError, LatentAttentionSpec, LinearHeadSpec, ModelSpec, MoeSpec, NormedAttentionSpec, RmsNormSpec,
                   RotaryBlendSpec, SandwichBlockSpec, ScheduleEntry)

ARCHITECTURE = "Netanex"
DEFAULT_MAX_POSITIONS = 1 << 20
MAGNITUDE_SLOPE = 0.1  # cos and sin of the blended rotary table are multiplied by this * ln(factor) + 1
MIXERS = ("attention", "attention_2", "latent_attention")


@dataclass(frozen=True)
class NetanexConfig:
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
    def from_dict(cls, d: Dict[str, Any]) -> "NetanexConfig":
        layers = _need(d, "layers", "the file")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        if not _num(_need(d, "norm", "the file"), "eps", "norm") > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        mp = d.get("max_positions") or DEFAULT_MAX_POSITIONS
        cfg = cls(text=json.dumps(d, sort_keys=True), vocab=_int(d, "vocab", "the file"), width=_int(d, "width", "the file"),
                  n_layers=len(layers), max_positions=int(mp))
        cfg.to_spec()  # every layer is checked by building its spec
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return self.data

    def with_max_positions(self, max_seq: int) -> "NetanexConfig":
        if max_seq and 0 < max_seq < self.max_positions:
            d = self.data
            d["max_positions"] = int(max_seq)
            return NetanexConfig.from_dict(d)
        return self

    # ---- translation into parts ------------------------------------------------------------
    @staticmethod
    def _window(m: Dict[str, Any], where: str) -> int:
        window = int((m.get("mask") or {}).get("size") or 0)
        if window < 0:
            raise ConfigError(f"config.json: {where}.mask.size={window} must not be negative")
        return window

    def _grouped(self, m: Dict[str, Any], where: str):
        heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        return heads, kv_heads

    def _mixer(self, i: int, layer: Dict[str, Any], eps: float) -> Any:
        where = f"layers[{i}].mixer"
        m = _need(layer, "mixer", f"layers[{i}]")
        kind = _need(layer, "type", f"layers[{i}]")
        if kind == "attention":
            heads, kv_heads = self._grouped(m, where)
            temp = m.get("q_temp") or None
            diff = _num(m, "diff", where)
            return NormedAttentionSpec(width=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=_int(m, "dim", where),
                                       v_head_dim=_int(m, "vdim", where), scale=_num(m, "scale", where),
                                       window=self._window(m, where), qk_norm="head", norm_eps=eps, proj_bias=True, out_bias=True,
                                       temp_coef=_num(temp, "coef", where + ".q_temp") if temp else 0.0,
                                       temp_every=_int(temp, "every", where + ".q_temp") if temp else 0, maps=2, diff=diff)
        if kind == "attention_2":
            heads, kv_heads = self._grouped(m, where)
            return NormedAttentionSpec(width=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=_int(m, "dim", where),
                                       v_head_dim=_int(m, "vdim", where), scale=_num(m, "scale", where),
                                       window=self._window(m, where), qk_norm="whole", norm_eps=eps, proj_bias=True,
                                       sink="zero", head_gate=True)
        if kind == "latent_attention":
            rot = _need(m, "rot", where)
            rot_dim = _int(m, "rot_dim", where)
            dims = _int(rot, "dims", where + ".rot")
            if dims > rot_dim or dims % 2:  # the first rot.dims numbers of the rotated part turn, the rest pass unchanged
                raise ConfigError(f"config.json: {where}.rot.dims={dims} must be even and at most rot_dim={rot_dim}")
            sc = rot.get("scaling") or None
            position = RotaryBlendSpec(dims=dims, base=_num(rot, "base", where + ".rot"),
                                       factor=_num(sc, "factor", where + ".rot.scaling") if sc else 1.0,
                                       original=_num(sc, "original", where + ".rot.scaling") if sc else 0.0,
                                       fast=_num(sc, "fast", where + ".rot.scaling") if sc else 32.0,
                                       slow=_num(sc, "slow", where + ".rot.scaling") if sc else 1.0,
                                       magnitude_slope=MAGNITUDE_SLOPE, pairing="halves")
            return LatentAttentionSpec(width=self.width, n_heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
                                       rot_dim=rot_dim, v_head_dim=_int(m, "vdim", where), q_rank=0,
                                       kv_rank=_int(m, "kv_rank", where), scale=_num(m, "scale", where), position=position,
                                       norm_eps=eps, window=self._window(m, where), head_gate=False, element_gate=True, sink=True)
        raise ConfigError(f"config.json: layers[{i}].type is one of {', '.join(MIXERS)}, not {kind!r}")

    def _ffn(self, i: int, layer: Dict[str, Any]) -> Any:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        where = f"layers[{i}].mlp"
        kind = _need(mlp, "kind", where)
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind is 'moe', not {kind!r}")
        router, expert = _need(mlp, "router", where), _need(mlp, "expert", where)
        experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router.top={top} exceeds its {experts} experts")
        return MoeSpec(width=self.width, n_experts=experts, top=top, expert_ff=_int(expert, "ff", where + ".expert"),
                       expert_limit=0.0, weight_on_input=False, scores="table", table_rows=self.vocab, activation="silu")

    def to_spec(self) -> ModelSpec:
        d = self.data
        eps = float(d["norm"]["eps"])
        norm = RmsNormSpec(width=self.width, eps=eps, one_plus=True)
        blocks, schedule = [], []
        block_of: Dict[int, int] = {}  # layer that owns tensors -> its block
        for i, layer in enumerate(d["layers"]):
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            # built (and so checked) for every layer, also for one that runs with another's weights
            ffn = self._ffn(i, layer)
            block = SandwichBlockSpec(mixer=self._mixer(i, layer, eps), ffn=ffn, mixer_norm=norm, mixer_post_norm=norm,
                                      ffn_norm=norm if ffn is not None else None,
                                      ffn_post_norm=norm if ffn is not None else None, label=str(i))
            j = layer.get("weights_of")
            if j is None:
                block_of[i] = len(blocks)
                blocks.append(block)
                schedule.append(ScheduleEntry(block=block_of[i]))
                continue
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
                raise ConfigError(f"config.json: layers[{i}].weights_of={j!r} must name an earlier layer")
            while d["layers"][j].get("weights_of") is not None:  # a layer that itself runs with another's weights
                j = d["layers"][j]["weights_of"]
            other = blocks[block_of[j]]
            if (block.mixer, block.ffn) == (other.mixer, other.ffn):
                schedule.append(ScheduleEntry(block=block_of[j]))  # the same block once more, with a cache of its own
                continue
            if d["layers"][j]["type"] != layer["type"] or (ffn is None) != (other.ffn is None):
                raise ConfigError(f"config.json: layers[{i}] uses the weights of layer {j} but is of another kind than that layer")
            # the same tensors under other constants (a window, a scale): a block of its own whose parameters carry the
            # owner's tensor names, so the file's tensors are read once and bound to both (sizes that do not fit the
            # owner's tensors show when the weights are loaded)
            schedule.append(ScheduleEntry(block=len(blocks)))
            blocks.append(SandwichBlockSpec(mixer=block.mixer, ffn=block.ffn, mixer_norm=norm, mixer_post_norm=norm,
                                            ffn_norm=block.ffn_norm, ffn_post_norm=block.ffn_post_norm, label=f"{j}@{i}"))
        spec = ModelSpec(vocab_size=self.vocab, width=self.width, blocks=tuple(blocks), schedule=tuple(schedule),
                         final_norm=norm, max_positions=self.max_positions, tie_embeddings=True, embedding_norm=norm,
                         head=LinearHeadSpec())
        spec.validate()
        return spec


def tensor_name(path: str) -> str:
    """Checkpoint name of the parameter at ``path``: ``blocks.3.mixer.q`` is ``l3.mix.q`` (the block's label is
    the number of the layer that owns the tensors)."""
    fixed = {"embedding.table": "embed", "embedding_norm.weight": "embed.norm", "final_norm.weight": "final.norm"}
    if path in fixed:
        return fixed[path]
    parts = path.split(".")
    if parts[0] == "blocks" and len(parts) >= 4:
        i, role, rest = parts[1].split("@")[0], parts[2], ".".join(parts[3:])  # "j@i": layer i's block on layer j's tensors
        norms = {"mixer_norm": "norm1", "mixer_post_norm": "norm1b", "ffn_norm": "norm2", "ffn_post_norm": "norm2b"}
        if role in norms and rest == "weight":
            return f"l{i}.{norms[role]}"
        if role == "mixer":
            return f"l{i}.mix.{rest}"
        if role == "ffn":
            return f"l{i}.mlp.{rest}"
    raise KeyError(f"the Netanex architecture has no tensor for parameter '{path}'")
