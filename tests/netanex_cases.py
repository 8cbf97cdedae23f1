"""Small Netanex configurations and weights for the tests.

The weights are drawn here, by tensor name and shape as the design names them (not from the library's
parameter table), with scales that make faults show: after their norms queries and keys have components of
size one, so with scales of about 2 / sqrt(dim) the scores spread over several units; sinks around three, so
that a softmax without them is visibly another; gains whose stored offsets from one are of size 0.2; biases of size one
half; gates' pre-activations of size two; the four vectors behind the second map's factor large enough that
the factor is far from the constant it would be without them.  All values are exactly representable in
bfloat16, so the same folder serves both number formats.
"""
import json
import os

import numpy as np
import torch

from plain_netanex import to_bf16

# every size differs from layer to layer; two, three and one query heads on a key/value head; key and value
# widths equal in no layer; rotated parts narrower than the plain ones; a window shorter than a page; layers that
# run with another layer's weights (not in the order of their owners); a layer without a feed-forward; experts of
# which a token takes some, all, or the only one
CASE_A = {
    "architecture": "Netanex", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.5},
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 24}}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 16, "scale": 0.7, "diff": 0.35,
                                        "q_temp": {"coef": 0.8, "every": 16}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 3}, "expert": {"ff": 16}}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "scale": 0.3,
                                               "mask": {"size": 37},
                                               "rot": {"base": 10000.0, "dims": 8,
                                                       "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}},
         "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "scale": 0.3,
                                               "mask": {"size": 37},
                                               "rot": {"base": 10000.0, "dims": 8,
                                                       "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}},
         "mlp": None, "weights_of": 2},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 16, "scale": 0.7, "diff": 0.35,
                                        "q_temp": {"coef": 0.8, "every": 16}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 3}, "expert": {"ff": 16}}, "weights_of": 1},
        {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 8, "scale": 0.35},
         "mlp": {"kind": "moe", "router": {"experts": 1, "top": 1}, "expert": {"ff": 40}}},
    ],
}

# sizes that are no multiples of 8 (and mostly not of 4) anywhere: rows of no whole 16-byte pieces, so the kernels
# take their number-by-number paths and the products the library's; a rotary table without scaling; a window of
# exactly a page; queries that grow at every position; one key/value head
CASE_B = {
    "architecture": "Netanex", "vocab": 61, "width": 50, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 5, "dim": 6, "rot_dim": 6, "vdim": 7, "kv_rank": 18, "scale": 0.4,
                                               "mask": {"size": 64}, "rot": {"base": 500.0, "dims": 6}},
         "mlp": {"kind": "moe", "router": {"experts": 4, "top": 1}, "expert": {"ff": 18}}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 12, "scale": 0.15, "diff": 0.8,
                                        "q_temp": {"coef": 1.5, "every": 1}},
         "mlp": {"kind": "moe", "router": {"experts": 2, "top": 2}, "expert": {"ff": 10}}},
        {"type": "attention_2", "mixer": {"heads": 3, "kv_heads": 3, "dim": 10, "vdim": 7, "scale": 0.6},
         "mlp": None},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 12, "scale": 0.15, "diff": 0.8,
                                        "q_temp": {"coef": 1.5, "every": 1}},
         "mlp": {"kind": "moe", "router": {"experts": 2, "top": 2}, "expert": {"ff": 10}}, "weights_of": 1},
    ],
}

# key and value rows in multiples of 16 (the tensor-core kernel for runs of tokens); latent rows of 64 numbers (the
# cached rows serve it) and of 56 (per-head keys are made for it); windows that are no multiples of a page and
# shorter than the prompts; four and two query heads on a key/value head; a factor on the queries that changes
# inside a prompt
CASE_C = {
    "architecture": "Netanex", "vocab": 150, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 4, "dim": 16, "vdim": 32, "scale": 0.5, "diff": 0.5,
                                        "q_temp": {"coef": 0.4, "every": 50}},
         "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 32}}},
        {"type": "latent_attention", "mixer": {"heads": 4, "dim": 32, "rot_dim": 16, "vdim": 32, "kv_rank": 48, "scale": 0.2,
                                               "mask": {"size": 70},
                                               "rot": {"base": 100000.0, "dims": 16,
                                                       "scaling": {"factor": 2.5, "original": 128, "fast": 16.0, "slow": 0.5}}},
         "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 32}}},
        {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 1, "dim": 32, "vdim": 16, "scale": 0.35},
         "mlp": {"kind": "moe", "router": {"experts": 4, "top": 3}, "expert": {"ff": 16}}},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 16, "rot_dim": 16, "vdim": 16, "kv_rank": 40, "scale": 0.25,
                                               "mask": {"size": 150},
                                               "rot": {"base": 1000.0, "dims": 16,
                                                       "scaling": {"factor": 8.0, "original": 32, "fast": 4.0, "slow": 1.0}}},
         "mlp": None},
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 4, "dim": 16, "vdim": 32, "scale": 0.5, "diff": 0.5,
                                        "q_temp": {"coef": 0.4, "every": 50}},
         "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 32}}, "weights_of": 0},
    ],
}

CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C}


def layer_shapes(layer: dict, W: int, V: int, p: str) -> dict:
    """The tensors of one layer that owns its weights, by name."""
    m, kind = layer["mixer"], layer["type"]
    t = {p + "norm1": (W,), p + "norm1b": (W,)}
    if kind in ("attention", "attention_2"):
        maps = 2 if kind == "attention" else 1
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t.update({p + "mix.q": (H * maps * d, W), p + "mix.q.b": (H * maps * d,), p + "mix.k": (G * maps * d, W),
                  p + "mix.k.b": (G * maps * d,), p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,), p + "mix.o": (W, H * dv)})
        if kind == "attention":
            t.update({p + "mix.q.norm": (d,), p + "mix.k.norm": (d,), p + "mix.o.b": (W,)})
            t.update({p + f"mix.{n}": (d,) for n in ("lq1", "lk1", "lq2", "lk2")})
        else:
            t.update({p + "mix.q.norm": (H * d,), p + "mix.k.norm": (G * d,), p + "mix.g": (H, W)})
    else:
        H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        t.update({p + "mix.q": (H * (d + dr), W), p + "mix.dkv": (rank + dr, W), p + "mix.dkv.norm": (rank,),
                  p + "mix.uk": (H * d, rank), p + "mix.uv": (H * dv, rank), p + "mix.sink": (H,), p + "mix.g": (H * dv, W),
                  p + "mix.o": (W, H * dv)})
    mlp = layer.get("mlp")
    if mlp is not None:
        t.update({p + "norm2": (W,), p + "norm2b": (W,), p + "mlp.table": (V, mlp["router"]["top"])})
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            t.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
    return t


def tensor_shapes(cfg: dict) -> dict:
    """Every tensor of the design by name, from the configuration."""
    W, V = cfg["width"], cfg["vocab"]
    t = {"embed": (V, W), "embed.norm": (W,), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is None:
            t.update(layer_shapes(layer, W, V, f"l{i}."))
    return t


def draw_weights(cfg: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    experts = {f"l{i}.mlp.table": layer["mlp"]["router"]["experts"] for i, layer in enumerate(cfg["layers"]) if layer.get("mlp")}
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last == "table":
            out[name] = np.stack([rng.permutation(experts[name])[: shape[1]] for _ in range(shape[0])]).astype(np.int32)
            continue
        if name.endswith((".q.norm", ".k.norm", ".dkv.norm")):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last in ("norm1", "norm1b", "norm2", "norm2b", "norm"):
            a = 0.2 * rng.standard_normal(shape)  # the offset from one
        elif last == "embed":
            a = rng.standard_normal(shape)
        elif last == "sink":
            a = rng.standard_normal(shape) + 3.0  # e^3: as much as a score of twenty keys
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            a = rng.standard_normal(shape) * 0.4
        elif last == "b":
            a = rng.standard_normal(shape) * 0.5
        elif last == "g":
            a = rng.standard_normal(shape) * 2.0 / np.sqrt(shape[-1])  # inputs have unit rms: pre-activations of size 2
        elif last == "o":
            a = rng.standard_normal(shape) * 0.5 / np.sqrt(shape[-1])
        else:
            a = rng.standard_normal(shape) * 1.3 / np.sqrt(shape[-1])
        out[name] = to_bf16(np.asarray(a, dtype=np.float64))
    return out


def write_folder(folder: str, cfg: dict, weights: dict, storage: str = "bfloat16") -> str:
    from bitnet_c_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[storage]
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(n, torch.from_numpy(a) if a.dtype == np.int32 else torch.tensor(np.asarray(a, dtype=np.float32)).to(dt))
                       for n, a in weights.items()])
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return folder
