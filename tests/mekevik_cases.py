"""Small Mekevik configurations and weights for the tests.

The weights are drawn here, by tensor name and shape as the design names them (not from the library's
parameter table), with scales that make faults show: after the norms over the whole projections queries and
keys have components of size one, so with scales of 2 / sqrt(dim) the scores spread over several units and the
logistic weights over their whole range; biases by distance and per head of order one; mixing matrices that are
far from the identity; blends between 0.2 and 0.8; gates' pre-activations of size two.  All values are exactly
representable in bfloat16, so the same folder serves both number formats.
"""
import json
import os

import numpy as np
import torch

from plain_mekevik import to_bf16

# every size differs from layer to layer; two, three and one query heads on a key/value head; key and value
# widths equal in no layer; a window shorter than a page, one of exactly a page, one longer than the prompts, one
# of a single position; blending from the first layer on, with a layer in between that does not blend; a dense
# feed-forward, experts of which a token takes some, experts of which it takes all, and none
CASE_A = {
    "architecture": "Mekevik", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "logit_scale": 0.5,
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.5, "bias_max": 30,
                                        "mask": {"size": 37}, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 40, "limit": 1.5}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 24, "scale": 0.7, "bias_max": 50,
                                        "mask": {"size": 64}, "v_mix": True},
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2, "scale": 0.7}, "expert": {"ff": 24}}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 8, "scale": 0.35, "bias_max": 9,
                                        "mask": {"size": 1000}, "v_mix": False},
         "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 24, "scale": 0.7, "bias_max": 20,
                                        "mask": {"size": 1}, "v_mix": True},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 3, "scale": 1.5}, "expert": {"ff": 16}}},
    ],
}
BUCKETS_A = {0: 16, 1: 32, 2: 8, 3: 6}  # layer -> rows of its distance-bias table

# sizes that are no multiples of 8 (and in one layer of 4) anywhere: rows of no whole 16-byte pieces, so the
# kernels take their number-by-number paths and the products the library's; the first layer does not blend, so
# the source of the blend is not layer 0; one expert of one; a mixer without a mask (every earlier key)
CASE_B = {
    "architecture": "Mekevik", "vocab": 61, "width": 50, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
    "layers": [
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 10, "vdim": 12, "scale": 0.6, "bias_max": 40,
                                        "mask": {"size": 30}},
         "mlp": {"kind": "moe", "router": {"experts": 1, "top": 1, "scale": 2.0}, "expert": {"ff": 18}}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 20, "vdim": 7, "scale": 0.45, "bias_max": 12,
                                        "mask": {"size": 23}, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 18, "limit": 0.75}},
        {"type": "attention", "mixer": {"heads": 5, "kv_heads": 1, "dim": 6, "vdim": 7, "scale": 0.8, "bias_max": 100,
                                        "v_mix": True},
         "mlp": {"kind": "dense", "ff": 10, "limit": 3.0}},
    ],
}
BUCKETS_B = {0: 10, 1: 4, 2: 20}

# key and value rows in multiples of 16, four and two query heads on a key/value head, windows shorter than the
# prompts that are no multiples of a page, more tokens than a window in one step
CASE_C = {
    "architecture": "Mekevik", "vocab": 150, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0}, "logit_scale": 0.25,
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.35, "bias_max": 60,
                                        "mask": {"size": 70}, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 64, "limit": 2.0}},
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.5, "bias_max": 120,
                                        "mask": {"size": 150}, "v_mix": True},
         "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2, "scale": 1.0}, "expert": {"ff": 32}}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 32, "scale": 0.25, "bias_max": 30,
                                        "mask": {"size": 33}, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 32, "limit": 1.0}},
    ],
}
BUCKETS_C = {0: 32, 1: 32, 2: 16}

CASES = {"A": (CASE_A, BUCKETS_A), "B": (CASE_B, BUCKETS_B), "C": (CASE_C, BUCKETS_C)}


def tensor_shapes(cfg: dict, buckets: dict) -> dict:
    """Every tensor of the design by name, from the configuration (and the rows that only the tensors fix)."""
    W, V = cfg["width"], cfg["vocab"]
    t = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = (W,)
        t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = (H * d, W), (G * d, W), (G * dv, W)
        t[p + "mix.q.norm"], t[p + "mix.k.norm"] = (H * d,), (G * d,)
        t[p + "mix.rel"], t[p + "mix.pb"], t[p + "mix.talk"] = (buckets[i], H), (H,), (H, H)
        t[p + "mix.vmix"] = ()
        t[p + "mix.g"], t[p + "mix.o"] = (H * dv, W), (W, H * dv)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        t[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = (mlp["ff"], W), (mlp["ff"], W), (W, mlp["ff"])
        else:
            t[p + "mlp.router"] = (mlp["router"]["experts"], W)
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                t[p + f"mlp.e{e}.gate"], t[p + f"mlp.e{e}.up"], t[p + f"mlp.e{e}.down"] = (ff, W), (ff, W), (W, ff)
    return t


def draw_weights(cfg: dict, buckets: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, buckets).items():
        last = name.split(".")[-1]
        if last in ("norm1", "norm2", "norm"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "embed":
            a = rng.standard_normal(shape)
        elif last == "rel":
            a = rng.standard_normal(shape)
        elif last == "pb":
            a = rng.standard_normal(shape) - 1.5  # most weights well below a half: sums over a window stay of order one
        elif last == "talk":
            a = np.eye(shape[0]) * 0.6 + 0.4 * rng.standard_normal(shape)
        elif last == "vmix":
            a = np.asarray(rng.uniform(0.2, 0.8))
        elif last in ("g", "router"):
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
                      [(n, torch.tensor(np.asarray(a, dtype=np.float32)).to(dt)) for n, a in weights.items()])  # a blend's weight keeps its shape ()
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return folder
