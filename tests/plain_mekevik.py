"""A plain, slow statement of the Mekevik decoder: one function per mechanism, NumPy float64,
whole sequences, no cache, no batching.  It shares no code with the library under test.

The design: a stream x that every layer reads through two RMS norms at once,
x <- x + (mixer(norm1(x)) + ff(norm2(x))); a mixer that is attention without a softmax (each visible
key weighs sigmoid(score + head bias), nothing is normalised over the keys), with one RMS norm over the
whole query projection and one over the whole key projection, a learned bias by log-bucketed distance,
a sliding window, the heads' weights mixed by a matrix, values blended with the values of the first
blending layer, and an element-wise logistic gate on the heads' outputs; a feed-forward that is a clamped
gated unit or a mixture of SiLU-gated experts with softmax router scores renormalised over the chosen ones.

``round_fn`` rounds what a bfloat16 engine stores in bfloat16 (projections, cached keys and values,
activations); the stream, norms, scores, weights and routers stay unrounded, as they do there.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np


def _id(a):
    return a


def to_bf16(a):
    """Round to the nearest bfloat16 (ties to even), returned as float64."""
    f = np.ascontiguousarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(a))


# ---- small pieces ------------------------------------------------------------------------------
def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def silu(z: np.ndarray) -> np.ndarray:
    return z * sigmoid(z)


# ---- attention mixer ---------------------------------------------------------------------------
def distance_bucket(n: int, n_buckets: int, max_distance: int) -> int:
    """Distances below half the table are their own bucket; beyond, buckets grow logarithmically up to
    ``max_distance`` and the last bucket takes the rest."""
    half = n_buckets // 2
    if n < half:
        return n
    t = math.log(n / half) / math.log(max_distance / half)
    return min(n_buckets - 1, half + int(math.floor(t * (n_buckets - half))))


def visible(i: int, j: int, window: int) -> bool:
    """Whether the query at position i sees the key at position j: itself and the window - 1 before it
    (window 0: every earlier key)."""
    return 0 <= i - j and (window <= 0 or i - j < window)


def attention_queries_keys(h, w, p, m, eps, r=_id):
    """Queries and keys after the norm over the whole projection (all heads of a token at once)."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = r(rms_norm(r(h @ w[p + "q"].T), w[p + "q.norm"], eps)).reshape(T, H, d)
    k = r(rms_norm(r(h @ w[p + "k"].T), w[p + "k.norm"], eps)).reshape(T, G, d)
    return q, k


def attention_values(h, w, p, m, v_first, r=_id):
    """Values [T, G, vdim]; blended with the first blending layer's when ``v_first`` is given."""
    T = h.shape[0]
    v = r(h @ w[p + "v"].T).reshape(T, m["kv_heads"], m["vdim"])
    if v_first is not None:
        lam = float(w[p + "vmix"])
        v = r((1.0 - lam) * v + lam * v_first.reshape(v.shape))  # number by number over all heads
    return v


def attention_weights(q, k, w, p, m):
    """[H, T, T]: sigmoid(q.k * scale + bias by distance + head bias) on visible keys, 0 elsewhere; then
    the heads' weights mixed: weight_h <- sum_g talk[h, g] weight_g."""
    T, H, _ = q.shape
    G = k.shape[1]
    rel = w[p + "rel"]
    B = rel.shape[0]
    window = int((m.get("mask") or {}).get("size", 0))
    bucket_of = np.array([distance_bucket(n, B, m["bias_max"]) for n in range(T)])
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = np.array([[visible(a, b, window) for b in range(T)] for a in range(T)]) if T <= 48 else \
        (i - j >= 0) & ((window <= 0) | (i - j < window))
    a = np.zeros((H, T, T))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] + rel[bucket_of[np.maximum(i - j, 0)], hd] + w[p + "pb"][hd]
        a[hd] = np.where(seen, sigmoid(np.where(seen, s, 0.0)), 0.0)
    return np.einsum("hg,gij->hij", w[p + "talk"], a)


def attention_mixer(h, w, p, m, eps, v_first, r=_id):
    """h [T, width] -> ([T, width], the values this layer caches)."""
    T = h.shape[0]
    H, G, dv = m["heads"], m["kv_heads"], m["vdim"]
    q, k = attention_queries_keys(h, w, p, m, eps, r)
    v = attention_values(h, w, p, m, v_first, r)
    a = attention_weights(q, k, w, p, m)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        out[:, hd] = a[hd] @ v[:, hd // (H // G)]
    gate = sigmoid(r(h @ w[p + "g"].T))
    out = r(out.reshape(T, H * dv) * gate)
    return r(out @ w[p + "o"].T), v


# ---- feed-forwards -----------------------------------------------------------------------------
def dense_ffn(h, w, p, mlp, r=_id):
    """down(g * sigmoid(1.702 g) * (u + 1)), g = min(gate h, limit), u = clamp(up h, -limit, limit)."""
    lim = mlp["limit"]
    g = np.minimum(r(h @ w[p + "gate"].T), lim)
    u = np.clip(r(h @ w[p + "up"].T), -lim, lim)
    return r(r(g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T)


def router(h, w, p, mlp):
    """Per token the chosen experts and their weights: softmax over all experts, the ``top`` largest,
    their scores divided by their sum (+ 1e-20) times the router's scale."""
    ro = mlp["router"]
    z = h @ w[p + "router"].T
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    s = e / e.sum(axis=-1, keepdims=True)
    ids = np.argsort(-s, axis=-1, kind="stable")[:, : ro["top"]]
    chosen = np.take_along_axis(s, ids, axis=-1)
    return ids, chosen / (chosen.sum(axis=-1, keepdims=True) + 1e-20) * ro["scale"]


def expert(h, w, p, r=_id):
    """down(silu(gate h) * (up h))."""
    return r(r(silu(r(h @ w[p + "gate"].T)) * r(h @ w[p + "up"].T)) @ w[p + "down"].T)


def router_margins(h, w, p, mlp):
    """Per token how far the last chosen expert's logit lies above the first one left out (inf when all are chosen)."""
    z = np.sort(h @ w[p + "router"].T, axis=-1)[:, ::-1]
    top = mlp["router"]["top"]
    return z[:, top - 1] - z[:, top] if top < z.shape[1] else np.full(h.shape[0], np.inf)


def moe_ffn(h, w, p, mlp, r=_id):
    ids, weights = router(h, w, p, mlp)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t], weights[t]):
            out[t] += wt * expert(h[t:t + 1], w, f"{p}e{e}.", r)[0]
    return out


# ---- the model ---------------------------------------------------------------------------------
def forward(cfg: Dict, w: Dict[str, np.ndarray], tokens: Sequence[int], round_fn=_id, layers_out: Optional[List] = None,
            margins_out: Optional[List] = None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the stream after every layer;
    ``margins_out``: one that receives every router's margins per token."""
    r = round_fn
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        m, mlp = layer["mixer"], layer.get("mlp")
        p = f"l{i}."
        h1 = r(rms_norm(x, w[p + "norm1"], eps))
        blend = bool(m.get("v_mix"))
        d, v = attention_mixer(h1, w, p + "mix.", m, eps, v_first if blend else None, r)
        if blend and v_first is None:
            v_first = v
        if mlp is not None:
            h2 = r(rms_norm(x, w[p + "norm2"], eps))
            if margins_out is not None and mlp["kind"] == "moe":
                margins_out.append(router_margins(h2, w, p + "mlp.", mlp))
            d = d + (dense_ffn(h2, w, p + "mlp.", mlp, r) if mlp["kind"] == "dense" else moe_ffn(h2, w, p + "mlp.", mlp, r))
        x = x + d
        if layers_out is not None:
            layers_out.append(x.copy())
    h = r(rms_norm(x, w["final.norm"], eps))
    return (h @ w["head"].T) * cfg["logit_scale"]
