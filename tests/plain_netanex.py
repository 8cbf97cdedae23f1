"""A plain, slow statement of the Netanex decoder: one function per mechanism, NumPy float64,
whole sequences, no cache, no batching.  It shares no code with the library under test.

The design: the embedding row of a token, normed; layers x <- x + n1b(mixer(n1(x))), x <- x + n2b(ff(n2(x)))
whose four norms are RMS norms with a gain kept as its offset from one (the factor is 1 + w); three mixers
(differential attention: two softmax maps per head over the same values, the second subtracted with a
learned factor, queries growing with the logarithm of the position; attention through a cached low-rank
latent with a rotated key part shared by all heads, a sliding window, a learned sink in the softmax's
denominator and an element-wise output gate; grouped-query attention with norms over the whole query and
key projections, a one in the softmax's denominator and a gate per head); a feed-forward of SiLU-gated
experts that a table chooses by token id; a layer may run with another layer's weights; the output head
is the embedding table.

``round_fn`` rounds what a bfloat16 engine stores in bfloat16 (projections, cached rows, activations);
the stream, norms, scores, weights and angles stay unrounded, as they do there.
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
def rms(x: np.ndarray, eps: float) -> np.ndarray:
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """The layers' norm: the file holds the gain minus one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def kv_head_of(h: int, heads: int, kv_heads: int) -> int:
    return h // (heads // kv_heads)


def visible(i: int, j: int, window: int) -> bool:
    """Itself and the window - 1 positions before it (window 0: every earlier position)."""
    return 0 <= i - j and (window <= 0 or i - j < window)


def softmax_with_sink(scores: np.ndarray, sink: Optional[float]) -> np.ndarray:
    """Softmax weights of ``scores`` whose denominator also holds exp(sink): the sink has no value, so the
    weights sum to less than one."""
    top = np.max(scores) if sink is None else max(np.max(scores), sink)
    e = np.exp(scores - top)
    den = e.sum() + (0.0 if sink is None else math.exp(sink - top))
    return e / den


def query_temperature(p: int, coef: float, every: int) -> float:
    """The factor on a query at position p: it grows by steps, with the logarithm of the position."""
    return 1.0 + coef * math.log((p + 1) // every + 1)


# ---- rotary positions with the blended frequencies -----------------------------------------------
def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequencies [dims / 2], factor on cos and sin)."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x: np.ndarray, pos: np.ndarray, dims: int, base: float, scaling: Optional[dict]) -> np.ndarray:
    """x[..., :dims] rotated, number i with number i + dims / 2; x is [T, ..., n], pos [T]."""
    f, mag = yarn_frequencies(dims, base, scaling)
    shape = (len(pos),) + (1,) * (x.ndim - 2) + (dims // 2,)
    a = (np.asarray(pos, dtype=np.float64)[:, None] * f[None, :]).reshape(shape)
    c, s = np.cos(a) * mag, np.sin(a) * mag
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    out = x.copy()
    out[..., : dims // 2] = u * c - v * s
    out[..., dims // 2: dims] = v * c + u * s
    return out


# ---- mixers ------------------------------------------------------------------------------------------
def attend(q, k, v, scale, window, sink, r=_id):
    """One head: q [T, d], k [T, d], v [T, dv] -> [T, dv]; ``sink`` None, or a score in the denominator."""
    T = q.shape[0]
    seen = np.array([[visible(i, j, window) for j in range(T)] for i in range(T)])
    s = np.where(seen, (q @ k.T) * scale, -np.inf)
    top = s.max(axis=1, keepdims=True) if sink is None else np.maximum(s.max(axis=1, keepdims=True), sink)
    e = np.exp(s - top)
    den = e.sum(axis=1, keepdims=True) + (0.0 if sink is None else np.exp(sink - top))
    return (e / den) @ v


def differential_lambda(w, p, diff):
    return (math.exp(float(np.sum(w[p + "lq1"] * w[p + "lk1"]))) - math.exp(float(np.sum(w[p + "lq2"] * w[p + "lk2"]))) + diff)


def mixer_differential(h, w, p, m, eps, r=_id):
    """Two maps per head over the same values; o = a1 - lambda a2, divided by its root mean square, times
    1 - diff."""
    T = h.shape[0]
    H, G, d, dv, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], float(m["diff"])
    q = r(h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, 2, d)
    k = r(h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, 2, d)
    v = r(h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q = norm_plain(q, w[p + "q.norm"], eps)
    k = r(norm_plain(k, w[p + "k.norm"], eps))
    qt = m.get("q_temp")
    if qt:
        t = np.array([query_temperature(i, float(qt["coef"]), int(qt["every"])) for i in range(T)])
        q = q * t[:, None, None, None]
    q = r(q)
    lam = differential_lambda(w, p, diff)
    window = int((m.get("mask") or {}).get("size", 0))
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = kv_head_of(hh, H, G)
        a1 = attend(q[:, hh, 0], k[:, g, 0], v[:, g], m["scale"], window, None)
        a2 = attend(q[:, hh, 1], k[:, g, 1], v[:, g], m["scale"], window, None)
        out[:, hh] = rms(a1 - lam * a2, eps) * (1.0 - diff)
    return r(out).reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def mixer_latent(h, w, p, m, eps, r=_id):
    """Keys and values of all heads from one cached latent per token, one rotated key part for all heads."""
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    pos = np.arange(T)
    q = r(h @ w[p + "q"].T).reshape(T, H, d + dr)
    ckv = r(h @ w[p + "dkv"].T)
    c = r(norm_plain(ckv[:, :rank], w[p + "dkv.norm"], eps))
    k_rot = r(rotate_half(ckv[:, rank:], pos, int(rot["dims"]), float(rot["base"]), rot.get("scaling")))
    q_rot = r(rotate_half(q[:, :, d:], pos, int(rot["dims"]), float(rot["base"]), rot.get("scaling")))
    k_plain = r(c @ w[p + "uk"].T).reshape(T, H, d)
    val = r(c @ w[p + "uv"].T).reshape(T, H, dv)
    window = int((m.get("mask") or {}).get("size", 0))
    out = np.zeros((T, H, dv))
    for hh in range(H):
        qh = np.concatenate([q[:, hh, :d], q_rot[:, hh]], axis=1)
        kh = np.concatenate([k_plain[:, hh], k_rot], axis=1)
        out[:, hh] = attend(qh, kh, val[:, hh], m["scale"], window, float(w[p + "sink"][hh]))
    gate = sigmoid(r(h @ w[p + "g"].T))
    return r(r(out).reshape(T, H * dv) * gate) @ w[p + "o"].T


def mixer_whole_norm(h, w, p, m, eps, r=_id):
    """Norms over the whole query and key projections; a one in the softmax's denominator; a gate per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = r(norm_plain(r(h @ w[p + "q"].T + w[p + "q.b"]), w[p + "q.norm"], eps)).reshape(T, H, d)
    k = r(norm_plain(r(h @ w[p + "k"].T + w[p + "k.b"]), w[p + "k.norm"], eps)).reshape(T, G, d)
    v = r(h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    gate = sigmoid(r(h @ w[p + "g"].T))  # [T, H]
    window = int((m.get("mask") or {}).get("size", 0))
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = kv_head_of(hh, H, G)
        out[:, hh] = attend(q[:, hh], k[:, g], v[:, g], m["scale"], window, 0.0) * gate[:, hh: hh + 1]
    return r(out).reshape(T, H * dv) @ w[p + "o"].T


MIXERS = {"attention": mixer_differential, "latent_attention": mixer_latent, "attention_2": mixer_whole_norm}


# ---- feed-forward ------------------------------------------------------------------------------------
def expert(h, w, p, r=_id):
    return r(r(silu(r(h @ w[p + "gate"].T))) * r(h @ w[p + "up"].T)) @ w[p + "down"].T


def experts_by_table(h, tokens, w, p, f, r=_id):
    """Every token's experts come from a table by token id; each weighs 1 / top."""
    top = int(f["router"]["top"])
    table = np.asarray(w[p + "table"]).astype(np.int64)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t, tok in enumerate(tokens):
        for e in table[tok, :top]:
            out[t] += r(expert(h[t: t + 1], w, f"{p}e{int(e)}.", r))[0] / top
    return out


# ---- the model -----------------------------------------------------------------------------------------
def layer_prefix(cfg, i: int) -> str:
    while cfg["layers"][i].get("weights_of") is not None:
        i = int(cfg["layers"][i]["weights_of"])
    return f"l{i}."


def layer(x, tokens, w, cfg, i, r=_id):
    L = cfg["layers"][i]
    eps = float(cfg["norm"]["eps"])
    p = layer_prefix(cfg, i)
    d = MIXERS[L["type"]](r(norm_one_plus(x, w[p + "norm1"], eps)), w, p + "mix.", L["mixer"], eps, r)
    x = x + norm_one_plus(d, w[p + "norm1b"], eps)
    if L.get("mlp") is not None:
        f = experts_by_table(r(norm_one_plus(x, w[p + "norm2"], eps)), tokens, w, p + "mlp.", L["mlp"], r)
        x = x + norm_one_plus(f, w[p + "norm2b"], eps)
    return x


def forward(tokens: Sequence[int], w: Dict[str, np.ndarray], cfg: dict, r=_id, taps: Optional[List[np.ndarray]] = None):
    """Logits [T, vocab] of one whole sequence; ``taps`` collects the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = norm_one_plus(w["embed"][np.asarray(tokens)], w["embed.norm"], eps)
    for i in range(len(cfg["layers"])):
        x = layer(x, tokens, w, cfg, i, r)
        if taps is not None:
            taps.append(x.copy())
    return r(norm_one_plus(x, w["final.norm"], eps)) @ w["embed"].T
