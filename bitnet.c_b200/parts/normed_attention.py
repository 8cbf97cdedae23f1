"""Grouped-query softmax attention with normed queries and keys, projection biases, a sink, and one or two maps."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import KvRequest, Mixer, ParamSpec
from .registry import register_mixer


@register_mixer("normed_attention")
class NormedAttention(Mixer):
    """[q | k | v | gate] = W h + b in one product that leaves float32; one launch then norms queries and keys
    (RMS with a gain: per head with one gain for all heads, or over a token's whole projection), multiplies the
    queries by 1 + coef ln(floor((p + 1) / every) + 1), rounds to the compute type and writes keys and values
    into the pages; softmax over the keys the window lets through, optionally with a sink in the denominator (a
    score of 0, or a learned one per head) that has no key and no value; the head's output times the logistic
    function of its gate; output projection (with a bias).

    With two maps every head has two sets of scores over the same values: queries and keys are twice as wide,
    head by head [map 1 | map 2]; the maps run as twice the heads over twice the key heads, every two key heads
    reading one value head, and leave their sums in float32; then o = a1 - lambda a2 with
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, divided by its root mean square over the head's values,
    times 1 - diff.  The rows of the query projection are reordered when the weights are bound so that the maps
    of the heads that share a key head lie side by side, [group][map][head in group]."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "attention", "attention_prefill", "unit_norm")
    TILED_MIN_TOKENS = 16  # runs of new tokens from this many on take the tensor-core kernel (bfloat16)
    graph_safe = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        s = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads are not a multiple of {s.n_kv_heads} key/value heads")
        if s.maps not in (1, 2):
            raise ValueError(f"one or two maps of scores per head, not {s.maps}")
        if s.qk_norm not in ("none", "head", "whole") or s.sink not in ("none", "zero", "learned"):
            raise ValueError(f"qk_norm={s.qk_norm!r} / sink={s.sink!r} are not known")
        if s.maps == 2 and s.head_gate:
            raise ValueError("two maps and a gate per head are not built together")
        if not 0 < s.head_dim <= 2048 or not 0 < s.v_head_dim <= 1024:
            raise ValueError(f"head_dim={s.head_dim} (at most 2048) or v_head_dim={s.v_head_dim} (at most 1024) is not supported")
        self.per_group = s.n_heads // s.n_kv_heads
        self.q_len = s.n_heads * s.maps * s.head_dim
        self.k_len = s.n_kv_heads * s.maps * s.head_dim
        self.v_len = s.n_kv_heads * s.v_head_dim
        self.w_in: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p = {"q": ParamSpec((self.q_len, s.width)), "k": ParamSpec((self.k_len, s.width)), "v": ParamSpec((self.v_len, s.width)),
             "o": ParamSpec((s.width, s.n_heads * s.v_head_dim))}
        if s.proj_bias:
            p.update({"q.b": ParamSpec((self.q_len,)), "k.b": ParamSpec((self.k_len,)), "v.b": ParamSpec((self.v_len,))})
        if s.out_bias:
            p["o.b"] = ParamSpec((s.width,))
        if s.qk_norm == "head":
            p.update({"q.norm": ParamSpec((s.head_dim,), init="ones"), "k.norm": ParamSpec((s.head_dim,), init="ones")})
        elif s.qk_norm == "whole":
            p.update({"q.norm": ParamSpec((self.q_len,), init="ones"), "k.norm": ParamSpec((self.k_len,), init="ones")})
        if s.head_gate:
            p["g"] = ParamSpec((s.n_heads, s.width))
        if s.sink == "learned":
            p["sink"] = ParamSpec((s.n_heads,))
        if s.maps == 2:
            for name in ("lq1", "lk1", "lq2", "lk2"):
                p[name] = ParamSpec((s.head_dim,))
        return p

    def _by_group(self, t: torch.Tensor) -> torch.Tensor:
        """Rows (or numbers) of the query projection from [head][map] to [group][map][head in group]."""
        s = self.spec
        if s.maps == 1:
            return t
        rest = tuple(t.shape[1:])
        t = t.reshape((s.n_kv_heads, self.per_group, s.maps, s.head_dim) + rest).transpose(1, 2)
        return t.reshape((self.q_len,) + rest).contiguous()

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        parts = [self._by_group(tensors["q"]), tensors["k"], tensors["v"]]
        self.k_off, self.v_off = self.q_len, self.q_len + self.k_len
        at = self.v_off + self.v_len
        self.g_off = at
        if s.head_gate:
            parts.append(tensors["g"])
            at += s.n_heads
        dt = parts[0].dtype if all(t.dtype == parts[0].dtype for t in parts) else torch.float32
        pad = -at % 8  # rows of the product's result stay 16-byte aligned
        if pad:
            parts.append(torch.zeros((pad, s.width), dtype=dt, device=parts[0].device))
        # one stacked matrix: all projections of the mixer's input are one product
        self.w_in = torch.cat([t.to(dt) for t in parts], dim=0).contiguous()
        self.row = at + pad
        dev = self.w_in.device
        self.b_in = None
        if s.proj_bias:
            self.b_in = torch.zeros(self.row, dtype=torch.float32, device=dev)
            self.b_in[: self.q_len] = self._by_group(tensors["q.b"]).float()
            self.b_in[self.k_off: self.v_off] = tensors["k.b"].float()
            self.b_in[self.v_off: self.v_off + self.v_len] = tensors["v.b"].float()
        self.w_o = tensors["o"]
        self.b_o = tensors["o.b"].float().contiguous() if s.out_bias else None
        self.tail = 0
        if s.out_bias and s.maps == 2:
            # the output bias as a column of the output matrix: the kernel that combines the maps leaves a one behind
            # the heads of every row (and zeros up to a 16-byte boundary), so the product adds the bias itself
            self.tail = 8
            extra = torch.zeros((s.width, self.tail), dtype=self.w_o.dtype, device=dev)
            extra[:, 0] = tensors["o.b"].to(self.w_o.dtype)
            self.w_o = torch.cat([self.w_o, extra], dim=1).contiguous()
            self.b_o = None
        self.wq = self.wk = None
        self.q_span = self.k_span = 0
        if s.qk_norm == "head":
            self.wq, self.wk = tensors["q.norm"].float().contiguous(), tensors["k.norm"].float().contiguous()
            self.q_span = self.k_span = s.head_dim
        elif s.qk_norm == "whole":
            self.wq, self.wk = self._by_group(tensors["q.norm"]).float().contiguous(), tensors["k.norm"].float().contiguous()
            self.q_span, self.k_span = self.q_len, self.k_len
        self.sink = None
        if s.sink == "zero":
            self.sink = torch.zeros(s.n_heads * s.maps, dtype=torch.float32, device=dev)
        elif s.sink == "learned":
            self.sink = tensors["sink"].float().repeat_interleave(s.maps).contiguous() if s.maps == 1 else \
                self._sink_by_group(tensors["sink"].float())
        self.lam = 0.0
        if s.maps == 2:
            dot = lambda a, b: float((tensors[a].float() * tensors[b].float()).sum().item())
            self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + s.diff

    def _sink_by_group(self, sink: torch.Tensor) -> torch.Tensor:
        s = self.spec  # a head's sink serves both of its maps: [group][map][head in group]
        return sink.reshape(s.n_kv_heads, 1, self.per_group).expand(-1, s.maps, -1).reshape(-1).contiguous()

    def cache_request(self) -> KvRequest:
        s = self.spec
        return KvRequest(n_kv_heads=s.n_kv_heads * s.maps, head_dim=s.head_dim, window=s.window, v_head_dim=s.v_head_dim,
                         v_heads=s.n_kv_heads if s.maps > 1 else 0)

    def forward(self, h, ctx, kv, state):
        s = self.spec
        n = h.shape[0]
        dt, dev = self.build.dtype, h.device
        H, G = s.n_heads * s.maps, s.n_kv_heads * s.maps
        wide = ops.linear(h, self.w_in, out_dtype=torch.float32)
        proj = torch.empty((n, self.row), dtype=dt, device=dev)
        ops.qk_norm_append(wide, proj, ctx.tok_pos, q_len=self.q_len, k_off=self.k_off, k_len=self.k_len, bias=self.b_in,
                           q_span=self.q_span, wq=self.wq, k_span=self.k_span, wk=self.wk, eps=s.norm_eps,
                           temp_coef=s.temp_coef, temp_every=s.temp_every, v_off=self.v_off, n_kv_heads=G, head_dim=s.head_dim,
                           n_v_heads=s.n_kv_heads, v_dim=s.v_head_dim, tok_seq=ctx.tok_seq, slots=ctx.slots,
                           page_table=kv.page_table, k_cache=kv.k, v_cache=kv.v)
        if ctx.diag is not None:
            ctx.tap("attn_q", lambda: proj[:, : self.q_len])
        # two maps leave their sums unrounded for the difference that follows
        out = torch.empty((n, H * s.v_head_dim), dtype=torch.float32 if s.maps == 2 else dt, device=dev)
        gate = proj[:, self.g_off:] if s.head_gate else None
        if (dt == torch.bfloat16 and not ctx.decode and ctx.tile_seq is not None and ctx.max_new >= self.TILED_MIN_TOKENS
                and s.v_head_dim % 16 == 0 and s.head_dim % 16 == 0 and s.head_dim <= 256 and s.v_head_dim <= 256):
            # runs of new tokens: 64 tokens of a sequence and a head per block on the tensor cores, the
            # softmax weights with 16 bits of mantissa
            ops.attention_prefill(proj, self.row, out, H, G, s.head_dim, s.scale, s.window, ctx.tile_seq, ctx.tile_row0,
                                  ctx.seq_start, ctx.seq_pos0, ctx.slots, kv.page_table, kv.k, kv.v, gate=gate,
                                  gate_stride=self.row, precise=True, sink=self.sink, v_share=s.maps)
        else:
            ops.attention_general(proj, self.row, out, n, H, G, s.head_dim, s.scale, s.window, ctx.tok_seq, ctx.tok_pos,
                                  ctx.slots, kv.page_table, kv.k, kv.v, gate=gate, gate_stride=self.row, sink=self.sink,
                                  v_share=s.maps, max_keys=min(ctx.max_len, s.window) if s.window > 0 else ctx.max_len)
        if s.maps == 2:
            both = out
            out = torch.empty((n, s.n_heads * s.v_head_dim + self.tail), dtype=dt, device=dev)
            ops.diff_combine(both, out, s.n_heads, self.per_group, s.v_head_dim, self.lam, s.norm_eps, 1.0 - s.diff, tail=self.tail)
        ctx.tap("attn_out", out)
        d = ops.linear(out, self.w_o, out_dtype=torch.float32)
        if self.b_o is not None:
            d += self.b_o
        return d
