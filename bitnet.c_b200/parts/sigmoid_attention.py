"""Attention without a softmax: logistic weights that are not normalised over the keys, mixed across heads."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..csrc import ops
from ..csrc.ops import PAGE
from .base import KvRequest, Mixer, ParamSpec
from .registry import register_mixer


@register_mixer("sigmoid_attention")
class SigmoidAttention(Mixer):
    """q, k, v and the output gate's pre-activations = W h in one product; an RMS norm with a gain over the whole
    query projection and one over the whole key projection (``whole_norm``); values blended with the source
    layer's of the same tokens (``value_mix``), and that is what the cache holds; a visible key weighs
    sigmoid(q . k * scale + bias[bucket(distance)] + head bias); the heads' weights are mixed by a matrix
    (``head_mix``); every head sums the values of its own key/value head; the result times the logistic function
    of the gate's pre-activations, number by number; output projection.

    The source layer of a value group leaves its values (a view into its stacked projections) in the step's
    ``memo``; the layers that blend run after it in the same step and read the rows of the same tokens."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "unit_norm", "sigmoid_attention", "sigmoid_attention_prefill")
    graph_safe = True
    TILED_MIN_TOKENS = 16  # a sequence brings at least so many new tokens: the tensor-core kernel runs
    TILED_DECODE = True    # steps of one token per sequence take it too (where its sizes fit), pages dealt out over clusters

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads are not a multiple of {spec.n_kv_heads} key/value heads")
        if spec.value_mix not in ("none", "source", "blend"):
            raise ValueError(f"value_mix is 'none', 'source' or 'blend', not {spec.value_mix!r}")
        if not spec.whole_norm:
            raise ValueError("this mixer is built with the norms over the whole query and key projections only")
        self.w_in: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.rel: Optional[torch.Tensor] = None
        self.mix: Optional[torch.Tensor] = None
        self.blend = 0.0

    @property
    def q_dim(self) -> int:
        return self.spec.n_heads * self.spec.head_dim

    @property
    def k_dim(self) -> int:
        return self.spec.n_kv_heads * self.spec.head_dim

    @property
    def v_dim(self) -> int:
        return self.spec.n_kv_heads * self.spec.v_head_dim

    @property
    def o_dim(self) -> int:
        return self.spec.n_heads * self.spec.v_head_dim

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p = {"q": ParamSpec((self.q_dim, s.width)), "k": ParamSpec((self.k_dim, s.width)), "v": ParamSpec((self.v_dim, s.width)),
             "q.norm": ParamSpec((self.q_dim,), init="ones"), "k.norm": ParamSpec((self.k_dim,), init="ones"),
             "o": ParamSpec((s.width, self.o_dim)),
             # the blend's weight: read by the layers that blend; a file may carry it for every layer
             "vmix": ParamSpec((), optional=s.value_mix != "blend")}
        if s.bias_buckets:
            p["rel"] = ParamSpec((s.bias_buckets, s.n_heads))
        if s.head_bias:
            p["pb"] = ParamSpec((s.n_heads,))
        if s.head_mix:
            p["talk"] = ParamSpec((s.n_heads, s.n_heads))
        if s.output_gate:
            p["g"] = ParamSpec((self.o_dim, s.width))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        parts = [tensors["q"], tensors["k"], tensors["v"]]
        self.k_off, self.v_off = self.q_dim, self.q_dim + self.k_dim
        at = self.v_off + self.v_dim
        self.g_off = at
        if s.output_gate:
            parts.append(tensors["g"])
            at += self.o_dim
        dt = parts[0].dtype if all(t.dtype == parts[0].dtype for t in parts) else torch.float32
        pad = -at % 8  # rows of the product's result stay 16-byte aligned
        if pad:
            parts.append(torch.zeros((pad, s.width), dtype=dt, device=parts[0].device))
        # one stacked matrix: all projections of the mixer's input are one product
        self.w_in = torch.cat([t.to(dt) for t in parts], dim=0).contiguous()
        self.row = at + pad
        self.w_o = tensors["o"]
        self.wq, self.wk = tensors["q.norm"], tensors["k.norm"].to(tensors["q.norm"].dtype)
        dev = tensors["q"].device
        # the bias by distance instead of by bucket (row n serves distance n, the last row every longer one), with
        # the heads' own biases added in: one table holds all that is added to a scaled score
        table = None
        if s.bias_buckets:
            buckets = bias_buckets(s.bias_buckets, s.bias_max_distance).to(dev)
            table = tensors["rel"].float()[buckets]
        if s.head_bias:
            pb = tensors["pb"].float()[None, :]
            table = pb if table is None else table + pb
        self.rel = table.contiguous() if table is not None else None
        self.mix = tensors["talk"].float().contiguous() if s.head_mix else None
        if s.value_mix == "blend":
            self.blend = float(tensors["vmix"].float().item())
        self.tiled_fits = (self.build.dtype == torch.bfloat16
                           and ops.sigmoid_attention_prefill_fits(s.n_heads, s.n_kv_heads, s.head_dim, s.v_head_dim))

    def cache_request(self) -> KvRequest:
        s = self.spec
        return KvRequest(n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window, v_head_dim=s.v_head_dim)

    def forward(self, h, ctx, kv, state):
        s = self.spec
        n = h.shape[0]
        proj = ops.linear(h, self.w_in, out_dtype=self.build.dtype)
        key = ("value_mix_source", s.value_group)
        other = None
        if s.value_mix == "blend":
            other = ctx.memo.get(key)
            if other is None or other.shape[0] != n:
                raise ValueError("a layer that blends values ran without the layer whose values it blends in")
        # norms over the whole projections, the blend, and keys and values into the cache: one launch
        ops.slice_norm_append(proj, self.q_dim, self.wq, self.k_off, self.wk, self.v_off, s.n_kv_heads, s.head_dim, s.v_head_dim,
                              s.norm_eps, v_other=other, blend=self.blend, tok_seq=ctx.tok_seq, tok_pos=ctx.tok_pos,
                              slots=ctx.slots, page_table=kv.page_table, k_cache=kv.k, v_cache=kv.v)
        if s.value_mix == "source":
            ctx.memo[key] = proj[:, self.v_off: self.v_off + self.v_dim]
        if ctx.diag is not None:
            ctx.tap("attn_q", lambda: proj[:, : self.q_dim])
        out = torch.empty((n, self.o_dim), dtype=self.build.dtype, device=h.device)
        gate = proj[:, self.g_off:] if s.output_gate else None
        if self.tiled_fits and ctx.decode and self.TILED_DECODE:
            # one token per sequence: a cluster per sequence and share of its pages; a block of rows is one row
            visible = min(ctx.max_len, s.window) if s.window > 0 else ctx.max_len
            pages = -(-visible // PAGE) + 1  # a window may begin and end inside a page
            splits = max(1, min(pages, 2 * ops.n_sms(h.device) // (n * s.n_kv_heads)))
            ops.sigmoid_attention_prefill(proj, self.row, out, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window, ctx.tok_seq,
                                          None if splits > 1 else torch.zeros_like(ctx.tok_seq), ctx.seq_start, ctx.seq_pos0, ctx.slots,
                                          kv.page_table, kv.k, kv.v, rel=self.rel, mix=self.mix, gate=gate, gate_stride=self.row,
                                          splits=splits)
            ctx.tap("attn_out", out)
            return ops.linear(out, self.w_o, out_dtype=torch.float32)
        if (self.tiled_fits and not ctx.decode and ctx.tile_seq is not None and ctx.max_new >= self.TILED_MIN_TOKENS):
            ops.sigmoid_attention_prefill(proj, self.row, out, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window, ctx.tile_seq,
                                          ctx.tile_row0, ctx.seq_start, ctx.seq_pos0, ctx.slots, kv.page_table, kv.k, kv.v,
                                          rel=self.rel, mix=self.mix, gate=gate, gate_stride=self.row)
            ctx.tap("attn_out", out)
            return ops.linear(out, self.w_o, out_dtype=torch.float32)
        ops.sigmoid_attention(proj, self.row, out, n, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window, ctx.tok_seq,
                              ctx.tok_pos, ctx.slots, kv.page_table, kv.k, kv.v, rel=self.rel, mix=self.mix, gate=gate,
                              gate_stride=self.row, max_keys=min(ctx.max_len, s.window) if s.window > 0 else ctx.max_len)
        ctx.tap("attn_out", out)
        return ops.linear(out, self.w_o, out_dtype=torch.float32)


def bias_buckets(n_buckets: int, max_distance: int) -> torch.Tensor:
    """The bucket of every distance 0 .. max_distance (int64): a distance below half the number of buckets is
    its own bucket; from there on buckets widen logarithmically and the last one begins at ``max_distance`` at
    the latest.  Double precision on the host, so that a bucket's edge falls where the real logarithm puts it."""
    half = n_buckets // 2
    if n_buckets < 2 or max_distance <= half:
        raise ValueError(f"{n_buckets} distance buckets up to a distance of {max_distance} cannot be laid out")
    span = math.log(max_distance / half)
    out = [n if n < half else min(n_buckets - 1, half + int(math.floor(math.log(n / half) / span * (n_buckets - half))))
           for n in range(max_distance + 1)]
    return torch.tensor(out, dtype=torch.int64)
