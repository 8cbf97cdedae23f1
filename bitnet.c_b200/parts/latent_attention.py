"""Softmax attention through low-rank latents, with the latent itself as the cached key and value."""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from ..csrc import ops
from .base import KvRequest, Mixer, ParamSpec
from .registry import build_part, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """c_q = norm(W_dq h), q = W_uq c_q (or, without a query latent, q = W_q h), per head [plain | rotated];
    W_dkv h = [latent | rotated key part], the
    latent normed; per head k = [W_uk c | rotated part], v = W_uv c; softmax over the window, optionally with a
    learned score per head in its denominator that has no key and no value (``sink``); the head's output
    times the logistic function of its gate (one number per head, or one per output number); output projection.

    Only the normed latent c and the rotated key part are cached, as one key row [c | k_rot] of one key/value
    head, and attention runs on those rows directly: since (W_uk c) . q = c . (W_uk^T q), every head's plain
    query part is carried into the latent space first (one small product per head), the scores are
    q' . [c | k_rot] with q' = [W_uk^T q_plain | q_rot], the weighted sum of the rows' first kv_rank numbers is
    the head's output in the latent space, and W_uv brings it back (another small product per head).  The
    values are a part of the key rows, so the cache holds no value plane.

    Runs of new tokens whose key rows are too wide for the tensor-core kernel (more than 256 numbers) take the
    other order: the rows every new token sees are read back from the cache, W_uk and W_uv make per-head keys
    [W_uk c | k_rot] and values of them (two products over all those rows), which go into scratch pages of the
    step, and the tensor-core kernel runs on these with the queries as projected."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "attention", "attention_prefill", "rotary_pairs", "norm")
    TILED_MIN_TOKENS = 16  # runs of new tokens from this many on take the tensor-core kernel (bfloat16)
    graph_safe = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if min(spec.n_heads, spec.head_dim, spec.rot_dim, spec.v_head_dim, spec.kv_rank) <= 0 or spec.q_rank < 0:
            raise ValueError("latent_attention: heads, head sizes and the key/value rank must be positive")
        self.element_gate = bool(getattr(spec, "element_gate", False))
        self.has_sink = bool(getattr(spec, "sink", False))
        if self.element_gate and spec.head_gate:
            raise ValueError("latent_attention: a gate per head or a gate per output number, not both")
        if spec.kv_rank + spec.rot_dim > 2048:
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {spec.kv_rank + spec.rot_dim} must be at most 2048")
        self.position = build_part("position", spec.position, build)
        self.w_dq: Optional[torch.Tensor] = None

    def children(self):
        return {"position": self.position}

    @property
    def key_row(self) -> int:
        return self.spec.kv_rank + self.spec.rot_dim

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p = {"dkv": ParamSpec((self.key_row, s.width)), "dkv.norm": ParamSpec((s.kv_rank,), init="ones"),
             "uk": ParamSpec((s.n_heads * s.head_dim, s.kv_rank)), "uv": ParamSpec((s.n_heads * s.v_head_dim, s.kv_rank)),
             "o": ParamSpec((s.width, s.n_heads * s.v_head_dim))}
        if s.q_rank:
            p.update({"dq": ParamSpec((s.q_rank, s.width)), "dq.norm": ParamSpec((s.q_rank,), init="ones"),
                      "uq": ParamSpec((s.n_heads * (s.head_dim + s.rot_dim), s.q_rank))})
        else:
            p["q"] = ParamSpec((s.n_heads * (s.head_dim + s.rot_dim), s.width))
        if s.head_gate or self.element_gate:
            p["g"] = ParamSpec((self.gate_len, s.width))
        if self.has_sink:
            p["sink"] = ParamSpec((s.n_heads,))
        return p

    @property
    def gate_len(self) -> int:
        s = self.spec
        return s.n_heads * s.v_head_dim if self.element_gate else (s.n_heads if s.head_gate else 0)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        if s.q_rank:
            self.w_dq, self.g_dq, self.w_uq = tensors["dq"], tensors["dq.norm"], tensors["uq"]
        self.g_dkv, self.w_o = tensors["dkv.norm"], tensors["o"]
        self.sink = tensors["sink"].float().contiguous() if self.has_sink else None
        # the latent, the rotated key part, the gates and (without a query latent) the queries are one product of
        # the mixer's input
        parts = [tensors["dkv"]] + ([tensors["g"]] if self.gate_len else [])
        self.g_off = self.key_row
        at = self.key_row + self.gate_len
        if not s.q_rank:
            gap = -at % 8  # the queries start at a 16-byte boundary of the row
            if gap:
                parts.append(torch.zeros((gap, s.width), dtype=parts[0].dtype, device=parts[0].device))
            self.q_off = at + gap
            parts.append(tensors["q"])
            at = self.q_off + s.n_heads * (s.head_dim + s.rot_dim)
        dt = parts[0].dtype if all(t.dtype == parts[0].dtype for t in parts) else torch.float32
        pad = -at % 8  # rows of the product's result stay 16-byte aligned
        if pad:
            parts.append(torch.zeros((pad, s.width), dtype=dt, device=parts[0].device))
        self.w_kv = torch.cat([t.to(dt) for t in parts], dim=0).contiguous()
        self.row = at + pad
        # per head: W_uk as [dim, kv_rank] (plain query part -> latent space), W_uv as [vdim, kv_rank]
        self.w_uk = tensors["uk"].reshape(s.n_heads, s.head_dim, s.kv_rank).contiguous()
        self.w_uv = tensors["uv"].reshape(s.n_heads, s.v_head_dim, s.kv_rank).contiguous()
        self.w_uk_flat, self.w_uv_flat = tensors["uk"], tensors["uv"]

    def cache_request(self) -> KvRequest:
        s = self.spec
        return KvRequest(n_kv_heads=1, head_dim=self.key_row, window=s.window, v_head_dim=s.kv_rank, values_in_keys=True)

    def forward(self, h, ctx, kv, state):
        s = self.spec
        n = h.shape[0]
        H, d, dr, rank, row = s.n_heads, s.head_dim, s.rot_dim, s.kv_rank, self.key_row
        dt = self.build.dtype
        ckv = ops.linear(h, self.w_kv, out_dtype=dt)  # [n, latent | rotated key part | gates | (queries) | padding]
        if s.q_rank:
            cq = ops.linear(h, self.w_dq, out_dtype=dt)
            ops.rmsnorm_slices(cq, s.norm_eps, 0, s.q_rank, self.g_dq)
            q, q_off = ops.linear(cq, self.w_uq, out_dtype=dt), 0  # [n, H * (d + dr)]
        else:
            q, q_off = ckv, self.q_off
        # the latent normed, the heads' rotated query parts and the shared key part rotated, the key row [c | k_rot]
        # to the cache: one launch
        self.position.apply(ckv, ctx, xq=q, q_off=q_off, n_q_heads=H, q_head_stride=d + dr, q_rot_off=d, k_off=0, n_k_heads=1,
                            k_head_stride=row, k_rot_off=rank, k_row=row, tok_seq=ctx.tok_seq, slots=ctx.slots,
                            page_table=kv.page_table, k_cache=kv.k, norm_len=rank, norm_w=self.g_dkv, norm_eps=s.norm_eps)
        gate = ckv[:, self.g_off:] if s.head_gate else None
        egate = ckv[:, self.g_off: self.g_off + self.gate_len] if self.element_gate else None
        tiled = dt == torch.bfloat16 and not ctx.decode and ctx.tile_seq is not None and ctx.max_new >= self.TILED_MIN_TOKENS
        if q_off:
            q = q[:, q_off: q_off + H * (d + dr)]
        if (tiled and (row > 256 or row % 16 or rank % 16) and (d + dr) % 16 == 0 and s.v_head_dim % 16 == 0 and d + dr <= 256
                and s.v_head_dim <= 256 and ctx.host_new):
            return self._per_head_keys(q, gate, ctx, kv, egate)
        # queries in the latent space: [W_uk^T q_plain | q_rot] per head
        q3 = q.unflatten(1, (H, d + dr))
        ql = torch.empty((n, H, row), dtype=q.dtype, device=q.device)
        torch.bmm(q3[:, :, :d].transpose(0, 1), self.w_uk.to(q.dtype), out=ql[:, :, :rank].transpose(0, 1))
        ql[:, :, rank:] = q3[:, :, d:]
        if ctx.diag is not None:
            ctx.tap("attn_q", lambda: ql.view(n, H * row))
        out = torch.empty((n, H * rank), dtype=dt, device=h.device)
        if tiled and row % 16 == 0 and rank % 16 == 0 and row <= 256:
            # runs of new tokens: 64 tokens of a sequence and a head per block on the tensor cores, the
            # softmax weights with 16 bits of mantissa
            ops.attention_prefill(ql, H * row, out, H, 1, row, s.scale, s.window, ctx.tile_seq, ctx.tile_row0, ctx.seq_start,
                                  ctx.seq_pos0, ctx.slots, kv.page_table, kv.k, None, gate=gate, gate_stride=self.row,
                                  precise=True, v_dim=rank, sink=self.sink)
        else:
            ops.attention_general(ql, H * row, out, n, H, 1, row, s.scale, s.window, ctx.tok_seq, ctx.tok_pos, ctx.slots,
                                  kv.page_table, kv.k, None, gate=gate, gate_stride=self.row, v_dim=rank,
                                  max_keys=min(ctx.max_len, s.window) if s.window > 0 else ctx.max_len, sink=self.sink)
        ctx.tap("attn_out", out)
        # back from the latent space: W_uv per head, heads side by side
        o = torch.empty((n, H, s.v_head_dim), dtype=dt, device=h.device)
        torch.bmm(out.view(n, H, rank).transpose(0, 1), self.w_uv.to(dt).transpose(1, 2), out=o.transpose(0, 1))
        o = o.view(n, H * s.v_head_dim)
        if egate is not None:
            ops.gate_rows(o, egate)
        return ops.linear(o, self.w_o, out_dtype=torch.float32)

    def _seen_rows(self, ctx, device):
        """For this step: which cached positions its new tokens see (sequence and position of each, on the device),
        and a page table of scratch pages that holds just those, by sequence of the step and page index within the
        sequence.  The same for every layer of one window, so it is made once per step."""
        key = ("latent_attention.seen", self.spec.window)
        if key not in ctx.memo:
            w = self.spec.window
            seq, pos, spans = [], [], []
            for i, (p0, n) in enumerate(zip(ctx.host_pos0, ctx.host_new)):
                lo = max(0, p0 - w + 1) if w > 0 else 0
                seq.append(np.full(p0 + n - lo, i, dtype=np.int64))
                pos.append(np.arange(lo, p0 + n, dtype=np.int64))
                spans.append((lo // ops.PAGE, (p0 + n - 1) // ops.PAGE))
            table = np.zeros((len(spans), max(b for _a, b in spans) + 1), dtype=np.int32)
            at = 0
            for i, (a, b) in enumerate(spans):
                table[i, a:b + 1] = np.arange(at, at + b - a + 1)
                at += b - a + 1
            both = torch.from_numpy(np.stack([np.concatenate(seq), np.concatenate(pos)])).pin_memory().to(device, non_blocking=True)
            ctx.memo[key] = (both[0], both[1], torch.from_numpy(table).pin_memory().to(device, non_blocking=True), at,
                             torch.arange(len(spans), dtype=torch.int32, device=device))
        return ctx.memo[key]

    def _per_head_keys(self, q, gate, ctx, kv, egate=None):
        s = self.spec
        H, d, dr, dv, rank = s.n_heads, s.head_dim, s.rot_dim, s.v_head_dim, s.kv_rank
        dt, dev = self.build.dtype, q.device
        seq, pos, table, n_pages, rows_of = self._seen_rows(ctx, dev)
        page, r = pos // ops.PAGE, pos % ops.PAGE
        rows = kv.k[kv.page_table[ctx.slots[seq].long(), page].long(), 0, r]  # [seen, latent | rotated key part]
        c = rows[:, :rank].contiguous()
        keys = torch.empty((rows.shape[0], H, d + dr), dtype=dt, device=dev)
        keys[:, :, :d] = ops.linear(c, self.w_uk_flat, out_dtype=dt).view(-1, H, d)
        keys[:, :, d:] = rows[:, None, rank:]
        values = ops.linear(c, self.w_uv_flat, out_dtype=dt).view(-1, H, dv)
        # scratch pages start as zeros: rows of a page that no position fills are masked, and zero times them is zero
        k_s = torch.zeros((n_pages, H, ops.PAGE, d + dr), dtype=dt, device=dev)
        v_s = torch.zeros((n_pages, H, ops.PAGE, dv), dtype=dt, device=dev)
        to = table[seq, page].long()
        k_s[to, :, r] = keys
        v_s[to, :, r] = values
        out = torch.empty((q.shape[0], H * dv), dtype=dt, device=dev)
        ops.attention_prefill(q, q.stride(0), out, H, H, d + dr, s.scale, s.window, ctx.tile_seq, ctx.tile_row0, ctx.seq_start,
                              ctx.seq_pos0, rows_of, table, k_s, v_s, gate=gate, gate_stride=self.row, precise=True, sink=self.sink)
        ctx.tap("attn_out", out)
        if egate is not None:
            ops.gate_rows(out, egate)
        return ops.linear(out, self.w_o, out_dtype=torch.float32)
