"""Mixture of gated experts: logistic or softmax router scores, clamped or plain gated units."""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from ..csrc import ops
from .base import FeedForward, ParamSpec
from .registry import register_ffn


@register_ffn("moe")
class Moe(FeedForward):
    """Router logits in float32; each token takes its ``top`` experts with the largest scores
    s = sigmoid(z) and weights them by s; the weight multiplies the expert's input
    (``weight_on_input``) or its output.  An expert is down(g * sigmoid(slope g) * (u + 1)) with
    g = min(gate x, limit), u = clamp(up x, -limit, limit); a shared expert of the same form (sizes and
    limit of its own) runs for every token and is added.  By the spec: ``scores`` "softmax" takes the softmax
    over all experts as scores; ``renormalise`` divides the chosen ones' by their sum (+ ``renormalise_eps``);
    ``weight_scale`` multiplies the weights; ``activation`` "silu" / "gelu_tanh" makes an expert
    down(act(gate x) * (up x)) without clamps; ``scores`` "table": no router, a table of expert ids by token id
    chooses and every chosen expert weighs 1 / top.

    Few rows (a decode step): two kernels stream the chosen experts once per (token, expert), from
    device memory alone.  Many rows: the (token, expert) items are sorted by expert and every expert's
    rows go through the ordinary products; the host then needs the experts' row counts, one copy per call."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "act", "moe")
    graph_safe = True  # the steps that are recorded are decode steps, which take the path without the host
    FEW_ITEMS = 64  # up to so many (token, expert) items the streaming kernels run
    PAD_FACTOR = 2.0  # blocks of equal size for all experts while they hold at most so many times the rows used

    def __init__(self, spec, build):
        super().__init__(spec, build)
        scores, activation = getattr(spec, "scores", "sigmoid"), getattr(spec, "activation", "limited")
        if scores not in ("sigmoid", "softmax", "table"):
            raise ValueError(f"router scores are 'sigmoid', 'softmax' or 'table', not {scores!r}")
        self.by_table = scores == "table"
        if self.by_table and (getattr(spec, "table_rows", 0) <= 0 or spec.shared_ff or spec.weight_on_input):
            raise ValueError("experts chosen by a table need its number of rows, weigh their outputs and have no shared expert")
        if activation != "limited" and activation not in ops.ACTIVATIONS:
            raise ValueError(f"expert activation {activation!r} is not built; known: limited, {', '.join(sorted(ops.ACTIVATIONS))}")
        self.softmax = scores == "softmax"
        self.act = -1 if activation == "limited" else ops.ACTIVATIONS[activation]  # -1: the clamped unit
        # experts too wide for the streaming kernels' shared memory always take the sorted path, which asks the
        # device for the experts' counts: such a model's steps are not recorded
        self.few_fits = ops.moe_few_fits(spec.width, spec.top, spec.expert_ff)
        self.graph_safe = self.few_fits

    def _activate(self, gate_up, out, limit):
        if self.act < 0:
            return ops.glu_limited(gate_up, out, limit, self.spec.slope)
        return ops.glu_halves(gate_up, out, self.act)

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        if self.by_table:  # token id -> the ids of its experts, different within a row
            p = {"table": ParamSpec((s.table_rows, s.top), init="distinct", integer=True, high=s.n_experts)}
        else:
            p = {"router": ParamSpec((s.n_experts, s.width))}
        for e in range(s.n_experts):
            p[f"e{e}.gate"] = ParamSpec((s.expert_ff, s.width))
            p[f"e{e}.up"] = ParamSpec((s.expert_ff, s.width))
            p[f"e{e}.down"] = ParamSpec((s.width, s.expert_ff))
        if s.shared_ff:
            p["shared.gate"] = ParamSpec((s.shared_ff, s.width))
            p["shared.up"] = ParamSpec((s.shared_ff, s.width))
            p["shared.down"] = ParamSpec((s.width, s.shared_ff))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        dt = self.build.dtype
        self.w_router = tensors.get("router")
        self.table = tensors.get("table")
        # the table on the host too: how many tokens of a step take each expert is then known without asking the device
        self.table_host = self.table.cpu().numpy() if self.table is not None else None
        # [experts, 2 ff, width]: an expert's gate rows, then its up rows; [experts, width, ff]
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"].to(dt), tensors[f"e{e}.up"].to(dt)], dim=0)
                                      for e in range(s.n_experts)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"].to(dt) for e in range(s.n_experts)]).contiguous()
        if s.shared_ff:
            self.w_shared_gate_up = torch.cat([tensors["shared.gate"].to(dt), tensors["shared.up"].to(dt)], dim=0).contiguous()
            self.w_shared_down = tensors["shared.down"]

    def _expert(self, x, w_gate_up, w_down, limit, out_dtype):
        gu = ops.linear(x, w_gate_up, out_dtype=self.build.dtype)
        act = torch.empty((x.shape[0], gu.shape[1] // 2), dtype=gu.dtype, device=gu.device)
        self._activate(gu, act, limit)
        return ops.linear(act, w_down, out_dtype=out_dtype)

    def forward(self, h, ctx):
        s = self.spec
        T = h.shape[0]
        shared = self._expert(h, self.w_shared_gate_up, self.w_shared_down, s.shared_limit, torch.float32) if s.shared_ff else None
        if self.by_table:
            # the choice depends on the step's token ids alone: runs that share a table share its rows of the step
            key = ("moe.table", self.table.data_ptr(), s.top)
            if key not in ctx.memo:
                ctx.memo[key] = ops.moe_table_route(ctx.tokens, self.table, s.top, s.n_experts)
            ids, weights = ctx.memo[key]
        else:
            ids, weights = ops.moe_route(h, self.w_router, s.top, s.renormalise, softmax=self.softmax,
                                         weight_scale=getattr(s, "weight_scale", 1.0), sum_eps=getattr(s, "renormalise_eps", 0.0))
        if ctx.diag is not None:
            ctx.tap("moe_ids", lambda: ids.float())
        if self.few_fits and (ctx.decode or T * s.top <= self.FEW_ITEMS):
            return ops.moe_experts_few(h, ids, weights, self.w_gate_up, self.w_down, s.expert_limit, s.slope,
                                       s.weight_on_input, add=shared, act=self.act)
        counts = ops.moe_count(ids, s.n_experts)
        host_tokens = getattr(ctx, "host_tokens", None)
        if self.by_table and host_tokens is not None:
            # chosen by token id: the counts follow from the step's ids on the host, nobody waits for the device
            ckey = ("moe.table.counts", self.table.data_ptr(), s.top)
            if ckey not in ctx.memo:
                rows = self.table_host.shape[0]
                chosen = self.table_host[np.clip(host_tokens, 0, rows - 1), : s.top]
                known = ((host_tokens >= 0) & (host_tokens < rows))[:, None] & (chosen >= 0) & (chosen < s.n_experts)
                chosen = np.where(known, chosen, 0)  # what the kernel cannot place goes to expert 0 with weight 0
                ctx.memo[ckey] = np.bincount(chosen.ravel(), minlength=s.n_experts).tolist()
            per_expert = ctx.memo[ckey]
        else:
            per_expert = counts.cpu().tolist()  # the one place where the host waits for the device
        dt, dev_ = self.build.dtype, h.device
        cap = -(-max(per_expert) // 8) * 8
        if cap * s.n_experts <= self.PAD_FACTOR * T * s.top:
            # the experts are about evenly used: each gets a block of ``cap`` rows, and all of them run as
            # one batched product each way (rows that no token took compute nothing that is read)
            x_pad, place, _ = ops.moe_sort(h, ids, weights, counts, s.weight_on_input, cap=cap)
            gate_up = ops.batched_matmul(x_pad.view(s.n_experts, cap, s.width), self.w_gate_up)
            act = torch.empty((s.n_experts * cap, s.expert_ff), dtype=dt, device=dev_)
            self._activate(gate_up.view(s.n_experts * cap, 2 * s.expert_ff), act, s.expert_limit)
            y_pad = ops.batched_matmul(act.view(s.n_experts, cap, s.expert_ff), self.w_down)
            return ops.moe_gather(y_pad.view(s.n_experts * cap, s.width), place, weights, not s.weight_on_input, add=shared)
        # uneven: the experts' rows packed side by side, their products one after another into slices
        x_sorted, place, _ = ops.moe_sort(h, ids, weights, counts, s.weight_on_input)
        at = [0]
        for c in per_expert:
            at.append(at[-1] + c)
        gate_up = torch.empty((T * s.top, 2 * s.expert_ff), dtype=dt, device=dev_)
        for e in range(s.n_experts):
            if at[e + 1] > at[e]:
                ops.matmul_into(x_sorted[at[e]: at[e + 1]], self.w_gate_up[e], gate_up[at[e]: at[e + 1]])
        act = torch.empty((T * s.top, s.expert_ff), dtype=dt, device=dev_)
        self._activate(gate_up, act, s.expert_limit)
        y_sorted = torch.empty((T * s.top, s.width), dtype=dt, device=dev_)
        for e in range(s.n_experts):
            if at[e + 1] > at[e]:
                ops.matmul_into(act[at[e]: at[e + 1]], self.w_down[e], y_sorted[at[e]: at[e + 1]])
        return ops.moe_gather(y_sorted, place, weights, not s.weight_on_input, add=shared)
