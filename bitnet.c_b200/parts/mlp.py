"""Dense gated feed-forward (SwiGLU, or with the tanh form of GELU on the gate)."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, ParamSpec
from .registry import register_ffn


@register_ffn("gated_mlp")
class GatedMlp(FeedForward):
    """y = W_down (act(W_gate h) * (W_up h)), act = SiLU (src/transformer/cpu.c:1247-1303) or, by the spec's
    ``activation``, the tanh form of GELU.  A width of the feed-forward that is no multiple of 8 is filled up with
    rows of zeros, which add nothing."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "act", "norm")
    graph_safe = True
    accepts_sink = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} is not built; known: {', '.join(sorted(ops.ACTIVATIONS))}")
        self.act = ops.ACTIVATIONS[spec.activation]

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        return {"gate": ParamSpec((s.intermediate, s.width)), "up": ParamSpec((s.intermediate, s.width)),
                "down": ParamSpec((s.width, s.intermediate))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors["gate"], tensors["up"]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        down = tensors["down"]
        pad = -g.shape[0] % 8
        if pad:
            zeros = torch.zeros((pad, g.shape[1]), dtype=dt, device=g.device)
            g, u = torch.cat([g.to(dt), zeros]), torch.cat([u.to(dt), zeros])
            down = torch.cat([down, torch.zeros((down.shape[0], pad), dtype=down.dtype, device=down.device)], dim=1).contiguous()
        # gate and up rows in alternating blocks of 8: one product gives both, and with few rows
        # its epilogue applies the activation (the reference stacks gate and up on upload,
        # src/gpu_cuda.cu:11521-11558, and fuses gate/up + SiLU for decode, src/gpu_cuda.cu:4547)
        self.w_gate_up = ops.interleave_gate_up(g.to(dt), u.to(dt))
        self.w_down = down

    def forward(self, h, ctx, sink=None):
        act = ops.linear(h, self.w_gate_up, out_dtype=self.build.dtype, swiglu=True, act=self.act)
        out_dtype = torch.float32 if getattr(self.spec, "wide_output", False) else self.build.dtype
        return ops.linear(act, self.w_down, out_dtype=out_dtype, sink=sink)


@register_ffn("limited_mlp")
class LimitedMlp(FeedForward):
    """y = W_down (g * sigmoid(slope g) * (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit):
    the clamped gated unit as a dense feed-forward.  Gate and up rows are one stacked product; the delta leaves
    the last product in float32."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "act")
    graph_safe = True

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        return {"gate": ParamSpec((s.intermediate, s.width)), "up": ParamSpec((s.intermediate, s.width)),
                "down": ParamSpec((s.width, s.intermediate))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u, down = tensors["gate"], tensors["up"], tensors["down"]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        pad = -g.shape[0] % 8  # rows of zeros add nothing: min(0, limit) * ... = 0
        if pad:
            zeros = torch.zeros((pad, g.shape[1]), dtype=dt, device=g.device)
            g, u = torch.cat([g.to(dt), zeros]), torch.cat([u.to(dt), zeros])
            down = torch.cat([down, torch.zeros((down.shape[0], pad), dtype=down.dtype, device=down.device)], dim=1)
        self.inter = g.shape[0]
        self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()  # the gate rows, then the up rows
        self.w_down = down.contiguous()

    def forward(self, h, ctx):
        s = self.spec
        gu = ops.linear(h, self.w_gate_up, out_dtype=self.build.dtype)
        act = torch.empty((h.shape[0], self.inter), dtype=gu.dtype, device=gu.device)
        ops.glu_limited(gu, act, s.limit, s.slope)
        return ops.linear(act, self.w_down, out_dtype=torch.float32)
