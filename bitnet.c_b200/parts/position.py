"""Position encodings."""
from __future__ import annotations

import numpy as np

from ..csrc import ops
from .base import Position
from .registry import register_position


@register_position("rotary")
class Rotary(Position):
    """Rotate-half rotary encoding; angle_i = pos * theta^(-2i/dims) as a running float32 product
    (src/transformer/cpu_backend.c:283-296, src/model_arch.c:322-338)."""

    kernels = ("rope",)
    graph_safe = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        dims = spec.dims
        if dims % 2 or dims > spec.head_dim or dims <= 0:
            raise ValueError(f"rotary_dims={dims} must be even and at most head_dim={spec.head_dim}")
        # powf(theta, -2/dims) in float32, the factor between consecutive angles.
        self.theta_scale = float(np.power(np.float32(spec.theta), np.float32(-2.0) / np.float32(dims)))

    def rotary_params(self):
        """(rotary_dims, theta_scale): lets a mixer's decode kernel apply this encoding itself."""
        return self.spec.dims, self.theta_scale

    def rotate(self, x, n_heads, head_dim, ctx):
        ops.rope_append(x, n_heads, head_dim, self.spec.dims, self.theta_scale, ctx.tok_pos)

    def rotate_and_append(self, x, n_heads, head_dim, ctx, kv, k_off, v_off):
        ops.rope_append(x, n_heads, head_dim, self.spec.dims, self.theta_scale, ctx.tok_pos,
                        k_off=k_off, v_off=v_off, n_kv_heads=kv.n_kv_heads, tok_seq=ctx.tok_seq,
                        slots=ctx.slots, page_table=kv.page_table, k_cache=kv.k, v_cache=kv.v)


@register_position("none")
class NoPosition(Position):
    graph_safe = True

    def rotary_params(self):
        return 0, 1.0

    def rotate(self, x, n_heads, head_dim, ctx):
        return None


def pair_frequencies(spec) -> np.ndarray:
    """The table of a ``RotaryPairsSpec``: base^(-2i/dims) for i < dims/2 in double precision, long wavelengths
    slowed down as ``scaling`` = (factor, low, high, original) says (wavelength l = 2 pi / f: f stays where
    l < original / high, becomes f / factor where l > original / low, and in between the blend
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)); rounded to float32 once."""
    i = np.arange(spec.dims // 2, dtype=np.float64)
    f = np.float64(spec.base) ** (-2.0 * i / spec.dims)
    if spec.scaling is not None:
        factor, low, high, original = (float(v) for v in spec.scaling)
        wavelength = 2.0 * np.pi / f
        s = (original / wavelength - low) / (high - low)
        blend = (1.0 - s) * f / factor + s * f
        f = np.where(wavelength < original / high, f, np.where(wavelength > original / low, f / factor, blend))
    return f.astype(np.float32)


@register_position("rotary_pairs")
class RotaryPairs(Position):
    """Rotary encoding in the interleaved pairing with a table of frequencies (``pair_frequencies``): the pair
    (2i, 2i + 1) of the rotated part of a head is turned by position * f_i, angles in float32.  Besides
    ``rotate`` it offers ``apply``, which places the rotated part anywhere inside the heads of two tensors and
    writes keys (and unrotated values) into the cache in the same launch."""

    kernels = ("rotary_pairs",)
    graph_safe = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if spec.dims % 2 or spec.dims <= 0 or spec.dims > 512:
            raise ValueError(f"rotary dims={spec.dims} must be even and at most 512")
        self._table = pair_frequencies(spec)
        self._freqs = None

    def freqs(self, device):
        if self._freqs is None or self._freqs.device != device:
            import torch
            self._freqs = torch.from_numpy(self._table).to(device)
        return self._freqs

    def rotate(self, x, n_heads, head_dim, ctx):
        ops.rotary_pairs_append(x, self.freqs(x.device), ctx.tok_pos, q_off=0, n_q_heads=n_heads, q_head_stride=head_dim)

    def apply(self, x, ctx, **places):
        """``ops.rotary_pairs_append`` with this encoding's table and the step's positions."""
        ops.rotary_pairs_append(x, self.freqs(x.device), ctx.tok_pos, **places)


def blended_frequencies(spec, wide: bool = False):
    """(table, magnitude) of a ``RotaryBlendSpec``: base^(-2i/dims) for i < dims/2 in double precision, the slow
    ones divided by ``factor`` along a ramp between the dimension that turns ``fast`` times within ``original``
    positions and the one that turns ``slow`` times; rounded to float32 once (``wide``: left in double precision).
    The magnitude multiplies cos and sin alike."""
    dims = spec.dims
    i = np.arange(dims // 2, dtype=np.float64)
    f = np.float64(spec.base) ** (-2.0 * i / dims)
    if spec.factor == 1.0 or spec.original <= 0:
        return (f if wide else f.astype(np.float32)), 1.0

    def turns(t):
        return dims * np.log(spec.original / (2.0 * np.pi * t)) / (2.0 * np.log(spec.base))

    lo = max(int(np.floor(turns(spec.fast))), 0)
    hi = min(int(np.ceil(turns(spec.slow))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    f = f / spec.factor * ramp + f * (1.0 - ramp)
    return (f if wide else f.astype(np.float32)), float(spec.magnitude_slope * np.log(spec.factor) + 1.0)


@register_position("rotary_blend")
class RotaryBlend(RotaryPairs):
    """Rotary encoding over a table whose slow frequencies are divided by a factor along a ramp
    (``blended_frequencies``), cos and sin both times a magnitude, in the halves pairing (number i of the rotated
    part with number i + dims / 2) or the neighbours pairing.  The same kernel and the same ``rotate`` / ``apply``
    as ``rotary_pairs``."""

    def __init__(self, spec, build):
        Position.__init__(self, spec, build)
        if spec.dims % 2 or spec.dims <= 0 or spec.dims > 512:
            raise ValueError(f"rotary dims={spec.dims} must be even and at most 512")
        if spec.pairing not in ("halves", "neighbours"):
            raise ValueError(f"rotary pairing is 'halves' or 'neighbours', not {spec.pairing!r}")
        self._table, self.magnitude = blended_frequencies(spec)
        self._table64 = blended_frequencies(spec, wide=True)[0]
        self._freqs = self._freqs64 = None
        self.split_halves = spec.pairing == "halves"

    def freqs64(self, device):
        """The table in double precision: the kernel then takes the angles in double precision as well, so that a
        position in the thousands costs no digits of the angle."""
        if self._freqs64 is None or self._freqs64.device != device:
            import torch
            self._freqs64 = torch.from_numpy(np.ascontiguousarray(self._table64, dtype=np.float64)).to(device)
        return self._freqs64

    def rotate(self, x, n_heads, head_dim, ctx):
        ops.rotary_pairs_append(x, self.freqs(x.device), ctx.tok_pos, q_off=0, n_q_heads=n_heads, q_head_stride=head_dim,
                                split_halves=self.split_halves, magnitude=self.magnitude, freqs64=self.freqs64(x.device))

    def apply(self, x, ctx, **places):
        ops.rotary_pairs_append(x, self.freqs(x.device), ctx.tok_pos, split_halves=self.split_halves, magnitude=self.magnitude,
                                freqs64=self.freqs64(x.device), **places)
