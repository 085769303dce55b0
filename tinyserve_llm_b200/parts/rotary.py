"""
Rotate-half rotary position encoding with optional llama3 frequency rescaling.

Reference formulas: inv_freq[i] = 1 / theta^(2i/d) in float32 (model/llama.py:148); llama3 rescaling
by wavelength bands (:107-128); angle[p, i] = float32(p) * inv_freq[i]; the table row of position p
is [cos(angle) | sin(angle)] (:157-160).  The table is built once on the host in float32, in that
order of operations, and the kernels gather rows of it by position.
"""

from __future__ import annotations

import math

import torch

from tinyserve_llm_b200.config.spec import Llama3Scaling, RotarySpec, SinusoidSpec
from tinyserve_llm_b200.parts.base import PositionEncoding, Runtime, register_part


def inverse_frequencies(head_dim: int, theta: float, scaling: Llama3Scaling | None) -> torch.Tensor:
    """float32 [head_dim // 2]."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta ** exponent)
    if scaling is None:
        return inv_freq
    window = scaling.original_max_position_embeddings
    longest_kept = window / scaling.low_freq_factor      # wavelengths above this are slowed by `factor`
    shortest_scaled = window / scaling.high_freq_factor  # wavelengths below this are left alone
    wavelength = 2 * math.pi / inv_freq
    slowed = torch.where(wavelength > longest_kept, inv_freq / scaling.factor, inv_freq)
    blend = (window / wavelength - scaling.low_freq_factor) / (scaling.high_freq_factor - scaling.low_freq_factor)
    blended = (1 - blend) * slowed / scaling.factor + blend * slowed
    in_band = (wavelength >= shortest_scaled) & (wavelength <= longest_kept)
    return torch.where(in_band, blended, slowed)


def cos_sin_table(spec: RotarySpec, num_positions: int | None = None) -> torch.Tensor:
    """float32 [positions, head_dim]: cos of the head_dim/2 angles, then their sin."""
    n = spec.max_positions if num_positions is None else num_positions
    inv_freq = inverse_frequencies(spec.head_dim, spec.theta, spec.scaling)
    angles = torch.outer(torch.arange(n, dtype=torch.float32), inv_freq)
    return torch.cat((angles.cos(), angles.sin()), dim=-1).contiguous()


@register_part("position", "rotary")
class Rotary(PositionEncoding):
    def __init__(self, spec: RotarySpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        key = ("rotary", spec)
        if key not in rt.shared:               # one table for all layers with the same settings
            rt.shared[key] = cos_sin_table(spec).to(rt.device)
        self.table = rt.shared[key]


def yarn_frequencies(dims: int, base: float, yarn) -> torch.Tensor:
    """float64 [dims / 2]: base^(-2i/dims), rescaled by `yarn` (a `YarnScaling`) where given."""
    i = torch.arange(0, dims // 2, dtype=torch.float64)
    freq = float(base) ** (-2.0 * i / dims)
    if yarn is None:
        return freq

    def turns(t: float) -> float:
        return dims * math.log(yarn.original / (2 * math.pi * t)) / (2 * math.log(base))

    lo = max(math.floor(turns(yarn.fast)), 0)
    hi = min(math.ceil(turns(yarn.slow)), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / yarn.factor * ramp + freq * (1.0 - ramp)


def band_scaled_frequencies(dims: int, base: float, bands) -> torch.Tensor:
    """
    float64 [dims / 2]: base^(-2i/dims) rescaled by wavelength l = 2 pi / f (`bands`: a `Llama3Scaling`): kept where
    l < original / high, divided by the factor where l > original / low, and in between, with
    s = (original / l - low) / (high - low), the blend (1 - s) f / factor + s f.
    """
    f = yarn_frequencies(dims, base, None)
    original, low, high = float(bands.original_max_position_embeddings), float(bands.low_freq_factor), float(bands.high_freq_factor)
    wavelength = 2 * math.pi / f
    s = (original / wavelength - low) / (high - low)
    blend = (1 - s) * f / bands.factor + s * f
    return torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / bands.factor, blend))


@register_part("position", "rotary_inline")
class InlineRotary(PositionEncoding):
    """
    Rotate-half rotation whose angles the kernels compute themselves, position * frequencies[i] in
    float32 with frequencies[i] = base^(-2i/dims) (rescaled by the spec's `yarn` or `bands`): no table,
    so no longest position.  Mixers that rotate inside their own kernels read `dims` and `frequencies`.
    """

    def __init__(self, spec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        if spec.dims <= 0 or spec.dims % 2:
            raise ValueError(f"rotation over {spec.dims} channels: the number must be positive and even")
        if spec.yarn is not None and getattr(spec, "bands", None) is not None:
            raise ValueError("a rotation takes one rescaling of its frequencies, YaRN or wavelength bands, not both")
        key = ("rotary_inline", spec)
        if key not in rt.shared:
            if getattr(spec, "bands", None) is not None:
                freq = band_scaled_frequencies(spec.dims, float(spec.base), spec.bands)
            else:
                freq = yarn_frequencies(spec.dims, float(spec.base), spec.yarn)
            rt.shared[key] = freq.to(torch.float32).to(rt.device)
        self.dims = spec.dims
        self.frequencies = rt.shared[key]
        # cos and sin are multiplied by this (1 without YaRN); a kernel that rotates with a YaRN rescaling has to apply it
        self.magnitude = 1.0 if spec.yarn is None else 0.1 * math.log(spec.yarn.factor) + 1.0


@register_part("position", "sinusoid")
class Sinusoid(PositionEncoding):
    """
    A position vector added to the token embedding: with angle_i = position * base^(-2i/size), entry 2i is
    sin(angle_i) and entry 2i + 1 cos(angle_i).  Only the frequencies are kept (worked out in float64, stored
    in float32); the kernel that gathers the embedding rows multiplies them by the position in float32 and
    takes sine and cosine itself, so there is no table and no longest position.
    """

    def __init__(self, spec: SinusoidSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        if spec.size <= 0 or spec.base <= 0:
            raise ValueError(f"a sinusoidal position vector of {spec.size} entries with base {spec.base}")
        key = ("sinusoid", spec)
        if key not in rt.shared:
            i = torch.arange((spec.size + 1) // 2, dtype=torch.float64)
            rt.shared[key] = (float(spec.base) ** (-2.0 * i / spec.size)).to(torch.float32).to(rt.device)
        self.frequencies = rt.shared[key]
