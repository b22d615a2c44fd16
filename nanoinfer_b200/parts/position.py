"""Position encodings.  A mixer asks its encoding for the constants its kernel needs."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..config.model_config import ConfigError
from ..config.registry import register_part
from .base import Part


def rope_inverse_frequencies(rotary_dim: int, theta: float, scaling) -> np.ndarray:
    """FP32 inverse frequencies of the rotary pairs, with the optional llama3 rescaling.

    freq_i = 1 / theta^(2i / rotary_dim); with scaling, by wavelength 2*pi/freq:
    >= original/low_freq_factor: freq / factor;  > original/high_freq_factor: blend
    (1 - s) * freq / factor + s * freq with s = (original / wavelen - low) / (high - low);
    else unchanged.  All in FP32, as src/op/kernels/cpu/rope_kernel.cpp:117-139 and
    src/op/kernels/cuda/rope_kernel.cu:95-132 compute them.
    """
    f32 = np.float32
    half = rotary_dim // 2
    freqs = np.empty(half, dtype=np.float32)
    for p in range(half):
        freq = f32(1.0) / np.power(f32(theta), f32(p * 2) / f32(rotary_dim), dtype=np.float32)
        if scaling is not None:
            orig = f32(scaling.original_max_position_embeddings)
            low, high = f32(scaling.low_freq_factor), f32(scaling.high_freq_factor)
            factor = f32(scaling.factor)
            wavelen = f32(2.0) * f32(math.pi) / freq
            if wavelen >= orig / low:
                freq = freq / factor
            elif wavelen > orig / high:
                smooth = (orig / wavelen - low) / (high - low)
                freq = (f32(1.0) - smooth) * freq / factor + smooth * freq
        freqs[p] = freq
    return freqs


class RotaryEncoding(Part):
    """Rotary encoding: holds inv_freq [rotary_dim/2] FP32 on the device and the pairing.

    What a mixer reads from ANY position encoding: ``rotary_dim`` (0: nothing is rotated), ``inv_freq``,
    ``interleaved``, and ``head_slopes`` - None, or float32 [num_heads] on the device: the encoding adds
    slope[h] * (key position - query position) to the scaled attention scores of head h (then the mixer
    uses the plain attention kernel, which takes such a bias, in either precision); and ``magnitude``: a factor on
    both the cosine and the sine (1 unless the encoding also scales what it rotates), which the kernels that take
    it apply to the rotated dimensions only."""
    head_slopes = None
    magnitude = 1.0

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ConfigError(f"rotary_dim {spec.rotary_dim} must be positive and even")
        if spec.pairing not in ("half", "interleaved"):
            raise ConfigError(f"rope pairing '{spec.pairing}' must be 'half' or 'interleaved'")
        if spec.scaling is not None and spec.scaling.rope_type != "llama3":
            raise ConfigError(f"rope scaling '{spec.scaling.rope_type}' is not supported")
        self.rotary_dim = spec.rotary_dim
        self.interleaved = spec.pairing == "interleaved"
        self.inv_freq = torch.from_numpy(
            rope_inverse_frequencies(spec.rotary_dim, spec.theta, spec.scaling)).to(rt.device)


class RotaryEncodingExact(RotaryEncoding):
    """Rotary encoding whose frequencies theta^(-2i / rotary_dim) are computed in double precision and rounded
    once to FP32 (no rescaling rule); angles stay FP32 products position * frequency on the device."""

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        if spec.scaling is not None:
            raise ConfigError("the exact rotary encoding has no rescaling rule")
        i = np.arange(spec.rotary_dim // 2, dtype=np.float64)
        self.inv_freq = torch.from_numpy(np.power(float(spec.theta), -2.0 * i / spec.rotary_dim).astype(np.float32)).to(rt.device)


class RotaryEncodingYarn(RotaryEncoding):
    """Rotary encoding stretched for longer contexts by a ramp over the frequencies.  With f_i = theta^(-2i / n)
    (n = rotary_dim) and the scaling's ``factor``, ``original`` (the context the frequencies were made for),
    ``fast`` and ``slow`` (carried in the spec's RopeScaling as high_freq_factor and low_freq_factor):

        c(t) = n ln(original / (2 pi t)) / (2 ln theta)        the dimension that turns t times over ``original``
        lo = max(floor(c(fast)), 0),  hi = min(ceil(c(slow)), n - 1)
        r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        f_i <- f_i / factor * r_i + f_i * (1 - r_i)

    so dimensions that turn often keep their frequency and slow ones are divided by ``factor``; cosine and sine
    are both multiplied by ``magnitude`` = 0.1 ln(factor) + 1.  Without a scaling rule it is the plain encoding.
    Frequencies are computed in double precision and rounded once; angles are FP32 products on the device."""

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        Part.__init__(self, spec, hidden_size, weights, rt)
        n = spec.rotary_dim
        if n <= 0 or n % 2:
            raise ConfigError(f"rotary_dim {n} must be positive and even")
        if spec.pairing not in ("half", "interleaved"):
            raise ConfigError(f"rope pairing '{spec.pairing}' must be 'half' or 'interleaved'")
        self.rotary_dim = n
        self.interleaved = spec.pairing == "interleaved"
        freq, self.magnitude = yarn_frequencies(n, spec.theta, spec.scaling)
        self.inv_freq = torch.from_numpy(freq.astype(np.float32)).to(rt.device)


def yarn_frequencies(rotary_dim: int, theta: float, scaling):
    """(float64 frequencies [rotary_dim / 2], magnitude) of RotaryEncodingYarn."""
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    freq = np.power(float(theta), -2.0 * i / rotary_dim)
    if scaling is None:
        return freq, 1.0
    if scaling.rope_type != "yarn":
        raise ConfigError(f"rope scaling '{scaling.rope_type}' is not the ramp rule ('yarn')")
    factor, original = float(scaling.factor), float(scaling.original_max_position_embeddings)
    fast, slow = float(scaling.high_freq_factor), float(scaling.low_freq_factor)
    if factor <= 0 or original <= 0 or fast <= 0 or slow <= 0 or theta <= 1.0:
        raise ConfigError("rope scaling: factor, original, fast and slow must be positive (and the base above 1)")

    def turns(t):
        return rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(theta))

    lo = max(math.floor(turns(fast)), 0)
    hi = min(math.ceil(turns(slow)), rotary_dim - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class RotaryEncodingScaled(RotaryEncoding):
    """Rotary encoding with f_i = theta^(-2i / n) (n = rotary_dim) and one of two rescaling rules, or none:

        "linear"   every f_i is divided by ``factor``;
        "llama3"   by wavelength l = 2 pi / f: l < original / high keeps f; l > original / low gives f / factor; between
                   the two, with s = (original / l - low) / (high - low), (1 - s) f / factor + s f.

    Unlike ``RotaryEncoding`` (which follows the reference's FP32 arithmetic step by step) the frequencies are computed
    in double precision and rounded once to FP32; angles stay FP32 products position * frequency on the device."""

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        Part.__init__(self, spec, hidden_size, weights, rt)
        n = spec.rotary_dim
        if n <= 0 or n % 2:
            raise ConfigError(f"rotary_dim {n} must be positive and even")
        if spec.pairing not in ("half", "interleaved"):
            raise ConfigError(f"rope pairing '{spec.pairing}' must be 'half' or 'interleaved'")
        self.rotary_dim = n
        self.interleaved = spec.pairing == "interleaved"
        self.inv_freq = torch.from_numpy(scaled_frequencies(n, spec.theta, spec.scaling).astype(np.float32)).to(rt.device)


def scaled_frequencies(rotary_dim: int, theta: float, scaling) -> np.ndarray:
    """float64 frequencies [rotary_dim / 2] of RotaryEncodingScaled."""
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    freq = np.power(float(theta), -2.0 * i / rotary_dim)
    if scaling is None:
        return freq
    factor = float(scaling.factor)
    if factor <= 0:
        raise ConfigError("rope scaling: the factor must be positive")
    if scaling.rope_type == "linear":
        return freq / factor
    if scaling.rope_type == "llama3":
        original = float(scaling.original_max_position_embeddings)
        low, high = float(scaling.low_freq_factor), float(scaling.high_freq_factor)
        if original <= 0 or low <= 0 or high <= low:
            raise ConfigError("rope scaling: original and low must be positive and high above low")
        wavelength = 2.0 * math.pi / freq
        s = (original / wavelength - low) / (high - low)
        blend = (1.0 - s) * freq / factor + s * freq
        return np.where(wavelength < original / high, freq, np.where(wavelength > original / low, freq / factor, blend))
    raise ConfigError(f"rope scaling '{scaling.rope_type}' is not one of linear, llama3")


class NoEncoding(Part):
    """No position encoding: queries and keys are used as projected."""
    head_slopes = None
    magnitude = 1.0

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.rotary_dim = 0
        self.interleaved = False
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=rt.device)


register_part("position", "rope", RotaryEncoding, replace=True)
register_part("position", "rope_exact", RotaryEncodingExact, replace=True)
register_part("position", "rope_yarn", RotaryEncodingYarn, replace=True)
register_part("position", "rope_scaled", RotaryEncodingScaled, replace=True)
register_part("position", "none", NoEncoding, replace=True)
