"""Position encodings.

``rotary``: tables of cos and sin of ``position * inv_freq`` with
``inv_freq[i] = theta^(-2i/head_dim)`` (engine/layers.py:57-79), applied to the
pairs (i, i + head_dim/2) of q and k (:82-115).  The optional llama3 frequency
scaling is not in the reference: wavelengths below ``orig/high_freq_factor``
are kept, above ``orig/low_freq_factor`` divided by ``factor``, and blended
linearly in ``orig/wavelength`` between.  Angles and tables are float32, built
once per distinct spec and shared by the layers that use it.
"""

from __future__ import annotations

import math

import torch

from ..weights.loader import ExpectedTensor
from .registry import register_position


def rotary_inv_freq(spec) -> torch.Tensor:
    hd = spec.head_dim
    inv_freq = 1.0 / (spec.theta ** (torch.arange(0, hd, 2).float() / hd))
    s = spec.scaling
    if s is not None:
        if s.rope_type != "llama3":
            raise ValueError(f"rope scaling {s.rope_type!r} is not built")
        f = inv_freq.double()
        orig = float(s.original_max_position_embeddings)
        wavelen = 2.0 * math.pi / f
        smooth = (orig / wavelen - s.low_freq_factor) / (s.high_freq_factor - s.low_freq_factor)
        blended = (1.0 - smooth) * f / s.factor + smooth * f
        out = torch.where(wavelen < orig / s.high_freq_factor, f,
                          torch.where(wavelen > orig / s.low_freq_factor, f / s.factor, blended))
        inv_freq = out.float()
    return inv_freq


def rotary_tables(spec) -> tuple[torch.Tensor, torch.Tensor]:
    """cos, sin: float32 [max_positions, head_dim/2] on the CPU."""
    inv_freq = rotary_inv_freq(spec)
    angles = torch.outer(torch.arange(spec.max_positions).float(), inv_freq)
    return angles.cos().contiguous(), angles.sin().contiguous()


@register_position("none")
class NoPosition:
    @staticmethod
    def expected_tensors(spec):
        return {}

    def __init__(self, spec, tensors, rt):
        self.spec = spec

    def rotary_tables(self):
        return None

    def rotate(self, q, k, ctx):
        return None


@register_position("rotary")
class Rotary:
    @staticmethod
    def expected_tensors(spec):
        return {}

    def __init__(self, spec, tensors, rt):
        if spec.head_dim % 2:
            raise ValueError("rotary embeddings need an even head_dim")
        self.spec = spec
        key = ("rotary", spec)
        if key not in rt.shared:
            cos, sin = rotary_tables(spec)
            rt.shared[key] = (cos.to(rt.device), sin.to(rt.device))
        self.cos, self.sin = rt.shared[key]

    def rotary_tables(self):
        return self.cos, self.sin

    def rotate(self, q, k, ctx):
        return None


@register_position("rotary_pairs")
class RotaryPairs:
    """Neighbouring dimensions (2i, 2i + 1) of the first ``rot_dims`` dimensions of every head turn by the angle
    ``position * theta^(-2i / rot_dims)``; the other dimensions pass unchanged.  There is no table: the kernel that
    norms q and k and writes the cache forms the angle from the position and these frequencies (float64, so that
    neither a large position nor a key far back costs digits; sine and cosine are float32), and positions have no
    limit."""

    @staticmethod
    def expected_tensors(spec):
        return {}

    def __init__(self, spec, tensors, rt):
        if spec.rot_dims % 2 or not 0 < spec.rot_dims <= spec.head_dim:
            raise ValueError(f"pair rotation needs an even number of dimensions up to the head's {spec.head_dim}, not {spec.rot_dims}")
        self.spec = spec
        key = ("rotary_pairs", spec.theta, spec.rot_dims)
        if key not in rt.shared:
            i = torch.arange(spec.rot_dims // 2, dtype=torch.float64)
            rt.shared[key] = (float(spec.theta) ** (-2.0 * i / spec.rot_dims)).to(rt.device)
        self.inv_freq = rt.shared[key]
        self.pair_rotation = (self.inv_freq, spec.rot_dims)

    def rotary_tables(self):
        return None

    def rotate(self, q, k, ctx):
        return None


def partial_rotation_frequencies(spec) -> tuple[torch.Tensor, float]:
    """(float64 frequencies [rot_dims / 2] on the CPU, multiplier of cosine and sine) of a ``rotary_partial`` spec:
    ``theta^(-2i / rot_dims)``, blended for a longer context when the spec carries a ``yarn`` entry."""
    dims = spec.rot_dims
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(spec.theta) ** (-2.0 * i / dims)
    y = spec.yarn
    if y is None:
        return f, 1.0
    ln_base = math.log(float(spec.theta))

    def dim_of(turns: float) -> float:       # the (fractional) pair index whose wavelength makes that many turns in the original context
        return dims * math.log(y.original / (2.0 * math.pi * turns)) / (2.0 * ln_base)

    lo = max(math.floor(dim_of(y.fast)), 0)
    hi = min(math.ceil(dim_of(y.slow)), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / y.factor * ramp + f * (1.0 - ramp), y.mult_slope * math.log(y.factor) + 1.0


@register_position("rotary_partial")
class PartialRotation:
    """``rot_dims`` dimensions of a head turn by ``position * frequency``, paired in halves or as neighbours; which
    dimensions of the head these are is the mixer's business (``kernels.head_prepare`` takes an offset).  No table: the
    kernel forms the angle from the position and the float64 frequencies, so positions have no limit."""

    @staticmethod
    def expected_tensors(spec):
        return {}

    def __init__(self, spec, tensors, rt):
        if spec.rot_dims % 2 or spec.rot_dims <= 0:
            raise ValueError(f"a rotation needs an even, positive number of dimensions, not {spec.rot_dims}")
        if spec.layout not in ("halves", "neighbours"):
            raise ValueError(f"rotation layout {spec.layout!r} is not built (known: halves, neighbours)")
        self.spec = spec
        key = ("rotary_partial", spec.theta, spec.rot_dims, spec.yarn)
        if key not in rt.shared:
            f, mult = partial_rotation_frequencies(spec)
            rt.shared[key] = (f.to(rt.device), float(mult))
        self.inv_freq, self.mult = rt.shared[key]
        self.rot_dims = spec.rot_dims
        self.neighbours = spec.layout == "neighbours"

    def rotary_tables(self):
        return None

    def rotate(self, q, k, ctx):
        return None


def distance_bucket(n: int, n_buckets: int, max_distance: int) -> int:
    """Row of a bucketed distance table for a key that lies ``n`` positions back.

    With h = n_buckets // 2: distances below h have a row each; from there on rows are spread evenly over
    ln(n / h) between h and ``max_distance``, and every distance from ``max_distance`` on shares the last row:
    ``min(n_buckets - 1, h + floor(ln(n / h) / ln(max_distance / h) * (n_buckets - h)))``.
    """
    h = n_buckets // 2
    if n < h:
        return n
    return min(n_buckets - 1, h + int(math.floor(math.log(n / h) / math.log(max_distance / h) * (n_buckets - h))))


@register_position("bucketed_bias")
class BucketedBias:
    """No rotation; a learned table [n_buckets, n_heads] is added to the scores by distance (``distance_bucket``).
    The table is unrolled once into one row per distance, [n_heads, max_distance + 1] float32, whose last column
    stands for every larger distance: what the attention kernels take as ``score_bias``."""

    @staticmethod
    def expected_tensors(spec):
        return {spec.table: ExpectedTensor((spec.n_buckets, spec.n_heads))}

    def __init__(self, spec, tensors, rt):
        if spec.n_buckets < 2 or spec.max_distance <= spec.n_buckets // 2:
            raise ValueError(f"a distance table of {spec.n_buckets} rows needs max_distance above {spec.n_buckets // 2}")
        self.spec = spec
        rows = torch.tensor([distance_bucket(n, spec.n_buckets, spec.max_distance) for n in range(spec.max_distance + 1)],
                            dtype=torch.long, device=rt.device)
        assert int(rows[-1]) == spec.n_buckets - 1
        self.bias = tensors[spec.table].float()[rows].t().contiguous()          # [n_heads, max_distance + 1]

    def rotary_tables(self):
        return None

    def rotate(self, q, k, ctx):
        return None

    def score_bias(self):
        return self.bias
