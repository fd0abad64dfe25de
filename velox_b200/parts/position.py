"""Position encodings that a mixer applies to its queries and keys.

`RotaryPosition`: the half-split rotation of the reference
(src/paged/metal_kernels.rs:199-202, 230-236): pairs (i, i + rot/2) turned by
position * inv_freq[i], inv_freq[i] = 1 / theta^(2i/rot), the power taken in
float64 and the quotient in float32 as the reference does
(src/paged/qwen3.rs:281-284).  The reference then tabulates cosines and sines
and rounds the table to the model's element type (src/paged/qwen3.rs:287-293);
here angle, sine and cosine are float32 inside the kernel and never rounded.

With `layout="interleaved"` the same angles turn neighbours instead: channel 2i is paired with channel 2i + 1.
The kernels that rotate take the layout as a flag (`interleaved`).

With `scaling` (factor, original, fast, slow) the frequencies are stretched for contexts longer than `original`
positions: channel pairs that turn fewer than `slow` times in `original` positions have their frequency divided by
`factor`, pairs that turn more than `fast` times keep it, and between the two pair indices
d(t) = rot ln(original / (2 pi t)) / (2 ln theta) the two are blended linearly; cosines and sines are then multiplied by
0.1 ln(factor) + 1 (`magnitude`, which the rotating kernels take as a parameter).

`NoPosition`: nothing is applied.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .base import Position


class RotaryPosition(Position):
    cuda_graph_safe = True

    def __init__(self, prefix: str = "", head_dim: int = 0, theta: float = 10000.0, rotary_dim: Optional[int] = None,
                 layout: str = "half", scaling: Optional[Dict[str, float]] = None):
        super().__init__(prefix)
        self.scaling = dict(scaling) if scaling else None
        if self.scaling is not None:
            missing = [k for k in ("factor", "original", "fast", "slow") if k not in self.scaling]
            if missing or not float(self.scaling["factor"]) > 0 or not float(self.scaling["original"]) > 0 \
                    or not float(self.scaling["fast"]) > 0 or not float(self.scaling["slow"]) > 0:
                raise ValueError("rotation scaling needs positive factor, original, fast and slow; got %r" % (scaling,))
        if layout not in ("half", "interleaved"):
            raise ValueError("rotation layout %r is not 'half' or 'interleaved'" % (layout,))
        self.interleaved = layout == "interleaved"
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim else self.head_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError("rotary_dim %d must be even and within head_dim %d" % (self.rotary_dim, self.head_dim))
        self._table = {}

    @property
    def magnitude(self) -> float:
        """What cosines and sines are multiplied by (1 without scaling)."""
        return 1.0 if self.scaling is None else 0.1 * math.log(float(self.scaling["factor"])) + 1.0

    def inverse_frequencies(self) -> np.ndarray:
        r = self.rotary_dim
        if self.scaling is None:
            vals = [np.float32(1.0) / np.float32(self.theta ** (i / r)) for i in range(0, r, 2)]
            return np.asarray(vals, dtype=np.float32)
        sc = self.scaling
        factor, original = float(sc["factor"]), float(sc["original"])

        def pair_index(turns: float) -> float:
            return r * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(pair_index(float(sc["fast"]))), 0)
        hi = min(math.ceil(pair_index(float(sc["slow"]))), r - 1)
        out = []
        for i in range(r // 2):
            f = self.theta ** (-2.0 * i / r)
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / factor * ramp + f * (1.0 - ramp))
        return np.asarray(out, dtype=np.float32)

    def rotary_table(self, device) -> Optional[Tuple[torch.Tensor, int]]:
        key = str(device)
        if key not in self._table:
            self._table[key] = torch.from_numpy(self.inverse_frequencies()).to(device)
        return self._table[key], self.rotary_dim


class NoPosition(Position):
    cuda_graph_safe = True

    def __init__(self, prefix: str = "", **_ignored):
        super().__init__(prefix)
