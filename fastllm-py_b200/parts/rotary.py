"""Rotary position encoding as a table.

The part turns its constants into cos/sin tables [max_positions, rot_dim/2] in
float32 on the host, once; the attention kernels index them by position.  Any
rotary variant is a different table, so the kernels do not change with it.

Formulas (fastllm_py/kernels/ops.py:77-81, fastllm_py/model.py:329-339):
inv_freq[j] = 1 / theta^(2j / D) in float32; with linear scaling the integer
positions are divided by the factor in float64 and then cast to float32;
angle = position * inv_freq in float32.

Blended scaling ("yarn": factor, original, fast, slow) stretches the slow pairs only.  With
D = rot_dim and pair index j, the pair that makes t turns over `original` positions sits at
d(t) = D ln(original / (2 pi t)) / (2 ln theta); lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), D - 1),
ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1); the frequency is
inv_freq[j] * ((1 - ramp_j) + ramp_j / factor), and cos and sin are both multiplied by
0.1 ln(factor) + 1.

Scaling by bands of wavelength ("bands": factor, original, low, high): a pair whose wavelength
2 pi / inv_freq is shorter than original / high keeps its frequency, one longer than
original / low turns `factor` times slower, and between the two the frequency is
(1 - s) inv_freq / factor + s inv_freq with s = (original / wavelength - low) / (high - low).
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Part
from .registry import register_part


@register_part("position", "rotary")
class Rotary(Part):
    """params: rot_dim (even, <= head_dim), theta, scaling: None | ("linear", factor) | ("yarn", factor, original,
    fast, slow) | ("bands", factor, original, low, high), exact (False: the
    frequencies and angles are rounded to float32 before cos and sin, as above; True: they are formed in
    float64 and only cos and sin are rounded, for models specified by the formula rather than by float32 code)."""
    category = "position"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.rot_dim = int(spec.params["rot_dim"])
        self.theta = float(spec.params["theta"])
        self.scaling = spec.params.get("scaling")
        self.exact = bool(spec.params.get("exact", False))
        if self.rot_dim % 2:
            raise ValueError(f"rotary: rot_dim {self.rot_dim} must be even")
        if self.scaling is not None and self.scaling[0] not in ("linear", "yarn", "bands"):
            raise ValueError(f"rotary: scaling {self.scaling[0]!r} is not supported")
        if self.scaling is not None and self.scaling[0] in ("yarn", "bands") and not self.exact:
            raise ValueError("rotary: blended scaling is formed in float64 (exact=True)")

    def tables(self):
        """(cos, sin) on the device, shared by all parts with the same constants."""
        key = ("rotary", self.rot_dim, self.theta, self.scaling, self.ctx.max_positions, self.exact)
        if key not in self.ctx.shared and self.exact:
            d = self.rot_dim
            inv_freq = self.theta ** (-np.arange(0, d, 2, dtype=np.float64) / d)
            pos = np.arange(self.ctx.max_positions, dtype=np.float64)
            gain = 1.0
            if self.scaling is not None and self.scaling[0] == "yarn":
                _, factor, original, fast, slow = (float(v) if i else v for i, v in enumerate(self.scaling))

                def pair_of(turns):
                    return d * np.log(original / (2.0 * np.pi * turns)) / (2.0 * np.log(self.theta))

                lo = max(int(np.floor(pair_of(fast))), 0)
                hi = min(int(np.ceil(pair_of(slow))), d - 1)
                ramp = np.clip((np.arange(d // 2, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
                inv_freq = inv_freq / factor * ramp + inv_freq * (1.0 - ramp)
                gain = 0.1 * np.log(factor) + 1.0
            elif self.scaling is not None and self.scaling[0] == "bands":
                factor, original, low, high = (float(v) for v in self.scaling[1:])
                wave = 2.0 * np.pi / inv_freq
                s = (original / wave - low) / (high - low)
                inv_freq = np.where(wave < original / high, inv_freq,
                                    np.where(wave > original / low, inv_freq / factor,
                                             (1.0 - s) * inv_freq / factor + s * inv_freq))
            elif self.scaling is not None:
                pos = pos / float(self.scaling[1])
            ang = pos[:, None] * inv_freq[None, :]
            cos = torch.from_numpy((np.cos(ang) * gain).astype(np.float32)).to(self.ctx.device)
            sin = torch.from_numpy((np.sin(ang) * gain).astype(np.float32)).to(self.ctx.device)
            self.ctx.shared[key] = (cos.contiguous(), sin.contiguous())
        if key not in self.ctx.shared:
            d = self.rot_dim
            inv_freq = 1.0 / (self.theta ** (np.arange(0, d, 2, dtype=np.float32) / d))
            inv_freq = inv_freq.astype(np.float32)
            pos = np.arange(self.ctx.max_positions)
            if self.scaling is not None:
                pos = pos / float(self.scaling[1])
            ang = pos.astype(np.float32)[:, None] * inv_freq[None, :]
            cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(self.ctx.device)
            sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(self.ctx.device)
            self.ctx.shared[key] = (cos.contiguous(), sin.contiguous())
        return self.ctx.shared[key]
