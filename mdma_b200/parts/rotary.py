"""Rotary position encoding with a per-pair frequency table.

angle = float32(position) * inv_freq[i]; the pair (x0, x1) becomes
(x0 cos - x1 sin, x0 sin + x1 cos) (src/backend/cpu.rs:68-84).  `layout`
chooses which elements pair up: "interleaved" (2i, 2i+1) as the reference's
Llama does, or "split_half" (i, i + rotary_dim/2) as in its split-half
rotation (src/backend/cpu.rs:135-156), which checkpoint folders use.  The
table is theta^(-2i/d) computed once on the host in float64 (the reference
builds it on the host too: src/backend/cuda.rs:383-398); llama3 scaling
divides each frequency by a factor chosen by its wavelength.  Rotated keys are
written straight into the cache, so the encoding is fixed at write time
(src/model/arch/llama.rs:198-209).

A second kind of scaling, a dict {kind: "ramp", factor, original, fast, slow, magnitude_slope}: with
turn(t) = d ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(turn(fast)), 0), hi = min(ceil(turn(slow)), d - 1)
and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at f_i / factor * ramp_i + f_i (1 - ramp_i),
and cos and sin are both multiplied by `magnitude` = magnitude_slope * ln(factor) + 1.  Kernels that take a
frequency table alone cannot apply the magnitude; `encode_and_store` refuses it, mixers that can take it read
`magnitude`.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..registry import POSITIONS
from .base import Part


def inverse_frequencies(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """float32 [rotary_dim/2]."""
    out = []
    if isinstance(scaling, dict):
        if scaling.get("kind") != "ramp":
            raise ValueError(f"unknown rotary scaling {scaling.get('kind')!r}")
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def turn(t: float) -> float:
            return rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(float(theta)))

        lo = max(math.floor(turn(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn(float(scaling["slow"]))), rotary_dim - 1)
        for i in range(rotary_dim // 2):
            f = float(theta) ** (-2.0 * i / rotary_dim)
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / factor * ramp + f * (1.0 - ramp))
        return torch.tensor(out, dtype=torch.float64).to(torch.float32)
    for i in range(rotary_dim // 2):
        f = float(theta) ** (-2.0 * i / rotary_dim)
        if scaling is not None:
            wavelength = 2.0 * math.pi / f
            span = float(scaling.original_max_position_embeddings)
            if wavelength < span / scaling.high_freq_factor:
                pass
            elif wavelength > span / scaling.low_freq_factor:
                f = f / scaling.factor
            else:
                s = (span / wavelength - scaling.low_freq_factor) / (
                    scaling.high_freq_factor - scaling.low_freq_factor)
                f = (1.0 - s) * f / scaling.factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


@POSITIONS.register("rotary")
class Rotary(Part):
    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.head_dim = int(p["head_dim"])
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        self.interleaved = p.get("layout", "split_half") == "interleaved"
        if p.get("layout", "split_half") not in ("split_half", "interleaved"):
            raise ValueError(f"unknown rotary layout {p['layout']!r}")
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.table_host = inverse_frequencies(self.rotary_dim, p["theta"], p.get("scaling"))
        scaling = p.get("scaling")
        self.magnitude = 1.0         # a factor on cos and sin (the "ramp" scaling sets it)
        if isinstance(scaling, dict):
            self.magnitude = float(scaling.get("magnitude_slope", 0.0)) * math.log(float(scaling["factor"])) + 1.0

    def bind(self, tensors, rt):
        if getattr(self, "rt", None) is rt and getattr(self, "inv_freq", None) is not None:
            return                  # bound by its mixer and again by the model: one table
        super().bind(tensors, rt)
        self.inv_freq = rt.derived(self.table_host)

    fuses_pending = True        # adds up a deferred K-split projection itself

    def resident_tensors(self):
        return []                 # the frequency table is derived, not a weight

    def device_tensors(self):
        return {"inv_freq": ((self.rotary_dim // 2,), torch.float32)}

    def rotary_table(self):
        """(inverse frequencies on the device, rotated width, interleaved?): what a mixer needs to do this
        encoding inside a kernel of its own instead of calling `encode_and_store`."""
        return self.inv_freq, self.rotary_dim, self.interleaved

    def encode_and_store(self, ctx, qkv, n_heads, n_kv_heads, head_dim, view, write_kv):
        if self.magnitude != 1.0:
            raise ValueError("this rotation multiplies cos and sin by a factor; the kernel behind encode_and_store has none")
        partial, splits, stride = None, 0, 0
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            pend = ops_tensor.take_pending(qkv, ops.GEMM_STORE, ctx.n_tokens, self.rt.tc)
            if pend is not None:
                partial, splits, stride = pend
            else:
                ops_tensor.flush_pending(qkv.device, self.rt.tc)
        ops.rope_cache_write(qkv, ctx.n_tokens, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, self.inv_freq,
                             view.k if write_kv else None, view.v if write_kv else None,
                             view.page_table if write_kv else None, view.max_pages, view.page_size,
                             n_heads, n_kv_heads, head_dim, self.rotary_dim, self.interleaved, write_kv,
                             partial, splits, stride)
