"""Grouped-query causal attention over the cache.

q, k, v = h Wq^T, h Wk^T, h Wv^T (no biases unless `bias` is set); q and k take the position
encoding, k and v go to the cache; a query at position p reads the keys
[first, p] of its own sequence (first = 0, or p+1-window), kv head = q head //
(heads / kv heads), scores (q.k) * scale through a float softmax; the result
times Wo^T is added to the residual stream (src/model/arch/llama.rs:195-212,
src/backend/cpu.rs:530-590).  Heads, groups, head size, scale and window are
parameters.  A site that reads another site's cache has no k/v matrices and
writes nothing.

Further options, each off unless set (a layer that sets any of them runs the path of `_forward_extended`):
`v_dim`, value heads of a size of their own; `qk_norm_eps`, after the position encoding every query and key head is
divided by its root mean square, x / sqrt(mean(x^2) + eps), without a weight; `sink`, a learned number per head
(tensor `sink`) whose exponential joins the softmax's denominator once, with no key and no value; `head_gate`, each
head's result is multiplied by sigmoid((Wg h)_head), one number per head (tensor `g_proj.weight` [heads, hidden],
computed with the q, k, v product); `out_scale`, a constant on the result.  `position` may be None (no encoding).
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..cache import KVNeed
from ..registry import MIXERS, POSITIONS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


FUSED_ROTARY = os.environ.get("MDMA_FUSED_ROTARY", "1") != "0"


@MIXERS.register("attention")
class Attention(Part):
    graph_safe = True      # forward reads no host-side per-step values
    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = int(p.get("window", 0) or 0)
        self.shared_cache = bool(p.get("shared_cache", False))
        self.bias = bool(p.get("bias", False))              # a vector added after each of the four products
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads do not divide over {self.n_kv_heads} kv heads")
        pos = p.get("position")
        self.position = POSITIONS.get(pos.kind)(pos) if pos is not None else None
        if getattr(self.position, "magnitude", 1.0) != 1.0:
            raise ValueError("this attention part takes rotations without a factor on cos and sin")
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        self.row_width = self.q_width + (0 if self.shared_cache else 2 * self.kv_width)
        self.v_dim = int(p.get("v_dim") or self.head_dim)
        self.qk_norm_eps = p.get("qk_norm_eps")
        self.sink, self.head_gate = bool(p.get("sink", False)), bool(p.get("head_gate", False))
        self.out_scale = float(p.get("out_scale", 1.0))
        self.extended = (self.v_dim != self.head_dim or self.qk_norm_eps is not None or self.sink or self.head_gate
                         or self.out_scale != 1.0 or self.position is None)
        if self.extended:
            if self.shared_cache or self.bias:
                raise ValueError("a shared cache or biases do not go with v_dim, qk_norm_eps, sink, head_gate or out_scale")
            if self.position is not None and not hasattr(self.position, "rotary_table"):
                raise ValueError("the extended attention path takes a rotation by a frequency table, or no position encoding")
            self.v_width, self.out_width = self.n_kv_heads * self.v_dim, self.n_heads * self.v_dim
            self.k_col, self.v_col = self.q_width, self.q_width + self.kv_width
            self.g_col = self.v_col + self.v_width
            self.row_width = self.g_col + (self.n_heads if self.head_gate else 0)
            self.row_pitch = -(-self.row_width // 8) * 8       # the attention kernels read query rows 16 bytes at a time

    def children(self):
        return [self.position] if self.position is not None else []

    def _extended_specs(self):
        specs = {"q_proj.weight": TensorSpec((self.q_width, self.hidden)),
                 "k_proj.weight": TensorSpec((self.kv_width, self.hidden)),
                 "v_proj.weight": TensorSpec((self.v_width, self.hidden))}
        if self.head_gate:
            specs["g_proj.weight"] = TensorSpec((self.n_heads, self.hidden))
        if self.sink:
            specs["sink"] = TensorSpec((self.n_heads,), "vector", "normal")
        specs["o_proj.weight"] = TensorSpec((self.hidden, self.out_width))
        return specs

    def tensor_specs(self):
        if self.extended:
            return self._extended_specs()
        specs = {"q_proj.weight": TensorSpec((self.q_width, self.hidden))}
        if not self.shared_cache:
            specs["k_proj.weight"] = TensorSpec((self.kv_width, self.hidden))
            specs["v_proj.weight"] = TensorSpec((self.kv_width, self.hidden))
        specs["o_proj.weight"] = TensorSpec((self.hidden, self.q_width))
        if self.bias:
            for name in [n for n in specs]:
                specs[name[:-len("weight")] + "bias"] = TensorSpec((specs[name].shape[0],), "vector", "normal")
        return specs

    MAX_HEAD_DIM = 256        # the plain attention kernel's limit (csrc/attention_simple.cu)

    def check_limits(self, rt):
        """Sizes no kernel of this library takes are refused when the engine is built, before
        anything is loaded (src/model/arch/llama/preflight.rs:35-42)."""
        if self.head_dim > self.MAX_HEAD_DIM:
            raise ValueError(f"head_dim {self.head_dim} is beyond the attention kernels' limit of {self.MAX_HEAD_DIM}")
        if self.v_dim > self.MAX_HEAD_DIM:
            raise ValueError(f"v_dim {self.v_dim} is beyond the attention kernels' limit of {self.MAX_HEAD_DIM}")

    def fused_tensors(self):
        # one product for q, k and v (and the heads' gate numbers)
        if self.shared_cache:
            return {}
        if self.extended:
            return {"qkv_proj.weight": ("q_proj.weight", "k_proj.weight", "v_proj.weight") + (("g_proj.weight",) if self.head_gate else ())}
        fused = {"qkv_proj.weight": ("q_proj.weight", "k_proj.weight", "v_proj.weight")}
        if self.bias:
            fused["qkv_proj.bias"] = ("q_proj.bias", "k_proj.bias", "v_proj.bias")
        return fused

    def device_tensors(self):
        return {"sink_f32": ((self.n_heads,), torch.float32), "sink_log2": ((self.n_heads,), torch.float32)} if self.sink else {}

    def kv_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window, v_dim=0 if self.v_dim == self.head_dim else self.v_dim)

    def state_need(self):
        return None

    def workspace(self):
        if self.extended:           # a buffer per geometry: rows of a shared, wider buffer would not be contiguous
            return {f"xqkv_{self.row_pitch}": (self.row_pitch, "act"), f"xattn_{self.out_width}": (self.out_width, "act")}
        return {"qkv": (self.row_width, "act"), "attn_out": (self.q_width, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        if self.position is not None and not self.position.tensor_specs():
            self.position.bind({}, rt)      # a position part with tensors of its own is bound by the model
        if self.extended:
            return self._bind_extended(tensors, rt)
        if self.shared_cache:
            fused = tensors["q_proj.weight"]
        elif "qkv_proj.weight" in tensors:
            fused = tensors["qkv_proj.weight"]        # the loader filled the one matrix (see fused_tensors)
        else:
            # bound by hand with three separate matrices: rows [q heads | k heads | v heads]
            fused = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                               tensors["v_proj.weight"]], dim=0).contiguous()
        fused_bias = None
        if self.bias:
            if self.shared_cache:
                fused_bias = tensors["q_proj.bias"]
            elif "qkv_proj.bias" in tensors:
                fused_bias = tensors["qkv_proj.bias"]
            else:
                fused_bias = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]]).contiguous()
        self._fast_ok = False
        if rt.attention == "fast":
            from .. import ops_tensor
            self._fast_ok = ops_tensor.attention_supported(self.n_heads, self.n_kv_heads, self.head_dim)
        self.qkv_proj = Linear(fused, rt, bias=fused_bias)
        self.o_proj = Linear(tensors["o_proj.weight"], rt, bias=tensors.get("o_proj.bias"))

    def _bind_extended(self, tensors, rt):
        names = ["q_proj.weight", "k_proj.weight", "v_proj.weight"] + (["g_proj.weight"] if self.head_gate else [])
        fused = tensors.get("qkv_proj.weight")
        if fused is None:
            fused = torch.cat([tensors[n] for n in names], dim=0).contiguous()
        self.qkv_proj = Linear(fused, rt)
        self.o_proj = Linear(tensors["o_proj.weight"], rt)
        self.sink_values = tensors.get("sink")
        self.sink_f32 = self.sink_log2 = None
        if self.sink:
            take = (lambda: rt.alloc((self.n_heads,), torch.float32)) if rt.alloc is not None else \
                   (lambda: torch.empty(self.n_heads, dtype=torch.float32, device=rt.device))
            self.sink_f32, self.sink_log2 = take(), take()
            self.sink_f32.copy_(self.sink_values.float())
            # the tensor-core attention kernels work in powers of two: the sinks times log2(e)
            self.sink_log2.copy_(self.sink_values.float() * 1.4426950408889634)
        self._fast_ok = False
        if rt.attention == "fast" and self.v_dim == self.head_dim:
            from .. import ops_tensor
            self._fast_ok = ops_tensor.attention_supported(self.n_heads, self.n_kv_heads, self.head_dim)
        self._tiled_ok = ops.attention_distance_tiled_fits(self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim)

    def _forward_extended(self, ctx, h, x, view, owns_cache):
        """One product for q, k, v and the gate numbers; one kernel rotates and norms q and k and writes the cache;
        attention on the tensor-core kernels where keys and values have one size they take (the sink is theirs, the
        gate a small kernel), else on the CUDA-core kernels, which take the sink, the gate and the scale themselves."""
        n = ctx.n_tokens
        row = ctx.buf(f"xqkv_{self.row_pitch}", self.row_pitch)
        out = ctx.buf(f"xattn_{self.out_width}", self.out_width)
        self.qkv_proj.store(h, row[:, :self.row_width], n)
        inv_freq, rotary_dim, interleaved = self.position.rotary_table() if self.position is not None else (None, 0, False)
        ops.qk_prepare(row, self.k_col, self.v_col, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, inv_freq, view.k, view.v,
                       view.page_table, view.max_pages, view.page_size, n, self.n_heads, self.n_kv_heads, self.head_dim,
                       self.v_dim, rotary_dim, interleaved, self.qk_norm_eps is not None, float(self.qk_norm_eps or 0.0),
                       owns_cache)
        gate = row[:, self.g_col:] if self.head_gate else None
        if self._fast_ok:
            from .. import ops_tensor
            ops_tensor.attention(ctx, row, view, out, self.n_heads, self.n_kv_heads, self.head_dim, self.window,
                                 self.scale, st=self.rt.tc, sink_log2=self.sink_log2)
            if gate is not None or self.out_scale != 1.0:
                ops.head_gate(out, gate, n, self.n_heads, self.v_dim, self.out_scale)
        else:
            # the 32-bit engine visits keys in position order, one warp per (token, head); the serving engine stages tiles
            tiled = self._tiled_ok and row.dtype != torch.float32
            ops.attention_distance(row, view.k, view.v, ctx, view.page_table, view.max_pages, view.page_size, None, gate,
                                   out, self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim, self.window, self.scale,
                                   tiled, sinks=self.sink_f32, gate_heads=True, out_scale=self.out_scale)
        self.o_proj.accumulate(out, x, n, defer=False)

    def forward(self, ctx, h, x, view, owns_cache=True):
        if self.extended:
            return self._forward_extended(ctx, h, x, view, owns_cache)
        n = ctx.n_tokens
        qkv = ctx.buf("qkv", self.row_width)
        out = ctx.buf("attn_out", self.q_width)
        write = owns_cache and not self.shared_cache
        if write and ctx.max_new == 1 and self._fast_ok and self._fusable(ctx, view):
            # single tokens: the attention kernel rotates q and k and writes the cache itself
            from .. import ops_tensor
            inv_freq, rotary_dim, interleaved = self.position.rotary_table()
            self.qkv_proj.store(h, qkv, n, defer=True)
            ops_tensor.attention_decode_rotary(ctx, qkv, view, out, self.n_heads, self.n_kv_heads, self.head_dim,
                                               self.window, self.scale, inv_freq, rotary_dim, interleaved, st=self.rt.tc)
            self.o_proj.accumulate(out, x, n)
            return
        self.qkv_proj.store(h, qkv, n, defer=getattr(self.position, "fuses_pending", False))
        self.position.encode_and_store(ctx, qkv, self.n_heads, self.n_kv_heads, self.head_dim, view, write)
        if self.rt.attention == "fast" and self._fast_ok:
            from .. import ops_tensor
            ops_tensor.attention(ctx, qkv, view, out, self.n_heads, self.n_kv_heads, self.head_dim,
                                 self.window, self.scale, st=self.rt.tc)
        else:
            if self.rt.gemm == "tensor":
                from .. import ops_tensor
                ops_tensor.flush_pending(qkv.device, self.rt.tc)
            ops.attention_simple(qkv, n, view.k, view.v, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                                 view.page_table, view.max_pages, view.page_size, out,
                                 self.n_heads, self.n_kv_heads, self.head_dim, self.window, self.scale)
        self.o_proj.accumulate(out, x, n)

    def _fusable(self, ctx, view) -> bool:
        """Whether this step's attention kernel should do the position encoding and the cache write
        itself.  It pays while the kernel's blocks have three warps or more (up to four blocks per SM).  Measured
        at the 8B layer shape, the chain of a layer with and without: batch 8 93.6 against 96.4 us; batch 32
        112.7 against 113.5, batch 64 136.6 against 138.2 (with the QKV product split four ways; with six it was
        the other way round, because every block adds up the projection's partial rows itself); batch 96 173.9
        against 163.3, batch 128 187.9 against 176.6 (blocks of one or two warps).  MDMA_FUSED_ROTARY=0 turns it
        off, for comparisons."""
        if self.rt.attention != "fast" or not hasattr(self.position, "rotary_table") or not FUSED_ROTARY:
            return False
        from .. import ops_tensor
        sms = self.rt.tc.sms if self.rt.tc is not None else 0
        return (ctx.n_seqs * self.n_kv_heads <= 4 * sms and
                ops_tensor.fused_rotary_supported(self.n_heads, self.n_kv_heads, self.head_dim, view.page_size,
                                                  self.position.rotary_table()[1]))

    def resident_tensors(self):
        extra = [self.sink_values] if self.extended else []
        return [t for t in [self.qkv_proj.w, self.o_proj.w, self.qkv_proj.bias, self.o_proj.bias] + extra if t is not None]
