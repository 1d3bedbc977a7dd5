"""Grouped-query causal attention whose heads' scores are mixed before the softmax.

q, k, v = h Wq^T (+ bq), h Wk^T (+ bk), h Wv^T (+ bv) with `bias`; with `qk_norm` every query and key head is divided
by its root mean square, x / sqrt(mean(x^2) + eps), and multiplied by a weight of `head_dim` numbers that all heads
share (tensors `q.norm`, `k.norm`), BEFORE the position encoding; the encoding turns the first `rotary_dim` numbers of
each head; k and v go to the cache (value heads of `v_dim` numbers).  A query at position p reads the keys up to p of
its own sequence, kv head = q head // (heads / kv heads).  With `talk`, the raw scores s_g = (q_g . k) * scale of all
query heads are mixed by a learned matrix T [heads, heads], s'_h = sum_g T[h, g] s_g, and head h takes the softmax of
s'_h.  `denominator_extra` c > 0 adds c to every softmax denominator (a key with score ln c and no value; 1 is a sink
whose score is 0).  The heads' results, concatenated, times Wo^T are added to the residual stream.

Scores, mixing and softmax are float in both engines.  Where the serving engine's tensor-core kernel takes the sizes,
the mixing is moved onto the queries: heads of one group share their key head, so s'_h = sum_c x_h,c . k_c with
x_h,c = scale * sum_{g in group c} T[h, g] q_g, one dot product of kv_heads * dim numbers against the token's key heads
side by side as the cache row holds them (x is formed in float and rounded once to bfloat16, the product sums in float).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..cache import KVNeed
from ..registry import MIXERS, POSITIONS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


@MIXERS.register("talking_attention")
class TalkingAttention(Part):
    graph_safe = True      # forward reads no host-side per-step values
    MAX_HEAD_DIM = 256     # the kernels' limits (csrc/attention_talking.cu)
    MAX_HEADS = 32

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads, self.n_kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.v_dim = int(p.get("v_dim") or self.head_dim)
        self.scale, self.eps = float(p["scale"]), float(p.get("eps", 0.0))
        self.window = int(p.get("window", 0) or 0)
        self.bias, self.qk_norm, self.talk = bool(p.get("bias", False)), bool(p.get("qk_norm", False)), bool(p.get("talk", False))
        self.extra = float(p.get("denominator_extra", 0.0) or 0.0)
        if self.extra < 0:
            raise ValueError("denominator_extra must not be negative")
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads do not divide over {self.n_kv_heads} kv heads")
        pos = p.get("position")
        self.position = POSITIONS.get(pos.kind)(pos) if pos is not None else None
        if self.position is not None and not hasattr(self.position, "rotary_table"):
            raise ValueError("this attention takes a rotation by a frequency table, or no position encoding")
        self.q_width, self.k_width = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        self.v_width, self.out_width = self.n_kv_heads * self.v_dim, self.n_heads * self.v_dim
        self.k_col, self.v_col = self.q_width, self.q_width + self.k_width
        self.row_width = self.v_col + self.v_width
        self.row_pitch = -(-self.row_width // 8) * 8
        # the tensor-core kernel works on queries mixed per kv group, side by side: kv_heads * dim numbers a head
        from ..ops_tensor import talking_attention_mma_warps
        self.mixed_width = self.n_heads * self.n_kv_heads * self.head_dim
        self._mma_shape = self.talk and talking_attention_mma_warps(self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim) > 0

    def children(self):
        return [self.position] if self.position is not None else []

    def check_limits(self, rt):
        if max(self.head_dim, self.v_dim) > self.MAX_HEAD_DIM:
            raise ValueError(f"head sizes {self.head_dim}/{self.v_dim} are beyond the attention kernels' limit of {self.MAX_HEAD_DIM}")
        if self.n_heads > self.MAX_HEADS:
            raise ValueError(f"{self.n_heads} heads are beyond the limit of {self.MAX_HEADS} of attention with mixed scores")

    def tensor_specs(self):
        specs = {"q": TensorSpec((self.q_width, self.hidden)), "k": TensorSpec((self.k_width, self.hidden)),
                 "v": TensorSpec((self.v_width, self.hidden))}
        if self.bias:
            for n in ("q", "k", "v"):
                specs[n + ".b"] = TensorSpec((specs[n].shape[0],), "vector", "normal")
        if self.qk_norm:
            specs["q.norm"] = TensorSpec((self.head_dim,), "vector")
            specs["k.norm"] = TensorSpec((self.head_dim,), "vector")
        if self.talk:
            specs["talk"] = TensorSpec((self.n_heads, self.n_heads), "vector", "normal")
        specs["o"] = TensorSpec((self.hidden, self.out_width))
        return specs

    def fused_tensors(self):
        fused = {"qkv": ("q", "k", "v")}
        if self.bias:
            fused["qkv.b"] = ("q.b", "k.b", "v.b")
        return fused

    def device_tensors(self):
        out = {}
        if self.talk:
            out["talk_f32"] = ((self.n_heads, self.n_heads), torch.float32)
        if self.extra > 0:
            out["sinks"] = ((self.n_heads,), torch.float32)
            out["sinks_log2"] = ((self.n_heads,), torch.float32)
        return out

    def kv_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window, v_dim=0 if self.v_dim == self.head_dim else self.v_dim)

    def state_need(self):
        return None

    def workspace(self):
        out = {f"tqkv_{self.row_pitch}": (self.row_pitch, "act"), f"tattn_{self.out_width}": (self.out_width, "act")}
        if self._mma_shape:
            out[f"tmixed_{self.mixed_width}"] = (self.mixed_width, "act")
        return out

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        if self.position is not None:
            self.position.bind({}, rt)
        fused = tensors.get("qkv")
        if fused is None:
            fused = torch.cat([tensors[n] for n in ("q", "k", "v")], dim=0).contiguous()
        fused_bias = None
        if self.bias:
            fused_bias = tensors.get("qkv.b")
            if fused_bias is None:
                fused_bias = torch.cat([tensors[n + ".b"] for n in ("q", "k", "v")]).contiguous()
        self.qkv = Linear(fused, rt, bias=fused_bias)
        self.o = Linear(tensors["o"], rt)
        self.q_weight, self.k_weight = tensors.get("q.norm"), tensors.get("k.norm")
        self.talk_values = tensors.get("talk")
        take = rt.alloc if rt.alloc is not None else (lambda shape, dt: torch.zeros(shape, dtype=dt, device=fused.device))
        self.talk_f32 = self.sinks = self.sinks_log2 = None
        if self.talk:
            self.talk_f32 = take((self.n_heads, self.n_heads), torch.float32)      # the mixing is done in float
            self.talk_f32.copy_(self.talk_values.float())
        if self.extra > 0:
            self.sinks = take((self.n_heads,), torch.float32)
            self.sinks.fill_(math.log(self.extra))
            self.sinks_log2 = take((self.n_heads,), torch.float32)      # the tensor-core kernel works in powers of two
            self.sinks_log2.fill_(math.log2(self.extra))
        self._tiled_ok = ops.talking_attention_tiled_fits(self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim)

    def forward(self, ctx, h, x, view, owns_cache=True):
        n = ctx.n_tokens
        row = ctx.buf(f"tqkv_{self.row_pitch}", self.row_pitch)
        out = ctx.buf(f"tattn_{self.out_width}", self.out_width)
        self.qkv.store(h, row[:, :self.row_width], n)
        inv_freq, rotary_dim, interleaved = self.position.rotary_table() if self.position is not None else (None, 0, False)
        magnitude = float(getattr(self.position, "magnitude", 1.0))
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            ops_tensor.flush_pending(row.device, self.rt.tc)
        ops.qk_norm_rotate(row, self.k_col, self.v_col, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, inv_freq, magnitude,
                           self.q_weight, self.k_weight, self.qk_norm, self.eps, view.k, view.v, view.page_table,
                           view.max_pages, view.page_size, n, self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim,
                           rotary_dim, interleaved, owns_cache)
        if self._mma_shape and self.rt.attention == "fast" and row.dtype == torch.bfloat16:
            from .. import ops_tensor
            mixed = ctx.buf(f"tmixed_{self.mixed_width}", self.mixed_width)
            splits, partial = 1, None
            if ctx.max_new == 1:
                # single tokens: the keys are divided over blocks.  The sums go through the rows of the mixed-query buffer
                # that a step of single tokens cannot reach (it has a row per token of a pass, a step of single tokens
                # uses a row per sequence); where those do not hold them, the keys stay whole.
                most = int(getattr(ctx, "most_seqs", None) or ctx.n_seqs)
                sms = self.rt.tc.sms if self.rt.tc is not None else 148
                splits = ops_tensor.talking_attention_splits(most, self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim, sms)
                spare = (mixed.shape[0] - most) * self.mixed_width // 2            # floats behind the rows in use
                if splits > 1 and mixed.is_contiguous() and spare >= most * self.n_heads * splits * (self.v_dim + 2):
                    partial = mixed.view(-1)[most * self.mixed_width:].view(torch.float32)
                else:
                    splits = 1
            ops_tensor.talking_attention_mma(ctx, row, self.talk_f32, mixed, view, self.sinks_log2, out, self.n_heads,
                                             self.n_kv_heads, self.head_dim, self.v_dim, self.window, self.scale, st=self.rt.tc,
                                             splits=splits, partial=partial)
            self.o.accumulate(out, x, n)
            return
        # the 32-bit engine visits keys in position order, a block per token; the serving engine stages tiles
        tiled = self._tiled_ok and row.dtype != torch.float32
        ops.talking_attention(row, view.k, view.v, self.talk_f32, self.sinks, ctx, view.page_table, view.max_pages,
                              view.page_size, out, self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim, self.window,
                              self.scale, tiled=tiled)
        self.o.accumulate(out, x, n)

    def resident_tensors(self):
        return [t for t in (self.qkv.w, self.qkv.bias, self.o.w, self.q_weight, self.k_weight, self.talk_values)
                if t is not None]
