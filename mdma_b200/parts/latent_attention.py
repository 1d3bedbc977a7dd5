"""Attention over a cached latent, without positions.

q = Wq h (heads x dim); c = rms_unit(Wdkv h) * w, `kv_rank` numbers, the only thing the
cache keeps of a token; per head k = Wuk c and v = Wuv c; a query at position p sees every
key up to p; score = (q . k) * scale; the softmax's denominator also holds exp(sink_h), a
learned number per head with no key and no value; the heads' results go through Wo.

Computed in the absorbed form: q'_h = Wuk,h^T q_h lives in the latent space, so that
score = q'_h . c and o_h = Wuv,h (sum_j p_j c_j); the cache is read as one shared head of
size kv_rank that serves as key and as value, whatever the number of heads.

`rotary_latent_attention` is the form with positions: the queries come from a latent of their own,
cq = rms_unit(Wdq h) * w, q = Wuq cq, each head [dim plain | rot_dim turned]; Wdkv h has kv_rank + rot_dim
numbers, the first kv_rank normed into c, the last rot_dim turned by the position into one key part r that
all heads share; score = (q_plain . Wuk,h c + q_turned . r) * scale.  The cache keeps [c | r] per token.  In
the absorbed form the query of head h in the cache's space is [Wuk,h^T q_plain | q_turned] and the score its
dot product with the cached vector; the weighted sum of cached vectors is taken whole and Wuv,h reads its
first kv_rank numbers.  Options: `sink` (a learned number per head in the softmax's denominator), `gate`
("element": the heads' results times sigmoid(Wg h), a number per number; "head": one number per head),
`shared_cache` (the site reads another site's cached vectors and has no Wdkv).
"""
from __future__ import annotations

import dataclasses

import torch

from .. import ops
from ..cache import KVNeed
from ..registry import MIXERS, POSITIONS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


class HeadwiseLinear:
    """out[:, h*N:(h+1)*N] = a[:, h*K:(h+1)*K] @ w[h].T for every head h; w is [heads, N, K].  Steps of
    many tokens (256 or more) run head by head on the tensor cores when the shapes allow, others as one
    launch on the CUDA cores."""

    TENSOR_TOKENS = 256       # below this a launch per head costs more than the CUDA-core launch for all heads

    def __init__(self, w: torch.Tensor, rt):
        self.w, self.rt = w, rt
        self.heads, self.n, self.k = w.shape
        self._tensor_ok = False
        if rt.gemm == "tensor" and w.dtype == torch.bfloat16:
            from .. import ops_tensor
            self._tensor_ok = ops_tensor.gemm_supported(self.n, self.k) and self.n % 8 == 0

    def run(self, a, out, m):
        if (self._tensor_ok and m >= self.TENSOR_TOKENS and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
                and out.dtype == torch.bfloat16):
            from .. import ops_tensor
            for h in range(self.heads):
                ops_tensor.gemm(a[:, h * self.k:(h + 1) * self.k], self.w[h], out[:, h * self.n:(h + 1) * self.n],
                                ops.GEMM_STORE, None, m, st=self.rt.tc)
            return
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            ops_tensor.flush_pending(a.device, self.rt.tc)
        ops.gemm_simt_batched(a, self.w, out, m)


@MIXERS.register("latent_attention")
class LatentAttention(Part):
    graph_safe = True      # forward reads no host-side per-step values
    MAX_RANK = 1024        # the attention kernel's limit (csrc/latent_attention.cu)

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads, self.dim, self.vdim, self.rank = int(p["heads"]), int(p["dim"]), int(p["vdim"]), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.window = int(p.get("window", 0) or 0)
        # as the attention kernels and the engine's scratch plan see it: every head reads one shared head of the cache
        self.n_kv_heads, self.head_dim = 1, self.rank
        self.q_width, self.v_width, self.lat_width = self.n_heads * self.dim, self.n_heads * self.vdim, self.n_heads * self.rank

    def check_limits(self, rt):
        if self.rank > self.MAX_RANK:
            raise ValueError(f"kv_rank {self.rank} is beyond the attention kernel's limit of {self.MAX_RANK}")

    def tensor_specs(self):
        return {"q": TensorSpec((self.q_width, self.hidden)), "dkv": TensorSpec((self.rank, self.hidden)),
                "dkv.norm": TensorSpec((self.rank,), "vector"),
                "uk": TensorSpec((self.q_width, self.rank)), "uv": TensorSpec((self.v_width, self.rank)),
                "sink": TensorSpec((self.n_heads,), "vector", "zeros"), "o": TensorSpec((self.hidden, self.v_width))}

    def fused_tensors(self):
        return {"q_dkv": ("q", "dkv")}           # one product for the queries and the latent

    def device_tensors(self):
        # the keys' map per head, transposed, so that it is applied to the queries as an ordinary product
        # (counted at four bytes an element: the plan is made before the compute dtype is known to the part)
        return {"uk_t": ((self.n_heads, self.rank, self.dim), torch.float32),
                "sink_log2": ((self.n_heads,), torch.float32)}

    def kv_need(self):
        return KVNeed(1, self.rank, self.window, values=False)

    def state_need(self):
        return None

    def _names(self):
        tag = f"{self.n_heads}_{self.dim}_{self.vdim}_{self.rank}"
        return f"latent_proj_{tag}", f"latent_q_{tag}", f"latent_o_{tag}", f"latent_v_{tag}"

    def workspace(self):
        proj, q, o, v = self._names()
        return {proj: (self.q_width + self.rank, "act"), q: (self.lat_width, "act"), o: (self.lat_width, "act"),
                v: (self.v_width, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        fused = tensors.get("q_dkv")
        if fused is None:
            fused = torch.cat([tensors["q"], tensors["dkv"]], dim=0).contiguous()
        self.q_dkv = Linear(fused, rt)
        self.o = Linear(tensors["o"], rt)
        self.latent_norm, self.sink = tensors["dkv.norm"], tensors["sink"]
        uk = self.uk = tensors["uk"]
        shape = (self.n_heads, self.rank, self.dim)
        uk_t = rt.alloc(shape, uk.dtype) if rt.alloc is not None else torch.empty(shape, dtype=uk.dtype, device=uk.device)
        uk_t.copy_(uk.view(self.n_heads, self.dim, self.rank).transpose(1, 2))
        self.absorb = HeadwiseLinear(uk_t, rt)
        # the tensor-core attention kernels work in powers of two: the sinks times log2(e), as floats
        self.sink_log2 = (rt.alloc((self.n_heads,), torch.float32) if rt.alloc is not None
                          else torch.empty(self.n_heads, dtype=torch.float32, device=uk.device))
        self.sink_log2.copy_(self.sink.float() * 1.4426950408889634)
        self._fast_ok = False
        if rt.attention == "fast":
            from .. import ops_tensor
            self._fast_ok = ops_tensor.attention_supported(self.n_heads, 1, self.rank) and self.scale > 0
        self.expand = HeadwiseLinear(tensors["uv"].view(self.n_heads, self.vdim, self.rank), rt)

    def forward(self, ctx, h, x, view, owns_cache=True):
        self._run(ctx, h, x, view, owns_cache, accumulate=True)

    def produce(self, ctx, h, out, view, owns_cache=True, defer=False):
        """`defer`: the last product may leave K-split partial sums of `out` for the caller's next kernel."""
        self._run(ctx, h, out, view, owns_cache, accumulate=False, defer=defer)

    def _run(self, ctx, h, target, view, owns_cache, accumulate, defer=False):
        n = ctx.n_tokens
        names = self._names()
        proj = ctx.buf(names[0], self.q_width + self.rank)
        q_lat, o_lat, v = ctx.buf(names[1], self.lat_width), ctx.buf(names[2], self.lat_width), ctx.buf(names[3], self.v_width)
        self.q_dkv.store(h, proj, n)
        if owns_cache:
            ops.latent_norm_store(proj, self.q_width, self.latent_norm, self.eps, self.rank, ctx.tok_seq, ctx.tok_pos,
                                  ctx.seq_slot, view.page_table, view.max_pages, view.page_size, view.k, n)
        self.absorb.run(proj, q_lat, n)
        if self._fast_ok:
            # the latent rows serve as the one key head and as the one value head
            from .. import ops_tensor
            ops_tensor.attention(ctx, q_lat, dataclasses.replace(view, v=view.k), o_lat, self.n_heads, 1, self.rank,
                                 self.window, self.scale, st=self.rt.tc, sink_log2=self.sink_log2)
        else:
            if self.rt.gemm == "tensor":
                from .. import ops_tensor
                ops_tensor.flush_pending(q_lat.device, self.rt.tc)
            ops.latent_attention(q_lat, view.k, self.sink, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, view.page_table,
                                 view.max_pages, view.page_size, o_lat, n, self.n_heads, self.rank, self.window, self.scale)
        self.expand.run(o_lat, v, n)
        if accumulate:
            self.o.accumulate(v, target, n, defer=False)
        else:
            self.o.store(v, target, n, defer=defer)

    def resident_tensors(self):
        return [self.q_dkv.w, self.o.w, self.latent_norm, self.sink, self.uk, self.expand.w]


@MIXERS.register("rotary_latent_attention")
class RotaryLatentAttention(Part):
    graph_safe = True      # forward reads no host-side per-step values
    MAX_RANK = LatentAttention.MAX_RANK

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads, self.dim, self.rot_dim = int(p["heads"]), int(p["dim"]), int(p["rot_dim"])
        self.vdim, self.rank, self.q_rank = int(p["vdim"]), int(p["kv_rank"]), int(p["q_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.sink = bool(p.get("sink", False))
        self.gate = p.get("gate")
        if self.gate not in (None, "element", "head"):
            raise ValueError(f"unknown gate {self.gate!r} (have 'element', 'head' or None)")
        self.shared_cache = bool(p.get("shared_cache", False))
        pos = p["position"]
        self.position = POSITIONS.get(pos.kind)(pos)
        if not hasattr(self.position, "rotary_table"):
            raise ValueError("the turned key part takes a rotation by a frequency table")
        if self.position.rotary_dim > self.rot_dim:
            raise ValueError(f"{self.position.rotary_dim} turned numbers do not fit a key part of {self.rot_dim}")
        # as the attention kernels and the engine's scratch plan see it: one shared head of cached vectors
        self.row = self.rank + self.rot_dim                  # a cached vector: [latent | turned key part]
        self.head_in = self.dim + self.rot_dim               # a query head as Wuq makes it
        self.n_kv_heads, self.head_dim = 1, self.row
        self.q_width, self.v_width, self.lat_width = self.n_heads * self.head_in, self.n_heads * self.vdim, self.n_heads * self.row
        self.g_width = {None: 0, "element": self.v_width, "head": self.n_heads}[self.gate]
        self.kv_col = self.q_rank
        self.g_col = self.q_rank + (0 if self.shared_cache else self.row)
        self.proj_width = self.g_col + self.g_width
        self.proj_pitch = -(-self.proj_width // 8) * 8

    def children(self):
        return [self.position]

    def check_limits(self, rt):
        if self.row > self.MAX_RANK:
            raise ValueError(f"kv_rank + rot_dim = {self.row} is beyond the attention kernel's limit of {self.MAX_RANK}")

    def tensor_specs(self):
        specs = {"dq": TensorSpec((self.q_rank, self.hidden)), "dq.norm": TensorSpec((self.q_rank,), "vector"),
                 "uq": TensorSpec((self.q_width, self.q_rank))}
        if not self.shared_cache:
            specs["dkv"] = TensorSpec((self.row, self.hidden))
            specs["dkv.norm"] = TensorSpec((self.rank,), "vector")
        specs["uk"] = TensorSpec((self.n_heads * self.dim, self.rank))
        specs["uv"] = TensorSpec((self.v_width, self.rank))
        if self.sink:
            specs["sink"] = TensorSpec((self.n_heads,), "vector", "zeros")
        if self.gate:
            specs["g"] = TensorSpec((self.g_width, self.hidden))
        specs["o"] = TensorSpec((self.hidden, self.v_width))
        return specs

    def _fused_names(self):
        return ("dq",) + (() if self.shared_cache else ("dkv",)) + (("g",) if self.gate else ())

    def fused_tensors(self):
        return {"down": self._fused_names()}      # one product for both latents and the gate

    def device_tensors(self):
        # counted at four bytes an element: the plan is made before the compute dtype is known to the part
        out = {"uk_x": ((self.n_heads, self.row, self.head_in), torch.float32),
               "uv_x": ((self.n_heads, self.vdim, self.row), torch.float32)}
        if self.sink:
            out["sink_log2"] = ((self.n_heads,), torch.float32)
        return out

    def kv_need(self):
        return KVNeed(1, self.row, 0, values=False)

    def state_need(self):
        return None

    def _names(self):
        tag = f"{self.n_heads}_{self.dim}_{self.rot_dim}_{self.vdim}_{self.rank}_{self.q_rank}_{self.proj_pitch}"
        return tuple(f"rlat_{n}_{tag}" for n in ("proj", "cq", "q", "ql", "ol", "v"))

    def workspace(self):
        proj, cq, q, ql, ol, v = self._names()
        return {proj: (self.proj_pitch, "act"), cq: (self.q_rank, "act"), q: (self.q_width, "act"),
                ql: (self.lat_width, "act"), ol: (self.lat_width, "act"), v: (self.v_width, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.position.bind({}, rt)
        fused = tensors.get("down")
        if fused is None:
            fused = torch.cat([tensors[n] for n in self._fused_names()], dim=0).contiguous()
        self.down = Linear(fused, rt)
        self.uq = Linear(tensors["uq"], rt)
        self.o = Linear(tensors["o"], rt)
        self.q_norm, self.kv_norm = tensors["dq.norm"], tensors.get("dkv.norm")
        self.sink_values = tensors.get("sink")
        uk, uv = tensors["uk"], tensors["uv"]
        self.uk, self.uv = uk, uv
        take = rt.alloc if rt.alloc is not None else (lambda shape, dt: torch.zeros(shape, dtype=dt, device=uk.device))
        H, R, D, r = self.n_heads, self.rank, self.dim, self.rot_dim
        # [Wuk,h^T 0; 0 I]: the plain part of a query head goes into the latent's space, the turned part is kept
        uk_x = take((H, self.row, self.head_in), uk.dtype)
        uk_x.zero_()
        uk_x[:, :R, :D].copy_(uk.view(H, D, R).transpose(1, 2))
        uk_x[:, R:, D:].copy_(torch.eye(r, dtype=uk.dtype, device=uk.device).expand(H, r, r))
        # [Wuv,h 0]: the values' map reads the latent part of the weighted sum of cached vectors
        uv_x = take((H, self.vdim, self.row), uv.dtype)
        uv_x.zero_()
        uv_x[:, :, :R].copy_(uv.view(H, self.vdim, R))
        self.absorb, self.expand = HeadwiseLinear(uk_x, rt), HeadwiseLinear(uv_x, rt)
        self.sink_log2 = None
        if self.sink:
            # the tensor-core attention kernels work in powers of two: the sinks times log2(e), as floats
            self.sink_log2 = take((H,), torch.float32)
            self.sink_log2.copy_(self.sink_values.float() * 1.4426950408889634)
        self._fast_ok = False
        if rt.attention == "fast":
            from .. import ops_tensor
            self._fast_ok = ops_tensor.attention_supported(H, 1, self.row) and self.scale > 0

    def forward(self, ctx, h, x, view, owns_cache=True):
        if owns_cache == self.shared_cache:
            raise ValueError("a site with a Wdkv of its own writes its cache; one without reads another site's")
        n = ctx.n_tokens
        names = self._names()
        proj, cq, q = ctx.buf(names[0], self.proj_pitch), ctx.buf(names[1], self.q_rank), ctx.buf(names[2], self.q_width)
        q_lat, o_lat, v = ctx.buf(names[3], self.lat_width), ctx.buf(names[4], self.lat_width), ctx.buf(names[5], self.v_width)
        inv_freq, rotary_dim, interleaved = self.position.rotary_table()
        magnitude = float(getattr(self.position, "magnitude", 1.0))
        self.down.store(h, proj[:, :self.proj_width], n)
        ops.latent_prepare(proj, 0, self.q_rank, self.q_norm, self.kv_col, self.rank, self.kv_norm, self.eps, self.rot_dim,
                           rotary_dim, interleaved, inv_freq, magnitude, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                           view.page_table, view.max_pages, view.page_size, cq, view.k, owns_cache, n)
        self.uq.store(cq, q, n)
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            ops_tensor.flush_pending(q.device, self.rt.tc)
        ops.rotate_heads(q, self.n_heads, self.head_in, self.dim, rotary_dim, interleaved, inv_freq, magnitude, ctx.tok_pos, n)
        self.absorb.run(q, q_lat, n)
        if self._fast_ok:
            # the cached vectors serve as the one key head and as the one value head
            from .. import ops_tensor
            ops_tensor.attention(ctx, q_lat, dataclasses.replace(view, v=view.k), o_lat, self.n_heads, 1, self.row,
                                 0, self.scale, st=self.rt.tc, sink_log2=self.sink_log2)
        else:
            if self.rt.gemm == "tensor":
                from .. import ops_tensor
                ops_tensor.flush_pending(q_lat.device, self.rt.tc)
            ops.latent_attention(q_lat, view.k, self.sink_values, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, view.page_table,
                                 view.max_pages, view.page_size, o_lat, n, self.n_heads, self.row, 0, self.scale)
        self.expand.run(o_lat, v, n)
        if self.gate == "element":
            ops.sigmoid_gate(v, proj[:, self.g_col:self.g_col + self.g_width], n)
        elif self.gate == "head":
            ops.head_gate(v, proj[:, self.g_col:self.g_col + self.g_width], n, self.n_heads, self.vdim, 1.0)
        self.o.accumulate(v, x, n)

    def resident_tensors(self):
        return [t for t in (self.down.w, self.uq.w, self.o.w, self.q_norm, self.kv_norm, self.sink_values, self.uk, self.uv,
                            self.absorb.w, self.expand.w) if t is not None]
