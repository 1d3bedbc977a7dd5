"""Linear attention with a fixed decay per head (`linear_attention`), and a mixer made of two mixers side by
side (`side_by_side`).

Linear attention.  q = silu(Wq h), k = silu(Wk h) [heads x dim], v = silu(Wv h) [heads x v_dim]; per head

    S_t = decay_h S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t,

S [dim, v_dim] starting at zero, kept in float per sequence (the site's state) and carried from step to step.
The heads side by side are RMS-normed together with the weight `norm`, multiplied by sigmoid(Wg h), by the
constant `out_scale`, and projected by Wo.  The decays are parameters (one per head).  The activations, the state, the
sums over it, the norm and the gate are float in both engines; the projections are one product in the compute dtype.
The 32-bit engine and short portions walk row by row in one fixed order; single tokens in the serving engine update
the state row in place without staging it; the serving engine walks portions of
`CHUNKS_FROM` rows or more a chunk of rows at a time, and long ones in runs of `RUN_ROWS` rows side by side (the
recurrence is linear in S: every run's last state from zero, then the runs' starting states in order, then every
run from its start), if the scratch holds the runs' states.

Side by side.  Two mixers read the same rows and their results are added, each times a constant:
`left_scale * left(h) + right_scale * right(h)`.  A child that takes an `out_scale` applies its constant itself;
any other mixer runs into a scratch buffer that is then added.  At most one child keeps keys and values; the
children's states lie one after the other in the site's state row.
"""
from __future__ import annotations

import dataclasses

import torch

from .. import ops
from ..cache import StateNeed
from ..registry import MIXERS
from ..spec import PartSpec, TensorSpec
from .base import Part
from .linear import Linear


@MIXERS.register("linear_attention")
class LinearAttention(Part):
    graph_safe = True
    takes_out_scale = True
    CHUNKS_FROM = 16          # rows of a sequence in a step from which the serving engine walks chunk by chunk
    RUN_ROWS = 128            # rows of a run; sequences of two runs and more are walked as runs side by side

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim = int(p["num_heads"]), int(p["head_dim"])
        self.v_dim = int(p.get("v_dim") or self.dim)
        self.decay = [float(d) for d in p["decay"]]
        self.eps = float(p["eps"])
        self.out_scale = float(p.get("out_scale", 1.0))
        if len(self.decay) != self.heads:
            raise ValueError(f"{len(self.decay)} decays for {self.heads} heads")
        self.qk_width, self.v_width = self.heads * self.dim, self.heads * self.v_dim
        self.k_col, self.v_col, self.g_col = self.qk_width, 2 * self.qk_width, 2 * self.qk_width + self.v_width
        self.row_width = self.g_col + self.v_width

    def check_limits(self, rt):
        if self.v_dim > 256 or self.dim > 4096:
            raise ValueError(f"linear attention heads of {self.dim} x {self.v_dim} are beyond the kernels' limits")

    def tensor_specs(self):
        W = self.hidden
        return {"q": TensorSpec((self.qk_width, W)), "k": TensorSpec((self.qk_width, W)), "v": TensorSpec((self.v_width, W)),
                "g": TensorSpec((self.v_width, W)), "norm": TensorSpec((self.v_width,), "vector"),
                "o": TensorSpec((W, self.v_width))}

    def fused_tensors(self):
        return {"qkvg": ("q", "k", "v", "g")}

    def device_tensors(self):
        return {"decay": ((self.heads,), torch.float32)}

    def kv_need(self):
        return None

    def state_need(self):
        return StateNeed((self.heads * self.dim * self.v_dim,), torch.float32)

    def workspace(self):
        tag = f"{self.row_width}_{self.v_width}"
        return {f"lin_proj_{tag}": (self.row_width, "act"), f"lin_sum_{tag}": (self.v_width, "f32"),
                f"lin_out_{tag}": (self.v_width, "act"), f"lin_runs_{tag}_{self.dim}": (self._run_columns(), "f32")}

    def _run_columns(self) -> int:
        # scratch for the runs side by side: room for two runs' states per RUN_ROWS rows of a step
        return -(-2 * self.heads * self.dim * self.v_dim // self.RUN_ROWS)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        fused = tensors.get("qkvg")
        if fused is None:
            fused = torch.cat([tensors[n] for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.proj = Linear(fused, rt)
        self.norm = tensors["norm"]
        self.o = Linear(tensors["o"], rt)
        self.decay_dev = rt.derived(torch.tensor(self.decay, dtype=torch.float64).to(torch.float32))
        if not ops.linear_attention_fits(self.dim, self.v_dim):
            raise ValueError(f"linear attention heads of {self.dim} x {self.v_dim} do not fit the kernels' shared memory")
        self.chunks_fit = ops.linear_attention_fits(self.dim, self.v_dim, chunked=True)

    def forward(self, ctx, h, x, view, owns_cache=True):
        n = ctx.n_tokens
        tag = f"{self.row_width}_{self.v_width}"
        proj = ctx.buf(f"lin_proj_{tag}", self.row_width)
        sums = ctx.buf(f"lin_sum_{tag}", self.v_width, torch.float32)
        out = ctx.buf(f"lin_out_{tag}", self.v_width)
        self.proj.store(h, proj, n)
        # portions of prompts in the serving engine: a chunk of rows at a time, long ones as runs side by side if the
        # scratch holds their states (it does unless one long prompt comes with many short ones); else, and always in
        # the 32-bit engine, row by row
        chunked = self.chunks_fit and proj.dtype != torch.float32 and ctx.max_new >= self.CHUNKS_FROM
        run_rows, max_runs, scratch = 0, 1, None
        if chunked and ctx.max_new >= 2 * self.RUN_ROWS:
            runs = ctx.buf(f"lin_runs_{tag}_{self.dim}", self._run_columns(), torch.float32).view(-1)
            most = -(-ctx.max_new // self.RUN_ROWS)
            if ctx.n_seqs * most * self.heads * self.dim * self.v_dim <= runs.numel():
                run_rows, max_runs, scratch = self.RUN_ROWS, most, runs
        ops.linear_attention(proj, 0, self.k_col, self.v_col, self.decay_dev, ctx.seq_start, ctx.seq_slot, view.state, sums,
                             ctx.n_seqs, self.heads, self.dim, self.v_dim, chunked, run_rows, max_runs, scratch,
                             single=ctx.max_new == 1 and proj.dtype != torch.float32)
        ops.gated_rmsnorm(sums, proj[:, self.g_col:], self.norm, out, n, self.eps, self.out_scale)
        self.o.accumulate(out, x, n, defer=False)

    def resident_tensors(self):
        return [self.proj.w, self.norm, self.o.w]


@MIXERS.register("side_by_side")
class SideBySide(Part):
    """`left` and `right`: the children's PartSpecs; `left_scale`, `right_scale`: the constants on their results."""

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.members = []
        for side in ("left", "right"):
            child: PartSpec = p[side]
            scale = float(p.get(side + "_scale", 1.0))
            cls = MIXERS.get(child.kind)
            folded = bool(getattr(cls, "takes_out_scale", False)) or (child.kind == "attention")
            if folded:
                child = dataclasses.replace(child, params=dict(child.params, out_scale=scale))
            self.members.append((cls(child), scale, folded))
        if sum(1 for m, _, _ in self.members if m.kv_need() is not None) > 1:
            raise ValueError("of two mixers side by side only one can keep keys and values")
        for m, _, _ in self.members:
            need = m.state_need()
            if need is not None and need.dtype != torch.float32:
                raise ValueError("mixers side by side keep their states in float rows")

    @property
    def graph_safe(self):
        return all(getattr(m, "graph_safe", False) for m, _, _ in self.members)

    def children(self):
        return [m for m, _, _ in self.members]

    def attention_shapes(self):
        return [(m.n_heads, m.n_kv_heads, m.head_dim) for m, _, _ in self.members
                if all(hasattr(m, a) for a in ("n_heads", "n_kv_heads", "head_dim"))]

    def workspace(self):
        return {"side_scratch": (self.hidden, "f32")} if any(not folded for _, _, folded in self.members) else {}

    def kv_need(self):
        for m, _, _ in self.members:
            if m.kv_need() is not None:
                return m.kv_need()
        return None

    @staticmethod
    def _floats(m) -> int:
        """Floats of a child's state, rounded up to a multiple of four (every part starts on a 16-byte boundary)."""
        need = m.state_need()
        if need is None:
            return 0
        n = 1
        for d in need.shape:
            n *= int(d)
        return -(-n // 4) * 4

    def state_need(self):
        total = sum(self._floats(m) for m, _, _ in self.members)
        return StateNeed((total,), torch.float32) if total else None

    def forward(self, ctx, h, x, view, owns_cache=True):
        at = 0
        for m, scale, folded in self.members:
            floats = self._floats(m)
            own = dataclasses.replace(view, state=view.state[:, at:at + floats] if floats else None)
            at += floats
            if folded:
                m.forward(ctx, h, x, own, owns_cache)
                continue
            tmp = ctx.buf("side_scratch", self.hidden, torch.float32)
            tmp[:ctx.n_tokens].zero_()
            m.forward(ctx, h, tmp, own, owns_cache)
            if ctx.rt.gemm == "tensor":
                from .. import ops_tensor
                ops_tensor.flush_pending(tmp.device, ctx.rt.tc)
            ops.add_scaled(x, tmp, scale, ctx.n_tokens)
