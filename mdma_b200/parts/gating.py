"""Small parts around a sublayer: the token shift in front of a mixer, the gate
on a sublayer's result, and the junction that re-enters a looped stack.

Token shift: what the mixer reads is h_t + (h_(t-1) - h_t) * mu, mu a learned
vector, h the normed rows as the arrangement hands them out, h_(-1) = 0.  The
last h of a sequence is part of its state (`width` floats).

Residual gate: the sublayer's result is multiplied by sigmoid(W h + b) before
it is added to the residual stream.

Loop input: before a pass over a looped stack of layers, x <- W [x ; x0] + s_t,
x0 the embedding's output and s_t a learned vector per pass.

Loop add: the same place, without a matrix: x <- x + x0 (not before the first
pass), then x <- x + s_t.

Depth average: AFTER run i of the schedule, what goes on is a learned weighted
sum of the embedding's output X_0 and the results X_1 .. X_(i+1) of all runs so
far, x <- sum_j w[j] X_j; X_(i+1) is the run's result before this sum.
"""
from __future__ import annotations

import torch

from .. import ops
from ..registry import AUXILIARIES, JUNCTIONS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


@AUXILIARIES.register("token_shift")
class TokenShift(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])

    def tensor_specs(self):
        return {"mu": TensorSpec((self.width,), "vector", "normal")}

    def state_floats(self) -> int:
        return self.width

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.mu = tensors["mu"]

    def forward(self, ctx, h, hs, state):
        """hs = shifted h; `state` [slots, width] holds each sequence's last h of the step before."""
        ops.token_shift(h, self.mu, ctx.tok_seq, ctx.seq_start, ctx.seq_slot, state, hs, ctx.n_tokens)

    def keep(self, ctx, h, state):
        """After everything that reads the old state has run: each sequence's last h goes to the state."""
        ops.keep_last_rows(h, ctx.seq_start, ctx.seq_slot, state, ctx.n_seqs)

    def resident_tensors(self):
        return [self.mu]


@AUXILIARIES.register("residual_gate")
class ResidualGate(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])

    def tensor_specs(self):
        return {"weight": TensorSpec((self.width, self.width)), "bias": TensorSpec((self.width,), "vector", "normal")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.proj = Linear(tensors["weight"], rt, bias=tensors["bias"])

    def project(self, ctx, h, g):
        """g = W h + b (the sigmoid is taken where the gate is applied)."""
        self.proj.store(h, g, ctx.n_tokens)

    def apply(self, ctx, x, g, y, keep_rows=None, state=None):
        """x += sigmoid(g) * y; with `keep_rows`, each sequence's last row of it goes to `state` in the same pass.
        If the product that made y left K-split partial sums, they are added up here instead of in a launch of their own."""
        partial, splits, stride = None, 0, 0
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            pend = ops_tensor.take_pending(y, ops.GEMM_STORE, ctx.n_tokens, self.rt.tc)
            if pend is not None:
                partial, splits, stride = pend
            else:
                ops_tensor.flush_pending(y.device, self.rt.tc)
        if keep_rows is None:
            ops.gated_add(x, g, y, ctx.n_tokens, partial=partial, splits=splits, split_stride=stride)
        else:
            ops.gated_add(x, g, y, ctx.n_tokens, keep_rows, ctx.tok_seq, ctx.seq_start, ctx.seq_slot, state,
                          partial=partial, splits=splits, split_stride=stride)

    def resident_tensors(self):
        return [self.proj.w, self.proj.bias]


@JUNCTIONS.register("loop_input")
class LoopInput(Part):
    """x <- W [x ; x0] + step[t] before pass t of a looped stack.  W is [width, 2 width] with x's
    columns first; `step` is [passes, width]."""
    needs_embedding = True

    def __init__(self, spec):
        super().__init__(spec)
        self.width, self.passes = int(self.params["width"]), int(self.params["passes"])

    def tensor_specs(self):
        return {"in": TensorSpec((self.width, 2 * self.width)),
                "step": TensorSpec((self.passes, self.width), "vector", "normal")}

    def workspace(self):
        return {"loop_pair": (2 * self.width, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.step = tensors["step"]
        self.proj = [Linear(tensors["in"], rt, bias=self.step[t]) for t in range(self.passes)]

    def forward(self, ctx, x, x0, t: int):
        pair = ctx.buf("loop_pair", 2 * self.width)
        ops.pack_pair(x, x0, pair, ctx.n_tokens)
        self.proj[t].store(pair, x, ctx.n_tokens)

    def resident_tensors(self):
        return [self.proj[0].w, self.step] if self.proj else [self.step]


@JUNCTIONS.register("loop_add")
class LoopAdd(Part):
    """Before pass t of a looped stack: x <- (x + x0) + step[t] for t > 0, x <- x + step[0] for the first pass.
    `step` is [passes, width].  `add_input` off: only the pass's vector is added, x <- x + step[t], and the
    embedding's output is not kept."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width, self.passes = int(self.params["width"]), int(self.params["passes"])
        self.needs_embedding = bool(self.params.get("add_input", True))

    def tensor_specs(self):
        return {"step": TensorSpec((self.passes, self.width), "vector", "normal")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.step = tensors["step"]

    def forward(self, ctx, x, x0, t: int):
        ops.loop_add(x, x0 if (t > 0 and self.needs_embedding) else None, self.step[t], ctx.n_tokens)

    def resident_tensors(self):
        return [self.step]


@JUNCTIONS.register("depth_average")
class DepthAverage(Part):
    """After run `arg` of the schedule: x <- sum_{j=0..arg+1} w[j] X_j, with X_0 the embedding's output and X_(j+1)
    the result of run j as that run left it (before its own average).  `terms` = arg + 2 weights; `depth` = runs in the
    schedule, which sizes the per-token history [depth, width] of float rows.  Sums in float, terms in the order of j."""
    needs_embedding = True

    def __init__(self, spec):
        super().__init__(spec)
        self.width, self.terms, self.depth = int(self.params["width"]), int(self.params["terms"]), int(self.params["depth"])
        if not 2 <= self.terms <= self.depth + 1:
            raise ValueError(f"a depth average of {self.terms} terms in a schedule of {self.depth} runs")

    def tensor_specs(self):
        return {"weight": TensorSpec((self.terms,), "vector", "ones")}

    def workspace(self):
        return {f"depth_history_{self.depth}": (self.depth * self.width, "f32")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors["weight"]

    def forward(self, ctx, x, x0, run: int):
        if run + 2 != self.terms:
            raise ValueError(f"a depth average of {self.terms} terms was placed after run {run}")
        history = ctx.buf(f"depth_history_{self.depth}", self.depth * self.width, torch.float32)
        ops.depth_mix(x, x0, history, self.depth, run, self.weight, ctx.n_tokens)

    def resident_tensors(self):
        return [self.weight]
