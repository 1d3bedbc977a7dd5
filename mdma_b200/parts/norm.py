"""Norms.  Both read the float residual stream and write the compute dtype.

RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w (src/backend/cpu.rs:388-401;
no +1 on the weight, no mean subtraction); sums in float.  `add_normed` is the
same norm on a sublayer's result, added into the residual stream: x += norm(y).
With `groups` g > 1 the row is split into g equal consecutive parts and every part is divided
by its own sqrt(mean(part^2) + eps); the weight spans the whole row.

Dynamic tanh: y = tanh(alpha * x) * w + b with a learned scalar alpha; no mean,
no variance, nothing summed over the row.

Layer norm with a weight and no bias: y = (x - mean) / sqrt(var + eps) * w, var
the mean of the squared deviations; sums in float."""
from __future__ import annotations

from .. import ops
from ..registry import NORMS
from ..spec import TensorSpec
from .base import Part


@NORMS.register("rmsnorm")
class RMSNorm(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.eps = float(self.params["eps"])
        self.groups = int(self.params.get("groups", 1) or 1)
        if self.groups < 1 or self.width % self.groups:
            raise ValueError(f"a row of {self.width} numbers does not split into {self.groups} equal parts")
        if self.groups > 1:
            self.fuses_pending = False      # the grouped kernel reads complete rows of x

    def tensor_specs(self):
        return {"weight": TensorSpec((self.width,), "vector")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors["weight"]

    fuses_pending = True        # adds up a deferred K-split product on x itself

    def forward(self, ctx, x, out, rows=None, n_rows=None):
        n = n_rows if n_rows is not None else (None if rows is not None else ctx.n_tokens)
        if self.groups > 1:
            if self.rt.gemm == "tensor":
                from .. import ops_tensor
                ops_tensor.flush_pending(x.device, self.rt.tc)
            ops.group_rmsnorm(x, self.weight, self.eps, self.groups, out, rows, n)
            return
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            pend = ops_tensor.take_pending(x, ops.GEMM_ACCUMULATE, ctx.n_tokens, self.rt.tc) if rows is None else None
            if pend is not None:
                scratch, splits, stride = pend
                ops.rmsnorm(x, self.weight, self.eps, out, None, n, scratch, splits, stride)
                return
            ops_tensor.flush_pending(x.device, self.rt.tc)
        ops.rmsnorm(x, self.weight, self.eps, out, rows, n)

    def add_normed(self, ctx, y, x):
        """x += norm(y), both float rows: the norm on a sublayer's result.  Partial sums that a K-split product left
        of y are added up on the way."""
        partial, splits, stride = None, 0, 0
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            pend = ops_tensor.take_pending(y, ops.GEMM_ACCUMULATE, ctx.n_tokens, self.rt.tc)
            if pend is not None:
                partial, splits, stride = pend
            else:
                ops_tensor.flush_pending(y.device, self.rt.tc)
        if self.groups > 1:
            ops.group_rmsnorm_add(x, y, self.weight, self.eps, self.groups, ctx.n_tokens, partial, splits, stride)
            return
        ops.rmsnorm_add(x, y, self.weight, self.eps, ctx.n_tokens, partial, splits, stride)

    def resident_tensors(self):
        return [self.weight]


@NORMS.register("dyt")
class DynamicTanh(Part):
    """tanh(alpha * x) * w + b.  Because nothing is summed over a row, the arrangement that shifts
    tokens may ask for the shifted rows in the same pass (`forward_shifted`)."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])

    def tensor_specs(self):
        return {"weight": TensorSpec((self.width,), "vector"),
                "b": TensorSpec((self.width,), "vector", "zeros"),
                "alpha": TensorSpec((), "vector", "ones")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight, self.b, self.alpha = tensors["weight"], tensors["b"], tensors["alpha"]

    def forward(self, ctx, x, out, rows=None, n_rows=None):
        n = n_rows if n_rows is not None else (None if rows is not None else ctx.n_tokens)
        ops.dyt_norm(x, self.weight, self.b, self.alpha, out, rows, n)

    def forward_shifted(self, ctx, x, h, hs, mu, state):
        """h = norm(x) and hs = h + (h' - h) * mu, h' the normed row before (or the kept one)."""
        ops.dyt_shift(x, self.weight, self.b, self.alpha, mu, ctx.tok_seq, ctx.seq_start, ctx.seq_slot, state,
                      h, hs, ctx.n_tokens)

    def resident_tensors(self):
        return [self.weight, self.b, self.alpha]


@NORMS.register("layernorm")
class LayerNorm(Part):
    """(x - mean) / sqrt(var + eps) * w; no bias."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.eps = float(self.params["eps"])

    def tensor_specs(self):
        return {"weight": TensorSpec((self.width,), "vector")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors["weight"]

    def forward(self, ctx, x, out, rows=None, n_rows=None):
        n = n_rows if n_rows is not None else (None if rows is not None else ctx.n_tokens)
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            ops_tensor.flush_pending(x.device, self.rt.tc)
        ops.layernorm(x, self.weight, self.eps, out, rows, n)

    def resident_tensors(self):
        return [self.weight]
