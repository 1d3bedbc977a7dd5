"""A feed-forward of many small gated feed-forwards of which each token uses a few (`routed_mlp`).

Router, in float:  z = R h over all routed outputs, s = softmax(z) (`scoring` "sigmoid": s = sigmoid(z), each
on its own), choice scores c = s + correction (`correction` off: c = s).
The routed outputs form `groups` equal groups of neighbours; a group's score is the sum of its `group_top`
largest c (1, the default: its largest), and only
members of the `keep_groups` best groups can be chosen (the others count as minus infinity).  The
`top` eligible outputs with the largest c are chosen; their weights are their s divided by the sum of
the chosen s (+ 1e-20), or with `renormalize` off their s as they are.  The first `experts` routed outputs are experts,
D_e (silu(G_e h) * (U_e h)), or with `activation` "swish_limit" D_e (g sigmoid(act_alpha g) (u + 1)) where
g = min(G_e h, act_limit) and u = U_e h kept within +-act_limit;
the last `identity` ones have no matrices and return h itself.  The result is the weighted sum.  A
shared expert of the same form (`shared_ff` > 0) runs for every token and is added, multiplied by
sigmoid(g . h), one number per token (`shared_gate`).

Tensors: `e<i>.gate|up|down`, `router` [experts + identity, width], `correction` [experts + identity],
`shared.gate|up|down`, `shared.sg` [1, width].  The experts' matrices are laid out as three stacked
matrices, so that a kernel finds expert e at a row offset.

Steps of few tokens read each chosen expert's matrices token by token; steps of many tokens sort the
(token, choice) pairs by expert on the device and compute expert by expert.  Nothing is read on the host
there.  Prompts of the serving engine (steps of `PRODUCTS_FROM` tokens or more that are not a replayed
decode step) gather each expert's input rows and run ONE tensor-core product pair per expert over its
run of rows; how many rows an expert got is read back from the device for that (the only host read of
this part; a replayed step never takes this way).
"""
from __future__ import annotations

import torch

from .. import ops
from ..registry import FEED_FORWARDS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


@FEED_FORWARDS.register("routed_mlp")
class RoutedMLP(Part):
    graph_safe = True
    MAX_ROUTED, MAX_TOP = 1024, 32       # the router kernel's limits
    SORTED_FROM = 33                     # tokens in a step from which the serving engine computes expert by expert
    PRODUCTS_FROM = 128                  # tokens in a step from which it does so with a matrix product per expert

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_experts, self.n_identity = int(p["experts"]), int(p.get("identity", 0) or 0)
        self.ff, self.top = int(p["intermediate_size"]), int(p["top"])
        self.groups, self.keep_groups = int(p.get("groups", 1) or 1), int(p.get("keep_groups", 0) or 0)
        self.keep_groups = self.keep_groups or self.groups
        self.shared_ff = int(p.get("shared_ff", 0) or 0)
        self.shared_gate = bool(p.get("shared_gate", True)) and self.shared_ff > 0
        self.correction = bool(p.get("correction", True))
        self.scoring = str(p.get("scoring", "softmax"))
        self.group_top = int(p.get("group_top", 1) or 1)
        self.renormalize = bool(p.get("renormalize", True))
        self.activation = str(p.get("activation", "silu"))
        self.act_limit, self.act_alpha = float(p.get("act_limit", 0.0) or 0.0), float(p.get("act_alpha", 1.0))
        if self.scoring not in ("softmax", "sigmoid") or not 1 <= self.group_top <= 8:
            raise ValueError(f"router scoring {self.scoring!r} with groups scored by their {self.group_top} largest is not implemented")
        if self.activation not in ("silu", "gelu_tanh", "gelu", "swish_limit"):
            raise ValueError(f"expert activation {self.activation!r} is not implemented")
        self.pair_act = ops.ACTIVATIONS[self.activation]
        self.n_routed = self.n_experts + self.n_identity
        if not 0 < self.top <= min(self.n_routed, self.MAX_TOP) or self.n_routed > self.MAX_ROUTED:
            raise ValueError(f"top {self.top} of {self.n_routed} routed outputs is outside the router kernel's limits "
                             f"({self.MAX_TOP} of {self.MAX_ROUTED})")
        if self.n_routed % self.groups or not 1 <= self.keep_groups <= self.groups:
            raise ValueError(f"{self.n_routed} routed outputs do not form {self.groups} groups of which {self.keep_groups} are kept")

    def tensor_specs(self):
        W, F = self.hidden, self.ff
        specs = {}
        for e in range(self.n_experts):
            specs[f"e{e}.gate"] = TensorSpec((F, W))
            specs[f"e{e}.up"] = TensorSpec((F, W))
            specs[f"e{e}.down"] = TensorSpec((W, F))
        specs["router"] = TensorSpec((self.n_routed, W))
        if self.correction:
            specs["correction"] = TensorSpec((self.n_routed,), "vector", "zeros")
        if self.shared_ff:
            specs["shared.gate"] = TensorSpec((self.shared_ff, W))
            specs["shared.up"] = TensorSpec((self.shared_ff, W))
            specs["shared.down"] = TensorSpec((W, self.shared_ff))
            if self.shared_gate:
                specs["shared.sg"] = TensorSpec((1, W))
        return specs

    def fused_tensors(self):
        if not self.n_experts:
            return {}
        return {f"experts.{part}": tuple(f"e{e}.{part}" for e in range(self.n_experts)) for part in ("gate", "up", "down")}

    def device_tensors(self):
        return {"first": ((2 * (self.n_experts + 1),), torch.int32)}          # the experts' starts in the sorted list, and counters

    def _names(self):
        tag = f"{self.top}_{self.ff}_{self.hidden}"
        return (f"routed_chosen_{tag}", f"routed_weight_{tag}", f"routed_order_{tag}", f"routed_act_{tag}",
                f"routed_y_{tag}", f"routed_shared_{self.shared_ff}", "routed_scale", f"routed_where_{tag}",
                f"routed_rows_{tag}")

    def workspace(self):
        chosen, weight, order, act, y, shared, scale, where, rows = self._names()
        ws = {chosen: (self.top, "f32"), weight: (self.top, "f32"), order: (self.top, "f32"), where: (self.top, "f32"),
              act: (self.top * self.ff, "act"), y: (self.top * self.hidden, "f32"), scale: (1, "f32"),
              rows: (self.top * self.hidden, "act")}
        if self.shared_ff:
            ws[shared] = (self.shared_ff, "act")
        return ws

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w_gate = self.w_up = self.w_down = None
        if self.n_experts:
            stacked = {}
            for part in ("gate", "up", "down"):
                t = tensors.get(f"experts.{part}")
                if t is None:
                    t = torch.cat([tensors[f"e{e}.{part}"] for e in range(self.n_experts)], dim=0).contiguous()
                stacked[part] = t
            self.w_gate, self.w_up, self.w_down = stacked["gate"], stacked["up"], stacked["down"]
        self.router = tensors["router"]
        self.correction_values = tensors.get("correction")
        self.shared_up = self.shared_down = self.sg = None
        if self.shared_ff:
            self.shared_up = Linear(tensors["shared.gate"], rt, tensors["shared.up"], activation=self.activation,
                                    act_limit=self.act_limit, act_alpha=self.act_alpha)
            self.shared_down = Linear(tensors["shared.down"], rt)
            if self.shared_gate:
                self.sg = tensors["shared.sg"].reshape(-1)
        self.first = rt.derived(torch.zeros(2 * (self.n_experts + 1), dtype=torch.int32))
        # long prompts in the serving engine: a tensor-core product pair per expert over its run of gathered rows
        self.by_products = False
        if self.n_experts and rt.gemm == "tensor" and self.w_gate.dtype == torch.bfloat16:
            from .. import ops_tensor
            self.by_products = (ops_tensor.gemm_supported(self.ff, self.hidden) and ops_tensor.gemm_supported(self.hidden, self.ff))

    def forward(self, ctx, h, x):
        n = ctx.n_tokens
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            ops_tensor.flush_pending(x.device, self.rt.tc)      # x is complete before a kernel of this part adds to it
        names = self._names()
        chosen = ctx.buf(names[0], self.top, torch.float32).view(torch.int32)
        weight = ctx.buf(names[1], self.top, torch.float32)
        act = ctx.buf(names[3], self.top * self.ff)
        scale = ctx.buf(names[6], 1, torch.float32)
        ops.route(h, self.router, self.correction_values, self.sg, n, self.top, self.groups, self.keep_groups, chosen,
                  weight, scale if self.sg is not None else None, self.scoring, self.group_top, self.renormalize)
        if (self.by_products and n >= self.PRODUCTS_FROM and not getattr(ctx, "decode_only", False)
                and not torch.cuda.is_current_stream_capturing()):
            self._experts_by_products(ctx, h, x, chosen, weight, act, names)
            self._shared(ctx, h, x, scale)
            return
        # the 32-bit engine keeps ONE order of additions whatever the step's size: always expert by expert
        scratch = None
        if act.dtype == torch.float32 or n >= self.SORTED_FROM:
            order = ctx.buf(names[2], self.top, torch.float32).view(torch.int32)
            scratch = (self.first, order, ctx.buf(names[4], self.top * self.hidden, torch.float32))
        ops.experts(h, self.w_gate, self.w_up, self.w_down, chosen, weight, n, self.n_experts, self.top, self.ff,
                    act.view(-1, self.ff), x, scratch, self.pair_act, self.act_limit, self.act_alpha)
        self._shared(ctx, h, x, scale)

    def _experts_by_products(self, ctx, h, x, chosen, weight, act, names):
        n = ctx.n_tokens
        order = ctx.buf(names[2], self.top, torch.float32).view(torch.int32)
        where = ctx.buf(names[7], self.top, torch.float32).view(torch.int32)
        y = ctx.buf(names[4], self.top * self.hidden, torch.float32).view(-1, self.hidden)
        rows = ctx.buf(names[8], self.top * self.hidden).view(-1, self.hidden)
        act = act.view(-1, self.ff)
        ops.experts_gather(h, chosen, n, self.n_experts, self.top, self.first, order, where, rows)
        first = self.first[:self.n_experts + 1].tolist()     # how many rows each expert got: read on the host
        from .. import ops_tensor
        ops_tensor.gemm_runs(rows, self.w_gate, act, first, self.ff, ops.GEMM_SWIGLU, self.w_up, st=self.rt.tc,
                             act=self.pair_act, act_limit=self.act_limit, act_alpha=self.act_alpha)
        ops_tensor.gemm_runs(act, self.w_down, y, first, self.hidden, ops.GEMM_STORE, st=self.rt.tc)
        ops.experts_combine(y, h, chosen, weight, where, n, self.n_experts, self.top, x)

    def _shared(self, ctx, h, x, scale):
        n = ctx.n_tokens
        if self.shared_ff:
            sact = ctx.buf(self._names()[5], self.shared_ff)
            self.shared_up.gated(h, sact, n)
            if self.sg is not None:
                ops.scale_rows(sact, scale.view(-1), n)      # the down product is linear: scaling its input scales its result
            self.shared_down.accumulate(sact, x, n, defer=False)

    def resident_tensors(self):
        ts = [self.w_gate, self.w_up, self.w_down, self.router, self.correction_values, self.sg]
        if self.shared_ff:
            ts += [self.shared_up.w, self.shared_up.w2, self.shared_down.w]
        return [t for t in ts if t is not None]
