"""How a layer's parts are arranged.  "prenorm": x += mixer(norm(x)); x +=
feed_forward(norm(x)), the residual stream x kept in float
(src/model/arch/llama.rs:181-231).  "shift_gated": the same with a token shift
in front of the mixer and a learned gate on each sublayer's result.  "parallel":
one norm whose output both sublayers read, x += mixer(h) + feed_forward(h).
"sandwich": a norm in front of each sublayer and one on its result,
x += norm_b(mixer(norm_a(x))); x += norm_d(feed_forward(norm_c(x)))."""
from __future__ import annotations

import dataclasses

import torch

from ..registry import AUXILIARIES, BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from ..spec import LayerSpec


@BLOCKS.register("prenorm")
class PreNormBlock:
    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer)
        self.ffn_norm = NORMS.get(spec.ffn_norm.kind)(spec.ffn_norm)
        self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn)

    handles_pending = True      # completes x itself where a product left partial sums (see _settle)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def workspace(self):
        """Per-token workspace of the arrangement itself: name -> (columns, 'act' | 'f32')."""
        return {"normed": (int(self.mixer_norm.params["width"]), "act")}

    def forward(self, ctx, x, view, owns_cache=True):
        h = ctx.buf("normed", x.shape[1])
        self._settle(ctx, x, self.mixer_norm)
        self.mixer_norm.forward(ctx, x, h)
        self.mixer.forward(ctx, h, x, view, owns_cache)
        self._settle(ctx, x, self.ffn_norm)
        self.ffn_norm.forward(ctx, x, h)
        self.ffn.forward(ctx, h, x)

    @staticmethod
    def _settle(ctx, x, norm):
        """A matrix product may have left partial sums of x for the next norm to add up;
        a norm that does not do that gets x completed first."""
        if ctx.rt.gemm == "tensor" and not getattr(norm, "fuses_pending", False):
            from .. import ops_tensor
            ops_tensor.flush_pending(x.device, ctx.rt.tc)


@BLOCKS.register("shift_gated")
class ShiftGatedBlock:
    """Pre-norm with a token shift and gated residuals:

        h = norm1(x);  x += sigmoid(Wg1 h + b1) * mixer(shift(h))
        h = norm2(x);  x += sigmoid(Wg2 h + b2) * feed_forward(h)       (if the layer has one)

    The gates read h as the norm hands it out, before the shift; only the mixer reads shifted rows.
    Parts beyond a layer's four come from `LayerSpec.extras`: "shift" (token_shift), "mixer_gate" and
    "ffn_gate" (residual_gate).  The run's state rows hold the mixer's own state first (padded to a
    multiple of four floats, so that both parts start on 16-byte boundaries), then the shift's last h.  Mixers and feed-forwards that offer `produce` (store their result as float rows) are
    used that way; others run into a zeroed buffer through their ordinary `forward`."""

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer)
        self.width = int(spec.mixer_norm.params["width"])
        self.shift = AUXILIARIES.get(spec.extras["shift"].kind)(spec.extras["shift"])
        self.mixer_gate = AUXILIARIES.get(spec.extras["mixer_gate"].kind)(spec.extras["mixer_gate"])
        self.ffn_norm = self.ffn = self.ffn_gate = None
        if spec.ffn is not None:
            self.ffn_norm = NORMS.get(spec.ffn_norm.kind)(spec.ffn_norm)
            self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn)
            self.ffn_gate = AUXILIARIES.get(spec.extras["ffn_gate"].kind)(spec.extras["ffn_gate"])

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.shift, self.mixer_gate, self.ffn_norm, self.ffn,
                            self.ffn_gate) if p is not None]

    def workspace(self):
        W = self.width
        return {"normed": (W, "act"), "shifted": (W, "act"), "gate": (W, "act"), "sublayer": (W, "f32")}

    def state_need(self):
        from ..cache import StateNeed
        # rows of a multiple of four floats: every row, and the mixer's part of it, starts on a 16-byte boundary
        return StateNeed((-(-(self._mixer_floats() + self.shift.state_floats()) // 4) * 4,), torch.float32)

    def _mixer_floats(self) -> int:
        """Floats of the mixer's state, rounded up to a multiple of four."""
        inner = self.mixer.state_need()
        if inner is None:
            return 0
        if inner.dtype != torch.float32:
            raise ValueError("the arrangement keeps its state in float rows; so must its mixer")
        n = 1
        for d in inner.shape:
            n *= int(d)
        return -(-n // 4) * 4

    def forward(self, ctx, x, view, owns_cache=True):
        W = self.width
        mixer_floats = self._mixer_floats()
        shift_state = view.state[:, mixer_floats:mixer_floats + self.shift.state_floats()]
        mixer_view = dataclasses.replace(view, state=view.state[:, :mixer_floats] if mixer_floats else None)
        h, hs, g = ctx.buf("normed", W), ctx.buf("shifted", W), ctx.buf("gate", W)
        y = ctx.buf("sublayer", W, torch.float32)
        if hasattr(self.mixer_norm, "forward_shifted"):
            self.mixer_norm.forward_shifted(ctx, x, h, hs, self.shift.mu, shift_state)
        else:
            self.mixer_norm.forward(ctx, x, h)
            self.shift.forward(ctx, h, hs, shift_state)
        self.mixer_gate.project(ctx, h, g)
        self._run(ctx, self.mixer, hs, y, mixer_view, owns_cache)
        # the shift's kept row is replaced only now, after the launch that read it
        self.mixer_gate.apply(ctx, x, g, y, keep_rows=h, state=shift_state)
        if self.ffn is None:
            return
        self.ffn_norm.forward(ctx, x, h)
        self.ffn_gate.project(ctx, h, g)
        self._run(ctx, self.ffn, h, y)
        self.ffn_gate.apply(ctx, x, g, y)

    @staticmethod
    def _run(ctx, part, h, y, *more):
        if hasattr(part, "produce"):
            # the gate's kernel adds up what a K-split product leaves (see ResidualGate.apply)
            part.produce(ctx, h, y, *more, defer=True)
            return
        y[:ctx.n_tokens].zero_()
        part.forward(ctx, h, y, *more)
        if ctx.rt.gemm == "tensor":
            from .. import ops_tensor
            ops_tensor.flush_pending(y.device, ctx.rt.tc)


@BLOCKS.register("parallel")
class ParallelBlock:
    """One norm, two readers:  h = norm(x);  x += mixer(h) + feed_forward(h)  (the feed-forward may be absent).
    Both sublayers add into the float residual stream, the mixer first."""

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer)
        self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn) if spec.ffn is not None else None
        if spec.ffn_norm is not None:
            raise ValueError("the parallel arrangement has one norm; its feed-forward reads the mixer's")

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn) if p is not None]

    def workspace(self):
        return {"normed": (int(self.mixer_norm.params["width"]), "act")}

    def forward(self, ctx, x, view, owns_cache=True):
        h = ctx.buf("normed", x.shape[1])
        self.mixer_norm.forward(ctx, x, h)
        self.mixer.forward(ctx, h, x, view, owns_cache)
        if self.ffn is not None:
            self.ffn.forward(ctx, h, x)


@BLOCKS.register("sandwich")
class SandwichBlock:
    """A norm before and after each sublayer:

        x += post1(mixer(norm1(x)));   x += post2(feed_forward(norm2(x)))       (if the layer has one)

    The two norms on the results come from `LayerSpec.extras`: "mixer_post_norm" and "ffn_post_norm"; they must offer
    `add_normed(ctx, y, x)` (x += norm(y) over float rows).  A sublayer adds its result into a zeroed float buffer
    through its ordinary `forward`, so any mixer and feed-forward of the registries fits."""

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.width = int(spec.mixer_norm.params["width"])
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer)
        self.mixer_post = NORMS.get(spec.extras["mixer_post_norm"].kind)(spec.extras["mixer_post_norm"])
        self.ffn_norm = self.ffn = self.ffn_post = None
        if spec.ffn is not None:
            self.ffn_norm = NORMS.get(spec.ffn_norm.kind)(spec.ffn_norm)
            self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn)
            self.ffn_post = NORMS.get(spec.extras["ffn_post_norm"].kind)(spec.extras["ffn_post_norm"])
        for norm in (self.mixer_post, self.ffn_post):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError(f"norm {norm.spec.kind!r} cannot follow a sublayer: it has no `add_normed`")

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_post, self.ffn_norm, self.ffn, self.ffn_post)
                if p is not None]

    def workspace(self):
        return {"normed": (self.width, "act"), "sublayer": (self.width, "f32")}

    def forward(self, ctx, x, view, owns_cache=True):
        n = ctx.n_tokens
        h = ctx.buf("normed", self.width)
        y = ctx.buf("sublayer", self.width, torch.float32)
        self.mixer_norm.forward(ctx, x, h)
        y[:n].zero_()
        self.mixer.forward(ctx, h, y, view, owns_cache)
        self.mixer_post.add_normed(ctx, y, x)
        if self.ffn is None:
            return
        self.ffn_norm.forward(ctx, x, h)
        y[:n].zero_()
        self.ffn.forward(ctx, h, y)
        self.ffn_post.add_normed(ctx, y, x)
