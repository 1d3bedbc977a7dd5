"""The Tubusun decoder as a `ModelSpec`.

Every layer is the "sandwich" arrangement: an RMS norm in front of each sublayer and one on its result,
x += norm_b(sublayer(norm_a(x))).  The mixer is a pair side by side, both reading the same rows: grouped-query
softmax attention over a sliding window (a rotation of the first numbers of each head in interleaved pairs, query and
key heads divided by their root mean square, a sink in the softmax's denominator, one sigmoid gate number per head)
and linear attention with a fixed decay per head (SiLU on q, k, v, a float state per sequence, an RMS norm over the
heads side by side and a sigmoid gate); their results are added, each times a constant.  The feed-forward is dense
(the exact GELU, biases) or routed (sigmoid scores, groups scored by their two largest, weights not renormalised,
experts g sigmoid(1.702 g) (u + 1) on bounded products), or absent.  The embedding's rows are multiplied by a
constant; the output head is the embedding table itself, and the logits go through a soft cap.  A run of layers may
be looped: it is scheduled `times` times with the same weights, every pass with a cache and state of its own, and a
"loop_add" junction that adds the pass's vector in front of each pass.

Tensor names: `embed`, `final.norm`, `loop.step`, and per layer i `l<i>.norm1|norm1b|norm2|norm2b`,
`l<i>.mix.left.q|k|v|g|sink|o`, `l<i>.mix.right.q|k|v|g|norm|o`, `l<i>.mlp.up|down[.b]` or
`l<i>.mlp.router`, `l<i>.mlp.e<j>.gate|up|down`.
"""
from __future__ import annotations

from ..registry import ARCHITECTURES
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .tubusun import TubusunConfig, TubusunFeedForward, TubusunPair

GROUP_TOP = 2            # a group of experts is scored by the sum of its two largest scores
SWISH_ALPHA = 1.702      # the experts' g sigmoid(1.702 g)


def _norm(width: int, eps: float, name: str) -> PartSpec:
    return PartSpec("rmsnorm", dict(width=width, eps=eps), aliases={"weight": name})


def _mixer(c: TubusunConfig, m: TubusunPair, prefix: str) -> PartSpec:
    a, b = m.left, m.right
    position = None
    if a.rot_dims:
        position = PartSpec("rotary", dict(head_dim=a.dim, rotary_dim=a.rot_dims, theta=a.rot_base, layout="interleaved"))
    left = PartSpec("attention",
                    dict(hidden_size=c.width, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, v_dim=a.vdim,
                         scale=a.scale, window=a.window, position=position, qk_norm_eps=c.eps, sink=True, head_gate=True),
                    prefix=prefix + "left.",
                    aliases={n + "_proj.weight": prefix + "left." + n for n in ("q", "k", "v", "g", "o")})
    right = PartSpec("linear_attention",
                     dict(hidden_size=c.width, num_heads=b.heads, head_dim=b.dim, v_dim=b.vdim, decay=list(b.decay),
                          eps=c.eps), prefix=prefix + "right.")
    return PartSpec("side_by_side", dict(hidden_size=c.width, left=left, right=right, left_scale=m.left_scale,
                                         right_scale=m.right_scale), prefix=prefix)


def _feed_forward(c: TubusunConfig, f: TubusunFeedForward, prefix: str) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("dense_mlp", dict(hidden_size=c.width, intermediate_size=f.ff, activation="gelu", bias=True),
                        prefix=prefix)
    return PartSpec("routed_mlp",
                    dict(hidden_size=c.width, intermediate_size=f.ff, experts=f.experts, identity=0, top=f.top,
                         groups=f.groups, keep_groups=f.keep, group_top=GROUP_TOP, scoring="sigmoid", renormalize=False,
                         correction=False, shared_ff=0, activation="swish_limit", act_limit=f.limit, act_alpha=SWISH_ALPHA),
                    prefix=prefix)


def describe_tubusun(c: TubusunConfig) -> ModelSpec:
    W = c.width
    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        extras = {"mixer_post_norm": _norm(W, c.eps, p + "norm1b")}
        ffn_norm = ffn = None
        if layer.mlp is not None:
            ffn_norm, ffn = _norm(W, c.eps, p + "norm2"), _feed_forward(c, layer.mlp, p + "mlp.")
            extras["ffn_post_norm"] = _norm(W, c.eps, p + "norm2b")
        layers.append(LayerSpec("sandwich", _norm(W, c.eps, p + "norm1"), _mixer(c, layer.mixer, p + "mix."), ffn_norm, ffn,
                                extras))
    n = len(layers)
    junctions = []
    if c.loop_times:
        junctions.append(PartSpec("loop_add", dict(width=W, passes=c.loop_times, add_input=False), prefix="loop."))
        schedule = [ScheduleEntry(i) for i in range(c.loop_start)]
        for t in range(c.loop_times):
            for i in range(c.loop_start, c.loop_stop):
                first = i == c.loop_start
                schedule.append(ScheduleEntry(i, junction=0 if first else None, junction_arg=t if first else 0))
        schedule += [ScheduleEntry(i) for i in range(c.loop_stop, n)]
    else:
        schedule = [ScheduleEntry(i) for i in range(n)]
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab, max_positions=c.max_context,
        embedding=PartSpec("embedding", dict(vocab_size=c.vocab, width=W, scale=c.embedding_scale), aliases={"weight": "embed"}),
        layers=layers, schedule=schedule, final_norm=_norm(W, c.eps, "final.norm"),
        lm_head=PartSpec("lm_head", dict(vocab_size=c.vocab, width=W, softcap=c.logit_softcap or None),
                         aliases={"weight": "embed"}),
        stop_token_ids=tuple(c.eos_token_id), junctions=junctions)


def _register() -> None:
    from . import Architecture
    ARCHITECTURES.register("Tubusun", Architecture("Tubusun", TubusunConfig.from_dict, describe_tubusun), replace=True)


_register()
