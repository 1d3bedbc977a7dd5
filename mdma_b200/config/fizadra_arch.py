"""The Fizadra decoder as a `ModelSpec`.

Every layer is the "sandwich" arrangement with RMS norms that work on `norm.groups` equal parts of a row, each part
divided by its own root mean square: x += norm_b(mixer(norm_a(x))); x += norm_d(feed_forward(norm_c(x))).  Three
mixers: attention over a cached latent with a turned key part shared by all heads, in two forms
("latent_attention": interleaved pairs, frequencies that may be scaled, a learned sink in the softmax, a sigmoid gate
per number of the result; "latent_attention_2": pairs half a width apart, the ordinary softmax, a gate per head), a
layer of either form may read an earlier layer's cached latent instead of making one; and grouped-query attention
with biases, normed query and key heads, part of a head turned, the heads' scores mixed by a learned matrix and one
added to the softmax's denominator.  The feed-forward is dense with a squared relu.  After each layer the stream
that goes on is a learned weighted sum of the embedding's output and the results of all layers so far (a
"depth_average" junction after every run).  The model's norm is grouped too; the head has a matrix of its own.

Tensor names: `embed`, `final.norm`, `head`, and per layer i `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.dwa`,
`l<i>.mlp.up|down`, `l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|sink|g|o` or
`l<i>.mix.q|k|v[.b]`, `l<i>.mix.q.norm|k.norm|talk|o`.
"""
from __future__ import annotations

from ..registry import ARCHITECTURES
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .fizadra import FizadraAttention, FizadraConfig, FizadraLatent, FizadraRotation

YARN_MAGNITUDE_SLOPE = 0.1      # cos and sin of scaled frequencies are multiplied by 0.1 ln(factor) + 1


def _norm(c: FizadraConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", dict(width=c.width, eps=c.eps, groups=c.groups), aliases={"weight": name})


def _rotary(rot: FizadraRotation, head: int, layout: str) -> PartSpec:
    scaling = None
    if rot.scaling is not None:
        factor, original, fast, slow = rot.scaling
        scaling = dict(kind="ramp", factor=factor, original=original, fast=fast, slow=slow,
                       magnitude_slope=YARN_MAGNITUDE_SLOPE)
    return PartSpec("rotary", dict(head_dim=head, rotary_dim=rot.dims, theta=rot.base, layout=layout, scaling=scaling))


def _mixer(c: FizadraConfig, kind: str, m, prefix: str) -> PartSpec:
    if isinstance(m, FizadraAttention):
        return PartSpec("talking_attention",
                        dict(hidden_size=c.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_dim=m.vdim,
                             scale=m.scale, eps=c.eps, position=_rotary(m.rot, m.dim, "split_half"), bias=True,
                             qk_norm=True, talk=True, denominator_extra=1.0), prefix=prefix)
    assert isinstance(m, FizadraLatent)
    first = kind == "latent_attention"
    return PartSpec("rotary_latent_attention",
                    dict(hidden_size=c.width, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank,
                         q_rank=m.q_rank, scale=m.scale, eps=c.eps,
                         position=_rotary(m.rot, m.rot_dim, "interleaved" if first else "split_half"),
                         sink=first, gate="element" if first else "head", shared_cache=m.kv_from is not None),
                    prefix=prefix)


def describe_fizadra(c: FizadraConfig) -> ModelSpec:
    W, n = c.width, len(c.layers)
    layers, schedule, junctions = [], [], []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        extras = {"mixer_post_norm": _norm(c, p + "norm1b")}
        ffn_norm = ffn = None
        if layer.ff:
            ffn_norm = _norm(c, p + "norm2")
            ffn = PartSpec("dense_mlp", dict(hidden_size=W, intermediate_size=layer.ff, activation="relu_squared"),
                           prefix=p + "mlp.")
            extras["ffn_post_norm"] = _norm(c, p + "norm2b")
        layers.append(LayerSpec("sandwich", _norm(c, p + "norm1"), _mixer(c, layer.type, layer.mixer, p + "mix."), ffn_norm,
                                ffn, extras))
        junctions.append(PartSpec("depth_average", dict(width=W, terms=i + 2, depth=n), aliases={"weight": p + "dwa"}))
        schedule.append(ScheduleEntry(i, cache=getattr(layer.mixer, "kv_from", None), after=i))
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab, max_positions=c.max_context,
        embedding=PartSpec("embedding", dict(vocab_size=c.vocab, width=W), aliases={"weight": "embed"}),
        layers=layers, schedule=schedule, final_norm=_norm(c, "final.norm"),
        lm_head=PartSpec("lm_head", dict(vocab_size=c.vocab, width=W), aliases={"weight": "head"}),
        stop_token_ids=tuple(c.eos_token_id), junctions=junctions)


def _register() -> None:
    from . import Architecture
    ARCHITECTURES.register("Fizadra", Architecture("Fizadra", FizadraConfig.from_dict, describe_fizadra), replace=True)


_register()
