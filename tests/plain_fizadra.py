"""A plain statement of the Fizadra decoder in float64: whole sequences, no cache, no batching, one function
per mechanism.  It shares no code with the engine; the tests compare the engine with it.

`config` is the dict of config.json, `w` maps tensor names to float64 tensors, matrices stored [out, in].
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The row in `groups` equal consecutive parts, each divided by its own root mean square; then the weight."""
    rows, width = x.shape
    return rms_unit(x.reshape(rows, groups, width // groups), eps).reshape(rows, width) * weight


def frequencies(rot: dict):
    """(frequency per pair, factor on cos and sin) of a rotation {base, dims[, scaling]}."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    s = rot.get("scaling")
    if not s:
        return torch.tensor(f, dtype=F64), 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo, hi = max(math.floor(turn_dim(float(s["fast"]))), 0), min(math.ceil(turn_dim(float(s["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict, layout: str) -> torch.Tensor:
    """x [T, heads, d]: the first rot.dims numbers of every head turned by the token's position."""
    dims = int(rot["dims"])
    f, mag = frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]                 # [T, dims/2]
    cos, sin = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        half = dims // 2
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


def causal_weights(scores: torch.Tensor, sink=None) -> torch.Tensor:
    """scores [H, T, T] -> softmax over the keys j <= i; `sink` [H] (or a number) joins the denominator only."""
    H, T, _ = scores.shape
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = scores.masked_fill(~mask, -math.inf)
    if sink is None:
        return torch.softmax(s, -1)
    extra = (sink if torch.is_tensor(sink) else torch.full((H,), float(sink), dtype=F64)).to(F64)[:, None, None].expand(H, T, 1)
    return torch.softmax(torch.cat([s, extra], -1), -1)[..., :T]


def latent_kv(h, w, p, m, positions, eps, layout):
    """What a latent-attention layer caches of its input rows: the normed latent [T, kv_rank] and the turned key
    part [T, rot_dim] that all heads share."""
    rank, rot_dim = int(m["kv_rank"]), int(m["rot_dim"])
    kv = h @ w[p + "dkv"].T
    c = rms_unit(kv[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate(kv[:, None, rank:rank + rot_dim], positions, m["rot"], layout)[:, 0]
    return c, k_rot


def latent_attention(h, w, p, m, positions, eps, kind, shared=None):
    """`kind` "latent_attention": interleaved pairs (with scaled frequencies where given), a learned sink, a gate per
    number; "latent_attention_2": pairs half a width apart, the ordinary softmax, a gate per head."""
    first = kind == "latent_attention"
    layout = "interleaved" if first else "split_half"
    H, dim, rot_dim, vdim, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    T = h.shape[0]
    cq = rms_unit(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], positions, m["rot"], layout)
    c, k_rot = shared if shared is not None else latent_kv(h, w, p, m, positions, eps, layout)
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dim)
    v = (c @ w[p + "uv"].T).reshape(T, H, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    pr = causal_weights(scores, w[p + "sink"] if first else None)
    o = torch.einsum("hij,jhd->ihd", pr, v)
    g = torch.sigmoid(h @ w[p + "g"].T)
    o = o * (g.reshape(T, H, vdim) if first else g[:, :, None])
    return o.reshape(T, H * vdim) @ w[p + "o"].T, (c, k_rot)


def talking_attention(h, w, p, m, positions, eps):
    """Grouped-query attention with biases, normed query and key heads, a partial turn, the heads' scores mixed by a
    matrix, and one added to the softmax's denominator."""
    H, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    G = int(m.get("kv_heads", H))
    T = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, dim)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, dim)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, vdim)
    q = rotate(rms_unit(q, eps) * w[p + "q.norm"], positions, m["rot"], "split_half")
    k = rotate(rms_unit(k, eps) * w[p + "k.norm"], positions, m["rot"], "split_half")
    rep = H // G
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    scores = torch.einsum("hg,gij->hij", w[p + "talk"], scores)
    pr = causal_weights(scores, 0.0)
    o = torch.einsum("hij,jhd->ihd", pr, v)
    return o.reshape(T, H * vdim) @ w[p + "o"].T


def feed_forward(h, w, p):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def forward(config: dict, w: dict, tokens, leave_out: str = "", return_layers: bool = False):
    """Logits [T, vocab] of one sequence from position 0.  `leave_out` names a mechanism that is skipped (the tests use
    it to show that each one matters): "groups", "post_norm", "depth", "sink", "gate", "talk", "one", "qk_norm",
    "bias", "scaling", "rotation", "shared"."""
    eps, groups = float(config["norm"]["eps"]), int(config["norm"]["groups"])
    if leave_out == "groups":
        groups = 1
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = w["embed"][ids]
    history, cached, layers = [x], {}, []
    for i, layer in enumerate(config["layers"]):
        p, m, kind = f"l{i}.", dict(layer["mixer"]), layer["type"]
        if leave_out == "scaling" and "scaling" in m["rot"]:
            m["rot"] = {k: v for k, v in m["rot"].items() if k != "scaling"}
        if leave_out == "rotation":
            m["rot"] = dict(m["rot"], base=1e30)
        ww = w
        if leave_out in ("sink", "gate", "talk", "bias", "qk_norm"):
            ww = dict(w)
            for name in list(ww):
                if not name.startswith(p + "mix."):
                    continue
                if leave_out == "sink" and name.endswith(".sink"):
                    ww[name] = torch.full_like(w[name], -1e30)
                if leave_out == "gate" and name.endswith(".g"):
                    ww[name] = torch.zeros_like(w[name])
                if leave_out == "talk" and name.endswith(".talk"):
                    ww[name] = torch.eye(w[name].shape[0], dtype=F64)
                if leave_out == "bias" and name.endswith(".b"):
                    ww[name] = torch.zeros_like(w[name])
                if leave_out == "qk_norm" and name.endswith((".q.norm", ".k.norm")):
                    ww[name] = torch.ones_like(w[name])
        h = group_norm(x, w[p + "norm1"], groups, eps)
        if kind in ("latent_attention", "latent_attention_2"):
            src = m.get("kv_from")
            shared = cached[int(src)] if src is not None and leave_out != "shared" else None
            if src is not None and leave_out == "shared":
                ww = dict(ww)
                for name in ("dkv", "dkv.norm"):
                    ww[p + "mix." + name] = w[f"l{int(src)}.mix.{name}"]
            y, cached[i] = latent_attention(h, ww, p + "mix.", m, positions, eps, kind, shared)
        elif kind == "attention":
            y = talking_attention(h, ww, p + "mix.", m, positions, eps)
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        x = x + (group_norm(y, w[p + "norm1b"], groups, eps) if leave_out != "post_norm" else y)
        if layer.get("mlp") is not None:
            y = feed_forward(group_norm(x, w[p + "norm2"], groups, eps), w, p + "mlp.")
            x = x + (group_norm(y, w[p + "norm2b"], groups, eps) if leave_out != "post_norm" else y)
        history.append(x)
        if leave_out != "depth":
            x = sum(w[p + "dwa"][j] * history[j] for j in range(i + 2))
        layers.append(x)
    logits = group_norm(x, w["final.norm"], groups, eps) @ w["head"].T
    return (logits, layers) if return_layers else logits
