"""A plain statement of the Tubusun decoder in float64: whole sequences, no cache, no batches, one
function per mechanism, written from the equations and sharing nothing with the engine.

Notation: x [T, W] the residual stream of one sequence, positions 0..T-1; W[name] the tensors.
"""
import math

import torch

F64 = torch.float64


def silu(z):
    return z * torch.sigmoid(z)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def rotate_pairs(x, dims, base, positions=None):
    """x [T, heads, D]: the pair (2i, 2i+1), i < dims/2, turns by p * base^(-2i/dims); the other columns stay."""
    T = x.shape[0]
    pos = torch.arange(T, dtype=F64) if positions is None else positions.to(F64)
    out = x.clone()
    for i in range(dims // 2):
        a = pos * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def window_attention(h, W, p, sizes, eps, skip=None):
    """Grouped-query attention over a sliding window: rotated and unit-normed q and k, a sink in the softmax's
    denominator, one sigmoid gate number per head, through Wo."""
    H, G, D = sizes["heads"], sizes["kv_heads"], sizes["dim"]
    V = sizes.get("vdim", D)
    window = (sizes.get("mask") or {}).get("size") or 0
    T = h.shape[0]
    q = (h @ W[p + "q"].T).view(T, H, D)
    k = (h @ W[p + "k"].T).view(T, G, D)
    v = (h @ W[p + "v"].T).view(T, G, V)
    rot = sizes.get("rot")
    if rot and skip != "rotation":
        q, k = rotate_pairs(q, rot["dims"], rot["base"]), rotate_pairs(k, rot["dims"], rot["base"])
    if skip != "qk_norm":
        q, k = unit_rms(q, eps), unit_rms(k, eps)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        sink = W[p + "sink"][head]
        for i in range(T):
            lo = max(0, i + 1 - window) if window and skip != "window" else 0
            score = (k[lo:i + 1, g] @ q[i, head]) * sizes["scale"]
            m = torch.maximum(score.max(), sink) if skip != "sink" else score.max()
            e = torch.exp(score - m)
            denom = e.sum() + (torch.exp(sink - m) if skip != "sink" else 0.0)
            out[i, head] = (e / denom) @ v[lo:i + 1, g]
    if skip != "head_gate":
        out = out * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return out.reshape(T, H * V) @ W[p + "o"].T


def lightning_attention(h, W, p, sizes, eps, skip=None):
    """Per head S_t = decay_h S_(t-1) + k_t v_t^T from S = 0, o_t = S_t^T q_t with q, k, v = silu of their
    projections; the heads side by side are RMS-normed together, times sigmoid(Wg h), through Wo."""
    H, D, V = sizes["heads"], sizes["dim"], sizes["vdim"]
    T = h.shape[0]
    q = silu(h @ W[p + "q"].T).view(T, H, D)
    k = silu(h @ W[p + "k"].T).view(T, H, D)
    v = silu(h @ W[p + "v"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        decay = 1.0 if skip == "decay" else float(sizes["decay"][head])
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = decay * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    o = out.reshape(T, H * V)
    if skip != "state_norm":
        o = rms_norm(o, W[p + "norm"], eps)
    if skip != "state_gate":
        o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def side_by_side(h, W, p, mixer, eps, skip=None):
    left = 0.0 if skip == "left" else window_attention(h, W, p + "left.", mixer["left"], eps, skip)
    right = 0.0 if skip == "right" else lightning_attention(h, W, p + "right.", mixer["right"], eps, skip)
    return mixer["left_scale"] * left + mixer["right_scale"] * right


def dense_ffn(h, W, p):
    return gelu_erf(h @ W[p + "up"].T + W[p + "up.b"]) @ W[p + "down"].T + W[p + "down.b"]


def route(h, W, p, router, skip=None, margins=None):
    """(chosen [T, top], weights [T, top]): sigmoid scores; a group's score is the sum of its two largest; the
    `top` largest scores among the members of the `keep` best groups; weights are the scores themselves."""
    n, top = router["experts"], router["top"]
    s = torch.sigmoid(h @ W[p + "router"].T)
    T = h.shape[0]
    c = s.clone()
    margin = torch.full((T,), float("inf"), dtype=h.dtype)
    groups = router.get("groups")
    if groups and groups["keep"] < groups["count"] and skip != "groups":
        per = n // groups["count"]
        for t in range(T):
            scores = [float(s[t, g * per:(g + 1) * per].sort(descending=True).values[:2].sum()) for g in range(groups["count"])]
            order = sorted(range(groups["count"]), key=lambda g: (-scores[g], g))
            margin[t] = scores[order[groups["keep"] - 1]] - scores[order[groups["keep"]]]
            for g in order[groups["keep"]:]:
                c[t, g * per:(g + 1) * per] = float("-inf")
    chosen = torch.empty(T, top, dtype=torch.long)
    for t in range(T):
        order = sorted(range(n), key=lambda e: (-float(c[t, e]), e))
        chosen[t] = torch.tensor(order[:top])
        if top < n and float(c[t, order[top]]) > float("-inf"):
            margin[t] = min(float(margin[t]), float(c[t, order[top - 1]] - c[t, order[top]]))
    if margins is not None:
        margins.append(margin)
    return chosen, s.gather(1, chosen)


def expert(h, W, p, limit, skip=None):
    g, u = h @ W[p + "gate"].T, h @ W[p + "up"].T
    if skip != "limit":
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def routed_ffn(h, W, p, mlp, skip=None, margins=None):
    router = mlp["router"]
    chosen, weights = route(h, W, p, router, skip, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(router["top"]):
            out[t] += weights[t, j] * expert(h[t:t + 1], W, f"{p}e{int(chosen[t, j])}.", mlp["expert"]["limit"], skip)[0]
    return out


def schedule(cfg):
    """[(layer, pass number if a pass starts here else None)]"""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, tensors, ids, trace=None, skip=None, margins=None):
    """Logits [T, vocab] of one sequence.  `trace`: a list that receives the residual stream after every run of a
    layer.  `skip`: the name of one mechanism to leave out (tests use it to show that each one matters).  `margins`:
    a list that receives ONE tensor [T]: per token, the smallest distance by which any router of any run decided."""
    W = {k: v.to(F64) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    seen = [] if margins is not None else None
    x = W["embed"][torch.tensor(ids)] * (1.0 if skip == "embedding_scale" else (cfg.get("embedding") or {}).get("scale", 1.0))
    for i, t in schedule(cfg):
        if t is not None and skip != "loop_step":
            x = x + W["loop.step"][t]
        layer, p = cfg["layers"][i], f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(layer["type"])
        y = side_by_side(rms_norm(x, W[p + "norm1"], eps), W, p + "mix.", layer["mixer"], eps, skip)
        x = x + (y if skip == "post_norm" else rms_norm(y, W[p + "norm1b"], eps))
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            y = dense_ffn(h, W, p + "mlp.") if mlp["kind"] == "dense" else routed_ffn(h, W, p + "mlp.", mlp, skip, seen)
            x = x + (y if skip == "post_norm" else rms_norm(y, W[p + "norm2b"], eps))
        if trace is not None:
            trace.append(x.clone())
    if margins is not None:
        margins.append(torch.stack(seen).min(0).values if seen else torch.full((len(ids),), float("inf"), dtype=F64))
    logits = rms_norm(x, W["final.norm"], eps) @ W["embed"].T
    cap = cfg.get("logit_softcap")
    if cap and skip != "softcap":
        logits = cap * torch.tanh(logits / cap)
    return logits
