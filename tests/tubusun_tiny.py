"""Small Tubusun configurations and weights for the tests.  The sizes differ from one another in every respect.
Weights are made here, tensor kind by tensor kind, so that every mechanism carries signal: sinks of the size of the
scores, gates that are not all half open, decays from fast to none at all, routers whose sigmoid scores spread out,
experts whose products reach their bound, biases and post-norm weights that are not trivial."""
import json
import os
import tempfile

import torch


def _left(heads, kv_heads, dim, vdim, scale, window, rot):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": None if window is None else {"size": window},
            "rot": None if rot is None else {"dims": rot[0], "base": rot[1]}}


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _pair(left, right, left_scale, right_scale):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def _moe(ff, limit, experts, top, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _layer(mixer, mlp):
    return {"type": "parallel", "mixer": mixer, "mlp": mlp}


# a loop in the middle with three passes; every head rotated whole and partly; grouped queries with value heads wider
# than key heads; windows that are no multiple of anything; groups of which some are kept; a layer without a
# feed-forward; a router without groups that takes one expert; a decay of exactly one (a state that never forgets)
CFG_A = {
    "architecture": "Tubusun", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "logit_softcap": 6.0, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _layer(_pair(_left(4, 4, 8, 8, 0.35, 20, (8, 100.0)), _right(3, 8, 16, (0.5, 0.9, 0.995)), 0.7, 0.4), _dense(48)),
        _layer(_pair(_left(6, 2, 16, 24, 0.25, 37, (6, 10000.0)), _right(2, 16, 8, (1.0, 0.8)), 1.2, 0.5),
               _moe(24, 0.8, 6, 3, groups=(3, 2))),
        _layer(_pair(_left(2, 1, 24, 40, 0.2, None, None), _right(5, 4, 12, (0.3, 0.6, 0.9, 0.97, 0.99)), 0.5, 1.0), None),
        _layer(_pair(_left(3, 3, 12, 4, 0.4, 9, (12, 50.0)), _right(1, 20, 20, (0.93,)), 1.0, 1.0), _moe(16, 2.0, 5, 1)),
    ],
}

# no loop, no soft cap, no embedding scale; a width that is no multiple of 8 (no tensor-core product takes it); one kv
# head for all query heads; key heads wider than value heads; no window at all; a rotation of two numbers; every
# group kept; as many chosen experts as there are eligible ones
CFG_B = {
    "architecture": "Tubusun", "vocab": 53, "width": 36, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_pair(_left(5, 1, 12, 4, 0.3, None, (2, 7.0)), _right(4, 6, 10, (0.7, 0.8, 0.9, 0.99)), 1.0, 0.3),
               _moe(20, 1.5, 8, 4, groups=(4, 2))),
        _layer(_pair(_left(2, 2, 10, 14, 0.33, 5, (10, 1000.0)), _right(3, 12, 5, (0.95, 0.5, 0.2)), 0.4, 0.9), _dense(30)),
        _layer(_pair(_left(1, 1, 18, 18, 0.25, 64, None), _right(2, 9, 9, (0.9, 0.99)), 0.8, 0.8), _moe(28, 0.5, 7, 2, groups=(7, 7))),
    ],
}

# sizes the tensor-core kernels take (key and value heads of one size, multiples of 16); one pass of a loop over the
# first layers; a window of exactly one page; groups of two scored by their two members
CFG_C = {
    "architecture": "Tubusun", "vocab": 160, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.7},
    "logit_softcap": 20.0, "loop": {"start": 0, "stop": 2, "times": 1},
    "layers": [
        _layer(_pair(_left(8, 2, 32, 32, 0.18, 64, (16, 10000.0)), _right(4, 32, 32, (0.6, 0.9, 0.98, 0.999)), 0.6, 0.5),
               _moe(64, 1.0, 16, 6, groups=(8, 4))),
        _layer(_pair(_left(2, 2, 64, 64, 0.12, 150, (64, 500000.0)), _right(2, 64, 16, (0.97, 0.75)), 0.9, 0.7), _dense(192)),
        _layer(_pair(_left(4, 1, 16, 16, 0.3, 33, (4, 10000.0)), _right(8, 16, 48, [0.9] * 8), 0.5, 0.5),
               _moe(48, 3.0, 4, 2, groups=(2, 1))),
    ],
}

# the whole model looped twice; one layer
CFG_D = {
    "architecture": "Tubusun", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [
        _layer(_pair(_left(4, 2, 16, 16, 0.25, 11, (8, 10000.0)), _right(2, 24, 24, (0.9, 0.99)), 1.0, 1.0), _moe(32, 1.0, 6, 2, groups=(3, 2))),
    ],
}


def make_tensors(cfg, seed):
    """name -> float32 tensor, for every tensor the architecture declares."""
    from mdma_b200.config import load_config
    from mdma_b200.engine.model import expected_tensors
    arch, typed = load_config(cfg)
    g = torch.Generator().manual_seed(seed)
    rn = lambda *shape: torch.randn(tuple(shape), generator=g)
    out = {}
    for name, ts in expected_tensors(arch.describe(typed)).items():
        shape = tuple(ts.shape)
        parts = name.split(".")
        last = parts[-1]
        if name == "embed":
            t = rn(*shape) * (1.6 / shape[1] ** 0.5)          # also the output head
        elif name == "loop.step":
            t = rn(*shape) * 0.5
        elif last in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.25 * rn(*shape)
        elif last in ("norm1b", "norm2b"):
            t = 0.7 + 0.2 * rn(*shape)                        # a sublayer's result has unit size before this weight
        elif last == "norm":                                  # the linear attention's
            t = 1.0 + 0.3 * rn(*shape)
        elif last == "sink":
            t = 1.5 * rn(*shape)                              # of the size of the scores
        elif last == "router":
            t = rn(*shape) * (2.5 / shape[1] ** 0.5)
        elif last == "b":
            t = 0.5 * rn(*shape)
        elif last == "g" and "left" in parts:
            t = rn(*shape) * (2.0 / shape[1] ** 0.5)          # one number per head: open and shut
        elif len(shape) == 2:
            t = rn(*shape) * (1.3 / shape[1] ** 0.5)
        else:
            raise AssertionError(f"no recipe for {name} {shape}")
        out[name] = t.to(torch.float32)
    return out


def make_model(cfg, seed, dtype=torch.float32, root=None):
    """Write a folder (config.json + model.safetensors in `dtype`); returns (dir, tensors as stored, in float32)."""
    from mdma_b200.weights import write_safetensors
    d = tempfile.mkdtemp(prefix="tubusun_tiny_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = {n: t.to(dtype) for n, t in make_tensors(cfg, seed).items()}
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d, {n: t.float() for n, t in tensors.items()}
