"""Small Fizadra configurations and weights for the tests.  The sizes differ from one another in every respect.
Weights are made here, tensor kind by tensor kind, so that every mechanism carries signal: sinks of the size of the
scores, gates that are not all half open, mixing matrices far from the identity, biases and norm weights that are
not trivial, depth weights that give every earlier layer a say."""
import json
import os
import tempfile

import torch


def _rot(dims, base, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def _latent(kind, heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, scaling=None, kv_from=None, ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale, "rot": _rot(rot_dim, base, scaling)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": kind, "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _attention(heads, kv_heads, dim, vdim, scale, rot_dims, base, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": _rot(rot_dims, base)}
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


L1, L2 = "latent_attention", "latent_attention_2"

# two parts a row; grouped queries with value heads wider than key heads and a third of a head turned; a latent layer
# that reads the first layer's cache; scaled frequencies whose ramp lies inside the table; a layer without a
# feed-forward; query and kv latents of different sizes
CFG_A = {
    "architecture": "Fizadra", "vocab": 97, "width": 64, "norm": {"eps": 1e-5, "groups": 2},
    "layers": [
        _latent(L1, 3, 8, 12, 12, 20, 10, 0.3, 100.0, scaling=(4.0, 16, 2.0, 0.5), ff=48),
        _attention(6, 2, 24, 40, 0.25, 8, 10000.0, ff=40),
        _latent(L1, 5, 16, 12, 4, 20, 24, 0.22, 100.0, scaling=(4.0, 16, 2.0, 0.5), kv_from=0),
        _latent(L2, 2, 12, 6, 8, 18, 14, 0.35, 50.0, ff=56),
        _attention(3, 3, 12, 12, 0.4, 12, 50.0, ff=32),
    ],
}

# three parts a row and a width no tensor-core product takes; one kv head for all query heads and two turned numbers;
# two layers of the second latent form sharing a cache; a rotation base of 7
CFG_B = {
    "architecture": "Fizadra", "vocab": 53, "width": 36, "norm": {"eps": 1e-6, "groups": 3},
    "layers": [
        _attention(5, 1, 12, 4, 0.3, 2, 7.0, ff=30),
        _latent(L2, 4, 6, 10, 10, 9, 7, 0.4, 7.0, ff=20),
        _latent(L2, 2, 10, 10, 14, 9, 12, 0.33, 7.0, kv_from=1, ff=28),
        _latent(L1, 1, 18, 2, 18, 30, 5, 0.25, 1000.0),
    ],
}

# sizes the tensor-core kernels take (cached vectors of 128 and 64 numbers, heads of 64); rows normed whole; a
# latent layer with a sink that reads an earlier cache across an attention layer
CFG_C = {
    "architecture": "Fizadra", "vocab": 160, "width": 128, "norm": {"eps": 1e-5, "groups": 1},
    "layers": [
        _latent(L1, 8, 32, 32, 32, 96, 64, 0.13, 10000.0, scaling=(2.0, 64, 8.0, 1.0), ff=192),
        _attention(8, 2, 64, 64, 0.12, 32, 500000.0, ff=128),
        _latent(L2, 4, 16, 16, 48, 48, 32, 0.2, 10000.0, ff=64),
        _latent(L1, 2, 64, 32, 16, 96, 16, 0.1, 10000.0, scaling=(2.0, 64, 8.0, 1.0), kv_from=0, ff=256),
    ],
}

# one layer; eight parts a row of six numbers each
CFG_D = {
    "architecture": "Fizadra", "vocab": 61, "width": 48, "norm": {"eps": 1e-5, "groups": 8},
    "layers": [_attention(4, 2, 16, 8, 0.25, 4, 10000.0, ff=32)],
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
        last = name.split(".")[-1]
        if name == "embed":
            t = rn(*shape)
        elif name == "head":
            t = rn(*shape) * (1.6 / shape[1] ** 0.5)
        elif last in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.25 * rn(*shape)
        elif last in ("norm1b", "norm2b"):
            t = 0.7 + 0.2 * rn(*shape)                        # a sublayer's result has unit size before this weight
        elif last == "norm":                                  # the latents' and the heads' norms
            t = 1.0 + 0.3 * rn(*shape)
        elif last == "dwa":
            t = 0.3 * rn(*shape)
            t[-1] += 1.0                                      # the layer's own result leads, the others have a say
        elif last == "sink":
            t = 1.5 * rn(*shape)                              # of the size of the scores
        elif last == "talk":
            t = torch.eye(shape[0]) + 0.4 * rn(*shape)
        elif last == "b":
            t = 0.5 * rn(*shape)
        elif last == "g":
            t = rn(*shape) * (2.0 / shape[1] ** 0.5)          # open and shut
        elif len(shape) == 2:
            t = rn(*shape) * (1.3 / shape[1] ** 0.5)
        else:
            raise AssertionError(f"no recipe for {name} {shape}")
        out[name] = t.to(torch.float32)
    return out


def make_model(cfg, seed, dtype=torch.float32, root=None):
    """Write a folder (config.json + model.safetensors in `dtype`); returns (dir, tensors as stored, in float64)."""
    from mdma_b200.weights import write_safetensors
    d = tempfile.mkdtemp(prefix="fizadra_tiny_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = {n: t.to(dtype) for n, t in make_tensors(cfg, seed).items()}
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d, {n: t.double() for n, t in tensors.items()}
