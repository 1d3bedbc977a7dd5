"""The Tubusun architecture against its plain statement (tests/plain_tubusun.py): every mechanism alone through its
kernel, then whole models through the engine's step function, the cache and state manager, the scheduler and the
generation loop.  Configurations and weights are made here (tests/tubusun_tiny.py)."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_tubusun as pt
from tubusun_tiny import CFG_A, CFG_B, CFG_C, CFG_D, make_model, make_tensors

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}
# float32: absolute, against the float64 statement.  bfloat16: the largest error as a share of the deviation of the
# reference logits, and a row's root-mean-square error as a share of the row's own deviation.
TOL_F32 = 5e-5
TOL_BF16, TOL_ROW_BF16 = 0.12, 0.04
# A router that decided by less than this may decide the other way in bfloat16: after several layers the normed rows are
# off by a few percent, the router's logits (deviation ~2.5 with the tests' weights) by ~0.05, a sigmoid score by ~0.01,
# and a group's score is the sum of two.
CLOSE_CALL = 0.05


def ids_of(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


_largest = {}        # the largest errors seen, printed at exit when TUBUSUN_TEST_REPORT is set


def close(got, ref, dtype, what="", margins=None):
    """float32: every logit within TOL_F32 of the float64 statement.  bfloat16: every row within the tolerances, as
    long as no router of its sequence has had a close call.  A close call can fall the other way in bfloat16; the token
    then takes another expert, which moves that row by a good part of its deviation, and the linear attention's state
    (a decay of 1 forgets nothing) and the cache carry it to every later row of the sequence, most of all near the
    sequence's start, where the state holds little else.  `margins` [rows, 2]: per row, the least distance by which any
    router decided at this row, and at this row or an earlier one of its sequence.  Rows at or after a close call only
    have to stay finite and correlated with the statement (a wrong key, window or state gives a row error near 1.4,
    and float32 is the sharp test of those)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: logits that are not finite"
    err = np.abs(got - ref)
    if dtype == "float32":
        _largest[dtype] = max(_largest.get(dtype, 0.0), float(err.max()))
        assert err.max() < TOL_F32, f"{what}: {err.max()}"
        return
    err2, ref2 = np.atleast_2d(err), np.atleast_2d(ref)
    share = err2.max(axis=-1) / max(float(ref.std()), 0.25)
    rel = np.sqrt((err2 ** 2).mean(axis=-1)) / np.maximum(ref2.std(axis=-1), 1e-3)
    strict = np.ones(len(share), dtype=bool)
    if margins is not None:
        strict = np.asarray(margins, dtype=np.float64).reshape(-1, 2)[:, 1] >= CLOSE_CALL
    off = (share >= TOL_BF16) | (rel >= TOL_ROW_BF16)
    if strict.any():
        _largest[dtype] = max(_largest.get(dtype, 0.0), float(share[strict].max()))
        _largest["row"] = max(_largest.get("row", 0.0), float(rel[strict].max()))
    bad = strict & off
    assert not bad.any(), f"{what}: rows {np.nonzero(bad)[0].tolist()} are off (share {share[bad]}, row error {rel[bad]})"
    loose = ~strict
    if loose.any():
        assert rel[loose].max() < 0.9, f"{what}: rows after a close call are unrelated to the statement: {rel[loose]}"
        assert loose.sum() < 8 or np.median(rel[loose]) < 0.2, f"{what}: rows after a close call: {rel[loose]}"


def margins_of(per_row):
    """[T, 2] from the plain statement's per-row margins of one sequence: (own, least so far)."""
    own = np.asarray(per_row, dtype=np.float64)
    return np.stack([own, np.minimum.accumulate(own)], axis=1)


if os.environ.get("TUBUSUN_TEST_REPORT"):
    import atexit
    atexit.register(lambda: print("largest errors seen:", _largest))


# =====================================================================================================
# Without a GPU: configuration, description, and that the plain statement itself notices each mechanism.

def test_config_is_read_and_checked():
    from mdma_b200.config import ConfigError, load_config
    arch, c = load_config(CFG_A)
    assert arch.name == "Tubusun" and c.width == 64 and c.loop_times == 3 and c.layers[2].mlp is None
    assert c.embedding_scale == 3.0 and c.logit_softcap == 6.0 and c.eps == 1e-5
    left, right = c.layers[1].mixer.left, c.layers[1].mixer.right
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.window, left.rot_dims, left.rot_base) == (6, 2, 16, 24, 37, 6, 10000.0)
    assert right.decay == (1.0, 0.8) and c.layers[1].mixer.left_scale == 1.2 and c.layers[1].mixer.right_scale == 0.5
    assert c.layers[2].mixer.left.window == 0 and c.layers[2].mixer.left.rot_dims == 0
    assert c.layers[0].mlp.kind == "dense" and c.layers[0].mlp.ff == 48
    moe = c.layers[1].mlp
    assert (moe.kind, moe.ff, moe.limit, moe.experts, moe.top, moe.groups, moe.keep) == ("moe", 24, 0.8, 6, 3, 3, 2)
    assert c.layers[3].mlp.groups == 1
    spec = arch.describe(c)
    runs = [(e.layer, e.junction, e.junction_arg) for e in spec.schedule]
    assert runs == [(0, None, 0), (1, 0, 0), (2, None, 0), (1, 0, 1), (2, None, 0), (1, 0, 2), (2, None, 0), (3, None, 0)]
    assert pt.schedule(CFG_A) == [(l, a if j is not None else None) for l, j, a in runs]
    _, b = load_config(CFG_B)
    assert b.loop_times == 0 and not arch.describe(b).junctions and b.logit_softcap == 0.0 and b.embedding_scale == 1.0
    for breaker in (lambda d: d.pop("width"),
                    lambda d: d["layers"][0].update(type="lstm"),
                    lambda d: d["layers"][1]["mixer"].pop("left"),
                    lambda d: d["layers"][1]["mixer"]["right"].update(decay=[0.5]),
                    lambda d: d["layers"][1]["mixer"]["left"].update(kv_heads=4),
                    lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=7),
                    lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=18),
                    lambda d: d["layers"][0]["mlp"].update(kind="glu"),
                    lambda d: d["layers"][1]["mlp"]["expert"].pop("limit"),
                    lambda d: d["layers"][1]["mlp"]["router"].update(top=9),
                    lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=4),
                    lambda d: d["loop"].update(stop=9), lambda d: d["loop"].update(times=0)):
        bad = json.loads(json.dumps(CFG_A))
        breaker(bad)
        with pytest.raises(ConfigError):
            load_config(bad)


def test_tensor_inventory_and_plan_without_a_device(tmp_path):
    from mdma_b200.config import load_config
    from mdma_b200.engine.model import DecoderModel
    from mdma_b200.engine.step import plan_only
    arch, c = load_config(CFG_A)
    model = DecoderModel(arch.describe(c))
    specs = model.expected_tensors()
    names = set(specs)
    assert {"embed", "final.norm", "loop.step", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.left.q",
            "l0.mix.left.sink", "l0.mix.left.g", "l0.mix.left.o", "l0.mix.right.norm", "l0.mix.right.g", "l0.mlp.up.b",
            "l0.mlp.down.b", "l1.mlp.e5.down", "l1.mlp.router", "l2.norm1b", "l3.mlp.e4.gate"} <= names
    assert not {"head", "l2.norm2", "l2.norm2b", "l2.mlp.router", "l1.mlp.e6.up", "l1.mlp.correction", "l1.mlp.up.b"} & names
    assert specs["l1.mix.left.q"].shape == (96, 64) and specs["l1.mix.left.v"].shape == (48, 64)
    assert specs["l1.mix.left.g"].shape == (6, 64) and specs["l1.mix.left.o"].shape == (64, 144)
    assert specs["l1.mix.right.k"].shape == (32, 64) and specs["l1.mix.right.g"].shape == (16, 64)
    assert specs["l1.mix.right.norm"].shape == (16,) and specs["loop.step"].shape == (3, 64)
    # every run of a looped layer owns its state and its cache
    state, kv = model.state_needs(), model.kv_needs()
    assert len(state) == len(kv) == 8 and all(n is not None for n in state) and all(n is not None for n in kv)
    assert state[0].shape == (3 * 8 * 16,) and state[1].shape == state[3].shape == (2 * 16 * 8,) and state[7].shape == (400,)
    assert (kv[1].n_kv_heads, kv[1].head_dim, kv[1].v_dim, kv[1].window) == (2, 16, 24, 37) and kv[0].v_dim == 0 and kv[2].window == 0
    d, _ = make_model(CFG_A, 3, root=str(tmp_path))
    plan = plan_only(d, dtype="float32", max_batch=2, max_context=128)
    assert plan["total_bytes"] > 0 and plan["cache_bytes"] > 0


def test_the_plain_statement_notices_each_mechanism():
    """Leaving a mechanism out of the plain statement moves the logits by far more than any tolerance here."""
    W = make_tensors(CFG_A, 5)
    ids = ids_of(CFG_A, 60, 1)
    ref = pt.forward(CFG_A, W, ids)

    def moved(changes=None, skip=None):
        W2 = dict(W)
        W2.update(changes or {})
        return float((pt.forward(CFG_A, W2, ids, skip=skip) - ref).abs().max())
    for skip in ("embedding_scale", "loop_step", "rotation", "qk_norm", "window", "sink", "head_gate", "decay", "state_norm",
                 "state_gate", "left", "right", "groups", "limit", "post_norm", "softcap"):
        assert moved(skip=skip) > 0.02, skip
    assert moved({"l0.mlp.up.b": torch.zeros_like(W["l0.mlp.up.b"])}) > 0.02
    assert moved({"l0.mlp.down.b": torch.zeros_like(W["l0.mlp.down.b"])}) > 0.02
    assert moved({"l1.norm2b": torch.ones_like(W["l1.norm2b"])}) > 0.02
    # the rotation is of interleaved pairs: with the halves paired instead, the logits differ
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    r = pt.rotate_pairs(x, 4, 100.0)
    assert torch.equal(r[..., 4:], x[..., 4:]) and torch.equal(r[0], x[0]) and not torch.allclose(r[1:, :, :4], x[1:, :, :4])
    a = 3 * 100.0 ** (-2.0 / 4)
    assert abs(float(r[3, 1, 2]) - float(x[3, 1, 2] * math.cos(a) - x[3, 1, 3] * math.sin(a))) < 1e-12
    assert abs(float(r[3, 1, 3]) - float(x[3, 1, 3] * math.cos(a) + x[3, 1, 2] * math.sin(a))) < 1e-12


# =====================================================================================================
# Kernels alone (GPU).

def _dev(t, dtype=torch.float32):
    return t.to(device="cuda", dtype=dtype).contiguous()


def _i32(a):
    return torch.as_tensor(np.asarray(a, dtype=np.int32), device="cuda")


class _Step:
    """The step metadata the kernels' entry points read, for a call outside an engine."""

    def __init__(self, lengths, pos0, slots):
        self.n_seqs, self.n_tokens = len(lengths), sum(lengths)
        self.max_new, self.max_len = max(lengths), max(p + n for p, n in zip(pos0, lengths))
        self.seq_start = _i32(np.concatenate([[0], np.cumsum(lengths)]))
        self.seq_pos0, self.seq_slot = _i32(pos0), _i32(slots)
        self.tok_seq = _i32(np.concatenate([np.full(n, s) for s, n in enumerate(lengths)]))
        self.tok_pos = _i32(np.concatenate([np.arange(p, p + n) for p, n in zip(pos0, lengths)]))
        self.most_seqs = None


def _plain_attention(q, k, v, sinks, gate, scale, window, pos0):
    """q [n, H, D] at positions pos0.., k [L, G, D], v [L, G, V] (the whole sequence), sinks [H] or None, gate [n, H] or
    None: softmax over the visible keys with exp(sink) in the denominator, times sigmoid(gate) per head."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=torch.float64)
    for r in range(n):
        i = pos0 + r
        lo = max(0, i + 1 - window) if window else 0
        for h in range(H):
            kv = h // (H // G)
            s = (k[lo:i + 1, kv] @ q[r, h]) * scale
            m = s.max() if sinks is None else torch.maximum(s.max(), sinks[h])
            e = torch.exp(s - m)
            denom = e.sum() + (0.0 if sinks is None else torch.exp(sinks[h] - m))
            out[r, h] = (e / denom) @ v[lo:i + 1, kv]
    if gate is not None:
        out = out * torch.sigmoid(gate)[:, :, None]
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,V,rot,interleaved,unit", [(3, 3, 8, 8, 8, True, True), (6, 2, 16, 24, 6, True, True),
                                                          (2, 1, 24, 40, 0, True, True), (5, 1, 12, 4, 2, True, False),
                                                          (6, 3, 96, 32, 32, False, True), (1, 1, 200, 256, 200, True, True)])
def test_rotation_unit_norm_and_cache_write_in_one_pass(dtype, H, G, D, V, rot, interleaved, unit):
    """Rows [q | k | v | gate numbers] of two sequences at positions far from zero: q comes back rotated and normed in
    place, k likewise in the token's cache row, v as it is; the columns behind and every other cache row stay."""
    from mdma_b200 import ops
    g = torch.Generator().manual_seed(H * D + rot)
    lengths, pos0, slots, page, max_pages, eps = [7, 3], [61, 1000], [2, 0], 16, 70, 1e-5
    n = sum(lengths)
    pitch = -(-(H * D + G * D + G * V + H) // 8) * 8
    rows = (torch.randn(n, pitch, generator=g) * 2).to(dtype)
    step = _Step(lengths, pos0, slots)
    table = torch.randperm(3 * max_pages, generator=g).to(torch.int32).view(3, max_pages).cuda()
    kc = torch.full((3 * max_pages, page, G, D), float("nan"), dtype=dtype, device="cuda")
    vc = torch.full((3 * max_pages, page, G, V), float("nan"), dtype=dtype, device="cuda")
    inv_freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64)
    proj = _dev(rows, dtype)
    ops.qk_prepare(proj, H * D, H * D + G * D, step.tok_seq, step.tok_pos, step.seq_slot, _dev(inv_freq) if rot else None, kc, vc,
                   table, max_pages, page, n, H, G, D, V, rot, interleaved, unit, eps, True)
    got = proj.double().cpu()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert torch.equal(got[:, H * D:], rows.double()[:, H * D:])
    seen = 0
    for s, (ln, p0) in enumerate(zip(lengths, pos0)):
        sl = slice(seen, seen + ln)
        seen += ln
        positions = torch.arange(p0, p0 + ln)
        q = rows.double()[sl, :H * D].view(ln, H, D)
        k = rows.double()[sl, H * D:H * D + G * D].view(ln, G, D)
        f32 = inv_freq.float()                  # float frequencies, as the engine's table holds them

        def turn(x):
            out = x.clone()
            for i in range(rot // 2):
                d0, d1 = (2 * i, 2 * i + 1) if interleaved else (i, i + rot // 2)
                a = (positions.float() * f32[i]).double()      # the angle is a float product
                c, sn = torch.cos(a)[:, None], torch.sin(a)[:, None]
                out[..., d0], out[..., d1] = x[..., d0] * c - x[..., d1] * sn, x[..., d1] * c + x[..., d0] * sn
            return out
        q, k = turn(q), turn(k)
        if unit:
            q, k = pt.unit_rms(q, eps), pt.unit_rms(k, eps)
        assert (got[sl, :H * D].view(ln, H, D) - q).abs().max() < tol
        for r, p in enumerate(positions.tolist()):
            row = int(table[slots[s], p // page]) * page + p % page
            assert (kc.view(-1, G, D)[row].double().cpu() - k[r]).abs().max() < tol
            assert torch.equal(vc.view(-1, G, V)[row].double().cpu(), rows.double()[seen - ln + r, H * D + G * D:H * D + G * D + G * V].view(G, V))
    assert int((~torch.isnan(kc.view(-1, G * D)[:, 0])).sum()) == n and int((~torch.isnan(vc.view(-1, G * V)[:, 0])).sum()) == n


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("H,G,D,V,window", [(3, 3, 16, 16, 0), (6, 2, 24, 40, 37), (4, 1, 40, 8, 64), (8, 4, 72, 20, 129), (2, 2, 8, 8, 1)])
def test_attention_with_sink_and_head_gate_far_key_window_edges_and_pages(dtype, tiled, H, G, D, V, window):
    """A cache of scattered 16-row pages with NaN in every row nobody owns.  The prompt comes in two portions (a long
    one, then the rest on the cached prefix) and the last rows again one by one.  One far key (position 3) is made to
    stand out for the last query of head 1; the key at the window's edge is asked for by the query that still sees it
    and by the next one, which must not.  Sinks from far below the scores to far above them."""
    from mdma_b200 import ops
    g = torch.Generator().manual_seed(40 + H)
    T, page, scale, out_scale = 200, 16, 0.3, 0.6
    sinks = torch.linspace(-4.0, 5.0, H, dtype=torch.float64)
    k = torch.randn(T, G, D, generator=g).to(dtype).double()
    v = torch.randn(T, G, V, generator=g).to(dtype).double()
    q = torch.randn(T, H, D, generator=g) * 0.5
    gate = (2 * torch.randn(T, H, generator=g)).to(dtype).double()
    far = 3
    # coordinate 0 of the keys is zero except at the far key, coordinate 1 except at the window's edge key: a query
    # along one of them scores that key alone, e^12 above the others and the sink
    k[:, :, 0] = 0
    k[:, :, 1] = 0
    k[far, 1 // (H // G), 0] = 8.0
    q[T - 1, 1] = 0
    q[T - 1, 1, 0] = float((12.0 + 5.0) / (8.0 * scale))
    if window > 1:
        edge = T - 1 - window          # seen from row T-2 (distance window-1), not from row T-1
        k[edge, 0, 1] = 8.0
        q[T - 2, 0] = 0
        q[T - 2, 0, 1] = float((12.0 + 5.0) / (8.0 * scale))
        q[T - 1, 0] = q[T - 2, 0]
    q = q.to(dtype).double()
    n_pages, max_pages = 40, 13
    perm = torch.randperm(n_pages, generator=g)[:max_pages].to(torch.int32)
    kc = torch.full((n_pages, page, G, D), float("nan"), dtype=dtype, device="cuda")
    vc = torch.full((n_pages, page, G, V), float("nan"), dtype=dtype, device="cuda")
    table = torch.zeros(5, max_pages, dtype=torch.int32)
    table[2] = perm
    table = table.cuda()
    want = _plain_attention(q, k, v, sinks, gate, scale, window, 0) * out_scale
    got = torch.empty(T, H, V, dtype=torch.float64)
    portions = [150, 44] + [1] * 6
    at = 0
    for n in portions:
        step = _Step([n], [at], [2])
        proj = torch.cat([q[at:at + n].reshape(n, -1), k[at:at + n].reshape(n, -1), v[at:at + n].reshape(n, -1), gate[at:at + n]], 1)
        proj = _dev(proj, dtype)
        ops.qk_prepare(proj, H * D, H * D + G * D, step.tok_seq, step.tok_pos, step.seq_slot, None, kc, vc, table, max_pages, page,
                       n, H, G, D, V, 0, True, False, 0.0, True)
        out = torch.empty(n, H * V, device="cuda", dtype=dtype)
        ops.attention_distance(proj, kc, vc, step, table, max_pages, page, None, proj[:, H * D + G * D + G * V:], out, H, G, D, V,
                               window, scale, tiled, sinks=_dev(sinks), gate_heads=True, out_scale=out_scale)
        got[at:at + n] = out.double().cpu().view(n, H, V)
        at += n
    assert torch.isfinite(got).all()
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    assert (got - want).abs().max() < tol
    plain = _plain_attention(q, k, v, sinks, None, scale, window, 0)
    no_sink = _plain_attention(q, k, v, None, None, scale, window, 0)
    assert (plain[:, H - 1] - no_sink[:, H - 1]).abs().max() > 0.2          # the largest sink takes most of the weight
    if not window:      # the far key carries the last query's head 1
        assert (plain[T - 1, 1] - v[far, 1 // (H // G)]).abs().max() < 0.05 * v[far].abs().max()
    elif window > 1:    # the edge key is seen from T-2 and not from T-1; the far key is outside every window
        assert (plain[T - 2, 0] - v[edge, 0]).abs().max() < 0.05 * v[edge, 0].abs().max()
        assert (plain[T - 1, 0] - v[edge, 0]).abs().max() > 0.2 * v[edge, 0].abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("H,G,D,window", [(4, 4, 64, 0), (8, 2, 128, 100), (3, 1, 32, 37), (6, 3, 96, 50), (6, 2, 16, 129)])
@pytest.mark.parametrize("impl", ["tc", "mma", None])
def test_tensor_core_attention_with_sinks_then_head_gate(H, G, D, window, impl):
    """The tensor-core attention kernels with a sink per head, followed by the kernel that applies one gate number per
    head and a constant: a prompt in one step, a portion on the cached prefix, then single tokens (the decode kernel),
    against the plain statement.  A far key stands out for one query; the window's edge is asked for from both sides."""
    from mdma_b200 import ops, ops_tensor
    from mdma_b200.cache import KVView
    g = torch.Generator().manual_seed(H * D + window)
    T, page, scale, out_scale = 300, 64, 0.25, 1.3
    if impl == "tc" and not ops_tensor.attention_tc_supported(H, G, D, page):
        pytest.skip("outside the tcgen05 kernel's limits")
    bf = torch.bfloat16
    sinks = torch.linspace(-3.0, 4.0, H, dtype=torch.float64)
    k = torch.randn(T, G, D, generator=g).to(bf).double()
    v = torch.randn(T, G, D, generator=g).to(bf).double()
    q = torch.randn(T, H, D, generator=g) * 0.4
    gate = (2 * torch.randn(T, H, generator=g)).to(bf).double()
    k[:, :, 0] = 0
    k[:, :, 1] = 0
    far = 5
    k[far, 1 // (H // G), 0] = 8.0
    q[T - 1, 1] = 0
    q[T - 1, 1, 0] = float(16.0 / (8.0 * scale))
    if window:
        edge = T - 1 - window
        k[edge, 0, 1] = 8.0
        q[T - 2, 0] = 0
        q[T - 2, 0, 1] = float(16.0 / (8.0 * scale))
        q[T - 1, 0] = q[T - 2, 0]
    q = q.to(bf).double()
    n_pages, max_pages = 12, 6
    table = torch.zeros(3, max_pages, dtype=torch.int32)
    table[1] = torch.tensor([7, 2, 9, 0, 11, 4], dtype=torch.int32)
    table = table.cuda()
    kc = torch.full((n_pages, page, G, D), float("nan"), dtype=bf, device="cuda")
    vc = torch.full((n_pages, page, G, D), float("nan"), dtype=bf, device="cuda")
    view = KVView(k=kc, v=vc, page_table=table, page_size=page, max_pages=max_pages, window=window)
    want = _plain_attention(q, k, v, sinks, gate, scale, window, 0) * out_scale
    got = torch.empty(T, H, D, dtype=torch.float64)
    sink_log2 = _dev(sinks * 1.4426950408889634)
    pitch = -(-(H * D + 2 * G * D + H) // 8) * 8
    at = 0
    for n in [200, 94] + [1] * 6:
        step = _Step([n], [at], [1])
        proj = torch.zeros(n, pitch, dtype=torch.float64)
        proj[:, :H * D] = q[at:at + n].reshape(n, -1)
        proj[:, H * D:H * D + G * D] = k[at:at + n].reshape(n, -1)
        proj[:, H * D + G * D:H * D + 2 * G * D] = v[at:at + n].reshape(n, -1)
        proj[:, H * D + 2 * G * D:H * D + 2 * G * D + H] = gate[at:at + n]
        proj = _dev(proj, bf)
        ops.qk_prepare(proj, H * D, H * D + G * D, step.tok_seq, step.tok_pos, step.seq_slot, None, kc, vc, table, max_pages, page,
                       n, H, G, D, D, 0, True, False, 0.0, True)
        out = torch.empty(n, H * D, device="cuda", dtype=bf)
        ops_tensor.attention(step, proj, view, out, H, G, D, window, scale, impl=impl if n > 1 else None, sink_log2=sink_log2)
        ops.head_gate(out, proj[:, H * D + 2 * G * D:], n, H, D, out_scale)
        got[at:at + n] = out.double().cpu().view(n, H, D)
        at += n
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 5e-2
    plain = _plain_attention(q, k, v, sinks, None, scale, window, 0)
    if not window:
        assert (plain[T - 1, 1] - v[far, 1 // (H // G)]).abs().max() < 0.05 * v[far].abs().max()
    else:
        assert (plain[T - 2, 0] - v[edge, 0]).abs().max() < 0.05 * v[edge, 0].abs().max()
        assert (plain[T - 1, 0] - v[edge, 0]).abs().max() > 0.2 * v[edge, 0].abs().max()


def _plain_linear_attention(q, k, v, decay, S0):
    """Row by row in float64 from state S0 [H, D, V]: q, k [T, H, D], v [T, H, V] after their SiLU: (o [T, H, V], last S)."""
    S = S0.clone()
    out = torch.zeros(q.shape[0], q.shape[1], v.shape[2], dtype=torch.float64)
    for t in range(q.shape[0]):
        for h in range(q.shape[1]):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out, S


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,V", [(3, 8, 16), (2, 16, 8), (5, 4, 12), (1, 20, 20), (2, 64, 100), (2, 200, 24)])
def test_linear_attention_in_portions_slots_reused_and_runs_side_by_side(dtype, H, D, V):
    """Three sequences in slots out of order, each brought in portions down to one and two rows, row by row, by the kernel
    for single rows, a chunk of rows at a time,
    and in runs of rows walked side by side (several runs where a portion is long); outputs and the final state equal the whole-sequence walk in float64;
    a decay of exactly one and a fast one; the floats beyond a slot's own part of the state row are not touched; a
    slot that is zeroed and used again starts clean."""
    from mdma_b200 import ops
    g = torch.Generator().manual_seed(H * D + V)
    decay = torch.tensor(([1.0, 0.35, 0.9, 0.99, 0.999] * 2)[:H], dtype=torch.float64)
    lengths, slots = [75, 5, 140], [4, 0, 2]
    plans = [[2, 1, 69, 3], [5], [1, 1, 2, 100, 36]]
    width = 2 * H * D + H * V
    seqs = [(0.8 * torch.randn(n, width + 5, generator=g)).to(dtype) for n in lengths]
    floats = H * D * V
    for mode in ("rows", "singles", "chunks", "runs of 32", "runs of 48"):
        run_rows = int(mode.split()[-1]) if mode.startswith("runs") else 0
        most = -(-100 // run_rows) if run_rows else 1
        scratch = torch.full((3 * most * floats,), float("nan"), device="cuda") if run_rows else None
        # the single-row kernel reads four floats at a time: its rows start on 16 bytes (else it is the walk row by row)
        state = torch.full((6, floats + (4 if mode == "singles" else 3)), float("nan"), device="cuda")
        state[:, :floats] = 0
        got = [[] for _ in seqs]
        at = [0, 0, 0]
        for step in range(5):
            live = [s for s in range(3) if step < len(plans[s])]
            ns = [plans[s][step] for s in live]
            st = _Step(ns, [at[s] for s in live], [slots[s] for s in live])
            proj = _dev(torch.cat([seqs[s][at[s]:at[s] + n] for s, n in zip(live, ns)]), dtype)
            out = torch.full((sum(ns), H * V), float("nan"), device="cuda")
            ops.linear_attention(proj, 0, H * D, 2 * H * D, _dev(decay), st.seq_start, st.seq_slot, state[:, :floats], out,
                                 len(live), H, D, V, mode not in ("rows", "singles"), run_rows, most, scratch,
                                 single=mode == "singles")
            o = 0
            for s, n in zip(live, ns):
                got[s].append(out[o:o + n].double().cpu())
                o += n
                at[s] += n
        for s, n in enumerate(lengths):
            x = seqs[s].double()
            q, k = pt.silu(x[:, :H * D]).view(n, H, D), pt.silu(x[:, H * D:2 * H * D]).view(n, H, D)
            v = pt.silu(x[:, 2 * H * D:width]).view(n, H, V)
            want, S = _plain_linear_attention(q, k, v, decay, torch.zeros(H, D, V, dtype=torch.float64))
            size = max(1.0, float(want.abs().max()))
            assert (torch.cat(got[s]).view(n, H, V) - want).abs().max() < 3e-5 * size, (s, mode)
            assert (state[slots[s], :floats].double().cpu().view(H, D, V) - S).abs().max() < 3e-5 * max(1.0, float(S.abs().max())), (s, mode)
        assert torch.isnan(state[:, floats:]).all() and not state[[1, 3, 5], :floats].any()
    # a state that is not zero goes on from where it was; the same rows from a zeroed slot start clean
    S0 = torch.randn(H, D, V, generator=g, dtype=torch.float64)
    state = torch.zeros(2, floats, device="cuda")
    state[1] = _dev(S0.reshape(-1))
    rows = seqs[0][:40]
    x = rows.double()
    q, k = pt.silu(x[:, :H * D]).view(40, H, D), pt.silu(x[:, H * D:2 * H * D]).view(40, H, D)
    v = pt.silu(x[:, 2 * H * D:width]).view(40, H, V)
    st = _Step([40, 40], [7, 0], [1, 0])
    out = torch.empty(80, H * V, device="cuda")
    ops.linear_attention(_dev(torch.cat([rows, rows]), dtype), 0, H * D, 2 * H * D, _dev(decay), st.seq_start, st.seq_slot, state, out,
                         2, H, D, V, True)
    for n, start in enumerate((S0, torch.zeros_like(S0))):
        want, _ = _plain_linear_attention(q, k, v, decay, start)
        assert (out[40 * n:40 * n + 40].double().cpu().view(40, H, V) - want).abs().max() < 3e-5 * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norms_on_results_gates_and_scaled_sums(dtype):
    from mdma_b200 import ops
    g = torch.Generator().manual_seed(7)
    for width in (12, 36, 64, 1000):
        T, eps = 9, 1e-5
        o = torch.randn(T, width, generator=g) * 3
        gate = (2 * torch.randn(T, width + 8, generator=g)).to(dtype)
        w = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype)
        out = torch.empty(T, width, device="cuda", dtype=dtype)
        ops.gated_rmsnorm(_dev(o), _dev(gate, dtype)[:, 3:], _dev(w, dtype), out, T, eps, 0.45)
        want = pt.rms_norm(o.double(), w.double(), eps) * torch.sigmoid(gate.double()[:, 3:3 + width]) * 0.45
        assert (out.double().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2)
        # x += norm(y), with and without partial sums that complete y first
        x, y = torch.randn(T, width, generator=g), torch.randn(T, width, generator=g) * 5
        xd = _dev(x)
        ops.rmsnorm_add(xd, _dev(y), _dev(w, dtype), eps, T)
        want = x.double() + pt.rms_norm(y.double(), w.double(), eps)
        assert (xd.double().cpu() - want).abs().max() < 1e-5
        parts = torch.randn(3, T, width, generator=g)
        xd, yd = _dev(x), _dev(y)
        ops.rmsnorm_add(xd, yd, _dev(w, dtype), eps, T, _dev(parts), 3, T * width)
        whole = y.double() + parts.double().sum(0)
        assert (yd.double().cpu() - whole).abs().max() < 1e-5
        assert (xd.double().cpu() - x.double() - pt.rms_norm(whole, w.double(), eps)).abs().max() < 1e-5
        yd = _dev(y)
        ops.add_scaled(yd, _dev(x), -0.3, T)
        assert (yd.cpu() - (y - 0.3 * x)).abs().max() < 1e-6
    heads, vd = 5, 12
    out = (torch.randn(7, heads * vd, generator=g)).to(dtype)
    gate = (2 * torch.randn(7, heads + 3, generator=g)).to(dtype)
    od = _dev(out, dtype)
    ops.head_gate(od, _dev(gate, dtype), 7, heads, vd, 0.8)
    want = (out.double().view(7, heads, vd) * torch.sigmoid(gate.double()[:, :heads])[:, :, None] * 0.8).view(7, -1)
    assert (od.double().cpu() - want).abs().max() < (1e-6 if dtype == torch.float32 else 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,ff,experts,top,groups,limit", [(64, 24, 6, 3, (3, 2), 0.8), (36, 20, 8, 4, (4, 2), 1.5), (128, 64, 16, 6, (8, 4), 1.0),
                                                           (48, 16, 5, 1, None, 2.0), (40, 28, 7, 2, (7, 7), 0.5), (64, 32, 12, 3, (2, 1), 1.0)])
def test_sigmoid_router_and_bounded_experts(dtype, W, ff, experts, top, groups, limit):
    """The router's choice and weights against the plain statement (rows that decide by a hair are left out), the
    groups' scores as sums of two (a case where the largest alone would keep another group), weights that are the
    scores themselves, and the experts token by token and expert by expert."""
    from mdma_b200 import ops
    g = torch.Generator().manual_seed(W + experts)
    T = 90
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    Wt = {"m.router": (torch.randn(experts, W, generator=g) * (2.5 / W ** 0.5)).to(dtype).float()}
    for e in range(experts):
        Wt[f"m.e{e}.gate"] = (torch.randn(ff, W, generator=g) * (1.5 / W ** 0.5)).to(dtype).float()
        Wt[f"m.e{e}.up"] = (torch.randn(ff, W, generator=g) * (1.5 / W ** 0.5)).to(dtype).float()
        Wt[f"m.e{e}.down"] = (torch.randn(W, ff, generator=g) * (1.3 / ff ** 0.5)).to(dtype).float()
    W64 = {k: v.double() for k, v in Wt.items()}
    h = torch.randn(T, W, generator=g).to(dtype)
    margins = []
    chosen_ref, weight_ref = pt.route(h.double(), W64, "m.", router, margins=margins)
    chosen = torch.full((T, top), -7, dtype=torch.int32, device="cuda")
    weight = torch.full((T, top), float("nan"), device="cuda")
    ops.route(_dev(h, dtype), _dev(Wt["m.router"], dtype), None, None, T, top, groups[0] if groups else 1,
              groups[1] if groups else 1, chosen, weight, None, "sigmoid", 2, False)
    chosen, weight = chosen.cpu(), weight.cpu()
    sure = margins[0] > 1e-5
    assert sure.sum() >= T - 2
    for t in torch.nonzero(sure).view(-1).tolist():
        assert sorted(chosen[t].tolist()) == sorted(chosen_ref[t].tolist()), t
        order = {e: j for j, e in enumerate(chosen[t].tolist())}
        for j, e in enumerate(chosen_ref[t].tolist()):
            assert abs(float(weight[t, order[e]]) - float(weight_ref[t, j])) < 1e-5
    assert float(weight.sum()) != pytest.approx(T, abs=1.0) or top == 1        # not renormalised
    if groups and groups[1] < groups[0]:
        other, _ = pt.route(h.double(), W64, "m.", router, skip="groups")
        assert (other.sort(1).values != chosen_ref.sort(1).values).any()        # the groups change who is chosen
    stack = lambda part: _dev(torch.cat([Wt[f"m.e{e}.{part}"] for e in range(experts)]), dtype)
    want = torch.zeros(T, W, dtype=torch.float64)
    clipped = 0
    for t in range(T):
        for j in range(top):
            e = int(chosen[t, j])
            want[t] += float(weight[t, j]) * pt.expert(h[t:t + 1].double(), W64, f"m.e{e}.", limit)[0]
            clipped += int((h[t].double() @ W64[f"m.e{e}.gate"].T > limit).sum())
    assert clipped > 10
    x0 = torch.randn(T, W, generator=g)
    for way in ("token", "expert"):
        x = _dev(x0)
        act = torch.empty(T * top, ff, device="cuda", dtype=dtype)
        scratch = None
        if way == "expert":
            scratch = (torch.full((2 * (experts + 1),), -1, dtype=torch.int32, device="cuda"),
                       torch.full((T * top,), -1, dtype=torch.int32, device="cuda"),
                       torch.full((T * top * W,), float("nan"), device="cuda"))
        ops.experts(_dev(h, dtype), stack("gate"), stack("up"), stack("down"), chosen.cuda(), weight.cuda(), T, experts, top, ff, act, x,
                    scratch, ops.ACT_SWISH_LIMIT, limit, 1.702)
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        assert (x.double().cpu() - x0.double() - want).abs().max() < tol, way


def test_a_group_is_scored_by_its_two_largest():
    """Scores chosen so that the single largest would keep group 0, the sum of two keeps group 1."""
    z = torch.tensor([[3.0, -4.0, -4.0, 1.5, 1.4, -4.0]], dtype=torch.float64)
    W = {"m.router": torch.eye(6, dtype=torch.float64)}
    chosen, weights = pt.route(z, W, "m.", {"experts": 6, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert sorted(chosen[0].tolist()) == [3, 4]
    assert torch.allclose(weights[0].sort().values, torch.sigmoid(torch.tensor([1.4, 1.5], dtype=torch.float64)))


@pytest.mark.gpu
def test_router_kernel_scores_a_group_by_its_two_largest():
    from mdma_b200 import ops
    z = torch.tensor([[3.0, -4.0, -4.0, 1.5, 1.4, -4.0, 0, 0], [0.2, 0.1, 0.0, 2.0, -3.0, -3.0, 0, 0]])
    chosen = torch.zeros(2, 2, dtype=torch.int32, device="cuda")
    weight = torch.zeros(2, 2, device="cuda")
    router = torch.eye(8)[:6].contiguous()
    ops.route(_dev(z), _dev(router), None, None, 2, 2, 2, 1, chosen, weight, None, "sigmoid", 2, False)
    assert sorted(chosen[0].tolist()) == [3, 4] and sorted(chosen[1].tolist()) == [0, 1]
    assert abs(float(weight[0].sum()) - float(torch.sigmoid(torch.tensor([1.5, 1.4])).sum())) < 1e-6
    ops.route(_dev(z), _dev(router), None, None, 2, 2, 2, 1, chosen, weight, None, "sigmoid", 1, False)
    assert sorted(chosen[0].tolist()) == [0, 1] and sorted(chosen[1].tolist()) == [3, 4]


@pytest.mark.gpu
@pytest.mark.parametrize("engine", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,ff", [(36, 30), (64, 48), (128, 192)])
def test_dense_feed_forward_with_biases_and_the_exact_gelu(engine, W, ff):
    """`dense_mlp` with activation "gelu" and biases through the part itself (CUDA-core products for float32 and for
    widths the tensor-core product does not take, tcgen05 products otherwise)."""
    from mdma_b200.parts.base import Runtime
    from mdma_b200.parts.mlp import DenseMLP
    from mdma_b200.spec import PartSpec
    dtype = torch.float32 if engine == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(W)
    T = 70
    Wt = {"m.up": torch.randn(ff, W, generator=g) * (1.3 / W ** 0.5), "m.up.b": 0.5 * torch.randn(ff, generator=g),
          "m.down": torch.randn(W, ff, generator=g) * (1.3 / ff ** 0.5), "m.down.b": 0.5 * torch.randn(W, generator=g)}
    Wt = {k: v.to(dtype).float() for k, v in Wt.items()}
    h = torch.randn(T, W, generator=g).to(dtype)
    want = pt.dense_ffn(h.double(), {k: v.double() for k, v in Wt.items()}, "m.")
    part = DenseMLP(PartSpec("dense_mlp", dict(hidden_size=W, intermediate_size=ff, activation="gelu", bias=True), prefix="m."))
    rt = Runtime(dtype, torch.device("cuda"), gemm="tensor" if engine == "bfloat16" else "simt")
    part.bind({k[2:]: _dev(v, dtype) for k, v in Wt.items()}, rt)

    class Ctx:
        n_tokens = T

        def __init__(self):
            self.rt = rt
            self.bufs = {}

        def buf(self, name, cols, dt=None):
            return self.bufs.setdefault(name, torch.empty(T, cols, device="cuda", dtype=dt or dtype))
    x = torch.zeros(T, W, device="cuda")
    part.forward(Ctx(), _dev(h, dtype), x)
    if engine == "bfloat16":
        from mdma_b200 import ops_tensor
        ops_tensor.flush_pending(x.device, rt.tc)
    assert (x.double().cpu() - want).abs().max() < (2e-5 if engine == "float32" else 4e-2)
    assert (pt.gelu_erf(torch.tensor([1.0], dtype=torch.float64)) - 0.8413447460685429).abs() < 1e-12      # not the tanh form (0.84119)


# =====================================================================================================
# Whole models through the engine (GPU).

_models: dict = {}


def model_of(key, dtype):
    """(folder, config, float64-ready tensors as the engine holds them) of configuration `key`."""
    k = (key, dtype)
    if k not in _models:
        store = torch.float32 if dtype == "float32" else torch.bfloat16
        d, W = make_model(CONFIGS[key], 23 + ord(key), store)
        _models[k] = (d, CONFIGS[key], W)
    return _models[k]


_refs: dict = {}


def ref_of(key, dtype, ids):
    """(logits [T, vocab], margins [T, 2], see `close`)."""
    k = (key, dtype, tuple(ids))
    if k not in _refs:
        _, cfg, W = model_of(key, dtype)
        margins = []
        logits = pt.forward(cfg, W, ids, margins=margins).numpy()
        _refs[k] = (logits, margins_of(margins[-1].numpy()))
    return _refs[k]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C", "D"])
def test_every_layer_against_the_plain_statement(key, dtype):
    """The residual stream after every run of a layer, then the logits; one short prompt."""
    from mdma_b200.engine import Engine, StepEntry
    d, cfg, W = model_of(key, dtype)
    ids = ids_of(cfg, 21, 4)
    trace, margins = [], []
    ref = pt.forward(cfg, W, ids, trace, margins=margins)
    m = margins_of(margins[-1].numpy())
    eng = Engine(d, dtype=dtype, max_batch=2, max_context=64, logit_rows=64, page_size=16)
    got = []
    eng.model.on_layer = lambda n, x: got.append(x.detach().double().cpu())
    s = eng.acquire()
    logits = eng.step([StepEntry(s, ids, list(range(len(ids))))]).cpu().numpy()
    assert len(got) == len(trace) == len(pt.schedule(cfg))
    tol = 1e-4 if dtype == "float32" else 0.04
    for n, (a, b) in enumerate(zip(got, trace)):
        row_err = (a - b).abs().max(dim=-1).values.numpy()
        bad = row_err >= tol * max(1.0, float(b.abs().max()))
        if dtype != "float32":
            bad &= m[:, 1] >= CLOSE_CALL            # rows before their sequence's first close call
        assert not bad.any(), f"after run {n} of the schedule: rows {np.nonzero(bad)[0].tolist()}, {row_err.max()}"
    close(logits, ref.numpy(), dtype, "logits", None if dtype == "float32" else m)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C", "D"])
def test_batches_portions_decoding_and_reuse(key, dtype):
    """Unequal prompts in one step; the same prompts cut in portions down to one and two tokens on a cached prefix;
    token-by-token decoding past every window; sequences that end early while others go on; slots and pages freed and
    taken again (rows nobody owns hold NaN throughout).  In float32 every way of cutting gives the same logits to
    within a few units of the last place."""
    from mdma_b200.engine import Engine, StepEntry
    d, cfg, W = model_of(key, dtype)
    lengths = [70, 1, 33, 2, 17]
    seqs = [ids_of(cfg, n, 20 + i) for i, n in enumerate(lengths)]
    refs = [ref_of(key, dtype, s) for s in seqs]
    eng = Engine(d, dtype=dtype, max_batch=5, max_context=96, logit_rows=160, page_size=16)

    def run(plan):
        """plan: per sequence, the sizes of its portions.  All sequences advance together, one portion a step."""
        slots = [eng.acquire() for _ in seqs]
        rows = [[] for _ in seqs]
        at = [0] * len(seqs)
        for step in range(max(len(p) for p in plan)):
            live = [i for i in range(len(seqs)) if step < len(plan[i])]
            eng.cache.poison_unused()
            out = eng.step([StepEntry(slots[i], seqs[i][at[i]:at[i] + plan[i][step]], list(range(plan[i][step])))
                            for i in live]).cpu().numpy()
            o = 0
            for i in live:
                n = plan[i][step]
                rows[i].append(out[o:o + n].copy())
                o += n
                at[i] += n
                if at[i] == len(seqs[i]):
                    eng.release(slots[i])           # ends early; its slot, its state row and its pages go back
        eng.cache.check()
        return [np.concatenate(r) for r in rows]

    whole = run([[n] for n in lengths])
    for i, (got, (ref, margin)) in enumerate(zip(whole, refs)):
        close(got, ref, dtype, f"whole prompts, sequence {i}", margin)
    alone = []
    for i, s in enumerate(seqs):                    # each alone, in a slot that the batch used
        slot = eng.acquire()
        alone.append(eng.step([StepEntry(slot, s, list(range(len(s))))]).cpu().numpy().copy())
        eng.release(slot)
    pieces = run([[2, 1, 30, 17, 1, 2, 16, 1], [1], [16, 1, 15, 1], [1, 1], [3, 14]])
    decoded = run([[25] + [1] * 45, [1], [1] * 33, [2], [16, 1]])
    for name, other in (("alone", alone), ("portions", pieces), ("decoded", decoded)):
        for i, (got, (ref, margin)) in enumerate(zip(other, refs)):
            close(got, ref, dtype, f"{name}, sequence {i}", margin)
            if dtype == "float32":
                assert np.abs(got - whole[i]).max() <= 4e-6, f"{name}, sequence {i}: differs from the whole prompt"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_passes_smaller_than_a_step_and_long_decoding(dtype):
    """A step run as passes of 7 tokens (cuts inside sequences), then 150 tokens decoded one by one across many page
    borders and past the windows (whose pages go back on the way), beside a batch mate that ends on the way and whose
    slot another request takes."""
    from mdma_b200.engine import Engine, StepEntry
    d, cfg, W = model_of("A", dtype)
    long_ids, mate, late = ids_of(cfg, 190, 31), ids_of(cfg, 60, 32), ids_of(cfg, 25, 33)
    (r_long, m_long), (r_mate, m_mate), (r_late, m_late) = (ref_of("A", dtype, s) for s in (long_ids, mate, late))
    eng = Engine(d, dtype=dtype, max_batch=2, max_context=192, logit_rows=64, page_size=16, chunk_tokens=7)
    a, b = eng.acquire(), eng.acquire()
    out = eng.step([StepEntry(a, long_ids[:40], [0, 39, 6, 7]), StepEntry(b, mate[:41], [40, 13])]).cpu().numpy()
    assert eng.forward_passes > 10
    close(out, np.stack([r_long[0], r_long[39], r_long[6], r_long[7], r_mate[40], r_mate[13]]), dtype, "passes",
          [m_long[0], m_long[39], m_long[6], m_long[7], m_mate[40], m_mate[13]])
    pb = 41
    for p in range(40, 190):
        entries = [StepEntry(a, [long_ids[p]], [0])]
        second = None
        if pb < len(mate):
            entries.append(StepEntry(b, [mate[pb]], [0]))
            second = (r_mate[pb], m_mate[pb])
            pb += 1
        elif pb == len(mate):                       # the mate is done: its slot goes to a late request
            eng.release(b)
            b = eng.acquire()
            entries.append(StepEntry(b, late, [len(late) - 1]))
            second = (r_late[-1], m_late[-1])
            pb += 1
        eng.cache.poison_unused()
        out = eng.step(entries).cpu().numpy()
        close(out[0], r_long[p], dtype, f"decoded position {p}", m_long[p])
        if second is not None:
            close(out[1], second[0], dtype, f"batch mate at step {p}", second[1])
    # the windowed groups gave pages back on the way: fewer are held than the sequence is long
    held = [len(g.seq_pages[a]) for g in eng.cache.groups]
    assert min(held) <= 3
    eng.cache.check()


@pytest.mark.gpu
def test_a_token_far_back_reaches_the_end_through_the_state_and_only_so():
    """Windowed attention beside linear attention: one early token is changed; the logits 300 positions later move (the
    state of the slow heads carries it) although every attention window has long passed it; with the linear attention
    left out of the plain statement they do not.  The engine agrees with the plain statement on both prompts, in
    portions that cut across the chunked walk."""
    from mdma_b200.engine import Engine, StepEntry
    d, cfg, W = model_of("D", "float32")
    ids = ids_of(cfg, 330, 61)
    other = list(ids)
    other[5] = (other[5] + 11) % cfg["vocab"]
    ra, rb = ref_of("D", "float32", ids)[0], ref_of("D", "float32", other)[0]
    assert np.abs(ra[-1] - rb[-1]).max() > 20 * TOL_F32
    blind = [pt.forward(cfg, W, s, skip="right")[-1] for s in (ids, other)]
    assert float((blind[0] - blind[1]).abs().max()) < 1e-9
    eng = Engine(d, dtype="float32", max_batch=2, max_context=384, logit_rows=16, page_size=16)
    s, t = eng.acquire(), eng.acquire()
    eng.step([StepEntry(s, ids[:300], []), StepEntry(t, other[:280], [])])
    out = eng.step([StepEntry(s, ids[300:], [29]), StepEntry(t, other[280:], [49])]).cpu().numpy()
    close(out[0], ra[-1], "float32", "the prompt")
    close(out[1], rb[-1], "float32", "the prompt with one early token changed")


@pytest.mark.gpu
def test_long_prompts_on_the_serving_kernels():
    """Prompts long enough for the chunked linear attention, the tiled and tcgen05 attention and the expert-by-expert
    products, in bfloat16, two unequal prompts in one step and then decoded; against the plain statement."""
    from mdma_b200.engine import Engine, StepEntry
    for key in ("A", "C"):
        d, cfg, W = model_of(key, "bfloat16")
        seqs = [ids_of(cfg, 620, 71), ids_of(cfg, 301, 72)]
        refs = [ref_of(key, "bfloat16", s) for s in seqs]
        eng = Engine(d, dtype="bfloat16", max_batch=2, max_context=640, logit_rows=64)
        slots = [eng.acquire(), eng.acquire()]
        want = [[0, 1, 30, 64, 65, 299, 300, 500, 610], [0, 20, 150, 295]]
        eng.cache.poison_unused()
        out = eng.step([StepEntry(slots[0], seqs[0][:611], want[0]), StepEntry(slots[1], seqs[1][:296], want[1])]).cpu().numpy()
        rows = np.concatenate([refs[0][0][want[0]], refs[1][0][want[1]]])
        margins = np.concatenate([refs[0][1][want[0]], refs[1][1][want[1]]])
        # long prompts meet close calls; the rows before them must agree, and most rows whatever the margins say
        got, ref = np.asarray(out, dtype=np.float64), rows
        rel = np.sqrt(((got - ref) ** 2).mean(-1)) / ref.std(-1)
        assert (rel[margins[:, 0] >= CLOSE_CALL] < 2 * TOL_ROW_BF16).all(), (key, rel, margins)
        assert (rel[margins[:, 1] >= CLOSE_CALL] < TOL_ROW_BF16).all() and rel.max() < 0.5, (key, rel, margins)
        eng.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("key", ["A", "C"])
def test_greedy_generation_through_the_scheduler(key):
    """`Engine.generate`: batches, the decode session's replayed graphs, argmax.  float32 tokens equal the plain
    statement's greedy continuation; replayed and step-by-step runs give the same tokens in both dtypes."""
    from mdma_b200.engine import Engine
    d, cfg, W = model_of(key, "float32")
    prompts = [ids_of(cfg, n, 40 + n) for n in (9, 30, 3)]
    want = []
    for p in prompts:
        ids = list(p)
        for _ in range(12):
            ids.append(int(pt.forward(cfg, W, ids)[-1].argmax()))
        want.append(ids[len(p):])
    eng = Engine(d, dtype="float32", max_batch=2, max_context=64)            # three requests, two slots: two batches
    assert eng.decode_session().graph_safe
    for graphs in (True, False):
        outs = eng.generate(prompts, max_tokens=12, use_graphs=graphs)
        assert [o.tokens for o in outs] == want, graphs
    d16, _, _ = model_of(key, "bfloat16")
    eng = Engine(d16, dtype="bfloat16", max_batch=3, max_context=64)
    a = eng.generate(prompts, max_tokens=12, use_graphs=True)
    b = eng.generate(prompts, max_tokens=12, use_graphs=False)
    assert [o.tokens for o in a] == [o.tokens for o in b]
    sampled = eng.generate(prompts, max_tokens=8, temperature=0.9, top_p=0.9, seed=3)
    assert all(len(o.tokens) == 8 for o in sampled)


@pytest.mark.gpu
def test_forty_sequences_decoded_together_replayed_and_step_by_step():
    """More sequences than the token-by-token expert kernels take in one step: a decode step of forty sorts its pairs by
    expert on the device, also inside a replayed graph."""
    from mdma_b200.engine import Engine
    d, cfg, W = model_of("A", "float32")
    prompts = [ids_of(cfg, 3 + (7 * i) % 23, 400 + i) for i in range(40)]
    eng = Engine(d, dtype="float32", max_batch=40, max_context=48)
    a = eng.generate(prompts, max_tokens=6, use_graphs=True)
    b = eng.generate(prompts, max_tokens=6, use_graphs=False)
    assert [o.tokens for o in a] == [o.tokens for o in b]
    for i in (0, 17, 39):
        ids = list(prompts[i])
        for _ in range(6):
            ids.append(int(pt.forward(cfg, W, ids)[-1].argmax()))
        assert a[i].tokens == ids[len(prompts[i]):], i


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_and_the_command_line(dtype, tmp_path):
    """`bin/trace_run` on a folder of this architecture: a prompt in a step, two requests decoded together, one ends,
    its slot is taken by a new request; `mdma plan` and `mdma run` take the folder too."""
    import subprocess
    import sys
    d, cfg, W = model_of("B", dtype)
    a, b, c = ids_of(cfg, 40, 81), ids_of(cfg, 9, 82), ids_of(cfg, 12, 83)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for j in range(4):
        steps.append({"step": 1 + j, "entries": [{"id": "a", "tokens": [a[30 + j]], "want": [0]}, {"id": "b", "tokens": [b[5 + j]], "want": [0]}],
                      "end": ["b"] if j == 3 else []})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": c, "want": [11]}], "end": ["c"]})
    steps.append({"step": 6, "entries": [{"id": "a", "tokens": a[34:], "want": [5]}], "end": ["a"]})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    res = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(7)]
    (ra, ma), (rb, mb), (rc, mc) = (ref_of("B", dtype, s) for s in (a, b, c))
    read = lambda i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    m = None if dtype == "float32" else [ma[0], ma[29], mb[4]]
    close(read(0), np.stack([ra[0], ra[29], rb[4]]), dtype, "step 0", m)
    for j in range(4):
        close(read(1 + j), np.stack([ra[30 + j], rb[5 + j]]), dtype, f"step {1 + j}", None if dtype == "float32" else [ma[30 + j], mb[5 + j]])
    close(read(5), rc[11:12], dtype, "step 5", None if dtype == "float32" else mc[11:12])
    close(read(6), ra[39:40], dtype, "step 6", None if dtype == "float32" else ma[39:40])
    if dtype == "float32":
        from mdma_b200.cli import main
        assert main(["run", d, " ".join(map(str, a[:5])), "--max-tokens", "4", "--dtype", "float32", "--max-context", "64"]) == 0
        assert main(["plan", d, "--ctx", "64"]) == 0
        assert main(["run", os.path.join(d, "config.json"), "3 1 4", "--random-weights", "7", "--max-tokens", "3", "--max-context", "32"]) == 0


def random_config(seed):
    """A configuration drawn from plausible sizes: sizes that are and are not multiples of 8 and 16, one to sixteen heads
    in one to as many groups, key and value heads of one size or two, windows from 1 to beyond the prompt or none,
    rotations of the whole head, a part of it or none, decays from fast to one, dense and routed feed-forwards and none,
    routers with and without groups, loops anywhere or nowhere, with and without the soft cap and the embedding's scale."""
    import random
    r = random.Random(seed)
    width = r.choice([32, 40, 48, 64, 96, 128, 160, 256])

    def mixer():
        heads = r.choice([1, 2, 3, 4, 6, 8, 12, 16])
        kv = r.choice([g for g in (1, 2, 3, 4, 6, 8, 12, 16) if heads % g == 0])
        dim = r.choice([8, 16, 24, 32, 48, 64, 80])
        left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": r.choice([dim, dim, 8, 16, 20, 32, 64, 96]),
                "scale": round(r.uniform(0.05, 0.4), 3), "mask": r.choice([None, {"size": r.choice([1, 2, 5, 16, 33, 64, 100, 400])}]),
                "rot": r.choice([None, {"dims": dim, "base": 10000.0}, {"dims": 2 * r.randint(1, dim // 2), "base": r.choice([100.0, 1e6])}])}
        rh = r.choice([1, 2, 3, 4, 6, 8])
        right = {"heads": rh, "dim": r.choice([4, 8, 16, 24, 32, 64]), "vdim": r.choice([4, 8, 12, 16, 32, 64]),
                 "decay": [round(r.choice([1.0, r.uniform(0.2, 0.9), r.uniform(0.9, 0.9999)]), 6) for _ in range(rh)]}
        return {"left": left, "right": right, "left_scale": round(r.uniform(0.3, 1.5), 2), "right_scale": round(r.uniform(0.3, 1.5), 2)}

    def mlp():
        kind = r.random()
        if kind < 0.15:
            return None
        if kind < 0.4:
            return {"kind": "dense", "ff": r.choice([8, 20, 32, 64, 100, 256])}
        count = r.choice([1, 1, 2, 3, 4])
        per = r.randint(1, 4)
        keep = r.randint(1, count)
        router = {"experts": count * per, "top": r.randint(1, min(keep * per, 6))}
        if count > 1 or r.random() < 0.3:
            router["groups"] = {"count": count, "keep": keep}
        return {"kind": "moe", "expert": {"ff": r.choice([8, 20, 32, 64, 100]), "limit": round(r.uniform(0.3, 4.0), 2)}, "router": router}
    n = r.randint(1, 4)
    cfg = {"architecture": "Tubusun", "vocab": r.randint(40, 500), "width": width, "norm": {"eps": r.choice([1e-5, 1e-6])},
           "layers": [{"type": "parallel", "mixer": mixer(), "mlp": mlp()} for _ in range(n)]}
    if r.random() < 0.7:
        cfg["embedding"] = {"scale": round(r.uniform(0.3, 4.0), 2)}
    if r.random() < 0.7:
        cfg["logit_softcap"] = round(r.uniform(3.0, 30.0), 1)
    if r.random() < 0.7:
        start = r.randint(0, n - 1)
        cfg["loop"] = {"start": start, "stop": r.randint(start + 1, n), "times": r.randint(1, 3)}
    return cfg


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(int(os.environ.get("TUBUSUN_DRAWN_CONFIGS", "12"))))
def test_random_configurations(seed):
    """Drawn configurations in both engines: two unequal prompts in one step, six tokens decoded, against the plain
    statement; pages of 16 or 64 rows."""
    import random
    import shutil
    from mdma_b200.engine import Engine, StepEntry
    cfg = random_config(seed)
    r = random.Random(1000 + seed)
    lengths = [r.randint(1, 90), r.randint(20, 150)]
    seqs = [ids_of(cfg, n + 6, 500 + seed + i) for i, n in enumerate(lengths)]
    for dtype in ("float32", "bfloat16"):
        d, W = make_model(cfg, 77 + seed, torch.float32 if dtype == "float32" else torch.bfloat16)
        try:
            refs = []
            for s in seqs:
                margins = []
                logits = pt.forward(cfg, W, s, margins=margins).numpy()
                refs.append((logits, margins_of(margins[-1].numpy())))
            eng = Engine(d, dtype=dtype, max_batch=2, max_context=192, logit_rows=256, page_size=r.choice([16, 64]))
            slots = [eng.acquire(), eng.acquire()]
            eng.cache.poison_unused()
            out = eng.step([StepEntry(slots[i], seqs[i][:lengths[i]], list(range(lengths[i]))) for i in range(2)]).cpu().numpy()
            m = np.concatenate([refs[i][1][:lengths[i]] for i in range(2)])
            ref = np.concatenate([refs[i][0][:lengths[i]] for i in range(2)])
            close(out, ref, dtype, f"seed {seed}: prompts {cfg}", m)
            for p in range(6):
                eng.cache.poison_unused()
                out = eng.step([StepEntry(slots[i], [seqs[i][lengths[i] + p]], [0]) for i in range(2)]).cpu().numpy()
                for i in range(2):
                    close(out[i], refs[i][0][lengths[i] + p], dtype, f"seed {seed}: decoded {p}, sequence {i}: {cfg}", refs[i][1][lengths[i] + p])
            eng.check_status()
            eng.cache.check()
            del eng
        finally:
            shutil.rmtree(d, ignore_errors=True)
