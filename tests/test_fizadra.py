"""The Fizadra architecture against its plain statement (tests/plain_fizadra.py): every mechanism alone through its
kernel, then whole models through the engine's step function, the cache manager, the scheduler and the generation
loop.  Configurations and weights are made here (tests/fizadra_tiny.py)."""
import dataclasses
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_fizadra as pf
from fizadra_tiny import CFG_A, CFG_B, CFG_C, CFG_D, L1, L2, _attention, _latent, make_model, make_tensors

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}
# float32: absolute, against the float64 statement.  bfloat16: the largest error as a share of the deviation of the
# reference logits, and a row's root-mean-square error as a share of the row's own deviation.
TOL_F32 = 5e-5
TOL_BF16, TOL_ROW_BF16 = 0.12, 0.04


def ids_of(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


_largest = {}        # the largest errors seen, printed at exit when FIZADRA_TEST_REPORT is set


_tally = {}          # per test: [rows compared in bfloat16, rows beyond the tight tolerances]
LOOSE_BF16, LOOSE_ROW_BF16, OFF_SHARE = 0.6, 0.25, 0.04


def close(got, ref, dtype, what=""):
    """float32: every logit within TOL_F32 of the float64 statement; this is the sharp test.  bfloat16: every row within
    the loose bounds (a wrong key, page or head gives a row error near 1.4), and all but a few of a test's rows (4 %, two
    at least) within the tight ones: a norm on a sublayer's result divides by that result's size, so a row whose mixer
    output is small in one part of the row turns the rounding of its inputs into several percent of the logits."""
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
    _largest[dtype] = max(_largest.get(dtype, 0.0), float(share.max()))
    _largest["row"] = max(_largest.get("row", 0.0), float(rel.max()))
    bad = (share >= LOOSE_BF16) | (rel >= LOOSE_ROW_BF16)
    assert not bad.any(), f"{what}: rows {np.nonzero(bad)[0].tolist()} are off (share {share[bad]}, row error {rel[bad]})"
    t = _tally.setdefault(os.environ.get("PYTEST_CURRENT_TEST", "").split(" (")[0], [0, 0])
    t[0] += len(share)
    t[1] += int(((share >= TOL_BF16) | (rel >= TOL_ROW_BF16)).sum())


@pytest.fixture(autouse=True)
def _few_rows_beyond_the_tight_tolerances():
    yield
    rows, off = _tally.pop(os.environ.get("PYTEST_CURRENT_TEST", "").split(" (")[0], [0, 0])
    assert off <= max(2, int(OFF_SHARE * rows)), f"{off} of {rows} bfloat16 rows are beyond the tight tolerances"


if os.environ.get("FIZADRA_TEST_REPORT"):
    import atexit
    atexit.register(lambda: print("largest errors seen:", _largest))


# =====================================================================================================
# Without a GPU: configuration, description, and that the plain statement itself notices each mechanism.

def test_config_is_read_and_checked():
    from mdma_b200.config import ConfigError, load_config
    arch, c = load_config(CFG_A)
    assert arch.name == "Fizadra" and c.groups == 2 and len(c.layers) == 5
    assert c.layers[2].mixer.kv_from == 0 and c.layers[0].mixer.rot.scaling == (4.0, 16.0, 2.0, 0.5)
    assert c.layers[1].mixer.kv_heads == 2 and c.layers[3].ff == 56 and c.layers[2].ff == 0
    spec = arch.describe(c)
    assert [e.cache for e in spec.schedule] == [None, None, 0, None, None]
    assert [e.after for e in spec.schedule] == [0, 1, 2, 3, 4]
    assert [j.params["terms"] for j in spec.junctions] == [2, 3, 4, 5, 6]

    def broken(change):
        cfg = json.loads(json.dumps(CFG_A))
        change(cfg)
        with pytest.raises(ConfigError):
            load_config(cfg)

    broken(lambda c: c["layers"][0].update(type="something_else"))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="moe"))
    broken(lambda c: c["norm"].update(groups=5))                        # 64 numbers do not split into five parts
    broken(lambda c: c["layers"][2]["mixer"].update(kv_from=2))        # not an earlier layer
    broken(lambda c: c["layers"][2]["mixer"].update(kv_from=1))        # that layer keeps no latent
    broken(lambda c: c["layers"][2]["mixer"].update(kv_rank=24))       # not the size of the cache it reads
    broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=4))       # six heads over four
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=26))   # more than a head
    broken(lambda c: c.pop("norm"))


def test_tensor_inventory_and_plan_without_a_device():
    from mdma_b200.config import load_config
    from mdma_b200.engine.model import expected_tensors
    arch, c = load_config(CFG_A)
    names = expected_tensors(arch.describe(c))
    assert names["l0.mix.dkv"].shape == (32, 64) and names["l0.mix.uq"].shape == (3 * 20, 10)
    assert "l2.mix.dkv" not in names and "l2.mix.dkv.norm" not in names and names["l2.mix.g"].shape == (20, 64)
    assert names["l3.mix.g"].shape == (2, 64) and "l3.mix.sink" not in names and names["l0.mix.sink"].shape == (3,)
    assert names["l1.mix.talk"].shape == (6, 6) and names["l1.mix.k.b"].shape == (48,) and names["l1.mix.v"].shape == (80, 64)
    assert names["l4.dwa"].shape == (6,) and "l2.mlp.up" not in names and names["head"].shape == (97, 64)
    d, _ = make_model(CFG_B, 5)
    from mdma_b200.engine.step import plan_only
    plan = plan_only(d, dtype="bfloat16", max_batch=3, max_context=128)
    assert plan["total_bytes"] > 0 and plan["slots"] == 3


def test_the_benchmark_configuration_is_a_valid_model():
    import bench
    from mdma_b200.config import load_config
    from mdma_b200.ops_tensor import attention_supported, talking_attention_mma_warps
    for width, layers in ((1024, 4), (2048, 6), (4096, 3)):
        arch, c = load_config(bench.fizadra_config(width, layers, 32000))
        spec = arch.describe(c)
        assert len(spec.schedule) == layers and all(e.cache in (None, n - 2) for n, e in enumerate(spec.schedule))
        latent = c.layers[0].mixer
        assert attention_supported(latent.heads, 1, latent.kv_rank + latent.rot_dim)       # the tensor-core kernels take it
        mixed = c.layers[1].mixer
        assert talking_attention_mma_warps(mixed.heads, mixed.kv_heads, mixed.dim, mixed.vdim) >= 2


def test_the_plain_statement_notices_each_mechanism():
    W = {n: t.double() for n, t in make_tensors(CFG_A, 3).items()}
    ids = ids_of(CFG_A, 40, 1)
    base = pf.forward(CFG_A, W, ids)
    spread = float(base.std())
    for what in ("groups", "post_norm", "depth", "sink", "gate", "talk", "one", "qk_norm", "bias", "scaling", "rotation", "shared"):
        if what == "one":
            continue
        moved = float((pf.forward(CFG_A, W, ids, leave_out=what) - base).abs().max())
        assert moved > 0.02 * spread, (what, moved, spread)
    # one added to the denominator: with keys that all score very low the weights must sum to far less than one
    s = torch.full((2, 3, 3), -4.0, dtype=torch.float64)
    assert float(pf.causal_weights(s, 0.0).sum(-1).max()) < 0.06 and abs(float(pf.causal_weights(s).sum(-1).min()) - 1) < 1e-12


def test_scaled_frequencies_of_the_rotary_part():
    from mdma_b200.parts.rotary import Rotary
    from mdma_b200.spec import PartSpec
    for rot in (CFG_A["layers"][0]["mixer"]["rot"], CFG_C["layers"][0]["mixer"]["rot"], {"base": 10000.0, "dims": 64,
                "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}):
        s = rot["scaling"]
        part = Rotary(PartSpec("rotary", dict(head_dim=rot["dims"], rotary_dim=rot["dims"], theta=rot["base"], layout="interleaved",
                                              scaling=dict(kind="ramp", magnitude_slope=0.1, **s))))
        f, mag = pf.frequencies(rot)
        assert torch.allclose(part.table_host.double(), f, rtol=1e-6) and abs(part.magnitude - mag) < 1e-12
        plainf, _ = pf.frequencies({"base": rot["base"], "dims": rot["dims"]})
        assert float((f - plainf).abs().max()) > 0 and f[0] == plainf[0]          # the fastest pair is kept, slow ones are not
    # by hand: four pairs, base 16 -> 1, 1/2, 1/4, 1/8; ramp 0, 1/2, 1, 1 from lo = 0, hi = 2; factor 2
    rot = {"base": 16.0, "dims": 8, "scaling": {"factor": 2.0, "original": 2 * math.pi * 4, "fast": 4.0, "slow": 1.0}}
    f, mag = pf.frequencies(rot)
    assert torch.allclose(f, torch.tensor([1.0, 0.375, 0.125, 0.0625], dtype=torch.float64)) and abs(mag - (0.1 * math.log(2) + 1)) < 1e-15


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


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,groups", [(64, 2), (36, 3), (128, 1), (48, 8), (320, 5), (4096, 4), (2048, 32), (96, 96)])
def test_norm_in_groups_plain_gathered_and_added(dtype, width, groups):
    from mdma_b200 import ops
    g = torch.Generator().manual_seed(width + groups)
    rows = 13
    x = torch.randn(rows, width, generator=g) * torch.linspace(0.1, 3.0, width)      # parts of very different sizes
    w = 1.0 + 0.3 * torch.randn(width, generator=g)
    wd = _dev(w, dtype)
    ref = pf.group_norm(x.double(), wd.double().cpu(), groups, 1e-5)
    out = torch.full((rows, width), 7.0, device="cuda", dtype=dtype)
    ops.group_rmsnorm(_dev(x), wd, 1e-5, groups, out)
    assert torch.allclose(out.double().cpu(), ref, **_tol(dtype))
    pick = [5, 0, 12, 5]
    out2 = torch.zeros(len(pick) + 1, width, device="cuda", dtype=dtype)
    ops.group_rmsnorm(_dev(x), wd, 1e-5, groups, out2, _i32(pick), len(pick))
    assert torch.allclose(out2[:4].double().cpu(), ref[pick], **_tol(dtype)) and float(out2[4].abs().max()) == 0
    # x += norm(y), with y still in three partial sums
    base = torch.randn(rows, width, generator=g)
    parts = torch.randn(3, rows + 2, width, generator=g)
    y0 = torch.randn(rows, width, generator=g)
    y_full = y0 + parts[:, :rows].sum(0)
    want = base.double() + pf.group_norm(y_full.double(), wd.double().cpu(), groups, 1e-5)
    xd, yd = _dev(base), _dev(y0)
    ops.group_rmsnorm_add(xd, yd, wd, 1e-5, groups, rows, _dev(parts), 3, (rows + 2) * width)
    assert torch.allclose(xd.double().cpu(), want, rtol=2e-5, atol=3e-5)
    assert torch.allclose(yd.cpu(), y_full, rtol=1e-6, atol=1e-6)                       # y is left complete
    xd, yd = _dev(base), _dev(y_full)
    ops.group_rmsnorm_add(xd, yd, wd, 1e-5, groups, rows)
    assert torch.allclose(xd.double().cpu(), want, rtol=2e-5, atol=3e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_weighted_sum_over_the_depth(wdtype):
    from mdma_b200 import ops
    g = torch.Generator().manual_seed(9)
    rows, width, depth = 11, 40, 4
    x0 = torch.randn(rows, width, generator=g)
    history = torch.full((rows + 1, depth * width), float("nan"), device="cuda")
    results, x0d = [x0.double()], _dev(x0)
    for run in range(depth):
        w = _dev(torch.randn(run + 2, generator=g), wdtype)
        mine = torch.randn(rows, width, generator=g)
        results.append(mine.double())
        xd = _dev(mine)
        ops.depth_mix(xd, x0d, history, depth, run, w, rows)
        want = sum(w.double().cpu()[j] * results[j] for j in range(run + 2))
        assert torch.allclose(xd.double().cpu(), want, rtol=1e-5, atol=1e-5), run
    assert torch.isnan(history[rows]).all()


def _turn(x, pos, dims, base, layout, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return pf.rotate(x, torch.as_tensor(pos), rot, layout)


def _rotary_part(head, dims, base, layout, scaling=None):
    from mdma_b200.parts.base import Runtime
    from mdma_b200.parts.rotary import Rotary
    from mdma_b200.spec import PartSpec
    sc = None if scaling is None else dict(kind="ramp", magnitude_slope=0.1, **dict(zip(("factor", "original", "fast", "slow"), scaling)))
    part = Rotary(PartSpec("rotary", dict(head_dim=head, rotary_dim=dims, theta=base, layout=layout, scaling=sc)))
    part.bind({}, Runtime(torch.float32, torch.device("cuda")))
    return part


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_rank,rank,rot_dim,dims,layout,scaling", [
    (10, 20, 12, 12, "interleaved", (4.0, 16, 2.0, 0.5)), (7, 9, 10, 10, "split_half", None), (64, 96, 32, 32, "interleaved", None),
    (5, 30, 2, 2, "split_half", None), (24, 200, 16, 8, "interleaved", (2.0, 64, 8.0, 1.0))])
def test_latents_normed_key_part_turned_and_cached(dtype, q_rank, rank, rot_dim, dims, layout, scaling):
    """Two sequences with cached prefixes, scattered pages; a second call that must not write; query heads turned in
    place at an offset."""
    from mdma_b200 import ops
    g = torch.Generator().manual_seed(q_rank * 7 + rank)
    page, max_pages = 4, 8
    st = _Step([5, 3], [6, 0], [2, 0])
    pos = st.tok_pos.cpu().numpy()
    n = st.n_tokens
    width = q_rank + rank + rot_dim + 3
    proj = torch.randn(n, width + 5, generator=g)[:, :width] * 2.0
    qw, kw = 1 + 0.3 * torch.randn(q_rank, generator=g), 1 + 0.3 * torch.randn(rank, generator=g)
    projd = _dev(torch.cat([proj, torch.zeros(n, 5)], 1), dtype)[:, :width]
    qwd, kwd = _dev(qw, dtype), _dev(kw, dtype)
    table = torch.zeros(3, max_pages, dtype=torch.int32)
    table[2, :3] = torch.tensor([9, 1, 6], dtype=torch.int32)
    table[0, :1] = torch.tensor([4], dtype=torch.int32)
    cache = torch.full((12, page, 1, rank + rot_dim), float("nan"), device="cuda", dtype=dtype)
    cq = torch.zeros(n, q_rank, device="cuda", dtype=dtype)
    part = _rotary_part(rot_dim, dims, 100.0, layout, scaling)
    inv_freq, rd, inter = part.rotary_table()
    ops.latent_prepare(projd, 0, q_rank, qwd, q_rank, rank, kwd, 1e-5, rot_dim, rd, inter, inv_freq, part.magnitude,
                       st.tok_seq, st.tok_pos, st.seq_slot, table.cuda(), max_pages, page, cq, cache, True, n)
    p64 = projd.double().cpu()
    want_q = pf.rms_unit(p64[:, :q_rank], 1e-5) * qwd.double().cpu()
    want_c = pf.rms_unit(p64[:, q_rank:q_rank + rank], 1e-5) * kwd.double().cpu()
    want_r = _turn(p64[:, None, q_rank + rank:q_rank + rank + rot_dim], pos, dims, 100.0, layout, scaling)[:, 0]
    assert torch.allclose(cq.double().cpu(), want_q, **_tol(dtype))
    slots = [2] * 5 + [0] * 3
    for t in range(n):
        row = cache[int(table[slots[t], pos[t] // page]), pos[t] % page, 0].double().cpu()
        assert torch.allclose(row[:rank], want_c[t], **_tol(dtype)) and torch.allclose(row[rank:], want_r[t], **_tol(dtype)), t
    assert int(torch.isfinite(cache.float()).all(-1).sum()) == n                     # no other row was touched
    before = cache.clone()
    ops.latent_prepare(projd, 0, q_rank, qwd, 0, 0, None, 1e-5, 0, 0, inter, None, 1.0, st.tok_seq, st.tok_pos, st.seq_slot,
                       None, 0, 0, cq, None, False, n)
    assert torch.equal(torch.nan_to_num(cache.float()), torch.nan_to_num(before.float()))
    # query heads [plain | turned] turned in place
    H, plain = 3, 5
    q = torch.randn(n, H, plain + rot_dim, generator=g)
    qd = _dev(q.reshape(n, -1), dtype)
    ops.rotate_heads(qd, H, plain + rot_dim, plain, rd, inter, inv_freq, part.magnitude, st.tok_pos, n)
    q64 = _dev(q.reshape(n, -1), dtype).double().cpu().reshape(n, H, -1)
    want = q64.clone()
    want[..., plain:] = _turn(q64[..., plain:], pos, dims, 100.0, layout, scaling)
    assert torch.allclose(qd.double().cpu().reshape(n, H, -1), want, **_tol(dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,V,dims,norm", [(6, 2, 24, 40, 8, True), (5, 1, 12, 4, 2, True), (8, 2, 64, 64, 32, True),
                                               (3, 3, 12, 12, 12, False), (4, 2, 16, 8, 0, True)])
def test_heads_normed_then_turned_and_cached(dtype, H, G, D, V, dims, norm):
    from mdma_b200 import ops
    g = torch.Generator().manual_seed(H * 11 + D)
    page, max_pages = 4, 8
    st = _Step([4, 6], [3, 0], [1, 2])
    pos, n = st.tok_pos.cpu().numpy(), st.n_tokens
    width = H * D + G * D + G * V
    rows = _dev(torch.randn(n, width + 8, generator=g) * 1.5, dtype)[:, :width]
    qw, kw = _dev(1 + 0.3 * torch.randn(D, generator=g), dtype), _dev(1 + 0.3 * torch.randn(D, generator=g), dtype)
    table = torch.zeros(3, max_pages, dtype=torch.int32)
    table[1, :2] = torch.tensor([7, 2], dtype=torch.int32)
    table[2, :2] = torch.tensor([5, 0], dtype=torch.int32)
    kc = torch.full((9, page, G, D), float("nan"), device="cuda", dtype=dtype)
    vc = torch.full((9, page, G, V), float("nan"), device="cuda", dtype=dtype)
    src = rows.double().cpu()
    part = _rotary_part(D, dims, 50.0, "split_half") if dims else None
    inv_freq, rd, inter = part.rotary_table() if part else (None, 0, False)
    ops.qk_norm_rotate(rows, H * D, H * D + G * D, st.tok_seq, st.tok_pos, st.seq_slot, inv_freq, 1.0, qw if norm else None,
                       kw if norm else None, norm, 1e-5, kc, vc, table.cuda(), max_pages, page, n, H, G, D, V, rd, inter, True)
    q, k = src[:, :H * D].reshape(n, H, D), src[:, H * D:H * D + G * D].reshape(n, G, D)
    if norm:
        q, k = pf.rms_unit(q, 1e-5) * qw.double().cpu(), pf.rms_unit(k, 1e-5) * kw.double().cpu()
    if dims:
        q, k = _turn(q, pos, dims, 50.0, "split_half"), _turn(k, pos, dims, 50.0, "split_half")
    assert torch.allclose(rows[:, :H * D].double().cpu().reshape(n, H, D), q, **_tol(dtype))
    slots = [1] * 4 + [2] * 6
    for t in range(n):
        pg, r = int(table[slots[t], pos[t] // page]), pos[t] % page
        assert torch.allclose(kc[pg, r].double().cpu(), k[t], **_tol(dtype)), t
        assert torch.equal(vc[pg, r].double().cpu(), src[t, H * D + G * D:].reshape(G, V)), t
    assert int(torch.isfinite(kc.float()).all(-1).all(-1).sum()) == n


def _plain_mixed_attention(q, k, v, talk, sink, scale, pos0):
    """q [n, H, D] at positions pos0.., k [len, G, D], v [len, G, V] of one sequence; float64."""
    n, H, _ = q.shape
    rep = H // k.shape[1]
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if talk is not None:
        s = torch.einsum("hg,gij->hij", talk, s)
    j = torch.arange(kk.shape[0])[None, :]
    i = (pos0 + torch.arange(n))[:, None]
    s = s.masked_fill((j > i)[None], -math.inf)
    if sink is not None:
        s = torch.cat([s, sink.double()[:, None, None].expand(H, n, 1)], -1)
    p = torch.softmax(s, -1)[..., :kk.shape[0]]
    return torch.einsum("hij,jhd->ihd", p, vv)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tiled", [False, True, "mma"])
@pytest.mark.parametrize("H,G,D,V,talk,sink", [(6, 2, 24, 40, True, True), (6, 2, 24, 48, True, True), (7, 1, 16, 16, True, False), (5, 1, 12, 4, True, True), (4, 4, 96, 96, True, True),
                                               (8, 2, 64, 64, True, False), (3, 3, 16, 16, False, True), (16, 4, 128, 128, True, True),
                                               (32, 8, 32, 48, True, True)])
def test_attention_with_mixed_scores_far_key_pages_and_batches(dtype, tiled, H, G, D, V, talk, sink):
    """Three sequences of unequal lengths in one call: a prompt from position 0, a portion on a cached prefix that
    crosses page borders, a single token far into its sequence.  In the long sequence one early key is made to stand
    out for one head through one coordinate, so that a kernel that loses far keys, mixes the wrong heads or reads the
    wrong page shows.  Pages are scattered; every row nobody owns holds NaN."""
    from mdma_b200 import ops
    if tiled == "mma":
        from mdma_b200 import ops_tensor
        from mdma_b200.cache import KVView
        if dtype != torch.bfloat16 or not talk or not ops_tensor.talking_attention_mma_warps(H, G, D, V):
            pytest.skip("the tensor-core kernel takes bfloat16, a mixing matrix and sizes in sixteens")
    elif tiled and not ops.talking_attention_tiled_fits(H, G, D, V):
        pytest.skip("beyond the tiled kernel's shared memory")
    g = torch.Generator().manual_seed(H * 13 + D + V)
    page, max_pages = 16, 24
    lens, new = [37, 150, 333], [37, 50, 1]
    pos0 = [l - n for l, n in zip(lens, new)]
    st = _Step(new, pos0, [3, 0, 5])
    n = st.n_tokens
    ks = [torch.randn(l, G, D, generator=g) for l in lens]
    vs = [torch.randn(l, G, V, generator=g) for l in lens]
    qs = [torch.randn(m, H, D, generator=g) for m in new]
    ks[2][7, 0, 3] = 12.0                                # the far key: position 7 of 333
    qs[2][0, 0, 3] = 6.0
    vs[2][7, 0] += 2.0
    ks[1][2, G - 1, 1] = 8.0
    qs[1][:, H - 1, 1] = 4.0
    T = (torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)) if talk else None
    S = (1.5 * torch.randn(H, generator=g)) if sink else None
    scale = 0.3
    perm = torch.randperm(60, generator=g).tolist()
    table = torch.zeros(6, max_pages, dtype=torch.int32)
    kc = torch.full((60, page, G, D), float("nan"), device="cuda", dtype=dtype)
    vc = torch.full((60, page, G, V), float("nan"), device="cuda", dtype=dtype)
    for s, slot in enumerate([3, 0, 5]):
        for p in range(-(-lens[s] // page)):
            pg = perm.pop()
            table[slot, p] = pg
            m = min(page, lens[s] - p * page)
            kc[pg, :m] = _dev(ks[s][p * page:p * page + m], dtype)
            vc[pg, :m] = _dev(vs[s][p * page:p * page + m], dtype)
    qd = _dev(torch.cat([q.reshape(q.shape[0], -1) for q in qs]), dtype)
    out = torch.zeros(n, H * V, device="cuda", dtype=dtype)
    Td, Sd = (None if T is None else _dev(T)), (None if S is None else _dev(S))

    def attend(q_rows, step, o):
        if tiled == "mma":
            x = torch.full((step.n_tokens + 1, H * G * D), float("nan"), device="cuda", dtype=dtype)
            parts = 5 if step.max_new == 1 else 1             # a single token: its keys divided over five blocks
            scratch = torch.full((step.n_tokens * H * parts * (V + 2) + 3,), float("nan"), device="cuda")
            ops_tensor.talking_attention_mma(step, q_rows, Td, x, KVView(kc, vc, table.cuda(), page, max_pages, 0),
                                             None if S is None else _dev(S * 1.4426950408889634), o, H, G, D, V, 0, scale,
                                             splits=parts, partial=scratch)
            assert torch.isnan(scratch[-3:]).all() and torch.isnan(x[-1]).all()
        else:
            ops.talking_attention(q_rows, kc, vc, Td, Sd, step, table.cuda(), max_pages, page, o, H, G, D, V, 0, scale, tiled=tiled)

    attend(qd, st, out)
    rd = lambda t: _dev(t, dtype).double().cpu()
    want = torch.cat([_plain_mixed_attention(rd(qs[s]), rd(ks[s]), rd(vs[s]), None if T is None else T.double(), S, scale, pos0[s])
                      .reshape(new[s], -1) for s in range(3)])
    got = out.double().cpu()
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **(dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)))
    # the far key carries most of head 0's weight at the last token: without it the row would be another
    blind_k = rd(ks[2]).clone()
    blind_k[7, 0, 3] = 0.0
    blind = _plain_mixed_attention(rd(qs[2]), blind_k, rd(vs[2]), None if T is None else T.double(), S, scale, pos0[2]).reshape(1, -1)
    assert float((blind - want[-1:]).abs().max()) > 0.5
    # each sequence alone gives the same rows
    o = 0
    for s, slot in enumerate([3, 0, 5]):
        one = _Step([new[s]], [pos0[s]], [slot])
        alone = torch.zeros(new[s], H * V, device="cuda", dtype=dtype)
        attend(qd[o:o + new[s]], one, alone)
        if dtype == torch.float32 and not tiled:
            assert torch.equal(alone, out[o:o + new[s]])
        else:
            assert torch.allclose(alone.float(), out[o:o + new[s]].float(), rtol=2e-2, atol=2e-2)
        o += new[s]


@pytest.mark.gpu
@pytest.mark.parametrize("impl", ["plain32", "plain16", "mma", "tc"])
@pytest.mark.parametrize("H,rank,rot,sink", [(3, 20, 12, True), (8, 96, 32, True), (4, 48, 16, False), (2, 96, 32, False), (5, 112, 16, True)])
def test_cached_vectors_as_key_and_value_far_key_with_and_without_sink(impl, H, rank, rot, sink):
    """The attention of the latent layers over cached vectors [latent | key part]: the plain kernel in both dtypes and
    the tensor-core kernels where they take the size.  A far key is made to stand out through a coordinate of the key
    part; without a sink pointer the softmax is the ordinary one."""
    from mdma_b200 import ops
    from mdma_b200.cache import KVView
    row = rank + rot
    dtype = torch.float32 if impl == "plain32" else torch.bfloat16
    if impl in ("mma", "tc"):
        from mdma_b200 import ops_tensor
        if not ops_tensor.attention_supported(H, 1, row) or (impl == "tc" and not ops_tensor.attention_tc_supported(H, 1, row, 64)):
            pytest.skip("the tensor-core kernels do not take this size")
    g = torch.Generator().manual_seed(H + row)
    page, max_pages = 64, 8
    lens, new = [300, 70], [300, 1]
    st = _Step(new, [0, 69], [1, 0])
    cs = [torch.randn(l, row, generator=g) * 0.7 for l in lens]
    qs = [torch.randn(m, H, row, generator=g) * 0.7 for m in new]
    cs[0][5, rank + 1] = 6.0
    qs[0][250:, 1 % H, rank + 1] = 6.0
    cs[1][3, rank] = 7.0
    qs[1][0, 0, rank] = 5.0
    S = (1.5 * torch.randn(H, generator=g)) if sink else None
    scale = 0.25
    table = torch.zeros(2, max_pages, dtype=torch.int32)
    cache = torch.full((9, page, 1, row), float("nan"), device="cuda", dtype=dtype)
    pages = [[6, 2, 8, 0, 4], [7, 3]]
    for s, slot in enumerate([1, 0]):
        for p, pg in enumerate(pages[s]):
            table[slot, p] = pg
            m = min(page, lens[s] - p * page)
            cache[pg, :m, 0] = _dev(cs[s][p * page:p * page + m], dtype)
    qd = _dev(torch.cat([q.reshape(q.shape[0], -1) for q in qs]), dtype)
    out = torch.zeros(st.n_tokens, H * row, device="cuda", dtype=dtype)
    if impl.startswith("plain"):
        Sd = None if S is None else _dev(S, dtype)
        ops.latent_attention(qd, cache, Sd, st.tok_seq, st.tok_pos, st.seq_slot, table.cuda(), max_pages, page, out, st.n_tokens,
                             H, row, 0, scale)
        S_used = None if S is None else Sd.double().cpu()
    else:
        view = KVView(cache, cache, table.cuda(), page, max_pages, 0)
        s2 = None if S is None else _dev(S * 1.4426950408889634)
        ops_tensor.attention(_Step([300], [0], [1]), qd[:300], view, out[:300], H, 1, row, 0, scale, impl=impl, sink_log2=s2)
        ops_tensor.attention(_Step([1], [69], [0]), qd[300:], view, out[300:], H, 1, row, 0, scale, impl="mma", sink_log2=s2)
        S_used = None if S is None else S.double()
    rd = lambda t: _dev(t, dtype).double().cpu()
    want = torch.cat([_plain_mixed_attention(rd(qs[s]), rd(cs[s])[:, None, :], rd(cs[s])[:, None, :], None, S_used, scale, [0, 69][s])
                      .reshape(new[s], -1) for s in range(2)])
    got = out.double().cpu().reshape(-1, H, row)[..., :rank]
    want = want.reshape(-1, H, row)[..., :rank]
    assert torch.allclose(got, want, **(dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)))
    blind_c = rd(cs[1]).clone()
    blind_c[3, rank] = 0.0
    blind = _plain_mixed_attention(rd(qs[1]), blind_c[:, None, :], blind_c[:, None, :], None, S_used, scale, 69).reshape(1, H, row)[..., :rank]
    assert float((blind - want[-1:]).abs().max()) > 0.1


@pytest.mark.gpu
@pytest.mark.parametrize("engine", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,ff", [(36, 30), (64, 48), (128, 192)])
def test_feed_forward_with_the_squared_relu(engine, W, ff):
    from mdma_b200.engine.step import StepContext
    from mdma_b200.parts.base import Runtime
    from mdma_b200.parts.mlp import DenseMLP
    from mdma_b200.spec import PartSpec
    dtype = torch.float32 if engine == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(W)
    n = 9
    up, down = torch.randn(ff, W, generator=g) / W ** 0.5, torch.randn(W, ff, generator=g) / ff ** 0.5
    h = torch.randn(n, W, generator=g)
    rt = Runtime(dtype, torch.device("cuda"), gemm="tensor" if engine == "bfloat16" else "simt")
    if engine == "bfloat16":
        from mdma_b200 import ops_tensor
        rt.tc = ops_tensor._device_state(torch.device("cuda", torch.cuda.current_device()))
    part = DenseMLP(PartSpec("dense_mlp", dict(hidden_size=W, intermediate_size=ff, activation="relu_squared")))
    tensors = {"up": _dev(up, dtype), "down": _dev(down, dtype)}
    part.bind(tensors, rt)

    class Ctx:
        n_tokens = n

        def __init__(self):
            self.rt = rt
            self.bufs = {k: torch.zeros(n, c, device="cuda", dtype=dtype if kind == "act" else torch.float32)
                         for k, (c, kind) in part.workspace().items()}

        def buf(self, name, cols, dt=None):
            return self.bufs[name][:, :cols]

    x = torch.zeros(n, W, device="cuda")
    hd = _dev(h, dtype)
    part.forward(Ctx(), hd, x)
    if engine == "bfloat16":
        ops_tensor.flush_pending(x.device, rt.tc)
    want = pf.feed_forward(hd.double().cpu(), {"up": tensors["up"].double().cpu(), "down": tensors["down"].double().cpu()}, "")
    assert torch.allclose(x.double().cpu(), want, **(dict(rtol=1e-4, atol=1e-4) if engine == "float32" else dict(rtol=3e-2, atol=3e-2)))


# =====================================================================================================
# Whole models through the engine (GPU).

_models: dict = {}


def model_of(key, dtype, cfg=None, seed=None):
    """(folder, config, float64 tensors as the engine holds them) of configuration `key`."""
    k = (key, dtype)
    if k not in _models:
        store = torch.float32 if dtype == "float32" else torch.bfloat16
        cfg = cfg or CONFIGS[key]
        d, W = make_model(cfg, seed if seed is not None else 23 + ord(key[0]), store)
        _models[k] = (d, cfg, W)
    return _models[k]


_refs: dict = {}


def ref_of(key, dtype, ids):
    k = (key, dtype, tuple(ids))
    if k not in _refs:
        _, cfg, W = model_of(key, dtype)
        _refs[k] = pf.forward(cfg, W, ids).numpy()
    return _refs[k]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C", "D"])
def test_every_layer_against_the_plain_statement(key, dtype):
    """The residual stream after every layer (after its weighted sum over the depth), then the logits; one short
    prompt, the first tokens among the rows."""
    from mdma_b200.engine import Engine, StepEntry
    d, cfg, W = model_of(key, dtype)
    ids = ids_of(cfg, 21, 4)
    ref, trace = pf.forward(cfg, W, ids, return_layers=True)
    eng = Engine(d, dtype=dtype, max_batch=2, max_context=64, logit_rows=64, page_size=16)
    got = []
    eng.model.on_layer = lambda n, x: got.append(x.detach().double().cpu())
    s = eng.acquire()
    logits = eng.step([StepEntry(s, ids, list(range(len(ids))))]).cpu().numpy()
    assert len(got) == len(trace) == len(cfg["layers"])
    tol = 1e-4 if dtype == "float32" else 0.04
    for n, (a, b) in enumerate(zip(got, trace)):
        err = float((a - b).abs().max())
        assert err < tol * max(1.0, float(b.abs().max())), f"after layer {n}: {err}"
    close(logits, ref.numpy(), dtype, "logits")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C", "D"])
def test_batches_portions_decoding_and_reuse(key, dtype):
    """Unequal prompts in one step; the same prompts cut in portions down to one and two tokens on a cached prefix;
    token-by-token decoding; sequences that end early while others go on; slots and pages freed and taken again (rows
    nobody owns hold NaN throughout).  In float32 every way of cutting gives the same logits to within a few units of
    the last place."""
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
                    eng.release(slots[i])           # ends early; its slot and its pages go back
        eng.cache.check()
        return [np.concatenate(r) for r in rows]

    whole = run([[n] for n in lengths])
    for i, (got, ref) in enumerate(zip(whole, refs)):
        close(got, ref, dtype, f"whole prompts, sequence {i}")
    alone = []
    for i, s in enumerate(seqs):                    # each alone, in a slot that the batch used
        slot = eng.acquire()
        alone.append(eng.step([StepEntry(slot, s, list(range(len(s))))]).cpu().numpy().copy())
        eng.release(slot)
    pieces = run([[2, 1, 30, 17, 1, 2, 16, 1], [1], [16, 1, 15, 1], [1, 1], [3, 14]])
    decoded = run([[25] + [1] * 45, [1], [1] * 33, [2], [16, 1]])
    for name, other in (("alone", alone), ("portions", pieces), ("decoded", decoded)):
        for i, (got, ref) in enumerate(zip(other, refs)):
            close(got, ref, dtype, f"{name}, sequence {i}")
            if dtype == "float32":
                assert np.abs(got - whole[i]).max() <= 4e-6, f"{name}, sequence {i}: differs from the whole prompt"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_passes_smaller_than_a_step_and_long_decoding(dtype):
    """A step run as passes of 7 tokens (cuts inside sequences), then 150 tokens decoded one by one across many page
    borders, beside a batch mate that ends on the way and whose slot another request takes."""
    from mdma_b200.engine import Engine, StepEntry
    d, cfg, W = model_of("A", dtype)
    long_ids, mate, late = ids_of(cfg, 190, 31), ids_of(cfg, 60, 32), ids_of(cfg, 25, 33)
    r_long, r_mate, r_late = (ref_of("A", dtype, s) for s in (long_ids, mate, late))
    eng = Engine(d, dtype=dtype, max_batch=2, max_context=192, logit_rows=64, page_size=16, chunk_tokens=7)
    a, b = eng.acquire(), eng.acquire()
    out = eng.step([StepEntry(a, long_ids[:40], [0, 39, 6, 7]), StepEntry(b, mate[:41], [40, 13])]).cpu().numpy()
    assert eng.forward_passes > 10
    close(out, np.stack([r_long[0], r_long[39], r_long[6], r_long[7], r_mate[40], r_mate[13]]), dtype, "passes")
    pb = 41
    for p in range(40, 190):
        entries = [StepEntry(a, [long_ids[p]], [0])]
        second = None
        if pb < len(mate):
            entries.append(StepEntry(b, [mate[pb]], [0]))
            second = r_mate[pb]
            pb += 1
        elif pb == len(mate):                       # the mate is done: its slot goes to a late request
            eng.release(b)
            b = eng.acquire()
            entries.append(StepEntry(b, late, [len(late) - 1]))
            second = r_late[-1]
            pb += 1
        eng.cache.poison_unused()
        out = eng.step(entries).cpu().numpy()
        close(out[0], r_long[p], dtype, f"decoded position {p}")
        if second is not None:
            close(out[1], second, dtype, f"batch mate at step {p}")
    eng.cache.check()


@pytest.mark.gpu
def test_a_token_far_back_moves_the_end_and_the_engine_follows():
    """One early token of a prompt of 330 is changed: the last logits move, in the plain statement and in the engine
    alike, in portions that cut across pages."""
    from mdma_b200.engine import Engine, StepEntry
    d, cfg, W = model_of("B", "float32")
    ids = ids_of(cfg, 330, 61)
    other = list(ids)
    other[5] = (other[5] + 11) % cfg["vocab"]
    ra, rb = ref_of("B", "float32", ids), ref_of("B", "float32", other)
    assert np.abs(ra[-1] - rb[-1]).max() > 20 * TOL_F32
    eng = Engine(d, dtype="float32", max_batch=2, max_context=384, logit_rows=16, page_size=16)
    s, t = eng.acquire(), eng.acquire()
    eng.step([StepEntry(s, ids[:300], []), StepEntry(t, other[:280], [])])
    out = eng.step([StepEntry(s, ids[300:], [29]), StepEntry(t, other[280:], [49])]).cpu().numpy()
    close(out[0], ra[-1], "float32", "the prompt")
    close(out[1], rb[-1], "float32", "the prompt with one early token changed")


@pytest.mark.gpu
@pytest.mark.parametrize("key", ["A", "C"])
def test_long_prompts_on_the_serving_kernels(key):
    """Prompts long enough for the tiled attention with mixed scores, the tensor-core attention over cached vectors and
    the per-head tensor-core products, in bfloat16: two unequal prompts in one step, then decoded."""
    from mdma_b200.engine import Engine, StepEntry
    d, cfg, W = model_of(key, "bfloat16")
    seqs = [ids_of(cfg, 620, 71), ids_of(cfg, 301, 72)]
    refs = [ref_of(key, "bfloat16", s) for s in seqs]
    eng = Engine(d, dtype="bfloat16", max_batch=2, max_context=640, logit_rows=64)
    slots = [eng.acquire(), eng.acquire()]
    want = [[0, 1, 30, 64, 65, 299, 300, 500, 610], [0, 20, 150, 295]]
    eng.cache.poison_unused()
    out = eng.step([StepEntry(slots[0], seqs[0][:611], want[0]), StepEntry(slots[1], seqs[1][:296], want[1])]).cpu().numpy()
    close(out, np.concatenate([refs[0][want[0]], refs[1][want[1]]]), "bfloat16", "long prompts")
    for j in range(5):
        eng.cache.poison_unused()
        out = eng.step([StepEntry(slots[0], [seqs[0][611 + j]], [0]), StepEntry(slots[1], [seqs[1][296 + j]], [0])]).cpu().numpy()
        close(out, np.stack([refs[0][611 + j], refs[1][296 + j]]), "bfloat16", f"decoded token {j}")
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
            ids.append(int(pf.forward(cfg, W, ids)[-1].argmax()))
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
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_and_the_command_line(dtype, tmp_path):
    """`bin/trace_run` on a folder of this architecture: a prompt in a step, two requests decoded together, one ends,
    its slot is taken by a new request; `mdma plan` and `mdma run` take the folder too."""
    import subprocess
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
    ra, rb, rc = (ref_of("B", dtype, s) for s in (a, b, c))
    read = lambda i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    close(read(0), np.stack([ra[0], ra[29], rb[4]]), dtype, "step 0")
    for j in range(4):
        close(read(1 + j), np.stack([ra[30 + j], rb[5 + j]]), dtype, f"step {1 + j}")
    close(read(5), rc[11:12], dtype, "step 5")
    close(read(6), ra[39:40], dtype, "step 6")
    if dtype == "float32":
        from mdma_b200.cli import main
        assert main(["run", d, " ".join(map(str, a[:5])), "--max-tokens", "4", "--dtype", "float32", "--max-context", "64"]) == 0
        assert main(["plan", d, "--ctx", "64"]) == 0
        assert main(["run", os.path.join(d, "config.json"), "3 1 4", "--random-weights", "7", "--max-tokens", "3", "--max-context", "32"]) == 0


def random_config(seed):
    """A configuration drawn from a seed: layer kinds in any order, shared caches where a source exists, head counts,
    head sizes, latents and parts of a row of many sizes, some multiples of 8 or 16 and some not."""
    rng = np.random.default_rng(1000 + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]
    groups = pick([1, 2, 3, 4, 6])
    width = groups * pick([16, 20, 24, 32, 48])
    layers, sources = [], {}
    for i in range(int(rng.integers(1, 6))):
        ff = pick([None, 24, 40, 64])
        kind = pick([L1, L2, "attention"])
        if kind == "attention":
            G = pick([1, 2, 3, 4])
            H = G * pick([1, 2, 3])
            D = pick([8, 12, 16, 32, 48])
            dims = pick([2, D // 2 // 2 * 2, D])
            layers.append(_attention(H, G, D, pick([4, 8, D, 24]), float(rng.uniform(0.15, 0.4)), dims, pick([7.0, 1e4, 1e6]), ff=ff))
            continue
        share = [j for j, k in sources.items() if k[0] == kind]
        if share and rng.random() < 0.5:
            j = pick(share)
            _, rank, rot_dim, base, scaling = sources[j]
            kv_from = j
        else:
            rank, rot_dim, base = pick([9, 16, 24, 48, 96, 112]), pick([2, 8, 16, 32]), pick([7.0, 1e4, 1e6])
            scaling = pick([None, (2.0, 32, 8.0, 1.0), (8.0, 16, 4.0, 0.5)]) if kind == L1 else None
            kv_from = None
            sources[i] = (kind, rank, rot_dim, base, scaling)
        layers.append(_latent(kind, pick([1, 2, 3, 5, 8]), pick([4, 8, 16, 24, 32]), rot_dim, pick([4, 8, 16, 20]), rank,
                              pick([6, 8, 16, 40]), float(rng.uniform(0.15, 0.4)), base, scaling=scaling, kv_from=kv_from, ff=ff))
    return {"architecture": "Fizadra", "vocab": int(rng.integers(40, 200)), "width": width,
            "norm": {"eps": pick([1e-5, 1e-6]), "groups": groups}, "layers": layers}


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(int(os.environ.get("FIZADRA_DRAWN_CONFIGS", "12"))))
def test_random_configurations(seed):
    """Drawn configurations in both engines: a batch of unequal prompts, portions on a cached prefix, decoding."""
    from mdma_b200.engine import Engine, StepEntry
    cfg = random_config(seed)
    for dtype in ("float32", "bfloat16"):
        d, _, W = model_of(f"drawn{seed}", dtype, cfg, seed)
        seqs = [ids_of(cfg, n, 90 + i) for i, n in enumerate((75, 12, 300))]
        refs = [pf.forward(cfg, W, s).numpy() for s in seqs]
        eng = Engine(d, dtype=dtype, max_batch=3, max_context=320, logit_rows=128)
        slots = [eng.acquire() for _ in seqs]
        eng.cache.poison_unused()
        first = [60, 12, 280]
        out = eng.step([StepEntry(slots[i], seqs[i][:first[i]], [0, 1, first[i] - 1]) for i in range(3)]).cpu().numpy()
        want = np.concatenate([refs[i][[0, 1, first[i] - 1]] for i in range(3)])
        check = lambda g, r, what: close(g, r, dtype, what)
        check(out, want, f"seed {seed} {dtype}: prompts")
        eng.release(slots[1])
        eng.cache.poison_unused()
        out = eng.step([StepEntry(slots[0], seqs[0][60:67], [6]), StepEntry(slots[2], seqs[2][280:282], [0, 1])]).cpu().numpy()
        check(out, np.stack([refs[0][66], refs[2][280], refs[2][281]]), f"seed {seed} {dtype}: portions")
        for j in range(8):
            eng.cache.poison_unused()
            out = eng.step([StepEntry(slots[0], [seqs[0][67 + j]], [0]), StepEntry(slots[2], [seqs[2][282 + j]], [0])]).cpu().numpy()
            check(out, np.stack([refs[0][67 + j], refs[2][282 + j]]), f"seed {seed} {dtype}: decoded {j}")
        eng.cache.check()
        eng.check_status()
