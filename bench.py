#!/usr/bin/env python3
"""Benchmark: decode tokens/s and prefill tokens/s at the Llama-3.1-8B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]
    python bench.py --shape llama-2-7b | llama-3.2-1b [--batch B] [--prompt-len P] [--prefill-tokens T]
    python bench.py --compare gevonex|mogevik|tubusun|fizadra [--compare-widths 1024,2048,4096] [--compare-layers 4]

Prints ONE JSON line.  The default run has the layer sizes of the
Llama-3.1-8B shape with random bfloat16 weights, a batch of 8 sequences
decoding after 512-token prompts in a cache sized for a context of 4096.  A
"step" is one decode step of the whole batch (forward, token selection,
feeding the tokens back).  `value` is timed on the device with CUDA events
around exactly K steps; `e2e` is the same through the Python entry point
(`Generator.generate`, host token lists in and out).  Decoding streams 15 GB
of weights per step, far more than the 126 MB L2, so nothing is flushed
between steps.

`--compare gevonex` is another program: prefill and decode throughput of the
Gevonex architecture (recurrent and latent-attention mixers, random weights)
at a few layer sizes, beside a Llama of the same width, depth and vocabulary,
each with the share of the measured peaks it reaches.  It prints one JSON line
of its own; the default workload and its line are unchanged.

`--compare mogevik` does the same for the Mogevik architecture (RG-LRU and
windowed attention with a distance penalty, routed feed-forwards) beside a
Gevonex and a Llama of the same width, depth and vocabulary and the same
number of matrix elements a token uses.

`--compare tubusun` does the same for the Tubusun architecture (windowed
attention with a sink and head gates side by side with linear attention,
norms around every sublayer, dense and routed feed-forwards) beside a Mogevik
and a Llama of the same width, depth and vocabulary.

`--compare fizadra` does the same for the Fizadra architecture (attention
over a cached latent with a turned key part, attention whose heads' scores
are mixed, grouped norms around every sublayer, a weighted sum over the
depth) beside a Gevonex (the other model with a cached latent) and a Llama.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_31_8B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=32, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
    rope_theta=500000.0, rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                           high_freq_factor=4.0, original_max_position_embeddings=8192),
    rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=131072)
# The other shapes that the baseline names (same architecture, other sizes): `--shape` picks one.
LLAMA_2_7B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=32, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=32, head_dim=128, intermediate_size=11008, vocab_size=32000,
    rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=4096)
LLAMA_32_1B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=16, hidden_size=2048,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256,
    rope_theta=500000.0, rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0,
                                           high_freq_factor=4.0, original_max_position_embeddings=8192),
    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)
SHAPES = {"llama-3.1-8b": ("Llama-3.1-8B shape", LLAMA_31_8B), "llama-2-7b": ("Llama-2-7B shape", LLAMA_2_7B),
          "llama-3.2-1b": ("Llama-3.2-1B shape", LLAMA_32_1B)}


def peaks():
    """Measured peaks if the driver wrote them, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src, sustained = 6650.0, 1590.0, "fallback", None
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            hbm = float(d.get("hbm_gbs", hbm))
            tf = float(d.get("bf16_tflops", tf))
            sustained = float(d["bf16_tflops_sustained"]) if d.get("bf16_tflops_sustained") else None
            src = "measured"
        except (ValueError, OSError):
            pass
    return hbm, tf, src, sustained


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(float(s[0])) for s in self.samples if s[0].replace(".", "").isdigit())
        mx = [int(float(s[1])) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[3:7]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def matmul_params(cfg, layers):
    E, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = E * (q + 2 * kv) + q * E + 3 * E * F
    return layers * per_layer, V * E


def prefill_flops(cfg, layers, T):
    body, head = matmul_params(cfg, layers)
    attn = layers * 2 * 2 * cfg["num_attention_heads"] * cfg["head_dim"] * (T * (T + 1) // 2)
    return 2 * T * body + 2 * head + attn          # the head runs on the last row only


def decode_bytes(cfg, layers, batch, context, elem_bytes=2):
    body, head = matmul_params(cfg, layers)
    kv_row = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * layers
    return (2 * (body + head) + batch * context * kv_row) * elem_bytes // 2


def gevonex_config(width: int, layers: int, vocab: int) -> dict:
    """A Gevonex of `layers` layers (Mamba-2, latent attention, minGRU, Mamba-2, ...) whose sizes follow the width
    the way released models of these mixers do: heads of 64, state 128, an inner width of 2 x width for Mamba-2;
    heads of 128 and a latent of 128 for the attention; a feed-forward of 4 x width."""
    kinds = ["mamba2", "latent_attention", "mingru", "mamba2"]
    mixers = {"mamba2": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4},
              "latent_attention": {"heads": width // 128, "dim": 128, "vdim": 128, "kv_rank": 128, "scale": 128 ** -0.5},
              "mingru": {"width": width}}
    return {"architecture": "Gevonex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
            "loop": {"start": 0, "stop": layers, "times": 1},
            "layers": [{"type": kinds[i % 4], "mixer": mixers[kinds[i % 4]], "mlp": {"kind": "dense", "ff": 4 * width}}
                       for i in range(layers)]}


def mogevik_config(width: int, layers: int, vocab: int) -> dict:
    """A Mogevik of `layers` layers (two recurrent layers, then one of attention, ...) whose sizes follow the width:
    a recurrence as wide as the model in blocks of 256 channels with four taps; query heads of 128 in groups of four
    over a window of 1,024; fourteen experts of width / 2 and two identity experts in four groups of which three are
    kept, four per token, and a shared expert of 2/3 width: the matrix elements a token uses are those of a dense
    feed-forward of 4 x width."""
    heads = max(1, width // 128)
    kinds = ["rglru", "rglru", "attention"]
    mixers = {"rglru": {"width": width, "blocks": max(1, width // 256), "conv": 4},
              "attention": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                            "mask": {"size": 1024}}}
    mlp = {"kind": "moe", "expert": {"ff": width // 2}, "shared": {"ff": (2 * width // 3 + 63) // 64 * 64},
           "router": {"experts": 14, "identity": 2, "top": 4, "groups": {"count": 4, "keep": 3}}}
    return {"architecture": "Mogevik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": float(width) ** 0.5}, "loop": {"start": 0, "stop": layers, "times": 1},
            "layers": [{"type": kinds[i % 3], "mixer": mixers[kinds[i % 3]], "mlp": mlp} for i in range(layers)]}


def tubusun_config(width: int, layers: int, vocab: int) -> dict:
    """A Tubusun of `layers` layers whose sizes follow the width: query heads of 128 in groups of four over a window of
    1,024 with half of each head rotated, beside linear-attention heads of 128 x 128 whose decays spread from 0.9 to
    0.999; a dense feed-forward of 4 x width in the odd layers and sixteen bounded experts of width / 2 in four groups
    of which three are kept, four per token, in the even ones."""
    heads = max(1, width // 128)
    left = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 0.09,
            "mask": {"size": 1024}, "rot": {"dims": 64, "base": 10000.0}}
    right = {"heads": heads, "dim": 128, "vdim": 128,
             "decay": [1.0 - 0.1 * (0.01 ** (h / max(1, heads - 1))) for h in range(heads)]}
    mixer = {"left": left, "right": right, "left_scale": 0.6, "right_scale": 0.5}
    moe = {"kind": "moe", "expert": {"ff": width // 2, "limit": 7.0},
           "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 3}}}
    dense = {"kind": "dense", "ff": 4 * width}
    return {"architecture": "Tubusun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "logit_softcap": 30.0,
            "layers": [{"type": "parallel", "mixer": mixer, "mlp": dense if i % 2 else moe} for i in range(layers)]}


def fizadra_config(width: int, layers: int, vocab: int) -> dict:
    """A Fizadra of `layers` layers (latent attention with a sink, attention with mixed scores, latent attention that
    reads the first layer's cache, latent attention of the second form, ...) whose sizes follow the width: heads of
    96 + 32 numbers over a latent of 96 with a turned part of 32 (cached vectors of 128, the widest the tensor-core
    attention kernels take), a query latent of width / 4; query heads of 128 in groups of four with half a head
    turned; a feed-forward of 4 x width; rows normed in four parts."""
    heads = max(1, width // 128)
    rot = {"base": 10000.0, "dims": 32}
    scaled = dict(rot, scaling={"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0})
    latent = {"heads": heads, "dim": 96, "rot_dim": 32, "vdim": 128, "kv_rank": 96, "q_rank": max(64, width // 4 // 64 * 64),
              "scale": 128 ** -0.5}
    kinds = ["latent_attention", "attention", "latent_attention", "latent_attention_2"]
    mixers = [dict(latent, rot=scaled), {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128,
                                         "scale": 128 ** -0.5, "rot": {"base": 500000.0, "dims": 64}},
              dict(latent, rot=scaled, kv_from=0), dict(latent, rot=rot)]
    out = []
    for i in range(layers):
        m = dict(mixers[i % 4])
        if "kv_from" in m:
            m["kv_from"] = i - 2
        out.append({"type": kinds[i % 4], "mixer": m, "mlp": {"kind": "dense", "ff": 4 * width}})
    return {"architecture": "Fizadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5, "groups": 4}, "layers": out}


def expert_share(cfg: dict, name: str, draws: int) -> float:
    """The share of an expert's matrix that a step of `draws` tokens reads (decode: distinct experts among the
    draws, chosen evenly) or, with draws = 0, the share of tokens that use it (prefill)."""
    parts = name.split(".")
    if len(parts) < 3 or parts[1] != "mlp" or not parts[2].startswith("e") or not parts[2][1:].isdigit():
        return 1.0
    mlp = cfg["layers"][int(parts[0][1:])]["mlp"]
    if "router" not in mlp:
        return 1.0
    router = mlp["router"]
    n = router["experts"] + (router.get("identity") or 0)
    if draws == 0:
        return router["top"] / n
    return 1.0 - (1.0 - 1.0 / n) ** (draws * router["top"])


def llama_like(width: int, layers: int, vocab: int) -> dict:
    """The closest existing model at equal size: the same width, depth and vocabulary, heads of 128 in groups of
    four, a gated feed-forward of 8/3 x width (the same three-matrix parameter count as 4 x width ungated + gate)."""
    heads = width // 128
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=layers, hidden_size=width,
                num_attention_heads=heads, num_key_value_heads=max(1, heads // 4), head_dim=128,
                intermediate_size=(8 * width // 3 + 255) // 256 * 256, vocab_size=vocab, rope_theta=500000.0,
                rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=8192)


def compare(args) -> int:
    import gc
    import torch
    from mdma_b200.engine import Engine, StepEntry
    from mdma_b200.sampling import SamplingParams
    hbm_gbs, bf16_tflops, peak_src, _ = peaks()
    torch.cuda.set_device(0)
    warmup = max(3, args.warmup)
    vocab, T, prompt = 32000, args.prefill_tokens, args.prompt_len
    gen = torch.Generator().manual_seed(0)
    ids = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()

    def measure(cfg, batch):
        eng = Engine(config=cfg, seed=0, dtype=args.dtype, max_batch=batch, max_context=max(T, prompt + 512))
        matrix_bytes = prefill_elements = 0          # bytes a decode step reads; matrix elements a prompt token uses
        for name, ts in eng.model.expected_tensors().items():
            if len(ts.shape) >= 2 and ts.kind == "matrix" and "embed" not in name:
                n = 1
                for d in ts.shape:
                    n *= d
                routed = cfg.get("architecture") in ("Mogevik", "Tubusun")
                matrix_bytes += 2 * n * (expert_share(cfg, name, batch) if routed else 1.0)
                prefill_elements += n * (expert_share(cfg, name, 0) if routed else 1.0)
        # what a decode step moves besides the matrices: every live sequence's fixed-size state is read and written,
        # and its cached rows (keys and values, or latents) are read
        state_per_seq = eng.cache.state_bytes / eng.cache.max_slots
        cache_per_token = sum(g.bytes for g in eng.cache.groups) / (eng.cache.n_pages * eng.page_size)
        times = []
        for i in range(warmup + 5):
            s = eng.acquire()
            p = ids(T)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step([StepEntry(s, p, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            eng.release(s)
            if i >= warmup:
                times.append(e0.elapsed_time(e1))
        ms_p = sorted(times)[len(times) // 2]
        slots = [eng.acquire() for _ in range(batch)]
        ps = [ids(prompt) for _ in range(batch)]
        logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, ps)])
        toks, _ = eng.sampler.sample(logits, SamplingParams.greedy(), list(range(batch)), [0] * batch)
        sess = eng.decode_session()
        sess.start(slots, toks)
        for _ in range(warmup):
            sess.run(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = max(8, args.steps // 2)
        e0.record()
        done = 0
        while done < steps:
            done += sess.run(min(sess.max_run, steps - done))
        e1.record()
        torch.cuda.synchronize()
        ms_d = e0.elapsed_time(e1) / steps
        launches = sess.launches_per_step
        decode_bytes = matrix_bytes + batch * (2 * state_per_seq + (prompt + warmup + steps / 2) * cache_per_token)
        eng.check_status()
        del sess, eng
        gc.collect()
        torch.cuda.empty_cache()
        # prefill: two operations per token and matrix element (attention and the scans are not counted, so the
        # share is a lower bound); decode: the matrices once, every sequence's state twice, its cached rows once
        return {"matrix_gb": round(matrix_bytes / 1e9, 3), "decode_gb_per_step": round(decode_bytes / 1e9, 3),
                "prefill_tokens_per_s": round(T * 1000.0 / ms_p, 1), "prefill_ms": round(ms_p, 3),
                "prefill_frac_of_bf16_peak": round(2 * T * prefill_elements / (ms_p * 1e-3) / (bf16_tflops * 1e12), 4),
                "decode_tokens_per_s": round(batch * 1000.0 / ms_d, 1), "decode_ms_per_step": round(ms_d, 4),
                "decode_frac_of_hbm_peak": round(decode_bytes / (ms_d * 1e-3) / 1e9 / hbm_gbs, 4),
                "launches_per_decode_step": launches}

    clock = ClockSampler()
    clock.start()
    rows = []
    for width in [int(w) for w in args.compare_widths.split(",")]:
        row = {"width": width, "layers": args.compare_layers, "vocab": vocab, "batch": args.batch}
        if args.compare == "fizadra":
            row["fizadra"] = measure(fizadra_config(width, args.compare_layers, vocab), args.batch)
        if args.compare == "tubusun":
            row["tubusun"] = measure(tubusun_config(width, args.compare_layers, vocab), args.batch)
        if args.compare in ("mogevik", "tubusun"):
            row["mogevik"] = measure(mogevik_config(width, args.compare_layers, vocab), args.batch)
        if args.compare != "tubusun":
            row["gevonex"] = measure(gevonex_config(width, args.compare_layers, vocab), args.batch)
        row["llama"] = measure(llama_like(width, args.compare_layers, vocab), args.batch)
        rows.append(row)
    beside = {"fizadra": "fizadra beside gevonex and llama", "tubusun": "tubusun beside mogevik and llama", "mogevik": "mogevik beside gevonex and llama",
              "gevonex": "gevonex beside llama"}[args.compare]
    print(json.dumps({"compare": beside + " at equal width, depth and vocabulary", "dtype": args.dtype,
                      "prefill_tokens": T, "decode_after_prompts_of": prompt, "peaks": peak_src,
                      "hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops,
                      "timing": "CUDA events; every step reads its matrices (0.15 GB and more at the default widths), more than the 126 MB of L2, so nothing is flushed",
                      "sizes": rows, "clocks": clock.stop()}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--prompt-len-range", type=int, nargs=2, default=None, metavar=("LO", "HI"),
                    help="prompt lengths drawn uniformly from [LO, HI] instead of equal prompts (seeded)")
    ap.add_argument("--shape", default="llama-3.1-8b", choices=sorted(SHAPES), help="layer sizes (default: the headline shape)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in config)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill measurements")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end measurement (profiling runs)")
    ap.add_argument("--prefill-only", action="store_true", help="run only the 2,048-token prefill (profiling runs)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the true 32-bit engine (CUDA-core kernels), for the record; the headline is bfloat16")
    ap.add_argument("--compare", default=None, choices=["gevonex", "mogevik", "tubusun", "fizadra"],
                    help="another program: the named architecture beside a Llama of equal size (see the header)")
    ap.add_argument("--compare-widths", default="1024,2048,4096")
    ap.add_argument("--compare-layers", type=int, default=4)
    args = ap.parse_args()

    if args.compare is not None and args.impl != "reference":
        return compare(args)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "AliOsm/mdma is a Rust crate (Cargo.toml, no setup.py/pyproject.toml); pip cannot "
                          "install it and no cargo/rustc is in the image"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built in this library")
        return 2
    warmup = max(3, args.warmup)

    import torch
    from mdma_b200 import ops
    from mdma_b200.engine import Engine, StepEntry
    from mdma_b200.engine.generate import Generator
    from mdma_b200.sampling import SamplingParams

    shape_name, shape_cfg = SHAPES[args.shape]
    FULL_LAYERS = shape_cfg["num_hidden_layers"]
    if args.layers is None:
        args.layers = FULL_LAYERS
    cfg = dict(shape_cfg, num_hidden_layers=args.layers)
    hbm_gbs, bf16_tflops, peak_src, sustained = peaks()
    torch.cuda.set_device(0)
    max_batch = args.batch
    eng = Engine(config=cfg, seed=0, dtype=args.dtype, max_batch=max_batch,
                 max_context=max(args.context, args.prefill_tokens))
    sampler = eng.sampler
    gen = torch.Generator().manual_seed(0)

    def prompts(n, length):
        if args.prompt_len_range is not None and length == args.prompt_len:
            lo, hi = args.prompt_len_range
            lens = torch.randint(lo, hi + 1, (n,), generator=gen).tolist()
        else:
            lens = [length] * n
        return [torch.randint(0, cfg["vocab_size"], (m,), generator=gen).tolist() for m in lens]

    def time_decode(batch, steps):
        """Device time of `steps` decode steps of `batch` sequences after prompt_len-token prompts."""
        slots = [eng.acquire() for _ in range(batch)]
        ps = prompts(batch, args.prompt_len)
        logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, ps)])
        toks, _ = sampler.sample(logits, SamplingParams.greedy(), list(range(batch)), [0] * batch)
        sess = eng.decode_session()
        sess.start(slots, toks)
        for _ in range(warmup):
            sess.run(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        done = 0
        while done < steps:             # exactly `steps` steps, replayed in runs as generation does
            done += sess.run(min(sess.max_run, steps - done))
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        per_graph = sess.launches_per_step
        mean_prompt = sum(len(p) for p in ps) / batch
        for s in slots:
            eng.release(s)
        return ms / steps, per_graph * steps, mean_prompt

    def time_prefill(T=args.prefill_tokens):
        times = []
        for i in range(warmup + 5):
            s = eng.acquire()
            p = prompts(1, T)[0]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step([StepEntry(s, p, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            eng.release(s)
            if i >= warmup:
                times.append(e0.elapsed_time(e1))
        ms_p = sorted(times)[len(times) // 2]
        fl = prefill_flops(cfg, args.layers, T)
        out = {"value": round(T * 1000.0 / ms_p, 1), "tokens": T, "ms": round(ms_p, 3),
               "frac": round(fl / (ms_p * 1e-3) / (bf16_tflops * 1e12), 4), "frac_of": f"{peak_src} burst peak"}
        if sustained:          # the same against what the library GEMM holds over seconds under the power cap
            out["frac_sustained"] = round(fl / (ms_p * 1e-3) / (sustained * 1e12), 4)
        return out

    if args.prefill_only:
        print(json.dumps({"prefill": time_prefill(), "config": {"layers": args.layers, "layers_full": FULL_LAYERS}}))
        return 0

    clock = ClockSampler()          # samples until every measurement of this run is done
    clock.start()
    ms_step, launches, mean_prompt = time_decode(args.batch, args.steps)
    value = args.batch * 1000.0 / ms_step
    ctx_end = int(mean_prompt) + warmup + args.steps
    avg_ctx = mean_prompt + warmup + args.steps / 2
    bytes_step = decode_bytes(cfg, args.layers, args.batch, avg_ctx, 2 if args.dtype == "bfloat16" else 4)
    achieved = bytes_step / (ms_step * 1e-3) / 1e9

    # end to end: host token lists in, host token lists out, through Generator.generate
    e2e = None
    if not args.no_e2e:
        stamps = []
        g = Generator(eng)
        n_e2e = args.steps + warmup + 1
        g.generate(prompts(args.batch, args.prompt_len), max_tokens=2 * g.run_ahead + 2)        # warm the path
        up0, down0 = eng.h2d_bytes, eng.d2h_bytes + sampler.d2h_bytes
        t_start = time.perf_counter()
        g.generate(prompts(args.batch, args.prompt_len), max_tokens=n_e2e,
                   on_token=lambda r, t: stamps.append(time.perf_counter()) if r == args.batch - 1 else None)
        # Host token lists go in, host token lists come out.  The tokens of `run_ahead` replayed steps reach
        # the host in one copy, so the rate is taken over the whole call but for the prompt step: from the
        # moment the first tokens are on the host to the moment the last ones are.
        e2e_value = args.batch * (len(stamps) - 1) / (stamps[-1] - stamps[0])
        n_steps = len(stamps) - 1
        e2e = {"value": round(e2e_value, 2), "unit": "tokens/s",
               # counted from the tensors copied during the call (prompt ids and step metadata up from pinned
               # memory; tokens, flags and the kernels' status word down), divided by its decode steps
               "h2d_bytes_per_step": round((eng.h2d_bytes - up0) / n_steps, 1),
               "d2h_bytes_per_step": round((eng.d2h_bytes + sampler.d2h_bytes - down0) / n_steps, 1),
               "steps": n_steps, "run_ahead": g.run_ahead,
               "with_prompt_step": round(args.batch * len(stamps) / (stamps[-1] - t_start), 2)}

    out = {
        "metric": f"decode tokens/s ({shape_name}, batch {args.batch}, after " + (
            f"{args.prompt_len}-token prompts)" if args.prompt_len_range is None else
            f"prompts of {args.prompt_len_range[0]}-{args.prompt_len_range[1]} tokens)"),
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic (uniform random token ids, random N(0,0.02) weights)",
        "impl": "ours",
        "config": {"model": shape_name, "layers": args.layers, "layers_full": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": args.context, "prompt_len": args.prompt_len,
                   "context_at_end": ctx_end, "parallelism": "single GPU", "page_size": eng.page_size,
                   "cuda_graph": True,
                   "l2": f"inputs ({bytes_step / 1e9:.1f} GB of weights and cache per step) larger than L2, no flush",
                   "peaks": peak_src},
        "e2e": e2e, "gpu_launches": launches, "clocks": None,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
    }

    if not args.no_points:
        # the other batch sizes, each on an engine built for that many sequences (as a deployment for that
        # batch size would be: the kernels plan some choices for the most sequences an engine holds)
        out["prefill"] = time_prefill()
        points = {}
        for b in (1, 64):
            if b != eng.max_slots:
                eng.check_status()
                sampler = eng = None
                import gc
                gc.collect()
                torch.cuda.empty_cache()
                eng = Engine(config=cfg, seed=0, dtype=args.dtype, max_batch=b, max_context=max(args.context, args.prefill_tokens))
                sampler = eng.sampler
            ms_b, _, _ = time_decode(b, max(8, args.steps // 2))
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 2)
        out["points"] = points
    out["clocks"] = clock.stop()
    eng.check_status()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
