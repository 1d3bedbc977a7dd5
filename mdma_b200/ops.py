"""Python faces of the CUDA kernels.

Each function checks what the kernel cannot check (devices, dtypes,
contiguity, sizes), passes raw pointers and the current stream to the C entry
point and raises `KernelError` with the library's message on failure.  There
is no fallback: without the compiled library, or off the GPU, these raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
GEMM_STORE, GEMM_ACCUMULATE, GEMM_SWIGLU = 0, 1, 2


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream of the current device, as the launches take it (the stream object
    of torch costs several microseconds to make, and a step makes hundreds of launches)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch._C._cuda_getDevice()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


LAUNCHES = 0      # kernel launches made through this module (a claim bench.py reports)


def _call(libname: str, fn: str, *args, launches: int = 1):
    global LAUNCHES
    LAUNCHES += launches
    lib = _build._loaded.get(libname) or _build.load(libname)
    rc = getattr(lib, fn)(*args)
    if rc != 0:
        raise KernelError(lib.mdma_last_error().decode(errors="replace"))


_i = ctypes.c_int
_f = ctypes.c_float


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale, as float rows."""
    _need_cuda(table, ids, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous()
    n = ids.numel()
    assert out.shape[0] >= n and out.shape[1] == table.shape[1] and out.is_contiguous()
    _call("core", "mdma_embed_rows_scaled", _ptr(table), _i(dtype_code(table.dtype)), _ptr(ids), _ptr(out),
          _i(n), _i(table.shape[1]), _i(table.shape[0]), _f(scale), _stream())


def fill_normal(out: torch.Tensor, key: int, table: torch.Tensor, std: float) -> None:
    """out.flat[i] = std * (a normal quantile picked by a hash of (key, i)); the host side of the same
    arithmetic is `weights.random_init.normal_values`.  `table`: 65,537 float quantiles on the device."""
    _need_cuda(out, table)
    assert out.is_contiguous() and table.dtype == torch.float32 and table.numel() == 65537
    _call("core", "mdma_fill_normal", _ptr(out), _i(dtype_code(out.dtype)), ctypes.c_long(out.numel()),
          ctypes.c_ulonglong(key & ((1 << 64) - 1)), _ptr(table), _f(std), _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
            partial: Optional[torch.Tensor] = None, splits: int = 0, split_stride: int = 0) -> None:
    """out[i] = rmsnorm(x[rows[i]] or x[i]) * w; x is the float residual stream.  With
    `partial` [splits, rows, width] the rows of x are first completed: x += sum of the partials."""
    _need_cuda(x, w, out, rows)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    width = x.shape[-1]
    assert w.numel() == width and out.shape[-1] == width
    n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert out.shape[0] >= n
    if rows is not None:
        assert rows.dtype == torch.int32
    _call("core", "mdma_rmsnorm", _ptr(x), _ptr(w), _i(dtype_code(w.dtype)), _ptr(rows), _ptr(out),
          _i(dtype_code(out.dtype)), _i(n), _i(width), _f(eps), _ptr(partial), _i(splits if partial is not None else 0),
          ctypes.c_long(split_stride), _stream())


ACT_SILU, ACT_GELU_TANH, ACT_GELU, ACT_SWISH_LIMIT, ACT_RELU_SQUARED = 0, 1, 2, 3, 4
# "gelu" is the exact one, 0.5 z (1 + erf(z / sqrt 2)).  "swish_limit" belongs to gated products only: with the gate's
# product g cut off above `limit` and the other product u kept within +-limit, g sigmoid(alpha g) (u + 1).
ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH, "gelu": ACT_GELU, "swish_limit": ACT_SWISH_LIMIT,
               "relu_squared": ACT_RELU_SQUARED}


def ending_args(n_features: int, bias: Optional[torch.Tensor], bias2: Optional[torch.Tensor], act: int,
                act_limit: float = 0.0, act_alpha: float = 1.0):
    """The arguments by which the product kernels take their bias vectors, the gate's activation and its constants."""
    for b in (bias, bias2):
        if b is not None:
            assert b.is_cuda and b.is_contiguous() and b.shape == (n_features,)
            assert bias.dtype == b.dtype and b.dtype in (torch.float32, torch.bfloat16)
    assert bias2 is None or bias is not None
    return (_ptr(bias), _ptr(bias2), _i(dtype_code(bias.dtype) if bias is not None else F32), _i(act), _f(act_limit),
            _f(act_alpha))


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = GEMM_STORE,
              w2: Optional[torch.Tensor] = None, m: Optional[int] = None, bias: Optional[torch.Tensor] = None,
              bias2: Optional[torch.Tensor] = None, act: int = ACT_SILU, act_limit: float = 0.0,
              act_alpha: float = 1.0) -> None:
    """out[:m] (=, +=) a[:m] @ w.T (+ bias) on the CUDA cores; the gated mode takes gate=w, up=w2 and
    gives act(gate) * up."""
    _need_cuda(a, w, out, w2)
    assert a.dim() == 2 and w.dim() == 2 and out.dim() == 2
    assert a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
    M = a.shape[0] if m is None else m
    N, K = w.shape
    assert a.shape[1] == K and out.shape[1] == N and out.shape[0] >= M and a.shape[0] >= M
    if w2 is not None:
        assert w2.shape == w.shape and w2.dtype == w.dtype and w2.is_contiguous()
    _call("core", "mdma_gemm_simt", _i(mode), _ptr(a), _i(dtype_code(a.dtype)), _i(a.stride(0)),
          _ptr(w), _ptr(w2), _i(dtype_code(w.dtype)), _ptr(out), _i(dtype_code(out.dtype)),
          _i(out.stride(0)), _i(M), _i(N), _i(K), *ending_args(N, bias, bias2, act, act_limit, act_alpha), _stream())


def rope_cache_write(qkv: torch.Tensor, n_tokens: int, tok_seq, tok_pos, seq_slot, inv_freq,
                     k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                     page_table: Optional[torch.Tensor], max_pages: int, page_size: int,
                     n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                     interleaved: bool, write_kv: bool, partial: Optional[torch.Tensor] = None,
                     splits: int = 0, split_stride: int = 0) -> None:
    """Rotate q (in place) and k, write k and v to the cache.  With `partial`
    [splits, tokens, row width] floats the projection row is their sum instead of qkv's content."""
    _need_cuda(qkv, tok_seq, tok_pos, seq_slot, inv_freq, k_cache, v_cache, page_table)
    assert qkv.stride(1) == 1 and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2
    if write_kv:
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
        assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    _call("core", "mdma_rope_cache_write", _ptr(qkv), _i(dtype_code(qkv.dtype)), _i(qkv.stride(0)),
          _ptr(partial), _i(splits if partial is not None else 0), ctypes.c_long(split_stride),
          _i(qkv.shape[1]), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot), _ptr(inv_freq), _ptr(k_cache), _ptr(v_cache),
          _ptr(page_table), _i(max_pages), _i(page_size),
          _i(n_tokens), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(rotary_dim), _i(int(interleaved)),
          _i(int(write_kv)), _stream())


def attention_simple(q: torch.Tensor, n_tokens: int, k_cache, v_cache, tok_seq, tok_pos, seq_slot,
                     page_table: torch.Tensor, max_pages: int, page_size: int,
                     out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                     window: int, scale: float) -> None:
    """q: rows of the fused projection (first n_heads*head_dim columns are the queries)."""
    _need_cuda(q, k_cache, v_cache, tok_seq, tok_pos, seq_slot, out, page_table)
    assert q.stride(1) == 1 and out.is_contiguous() and out.dtype == q.dtype == k_cache.dtype
    assert out.shape[1] == n_heads * head_dim and out.shape[0] >= n_tokens
    _call("core", "mdma_attention_simple", _ptr(q), _i(dtype_code(q.dtype)), _i(q.stride(0)),
          _ptr(k_cache), _ptr(v_cache), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot),
          _ptr(page_table), _i(max_pages), _i(page_size), _ptr(out),
          _i(n_tokens), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(window),
          _f(scale), _stream())


_argmax_scratch: dict = {}


def argmax_scratch_words(n_rows: int, vocab: int) -> int:
    return 3 * max(n_rows, 1) * (-(-vocab // 4096))


def argmax(logits: torch.Tensor, tokens: torch.Tensor, flags: Optional[torch.Tensor] = None,
           n_rows: Optional[int] = None, scratch: Optional[torch.Tensor] = None) -> None:
    """tokens[r] = index of the largest logit of row r (the lowest index among equals);
    flags[r] = 1 if the row holds a value that is not finite.  `scratch`: floats for the first
    stage's partial results (`argmax_scratch_words`); without it a buffer of this module is used."""
    _need_cuda(logits, tokens, flags, scratch)
    assert logits.dtype == torch.float32 and logits.is_contiguous() and tokens.dtype == torch.int32
    n = logits.shape[0] if n_rows is None else n_rows
    need = argmax_scratch_words(n, logits.shape[1])
    if scratch is not None:
        if scratch.numel() < need:
            raise KernelError(f"argmax needs {need} words of scratch, {scratch.numel()} given")
    else:
        scratch = _argmax_scratch.get(logits.device.index)
    if scratch is None or scratch.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("argmax scratch cannot grow during graph capture")
        scratch = _argmax_scratch[logits.device.index] = torch.empty(max(need, 1 << 16), dtype=torch.float32,
                                                                     device=logits.device)
    _call("core", "mdma_argmax", _ptr(logits), _i(n), _i(logits.shape[1]), _ptr(tokens), _ptr(flags),
          _ptr(scratch), ctypes.c_long(scratch.numel()), _stream(), launches=2)


def sample_scratch_words(n_rows: int, vocab: int) -> int:
    """Floats of scratch `sample` needs: exponentials, candidate probabilities and candidate ids of every row."""
    return 3 * n_rows * vocab


def sample(logits: torch.Tensor, uniforms: Optional[torch.Tensor], tokens: torch.Tensor, probs_scratch: torch.Tensor,
           temperature: float, top_p: float, min_p: float, penalty: float, penalty_window: int,
           history: Optional[torch.Tensor] = None, history_len: Optional[torch.Tensor] = None,
           flags: Optional[torch.Tensor] = None, n_rows: Optional[int] = None, impl: int = 0,
           requests: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None, seed: int = 0,
           advance: bool = False, dev_params: Optional[torch.Tensor] = None) -> None:
    """One token per row of `logits`.  The uniform number of a row is `uniforms[r]`, or, without
    `uniforms`, made on the device from (seed, requests[r], steps[r]).  `history` [rows, cap] is a ring of
    recent token ids per row and `history_len` the count of tokens ever added to it.  `advance`: the
    kernel appends the selected token to the ring and adds one to `steps`.
    `impl`: 0 picks (a cluster of eight blocks per row when the row fits), 1 one block per row, 2 the cluster.
    `dev_params` (eight 32-bit words on the device: temperature, top_p, min_p, penalty as floats, the
    window, an unused word, the seed's low and high halves) replaces the options given by value, so that
    a captured launch serves whatever the host writes there before a replay."""
    _need_cuda(logits, uniforms, tokens, probs_scratch, history, history_len, flags, requests, steps, dev_params)
    assert dev_params is None or (dev_params.dtype == torch.int32 and dev_params.numel() >= 8)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert tokens.dtype == torch.int32 and (uniforms is None or uniforms.dtype == torch.float32)
    assert uniforms is not None or (requests is not None and steps is not None)
    assert requests is None or (requests.dtype == torch.int32 and steps.dtype == torch.int32)
    n = logits.shape[0] if n_rows is None else n_rows
    assert probs_scratch.dtype == torch.float32 and probs_scratch.numel() >= sample_scratch_words(n, logits.shape[1])
    hstride = 0
    if history is not None:
        assert history.dtype == torch.int32 and history_len.dtype == torch.int32 and history.is_contiguous()
        hstride = history.shape[1]
    _call("core", "mdma_sample", _ptr(logits), _i(n), _i(logits.shape[1]), _ptr(history),
          _ptr(history_len), _i(hstride), _ptr(uniforms), _ptr(requests), _ptr(steps),
          ctypes.c_ulonglong(seed & ((1 << 64) - 1)), _i(int(advance)), _f(temperature), _f(top_p), _f(min_p),
          _f(penalty), _i(penalty_window), _ptr(probs_scratch), ctypes.c_long(probs_scratch.numel()), _ptr(tokens),
          _ptr(flags), _i(impl), _ptr(dev_params), _stream())


def advance_decode(tokens: torch.Tensor, ids: torch.Tensor, tok_pos: torch.Tensor, seq_pos0: torch.Tensor,
                   n: int, ring: Optional[torch.Tensor] = None, counter: Optional[torch.Tensor] = None) -> None:
    """ids <- tokens, positions += 1: what a decode step leaves for the next one.  With `ring`
    [rows, words] the first `words` integers at `tokens` (tokens, flags and what lies behind them in
    the same buffer) are also kept in row counter % rows, and the counter moves on."""
    _need_cuda(tokens, ids, tok_pos, seq_pos0, ring, counter)
    words, rows = (ring.shape[1], ring.shape[0]) if ring is not None else (0, 0)
    assert ring is None or (ring.dtype == torch.int32 and ring.is_contiguous() and counter.dtype == torch.int32)
    _call("core", "mdma_advance_decode", _ptr(tokens), _ptr(ids), _ptr(tok_pos), _ptr(seq_pos0), _i(n),
          _i(words), _ptr(ring), _i(rows), _ptr(counter), _stream())


# ---- layers with per-sequence state, and the small steps around them (csrc/sequence_mix.cu) ---------------
GEMM_STORE_ACT = 3        # out = act(a W^T + b): CUDA-core product only


def _state(state: torch.Tensor):
    """Pointer and row stride of a per-sequence state [slots, n] (a view of wider rows is fine)."""
    assert state.is_cuda and state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
    return _ptr(state), ctypes.c_long(state.stride(0))


def _same_dtype(*vectors):
    dt = vectors[0].dtype
    for v in vectors:
        assert v.is_cuda and v.is_contiguous() and v.dtype == dt, "the small vectors of a part are kept in one dtype"
    return dtype_code(dt)


def dyt_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> None:
    """out[i] = tanh(alpha * x[rows[i]] or x[i]) * w + b; x is the float residual stream."""
    _need_cuda(x, w, b, alpha, out, rows)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    width = x.shape[-1]
    assert w.numel() == width and b.numel() == width and alpha.numel() == 1 and out.shape[-1] == width
    n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert out.shape[0] >= n and (rows is None or rows.dtype == torch.int32)
    _call("core", "mdma_dyt_norm", _ptr(x), _ptr(w), _ptr(b), _ptr(alpha), _i(_same_dtype(w, b, alpha)), _ptr(rows),
          _ptr(out), _i(dtype_code(out.dtype)), _i(n), _i(width), _stream())


def dyt_shift(x, w, b, alpha, mu, tok_seq, seq_start, seq_slot, state, h, hs, n_rows: int) -> None:
    """h = dyt(x) and hs = h + (h' - h) * mu in one pass (h': the row before, or the kept row of `state`)."""
    _need_cuda(x, w, b, alpha, mu, tok_seq, seq_start, seq_slot, state, h, hs)
    width = x.shape[-1]
    assert x.dtype == torch.float32 and x.is_contiguous() and h.is_contiguous() and hs.is_contiguous()
    assert h.dtype == hs.dtype and h.shape[1] == hs.shape[1] == width and mu.numel() == width
    sp, ss = _state(state)
    _call("core", "mdma_dyt_shift", _ptr(x), _ptr(w), _ptr(b), _ptr(alpha), _ptr(mu), _i(_same_dtype(w, b, alpha, mu)),
          _ptr(tok_seq), _ptr(seq_start), _ptr(seq_slot), sp, ss, _ptr(h), _ptr(hs), _i(dtype_code(h.dtype)),
          _i(n_rows), _i(width), _stream())


def token_shift(h, mu, tok_seq, seq_start, seq_slot, state, hs, n_rows: int) -> None:
    """hs[t] = h[t] + (h' - h[t]) * mu, h' = h[t-1] within the step, else the sequence's kept row."""
    _need_cuda(h, mu, tok_seq, seq_start, seq_slot, state, hs)
    width = h.shape[1]
    assert h.is_contiguous() and hs.is_contiguous() and hs.dtype == h.dtype and hs.shape[1] == width and mu.numel() == width
    sp, ss = _state(state)
    _call("core", "mdma_token_shift", _ptr(h), _i(dtype_code(h.dtype)), _ptr(mu), _i(dtype_code(mu.dtype)),
          _ptr(tok_seq), _ptr(seq_start), _ptr(seq_slot), sp, ss, _ptr(hs), _i(n_rows), _i(width), _stream())


def keep_last_rows(rows, seq_start, seq_slot, state, n_seqs: int) -> None:
    """state[slot] = the last row each sequence brought."""
    _need_cuda(rows, seq_start, seq_slot, state)
    assert rows.is_contiguous()
    sp, ss = _state(state)
    _call("core", "mdma_keep_last_rows", _ptr(rows), _i(dtype_code(rows.dtype)), _ptr(seq_start), _ptr(seq_slot),
          sp, ss, _i(n_seqs), _i(rows.shape[1]), _stream())


def gated_add(x, g, y, n_rows: int, keep_rows=None, tok_seq=None, seq_start=None, seq_slot=None, state=None,
              partial=None, splits: int = 0, split_stride: int = 0) -> None:
    """x += sigmoid(g) * y (x, y float).  With `keep_rows` each sequence's last row of it goes to `state`.
    With `partial` [splits, rows, width] floats, y is their sum (a K-split product not yet added up)."""
    _need_cuda(x, g, y, keep_rows, tok_seq, seq_start, seq_slot, state)
    width = x.shape[1]
    assert x.dtype == torch.float32 and y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and g.is_contiguous()
    assert g.shape[1] == width and y.shape[1] == width
    sp, ss = (_ptr(None), ctypes.c_long(0))
    if keep_rows is not None:
        assert keep_rows.is_contiguous() and keep_rows.shape[1] == width
        sp, ss = _state(state)
    _call("core", "mdma_gated_add", _ptr(x), _ptr(g), _i(dtype_code(g.dtype)), _ptr(y), _ptr(partial),
          _i(splits if partial is not None else 0), ctypes.c_long(split_stride), _i(n_rows), _i(width),
          _ptr(keep_rows), _i(dtype_code(keep_rows.dtype) if keep_rows is not None else F32), _ptr(tok_seq),
          _ptr(seq_start), _ptr(seq_slot), sp, ss, _stream())


def activation(v: torch.Tensor, n_rows: int, act: int) -> None:
    """v[:n_rows] = act(v[:n_rows]) in place."""
    _need_cuda(v)
    assert v.is_contiguous()
    _call("core", "mdma_activation", _ptr(v), _i(dtype_code(v.dtype)), ctypes.c_long(n_rows * v.shape[1]), _i(act), _stream())


def softcap(logits: torch.Tensor, n_rows: int, cap: float) -> None:
    """logits[:n_rows] = cap * tanh(logits / cap) in place (float)."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _call("core", "mdma_softcap", _ptr(logits), ctypes.c_long(n_rows * logits.shape[1]), _f(cap), _stream())


def pack_pair(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    """out[t] = [a[t] | b[t]] in out's dtype; a and b are float rows of one width."""
    _need_cuda(a, b, out)
    width = a.shape[1]
    assert a.dtype == b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous() and out.is_contiguous()
    assert b.shape[1] == width and out.shape[1] == 2 * width
    _call("core", "mdma_pack_pair", _ptr(a), _ptr(b), _ptr(out), _i(dtype_code(out.dtype)), _i(n_rows), _i(width), _stream())


def mingru_scan(p, bz, bu, seq_start, seq_slot, state, out, n_seqs: int, width: int, chunked: bool = False) -> None:
    """p [T, 3*width] float = the three projections (z | u | g); runs S = (1-z) S + z cand over each
    sequence's rows and writes S * silu(g).  `chunked`: the kernel for steps of many rows per sequence, which
    walks 32 runs of a sequence side by side (equal to the row-by-row kernel up to rounding)."""
    _need_cuda(p, bz, bu, seq_start, seq_slot, state, out)
    assert p.dtype == torch.float32 and p.stride(1) == 1 and p.shape[1] == 3 * width and out.is_contiguous() and out.shape[1] == width
    sp, ss = _state(state)
    _call("core", "mdma_mingru_scan", _ptr(p), _i(p.stride(0)), _ptr(bz), _ptr(bu), _i(_same_dtype(bz, bu)),
          _ptr(seq_start), _ptr(seq_slot), sp, ss, _ptr(out), _i(dtype_code(out.dtype)), _i(n_seqs), _i(width), _i(int(chunked)), _stream())


def causal_conv_silu(proj, in_col: int, w, b, taps: int, channels: int, tok_seq, seq_start, seq_slot, state, out,
                     n_rows: int, n_seqs: int, silu: bool = True) -> None:
    """out[t, c] = silu(bias + sum_j w[c, j] * input(t - taps + 1 + j, c)) over columns in_col.. of the float
    projection rows; inputs before the step come from `state` ([taps-1, channels] per slot), which is then
    brought up to date.  `silu=False`: the sum itself, no activation."""
    _need_cuda(proj, w, b, tok_seq, seq_start, seq_slot, state, out)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and out.dtype == torch.float32 and out.is_contiguous()
    assert w.is_contiguous() and tuple(w.shape) == (channels, taps) and b.numel() == channels and out.shape[1] == channels
    sp, ss = _state(state)
    _call("core", "mdma_causal_conv", _ptr(proj), _i(proj.stride(0)), _i(in_col), _ptr(w), _i(dtype_code(w.dtype)),
          _ptr(b), _i(dtype_code(b.dtype)), _i(taps), _i(channels), _ptr(tok_seq), _ptr(seq_start), _ptr(seq_slot),
          sp, ss, _ptr(out), _i(n_rows), _i(n_seqs), _i(int(silu)), _stream(), launches=2 if taps > 1 else 1)


def mamba2_scan(conv, proj, dt_col: int, dt_bias, a_log, d, seq_start, seq_slot, state, y, n_seqs: int, heads: int,
                vdim: int, n_state: int, groups: int, chunk_rows: int = 0, max_chunks: int = 1, scratch=None,
                wide_state: bool = False) -> None:
    """The selective scan over each sequence's rows; `conv` rows are [x | B | C] after the convolution,
    `proj` holds the raw step sizes at columns dt_col + head; state [slots, heads * n_state * vdim] float.
    `chunk_rows` > 0: sequences are walked as runs of that many rows side by side (`max_chunks`: the most runs
    of a sequence; `scratch`: n_seqs * max_chunks * (state size + heads) floats); equal up to rounding.
    `wide_state`: the state rows hold doubles (two floats an element), and step sizes, decays and the sums over
    the state are computed in double: the exact engine's walk."""
    _need_cuda(scratch)
    assert chunk_rows == 0 or (scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous())
    _need_cuda(conv, proj, dt_bias, a_log, d, seq_start, seq_slot, state, y)
    assert conv.dtype == proj.dtype == y.dtype == torch.float32 and conv.stride(1) == 1 and proj.stride(1) == 1
    assert y.is_contiguous() and y.shape[1] == heads * vdim and conv.shape[1] == heads * vdim + 2 * groups * n_state
    sp, ss = _state(state)
    _call("core", "mdma_mamba2_scan", _ptr(conv), _i(conv.stride(0)), _ptr(proj), _i(proj.stride(0)), _i(dt_col),
          _ptr(dt_bias), _ptr(a_log), _ptr(d), _i(_same_dtype(dt_bias, a_log, d)), _ptr(seq_start), _ptr(seq_slot),
          sp, ss, _ptr(y), _i(n_seqs), _i(heads), _i(vdim), _i(n_state), _i(groups), _i(chunk_rows), _i(max_chunks),
          _ptr(scratch), ctypes.c_long(scratch.numel() if scratch is not None else 0), _i(int(wide_state)), _stream(),
          launches=3 if chunk_rows > 0 else 1)


def gated_group_rmsnorm(y, z, w, out, n_rows: int, groups: int, eps: float) -> None:
    """out = rms_unit_per_part(y * silu(z)) * w; y and z float rows (z may be a view of wider rows)."""
    _need_cuda(y, z, w, out)
    width = y.shape[1]
    assert y.dtype == z.dtype == torch.float32 and y.stride(1) == 1 and z.stride(1) == 1 and z.shape[1] == width
    assert out.is_contiguous() and out.shape[1] == width and w.numel() == width and w.is_contiguous()
    _call("core", "mdma_gated_group_rmsnorm", _ptr(y), _i(y.stride(0)), _ptr(z), _i(z.stride(0)), _ptr(w),
          _i(dtype_code(w.dtype)), _ptr(out), _i(dtype_code(out.dtype)), _i(n_rows), _i(width), _i(groups), _f(eps), _stream())


def gemm_simt_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, m: int) -> None:
    """out[:m, z*N:(z+1)*N] = a[:m, z*K:(z+1)*K] @ w[z].T for every z: w [batch, N, K]; the pieces of a
    row (one per head) lie side by side in a and in out."""
    _need_cuda(a, w, out)
    batch, N, K = w.shape
    assert w.is_contiguous() and a.stride(1) == 1 and out.stride(1) == 1
    assert a.shape[1] >= batch * K and out.shape[1] >= batch * N and a.shape[0] >= m and out.shape[0] >= m
    _call("core", "mdma_gemm_simt_batched", _ptr(a), _i(dtype_code(a.dtype)), _i(a.stride(0)), ctypes.c_long(K),
          _ptr(w), _i(dtype_code(w.dtype)), ctypes.c_long(N * K), _ptr(out), _i(dtype_code(out.dtype)),
          _i(out.stride(0)), ctypes.c_long(N), _i(batch), _i(m), _i(N), _i(K), _stream())


# ---- attention over a cached latent (csrc/latent_attention.cu) ------------------------------------------------
def latent_norm_store(proj, col0: int, w, eps: float, rank: int, tok_seq, tok_pos, seq_slot, page_table,
                      max_pages: int, page_size: int, cache, n_tokens: int) -> None:
    """cache[row of token] = rms_unit(proj[t, col0:col0+rank]) * w."""
    _need_cuda(proj, w, tok_seq, tok_pos, seq_slot, page_table, cache)
    assert proj.stride(1) == 1 and cache.is_contiguous() and cache.dtype == proj.dtype and w.numel() == rank
    _call("core", "mdma_latent_norm_store", _ptr(proj), _i(dtype_code(proj.dtype)), _i(proj.stride(0)), _i(col0),
          _ptr(w), _i(dtype_code(w.dtype)), _f(eps), _i(rank), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot),
          _ptr(page_table), _i(max_pages), _i(page_size), _ptr(cache), _i(n_tokens), _stream())


def latent_attention(q, cache, sink, tok_seq, tok_pos, seq_slot, page_table, max_pages: int, page_size: int, out,
                     n_tokens: int, n_heads: int, rank: int, window: int, scale: float) -> None:
    """q [T, heads*rank]: queries already mapped into the latent; out [T, heads*rank]: the weighted sums of
    cached latents, softmax with one sink term per head in the denominator (`sink` None: none)."""
    _need_cuda(q, cache, sink, tok_seq, tok_pos, seq_slot, page_table, out)
    assert q.stride(1) == 1 and out.is_contiguous() and out.dtype == q.dtype == cache.dtype and cache.is_contiguous()
    assert out.shape[1] == n_heads * rank and (sink is None or (sink.numel() == n_heads and sink.is_contiguous()))
    _call("core", "mdma_latent_attention", _ptr(q), _i(dtype_code(q.dtype)), _i(q.stride(0)), _ptr(cache), _ptr(sink),
          _i(dtype_code(sink.dtype) if sink is not None else F32), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot), _ptr(page_table), _i(max_pages),
          _i(page_size), _ptr(out), _i(n_tokens), _i(n_heads), _i(rank), _i(window), _f(scale), _stream())


# ---- layer norm, loop re-entry by addition, row scale, the real-gated linear recurrence (csrc/rglru.cu) ---------
def layernorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None,
              n_rows: Optional[int] = None) -> None:
    """out[i] = (x[r] - mean) / sqrt(var + eps) * w, r = rows[i] or i; x is the float residual stream."""
    _need_cuda(x, w, out, rows)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    width = x.shape[-1]
    assert w.numel() == width and out.shape[-1] == width and w.is_contiguous()
    n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert out.shape[0] >= n and (rows is None or rows.dtype == torch.int32)
    _call("core", "mdma_layernorm", _ptr(x), _ptr(w), _i(dtype_code(w.dtype)), _ptr(rows), _ptr(out),
          _i(dtype_code(out.dtype)), _i(n), _i(width), _f(eps), _stream())


def loop_add(x: torch.Tensor, x0: Optional[torch.Tensor], step: torch.Tensor, n_rows: int) -> None:
    """x[t] = (x[t] + x0[t]) + step (x0 None: only the vector is added); x, x0 float rows."""
    _need_cuda(x, x0, step)
    width = x.shape[1]
    assert x.dtype == torch.float32 and x.is_contiguous() and step.numel() == width and step.is_contiguous()
    assert x0 is None or (x0.dtype == torch.float32 and x0.is_contiguous() and x0.shape[1] == width)
    _call("core", "mdma_loop_add", _ptr(x), _ptr(x0), _ptr(step), _i(dtype_code(step.dtype)), _i(n_rows), _i(width), _stream())


def scale_rows(v: torch.Tensor, s: torch.Tensor, n_rows: int) -> None:
    """v[t, :] *= s[t] in place; s float."""
    _need_cuda(v, s)
    assert v.is_contiguous() and s.dtype == torch.float32 and s.is_contiguous() and s.numel() >= n_rows
    _call("core", "mdma_scale_rows", _ptr(v), _i(dtype_code(v.dtype)), _ptr(s), _i(n_rows), _i(v.shape[1]), _stream())


def sigmoid_gate(v: torch.Tensor, g: torch.Tensor, n_rows: int) -> None:
    """v[t, :] *= sigmoid(g[t, :]) in place; g may be a view of wider rows."""
    _need_cuda(v, g)
    assert v.is_contiguous() and g.dtype == v.dtype and g.stride(1) == 1 and g.shape[1] >= v.shape[1]
    _call("core", "mdma_sigmoid_gate", _ptr(v), _ptr(g), _i(dtype_code(v.dtype)), _i(g.stride(0)), _i(n_rows), _i(v.shape[1]), _stream())


def rglru_scan(gates_r, gates_i, u, y, rb, ib, lam, decay: float, seq_start, seq_slot, state, out, n_seqs: int,
               width: int, runs: bool = False) -> None:
    """The real-gated linear recurrence over each sequence's rows: gates_r, gates_i, u [T, width] floats (the
    gates' products before bias and sigmoid, the convolved branch), y float rows (the other branch before its
    GELU; may be a view of wider rows), rb, ib, lam [width]; writes S * gelu(y) and keeps S in `state`.
    `runs`: the side-by-side walk for steps of many rows per sequence (equal up to rounding)."""
    _need_cuda(gates_r, gates_i, u, y, rb, ib, lam, seq_start, seq_slot, state, out)
    for t in (gates_r, gates_i, u):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape[1] == width
    assert y.dtype == torch.float32 and y.stride(1) == 1 and y.shape[1] == width
    assert out.is_contiguous() and out.shape[1] == width
    sp, ss = _state(state)
    _call("core", "mdma_rglru_scan", _ptr(gates_r), _ptr(gates_i), _ptr(u), _ptr(y), _i(y.stride(0)), _ptr(rb), _ptr(ib),
          _ptr(lam), _i(_same_dtype(rb, ib, lam)), _f(decay), _ptr(seq_start), _ptr(seq_slot), sp, ss, _ptr(out),
          _i(dtype_code(out.dtype)), _i(n_seqs), _i(width), _i(int(runs)), _stream())


# ---- attention with a penalty on distance (csrc/attention_distance.cu) -------------------------------------------
def kv_store(proj, k_col: int, v_col: int, k_width: int, v_width: int, tok_seq, tok_pos, seq_slot, page_table,
             max_pages: int, page_size: int, k_cache, v_cache, n_tokens: int) -> None:
    """The k and v parts of the projection rows go to the tokens' cache rows (no position encoding)."""
    _need_cuda(proj, tok_seq, tok_pos, seq_slot, page_table, k_cache, v_cache)
    assert proj.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.dtype == proj.dtype == v_cache.dtype
    _call("core", "mdma_kv_store", _ptr(proj), _i(dtype_code(proj.dtype)), _i(proj.stride(0)), _i(k_col), _i(v_col),
          _i(k_width), _i(v_width), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot), _ptr(page_table), _i(max_pages),
          _i(page_size), _ptr(k_cache), _ptr(v_cache), _i(n_tokens), _stream())


def attention_distance_tiled_fits(n_heads: int, n_kv_heads: int, dim: int, v_dim: int) -> bool:
    lib = _build._loaded.get("core") or _build.load("core")
    return bool(lib.mdma_attention_distance_tiled_fits(_i(n_heads), _i(n_kv_heads), _i(dim), _i(v_dim)))


def attention_distance(q, k_cache, v_cache, ctx, page_table, max_pages: int, page_size: int, slopes, gate, out,
                       n_heads: int, n_kv_heads: int, dim: int, v_dim: int, window: int, scale: float,
                       tiled: bool = False, sinks=None, gate_heads: bool = False, out_scale: float = 1.0) -> None:
    """Softmax attention with score (q.k) * scale - slopes[h] * distance over the paged cache; q: rows whose first
    n_heads * dim columns are the queries; `gate` (rows of n_heads * v_dim, optional): the result is multiplied by
    its sigmoid; out [T, n_heads * v_dim].  `tiled`: the kernel that stages keys and values per tile of query rows.
    `sinks` [n_heads] floats: exp(sink) joins each head's normaliser once; `gate_heads`: the gate has one number per
    head (rows of n_heads); `out_scale` multiplies the result."""
    _need_cuda(q, k_cache, v_cache, page_table, slopes, gate, out)
    assert q.stride(1) == 1 and out.is_contiguous() and out.dtype == q.dtype == k_cache.dtype == v_cache.dtype
    assert out.shape[1] == n_heads * v_dim and out.shape[0] >= ctx.n_tokens
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == n_heads and slopes.is_contiguous())
    assert gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1 and gate.shape[1] >= (n_heads if gate_heads else n_heads * v_dim))
    assert sinks is None or (sinks.is_cuda and sinks.dtype == torch.float32 and sinks.numel() == n_heads and sinks.is_contiguous())
    _call("core", "mdma_attention_distance", _ptr(q), _i(dtype_code(q.dtype)), _i(q.stride(0)), _ptr(k_cache), _ptr(v_cache),
          _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.seq_pos0),
          _ptr(page_table), _i(max_pages), _i(page_size), _ptr(slopes), _ptr(gate),
          _i(gate.stride(0) if gate is not None else 0), _ptr(out), _i(ctx.n_tokens), _i(ctx.n_seqs), _i(ctx.max_new),
          _i(n_heads), _i(n_kv_heads), _i(dim), _i(v_dim), _i(window), _f(scale), _i(int(tiled)), _ptr(sinks),
          _i(int(gate_heads)), _f(out_scale), _stream())


# ---- routed feed-forward (csrc/routed_ffn.cu) -----------------------------------------------------------------------
def route(h, router, correction, shared_gate, n_tokens: int, top: int, n_groups: int, keep_groups: int, chosen, weights,
          shared_scale, scoring: str = "softmax", group_top: int = 1, renormalize: bool = True) -> None:
    """Per token: scores over the router's logits (`scoring`: "softmax" over all, or "sigmoid" of each), choice among the
    best groups (a group's score: the sum of its `group_top` largest), `top` experts and their weights (their scores,
    divided by their sum if `renormalize`); with `shared_gate` [width] also sigmoid(shared_gate . h) into `shared_scale`."""
    assert scoring in ("softmax", "sigmoid")
    _need_cuda(h, router, correction, shared_gate, chosen, weights, shared_scale)
    n_routed, width = router.shape
    assert h.stride(1) == 1 and h.shape[1] == width and router.is_contiguous()
    assert chosen.dtype == torch.int32 and weights.dtype == torch.float32 and chosen.is_contiguous() and weights.is_contiguous()
    assert correction is None or (correction.numel() == n_routed and correction.is_contiguous())
    assert shared_gate is None or (shared_gate.numel() == width and shared_gate.dtype == router.dtype and shared_gate.is_contiguous())
    _call("core", "mdma_route", _ptr(h), _i(dtype_code(h.dtype)), _i(h.stride(0)), _ptr(router), _i(dtype_code(router.dtype)),
          _ptr(correction), _i(dtype_code(correction.dtype) if correction is not None else F32), _ptr(shared_gate),
          _i(n_tokens), _i(width), _i(n_routed), _i(top), _i(n_groups), _i(keep_groups), _i(int(scoring == "sigmoid")),
          _i(group_top), _i(int(renormalize)), _ptr(chosen), _ptr(weights), _ptr(shared_scale), _stream())


def experts(h, gate_w, up_w, down_w, chosen, weights, n_tokens: int, n_experts: int, top: int, ff: int, act, x,
            sorted_scratch=None, pair_act: int = ACT_SILU, act_limit: float = 0.0, act_alpha: float = 1.0) -> None:
    """x += sum over each token's chosen experts of weight * expert(h) (identity experts: weight * h).  gate_w, up_w
    [experts * ff, width], down_w [experts * width, ff]; act [tokens * top, ff] scratch in h's dtype.
    `sorted_scratch` = (first [2 * (experts + 1)] ints, order, y): the expert-by-expert kernels (steps of many tokens); else token by token."""
    _need_cuda(h, gate_w, up_w, down_w, chosen, weights, act, x)
    width = h.shape[1]
    assert h.stride(1) == 1 and x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == width
    assert act.is_contiguous() and act.dtype == h.dtype and act.shape[1] == ff
    if n_experts:
        assert gate_w.is_contiguous() and up_w.is_contiguous() and down_w.is_contiguous()
        assert tuple(gate_w.shape) == (n_experts * ff, width) == tuple(up_w.shape) and tuple(down_w.shape) == (n_experts * width, ff)
        assert gate_w.dtype == up_w.dtype == down_w.dtype
    wd = dtype_code(gate_w.dtype) if n_experts else dtype_code(h.dtype)
    if sorted_scratch is None:
        _call("core", "mdma_experts_by_token", _ptr(h), _i(dtype_code(h.dtype)), _i(h.stride(0)), _ptr(gate_w), _ptr(up_w),
              _ptr(down_w), _i(wd), _ptr(chosen), _ptr(weights), _i(n_tokens), _i(n_experts), _i(top), _i(width), _i(ff),
              _ptr(act), _ptr(x), _i(pair_act), _f(act_limit), _f(act_alpha), _stream(), launches=2)
        return
    first, order, y = sorted_scratch
    _need_cuda(first, order, y)
    assert first.dtype == order.dtype == torch.int32 and first.numel() >= 2 * (n_experts + 1) and order.numel() >= n_tokens * top
    assert y.dtype == torch.float32 and y.is_contiguous() and y.numel() >= n_tokens * top * width
    _call("core", "mdma_experts_sorted", _ptr(h), _i(dtype_code(h.dtype)), _i(h.stride(0)), _ptr(gate_w), _ptr(up_w),
          _ptr(down_w), _i(wd), _ptr(chosen), _ptr(weights), _i(n_tokens), _i(n_experts), _i(top), _i(width), _i(ff),
          _ptr(first), _ptr(order), _ptr(act), _ptr(y), _ptr(x), _i(pair_act), _f(act_limit), _f(act_alpha), _stream(),
          launches=4)


def experts_gather(h, chosen, n_tokens: int, n_experts: int, top: int, first, order, where, rows) -> None:
    """Sort the (token, choice) pairs by expert (first [n_experts + 1], order and its inverse `where` [tokens * top])
    and copy each sorted pair's input row to `rows` [tokens * top, width], expert after expert."""
    _need_cuda(h, chosen, first, order, where, rows)
    width = h.shape[1]
    assert h.stride(1) == 1 and rows.is_contiguous() and rows.dtype == h.dtype and rows.shape[1] == width
    assert first.dtype == order.dtype == where.dtype == chosen.dtype == torch.int32
    assert first.numel() >= 2 * (n_experts + 1) and order.numel() >= n_tokens * top and where.numel() >= n_tokens * top
    assert rows.shape[0] >= n_tokens * top
    _call("core", "mdma_experts_gather", _ptr(h), _i(dtype_code(h.dtype)), _i(h.stride(0)), _ptr(chosen), _i(n_tokens),
          _i(n_experts), _i(top), _i(width), _ptr(first), _ptr(order), _ptr(where), _ptr(rows), _stream(), launches=2)


def experts_combine(y, h, chosen, weights, where, n_tokens: int, n_experts: int, top: int, x) -> None:
    """x[t] += sum_j weights[t, j] * (y[where[t * top + j]] or, for an identity expert, h[t]); y float rows in the
    sorted list's order."""
    _need_cuda(y, h, chosen, weights, where, x)
    width = h.shape[1]
    assert y.dtype == torch.float32 and y.is_contiguous() and x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == width
    _call("core", "mdma_experts_combine", _ptr(y), _ptr(h), _i(dtype_code(h.dtype)), _i(h.stride(0)), _ptr(chosen),
          _ptr(weights), _ptr(where), _i(n_tokens), _i(n_experts), _i(top), _i(width), _ptr(x), _stream())


# ---- attention made ready in one pass, per-head gates, a norm on a sublayer's result (csrc/attention_prepare.cu) -------
def qk_prepare(proj, k_col: int, v_col: int, tok_seq, tok_pos, seq_slot, inv_freq, k_cache, v_cache, page_table,
               max_pages: int, page_size: int, n_tokens: int, n_heads: int, n_kv_heads: int, dim: int, v_dim: int,
               rotary_dim: int, interleaved: bool, unit_norm: bool, eps: float, write_kv: bool) -> None:
    """Rows [q heads | ... k heads at k_col | ... v heads at v_col]: q and k heads are rotated by the token's position
    (the first `rotary_dim` numbers of each head) and, with `unit_norm`, divided by their root mean square (eps inside
    the root); q in place, k and v to the token's cache row (`write_kv`)."""
    _need_cuda(proj, tok_seq, tok_pos, seq_slot, inv_freq, k_cache, v_cache, page_table)
    assert proj.stride(1) == 1 and (inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2))
    if write_kv:
        assert k_cache.dtype == proj.dtype == v_cache.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert k_cache.shape[-1] == dim and v_cache.shape[-1] == v_dim
        assert proj.shape[1] >= v_col + n_kv_heads * v_dim and v_col >= k_col + n_kv_heads * dim >= 0
    _call("core", "mdma_qk_prepare", _ptr(proj), _i(dtype_code(proj.dtype)), _i(proj.stride(0)), _i(k_col), _i(v_col),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot), _ptr(inv_freq), _ptr(k_cache), _ptr(v_cache), _ptr(page_table),
          _i(max_pages), _i(page_size), _i(n_tokens), _i(n_heads), _i(n_kv_heads), _i(dim), _i(v_dim), _i(rotary_dim),
          _i(int(interleaved)), _i(int(unit_norm)), _f(eps), _i(int(write_kv)), _stream())


def head_gate(out: torch.Tensor, gate: Optional[torch.Tensor], n_rows: int, n_heads: int, v_dim: int, scale: float = 1.0) -> None:
    """out[t, h * v_dim + d] *= sigmoid(gate[t, h]) * scale in place; gate may be a view of wider rows."""
    _need_cuda(out, gate)
    assert out.is_contiguous() and out.shape[1] == n_heads * v_dim
    assert gate is None or (gate.dtype == out.dtype and gate.stride(1) == 1 and gate.shape[1] >= n_heads)
    _call("core", "mdma_head_gate", _ptr(out), _ptr(gate), _i(dtype_code(out.dtype)), _i(gate.stride(0) if gate is not None else 0), _i(n_rows),
          _i(n_heads), _i(v_dim), _f(scale), _stream())


def rmsnorm_add(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, n_rows: int,
                partial: Optional[torch.Tensor] = None, splits: int = 0, split_stride: int = 0) -> None:
    """x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w; x and y float rows.  With `partial` [splits, rows, width], y is first
    completed by those sums (a K-split product not yet added up)."""
    _need_cuda(x, y, w, partial)
    width = x.shape[1]
    assert x.dtype == y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape[1] == width
    assert w.numel() == width and w.is_contiguous()
    _call("core", "mdma_rmsnorm_add", _ptr(x), _ptr(y), _ptr(partial), _i(splits if partial is not None else 0),
          ctypes.c_long(split_stride), _ptr(w), _i(dtype_code(w.dtype)), _i(n_rows), _i(width), _f(eps), _stream())


def add_scaled(y: torch.Tensor, z: torch.Tensor, a: float, n_rows: int) -> None:
    """y[:n_rows] += a * z[:n_rows]; float rows of one width."""
    _need_cuda(y, z)
    assert y.dtype == z.dtype == torch.float32 and y.is_contiguous() and z.is_contiguous() and y.shape[1] == z.shape[1]
    _call("core", "mdma_add_scaled", _ptr(y), _ptr(z), _f(a), ctypes.c_long(n_rows * y.shape[1]), _stream())


# ---- linear attention with a decay per head (csrc/linear_attention.cu) -----------------------------------------------------
def linear_attention_fits(dim: int, vdim: int, chunked: bool = False) -> bool:
    """Whether heads of dim x vdim fit a block's shared memory in the walk row by row, or a chunk of rows at a time."""
    lib = _build._loaded.get("core") or _build.load("core")
    return bool(lib.mdma_linear_attention_fits(_i(dim), _i(vdim), _i(int(chunked))))


def linear_attention(proj, q_col: int, k_col: int, v_col: int, decay, seq_start, seq_slot, state, out, n_seqs: int,
                     heads: int, dim: int, vdim: int, chunked: bool = False, run_rows: int = 0, max_runs: int = 1,
                     scratch=None, single: bool = False) -> None:
    """S = decay_h S + k v^T, o = S^T q per head over each sequence's rows, q, k, v = SiLU of the columns q_col.., k_col..,
    v_col.. of `proj`; state [slots, heads * dim * vdim] floats is read and brought up to date; out [T, heads * vdim]
    floats.  `chunked`: the walk a chunk of rows at a time, and with `run_rows` > 0 in runs of that many rows side by
    side (`max_runs`: the most runs of a sequence; `scratch`: n_seqs * max_runs * heads * dim * vdim floats); `single`:
    the kernel for steps in which no sequence brings more than one row.  Equal up to rounding."""
    _need_cuda(proj, decay, seq_start, seq_slot, state, out)
    _need_cuda(scratch)
    assert proj.stride(1) == 1 and decay.dtype == torch.float32 and decay.numel() == heads and decay.is_contiguous()
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape[1] == heads * vdim
    assert proj.shape[1] >= max(q_col + heads * dim, k_col + heads * dim, v_col + heads * vdim)
    assert run_rows == 0 or (chunked and scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous())
    assert not (single and chunked)
    sp, ss = _state(state)
    assert state.shape[1] >= heads * dim * vdim
    _call("core", "mdma_linear_attention", _ptr(proj), _i(dtype_code(proj.dtype)), _i(proj.stride(0)), _i(q_col), _i(k_col),
          _i(v_col), _ptr(decay), _ptr(seq_start), _ptr(seq_slot), sp, ss, _ptr(out), _i(n_seqs), _i(heads), _i(dim),
          _i(vdim), _i(2 if single else int(chunked)), _i(run_rows), _i(max_runs), _ptr(scratch),
          ctypes.c_long(scratch.numel() if scratch is not None else 0), _stream(), launches=2 if run_rows > 0 else 1)


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n_rows: int, eps: float,
                  scale: float = 1.0) -> None:
    """out = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate) * scale; o float rows, gate may be a view of wider rows."""
    _need_cuda(o, gate, w, out)
    width = o.shape[1]
    assert o.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous() and out.shape[1] == width
    assert gate.stride(1) == 1 and gate.shape[1] >= width and w.numel() == width and w.is_contiguous()
    _call("core", "mdma_gated_rmsnorm", _ptr(o), _ptr(gate), _i(dtype_code(gate.dtype)), _i(gate.stride(0)), _ptr(w),
          _i(dtype_code(w.dtype)), _ptr(out), _i(dtype_code(out.dtype)), _i(n_rows), _i(width), _f(eps), _f(scale), _stream())


# ---- RMS norm in groups, the weighted sum over the depth (csrc/group_norm.cu) ----------------------------------------
def group_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, groups: int, out: torch.Tensor,
                  rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> None:
    """out[i] = the row x[rows[i]] (or x[i]) in `groups` equal parts, each divided by its own root mean square, times w."""
    _need_cuda(x, w, out, rows)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    width = x.shape[-1]
    assert w.numel() == width and out.shape[-1] == width and w.is_contiguous()
    n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert out.shape[0] >= n and (rows is None or rows.dtype == torch.int32)
    _call("core", "mdma_group_rmsnorm", _ptr(x), _ptr(w), _i(dtype_code(w.dtype)), _ptr(rows), _ptr(out),
          _i(dtype_code(out.dtype)), _i(n), _i(width), _i(groups), _f(eps), _stream())


def group_rmsnorm_add(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, groups: int, n_rows: int,
                      partial: Optional[torch.Tensor] = None, splits: int = 0, split_stride: int = 0) -> None:
    """x[t] += group norm of y[t] times w; x and y float rows.  With `partial` [splits, rows, width], y is first
    completed by those sums (a K-split product not yet added up)."""
    _need_cuda(x, y, w, partial)
    width = x.shape[1]
    assert x.dtype == y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape[1] == width
    assert w.numel() == width and w.is_contiguous()
    _call("core", "mdma_group_rmsnorm_add", _ptr(x), _ptr(y), _ptr(partial), _i(splits if partial is not None else 0),
          ctypes.c_long(split_stride), _ptr(w), _i(dtype_code(w.dtype)), _i(n_rows), _i(width), _i(groups), _f(eps), _stream())


def depth_mix(x: torch.Tensor, x0: torch.Tensor, history: torch.Tensor, depth: int, run: int, w: torch.Tensor,
              n_rows: int) -> None:
    """history[t, run] = x[t]; x[t] = w[0] x0[t] + sum_{j<=run} w[j+1] history[t, j].  Float rows; history
    [rows, depth * width]."""
    _need_cuda(x, x0, history, w)
    width = x.shape[1]
    assert x.dtype == x0.dtype == history.dtype == torch.float32 and x.is_contiguous() and x0.is_contiguous()
    assert history.is_contiguous() and history.shape[1] == depth * width and w.numel() >= run + 2 and w.is_contiguous()
    _call("core", "mdma_depth_mix", _ptr(x), _ptr(x0), _ptr(history), _i(depth), _i(run), _ptr(w), _i(dtype_code(w.dtype)),
          _i(n_rows), _i(width), _stream())


# ---- a cached latent with a turned key part (csrc/rotary_latent.cu) ----------------------------------------------------
def latent_prepare(proj, q_col: int, q_rank: int, q_w, kv_col: int, kv_rank: int, kv_w, eps: float, rot_dim: int,
                   rotary_dim: int, interleaved: bool, inv_freq, magnitude: float, tok_seq, tok_pos, seq_slot, page_table,
                   max_pages: int, page_size: int, cq, cache, write_cache: bool, n_tokens: int) -> None:
    """cq[t] = rms_unit(proj[t, q_col:+q_rank]) * q_w; with `write_cache`, the token's cache row becomes
    [rms_unit(proj[t, kv_col:+kv_rank]) * kv_w | the next rot_dim numbers, turned by the token's position]."""
    _need_cuda(proj, q_w, kv_w, inv_freq, tok_seq, tok_pos, seq_slot, page_table, cq, cache)
    assert proj.stride(1) == 1 and cq.is_contiguous() and cq.dtype == proj.dtype and cq.shape[1] == q_rank
    assert q_w.numel() == q_rank and q_w.is_contiguous()
    w_dtype = dtype_code(q_w.dtype)
    if write_cache:
        assert cache.is_contiguous() and cache.dtype == proj.dtype and cache.shape[-1] == kv_rank + rot_dim
        assert kv_w.numel() == kv_rank and kv_w.dtype == q_w.dtype and kv_w.is_contiguous()
        assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2)
    _call("core", "mdma_latent_prepare", _ptr(proj), _i(dtype_code(proj.dtype)), _i(proj.stride(0)), _i(q_col), _i(q_rank),
          _ptr(q_w), _i(kv_col), _i(kv_rank), _ptr(kv_w), _i(w_dtype), _f(eps), _i(rot_dim), _i(rotary_dim),
          _i(int(interleaved)), _ptr(inv_freq), _f(magnitude), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot), _ptr(page_table),
          _i(max_pages), _i(page_size), _ptr(cq), _ptr(cache), _i(int(write_cache)), _i(n_tokens), _stream())


def rotate_heads(q, n_heads: int, head_pitch: int, offset: int, rotary_dim: int, interleaved: bool, inv_freq,
                 magnitude: float, tok_pos, n_tokens: int) -> None:
    """Columns [offset, offset + rotary_dim) of every head of q [tokens, heads * head_pitch] turned in place."""
    _need_cuda(q, inv_freq, tok_pos)
    assert q.stride(1) == 1 and q.shape[1] >= n_heads * head_pitch
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2)
    _call("core", "mdma_rotate_heads", _ptr(q), _i(dtype_code(q.dtype)), _i(q.stride(0)), _i(n_heads), _i(head_pitch),
          _i(offset), _i(rotary_dim), _i(int(interleaved)), _ptr(inv_freq), _f(magnitude), _ptr(tok_pos), _i(n_tokens), _stream())


# ---- attention whose heads' scores are mixed before the softmax (csrc/attention_talking.cu) --------------------------
def qk_norm_rotate(proj, k_col: int, v_col: int, tok_seq, tok_pos, seq_slot, inv_freq, magnitude: float, q_w, k_w,
                   norm: bool, eps: float, k_cache, v_cache, page_table, max_pages: int, page_size: int, n_tokens: int,
                   n_heads: int, n_kv_heads: int, dim: int, v_dim: int, rotary_dim: int, interleaved: bool,
                   write_kv: bool) -> None:
    """Rows [q heads | k heads at k_col | v heads at v_col]: q and k heads are (with `norm`) divided by their root mean
    square and multiplied by q_w / k_w [dim], then their first `rotary_dim` numbers are turned by the token's position;
    q in place, k and v to the token's cache row (`write_kv`)."""
    _need_cuda(proj, tok_seq, tok_pos, seq_slot, inv_freq, q_w, k_w, k_cache, v_cache, page_table)
    assert proj.stride(1) == 1 and (inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2))
    w_dtype = F32
    if q_w is not None:
        assert q_w.numel() == dim and k_w.numel() == dim and q_w.dtype == k_w.dtype and q_w.is_contiguous() and k_w.is_contiguous()
        w_dtype = dtype_code(q_w.dtype)
    if write_kv:
        assert k_cache.dtype == proj.dtype == v_cache.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert k_cache.shape[-1] == dim and v_cache.shape[-1] == v_dim
        assert proj.shape[1] >= v_col + n_kv_heads * v_dim and v_col >= k_col + n_kv_heads * dim >= 0
    _call("core", "mdma_qk_norm_rotate", _ptr(proj), _i(dtype_code(proj.dtype)), _i(proj.stride(0)), _i(k_col), _i(v_col),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot), _ptr(inv_freq), _f(magnitude), _ptr(q_w), _ptr(k_w), _i(w_dtype),
          _i(int(norm)), _f(eps), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _i(max_pages), _i(page_size), _i(n_tokens),
          _i(n_heads), _i(n_kv_heads), _i(dim), _i(v_dim), _i(rotary_dim), _i(int(interleaved)), _i(int(write_kv)), _stream())


def talking_attention_tiled_fits(n_heads: int, n_kv_heads: int, dim: int, v_dim: int) -> bool:
    """Whether the tiled kernel's shared memory takes this geometry at all (with tiles of one row at least)."""
    lib = _build._loaded.get("core") or _build.load("core")
    return n_heads % n_kv_heads == 0 and bool(lib.mdma_talking_attention_tile_rows(_i(n_heads), _i(n_kv_heads), _i(dim), _i(v_dim), _i(1)))


def talking_attention(q, k_cache, v_cache, talk, sinks, ctx, page_table, max_pages: int, page_size: int, out,
                      n_heads: int, n_kv_heads: int, dim: int, v_dim: int, window: int, scale: float,
                      tiled: bool = False) -> None:
    """out[t, h] = sum_j p_hj v_j with p_h the softmax over the keys up to the token's position of the MIXED scores
    sum_g talk[h, g] (q_g . k_j) scale; `sinks` [heads] float join each denominator as exp(sink_h); `talk` None: heads
    on their own.  `tiled`: the kernel that stages keys and values per tile of query rows (else a block per token
    that visits the keys in position order)."""
    _need_cuda(q, k_cache, v_cache, talk, sinks, page_table, out)
    assert q.stride(1) == 1 and out.is_contiguous() and out.dtype == q.dtype == k_cache.dtype == v_cache.dtype
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and out.shape[1] == n_heads * v_dim and out.shape[0] >= ctx.n_tokens
    assert talk is None or (talk.dtype == torch.float32 and talk.is_contiguous() and talk.numel() == n_heads * n_heads)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == n_heads)
    if tiled:
        _call("core", "mdma_talking_attention_tiled", _ptr(q), _i(dtype_code(q.dtype)), _i(q.stride(0)), _ptr(k_cache),
              _ptr(v_cache), _ptr(talk), _ptr(sinks), _ptr(ctx.seq_start), _ptr(ctx.seq_pos0), _ptr(ctx.seq_slot),
              _ptr(page_table), _i(max_pages), _i(page_size), _ptr(out), _i(ctx.n_tokens), _i(ctx.n_seqs), _i(ctx.max_new),
              _i(n_heads), _i(n_kv_heads), _i(dim), _i(v_dim), _i(window), _f(scale), _stream())
        return
    _call("core", "mdma_talking_attention", _ptr(q), _i(dtype_code(q.dtype)), _i(q.stride(0)), _ptr(k_cache), _ptr(v_cache),
          _ptr(talk), _ptr(sinks), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(ctx.seq_slot), _ptr(page_table), _i(max_pages),
          _i(page_size), _ptr(out), _i(ctx.n_tokens), _i(n_heads), _i(n_kv_heads), _i(dim), _i(v_dim), _i(window), _f(scale),
          _stream())
