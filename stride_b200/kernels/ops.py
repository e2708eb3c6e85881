"""Python faces of the CUDA kernels: torch tensors in, raw pointers down.

Every function here launches hand-written CUDA from `stride_b200/csrc` on the
current torch stream. There is no torch or CPU implementation behind them: a
tensor that is not on a CUDA device, or a library that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from .build import library

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_configured: set = set()


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"stride_b200 kernels take float32 or bfloat16 tensors, not {dtype}") from None


def _fn(lib_name: str, fn_name: str, argtypes):
    lib = library(lib_name)
    fn = getattr(lib, fn_name)
    if (lib_name, fn_name) not in _configured:
        fn.argtypes = argtypes
        fn.restype = c_int
        _configured.add((lib_name, fn_name))
    return lib, fn


launches = 0    # kernels launched through this module since import (bench.py reports the difference)


def _check(lib, rc: int) -> None:
    global launches
    launches += 1
    if rc != 0:
        raise RuntimeError(lib.sb_last_error().decode(errors="replace"))


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("stride_b200 kernels run on CUDA tensors only; got a tensor on " + str(t.device))


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current torch stream's handle (kernels are launched on it, so they order with torch's own work)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, slots=None, sampled=None, copy=None, scale: float = 1.0) -> None:
    """out[i, :] = float32(table[tokens[i], :]) * scale; a token of -1 means sampled[slots[i]] (the request's last sampled token).
    `copy` (float32, the shape of out) receives the same rows."""
    _cuda(tokens, table, out, slots, sampled, copy)
    lib, fn = _fn("elementwise", "sb_embed", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float,
                                              c_void_p])
    n, H = out.shape
    _check(lib, fn(_ptr(tokens), _ptr(table), dtype_code(table.dtype), _ptr(out), n, H, table.shape[0], _ptr(slots),
                   _ptr(sampled) if slots is not None else 0, _ptr(copy), scale, _stream()))


def layernorm(h: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float, out: torch.Tensor, partials=None) -> None:
    """out = (x - mean(x)) / sqrt(var(x) + eps) * weight + bias with x = h (+ partials[0] + partials[1] ...), folded into h
    in place as `rmsnorm` does."""
    _cuda(h, weight, bias, out, partials)
    if weight.dtype != bias.dtype:
        raise TypeError("layernorm takes a gain and a bias of one dtype")
    lib, fn = _fn("norm", "sb_layernorm", [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                           c_int, c_int, c_float, c_void_p])
    n, H = h.shape
    S = 0 if partials is None else partials.shape[0]
    stride = 0 if partials is None else partials.stride(0)
    _check(lib, fn(_ptr(h), _ptr(partials), S, stride, _ptr(weight), _ptr(bias), dtype_code(weight.dtype), _ptr(out),
                   dtype_code(out.dtype), n, H, eps, _stream()))


def concat_rows(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, partials=None, clear_a: bool = False) -> None:
    """out[i] = [a[i] (+ partials[s, i] for every s, ascending); b[i]]: float32 [n, H] twice into [n, 2 H] of out's dtype.
    With `clear_a`, a is zero afterwards."""
    _cuda(a, b, out, partials)
    lib, fn = _fn("elementwise", "sb_concat_rows", [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    n, H = a.shape
    S = 0 if partials is None else partials.shape[0]
    stride = 0 if partials is None else partials.stride(0)
    _check(lib, fn(_ptr(a), _ptr(partials), S, stride, _ptr(b), _ptr(out), dtype_code(out.dtype), n, H, int(clear_a), _stream()))


def lightning_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, entry_meta: torch.Tensor, entries: int, decay: torch.Tensor,
                   state: torch.Tensor, out: torch.Tensor, heads: int, key_dim: int, value_dim: int, act=None) -> None:
    """The decayed linear-attention recurrence for every entry of a step (csrc/lightning.cu). proj [S, n, width] float32:
    partial sums of the projection with q, k, v at the given columns; entry_meta [4, E] on the device; state
    [slots, heads, key_dim, value_dim] float32 (read unless the entry starts at position 0, written back); out [n, heads * value_dim].
    `act`: float32 scratch of n * (columns of q, k, v) elements; with it a long step's activations are made by a kernel of their own."""
    _cuda(proj, entry_meta, decay, state, out, act)
    lib, fn = _fn("lightning", "sb_lightning_scan", [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                                    c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    if proj.dim() == 2:
        proj = proj.unsqueeze(0)
    _check(lib, fn(_ptr(proj), proj.shape[0], proj.stride(0), proj.shape[2], q_off, k_off, v_off, _ptr(entry_meta), entry_meta.stride(0),
                   entries, proj.shape[1], _ptr(decay), _ptr(state), _ptr(out), _ptr(act), heads, key_dim, value_dim, _stream()))


def gated_rmsnorm(o: torch.Tensor, proj: torch.Tensor, g_off: int, gain: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out = o / sqrt(mean(o^2) + eps) * gain * sigmoid(gate), the gate being columns g_off.. of proj [S, n, width] (partial sums)."""
    _cuda(o, proj, gain, out)
    lib, fn = _fn("lightning", "sb_gated_rmsnorm", [c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                                   c_int, c_int, c_float, c_void_p])
    if proj.dim() == 2:
        proj = proj.unsqueeze(0)
    n, W = o.shape
    _check(lib, fn(_ptr(o), _ptr(proj), proj.shape[0], proj.stride(0), proj.shape[2], g_off, _ptr(gain), dtype_code(gain.dtype), _ptr(out),
                   dtype_code(out.dtype), n, W, eps, _stream()))


def rmsnorm(h: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, partials=None) -> None:
    """out = weight * (x / sqrt(mean(x^2) + eps)) with x = h (+ partials[0] + partials[1] ...).

    `partials` [S, n, H] float32 are summed into h left to right and h is updated in place.
    """
    _cuda(h, weight, out, partials)
    lib, fn = _fn("norm", "sb_rmsnorm", [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p, c_int,
                                               c_int, c_int, c_float, c_void_p])
    n, H = h.shape
    S = 0 if partials is None else partials.shape[0]
    stride = 0 if partials is None else partials.stride(0)
    _check(lib, fn(_ptr(h), _ptr(partials), S, stride, _ptr(weight), dtype_code(weight.dtype), _ptr(out),
                   dtype_code(out.dtype), n, H, eps, _stream()))


def rope_append(qkv: torch.Tensor, positions, slots, cos_sin, rotary_dim: int, q_out, cache_layer, block_table,
                num_heads: int, num_kv_heads: int, head_dim: int, write_kv: bool = True, values_from_keys: bool = False) -> None:
    """Rotate q and k of `qkv` [S, n, (Hq + 2 Hkv) D] (partials summed), store q, append k and v to the pages.
    With `values_from_keys` qkv is [S, n, (Hq + Hkv) D] and a value head is its key head before rotation.

    `cache_layer` is this layer's view [pages, 2, Hkv, page_size, D] of the arena.
    """
    _cuda(qkv, positions, slots, cos_sin, q_out, cache_layer, block_table)
    lib, fn = _fn("elementwise", "sb_rope_append",
                  [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                   c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    if qkv.dim() == 2:
        qkv = qkv.unsqueeze(0)
    S, n, _ = qkv.shape
    _check(lib, fn(_ptr(qkv), S, qkv.stride(0), _ptr(positions), _ptr(slots), _ptr(cos_sin), rotary_dim, _ptr(q_out),
                   dtype_code(q_out.dtype), _ptr(cache_layer), dtype_code(cache_layer.dtype), _ptr(block_table),
                   block_table.shape[1], cache_layer.shape[3], cache_layer.stride(0), cache_layer.stride(1),
                   cache_layer.stride(2), n, num_heads, num_kv_heads, head_dim, int(write_kv), int(values_from_keys), _stream()))


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[n, I] = act(gate_up[:, :I]) * gate_up[:, I:], act = silu or the tanh form of gelu."""
    _cuda(gate_up, out)
    lib, fn = _fn("elementwise", "sb_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    n, I = out.shape
    _check(lib, fn(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), n, I, GATE_ACTIVATIONS[activation], _stream()))


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor, partials=None) -> None:
    """out[i, :] = src[rows[i], :] (+ partials[s, rows[i], :] for every s)."""
    _cuda(src, rows, out, partials)
    lib, fn = _fn("elementwise", "sb_gather_rows", [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p])
    S = 0 if partials is None else partials.shape[0]
    stride = 0 if partials is None else partials.stride(0)
    _check(lib, fn(_ptr(src), _ptr(partials), S, stride, _ptr(rows), _ptr(out), out.shape[0], out.shape[1], _stream()))


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out[n, M] (+)= x[n, K] . weight[M, K]^T in true 32-bit FMA; x and weight float32 or bfloat16."""
    _cuda(x, weight, out)
    if out.dtype != torch.float32:
        raise TypeError("gemm_f32 writes float32")
    lib, fn = _fn("gemm_f32", "sb_gemm_f32", [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_void_p, c_int64, c_int,
                                              c_int, c_int, c_int, c_void_p])
    n, K = x.shape
    M = weight.shape[0]
    if weight.shape[1] != K or out.shape[0] != n or out.shape[1] != M:
        raise ValueError(f"gemm_f32 shapes: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    _check(lib, fn(_ptr(x), dtype_code(x.dtype), x.stride(0), _ptr(weight), dtype_code(weight.dtype), weight.stride(0), _ptr(out),
                   out.stride(0), n, M, K, int(accumulate), _stream()))


def attention_generic(q, out, cache_layer, block_table, positions, slots, num_heads: int, num_kv_heads: int,
                      head_dim: int, window: int, scale: float) -> None:
    """Causal paged attention of every token of the step over its request's cache (any head size)."""
    _cuda(q, out, cache_layer, block_table, positions, slots)
    if not (q.dtype == out.dtype == cache_layer.dtype):
        raise TypeError("attention_generic takes q, out and cache of one dtype")
    lib, fn = _fn("attention_generic", "sb_attention_generic",
                  [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p,
                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), dtype_code(q.dtype), _ptr(cache_layer), _ptr(block_table), block_table.shape[1],
                   cache_layer.shape[3], cache_layer.stride(0), cache_layer.stride(1), cache_layer.stride(2),
                   _ptr(positions), _ptr(slots), q.shape[0], num_heads, num_kv_heads, head_dim, window, scale, _stream()))


def argmax(logits: torch.Tensor, tokens: torch.Tensor, values: torch.Tensor, scatter_index=None, scatter=None) -> None:
    """tokens[i] = index of the largest logit of row i (smallest index among equals); values[i] = that logit.
    With `scatter`, also scatter[scatter_index[i]] = tokens[i]."""
    _cuda(logits, tokens, values, scatter_index, scatter)
    lib, fn = _fn("sampling", "sb_argmax", [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(lib, fn(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(tokens), _ptr(values),
                   _ptr(scatter_index), _ptr(scatter) if scatter_index is not None else 0, _stream()))


def sample_temperature(logits, temperatures, seeds, lengths, tokens, values, scatter_index=None, scatter=None) -> None:
    """Temperature sampling keyed on (seed, sequence length) for every row with temperature > 0 (other rows are left
    alone); see csrc/sampling.cu. With `scatter`, also scatter[scatter_index[i]] = tokens[i]."""
    _cuda(logits, temperatures, seeds, lengths, tokens, values, scatter_index, scatter)
    lib, fn = _fn("sampling", "sb_sample_temperature", [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(lib, fn(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(temperatures), _ptr(seeds),
                   _ptr(lengths), _ptr(tokens), _ptr(values), _ptr(scatter_index),
                   _ptr(scatter) if scatter_index is not None else 0, _stream()))


STORE, ADD, SWIGLU, GEGLU_TANH = 0, 1, 2, 3     # GEGLU_TANH: SWIGLU with the tanh form of gelu on the gate


def gemm_tc_splits(M: int, K: int) -> int:
    """How many K ranges `gemm_tc` cuts a [M, K] weight into: a function of the weight's shape alone."""
    lib = library("gemm_tc")
    lib.sb_gemm_tc_splits.argtypes = [c_int, c_int]
    lib.sb_gemm_tc_splits.restype = c_int
    return lib.sb_gemm_tc_splits(M, K)


def gemm_tc_partial_tokens() -> int:
    """Up to this many tokens `gemm_tc` leaves one partial buffer per K range; with more it adds the ranges itself."""
    lib = library("gemm_tc")
    lib.sb_gemm_tc_partial_tokens.restype = c_int
    return lib.sb_gemm_tc_partial_tokens()


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int = STORE, splits: int = 1,
            half_rows: int = 0) -> None:
    """out = x . weight^T on the tcgen05 tensor cores; x [n, K] and weight [M, K] bfloat16.

    STORE: out float32 [n, M]. With splits > 1 (= gemm_tc_splits) and at most gemm_tc_partial_tokens() tokens, out is
    [splits, n, M]: one partial sum per K range, to be added in ascending order; with more tokens the kernel adds the
    ranges itself, in the same order, and out is [n, M].
    ADD: out float32 [n, M] += result (one range only).
    SWIGLU: weight is [2 I, K] (gate rows, then up rows) and out bfloat16 [n, I] = silu(x . gate^T) * (x . up^T).
    """
    _cuda(x, weight, out)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("gemm_tc takes bfloat16 operands")
    want = torch.bfloat16 if epilogue in (SWIGLU, GEGLU_TANH) else torch.float32
    if out.dtype != want:
        raise TypeError(f"gemm_tc epilogue {epilogue} writes {want}")
    lib, fn = _fn("gemm_tc", "sb_gemm_tc", [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int,
                                            c_int, c_int, c_int64, c_int, c_void_p])
    n, K = x.shape
    M = weight.shape[0]
    if weight.shape[1] != K:
        raise ValueError(f"gemm_tc shapes: x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    if splits > 1 and n <= gemm_tc_partial_tokens():
        if out.dim() != 3 or out.shape[0] != splits:
            raise ValueError("gemm_tc with K ranges and few tokens writes [splits, n, M]")
        ldo, split_stride = out.stride(1), out.stride(0)
    else:
        o2 = out[0] if out.dim() == 3 else out
        ldo, split_stride = o2.stride(0), 0
    _check(lib, fn(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), ldo, n, M, K, epilogue, splits,
                   split_stride, half_rows, _stream()))


def gemm_tc_status() -> int:
    """0 if every wait inside the tensor-core kernels completed since the last call; synchronises."""
    lib = library("gemm_tc")
    lib.sb_gemm_tc_status.restype = c_int
    return lib.sb_gemm_tc_status()


_status_word = None
_status_users = {"gemm_tc": "sb_gemm_tc_use_status_word", "attention_tc5": "sb_attention_tc5_use_status_word",
                 "decode_chain": "sb_decode_chain_use_status_word",
                 "sampling": "sb_sampling_use_status_word"}   # the sampling kernels only read it
_status_registered: set = set()


def shared_status_word(libraries=("gemm_tc",)) -> torch.Tensor:
    """One int32 on the device into which the bounded waits of the tensor-core kernels report when they give up:
    0 = every wait completed. Made at the first call; those of `libraries` that have such waits (gemm_tc,
    attention_tc5) use it from then on, and the sampling kernels report -1 - its value instead of a token while it is
    not 0, so that a lost signal is an error and not a wrong token."""
    global _status_word
    if _status_word is None:
        _status_word = torch.zeros(1, dtype=torch.int32, device="cuda")
    for lib_name in sorted(set(libraries) & set(_status_users) - _status_registered):
        fn = getattr(library(lib_name), _status_users[lib_name])
        fn.argtypes, fn.restype = [c_void_p], None
        fn(_status_word.data_ptr())
        _status_registered.add(lib_name)
    return _status_word


def lost_signal_selftest(code: int = 9) -> None:
    """Launches a kernel whose only wait is never answered: after about a second it gives up and the status word
    reads `code`. Exercises the path by which a lost signal inside a tensor-core kernel becomes an error."""
    lib, fn = _fn("gemm_tc", "sb_gemm_tc_lost_signal_selftest", [c_int, c_void_p])
    _check(lib, fn(code, _stream()))


def attention_tc_scratch(items: int, num_kv_heads: int, chunks: int, head_dim: int) -> int:
    """Floats of scratch `attention_tc` needs."""
    return items * num_kv_heads * chunks * 16 * (head_dim + 2)


_decode_rope_limit = None


def attention_decode_rope_limit() -> int:
    """Up to this many CTAs (entries x key/value heads x chunks) `attention_decode_rope` runs all at once on this
    device and is the faster choice; asked of the library once."""
    global _decode_rope_limit
    if _decode_rope_limit is None:
        lib = library("attention_tc")
        lib.sb_attention_decode_rope_resident_ctas.restype = c_int
        _decode_rope_limit = int(lib.sb_attention_decode_rope_resident_ctas())
    return _decode_rope_limit


def attention_tc(q, out, cache_layer, block_table, entry_meta, work, n_tiles: int, n_items: int, chunks: int,
                 scratch, num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                 counters=None) -> None:
    """Tensor-core paged attention (bfloat16, head_dim 64 or 128); see csrc/attention_tc.cu for `work`.
    `counters`: int32 zeros, one per (decode entry, kv head); with them the decode kernel folds its own chunks."""
    _cuda(q, out, cache_layer, block_table, entry_meta, work, scratch, counters)
    if not (q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16):
        raise TypeError("attention_tc takes bfloat16 q, out and cache")
    lib, fn = _fn("attention_tc", "sb_attention_tc",
                  [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int,
                   c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), _ptr(cache_layer), _ptr(block_table), block_table.shape[1], cache_layer.shape[3],
                   cache_layer.stride(0), cache_layer.stride(1), cache_layer.stride(2), _ptr(entry_meta),
                   entry_meta.stride(0), _ptr(work), n_tiles, n_items, chunks, _ptr(scratch), _ptr(counters), num_heads, num_kv_heads,
                   head_dim, window, scale, _stream()))


def attention_decode_rope(qkv, cos_sin, out, cache_layer, block_table, entry_meta, items, n_items: int, chunks: int, scratch,
                          counters, num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float) -> None:
    """The decode kernel of `attention_tc` with `rope_append` fused in, for steps whose entries all fit it: qkv
    [S, n, (Hq + 2 Hkv) D] float32 partial sums of the projection, cos_sin the table of a fully rotated head. Rotates
    q in shared memory, appends the step's rotated k and its v to the pages, attends. Same bits as the two kernels."""
    _cuda(qkv, cos_sin, out, cache_layer, block_table, entry_meta, items, scratch, counters)
    if not (out.dtype == cache_layer.dtype == torch.bfloat16) or qkv.dtype != torch.float32:
        raise TypeError("attention_decode_rope takes float32 qkv and bfloat16 out and cache")
    lib, fn = _fn("attention_tc", "sb_attention_decode_rope",
                  [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64,
                   c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    if qkv.dim() == 2:
        qkv = qkv.unsqueeze(0)
    _check(lib, fn(_ptr(qkv), qkv.shape[0], qkv.stride(0), _ptr(cos_sin), _ptr(out), _ptr(cache_layer), _ptr(block_table),
                   block_table.shape[1], cache_layer.shape[3], cache_layer.stride(0), cache_layer.stride(1),
                   cache_layer.stride(2), _ptr(entry_meta), entry_meta.stride(0), _ptr(items), n_items, chunks, _ptr(scratch),
                   _ptr(counters), num_heads, num_kv_heads, head_dim, window, scale, _stream()))


def attention_tc5_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """True if the tcgen05 prompt-attention kernel takes this shape (head size 64 or 128, pages of a power of two >= 8)."""
    if head_dim not in (64, 128) or num_kv_heads <= 0 or num_heads % num_kv_heads or num_heads // num_kv_heads > 128:
        return False
    return page_size >= 8 and page_size & (page_size - 1) == 0


def attention_tc5(q, out, cache_layer, block_table, entry_meta, work, n_tiles: int, num_heads: int, num_kv_heads: int,
                  head_dim: int, window: int, scale: float) -> None:
    """Prompt-portion attention on the tcgen05 tensor cores; `work` is [n_tiles, 2] = (entry, tile of 128 // G positions)."""
    _cuda(q, out, cache_layer, block_table, entry_meta, work)
    if not (q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16):
        raise TypeError("attention_tc5 takes bfloat16 q, out and cache")
    lib, fn = _fn("attention_tc5", "sb_attention_tc5",
                  [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int,
                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), _ptr(cache_layer), cache_layer.shape[0], _ptr(block_table), block_table.shape[1],
                   cache_layer.shape[3], cache_layer.stride(0), cache_layer.stride(1), cache_layer.stride(2), _ptr(entry_meta),
                   entry_meta.stride(0), _ptr(work), n_tiles, q.shape[0], num_heads, num_kv_heads, head_dim, window, scale,
                   _stream()))


def attention_tc5_status() -> int:
    """0 if every wait inside the tcgen05 attention kernel completed since the last call; synchronises."""
    lib = library("attention_tc5")
    lib.sb_attention_tc5_status.restype = c_int
    return lib.sb_attention_tc5_status()


# ---------------------------------------------------------------------------------------------------------------------
# Branches beside the residual stream, feed-forwards that are no plain gated product, attention without softmax, and
# recurrences with a gate per channel (csrc/branch.cu, feed_forward.cu, sigmoid_attention.cu, gated_recurrence.cu, rglru.cu)

def _partials(p):
    """(pointer, count, stride) of partial sums [P, n, M] (a 2-D tensor counts as P = 1), or zeros for None."""
    if p is None:
        return 0, 0, 0
    if p.dim() == 2:
        p = p.unsqueeze(0)
    return p.data_ptr(), p.shape[0], p.stride(0)


def branch_fold(dst: torch.Tensor, a=None, a_partials=None, ca: float = 1.0, b=None, b_partials=None, cb: float = 1.0, gain=None) -> None:
    """dst += gain * (ca * (a + sum of a_partials) + cb * (b + sum of b_partials)), all float32 [n, W]; a and b are zero afterwards."""
    _cuda(dst, a, a_partials, b, b_partials, gain)
    lib, fn = _fn("branch", "sb_branch_fold", [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_float, c_void_p, c_void_p, c_int, c_int64, c_float,
                                               c_void_p, c_int, c_int, c_int, c_void_p])
    n, W = dst.shape
    pa, na, sa = _partials(a_partials)
    pb, nb, sb = _partials(b_partials)
    _check(lib, fn(_ptr(dst), _ptr(a), pa, na, sa, ca, _ptr(b), pb, nb, sb, cb, _ptr(gain), dtype_code(gain.dtype) if gain is not None else 0,
                   n, W, _stream()))


def branch_norm_fold(dst: torch.Tensor, gain, eps: float, a=None, a_partials=None, ca: float = 1.0, b=None, b_partials=None, cb: float = 1.0) -> None:
    """y = ca * (a + sum of a_partials) + cb * (b + sum of b_partials); dst += gain * y / sqrt(mean(y^2) + eps) per row; a and b are zero afterwards."""
    _cuda(dst, a, a_partials, b, b_partials, gain)
    lib, fn = _fn("branch", "sb_branch_norm_fold", [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_float, c_void_p, c_void_p, c_int, c_int64, c_float,
                                                    c_void_p, c_int, c_float, c_int, c_int, c_void_p])
    n, W = dst.shape
    pa, na, sa = _partials(a_partials)
    pb, nb, sb = _partials(b_partials)
    _check(lib, fn(_ptr(dst), _ptr(a), pa, na, sa, ca, _ptr(b), pb, nb, sb, cb, _ptr(gain), dtype_code(gain.dtype) if gain is not None else 0,
                   eps, n, W, _stream()))


def stream_add(dst: torch.Tensor, other=None, vector=None, partials=None) -> None:
    """dst[r, :] = ((dst[r, :] + sum of partials) + other[r, :]) + vector[:], float32 rows; `other`, `vector` and `partials` may be None."""
    _cuda(dst, other, vector, partials)
    lib, fn = _fn("branch", "sb_stream_add", [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    n, W = dst.shape
    p, P, stride = _partials(partials)
    _check(lib, fn(_ptr(dst), p, P, stride, _ptr(other), _ptr(vector), dtype_code(vector.dtype) if vector is not None else 0, n, W, _stream()))


def row_scaled_add(dst: torch.Tensor, x: torch.Tensor, weights: torch.Tensor, first: int, count: int) -> None:
    """dst[r, :] += (weights[r, first] + .. + weights[r, first + count - 1]) * x[r, :]."""
    _cuda(dst, x, weights)
    lib, fn = _fn("branch", "sb_row_scaled_add", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    n, W = dst.shape
    _check(lib, fn(_ptr(dst), _ptr(x), dtype_code(x.dtype), _ptr(weights), weights.stride(0), first, count, n, W, _stream()))


def polynorm(up: torch.Tensor, out: torch.Tensor, coefficients, eps: float) -> None:
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row of z = the sum of `up` [P, n, F]; N(y) = y / sqrt(mean(y^2) + eps)."""
    _cuda(up, out)
    lib, fn = _fn("feed_forward", "sb_polynorm", [c_void_p, c_int, c_int64, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float, c_float,
                                                   c_float, c_void_p])
    p, P, stride = _partials(up)
    n, F = out.shape
    a, b, c, e = (float(v) for v in coefficients)
    _check(lib, fn(p, P, stride, _ptr(out), dtype_code(out.dtype), n, F, a, b, c, e, eps, _stream()))


def moe_route(logits: torch.Tensor, correction: torch.Tensor, weights: torch.Tensor, top: int, scale: float, biased: bool = False) -> None:
    """weights[r, x] = softmax(logits[r])[x] / (sum over the chosen + 1e-20) * scale for the `top` experts with the largest
    softmax + correction, 0 for the others. `biased`: the correction is the router's bias; the experts with the largest
    logits + bias are chosen and weigh by the softmax over those alone (times scale)."""
    _cuda(logits, correction, weights)
    lib, fn = _fn("feed_forward", "sb_moe_route", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p])
    n, X = weights.shape
    _check(lib, fn(_ptr(logits), logits.stride(0), _ptr(correction), dtype_code(correction.dtype), _ptr(weights), n, X, top, scale, int(biased),
                   _stream()))


def moe_activate(up: torch.Tensor, weights: torch.Tensor, out: torch.Tensor, experts: int, ff: int, gated: bool = False) -> None:
    """out[r, e ff + j] = weights[r, e] * relu(sum of up [P, n, E ff])^2; `gated`: weights[r, e] * silu(gate) * up with
    up [P, n, E 2 ff], an expert's ff gate rows in front of its ff up rows."""
    _cuda(up, weights, out)
    lib, fn = _fn("feed_forward", "sb_moe_activate", [c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                      c_void_p])
    p, P, stride = _partials(up)
    _check(lib, fn(p, P, stride, _ptr(weights), weights.stride(0), _ptr(out), dtype_code(out.dtype), out.shape[0], experts, ff, int(gated),
                   _stream()))


def qkv_rotate_append(qkv: torch.Tensor, positions, slots, cos_sin, rotary_dim: int, q_out, cache_layer, block_table, num_heads: int,
                      num_kv_heads: int, key_dim: int, value_dim: int, write_kv: bool = True) -> None:
    """Rotate q and k of `qkv` [P, n, Hq D + Hkv D + Hkv Dv] (partial sums added), store q, append k and v to the pages
    [pages, 2, Hkv, page_size, >= max(D, Dv)]."""
    _cuda(qkv, positions, slots, cos_sin, q_out, cache_layer, block_table)
    lib, fn = _fn("sigmoid_attention", "sb_qkv_rotate_append",
                  [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                   c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    p, P, stride = _partials(qkv)
    n = q_out.shape[0]
    _check(lib, fn(p, P, stride, _ptr(positions), _ptr(slots), _ptr(cos_sin), rotary_dim, _ptr(q_out), dtype_code(q_out.dtype), _ptr(cache_layer),
                   dtype_code(cache_layer.dtype), _ptr(block_table), block_table.shape[1], cache_layer.shape[3], cache_layer.stride(0),
                   cache_layer.stride(1), cache_layer.stride(2), n, num_heads, num_kv_heads, key_dim, value_dim, cache_layer.shape[4],
                   int(write_kv), _stream()))


def sigmoid_attention(q, out, cache_layer, block_table, positions, slots, bias, num_heads: int, num_kv_heads: int, key_dim: int,
                      value_dim: int, window: int, scale: float) -> None:
    """out[i] = sum over the visible keys j of sigmoid(scale q_i.k_j + bias[head]) v_j over the paged cache."""
    _cuda(q, out, cache_layer, block_table, positions, slots, bias)
    if not (q.dtype == out.dtype == cache_layer.dtype):
        raise TypeError("sigmoid_attention takes q, out and cache of one dtype")
    lib, fn = _fn("sigmoid_attention", "sb_sigmoid_attention",
                  [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), dtype_code(q.dtype), _ptr(cache_layer), _ptr(block_table), block_table.shape[1], cache_layer.shape[3],
                   cache_layer.stride(0), cache_layer.stride(1), cache_layer.stride(2), _ptr(positions), _ptr(slots), _ptr(bias), q.shape[0],
                   num_heads, num_kv_heads, key_dim, value_dim, cache_layer.shape[4], window, scale, _stream()))


def sigmoid_attention_tiles_supported(num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, row: int) -> bool:
    """True if the tensor-core form of the sigmoid attention takes this shape (bfloat16 only)."""
    lib = library("sigmoid_attention")
    lib.sb_sigmoid_attention_tiles_supported.argtypes = [c_int] * 5
    lib.sb_sigmoid_attention_tiles_supported.restype = c_int
    return bool(lib.sb_sigmoid_attention_tiles_supported(num_heads, num_kv_heads, key_dim, value_dim, row))


def sigmoid_attention_tiles(q, out, cache_layer, block_table, entry_meta, entries: int, bias, num_heads: int, num_kv_heads: int, key_dim: int,
                            value_dim: int, window: int, scale: float) -> None:
    """`sigmoid_attention` on the tensor cores (bfloat16 q, out and cache), entry by entry of the step."""
    _cuda(q, out, cache_layer, block_table, entry_meta, bias)
    if not (q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16):
        raise TypeError("sigmoid_attention_tiles takes bfloat16 q, out and cache")
    lib, fn = _fn("sigmoid_attention", "sb_sigmoid_attention_tiles",
                  [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_int, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), _ptr(cache_layer), _ptr(block_table), block_table.shape[1], cache_layer.shape[3], cache_layer.stride(0),
                   cache_layer.stride(1), cache_layer.stride(2), _ptr(entry_meta), entry_meta.stride(0), entries, _ptr(bias), q.shape[0],
                   num_heads, num_kv_heads, key_dim, value_dim, cache_layer.shape[4], window, scale, _stream()))


def hgrn2_activate(proj: torch.Tensor, f_bias, lower, act: torch.Tensor, HD: int, HV: int) -> None:
    """act [n, 3 HD + HV] = q | g | k | v from the sums of proj [P, n, 2 HD + HV] = q | f | v: q = silu, g = lower + (1 - lower) sigmoid(f + bias),
    k = 1 - g, v as projected."""
    _cuda(proj, f_bias, lower, act)
    if f_bias.dtype != lower.dtype:
        raise TypeError("hgrn2_activate takes the gate's bias and lower bound in one dtype")
    lib, fn = _fn("gated_recurrence", "sb_hgrn2_activate", [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    p, P, stride = _partials(proj)
    _check(lib, fn(p, P, stride, _ptr(f_bias), _ptr(lower), dtype_code(lower.dtype), _ptr(act), act.shape[0], HD, HV, _stream()))


def gated_scan(act: torch.Tensor, q_off: int, g_off: int, k_off: int, v_off: int, entry_meta: torch.Tensor, entries: int, state: torch.Tensor,
               out: torch.Tensor, heads: int, key_dim: int, value_dim: int) -> None:
    """S <- diag(g) S + k v^T, o = S^T q for every entry of the step, token by token; state [slots, heads, key_dim, value_dim] float32."""
    _cuda(act, entry_meta, state, out)
    lib, fn = _fn("gated_recurrence", "sb_gated_scan", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                         c_int, c_int, c_int, c_void_p])
    _check(lib, fn(_ptr(act), act.stride(0), q_off, g_off, k_off, v_off, _ptr(entry_meta), entry_meta.stride(0), entries, _ptr(state), _ptr(out),
                   heads, key_dim, value_dim, _stream()))


def group_rmsnorm(o: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor, heads: int, value_dim: int) -> None:
    """Every head's value_dim outputs RMS-normed on their own, times gain [value_dim]."""
    _cuda(o, gain, out)
    lib, fn = _fn("gated_recurrence", "sb_group_rmsnorm", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(o), _ptr(gain), dtype_code(gain.dtype), _ptr(out), dtype_code(out.dtype), o.shape[0], heads, value_dim, eps, _stream()))


def rglru_conv(proj: torch.Tensor, x_bias, taps, conv_bias, positions, slots, state: torch.Tensor, u: torch.Tensor) -> None:
    """u = causal convolution per channel of x = (columns C.. of the sums of proj [P, n, 2 C]) + x_bias; taps [C, K], the last one on
    the token itself; earlier inputs from the step's rows or from state [slots, K, C]."""
    _cuda(proj, x_bias, taps, conv_bias, positions, slots, state, u)
    lib, fn = _fn("rglru", "sb_rglru_conv", [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int, c_int, c_int, c_void_p])
    p, P, stride = _partials(proj)
    n, C = u.shape
    _check(lib, fn(p, P, stride, _ptr(x_bias), _ptr(taps), _ptr(conv_bias), dtype_code(taps.dtype), _ptr(positions), _ptr(slots), _ptr(state),
                   _ptr(u), n, C, taps.shape[1], _stream()))


def rglru_gates(gate_weights: torch.Tensor, r_bias, i_bias, lam, y_bias, u, proj, a, d, y) -> None:
    """a = exp(-8 sigmoid(A_b u_b + r_bias) softplus(lam)), d = sqrt(1 - a^2) sigmoid(I_b u_b + i_bias) u, y = gelu_tanh(proj_y + y_bias);
    gate_weights [blocks, bw, 2 bw]: per block of channels A_b and I_b side by side, transposed ([input, output])."""
    _cuda(gate_weights, r_bias, i_bias, lam, y_bias, u, proj, a, d, y)
    lib, fn = _fn("rglru", "sb_rglru_gates", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64,
                                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    p, P, stride = _partials(proj)
    n, C = u.shape
    _check(lib, fn(_ptr(gate_weights), dtype_code(gate_weights.dtype), _ptr(r_bias), _ptr(i_bias), _ptr(lam), _ptr(y_bias), dtype_code(lam.dtype),
                   _ptr(u), p, P, stride, _ptr(a), _ptr(d), _ptr(y), n, C, gate_weights.shape[0], _stream()))


def rglru_scan(a, d, y, proj, x_bias, entry_meta: torch.Tensor, entries: int, state: torch.Tensor, out: torch.Tensor, taps: int) -> None:
    """S <- a S + d token by token for every entry of the step, out = S * y; writes S and the convolution's last inputs back to state."""
    _cuda(a, d, y, proj, x_bias, entry_meta, state, out)
    lib, fn = _fn("rglru", "sb_rglru_scan", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p, c_int, c_int,
                                             c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    p, P, stride = _partials(proj)
    _check(lib, fn(_ptr(a), _ptr(d), _ptr(y), p, P, stride, _ptr(x_bias), dtype_code(x_bias.dtype), _ptr(entry_meta), entry_meta.stride(0), entries,
                   _ptr(state), _ptr(out), dtype_code(out.dtype), out.shape[1], taps, _stream()))


# ---------------------------------------------------------------------------------------------- csrc/masked_attention.cu
def _page_args(cache_layer, block_table):
    """(pages, block table, pages per sequence, page size, page stride, value offset, head stride) of a `[pages, planes, Hkv, page_size, Dc]`
    cache; with one plane the values lie in the key rows themselves (offset 0)."""
    v_offset = cache_layer.stride(1) if cache_layer.shape[1] > 1 else 0
    return [_ptr(cache_layer), _ptr(block_table), block_table.shape[1], cache_layer.shape[3], cache_layer.stride(0), v_offset, cache_layer.stride(2)]


def qkv_norm_append(qkv: torch.Tensor, bias, q_gain, k_gain, eps: float, positions, slots, q_out, cache_layer, block_table, num_heads: int,
                    num_kv_heads: int, key_dim: int, value_dim: int, write_kv: bool = True) -> None:
    """qkv [P, n, Hq D + Hkv D + Hkv Dv] partial sums, + bias; the whole query projection RMS-normed times q_gain [Hq D], the whole key
    projection times k_gain [Hkv D] (None: not normed); q stored, k and v appended to the pages. bias and gains float32."""
    _cuda(qkv, bias, q_gain, k_gain, positions, slots, q_out, cache_layer, block_table)
    lib, fn = _fn("masked_attention", "sb_qkv_norm_append",
                  [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                   c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    p, P, stride = _partials(qkv)
    if q_out.dtype != cache_layer.dtype:
        raise TypeError("qkv_norm_append takes q and cache of one dtype")
    _check(lib, fn(p, P, stride, _ptr(bias), _ptr(q_gain), _ptr(k_gain), eps, _ptr(positions), _ptr(slots), _ptr(q_out), dtype_code(q_out.dtype),
                   *_page_args(cache_layer, block_table), q_out.shape[0], num_heads, num_kv_heads, key_dim, value_dim, cache_layer.shape[4],
                   int(write_kv), _stream()))


def latent_prepare(proj: torch.Tensor, q_gain, kv_gain, eps: float, positions, slots, cos_sin, q_latent, cache_layer, block_table, q_rank: int,
                   kv_rank: int, rot: int, write_kv: bool = True) -> None:
    """proj [P, n, q_rank + kv_rank + rot] partial sums: both latents RMS-normed with their gains (float32), the query latent stored, the
    key/value latent and the rotated last `rot` elements appended as one row [kv_rank | rot] of the token's page (one plane, one head)."""
    _cuda(proj, q_gain, kv_gain, positions, slots, cos_sin, q_latent, cache_layer, block_table)
    lib, fn = _fn("masked_attention", "sb_latent_prepare",
                  [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                   c_int, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    p, P, stride = _partials(proj)
    if q_latent.dtype != cache_layer.dtype:
        raise TypeError("latent_prepare takes the query latent and the cache of one dtype")
    _check(lib, fn(p, P, stride, _ptr(q_gain), _ptr(kv_gain), eps, _ptr(positions), _ptr(slots), _ptr(cos_sin), _ptr(q_latent),
                   dtype_code(q_latent.dtype), _ptr(cache_layer), _ptr(block_table), block_table.shape[1], cache_layer.shape[3], cache_layer.stride(0),
                   q_latent.shape[0], q_rank, kv_rank, rot, cache_layer.shape[4], int(write_kv), _stream()))


def rotate_heads(q: torch.Tensor, positions, cos_sin, out: torch.Tensor, num_heads: int, head_dim: int, offset: int, rot: int) -> None:
    """q [P, n, H D] partial sums -> out [n, H D]: elements offset .. offset + rot - 1 of every head rotated (pairs d, d + rot / 2)."""
    _cuda(q, positions, cos_sin, out)
    lib, fn = _fn("masked_attention", "sb_rotate_heads", [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                          c_int, c_void_p])
    p, P, stride = _partials(q)
    _check(lib, fn(p, P, stride, _ptr(positions), _ptr(cos_sin), _ptr(out), dtype_code(out.dtype), out.shape[0], num_heads, head_dim, offset, rot,
                   _stream()))


def masked_attention(q, out, cache_layer, block_table, positions, slots, slopes, sinks, num_heads: int, num_kv_heads: int, key_dim: int,
                     value_dim: int, window: int, keep_first: int, scale: float) -> None:
    """Softmax attention over the paged cache: score = scale q_i.k_j - slopes[h] (i - j); i sees j <= i with i - j < window or j < keep_first
    (window 0: all); the denominator also holds exp(sinks[h]). slopes and sinks: float32 [H] or None."""
    _cuda(q, out, cache_layer, block_table, positions, slots, slopes, sinks)
    if not (q.dtype == out.dtype == cache_layer.dtype):
        raise TypeError("masked_attention takes q, out and cache of one dtype")
    lib, fn = _fn("masked_attention", "sb_masked_attention",
                  [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), dtype_code(q.dtype), *_page_args(cache_layer, block_table), _ptr(positions), _ptr(slots), _ptr(slopes),
                   _ptr(sinks), q.shape[0], num_heads, num_kv_heads, key_dim, value_dim, cache_layer.shape[4], window, keep_first, scale, _stream()))


def masked_attention_tiles_supported(num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, row: int, v_offset: int) -> bool:
    """True if the tensor-core form of the masked attention takes this shape (bfloat16 only)."""
    lib = library("masked_attention")
    lib.sb_masked_attention_tiles_supported.argtypes = [c_int] * 5 + [c_int64]
    lib.sb_masked_attention_tiles_supported.restype = c_int
    return bool(lib.sb_masked_attention_tiles_supported(num_heads, num_kv_heads, key_dim, value_dim, row, v_offset))


def masked_attention_tiles(q, out, cache_layer, block_table, entry_meta, entries: int, slopes, sinks, num_heads: int, num_kv_heads: int,
                           key_dim: int, value_dim: int, window: int, keep_first: int, scale: float) -> None:
    """`masked_attention` on the tensor cores (bfloat16 q, out and cache), entry by entry of the step."""
    _cuda(q, out, cache_layer, block_table, entry_meta, slopes, sinks)
    if not (q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16):
        raise TypeError("masked_attention_tiles takes bfloat16 q, out and cache")
    lib, fn = _fn("masked_attention", "sb_masked_attention_tiles",
                  [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_int, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), *_page_args(cache_layer, block_table), _ptr(entry_meta), entry_meta.stride(0), entries, _ptr(slopes),
                   _ptr(sinks), q.shape[0], num_heads, num_kv_heads, key_dim, value_dim, cache_layer.shape[4], window, keep_first, scale, _stream()))


def head_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, tail: int = 0) -> None:
    """out[r, h, :N] = weight[h]^T x[r, h, :K] (weight [H, K, N]); the `tail` elements of x behind the K are copied behind the N of out.
    x [n, H, >= K + tail] and out [n, H, >= N + tail] may be views with any row and head strides; sums in 32-bit."""
    _cuda(x, weight, out)
    if not (x.dtype == weight.dtype == out.dtype):
        raise TypeError("head_linear takes input, weights and output of one dtype")
    H, K, N = weight.shape
    if x.shape[1] != H or out.shape[1] != H or x.shape[2] < K + tail or out.shape[2] < N + tail or x.stride(2) != 1 or out.stride(2) != 1:
        raise ValueError(f"head_linear: {tuple(x.shape)} -> {tuple(out.shape)} through {tuple(weight.shape)} with a tail of {tail}")
    lib, fn = _fn("masked_attention", "sb_head_linear", [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int,
                                                         c_int, c_int, c_int, c_void_p])
    _check(lib, fn(_ptr(x), x.stride(0), x.stride(1), _ptr(weight), _ptr(out), out.stride(0), out.stride(1), dtype_code(x.dtype), x.shape[0], H, K, N,
                   tail, _stream()))
