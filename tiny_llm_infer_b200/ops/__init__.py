"""Python face of the hand-written CUDA kernels (``csrc/*.cu``) and of the library matrix
product.  Every function here works on CUDA tensors on the current stream and has no
other implementation: if the kernel library cannot be built or loaded, the first call
raises ``KernelLibraryError``.

The matrix product (``linear``, ``linear_swiglu``) has two kernels of this package for
bfloat16, chosen by the number of rows: up to 8 the weight-streaming mma.sync product
(``gemm_skinny``), from 256 on, where the tiles fill the GPU, the TMA + tcgen05 product
(``gemm_tcgen05``).  Everything else is the library's (cuBLAS through ``torch.mm``), as in the reference, which calls
``cublasHgemm`` for every projection with more than one row
(kernels/src/matmul_kernel_cuda.cu:83-91); in float32 mode it runs with the
reduced-precision matrix modes switched off.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

# flags of qk_norm_rope_store (csrc/qk_rope_store.cu)
QK_NORM, QK_ROPE, QK_STORE, QK_QOUT, QK_KVOUT = 1, 2, 4, 8, 16


class KernelLibraryError(RuntimeError):
    pass


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    """The loaded kernel library (built on first use)."""
    global _lib
    if _lib is not None:
        return _lib
    try:
        path = _build.library_path()
    except Exception as exc:  # BuildError and anything the toolchain throws
        raise KernelLibraryError(f"the CUDA kernel library is not available: {exc}") from exc
    try:
        handle = ctypes.CDLL(str(path))
    except OSError as exc:
        raise KernelLibraryError(f"cannot load {path}: {exc}") from exc
    _declare(handle)
    _lib = handle
    return handle


def _declare(h) -> None:
    vp, i32, f32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    h.tllm_last_error.restype = ctypes.c_char_p
    h.tllm_last_error.argtypes = []
    sigs = {
        "tllm_embedding": [vp, vp, i32, vp, i32, i32, i32, f32, vp],
        "tllm_postnorm_add_rmsnorm": [vp, vp, vp, f32, vp, i32, f32, vp, i32, vp, i32, i32, vp],
        "tllm_qkv_unit_store": [vp, i32, vp, vp, f32, i32, vp, vp, vp, i32, i32, vp, vp, i64, vp, i32, i32,
                                i32, i32, i32, i32, i32, vp, i32, f32, i32, i32, vp, vp],
        "tllm_attention_biased_general": [vp, vp, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32,
                                          f32, f32, i32, i32, i32, vp, vp, vp, i32, i32, vp, i32, i32, vp, vp],
        "tllm_attention_biased_prefill": [vp, vp, vp, i64, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32,
                                          f32, f32, i32, i32, i32, vp, vp, vp, i32, i32, vp, i32, i32, vp, vp],
        "tllm_attention_biased_decode": [vp, vp, vp, i64, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32,
                                         f32, f32, i32, i32, i32, vp, vp, vp, i32, i32, vp, i32, i32, i32, vp, vp, vp],
        "tllm_scaled_add_layernorm": [vp, vp, vp, i32, vp, i32, f32, vp, i32, vp, i32, i32, vp],
        "tllm_linear_prepare": [vp, i32, i32, vp, i32, vp, i32, f32, vp, i32, i32, i32, f32, vp, vp, vp, vp, vp, vp,
                                i32, vp],
        "tllm_embedding_norm": [vp, vp, vp, vp, i32, vp, f32, f32, vp, i32, i32, i32, i32, vp],
        "tllm_softcap": [vp, f32, i64, vp],
        "tllm_stream_add": [vp, vp, vp, i32, f32, vp, i32, i32, i32, vp],
        "tllm_activation": [vp, vp, i32, i32, i32, i32, vp, vp, i32, i32, i32, vp],
        "tllm_delta_prepare": [vp, i32, i32, vp, vp, i32, vp, i32, vp, vp, vp, vp, i64, i32, i32, i32, i32, f32, f32,
                               vp, vp, vp, vp, vp, i32, i32, i32, vp],
        "tllm_delta_scan": [vp, i32, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, vp, i32, vp, i64, f32, vp, vp],
        "tllm_delta_finish": [vp, vp, i32, i32, vp, f32, vp, i32, i32, i32, i32, i32, vp, i32, vp, i32, i32, vp, i64,
                              vp, i32, i32, vp],
        "tllm_latent_norm_store": [vp, i32, i32, i32, i32, i32, i32, vp, vp, f32, vp, f32, vp, vp, vp, i32, i32,
                                   vp, i64, vp, i32, i32, i32, vp],
        "tllm_latent_query": [vp, i32, vp, i32, i32, i32, i32, i32, i32, vp, f32, vp, vp, i32, vp, i32, vp],
        "tllm_heads_gate": [vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp],
        "tllm_moe_route": [vp, i32, i32, i32, i32, vp, vp, vp],
        "tllm_moe_route_grouped": [vp, i32, i32, i32, i32, vp, i32, i32, vp, vp, vp],
        "tllm_moe_plan": [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp],
        "tllm_moe_grouped": [vp, i32, vp, vp, i32, vp, i64, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32,
                             i32, i32, i32, i32, vp, vp],
        "tllm_moe_gather": [vp, vp, vp, i32, vp, i32, i32, vp],
        "tllm_moe_combine": [vp, i32, vp, vp, i32, vp, vp, i32, i32, i32, vp, vp, i32, vp],
        "tllm_sum_rmsnorm": [vp, vp, vp, i32, f32, vp, vp, f32, vp, i32, i32, i32, vp],
        "tllm_ssd_prepare": [vp, i32, i32, vp, vp, vp, i32, vp, vp, vp, vp, i64, i64, i32, i32, i32, i32, vp, vp, vp,
                             vp, vp, i32, vp],
        "tllm_ssd_finish": [vp, vp, vp, i32, vp, i32, i32, vp, f32, i32, vp, i32, i32, i32, i32, vp, i64, i64, vp, vp],
        "tllm_gemm_tcgen05_grouped": [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, i32, vp, vp],
        "tllm_add_rmsnorm": [vp, vp, vp, i32, f32, vp, i32, vp, i32, i32, vp],
        "tllm_swiglu": [vp, vp, i32, i32, i32, i32, i32, vp],
        "tllm_cast": [vp, i32, vp, i32, i64, vp],
        "tllm_feed_tokens": [vp, vp, vp, vp, i32, vp],
        "tllm_qk_norm_rope_store": [vp, vp, vp, i32, f32, vp, i32, vp, vp, vp, i32, vp, i32, vp,
                                    i32, i32, i32, i32, i32, i32, vp, vp],
        "tllm_rope_table": [vp, vp, i32, i32, vp, vp],
        "tllm_paged_attention_general": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32,
                                         i32, f32, vp, vp],
        "tllm_sample": [vp, i32, i32, i64, vp, vp, vp, vp],
        "tllm_sample_split": [vp, i32, i32, i64, vp, vp, vp, vp, i32, vp, vp],
        "tllm_gemm_skinny": [vp, vp, vp, i32, i32, i32, i32, vp],
        "tllm_gemm_plain": [vp, i32, vp, i32, vp, i32, i32, i32, i32, vp],
        "tllm_gemm_tcgen05": [vp, vp, vp, i32, i32, i32, i32, vp, vp],
        "tllm_gemm_skinny_swiglu": [vp, vp, vp, i32, i32, i32, i32, vp],
        "tllm_gemm_skinny_act": [vp, vp, vp, i32, i32, i32, i32, vp],
        "tllm_paged_attention_decode": [vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32,
                                        i32, vp, vp, vp, vp],
        "tllm_paged_attention_prefill": [vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp],
        "tllm_paged_attention_prefill_tc": [vp, i32, vp, i32, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32,
                                            vp, i32, vp, vp, vp, vp],
        "tllm_attention_planes_prefill_tc": [vp, i32, vp, vp, ctypes.c_longlong, i32, vp, vp, i32, vp, i32, i32,
                                             i32, i32, i32, f32, vp, i32, vp, vp, i32, vp, vp, vp, vp],
    }
    for name, args in sigs.items():
        fn = getattr(h, name)
        fn.argtypes = args
        fn.restype = i32
    h.tllm_delta_rule_lanes.argtypes = [i32]
    h.tllm_delta_rule_lanes.restype = i32
    h.tllm_delta_rule_state_floats.argtypes = [i32, i32, i32, i32, i32]
    h.tllm_delta_rule_state_floats.restype = i64
    h.tllm_attention_biased_fast_ok.argtypes = [i32, i32, i32, i32]
    h.tllm_attention_biased_fast_ok.restype = i32
    h.tllm_moe_tile_rows.argtypes = []
    h.tllm_moe_tile_rows.restype = i32
    h.tllm_paged_attention_prefill_tc_rows.argtypes = [i32, i32]
    h.tllm_paged_attention_prefill_tc_rows.restype = i32
    h.tllm_sample_nucleus_scratch_bytes.argtypes = [i32]
    h.tllm_sample_nucleus_scratch_bytes.restype = i64
    h.tllm_uniform_of.argtypes = [ctypes.c_ulonglong, i32]
    h.tllm_uniform_of.restype = f32


launches = 0      # kernels of csrc/ launched so far (graph replays are added by the runner)


def _check(code: int, what: str, kernels: int = 1) -> None:
    global launches
    launches += kernels
    if code != 0:
        raise KernelError(f"{what}: {lib().tllm_last_error().decode(errors='replace')} (code {code})")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current CUDA stream of the current device (the raw getter costs a fraction
    of a microsecond, the Stream object several)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernels take contiguous CUDA tensors")


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}") from None


# --------------------------------------------------------------------------- ops
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[ids[t]] * scale as float32; rows with a negative id become zero."""
    _cuda(ids, table, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32
    vocab, hidden = table.shape
    _check(lib().tllm_embedding(_p(ids), _p(table), _dt(table), _p(out), ids.numel(), hidden, vocab,
                                float(scale), _stream()), "embedding")
    return out


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None,
                post_gain: Optional[torch.Tensor] = None, post_eps: float = 0.0) -> torch.Tensor:
    """h += delta (float32 sum, written back) and out = gain * h / sqrt(mean(h^2) + eps).
    With ``rows`` only those rows are normed, into out[0..len(rows)), and h is not written.
    With ``post_gain`` the delta is normed itself before it is added:
    h += post_gain * delta / sqrt(mean(delta^2) + post_eps), in float32 inside the same kernel."""
    _cuda(h, delta, gain, out, rows, post_gain)
    assert h.dtype == torch.float32
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape == h.shape
    n_out = out.shape[0] if rows is None else rows.numel()
    if post_gain is not None:
        assert delta is not None and post_gain.dtype == gain.dtype
        _check(lib().tllm_postnorm_add_rmsnorm(_p(h), _p(delta), _p(post_gain), float(post_eps), _p(gain), _dt(gain),
                                               float(eps), _p(out), _dt(out), _p(rows), n_out, h.shape[-1], _stream()),
               "postnorm_add_rmsnorm")
        return out
    _check(lib().tllm_add_rmsnorm(_p(h), _p(delta), _p(gain), _dt(gain), float(eps), _p(out), _dt(out),
                                  _p(rows), n_out, h.shape[-1], _stream()), "add_rmsnorm")
    return out


def scaled_add_layernorm(h: torch.Tensor, deltas, scales, gain: torch.Tensor, eps: float, out: torch.Tensor,
                         rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h += sum_i scales[i] * deltas[i] (float32, written back; ``scales[i]`` a float32 vector of the row's width,
    ``deltas[i]`` [T, width] in the storage type; at most four), then out = gain * (h - mean) / sqrt(mean of the
    squared deviations + eps).  With ``rows`` only those rows are normed, into out[0..len(rows)), and h is not
    written."""
    _cuda(h, gain, out, rows, *deltas, *scales)
    assert h.dtype == torch.float32 and len(deltas) == len(scales) <= 4
    for d, s in zip(deltas, scales):
        assert d.dtype == out.dtype and d.shape == h.shape and s.dtype == torch.float32 and s.numel() == h.shape[1]
    n = len(deltas)
    dp = (ctypes.c_void_p * 4)(*[d.data_ptr() for d in deltas])
    sp = (ctypes.c_void_p * 4)(*[s.data_ptr() for s in scales])
    n_out = out.shape[0] if rows is None else rows.numel()
    _check(lib().tllm_scaled_add_layernorm(_p(h), ctypes.cast(dp, ctypes.c_void_p), ctypes.cast(sp, ctypes.c_void_p), n,
                                           _p(gain), _dt(gain), float(eps), _p(out), _dt(out), _p(rows), n_out,
                                           h.shape[-1], _stream()), "scaled_add_layernorm")
    return out


def sum_rmsnorm(h: torch.Tensor, deltas, coefs, alpha: float, gain: torch.Tensor, eps: float, out: torch.Tensor,
                bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h <- gain * v / sqrt(mean(v^2) + eps) with v = alpha * h + sum_i coefs[i] * deltas[i] (+ bias), for every row:
    the norm of a weighted sum becomes the stream itself (float32); ``out`` receives the new stream in the storage
    type.  ``deltas[i]`` [T, width] in the storage type with one float each (at most four), ``gain`` and ``bias``
    float32 vectors."""
    _cuda(h, gain, out, bias, *deltas)
    assert h.dtype == torch.float32 and gain.dtype == torch.float32 and len(deltas) == len(coefs) <= 4
    assert out.shape == h.shape and gain.numel() == h.shape[1] and (bias is None or (bias.dtype == torch.float32 and bias.numel() == h.shape[1]))
    for d in deltas:
        assert d.dtype == out.dtype and d.shape == h.shape
    n = len(deltas)
    dp = (ctypes.c_void_p * 4)(*[d.data_ptr() for d in deltas])
    cp = (ctypes.c_float * 4)(*[float(c) for c in coefs])
    _check(lib().tllm_sum_rmsnorm(_p(h), ctypes.cast(dp, ctypes.c_void_p), ctypes.cast(cp, ctypes.c_void_p), n, float(alpha),
                                  _p(bias), _p(gain), float(eps), _p(out), _dt(out), h.shape[0], h.shape[1], _stream()),
           "sum_rmsnorm")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2 I, K] with the rows of ``gate`` and ``up`` ([I, K], I a multiple of 8) interleaved by
    eight: eight gate rows, the eight up rows that belong to them, and so on.  A block of the
    weight-streaming product and a tile of the tcgen05 product then read neighbouring rows and
    find a gate and its up in one accumulator, so SwiGLU fits their epilogues."""
    inter, k = gate.shape
    assert up.shape == gate.shape and inter % 8 == 0
    return torch.stack([gate.reshape(inter // 8, 8, k), up.reshape(inter // 8, 8, k)], dim=1).reshape(2 * inter, k)


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}      # codes of csrc/common.cuh (GateAct)


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False, act: str = "silu") -> torch.Tensor:
    """out[t, i] = act(gate) * up with gate = gate_up[t, i], up = gate_up[t, I + i], or, for columns
    interleaved by eight, gate = gate_up[t, 16 (i // 8) + i % 8] and up eight columns further.
    ``act``: ``silu`` or ``gelu_tanh``."""
    _cuda(gate_up, out)
    tokens, two_i = gate_up.shape
    assert out.shape == (tokens, two_i // 2) and out.dtype == gate_up.dtype
    _check(lib().tllm_swiglu(_p(gate_up), _p(out), _dt(out), tokens, two_i // 2, int(interleaved),
                             ACTIVATIONS[act], _stream()), "swiglu")
    return out


def cast(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _cuda(src)
    if src.dtype == dtype:
        return src
    dst = torch.empty_like(src, dtype=dtype)
    _check(lib().tllm_cast(_p(src), _dt(src), _p(dst), _dt(dst), src.numel(), _stream()), "cast")
    return dst


def feed_tokens(ids: torch.Tensor, places: torch.Tensor, rows: torch.Tensor, sampled: torch.Tensor) -> None:
    """ids[places[i]] = sampled[rows[i]] (all int32, on the device): the tokens that the step before
    is still sampling go into this step's token ids without passing through the host."""
    _cuda(ids, places, rows, sampled)
    assert ids.dtype == places.dtype == rows.dtype == sampled.dtype == torch.int32 and places.numel() == rows.numel()
    _check(lib().tllm_feed_tokens(_p(ids), _p(places), _p(rows), _p(sampled), places.numel(), _stream()), "feed_tokens")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[tokens, 2, half] float32: cosines and sines of position * inv_freq (the float32 product), made
    once per step and read by every layer's ``qk_norm_rope_store``."""
    _cuda(positions, inv_freq)
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32
    tokens, half = positions.numel(), inv_freq.numel()
    table = torch.empty((tokens, 2, half), dtype=torch.float32, device=positions.device)
    _check(lib().tllm_rope_table(_p(positions), _p(inv_freq), half, tokens, _p(table), _stream()), "rope_table")
    return table


def qk_norm_rope_store(qkv: torch.Tensor, q_gain, k_gain, eps: float, inv_freq, rotary_dim: int,
                       positions: torch.Tensor, token_slot: torch.Tensor, block_table, cache,
                       page_size: int, q_out, q_heads: int, kv_heads: int, head_dim: int,
                       flags: int, table: Optional[torch.Tensor] = None) -> None:
    """One pass over the fused q|k|v rows [T, (q_heads + 2 kv_heads) * head_dim]: per-head
    RMSNorm of q and k (QK_NORM), rotate-half rotation (QK_ROPE), write of k and v into
    their page (QK_STORE), write of q to ``q_out`` (QK_QOUT), write of the processed k back
    in place (QK_KVOUT).  Rows whose token_slot is negative are skipped.  ``table``: the step's
    ``rope_table`` for these positions and frequencies (same values, no sincosf per layer)."""
    _cuda(qkv, q_gain, k_gain, inv_freq, positions, token_slot, block_table, cache, q_out, table)
    if table is not None:
        assert table.dtype == torch.float32 and tuple(table.shape) == (qkv.shape[0], 2, rotary_dim // 2)
    tokens = qkv.shape[0]
    assert qkv.shape[1] == (q_heads + 2 * kv_heads) * head_dim
    gain_dt = _dt(q_gain) if q_gain is not None else F32
    max_pages = block_table.shape[1] if block_table is not None else 0
    if cache is not None:
        assert cache.dtype == qkv.dtype and tuple(cache.shape[1:]) == (2, kv_heads, page_size, head_dim)
    _check(lib().tllm_qk_norm_rope_store(
        _p(qkv), _p(q_gain), _p(k_gain), gain_dt, float(eps), _p(inv_freq), rotary_dim,
        _p(positions), _p(token_slot), _p(block_table), max_pages, _p(cache), page_size, _p(q_out),
        _dt(qkv), tokens, q_heads, kv_heads, head_dim, flags, _p(table), _stream()), "qk_norm_rope_store")


_workspaces = {}


WORKSPACE_FLOATS = 16 << 20


def workspace(device, floats: int) -> torch.Tensor:
    """Float32 scratch for one call.  Up to WORKSPACE_FLOATS it is one buffer per device
    that lives as long as the process and never moves (captured CUDA graphs keep its
    address); a larger request gets a tensor of its own."""
    if floats > WORKSPACE_FLOATS:
        return torch.empty(floats, dtype=torch.float32, device=device)
    key = str(device)
    buf = _workspaces.get(key)
    if buf is None:
        buf = torch.empty(WORKSPACE_FLOATS, dtype=torch.float32, device=device)
        _workspaces[key] = buf
    return buf


SM_COUNT = 148


def decode_splits(rows: int, kv_heads: int, max_context: int) -> int:
    """How many blocks share the keys of one (row, key/value head): enough blocks for
    about four per multiprocessor, each with at least 128 keys."""
    by_length = -(-max_context // 1024)                       # about a thousand keys per block
    by_count = -(-128 // max(rows * kv_heads, 1))             # but at least 128 blocks in all
    return max(1, min(max(by_length, by_count), -(-max_context // 128), 64))


def fast_attention_ok(dtype, page_size: int, q_heads: int, kv_heads: int, head_dim: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0
            and q_heads % kv_heads == 0 and q_heads // kv_heads <= 16)


def paged_attention_decode(q, cache, positions, token_slot, rows, n_rows, block_table, page_size,
                           q_heads, kv_heads, head_dim, window, scale, out, max_context, splits=None):
    """Attention of one-token rows (``rows``: their indices, None for all), keys split over
    ``splits`` blocks per (row, key/value head); the splits' partial results go through scratch
    in global memory to a second small kernel that combines them in the order of the splits."""
    _cuda(q, cache, positions, token_slot, rows, block_table, out)
    if splits is None:
        splits = decode_splits(n_rows, kv_heads, max_context)
    part_o = part_ml = None
    if splits > 1:
        n = n_rows * q_heads * splits
        ws = workspace(q.device, n * (head_dim + 2))
        part_o, part_ml = ws[:n * head_dim], ws[n * head_dim:n * (head_dim + 2)]
    _check(lib().tllm_paged_attention_decode(
        _p(q), _p(cache), _p(positions), _p(token_slot), _p(rows), n_rows, _p(block_table),
        block_table.shape[1], page_size, q_heads, kv_heads, head_dim, int(window or 0), float(scale),
        splits, _p(part_o), _p(part_ml), _p(out), _stream()), "paged_attention_decode",
        kernels=2 if splits > 1 else 1)
    return out


def paged_attention_prefill(q, cache, seg_info, tiles, n_tiles, block_table, page_size, q_heads,
                            kv_heads, head_dim, window, scale, out):
    """Attention of the segments' query blocks listed in ``tiles`` ([n, 2] = segment, offset)."""
    _cuda(q, cache, seg_info, tiles, block_table, out)
    _check(lib().tllm_paged_attention_prefill(
        _p(q), _p(cache), _p(seg_info), _p(tiles), n_tiles, _p(block_table), block_table.shape[1],
        page_size, q_heads, kv_heads, head_dim, int(window or 0), float(scale), _p(out), _stream()),
        "paged_attention_prefill")
    return out


PREFILL_TCGEN05 = True     # head width 128 takes the tcgen05 kernel; False keeps the mma.sync one


def prefill_tcgen05_block_rows(q_heads: int, kv_heads: int) -> int:
    """Query rows per entry of the tile list that ``paged_attention_prefill_tcgen05`` wants: 128
    where two heads of one key/value head share a thread block (an even group), else 256."""
    return int(lib().tllm_paged_attention_prefill_tc_rows(q_heads, kv_heads))


def prefill_splits(blocks: int, max_context: int) -> int:
    """Runs of keys per block of query rows in ``paged_attention_prefill_tcgen05``: 1, 2, 4 or 8.
    A step with few query rows (a short portion of a prompt) has few blocks, each walking all keys
    of its request; cutting the keys fills the GPU (148 SMs, one block each), as long as a run
    keeps eight tiles of 64 keys, below which a block's start and end outweigh its work."""
    fit = min(SM_COUNT // max(blocks, 1), -(-max_context // 64) // 8)
    splits = 1
    while splits * 2 <= min(fit, 8):
        splits *= 2
    return splits



def paged_attention_prefill_tcgen05(q, cache, seg_info, tiles, n_tiles, block_table, page_size, q_heads,
                                    kv_heads, head_dim, window, scale, out, splits=1):
    """As ``paged_attention_prefill`` on tcgen05 tensor cores with TMA loads: bfloat16, head width
    128, ``tiles`` at multiples of ``prefill_tcgen05_block_rows`` rows.  With ``splits`` > 1 every
    block's keys are shared by that many blocks and a second kernel combines what they leave.
    The kernel's waits are bounded; what they report is read by ``check_error_word``."""
    _cuda(q, cache, seg_info, tiles, block_table, out)
    assert q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.shape[1] == q_heads * head_dim and tuple(out.shape) == tuple(q.shape)
    global tcgen05_calls
    tcgen05_calls += 1
    part_o = part_ml = None
    if splits > 1:
        n = q.shape[0] * q_heads * splits
        ws = workspace(q.device, n * (head_dim + 2))
        part_o, part_ml = ws[:n * head_dim], ws[n * head_dim:n * (head_dim + 2)]
    _check(lib().tllm_paged_attention_prefill_tc(
        _p(q), q.shape[0], _p(cache), cache.shape[0], _p(seg_info), _p(tiles), n_tiles, _p(block_table),
        block_table.shape[1], page_size, q_heads, kv_heads, head_dim, int(window or 0), float(scale),
        _p(out), splits, _p(part_o), _p(part_ml), _p(error_word(q.device)), _stream()), "paged_attention_prefill_tc",
        kernels=2 if splits > 1 else 1)
    return out


def paged_attention(q: torch.Tensor, cache: torch.Tensor, positions, token_slot, block_table,
                    page_size: int, q_heads: int, kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float, out: torch.Tensor, ctx=None) -> torch.Tensor:
    """Attention of every row of ``q`` over the keys of its own request in the paged cache:
    positions max(0, pos - window + 1) .. pos.  With the step's context and a shape the
    tensor-core kernels take (bfloat16, head width 64 or 128, pages of a multiple of 16),
    one-token rows go to the split-key decode kernel and longer segments to the tiled
    prefill kernel; everything else runs the general kernel."""
    _cuda(q, cache, positions, token_slot, block_table, out)
    tokens = q.shape[0]
    assert tuple(cache.shape[1:]) == (2, kv_heads, page_size, head_dim) and cache.dtype == q.dtype
    if ctx is not None and ctx.pf_tiles is not None and ctx.tokens == tokens \
            and fast_attention_ok(q.dtype, page_size, q_heads, kv_heads, head_dim):
        if ctx.n_dec:
            paged_attention_decode(q, cache, positions, token_slot, ctx.dec_rows, ctx.n_dec, block_table,
                                   page_size, q_heads, kv_heads, head_dim, window, scale, out,
                                   ctx.max_context)
        if ctx.n_tiles:
            if PREFILL_TCGEN05 and head_dim == 128 and getattr(ctx, "n_tiles256", 0):
                pairs = prefill_tcgen05_block_rows(q_heads, kv_heads) == 128
                blocks = ctx.n_tiles128 if pairs else ctx.n_tiles256
                keys = ctx.max_context if not window else min(ctx.max_context, window + 256)
                splits = prefill_splits(blocks * (q_heads // 2 if pairs else q_heads), keys)
                paged_attention_prefill_tcgen05(q, cache, ctx.seg_info, ctx.pf_tiles, blocks,
                                                block_table, page_size, q_heads, kv_heads, head_dim,
                                                window, scale, out, splits)
            else:
                paged_attention_prefill(q, cache, ctx.seg_info, ctx.pf_tiles, ctx.n_tiles, block_table,
                                        page_size, q_heads, kv_heads, head_dim, window, scale, out)
        return out
    _check(lib().tllm_paged_attention_general(
        _p(q), _p(cache), _p(positions), _p(token_slot), _p(block_table), block_table.shape[1],
        page_size, _dt(q), tokens, q_heads, kv_heads, head_dim, int(window or 0), float(scale),
        _p(out), _stream()), "paged_attention")
    return out


SAMPLE_BLOCKS = 1024     # blocks over all rows beyond which a row's vocabulary is cut less finely


def sample(logits: torch.Tensor, params: torch.Tensor, seeds: torch.Tensor,
           out: torch.Tensor, any_nucleus: Optional[bool] = None) -> torch.Tensor:
    """Token per row of float32 ``logits`` [S, V]: params[s] = (temperature, top_p), seeds[s]
    an int64 key.  temperature <= 1e-6 is argmax (lowest id on ties).  ``any_nucleus`` says
    whether some row samples with top_p < 1 (None: not known, assume so)."""
    _cuda(logits, params, seeds, out)
    assert logits.dtype == torch.float32 and params.dtype == torch.float32
    assert seeds.dtype == torch.int64 and out.dtype == torch.int32
    rows, vocab = logits.shape
    if vocab >= 4096 and rows > 0:
        # a row's vocabulary shared by several blocks; rows with top-p take four more passes
        blocks = min(64, -(-vocab // 2048), max(8, SAMPLE_BLOCKS // rows))
        partial = torch.empty((rows, blocks, 2), dtype=torch.float32, device=logits.device)
        scratch = None
        if any_nucleus is None or any_nucleus:
            size = lib().tllm_sample_nucleus_scratch_bytes(rows)
            scratch = torch.empty(size // 8, dtype=torch.int64, device=logits.device)
        _check(lib().tllm_sample_split(_p(logits), rows, vocab, logits.stride(0), _p(params), _p(seeds),
                                       _p(out), _p(partial), blocks, _p(scratch), _stream()), "sample",
               kernels=2 if scratch is None else 7)
        return out
    _check(lib().tllm_sample(_p(logits), rows, vocab, logits.stride(0), _p(params), _p(seeds),
                             _p(out), _stream()), "sample")
    return out


def uniform_of(seed: int, token: int) -> float:
    """The uniform number the sampler draws for (seed, token); for host-side checks."""
    return float(lib().tllm_uniform_of(seed & 0xFFFFFFFFFFFFFFFF, token))


SKINNY_MAX_ROWS = 8       # up to this many rows the weight-streaming product beats the library


def gemm_skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """y = x . weight^T for at most 32 bfloat16 rows: every weight is read once, straight from
    HBM into tensor-core fragments (csrc/gemm_skinny.cu)."""
    _cuda(x, weight)
    rows, k = x.shape
    n = weight.shape[0]
    assert weight.shape[1] == k and x.dtype == weight.dtype == torch.bfloat16
    y = torch.empty((rows, n), dtype=out_dtype, device=x.device)
    _check(lib().tllm_gemm_skinny(_p(x), _p(weight), _p(y), _DT[out_dtype], rows, n, k, _stream()),
           "gemm_skinny")
    return y


def gemm_plain(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """y = x . weight^T by the plain kernel (csrc/gemm_plain.cu): one thread per output, the sum over
    k in order in float32, any sizes, bfloat16 or float32 operands.  Slow; it is what the fast products
    are checked against at sizes too large for the host."""
    _cuda(x, weight)
    rows, k = x.shape
    n = weight.shape[0]
    assert weight.shape[1] == k
    y = torch.empty((rows, n), dtype=out_dtype, device=x.device)
    _check(lib().tllm_gemm_plain(_p(x), _dt(x), _p(weight), _dt(weight), _p(y), _dt(y), rows, n, k, _stream()), "gemm_plain")
    return y


_error_words = {}


def error_word(device) -> torch.Tensor:
    """Device int32 that kernels with bounded waits (the tcgen05 product) set to a non-zero
    code when a wait ran out.  ``check_error_word`` reads it (a synchronisation)."""
    key = str(device)
    if key not in _error_words:
        _error_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_words[key]


def check_error_word(device) -> None:
    code = int(error_word(device).item())
    if code:
        error_word(device).zero_()
        raise KernelError(f"a bounded wait ran out inside a kernel (code {code}); its result is invalid")


tcgen05_calls = 0          # products issued on the tcgen05 path (their bounded waits report to error_word)


def tcgen05_pays(rows: int, out_cols: int, k: int, dtype, col_tile: int = 256) -> bool:
    """Whether the hand-written tcgen05 product is used instead of the library's: bfloat16, at
    least 256 rows, and a tile count that fills the SMs' last round to 85% (blocks of 256 rows;
    with fewer tiles per round the library's 2-CTA kernels are faster)."""
    if dtype != torch.bfloat16 or rows < 256 or k % 8 or out_cols % 8:
        return False
    tiles = -(-rows // 256) * -(-out_cols // col_tile)
    rounds = -(-tiles // SM_COUNT)
    return tiles / (rounds * SM_COUNT) >= 0.85


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, swiglu: bool = False, short_tiles: bool = False,
                 interleaved: bool = False, act: str = "silu", unary: bool = False) -> torch.Tensor:
    """y = x . weight^T on tcgen05 tensor cores fed by TMA (csrc/gemm_tcgen05.cu), bfloat16 in
    and out, float32 accumulation in tensor memory.  With ``swiglu`` the weight is [gate; up]
    (or, ``interleaved``, gate and up rows interleaved by eight) and the result is
    silu(x . gate^T) * (x . up^T), [rows, weight rows / 2].  ``short_tiles`` keeps blocks of 128
    rows even when there are more (for measurements)."""
    _cuda(x, weight)
    rows, k = x.shape
    n = weight.shape[0]
    assert weight.shape[1] == k and x.dtype == weight.dtype == torch.bfloat16
    y = torch.empty((rows, n // 2 if swiglu else n), dtype=torch.bfloat16, device=x.device)
    if rows == 0:
        return y
    global tcgen05_calls
    tcgen05_calls += 1
    _check(lib().tllm_gemm_tcgen05(_p(x), _p(weight), _p(y), rows, n, k, int(swiglu) | (2 if short_tiles else 0) | (4 if interleaved else 0) | (16 if unary else 0)
                                   | (ELEMENTWISE_ACTIVATIONS[act] << 8 if (swiglu or unary) else 0),
                                   _p(error_word(x.device)), _stream()), "gemm_tcgen05")
    return y


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[T, N] = x[T, K] . weight[N, K]^T with float32 accumulation.  A weight kept in
    float32 is multiplied in float32 whatever the activations are stored in.  ``bias`` [N] (the weight's type) is
    added in the library product's epilogue."""
    if not x.is_cuda:
        raise KernelError("linear takes CUDA tensors")
    want = out_dtype or x.dtype
    if bias is not None:
        if weight.dtype == torch.float32 and (torch.backends.cuda.matmul.allow_tf32 or torch.get_float32_matmul_precision() != "highest"):
            raise KernelError("float32 products need the reduced-precision matrix modes off")
        y = torch.addmm(bias.to(weight.dtype), cast(x, weight.dtype), weight.t())
        return y if want == y.dtype else cast(y, want)
    if weight.dtype == torch.float32:
        if torch.backends.cuda.matmul.allow_tf32 or torch.get_float32_matmul_precision() != "highest":
            raise KernelError("float32 products need the reduced-precision matrix modes off")
        y = torch.mm(cast(x, torch.float32), weight.t())
        return y if want == torch.float32 else cast(y, want)
    if x.dtype != weight.dtype:
        x = cast(x, weight.dtype)
    rows, k = x.shape
    if weight.dtype == torch.bfloat16 and 0 < rows <= SKINNY_MAX_ROWS and k % 8 == 0 \
            and x.is_contiguous() and weight.is_contiguous() and want in _DT:
        return gemm_skinny(x, weight, want)
    if want == torch.bfloat16 and tcgen05_pays(rows, weight.shape[0], k, weight.dtype) \
            and x.is_contiguous() and weight.is_contiguous():
        return gemm_tcgen05(x, weight)
    if want == weight.dtype:
        return torch.mm(x, weight.t())
    return torch.mm(x, weight.t(), out_dtype=want)


def gemm_skinny_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for at most 16 bfloat16 rows as one weight-streaming kernel;
    ``w_gate_up`` holds the rows of Wg and Wu interleaved by eight (``interleave_gate_up``)."""
    _cuda(x, w_gate_up)
    rows, k = x.shape
    inter = w_gate_up.shape[0] // 2
    out = torch.empty((rows, inter), dtype=torch.bfloat16, device=x.device)
    _check(lib().tllm_gemm_skinny_swiglu(_p(x), _p(w_gate_up), _p(out), rows, inter, k, ACTIVATIONS[act], _stream()),
           "gemm_skinny_swiglu")
    return out


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out_dtype: torch.dtype,
                  interleaved: bool = False, act: str = "silu") -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for w_gate_up = [Wg; Wu], or with the rows of Wg and Wu
    interleaved by eight (``interleave_gate_up``).  With enough bfloat16 rows the product and the
    activation are one tcgen05 kernel, with few rows and interleaved weights one weight-streaming
    kernel; otherwise the product is followed by the SwiGLU kernel."""
    rows, k = x.shape
    inter = w_gate_up.shape[0] // 2
    plain = x.dtype == w_gate_up.dtype == out_dtype == torch.bfloat16 and x.is_contiguous() \
        and w_gate_up.is_contiguous()
    if plain and tcgen05_pays(rows, inter, k, w_gate_up.dtype, col_tile=128):
        return gemm_tcgen05(x, w_gate_up, swiglu=True, interleaved=interleaved, act=act)
    if plain and interleaved and 0 < rows <= SKINNY_MAX_ROWS and k % 8 == 0:
        return gemm_skinny_swiglu(x, w_gate_up, act)
    gate_up = linear(x, w_gate_up, out_dtype=out_dtype)
    out = torch.empty((rows, inter), dtype=out_dtype, device=x.device)
    return swiglu(gate_up, out, interleaved, act)


# --------------------------------------------------------------------------- attention with a modified score
def _plane(plane: torch.Tensor):
    """(pointer, elements from one page to the next) of a cache plane [pages, heads, page, width]: a
    view into the pages whose last three axes are dense."""
    heads, page, width = plane.shape[1:]
    assert plane.stride(3) == 1 and plane.stride(2) == width and plane.stride(1) == page * width
    return plane.data_ptr(), plane.stride(0)


BIASED_FAST = True       # False: every row takes the general kernel (for comparisons)


def biased_decode_splits(rows: int, kv_heads: int, reach: int) -> int:
    """Runs of keys per (row, key/value head) of ``attention_biased``'s one-token kernel: enough blocks
    for two per multiprocessor, each run with at least 256 keys of the ``reach`` a row can see."""
    want = -(-2 * SM_COUNT // max(rows * kv_heads, 1))
    return max(1, min(want, reach // 256, 64))


def qkv_unit_store(proj: torch.Tensor, q_out: torch.Tensor, positions, token_slot, block_table,
                   k_plane: Optional[torch.Tensor], v_plane: Optional[torch.Tensor], page_size: int,
                   q_heads: int, kv_heads: int, dk: int, dv: int, eps: Optional[float],
                   q_gain: Optional[torch.Tensor] = None, k_gain: Optional[torch.Tensor] = None,
                   store: bool = True, inv_freq: Optional[torch.Tensor] = None, rot_dims: int = 0,
                   q_temperature=None, values_are_keys: bool = False, bias: Optional[torch.Tensor] = None) -> None:
    """Rows of ``proj`` = q heads | k heads | v heads | anything: queries and keys divided per head by
    their root mean square (``eps`` None: left as they are; gains optional), queries to ``q_out``,
    keys and values of every row into their planes of the paged cache (``store``).  Keys have width
    ``dk``, values ``dv``.  Rows with a negative slot are skipped.  ``inv_freq`` [rot_dims / 2] float32: the first
    ``rot_dims`` elements of every query and key head turn by position * inv_freq (pairs half the rotated width
    apart), after the norm.  ``q_temperature`` (coef, every): queries times 1 + coef ln(floor((pos + 1) / every) + 1).
    ``values_are_keys``: the rows carry no values; a value is its key as projected, before the norm (dv = dk).
    ``bias`` float32, one number per q | k | v column: added to the rows, in float32, before anything else."""
    _cuda(proj, q_out, positions, token_slot, block_table, q_gain, k_gain, inv_freq, bias)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == (q_heads + kv_heads) * dk + (0 if values_are_keys else kv_heads * dv)
    if inv_freq is not None:
        assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2
    if q_gain is not None:
        assert q_gain.dtype == k_gain.dtype == proj.dtype
    coef, every = q_temperature if q_temperature is not None else (0.0, 0)
    assert q_out.dtype == proj.dtype and tuple(q_out.shape) == (proj.shape[0], q_heads * dk)
    kp = vp = None
    stride = 0
    if store:
        assert k_plane.dtype == v_plane.dtype == proj.dtype
        assert tuple(k_plane.shape[1:]) == (kv_heads, page_size, dk) and tuple(v_plane.shape[1:]) == (kv_heads, page_size, dv)
        (kp, stride), (vp, stride_v) = _plane(k_plane), _plane(v_plane)
        assert stride == stride_v
    _check(lib().tllm_qkv_unit_store(
        _p(proj), proj.shape[1], _p(q_gain), _p(k_gain), float(eps or 1.0), int(eps is not None), _p(positions),
        _p(token_slot), _p(block_table), block_table.shape[1] if block_table is not None else 0, page_size,
        kp, vp, stride, _p(q_out), _dt(proj), proj.shape[0], q_heads, kv_heads, dk, dv, int(store),
        _p(inv_freq), int(rot_dims if inv_freq is not None else 0), float(coef), int(every), int(values_are_keys),
        _p(bias), _stream()), "qkv_unit_store")


def attention_biased(q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor, positions, token_slot,
                     block_table, page_size: int, q_heads: int, kv_heads: int, dk: int, dv: int, scale: float,
                     out: torch.Tensor, softcap: float = 0.0, chunk: int = 0, window: int = 0,
                     sink: bool = False, slopes: Optional[torch.Tensor] = None,
                     gate: Optional[torch.Tensor] = None, ctx=None, sink_logits: Optional[torch.Tensor] = None,
                     values_in_keys: bool = False, distance_bias: Optional[torch.Tensor] = None,
                     gate_per_head: bool = False) -> torch.Tensor:
    """Attention of every row of ``q`` [T, q_heads * dk] over the keys of its own request, with the
    score s = (q . k) * scale changed in this order by whatever is given: ``softcap`` (s <- cap *
    tanh(s / cap)), ``slopes`` [q_heads] float32 (s <- s - slope * (pos - key pos)); keys j <= pos from
    the row's own ``chunk`` of positions and from its ``window``; ``sink``: one is added to the softmax's
    denominator, or exp(sink_logits[head]) with ``sink_logits`` [q_heads] float32 (a learned score that is
    neither scaled nor capped).  ``gate`` (a view [T, q_heads * dv], or with ``gate_per_head`` [T, q_heads],
    whose rows may be strided): out *= sigmoid(gate).  ``values_in_keys``: a value is the first ``dv`` elements of its key's row (``v_plane`` is
    not looked at), as in attention over compressed vectors that are key and, in part, value at once.
    ``distance_bias`` [q_heads, L] float32: entry [h, min(pos - key pos, L - 1)] is added to the score after
    everything else (a learned bias by distance; it is not scaled)."""
    _cuda(q, positions, token_slot, block_table, out, slopes, sink_logits, distance_bias)
    dist_len = 0
    if distance_bias is not None:
        assert distance_bias.dtype == torch.float32 and distance_bias.dim() == 2 and distance_bias.shape[0] == q_heads
        dist_len = distance_bias.shape[1]
    tokens = q.shape[0]
    assert tuple(out.shape) == (tokens, q_heads * dv) and out.dtype == q.dtype
    kp, stride = _plane(k_plane)
    if values_in_keys:
        assert dv <= dk
        vp, stride_v, v_row = kp, stride, dk
    else:
        (vp, stride_v), v_row = _plane(v_plane), dv
    assert stride == stride_v and k_plane.dtype == q.dtype
    if sink_logits is not None:
        assert sink and sink_logits.dtype == torch.float32 and sink_logits.numel() == q_heads
    gate_stride = 0
    if gate is not None:
        assert gate.dtype == q.dtype and gate.stride(1) == 1
        assert tuple(gate.shape) == ((tokens, q_heads) if gate_per_head else tuple(out.shape))
        gate_stride = gate.stride(0)
    if slopes is not None:
        assert slopes.dtype == torch.float32 and slopes.numel() == q_heads
    gate_ptr = None if gate is None else gate.data_ptr()
    mods = (float(scale), float(softcap or 0.0), int(chunk or 0), int(window or 0), int(bool(sink)), _p(slopes),
            _p(sink_logits), _p(distance_bias), dist_len, v_row, gate_ptr, gate_stride, int(gate_per_head))
    consts = mods + (_p(out), _stream())
    # the plain score, or one changed only by a table of biases and a learned sink, at width 128 on both
    # sides: prompt portions go to the tcgen05 kernel of the plain cache, which reads the two planes
    tcgen05 = PREFILL_TCGEN05 and dk == 128 and dv == 128 and not values_in_keys and not softcap and not chunk \
        and slopes is None and gate is None and (sink_logits is not None or not sink) \
        and page_size % 16 == 0 and stride % 128 == 0 and q_heads <= 65535
    if BIASED_FAST and ctx is not None and ctx.pf_tiles is not None and ctx.tokens == tokens \
            and q.dtype == torch.bfloat16 and (gate_stride % 2 == 0 or gate_per_head) and v_row % 8 == 0 \
            and lib().tllm_attention_biased_fast_ok(q_heads, kv_heads, dk, dv):
        # one-token rows: keys read once per group of query heads; longer portions: tensor-core tiles
        if ctx.n_dec:
            reach = min(v for v in (chunk, window, ctx.max_context or 1 << 30) if v)
            splits = biased_decode_splits(ctx.n_dec, kv_heads, reach)
            part = None
            if splits > 1:
                part = workspace(q.device, ctx.n_dec * q_heads * splits * (dv + 2))
            _check(lib().tllm_attention_biased_decode(
                _p(q), kp, vp, stride, _p(positions), _p(token_slot), _p(ctx.dec_rows), ctx.n_dec, _p(block_table),
                block_table.shape[1], page_size, q_heads, kv_heads, dk, dv, *mods, splits, _p(part), _p(out), _stream()),
                "attention_biased_decode", kernels=2 if splits > 1 else 1)
        if ctx.n_tiles and tcgen05 and getattr(ctx, "n_tiles256", 0):
            pairs = prefill_tcgen05_block_rows(q_heads, kv_heads) == 128
            blocks = ctx.n_tiles128 if pairs else ctx.n_tiles256
            keys = ctx.max_context if not window else min(ctx.max_context, window + 256)
            splits = prefill_splits(blocks * (q_heads // 2 if pairs else q_heads), keys)
            part_o = part_ml = None
            if splits > 1:
                n = tokens * q_heads * splits
                ws = workspace(q.device, n * (dv + 2))
                part_o, part_ml = ws[:n * dv], ws[n * dv:n * (dv + 2)]
            global tcgen05_calls
            tcgen05_calls += 1
            _check(lib().tllm_attention_planes_prefill_tc(
                _p(q), tokens, kp, vp, stride, k_plane.shape[0], _p(ctx.seg_info), _p(ctx.pf_tiles), blocks,
                _p(block_table), block_table.shape[1], page_size, q_heads, kv_heads, int(window or 0), float(scale),
                _p(distance_bias), dist_len, _p(sink_logits), _p(out), splits, _p(part_o), _p(part_ml),
                _p(error_word(q.device)), _stream()), "attention_planes_prefill_tc", kernels=2 if splits > 1 else 1)
        elif ctx.n_tiles:
            _check(lib().tllm_attention_biased_prefill(
                _p(q), kp, vp, stride, _p(ctx.seg_info), _p(ctx.pf_tiles), ctx.n_tiles, _p(block_table),
                block_table.shape[1], page_size, q_heads, kv_heads, dk, dv, *consts), "attention_biased_prefill")
        return out
    _check(lib().tllm_attention_biased_general(
        _p(q), kp, vp, stride, _p(positions), _p(token_slot), _p(block_table), block_table.shape[1], page_size,
        _dt(q), tokens, q_heads, kv_heads, dk, dv, float(scale), float(softcap or 0.0), int(chunk or 0),
        int(window or 0), int(bool(sink)), _p(slopes), _p(sink_logits), _p(distance_bias), dist_len, v_row,
        None if gate is None else gate.data_ptr(), gate_stride, int(gate_per_head), _p(out), _stream()), "attention_biased")
    return out


# --------------------------------------------------------------------------- stream, embedding with positions, activations
ELEMENTWISE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "gelu_erf": 2, "relu2": 3}      # codes of csrc/common.cuh (GateAct); relu2 = max(x, 0)^2


def embedding_norm(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
                   positions: Optional[torch.Tensor] = None, pos_table: Optional[torch.Tensor] = None,
                   gain: Optional[torch.Tensor] = None, eps: float = 0.0) -> torch.Tensor:
    """out[t] = norm(table[ids[t]] * scale + pos_table[positions[t]]) in float32: the position table and the
    norm (``gain`` float32, the factor itself; x / sqrt(mean(x^2) + eps) * gain) only where they are given."""
    _cuda(ids, table, out, positions, pos_table, gain)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32
    vocab, hidden = table.shape
    if pos_table is not None:
        assert pos_table.dtype == table.dtype and pos_table.shape[1] == hidden and positions.dtype == torch.int32
    if gain is not None:
        assert gain.dtype == torch.float32 and gain.numel() == hidden
    _check(lib().tllm_embedding_norm(_p(ids), _p(positions), _p(table), _p(pos_table), _dt(table), _p(gain), float(eps),
                                     float(scale), _p(out), ids.numel(), hidden, vocab,
                                     0 if pos_table is None else pos_table.shape[0], _stream()), "embedding_norm")
    return out


def stream_add(h: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
               post_gain: Optional[torch.Tensor] = None, post_eps: float = 0.0) -> torch.Tensor:
    """h += delta (float32, written back) and out = h in the storage type, with no norm on the way out.  With
    ``post_gain`` the delta is normed first: h += post_gain * delta / sqrt(mean(delta^2) + post_eps)."""
    _cuda(h, delta, out, post_gain)
    assert h.dtype == torch.float32 and out.shape == h.shape
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape == h.shape
    gdt = _dt(post_gain) if post_gain is not None else F32
    _check(lib().tllm_stream_add(_p(h), _p(delta), _p(post_gain), gdt, float(post_eps), _p(out), _dt(out), h.shape[0],
                                 h.shape[1], _stream()), "stream_add")
    return out


def linear_act(x: torch.Tensor, weight: torch.Tensor, act: str, out_dtype: torch.dtype) -> torch.Tensor:
    """act(x . weight^T) with ``act`` one of ``ELEMENTWISE_ACTIVATIONS``.  In bfloat16 the activation sits in the
    product's epilogue where this package's own products run (at most 8 rows: the weight-streaming kernel; from
    256 rows on, where the tiles fill the GPU: the tcgen05 kernel); else the product is followed by the
    activation kernel."""
    rows, k = x.shape
    plain = x.dtype == weight.dtype == out_dtype == torch.bfloat16 and x.is_contiguous() and weight.is_contiguous()
    if plain and 0 < rows <= SKINNY_MAX_ROWS and k % 8 == 0:
        _cuda(x, weight)
        out = torch.empty((rows, weight.shape[0]), dtype=torch.bfloat16, device=x.device)
        _check(lib().tllm_gemm_skinny_act(_p(x), _p(weight), _p(out), rows, weight.shape[0], k,
                                          ELEMENTWISE_ACTIVATIONS[act], _stream()), "gemm_skinny_act")
        return out
    if plain and tcgen05_pays(rows, weight.shape[0], k, weight.dtype):
        return gemm_tcgen05(x, weight, act=act, unary=True)
    return activation(linear(x, weight, out_dtype=out_dtype), act)


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place, float32."""
    _cuda(x)
    assert x.dtype == torch.float32
    _check(lib().tllm_softcap(_p(x), float(cap), x.numel(), _stream()), "softcap")
    return x


def activation(x: torch.Tensor, act: str, ids: Optional[torch.Tensor] = None, table: Optional[torch.Tensor] = None,
               col0: int = 0) -> torch.Tensor:
    """act(x) element by element (``silu``, ``gelu_tanh``, ``gelu_erf``; float32 inside); with ``table`` [vocab,
    columns] and ``ids``, times table[ids[t], col0 + j]: a gate on a vector looked up by the row's token."""
    _cuda(x, ids, table)
    tokens, width = x.shape
    out = torch.empty_like(x)
    if table is not None:
        assert table.dtype == x.dtype and ids.dtype == torch.int32 and ids.numel() == tokens
    _check(lib().tllm_activation(_p(x), _p(out), _dt(x), ELEMENTWISE_ACTIVATIONS[act], tokens, width, _p(ids), _p(table),
                                 0 if table is None else table.shape[1], int(col0),
                                 0 if table is None else table.shape[0], _stream()), "activation")
    return out


# --------------------------------------------------------------------------- delta rule with channel-wise decay
def delta_rule_state_floats(heads: int, kv_heads: int, dk: int, dv: int, taps: int) -> int:
    """Float32 words of one request's state: S of every head in the scan kernel's layout, then the
    convolution's last ``taps - 1`` inputs."""
    return int(lib().tllm_delta_rule_state_floats(heads, kv_heads, dk, dv, taps))


SCAN_DELTA, SCAN_PLAIN, SCAN_MEMORY, SCAN_HEAD_DECAY = 0, 1, 2, 3     # recurrences of the scan kernel (csrc/delta_rule.cu, ScanMode)
GATE_ACTS = {"sigmoid": 0, "silu": 1}                # what the read-out is multiplied by: act(gate)


def _delta_finish(o_raw, gate, out_weight, weight_per_head, eps, token_slot, tokens, heads, kv_heads, dk, dv, out_dtype,
                  proj, ld, taps, state, den, gate_act):
    out = torch.empty((tokens, heads * dv), dtype=out_dtype, device=o_raw.device)
    assert gate.stride(1) == 1 and gate.dtype in (torch.float32, out_dtype) and out_weight.dtype == torch.float32
    assert out_weight.numel() == (heads * dv if weight_per_head else dv)
    _check(lib().tllm_delta_finish(_p(o_raw), gate.data_ptr(), int(gate.dtype == torch.float32), gate.stride(0), _p(out_weight),
                                   float(eps), _p(token_slot), tokens, heads, kv_heads, dk, dv, _p(out), _dt(out), _p(proj), ld,
                                   taps, _p(state), state.stride(0), _p(den), GATE_ACTS[gate_act],
                                   dv if weight_per_head else 0, _stream()), "delta_finish")
    return out


def delta_rule(proj: torch.Tensor, conv_w: torch.Tensor, taps: int, a: torch.Tensor, dt_bias: torch.Tensor,
               rate: torch.Tensor, gate: torch.Tensor, out_weight: torch.Tensor, eps: float, token_slot: torch.Tensor,
               seg_info: Optional[torch.Tensor], state: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int,
               q_scale: float, unit_eps: float, out_dtype: torch.dtype, conv_t: Optional[torch.Tensor] = None,
               decay_per_head: bool = False, beta_col: Optional[int] = None, gate_act: str = "sigmoid") -> torch.Tensor:
    """One step of the delta rule for every row of ``proj`` [T, >= channels + heads] = q channels | k channels | v
    channels | ... with the beta logits at column ``beta_col`` (None: right behind the channels), in the storage
    type: convolution with ``conv_w`` [channels, taps] and SiLU, unit q and k, g = exp(-rate_h softplus(a + dt_bias))
    with ``a`` float32 [T, heads * dk] (a decay per head and key channel) or, ``decay_per_head``, [T, heads]; the
    recurrence over each portion's rows from ``state[slot]`` (float32, updated in place), then the read-out divided
    by its root mean square per head, times ``out_weight`` [dv] float32, times ``gate_act``(``gate``) ([T, heads * dv]
    float32 or storage type, rows may be strided).  ``seg_info`` [segments, 4] = slot, first row, length, first
    position; None: every row is a portion of one token.  ``conv_t``: the taps once more as [taps, channels], which
    lets the kernels take eight channels per access.  Returns [T, heads * dv] in ``out_dtype``."""
    _cuda(proj, conv_w, dt_bias, rate, out_weight, token_slot, seg_info, state, conv_t)
    tokens, ld = proj.shape
    assert a.dtype == dt_bias.dtype == rate.dtype == out_weight.dtype == state.dtype == torch.float32
    assert a.stride(1) == 1 and conv_w.dtype == proj.dtype and state.dim() == 2
    assert dt_bias.numel() == (heads if decay_per_head else heads * dk)
    dev = proj.device
    ws = workspace(dev, tokens * (2 * kv_heads * dk + 2 * heads * dv + heads * dk + heads))
    at = 0

    def take(n):
        nonlocal at
        t = ws[at:at + tokens * n]
        at += tokens * n
        return t
    # q, k and the decays first: their rows start on 16-byte boundaries wherever dk is a multiple of four
    qn, kn, decay, vv, o_raw, beta = (take(kv_heads * dk), take(kv_heads * dk), take(heads * dk), take(heads * dv),
                                      take(heads * dv), take(heads))
    _check(lib().tllm_delta_prepare(_p(proj), ld, _dt(proj), _p(conv_w), _p(conv_t), taps, a.data_ptr(), a.stride(0), _p(dt_bias), _p(rate),
                                    _p(token_slot), _p(state), state.stride(0), heads, kv_heads, dk, dv, float(q_scale),
                                    float(unit_eps), _p(qn), _p(kn), _p(vv), _p(decay), _p(beta), tokens,
                                    int(decay_per_head), -1 if beta_col is None else int(beta_col), _stream()),
           "delta_prepare")
    segments = tokens if seg_info is None else seg_info.shape[0]
    _check(lib().tllm_delta_scan(_p(seg_info), segments, _p(token_slot), _p(qn), _p(kn), _p(vv), _p(decay), _p(beta),
                                 _p(state), state.stride(0), heads, kv_heads, dk, dv, _p(o_raw), SCAN_DELTA, None, 0, 0.0,
                                 None, _stream()), "delta_scan")
    return _delta_finish(o_raw, gate, out_weight, False, eps, token_slot, tokens, heads, kv_heads, dk, dv, out_dtype,
                         proj, ld, taps, state, None, gate_act)


LINEAR_KINDS = {"channel_decay": 0, "log_gates": 1}      # csrc/delta_rule.cu, LinearKind


def linear_recurrence_state_floats(kind: str, heads: int, dk: int, dv: int) -> int:
    """Float32 words of one request's state of ``linear_recurrence``: S of every head in the scan kernel's layout
    (with ``log_gates`` one more column, the normaliser) and, with ``log_gates``, the running maximum per column."""
    cols = dv + 1 if kind == "log_gates" else dv
    s_floats = delta_rule_state_floats(heads, heads, dk, cols, 1)
    return s_floats + (heads * cols if kind == "log_gates" else 0)


def linear_recurrence(proj: torch.Tensor, kind: str, z: torch.Tensor, z_bias: torch.Tensor, p0: float,
                      gate: torch.Tensor, gate_act: str, out_weight: torch.Tensor, weight_per_head: bool, eps: float,
                      token_slot: torch.Tensor, seg_info: Optional[torch.Tensor], state: torch.Tensor, heads: int,
                      dk: int, dv: int, q_scale: float, out_dtype: torch.dtype, floor_eps: float = 1e-6) -> torch.Tensor:
    """One step of a recurrence S <- decay S + k (w v)^T, o = S^T q per head, for every row of ``proj`` [T, >= heads
    (2 dk + dv)] = q | k | v in the storage type (q is multiplied by ``q_scale``), from ``state[slot]`` (float32,
    updated in place).  ``kind``:

    * ``channel_decay``: a decay per key channel sigmoid(z + z_bias)^p0 with ``z`` [T, heads * dk] float32, w = 1;
    * ``log_gates``: ``z`` [T, 2 heads] float32 = write | keep logits (plus ``z_bias``), each capped as p0 tanh(. /
      p0); with i the capped write logit and f = logsigmoid(capped keep logit), a running maximum m <- max(f + m, i)
      that starts at zero: decay = exp(f + m_before - m), w = exp(i - m); a vector n <- decay n + w k is kept beside
      S and the read-out is S^T q / (max(|n . q|, exp(-m)) + ``floor_eps``).

    Then the read-out is divided by its root mean square per head (``eps``), times ``out_weight`` ([dv], or [heads *
    dv] with ``weight_per_head``) float32, times ``gate_act``(``gate``) ([T, heads * dv], rows may be strided).
    Returns [T, heads * dv] in ``out_dtype``."""
    _cuda(proj, z_bias, out_weight, token_slot, seg_info, state)
    tokens, ld = proj.shape
    assert z.dtype == z_bias.dtype == state.dtype == torch.float32 and z.stride(1) == 1 and state.dim() == 2
    memory = kind == "log_gates"
    cols = dv + 1 if memory else dv
    assert state.shape[1] == linear_recurrence_state_floats(kind, heads, dk, dv)
    dev = proj.device
    ws = workspace(dev, tokens * (3 * heads * dk + heads * (cols + dv) + 3 * heads + 8))
    at = 0

    def take(n):
        nonlocal at
        t = ws[at:at + tokens * n]
        at += -(-tokens * n // 4) * 4
        return t
    qn, kn = take(heads * dk), take(heads * dk)
    decay = None if memory else take(heads * dk)
    vv, o_raw = take(heads * cols), take(heads * dv)
    wgate, fgate, den = (take(heads), take(heads), take(heads)) if memory else (None, None, None)
    _check(lib().tllm_linear_prepare(_p(proj), ld, _dt(proj), z.data_ptr(), z.stride(0), _p(z_bias), LINEAR_KINDS[kind],
                                     float(p0), _p(token_slot), heads, dk, dv, float(q_scale), _p(qn), _p(kn), _p(vv),
                                     _p(decay), _p(wgate), _p(fgate), tokens, _stream()), "linear_prepare")
    segments = tokens if seg_info is None else seg_info.shape[0]
    aux_off = delta_rule_state_floats(heads, heads, dk, cols, 1) if memory else 0
    _check(lib().tllm_delta_scan(_p(seg_info), segments, _p(token_slot), _p(qn), _p(kn), _p(vv), _p(decay), _p(wgate),
                                 _p(state), state.stride(0), heads, heads, dk, cols, _p(o_raw),
                                 SCAN_MEMORY if memory else SCAN_PLAIN, _p(fgate), aux_off, float(floor_eps), _p(den),
                                 _stream()), "delta_scan")
    return _delta_finish(o_raw, gate, out_weight, weight_per_head, eps, token_slot, tokens, heads, heads, dk, dv,
                         out_dtype, None, 0, 1, state, den, gate_act)


# --------------------------------------------------------------------------- selective state space
def state_space_state_floats(heads: int, groups: int, state: int, head_dim: int, taps: int) -> int:
    """Float32 words of one request's state of ``state_space``: S [state, head_dim] of every head in the scan
    kernel's layout, then the convolution's last ``taps - 1`` inputs over the channels x | B | C."""
    return delta_rule_state_floats(heads, groups, state, head_dim, 1) + (taps - 1) * (heads * head_dim + 2 * groups * state)


def state_space(proj: torch.Tensor, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor], taps: int,
                dt_bias: torch.Tensor, rate: torch.Tensor, skip: torch.Tensor, out_weight: torch.Tensor, eps: float,
                norm_groups: int, token_slot: torch.Tensor, seg_info: Optional[torch.Tensor], state: torch.Tensor,
                heads: int, groups: int, n_state: int, head_dim: int, out_dtype: torch.dtype,
                conv_t: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One step of a selective state space with a decay per head, for every row of ``proj`` [T, >= 2 heads P + 2 G N
    + heads] = z | x | B | C | dt in the storage type (P = ``head_dim``, N = ``n_state``, G = ``groups``): the causal
    convolution ``conv_w`` [channels, taps] with bias ``conv_b`` over x | B | C and SiLU, dt = softplus(dt +
    ``dt_bias``), per head S <- exp(-rate_h dt) S + B (dt x)^T from ``state[slot]`` (float32, updated in place), y =
    S^T C + skip_h x, then y silu(z), an RMS norm over each of ``norm_groups`` equal parts of the row and
    ``out_weight``.  ``dt_bias``, ``rate``, ``skip`` [heads], ``conv_b`` and ``out_weight`` are float32.  ``seg_info``
    as in ``delta_rule``.  ``conv_t``: the taps once more as [taps, channels], which lets the kernels take eight
    channels per access.  Returns [T, heads P] in ``out_dtype``."""
    _cuda(proj, conv_w, conv_b, dt_bias, rate, skip, out_weight, token_slot, seg_info, state, conv_t)
    tokens, ld = proj.shape
    inner, gn = heads * head_dim, groups * n_state
    channels = inner + 2 * gn
    assert dt_bias.dtype == rate.dtype == skip.dtype == out_weight.dtype == state.dtype == torch.float32
    assert conv_w.dtype == proj.dtype and tuple(conv_w.shape) == (channels, taps) and state.dim() == 2
    assert conv_b is None or (conv_b.dtype == torch.float32 and conv_b.numel() == channels)
    assert out_dtype == proj.dtype and state.shape[1] == state_space_state_floats(heads, groups, n_state, head_dim, taps)
    tail_off = delta_rule_state_floats(heads, groups, n_state, head_dim, 1)
    ws = workspace(proj.device, tokens * (2 * gn + 2 * inner + 2 * heads) + 32)
    at = 0

    def take(n):
        nonlocal at
        t = ws[at:at + tokens * n]
        at += -(-tokens * n // 4) * 4
        return t
    qn, kn, decay, step, vv, o_raw = take(gn), take(gn), take(heads), take(heads), take(inner), take(inner)
    _check(lib().tllm_ssd_prepare(_p(proj), ld, _dt(proj), _p(conv_w), _p(conv_t), _p(conv_b), taps, _p(dt_bias), _p(rate),
                                  _p(token_slot), _p(state), state.stride(0), tail_off, heads, groups, n_state, head_dim,
                                  _p(qn), _p(kn), _p(vv), _p(decay), _p(step), tokens, _stream()), "ssd_prepare")
    segments = tokens if seg_info is None else seg_info.shape[0]
    _check(lib().tllm_delta_scan(_p(seg_info), segments, _p(token_slot), _p(qn), _p(kn), _p(vv), None, _p(decay),
                                 _p(state), state.stride(0), heads, groups, n_state, head_dim, _p(o_raw), SCAN_HEAD_DECAY,
                                 _p(step), 0, 0.0, None, _stream()), "delta_scan")
    out = torch.empty((tokens, inner), dtype=out_dtype, device=proj.device)
    _check(lib().tllm_ssd_finish(_p(o_raw), _p(vv), _p(skip), head_dim, _p(proj), ld, _dt(proj), _p(out_weight), float(eps),
                                 int(norm_groups), _p(token_slot), tokens, inner, channels, taps, _p(state),
                                 state.stride(0), tail_off, _p(out), _stream()), "ssd_finish")
    return out


# --------------------------------------------------------------------------- attention over compressed vectors
def latent_norm_store(proj: torch.Tensor, q_rank: int, rank: int, rot: int, rot_dims: int, q_gain, c_gain,
                      eps: float, freq: torch.Tensor, mag: float, positions, token_slot, block_table,
                      plane: torch.Tensor, page_size: int, store: bool = True,
                      half_pairs: bool = False) -> Optional[torch.Tensor]:
    """Rows of ``proj`` (a view whose rows may be strided) = query latent (q_rank) | key/value latent (rank) |
    shared key part (rot) | anything.  ``half_pairs``: the rotation pairs element i with i + rot_dims / 2 instead of
    its neighbour.
    Returns the query latent divided by its root mean square times ``q_gain`` (None if q_rank is 0) and
    writes [normed latent times ``c_gain`` | rotated key part] of every row into its place of ``plane``
    ([pages, 1, page, rank + rot]).  Gains and ``freq`` [rot_dims / 2] are float32."""
    _cuda(q_gain, c_gain, freq, positions, token_slot, block_table)
    assert proj.is_cuda and proj.stride(1) == 1
    tokens = proj.shape[0]
    cq = torch.empty((tokens, q_rank), dtype=proj.dtype, device=proj.device) if q_rank else None
    pp, stride = _plane(plane)
    assert plane.dtype == proj.dtype and tuple(plane.shape[1:]) == (1, page_size, rank + rot)
    _check(lib().tllm_latent_norm_store(proj.data_ptr(), proj.stride(0), _dt(proj), q_rank, rank, rot, rot_dims, _p(q_gain),
                                        _p(c_gain), float(eps), _p(freq), float(mag), _p(positions), _p(token_slot),
                                        _p(block_table), block_table.shape[1], page_size, pp, stride, _p(cq), int(store),
                                        tokens, int(half_pairs), _stream()), "latent_norm_store")
    return cq


def latent_query(q: torch.Tensor, lat: torch.Tensor, heads: int, plain: int, rot: int, rot_dims: int, rank: int,
                 freq: torch.Tensor, mag: float, positions, token_slot, half_pairs: bool = False) -> torch.Tensor:
    """[T, heads, rank + rot]: per head ``lat`` [heads, T, rank] followed by the rotated last ``rot`` elements
    of the head's query in ``q`` [T, heads * (plain + rot)] (a view whose rows may be strided)."""
    _cuda(lat, freq, positions, token_slot)
    assert q.is_cuda and q.stride(1) == 1
    tokens = q.shape[0]
    assert tuple(lat.shape) == (heads, tokens, rank) and lat.dtype == q.dtype and q.shape[1] == heads * (plain + rot)
    out = torch.empty((tokens, heads * (rank + rot)), dtype=q.dtype, device=q.device)
    _check(lib().tllm_latent_query(q.data_ptr(), q.stride(0), _p(lat), _dt(q), heads, plain, rot, rot_dims, rank, _p(freq), float(mag),
                                   _p(positions), _p(token_slot), tokens, _p(out), int(half_pairs), _stream()), "latent_query")
    return out


def heads_gate(x: torch.Tensor, gate: Optional[torch.Tensor], token_slot=None, per_head: bool = False) -> torch.Tensor:
    """[T, heads * width] = x[h, t, :] * sigmoid(gate[t, h * width + :]) for ``x`` [heads, T, width]; ``gate`` is a
    view whose rows may be strided (None: no gate); with ``per_head`` it is [T, heads], one number per head."""
    _cuda(x, token_slot)
    heads, tokens, width = x.shape
    out = torch.empty((tokens, heads * width), dtype=x.dtype, device=x.device)
    ldg = 0
    if gate is not None:
        assert gate.dtype == x.dtype and gate.stride(1) == 1
        assert tuple(gate.shape) == (tokens, heads if per_head else heads * width)
        ldg = gate.stride(0)
    _check(lib().tllm_heads_gate(_p(x), None if gate is None else gate.data_ptr(), ldg, _dt(x), heads, width, tokens,
                                 _p(token_slot), _p(out), int(per_head), _stream()), "heads_gate")
    return out


# --------------------------------------------------------------------------- mixture of experts
def moe_tile_rows() -> int:
    return int(lib().tllm_moe_tile_rows())


def moe_route(z: torch.Tensor, top: int, softmax_weights: bool = False):
    """(ids [T, top] int32, weights [T, top] float32) from float32 router logits ``z`` [T, E]: the
    ``top`` experts with the largest logits; weight sigmoid(z), or softmax over the chosen ones."""
    _cuda(z)
    assert z.dtype == torch.float32
    tokens, experts = z.shape
    ids = torch.empty((tokens, top), dtype=torch.int32, device=z.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=z.device)
    _check(lib().tllm_moe_route(_p(z), tokens, experts, top, int(softmax_weights), _p(ids), _p(weights), _stream()),
           "moe_route")
    return ids, weights


ROUTER_SCORES = {"sigmoid": 0, "softmax": 1}      # scores over all experts (csrc/moe.cu, moe_route_grouped)


def moe_route_grouped(z: torch.Tensor, top: int, scores: str = "softmax", correction: Optional[torch.Tensor] = None,
                      groups: int = 1, keep: int = 1):
    """(ids [T, top] int32, weights [T, top] float32) from float32 router logits ``z`` [T, E]: scores s over all E
    experts (``softmax`` or ``sigmoid``); the choice goes by s + ``correction`` ([E] float32, if given), within the
    ``keep`` of ``groups`` equal groups of neighbouring experts whose best member scores highest; the weights are
    the chosen experts' s as they are.  Lowest index first on ties."""
    _cuda(z, correction)
    assert z.dtype == torch.float32 and (correction is None or (correction.dtype == torch.float32 and correction.numel() == z.shape[1]))
    tokens, experts = z.shape
    ids = torch.empty((tokens, top), dtype=torch.int32, device=z.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=z.device)
    _check(lib().tllm_moe_route_grouped(_p(z), tokens, experts, top, ROUTER_SCORES[scores], _p(correction), int(groups),
                                        int(keep), _p(ids), _p(weights), _stream()), "moe_route_grouped")
    return ids, weights


class MoePlan:
    """Device-side lists that sort a step's (token, choice) assignments by expert, with the rows cut
    into tiles of ``tile_rows`` per expert.  ``real``: experts that have matrices; assignments to later ones
    (identity experts) get rows and no tiles."""

    def __init__(self, ids: torch.Tensor, experts: int, tile_rows: Optional[int] = None, real: Optional[int] = None):
        n = ids.numel()
        self.n, self.experts = n, experts
        self.real = experts if real is None else int(real)
        self.tile_rows = tile_rows or moe_tile_rows()
        self.max_tiles = n // self.tile_rows + experts
        ints = torch.empty(experts + 2 + 3 * n + 2 * self.max_tiles, dtype=torch.int32, device=ids.device)
        at = 0

        def take(k):
            nonlocal at
            part = ints[at:at + k]
            at += k
            return part
        self.offsets, self.n_tiles = take(experts + 1), take(1)
        self.row_of, self.src_of, self.expert_of_row = take(n), take(n), take(n)
        self.tile_expert, self.tile_row0 = take(self.max_tiles), take(self.max_tiles)
        _check(lib().tllm_moe_plan(_p(ids), n, experts, self.real, self.tile_rows, _p(self.offsets), _p(self.n_tiles),
                                   _p(self.row_of), _p(self.src_of), _p(self.expert_of_row), _p(self.tile_expert),
                                   _p(self.tile_row0), _stream()), "moe_plan")


MOE_TCGEN05_ROWS = 1024     # from this many (token, choice) rows on the experts' products run on tcgen05
MOE_TCGEN05_TILE = 128


def moe_tcgen05_pays(rows: int, experts: int, n: int, k: int, dtype) -> bool:
    """Whether the experts' products of a step take the grouped tcgen05 kernel: bfloat16, whole 16-byte
    pieces, and enough rows that an expert's tile of 128 is on average at least a quarter full."""
    return (dtype == torch.bfloat16 and rows >= MOE_TCGEN05_ROWS and rows >= 32 * experts
            and k % 8 == 0 and n % 8 == 0)


def moe_grouped(a: torch.Tensor, w: torch.Tensor, plan: MoePlan, top: int, gated: bool, gather: bool,
                weights: Optional[torch.Tensor] = None, act: str = "silu", interleaved: bool = False,
                out_dtype: Optional[torch.dtype] = None, unary: bool = False) -> torch.Tensor:
    """Per row r of the plan, A[r] . W[expert of r]^T.  ``w`` is [E, N (or 2 N: gate rows, then up rows, or
    ``interleaved`` by eight), K].  ``gather``: ``a`` is [tokens, K] and a row reads its token, times ``weights``
    [tokens, top] if given.  ``gated``: the result is act(gate) * up [rows, N] in the storage type, else
    [rows, N] float32, or with ``unary`` act(.) [rows, N] in the storage type (``act`` then one of
    ``ELEMENTWISE_ACTIVATIONS``).  A plan cut into tiles of 128 rows goes to the grouped tcgen05 product (bfloat16
    in and out; the gathered rows are laid out by a kernel of their own first).  Rows of experts without matrices
    (``plan.real``) are left unwritten."""
    _cuda(a, w, weights)
    experts, n_total, k = w.shape
    assert a.shape[1] == k and a.dtype == w.dtype and experts == plan.real and not (gated and unary)
    act_code = ELEMENTWISE_ACTIVATIONS[act] if unary else ACTIVATIONS[act]
    n = n_total // 2 if gated else n_total
    if plan.tile_rows == MOE_TCGEN05_TILE:
        assert a.dtype == torch.bfloat16 and (interleaved or not gated)
        if gather:
            xs = torch.empty((plan.n, k), dtype=a.dtype, device=a.device)
            _check(lib().tllm_moe_gather(_p(a), _p(plan.src_of), _p(weights), top, _p(xs), plan.n, k, _stream()),
                   "moe_gather")
            a = xs
        out = torch.empty((plan.n, n), dtype=torch.bfloat16, device=a.device)
        global tcgen05_calls
        tcgen05_calls += 1
        flags = (1 | 4 | (act_code << 8)) if gated else ((16 | (act_code << 8)) if unary else 0)
        _check(lib().tllm_gemm_tcgen05_grouped(
            _p(a), _p(w), _p(out), plan.n, n_total, k, experts, flags, _p(plan.tile_expert), _p(plan.tile_row0),
            _p(plan.n_tiles), _p(plan.offsets), plan.max_tiles, _p(error_word(a.device)), _stream()),
            "gemm_tcgen05_grouped")
        return out
    out = torch.empty((plan.n, n), dtype=a.dtype if (gated or unary) else torch.float32, device=a.device)
    _check(lib().tllm_moe_grouped(
        _p(a), a.stride(0), _p(plan.src_of), _p(weights), top, _p(w), w.stride(0), _p(plan.tile_expert),
        _p(plan.tile_row0), _p(plan.n_tiles), _p(plan.offsets), _p(plan.expert_of_row), plan.n, plan.max_tiles,
        n, k, _dt(a), 1 if gated else (2 if unary else 0), int(gather), act_code, int(interleaved), plan.real, _p(out),
        _stream()), "moe_grouped")
    return out


def moe_combine(y: torch.Tensor, plan: MoePlan, top: int, shared: Optional[torch.Tensor], dtype: torch.dtype,
                weights: Optional[torch.Tensor] = None, identity_input: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = shared[t] + sum_k (weights[t, k] *) y[row of (t, k)], float32 sums, stored as ``dtype``;
    ``y`` float32 or in the storage type.  ``identity_input`` [T, width] (``dtype``): an assignment to an expert
    without matrices (``plan.real`` or later) adds the token's row of it instead of a row of ``y``."""
    _cuda(y, shared, weights, identity_input)
    if identity_input is not None:
        assert identity_input.dtype == dtype and tuple(identity_input.shape) == (plan.n // top, y.shape[1])
    tokens, width = plan.n // top, y.shape[1]
    out = torch.empty((tokens, width), dtype=dtype, device=y.device)
    if shared is not None:
        assert shared.dtype == dtype and tuple(shared.shape) == (tokens, width)
    _check(lib().tllm_moe_combine(_p(y), _dt(y), _p(plan.row_of), _p(weights), top, _p(shared), _p(out), _DT[dtype],
                                  tokens, width, _p(identity_input), _p(plan.expert_of_row), plan.real, _stream()),
           "moe_combine")
    return out
