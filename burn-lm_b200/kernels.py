"""Python faces of the CUDA kernels in `csrc/`.

Each function checks what it is given, hands raw device pointers to the C entry point of the same
name, and raises `KernelError` with the kernel's own message when that refuses.  Kernels run on
torch's current CUDA stream, so they can be captured in a CUDA graph with the matrix products
around them.  There is no fallback: without a CUDA device or without the compiled library these
functions raise.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_size_t, c_uint, c_ulonglong, c_void_p

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
PAGE = 64  # positions per cache page; the attention kernels are written for this size


class KernelError(RuntimeError):
    pass


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """How many multiprocessors the device has (asked once per device)."""
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = torch.cuda.current_device()
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return n


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """torch's current stream on the current device, as a raw handle.  Asked once per launch: the short way
    (two calls into torch's C module) costs a tenth of building a torch.cuda.Stream object each time."""
    if _raw_stream is not None and _current_device is not None:
        return c_void_p(_raw_stream(_current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("burn-lm_b200 kernels run on a CUDA device only; got a CPU tensor")
        if t is not None and not t.is_contiguous():
            raise KernelError("kernel arguments must be contiguous")


_protos = {
    "elementwise": {
        "blm_embed": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p],
        "blm_add_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                            c_float, c_void_p],
        "blm_rope_append": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                            c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p],
        "blm_rope_table": [c_void_p, c_void_p, c_int, c_int, c_void_p],
        "blm_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "blm_convert": [c_void_p, c_int, c_void_p, c_int, c_size_t, c_void_p],
        "blm_decode_advance": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "blm_step_tables": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "blm_embed_pairs": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                            c_int, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p,
                            c_void_p],
        "blm_add_dyt": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                        c_int, c_void_p],
    },
    "attention_sink": {
        "blm_qk_norm_append": [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_void_p],
        "blm_attention_sink": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_float, c_void_p],
        "blm_head_norm_rope_append": [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int,
                                      c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int, c_void_p],
        "blm_attention_sink_prompt_takes": [c_int, c_int, c_int, c_int, c_int, c_int],
        "blm_attention_sink_decode_takes": [c_int, c_int, c_int, c_int, c_int, c_int],
    },
    "stream_ops": {
        "blm_embed_scaled": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "blm_sandwich_norm": [c_void_p, c_void_p, c_void_p, c_float, c_float, c_int, c_void_p, c_void_p, c_void_p, c_float, c_float,
                              c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
        "blm_bias_act": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "blm_weighted_sum": [c_void_p, c_void_p, c_void_p, c_float, c_float, c_size_t, c_void_p],
        "blm_pack_cols": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_void_p],
        "blm_softcap": [c_void_p, c_float, c_size_t, c_void_p],
    },
    "recurrent": {
        "blm_causal_conv": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_longlong, c_int,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_longlong, c_longlong, c_longlong,
                            c_int, c_void_p, c_longlong, c_void_p],
        "blm_shift_mix": [c_void_p, c_longlong, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                          c_int, c_void_p, c_longlong, c_longlong, c_longlong, c_int, c_void_p],
        "blm_decay_scan": [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p, c_longlong,
                           c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                           c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_longlong, c_int, c_void_p],
        "blm_ssm_scan": [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p,
                         c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                         c_longlong, c_longlong, c_longlong, c_int, c_void_p],
        "blm_delta_scan": [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p,
                           c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int,
                           c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_longlong,
                           c_void_p],
        "blm_gated_group_norm": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                 c_float, c_void_p, c_int, c_longlong, c_int, c_void_p],
    },
    "attention_sigmoid": {
        "blm_bias_rope_append": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "blm_sigmoid_attention": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_float, c_float, c_int, c_void_p],
        "blm_sigmoid_attention_takes": [c_int, c_int, c_int, c_int, c_int, c_int],
    },
    "attention_latent": {
        "blm_latent_prepare": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p,
                               c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_void_p],
        "blm_latent_gather": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                              c_int, c_void_p],
        "blm_latent_expand": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_void_p],
        "blm_latent_attention": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                 c_void_p],
        "blm_latent_attention_tile_rows": [c_int, c_int, c_int, c_int, c_int],
        "blm_sigmoid_gate": [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p],
    },
    "moe": {
        "blm_moe_route": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                          c_void_p],
        "blm_moe_group": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
        "blm_moe_experts": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p],
        "blm_moe_down_splits": [c_int, c_int, c_int, c_int, c_int, c_int],
        "blm_moe_padded_tiles": [c_int, c_int, c_int],
        "blm_moe_group_padded": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
        "blm_moe_gather_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "blm_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    },
    "attention": {
        "blm_attention": [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
    },
    "gemm": {
        "blm_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                         c_longlong, c_void_p],
        "blm_gemm_f32_batched": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                                 c_longlong, c_longlong, c_longlong, c_void_p],
    },
    "gemv": {
        "blm_gemv": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int,
                     c_float, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p, c_int,
                     c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "blm_gemv_supported": [c_int, c_int, c_int, c_int],
    },
    "runtime": {
        "blm_graph_step": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
                           c_int, c_void_p],
        "blm_host_device_pointer": [c_void_p, c_void_p],
    },
    "gemm_tc": {
        "blm_gemm_tc": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                        c_void_p, c_void_p],
        "blm_gemm_tc_supported": [c_int, c_int, c_int],
        "blm_gemm_tc_grouped": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p,
                                c_int, c_void_p, c_void_p],
    },
    "gemm_sk": {
        "blm_gemm_sk": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p, c_int,
                        c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "blm_gemm_sk_supported": [c_int, c_int, c_int],
        "blm_gemm_sk_squares_row": [],
    },
    "sampling": {
        "blm_argmax": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_int, c_void_p],
        "blm_argmax_advances": [c_int],
        "blm_argmax_scratch_floats": [c_int, c_int],
        "blm_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, c_void_p],
    },
}
_bound: dict[str, ctypes.CDLL] = {}


def _lib(module: str) -> ctypes.CDLL:
    lib = _bound.get(module)
    if lib is None:
        lib = _build.load(module)
        for name, argtypes in _protos.get(module, {}).items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        err = getattr(lib, f"blm_{module}_last_error")
        err.restype = ctypes.c_char_p
        err.argtypes = []
        _bound[module] = lib
    return lib


def prebuild(dtype, modules=None) -> None:
    """Compile, side by side, the modules that every step of a model of this dtype uses, so that a first
    call waits for the slowest of them instead of for their sum.  The others are still built when first used.
    `modules`: the ones the model's parts name (their `kernel_modules`); None: those of the dense decoder."""
    if modules is None:
        modules = ["elementwise", "attention"]
    _build.build_many(sorted(set(modules)) + ["gemv" if dtype == torch.bfloat16 else "gemm"])


_launches = 0


def launch_count() -> int:
    """How many kernels of this package have been launched (or captured) by this process."""
    return _launches


def stream_handle() -> int:
    """torch's current stream as an integer."""
    return _stream().value or 0


def _call(module: str, name: str, *args, kernels: int = 1):
    global _launches
    lib = _lib(module)
    rc = getattr(lib, name)(*args)
    _launches += kernels
    if rc != 0:
        msg = getattr(lib, f"blm_{module}_last_error")().decode(errors="replace")
        raise KernelError(f"{name}: {msg}")


def loaded_modules():
    return sorted(_bound)


# ------------------------------------------------------------------------------------------------
def embed(tokens, table, out, hand_over=None):
    """out[n, :] = table[tokens[n], :] as fp32.  tokens int32 [N]; table [V, D]; out fp32 [N, D].
    `hand_over` = (gamma [D], scaled bfloat16 [N, D], squares float32 [1, SQUARES_ROWS]) for up to SQUARES_ROWS
    tokens: the kernel also leaves the input of the norm that reads the stream first, scaled = out * gamma and the
    rows' sums of squares in one part, as gemv's `hand_over` does."""
    _need_cuda(tokens, table, out)
    n, (v, d) = tokens.numel(), table.shape
    if tokens.dtype != torch.int32 or out.dtype != torch.float32 or tuple(out.shape) != (n, d):
        raise KernelError("embed: tokens int32 [N], out float32 [N, D]")
    gamma = scaled = squares = None
    if hand_over is not None:
        gamma, scaled, squares = hand_over
        _need_cuda(gamma, scaled, squares)
        if (n > SQUARES_ROWS or gamma.numel() != d or scaled.dtype != torch.bfloat16 or tuple(scaled.shape) != (n, d)
                or not scaled.is_contiguous() or squares.dtype != torch.float32 or tuple(squares.shape) != (1, SQUARES_ROWS)):
            raise KernelError("embed: hand_over = (gamma [D], scaled bfloat16 [N, D], squares float32 [1, 16]) for up to 16 tokens")
    _call("elementwise", "blm_embed", _ptr(tokens), _ptr(table), _code(table.dtype), _ptr(out), n, d, v,
          _ptr(gamma), 1 if (gamma is not None and gamma.dtype == torch.float32) else 0, _ptr(scaled), _ptr(squares),
          SQUARES_ROWS, _stream())


def add_rmsnorm(resid, delta, gamma, eps, out, rows=None):
    """Residual add fused with the RMS norm, in fp32.

    rows is None: resid[n] += delta[n] (stored), out[n] = norm(resid[n]) * gamma for every row.
    rows given (int32 [R]): out[i] = norm(resid[rows[i]] + delta[rows[i]]) * gamma; resid unchanged.
    delta may be None.  resid is fp32 [N, D]; delta and out have the activation dtype, or delta is float32 beside a
    bfloat16 out (a sublayer's unrounded output).  out may be resid itself (float32): the stream normed in place."""
    _need_cuda(resid, delta, gamma, out, rows)
    d = resid.shape[-1]
    n_out = rows.numel() if rows is not None else resid.shape[0]
    if resid.dtype != torch.float32 or gamma.numel() != d or tuple(out.shape) != (n_out, d):
        raise KernelError("add_rmsnorm: resid float32 [N, D], gamma [D], out [rows, D]")
    if delta is not None and ((delta.dtype != out.dtype and delta.dtype != torch.float32) or delta.shape != resid.shape):
        raise KernelError("add_rmsnorm: delta must match resid's shape and have out's dtype or float32")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("add_rmsnorm: rows must be int32")
    _call("elementwise", "blm_add_rmsnorm", _ptr(resid), _ptr(delta), _code(delta.dtype) if delta is not None else _code(out.dtype),
          _ptr(gamma), _code(gamma.dtype), _ptr(out),
          _code(out.dtype), _ptr(rows), n_out, d, c_float(eps), _stream())


def embed_pairs(tokens, table, pairs, out, step, ids_pool, block_table, buckets, mul_prev, mul_cur, norm=None):
    """out[n] = table[tokens[n]] + pairs[(previous token * mul_prev + token * mul_cur) mod buckets] as fp32 (the row
    `buckets` for a sequence's first token), then, with `norm` = (weight, bias, alpha) in float32, tanh(alpha x) * weight
    + bias.  The previous token of a portion's first row comes from the sequence's paged line of token ids `ids_pool`
    (int32 [pages, PAGE], looked up through `block_table`), to which every row appends its own token.  `step`: the
    step's tokens' sequences and positions (parts.base.StepContext)."""
    _need_cuda(tokens, table, pairs, out, ids_pool, block_table)
    n, (v, d) = tokens.numel(), table.shape
    if tokens.dtype != torch.int32 or out.dtype != torch.float32 or tuple(out.shape) != (n, d):
        raise KernelError("embed_pairs: tokens int32 [N], out float32 [N, D]")
    if pairs.dtype != table.dtype or tuple(pairs.shape) != (buckets + 1, d):
        raise KernelError(f"embed_pairs: the table of pairs must be [{buckets + 1}, {d}] in the token table's dtype")
    if ids_pool.dtype != torch.int32 or ids_pool.dim() != 2 or ids_pool.shape[1] != PAGE:
        raise KernelError(f"embed_pairs: the line of token ids must be int32 [pages, {PAGE}]")
    w = b = a = None
    if norm is not None:
        w, b, a = norm
        _need_cuda(w, b, a)
        if not (w.dtype == b.dtype == a.dtype == torch.float32) or w.numel() != d or b.numel() != d or a.numel() != 1:
            raise KernelError("embed_pairs: norm = (weight [D], bias [D], alpha []) in float32")
    _call("elementwise", "blm_embed_pairs", _ptr(tokens), _ptr(step.token_seq), _ptr(step.token_pos), _ptr(step.cu_seqlens),
          _ptr(step.slot_of_seq), _ptr(block_table), block_table.shape[1], _ptr(ids_pool), PAGE, _ptr(table), _ptr(pairs),
          _code(table.dtype), _ptr(out), n, d, v, int(buckets), int(mul_prev), int(mul_cur), _ptr(w), _ptr(b), _ptr(a), _stream())


def add_dyt(resid, deltas, weight, bias, alpha, out, rows=None):
    """Residual add fused with the Dynamic Tanh norm, in fp32: the stream takes the sum of up to three `deltas`
    (tensors of the activation dtype shaped like `resid`, or an empty list), then out = tanh(alpha x) * weight + bias.

    rows is None: resid += sum(deltas) (stored); out[n] from every row.  rows given (int32 [R]): out[i] from row rows[i]
    of resid + deltas; resid unchanged.  `out` None: the deltas are only added into the stream."""
    deltas = [t for t in (deltas or ()) if t is not None]
    _need_cuda(resid, weight, bias, alpha, out, rows, *deltas)
    d = resid.shape[-1]
    if len(deltas) > 3:
        raise KernelError("add_dyt: at most three deltas")
    if resid.dtype != torch.float32:
        raise KernelError("add_dyt: resid float32 [N, D]")
    act = out.dtype if out is not None else (deltas[0].dtype if deltas else torch.float32)
    for t in deltas:
        if t.dtype != act or t.shape != resid.shape:
            raise KernelError("add_dyt: deltas must match resid's shape and the activation dtype")
    n_out = rows.numel() if rows is not None else resid.shape[0]
    if out is not None:
        if tuple(out.shape) != (n_out, d) or weight.numel() != d or bias.numel() != d or alpha.numel() != 1 \
                or not (weight.dtype == bias.dtype == alpha.dtype == torch.float32):
            raise KernelError("add_dyt: out [rows, D]; weight [D], bias [D], alpha [] in float32")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("add_dyt: rows must be int32")
    ds = deltas + [None] * (3 - len(deltas))
    _call("elementwise", "blm_add_dyt", _ptr(resid), _ptr(ds[0]), _ptr(ds[1]), _ptr(ds[2]), _ptr(weight), _ptr(bias), _ptr(alpha),
          _ptr(out), _code(act), _ptr(rows), n_out, d, _stream())


def kv_page_elems(n_kv, key_dim, value_dim) -> int:
    """Elements of a cache page that holds its keys [n_kv, PAGE, key_dim] followed by its values [n_kv, PAGE, value_dim]."""
    return n_kv * PAGE * (key_dim + value_dim)


def _flat_pool(pool, n_kv, key_dim, value_dim):
    elems = kv_page_elems(n_kv, key_dim, value_dim)
    if not pool.is_contiguous() or pool.numel() != pool.shape[0] * elems:
        raise KernelError(f"the cache pool must hold pages of {elems} elements ({n_kv} kv heads, keys of {key_dim}, values of {value_dim})")
    return elems


def qk_norm_append(proj, step, pool, block_table, q_out, n_heads, n_kv, key_dim, value_dim, q_weight=None, k_weight=None,
                   eps=0.0, blend=None, values_in=None, values_out=None):
    """What follows a fused projection [q | k | v | ...] (float32 [N, >= (n_heads + n_kv) key_dim + n_kv value_dim]):
    q and k are each divided by the root mean square of their WHOLE row (all heads at once, eps inside the root) and
    multiplied by `q_weight` / `k_weight` (float32; None: q and k stay as they are); v becomes (1 - blend) v + blend
    values_in[n] when `values_in` (float32 [N, n_kv value_dim]) is given, `blend` a float32 scalar on the device;
    `values_out` receives v; q goes to `q_out` [N, n_heads key_dim], k and v to the token's place in the paged cache."""
    _need_cuda(proj, pool, block_table, q_out, q_weight, k_weight, blend, values_in, values_out)
    n = proj.shape[0]
    qc, kc, vc = n_heads * key_dim, n_kv * key_dim, n_kv * value_dim
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.shape[1] < qc + kc + vc:
        raise KernelError("qk_norm_append: the projection is float32 [N, q + k + v (+ more)]")
    if tuple(q_out.shape) != (n, qc) or q_out.dtype != pool.dtype:
        raise KernelError("qk_norm_append: q_out must be [N, heads * key_dim] in the cache's dtype")
    for t, size in ((q_weight, qc), (k_weight, kc), (blend, 1), (values_in, n * vc), (values_out, n * vc)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != size):
            raise KernelError("qk_norm_append: weights, blend and values are float32 of the sizes the head counts give")
    _call("attention_sink", "blm_qk_norm_append", _ptr(proj), proj.stride(0), n, n_heads, n_kv, key_dim, value_dim, _ptr(q_weight),
          _ptr(k_weight), c_float(eps), _ptr(blend), _ptr(values_in), _ptr(values_out), _ptr(q_out), _ptr(pool), _code(pool.dtype),
          _flat_pool(pool, n_kv, key_dim, value_dim), PAGE, _ptr(step.token_seq), _ptr(step.token_pos), _ptr(step.slot_of_seq),
          _ptr(block_table), block_table.shape[1], _stream())


def head_norm_rope_append(proj, step, pool, block_table, q_out, n_heads, n_kv, key_dim, value_dim, q_weight=None, k_weight=None,
                          eps=0.0, value_norm=False, freq=None, rotary_dims=0, halves=False):
    """What follows a fused projection [q | k | v | ...] (float32 [N, >= (n_heads + n_kv) key_dim + n_kv value_dim]), head by
    head: every head of q is divided by its root mean square (eps inside the root) and multiplied by `q_weight` (float32
    [key_dim], the same for all heads; None: q stays as it is), every head of k likewise with `k_weight`; the first
    `rotary_dims` lanes of every q and k head turn by position * freq[i] (freq float64 [rotary_dims / 2]), lanes (2i, 2i + 1)
    together, or (i, i + rotary_dims / 2) with `halves`; with `value_norm` every head of v is divided by its root mean square
    (no weight).  q goes to `q_out` [N, n_heads key_dim], k and v to the token's place in the paged cache."""
    _need_cuda(proj, pool, block_table, q_out, q_weight, k_weight, freq)
    _f32(proj, q_weight, k_weight)
    n = proj.shape[0]
    qc, kc, vc = n_heads * key_dim, n_kv * key_dim, n_kv * value_dim
    if proj.dim() != 2 or proj.shape[1] < qc + kc + vc or proj.stride(1) != 1:
        raise KernelError("head_norm_rope_append: the projection is float32 [N, q + k + v (+ more)]")
    if tuple(q_out.shape) != (n, qc) or q_out.dtype != pool.dtype or not q_out.is_contiguous():
        raise KernelError("head_norm_rope_append: q_out must be [N, heads * key_dim] in the cache's dtype")
    for t in (q_weight, k_weight):
        if t is not None and t.numel() != key_dim:
            raise KernelError("head_norm_rope_append: the norms' weights are float32 [key_dim]")
    if rotary_dims and (freq is None or freq.dtype != torch.float64 or freq.numel() != rotary_dims // 2):
        raise KernelError("head_norm_rope_append: freq must be float64 [rotary_dims / 2]")
    _call("attention_sink", "blm_head_norm_rope_append", _ptr(proj), c_longlong(proj.stride(0)), n, n_heads, n_kv, key_dim, value_dim,
          _ptr(q_weight), _ptr(k_weight), c_float(eps), 1 if value_norm else 0, _ptr(freq), int(rotary_dims), 1 if halves else 0,
          _ptr(q_out), _ptr(pool), _code(pool.dtype), c_longlong(_flat_pool(pool, n_kv, key_dim, value_dim)), PAGE, _ptr(step.token_seq),
          _ptr(step.token_pos), _ptr(step.slot_of_seq), _ptr(block_table), block_table.shape[1], _stream())


def attention_sink_scratch_floats(n_tokens, n_heads, value_dim, n_splits) -> int:
    return 0 if n_splits <= 1 else n_tokens * n_heads * n_splits * (value_dim + 2)


def attention_sink_prompt_takes(dtype, key_dim, value_dim, max_q_len, n_heads) -> bool:
    """Whether a step of this shape runs the tensor-core prompt kernel (else the row kernel, which takes every shape)."""
    return bool(_lib("attention_sink").blm_attention_sink_prompt_takes(_code(dtype), key_dim, value_dim, PAGE, max_q_len, n_heads))


def attention_sink_decode_takes(dtype, key_dim, value_dim, n_heads, n_kv) -> bool:
    """Whether single tokens and short portions of this shape run the tensor-core decode kernel, whose splits are cut by
    pages (else the row kernel, which takes every shape and cuts its splits by chunks of 32 keys)."""
    return bool(_lib("attention_sink").blm_attention_sink_decode_takes(_code(dtype), key_dim, value_dim, PAGE, n_heads, n_kv))


def attention_sink(q, step, pool, block_table, out, n_heads, n_kv, key_dim, value_dim, scale, window, keep_first=0, sink=True,
                   gate=None, gate_stride=0, max_q_len=1, n_splits=1, scratch=None, head_scale=None, sink_logit=None, softcap=0.0):
    """Attention of the step's tokens over the paged cache (after the append) where the query at position i sees the
    key at j when j <= i and (i - j < window or j < keep_first); softmax with `sink` added to its denominator (one more
    entry of score 0 without a value); keys of `key_dim` and values of `value_dim` lanes; `gate`: a float32 tensor
    whose element n * gate_stride + h is squashed by a sigmoid and multiplies head h's output of token n.
    q [N, n_heads key_dim] and out [N, n_heads value_dim] in the cache's dtype.
    `head_scale` float32 [n_heads]: head h's scores are scale * head_scale[h] * q.k; `softcap` > 0: a score s becomes
    softcap * tanh(s / softcap) before the softmax; `sink_logit` float32 [n_heads]: the sink's score is that number instead
    of 0 (exp(sink_logit[h]) joins the denominator).

    `max_q_len`: the longest run of new tokens of one sequence (a bound is enough): bfloat16 steps of 8 or more run
    the tensor-core prompt kernel, 64 query rows a block (it reads step.cu_seqlens and step.start_pos); shorter ones
    the tensor-core decode kernel (bfloat16, up to 16 query heads a kv head) or else the row kernel, a block per (row,
    kv head) either, whose keys `n_splits` > 1 cuts over that many blocks (it then needs `scratch`:
    attention_sink_scratch_floats(...) float32)."""
    _need_cuda(q, pool, block_table, out, scratch, head_scale, sink_logit)
    _f32(head_scale, sink_logit)
    for t in (head_scale, sink_logit):
        if t is not None and t.numel() != n_heads:
            raise KernelError("attention_sink: head_scale and sink_logit have a number per query head")
    n = q.shape[0]
    if tuple(q.shape) != (n, n_heads * key_dim) or tuple(out.shape) != (n, n_heads * value_dim) or q.dtype != pool.dtype \
            or out.dtype != pool.dtype:
        raise KernelError("attention_sink: q [N, heads * key_dim] and out [N, heads * value_dim] in the cache's dtype")
    if gate is not None and (not gate.is_cuda or gate.dtype != torch.float32):
        raise KernelError("attention_sink: the gate is float32")
    prompt = attention_sink_prompt_takes(pool.dtype, key_dim, value_dim, max_q_len, n_heads) and getattr(step, "cu_seqlens", None) is not None
    if prompt:
        n_splits = 1
    if n_splits > 1:
        need = attention_sink_scratch_floats(n, n_heads, value_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_sink: {n_splits} splits need {need} float32 of scratch")
    cu = step.cu_seqlens if prompt else None
    _call("attention_sink", "blm_attention_sink", _ptr(q), _ptr(pool), _code(pool.dtype), _flat_pool(pool, n_kv, key_dim, value_dim),
          _ptr(block_table), block_table.shape[1], _ptr(step.token_seq), _ptr(step.token_pos), _ptr(step.slot_of_seq), _ptr(cu),
          _ptr(step.start_pos if prompt else None), (cu.numel() - 1) if prompt else 0, int(max_q_len), _ptr(gate), int(gate_stride),
          _ptr(out), _ptr(scratch), int(n_splits), n, n_heads, n_kv, key_dim, value_dim, PAGE, int(window), int(keep_first),
          c_float(scale), 1 if sink else 0, _ptr(head_scale), _ptr(sink_logit if sink else None), c_float(softcap or 0.0), _stream(),
          kernels=2 if n_splits > 1 else 1)


def moe_route(h, router, top, softmax=False, correction=None, renormalise=False, n_groups=1, keep_groups=1):
    """(ids int32 [N, top], weights float32 [N, top]): every token's `top` experts of largest sigmoid(router h), in
    falling order (the lower index on a tie), with those scores.  router float32 [experts, D]; sums in float32.
    `softmax`: the scores are softmax(router h) over all experts.  `correction` float32 [experts]: added to the scores for
    the choice only; the weights stay the scores.  `renormalise`: the chosen weights are divided by their sum + 1e-20.
    `n_groups` > 1: the experts form that many equal groups of neighbours, a group's mark is the sum of its two largest
    choice scores (correction included), and only experts of the `keep_groups` groups of largest mark can be chosen."""
    _need_cuda(h, router, correction)
    _f32(correction)
    if correction is not None and correction.numel() != router.shape[0]:
        raise KernelError("moe_route: the correction has a number per expert")
    n, d = h.shape
    if router.dtype != torch.float32 or router.dim() != 2 or router.shape[1] != d:
        raise KernelError("moe_route: the router is float32 [experts, D]")
    ids = torch.empty((n, top), dtype=torch.int32, device=h.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=h.device)
    _call("moe", "blm_moe_route", _ptr(h), _code(h.dtype), _ptr(router), n, d, router.shape[0], top, _ptr(ids), _ptr(weights),
          1 if softmax else 0, _ptr(correction), 1 if renormalise else 0, int(n_groups), int(keep_groups if n_groups > 1 else 1), _stream())
    return ids, weights


UNIT_GATED, UNIT_GELU, UNIT_GELU_TANH = 0, 1, 2      # an expert's unit: gated (silu or clamped); W_down gelu(W_up x), exact or tanh form


def moe_experts(h, ids, weights, gate_up, down, extra=None, weight_on_input=True, clamp_limit=0.0, clamp_alpha=1.702, out_dtype=None,
                unit=UNIT_GATED):
    """sum over a token's chosen experts of expert(weight h) (`weight_on_input`) or of weight expert(h), plus `extra`
    [N, D] when given; expert(x) = down[e] (silu(gate[e] x) * (up[e] x)).  gate_up [experts, 2 ff, D] (an expert's
    gate rows, then its up rows) and down [experts, D, ff] in h's dtype.  Returns [N, D] in h's dtype, or in float32
    (`out_dtype`).  `clamp_limit` > 0: the experts' unit is the clamped one, g = min(gate x, limit), u = clamp(up x, -limit,
    limit), g sigmoid(clamp_alpha g) (u + 1).  `unit` UNIT_GELU or UNIT_GELU_TANH: the experts have no gate,
    expert(x) = down[e] gelu(up[e] x), and `gate_up` is [experts, ff, D], the up rows alone."""
    _need_cuda(h, ids, weights, gate_up, down, extra)
    n, d = h.shape
    top = ids.shape[1]
    e, rows, _ = gate_up.shape
    ff = rows // 2 if unit == UNIT_GATED else rows
    if (gate_up.dtype != h.dtype or down.dtype != h.dtype or tuple(gate_up.shape) != (e, (2 if unit == UNIT_GATED else 1) * ff, d)
            or tuple(down.shape) != (e, d, ff)):
        raise KernelError("moe_experts: gate_up [experts, 2 ff, D] (ff rows without a gate) and down [experts, D, ff] in the activations' dtype")
    if ids.dtype != torch.int32 or weights.dtype != torch.float32 or tuple(weights.shape) != (n, top):
        raise KernelError("moe_experts: ids int32 [N, top], weights float32 [N, top]")
    if extra is not None and (extra.dtype != h.dtype or tuple(extra.shape) != (n, d)):
        raise KernelError("moe_experts: extra must be [N, D] in the activations' dtype")
    dev = h.device
    pairs = n * top
    if (unit == UNIT_GELU and not weight_on_input and h.dtype == torch.bfloat16 and pairs >= MOE_TC_PAIRS * e and d % 8 == 0 and ff % 8 == 0
            and d >= 64 and ff >= 64 and e * max(d, ff) < (1 << 31)):
        return _moe_experts_tc(h, ids, weights, gate_up, down, extra, out_dtype or h.dtype)
    offsets = torch.empty(e + 1, dtype=torch.int32, device=dev)
    order = torch.empty(pairs, dtype=torch.int32, device=dev)
    place_of = torch.empty(pairs, dtype=torch.int32, device=dev)
    act = torch.empty((pairs, ff), dtype=h.dtype, device=dev)
    # steps that bring an expert a few tokens cut the second product's reduction over several blocks: a plane of sums each
    planes = int(_lib("moe").blm_moe_down_splits(_code(h.dtype), n, d, ff, e, top))
    y = torch.empty((planes, pairs, d), dtype=torch.float32, device=dev)
    out = torch.empty((n, d), dtype=out_dtype or h.dtype, device=dev)
    stream = _stream()
    _call("moe", "blm_moe_group", _ptr(ids), pairs, e, _ptr(offsets), _ptr(order), _ptr(place_of), stream)
    _call("moe", "blm_moe_experts", _ptr(h), _code(h.dtype), _ptr(weights), _ptr(order), _ptr(offsets), _ptr(gate_up), _ptr(down),
          _ptr(act), _ptr(y), n, d, ff, e, top, 1 if weight_on_input else 0, c_float(clamp_limit), c_float(clamp_alpha), int(unit), planes, stream, kernels=2)
    _call("moe", "blm_moe_combine", _ptr(y), _ptr(place_of), _ptr(weights), _ptr(extra), _ptr(out), _code(h.dtype), n, d, top,
          0 if weight_on_input else 1, _code(out.dtype), planes, stream)
    return out


# from this many (token, expert) pairs an expert on average, experts without a gate run on tcgen05 (BURN_LM_B200_MOE_TC_PAIRS=n
# to measure another border)
MOE_TC_PAIRS = int(os.environ.get("BURN_LM_B200_MOE_TC_PAIRS", "16"))
MOE_TC_ROWS = 128       # rows of a tile of the tcgen05 product: an expert's share of the pairs starts at a multiple of it


def _moe_experts_tc(h, ids, weights, up, down, extra, out_dtype):
    """Experts without a gate for prompts, both products on the tcgen05 tensor cores: the pairs' token rows are gathered expert
    by expert, every expert's share starting at a multiple of 128 places (a place no pair owns holds zeros), and one grouped
    product runs over all experts at once (kernels of gemm_tc.cu: a table names the expert of every tile of places); the
    first product's epilogue applies the exact GELU, the second leaves fp32 sums, and the sum over a token's experts weighs
    them as ever.  Everything is sized by the token count alone, so a step can be captured."""
    n, d = h.shape
    e, ff, _ = up.shape
    top = ids.shape[1]
    pairs, dev, stream = n * top, h.device, _stream()
    tiles = int(_lib("moe").blm_moe_padded_tiles(pairs, e, MOE_TC_ROWS))
    places = tiles * MOE_TC_ROWS
    place_of = torch.empty(pairs, dtype=torch.int32, device=dev)
    pair_of_place = torch.empty(places, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(tiles, dtype=torch.int32, device=dev)
    xs = torch.empty((places, d), dtype=torch.bfloat16, device=dev)
    act = torch.empty((places, ff), dtype=torch.bfloat16, device=dev)
    y = torch.empty((places, d), dtype=torch.float32, device=dev)
    out = torch.empty((n, d), dtype=out_dtype, device=dev)
    status = status_word(dev)
    _call("moe", "blm_moe_group_padded", _ptr(ids), pairs, e, MOE_TC_ROWS, _ptr(place_of), _ptr(pair_of_place), _ptr(tile_expert), stream)
    _call("moe", "blm_moe_gather_rows", _ptr(h), _ptr(pair_of_place), _ptr(xs), places, d, top, stream)
    _call("gemm_tc", "blm_gemm_tc_grouped", _ptr(xs), c_longlong(d), _ptr(up), c_longlong(d), _ptr(act), c_longlong(ff), places, ff, d, e,
          _ptr(tile_expert), 3, _ptr(status), stream)
    _call("gemm_tc", "blm_gemm_tc_grouped", _ptr(act), c_longlong(ff), _ptr(down), c_longlong(ff), _ptr(y), c_longlong(d), places, d, ff, e,
          _ptr(tile_expert), 4, _ptr(status), stream)
    _call("moe", "blm_moe_combine", _ptr(y), _ptr(place_of), _ptr(weights), _ptr(extra), _ptr(out), _code(h.dtype), n, d, top,
          1, _code(out.dtype), 1, stream)
    return out


def rope_table(inv_freq, n_positions):
    """(cos, sin) of position * inv_freq for positions below n_positions: float32 [n_positions, half, 2],
    computed in float64 on the device; rope_append reads it instead of computing angles per token."""
    _need_cuda(inv_freq)
    half = inv_freq.numel()
    table = torch.empty((n_positions, half, 2), dtype=torch.float32, device=inv_freq.device)
    _call("elementwise", "blm_rope_table", _ptr(inv_freq), _ptr(table), n_positions, half, _stream())
    return table


PAIRS_HALVES, PAIRS_INTERLEAVED, PAIRS_TILED = 0, 1, 2


def rope_append(qkv, token_seq, token_pos, slot_of_seq, block_table, inv_freq, rotary_dim, interleaved,
                pool, n_heads, n_kv, head_dim, write_cache=True, table=None, max_position=None):
    """Rotate q (in place) and k of every token by its position, and append k, v to the paged cache.

    `interleaved`: False or PAIRS_HALVES: pair i is lanes (i, i + rotary_dim / 2); True or
    PAIRS_INTERLEAVED: lanes (2i, 2i + 1); PAIRS_TILED: lanes (16 (i // 8) + i % 8, that + 8), the order
    of a head whose weight rows were dealt out with tiled_pair_order().

    qkv [N, (n_heads + 2 n_kv) * head_dim]; pool [pages, 2, n_kv, PAGE, head_dim] of one cache line;
    inv_freq float64 [rotary_dim / 2] or None when rotary_dim == 0; `table` (from rope_table) spares
    the per-token angles for positions it covers.  `max_position`: an upper bound of the step's
    positions known on the host; when the table covers it, the vector kernel may run."""
    _need_cuda(qkv, token_seq, token_pos, slot_of_seq, block_table, inv_freq, pool, table)
    if table is not None and (table.dtype != torch.float32 or tuple(table.shape[1:]) != (rotary_dim // 2, 2)):
        raise KernelError("rope_append: table must be float32 [positions, rotary_dim / 2, 2]")
    n = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("rope_append: qkv width does not match the head counts")
    if write_cache:
        if pool.dtype != qkv.dtype or tuple(pool.shape[1:]) != (2, n_kv, PAGE, head_dim):
            raise KernelError(f"rope_append: pool must be [pages, 2, {n_kv}, {PAGE}, {head_dim}] of {qkv.dtype}")
    if rotary_dim:
        if inv_freq.dtype != torch.float64 or inv_freq.numel() != rotary_dim // 2:
            raise KernelError("rope_append: inv_freq must be float64 [rotary_dim / 2]")
    _call("elementwise", "blm_rope_append", _ptr(qkv), _code(qkv.dtype), _ptr(token_seq), _ptr(token_pos),
          _ptr(slot_of_seq), _ptr(block_table), block_table.shape[1], _ptr(inv_freq), rotary_dim,
          int(interleaved), _ptr(pool), n, n_heads, n_kv, head_dim, PAGE, 1 if write_cache else 0,
          _ptr(table), table.shape[0] if table is not None else 0,
          1 if (table is not None and max_position is not None and max_position < table.shape[0]) else 0, _stream())


def tiled_pair_order(head_dim: int) -> list:
    """For PAIRS_TILED: which lane of a head (in the stored order, pairs (i, i + head_dim / 2)) goes to each
    place: every 16 places hold lanes 8j .. 8j + 7 and then their partners."""
    half = head_dim // 2
    return [(8 * (p // 16) + p % 16) if p % 16 < 8 else (half + 8 * (p // 16) + p % 16 - 8) for p in range(head_dim)]


GATE_TILE = 8   # a fused [gate; up] weight for the skinny kernel: tiles of 8 gate rows, then their 8 up rows


def swiglu(gate_up, out, tile=0):
    """out[n, i] = silu(gate_i) * up_i.  gate_up [N, 2 I] holds all gates then all ups (tile 0), or
    tiles of `tile` gates followed by the ups of the same outputs."""
    _need_cuda(gate_up, out)
    n, two_i = gate_up.shape
    if tuple(out.shape) != (n, two_i // 2) or out.dtype != gate_up.dtype or two_i % 2:
        raise KernelError("swiglu: out must be [N, I] for gate_up [N, 2 I], same dtype")
    _call("elementwise", "blm_swiglu", _ptr(gate_up), _ptr(out), _code(out.dtype), n, two_i // 2, tile, _stream())


def convert(src, dst):
    """dst = src in the other of float32 / bfloat16."""
    _need_cuda(src, dst)
    if src.numel() != dst.numel():
        raise KernelError("convert: sizes differ")
    _call("elementwise", "blm_convert", _ptr(src), _code(src.dtype), _ptr(dst), _code(dst.dtype),
          c_size_t(src.numel()), _stream())


def decode_advance(tokens, pos, sampled, history, step_no, counters=None):
    """Between two decode steps that run without the host: tokens = sampled, pos += 1 (and counters += 1),
    history[step_no] = sampled, step_no += 1.  All int32 on the device (counters int64)."""
    _need_cuda(tokens, pos, sampled, history, step_no, counters)
    b = tokens.numel()
    steps = history.shape[0] if history is not None else 0
    _call("elementwise", "blm_decode_advance", _ptr(tokens), _ptr(pos), _ptr(sampled), _ptr(history), _ptr(step_no),
          _ptr(counters), b, steps, _stream(), kernels=2)


def step_tables(token_seq, token_pos, slot_of_seq, block_table, n_seqs):
    """Looked up once per step for all layers that share a block table: (token_page int32 [N], the page every new
    token goes to, -1 for a row of no sequence; seq_table int32 [n_seqs, pages per sequence], the block table's
    rows in the order of the step's sequences)."""
    _need_cuda(token_seq, token_pos, slot_of_seq, block_table)
    n = token_seq.numel()
    token_page = torch.empty(n, dtype=torch.int32, device=block_table.device)
    seq_table = torch.empty((n_seqs, block_table.shape[1]), dtype=torch.int32, device=block_table.device)
    _call("elementwise", "blm_step_tables", _ptr(token_seq), _ptr(token_pos), _ptr(slot_of_seq), _ptr(block_table),
          block_table.shape[1], PAGE, n, n_seqs, _ptr(token_page), _ptr(seq_table), _stream())
    return token_page, seq_table


def attention_decode_is_specialised(dtype, head_dim, group) -> bool:
    """Whether a step of one token per sequence runs the specialised decode kernel (whose blocks
    split the keys by pages and skip splits a sequence does not need)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and 1 <= group <= 8


def attention_scratch_floats(n_tokens, n_heads, head_dim, n_splits):
    return 0 if n_splits <= 1 else n_tokens * n_heads * n_splits * (head_dim + 2)


def attention(q, q_stride, pool, block_table, cu_seqlens, slot_of_seq, start_pos, out, n_tokens, n_seqs,
              max_q_len, n_heads, n_kv, head_dim, scale, window=0, n_splits=1, scratch=None, general_only=False,
              max_kv_len=0, seq_table=None, ahead=False):
    """Causal grouped-query attention of the step's tokens over the paged cache (after the append).

    q: tensor whose token n, head h starts at element n * q_stride + h * head_dim (the qkv buffer).
    Token t of sequence s sits at position start_pos[s] + t and sees keys 0..that position (the last
    `window` of them when window > 0).  n_splits > 1 cuts every sequence's keys over that many
    blocks and combines the partial results; it needs `scratch` (float32,
    attention_scratch_floats(...) elements).  bfloat16 steps of one token per sequence with a head
    size of 64 or 128 and up to 8 query heads per kv head run a specialised kernel unless
    `general_only`; `max_kv_len` (the longest sequence after the step, when known) lets it size its
    rings of pages; `seq_table` (from step_tables) spares it the way through the slots.  `ahead`: the kernel
    launched just before this one was gemv() with `rope`, which lets its successor start only after its own wait;
    the specialised kernel then reads the step's tables and fetches the pages of earlier tokens before it waits
    for that kernel itself (for q and the page of the new token).  Say so only when it is so."""
    _need_cuda(q, pool, block_table, cu_seqlens, slot_of_seq, start_pos, out, scratch, seq_table)
    if seq_table is not None and (seq_table.dtype != torch.int32 or tuple(seq_table.shape) != (n_seqs, block_table.shape[1])):
        raise KernelError("attention: seq_table must be int32 [n_seqs, pages per sequence]")
    if tuple(out.shape) != (n_tokens, n_heads * head_dim) or out.dtype != q.dtype or pool.dtype != q.dtype:
        raise KernelError("attention: out must be [N, heads * head_dim] in q's dtype, as the pool")
    if tuple(pool.shape[1:]) != (2, n_kv, PAGE, head_dim):
        raise KernelError(f"attention: pool must be [pages, 2, {n_kv}, {PAGE}, {head_dim}]")
    if n_splits > 1:
        need = attention_scratch_floats(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention: {n_splits} splits need {need} float32 of scratch")
    _call("attention", "blm_attention", _ptr(q), q_stride, _ptr(pool), _code(q.dtype), _ptr(block_table),
          block_table.shape[1], _ptr(cu_seqlens), _ptr(slot_of_seq), _ptr(start_pos), _ptr(out), _ptr(scratch),
          n_tokens, n_seqs, max_q_len, n_heads, n_kv, head_dim, PAGE, int(window or 0), n_splits,
          c_float(scale), 1 if general_only else 0, _ptr(status_word(q.device)), pool.shape[0], int(max_kv_len), _ptr(seq_table),
          1 if ahead else 0, _stream(), kernels=2 if n_splits > 1 else 1)


def gemm_f32(x, w, out=None):
    """x [N, K] times w [M, K] transposed, in true fp32 (no tensor-core mode)."""
    _need_cuda(x, w, out)
    if x.dtype != torch.float32 or w.dtype != torch.float32 or x.shape[1] != w.shape[1]:
        raise KernelError("gemm_f32: float32 x [N, K] and w [M, K]")
    n, k = x.shape
    m = w.shape[0]
    if out is None:
        out = torch.empty((n, m), dtype=torch.float32, device=x.device)
    elif tuple(out.shape) != (n, m) or out.dtype != torch.float32:
        raise KernelError("gemm_f32: out must be float32 [N, M]")
    _call("gemm", "blm_gemm_f32", _ptr(x), _ptr(w), _ptr(out), n, m, k, k, k, m, _stream())
    return out


def batched_product(x, w, out=None, out_dtype=None):
    """out[b] = x[b] w[b]^T for a batch of small products of one shape: x [B, N, K], w [B, M, K], out [B, N, M]; the
    operands may be strided views (rows a fixed distance apart, unit stride along K and M).  float32 operands run this
    package's FFMA product, true 32-bit; bfloat16 operands the library's batched product, as the plain products of a
    prompt do, with a bfloat16 or (`out_dtype`) float32 result."""
    _need = [t for t in (x, w, out) if t is not None]
    for t in _need:
        if not t.is_cuda:
            raise KernelError("burn-lm_b200 kernels run on a CUDA device only; got a CPU tensor")
    b, n, k = x.shape
    m = w.shape[1]
    if tuple(w.shape) != (b, m, k) or x.dtype != w.dtype:
        raise KernelError("batched_product: x [B, N, K] and w [B, M, K] of one dtype")
    if x.dtype == torch.float32:
        if out is None:
            out = torch.empty((b, n, m), dtype=torch.float32, device=x.device)
        if out.dtype != torch.float32 or tuple(out.shape) != (b, n, m) or any(t.stride(2) != 1 for t in (x, w, out)):
            raise KernelError("batched_product: float32 out [B, N, M]; unit stride along the last axis")
        _call("gemm", "blm_gemm_f32_batched", _ptr(x), _ptr(w), _ptr(out), b, n, m, k, c_longlong(x.stride(1)), c_longlong(w.stride(1)),
              c_longlong(out.stride(1)), c_longlong(x.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)), _stream())
        return out
    if out is not None:
        return torch.bmm(x, w.transpose(1, 2), out=out)
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.bmm(x, w.transpose(1, 2), out_dtype=out_dtype)
    return torch.bmm(x, w.transpose(1, 2))


EPI_STORE, EPI_SWIGLU, EPI_RESID_ADD, EPI_ROPE = 0, 1, 2, 3


class _GemvRope(ctypes.Structure):
    _fields_ = [("token_pos", c_void_p), ("token_seq", c_void_p), ("slot_of_seq", c_void_p), ("block_table", c_void_p),
                ("table", c_void_p), ("pool", c_void_p), ("table_stride", c_int), ("n_heads", c_int), ("n_kv", c_int),
                ("hd", c_int), ("page_size", c_int), ("write_cache", c_int), ("token_page", c_void_p)]


def gemv_supported(n_tokens, m, k, plain_tokens=False) -> bool:
    """Whether gemv() takes the shape.  `plain_tokens`: the input is a bfloat16 [N, K] tensor used row by row
    (no stream to normalise, no gathered rows): then a very wide K is taken too."""
    return bool(_lib("gemv").blm_gemv_supported(n_tokens, m, k, 1 if plain_tokens else 0))


def gemm_tc_supported(m, n, k) -> bool:
    return bool(_lib("gemm_tc").blm_gemm_tc_supported(m, n, k))


def gemm_tc(x, w, out=None, swiglu=False, add_into=None):
    """x [M, K] times w [N, K] transposed on the tcgen05 tensor cores (bfloat16, fp32 accumulation in
    tensor memory).  out [M, N]; with `swiglu`, w is a fused gate/up weight in tiles of GATE_TILE gate
    rows followed by their up rows and out [M, N / 2] = silu(gate) * up, formed in the epilogue; with
    `add_into` (float32 [M, N], the residual stream) the product is added into it in the epilogue and
    nothing else is written."""
    _need_cuda(x, w, out, add_into)
    m, k = x.shape
    n = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k:
        raise KernelError("gemm_tc: bfloat16 x [M, K] and w [N, K]")
    if add_into is not None:
        if swiglu or out is not None or add_into.dtype != torch.float32 or tuple(add_into.shape) != (m, n) or add_into.stride(1) != 1:
            raise KernelError("gemm_tc: add_into must be float32 [M, N], alone")
        _call("gemm_tc", "blm_gemm_tc", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(add_into), add_into.stride(0), m, n, k,
              2, _ptr(status_word(x.device)), _stream())
        return
    if out is None or out.dtype != torch.bfloat16 or tuple(out.shape) != (m, n // 2 if swiglu else n):
        raise KernelError("gemm_tc: out must be bfloat16 [M, N] (or [M, N / 2] with the gated epilogue)")
    _call("gemm_tc", "blm_gemm_tc", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), m, n, k,
          1 if swiglu else 0, _ptr(status_word(x.device)), _stream())


SK_SQUARES_ROWS = 64     # row length of the sums of squares that go with a norm handed over between gemm_sk products
SK_TOKENS = 128          # gemm_sk takes up to this many tokens


def gemm_sk_supported(n_tokens, m, k) -> bool:
    return bool(_lib("gemm_sk").blm_gemm_sk_supported(n_tokens, m, k))


def gemm_sk(w, x, out=None, add_into=None, swiglu=False, squares=None, eps=0.0, hand_over=None, rope=None):
    """x [N, K] times w [M, K] transposed for up to 128 tokens on the tcgen05 tensor cores, the weight rows as the
    wide operand, K cut over the blocks of a cluster where the weight has few rows; bfloat16 operands, fp32 sums.

    Ends, one at a time: `out` [N, M] bfloat16 or float32; `swiglu`: w is [2 I, K] in tiles of GATE_TILE gate rows
    followed by their up rows and out [N, I] = silu(gate) * up; `add_into` (fp32 [N, M]) += the product, with
    `hand_over` = (gamma, scaled bfloat16 [N, M], squares float32 [ceil(M / 16), SK_SQUARES_ROWS]) also the next
    norm's input; `rope` (as for gemv): w is a step's [q; k; v] with q and k rows in tiled_pair_order(), q goes
    to `out`, the rotated k and the v to the cache.  `squares` (+ `eps`): x is a handed-over norm,
    bfloat16(stream * gamma), and the results' rows are divided by the stream rows' root mean square."""
    _need_cuda(w, x, out, add_into, squares)
    if w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KernelError("gemm_sk: bfloat16 x [N, K] and w [M, K]")
    n, k = x.shape
    m_rows = w.shape[0]
    m = m_rows // 2 if swiglu else m_rows
    epi = EPI_SWIGLU if swiglu else (EPI_RESID_ADD if add_into is not None else (EPI_ROPE if rope is not None else EPI_STORE))
    if sum(v is not None and v is not False for v in (add_into, rope, swiglu or None)) > 1:
        raise KernelError("gemm_sk: one epilogue at a time")
    rope_arg = None
    if rope is not None:
        r = rope
        hd, table, pool = r["head_dim"], r["table"], r["pool"]
        _need_cuda(r["token_pos"], r["token_seq"], r["slot_of_seq"], r["block_table"], table, pool)
        if table is None or table.dtype != torch.float32 or tuple(table.shape[1:]) != (hd // 2, 2) \
                or r.get("max_position") is None or r["max_position"] >= table.shape[0]:
            raise KernelError("gemm_sk: the rotary epilogue needs a table [positions, head_dim / 2, 2] that covers the step")
        if r["write_cache"] and (pool.dtype != torch.bfloat16 or tuple(pool.shape[1:]) != (2, r["n_kv"], PAGE, hd)):
            raise KernelError(f"gemm_sk: pool must be bfloat16 [pages, 2, {r['n_kv']}, {PAGE}, {hd}]")
        if out is None or out.dtype != torch.bfloat16 or tuple(out.shape) != (n, r["n_heads"] * hd):
            raise KernelError("gemm_sk: the rotary epilogue writes q to a bfloat16 out [N, n_heads * head_dim]")
        rope_arg = _GemvRope(r["token_pos"].data_ptr(), r["token_seq"].data_ptr(), r["slot_of_seq"].data_ptr(),
                             r["block_table"].data_ptr(), table.data_ptr(), pool.data_ptr() if pool is not None else 0,
                             r["block_table"].shape[1], r["n_heads"], r["n_kv"], hd, PAGE, 1 if r["write_cache"] else 0,
                             r["token_page"].data_ptr() if r.get("token_page") is not None else 0)
    if squares is not None and (squares.dtype != torch.float32 or squares.dim() != 2 or squares.shape[1] != SK_SQUARES_ROWS
                                or n > SK_SQUARES_ROWS):
        raise KernelError(f"gemm_sk: squares are float32 [parts, {SK_SQUARES_ROWS}] for up to {SK_SQUARES_ROWS} tokens")
    next_gamma = scaled = squares_out = None
    if hand_over is not None:
        next_gamma, scaled, squares_out = hand_over
        _need_cuda(next_gamma, scaled, squares_out)
        if (epi != EPI_RESID_ADD or scaled.dtype != torch.bfloat16 or tuple(scaled.shape) != (n, m) or squares_out.dtype != torch.float32
                or tuple(squares_out.shape) != ((m + 15) // 16, SK_SQUARES_ROWS) or next_gamma.numel() != m or n > SK_SQUARES_ROWS):
            raise KernelError(f"gemm_sk: hand_over = (gamma [M], scaled bfloat16 [N, M], squares float32 [ceil(M / 16), {SK_SQUARES_ROWS}]) "
                              "with add_into")
    if epi == EPI_RESID_ADD:
        if add_into.dtype != torch.float32 or tuple(add_into.shape) != (n, m):
            raise KernelError("gemm_sk: add_into must be float32 [N, M]")
    elif epi != EPI_ROPE and (out is None or tuple(out.shape) != (n, m) or out.dtype not in (torch.bfloat16, torch.float32)
                              or (swiglu and out.dtype != torch.bfloat16)):
        raise KernelError("gemm_sk: out must be [N, M] bfloat16 (or float32 for a plain store)")
    _call("gemm_sk", "blm_gemm_sk", _ptr(w), w.stride(0), m_rows, k, _ptr(x), x.stride(0), n, _ptr(out),
          out.stride(0) if out is not None else 0, 1 if (out is not None and out.dtype == torch.float32) else 0, _ptr(add_into), epi,
          _ptr(squares), squares.shape[0] if squares is not None else 0, c_float(eps), _ptr(next_gamma),
          1 if (next_gamma is not None and next_gamma.dtype == torch.float32) else 0, _ptr(scaled), _ptr(squares_out),
          ctypes.byref(rope_arg) if rope_arg is not None else None, _ptr(status_word(w.device)), _stream())


def graph_step(graph_exec: int, dev_in, host_in, host_out, dev_out, dev_in2=None, host_in2=None, written_by_graph=False):
    """One captured step driven from native code: host_in (pinned) -> dev_in (and host_in2 -> dev_in2), the
    instantiated graph `graph_exec` (a cudaGraphExec_t as an integer), dev_out -> host_out (pinned), and the
    wait, on the current stream.  `written_by_graph`: the graph's last kernel writes host_out itself (int32 >= 0,
    see `argmax`'s `mirror`); then nothing is copied out and the call returns as soon as every entry is there.

    Returns a function of no arguments that does the same again (same buffers, same stream) at the cost of one
    foreign call: every argument is converted once, here."""
    nbytes = lambda t: t.numel() * t.element_size() if t is not None else 0
    fn = getattr(_lib("runtime"), "blm_graph_step")
    args = (c_void_p(graph_exec), _ptr(dev_in), c_void_p(host_in.data_ptr()), nbytes(host_in),
            _ptr(dev_in2), c_void_p(host_in2.data_ptr()) if host_in2 is not None else c_void_p(0), nbytes(host_in2),
            c_void_p(host_out.data_ptr()), _ptr(dev_out), nbytes(host_out), 1 if written_by_graph else 0, _stream())

    def again():
        if fn(*args) != 0:
            raise KernelError("graph_step: " + _lib("runtime").blm_runtime_last_error().decode(errors="replace"))
    again()
    return again


def host_device_pointer(pinned) -> int:
    """The address under which kernels see a pinned host tensor."""
    if not pinned.is_pinned():
        raise KernelError("host_device_pointer: the tensor is not in pinned host memory")
    dev = c_void_p(0)
    _call("runtime", "blm_host_device_pointer", c_void_p(pinned.data_ptr()), ctypes.byref(dev), kernels=0)
    return int(dev.value or 0)


_status: dict = {}


def status_word(device) -> torch.Tensor:
    """The device word in which kernels with bounded waits record that a wait ran out (0: all well)."""
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    w = _status.get(key)
    if w is None:
        w = _status[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return w


def check_status(device) -> None:
    """Raise if a kernel gave up a bounded wait since the last check (reads one word from the device)."""
    w = status_word(device)
    code = int(w.item())
    if code:
        w.zero_()
        what = {21: "decode attention: a consumer waited in vain for a page", 22: "decode attention: the producer waited in vain for a free stage",
                1: "gemv: a consumer waited in vain for a weight stage", 2: "gemv: the producer waited in vain for a free stage",
                31: "prompt attention: the query tile did not arrive", 32: "prompt attention: a key tile did not arrive",
                33: "prompt attention: a value tile did not arrive", 34: "prompt attention: the scores did not arrive",
                35: "prompt attention: the probabilities were not written", 36: "prompt attention: the product with the values did not arrive",
                37: "prompt attention: the producer waited in vain for a free stage",
                11: "gemm_tc: the tensor-core thread waited in vain for a stage", 12: "gemm_tc: the producer waited in vain for a free stage",
                13: "gemm_tc: the epilogue waited in vain for the accumulator",
                41: "gemm_sk: the tensor-core thread waited in vain for a stage", 42: "gemm_sk: the producer waited in vain for a free stage",
                43: "gemm_sk: the epilogue waited in vain for the accumulator"}
        raise KernelError(f"{what.get(code, 'status ' + str(code))}; the step's results are not valid")


SQUARES_ROWS = 16     # row length of the sums of squares that go with a handed-over norm


def gemv(w, n_tokens, x=None, stream_rows=None, gamma=None, eps=0.0, rows=None, out=None, add_into=None, swiglu=False,
         squares=None, hand_over=None, rope=None):
    """Skinny product of n_tokens <= 16 tokens with a bfloat16 weight [M, K], with fused ends.

    Input: `x` bfloat16 [N, K], or the fp32 residual stream `stream_rows` [*, K] to be RMS-normalised
    with `gamma`, `eps` (optionally gathering `rows`), or a norm that the writer of the stream handed
    over: `x` = bfloat16(stream * gamma) with `squares` (fp32 [parts, SQUARES_ROWS], the stream rows'
    sums of squares in parts) and `eps`; the result is then divided by the rows' root mean square.
    Output: `out` [N, M] bfloat16 or float32;
    with `swiglu` the weight is [2 I, K] in tiles of GATE_TILE gate rows followed by the up rows of the
    same outputs, and out [N, I] = silu(gate) * up; with
    `add_into` (fp32 [N, M]) the product is added into it and nothing else is written, unless
    `hand_over` = (gamma, scaled, squares) asks for the next norm's input as well: scaled
    (bfloat16 [N, M]) = the new stream times gamma, squares (fp32 [ceil(M / 16), SQUARES_ROWS]) its
    sums of squares by tiles of 16 lanes.
    With `rope` (a dict: token_pos, token_seq, slot_of_seq, block_table, table from rope_table, pool,
    n_heads, n_kv, head_dim, write_cache, max_position) the weight is a step's [q; k; v] (or q alone without
    write_cache) whose q and k heads have their rows in tiled_pair_order(): q and k are rotated by their
    token's position, q goes to `out` [N, n_heads * head_dim] (lanes in that order), the rotated k and the
    v to the token's place in `pool`."""
    _need_cuda(w, x, stream_rows, gamma, rows, out, add_into, squares)
    m_rows, k = w.shape
    if w.dtype != torch.bfloat16:
        raise KernelError("gemv: the weight must be bfloat16")
    m = m_rows // 2 if swiglu else m_rows
    epi = EPI_SWIGLU if swiglu else (EPI_RESID_ADD if add_into is not None else (EPI_ROPE if rope is not None else EPI_STORE))
    rope_arg = None
    if rope is not None:
        if swiglu or add_into is not None:
            raise KernelError("gemv: one epilogue at a time")
        r = rope
        hd, table, pool = r["head_dim"], r["table"], r["pool"]
        _need_cuda(r["token_pos"], r["token_seq"], r["slot_of_seq"], r["block_table"], table, pool)
        if table is None or table.dtype != torch.float32 or tuple(table.shape[1:]) != (hd // 2, 2) \
                or r.get("max_position") is None or r["max_position"] >= table.shape[0]:
            raise KernelError("gemv: the rotary epilogue needs a table [positions, head_dim / 2, 2] that covers the step")
        if r["write_cache"] and (pool.dtype != torch.bfloat16 or tuple(pool.shape[1:]) != (2, r["n_kv"], PAGE, hd)):
            raise KernelError(f"gemv: pool must be bfloat16 [pages, 2, {r['n_kv']}, {PAGE}, {hd}]")
        if out is None or out.dtype != torch.bfloat16 or tuple(out.shape) != (n_tokens, r["n_heads"] * hd):
            raise KernelError("gemv: the rotary epilogue writes q to a bfloat16 out [N, n_heads * head_dim]")
        rope_arg = _GemvRope(r["token_pos"].data_ptr(), r["token_seq"].data_ptr(), r["slot_of_seq"].data_ptr(),
                             r["block_table"].data_ptr(), table.data_ptr(), pool.data_ptr() if pool is not None else 0,
                             r["block_table"].shape[1], r["n_heads"], r["n_kv"], hd, PAGE, 1 if r["write_cache"] else 0,
                             r["token_page"].data_ptr() if r.get("token_page") is not None else 0)
    if x is not None and (x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != k
                          or (rows is None and x.shape[0] != n_tokens)):
        raise KernelError("gemv: x must be bfloat16 [N, K]")
    if rows is not None and rows.numel() != n_tokens:
        raise KernelError("gemv: one row index per token")
    if squares is not None and (x is None or squares.dtype != torch.float32 or squares.dim() != 2
                                or squares.shape[1] != SQUARES_ROWS or not squares.is_contiguous()
                                or x.shape[0] > SQUARES_ROWS):
        raise KernelError("gemv: squares go with x and are float32 [parts, 16]")
    next_gamma = scaled = squares_out = None
    if hand_over is not None:
        next_gamma, scaled, squares_out = hand_over
        _need_cuda(next_gamma, scaled, squares_out)
        if (epi != EPI_RESID_ADD or scaled.dtype != torch.bfloat16 or tuple(scaled.shape) != (n_tokens, m)
                or not scaled.is_contiguous() or squares_out.dtype != torch.float32 or not squares_out.is_contiguous()
                or tuple(squares_out.shape) != ((m + 15) // 16, SQUARES_ROWS) or next_gamma.numel() != m):
            raise KernelError("gemv: hand_over = (gamma [M], scaled bfloat16 [N, M], squares float32 [ceil(M / 16), 16]) "
                              "with add_into")
    if stream_rows is not None and (stream_rows.dtype != torch.float32 or stream_rows.shape[1] != k or gamma is None):
        raise KernelError("gemv: the stream must be float32 [*, K] with a gamma")
    if epi == EPI_RESID_ADD:
        if add_into.dtype != torch.float32 or tuple(add_into.shape) != (n_tokens, m):
            raise KernelError("gemv: add_into must be float32 [N, M]")
    elif epi == EPI_ROPE:
        pass
    elif out is None or tuple(out.shape) != (n_tokens, m) or out.dtype not in (torch.bfloat16, torch.float32) \
            or (swiglu and out.dtype != torch.bfloat16):
        raise KernelError("gemv: out must be [N, M] bfloat16 (or float32 for a plain store)")
    _call("gemv", "blm_gemv", _ptr(w), w.stride(0), m, k, _ptr(x), x.stride(0) if x is not None else 0,
          _ptr(stream_rows), _ptr(gamma), 1 if (gamma is not None and gamma.dtype == torch.float32) else 0, c_float(eps),
          _ptr(rows), n_tokens, _ptr(out), out.stride(0) if out is not None else 0,
          1 if (out is not None and out.dtype == torch.float32) else 0, _ptr(add_into), epi,
          _ptr(squares), squares.shape[0] if squares is not None else 0,
          _ptr(next_gamma), 1 if (next_gamma is not None and next_gamma.dtype == torch.float32) else 0,
          _ptr(scaled), _ptr(squares_out), ctypes.byref(rope_arg) if rope_arg is not None else None,
          _ptr(status_word(w.device)), _stream())


def argmax(logits, out, mirror=None, tickets=None, advance=None):
    """out[b] = index of the largest logit of row b (the lowest index on a tie).  `mirror`: a pinned host int32
    tensor that the kernel fills as well, through the address the device sees it under, so that a host which
    polls it has the result without a copy (`graph_step`).  `tickets`: B + 1 zeroed int32 on the device that belong
    to the caller and to no other launch in flight (the kernel leaves them zero): a large vocabulary then takes one
    launch instead of two.  `advance` = (tokens, positions, history or None, step counter): the step feeds itself
    as `decode_advance` says, in that same launch where there is one."""
    _need_cuda(logits, out)
    if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() < logits.shape[0]:
        raise KernelError("argmax: float32 logits [B, V], int32 out [B]")
    b, v = logits.shape
    if mirror is not None and (mirror.dtype != torch.int32 or mirror.numel() < b or not mirror.is_contiguous()):
        raise KernelError("argmax: the mirror is a pinned int32 tensor of at least B entries")
    lib = _lib("sampling")
    need = lib.blm_argmax_scratch_floats(b, v)
    scratch = torch.empty(need, dtype=torch.float32, device=logits.device) if need else None
    if tickets is not None:
        _need_cuda(tickets)
        if tickets.dtype != torch.int32 or tickets.numel() < b + 1 or not tickets.is_contiguous():
            raise KernelError("argmax: the tickets are B + 1 int32")
        if not need:
            tickets = None
    fed = None
    if advance is not None and tickets is not None and lib.blm_argmax_advances(v):
        fed = advance
        tokens, pos, history, step_no = fed
        _need_cuda(tokens, pos, step_no)
        if tokens.dtype != torch.int32 or pos.dtype != torch.int32 or tokens.numel() != b or pos.numel() != b:
            raise KernelError("argmax: a step that feeds itself has int32 tokens and positions [B]")
        if history is not None and (history.dtype != torch.int32 or history.shape[1] != b or not history.is_contiguous()):
            raise KernelError("argmax: the history is int32 [steps, B]")
    tokens, pos, history, step_no = fed if fed is not None else (None, None, None, None)
    _call("sampling", "blm_argmax", _ptr(logits), logits.stride(0), b, v, _ptr(out),
          c_void_p(host_device_pointer(mirror) if mirror is not None else 0), _ptr(scratch), _ptr(tickets),
          _ptr(tokens), _ptr(pos), _ptr(history), _ptr(step_no), c_void_p(0), history.shape[0] if history is not None else 0,
          _stream(), kernels=(1 if tickets is not None else 2) if need else 1)
    if advance is not None and fed is None:
        decode_advance(advance[0], advance[1], out, advance[2], advance[3])


def sample(logits, temperature, top_p, seeds, stream_ids, counters, out, mirror=None):
    """Draw out[b] from softmax(logits[b] / temperature[b]) restricted to its top-p nucleus.

    temperature, top_p float32 [B]; seeds, stream_ids, counters int64 [B] (read as unsigned): the
    uniform number of a draw is a hash of the three, so it does not depend on the batch.
    `mirror`: as `argmax`'s."""
    _need_cuda(logits, temperature, top_p, seeds, stream_ids, counters, out)
    b = logits.shape[0]
    if logits.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("sample: float32 logits, int32 out")
    if mirror is not None and (mirror.dtype != torch.int32 or mirror.numel() < b or not mirror.is_contiguous()):
        raise KernelError("sample: the mirror is a pinned int32 tensor of at least B entries")
    for t, dt in ((temperature, torch.float32), (top_p, torch.float32), (seeds, torch.int64),
                  (stream_ids, torch.int64), (counters, torch.int64)):
        if t.dtype != dt or t.numel() < b:
            raise KernelError("sample: per-row arguments must be float32/int64 of length B")
    work = torch.empty((b, logits.shape[1]), dtype=torch.float32, device=logits.device)     # the rows' exponentials
    _call("sampling", "blm_sample", _ptr(logits), logits.stride(0), b, logits.shape[1], _ptr(temperature),
          _ptr(top_p), _ptr(seeds), _ptr(stream_ids), _ptr(counters), _ptr(out),
          c_void_p(host_device_pointer(mirror) if mirror is not None else 0), _ptr(work), _stream())


def uniform32(seed, stream_id, counter) -> int:
    """The 32-bit uniform number the sampling kernel uses for (seed, stream, counter); host side."""
    lib = _lib("sampling")
    fn = lib.blm_sampling_uniform32
    fn.argtypes = [c_ulonglong, c_ulonglong, c_ulonglong]
    fn.restype = c_uint
    return int(fn(seed & (2**64 - 1), stream_id & (2**64 - 1), counter & (2**64 - 1)))


# ------------------------------------------------------------------------------------------------
# blocks that norm a sublayer's output before it is added to the stream
# ------------------------------------------------------------------------------------------------
def _f32(*tensors):
    for t in tensors:
        if t is not None and t.dtype != torch.float32:
            raise KernelError("this argument must be float32")


def embed_scaled(tokens, table, out, scale: float):
    """out[n, :] = table[tokens[n], :] * scale as fp32.  tokens int32 [N]; table [V, D]; out fp32 [N, D]."""
    _need_cuda(tokens, table, out)
    n, (v, d) = tokens.numel(), table.shape
    if tokens.dtype != torch.int32 or out.dtype != torch.float32 or tuple(out.shape) != (n, d):
        raise KernelError("embed_scaled: tokens int32 [N], out float32 [N, D]")
    _call("stream_ops", "blm_embed_scaled", _ptr(tokens), _ptr(table), _code(table.dtype), _ptr(out), n, d, v, c_float(scale), _stream())


def sandwich_norm(resid, delta, post_weight, mult, eps_post, pre_weight, eps_pre, out, rows=None, delta_bias=None, second=None):
    """The add of a normed sublayer output fused with the norm that reads the stream next, in fp32.  With d = delta (+ delta_bias),
    or d = scale_a * delta + scale_b * delta_b (+ delta_bias) when `second` = (scale_a, delta_b, scale_b) names the output of
    a mixer that ran beside the first:

        h   = resid + mult * (d / sqrt(mean(d^2) + eps_post) * post_weight)       stored into resid (rows is None)
        out = h / sqrt(mean(h^2) + eps_pre) * pre_weight                          when pre_weight and out are given
        out = h in out's dtype                                                    when out is given without pre_weight

    delta None: h = resid.  rows (int32 [R]): row i of out comes from row rows[i], resid is left alone.
    resid fp32 [N, D]; delta [N, D] in float32 or bfloat16; the weights and the bias float32 [D]."""
    _need_cuda(resid, delta, post_weight, pre_weight, out, rows, delta_bias)
    _f32(resid, post_weight, pre_weight, delta_bias)
    d = resid.shape[-1]
    n_out = rows.numel() if rows is not None else resid.shape[0]
    if delta is not None and (delta.shape != resid.shape or post_weight is None or post_weight.numel() != d):
        raise KernelError("sandwich_norm: delta must match resid's shape and bring its norm's weight [D]")
    if out is not None and (tuple(out.shape) != (n_out, d) or (pre_weight is not None and pre_weight.numel() != d)):
        raise KernelError("sandwich_norm: out [rows, D]; the weight [D] of the norm that produces it, or none for the stream as it is")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("sandwich_norm: rows must be int32")
    sa, delta_b, sb = second if second is not None else (1.0, None, 0.0)
    _need_cuda(delta_b)
    if delta_b is not None and (delta is None or delta_b.shape != delta.shape or delta_b.dtype != delta.dtype):
        raise KernelError("sandwich_norm: the second output must match the first in shape and dtype")
    _call("stream_ops", "blm_sandwich_norm", _ptr(resid), _ptr(delta), _ptr(delta_b), c_float(sa), c_float(sb),
          _code(delta.dtype) if delta is not None else F32,
          _ptr(delta_bias), _ptr(post_weight), _ptr(pre_weight if out is not None else None), c_float(mult), c_float(eps_post),
          c_float(eps_pre), _ptr(out), _code(out.dtype) if out is not None else F32, _ptr(rows), n_out, d, _stream())


ACT_NONE, ACT_XIELU, ACT_TANH = 0, 1, 2


def bias_act(x, bias, out, kind=ACT_NONE, params=None):
    """out = act(x + bias) row by row; x, out [N, D] (float32 or bfloat16), bias float32 [D] or None.  ACT_XIELU with
    params = float32 [2] (p, q): z > 0: softplus(p) z^2 + z / 2; else (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.
    ACT_TANH: tanh(z)."""
    _need_cuda(x, bias, out, params)
    _f32(bias, params)
    n, d = x.shape
    if tuple(out.shape) != (n, d) or (bias is not None and bias.numel() != d):
        raise KernelError("bias_act: x and out [N, D], bias [D]")
    if kind == ACT_XIELU and (params is None or params.numel() != 2):
        raise KernelError("bias_act: the activation needs its two numbers")
    _call("stream_ops", "blm_bias_act", _ptr(x), _code(x.dtype), _ptr(bias), _ptr(params), _ptr(out), _code(out.dtype), n, d, int(kind),
          _stream())


def weighted_sum(a, scale_a, b, scale_b, out):
    """out = scale_a * a + scale_b * b, all float32 of one shape."""
    _need_cuda(a, b, out)
    _f32(a, b, out)
    if a.shape != b.shape or a.shape != out.shape:
        raise KernelError("weighted_sum: shapes differ")
    _call("stream_ops", "blm_weighted_sum", _ptr(a), _ptr(b), _ptr(out), c_float(scale_a), c_float(scale_b), c_size_t(a.numel()), _stream())


# ------------------------------------------------------------------------------------------------
# recurrent mixers
# ------------------------------------------------------------------------------------------------
def scan_state_floats(heads: int, rows: int, value_dim: int) -> int:
    """Floats of one copy of a scan's state: the rows are rounded up to what the kernel's instance holds (8 row groups
    times 1, 2, 4, 8, 16 or 32 rows a thread)."""
    groups = 8
    for rn in (1, 2, 4, 8, 16, 32):
        if rn * groups >= rows:
            return heads * rn * groups * value_dim
    raise KernelError(f"a recurrent state of {rows} rows: the scan kernels take up to 256")


def _state_args(state, offset):
    """state float32 [slots, 2, floats]: (pointer, floats a slot, floats a copy, this piece's offset in a copy)."""
    if state.dtype != torch.float32 or state.dim() != 3 or state.shape[1] != 2 or not state.is_contiguous():
        raise KernelError("a recurrent state is float32 [slots, 2, floats]")
    return _ptr(state), c_longlong(2 * state.shape[2]), c_longlong(state.shape[2]), c_longlong(offset)


def _cols(t, col0, width):
    if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or col0 < 0 or col0 + width > t.shape[1]:
        raise KernelError("a column range must lie inside a float32 [N, *] tensor with unit stride along its rows")
    return _ptr(t), c_longlong(t.stride(0)), int(col0)


def causal_conv(x, x_col0, channels, taps, bias, out, out_col0, step, state, state_offset, silu=True, out_bf16=None, residual=False):
    """y_t = sum_k taps[:, k] x_(t - (K-1) + k) (+ bias) per channel over each sequence's time, then silu; zeros before a
    sequence's start.  x, out float32 [N, *] (the channels at x_col0 / out_col0); taps float32 [C, K]; the last K - 1
    inputs of every sequence are carried in `state` (float32 [slots, 2, floats]) at state_offset, [K - 1, C].  A step in
    which every sequence brings one token (step.max_q_len == 1) moves the carried inputs on in the same launch.
    `out_bf16` (bfloat16 [N, C]): the result once more, rounded, for a product that reads it.  `residual` (without silu):
    y_t = x_t + the sum over the taps."""
    if residual and silu:
        raise KernelError("causal_conv: the input is added to the plain convolution, not to an activated one")
    _need_cuda(taps, bias, state, out_bf16)
    if out_bf16 is not None and (out_bf16.dtype != torch.bfloat16 or tuple(out_bf16.shape) != (step.n_tokens, channels)):
        raise KernelError("causal_conv: out_bf16 is bfloat16 [N, C]")
    _f32(taps, bias)
    k = taps.shape[1]
    if tuple(taps.shape) != (channels, k) or (bias is not None and bias.numel() != channels):
        raise KernelError("causal_conv: taps [C, K], bias [C]")
    xp, xs, xc = _cols(x, x_col0, channels)
    op, os_, oc = _cols(out, out_col0, channels)
    if x.shape[0] != step.n_tokens or out.shape[0] != step.n_tokens:
        raise KernelError("causal_conv: a row per token of the step")
    single = getattr(step, "max_q_len", 0) == 1
    _call("recurrent", "blm_causal_conv", xp, xs, xc, channels, _ptr(taps), _ptr(bias), k, 2 if residual else (1 if silu else 0), op, os_, oc,
          _ptr(step.token_seq), _ptr(step.cu_seqlens), _ptr(step.slot_of_seq), _ptr(step.start_pos), step.n_tokens, step.n_seqs,
          *_state_args(state, state_offset), 1 if single else 0, _ptr(out_bf16), c_longlong(channels), _stream(),
          kernels=2 if k > 1 and not single else 1)


def ssm_scan(xbc, x_col0, b_col0, c_col0, dt, dt_col0, dt_bias, a_log, d_skip, y, heads, groups, n_state, value_dim, step, state,
             state_offset, wide_sums=False):
    """The state-space scan per head: S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x with dt = softplus(dt_raw +
    dt_bias); x [heads x value_dim], B and C [groups x n_state] are column ranges of xbc, dt_raw [heads] one of dt;
    y float32 [N, heads * value_dim].  The state (fp32, carried per sequence) lies in `state` at state_offset.  `wide_sums`:
    inside a step the state and the sums over its rows are held in float64 (the 32-bit path: a head that decays slowly sums
    a long past into a state far larger than its read-out, whose cancellation float sums alone make visible)."""
    _need_cuda(dt_bias, a_log, d_skip, y, state)
    _f32(dt_bias, a_log, d_skip, y)
    xp, xs, xc = _cols(xbc, x_col0, heads * value_dim)
    _cols(xbc, b_col0, groups * n_state)
    _cols(xbc, c_col0, groups * n_state)
    dp, ds, dc = _cols(dt, dt_col0, heads)
    if tuple(y.shape) != (step.n_tokens, heads * value_dim) or not y.is_contiguous():
        raise KernelError("ssm_scan: y float32 [N, heads * value_dim]")
    _call("recurrent", "blm_ssm_scan", xp, xs, xc, int(b_col0), int(c_col0), dp, ds, dc, _ptr(dt_bias), _ptr(a_log), _ptr(d_skip),
          _ptr(y), c_longlong(y.stride(0)), heads, groups, n_state, value_dim, _ptr(step.cu_seqlens), _ptr(step.slot_of_seq),
          _ptr(step.start_pos), step.n_seqs, *_state_args(state, state_offset), 1 if wide_sums else 0, _stream())


def delta_scan(q, q_col0, k, k_col0, v, v_col0, b, b_col0, a, a_col0, dt_bias, a_log, out, heads, qk_heads, key_dim, value_dim,
               step, state, state_offset):
    """The gated delta rule per head: S <- g S (g per key channel); u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with
    q and k made unit vectors (q also times key_dim^-1/2), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)).
    q, k [qk_heads x key_dim], v [heads x value_dim], b [heads], a [heads x key_dim] are column ranges of float32 [N, *]
    tensors; out float32 [N, heads * value_dim]."""
    _need_cuda(dt_bias, a_log, out, state)
    _f32(dt_bias, a_log, out)
    qa = _cols(q, q_col0, qk_heads * key_dim)
    ka = _cols(k, k_col0, qk_heads * key_dim)
    va = _cols(v, v_col0, heads * value_dim)
    ba = _cols(b, b_col0, heads)
    aa = _cols(a, a_col0, heads * key_dim)
    if tuple(out.shape) != (step.n_tokens, heads * value_dim) or not out.is_contiguous() or dt_bias.numel() != heads * key_dim:
        raise KernelError("delta_scan: out float32 [N, heads * value_dim], dt_bias [heads * key_dim]")
    _call("recurrent", "blm_delta_scan", *qa, *ka, *va, *ba, *aa, _ptr(dt_bias), _ptr(a_log), _ptr(out), c_longlong(out.stride(0)),
          heads, qk_heads, key_dim, value_dim, _ptr(step.cu_seqlens), _ptr(step.slot_of_seq), _ptr(step.start_pos), step.n_seqs,
          *_state_args(state, state_offset), _stream())


def shift_mix(x, mu, out, step, state, state_offset):
    """out[s, n] = x[n] + (x[n - 1] - x[n]) * mu[s]: every one of S mixes of a token's input with the input of the token
    before it in its sequence (zeros before the first).  x float32 [N, C]; mu float32 [S, C]; out [S, N, C] in float32 or
    bfloat16.  The last input of every sequence is carried in `state` (float32 [slots, 2, floats]) at state_offset, [C]."""
    _need_cuda(x, mu, out, state)
    _f32(x, mu)
    n, c = x.shape
    s = mu.shape[0]
    if n != step.n_tokens or tuple(mu.shape) != (s, c) or tuple(out.shape) != (s, n, c):
        raise KernelError("shift_mix: x [N, C], mu [S, C], out [S, N, C]")
    single = getattr(step, "max_q_len", 0) == 1
    _call("recurrent", "blm_shift_mix", _ptr(x), c_longlong(x.stride(0)), c, _ptr(mu), s, _ptr(out), _code(out.dtype),
          _ptr(step.token_seq), _ptr(step.cu_seqlens), _ptr(step.slot_of_seq), _ptr(step.start_pos), n, step.n_seqs,
          *_state_args(state, state_offset), 1 if single else 0, _stream(), kernels=1 if single else 2)


DECAY_EXP_EXP, DECAY_LOWER_BOUND = 0, 1


def decay_scan(q, q_col0, k, k_col0, v, v_col0, a, a_col0, bias, extra, out, heads, key_dim, value_dim, kind, read_first, step,
               state, state_offset, wide_sums=False):
    """Linear attention with a decay per key channel, per head with a state S [key_dim x value_dim]:
    `read_first`: o = (S + diag(u) k v^T)^T q, then S <- diag(w) S + k v^T (u = `extra`, a bonus for the current token);
    else S <- diag(w) S + k v^T, then o = S^T q.  DECAY_EXP_EXP: w = exp(-exp(a + bias)), q and k as given.
    DECAY_LOWER_BOUND: w = low + (1 - low) sigmoid(a + bias) with low = `extra`, k = 1 - w (k is not read), q = silu(q).
    q, k, a [heads x key_dim] and v [heads x value_dim] are column ranges of float32 [N, *] tensors; bias, extra float32
    [heads * key_dim]; out float32 [N, heads * value_dim].  `wide_sums`: the state and the sums over its rows are held in
    float64 inside a step (the 32-bit path)."""
    _need_cuda(bias, extra, out, state)
    _f32(bias, extra, out)
    qa = _cols(q, q_col0, heads * key_dim)
    ka = _cols(k, k_col0, heads * key_dim) if k is not None else (c_void_p(0), c_longlong(0), 0)
    va = _cols(v, v_col0, heads * value_dim)
    aa = _cols(a, a_col0, heads * key_dim)
    if tuple(out.shape) != (step.n_tokens, heads * value_dim) or not out.is_contiguous() or bias.numel() != heads * key_dim:
        raise KernelError("decay_scan: out float32 [N, heads * value_dim], bias [heads * key_dim]")
    if extra is not None and extra.numel() != heads * key_dim:
        raise KernelError("decay_scan: extra [heads * key_dim]")
    _call("recurrent", "blm_decay_scan", *qa, *ka, *va, *aa, _ptr(bias), _ptr(extra), _ptr(out), c_longlong(out.stride(0)), heads,
          key_dim, value_dim, int(kind), 1 if read_first else 0, _ptr(step.cu_seqlens), _ptr(step.slot_of_seq), _ptr(step.start_pos),
          step.n_seqs, *_state_args(state, state_offset), 1 if wide_sums else 0, _stream())


GATE_FIRST, GATE_LAST, GATE_SILU_LAST, GATE_NONE = 0, 1, 2, 3


def gated_group_norm(y, gate, gate_col0, weight, group, mode, eps, out):
    """RMS norm over groups of `group` lanes of every row with a gate.  GATE_FIRST: u = y silu(gate), out = u / rms(u) *
    weight; GATE_LAST: out = y / rms(y) * weight * sigmoid(gate); GATE_SILU_LAST: ... * silu(gate); GATE_NONE: no gate
    (`gate` None).  weight float32 of a row's or of a group's size (then
    shared by the groups); y float32 [N, C]; the gate a column range of a float32 tensor; out [N, C]."""
    _need_cuda(y, weight, out)
    _f32(y, weight)
    n, c = y.shape
    if c % group or weight.numel() not in (c, group) or tuple(out.shape) != (n, c) or not y.is_contiguous() or not out.is_contiguous():
        raise KernelError("gated_group_norm: groups must divide the row; weight of a row's or a group's size")
    gp, gs, gc = _cols(gate, gate_col0, c) if gate is not None else (c_void_p(0), c_longlong(0), 0)
    _call("recurrent", "blm_gated_group_norm", _ptr(y), c_longlong(y.stride(0)), gp, gs, gc, _ptr(weight), weight.numel(), group,
          c // group, int(mode), c_float(eps), _ptr(out), _code(out.dtype), c_longlong(out.stride(0)), n, _stream())


# ------------------------------------------------------------------------------------------------
# attention without a softmax
# ------------------------------------------------------------------------------------------------
def bias_rope_append(proj, bias, freq, rotary_dim, q_out, pool, block_table, step, n_heads, n_kv, key_dim, value_dim):
    """proj float32 [N, q | k | v] (+ bias float32): the first rotary_dim lanes of every q and k head are rotated (lane i
    with lane i + rotary_dim / 2 by position * freq[i], freq float64 [rotary_dim / 2]; the angle, its sine and its cosine are
    taken in fp64 and applied in fp32); q goes to q_out
    [N, n_heads * key_dim], k and v to the token's place in the paged cache."""
    _need_cuda(proj, bias, freq, q_out, pool, block_table)
    _f32(proj, bias)
    n = step.n_tokens
    width = (n_heads + n_kv) * key_dim + n_kv * value_dim
    if proj.dim() != 2 or proj.shape[0] != n or proj.shape[1] != width or (bias is not None and bias.numel() != width):
        raise KernelError("bias_rope_append: proj [N, (heads + kv) * key_dim + kv * value_dim] and a bias of that width")
    if q_out.dtype != pool.dtype or tuple(q_out.shape) != (n, n_heads * key_dim):
        raise KernelError("bias_rope_append: q_out [N, heads * key_dim] in the cache's dtype")
    if pool.numel() % kv_page_elems(n_kv, key_dim, value_dim):
        raise KernelError("bias_rope_append: the pool does not consist of pages of keys [kv, PAGE, key_dim] and values [kv, PAGE, value_dim]")
    if rotary_dim and (freq is None or freq.dtype != torch.float64 or freq.numel() != rotary_dim // 2):
        raise KernelError("bias_rope_append: freq must be float64 [rotary_dim / 2]")
    _call("attention_sigmoid", "blm_bias_rope_append", _ptr(proj), c_longlong(proj.stride(0)), _ptr(bias), _ptr(freq), int(rotary_dim),
          _ptr(q_out), _ptr(pool), _code(pool.dtype), _ptr(step.token_seq), _ptr(step.token_pos), _ptr(step.slot_of_seq),
          _ptr(block_table), block_table.shape[1], n, n_heads, n_kv, key_dim, value_dim, PAGE, _stream())


def sigmoid_attention_takes(dtype, n_heads, n_kv, key_dim, value_dim) -> bool:
    return bool(_lib("attention_sigmoid").blm_sigmoid_attention_takes(_code(dtype), n_heads, n_kv, key_dim, value_dim, PAGE))


def sigmoid_attention(q, pool, block_table, step, out, n_heads, n_kv, key_dim, value_dim, scale, softcap=0.0, talk=None,
                      head_bias=None, ranges=1, partial=None, scalar_only=False):
    """Causal attention whose weights are sigmoid(cap(scale q.k) + head_bias) without a normalisation over the keys, mixed
    across heads by talk [heads, heads] (row h: what head h takes of every head's weights) before they meet the values.
    q [N, heads * key_dim] and out [N, heads * value_dim] in the cache's dtype (out must hold zeros in rows of no
    sequence); `ranges` > 1 cuts every query's keys over that many blocks whose partial outputs (`partial`, float32
    with room for ranges * N * heads * value_dim) are added in order.  Prompts in bfloat16 run the tensor-core kernel where
    it takes the shape (key lanes in multiples of 16, value lanes of 8); `scalar_only` keeps them off it."""
    _need_cuda(q, pool, block_table, out, talk, head_bias, partial)
    _f32(talk, head_bias, partial)
    n = step.n_tokens
    if q.dtype != pool.dtype or out.dtype != pool.dtype or tuple(q.shape) != (n, n_heads * key_dim) or tuple(out.shape) != (n, n_heads * value_dim):
        raise KernelError("sigmoid_attention: q [N, heads * key_dim], out [N, heads * value_dim] in the cache's dtype")
    if talk is not None and tuple(talk.shape) != (n_heads, n_heads):
        raise KernelError("sigmoid_attention: talk [heads, heads]")
    if head_bias is not None and head_bias.numel() != n_heads:
        raise KernelError("sigmoid_attention: head_bias [heads]")
    if ranges > 1 and (partial is None or partial.numel() < ranges * n * n_heads * value_dim):
        raise KernelError("sigmoid_attention: the workspace is too small for the key ranges")
    _call("attention_sigmoid", "blm_sigmoid_attention", _ptr(q), _ptr(pool), _code(pool.dtype), _ptr(block_table), block_table.shape[1],
          _ptr(step.cu_seqlens), _ptr(step.slot_of_seq), _ptr(step.start_pos), _ptr(step.token_seq), _ptr(talk), _ptr(head_bias),
          _ptr(out), _ptr(partial), n, step.n_seqs, step.max_q_len, n_heads, n_kv, key_dim, value_dim, PAGE, int(ranges),
          c_float(scale), c_float(softcap), 1 if scalar_only else 0, _stream(), kernels=2 if ranges > 1 else 1)


# ------------------------------------------------------------------------------------------------
# attention over a cached latent
# ------------------------------------------------------------------------------------------------
def latent_prepare(q_proj, down, c_weight, eps, freq, rot_dims, q_nope, q_rot, pool, block_table, step, n_heads, key_dim, rot_dim,
                   rank, q_full=None, halves=False):
    """q_proj float32 [N, heads * (key_dim + rot_dim)] (every head's unrotated lanes, then its rotated ones) and down
    float32 [N, rank + rot_dim]: q_nope [heads, N, key_dim] (the cache's dtype) takes the unrotated lanes, q_rot float32
    [N, heads, rot_dim] the rotated ones turned by the token's position (lanes 2i, 2i + 1 by position * freq[i] for the first
    rot_dims lanes; freq float64 [rot_dims / 2]); the first `rank` lanes of `down`, RMS-normed with c_weight, and its last
    rot_dim lanes, turned likewise, go to the token's place in the paged cache ([pages, PAGE, rank + rot_dim]).
    With `q_full` [N, heads, hd] (the cache's dtype, hd >= key_dim + rot_dim) the query goes there instead, a head's
    unrotated lanes, its turned ones and zeros side by side, and q_nope and q_rot are not written (they may be None).
    `halves`: the turning lanes are paired (i, i + rot_dims / 2) instead of (2i, 2i + 1)."""
    _need_cuda(c_weight, freq, q_nope, q_rot, q_full, pool, block_table)
    _f32(q_proj, down, c_weight, q_rot)
    if not q_proj.is_cuda or not down.is_cuda or q_proj.stride(1) != 1 or down.stride(1) != 1:
        raise KernelError("latent_prepare: q_proj and down are CUDA tensors (column ranges of a wider one will do)")
    n = step.n_tokens
    if tuple(q_proj.shape) != (n, n_heads * (key_dim + rot_dim)) or tuple(down.shape) != (n, rank + rot_dim) or c_weight.numel() != rank:
        raise KernelError("latent_prepare: q_proj [N, heads * (key_dim + rot_dim)], down [N, rank + rot_dim], c_weight [rank]")
    hd_full = 0
    if q_full is not None:
        hd_full = q_full.shape[-1]
        if q_full.dtype != pool.dtype or tuple(q_full.shape) != (n, n_heads, hd_full) or hd_full < key_dim + rot_dim or not q_full.is_contiguous():
            raise KernelError("latent_prepare: q_full [N, heads, hd >= key_dim + rot_dim] in the cache's dtype")
    elif (q_nope is None or q_rot is None or q_nope.dtype != pool.dtype or tuple(q_nope.shape) != (n_heads, n, key_dim)
          or tuple(q_rot.shape) != (n, n_heads, rot_dim)):
        raise KernelError("latent_prepare: q_nope [heads, N, key_dim] in the cache's dtype, q_rot float32 [N, heads, rot_dim]")
    if pool.numel() % (PAGE * (rank + rot_dim)):
        raise KernelError("latent_prepare: the pool does not consist of pages [PAGE, rank + rot_dim]")
    if rot_dims and (freq is None or freq.dtype != torch.float64 or freq.numel() != rot_dims // 2):
        raise KernelError("latent_prepare: freq must be float64 [rot_dims / 2]")
    _call("attention_latent", "blm_latent_prepare", _ptr(q_proj), c_longlong(q_proj.stride(0)), _ptr(down), c_longlong(down.stride(0)),
          _ptr(c_weight), c_float(eps), _ptr(freq), int(rot_dims), _ptr(q_nope), _ptr(q_rot), _ptr(q_full), int(hd_full), _ptr(pool),
          _code(pool.dtype), _ptr(step.token_seq), _ptr(step.token_pos), _ptr(step.slot_of_seq), _ptr(block_table), block_table.shape[1],
          n, n_heads, key_dim, rot_dim, rank, PAGE, 1 if halves else 0, _stream())


def latent_gather(pool, block_table, step, out, pages_each, lanes, window=0):
    """The cached pages of the step's sequences side by side: out [n_seqs * pages_each, PAGE, lanes] takes page p of
    sequence s at s * pages_each + p; positions a sequence has not reached are zeros.  `window` > 0: so are the pages
    that lie wholly before the window of the step's first token (the cache may have given them back)."""
    _need_cuda(pool, block_table, out)
    if out.dtype != pool.dtype or out.numel() != step.n_seqs * pages_each * PAGE * lanes or not out.is_contiguous():
        raise KernelError("latent_gather: out [n_seqs * pages_each, PAGE, lanes] in the cache's dtype")
    if pool.numel() % (PAGE * lanes) or pages_each > block_table.shape[1]:
        raise KernelError("latent_gather: the pool's pages are [PAGE, lanes]; a sequence has at most the table's pages")
    _call("attention_latent", "blm_latent_gather", _ptr(pool), _code(pool.dtype), _ptr(block_table), block_table.shape[1],
          _ptr(step.cu_seqlens), _ptr(step.slot_of_seq), _ptr(step.start_pos), _ptr(out), step.n_seqs, int(pages_each), int(lanes), PAGE,
          int(window), _stream())


def latent_expand(kv, gathered, out, n_heads, key_dim, rot_dim, value_dim, rank):
    """Pages of whole keys and values for the grouped-query attention kernels.  kv [rows, heads * key_dim + heads *
    value_dim]: every gathered position's unrotated keys of all heads, then its values; gathered [rows, rank + rot_dim]
    gives the rotated key part all heads share.  out [rows / PAGE, 2, heads, PAGE, hd]: keys [unrotated | rotated | zeros]
    and values [value | zeros]."""
    _need_cuda(kv, gathered, out)
    rows, hd = gathered.shape[0], out.shape[-1]
    if (kv.dtype != out.dtype or gathered.dtype != out.dtype or kv.stride(1) != 1 or not gathered.is_contiguous() or not out.is_contiguous()
            or tuple(kv.shape) != (rows, n_heads * (key_dim + value_dim)) or gathered.shape[1] != rank + rot_dim or rows % PAGE
            or tuple(out.shape) != (rows // PAGE, 2, n_heads, PAGE, hd) or hd < max(key_dim + rot_dim, value_dim)):
        raise KernelError("latent_expand: kv [rows, heads * (key_dim + value_dim)], gathered [rows, rank + rot_dim], "
                          "out [rows / PAGE, 2, heads, PAGE, hd]")
    _call("attention_latent", "blm_latent_expand", _ptr(kv), c_longlong(kv.stride(0)), _ptr(gathered), _ptr(out), _code(out.dtype),
          rows // PAGE, n_heads, key_dim, rot_dim, value_dim, rank, hd, PAGE, _stream())


def latent_attention_scratch_floats(n_tokens, n_heads, rank, n_splits) -> int:
    return n_splits * n_tokens * n_heads * (rank + 2) if n_splits > 1 else 0


def latent_attention_tile_rows(dtype, n_heads, rank, rot_dim, max_q_len) -> int:
    """How many rows (new token x head) a block of latent_attention owns at these sizes: 16 on the CUDA cores, 16 or 32
    on the tensor cores (a bfloat16 cache whose latent and rotated part are multiples of 16 lanes, up to 512)."""
    return int(_lib("attention_latent").blm_latent_attention_tile_rows(_code(dtype), n_heads, rank, rot_dim, max_q_len))


def latent_attention(q_lat, q_rot, pool, block_table, step, out, n_heads, rank, rot_dim, scale, n_splits=1, partial=None,
                     window=0, sink=None):
    """Causal softmax attention of every new token's heads over its sequence's cached positions, each one key of rank +
    rot_dim lanes shared by the heads, whose first `rank` lanes are the value: score = (q_lat . c + q_rot . k_rot) * scale.
    q_lat float32 [heads, N, rank], q_rot float32 [N, heads, rot_dim]; out [heads, N, rank] in float32 or the cache's dtype
    (rows of no sequence are left as they are).  `n_splits` > 1 cuts every row's keys over that many blocks (`partial`:
    float32 scratch of latent_attention_scratch_floats) whose shares are merged in order.  `window` > 0: position i sees
    j with 0 <= i - j < window.  `sink` float32 [heads]: exp(sink_h) joins the softmax's denominator (no key, no value,
    not scaled)."""
    _need_cuda(q_lat, q_rot, pool, block_table, out, partial, sink)
    _f32(q_lat, q_rot, partial, sink)
    if sink is not None and sink.numel() != n_heads:
        raise KernelError("latent_attention: the sink has a number per head")
    n = step.n_tokens
    if tuple(q_lat.shape) != (n_heads, n, rank) or tuple(q_rot.shape) != (n, n_heads, rot_dim) or tuple(out.shape) != (n_heads, n, rank):
        raise KernelError("latent_attention: q_lat and out [heads, N, rank], q_rot [N, heads, rot_dim]")
    if n_splits > 1 and (partial is None or partial.numel() < latent_attention_scratch_floats(n, n_heads, rank, n_splits)):
        raise KernelError("latent_attention: the workspace is too small for the key shares")
    _call("attention_latent", "blm_latent_attention", _ptr(q_lat), _ptr(q_rot), _ptr(pool), _code(pool.dtype), _ptr(block_table),
          block_table.shape[1], _ptr(step.cu_seqlens), _ptr(step.slot_of_seq), _ptr(step.start_pos), _ptr(step.token_seq), _ptr(out),
          _code(out.dtype), _ptr(partial), n, step.n_seqs, step.max_q_len, n_heads, rank, rot_dim, PAGE, c_float(scale), int(n_splits),
          int(window or 0), _ptr(sink), _stream(), kernels=2 if n_splits > 1 else 1)


def sigmoid_gate(o, gate, out, share=1):
    """out = o * sigmoid(gate); o and out [N, C]; gate [N, C / share] in float32 or o's dtype, possibly a column range of a
    wider tensor: a number for every `share` neighbouring columns of o (1: element by element; a head's value size: a gate
    per head)."""
    _need_cuda(o, out)
    if not gate.is_cuda or gate.dim() != 2 or gate.stride(1) != 1:
        raise KernelError("sigmoid_gate: the gate is a CUDA tensor [N, C / share] with unit stride along its rows")
    if (o.dim() != 2 or share < 1 or o.shape[1] % share or tuple(gate.shape) != (o.shape[0], o.shape[1] // share) or o.shape != out.shape
            or o.dtype != out.dtype):
        raise KernelError("sigmoid_gate: o and out [N, C], gate [N, C / share]; out in o's dtype")
    _call("attention_latent", "blm_sigmoid_gate", _ptr(o), _code(o.dtype), _ptr(gate), _code(gate.dtype), c_longlong(gate.stride(0)),
          _ptr(out), o.shape[0], o.shape[1], int(share), _stream())


# ------------------------------------------------------------------------------------------------
# the stream beside another row; capped logits
# ------------------------------------------------------------------------------------------------
def pack_cols(src, delta, dst, col0):
    """dst[:, col0 : col0 + D] = src (+ delta, the sum also stored into src), converted to dst's dtype.  src float32
    [N, D]; delta float32 or bfloat16 [N, D] or None; dst [N, W] with W >= col0 + D."""
    _need_cuda(src, delta, dst)
    _f32(src)
    n, d = src.shape
    if dst.dim() != 2 or dst.shape[0] != n or col0 < 0 or col0 + d > dst.shape[1] or (delta is not None and delta.shape != src.shape):
        raise KernelError("pack_cols: src [N, D], dst [N, W] with room for D columns at col0")
    _call("stream_ops", "blm_pack_cols", _ptr(src), _ptr(delta), _code(delta.dtype) if delta is not None else F32, _ptr(dst),
          _code(dst.dtype), c_longlong(dst.stride(0)), int(col0), n, d, _stream())


def softcap(x, cap: float):
    """x <- cap * tanh(x / cap) in place; x float32."""
    _need_cuda(x)
    _f32(x)
    _call("stream_ops", "blm_softcap", _ptr(x), c_float(cap), c_size_t(x.numel()), _stream())
