"""Python entry to the hand-written CUDA kernels.

Every function takes torch CUDA tensors (as containers only), hands raw pointers to
an ``extern "C"`` launcher on torch's current stream, and raises on any error.  There
is no CPU path and no library fallback: a tensor that is not on a CUDA device, a size
a kernel refuses, or a missing library is an error here.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .csrc.build import DEBUG_BUILD, load_library

F32, BF16 = 0, 1
_UNSUPPORTED = 10001


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


_SIGNATURES = {
    "elementwise": {
        "tl_embed": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "tl_rms_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "tl_rope_kv": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                       c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "tl_elementwise_debug_error": [c_void_p],
        "tl_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
    "gemm_simt": {
        "tl_gemm_simt": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_int, c_int, c_void_p],
    },
    "attention_generic": {
        "tl_attention_generic": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_int,
                                 c_void_p, c_int, c_void_p],
        "tl_attention_generic_debug_error": [c_void_p],
    },
    "gemm_tc": {
        "tl_gemm_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_longlong,
                       c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p],
        "tl_gemm_tc_glu": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p,
                           c_longlong, c_float, c_float, c_void_p],
        "tl_gemm_tc_gated": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_longlong,
                             c_longlong, c_void_p, c_longlong, c_int, c_void_p],
        "tl_gemm_tc_grouped": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                               c_float, c_float, c_void_p],
        "tl_gemm_tc_plan": [c_int, c_int, c_int, c_void_p, c_void_p],
        "tl_gemm_tc_error": [],
        "tl_gemm_tc_wait_selftest": [c_int, c_void_p],
    },
    "attention_mma": {
        "tl_attention_mma": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                             c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p],
        "tl_attention_mma_ex": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_float, c_int, c_void_p, c_longlong,
                                c_void_p, c_void_p, c_void_p],
        "tl_attention_mma_error": [],
        "tl_attention_mma_debug_error": [c_void_p],
    },
    "decode_fused": {
        "tl_finish_qkv_rope": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "tl_decode_fused_debug_error": [c_void_p],
        "tl_finish_accum_norm": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                 c_void_p],
    },
    "attention_tc": {
        "tl_attention_tc": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_float,
                            c_int, c_void_p, c_int, c_void_p, c_longlong, c_int, c_float, c_int, c_void_p, c_longlong,
                            c_void_p, c_void_p, c_void_p],
        "tl_attention_tc_merge": [c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                  c_longlong, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p],
        "tl_attention_tc_error": [],
        "tl_attention_tc_rows": [c_int],
    },
    "slots": {
        "tl_slot_gather": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "tl_slot_advance": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "tl_slot_command_words": [c_int, c_int],
        "tl_slot_record_rows": [],
        "tl_slots_debug_error": [c_void_p],
    },
    "stream_ops": {
        "tl_fill_zero": [c_void_p, c_longlong, c_void_p],
        "tl_scale": [c_void_p, c_float, c_longlong, c_void_p],
        "tl_scaled_add": [c_void_p, c_void_p, c_float, c_void_p, c_longlong, c_int, c_void_p],
        "tl_rms_scaled_add": [c_void_p, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int, c_void_p],
        "tl_rms_scaled_add_partials": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_float, c_float, c_int, c_int, c_int,
                                       c_void_p],
        "tl_gated_token_embed": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
        "tl_clamped_glu": [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p],
        "tl_glu_act": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "tl_stream_ops_debug_error": [c_void_p],
    },
    "delta_rule": {
        "tl_delta_prepare": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_void_p],
        "tl_delta_scan": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_int, c_void_p],
        "tl_delta_finish": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                            c_void_p],
        "tl_delta_rule_debug_error": [c_void_p],
    },
    "latent_attention": {
        "tl_latent_prepare": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float,
                              c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                              c_int, c_void_p],
        "tl_latent_absorb_q": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_void_p],
        "tl_latent_attention": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "tl_latent_expand_o": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
        "tl_latent_attention_debug_error": [c_void_p],
    },
    "latent_attention_mma": {
        "tl_latent_attention_mma_supported": [c_int, c_int],
        "tl_latent_attention_mma": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                    c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                    c_void_p, c_void_p],
        "tl_latent_attention_mma_debug_error": [c_void_p],
    },
    "gla": {
        "tl_gla_decay": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "tl_gla_scan": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                        c_int, c_int, c_float, c_int, c_void_p],
        "tl_rotate_heads_f32": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "tl_gla_finish": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                          c_void_p],
        "tl_gla_debug_error": [c_void_p],
    },
    "gated_attention": {
        "tl_normed_qk_store": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p,
                               c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_void_p],
        "tl_gated_attention_debug_error": [c_void_p],
    },
    "moe": {
        "tl_moe_tile_rows": [],
        "tl_moe_route": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_int, c_float, c_void_p, c_float, c_void_p, c_void_p, c_void_p],
        "tl_moe_plan": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "tl_moe_scatter": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "tl_moe_gemm_simt": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float,
                             c_float, c_void_p],
        "tl_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                           c_void_p],
    },
    "ssm": {
        "tl_ssm_conv": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_void_p],
        "tl_ssm_conv_state": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "tl_gated_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_float, c_void_p],
        "tl_activate_silu": [c_void_p, c_int, c_int, c_int, c_void_p],
        "tl_gate_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
        "tl_token_gate": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "tl_ssm_debug_error": [c_void_p],
    },
    "hyper": {
        "tl_hyper_fanout": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "tl_hyper_collapse": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "tl_hyper_read_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_int, c_void_p],
        "tl_hyper_conv": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_int, c_void_p],
        "tl_hyper_conv_state": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "tl_hyper_write": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "tl_hyper_debug_error": [c_void_p],
    },
    "pooled_attention": {
        "tl_pooled_store": [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_void_p],
        "tl_pooled_attention": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_float, c_int, c_int, c_void_p],
        "tl_pooled_prior": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
        "tl_pooled_attention_debug_error": [c_void_p],
    },
    "sampling": {
        "tl_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_longlong, c_void_p],
    },
}

_functions: dict[str, ctypes._CFuncPtr] = {}


def _fn(library: str, name: str):
    fn = _functions.get(name)
    if fn is None:
        lib = load_library(library)
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[library][name]
        fn.restype = c_longlong if name.endswith("_plan") else c_int
        _functions[name] = fn
    return fn


launch_count = 0  # kernels launched through this module (graph replays are counted by the runner)


def _check(code: int, what: str, kernels: int = 1) -> None:
    global launch_count
    if code == 0:
        launch_count += kernels
        return
    if code == _UNSUPPORTED:
        raise KernelError(f"{what}: sizes or types not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The handle of the current CUDA stream of the current device.  (Asked through the raw
    accessor where torch has one: building a ``torch.cuda.Stream`` object for every launch
    was a third of the host's time in a step of small kernels.)"""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


# ------------------------------------------------------------------ wrappers
def embed(table: torch.Tensor, ids: torch.Tensor, acc: torch.Tensor, scale: float = 1.0) -> None:
    """acc[t] = float32(table[ids[t]]) * scale;  ids int32 [T], acc float32 [T, hidden]."""
    _need_cuda(table, ids, acc)
    tokens, hidden = acc.shape
    assert ids.dtype == torch.int32 and acc.dtype == torch.float32 and acc.is_contiguous()
    assert table.is_contiguous() and table.shape[1] == hidden
    code = _fn("elementwise", "tl_embed")(
        table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), acc.data_ptr(), tokens, hidden,
        table.shape[0], float(scale), _stream())
    _check(code, "embed")


def rms_norm(acc: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, rows=None,
             groups: int = 1) -> None:
    """out[r] = rmsnorm(acc[rows[r] or r]) * weight;  acc float32, weight float32.  ``groups`` > 1:
    every row is normed in that many equal consecutive parts, each by its own root mean square."""
    _need_cuda(acc, weight, out, rows)
    hidden = acc.shape[1]
    num_rows = out.shape[0]
    assert acc.dtype == torch.float32 and weight.dtype == torch.float32
    assert acc.is_contiguous() and out.is_contiguous() and out.shape[1] == hidden
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= num_rows)
    code = _fn("elementwise", "tl_rms_norm")(
        acc.data_ptr(), weight.data_ptr(), _ptr(rows), out.data_ptr(), dtype_code(out.dtype), num_rows,
        hidden, float(eps), int(groups), _stream())
    _check(code, "rms_norm")


def rope_kv(qkv, positions, token_req, block_table, pages, inv_freq, nh, nkv, d, page_size, write_kv=True):
    """Rotate q (in place) and k by position, write k and v into cache pages."""
    _need_cuda(qkv, positions, token_req, block_table, pages, inv_freq)
    tokens = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d
    assert pages.dtype == qkv.dtype and inv_freq.dtype == torch.float32 and inv_freq.numel() == d // 2
    code = _fn("elementwise", "tl_rope_kv")(
        qkv.data_ptr(), dtype_code(qkv.dtype), positions.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], pages.data_ptr(), inv_freq.data_ptr(), tokens, nh, nkv,
        d, page_size, 1 if write_kv else 0, pages.shape[0], _stream())
    _check(code, "rope_kv")


def store_kv(qkv, positions, token_req, block_table, pages, nh, nkv, d, page_size) -> None:
    """Write the k and v heads of the fused ``qkv`` rows to the cache pages, unchanged (for a mixer
    whose position encoding, if any, does not store them itself)."""
    _need_cuda(qkv, positions, token_req, block_table, pages)
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d and pages.dtype == qkv.dtype
    code = _fn("elementwise", "tl_rope_kv")(
        qkv.data_ptr(), dtype_code(qkv.dtype), positions.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], pages.data_ptr(), None, qkv.shape[0], nh, nkv,
        d, page_size, 1, pages.shape[0], _stream())
    _check(code, "store_kv")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need_cuda(gate_up, out)
    tokens, inter = out.shape
    assert gate_up.shape == (tokens, 2 * inter) and gate_up.is_contiguous() and out.is_contiguous()
    assert gate_up.dtype == out.dtype
    code = _fn("elementwise", "tl_swiglu")(
        gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), tokens, inter, _stream())
    _check(code, "swiglu")


def gemm_simt(x, w, out, bias=None, accumulate=False) -> None:
    """out (+)= x @ w.T + bias on CUDA cores, float32 accumulation in ascending k."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and x.dtype == w.dtype
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == N)
    assert not accumulate or out.dtype == torch.float32
    code = _fn("gemm_simt", "tl_gemm_simt")(
        x.data_ptr(), w.data_ptr(), dtype_code(x.dtype), _ptr(bias), out.data_ptr(), dtype_code(out.dtype),
        1 if accumulate else 0, M, N, K, x.stride(0), w.stride(0), out.stride(0), _stream())
    _check(code, "gemm_simt")


def attention_generic(q, q_stride, pages, block_table, token_req, positions, out, tokens, nh, nkv, d,
                      page_size, window, scale, softcap=None, sink: bool = False, gate=None) -> None:
    """Paged causal GQA attention, one warp per (token, head); q may be a view into qkv.
    ``softcap``: scores become softcap * tanh(score / softcap); ``sink``: one is added to the softmax's
    denominator; ``gate`` (float32 [tokens, >= nh * d] rows): the output is multiplied by sigmoid(gate)."""
    _need_cuda(q, pages, block_table, token_req, positions, out, gate)
    assert q.dtype == pages.dtype == out.dtype and out.is_contiguous()
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    code = _fn("attention_generic", "tl_attention_generic")(
        q.data_ptr(), q_stride, pages.data_ptr(), dtype_code(q.dtype), block_table.data_ptr(),
        block_table.shape[1], token_req.data_ptr(), positions.data_ptr(), out.data_ptr(), out.stride(0),
        tokens, nh, nkv, d, page_size, int(window or 0), float(scale), pages.shape[0], float(softcap or 0.0),
        1 if sink else 0, _ptr(gate), gate.stride(0) if gate is not None else 0, _stream())
    _check(code, "attention_generic")


def sample(logits, out, temperature=None, seed=None, counter=None) -> None:
    """out[r] = argmax(logits[r]) or a seeded draw from softmax(logits[r] / temperature[r])."""
    _need_cuda(logits, out, temperature, seed, counter)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    if temperature is not None:
        assert temperature.dtype == torch.float32 and seed.dtype == torch.int64 and counter.dtype == torch.int32
    chunks = -(-vocab // 8192)
    scratch = _workspace(("sample", logits.device), rows * chunks * 8) if chunks > 1 else None
    code = _fn("sampling", "tl_sample")(
        logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(seed), _ptr(counter),
        out.data_ptr(), _ptr(scratch), scratch.numel() * 4 if scratch is not None else 0, _stream())
    _check(code, "sample", 2 if chunks > 1 else 1)


# ------------------------------------------------- around the residual stream
def fill_zero(x: torch.Tensor) -> None:
    """x = 0;  float32, contiguous."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(_fn("stream_ops", "tl_fill_zero")(x.data_ptr(), x.numel(), _stream()), "fill_zero")


def scale_(x: torch.Tensor, alpha: float) -> None:
    """x *= alpha;  float32, contiguous."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(_fn("stream_ops", "tl_scale")(x.data_ptr(), float(alpha), x.numel(), _stream()), "scale")


def scaled_add(acc: torch.Tensor, delta: torch.Tensor, m: float, cast: torch.Tensor | None = None,
               clear: bool = False) -> None:
    """acc += m * delta (float32); ``cast`` (bfloat16, same shape) also receives the updated acc; ``clear``: delta is
    left zeroed."""
    _need_cuda(acc, delta, cast)
    assert acc.dtype == delta.dtype == torch.float32 and acc.shape == delta.shape
    assert acc.is_contiguous() and delta.is_contiguous()
    assert cast is None or (cast.dtype == torch.bfloat16 and cast.shape == acc.shape and cast.is_contiguous())
    code = _fn("stream_ops", "tl_scaled_add")(acc.data_ptr(), delta.data_ptr(), float(m), _ptr(cast), acc.numel(),
                                              1 if clear else 0, _stream())
    _check(code, "scaled_add")


def rms_scaled_add(acc: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, m: float, eps: float,
                   clear: bool = False) -> None:
    """acc[r] += m * y[r] / sqrt(mean(y[r]^2) + eps) * weight;  all float32.  ``clear``: y is left zeroed."""
    _need_cuda(acc, y, weight)
    rows, hidden = acc.shape
    assert acc.dtype == y.dtype == weight.dtype == torch.float32 and y.shape == acc.shape
    assert acc.is_contiguous() and y.is_contiguous() and weight.numel() == hidden
    code = _fn("stream_ops", "tl_rms_scaled_add")(acc.data_ptr(), y.data_ptr(), weight.data_ptr(), float(m),
                                                  float(eps), rows, hidden, 1 if clear else 0, _stream())
    _check(code, "rms_scaled_add")


def rms_scaled_add_partials(acc: torch.Tensor, y: torch.Tensor, partials: torch.Tensor, splits: int, weight: torch.Tensor,
                            m: float, eps: float, clear: bool = False) -> None:
    """``rms_scaled_add`` for a y that still lacks ``splits`` float32 partial sums [splits, rows, hidden] (the start
    of ``partials``) which a product left: they are added inside the kernel (y then holds the sum, or zeros with
    ``clear``)."""
    _need_cuda(acc, y, partials, weight)
    rows, hidden = acc.shape
    assert acc.dtype == y.dtype == partials.dtype == weight.dtype == torch.float32 and acc.is_contiguous()
    assert y.is_contiguous() and y.shape == acc.shape
    assert partials.numel() >= splits * rows * hidden and weight.numel() == hidden
    code = _fn("stream_ops", "tl_rms_scaled_add_partials")(acc.data_ptr(), y.data_ptr(), partials.data_ptr(), splits,
                                                           weight.data_ptr(), float(m), float(eps), rows, hidden,
                                                           1 if clear else 0, _stream())
    _check(code, "rms_scaled_add_partials")


def gated_token_embed(gate: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = gelu_tanh(gate[t]) * table[ids[t]];  gate float32 [T, dim], table and out in the compute type."""
    _need_cuda(gate, table, ids, out)
    tokens, dim = out.shape
    assert gate.dtype == torch.float32 and gate.shape == out.shape and gate.is_contiguous() and out.is_contiguous()
    assert table.dtype == out.dtype and table.shape[1] == dim and table.stride(1) == 1 and ids.dtype == torch.int32
    code = _fn("stream_ops", "tl_gated_token_embed")(
        gate.data_ptr(), table.data_ptr(), table.stride(0), dtype_code(out.dtype), ids.data_ptr(), table.shape[0],
        out.data_ptr(), tokens, dim, _stream())
    _check(code, "gated_token_embed")


def clamped_glu(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
    """out = g * sigmoid(alpha * g) * (u + 1) with g = min(gate_up[:, :I], limit) and
    u = clamp(gate_up[:, I:], -limit, limit)."""
    _need_cuda(gate_up, out)
    tokens, inter = out.shape
    assert gate_up.shape == (tokens, 2 * inter) and gate_up.is_contiguous() and out.is_contiguous()
    assert gate_up.dtype == out.dtype
    code = _fn("stream_ops", "tl_clamped_glu")(gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), tokens,
                                               inter, float(limit), float(alpha), _stream())
    _check(code, "clamped_glu")


# ------------------------------------------------------------ delta-rule mixer
def delta_prepare(proj, w2, w0, a_bias, gates, heads: int, dim: int, rank: int) -> None:
    """From the float32 projections ``proj`` [T, 5 H D + rank] (r | k | v | g | a' | l) to
    ``gates`` [T, H, 3, D]: decay w, unit key u and a * u of every key channel (csrc/delta_rule.cu).
    ``w2`` is the decay's second matrix TRANSPOSED, [rank, H D]."""
    _need_cuda(proj, w2, w0, a_bias, gates)
    tokens = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] == 5 * heads * dim + rank
    assert w2.dtype == w0.dtype == a_bias.dtype == gates.dtype == torch.float32
    assert w2.is_contiguous() and w2.shape == (rank, heads * dim) and gates.is_contiguous()
    assert gates.numel() == tokens * heads * 3 * dim
    code = _fn("delta_rule", "tl_delta_prepare")(proj.data_ptr(), proj.stride(0), w2.data_ptr(), w0.data_ptr(),
                                                 a_bias.data_ptr(), gates.data_ptr(), tokens, heads, dim, rank,
                                                 _stream())
    _check(code, "delta_prepare")


def delta_scan(proj, gates, req_indptr, slots, state, out, requests: int, heads: int, dim: int) -> None:
    """Walks each request's tokens of the step through its slot's state [H, D, D] (float32);
    ``out`` float32 [T, H D] receives S_t^T r_t.  A request whose slot is negative is padding."""
    _need_cuda(proj, gates, req_indptr, slots, state, out)
    assert state.dtype == out.dtype == torch.float32 and state.is_contiguous() and out.is_contiguous()
    assert state.shape[1:] == (heads, dim, dim) and req_indptr.dtype == slots.dtype == torch.int32
    code = _fn("delta_rule", "tl_delta_scan")(proj.data_ptr(), proj.stride(0), gates.data_ptr(), req_indptr.data_ptr(),
                                              slots.data_ptr(), state.data_ptr(), out.data_ptr(), requests, heads, dim,
                                              state.shape[0], _stream())
    _check(code, "delta_scan")


def delta_finish(o, proj, weight, out, heads: int, dim: int, eps: float) -> None:
    """out = o / rms(o per head) * weight * sigmoid(g), g read from ``proj``; out in the compute type."""
    _need_cuda(o, proj, weight, out)
    tokens = o.shape[0]
    assert o.dtype == weight.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous()
    assert out.shape == o.shape == (tokens, heads * dim)
    code = _fn("delta_rule", "tl_delta_finish")(o.data_ptr(), proj.data_ptr(), proj.stride(0), weight.data_ptr(),
                                                out.data_ptr(), dtype_code(out.dtype), tokens, heads, dim, float(eps),
                                                _stream())
    _check(code, "delta_finish")


# ----------------------------------------------------- gated linear attention
def gla_decay(proj, low_offset: int, w2t, bias, decay, rank: int, tau: float) -> None:
    """decay[t, c] = sigmoid(z)^(1 / tau), z = W2 proj[t, low_offset : low_offset + rank] + bias, float32
    (csrc/gla.cu).  ``w2t`` is W2 TRANSPOSED, [rank, channels]."""
    _need_cuda(proj, w2t, bias, decay)
    tokens, channels = decay.shape
    assert proj.dtype == w2t.dtype == bias.dtype == decay.dtype == torch.float32 and proj.stride(1) == 1
    assert w2t.is_contiguous() and w2t.shape == (rank, channels) and decay.is_contiguous() and bias.numel() == channels
    code = _fn("gla", "tl_gla_decay")(proj.data_ptr(), proj.stride(0), low_offset, w2t.data_ptr(), bias.data_ptr(),
                                      decay.data_ptr(), tokens, channels, rank, float(tau), _stream())
    _check(code, "gla_decay")


def gla_scan(proj, decay, req_indptr, slots, state, out, requests: int, heads: int, dim: int, vdim: int,
             qscale: float, fixed_decay: bool = False, token_decay: bool = False, qk_heads: int | None = None) -> None:
    """Walks each request's tokens of the step through its slot's state [H, D, V] (float32):
    S = diag(decay) S + k v^T, out = S^T q * qscale; ``proj`` rows are [q (G D) | k (G D) | v (H V) | ...] with
    G = ``qk_heads`` (default H) heads of q and k, head h reading q/k head h // (H / G).
    ``decay`` is float32 [tokens, H D] (one number a key channel), or with ``fixed_decay`` one constant per head, [H]
    (a retention), or with ``token_decay`` [tokens, H] (one number a token and head).
    A request whose slot is negative is padding."""
    _need_cuda(proj, decay, req_indptr, slots, state, out)
    assert proj.dtype == decay.dtype == state.dtype == out.dtype == torch.float32
    assert not (fixed_decay and token_decay)
    qk_heads = heads if qk_heads is None else int(qk_heads)
    assert decay.numel() == (heads if fixed_decay else proj.shape[0] * heads * (1 if token_decay else dim))
    assert state.is_contiguous() and out.is_contiguous() and decay.is_contiguous() and proj.stride(1) == 1
    assert state.shape[1:] == (heads, dim, vdim) and req_indptr.dtype == slots.dtype == torch.int32
    code = _fn("gla", "tl_gla_scan")(proj.data_ptr(), proj.stride(0), decay.data_ptr(), req_indptr.data_ptr(),
                                     slots.data_ptr(), state.data_ptr(), out.data_ptr(), requests, heads, qk_heads, dim,
                                     vdim, state.shape[0], float(qscale), 1 if fixed_decay else (2 if token_decay else 0),
                                     _stream())
    _check(code, "gla_scan")


def rotate_heads_f32(rows, positions, inv_freq, heads: int, dim: int, dims: int) -> None:
    """Split-half rotation, in place, of the first ``dims`` entries of the first ``heads`` heads of ``dim`` entries
    of every float32 row: entry i pairs with i + dims / 2, angle = float(position) * inv_freq[i]."""
    _need_cuda(rows, positions, inv_freq)
    assert rows.dtype == inv_freq.dtype == torch.float32 and rows.stride(1) == 1 and rows.shape[1] >= heads * dim
    assert positions.dtype == torch.int32 and inv_freq.numel() == dims // 2
    code = _fn("gla", "tl_rotate_heads_f32")(rows.data_ptr(), rows.stride(0), positions.data_ptr(), inv_freq.data_ptr(),
                                             rows.shape[0], heads, dim, dims, _stream())
    _check(code, "rotate_heads_f32")


def gla_finish(o, proj, gate_offset: int, weight, out, heads: int, vdim: int, eps: float) -> None:
    """out = o / rms(o per head) * weight * silu(g), g = proj[:, gate_offset:]; ``weight`` covers one head
    (None: no weight)."""
    _need_cuda(o, proj, weight, out)
    tokens = o.shape[0]
    assert o.dtype == proj.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous()
    assert out.shape == o.shape == (tokens, heads * vdim)
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == vdim)
    code = _fn("gla", "tl_gla_finish")(o.data_ptr(), proj.data_ptr(), proj.stride(0), gate_offset, _ptr(weight),
                                       out.data_ptr(), dtype_code(out.dtype), tokens, heads, vdim, float(eps), _stream())
    _check(code, "gla_finish")


# ------------------------------------------- attention with normed queries and keys
def normed_qk_store(proj, wq, wk, inv_freq, magnitude: float, eps: float, positions, token_req, block_table, pages,
                    page_size: int, q_out, nh: int, nkv: int, d: int, dims: int, v_offset: int, write_kv: bool = True) -> None:
    """From float32 projection rows [q (nh d) | k (nkv d) | ...]: RMS norm of the whole q and the whole k
    (weights ``wq``, ``wk``; None: no norm), rotation of the first ``dims`` entries of every head, q to
    ``q_out``, the key to plane 0 and proj[:, v_offset : v_offset + nkv d] to plane 1 of the cache rows
    (csrc/gated_attention.cu)."""
    _need_cuda(proj, wq, wk, inv_freq, positions, token_req, block_table, pages, q_out)
    tokens = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.is_contiguous() and pages.is_contiguous()
    assert q_out.shape == (tokens, nh * d) and pages.dtype == q_out.dtype
    assert dims == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == dims // 2)
    code = _fn("gated_attention", "tl_normed_qk_store")(
        proj.data_ptr(), proj.stride(0), _ptr(wq), _ptr(wk), _ptr(inv_freq), float(magnitude), float(eps),
        positions.data_ptr(), token_req.data_ptr(), block_table.data_ptr(), block_table.shape[1], pages.data_ptr(),
        dtype_code(q_out.dtype), page_size, pages.shape[0], q_out.data_ptr(), tokens, nh, nkv, d, dims,
        1 if wq is not None else 0, 1 if wk is not None else 0, v_offset, 1 if write_kv else 0, _stream())
    _check(code, "normed_qk_store")


# ------------------------------------------- several residual streams, input convolution, layer norm
def hyper_fanout(acc, z) -> None:
    """z[t, s] = acc[t] for every stream s;  acc float32 [T, width], z float32 [T, n, width]."""
    _need_cuda(acc, z)
    tokens, n, width = z.shape
    assert acc.dtype == z.dtype == torch.float32 and acc.is_contiguous() and z.is_contiguous() and acc.shape == (tokens, width)
    _check(_fn("hyper", "tl_hyper_fanout")(acc.data_ptr(), z.data_ptr(), tokens, n, width, _stream()), "hyper_fanout")


def hyper_collapse(z, acc) -> None:
    """acc[t] = sum_s z[t, s] (ascending s)."""
    _need_cuda(acc, z)
    tokens, n, width = z.shape
    assert acc.dtype == z.dtype == torch.float32 and acc.is_contiguous() and z.is_contiguous() and acc.shape == (tokens, width)
    _check(_fn("hyper", "tl_hyper_collapse")(z.data_ptr(), acc.data_ptr(), tokens, n, width, _stream()), "hyper_collapse")


def hyper_read_norm(z, a, weight, bias, eps: float, out, centre: bool = True, rows=None, write=None, conv=None) -> None:
    """out[r] = norm(sum_s a[s] z[row, s]) * weight (+ bias): a layer norm (``centre``) or an RMS norm of the streams'
    weighted sum.  z float32 [T, n, width], or [T, width] with ``a`` None; ``rows`` (int32) gathers.
    ``write`` = (y, mix, b): ``hyper_write`` of these happens first, in the same pass over z.  ``conv`` = (w, state,
    token_req, slots) in a step whose requests bring ONE token each: out = h + conv(h) as ``hyper_conv`` gives it,
    and the slots' rows move as ``hyper_conv_state`` moves them."""
    _need_cuda(z, a, weight, bias, out, rows)
    y = mix = b = conv_w = conv_state = token_req = slots = None
    taps = max_slots = 0
    if write is not None:
        y, mix, b = write
        _need_cuda(y, mix, b)
        assert rows is None and y.dtype == mix.dtype == b.dtype == torch.float32 and y.is_contiguous() and mix.is_contiguous()
        assert y.shape == (z.shape[0], z.shape[-1]) and mix.shape == (z.shape[1], z.shape[1]) and b.numel() == z.shape[1]
    if conv is not None:
        conv_w, conv_state, token_req, slots = conv
        _need_cuda(conv_w, conv_state, token_req, slots)
        taps = conv_w.shape[1]
        assert conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[0] == z.shape[-1]
        if taps > 1:
            assert conv_state.dtype == torch.float32 and conv_state.is_contiguous()
            assert conv_state.shape[1:] == (taps - 1, z.shape[-1])
            max_slots = conv_state.shape[0]
        else:
            conv_state = None
    n = z.shape[1] if z.dim() == 3 else 1
    width = z.shape[-1]
    count = out.shape[0]
    assert z.dtype == weight.dtype == torch.float32 and z.is_contiguous() and out.is_contiguous() and out.shape[1] == width
    assert (a is None and n == 1) or (a is not None and a.dtype == torch.float32 and a.numel() == n)
    assert rows is not None or count == z.shape[0]
    code = _fn("hyper", "tl_hyper_read_norm")(z.data_ptr(), _ptr(a), weight.data_ptr(), _ptr(bias), _ptr(rows), out.data_ptr(),
                                              dtype_code(out.dtype), count, n, width, float(eps), 1 if centre else 0,
                                              _ptr(y), _ptr(mix), _ptr(b), _ptr(conv_w), _ptr(conv_state), _ptr(token_req),
                                              _ptr(slots), taps, max_slots, _stream())
    _check(code, "hyper_read_norm")


def hyper_conv(h, w, state, token_req, req_indptr, slots, out) -> None:
    """out[t] = h[t] + sum_j w[:, j] h[t - taps + 1 + j] along each request's tokens; the rows before a request's first
    token of the step come from ``state`` [slots, taps - 1, width] (float32; None with one tap, which has no history)."""
    _need_cuda(h, w, state, token_req, req_indptr, slots, out)
    tokens, width = h.shape
    taps = w.shape[1]
    assert h.dtype == w.dtype == torch.float32 and h.is_contiguous() and w.is_contiguous() and w.shape[0] == width
    assert out.is_contiguous() and out.shape == h.shape
    if taps > 1:
        assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (taps - 1, width)
    code = _fn("hyper", "tl_hyper_conv")(h.data_ptr(), w.data_ptr(), _ptr(state) if taps > 1 else 0, token_req.data_ptr(),
                                         req_indptr.data_ptr(), slots.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
                                         tokens, width, taps, state.shape[0] if taps > 1 else 0, _stream())
    _check(code, "hyper_conv")


def hyper_conv_state(h, state, req_indptr, slots, requests: int) -> None:
    """After ``hyper_conv``: every request's slot keeps the last taps - 1 rows of ``h`` it has seen."""
    _need_cuda(h, state, req_indptr, slots)
    width = h.shape[1]
    taps = state.shape[1] + 1
    assert h.dtype == state.dtype == torch.float32 and h.is_contiguous() and state.is_contiguous() and state.shape[2] == width
    code = _fn("hyper", "tl_hyper_conv_state")(h.data_ptr(), state.data_ptr(), req_indptr.data_ptr(), slots.data_ptr(),
                                               requests, width, taps, state.shape[0], _stream())
    _check(code, "hyper_conv_state")


def hyper_write(z, y, mix, b) -> None:
    """z[t, to] <- sum_s mix[s, to] z[t, s] + b[to] y[t], all streams from the old ones; y is left zeroed."""
    _need_cuda(z, y, mix, b)
    tokens, n, width = z.shape
    assert z.dtype == y.dtype == mix.dtype == b.dtype == torch.float32 and z.is_contiguous() and y.is_contiguous()
    assert y.shape == (tokens, width) and mix.is_contiguous() and mix.shape == (n, n) and b.numel() == n
    _check(_fn("hyper", "tl_hyper_write")(z.data_ptr(), y.data_ptr(), mix.data_ptr(), b.data_ptr(), tokens, n, width,
                                          _stream()), "hyper_write")


# ------------------------------ attention over a window of tokens and pooled blocks of older ones
def pooled_store(proj, k_offset: int, v_offset: int, pages, block_table, token_req, positions, req_indptr, slots, pooled,
                 nkv: int, d: int, dv: int, page_size: int, pool: int) -> None:
    """The step's keys and values (``proj[:, k_offset:]``: nkv x d, ``proj[:, v_offset:]``: nkv x dv) into the
    pages (one plane of rows [key | value], or a key plane and a value plane where d = dv); a token that completes a
    block of ``pool`` tokens also writes the block's mean row into ``pooled`` [slots, blocks, nkv, d + dv] (float32)
    of its request's slot (csrc/pooled_attention.cu)."""
    _need_cuda(proj, pages, block_table, token_req, positions, req_indptr, slots, pooled)
    assert pages.dtype == proj.dtype and proj.stride(1) == 1 and pages.is_contiguous() and pooled.is_contiguous()
    assert pooled.dtype == torch.float32 and pooled.shape[2:] == (nkv, d + dv)
    split = _pooled_split(pages, nkv, d, dv, page_size)
    code = _fn("pooled_attention", "tl_pooled_store")(
        proj.data_ptr(), proj.stride(0), k_offset, v_offset, pages.data_ptr(), dtype_code(proj.dtype),
        block_table.data_ptr(), block_table.shape[1], token_req.data_ptr(), positions.data_ptr(), req_indptr.data_ptr(),
        slots.data_ptr(), pooled.data_ptr(), pooled.shape[1], pooled.shape[0], proj.shape[0], nkv, d, dv, page_size, pool,
        pages.shape[0], split, _stream())
    _check(code, "pooled_store")


def _pooled_split(pages, nkv: int, d: int, dv: int, page_size: int) -> int:
    """1: the pages hold a key plane and a value plane; 0: one plane of joined rows."""
    if pages.shape[1] == 2:
        assert d == dv and pages.shape[1:] == (2, nkv, page_size, d)
        return 1
    assert pages.shape[1:] == (1, nkv, page_size, d + dv)
    return 0


def pooled_attention(q, pages, block_table, token_req, positions, slots, pooled, out, nh: int, nkv: int, d: int, dv: int,
                     page_size: int, size: int, pool: int, scale: float) -> None:
    """One softmax over the last ``size`` tokens and the pooled rows of the whole blocks before them; one warp a
    (token, head), float32 inside.  q: rows whose first nh x d entries are the queries."""
    _need_cuda(q, pages, block_table, token_req, positions, slots, pooled, out)
    tokens = q.shape[0]
    assert pages.dtype == q.dtype == out.dtype and q.stride(1) == 1 and out.stride(1) == 1 and pages.is_contiguous()
    assert out.shape == (tokens, nh * dv) and pooled.dtype == torch.float32 and pooled.is_contiguous()
    code = _fn("pooled_attention", "tl_pooled_attention")(
        q.data_ptr(), q.stride(0), pages.data_ptr(), dtype_code(q.dtype), block_table.data_ptr(), block_table.shape[1],
        token_req.data_ptr(), positions.data_ptr(), slots.data_ptr(), pooled.data_ptr(), pooled.shape[1], pooled.shape[0],
        out.data_ptr(), out.stride(0), tokens, nh, nkv, d, dv, page_size, size, pool, float(scale), pages.shape[0],
        _pooled_split(pages, nkv, d, dv, page_size), _stream())
    _check(code, "pooled_attention")


def pooled_prior(q, token_req, positions, slots, pooled, ml, acc, nh: int, nkv: int, d: int, dv: int, size: int,
                 pool: int, scale: float) -> None:
    """The softmax state of every (token, head) over the pooled rows of the whole blocks before its window, alone:
    ``ml`` [tokens, nh, 2] = (max in log2 units of the scaled score, sum; (-inf, 0) where no block is seen), ``acc``
    [tokens, nh, dv] the unnormalized weighted values, float32.  ``attention_mma`` and ``attention_tc`` take the two
    as their ``prior``."""
    _need_cuda(q, token_req, positions, slots, pooled, ml, acc)
    tokens = q.shape[0]
    assert q.stride(1) == 1 and pooled.dtype == ml.dtype == acc.dtype == torch.float32
    assert pooled.is_contiguous() and ml.is_contiguous() and acc.is_contiguous()
    assert ml.shape == (tokens, nh, 2) and acc.shape == (tokens, nh, dv) and pooled.shape[2:] == (nkv, d + dv)
    code = _fn("pooled_attention", "tl_pooled_prior")(
        q.data_ptr(), q.stride(0), dtype_code(q.dtype), token_req.data_ptr(), positions.data_ptr(), slots.data_ptr(),
        pooled.data_ptr(), pooled.shape[1], pooled.shape[0], ml.data_ptr(), acc.data_ptr(), tokens, nh, nkv, d, dv, size,
        pool, float(scale), _stream())
    _check(code, "pooled_prior")


# ------------------------------------------- state-space mixer, gated norms, gates
GLU_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def glu_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu", row_scale=None) -> None:
    """out = act(gate) * up over rows [gate (I) | up (I)], act "silu" or "gelu_tanh"; ``row_scale`` (float32 [tokens]):
    every row is multiplied by its token's number before it is rounded."""
    _need_cuda(gate_up, out, row_scale)
    tokens, inter = out.shape
    assert gate_up.is_contiguous() and out.is_contiguous() and gate_up.shape == (tokens, 2 * inter) and gate_up.dtype == out.dtype
    assert row_scale is None or (row_scale.dtype == torch.float32 and row_scale.numel() == tokens)
    code = _fn("stream_ops", "tl_glu_act")(gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), tokens, inter,
                                           GLU_ACTIVATIONS[activation], _ptr(row_scale), _stream())
    _check(code, "glu_act")


def ssm_conv(proj, xbc_offset: int, dt_offset: int, weight, bias, dt_bias, a_log, state, token_req, req_indptr, slots,
             scan_in, x_out, decay, heads: int, vdim: int, gn: int, update_state: bool = False) -> None:
    """The front of a selective state-space mixer (csrc/ssm.cu): causal convolution over time of the channels
    proj[:, xbc_offset:] = [x (H V) | B (G N) | C (G N)] with ``weight`` [channels, taps] (last column: the current
    token) and ``bias``, silu; dt = softplus(proj[:, dt_offset:] + dt_bias); writes the scan's rows
    ``scan_in`` [C | B | dt x], ``x_out`` and ``decay`` [tokens, H] = exp(-exp(a_log) dt).  ``state`` [slots, taps - 1,
    channels] holds each request's last raw inputs (None when taps == 1).  ``update_state``: every request brings ONE
    token, and the kernel also moves that token's raw inputs into the slot's rows (else ``ssm_conv_state`` does)."""
    _need_cuda(proj, weight, bias, dt_bias, a_log, state, token_req, req_indptr, slots, scan_in, x_out, decay)
    tokens = proj.shape[0]
    channels, taps = weight.shape
    assert channels == heads * vdim + 2 * gn and proj.dtype == torch.float32 and proj.stride(1) == 1
    assert all(t.dtype == torch.float32 and t.is_contiguous() for t in (weight, bias, dt_bias, a_log, scan_in, x_out, decay))
    assert scan_in.shape == (tokens, 2 * gn + heads * vdim) and x_out.shape == (tokens, heads * vdim) and decay.shape == (tokens, heads)
    assert taps == 1 or (state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (taps - 1, channels))
    code = _fn("ssm", "tl_ssm_conv")(proj.data_ptr(), proj.stride(0), xbc_offset, dt_offset, weight.data_ptr(), bias.data_ptr(),
                                     dt_bias.data_ptr(), a_log.data_ptr(), _ptr(state), token_req.data_ptr(),
                                     req_indptr.data_ptr(), slots.data_ptr(), scan_in.data_ptr(), x_out.data_ptr(),
                                     decay.data_ptr(), tokens, taps, heads, vdim, gn, state.shape[0] if state is not None else 0,
                                     1 if update_state else 0, _stream())
    _check(code, "ssm_conv")


def ssm_conv_state(proj, xbc_offset: int, state, req_indptr, slots, requests: int) -> None:
    """Moves the last taps - 1 raw inputs proj[:, xbc_offset : xbc_offset + channels] of every request into its slot's
    rows of ``state`` [slots, taps - 1, channels] (rows of the old state where the portion is shorter)."""
    _need_cuda(proj, state, req_indptr, slots)
    assert proj.dtype == state.dtype == torch.float32 and state.is_contiguous() and proj.stride(1) == 1
    code = _fn("ssm", "tl_ssm_conv_state")(proj.data_ptr(), proj.stride(0), xbc_offset, state.data_ptr(), req_indptr.data_ptr(),
                                           slots.data_ptr(), requests, state.shape[2], state.shape[1] + 1, state.shape[0],
                                           _stream())
    _check(code, "ssm_conv_state")


def gated_norm(o, gate, weight, out, groups: int, eps: float, gate_first: bool, gate_act: str, x=None, skip=None,
               vdim: int = 1) -> None:
    """out = rmsnorm_groups(y) * weight with a gate: y = o (+ skip[c // vdim] * x), ``gate_first``: y * act(gate) goes
    through the norm, else the normed and weighted row is multiplied by act(gate).  ``gate``: float32 rows (a view);
    act "silu" or "sigmoid"; the RMS norm is taken over ``groups`` equal parts of the row; all float32 inside."""
    _need_cuda(o, gate, weight, out, x, skip)
    tokens, width = o.shape
    assert o.dtype == gate.dtype == weight.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous()
    assert gate.stride(1) == 1 and gate.shape == o.shape == out.shape and weight.numel() == width
    assert (x is None) == (skip is None) and (x is None or (x.dtype == torch.float32 and x.is_contiguous() and x.shape == o.shape))
    code = _fn("ssm", "tl_gated_norm")(o.data_ptr(), _ptr(x), _ptr(skip), gate.data_ptr(), gate.stride(0), weight.data_ptr(),
                                       out.data_ptr(), dtype_code(out.dtype), tokens, width, int(groups), int(vdim),
                                       1 if gate_first else 0, {"silu": 0, "sigmoid": 1}[gate_act], float(eps), _stream())
    _check(code, "gated_norm")


def activate_silu_(rows, cols: int) -> None:
    """silu, in place, on the first ``cols`` columns of float32 rows."""
    _need_cuda(rows)
    assert rows.dtype == torch.float32 and rows.stride(1) == 1 and cols <= rows.shape[1]
    _check(_fn("ssm", "tl_activate_silu")(rows.data_ptr(), rows.stride(0), rows.shape[0], cols, _stream()), "activate_silu")


def gate_mul_(rows, gate) -> None:
    """rows *= sigmoid(gate): ``rows`` contiguous in the compute type, ``gate`` float32 rows (a view) of the same shape."""
    _need_cuda(rows, gate)
    assert rows.is_contiguous() and gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == rows.shape
    code = _fn("ssm", "tl_gate_mul")(rows.data_ptr(), dtype_code(rows.dtype), gate.data_ptr(), gate.stride(0), rows.shape[0],
                                     rows.shape[1], _stream())
    _check(code, "gate_mul")


def token_gate(x, w, out) -> None:
    """out[t] = sigmoid(w . x[t]) in float32; ``w`` float32 [hidden]."""
    _need_cuda(x, w, out)
    tokens, hidden = x.shape
    assert w.dtype == out.dtype == torch.float32 and w.numel() == hidden and out.numel() == tokens and x.stride(1) == 1
    code = _fn("ssm", "tl_token_gate")(x.data_ptr(), x.stride(0), dtype_code(x.dtype), w.data_ptr(), out.data_ptr(), tokens,
                                       hidden, _stream())
    _check(code, "token_gate")


# ------------------------------------------------------- routed feed-forward
def moe_tile_rows() -> int:
    """Rows of a tile of the grouped CUDA-core products (every expert's rows are padded to whole tiles)."""
    return _fn("moe", "tl_moe_tile_rows")()


def moe_route(x, router, choice, weight, softmax_scores: bool = False, renormalize: bool = False, groups: int = 1,
              keep: int = 1, renorm_eps: float = 0.0, correction=None, scale: float = 1.0, token_gate=None) -> None:
    """choice[t, j], weight[t, j]: the ``top`` experts of every token by score (sigmoid or softmax of the
    float32 router logits) and their scores (csrc/moe.cu), divided by their sum + ``renorm_eps`` if
    ``renormalize``.  ``groups`` > 1: the experts form that many equal groups of neighbours and only experts of the
    ``keep`` groups with the largest best score can be chosen.  ``correction`` (float32 [experts]): the choice goes
    by score + correction, the weights stay the scores.  ``scale`` multiplies the weights.  ``token_gate`` (w float32
    [hidden], out float32 [tokens]): the same kernel also writes out[t] = sigmoid(w . x[t]), the gate of an always-on
    expert beside the routed ones."""
    gate_w, gate_out = token_gate if token_gate is not None else (None, None)
    _need_cuda(x, router, choice, weight, correction, gate_w, gate_out)
    assert gate_w is None or (gate_w.dtype == gate_out.dtype == torch.float32 and gate_w.numel() == x.shape[1]
                              and gate_out.numel() == x.shape[0] and gate_w.is_contiguous() and gate_out.is_contiguous())
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == router.shape[0])
    tokens, hidden = x.shape
    experts, top = router.shape[0], choice.shape[1]
    assert router.dtype == torch.float32 and router.is_contiguous() and router.shape[1] == hidden and x.stride(1) == 1
    assert choice.dtype == torch.int32 and weight.dtype == torch.float32 and choice.is_contiguous() and weight.is_contiguous()
    code = _fn("moe", "tl_moe_route")(x.data_ptr(), x.stride(0), dtype_code(x.dtype), router.data_ptr(), choice.data_ptr(),
                                      weight.data_ptr(), tokens, hidden, experts, top, 1 if softmax_scores else 0,
                                      1 if renormalize else 0, int(groups), int(keep), float(renorm_eps), _ptr(correction),
                                      float(scale), _ptr(gate_w), _ptr(gate_out), _stream())
    _check(code, "moe_route")


def moe_plan(choice, position, plan, experts: int, tile: int) -> None:
    """position[t, j]: the row of (token, choice) in the expert-sorted order, every expert's rows padded to
    whole tiles of ``tile`` rows; plan[0] tiles in use, plan[1 + i] the expert of tile i.  A choice >= ``experts``
    (an identity expert) has no row: its position is -1."""
    _need_cuda(choice, position, plan)
    assert position.dtype == plan.dtype == torch.int32 and position.numel() == choice.numel()
    code = _fn("moe", "tl_moe_plan")(choice.data_ptr(), position.data_ptr(), plan.data_ptr(), choice.numel(), experts, tile,
                                     plan.numel() - 1, _stream())
    _check(code, "moe_plan")


def moe_scatter(x, position, weight, out, top: int, weighted: bool) -> None:
    """out[position[t, j]] = x[t] (* weight[t, j] if ``weighted``)."""
    _need_cuda(x, position, weight, out)
    tokens, hidden = x.shape
    assert out.dtype == x.dtype and out.is_contiguous() and out.shape[1] == hidden and x.stride(1) == 1
    code = _fn("moe", "tl_moe_scatter")(x.data_ptr(), x.stride(0), dtype_code(x.dtype), position.data_ptr(), weight.data_ptr(),
                                        out.data_ptr(), tokens, hidden, top, 1 if weighted else 0, _stream())
    _check(code, "moe_scatter")


def moe_gemm_simt(x, w, out, plan, glu: bool = False, limit: float = 0.0, alpha: float = 0.0) -> None:
    """Grouped product over expert-sorted rows on CUDA cores: out[r] = W_e(r) x[r]; ``w`` [experts, N, K], or
    with ``glu`` [experts, 2 N, K] ([gate; up]) and the clamped gated activation applied."""
    _need_cuda(x, w, out, plan)
    rows, K = x.shape
    N = out.shape[1]
    assert x.is_contiguous() and w.is_contiguous() and out.is_contiguous() and w.dtype == x.dtype
    assert w.shape[1:] == ((2 if glu else 1) * N, K) and rows == (plan.numel() - 1) * moe_tile_rows() == out.shape[0]
    code = _fn("moe", "tl_moe_gemm_simt")(x.data_ptr(), w.data_ptr(), dtype_code(x.dtype), out.data_ptr(),
                                          dtype_code(out.dtype), plan.data_ptr(), plan.numel() - 1, N, K, 1 if glu else 0,
                                          float(limit), float(alpha), _stream())
    _check(code, "moe_gemm_simt")


def moe_combine(y, position, weight, side, top: int, weighted: bool, x=None) -> None:
    """side[t] += sum_j y[position[t, j]] (* weight[t, j] if ``weighted``), float32, in the order of j.  Where a
    position is -1 (an identity expert) the token's own row of ``x`` stands for the product's row."""
    _need_cuda(y, position, weight, side, x)
    tokens, hidden = side.shape
    assert y.dtype == side.dtype == torch.float32 and y.is_contiguous() and side.is_contiguous() and y.shape[1] == hidden
    assert x is None or (x.shape == (tokens, hidden) and x.stride(1) == 1)
    code = _fn("moe", "tl_moe_combine")(y.data_ptr(), position.data_ptr(), weight.data_ptr(), side.data_ptr(), tokens,
                                        hidden, top, 1 if weighted else 0, _ptr(x), x.stride(0) if x is not None else 0,
                                        dtype_code(x.dtype) if x is not None else 0, _stream())
    _check(code, "moe_combine")


# ------------------------------------------------------------ latent attention
def latent_prepare(down, q_rank, kv_rank, rot_dim, rot_dims, q_norm, kv_norm, inv_freq, eps, positions, token_req,
                   block_table, pages, page_size, q_latent, write_kv: bool) -> None:
    """Norms of the query latent and (``write_kv``) of the key/value latent, rotation of the shared
    key part, and the write of the token's cache row (csrc/latent_attention.cu)."""
    _need_cuda(down, q_norm, kv_norm, inv_freq, positions, token_req, block_table, pages, q_latent)
    tokens = down.shape[0]
    assert down.dtype == torch.float32 and down.stride(1) == 1
    assert down.shape[1] == q_rank + ((kv_rank + rot_dim) if write_kv else 0)
    assert q_rank == 0 or (q_latent.is_contiguous() and q_latent.shape == (tokens, q_rank))
    assert not write_kv or ((q_latent is None or pages.dtype == q_latent.dtype) and pages.is_contiguous())
    code = _fn("latent_attention", "tl_latent_prepare")(
        down.data_ptr(), down.stride(0), q_rank, kv_rank, rot_dim, rot_dims, _ptr(q_norm), _ptr(kv_norm),
        inv_freq.data_ptr(), float(eps), positions.data_ptr(), token_req.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], pages.data_ptr(), dtype_code(pages.dtype), page_size, pages.shape[0],
        _ptr(q_latent), 1 if write_kv else 0, tokens, _stream())
    _check(code, "latent_prepare")


def latent_absorb_q(q, uk, inv_freq, positions, q_abs, heads, dim, rot_dim, rot_dims, kv_rank, fold: bool = True,
                    plain_out=None) -> None:
    """q float32 [T, H (dim + rot)] -> q_abs [T, H, kv_rank + rot]: W_uk,h^T q_plain and the rotated part.
    ``fold`` False: only the rotated part is written (the folded part comes from a tensor-core product of
    ``plain_out``, which receives q_plain [T, H dim] in the compute type)."""
    _need_cuda(q, uk, inv_freq, positions, q_abs, plain_out)
    tokens = q.shape[0]
    assert q.dtype == torch.float32 and q.stride(1) == 1 and q.shape[1] == heads * (dim + rot_dim)
    assert uk.dtype == q_abs.dtype and uk.is_contiguous() and uk.shape == (heads * dim, kv_rank)
    assert q_abs.is_contiguous() and q_abs.numel() == tokens * heads * (kv_rank + rot_dim)
    assert plain_out is None or (plain_out.dtype == q_abs.dtype and plain_out.is_contiguous()
                                 and plain_out.numel() == tokens * heads * dim)
    code = _fn("latent_attention", "tl_latent_absorb_q")(
        q.data_ptr(), q.stride(0), uk.data_ptr(), dtype_code(uk.dtype), inv_freq.data_ptr(), positions.data_ptr(),
        q_abs.data_ptr(), _ptr(plain_out), tokens, heads, dim, rot_dim, rot_dims, kv_rank, 1 if fold else 0, _stream())
    _check(code, "latent_absorb_q")


def latent_attention(q_abs, pages, block_table, token_req, positions, out, tokens, heads, dk, dv, page_size,
                     scale) -> None:
    """Causal attention of every (token, head) over the cached rows of its request, in the latent
    space: keys are whole rows (dk), values their first dv entries; one warp per (token, head)."""
    _need_cuda(q_abs, pages, block_table, token_req, positions, out)
    assert q_abs.dtype == pages.dtype == out.dtype and q_abs.is_contiguous() and out.is_contiguous()
    assert pages.is_contiguous()
    code = _fn("latent_attention", "tl_latent_attention")(
        q_abs.data_ptr(), pages.data_ptr(), dtype_code(out.dtype), block_table.data_ptr(), block_table.shape[1],
        token_req.data_ptr(), positions.data_ptr(), out.data_ptr(), tokens, heads, dk, dv, page_size, float(scale),
        pages.shape[0], _stream())
    _check(code, "latent_attention")


def latent_attention_mma_supported(dk: int, dv: int) -> bool:
    """Sizes the tensor-core latent attention takes (multiples of 16, value size up to 512)."""
    return bool(_fn("latent_attention_mma", "tl_latent_attention_mma_supported")(dk, dv))


def latent_attention_mma(q_abs, pages, block_table, req_indptr, kv_before, tile_req, tile_row, tiles, out, tokens,
                         heads, dk, dv, page_size, scale, splits: int = 1) -> None:
    """Latent-space attention on the tensor cores (csrc/latent_attention_mma.cu), bfloat16.  Row tiles
    of 64 packed (token, head) rows: ``tile_req``/``tile_row`` name each tile's request and first row,
    or are None when every request brings one token.  ``splits`` > 1 (single tokens only): that many
    CTAs share a request's keys and a second kernel merges them."""
    _need_cuda(q_abs, pages, block_table, req_indptr, kv_before, tile_req, tile_row, out)
    assert q_abs.dtype == pages.dtype == out.dtype == torch.bfloat16
    assert q_abs.is_contiguous() and out.is_contiguous() and pages.is_contiguous()
    part_o = part_ml = None
    if splits > 1:
        rows = tokens * heads
        ws = _workspace(("latent_attention", q_abs.device), rows * splits * (dv + 2) * 4)
        part_o, part_ml = ws, ws[rows * splits * dv:]
    code = _fn("latent_attention_mma", "tl_latent_attention_mma")(
        q_abs.data_ptr(), pages.data_ptr(), block_table.data_ptr(), block_table.shape[1], req_indptr.data_ptr(),
        kv_before.data_ptr(), _ptr(tile_req), _ptr(tile_row), tiles, out.data_ptr(), tokens, heads, dk, dv, page_size,
        float(scale), pages.shape[0], splits, _ptr(part_o), _ptr(part_ml), _stream())
    _check(code, "latent_attention_mma", 2 if splits > 1 else 1)


def latent_expand_o(o_lat, uv, out, heads, vdim, kv_rank, gate=None) -> None:
    """out[t, h] = W_uv,h o_lat[t, h] (* sigmoid(gate[t, h]));  uv [H vdim, kv_rank], out [T, H vdim]; ``gate``: float32
    rows (a view) of out's shape."""
    _need_cuda(o_lat, uv, out, gate)
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == out.shape)
    tokens = out.shape[0]
    assert o_lat.dtype == uv.dtype == out.dtype and o_lat.is_contiguous() and uv.is_contiguous() and out.is_contiguous()
    assert uv.shape == (heads * vdim, kv_rank) and out.shape == (tokens, heads * vdim)
    code = _fn("latent_attention", "tl_latent_expand_o")(o_lat.data_ptr(), uv.data_ptr(), out.data_ptr(),
                                                         dtype_code(out.dtype), tokens, heads, vdim, kv_rank, _ptr(gate),
                                                         gate.stride(0) if gate is not None else 0, _stream())
    _check(code, "latent_expand_o")


# ---------------------------------------------------------------- slot records
def slot_record_rows() -> int:
    return _fn("slots", "tl_slot_record_rows")()


def slot_command_words(lanes: int, capacity: int) -> int:
    """int32 words of the command block of a decode step (csrc/slots.cu)."""
    return _fn("slots", "tl_slot_command_words")(lanes, capacity)


def slot_gather(command, lanes: int, groups: int, max_slots: int, width: int, page_size: int, records, slot_tables,
                token, position, kv_before, slot, seed, temperature, counter, lane_tables) -> None:
    """From the slot records (and the command block's news) to the lane-indexed words a decode
    step's kernels read: tokens, positions, sampling words, block-table rows."""
    _need_cuda(command, records, slot_tables, token, position, kv_before, slot, seed, temperature, counter, lane_tables)
    assert records.dtype == torch.int32 and records.is_contiguous() and records.shape[1] == max_slots
    assert seed.dtype == torch.int64 and temperature.dtype == torch.float32
    code = _fn("slots", "tl_slot_gather")(
        command.data_ptr(), lanes, groups, max_slots, width, page_size, records.data_ptr(), _ptr(slot_tables),
        token.data_ptr(), position.data_ptr(), kv_before.data_ptr(), slot.data_ptr(), seed.data_ptr(),
        temperature.data_ptr(), counter.data_ptr(), _ptr(lane_tables), _stream())
    _check(code, "slot_gather")


def slot_advance(command, lanes: int, max_slots: int, sampled, records) -> None:
    """After sampling: each live lane's slot takes the sampled token, position + 1, counter + 1."""
    _need_cuda(command, sampled, records)
    code = _fn("slots", "tl_slot_advance")(command.data_ptr(), lanes, max_slots, sampled.data_ptr(),
                                           records.data_ptr(), _stream())
    _check(code, "slot_advance")


# ------------------------------------------------------- tensor-core products
EPI_STORE_BF16, EPI_ACCUM_F32, EPI_SWIGLU_BF16, EPI_STORE_F32 = 0, 1, 2, 3
_workspaces: dict = {}
_outgrown: list = []  # kept alive: captured CUDA graphs may still hold their addresses


def _workspace(device, nbytes: int) -> torch.Tensor:
    """A float32 scratch buffer per device that only grows (split-K partial sums)."""
    ws = _workspaces.get(device)
    if ws is None or ws.numel() * 4 < nbytes:
        if ws is not None:
            _outgrown.append(ws)
        where = device[1] if isinstance(device, tuple) else device
        ws = torch.empty(max(nbytes // 4 + 1, 1 << 22), dtype=torch.float32, device=where)
        _workspaces[device] = ws
    return ws


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Sizes the tcgen05 product takes: K and both row strides multiples of 8 elements,
    16-byte aligned bases."""
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.stride(1) == 1 and w.stride(1) == 1)


# The step context that holds unfinished partial sums in the shared workspace, if any; it
# is asked to finish them before another product overwrites the workspace.
workspace_holder = None


def _release_workspace() -> None:
    if workspace_holder is not None:
        workspace_holder.flush_pending()


_plans: dict = {}  # (M, N, K) -> (workspace bytes, swapped orientation, splits): fixed for a process


def _gemm_plan(M: int, N: int, K: int) -> tuple:
    plan = _plans.get((M, N, K))
    if plan is None:
        swap, splits = ctypes.c_int(0), ctypes.c_int(0)
        need = _fn("gemm_tc", "tl_gemm_tc_plan")(M, N, K, ctypes.byref(swap), ctypes.byref(splits))
        plan = _plans[(M, N, K)] = (need, bool(swap.value), splits.value)
    return plan


def gemm_tc(x, w, out, bias=None, epilogue=EPI_STORE_BF16, cta_pairs=None) -> None:
    """out (+)= x @ w.T (+ bias) on the tcgen05 tensor cores; see csrc/gemm_tc.cu.
    ``cta_pairs``: for many tokens, True forces the kernel in which two CTAs share one 256-row
    MMA, False the single-CTA kernel; None lets the library choose (pairs where their 256-row tiles cover no more rows than 128-row tiles)."""
    _need_cuda(x, w, out, bias)
    _release_workspace()
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1
    want = torch.bfloat16 if epilogue in (EPI_STORE_BF16, EPI_SWIGLU_BF16) else torch.float32
    assert out.dtype == want and out.shape == (M, N // 2 if epilogue == EPI_SWIGLU_BF16 else N)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == N)
    need, _, splits = _gemm_plan(M, N, K)
    ws = _workspace(x.device, need) if need else None
    kernels = 2 if need and splits > 1 else 1  # several splits: product + finishing pass
    code = _fn("gemm_tc", "tl_gemm_tc")(
        x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), out.stride(0), epilogue, M, N, K, x.stride(0),
        w.stride(0), _ptr(ws), ws.numel() * 4 if ws is not None else 0, {None: 0, True: 2, False: 3}[cta_pairs], None,
        _stream())
    _check(code, "gemm_tc", kernels)


def gemm_tc_glu(x, w, out, limit: float, alpha: float) -> None:
    """out = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit), where gate
    and up are the 16-interleaved rows of ``w`` applied to ``x``: the product and the activation as one kernel
    (the gated epilogue of csrc/gemm_tc.cu).  out bfloat16 [M, N / 2]."""
    _need_cuda(x, w, out)
    _release_workspace()
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1 and out.dtype == torch.bfloat16 and out.shape == (M, N // 2)
    need, _, splits = _gemm_plan(M, N, K)
    ws = _workspace(x.device, need) if need else None
    code = _fn("gemm_tc", "tl_gemm_tc_glu")(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), out.stride(0), M, N, K, x.stride(0), w.stride(0), _ptr(ws),
        ws.numel() * 4 if ws is not None else 0, float(limit), float(alpha), _stream())
    _check(code, "gemm_tc_glu", 2 if need and splits > 1 else 1)


def gemm_tc_gated(x, w, out, activation: str = "silu", bias=None, row_scale=None) -> None:
    """out = act(gate + b_gate) * (up + b_up) (* row_scale[token]), where gate and up are the 16-interleaved rows of
    ``w`` applied to ``x``: the product, the biases, the activation ("silu" or "gelu_tanh") and the token's factor as
    one kernel (the gated epilogue of csrc/gemm_tc.cu).  ``bias`` float32 [N], interleaved like the rows of ``w``;
    ``row_scale`` float32 [M]; out bfloat16 [M, N / 2]."""
    _need_cuda(x, w, out, bias, row_scale)
    _release_workspace()
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1 and out.dtype == torch.bfloat16 and out.shape == (M, N // 2)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous())
    assert row_scale is None or (row_scale.dtype == torch.float32 and row_scale.numel() == M and row_scale.is_contiguous())
    need, _, splits = _gemm_plan(M, N, K)
    ws = _workspace(x.device, need) if need else None
    code = _fn("gemm_tc", "tl_gemm_tc_gated")(
        x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(row_scale), out.data_ptr(), out.stride(0), M, N, K, x.stride(0),
        w.stride(0), _ptr(ws), ws.numel() * 4 if ws is not None else 0, GLU_ACTIVATIONS[activation], _stream())
    _check(code, "gemm_tc_gated", 2 if need and splits > 1 else 1)


GROUPED_TILE_ROWS = 128  # rows of a tile of the grouped tcgen05 product: every group's rows are padded to these
GROUPED_TILE_ROWS_FEW = 16  # ... and where a group has few rows (the weight-streaming orientation)


def gemm_tc_grouped(x, w, out, plan, glu: bool = False, limit: float = 0.0, alpha: float = 0.0,
                    tile_rows: int = GROUPED_TILE_ROWS) -> None:
    """Grouped product over group-sorted rows on the tcgen05 tensor cores (csrc/gemm_tc.cu with a plan):
    out[r] = W_g(r) x[r].  ``x`` [rows, K] bfloat16 with rows = tile_rows * tiles; ``tile_rows`` 128 (the
    persistent kernel) or 16 (few rows a group: the weight-streaming orientation);
    ``plan`` int32 [1 + tiles] on the device: plan[0] tiles in use, plan[1 + i] the group of row tile i;
    ``w`` [groups, N, K]; ``out`` [rows, N] float32 or bfloat16, or with ``glu`` (``w`` [groups, 2 F, K], gate
    and up rows interleaved by 16) [rows, F] bfloat16 with the clamped gated activation applied."""
    _need_cuda(x, w, out, plan)
    _release_workspace()
    rows, K = x.shape
    groups, N = w.shape[0], w.shape[1]
    assert x.dtype == w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous() and w.shape[2] == K
    assert rows == (plan.numel() - 1) * tile_rows == out.shape[0] and plan.dtype == torch.int32
    assert out.stride(1) == 1 and out.shape[1] == (N // 2 if glu else N)
    if glu:
        assert out.dtype == torch.bfloat16
        epilogue = EPI_SWIGLU_BF16
    else:
        epilogue = EPI_STORE_BF16 if out.dtype == torch.bfloat16 else EPI_STORE_F32
    code = _fn("gemm_tc", "tl_gemm_tc_grouped")(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), out.stride(0), epilogue, rows, N, K, groups, plan.data_ptr(),
        tile_rows, float(limit), float(alpha), _stream())
    _check(code, "gemm_tc_grouped")


def gemm_tc_deferred(x, w):
    """The product x @ w.T left as float32 partial sums ``[splits, M, N]`` for a fused
    finishing kernel.  Returns (partials, splits), or None when the sizes run in a
    kernel that writes its output directly (many tokens, no K splits)."""
    _need_cuda(x, w)
    _release_workspace()
    M, K = x.shape
    N = w.shape[0]
    need, swap, planned = _gemm_plan(M, N, K)
    if not swap and planned <= 1:
        return None
    ws = _workspace(x.device, need)
    splits = ctypes.c_int(0)
    code = _fn("gemm_tc", "tl_gemm_tc")(
        x.data_ptr(), w.data_ptr(), None, None, 0, EPI_STORE_F32, M, N, K, x.stride(0), w.stride(0), ws.data_ptr(),
        ws.numel() * 4, 1, ctypes.byref(splits), _stream())
    _check(code, "gemm_tc (deferred)")
    return ws, splits.value


def finish_qkv_rope(partials, splits, bias, qkv, positions, token_req, block_table, pages, inv_freq, nh, nkv, d,
                    page_size, write_kv=True) -> None:
    """Sum the qkv product's splits (+ bias), rotate q and k, store q to ``qkv`` and k, v to pages."""
    _need_cuda(partials, bias, qkv, positions, token_req, block_table, pages, inv_freq)
    assert qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d
    code = _fn("decode_fused", "tl_finish_qkv_rope")(
        partials.data_ptr(), splits, _ptr(bias), qkv.data_ptr(), positions.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], pages.data_ptr(), inv_freq.data_ptr(), qkv.shape[0], nh, nkv,
        d, page_size, 1 if write_kv else 0, pages.shape[0], _stream())
    _check(code, "finish_qkv_rope")


def finish_accum_norm(partials, splits, bias, acc, weight=None, eps=0.0, out=None) -> None:
    """acc += sum of the splits (+ bias); with ``out``: out = rmsnorm(acc) * weight (bfloat16)."""
    _need_cuda(partials, bias, acc, weight, out)
    tokens, hidden = acc.shape
    assert acc.dtype == torch.float32 and acc.is_contiguous()
    assert out is None or (out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == acc.shape)
    code = _fn("decode_fused", "tl_finish_accum_norm")(
        partials.data_ptr(), splits, _ptr(bias), acc.data_ptr(), _ptr(weight), _ptr(out), tokens, hidden,
        float(eps), _stream())
    _check(code, "finish_accum_norm")


def gemm_tc_error() -> int:
    """0, or the code a bounded wait in a tensor-core kernel left when it gave up
    (1 producer, 2 MMA issuer, 3 epilogue).  Reading clears it."""
    return _fn("gemm_tc", "tl_gemm_tc_error")()


def wait_selftest(code: int = 99) -> None:
    """Launches one block whose bounded wait runs out (nothing ever arrives at its barrier; the
    limit is 2^16 cycles) and that then returns normally: ``gemm_tc_error()`` afterwards gives
    ``code`` and ``raise_on_wait_errors()`` raises.  Nothing faults or hangs; for tests."""
    _check(_fn("gemm_tc", "tl_gemm_tc_wait_selftest")(code, _stream()), "wait_selftest")


_arrival_counters: dict = {}
_outgrown_counters: list = []  # kept alive: captured CUDA graphs may still hold their addresses


def _arrivals(device, count: int) -> torch.Tensor:
    """Per device, ints that are zero between launches: the decode attention counts the key
    splits of a (request, KV head) that have finished; the last one merges and zeroes its counter."""
    counters = _arrival_counters.get(device)
    if counters is None or counters.numel() < count:
        if counters is not None:
            _outgrown_counters.append(counters)
        counters = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
        _arrival_counters[device] = counters
    return counters


# TORCHLET_B200_DECODE_MERGE=kernel: a second kernel merges the key splits (for measurements)
_merge_in_kernel = os.environ.get("TORCHLET_B200_DECODE_MERGE", "") != "kernel"


def attention_mma(qkv, pages, block_table, req_indptr, kv_before, tile_req, tile_row, tiles, out, tokens, nh, nkv,
                  d, page_size, window, scale, rows16: bool, splits: int = 1, late_wait: bool = False,
                  softcap=None, sink: bool = False, gate=None, prior=None) -> None:
    """Tensor-core paged attention (csrc/attention_mma.cu).  ``tile_req``/``tile_row`` None:
    tile i is request i from its first packed row.  With ``splits`` > 1 every tile is a request
    that brings one token; only those tokens' rows of ``out`` are written.  ``splits`` is the
    number of CTAs the grid holds for a request's keys; the kernel uses as many as the request's
    own length warrants.  ``late_wait`` (16-row tiles): the launch just before this one on the
    stream was ``attention_tc`` for the other requests of the same step; this grid starts beside
    it and waits for it at its end instead of at its start.  ``softcap``: scores become
    softcap * tanh(score / softcap); ``sink``: one is added to the softmax's denominator; ``gate`` (float32
    rows [tokens, >= nh * d]): the output is multiplied by sigmoid(gate).  ``prior`` = (ml [tokens, nh, 2], acc
    [tokens, nh, d]), float32: a softmax state over keys the kernel does not walk (``pooled_prior``), joined with every
    row's own where the row is normalized."""
    _need_cuda(qkv, pages, block_table, req_indptr, kv_before, tile_req, tile_row, out, gate)
    prior_ml, prior_acc = _prior(prior, qkv.shape[0], nh, d)
    assert qkv.dtype == pages.dtype == out.dtype == torch.bfloat16
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    # key splits: float32 partial results of every (decode tile, head, split); the split that finishes last merges
    need = tiles * nh * splits * (d + 2) * 4 if splits > 1 else 0
    ws = _workspace(("attention", qkv.device), need) if need else None
    # up to 16 splits the last split to finish merges them inside the kernel (one round of loads;
    # measured -1 % of a decode step at batch 8 to 32); more are merged by a second kernel, whose
    # many small CTAs do better than one CTA's two rounds (batch 1 at 4,096 tokens: 32 splits)
    arrivals = _arrivals(qkv.device, tiles * nkv) if need and _merge_in_kernel and splits <= 16 else None
    code = _fn("attention_mma", "tl_attention_mma_ex")(
        qkv.data_ptr(), qkv.stride(0), pages.data_ptr(), pages.shape[0], block_table.data_ptr(),
        block_table.shape[1], req_indptr.data_ptr(), kv_before.data_ptr(), _ptr(tile_req), _ptr(tile_row), tiles,
        out.data_ptr(), out.stride(0), tokens, nh, nkv, d, page_size, int(window or 0), float(scale),
        1 if rows16 else 0, splits,
        _ptr(ws), ws.numel() * 4 if ws is not None else 0, _ptr(arrivals), 1 if late_wait else 0,
        float(softcap or 0.0), 1 if sink else 0, _ptr(gate), gate.stride(0) if gate is not None else 0,
        _ptr(prior_ml), _ptr(prior_acc), _stream())
    _check(code, "attention_mma", 2 if splits > 1 and arrivals is None else 1)


def _prior(prior, tokens: int, nh: int, d: int):
    if prior is None:
        return None, None
    ml, acc = prior
    _need_cuda(ml, acc)
    assert ml.dtype == acc.dtype == torch.float32 and ml.is_contiguous() and acc.is_contiguous()
    assert ml.shape == (tokens, nh, 2) and acc.shape == (tokens, nh, d)
    return ml, acc


def attention_tc_rows(group: int) -> int:
    """Packed rows a tile of the tcgen05 attention kernel holds for ``group`` heads a KV head."""
    return _fn("attention_tc", "tl_attention_tc_rows")(group)


def attention_tc_supported(d: int, group: int, page_size: int) -> bool:
    return d in (64, 128) and 1 <= group <= 128 and 8 <= page_size <= 128 and 128 % page_size == 0


def attention_tc(qkv, pages, block_table, req_indptr, kv_before, tile_req, tile_row, tiles, out, nh, nkv, d,
                 page_size, window, scale, splits: int = 1, token_req=None, defer_merge: bool = False,
                 softcap=None, sink: bool = False, gate=None, prior=None):
    """Prompt-portion attention on tcgen05 (csrc/attention_tc.cu): tiles of packed rows
    (``tile_row`` multiples of ``attention_tc_rows(nh // nkv)``) that cover every request of the
    step with more than one token.  ``splits`` > 1: that many CTAs share the key tiles of each
    (row tiles, KV head) and a second kernel merges them (``token_req``: each token's request).
    ``defer_merge``: that second kernel is not launched; the call returns a function that launches
    it (None when there is nothing to merge), so that the decode attention may run between the two.
    The partial results have a workspace of their own.  ``softcap``, ``sink``, ``gate``, ``prior``: as in
    ``attention_mma``."""
    _need_cuda(qkv, pages, block_table, req_indptr, kv_before, tile_req, tile_row, out, token_req, gate)
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    gate_stride = gate.stride(0) if gate is not None else 0
    assert qkv.dtype == pages.dtype == out.dtype == torch.bfloat16 and pages.is_contiguous()
    tokens = qkv.shape[0]
    prior_ml, prior_acc = _prior(prior, tokens, nh, d)
    need = tokens * nh * splits * (d + 2) * 4 if splits > 1 else 0
    ws = _workspace(("attention_tc", qkv.device), need) if need else None
    ws_bytes = ws.numel() * 4 if ws is not None else 0
    defer = defer_merge and splits > 1
    code = _fn("attention_tc", "tl_attention_tc")(
        qkv.data_ptr(), qkv.stride(0), pages.data_ptr(), pages.shape[0], block_table.data_ptr(),
        block_table.shape[1], req_indptr.data_ptr(), kv_before.data_ptr(), tile_req.data_ptr(), tile_row.data_ptr(),
        tiles, out.data_ptr(), out.stride(0), nh, nkv, d, page_size, int(window or 0), float(scale), splits,
        _ptr(token_req), tokens, _ptr(ws), ws_bytes, 1 if defer else 0, float(softcap or 0.0), 1 if sink else 0,
        _ptr(gate), gate_stride, _ptr(prior_ml), _ptr(prior_acc), _stream())
    _check(code, "attention_tc", 2 if splits > 1 and not defer else 1)
    if not defer:
        return None

    def merge() -> None:
        code = _fn("attention_tc", "tl_attention_tc_merge")(
            req_indptr.data_ptr(), out.data_ptr(), out.stride(0), nh, d, splits, token_req.data_ptr(), tokens,
            ws.data_ptr(), ws_bytes, 1 if sink else 0, _ptr(gate), gate_stride, _ptr(prior_ml), _ptr(prior_acc),
            _stream())
        _check(code, "attention_tc_merge", 1)

    return merge


def attention_mma_error() -> int:
    """0, or the code a bounded wait of the decode attention's TMA loader left.  Reading clears it
    (and the arrival counters, which a kernel that gave up may have left half counted)."""
    code = _fn("attention_mma", "tl_attention_mma_error")()
    if code:
        for counters in _arrival_counters.values():
            counters.zero_()
    return code


def attention_tc_error() -> int:
    """0, or the code a bounded wait in the tcgen05 attention kernel left when it gave up."""
    return _fn("attention_tc", "tl_attention_tc_error")()


_DEBUG_CODES = {1: "a token id outside the vocabulary", 2: "a position beyond its request's block table",
                3: "a page id outside the pool", 4: "a slot outside the slot range"}


def debug_errors() -> list:
    """What the debug build's index checks have caught since the last call: (library, meaning,
    offending value) for every loaded library whose check failed; reading clears.  Always empty
    in the ordinary build (``TORCHLET_B200_DEBUG`` unset), whose kernels carry no checks."""
    found = []
    for library in ("elementwise", "attention_generic", "attention_mma", "decode_fused", "slots", "stream_ops",
                    "delta_rule", "latent_attention", "latent_attention_mma", "gla", "gated_attention", "hyper",
                    "pooled_attention", "ssm"):
        if any(name in _functions for name in _SIGNATURES[library]):
            value = ctypes.c_int(0)
            code = _fn(library, f"tl_{library}_debug_error")(ctypes.byref(value))
            if code:
                found.append((library, _DEBUG_CODES.get(code, f"code {code}"), value.value))
    return found


def raise_on_wait_errors() -> None:
    """Raises if a bounded wait inside a tensor-core kernel has given up since the last call
    (the kernel then ran to its end with whatever it had, so its output is not to be used), or,
    in the debug build, if an index check inside a kernel has failed.
    Only libraries that are loaded are asked.  The read is a blocking copy on the default
    stream, so it sees every kernel launched before it."""
    for library, read in (("gemm_tc", gemm_tc_error), ("attention_tc", attention_tc_error),
                          ("attention_mma", attention_mma_error)):
        if any(name in _functions for name in _SIGNATURES[library]):
            code = read()
            if code:
                raise KernelError(f"{library}: a bounded wait gave up inside a kernel (code {code}); "
                                  "the results of this step are invalid")
    if DEBUG_BUILD:
        for library, meaning, value in debug_errors():
            raise KernelError(f"{library} (debug build): {meaning}: {value}; the access was skipped, "
                              "the results of this step are invalid")