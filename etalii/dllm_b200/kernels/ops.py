"""Python entry points of the hand-written kernels. Each takes torch CUDA tensors, checks what the kernel assumes
(device, dtype, contiguity, sizes), launches on torch's current stream and raises on a refused argument. There is
no CPU path and no library fallback: a tensor that is not on a CUDA device is an error."""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_void_p

import torch

from .build import library

EPI_STORE_F32, EPI_STORE_T, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
EPI_GLU_CLAMPED = 10
"""W interleaves gate and up rows; c[M,N/2] = g sigmoid(1.702 g) (u + 1) with g = min(gate, limit), u = clamp(up,
-limit, limit). Only the weight-streaming kernels have it (`glu_clamped_fuses`); `eps` carries the limit."""
_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_STATUS = {-1: "bad argument", -2: "unsupported size", -3: "kernel launch failed"}
EPI_GLU_GELU_TANH = 11
"""Gate and up rows interleaved as for SwiGLU: c[M, N/2] = gelu(gate) * up with the tanh form of gelu. Where
EPI_GLU_CLAMPED is: the weight-streaming kernels (`glu_clamped_fuses`)."""
_EPILOGUE_NAMES = {0: "store_f32", 1: "store", 2: "residual", 3: "swiglu", 10: "glu_clamped", 11: "glu_gelu_tanh"}


class KernelError(RuntimeError):
    pass


_prototypes = {
    ("elementwise", "dllm_embed"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ("elementwise", "dllm_embed_scaled"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                           c_void_p],
    ("elementwise", "dllm_rmsnorm"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    ("elementwise", "dllm_layernorm"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    ("elementwise", "dllm_glu_clamped"): [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float, c_int, c_void_p],
    ("elementwise", "dllm_dynamic_tanh"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                           c_int, c_void_p],
    ("elementwise", "dllm_glu_act"): [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("sigmoid_attention", "dllm_sigmoid_prepare"): [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                                    c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                    c_void_p, c_int, c_int, c_int, c_void_p],
    ("sigmoid_attention", "dllm_sigmoid_attention"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                      c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                      c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                      c_int, c_int, c_void_p, c_int, c_void_p],
    ("sigmoid_attention_tiled", "dllm_sigmoid_attention_tiled_fits"): [c_int, c_int, c_int, c_int, c_int],
    ("sigmoid_attention_tiled", "dllm_sigmoid_attention_tiled"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                                  c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                                                  c_void_p, c_void_p, c_int, c_float, c_int, c_int,
                                                                  c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                                  c_int, c_void_p, c_int, c_void_p],
    ("sigmoid_attention", "dllm_sigmoid_combine"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                    c_void_p],
    ("elementwise", "dllm_norm_sum_residual"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                                c_float, c_void_p],
    ("elementwise", "dllm_norm_add_residual"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    ("elementwise", "dllm_cast_rows"): [c_void_p, c_void_p, c_longlong, c_void_p],
    ("diff_attention", "dllm_map_prepare"): [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                             c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
                                             c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    ("diff_attention", "dllm_diff_attention"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                c_float, c_float, c_float, c_float, c_float, c_int, c_int, c_int, c_int,
                                                c_void_p],
    ("diff_attention_prefill", "dllm_diff_attention_prefill"): [
        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_float, c_float, c_float, c_int, c_int,
        c_void_p],
    ("diff_attention_decode", "dllm_diff_attention_decode_fits"): [c_int, c_int, c_int, c_int, c_int],
    ("diff_attention_decode", "dllm_diff_attention_decode"): [
        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
        c_void_p, c_void_p, c_int, c_float, c_float, c_float, c_float, c_float, c_int, c_int, c_int, c_void_p, c_void_p,
        c_void_p],
    ("moe", "dllm_moe_route"): [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                c_int, c_void_p],
    ("moe", "dllm_moe_up_plain"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                   c_void_p],
    ("elementwise", "dllm_norm_conv"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
    ("elementwise", "dllm_bias_act"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p],
    ("elementwise", "dllm_add_row"): [c_void_p, c_void_p, c_int, c_int, c_void_p],
    ("elementwise", "dllm_gate_embed"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                         c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ("latent_attention", "dllm_latent_prepare"): [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                  c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                  c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    ("latent_attention", "dllm_latent_queries"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                  c_int, c_float, c_void_p, c_int, c_void_p],
    ("latent_attention", "dllm_latent_attention"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                    c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                                    c_void_p],
    ("latent_attention_tiled", "dllm_latent_attention_tiled"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                                c_void_p, c_int,
                                                                c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                                c_void_p, c_void_p, ctypes.c_longlong, c_void_p],
    ("latent_attention", "dllm_latent_values"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                                 c_int, c_int, c_void_p],
    ("recurrent", "dllm_gated_scan"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                       c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                       c_void_p],
    ("recurrent", "dllm_running_max_gates"): [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p,
                                              c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
    ("recurrent", "dllm_normalised_readout"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                               c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    ("moe", "dllm_moe_up"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_float, c_float,
                             c_float, c_int, c_void_p],
    ("moe", "dllm_moe_down"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                               c_int, c_void_p],
    ("moe_grouped", "dllm_moe_sort"): [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
    ("moe_grouped", "dllm_moe_grouped_up"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                             c_void_p, c_float, c_float, c_float, c_void_p],
    ("moe_grouped", "dllm_moe_grouped_up_plain"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                   c_void_p, c_void_p, c_int, c_void_p],
    ("moe_grouped", "dllm_moe_grouped_down"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                               c_void_p, c_void_p, c_void_p],
    ("moe_grouped", "dllm_moe_combine"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("elementwise", "dllm_concat_restart"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    ("recurrent", "dllm_decay_scan"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                       c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    ("recurrent", "dllm_silu_columns"): [c_void_p, c_int, c_int, c_int, c_void_p],
    ("recurrent", "dllm_delta_scan"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                       c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    ("recurrent", "dllm_delta_prepare"): [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_int, c_void_p],
    ("recurrent", "dllm_gated_norm"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                       c_int, c_int, c_void_p],
    ("elementwise", "dllm_rope_cache_write"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                               c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                               c_int, c_int, c_longlong, c_void_p],
    ("elementwise", "dllm_copy_to_device"): [c_void_p, c_void_p, c_longlong, c_void_p],
    ("elementwise", "dllm_add_residual"): [c_void_p, c_void_p, c_longlong, c_int, c_void_p],
    ("elementwise", "dllm_sum_parts_residual"): [c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_split"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                  c_void_p, c_void_p],
    ("elementwise", "dllm_decode_advance"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_void_p],
    ("elementwise", "dllm_mask_tokens"): [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p],
    ("gemm_simt", "dllm_gemm_f32"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("gemm_bf16", "dllm_gemm_bf16"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                            c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_qkv_rope"): [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                     c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                                     c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_normed"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                                   c_int, c_float, c_void_p, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_residual_norm"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                          c_int, c_int, c_int, c_void_p, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_qkv_rope_normed"): [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                            c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                            c_void_p, c_int, c_float, c_void_p, c_void_p],
    ("elementwise", "dllm_cast_ssq"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    ("gemv", "dllm_gemv_bf16"): [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int,
                                 c_void_p, c_longlong, c_void_p],
    ("gemv_cluster", "dllm_gemv_cluster"): [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int,
                                            c_int, c_void_p, c_longlong, c_void_p],
    ("gemv_cluster", "dllm_gemv_cluster_qkv_rope"): [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p,
                                                     c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                     c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                     c_void_p, c_longlong, c_void_p],
    ("mlp_decode", "dllm_mlp_decode"): [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                        c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p],
    ("gemv", "dllm_argmax_candidates"): [c_void_p, c_void_p, c_int, c_int, c_void_p],
    ("gemv_tma", "dllm_gemv_tma"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ("gemv", "dllm_gemv_qkv_rope"): [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                     c_void_p, c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p],
    ("attention", "dllm_attention_general"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                              c_int, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int,
                                              c_void_p],
    ("attention", "dllm_attention_blocks"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int,
                                             c_void_p],
    ("attention_decode", "dllm_attention_decode"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                    c_int, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int,
                                                    c_void_p, c_void_p, c_void_p],
    ("attention_decode_cluster", "dllm_attention_decode_cluster"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                                    c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                                                    c_int, c_float, c_int, c_int, c_void_p],
    ("attention_prefill", "dllm_attention_prefill"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                      c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                      c_int, c_float, c_int, c_void_p],
    ("attention_prefill_tcgen05", "dllm_attention_prefill_tcgen05"): [
        c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p],
    ("sampling", "dllm_sample"): [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                  c_float, c_int, c_double, c_double, c_void_p],
    ("sampling", "dllm_seed_rng"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
}
_functions: dict[tuple[str, str], ctypes._CFuncPtr] = {}


launches = 0
"""How many kernels this module has launched (every call below launches exactly one)."""

trace: list | None = None
"""A list while a measurement wants every launch timed: each launch appends (name, CUDA event recorded behind it).
On one stream the time between consecutive events is the kernel's (plus the gap before it)."""


def _fn(lib: str, name: str):
    key = (lib, name)
    found = _functions.get(key)
    if found is None:
        found = getattr(library(lib), name)
        found.argtypes = _prototypes[key]
        found.restype = c_int
        _functions[key] = found
    return found


def _check(status: int, what: str, detail="") -> None:
    """Counts the launch; a refusal raises. `detail` may be a callable that makes the text (only then is it made:
    formatting a message costs a launch's worth of host time)."""
    global launches
    launches += 1
    if callable(what):
        what = what()
    if trace is not None and status == 0:
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        trace.append((what, event))
    if status != 0:
        if callable(detail):
            detail = detail()
        raise KernelError(f"{what}: {_STATUS.get(status, status)}{(' (' + detail + ')') if detail else ''}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (the raw getter costs a fraction of a microsecond; the Stream object ten times
    that, once per launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernels take contiguous CUDA tensors only (there is no CPU path)")


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported (float32 and bfloat16 are)") from None


def embed(out: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, status: torch.Tensor | None = None,
          scale: float = 1.0) -> None:
    """out[r] = float32(table[tokens[r]]) * scale; a token outside the table gives a zero row and sets the status word
    (`status`: an int32 word the device can write; default: the pinned word that `raise_if_failed` reads)."""
    _cuda(out, table, tokens)
    if status is None:
        status = _status_word()
    assert out.dtype == torch.float32 and tokens.dtype == torch.int32 and status.dtype == torch.int32
    rows, hidden = out.shape
    assert tokens.numel() >= rows and table.shape[1] == hidden
    _check(_fn("elementwise", "dllm_embed_scaled")(out.data_ptr(), table.data_ptr(), tokens.data_ptr(), rows, hidden,
                                                   table.shape[0], _code(table.dtype), float(scale),
                                                   status.data_ptr(), _stream()), "embed")


def copy_to_device(dst_ptr: int, src_ptr: int, nbytes: int) -> None:
    """Copies `nbytes` from pinned host memory to device memory on the current stream, without a host wait (the
    caller keeps the source alive and unchanged until the copy has run: an event behind it tells)."""
    status = _fn("elementwise", "dllm_copy_to_device")(dst_ptr, src_ptr, int(nbytes), _stream())
    if status != 0:
        raise KernelError(f"copy to the device: {_STATUS.get(status, status)}")


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float,
            rows: torch.Tensor | None = None) -> None:
    """out[r] = norm(x[rows[r]] if rows is given else x[r]) * weight; x and weight float32."""
    _cuda(out, x, weight, rows)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == x.shape[-1]
    n = out.shape[0]
    assert out.shape[-1] == x.shape[-1] and (rows is not None or x.shape[0] >= n)
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= n)
    _check(_fn("elementwise", "dllm_rmsnorm")(out.data_ptr(), x.data_ptr(), weight.data_ptr(),
                                              rows.data_ptr() if rows is not None else None, n, x.shape[-1],
                                              float(eps), _code(out.dtype), _stream()), "rmsnorm")


def layernorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float,
              rows: torch.Tensor | None = None) -> None:
    """out[r] = (x - mean) / sqrt(variance + eps) * weight of row r (or of row rows[r]); x and weight float32, the
    variance the mean of the squared deviations."""
    _cuda(out, x, weight, rows)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == x.shape[-1]
    n = out.shape[0]
    assert out.shape[-1] == x.shape[-1] and (rows is not None or x.shape[0] >= n)
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= n)
    _check(_fn("elementwise", "dllm_layernorm")(out.data_ptr(), x.data_ptr(), weight.data_ptr(),
                                                rows.data_ptr() if rows is not None else None, n, x.shape[-1],
                                                float(eps), _code(out.dtype), _stream()), "layernorm")


def dynamic_tanh(out: torch.Tensor, x: torch.Tensor, alpha: float, weight: torch.Tensor, bias: torch.Tensor,
                 rows: torch.Tensor | None = None) -> None:
    """out[r] = tanh(alpha * x[rows[r]] if rows is given else x[r]) * weight + bias; x, weight and bias float32."""
    _cuda(out, x, weight, bias, rows)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and bias.dtype == torch.float32
    assert weight.numel() == x.shape[-1] and bias.numel() == x.shape[-1]
    n = out.shape[0]
    assert out.shape[-1] == x.shape[-1] and (rows is not None or x.shape[0] >= n)
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= n)
    _check(_fn("elementwise", "dllm_dynamic_tanh")(out.data_ptr(), x.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                                   rows.data_ptr() if rows is not None else None, n, x.shape[-1],
                                                   float(alpha), _code(out.dtype), _stream()), "dynamic_tanh")


def glu_act(out: torch.Tensor, gate_up: torch.Tensor, activation: int) -> None:
    """gate_up float32 [rows, 2 width] = gate_0, up_0, gate_1, up_1, ...; out[rows, width] = act(gate) * up in float32
    (`activation`: a value of `ACTIVATIONS`), rounded once to out's type."""
    _cuda(out, gate_up)
    rows, width = out.shape
    assert gate_up.shape == (rows, 2 * width) and gate_up.dtype == torch.float32
    _check(_fn("elementwise", "dllm_glu_act")(out.data_ptr(), gate_up.data_ptr(), rows, width, int(activation),
                                              _code(out.dtype), _stream()), "glu_act")


def sigmoid_prepare(rows: torch.Tensor, q_at: int, k_at: int, v_at: int, q_out: torch.Tensor, cache, heads: int,
                    biases, norm_weights, eps: float, batch, write_cache: bool = True) -> None:
    """From a token's projected float32 row (q at q_at: heads x dim; k at k_at: kv_heads x dim; v at v_at: kv_heads x
    value_dim): `biases` = (q, k, v) float32 vectors added first (None: no biases); `norm_weights` = (q, k) float32
    weights of an RMS norm over the WHOLE q and the whole k, all heads at once (None: no norm). Queries go to q_out
    (the cache's type), keys and values into the token's place in the cache."""
    qb, kb, vb = biases if biases is not None else (None, None, None)
    qw, kw = norm_weights if norm_weights is not None else (None, None)
    _cuda(rows, q_out, qb, kb, vb, qw, kw)
    dim, vdim, kv_heads = cache.head_dim, cache.value_dim, cache.kv_heads
    assert rows.dtype == torch.float32 and q_out.dtype == cache.dtype and not cache.keys_only
    assert q_out.shape[1] == heads * dim
    for tensor, size in ((qb, heads * dim), (kb, kv_heads * dim), (vb, kv_heads * vdim), (qw, heads * dim),
                         (kw, kv_heads * dim)):
        assert tensor is None or (tensor.dtype == torch.float32 and tensor.numel() == size)
    ptr = lambda tensor: tensor.data_ptr() if tensor is not None else None  # noqa: E731
    _check(_fn("sigmoid_attention", "dllm_sigmoid_prepare")(
        rows.data_ptr(), rows.shape[1], int(q_at), int(k_at), int(v_at), heads, kv_heads, dim, vdim, ptr(qb), ptr(kb),
        ptr(vb), ptr(qw), ptr(kw), float(eps), q_out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(),
        cache.max_pages, cache.page_size, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(),
        batch.n_tokens, 1 if write_cache else 0, _code(cache.dtype), _stream()), "sigmoid_prepare")


def sigmoid_attention_splits(batch, window: int, keep: int) -> int:
    """Over how many blocks the general kernel deals a token's keys: one where the step's tokens fill the device by
    themselves, else enough for about two blocks a multiprocessor, every block with two tiles of keys or more."""
    reach = batch.max_context if window <= 0 else min(batch.max_context, window + keep + 32)
    return max(1, min(296 // max(1, batch.n_tokens), reach // 64))


def sigmoid_attention(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int, keep: int,
                      mix: torch.Tensor | None, slopes: torch.Tensor | None, head_bias: torch.Tensor | None,
                      gates: torch.Tensor | None, gate_at: int, batch, ws=None) -> None:
    """Attention without a softmax over a cache of keys [dim] and values [value_dim]: token i weighs a visible key j
    (j <= i and i - j < window, or j < keep; window 0: all) with sigmoid(q . k * scale - slopes[h] (i - j) +
    head_bias[h]); `mix` float32 [heads, heads] then mixes the heads' weights, weight_h <- sum_g mix[h, g] weight_g;
    head h applies its weights to the values of its kv head. out [tokens, heads x value_dim] in the cache's type, times
    sigmoid(gates[t, gate_at + o]) where `gates` (float32 rows) is given. The general kernel: float32 arithmetic, either
    cache type, every size up to heads x value_dim = 8192; with `ws` a step of few tokens deals each token's keys to
    several blocks."""
    _cuda(out, q, mix, slopes, head_bias, gates)
    dim, vdim = cache.head_dim, cache.value_dim
    assert q.dtype == cache.dtype and out.dtype == cache.dtype and not cache.keys_only
    assert q.shape[1] == heads * dim and out.shape[1] == heads * vdim
    assert mix is None or (mix.dtype == torch.float32 and tuple(mix.shape) == (heads, heads))
    for tensor in (slopes, head_bias):
        assert tensor is None or (tensor.dtype == torch.float32 and tensor.numel() == heads)
    tokens = batch.n_tokens
    splits = sigmoid_attention_splits(batch, window, keep) if ws is not None else 1
    part = ws.buffer("sigmoid_part", (splits * tokens * heads * vdim,), torch.float32) if splits > 1 else None
    gate_ptr = (gates.data_ptr() + 4 * int(gate_at)) if gates is not None else None
    ptr = lambda tensor: tensor.data_ptr() if tensor is not None else None  # noqa: E731
    _check(_fn("sigmoid_attention", "dllm_sigmoid_attention")(
        q.data_ptr(), out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, dim, vdim, ptr(mix), ptr(slopes), ptr(head_bias), gate_ptr,
        gates.shape[1] if gates is not None else 0, float(scale), int(window), int(keep), batch.tok_seq.data_ptr(),
        batch.tok_pos.data_ptr(), batch.slots.data_ptr(), tokens, splits, ptr(part), _code(cache.dtype), _stream()),
        "sigmoid_attention", lambda: f"heads={heads} dim={dim} value_dim={vdim} page={cache.page_size}")


_sigmoid_tiles: dict[tuple, bool] = {}


def sigmoid_attention_tiles(dtype, heads: int, kv_heads: int, dim: int, vdim: int, page_size: int = 64) -> bool:
    """Whether the tensor-core kernel runs these sizes: bfloat16, dim and vdim multiples of 16 (vdim at most 128, dim
    at most 256), pages of a multiple of 32 positions, a block's queries, one tile of every kv head's keys and values
    and all heads' weights within its shared memory (the library answers, once per combination of sizes)."""
    if dtype != torch.bfloat16 or dim % 16 or vdim % 16 or (heads * vdim) % 2:
        return False
    key = (heads, kv_heads, dim, vdim, page_size)
    if key not in _sigmoid_tiles:
        _sigmoid_tiles[key] = bool(_fn("sigmoid_attention_tiled", "dllm_sigmoid_attention_tiled_fits")(*key))
    return _sigmoid_tiles[key]


def sigmoid_tiled_splits(batch, window: int, keep: int) -> int:
    """Over how many blocks the tile kernel deals the keys of a block of sixteen tokens: one where the step's blocks
    cover half the multiprocessors by themselves, else enough for about two blocks each, every block with two tiles
    of 32 keys or more."""
    blocks = batch.n_seqs * (-(-batch.max_new // 16))
    if blocks >= 74:
        return 1
    reach = batch.max_context if window <= 0 else min(batch.max_context, window + keep + 32)
    return max(1, min(296 // blocks, reach // 64))


def sigmoid_attention_tiled(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int,
                            keep: int, mix: torch.Tensor | None, slopes: torch.Tensor | None,
                            head_bias: torch.Tensor | None, gates: torch.Tensor | None, gate_at: int, batch,
                            ws=None) -> None:
    """`sigmoid_attention` on the tensor cores: a block takes sixteen consecutive new tokens of a sequence and all
    heads; the weights are rounded to bfloat16 before the mixing (itself a tensor-core product) and after it, as the
    operand of the product with the values (accumulation float32). With `ws`, a step of few blocks (single tokens)
    deals each block's keys to several blocks and a second kernel adds their float32 sums. Sizes:
    `sigmoid_attention_tiles`."""
    _cuda(out, q, mix, slopes, head_bias, gates)
    dim, vdim = cache.head_dim, cache.value_dim
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
    assert q.shape[1] == heads * dim and out.shape[1] == heads * vdim and not cache.keys_only
    assert mix is None or (mix.dtype == torch.float32 and tuple(mix.shape) == (heads, heads))
    for tensor in (slopes, head_bias):
        assert tensor is None or (tensor.dtype == torch.float32 and tensor.numel() == heads)
    gate_ptr = (gates.data_ptr() + 4 * int(gate_at)) if gates is not None else None
    gate_ld = gates.shape[1] if gates is not None else 0
    ptr = lambda tensor: tensor.data_ptr() if tensor is not None else None  # noqa: E731
    tokens = batch.n_tokens
    splits = sigmoid_tiled_splits(batch, window, keep) if ws is not None else 1
    part = ws.buffer("sigmoid_part", (splits * tokens * heads * vdim,), torch.float32) if splits > 1 else None
    _check(_fn("sigmoid_attention_tiled", "dllm_sigmoid_attention_tiled")(
        q.data_ptr(), out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, dim, vdim, ptr(mix), ptr(slopes), ptr(head_bias), gate_ptr, gate_ld, float(scale),
        int(window), int(keep), batch.cu_seqlens.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(),
        batch.n_seqs, int(batch.max_new), splits, ptr(part), tokens, _stream()),
        "sigmoid_attention_tiled",
        lambda: f"heads={heads} dim={dim} value_dim={vdim} page={cache.page_size} gate_at={gate_at}")
    if splits > 1:
        _check(_fn("sigmoid_attention", "dllm_sigmoid_combine")(
            part.data_ptr(), gate_ptr, gate_ld, out.data_ptr(), tokens, heads * vdim, splits, _code(out.dtype),
            _stream()), "sigmoid_combine")


def glu_clamped_fuses(rows: int, outputs: int, inner: int) -> bool:
    """Whether a bfloat16 product of these sizes runs in one of the two weight-streaming kernels that can end in the
    clamped GLU (a block per 16 rows of W, or the reduction split over a cluster)."""
    return streams(rows, outputs, inner) and not takes_weights_as_rows(rows, outputs, inner) and \
        not streams_through_shared_memory(rows, outputs, inner)


def glu_clamped(out: torch.Tensor, gate_up: torch.Tensor, limit: float, alpha: float, shift: float) -> None:
    """gate_up [rows, 2 width] = gate_0, up_0, gate_1, up_1, ...; out[rows, width] = g sigmoid(alpha g) (u + shift)
    with g = min(gate, limit), u = clamp(up, -limit, limit), in float32, rounded once."""
    _cuda(out, gate_up)
    rows, width = out.shape
    assert gate_up.shape == (rows, 2 * width) and gate_up.dtype == out.dtype
    _check(_fn("elementwise", "dllm_glu_clamped")(out.data_ptr(), gate_up.data_ptr(), rows, width, float(limit),
                                                  float(alpha), float(shift), _code(out.dtype), _stream()),
           "glu_clamped")


def norm_sum_residual(residual: torch.Tensor, a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor,
                      eps: float, factor: float) -> None:
    """residual += factor * (a / rms(a) * wa + b / rms(b) * wb), row by row, all float32."""
    _cuda(residual, a, wa, b, wb)
    rows, hidden = a.shape
    assert all(t.dtype == torch.float32 for t in (residual, a, wa, b, wb))
    assert b.shape == a.shape and residual.shape[0] >= rows and residual.shape[1] == hidden
    assert wa.numel() == hidden and wb.numel() == hidden
    _check(_fn("elementwise", "dllm_norm_sum_residual")(residual.data_ptr(), a.data_ptr(), wa.data_ptr(), b.data_ptr(),
                                                        wb.data_ptr(), rows, hidden, float(eps), float(factor),
                                                        _stream()), "norm_sum_residual")


def norm_add_residual(residual: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                      copy: torch.Tensor | None = None) -> None:
    """residual += y / sqrt(mean(y^2) + eps) * weight, row by row, all float32 (a sublayer whose OUTPUT is normed).
    With `copy` (bfloat16, the rows' shape) the new rows are also left there rounded: the next product's operand."""
    _cuda(residual, y, weight, copy)
    assert copy is None or (copy.dtype == torch.bfloat16 and copy.numel() >= y.numel())
    rows, hidden = y.shape
    assert all(t.dtype == torch.float32 for t in (residual, y, weight))
    assert residual.shape[0] >= rows and residual.shape[1] == hidden and weight.numel() == hidden
    _check(_fn("elementwise", "dllm_norm_add_residual")(residual.data_ptr(), y.data_ptr(), weight.data_ptr(),
                                                        copy.data_ptr() if copy is not None else None, rows,
                                                        hidden, float(eps), _stream()), "norm_add_residual")


def cast_rows(out: torch.Tensor, x: torch.Tensor) -> None:
    """out = bfloat16(x), x float32 of the same shape: the stream as the operand of a product that has no norm in
    front."""
    _cuda(out, x)
    assert x.dtype == torch.float32 and out.dtype == torch.bfloat16 and out.numel() == x.numel()
    _check(_fn("elementwise", "dllm_cast_rows")(out.data_ptr(), x.data_ptr(), x.numel(), _stream()), "cast_rows")


def map_prepare(rows: torch.Tensor, q_at: int, k_at: int, v_at: int, q_out: torch.Tensor, cache, heads: int, dim: int,
                q_weight: torch.Tensor, k_weight: torch.Tensor | None, eps: float, table: torch.Tensor | None,
                rotary_dim: int, batch, write_cache: bool = True) -> None:
    """Queries and keys of two score maps per head, from the projected rows [tokens, n] float32 (q at column q_at:
    heads x 2 x dim; k at k_at: kv_heads x 2 x dim; v at v_at: kv_heads x value_dim): every (head, map) vector is
    divided by its root mean square and multiplied by the weight [dim] (one for q, one for k), its first
    `rotary_dim` places are rotated in halves by the token's position; q goes to q_out [tokens, heads x 2 x dim]
    float32, k and v into the token's place in the cache (keys of 2 dim, values of `cache.value_dim`). With
    `write_cache` False only the queries are made."""
    _cuda(rows, q_out, q_weight, k_weight, table)
    tokens = batch.n_tokens
    assert rows.dtype == torch.float32 and q_out.dtype == torch.float32 and q_weight.dtype == torch.float32
    assert cache.head_dim == 2 * dim and q_weight.numel() == dim and q_out.shape[1] == heads * 2 * dim
    assert rows.shape[0] >= tokens and q_out.shape[0] >= tokens
    assert not write_cache or (k_weight is not None and k_weight.dtype == torch.float32 and k_weight.numel() == dim)
    if table is not None and rotary_dim > 0:
        assert table.dtype == torch.float32 and table.shape[0] > batch.max_position, "position beyond the table"
        assert table.shape[1] == rotary_dim // 2 and table.shape[2] == 2
    _check(_fn("diff_attention", "dllm_map_prepare")(
        rows.data_ptr(), rows.shape[1], int(q_at), int(k_at), int(v_at), q_out.data_ptr(), cache.base_ptr,
        cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads, cache.kv_heads, dim, cache.value_dim,
        q_weight.data_ptr(), k_weight.data_ptr() if k_weight is not None else None, float(eps),
        table.data_ptr() if table is not None else None, int(rotary_dim) if table is not None else 0,
        batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(), tokens, 1 if write_cache else 0,
        _code(cache.dtype), _stream()), "map_prepare",
        lambda: f"dim={dim}, value_dim={cache.value_dim} (at most 256), rotary_dim={rotary_dim} (even, at most dim)")


def diff_attention(out: torch.Tensor, q: torch.Tensor, gates: torch.Tensor | None, gate_at: int, cache, heads: int,
                   dim: int, scale: float, softcap: float, weight: float, eps: float, out_scale: float, chunk: int,
                   window: int, batch, split: bool | None = None) -> None:
    """Differential attention of every token over its own sequence's cache: two softmax maps per head (scores
    q_m . k_m * scale, then softcap * tanh(score / softcap) if softcap > 0) over the keys of the token's chunk of
    `chunk` positions (0: none), of the last `window` positions (0: all), up to itself; out = (a1 - weight * a2) /
    sqrt(mean(.^2) + eps) * out_scale * sigmoid(gates[t, gate_at + head]). q float32 [tokens, heads x 2 x dim]; out
    [tokens, heads x value_dim] in the cache's dtype; `gates` float32 rows (None: no gate). `split`: a block of sixteen
    warps per (token, head) instead of a warp (default: for steps of few tokens)."""
    _cuda(out, q, gates)
    tokens = batch.n_tokens
    assert q.dtype == torch.float32 and out.dtype == cache.dtype and cache.head_dim == 2 * dim
    assert q.shape[1] == heads * 2 * dim and out.shape[1] == heads * cache.value_dim
    assert gates is None or (gates.dtype == torch.float32 and gates.shape[0] >= tokens)
    if split is None:
        split = tokens * heads <= 4 * _multiprocessors()
    gate_ptr = (gates.data_ptr() + 4 * int(gate_at)) if gates is not None else None
    _check(_fn("diff_attention", "dllm_diff_attention")(
        out.data_ptr(), q.data_ptr(), gate_ptr, gates.shape[1] if gates is not None else 0, cache.base_ptr,
        cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads, cache.kv_heads, dim, cache.value_dim,
        batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(), tokens, float(scale),
        float(softcap or 0.0), float(weight), float(eps), float(out_scale), int(chunk or 0), int(window or 0),
        1 if split else 0, _code(cache.dtype), _stream()), "diff_attention",
        lambda: f"dim={dim}, value_dim={cache.value_dim} (at most 256)")


_decode_fits: dict[tuple, bool] = {}


def diff_attention_decode_supported(cache, heads: int, dim: int) -> bool:
    """Whether the kernel that serves a token's whole group of query heads per block takes these sizes (bfloat16, at
    most 8 query heads per kv head, dim and value_dim multiples of 8, the stages of keys and values in shared memory:
    the library itself says)."""
    if cache.dtype != torch.bfloat16 or heads % cache.kv_heads:
        return False
    key = (heads, cache.kv_heads, dim, cache.value_dim, cache.page_size)
    if key not in _decode_fits:
        _decode_fits[key] = _fn("diff_attention_decode", "dllm_diff_attention_decode_fits")(*key) == 0
    return _decode_fits[key]


def diff_attention_decode_splits(tokens: int, kv_heads: int, longest: int) -> int:
    """Into how many stretches a token's keys are cut: enough blocks (tokens x kv heads x stretches) for two a
    multiprocessor, at most 16 and at most one per two pages of the longest context."""
    wanted = max(1, (2 * _multiprocessors()) // max(1, tokens * kv_heads))
    return max(1, min(16, wanted, -(-int(longest) // 128)))


def diff_attention_decode(out: torch.Tensor, q: torch.Tensor, gates: torch.Tensor | None, gate_at: int, cache,
                          heads: int, dim: int, scale: float, softcap: float, weight: float, eps: float,
                          out_scale: float, chunk: int, window: int, batch, splits: int, partial: torch.Tensor | None,
                          tickets: torch.Tensor | None) -> None:
    """`diff_attention` for a step of single tokens (bfloat16): a block per (token, kv head, stretch of keys) serves all
    query heads of the group from pages staged in shared memory; with `splits` > 1 the last block of a token combines
    the stretches through `partial` (tokens x kv_heads x splits x 2 group x (value_dim + 2) floats) and `tickets`
    (tokens x kv_heads int32 zeros, left zero)."""
    _cuda(out, q, gates, partial, tickets)
    tokens = batch.n_tokens
    assert diff_attention_decode_supported(cache, heads, dim) and batch.n_tokens == batch.n_seqs
    assert q.dtype == torch.float32 and out.dtype == torch.bfloat16 and cache.head_dim == 2 * dim
    assert q.shape[1] == heads * 2 * dim and out.shape[1] == heads * cache.value_dim
    group = heads // cache.kv_heads
    if splits > 1:
        assert partial.dtype == torch.float32 and tickets.dtype == torch.int32
        assert partial.numel() >= tokens * cache.kv_heads * splits * 2 * group * (cache.value_dim + 2)
        assert tickets.numel() >= tokens * cache.kv_heads
    gate_ptr = (gates.data_ptr() + 4 * int(gate_at)) if gates is not None else None
    _check(_fn("diff_attention_decode", "dllm_diff_attention_decode")(
        out.data_ptr(), q.data_ptr(), gate_ptr, gates.shape[1] if gates is not None else 0, cache.base_ptr,
        cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads, cache.kv_heads, dim, cache.value_dim,
        batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(), tokens, float(scale),
        float(softcap or 0.0), float(weight), float(eps), float(out_scale), int(chunk or 0), int(window or 0),
        int(splits), partial.data_ptr() if partial is not None else None,
        tickets.data_ptr() if tickets is not None else None, _stream()), "diff_attention_decode",
        lambda: f"dim={dim}, value_dim={cache.value_dim}, {group} query heads per kv head")


def diff_attention_prefill_supported(cache, dim: int) -> bool:
    return cache.dtype == torch.bfloat16 and cache.page_size == 64 and dim % 8 == 0 and dim <= 128 and \
        cache.value_dim % 8 == 0 and cache.value_dim <= 128


def diff_attention_prefill(out: torch.Tensor, q: torch.Tensor, gates: torch.Tensor | None, gate_at: int, cache,
                           heads: int, dim: int, scale: float, softcap: float, weight: float, eps: float,
                           out_scale: float, chunk: int, window: int, batch) -> None:
    """`diff_attention` for the new tokens of a prompt-sized step on the tensor cores (bfloat16; dim and value_dim
    multiples of 8 up to 128; pages of 64): tiles of 64 queries of one sequence and head, a group of warps per map."""
    _cuda(out, q, gates)
    assert diff_attention_prefill_supported(cache, dim) and q.dtype == torch.float32 and out.dtype == torch.bfloat16
    assert q.shape[1] == heads * 2 * dim and out.shape[1] == heads * cache.value_dim and cache.head_dim == 2 * dim
    assert gates is None or (gates.dtype == torch.float32 and gates.shape[0] >= batch.n_tokens)
    gate_ptr = (gates.data_ptr() + 4 * int(gate_at)) if gates is not None else None
    _check(_fn("diff_attention_prefill", "dllm_diff_attention_prefill")(
        out.data_ptr(), q.data_ptr(), gate_ptr, gates.shape[1] if gates is not None else 0, cache.base_ptr,
        cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads, cache.kv_heads, dim, cache.value_dim,
        batch.tile_seq.data_ptr(), batch.tile_first.data_ptr(), batch.cu_seqlens.data_ptr(), batch.start.data_ptr(),
        batch.slots.data_ptr(), batch.n_tiles, float(scale), float(softcap or 0.0), float(weight), float(eps),
        float(out_scale), int(chunk or 0), int(window or 0), _stream()), "diff_attention_prefill",
        lambda: f"dim={dim}, value_dim={cache.value_dim}: multiples of 8 up to 128; pages of 64")


def moe_route(chosen: torch.Tensor, weights: torch.Tensor, x: torch.Tensor, router: torch.Tensor,
              bias: torch.Tensor | None, top: int, all_experts: bool = False) -> None:
    """Per row of x (float32, or the activations in bfloat16): logits = router x + bias in float32; chosen[t] = the `top` experts with the largest
    logits, largest first (the lower expert on ties); weights[t] = the softmax over those logits only, or with
    `all_experts` the chosen experts' shares of the softmax over every expert's logit, as they are."""
    _cuda(chosen, weights, x, router, bias)
    tokens, width = x.shape
    experts = router.shape[0]
    assert router.dtype == torch.float32 and router.shape[1] == width
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == experts)
    assert chosen.dtype == torch.int32 and weights.dtype == torch.float32
    assert chosen.numel() >= tokens * top and weights.numel() >= tokens * top
    _check(_fn("moe", "dllm_moe_route")(x.data_ptr(), width, router.data_ptr(),
                                        bias.data_ptr() if bias is not None else None, experts, int(top), tokens,
                                        chosen.data_ptr(), weights.data_ptr(), 1 if all_experts else 0,
                                        _code(x.dtype), _stream()), "moe_route",
           lambda: f"experts={experts} (at most 256), top={top} (at most 16 and at most experts)")


def moe_up(act: torch.Tensor, h: torch.Tensor, w_gate_up: torch.Tensor, chosen: torch.Tensor, top: int, limit: float,
           alpha: float, shift: float) -> None:
    """act[t, k] = glu(W[chosen[t, k]] h[t]) for every token and choice: W [experts, 2 ff, width] interleaves gate and
    up rows; glu = g sigmoid(alpha g) (u + shift), g = min(gate, limit), u = clamp(up, -limit, limit), in float32."""
    _cuda(act, h, w_gate_up, chosen)
    tokens, width = h.shape
    ff = w_gate_up.shape[1] // 2
    assert h.dtype == w_gate_up.dtype == act.dtype and w_gate_up.shape[2] == width and chosen.dtype == torch.int32
    assert act.numel() >= tokens * top * ff and chosen.numel() >= tokens * top
    _check(_fn("moe", "dllm_moe_up")(act.data_ptr(), h.data_ptr(), width, w_gate_up.data_ptr(), ff, int(top), tokens,
                                     chosen.data_ptr(), float(limit), float(alpha), float(shift), _code(h.dtype),
                                     _stream()), "moe_up")


ACT_NONE, ACT_GELU, ACT_GELU_TANH, ACT_RELU_SQUARED = 0, 1, 2, 3
ACTIVATIONS = {None: ACT_NONE, "gelu": ACT_GELU, "gelu_tanh": ACT_GELU_TANH, "relu_squared": ACT_RELU_SQUARED}
"""The activations the pointwise kernels know, by name: the exact (erf) gelu, its tanh form 0.5 z (1 + tanh(sqrt(2/pi)
(z + 0.044715 z^3))), and the square of relu."""


def moe_up_plain(act: torch.Tensor, h: torch.Tensor, w_up: torch.Tensor, chosen: torch.Tensor, top: int,
                 activation: int) -> None:
    """act[t, k] = activation(W[chosen[t, k]] h[t]) for every token and choice: experts without a gate, W [experts,
    ff, width]; the activation (ACT_GELU, ACT_GELU_TANH or ACT_RELU_SQUARED) in float32."""
    _cuda(act, h, w_up, chosen)
    tokens, width = h.shape
    ff = w_up.shape[1]
    assert h.dtype == w_up.dtype == act.dtype and w_up.shape[2] == width and chosen.dtype == torch.int32
    assert act.numel() >= tokens * top * ff and chosen.numel() >= tokens * top
    _check(_fn("moe", "dllm_moe_up_plain")(act.data_ptr(), h.data_ptr(), width, w_up.data_ptr(), ff, int(top), tokens,
                                           chosen.data_ptr(), int(activation), _code(h.dtype), _stream()),
           "moe_up_plain")


def moe_plain_grouped_built() -> bool:
    """Whether the grouped tile products know experts without a gate matrix."""
    return True


def norm_conv(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, taps: torch.Tensor,
              history: torch.Tensor | None, eps: float, batch) -> None:
    """out = h + conv(h) with h = x / rms(x) * weight: every channel of the normed rows is filtered over time inside
    its own sequence, conv(h)_t = sum_j taps[:, j] h_(t - n + 1 + j) (taps [hidden, n] float32, the last column on the
    token itself, zeros before a sequence's start). `history` [slots, n - 1, hidden] float32 holds the normed rows of
    the tokens before the step and is moved on. x float32 [tokens, hidden]; out in either type."""
    _cuda(out, x, weight, taps, history)
    tokens, hidden = batch.n_tokens, x.shape[1]
    n_taps = taps.shape[1]
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and taps.dtype == torch.float32
    assert weight.numel() == hidden and taps.shape[0] == hidden and out.shape[1] == hidden
    assert x.shape[0] >= tokens and out.shape[0] >= tokens
    assert n_taps == 1 or (history is not None and history.dtype == torch.float32 and
                           tuple(history.shape[1:]) == (n_taps - 1, hidden))
    _check(_fn("elementwise", "dllm_norm_conv")(
        out.data_ptr(), x.data_ptr(), weight.data_ptr(), taps.data_ptr(), n_taps,
        history.data_ptr() if history is not None else None, batch.tok_seq.data_ptr(), batch.cu_seqlens.data_ptr(),
        batch.slots.data_ptr(), tokens, batch.n_seqs, hidden, float(eps), 1 if batch.is_decode else 0,
        _code(out.dtype), _stream()), "norm_conv", lambda: f"taps={n_taps} (at most 8)")
    if not batch.is_decode and n_taps > 1:
        global launches
        launches += 1  # (the history's own small kernel)


def bias_act(out: torch.Tensor, rows: torch.Tensor, bias: torch.Tensor | None, activation: int, width: int,
             gated: bool = False) -> None:
    """out[r, i] = activation(rows[r, i] + bias[i]) for i < width, times sigmoid(rows[r, width]) if `gated` (the
    column behind the activated ones is then the row's gate); out's columns behind `width` are set to zero. rows
    float32 (a product's output); out either type."""
    _cuda(out, rows, bias)
    n = out.shape[0]
    assert out.shape[1] >= width
    assert rows.dtype == torch.float32 and rows.shape[0] >= n and rows.shape[1] >= width + (1 if gated else 0)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == width)
    _check(_fn("elementwise", "dllm_bias_act")(out.data_ptr(), rows.data_ptr(),
                                               bias.data_ptr() if bias is not None else None, n, int(width),
                                               out.shape[1], rows.shape[1],
                                               int(activation), 1 if gated else 0, _code(out.dtype), _stream()),
           "bias_act")


def add_row(residual: torch.Tensor, row: torch.Tensor) -> None:
    """residual[r] += row for every r (float32): a bias behind a product that added into the stream."""
    _cuda(residual, row)
    assert residual.dtype == torch.float32 and row.dtype == torch.float32 and row.numel() == residual.shape[1]
    _check(_fn("elementwise", "dllm_add_row")(residual.data_ptr(), row.data_ptr(), residual.shape[0],
                                              residual.shape[1], _stream()), "add_row")


def gate_embed(out: torch.Tensor, z: torch.Tensor, table: torch.Tensor, offset: int, width: int, tokens: torch.Tensor,
               activation: int, status: torch.Tensor | None = None) -> None:
    """out[r, i] = activation(z[r, i]) * table[tokens[r], offset + i] for i < width, zeros in out's columns behind (a
    reduction width padded for the next product). z float32 [rows, >= width]; table and out in the same type."""
    _cuda(out, z, table, tokens)
    if status is None:
        status = _status_word()
    rows = out.shape[0]
    assert z.dtype == torch.float32 and z.shape[0] >= rows and z.shape[1] >= width and out.shape[1] >= width
    assert table.dtype == out.dtype and tokens.dtype == torch.int32 and tokens.numel() >= rows
    _check(_fn("elementwise", "dllm_gate_embed")(out.data_ptr(), z.data_ptr(), z.shape[1], table.data_ptr(),
                                                 table.shape[1], table.shape[0], int(offset), tokens.data_ptr(), rows,
                                                 int(width), out.shape[1], int(activation), _code(out.dtype),
                                                 status.data_ptr(), _stream()), "gate_embed")


def latent_prepare(rows: torch.Tensor, cq_at: int, q_rank: int, c_at: int, rank: int, rot: int,
                   q_weight: torch.Tensor | None, c_weight: torch.Tensor, eps: float, table: torch.Tensor | None,
                   cq_out: torch.Tensor | None, cache, batch, write_cache: bool = True) -> None:
    """From a token's projected float32 row: the query latent (q_rank values at column cq_at) divided by its root mean
    square times q_weight -> cq_out (activation type); the key latent (rank values at c_at) normed likewise with
    c_weight and the `rot` values behind it rotated in halves by the token's position -> the token's row [rank + rot]
    of the keys-only cache entry."""
    _cuda(rows, q_weight, c_weight, table, cq_out)
    tokens = batch.n_tokens
    assert rows.dtype == torch.float32 and c_weight.dtype == torch.float32 and cache.head_dim == rank + rot
    assert cache.keys_only and cache.kv_heads == 1
    assert q_rank == 0 or (cq_out.dtype == cache.dtype and q_weight.numel() == q_rank)
    if rot:
        assert table.dtype == torch.float32 and table.shape[0] > batch.max_position, "position beyond the table"
        assert table.shape[1] == rot // 2 and table.shape[2] == 2
    _check(_fn("latent_attention", "dllm_latent_prepare")(
        rows.data_ptr(), rows.shape[1], int(cq_at), int(q_rank), int(c_at), int(rank), int(rot),
        q_weight.data_ptr() if q_weight is not None else None, c_weight.data_ptr(), float(eps),
        table.data_ptr() if table is not None else None, cq_out.data_ptr() if cq_out is not None else None,
        cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size, batch.tok_seq.data_ptr(),
        batch.tok_pos.data_ptr(), batch.slots.data_ptr(), tokens, 1 if write_cache else 0, _code(cache.dtype),
        _stream()), "latent_prepare")


def latent_queries(out: torch.Tensor, q: torch.Tensor, uk: torch.Tensor, table: torch.Tensor | None, heads: int,
                   dim: int, rot: int, rank: int, scale: float, batch) -> None:
    """Queries in the latent's coordinates: q float32 [tokens, heads x (dim + rot)] head by head [plain | rotated
    part]; out float32 [tokens, heads x (rank + rot)] = [uk_h^T q_plain | rotate(q_rot)] x scale, uk [heads x dim,
    rank] the map from the latent to the heads' keys."""
    _cuda(out, q, uk, table)
    tokens = batch.n_tokens
    assert q.dtype == torch.float32 and out.dtype == torch.float32
    assert q.shape[1] == heads * (dim + rot) and out.shape[1] == heads * (rank + rot)
    assert tuple(uk.shape) == (heads * dim, rank)
    _check(_fn("latent_attention", "dllm_latent_queries")(
        q.data_ptr(), uk.data_ptr(), table.data_ptr() if table is not None else None, out.data_ptr(), tokens, heads,
        dim, rot, rank, float(scale), batch.tok_pos.data_ptr(), _code(uk.dtype), _stream()), "latent_queries")


def latent_attention(out: torch.Tensor, q: torch.Tensor, cache, heads: int, rank: int, rot: int, batch,
                     sinks: torch.Tensor | None = None) -> None:
    """Causal softmax attention of every (token, head) over the rows [rank + rot] its sequence has cached: scores
    q . row (the queries carry the scale), out float32 [tokens, heads x rank] = the weighted sum of the rows' first
    `rank` values. With `sinks` (float32 [heads]) the softmax's denominator also holds exp(sinks[head]), a score that
    has no key and no value. The general kernel: float32 arithmetic, either cache type, rank up to 512."""
    _cuda(out, q, sinks)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == heads)
    assert q.dtype == torch.float32 and out.dtype == torch.float32 and cache.head_dim == rank + rot
    assert q.shape[1] == heads * (rank + rot) and out.shape[1] == heads * rank
    _check(_fn("latent_attention", "dllm_latent_attention")(
        q.data_ptr(), out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, rank, rot, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(), batch.n_tokens,
        _code(cache.dtype), sinks.data_ptr() if sinks is not None else None, _stream()), "latent_attention",
        lambda: f"rank={rank} (at most 512)")


def latent_values(out: torch.Tensor, mixed: torch.Tensor, uv: torch.Tensor, gates: torch.Tensor | None, gate_at: int,
                  heads: int, rank: int, vdim: int) -> None:
    """out[t, h] = (uv_h mixed[t, h]) x sigmoid(gates[t, gate_at + h]): the heads' values from their weighted sums of
    the latent; mixed float32 [tokens, heads x rank], uv [heads x vdim, rank], out [tokens, heads x vdim] in uv's
    type; gates float32 rows (None: no gate)."""
    _cuda(out, mixed, uv, gates)
    tokens = out.shape[0]
    assert mixed.dtype == torch.float32 and out.dtype == uv.dtype and tuple(uv.shape) == (heads * vdim, rank)
    assert mixed.shape[1] == heads * rank and out.shape[1] == heads * vdim
    gate_ptr = (gates.data_ptr() + 4 * int(gate_at)) if gates is not None else None
    _check(_fn("latent_attention", "dllm_latent_values")(
        mixed.data_ptr(), uv.data_ptr(), gate_ptr, gates.shape[1] if gates is not None else 0, out.data_ptr(), tokens,
        heads, rank, vdim, _code(out.dtype), _stream()), "latent_values")


def latent_tiles(dtype, rank: int, rot: int, page_size: int = 64):
    """The padded rank the tensor-core kernel runs a latent of these sizes with, or None where only the general kernel
    runs: float32, a rank above 256, rows that are no whole 16-byte pieces or too long for a block's shared memory,
    pages that are no multiple of 32."""
    if dtype != torch.bfloat16 or rank > 256 or rank % 8 or (rank + rot) % 8 or rot % 2 or page_size % 32:
        return None
    padded = 64 if rank <= 64 else (128 if rank <= 128 else 256)
    row = max(-(-(rank + rot) // 16) * 16, padded) + 8  # values of a shared-memory row
    if 128 * row * 2 > 200 * 1024:  # (64 query rows and two stages of 32 keys)
        return None
    return padded


def latent_splits(batch, heads: int) -> int:
    """Over how many blocks the tile kernel deals a sequence's keys: one where the step's rows fill the
    multiprocessors by themselves, else enough for two blocks each, every block with 64 positions or more."""
    blocks = batch.n_seqs * (-(-batch.max_new * heads // 64))
    return max(1, min(64, 296 // max(1, blocks), batch.max_context // 64))


def latent_attention_tiled(out: torch.Tensor, q: torch.Tensor, table: torch.Tensor | None, gates: torch.Tensor | None,
                           gate_at: int, cache, heads: int, rank: int, rot: int, batch, ws=None,
                           sinks: torch.Tensor | None = None) -> None:
    """`latent_attention` on the tensor cores over a bfloat16 cache. q float32 [tokens, heads x (rank + rot)] in the
    latent's coordinates, scale included; with `table` its rotated parts are rotated on the way in. out [tokens,
    heads x rank]: float32, or bfloat16; with `gates` (float32 rows, head h at column gate_at + h) every head's sum
    is multiplied by the sigmoid of its gate; with `sinks` (float32 [heads]) the softmax's denominator also holds
    exp(sinks[head])."""
    _cuda(out, q, table, gates, sinks)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == heads)
    assert q.dtype == torch.float32 and out.dtype in (torch.float32, torch.bfloat16)
    assert cache.dtype == torch.bfloat16 and cache.keys_only and cache.kv_heads == 1 and cache.head_dim == rank + rot
    assert q.shape[1] == heads * (rank + rot) and out.shape[1] == heads * rank and out.is_contiguous()
    if table is not None:
        assert table.dtype == torch.float32 and table.shape[0] > batch.max_position, "position beyond the table"
        assert table.shape[1] == rot // 2 and table.shape[2] == 2
    gate_ptr = (gates.data_ptr() + 4 * int(gate_at)) if gates is not None else None
    pairs = batch.n_tokens * heads
    splits = latent_splits(batch, heads) if ws is not None else 1
    part_o = ws.buffer("latent_part_o", (pairs * splits * rank,), torch.float32) if splits > 1 else None
    part_ml = ws.buffer("latent_part_ml", (pairs * splits * 2,), torch.float32) if splits > 1 else None
    _check(_fn("latent_attention_tiled", "dllm_latent_attention_tiled")(
        q.data_ptr(), table.data_ptr() if table is not None else None, gate_ptr,
        gates.shape[1] if gates is not None else 0, sinks.data_ptr() if sinks is not None else None, out.data_ptr(),
        1 if out.dtype == torch.bfloat16 else 0,
        cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads, rank, rot,
        batch.cu_seqlens.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(), batch.n_seqs,
        int(batch.max_new), splits, part_o.data_ptr() if splits > 1 else None,
        part_ml.data_ptr() if splits > 1 else None, pairs, _stream()), "latent_attention_tiled",
        lambda: f"rank={rank} (a multiple of 8, at most 256) rot={rot} page={cache.page_size}")


def running_max_gates(aux: torch.Tensor, rows: torch.Tensor, i_at: int, f_at: int, i_bias: torch.Tensor | None,
                      f_bias: torch.Tensor | None, cap: float, heads: int, state: torch.Tensor, batch) -> None:
    """The per-token factors of the gated outer products: log input gate i = cap tanh((z_i + b_i) / cap), log forget
    gate f = logsigmoid(cap tanh((z_f + b_f) / cap)), running maximum m' = max(f + m, i) carried in `state` [slots,
    heads] from step to step (zero at a sequence's start); aux [tokens, 3 heads] = [exp(f + m - m') | exp(i - m') |
    exp(-m')]. z_i, z_f: columns i_at, f_at of `rows` (float32)."""
    _cuda(aux, rows, i_bias, f_bias, state)
    assert all(t.dtype == torch.float32 for t in (aux, rows, state)) and aux.shape[1] >= 3 * heads
    assert tuple(state.shape[1:]) == (heads,) and aux.shape[0] >= batch.n_tokens
    _check(_fn("recurrent", "dllm_running_max_gates")(
        _columns(rows, i_at), _columns(rows, f_at), rows.shape[1], i_bias.data_ptr() if i_bias is not None else None,
        f_bias.data_ptr() if f_bias is not None else None, float(cap), state.data_ptr(), batch.cu_seqlens.data_ptr(),
        batch.slots.data_ptr(), batch.n_seqs, heads, aux.data_ptr(), aux.shape[1], _stream()), "running_max_gates")


def gated_scan(out: torch.Tensor, nq: torch.Tensor, rows: torch.Tensor, q_at: int, k_at: int, v_at: int, heads: int,
               dim: int, vdim: int, aux: torch.Tensor, q_scale: float, state: torch.Tensor, batch) -> None:
    """Per sequence and head, over the step's tokens in order: S <- a_t S + b_t k v^T, out = S^T q x q_scale, and the
    same with v = 1 in one more column of S, read out as nq [tokens, heads] = n . q x q_scale. a_t, b_t: the first
    two blocks of `aux` (`running_max_gates`). state [slots, heads, vdim + 1, dim] float32."""
    _cuda(out, nq, rows, aux, state)
    assert all(t.dtype == torch.float32 for t in (out, nq, rows, aux, state))
    assert tuple(state.shape[1:]) == (heads, vdim + 1, dim) and out.shape[1] == heads * vdim and nq.shape[1] == heads
    _check(_fn("recurrent", "dllm_gated_scan")(
        _columns(rows, q_at), _columns(rows, k_at), _columns(rows, v_at), rows.shape[1], heads, dim, vdim,
        aux.data_ptr(), aux.shape[1], float(q_scale), state.data_ptr(), batch.cu_seqlens.data_ptr(),
        batch.slots.data_ptr(), batch.n_seqs, int(batch.max_new), out.data_ptr(), nq.data_ptr(), _stream()),
        "gated_scan", lambda: f"dim={dim} (a multiple of 4, at most 256)")


def normalised_readout(out: torch.Tensor, x: torch.Tensor, nq: torch.Tensor, aux: torch.Tensor, floor_at: int,
                       weight: torch.Tensor | None, rows: torch.Tensor, gate_at: int, heads: int, vdim: int,
                       eps: float) -> None:
    """out = x / (max(|nq|, floor) + 1e-6) per head (floor: column floor_at + head of `aux`), then divided by its
    root mean square over the head, times weight [heads x vdim], times sigmoid of the gate pre-activations at column
    gate_at of `rows`; x float32 [tokens, heads x vdim]."""
    _cuda(out, x, nq, aux, weight, rows)
    tokens = out.shape[0]
    assert all(t.dtype == torch.float32 for t in (x, nq, aux, rows)) and x.shape[1] == heads * vdim
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == heads * vdim)
    _check(_fn("recurrent", "dllm_normalised_readout")(
        out.data_ptr(), x.data_ptr(), nq.data_ptr(), _columns(aux, floor_at), aux.shape[1],
        weight.data_ptr() if weight is not None else None, _columns(rows, gate_at), rows.shape[1], tokens, heads, vdim,
        float(eps), _code(out.dtype), _stream()), "normalised_readout")


def moe_down(out: torch.Tensor, act: torch.Tensor, w_down: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor,
             top: int, accumulate: bool = False) -> None:
    """out[t] (float32) = sum over k of weights[t, k] * W_down[chosen[t, k]] act[t, k] (added to out if
    `accumulate`). W_down [experts, width, ff]."""
    _cuda(out, act, w_down, chosen, weights)
    tokens, width = out.shape
    ff = w_down.shape[2]
    assert out.dtype == torch.float32 and act.dtype == w_down.dtype and w_down.shape[1] == width
    assert act.numel() >= tokens * top * ff and chosen.dtype == torch.int32 and weights.dtype == torch.float32
    _check(_fn("moe", "dllm_moe_down")(out.data_ptr(), act.data_ptr(), ff, w_down.data_ptr(), width, int(top), tokens,
                                       chosen.data_ptr(), weights.data_ptr(), 1 if accumulate else 0,
                                       _code(act.dtype), _stream()), "moe_down")


MOE_GROUPED_FROM = 64
"""Steps of more tokens than this run the experts as grouped tile products (`moe_experts_grouped`); smaller ones read
each chosen expert's rows once per token (`moe_up`, `moe_down`), which is what few tokens need."""


def moe_grouped_supported(tokens: int, dtype, width: int, ff: int) -> bool:
    return dtype == torch.bfloat16 and tokens > MOE_GROUPED_FROM and width % 8 == 0 and ff % 8 == 0


def moe_experts_grouped(out: torch.Tensor, h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                        chosen: torch.Tensor, weights: torch.Tensor, top: int, limit: float, alpha: float, shift: float,
                        offsets: torch.Tensor, place_pair: torch.Tensor, act: torch.Tensor, y: torch.Tensor,
                        accumulate: bool = False) -> None:
    """What `moe_up` and `moe_down` compute, for many tokens (bfloat16): the (token, choice) pairs are put in expert
    order on the device, every expert's rows run as tile products on the tensor cores (gate/up with the gated unit in
    the epilogue, then down, scattered back by pair), and a last kernel forms each token's weighted sum. Four launches
    whose shapes depend on the sizes only. Scratch: offsets [experts + 1] and place_pair [pairs] int32, act [pairs, ff]
    bfloat16, y [pairs, width] float32."""
    _cuda(out, h, w_gate_up, w_down, chosen, weights, offsets, place_pair, act, y)
    tokens, width = h.shape
    experts, ff = w_gate_up.shape[0], w_gate_up.shape[1] // 2
    pairs = tokens * top
    assert h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
    assert tuple(w_down.shape) == (experts, width, ff) and w_gate_up.shape[2] == width
    assert out.dtype == torch.float32 and tuple(out.shape) == (tokens, width)
    assert offsets.dtype == torch.int32 and offsets.numel() >= experts + 1 and place_pair.numel() >= pairs
    assert act.dtype == torch.bfloat16 and act.numel() >= pairs * ff and y.dtype == torch.float32
    assert y.numel() >= pairs * width and chosen.dtype == torch.int32 and weights.dtype == torch.float32
    stream = _stream()
    _check(_fn("moe_grouped", "dllm_moe_sort")(chosen.data_ptr(), pairs, experts, offsets.data_ptr(),
                                               place_pair.data_ptr(), stream), "moe_sort",
           lambda: f"experts={experts} (at most 256)")
    _check(_fn("moe_grouped", "dllm_moe_grouped_up")(
        act.data_ptr(), h.data_ptr(), width, w_gate_up.data_ptr(), ff, experts, int(top), tokens, offsets.data_ptr(),
        place_pair.data_ptr(), float(limit), float(alpha), float(shift), stream), "moe_grouped_up",
        lambda: f"width={width} (a multiple of 8)")
    _check(_fn("moe_grouped", "dllm_moe_grouped_down")(
        y.data_ptr(), act.data_ptr(), ff, w_down.data_ptr(), width, experts, int(top), tokens, offsets.data_ptr(),
        place_pair.data_ptr(), stream), "moe_grouped_down", lambda: f"ff={ff} (a multiple of 8)")
    _check(_fn("moe_grouped", "dllm_moe_combine")(out.data_ptr(), y.data_ptr(), weights.data_ptr(), width, int(top),
                                                  tokens, 1 if accumulate else 0, stream), "moe_combine")


def moe_plain_experts_grouped(out: torch.Tensor, h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                              chosen: torch.Tensor, weights: torch.Tensor, top: int, kind: int, offsets: torch.Tensor,
                              place_pair: torch.Tensor, act: torch.Tensor, y: torch.Tensor,
                              accumulate: bool = False) -> None:
    """`moe_experts_grouped` for experts without a gate matrix: W_down act(W_up h) with the activation `kind` in the
    first product's epilogue. w_up [experts, ff, width], w_down [experts, width, ff]; the same scratch."""
    _cuda(out, h, w_up, w_down, chosen, weights, offsets, place_pair, act, y)
    tokens, width = h.shape
    experts, ff = w_up.shape[0], w_up.shape[1]
    pairs = tokens * top
    assert h.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
    assert tuple(w_down.shape) == (experts, width, ff) and w_up.shape[2] == width
    assert out.dtype == torch.float32 and tuple(out.shape) == (tokens, width)
    assert offsets.dtype == torch.int32 and offsets.numel() >= experts + 1 and place_pair.numel() >= pairs
    assert act.dtype == torch.bfloat16 and act.numel() >= pairs * ff and y.dtype == torch.float32
    assert y.numel() >= pairs * width and chosen.dtype == torch.int32 and weights.dtype == torch.float32
    stream = _stream()
    _check(_fn("moe_grouped", "dllm_moe_sort")(chosen.data_ptr(), pairs, experts, offsets.data_ptr(),
                                               place_pair.data_ptr(), stream), "moe_sort",
           lambda: f"experts={experts} (at most 256)")
    _check(_fn("moe_grouped", "dllm_moe_grouped_up_plain")(
        act.data_ptr(), h.data_ptr(), width, w_up.data_ptr(), ff, experts, int(top), tokens, offsets.data_ptr(),
        place_pair.data_ptr(), int(kind), stream), "moe_grouped_up",
        lambda: f"width={width} (a multiple of 8) ff={ff} (even)")
    _check(_fn("moe_grouped", "dllm_moe_grouped_down")(
        y.data_ptr(), act.data_ptr(), ff, w_down.data_ptr(), width, experts, int(top), tokens, offsets.data_ptr(),
        place_pair.data_ptr(), stream), "moe_grouped_down", lambda: f"ff={ff} (a multiple of 8)")
    _check(_fn("moe_grouped", "dllm_moe_combine")(out.data_ptr(), y.data_ptr(), weights.data_ptr(), width, int(top),
                                                  tokens, 1 if accumulate else 0, stream), "moe_combine")


def concat_restart(both: torch.Tensor, x: torch.Tensor, kept: torch.Tensor, start: torch.Tensor | None) -> None:
    """both[r] = [x[r] | kept[r]] in both's dtype, then x[r] = start (a row of float32, or zeros)."""
    _cuda(both, x, kept, start)
    rows, hidden = kept.shape
    assert x.dtype == torch.float32 and kept.dtype == torch.float32 and x.shape == kept.shape
    assert both.shape == (rows, 2 * hidden) and (start is None or (start.dtype == torch.float32 and
                                                                    start.numel() == hidden))
    _check(_fn("elementwise", "dllm_concat_restart")(both.data_ptr(), x.data_ptr(), kept.data_ptr(),
                                                     start.data_ptr() if start is not None else None, rows, hidden,
                                                     _code(both.dtype), _stream()), "concat_restart")


def _columns(rows: torch.Tensor, offset: int) -> int:
    return rows.data_ptr() + 4 * int(offset)


def decay_scan(out: torch.Tensor, rows: torch.Tensor, q_at: int, k_at: int, v_at: int, heads: int, dim: int, vdim: int,
               decay: torch.Tensor, silu_inputs: bool, k_scale: float, state: torch.Tensor, batch) -> None:
    """Per sequence and head, over the step's tokens in order: S <- decay_h S + k v^T, out = S^T q, from and to
    `state` [slots, heads, vdim, dim] (float32, S stored column by column). `rows` [tokens, n] float32 holds q, k
    and v of a token at the column offsets q_at, k_at, v_at; with `silu_inputs` the columns from q_at to the end of v
    (which must lie one behind the other) pass silu first, in place; k counts k_scale times (the sums are linear in
    k: the state holds the unscaled sum and the read-out is multiplied)."""
    _cuda(out, rows, decay, state)
    assert rows.dtype == torch.float32 and out.dtype == torch.float32 and state.dtype == torch.float32
    assert decay.dtype == torch.float32 and decay.numel() == heads
    assert tuple(state.shape[1:]) == (heads, vdim, dim) and out.shape[1] == heads * vdim
    assert rows.shape[0] >= batch.n_tokens and out.shape[0] >= batch.n_tokens
    if silu_inputs:
        assert q_at == 0 and k_at == heads * dim and v_at == 2 * heads * dim
        _check(_fn("recurrent", "dllm_silu_columns")(rows.data_ptr(), batch.n_tokens, v_at + heads * vdim,
                                                     rows.shape[1], _stream()), "silu_columns")
    _check(_fn("recurrent", "dllm_decay_scan")(
        _columns(rows, q_at), _columns(rows, k_at), _columns(rows, v_at), rows.shape[1], heads, dim, vdim,
        decay.data_ptr(), float(k_scale), state.data_ptr(), batch.cu_seqlens.data_ptr(),
        batch.slots.data_ptr(), batch.n_seqs, int(batch.max_new), out.data_ptr(), _stream()), "decay_scan",
        lambda: f"dim={dim} (a multiple of 4, at most 256)")


def delta_prepare(prepared: torch.Tensor, aux: torch.Tensor, rows: torch.Tensor, b_at: int, a_at: int,
                  taps: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, history: torch.Tensor | None,
                  heads: int, qk_heads: int, dim: int, vdim: int, batch) -> None:
    """What the gated delta rule's scan reads, from the projected rows [tokens, n] float32 = [q | k | v | ...]:
    the causal convolution over time per channel (taps [channels, width] float32; inputs of earlier steps from
    `history` [slots, width - 1, channels], which is moved on), silu, unit vectors for q and k per head (q times
    dim^-1/2) -> prepared [tokens, channels]; and aux [tokens, 2 heads + qk_heads] = decay g, step size beta (from
    the columns at a_at and b_at), and k.q."""
    _cuda(prepared, aux, rows, taps, a_log, dt_bias, history)
    channels = 2 * qk_heads * dim + heads * vdim
    assert all(t.dtype == torch.float32 for t in (prepared, aux, rows, taps, a_log, dt_bias))
    assert taps.shape[0] == channels and prepared.shape[1] == channels and aux.shape[1] == 2 * heads + qk_heads
    width = taps.shape[1]
    assert history is None or (history.dtype == torch.float32 and tuple(history.shape[1:]) == (width - 1, channels))
    _check(_fn("recurrent", "dllm_delta_prepare")(
        rows.data_ptr(), rows.shape[1], int(b_at), int(a_at), taps.data_ptr(), width, a_log.data_ptr(),
        dt_bias.data_ptr(), history.data_ptr() if history is not None else None, batch.tok_seq.data_ptr(),
        batch.cu_seqlens.data_ptr(), batch.slots.data_ptr(), batch.n_tokens, batch.n_seqs, heads, qk_heads, dim, vdim,
        prepared.data_ptr(), aux.data_ptr(), 1 if batch.is_decode else 0, _stream()), "delta_prepare",
        lambda: f"taps={width} (at most 16), dim={dim} (a multiple of 4, at most 256)")
    if not batch.is_decode and width > 1:
        global launches
        launches += 1  # (the history's own small kernel)


def delta_scan(out: torch.Tensor, prepared: torch.Tensor, aux: torch.Tensor, heads: int, qk_heads: int, dim: int,
               vdim: int, state: torch.Tensor, batch) -> None:
    """Per sequence and head, over the step's tokens in order: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    out = S^T q, from and to `state` [slots, heads, vdim, dim]. `prepared`, `aux`: what `delta_prepare` wrote."""
    _cuda(out, prepared, aux, state)
    assert all(t.dtype == torch.float32 for t in (out, prepared, aux, state))
    assert tuple(state.shape[1:]) == (heads, vdim, dim) and out.shape[1] == heads * vdim
    _check(_fn("recurrent", "dllm_delta_scan")(
        prepared.data_ptr(), _columns(prepared, qk_heads * dim), _columns(prepared, 2 * qk_heads * dim),
        prepared.shape[1], heads, qk_heads, dim, vdim, aux.data_ptr(), aux.shape[1], state.data_ptr(),
        batch.cu_seqlens.data_ptr(), batch.slots.data_ptr(), batch.n_seqs, int(batch.max_new), out.data_ptr(),
        _stream()), "delta_scan",
        lambda: f"dim={dim} (a multiple of 4, at most 256)")


GATE_SILU, GATE_SIGMOID = 1, 2


def gated_norm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor | None, rows: torch.Tensor, gate_at: int,
               group: int, eps: float, gate: int) -> None:
    """out = x / rms(x over groups of `group` values) * weight[i % group] * gate(z), z the token's gate values at
    column offset gate_at of `rows` [tokens, n] float32; gate GATE_SILU or GATE_SIGMOID. x float32 [tokens, width]."""
    _cuda(out, x, weight, rows)
    tokens, width = out.shape
    assert x.dtype == torch.float32 and rows.dtype == torch.float32 and x.shape[1] == width
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == group)
    _check(_fn("recurrent", "dllm_gated_norm")(
        out.data_ptr(), x.data_ptr(), weight.data_ptr() if weight is not None else None, _columns(rows, gate_at),
        rows.shape[1], tokens, width, int(group), float(eps), int(gate), _code(out.dtype), _stream()), "gated_norm")


prefetch_hints: dict[int, torch.Tensor] = {}
"""Weight tensor (by address) -> the weight tensor a later kernel of the step streams. A decode-sized product whose
weights are a key asks the L2 cache for the value while it runs. The model fills this from its run order."""


PREFETCH_LIMIT = 16 << 20
"""Larger weights are not asked into L2 ahead of time: four products of them would not fit there anyway."""


PREFETCH_SLICED_LIMIT = 64 << 20
"""A step's last matrix (the head's) up to this size is asked into L2 in slices by the products before it."""


def _prefetch_of(w: torch.Tensor):
    hint = prefetch_hints.get(w.data_ptr())
    if hint is None or hint.numel() * hint.element_size() > PREFETCH_LIMIT:
        return (None, 0)
    return (hint.data_ptr(), hint.numel() * hint.element_size())


_async_status = None


def _status_word() -> torch.Tensor:
    """A pinned host word that kernels with bounded waits set when a wait runs out; the host can read it at any
    time without a synchronisation."""
    global _async_status
    if _async_status is None:
        _async_status = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _async_status


def raise_if_failed() -> None:
    """Raises if a kernel has set the status word since the last look: a bounded wait on an mbarrier ran out
    (codes 2-5 the tile product, 12-21 the tcgen05 attention, 32-33 the product that streams through shared memory)
    or the embedding met a token outside its table (64). Results computed since are not valid. The word lives in
    pinned host memory, so the look costs no synchronisation; it is meaningful after the host has waited for the
    kernels in question (a `.tolist()`, a copy to the host, a synchronize)."""
    if _async_status is not None and int(_async_status[0]) != 0:
        code = int(_async_status[0])
        _async_status[0] = 0
        if code == 64:
            raise KernelError("the embedding was given a token outside its table; the step's results are invalid")
        raise KernelError(f"a kernel gave up waiting on an mbarrier (role code {code}); the step's results are invalid")


GEMV_MAX_ROWS = 64
"""The weight-streaming kernel takes at most this many activation rows."""


CLUSTER_SPLIT_BYTES = (1 << 20, 16 << 20)
CLUSTER_NARROW_ROWS = 8192


def splits_over_clusters(rows: int, outputs: int, inner: int) -> bool:
    """Whether a product with 9 to 64 rows of activations takes the kernel that splits the reduction over the
    blocks of a thread-block cluster (`gemv_cluster.cu`): weights of a few megabytes, where bringing the activations
    to the multiprocessors is the cost and a block per 16 rows of W reads them far too often. Measured at the layer
    sizes of a 576-wide model, as links of a chain of dependent launches: with 64 rows 4.0 to 7.4 µs against 4.9 to
    10.8; with 16 rows 3.2 to 3.6 against 3.8 to 4.5, but 2.5 against 2.3 for the smallest matrix (576 x 576); with 8
    rows the kernel with a block per 16 rows of W wins everywhere (1.5 to 2.5 against 2.4 to 3.3).
    With 17 to 64 rows it also takes larger weights of few rows (at most 8,192: 6144 x 4096 with 32 rows 16.6 µs
    against 21.1 for a block per 16 rows and 23.7 for the tile kernel, with 64 rows 22.3 against 47.3 and 23.9;
    4096 x 14336 with 32 rows 29.9 against 40.0 and 73.9), where the tile kernel has too few tiles for the device."""
    size = 2 * outputs * inner
    if 16 < rows <= GEMV_MAX_ROWS:
        return size <= CLUSTER_SPLIT_BYTES[1] or outputs <= CLUSTER_NARROW_ROWS
    return 8 < rows <= 16 and CLUSTER_SPLIT_BYTES[0] <= size <= CLUSTER_SPLIT_BYTES[1]


def streams(rows: int, outputs: int, inner: int | None = None) -> bool:
    """Whether a bfloat16 product of `rows` activation rows and `outputs` weight rows (of `inner` values, if given)
    runs in one of the weight-streaming kernels, which can take an RMSNorm in front: always up to 16 rows; up to 64
    rows where the weights are small enough for the kernel that splits the reduction over a cluster, or unless the
    matrix has so many rows that its blocks (16 weight rows each) would together re-read the activations far more
    often than the weights."""
    if rows <= 16:
        return True
    if inner is not None and splits_over_clusters(rows, outputs, inner):
        return True
    if rows <= 32:
        return outputs <= 4096
    # 33 to 64 rows: measured at 576-wide layers, the tile kernel (with a separate norm) wins from 2,048 weight rows
    # on (gate/up 3072 x 576 with 48 rows: 9.0 against 10.6 µs), the streaming kernel below that
    return rows <= GEMV_MAX_ROWS and outputs < 2048


TMA_STREAM_BYTES = 48 << 20


def streams_through_shared_memory(rows: int, outputs: int, inner: int) -> bool:
    """Whether a decode-sized product takes the kernel that streams W through a ring of shared-memory stages.
    Measured against the kernel that streams through registers: it wins (0.71 to 0.97 of the HBM rate against 0.65 to
    0.89) for few rows of activations, long rows of W (its copies are 2 KB pieces of a row) and matrices of tens of
    megabytes; with more rows the copies of the activations cost it the lead."""
    if inner % 64 or 2 * outputs * inner < TMA_STREAM_BYTES:
        return False
    # (up to 4 rows its lead holds, 6144 x 4096: 11.3 µs against 12.2; up to 8 rows only for very long rows of W,
    # 4096 x 14336: 24.2 against 28.8)
    return (rows <= 4 and inner >= 4096) or (rows <= 8 and inner >= 8192)


def takes_weights_as_rows(rows: int, outputs: int, inner: int) -> bool:
    """Whether a product with 3 to 64 rows of activations runs the other way round on the tile kernel (W as the
    128-row operand, read once). Measured: it wins where W has at least as many 128-row tiles as the device has
    multiprocessors (28672 x 4096 with 64 rows: 49 µs against 89 µs for the tile kernel and 187 µs for the streaming
    one; 16384 x 2048: 17 against 25); with fewer tiles a block's rate is bound by its one lane issuing products."""
    if not (outputs >= 16384 and 2 * outputs * inner >= (32 << 20)):
        return False
    # with 3 to 16 rows (the tile kernel's time does not depend on the rows): from 9 rows on, where the streaming
    # kernels need a second fragment of tokens (16384 x 2048 with 16 rows: 16.6 µs against 19.6; 49152 x 2048: 39.0
    # against 47.1), and from 3 rows on for rows of W of 4,096 values or more (128256 x 4096 with 8 rows: 176 against
    # 194; 28672 x 4096: 43.8 against 46.6; with rows of 2,048 values and up to 8 rows the streaming kernel reads at
    # 0.9 to 1.0 of the memory rate and keeps them)
    return 16 < rows <= 64 or (8 < rows <= 16 and inner >= 2048) or (3 <= rows <= 8 and inner >= 4096)


SPLIT_MIN_BYTES = 16 << 20
MAX_REDUCTION_SPLIT = 8


B200_MULTIPROCESSORS = 148


_sm_count = 0


def _multiprocessors() -> int:
    """The device's multiprocessors (a B200's where no device is present: the rules are plain functions of sizes)."""
    global _sm_count
    if _sm_count == 0:
        _sm_count = (torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
                     if torch.cuda.is_available() else B200_MULTIPROCESSORS)
    return _sm_count


def reduction_split(rows: int, outputs: int, inner: int, multiprocessors: int | None = None) -> int:
    """Into how many stretches the reduction of a residual product with 33 to 64 rows of activations is cut, 1 for
    not at all. A W of few rows and a long reduction (an output or down projection: 4096 x 14336, 2048 x 8192) has
    fewer 128-row tiles than the device has multiprocessors, and a multiprocessor takes in about 80 GB/s: with 32
    tiles the whole device reads W at a quarter of its memory rate. Cut, the tiles of every stretch run side by side
    and a second small kernel sums their partial results in order. Measured with 64 rows, both kernels together,
    against the best of the other kernels: 4096 x 14336 29.3 µs against 73.3, 4096 x 4096 12.9 against 20.0,
    2048 x 8192 13.4 against 19.1; with 32 rows and fewer, and for weights under 16 MB, the kernel that splits the
    reduction over a cluster is as fast or faster (2048 x 2048 with 64 rows: 7.6 against 8.9)."""
    if not (32 < rows <= GEMV_MAX_ROWS) or inner % 8 or outputs % 4 or 2 * outputs * inner <= SPLIT_MIN_BYTES:
        return 1
    multiprocessors = multiprocessors or _multiprocessors()
    tiles, k_tiles = -(-outputs // 128), -(-inner // 64)
    if tiles >= multiprocessors:
        return 1
    # doubled while the work items stay within two a multiprocessor and a stretch keeps eight k tiles or more
    split = 1
    while split < MAX_REDUCTION_SPLIT and tiles * split <= multiprocessors and k_tiles // (split * 2) >= 8:
        split *= 2
    return split


_parts: dict = {}


def _parts_buffer(device, floats: int) -> torch.Tensor:
    """Scratch for partial results, one buffer per size for the life of the process: a captured graph may hold its
    address. Like the work buffers, it serves one stream: a product's parts are read by the kernel behind it."""
    key = (str(device), floats)
    if key not in _parts:
        _parts[key] = torch.empty(floats, device=device, dtype=torch.float32)
    return _parts[key]


def gemm_parts(a: torch.Tensor, w: torch.Tensor, split: int) -> torch.Tensor:
    """The product a[M,K] @ w[N,K]^T (bfloat16, M <= 64) as `split` partial results over stretches of the reduction:
    a float32 tensor [split, M, N] in scratch that the next call of the same width overwrites. The tile kernel runs
    it with W as the 128-row operand; whoever reads the parts sums them in order."""
    _cuda(a, w)
    m, k = a.shape
    n = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == k
    assert 0 < m <= GEMV_MAX_ROWS and 1 <= split <= MAX_REDUCTION_SPLIT
    parts = _parts_buffer(a.device, MAX_REDUCTION_SPLIT * GEMV_MAX_ROWS * n)
    _check(_fn("gemm_tcgen05", "dllm_gemm_tcgen05_split")(
        parts.data_ptr(), w.data_ptr(), a.data_ptr(), n, m, k, split, 32 if m <= 32 else 64,
        _status_word().data_ptr(), _stream()), "gemm_parts",
        lambda: f"M={m} N={n} K={k} (multiple of 8) in {split} stretches (at most one per 64 values of K)")
    return parts[:split * m * n].view(split, m, n)


def gemm(c: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int = EPI_STORE_T, kernel: int = 0,
         norm_weight: torch.Tensor | None = None, eps: float = 0.0, tile_n: int = 0, cluster: int = 0) -> None:
    """c = a[M,K] @ w[N,K]^T with float32 accumulation, then the epilogue: EPI_STORE_F32 (c float32), EPI_STORE_T
    (c in the weights' dtype), EPI_RESIDUAL (c float32 += product), EPI_SWIGLU (w interleaves gate and up rows;
    c[M,N/2] = silu(gate) * up). float32 weights run the true 32-bit kernel; bfloat16 the tcgen05/TMA tile kernel
    or, for M <= 64, a weight-streaming kernel (`kernel`: 0 chooses by the sizes, 1 forces the mma.sync tile kernel,
    2 forces streaming through registers, 3 forces tcgen05, 4 forces streaming through shared memory, 5 forces
    tcgen05 with W as the 128-row operand (for at most 256 rows of `a`), 6 forces the reduction split over a cluster
    (`cluster` blocks, 0 chooses), 7 forces W as the 128-row operand with the reduction cut into `cluster` stretches
    (residual epilogue, at most 64 rows; 0 chooses); `tile_n` picks the tcgen05 tile width).
    With `norm_weight` (streaming kernel only), `a` is the float32 residual stream and is RMS-normed on the way in."""
    _cuda(c, a, w, norm_weight)
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k, (a.shape, w.shape)
    want_cols = n // 2 if epilogue in (EPI_SWIGLU, EPI_GLU_CLAMPED, EPI_GLU_GELU_TANH) else n
    if epilogue in (EPI_GLU_CLAMPED, EPI_GLU_GELU_TANH):
        assert w.dtype == torch.bfloat16 and kernel == 0 and norm_weight is None and glu_clamped_fuses(m, n, k)
    want_dtype = torch.float32 if epilogue in (EPI_STORE_F32, EPI_RESIDUAL) else w.dtype
    assert tuple(c.shape) == (m, want_cols) and c.dtype == want_dtype, (c.shape, c.dtype, m, want_cols, want_dtype)
    def detail() -> str:
        return (f"M={m} N={n} K={k}: K must be a multiple of {4 if w.dtype == torch.float32 else 8}; N even for the "
                f"SwiGLU epilogue; the weight-streaming kernel takes M up to {GEMV_MAX_ROWS}")
    if w.dtype == torch.float32:
        assert a.dtype == torch.float32 and norm_weight is None
        status = _fn("gemm_simt", "dllm_gemm_f32")(c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue,
                                                   _stream())
    elif w.dtype == torch.bfloat16:
        streaming = (kernel == 2 and m <= GEMV_MAX_ROWS) or (kernel == 0 and streams(m, n, k))
        split = reduction_split(m, n, k) if (kernel == 0 and epilogue == EPI_RESIDUAL and norm_weight is None) else 1
        if kernel == 7 or split > 1:
            # W as the 128-row operand, the reduction cut into stretches, the parts summed into c by a second kernel
            assert a.dtype == torch.bfloat16 and norm_weight is None and epilogue == EPI_RESIDUAL and m <= 64
            split = split if kernel == 0 else max(1, int(cluster) or reduction_split(m, n, k))
            parts = gemm_parts(a, w, split)
            status = _fn("elementwise", "dllm_sum_parts_residual")(c.data_ptr(), parts.data_ptr(), split, m * n,
                                                                   _stream())
        elif kernel == 5 or (kernel == 0 and norm_weight is None and takes_weights_as_rows(m, n, k)):
            # the product the other way round: W is the 128-row operand, the tokens are the tile's columns
            assert a.dtype == torch.bfloat16 and norm_weight is None and m <= 256
            width = 32 if m <= 32 else (64 if m <= 64 else (128 if m <= 128 else 256))
            status = _fn("gemm_tcgen05", "dllm_gemm_tcgen05")(
                c.data_ptr(), w.data_ptr(), a.data_ptr(), n, m, k, epilogue + 5, width, _status_word().data_ptr(),
                _stream())
        elif kernel == 4 or (kernel == 0 and norm_weight is None and streams_through_shared_memory(m, n, k)):
            assert a.dtype == torch.bfloat16 and norm_weight is None
            status = _fn("gemv_tma", "dllm_gemv_tma")(c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue,
                                                      _status_word().data_ptr(), _stream())
        elif (kernel == 6 and m <= GEMV_MAX_ROWS) or (kernel == 0 and streaming and splits_over_clusters(m, n, k)):
            if norm_weight is not None:
                assert a.dtype == torch.float32 and norm_weight.dtype == torch.float32 and norm_weight.numel() == k
            else:
                assert a.dtype == torch.bfloat16
            status = _fn("gemv_cluster", "dllm_gemv_cluster")(
                c.data_ptr(), a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps),
                w.data_ptr(), m, n, k, epilogue, int(cluster), *_prefetch_of(w), _stream())
        elif streaming:
            if norm_weight is not None:
                assert a.dtype == torch.float32 and norm_weight.dtype == torch.float32 and norm_weight.numel() == k
            else:
                assert a.dtype == torch.bfloat16
            status = _fn("gemv", "dllm_gemv_bf16")(
                c.data_ptr(), a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps),
                w.data_ptr(), m, n, k, epilogue, *_prefetch_of(w), _stream())
        elif kernel == 1:
            assert a.dtype == torch.bfloat16 and norm_weight is None
            status = _fn("gemm_bf16", "dllm_gemm_bf16")(c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue,
                                                        _stream())
        else:
            assert a.dtype == torch.bfloat16 and norm_weight is None
            status = _fn("gemm_tcgen05", "dllm_gemm_tcgen05")(
                c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue, tile_n, _status_word().data_ptr(),
                _stream())
    else:
        raise KernelError(f"gemm: dtype {w.dtype} is not supported")
    _check(status, (lambda: f"gemm {_EPILOGUE_NAMES[epilogue]} M={m} N={n} K={k}"
                    + (" +norm" if norm_weight is not None else "")) if trace is not None else "gemm", detail)


MLP_DECODE_MAX_ROWS = 16
FUSED_FEED_FORWARD = False
"""Whether decode steps take the one-kernel feed-forward (`mlp_decode`) where it fits. Off: measured on a B200 at the
SmolLM2-135M layer sizes with 8 tokens, as one link of a chain of dependent launches in a CUDA graph, the fused kernel
takes 7.4 us against 4.7 us for the two kernels it replaces. Its gate/up part costs 2.65 us, the exchange inside the
cluster 0.6 us, the down product 0.8 us, and the fixed-order sum of the clusters' partial results through global
memory (fence, ticket, fence, loads) 3.3 us: more than the second launch it saves. The kernel stays as a tested
option."""


def mlp_decode_supported(rows: int, hidden: int, intermediate: int) -> bool:
    """Whether the feed-forward of a decode step may run as one kernel: up to 16 tokens and an intermediate size
    that slices of 16 tile."""
    return 0 < rows <= MLP_DECODE_MAX_ROWS and intermediate % 16 == 0 and hidden % 8 == 0


def mlp_decode_scratch(rows: int, hidden: int, intermediate: int) -> int:
    """Floats of scratch `mlp_decode` needs: a partial result [8 or 16 tokens, hidden] per cluster of blocks."""
    cluster = next(c for c in (8, 4, 2, 1) if intermediate % (16 * c) == 0)
    return (intermediate // (16 * cluster)) * (8 if rows <= 8 else 16) * hidden


def mlp_decode(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w_gate_up: torch.Tensor, w_down: torch.Tensor,
               scratch: torch.Tensor, tickets: torch.Tensor) -> None:
    """x (float32 residual [rows, hidden]) += down(silu(gate(h)) * up(h)), h = RMSNorm(x) rounded to bfloat16, in one
    kernel. w_gate_up [2 * intermediate, hidden] interleaves gate and up rows; w_down is [hidden, intermediate].
    `scratch`: `mlp_decode_scratch` floats; `tickets`: 8 int32 zeros (the kernel leaves them zero)."""
    _cuda(x, norm_weight, w_gate_up, w_down, scratch, tickets)
    rows, hidden = x.shape
    intermediate = w_down.shape[1]
    assert x.dtype == torch.float32 and norm_weight.dtype == torch.float32 and norm_weight.numel() == hidden
    assert w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
    assert tuple(w_gate_up.shape) == (2 * intermediate, hidden) and w_down.shape[0] == hidden
    assert scratch.dtype == torch.float32 and scratch.numel() >= mlp_decode_scratch(rows, hidden, intermediate)
    assert tickets.dtype == torch.int32 and tickets.numel() >= 8
    _check(_fn("mlp_decode", "dllm_mlp_decode")(
        x.data_ptr(), norm_weight.data_ptr(), float(eps), w_gate_up.data_ptr(), w_down.data_ptr(), rows, hidden,
        intermediate, scratch.data_ptr(), tickets.data_ptr(), *_prefetch_of(w_gate_up), *_prefetch_of(w_down),
        _stream()), "mlp_decode",
        lambda: f"rows={rows} (at most 16), hidden={hidden} (multiple of 8), intermediate={intermediate} (multiple of 16)")


EPI_ARGMAX = 9
ARGMAX_MAX_ROWS = 16


def head_argmax_supported(rows: int, w: torch.Tensor) -> bool:
    """Whether the greedy choice can be made inside the head product: bfloat16 weights and a step small enough for
    the weight-streaming kernel (up to 16 rows)."""
    return w.dtype == torch.bfloat16 and 0 < rows <= ARGMAX_MAX_ROWS and w.shape[1] % 8 == 0


def head_argmax_scratch(rows: int, outputs: int) -> int:
    """Floats of scratch: a (value, feature) candidate per token and tile of 16 output features."""
    return 2 * rows * (-(-outputs // 16))


def head_argmax(out_tokens: torch.Tensor, a: torch.Tensor, w: torch.Tensor, scratch: torch.Tensor,
                norm_weight: torch.Tensor | None = None, eps: float = 0.0) -> None:
    """out_tokens[r] = the index of the largest of a[r] @ w^T (the lowest index on ties; 0 if no value is above
    -inf), without the logits ever being stored: the product's tiles leave one candidate each, a second small
    kernel picks the winner. With `norm_weight`, `a` is the float32 residual stream, RMS-normed on the way in."""
    _cuda(out_tokens, a, w, scratch, norm_weight)
    m, k = a.shape
    n = w.shape[0]
    assert head_argmax_supported(m, w) and w.shape[1] == k and out_tokens.dtype == torch.int32
    assert scratch.dtype == torch.float32 and scratch.numel() >= head_argmax_scratch(m, n)
    assert a.dtype == (torch.float32 if norm_weight is not None else torch.bfloat16)
    _check(_fn("gemv", "dllm_gemv_bf16")(
        scratch.data_ptr(), a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps),
        w.data_ptr(), m, n, k, EPI_ARGMAX, *_prefetch_of(w), _stream()), "head_argmax product",
        lambda: f"M={m} N={n} K={k}")
    _check(_fn("gemv", "dllm_argmax_candidates")(out_tokens.data_ptr(), scratch.data_ptr(), m, -(-n // 16),
                                                 _stream()), "head_argmax choice")


def cast_ssq(copy: torch.Tensor, ssq: torch.Tensor, x: torch.Tensor) -> None:
    """copy = bfloat16(x) and ssq[r] = sum of x[r]^2: what a norm folded around the next tile product needs of rows
    that no product's epilogue has written (a step's first rows)."""
    _cuda(copy, ssq, x)
    rows, hidden = x.shape
    assert x.dtype == torch.float32 and copy.dtype == torch.bfloat16 and tuple(copy.shape) == (rows, hidden)
    assert ssq.dtype == torch.float32 and ssq.numel() >= rows
    _check(_fn("elementwise", "dllm_cast_ssq")(copy.data_ptr(), ssq.data_ptr(), x.data_ptr(), rows, hidden, _stream()),
           "cast_ssq", lambda: f"hidden={hidden} must be a multiple of 4")


def gemm_normed(c: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int, ssq: torch.Tensor, parts: int,
                eps: float) -> None:
    """c = epilogue((a @ w^T) * 1 / sqrt(sum(ssq[:parts, row]) / K + eps)): the tile product with an RMSNorm folded
    around it. `a` is the bfloat16 copy of the un-normed rows, `w` carries the norm's weight in its columns;
    epilogues EPI_STORE_F32, EPI_STORE_T and EPI_SWIGLU."""
    _cuda(c, a, w, ssq)
    m, k = a.shape
    n = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ssq.dtype == torch.float32
    assert ssq.numel() >= m * parts
    _check(_fn("gemm_tcgen05", "dllm_gemm_tcgen05_normed")(
        c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue, ssq.data_ptr(), int(parts), float(eps),
        _status_word().data_ptr(), _stream()), "gemm_normed", lambda: f"M={m} N={n} K={k}")


def gemm_residual_norm(x: torch.Tensor, copy: torch.Tensor, ssq: torch.Tensor, a: torch.Tensor,
                       w: torch.Tensor) -> int:
    """x (float32) += a @ w^T; copy = bfloat16(new x); ssq[tile, row] = the sum of the squares of the new values of
    the row in each half tile of columns. Returns the number of parts (the reader's `parts`). N a multiple of 16."""
    _cuda(x, copy, ssq, a, w)
    m, k = a.shape
    n = w.shape[0]
    assert x.dtype == torch.float32 and tuple(x.shape) == (m, n) and copy.dtype == torch.bfloat16
    assert tuple(copy.shape) == (m, n) and ssq.dtype == torch.float32 and ssq.numel() >= m * (-(-n // 16))
    parts = c_int(0)
    _check(_fn("gemm_tcgen05", "dllm_gemm_tcgen05_residual_norm")(
        x.data_ptr(), copy.data_ptr(), ssq.data_ptr(), ctypes.addressof(parts), a.data_ptr(), w.data_ptr(), m, n, k,
        _status_word().data_ptr(), _stream()), "gemm_residual_norm", lambda: f"M={m} N={n} (multiple of 16) K={k}")
    return parts.value


def gemm_qkv_rope_supported(cache, rotary_dim: int, has_table: bool) -> bool:
    """Whether the tile kernel can end in the rotation and cache write: one head per tile, full rotation."""
    return cache.dtype == torch.bfloat16 and cache.head_dim in (32, 64, 128) and \
        (not has_table or rotary_dim == cache.head_dim)


_tables_by_pair: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def table_by_pair(table: torch.Tensor) -> torch.Tensor:
    """The rotary table [positions, pairs, (cos, sin)] laid out pair by pair, [pairs, positions, (cos, sin)], as the
    tile product reads it (a warp's tokens, at consecutive positions, then read consecutive bytes). Made once per
    table and kept with it."""
    found = _tables_by_pair.get(table.data_ptr())
    if found is None or found[0] is not table:
        if len(_tables_by_pair) > 64:
            _tables_by_pair.clear()
        found = _tables_by_pair[table.data_ptr()] = (table, table.transpose(0, 1).contiguous())
    return found[1]


def gemm_qkv_rope(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cache, table: torch.Tensor | None,
                  rotary_dim: int, heads: int, batch, write_cache: bool = True) -> None:
    """The q/k/v projection of a prefill-sized step in the tcgen05 tile kernel, ending in the rotation of q and k and
    the write of k and v into the paged cache (no float32 q/k/v in memory, no separate rotation kernel)."""
    _cuda(a, w, q_out, table)
    m, k = batch.n_tokens, a.shape[1]
    assert gemm_qkv_rope_supported(cache, rotary_dim, table is not None)
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16
    assert w.shape == ((heads + 2 * cache.kv_heads) * cache.head_dim, k) and a.shape[0] >= m
    if table is not None:
        assert table.dtype == torch.float32 and table.shape[0] > batch.max_position, "position beyond the table"
        assert table.shape[1] == rotary_dim // 2 and table.shape[2] == 2
    by_pair = table_by_pair(table) if table is not None else None  # (the layout this kernel reads)
    _check(_fn("gemm_tcgen05", "dllm_gemm_tcgen05_qkv_rope")(
        a.data_ptr(), w.data_ptr(), m, k, q_out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(),
        cache.max_pages, cache.page_size, heads, cache.kv_heads, cache.head_dim,
        by_pair.data_ptr() if by_pair is not None else None, rotary_dim if table is not None else 0,
        table.shape[0] if table is not None else 0,
        batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(), 1 if write_cache else 0,
        _status_word().data_ptr(), _stream()), "gemm_qkv_rope", lambda: f"M={m} K={k} head_dim={cache.head_dim}")


def gemv_qkv_rope(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cache, table: torch.Tensor | None,
                  rotary_dim: int, heads: int, batch, write_cache: bool = True,
                  norm_weight: torch.Tensor | None = None, eps: float = 0.0, prefetch_window: int = -1,
                  kernel: int = 0, cluster: int = 0) -> None:
    """The q/k/v projection of at most 64 tokens in one kernel (bfloat16): optional RMSNorm of the float32 residual
    in front, rotation of q and k, q to q_out, k and v into the paged cache. With `prefetch_window` >= 0 the kernel
    also asks L2 for the cached keys and values of the tokens' sequences (0: all of them, w: the last w), which the
    attention kernel behind it reads. `kernel`: 0 chooses, 2 forces a block per 16 rows of W, 6 the reduction split
    over a cluster (`cluster` blocks, 0 chooses)."""
    _cuda(a, w, q_out, table, norm_weight)
    m, k = batch.n_tokens, a.shape[1]
    assert w.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16
    assert w.shape == ((heads + 2 * cache.kv_heads) * cache.head_dim, k) and a.shape[0] >= m
    assert a.dtype == (torch.float32 if norm_weight is not None else torch.bfloat16)
    if table is not None:
        assert table.dtype == torch.float32 and table.shape[0] > batch.max_position, "position beyond the table"
        assert table.shape[1] == rotary_dim // 2 and table.shape[2] == 2
    if kernel == 6 or (kernel == 0 and splits_over_clusters(m, w.shape[0], k)):
        _check(_fn("gemv_cluster", "dllm_gemv_cluster_qkv_rope")(
            a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps), w.data_ptr(), m, k,
            q_out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads,
            cache.kv_heads, cache.head_dim, table.data_ptr() if table is not None else None,
            rotary_dim if table is not None else 0, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
            batch.slots.data_ptr(), 1 if write_cache else 0, int(prefetch_window), int(cluster), *_prefetch_of(w),
            _stream()),
            "gemv_cluster_qkv_rope",
            lambda: f"M={m} (at most 64), K={k} (multiple of 8), head_dim and rotary_dim multiples of 16")
        return
    _check(_fn("gemv", "dllm_gemv_qkv_rope")(
        a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps), w.data_ptr(), m, k,
        q_out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads,
        cache.kv_heads, cache.head_dim, table.data_ptr() if table is not None else None,
        rotary_dim if table is not None else 0, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
        batch.slots.data_ptr(), 1 if write_cache else 0, int(prefetch_window), *_prefetch_of(w), _stream()),
        "gemv_qkv_rope", lambda: f"M={m} (at most 64), K={k} (multiple of 8), head_dim and rotary_dim multiples of 16")


def rope_cache_write(qkv: torch.Tensor, q_out: torch.Tensor, cache, table: torch.Tensor | None, rotary_dim: int,
                     heads: int, batch, write_cache: bool = True) -> None:
    """Rotates queries and keys of qkv (float32 [tokens, (heads + 2 kv_heads) * head_dim]) by the table's angle for
    each token's position; queries go to q_out, keys and values into the token's place in the paged cache. A qkv
    of three dimensions is partial results [parts, tokens, ...] (`gemm_parts`), summed in order on the way in."""
    _cuda(qkv, q_out, table)
    tokens = batch.n_tokens
    assert qkv.dtype == torch.float32 and q_out.dtype == cache.dtype
    n_parts, part_stride = 1, 0
    if qkv.dim() == 3:
        assert qkv.is_contiguous()
        n_parts, part_stride = qkv.shape[0], qkv.shape[1] * qkv.shape[2]
        qkv = qkv[0]
    assert qkv.shape[0] >= tokens and qkv.shape[1] == (heads + 2 * cache.kv_heads) * cache.head_dim
    if table is not None:
        assert table.dtype == torch.float32 and table.shape[0] > batch.max_position, "position beyond the table"
        assert table.shape[1] == rotary_dim // 2 and table.shape[2] == 2
    _check(_fn("elementwise", "dllm_rope_cache_write")(
        qkv.data_ptr(), q_out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages,
        cache.page_size, heads, cache.kv_heads, cache.head_dim, table.data_ptr() if table is not None else None,
        rotary_dim if table is not None else 0, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
        batch.slots.data_ptr(), tokens, 1 if write_cache else 0, _code(cache.dtype), n_parts, part_stride,
        _stream()), "rope_cache_write")


def attention_general(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int,
                      batch) -> None:
    """Causal attention of every token in the batch over its own sequence's cache (keys up to its position, the
    last `window` of them if window > 0). out, q: [tokens, heads * head_dim] in the cache's dtype."""
    _cuda(out, q)
    assert q.dtype == cache.dtype and out.dtype == cache.dtype
    _check(_fn("attention", "dllm_attention_general")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
        batch.slots.data_ptr(), batch.n_tokens, float(scale), int(window or 0), _code(cache.dtype), _stream()),
        "attention", lambda: f"head_dim={cache.head_dim} must be a multiple of 8, at most 256")


def attention_blocks_supported(cache) -> bool:
    return cache.page_size == 64 and cache.head_dim % 8 == 0 and cache.head_dim <= 256


def attention_blocks(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int, batch) -> None:
    """`attention_general` blockwise: the keys and values of a kv head go through shared memory page by page and
    serve every (token, head) pair of a run of tokens at once. Without a window a pair's result has the same bits
    as `attention_general` gives; with one the same formula is rounded in other places. The float32 path's attention,
    for whole prompts and single tokens alike."""
    _cuda(out, q)
    assert q.dtype == cache.dtype and out.dtype == cache.dtype and attention_blocks_supported(cache)
    _check(_fn("attention", "dllm_attention_blocks")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
        batch.slots.data_ptr(), batch.n_tokens, int(batch.max_new), float(scale), int(window or 0),
        _code(cache.dtype), _stream()), "attention_blocks",
        lambda: f"head_dim={cache.head_dim} must be a multiple of 8, at most 256; pages of 64")


def add_residual(residual: torch.Tensor, update: torch.Tensor) -> None:
    """residual (float32) += update, summed in float32."""
    _cuda(residual, update)
    assert residual.dtype == torch.float32 and residual.numel() == update.numel()
    _check(_fn("elementwise", "dllm_add_residual")(residual.data_ptr(), update.data_ptr(), residual.numel(),
                                                   _code(update.dtype), _stream()), "add_residual")


def sample_scratch(rows: int, vocab: int) -> int:
    """Floats of scratch that temperature sampling needs: a float and a double per logit."""
    return 3 * rows * vocab + 2


def sample(out_tokens: torch.Tensor, logits: torch.Tensor, scratch: torch.Tensor | None, rng: torch.Tensor | None,
           rng_rows: torch.Tensor | None, temperature: float, top_k: int = 0, top_p: float = 1.0,
           min_p: float = 0.0) -> None:
    """One token per row of logits (float32 [rows, vocab]); see csrc/sampling.cu for the rule."""
    _cuda(out_tokens, logits, scratch, rng, rng_rows)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out_tokens.dtype == torch.int32 and out_tokens.numel() >= rows
    if temperature > 0:
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= sample_scratch(rows, vocab)
        assert scratch.data_ptr() % 8 == 0
        assert rng is not None and rng.dtype == torch.int64 and rng_rows.dtype == torch.int32
    _check(_fn("sampling", "dllm_sample")(
        out_tokens.data_ptr(), logits.data_ptr(), logits.stride(0), rows, vocab,
        scratch.data_ptr() if scratch is not None else None, rng.data_ptr() if rng is not None else None,
        rng_rows.data_ptr() if rng_rows is not None else None, float(temperature), int(top_k), float(top_p),
        float(min_p), _stream()), "sample")


def seed_rng(rng: torch.Tensor, rows: torch.Tensor, seeds: torch.Tensor) -> None:
    """rng[rows[i]] = xoshiro256** state seeded with seeds[i] (int64 bit patterns of unsigned 64-bit seeds)."""
    _cuda(rng, rows, seeds)
    assert rng.dtype == torch.int64 and rows.dtype == torch.int32 and seeds.dtype == torch.int64
    _check(_fn("sampling", "dllm_seed_rng")(rng.data_ptr(), rows.data_ptr(), seeds.data_ptr(), rows.numel(),
                                            _stream()), "seed_rng")


def decode_advance(tokens: torch.Tensor, tok_pos: torch.Tensor, start: torch.Tensor, chosen: torch.Tensor,
                   history: torch.Tensor, counter: torch.Tensor, batch: int) -> None:
    """tokens = chosen; positions and cached lengths + 1; history[counter] = chosen; counter + 1 (all int32)."""
    _cuda(tokens, tok_pos, start, chosen, history, counter)
    _check(_fn("elementwise", "dllm_decode_advance")(
        tokens.data_ptr(), tok_pos.data_ptr(), start.data_ptr(), chosen.data_ptr(), history.data_ptr(),
        counter.data_ptr(), batch, history.numel() // batch, _stream()), "decode_advance")


def mask_tokens(logits: torch.Tensor, ids: torch.Tensor, produced: torch.Tensor, steps: torch.Tensor | None,
                min_tokens: int) -> None:
    """logits[:, ids] = -inf in every row while produced[0] + steps[0] < min_tokens (float32 logits [rows, vocab];
    ids, produced and steps int32 on the device; `steps` may be None). Ids outside the vocabulary are skipped."""
    _cuda(logits, ids, produced)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    assert ids.dtype == torch.int32 and produced.dtype == torch.int32
    assert steps is None or (steps.is_cuda and steps.dtype == torch.int32)
    _check(_fn("elementwise", "dllm_mask_tokens")(
        logits.data_ptr(), logits.shape[0], logits.shape[1], ids.data_ptr(), ids.numel(), produced.data_ptr(),
        steps.data_ptr() if steps is not None else None, int(min_tokens), _stream()), "mask_tokens")


def attention_decode_scratch(sequences: int, heads: int, head_dim: int, chunk: int, max_context: int) -> int:
    """Floats of scratch `attention_decode` needs."""
    return sequences * heads * (-(-max_context // chunk)) * (head_dim + 2)


def attention_decode(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int, batch,
                     chunk: int, scratch: torch.Tensor, tickets: torch.Tensor) -> None:
    """Attention for a batch in which every sequence brings one token (bfloat16): keys are split into chunks of
    `chunk` positions across blocks, every block serves all query heads of its kv head, partial results are combined
    in chunk order by the block that finishes last. Serves any length up to batch.max_context. `tickets`: int32
    zeros, one per (sequence, kv head); the kernel leaves them zero."""
    _cuda(out, q, scratch, tickets)
    assert tickets.dtype == torch.int32 and tickets.numel() >= batch.n_seqs * cache.kv_heads
    assert cache.dtype == torch.bfloat16 and q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert batch.n_tokens == batch.n_seqs and scratch.dtype == torch.float32
    assert scratch.numel() >= attention_decode_scratch(batch.n_seqs, heads, cache.head_dim, chunk, batch.max_context)
    _check(_fn("attention_decode", "dllm_attention_decode")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tok_pos.data_ptr(), batch.slots.data_ptr(), batch.n_seqs,
        float(scale), int(window or 0), int(chunk), int(batch.max_context), scratch.data_ptr(),
        tickets.data_ptr(), _stream()),
        "attention_decode", lambda: f"head_dim={cache.head_dim} must be a multiple of 8, at most 256")


def attention_prefill_supported(cache) -> bool:
    return cache.dtype == torch.bfloat16 and cache.head_dim % 16 == 0 and cache.head_dim <= 128 \
        and cache.page_size == 64


def attention_prefill(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int,
                      batch) -> None:
    """Blockwise causal attention of the batch's new tokens over their sequences' caches on the tensor cores
    (bfloat16, head_dim a multiple of 16 up to 128, pages of 64 positions)."""
    _cuda(out, q)
    assert attention_prefill_supported(cache) and q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    _check(_fn("attention_prefill", "dllm_attention_prefill")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tile_seq.data_ptr(), batch.tile_first.data_ptr(),
        batch.cu_seqlens.data_ptr(), batch.start.data_ptr(), batch.slots.data_ptr(), batch.n_tiles, float(scale),
        int(window or 0), _stream()), "attention_prefill",
        lambda: f"head_dim={cache.head_dim} must be a multiple of 16, at most 128; pages of 64")


def attention_prefill_tcgen05_supported(cache) -> bool:
    return cache.dtype == torch.bfloat16 and cache.head_dim in (64, 128) and cache.page_size == 64


def attention_prefill_tcgen05(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int,
                              batch) -> None:
    """Blockwise causal attention of the batch's new tokens over their sequences' caches on the 5th-generation
    tensor cores (bfloat16, head_dim 64 or 128, pages of 64 positions): tiles of 128 queries, scores and outputs in tensor
    memory, pages of keys and values by TMA."""
    _cuda(out, q)
    assert attention_prefill_tcgen05_supported(cache) and q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    _check(_fn("attention_prefill_tcgen05", "dllm_attention_prefill_tcgen05")(
        out.data_ptr(), q.data_ptr(), q.shape[0], cache.base_ptr, cache.storage.shape[0],
        cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads, cache.kv_heads, cache.head_dim,
        batch.tile_seq.data_ptr(), batch.tile_first.data_ptr(), batch.cu_seqlens.data_ptr(), batch.start.data_ptr(),
        batch.slots.data_ptr(), batch.n_tiles, float(scale), int(window or 0), _status_word().data_ptr(),
        _stream()), "attention_prefill_tcgen05", lambda: f"head_dim={cache.head_dim} must be 64 or 128; pages of 64")


def attention_decode_cluster_supported(cache) -> bool:
    return cache.dtype == torch.bfloat16 and cache.head_dim % 16 == 0 and cache.head_dim <= 128 \
        and cache.page_size == 64


DECODE_CLUSTER_SHAPES = 5
"""Launch shapes of the cluster decode kernel: 0..3 are 1, 2, 4, 8 blocks per (sequence, kv head) pair, of four warps
(two when head_dim is above 64); 4 is eight blocks of four warps at any head_dim."""


def attention_decode_cluster(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int,
                             batch, shape: int = -1) -> None:
    """Attention for a batch in which every sequence brings one token (bfloat16, head_dim a multiple of 16 up to
    128): the blocks of a cluster split the keys of a (sequence, kv head) pair and combine through distributed
    shared memory; no scratch, and a launch shape that does not depend on the context length. shape -1 lets the
    kernel choose by the number of pairs; 0..4 name one of DECODE_CLUSTER_SHAPES."""
    _cuda(out, q)
    assert attention_decode_cluster_supported(cache) and q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert batch.n_tokens == batch.n_seqs
    _check(_fn("attention_decode_cluster", "dllm_attention_decode_cluster")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tok_pos.data_ptr(), batch.slots.data_ptr(), batch.n_seqs,
        float(scale), int(window or 0), int(shape), _stream()), "attention_decode_cluster",
        lambda: f"head_dim={cache.head_dim} must be a multiple of 16, at most 128; pages of 64")
