"""Thin Python layer over the kernel libraries (ctypes, raw device pointers).

Every function here launches hand-written sm_100a kernels on the current torch
stream and returns at once.  There is no eager or CPU fallback: tensors must be
CUDA tensors, and when a library cannot be built or loaded the call raises.
The reference pairs every kernel with an eager fallback inside the same
function (python/lyapunov_engine/ops.py:12-216); here the plain twins live in
the tests only.

Matrix products in bfloat16 go to the library (cuBLAS through torch), as the
reference's do (nn.Linear, python/lyapunov_engine/models/llama.py:45-48,112-117,177);
32-bit products use the package's own FP32 kernel, never a tensor-core mode.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a block table entry outside the page pool",
               4: "a position outside the rotary table", 8: "a bounded wait inside a kernel ran out"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _ptr(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle.  (torch.cuda.current_stream() without a
    device costs tens of microseconds, several times per decode step.)"""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("lyapunov_engine_b200 kernels run on CUDA tensors only (there is no CPU path)")


_core = None
_attention: dict[int, ctypes.CDLL] = {}

_CORE_SIGNATURES = {
    "le_embed": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "le_zero_fresh_state": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "le_zero_fresh_states": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "le_sm_count": [],
    "le_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "le_convert": [c_void_p, c_int, c_void_p, c_int, c_int64, c_void_p],
    "le_rmsnorm": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_float, c_int,
                   c_int, c_int, c_void_p, c_void_p],
    "le_rmsnorm_taps_applies": [c_int, c_int],
    "le_rmsnorm_taps": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_float, c_int, c_int, c_int,
                        c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p],
    "le_embed_sinusoid": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "le_glu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
    "le_head_gate": [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p],
    "le_short_conv": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                      c_int, c_int, c_int, c_void_p],
    "le_short_conv_general": [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "le_glu_bias": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p],
    "le_gated_delta_lanes": [c_int],
    "le_gated_delta_scratch": [c_int, c_int],
    "le_gated_delta_scan": [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_int64, c_int, c_int, c_int,
                            c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_float, c_float, c_void_p, c_void_p],
    "le_head_norm_gate": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_float, c_int, c_int,
                          c_int, c_int, c_int, c_float, c_void_p],
    "le_rope_norm_store": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_int,
                           c_void_p, c_void_p],
    "le_latent_rope_store": [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p,
                             c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_int, c_void_p, c_void_p],
    "le_rmsnorm_pair": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_float, c_void_p,
                        c_void_p, c_float, c_void_p, c_int, c_int, c_void_p],
    "le_residual_add": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int64, c_void_p, c_int, c_int, c_int64,
                        c_void_p, c_int, c_int, c_void_p],
    "le_gate_rows": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                     c_void_p],
    "le_stream_entry": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "le_sigmoid_gate": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_float, c_void_p],
    "le_ssm_scan": [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p,
                    c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                    c_int, c_int, c_int, c_float, c_void_p],
    "le_mlstm_rows": [c_int, c_int],
    "le_mlstm_scan": [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                      c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
    "le_rope_qknorm_store": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_int,
                             c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_void_p, c_void_p],
    "le_kv_store": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "le_latent_norm_store": [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "le_latent_prepare": [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p,
                          c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "le_gemm_heads": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                      c_void_p],
    "le_gemm_tc_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int,
                        c_int, c_float, c_float, c_void_p, c_void_p],
    "le_gemm_skinny_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int,
                            c_int64, c_int, c_int, c_float, c_float, c_void_p],
    "le_gemm_skinny_bias_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int,
                                 c_int64, c_int, c_int, c_float, c_float, c_void_p, c_void_p],
    "le_gemm_tc_bias_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int,
                             c_int, c_float, c_float, c_void_p, c_void_p, c_void_p],
    "le_gemm_skinny_rotary_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_void_p, c_void_p],
    "le_rope_kv_write": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "le_gemm_simt": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                     c_void_p],
    "le_stream_norm": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p],
    "le_stream_sum": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "le_rope_pairs_store": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_void_p, c_void_p],
    "le_maps_combine": [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                        c_float, c_void_p],
    "le_softcap": [c_void_p, c_int64, c_float, c_void_p],
    "le_moe_tile_rows": [c_int],
    "le_moe_route": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                     c_int, c_int, c_int, c_int, c_void_p],
    "le_moe_group": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_void_p, c_void_p],
    "le_moe_gather": [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "le_moe_combine_sorted": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_void_p],
    "le_gemm_tc_grouped_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int,
                                c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p, c_void_p],
    "le_moe_grouped": [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int, c_void_p, c_int,
                       c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                       c_float, c_float, c_void_p],
    "le_moe_combine": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "le_argmax": [c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p],
    "le_sample": [c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_void_p],
}
_ATTENTION_SIGNATURES = {
    "le_attention_generic": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_float, c_void_p, c_int, c_float, c_void_p, c_void_p],
}


def _declare(lib, signatures):
    for name, args in signatures.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = c_int
    lib.le_last_error_fn = getattr(lib, "le_last_error", None)
    if lib.le_last_error_fn is not None:
        lib.le_last_error_fn.restype = ctypes.c_char_p


def core():
    global _core
    if _core is None:
        lib = build.load_core()
        _declare(lib, _CORE_SIGNATURES)
        _core = lib
    return _core


def attention_lib(head_dim: int):
    lib = _attention.get(head_dim)
    if lib is None:
        lib = build.load_attention(head_dim)
        _declare(lib, _ATTENTION_SIGNATURES)
        _declare(lib, _EXTRA_ATTENTION_SIGNATURES)
        lib.le_attention_mma_available.restype = c_int
        lib.le_attention_mma_available.argtypes = []
        lib.le_attention_tc_available.restype = c_int
        lib.le_attention_tc_available.argtypes = [c_int]
        _attention[head_dim] = lib
    return lib


_EXTRA_ATTENTION_SIGNATURES: dict[str, list] = {
    "le_attention_prefill_bf16": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_void_p, c_int, c_float, c_void_p, c_void_p],
    "le_attention_prefill_tc_bf16": [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                     c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_float, c_void_p, c_void_p, c_void_p],
    "le_attention_decode_bf16": [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                 c_int, c_void_p, c_void_p],
    "le_attention_decode_bf16_form": [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                      c_void_p, c_int, c_float, c_int, c_int, c_void_p, c_void_p],
}


# Launch counters (own kernels, library products) for the benchmark's report.
counters = {"own_kernels": 0, "library_products": 0}


def _check(code: int, name: str, lib=None, launches: int = 1):
    counters["own_kernels"] += launches
    if code != 0:
        lib = lib or core()
        detail = ""
        fn = getattr(lib, "le_last_error_fn", None) or getattr(core(), "le_last_error_fn", None)
        if fn is not None:
            detail = (fn() or b"").decode(errors="replace")
        raise KernelError(f"{name} failed ({code}): {detail}")


def new_status(device) -> torch.Tensor:
    """The status word kernels set instead of faulting on bad indices."""
    return torch.zeros(4, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor) -> None:
    """Reads the status word (this waits for the device) and raises if a kernel
    met an index it refused to follow."""
    word = int(status[0].item())
    if word:
        status.zero_()
        what = "; ".join(text for bit, text in STATUS_BITS.items() if word & bit)
        raise KernelError(f"a kernel refused bad input: {what}")


# --------------------------------------------------------------------------
def embed(out_resid: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor, scale: float = 1.0) -> None:
    """out_resid[t] (float32) = table[ids[t]] * scale."""
    _need_cuda(out_resid, table, ids)
    T, H = out_resid.shape
    assert out_resid.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == H
    assert out_resid.is_contiguous() and table.is_contiguous()
    _check(core().le_embed(_ptr(out_resid), _ptr(table), dtype_code(table.dtype), _ptr(ids), T, H, table.shape[0],
                           float(scale), _ptr(status), _stream()), "le_embed")


def zero_fresh_state(state: torch.Tensor, state_slots: torch.Tensor, ctx_before: torch.Tensor, num_requests: int) -> None:
    """Zeroes row ``state_slots[b]`` of ``state`` [rows, ...] for every request b
    of the step that has nothing in the cache yet (``ctx_before[b]`` == 0)."""
    _need_cuda(state, state_slots, ctx_before)
    assert state.is_contiguous() and state_slots.dtype == torch.int32 and ctx_before.dtype == torch.int32
    row_bytes = state[0].numel() * state.element_size()
    _check(core().le_zero_fresh_state(_ptr(state), row_bytes, state.shape[0], _ptr(state_slots), _ptr(ctx_before),
                                      num_requests, _stream()), "le_zero_fresh_state")


def state_table(states: list) -> torch.Tensor | None:
    """What zero_fresh_states() takes: per state buffer its address and the
    4-byte words of one of its rows, as int64 pairs on the device."""
    if not states:
        return None
    rows = states[0].shape[0]
    flat = []
    for s in states:
        _need_cuda(s)
        assert s.is_contiguous() and s.shape[0] == rows and (s[0].numel() * s.element_size()) % 4 == 0
        flat += [s.data_ptr(), s[0].numel() * s.element_size() // 4]
    return torch.tensor(flat, dtype=torch.int64, device=states[0].device)


def zero_fresh_states(table: torch.Tensor, num_buffers: int, num_rows: int, state_slots: torch.Tensor,
                      ctx_before: torch.Tensor, num_requests: int) -> None:
    """zero_fresh_state() for all of a model's state buffers in one launch."""
    _check(core().le_zero_fresh_states(_ptr(table), num_buffers, num_rows, _ptr(state_slots), _ptr(ctx_before),
                                       num_requests, _stream()), "le_zero_fresh_states")


_sm_count: dict[int, int] = {}


def sm_count() -> int:
    """Multiprocessors of the current device (148 on a B200)."""
    dev = torch.cuda.current_device()
    n = _sm_count.get(dev)
    if n is None:
        n = int(core().le_sm_count())
        if n <= 0:
            raise KernelError("the device's multiprocessor count could not be read")
        _sm_count[dev] = n
    return n


def swiglu(out: torch.Tensor, gate_up: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need_cuda(out, gate_up)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and out.is_contiguous() and gate_up.is_contiguous()
    assert out.dtype == gate_up.dtype
    _check(core().le_swiglu(_ptr(out), _ptr(gate_up), dtype_code(out.dtype), T, I, _stream()), "le_swiglu")


GLU_SILU, GLU_CLAMPED, GLU_RELU = 0, 1, 2


def glu(out: torch.Tensor, gate_up: torch.Tensor, kind: int = GLU_SILU, alpha: float = 1.0, limit: float = 0.0,
        bias=None) -> None:
    """out[t, i] from gate g = gate_up[t, i] and u = gate_up[t, I + i], each
    plus its entry of ``bias`` (float32 [2 I]) where one is given.
    GLU_SILU: silu(g) * u.  GLU_CLAMPED: g' = min(g, limit), u' = clamp(u,
    -limit, limit); g' * sigmoid(alpha * g') * (u' + 1).  GLU_RELU: max(g, 0) * u."""
    _need_cuda(out, gate_up, bias)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and out.is_contiguous() and gate_up.is_contiguous() and out.dtype == gate_up.dtype
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == 2 * I)
    _check(core().le_glu_bias(_ptr(out), _ptr(gate_up), dtype_code(out.dtype), T, I, int(kind), float(alpha), float(limit),
                              _ptr(bias), _stream()), "le_glu_bias")


def embed_sinusoid(out_resid, table, ids, positions, rates, status) -> None:
    """out_resid[t] (float32) = table[ids[t]] + s(positions[t]), where entry 2i of
    s(p) is sin(p * rates[i]) and entry 2i + 1 is cos(p * rates[i])."""
    _need_cuda(out_resid, table, ids, positions, rates)
    T, H = out_resid.shape
    assert out_resid.dtype == torch.float32 and ids.dtype == torch.int32 and positions.dtype == torch.int32
    assert table.shape[1] == H and out_resid.is_contiguous() and table.is_contiguous()
    assert rates.dtype == torch.float32 and rates.is_contiguous() and rates.numel() >= (H + 1) // 2
    _check(core().le_embed_sinusoid(_ptr(out_resid), _ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(positions),
                                    _ptr(rates), T, H, table.shape[0], _ptr(status), _stream()), "le_embed_sinusoid")


def head_gate(x: torch.Tensor, gate: torch.Tensor, num_heads: int, head_width: int) -> None:
    """x[t, h, :] *= sigmoid(gate[t, h]) in place; ``gate`` may be a column
    range of a wider buffer."""
    _need_cuda(x, gate)
    assert x.dtype == gate.dtype and x.stride(1) == 1 and gate.stride(1) == 1 and x.shape[1] == num_heads * head_width
    assert gate.shape == (x.shape[0], num_heads)
    _check(core().le_head_gate(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), dtype_code(x.dtype), x.shape[0],
                               num_heads, head_width, _stream()), "le_head_gate")


SHORT_CONV_TILE = 16
SHORT_CONV_MAX_TAPS = 17


def short_conv(out, h, w_taps, state, state_slots, cu_q, tile_request, tile_q0, num_tiles) -> None:
    """out = h + causal convolution of h over time per channel, continuing
    each request from its state row.  ``w_taps``: float32 [taps, channels];
    ``state``: float32 [rows, taps - 1, channels] (None when taps is 1), row
    ``state_slots[b]`` holds request b's last taps - 1 inputs and is brought up
    to date; the tiles list SHORT_CONV_TILE tokens each.  ``tile_request`` and
    ``tile_q0`` None: every request of the step brings one token (request b is
    row b), ``num_tiles`` is their number."""
    _need_cuda(out, h, w_taps, state, state_slots, cu_q)
    T, C = h.shape
    taps = w_taps.shape[0]
    assert out.shape == h.shape and out.dtype == h.dtype and out.is_contiguous() and h.is_contiguous()
    assert w_taps.dtype == torch.float32 and w_taps.is_contiguous() and w_taps.shape[1] == C
    rows = 0
    if taps > 1:
        assert state is not None and state.dtype == torch.float32 and state.is_contiguous()
        assert tuple(state.shape[1:]) == (taps - 1, C)
        rows = state.shape[0]
    _check(core().le_short_conv(_ptr(out), _ptr(h), dtype_code(h.dtype), _ptr(w_taps), _ptr(state) if taps > 1 else None,
                                rows, _ptr(state_slots), _ptr(cu_q), _ptr(tile_request), _ptr(tile_q0), num_tiles,
                                SHORT_CONV_TILE, C, taps, _stream()), "le_short_conv")


def kv_store(src, k_col, v_col, k_cache, v_cache, positions, request_of_token, block_table, num_kv_heads, head_dim,
             page_size, status) -> None:
    """Copies keys (columns k_col ..) and values (columns v_col ..) of the rows
    of ``src`` into the paged cache, unrotated."""
    _need_cuda(src, k_cache, v_cache, positions, block_table)
    assert src.stride(1) == 1 and k_cache.dtype == src.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[1:] == (num_kv_heads, page_size, head_dim) and block_table.is_contiguous()
    _check(core().le_kv_store(_ptr(src), src.stride(0), k_col, v_col, _ptr(k_cache), _ptr(v_cache), dtype_code(src.dtype),
                              _ptr(positions), _ptr(request_of_token), _ptr(block_table), block_table.shape[1],
                              src.shape[0], num_kv_heads, head_dim, page_size, k_cache.shape[0], _ptr(status), _stream()),
           "le_kv_store")


def latent_norm_store(src, col, rank, weight, eps, cache, positions, request_of_token, block_table, page_size, status) -> None:
    """Columns col .. col + rank of each row of ``src``, divided by their root
    mean square and multiplied by ``weight`` (32-bit), into the paged pool
    ``cache`` [pages, 1, page, padded rank]; the padding columns get zeros."""
    _need_cuda(src, weight, cache, positions, block_table)
    assert src.stride(1) == 1 and cache.dtype == src.dtype and cache.is_contiguous() and block_table.is_contiguous()
    assert weight.dtype == torch.float32 and weight.numel() == rank
    assert cache.shape[1] == 1 and cache.shape[2] == page_size and cache.shape[3] >= rank
    _check(core().le_latent_norm_store(_ptr(src), src.stride(0), col, rank, cache.shape[3], _ptr(weight), float(eps),
                                       _ptr(cache), dtype_code(src.dtype), _ptr(positions), _ptr(request_of_token),
                                       _ptr(block_table), block_table.shape[1], src.shape[0], page_size, cache.shape[0],
                                       _ptr(status), _stream()), "le_latent_norm_store")


LATENT_PREPARE_ROWS = 32


def latent_prepare_applies(src: torch.Tensor, head_dim: int) -> bool:
    """Whether latent_prepare() takes these rows (few of them, 16-byte pieces)."""
    vec = 16 // src.element_size()
    return (src.shape[0] <= LATENT_PREPARE_ROWS and head_dim % vec == 0 and src.stride(0) % vec == 0
            and src.data_ptr() % 16 == 0 and src.stride(1) == 1)


def latent_prepare(q_latent, src, w_into, col, rank, weight, eps, cache, positions, request_of_token, block_table,
                   page_size, status) -> None:
    """For a step of few rows, in one launch: gemm_heads(q_latent, src[:, :heads
    * head_dim], w_into) and latent_norm_store(src, col, rank, ...) (``cache``
    None: the latent is not stored)."""
    _need_cuda(q_latent, src, w_into, weight, cache, positions, block_table)
    heads, padded, head_dim = w_into.shape
    T = src.shape[0]
    assert latent_prepare_applies(src, head_dim) and w_into.is_contiguous() and w_into.dtype == src.dtype == q_latent.dtype
    assert q_latent.shape == (T, heads * padded) and q_latent.stride(1) == 1 and padded >= rank
    assert weight.dtype == torch.float32 and weight.numel() == rank and block_table.is_contiguous()
    pages = 0
    if cache is not None:
        assert cache.dtype == src.dtype and cache.is_contiguous() and tuple(cache.shape[1:]) == (1, page_size, padded)
        pages = cache.shape[0]
    _check(core().le_latent_prepare(_ptr(src), src.stride(0), T, heads, head_dim, _ptr(w_into), _ptr(q_latent),
                                    q_latent.stride(0), col, rank, padded, _ptr(weight), float(eps), _ptr(cache),
                                    dtype_code(src.dtype), _ptr(positions), _ptr(request_of_token), _ptr(block_table),
                                    block_table.shape[1], page_size, pages, _ptr(status), _stream()), "le_latent_prepare")


def gemm_heads(out, a, w, gate=None) -> None:
    """One product per head: out[t, h, :] = w[h] @ a[t, h, :] (w: [heads, N,
    K]), times sigmoid(gate[t, h]) where ``gate`` is given.  ``a``, ``out`` and
    ``gate`` may be column ranges of wider buffers (rows of any stride)."""
    _need_cuda(out, a, w, gate)
    heads, N, K = w.shape
    M = a.shape[0]
    assert a.shape[1] == heads * K and out.shape == (M, heads * N) and a.stride(1) == 1 and out.stride(1) == 1
    assert w.is_contiguous() and a.dtype == w.dtype == out.dtype
    if gate is not None:
        assert gate.shape == (M, heads) and gate.stride(1) == 1 and gate.dtype == a.dtype
    _check(core().le_gemm_heads(_ptr(out), out.stride(0), _ptr(a), a.stride(0), _ptr(w), _ptr(gate),
                                gate.stride(0) if gate is not None else 0, dtype_code(a.dtype), M, heads, N, K, _stream()),
           "le_gemm_heads")


def convert(out: torch.Tensor, src: torch.Tensor) -> None:
    _need_cuda(out, src)
    assert out.numel() == src.numel() and out.is_contiguous() and src.is_contiguous()
    _check(core().le_convert(_ptr(out), dtype_code(out.dtype), _ptr(src), dtype_code(src.dtype), out.numel(),
                             _stream()), "le_convert")


def rmsnorm(out: torch.Tensor, resid: torch.Tensor, delta, weight: torch.Tensor, eps: float, rows=None,
            groups: int = 1, delta_scale=None) -> None:
    """resid += delta (when given and ``rows`` is None); out = rmsnorm(resid) * weight.
    ``delta_scale`` (float32 [H]): resid += delta_scale * delta instead.
    ``groups`` > 1: each of that many equal consecutive parts of a row is
    divided by its own root mean square.
    ``delta`` has the residual stream's shape [T, H] in the activations' type,
    or is float32 [S, T, H]: the partial sums of a split-K product, added in
    order.  With ``rows`` (int32 indices) only those rows are normed, into
    out[0..len(rows)), and ``resid`` is left as it is."""
    _need_cuda(out, resid, delta, weight, rows, delta_scale)
    H = resid.shape[1]
    n = out.shape[0]
    assert delta_scale is None or (delta_scale.dtype == torch.float32 and delta_scale.is_contiguous() and delta_scale.numel() == H)
    assert resid.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == H
    assert out.shape[1] == H and out.is_contiguous() and resid.is_contiguous()
    parts, stride, dcode = 1, 0, dtype_code(out.dtype)
    if delta is not None:
        assert delta.is_contiguous() and tuple(delta.shape[-2:]) == tuple(resid.shape)
        if delta.dim() == 3:
            assert delta.dtype == torch.float32
            parts, stride = delta.shape[0], delta.stride(0)
        else:
            assert delta.dtype in (out.dtype, torch.float32)
        dcode = dtype_code(delta.dtype)
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() >= n
    else:
        assert n == resid.shape[0]
    _check(core().le_rmsnorm(_ptr(out), dtype_code(out.dtype), _ptr(resid), _ptr(delta), dcode, parts, stride,
                             _ptr(weight), _ptr(rows), float(eps), n, H, int(groups), _ptr(delta_scale), _stream()),
           "le_rmsnorm")


def rmsnorm_taps_applies(hidden: int, groups: int) -> bool:
    """Whether rmsnorm_taps() has a form for rows of this width and grouping."""
    return bool(core().le_rmsnorm_taps_applies(int(hidden), int(groups)))


def rmsnorm_taps(out, resid, delta, weight, eps, groups, w_taps, state, state_slots) -> None:
    """rmsnorm() over every row of a step whose requests bring one token each
    (row b is request b), then, in the same kernel, short_conv() of the normed
    rows: same arithmetic and roundings as the two kernels one after the other."""
    _need_cuda(out, resid, delta, weight, w_taps, state, state_slots)
    n, H = out.shape
    taps = w_taps.shape[0]
    assert resid.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == H
    assert out.is_contiguous() and resid.is_contiguous() and resid.shape == (n, H)
    assert w_taps.dtype == torch.float32 and w_taps.is_contiguous() and w_taps.shape[1] == H
    parts, stride, dcode = 1, 0, dtype_code(out.dtype)
    if delta is not None:
        assert delta.is_contiguous() and tuple(delta.shape[-2:]) == tuple(resid.shape)
        if delta.dim() == 3:
            assert delta.dtype == torch.float32
            parts, stride = delta.shape[0], delta.stride(0)
        else:
            assert delta.dtype in (out.dtype, torch.float32)
        dcode = dtype_code(delta.dtype)
    rows = 0
    if taps > 1:
        assert state is not None and state.dtype == torch.float32 and state.is_contiguous()
        assert tuple(state.shape[1:]) == (taps - 1, H)
        rows = state.shape[0]
    _check(core().le_rmsnorm_taps(_ptr(out), dtype_code(out.dtype), _ptr(resid), _ptr(delta), dcode, parts, stride,
                                  _ptr(weight), float(eps), n, H, int(groups), _ptr(w_taps),
                                  _ptr(state) if taps > 1 else None, rows, _ptr(state_slots), taps, _stream()),
           "le_rmsnorm_taps")


def rope_kv_write(qkv, k_cache, v_cache, cos_sin, positions, request_of_token, block_table, num_heads, num_kv_heads,
                  head_dim, page_size, write_kv, status) -> None:
    """Rotates queries (in place) and keys of the fused qkv rows and writes keys
    and values into the paged cache [pages, kv_heads, page, head_dim]."""
    _need_cuda(qkv, k_cache, cos_sin, positions, block_table)
    T = qkv.shape[0]
    assert qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim and qkv.is_contiguous()
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    max_pos, rot = cos_sin.shape
    if write_kv:
        assert k_cache.dtype == qkv.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert k_cache.shape[1:] == (num_kv_heads, page_size, head_dim), (k_cache.shape, num_kv_heads, page_size)
    num_pages = k_cache.shape[0] if k_cache is not None else 0
    _check(core().le_rope_kv_write(_ptr(qkv), dtype_code(qkv.dtype), _ptr(k_cache), _ptr(v_cache), _ptr(cos_sin),
                                   _ptr(positions), _ptr(request_of_token), _ptr(block_table), block_table.shape[1],
                                   T, num_heads, num_kv_heads, head_dim, rot, max_pos, page_size, num_pages,
                                   1 if write_kv else 0, _ptr(status), _stream()), "le_rope_kv_write")


def gemm_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the FP32 pipes (inputs float32 or
    bfloat16, 32-bit accumulation in ascending k)."""
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and a.dtype == w.dtype
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(core().le_gemm_simt(_ptr(out), dtype_code(out.dtype), _ptr(a), _ptr(w), dtype_code(a.dtype), M, N, K,
                               a.stride(0), w.stride(0), out.stride(0), _stream()), "le_gemm_simt")


# Up to this many rows a product streams weights through the package's own kernel (mma.sync with the weights as
# the 16-row operand).  Up to 16 rows of x a block takes 16 weight rows, and every product of a decode step runs
# there.  From 17 to 32 rows a block takes 32 or 64 weight rows (so that the slice of x it streams beside them is
# no larger than they are), and the products that are bound by their weights' bytes stay: the gated one (12.5 us
# against 18.6 of the tcgen05 kernel and 13.2 + the activation of the library at the 1B sizes) and the split-K
# ones that feed the residual stream (o 3.9 against 5.7 us of the library, down 9.5 against 13.1); the plain qkv
# product goes to the library there (6.9 against 5.7).  Beyond 32 rows mma.sync is the limit (64 rows: 20.5 us
# gated against 18.5 of the tcgen05 kernel).
SKINNY_ROWS = int(os.environ.get("LYAPUNOV_SKINNY_ROWS", "32"))
SKINNY_NARROW_ROWS = 16   # rows of x up to which a block takes 16 weight rows (and the qkv product its rotary epilogue)
SKINNY_BLOCKS_PER_SM = 512 / 148   # blocks worth having in flight per multiprocessor (512 on a B200: 4 slices of K for 2048 columns, measured best of 1..8)


def skinny_applies(a: torch.Tensor, w: torch.Tensor, rows: int | None = None) -> bool:
    """``rows``: the most rows of x the caller's form is worth it for (SKINNY_ROWS by default)."""
    return (a.dtype == torch.bfloat16 and a.shape[0] <= (SKINNY_ROWS if rows is None else rows) and a.shape[1] % 8 == 0 and a.stride(1) == 1
            and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def gemm_skinny(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, splits: int = 1, gated: bool = False,
                activation=(0, 1.0, 0.0), bias=None) -> None:
    """The package's weight-streaming product for at most 64 rows (bfloat16
    inputs).  ``splits`` > 1: ``out`` is float32 [splits, M, N] partial sums.
    ``gated``: ``w`` is [2 I, K] (gate rows, then up rows), out = act(gate, up)
    with ``activation`` = (kind, slope, limit) as glu() takes them (silu(gate) * up by default), and
    ``bias`` (float32 [2 I] or None) added to the product's columns before it."""
    _need_cuda(out, a, w, bias)
    M, K = a.shape
    N = w.shape[0]
    assert bias is None or (gated and bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == N)
    if splits > 1:
        assert out.dtype == torch.float32 and out.shape == (splits, M, N) and out.is_contiguous()
        ldo, stride = N, out.stride(0)
    else:
        assert out.shape[-2:] == (M, N // 2 if gated else N) and out.stride(-1) == 1
        ldo, stride = out.stride(-2), 0
    _check(core().le_gemm_skinny_bias_bf16(_ptr(out), dtype_code(out.dtype), _ptr(a), _ptr(w), M, N, K, a.stride(0),
                                           w.stride(0), ldo, splits, stride, 1 if gated else 0, int(activation[0]),
                                           float(activation[1]), float(activation[2]), _ptr(bias), _stream()),
           "le_gemm_skinny_bf16")


FUSE_ROTARY = os.environ.get("LYAPUNOV_FUSE_ROTARY", "1") not in ("0", "")


def rotary_product_applies(a: torch.Tensor, w: torch.Tensor, head_dim: int, rot: int) -> bool:
    """Whether the qkv product, the rotation and the cache write can be one kernel."""
    return skinny_applies(a, w, SKINNY_NARROW_ROWS) and rot == head_dim and head_dim % 16 == 0 and head_dim >= 16


def gemm_skinny_rotary(qkv, a, w, k_cache, v_cache, cos_sin, positions, request_of_token, block_table, num_heads,
                       num_kv_heads, head_dim, page_size, write_kv, status) -> None:
    """The fused qkv projection of at most 64 rows with rotary encoding and
    cache write in its epilogue: rotated queries into ``qkv`` (its key and
    value columns are left alone), rotated keys and the values into the paged
    cache.  Same arithmetic and roundings as linear() then rope_kv_write()."""
    _need_cuda(qkv, a, w, k_cache, cos_sin, positions, block_table)
    M, K = a.shape
    assert M <= 64 and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and cos_sin.shape[1] == head_dim and head_dim % 16 == 0
    assert K % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
    assert w.shape == ((num_heads + 2 * num_kv_heads) * head_dim, K) and qkv.shape == (M, w.shape[0])
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    if write_kv:
        assert k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    num_pages = k_cache.shape[0] if k_cache is not None else 0
    _check(core().le_gemm_skinny_rotary_bf16(_ptr(qkv), _ptr(a), _ptr(w), M, K, a.stride(0), w.stride(0), qkv.stride(0),
                                             _ptr(k_cache), _ptr(v_cache), _ptr(cos_sin), _ptr(positions),
                                             _ptr(request_of_token), _ptr(block_table), block_table.shape[1], num_heads,
                                             num_kv_heads, head_dim, cos_sin.shape[0], page_size, num_pages,
                                             1 if write_kv else 0, _ptr(status), _stream()), "le_gemm_skinny_rotary_bf16")


_tc_status = {}


def gemm_tc(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, gated: bool = False, status=None,
            activation=(0, 1.0, 0.0), bias=None) -> None:
    """The package's tcgen05 / TMA product for many rows (bfloat16 inputs):
    out = a @ w^T (bfloat16 or float32), or with ``gated`` out = act(a Wg^T,
    a Wu^T) for w = [Wg; Wu], ``activation`` = (kind, slope, limit) as glu()
    takes them (silu(g) * u by default), and ``bias`` (float32 [2 I] or None)
    added to the product's columns before it."""
    _need_cuda(out, a, w, bias)
    M, K = a.shape
    N = w.shape[0]
    assert bias is None or (gated and bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == N)
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert out.shape == (M, N // 2 if gated else N) and out.stride(1) == 1 and a.stride(1) == 1 and w.stride(1) == 1
    if status is None:
        status = tc_status(a.device)
    _check(core().le_gemm_tc_bias_bf16(_ptr(out), dtype_code(out.dtype), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(0),
                                       out.stride(0), 1 if gated else 0, int(activation[0]), float(activation[1]),
                                       float(activation[2]), _ptr(bias), _ptr(status), _stream()), "le_gemm_tc_bf16")


def tc_status(device) -> torch.Tensor:
    """The status word of the tensor-core product (a bounded wait that ran out sets it)."""
    status = _tc_status.get(torch.device(device))
    if status is None:
        status = _tc_status[torch.device(device)] = new_status(device)
    return status


def tc_applies(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


# Plain products with many rows: the package's tcgen05 kernel (one block per SM, 128 x 256 tiles) measures 7-18 %
# behind the library's two-SM kernels on this model's shapes, so they go to the library unless this is set; the
# gated product, where the fused activation more than pays for it, always uses the package's kernel.
TC_PLAIN_PRODUCTS = os.environ.get("LYAPUNOV_TC_PLAIN", "0") not in ("0", "")


def tc_fills_the_gpu(m: int, n: int) -> bool:
    """Whether 128 x 256 tiles of an [m, n] product fill the 148 SMs in whole
    rounds.  The package's kernel has that one tile shape; where it leaves the
    last round mostly empty the library, which picks among many shapes, is
    faster, and a plain product may go to it."""
    tiles = ((m + 127) // 128) * ((n + 255) // 256)
    rounds = (tiles + 147) // 148
    return tiles >= 0.8 * rounds * 148


def split_k_for(n_out: int, k: int, rows: int = 1) -> int:
    """How many slices of K give a product enough blocks to fill the GPU."""
    if rows > SKINNY_NARROW_ROWS:
        # blocks of 64 weight rows, two to a multiprocessor
        blocks = (n_out + 63) // 64
        return max(1, min((2 * sm_count() + blocks - 1) // blocks, k // 256, 16))
    blocks = (n_out + 15) // 16
    in_flight = int(SKINNY_BLOCKS_PER_SM * sm_count() + 0.5)
    return max(1, min((in_flight + blocks - 1) // blocks, k // 512, 16))


def linear_for_residual(a: torch.Tensor, w: torch.Tensor, workspace, key: str, status=None):
    """a @ w^T for a product whose only use is to be added to the residual
    stream: returns either the tensor [M, N] in the activations' type or, for
    few rows, float32 partial sums [S, M, N] that the next norm adds up."""
    M, N = a.shape[0], w.shape[0]
    if skinny_applies(a, w):
        splits = split_k_for(N, a.shape[1], M)
        out = workspace.get(key + "_partials", (splits, M, N), torch.float32)
        if splits == 1:
            gemm_skinny(out[0], a, w)
        else:
            gemm_skinny(out, a, w, splits=splits)
        return out
    out = workspace.get(key, (M, N), a.dtype)
    linear(out, a, w, status)
    return out


def gated_linear(out: torch.Tensor, a: torch.Tensor, w_gate_up: torch.Tensor, workspace, status=None,
                 activation=(GLU_SILU, 1.0, 0.0)) -> None:
    """out = act(a @ w_gate^T, a @ w_up^T), w_gate_up = [gate rows; up rows];
    ``activation``: (kind, slope, limit) as glu() takes them, silu(g) * u by
    default.  bfloat16: one kernel of the package (weight-streaming for few
    rows, tcgen05 for many) with the activation in its epilogue."""
    if skinny_applies(a, w_gate_up):
        gemm_skinny(out, a, w_gate_up, gated=True, activation=activation)
        return
    if tc_applies(a, w_gate_up):
        gemm_tc(out, a, w_gate_up, gated=True, status=status, activation=activation)
        return
    gu = workspace.get("gate_up", (a.shape[0], w_gate_up.shape[0]), a.dtype)
    linear(gu, a, w_gate_up, status)
    glu(out, gu, *activation)


FUSE_GATED_BIAS = os.environ.get("LYAPUNOV_FUSE_GATED_BIAS", "1") not in ("0", "")


def gated_linear_bias(out: torch.Tensor, a: torch.Tensor, w_gate_up: torch.Tensor, bias: torch.Tensor, workspace, status=None,
                      activation=(GLU_SILU, 1.0, 0.0)) -> None:
    """gated_linear() with a bias [2 I] (float32) on the product's columns
    before the activation.  bfloat16: in the epilogue of the package's kernels,
    on the 32-bit sums (weight-streaming for few rows, tcgen05 for many);
    else the product, then the activation's kernel with the bias.
    LYAPUNOV_FUSE_GATED_BIAS=0 takes the second way always."""
    if FUSE_GATED_BIAS and skinny_applies(a, w_gate_up):
        gemm_skinny(out, a, w_gate_up, gated=True, activation=activation, bias=bias)
        return
    if FUSE_GATED_BIAS and tc_applies(a, w_gate_up):
        gemm_tc(out, a, w_gate_up, gated=True, status=status, activation=activation, bias=bias)
        return
    gu = workspace.get("gate_up", (a.shape[0], w_gate_up.shape[0]), a.dtype)
    linear(gu, a, w_gate_up, status)
    glu(out, gu, *activation, bias=bias)


def linear(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, status=None) -> None:
    """out = a @ w^T.  float32: the package's FP32 kernel.  bfloat16 with few
    rows: the package's weight-streaming kernel.  bfloat16 with many rows: the
    package's tcgen05 kernel where its tiles fill the GPU, else the library
    product (cuBLAS); 32-bit accumulation everywhere, and a float32 ``out`` is
    written without an intermediate rounding."""
    if a.dtype == torch.float32:
        gemm_simt(out, a, w)
        return
    _need_cuda(out, a, w)
    if skinny_applies(a, w, SKINNY_NARROW_ROWS):
        gemm_skinny(out, a, w)
        return
    if TC_PLAIN_PRODUCTS and tc_applies(a, w) and tc_fills_the_gpu(a.shape[0], w.shape[0]):
        gemm_tc(out, a, w, status=status)
        return
    if out.dtype == torch.bfloat16:
        counters["library_products"] += 1
        torch.mm(a, w.t(), out=out)
    else:
        gemm_bf16_f32out(out, a, w)


_mm_out_dtype_ok = None


def gemm_bf16_f32out(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """bfloat16 inputs, float32 output (the output head's logits)."""
    global _mm_out_dtype_ok
    if _mm_out_dtype_ok is None:
        try:
            torch.mm(a[:1], w[:8].t(), out_dtype=torch.float32)
            _mm_out_dtype_ok = True
        except (TypeError, RuntimeError):
            _mm_out_dtype_ok = False
    K, N = a.shape[1], w.shape[0]
    if _mm_out_dtype_ok and K % 8 == 0 and N % 8 == 0:
        counters["library_products"] += 1
        torch.mm(a, w.t(), out_dtype=torch.float32, out=out)
    else:
        gemm_simt(out, a, w)


def reach_code(window: int | None = None, chunk: int | None = None) -> int:
    """Which keys a query sees besides none after itself, as the one integer
    the attention kernels take: 0 every key, w > 0 the last w keys, -c < 0 the
    keys of its own chunk of c positions (chunks counted from position 0)."""
    if window and chunk:
        raise ValueError("a mixer's keys are visible through a window or chunk by chunk, not both")
    return int(window) if window else (-int(chunk) if chunk else 0)


def _head_scale(head_scale, num_heads):
    if head_scale is not None:
        assert head_scale.dtype == torch.float32 and head_scale.is_contiguous() and head_scale.numel() == num_heads
        _need_cuda(head_scale)
    return _ptr(head_scale)


def attention_generic(out, q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_before, tile_request, tile_q0,
                      num_tiles, num_heads, num_kv_heads, head_dim, page_size, reach, scale, status, head_scale=None,
                      keep_first: int = 0, softcap: float = 0.0) -> None:
    """``reach``: see reach_code.  ``head_scale`` (float32 [num_heads] or None):
    one more factor per query head on its scores.  ``keep_first`` n: the keys
    at positions below n stay visible behind a window.  ``softcap`` c > 0: a
    score s becomes c * tanh(s / c)."""
    _need_cuda(out, q, k_cache, v_cache, block_table)
    lib = attention_lib(head_dim)
    assert out.is_contiguous() and out.shape[1] == num_heads * head_dim
    assert k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    _check(lib.le_attention_generic(_ptr(out), out.stride(0), _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache),
                                    dtype_code(out.dtype), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
                                    _ptr(ctx_before), _ptr(tile_request), _ptr(tile_q0), num_tiles, num_heads,
                                    num_kv_heads, page_size, k_cache.shape[0], int(reach or 0), float(scale),
                                    _head_scale(head_scale, num_heads), int(keep_first), float(softcap), _ptr(status),
                                    _stream()), "le_attention_generic", lib)


def attention_mma_available(head_dim: int) -> bool:
    """Whether the tensor-core attention kernels exist for this head size."""
    lib = attention_lib(head_dim)
    return bool(lib.le_attention_mma_available())


def attention_prefill_bf16(out, q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_before, tile_request, tile_q0,
                           num_tiles, num_heads, num_kv_heads, head_dim, page_size, reach, scale, status,
                           head_scale=None, keep_first: int = 0, softcap: float = 0.0) -> None:
    """Tensor-core attention for requests that bring several tokens; the tiles
    list 128 query tokens each.  ``keep_first``, ``softcap``: as attention_generic."""
    _need_cuda(out, q, k_cache, v_cache, block_table)
    lib = attention_lib(head_dim)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == num_heads * head_dim
    assert k_cache.dtype == torch.bfloat16 and k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    _check(lib.le_attention_prefill_bf16(_ptr(out), out.stride(0), _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache),
                                         _ptr(block_table), block_table.shape[1], _ptr(cu_q), _ptr(ctx_before),
                                         _ptr(tile_request), _ptr(tile_q0), num_tiles, num_heads, num_kv_heads,
                                         page_size, k_cache.shape[0], int(reach or 0), float(scale),
                                         _head_scale(head_scale, num_heads), int(keep_first), float(softcap), _ptr(status),
                                         _stream()),
           "le_attention_prefill_bf16", lib)


def attention_tc_available(head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention exists for this head and page size."""
    return bool(attention_lib(head_dim).le_attention_tc_available(int(page_size)))


def attention_prefill_tc_bf16(out, q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_before, tile_request, tile_q0,
                              num_tiles, num_heads, num_kv_heads, head_dim, page_size, reach, scale, status,
                              head_scale=None) -> None:
    """tcgen05 / TMA attention for requests that bring several tokens (head
    sizes 64 and 128, pages of 8..128 keys); the tiles list 128 query tokens
    each.  ``q`` is the [T, width] buffer whose rows start with the query heads.
    ``head_scale`` must be positive here (the kernel folds it into the exponent's scale)."""
    _need_cuda(out, q, k_cache, v_cache, block_table)
    lib = attention_lib(head_dim)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == num_heads * head_dim
    assert k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[1:] == (num_kv_heads, page_size, head_dim) and q.dim() == 2 and q.stride(1) == 1
    _check(lib.le_attention_prefill_tc_bf16(_ptr(out), out.stride(0), _ptr(q), q_stride, q.shape[0], q.shape[1],
                                            _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
                                            _ptr(cu_q), _ptr(ctx_before), _ptr(tile_request), _ptr(tile_q0), num_tiles,
                                            num_heads, num_kv_heads, page_size, k_cache.shape[0], int(reach or 0),
                                            float(scale), _head_scale(head_scale, num_heads), _ptr(status), _stream()),
           "le_attention_prefill_tc_bf16", lib)


def attention_decode_scratch_floats(head_dim: int, num_requests: int, num_heads: int, num_splits: int) -> int:
    return 0 if num_splits <= 1 else num_requests * num_heads * num_splits * (head_dim + 2)


_decode_resident: dict[tuple, int] = {}


def attention_decode_resident_blocks(head_dim: int, num_splits: int, small: bool = False) -> int:
    """Blocks of the split-key decode attention that the current device holds
    at once when the keys are cut ``num_splits`` ways (asked once per size).
    Splits that run as a thread-block cluster come in whole clusters, and fewer
    of those fit than twice the multiprocessor count suggests.  ``small``: of
    the form with 16-key tiles, which the launcher takes where the blocks of the
    usual form (32-key tiles at head sizes up to 64) do not all fit at once."""
    key = (torch.cuda.current_device(), head_dim, num_splits, bool(small))
    n = _decode_resident.get(key)
    if n is None:
        fn = attention_lib(head_dim).le_attention_decode_resident_blocks
        fn.restype, fn.argtypes = c_int, [c_int, c_int]
        n = int(fn(num_splits, 1 if small else 0))
        if n <= 0:
            raise KernelError(f"the device did not say how many decode attention blocks of head size {head_dim} it holds")
        _decode_resident[key] = n
    return n


def attention_decode_bf16(out, scratch, q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_before, requests,
                          num_requests, num_heads, num_kv_heads, head_dim, page_size, reach, scale, num_splits,
                          status, small_form=None, head_scale=None, keep_first: int = 0, softcap: float = 0.0) -> None:
    """Split-key tensor-core attention for requests that bring one token
    (``keep_first``, ``softcap``: as attention_generic).
    ``scratch``: float32, attention_decode_scratch_floats(...) elements.
    ``small_form``: None lets the launcher choose between the kernel's usual
    form and the one with 16-key tiles by the number of blocks; a caller that
    knows how many of the requests are real says True or False."""
    _need_cuda(out, q, k_cache, v_cache, block_table, scratch)
    lib = attention_lib(head_dim)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == num_heads * head_dim
    assert k_cache.dtype == torch.bfloat16 and k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    if num_splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32
        assert scratch.numel() >= attention_decode_scratch_floats(head_dim, num_requests, num_heads, num_splits)
    form = 0 if small_form is None else (2 if small_form else 1)
    _check(lib.le_attention_decode_bf16_form(_ptr(out), out.stride(0), _ptr(scratch), _ptr(q), q_stride, _ptr(k_cache),
                                             _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
                                             _ptr(ctx_before), _ptr(requests), num_requests, num_heads, num_kv_heads,
                                             page_size, k_cache.shape[0], int(reach or 0), float(scale),
                                             _head_scale(head_scale, num_heads), int(keep_first), float(softcap), num_splits,
                                             form, _ptr(status), _stream()),
           "le_attention_decode_bf16", lib,
           launches=2 if num_splits > 1 else 1)       # the attention kernel and the merge


def argmax_scratch_floats(num_rows: int, vocab: int) -> int:
    return 2 * num_rows * ((vocab + 4095) // 4096)


def argmax(out: torch.Tensor, logits: torch.Tensor, scratch=None) -> None:
    """out[r] = index of the first maximum of logits[r].  ``scratch`` (float32,
    argmax_scratch_floats elements) lets many blocks search one wide row."""
    _need_cuda(out, logits, scratch)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and logits.stride(1) == 1
    if scratch is not None:
        assert scratch.dtype == torch.float32 and scratch.numel() >= argmax_scratch_floats(n, V)
    two_stages = scratch is not None and (V + 4095) // 4096 >= 4
    _check(core().le_argmax(_ptr(out), _ptr(logits), n, V, logits.stride(0), _ptr(scratch), _stream()), "le_argmax",
           launches=2 if two_stages else 1)


def sample(out, logits, temperature, top_p, top_k, seeds, uniforms=None, probs_out=None) -> None:
    """One token per row of ``logits`` [n, V] float32: greedy where temperature
    < 1e-4, else temperature / top-k / top-p sampling.  ``seeds`` is int32
    [n, 3]: seed low word, seed high word, counter."""
    _need_cuda(out, logits, temperature, top_p, top_k, seeds)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert top_k.dtype == torch.int32 and seeds.dtype == torch.int32
    _check(core().le_sample(_ptr(out), _ptr(logits), n, V, logits.stride(0), _ptr(temperature), _ptr(top_p),
                            _ptr(top_k), _ptr(seeds), _ptr(uniforms), _ptr(probs_out), _stream()), "le_sample")


# --------------------------------------------------------------------------
# a residual stream in several copies; rotary pairs over segmented heads; maps of a head combined; capped logits
def stream_norm(out, streams, weight, bias, eps, delta=None, mix=None, post=None, pre=None, init=None, rows=None) -> None:
    """One launch over a residual stream kept as S copies (``streams`` float32
    [T, S, W]): first the pending update x'_j = sum_s mix[s, j] x_s + post[j] *
    delta (``delta`` [T, W] in the activations' type, or float32 [P, T, W]
    partial sums added in order; None: no update; ``init`` float32 [T, W]:
    every copy starts as that row), written back; then u = sum_s pre[s] x'_s
    (``pre`` None: the plain sum); then out = layer norm of u with ``weight``
    and ``bias`` (``bias`` None: RMS norm).  ``mix`` / ``post`` None: identity /
    ones.  With ``rows`` (int32) only those rows are read and normed, into
    out[0 .. len(out)), and ``streams`` stays as it is."""
    _need_cuda(out, streams, weight, bias, delta, mix, post, pre, init, rows)
    T, S, W = streams.shape
    n = out.shape[0]
    assert streams.dtype == torch.float32 and streams.is_contiguous() and out.is_contiguous() and out.shape[1] == W
    assert weight.dtype == torch.float32 and weight.numel() == W and (bias is None or (bias.dtype == torch.float32 and bias.numel() == W))
    for v, count in ((mix, S * S), (post, S), (pre, S)):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == count)
    parts, stride, dcode = 1, 0, dtype_code(out.dtype)
    if delta is not None:
        assert delta.is_contiguous() and tuple(delta.shape[-2:]) == (T, W)
        if delta.dim() == 3:
            assert delta.dtype == torch.float32
            parts, stride = delta.shape[0], delta.stride(0)
        else:
            assert delta.dtype in (out.dtype, torch.float32)
        dcode = dtype_code(delta.dtype)
    if init is not None:
        assert init.dtype == torch.float32 and init.is_contiguous() and tuple(init.shape) == (T, W)
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() >= n
    else:
        assert n == T
    _check(core().le_stream_norm(_ptr(out), dtype_code(out.dtype), _ptr(streams), _ptr(init), _ptr(delta), dcode, parts,
                                 stride, _ptr(mix), _ptr(post), _ptr(pre), _ptr(weight), _ptr(bias), _ptr(rows), float(eps),
                                 n, W, S, _stream()), "le_stream_norm")


def stream_sum(out, streams) -> None:
    """out [T, W] float32 = the sum of the copies ``streams`` [T, S, W]."""
    _need_cuda(out, streams)
    T, S, W = streams.shape
    assert out.shape == (T, W) and out.dtype == streams.dtype == torch.float32 and out.is_contiguous() and streams.is_contiguous()
    _check(core().le_stream_sum(_ptr(out), _ptr(streams), T, W, S, _stream()), "le_stream_sum")


def rope_pairs_store(q_out, src, bias, k_cache, v_cache, rates, positions, request_of_token, block_table, heads, kv_heads,
                     segments, seg_dim, value_dim, rot, head_dim, page_size, write_kv, status) -> None:
    """Rows of ``src`` hold queries [heads, segments, seg_dim], keys [kv_heads,
    segments, seg_dim] and values [kv_heads, value_dim].  Adds ``bias``
    (float32, as wide as a row, or None), turns the entries (2i, 2i + 1) below
    ``rot`` of every segment by position * rates[i] in 32 bits, and writes
    every (head, segment) as a query head of ``head_dim`` columns into
    ``q_out`` (its segment at columns segment * seg_dim .., zeros elsewhere),
    keys (a kv head's segments side by side) and values (zero-padded) into the
    paged pools [pages, kv_heads, page, head_dim]."""
    _need_cuda(q_out, src, bias, k_cache, v_cache, rates, positions, block_table)
    T = src.shape[0]
    cols = (heads + kv_heads) * segments * seg_dim + kv_heads * value_dim
    assert src.shape[1] == cols and src.stride(1) == 1 and q_out.dtype == src.dtype and q_out.stride(1) == 1
    assert q_out.shape == (T, heads * segments * head_dim)
    assert rates.dtype == torch.float32 and rates.is_contiguous() and rates.numel() >= rot // 2
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == cols)
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    pages = 0
    if write_kv:
        assert k_cache.dtype == src.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (kv_heads, page_size, head_dim) and v_cache.shape == k_cache.shape
        pages = k_cache.shape[0]
    _check(core().le_rope_pairs_store(_ptr(src), src.stride(0), dtype_code(src.dtype), _ptr(bias), _ptr(q_out),
                                      q_out.stride(0), _ptr(k_cache) if write_kv else None,
                                      _ptr(v_cache) if write_kv else None, _ptr(rates), _ptr(positions),
                                      _ptr(request_of_token), _ptr(block_table), block_table.shape[1], T, heads, kv_heads,
                                      segments, seg_dim, value_dim, rot, head_dim, page_size, pages, 1 if write_kv else 0,
                                      _ptr(status), _stream()), "le_rope_pairs_store")


def maps_combine(out, attn, coef, heads, segments, head_dim, value_dim, eps, post) -> None:
    """out[t, h, :value_dim] = post * unit(sum_m coef[m] * attn[t, h * segments +
    m, :value_dim]) with unit(o) = o / sqrt(mean(o^2) + eps) (``eps`` None: no
    division), in 32 bits.  ``coef``: float32 [segments] on the device."""
    _need_cuda(out, attn, coef)
    T = attn.shape[0]
    assert attn.shape[1] == heads * segments * head_dim and attn.stride(1) == 1 and out.shape == (T, heads * value_dim)
    assert out.stride(1) == 1 and out.dtype == attn.dtype and coef.dtype == torch.float32 and coef.numel() == segments
    _check(core().le_maps_combine(_ptr(out), out.stride(0), _ptr(attn), attn.stride(0), dtype_code(attn.dtype), _ptr(coef), T,
                                  heads, segments, head_dim, value_dim, -1.0 if eps is None else float(eps), float(post),
                                  _stream()), "le_maps_combine")


def softcap(logits, cap: float) -> None:
    """logits <- cap * tanh(logits / cap), float32, in place."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous() and cap > 0
    _check(core().le_softcap(_ptr(logits), logits.numel(), float(cap), _stream()), "le_softcap")


# --------------------------------------------------------------------------
# routed experts
_moe_tile_rows: dict[bool, int] = {}
MOE_WIDE_ROWS = 64      # rows an expert has on average from which the wide row tiles pay
# 0: the experts' products of prompt portions stay on the mma.sync kernel (wide row tiles) instead of the tcgen05 one
TC_EXPERTS = os.environ.get("LYAPUNOV_TC_EXPERTS", "1") not in ("0", "")


def moe_tile_rows(wide: bool = False) -> int:
    """Sorted slots per row tile: 32, or 128 in the wide form (tensor cores, many rows per expert)."""
    if wide not in _moe_tile_rows:
        _moe_tile_rows[wide] = int(core().le_moe_tile_rows(1 if wide else 0))
    return _moe_tile_rows[wide]


def moe_wide_tiles(pairs: int, experts: int, dtype, width: int, inner: int) -> bool:
    """Whether the experts' products of ``pairs`` rows run on wide row tiles:
    bfloat16, rows in 16-byte pieces, and enough rows per expert."""
    return dtype == torch.bfloat16 and width % 8 == 0 and inner % 8 == 0 and pairs >= MOE_WIDE_ROWS * experts


def moe_max_tiles(pairs: int, experts: int, wide: bool = False) -> int:
    """Row tiles that ``pairs`` (token, choice) pairs can need at most, however they fall on the experts."""
    return pairs // moe_tile_rows(wide) + min(experts, pairs)


MOE_SOFTMAX_CHOSEN, MOE_SIGMOID = 0, 1


def moe_route(ids, weights, gate, h, w_router, b_router, w_gate, top: int, scratch=None, scoring: int = MOE_SOFTMAX_CHOSEN) -> None:
    """Per row of ``h``: router logits W h + b in 32 bits, the ``top`` largest
    (``ids`` int32 [T, top], best first), softmax over the chosen logits
    (``weights`` float32 [T, top]; ``scoring`` MOE_SIGMOID: each chosen
    logit's own sigmoid instead, not renormalized); with ``w_gate`` (float32 [W]) also
    ``gate`` [T] = sigmoid(w_gate . h).  ``scratch``: float32, T * (experts +
    1) elements, for the logits (made here when not given: a caller whose
    steps are captured passes its own)."""
    _need_cuda(ids, weights, gate, h, w_router, b_router, w_gate, scratch)
    T, W = h.shape
    E = w_router.shape[0]
    assert w_router.dtype == torch.float32 and w_router.is_contiguous() and w_router.shape[1] == W and h.stride(1) == 1
    assert b_router is None or (b_router.dtype == torch.float32 and b_router.numel() == E)
    assert ids.dtype == torch.int32 and ids.is_contiguous() and tuple(ids.shape) == (T, top)
    assert weights.dtype == torch.float32 and weights.is_contiguous() and tuple(weights.shape) == (T, top)
    if w_gate is not None:
        assert w_gate.dtype == torch.float32 and w_gate.numel() == W and gate.dtype == torch.float32 and gate.numel() >= T
    if scratch is None:
        scratch = torch.empty(T * (E + 1), dtype=torch.float32, device=h.device)
    assert scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= T * (E + 1)
    _check(core().le_moe_route(_ptr(h), h.stride(0), dtype_code(h.dtype), _ptr(w_router), _ptr(b_router), _ptr(w_gate),
                               _ptr(scratch), _ptr(ids), _ptr(weights), _ptr(gate), T, W, E, top, int(scoring), _stream()),
           "le_moe_route",
           launches=2)


def moe_group(ids, experts: int, slot_pair, tiles, meta, wide: bool = False, padded: bool = False, pair_slot=None) -> None:
    """Sorts the pairs (entries of ``ids``) by expert: ``slot_pair`` int32
    lists the pairs expert by expert; ``tiles`` int32 [3, max tiles] (expert,
    first slot, rows of each row tile; unused entries zero); ``meta[0]`` the
    tile count.  ``padded``: every expert's slots start at a multiple of the
    tile's rows, slots that stand for no pair hold -1, and ``slot_pair`` has
    room for max tiles * tile rows.  ``pair_slot`` (int32 [pairs]) receives
    each pair's slot."""
    _need_cuda(ids, slot_pair, tiles, meta, pair_slot)
    pairs = ids.numel()
    assert slot_pair.dtype == tiles.dtype == meta.dtype == torch.int32 and tiles.is_contiguous() and tiles.shape[0] == 3
    max_tiles = tiles.shape[1]
    assert max_tiles >= moe_max_tiles(pairs, experts, wide)
    assert slot_pair.numel() >= (max_tiles * moe_tile_rows(wide) if padded else pairs)
    assert pair_slot is None or (pair_slot.dtype == torch.int32 and pair_slot.numel() >= pairs)
    _check(core().le_moe_group(_ptr(ids), pairs, experts, moe_tile_rows(wide), 1 if padded else 0, max_tiles,
                               slot_pair.numel(), _ptr(slot_pair), _ptr(pair_slot), _ptr(tiles[0]), _ptr(tiles[1]),
                               _ptr(tiles[2]), _ptr(meta), _stream()), "le_moe_group")


def moe_gather(out, x, slot_pair, meta, src_div: int, wide: bool = True, pair_weight=None) -> None:
    """out[slot] = x[slot_pair[slot] // src_div] for the slots of the first
    meta[0] row tiles (zeros where a slot stands for no pair); with
    ``pair_weight`` (float32 [pairs]) the row times its pair's weight."""
    _need_cuda(out, x, slot_pair, meta, pair_weight)
    assert pair_weight is None or (pair_weight.dtype == torch.float32 and pair_weight.is_contiguous())
    assert out.dtype == x.dtype and out.is_contiguous() and x.stride(1) == 1 and out.shape[1] == x.shape[1]
    assert slot_pair.numel() >= out.shape[0]
    _check(core().le_moe_gather(_ptr(out), _ptr(x), x.stride(0), dtype_code(x.dtype), _ptr(slot_pair), int(src_div),
                                moe_tile_rows(wide), _ptr(meta), out.shape[0], x.shape[1], _ptr(pair_weight), _stream()),
           "le_moe_gather")


def moe_combine_sorted(out, y, pair_slot, share, top: int, shared_out=None, gate=None) -> None:
    """out[t] = sum_j share[t, j] * y[pair_slot[t * top + j]] (+ gate[t] * shared_out[t]); ``share`` None: plain sum."""
    _need_cuda(out, y, pair_slot, share, shared_out, gate)
    T, W = out.shape
    assert y.is_contiguous() and y.shape[1] == W and out.is_contiguous()
    assert share is None or (share.dtype == torch.float32 and share.is_contiguous() and share.numel() == T * top)
    assert pair_slot.dtype == torch.int32 and pair_slot.numel() >= T * top
    assert shared_out is None or (shared_out.dtype == out.dtype and shared_out.is_contiguous() and shared_out.shape == out.shape)
    _check(core().le_moe_combine_sorted(_ptr(out), dtype_code(out.dtype), _ptr(y), dtype_code(y.dtype), _ptr(pair_slot),
                                        _ptr(share), _ptr(shared_out), _ptr(gate), T, W, top, _stream()),
           "le_moe_combine_sorted")


def gemm_tc_grouped(out, a, w, tile_expert, tile_count, gated: bool = False, status=None, activation=(0, 1.0, 0.0)) -> None:
    """The tcgen05 / TMA product in its grouped form: ``a`` [M, K] holds row
    tiles of 128 rows, tile m is multiplied with matrix ``tile_expert[m]`` of
    ``w`` [experts, N, K] (gated: N = 2 F, gate rows then up rows, out =
    act(gate, up)), and only the first ``tile_count[0]`` tiles are computed;
    both lists are int32 on the device."""
    _need_cuda(out, a, w, tile_expert, tile_count)
    E, N, K = w.shape
    M = a.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and a.shape[1] == K and M % 128 == 0
    assert out.shape == (M, N // 2 if gated else N) and out.stride(1) == 1 and a.stride(1) == 1
    assert tile_expert.dtype == torch.int32 and tile_expert.numel() >= M // 128 and tile_count.dtype == torch.int32
    if status is None:
        status = tc_status(a.device)
    _check(core().le_gemm_tc_grouped_bf16(_ptr(out), dtype_code(out.dtype), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(1),
                                          out.stride(0), E, _ptr(tile_expert), _ptr(tile_count), 1 if gated else 0,
                                          int(activation[0]), float(activation[1]), float(activation[2]), _ptr(status),
                                          _stream()), "le_gemm_tc_grouped_bf16")


def moe_grouped(out, a, w, slot_pair, tiles, meta, max_tiles: int, src_div: int, scatter: bool, pair_weight=None,
                gated: bool = False, activation=(0, 1.0, 0.0), wide: bool = False) -> None:
    """The product of every sorted slot's row with its expert's matrix
    ``w`` [experts, N (2 F when gated), K].  Input row of a slot: row pair //
    src_div of ``a`` (``src_div`` 0: row slot).  Output row: the slot, or with
    ``scatter`` the pair, times ``pair_weight[pair]`` where given (in the
    gated form the weight multiplies both products before the activation: the
    weight on the expert's input).  bfloat16
    with rows in 16-byte pieces: tensor cores (``wide``: the tiles moe_group
    made are the wide ones); else the FP32 pipes."""
    _need_cuda(out, a, w, slot_pair, tiles, meta, pair_weight)
    E, N, K = w.shape
    if gated:
        N //= 2
    assert w.is_contiguous() and a.dtype == w.dtype and a.stride(1) == 1 and a.shape[1] == K and out.stride(1) == 1
    assert out.shape[1] == N
    _check(core().le_moe_grouped(_ptr(out), dtype_code(out.dtype), out.stride(0), _ptr(a), a.stride(0), _ptr(w), w.stride(0),
                                 w.stride(1), dtype_code(a.dtype), _ptr(slot_pair), int(src_div), 1 if scatter else 0,
                                 _ptr(pair_weight), _ptr(tiles[0]), _ptr(tiles[1]), _ptr(tiles[2]), _ptr(meta), max_tiles,
                                 moe_tile_rows(wide), N, K, 1 if gated else 0, int(activation[0]), float(activation[1]),
                                 float(activation[2]), _stream()), "le_moe_grouped")


def moe_combine(out, y, top: int, shared_out=None, gate=None) -> None:
    """out[t] = sum_j y[t * top + j] (+ gate[t] * shared_out[t]); ``y`` float32 [T * top, W]."""
    _need_cuda(out, y, shared_out, gate)
    T, W = out.shape
    assert y.dtype == torch.float32 and y.is_contiguous() and tuple(y.shape) == (T * top, W) and out.is_contiguous()
    assert shared_out is None or (shared_out.dtype == out.dtype and shared_out.is_contiguous() and shared_out.shape == out.shape)
    _check(core().le_moe_combine(_ptr(out), dtype_code(out.dtype), _ptr(y), _ptr(shared_out), _ptr(gate), T, W, top, _stream()),
           "le_moe_combine")


# -------------------------------------------------------------------------- convolution with activation, delta rule
def short_conv_general(out, h, w_taps, state, state_slots, cu_q, tile_request, tile_q0, num_tiles, add_input: bool,
                       silu: bool, bias=None) -> None:
    """short_conv() in its general form: ``h`` may be a column range of wider
    rows (any row stride); ``add_input`` False leaves the token's own
    input out of the sum (a plain causal convolution whose last tap is the
    current token's); ``silu`` puts silu over the sum; ``bias`` (float32
    [channels]) is added to the sum before it."""
    _need_cuda(out, h, w_taps, state, state_slots, cu_q, bias)
    T, C = h.shape
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C)
    taps = w_taps.shape[0]
    assert out.shape == h.shape and out.dtype == h.dtype and out.is_contiguous() and h.stride(1) == 1
    assert w_taps.dtype == torch.float32 and w_taps.is_contiguous() and w_taps.shape[1] == C
    rows = 0
    if taps > 1:
        assert state is not None and state.dtype == torch.float32 and state.is_contiguous()
        assert tuple(state.shape[1:]) == (taps - 1, C)
        rows = state.shape[0]
    _check(core().le_short_conv_general(_ptr(out), _ptr(h), h.stride(0), dtype_code(h.dtype), _ptr(w_taps),
                                        _ptr(state) if taps > 1 else None, rows, _ptr(state_slots), _ptr(cu_q),
                                        _ptr(tile_request), _ptr(tile_q0), num_tiles, SHORT_CONV_TILE, C, taps,
                                        1 if add_input else 0, 1 if silu else 0, _ptr(bias), _stream()),
           "le_short_conv_general")


GATED_DELTA_MAX_DIM = 1024


def gated_delta_scratch_width(heads: int, kv_heads: int) -> int:
    """Floats per token of the scratch rows that ``gated_delta_scan`` fills (inverse lengths, k . q, decay, step size)."""
    return 4 * int(kv_heads) + 2 * int(heads)


def gated_delta_scan(out, qkv, q_col, k_col, v_col, proj, b_col, a_col, a_log, dt_bias, state, state_slots, cu_q,
                     num_requests, heads, kv_heads, dim, vdim, unit_eps, q_scale, scratch=None) -> None:
    """The gated delta rule over the step's tokens, request by request, from
    each request's state row and back into it.  ``out``: float32 [T, heads *
    vdim].  ``qkv``: rows with queries and keys [kv_heads, dim] at columns
    ``q_col`` / ``k_col`` and values [heads, vdim] at ``v_col``; queries and
    keys are made unit vectors here (x / sqrt(sum x^2 + unit_eps)), queries
    times ``q_scale``.  ``proj``: rows with one number per head at ``b_col``
    (step size = its sigmoid) and ``a_col`` (decay = exp(-exp(a_log) *
    softplus(a + dt_bias))).  ``state``: float32 [rows, heads, vdim, dim].
    ``scratch``: float32 [T, gated_delta_scratch_width()], made here if None."""
    _need_cuda(out, qkv, proj, a_log, dt_bias, state, state_slots, cu_q)
    T = out.shape[0]
    assert out.dtype == torch.float32 and out.stride(1) == 1 and qkv.stride(1) == 1 and proj.stride(1) == 1
    assert qkv.dtype == proj.dtype and a_log.dtype == torch.float32 and dt_bias.dtype == torch.float32
    assert a_log.numel() == heads and dt_bias.numel() == heads and qkv.shape[0] == T and proj.shape[0] == T
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, vdim, dim)
    width = gated_delta_scratch_width(heads, kv_heads)
    if scratch is None:
        scratch = torch.empty((max(T, 1), width), dtype=torch.float32, device=out.device)
    assert scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.shape[0] >= T and scratch.shape[1] == width
    _check(core().le_gated_delta_scan(_ptr(out), out.stride(0), _ptr(qkv), qkv.stride(0), q_col, k_col, v_col, _ptr(proj),
                                      proj.stride(0), b_col, a_col, dtype_code(qkv.dtype), _ptr(a_log), _ptr(dt_bias),
                                      _ptr(state), state.shape[0], _ptr(state_slots), _ptr(cu_q), num_requests, T, heads,
                                      kv_heads, dim, vdim, float(unit_eps), float(q_scale), _ptr(scratch), _stream()),
           "le_gated_delta_scan")


def head_norm_gate(out, o, gate, weight, eps, heads, vdim, sigmoid: bool = False, out_scale: float = 1.0) -> None:
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight *
    silu(gate[t, h, :]); ``o`` float32, ``gate`` and ``out`` in the
    activations' type (column ranges of wider rows are fine).  ``weight``
    holds ``vdim`` numbers shared by the heads, or ``heads * vdim``.
    ``sigmoid``: the gate's sigmoid instead of its silu; ``out_scale``: one
    more factor on the result."""
    _need_cuda(out, o, gate, weight)
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.shape == (T, heads * vdim) and out.shape == o.shape and gate.shape == o.shape
    assert out.dtype == gate.dtype and o.stride(1) == 1 and out.stride(1) == 1 and gate.stride(1) == 1
    assert weight.dtype == torch.float32 and weight.numel() in (vdim, heads * vdim) and weight.is_contiguous()
    _check(core().le_head_norm_gate(_ptr(out), out.stride(0), _ptr(o), o.stride(0), _ptr(gate), gate.stride(0),
                                    dtype_code(out.dtype), _ptr(weight), float(eps), T, heads, vdim,
                                    1 if weight.numel() != vdim else 0, 1 if sigmoid else 0, float(out_scale), _stream()),
           "le_head_norm_gate")


# -------------------------------------------------------------------------- rotary pairs with a norm per head
def rope_norm_store(rows, k_cache, v_cache, rates, positions, request_of_token, block_table, heads, kv_heads, head_dim,
                    rot_col, rot, unit_eps, norm_dim, page_size, write_kv, values_are_keys, status) -> None:
    """Rows hold query heads, then key heads, ``head_dim`` entries each.  The
    entries (rot_col + 2i, rot_col + 2i + 1) below rot_col + ``rot`` of every
    head turn by position * rates[i]; with ``unit_eps`` not None the head is
    then divided by sqrt(mean over its first ``norm_dim`` entries of x^2 +
    unit_eps).  Queries are rewritten in place, keys go to ``k_cache``, and
    ``v_cache`` receives the keys as they were projected when
    ``values_are_keys``.  ``write_kv`` False: the queries only."""
    _need_cuda(rows, k_cache, v_cache, rates, positions, block_table)
    T = rows.shape[0]
    assert rows.stride(1) == 1 and rows.shape[1] >= (heads + (kv_heads if write_kv else 0)) * head_dim
    assert rates.dtype == torch.float32 and rates.is_contiguous() and rates.numel() >= rot // 2
    pages = 0
    if write_kv:
        assert k_cache.dtype == rows.dtype and k_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (kv_heads, page_size, head_dim)
        assert not values_are_keys or (v_cache.shape == k_cache.shape and v_cache.is_contiguous())
        pages = k_cache.shape[0]
    _check(core().le_rope_norm_store(_ptr(rows), rows.stride(0), dtype_code(rows.dtype), _ptr(k_cache) if write_kv else None,
                                     _ptr(v_cache) if write_kv and values_are_keys else None, _ptr(rates), _ptr(positions),
                                     _ptr(request_of_token), _ptr(block_table), block_table.shape[1], T, heads, kv_heads,
                                     head_dim, rot_col, rot, 0 if unit_eps is None else 1,
                                     0.0 if unit_eps is None else float(unit_eps), norm_dim, page_size, pages,
                                     1 if write_kv else 0, 1 if values_are_keys else 0, _ptr(status), _stream()),
           "le_rope_norm_store")


def latent_rope_store(src, col, rank, rot, padded, weight, eps, rates, cache, positions, request_of_token, block_table,
                      page_size, status, second=None) -> None:
    """The latent at columns [col, col + rank) of ``src`` is normed (weight
    [rank]) and the ``rot`` columns behind it are turned in neighbouring pairs
    by position * rates[i]; both go to ``cache`` [pages, 1, page, padded]
    (None: nothing is stored).  ``second`` = (col2, rank2, weight2, out2): a
    second latent of the row is normed into ``out2``."""
    _need_cuda(src, weight, rates, cache, positions, block_table)
    T = src.shape[0]
    assert src.stride(1) == 1 and weight.dtype == torch.float32 and weight.numel() == rank
    assert rot == 0 or (rates is not None and rates.dtype == torch.float32 and rates.numel() >= rot // 2)
    pages = 0
    if cache is not None:
        assert cache.dtype == src.dtype and cache.is_contiguous() and tuple(cache.shape[1:]) == (1, page_size, padded)
        pages = cache.shape[0]
    col2, rank2, weight2, out2 = second if second is not None else (0, 0, None, None)
    if out2 is not None:
        assert out2.dtype == src.dtype and out2.stride(1) == 1 and weight2.dtype == torch.float32 and weight2.numel() == rank2
    _check(core().le_latent_rope_store(_ptr(src), src.stride(0), dtype_code(src.dtype), col, rank, rot, padded, _ptr(weight),
                                       float(eps), _ptr(rates), _ptr(cache), col2, rank2, _ptr(weight2), _ptr(out2),
                                       out2.stride(0) if out2 is not None else 0, _ptr(positions), _ptr(request_of_token),
                                       _ptr(block_table), block_table.shape[1], T, page_size, pages, _ptr(status), _stream()),
           "le_latent_rope_store")


# -------------------------------------------------------------------------- sub-layers side by side; inputs per token
def _addend(t, rows: int, width: int):
    """(pointer, dtype code, partial sums, elements between them) of a
    sub-layer's output on its way into the stream: [rows, width] in the
    activations' type or float32, or float32 partial sums [parts, rows, width]."""
    if t is None:
        return None, F32, 1, 0
    assert t.is_contiguous() and tuple(t.shape[-2:]) == (rows, width)
    if t.dim() == 3:
        assert t.dtype == torch.float32
        return t.data_ptr(), F32, t.shape[0], t.stride(0)
    return t.data_ptr(), dtype_code(t.dtype), 1, 0


def rmsnorm_pair(out1, out2, resid, w1, w2, eps, addend=None, addend_weight=None, addend_eps: float = 0.0, rows=None) -> None:
    """``addend`` first enters the 32-bit stream ``resid`` [T, W]: plainly, or,
    with ``addend_weight`` [W], as addend / sqrt(mean(addend^2) + addend_eps) *
    addend_weight.  Then out1 = rmsnorm(resid) * w1 and (``out2`` given) out2 =
    rmsnorm(resid) * w2.  ``out1`` None: only the addend enters.  With ``rows``
    only those rows are normed and ``resid`` is left as it is."""
    _need_cuda(out1, out2, resid, w1, w2, addend, addend_weight, rows)
    T, W = resid.shape
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    n = T if rows is None else (out1.shape[0] if out1 is not None else 0)
    for o, w in ((out1, w1), (out2, w2)):
        if o is not None:
            assert o.is_contiguous() and o.shape == (n, W) and w.dtype == torch.float32 and w.numel() == W
    ptr, code, parts, stride = _addend(addend, T, W)
    out_code = dtype_code(out1.dtype) if out1 is not None else F32
    _check(core().le_rmsnorm_pair(_ptr(out1), _ptr(out2), out_code, _ptr(resid), ptr, code, parts, stride,
                                  _ptr(addend_weight), float(addend_eps), _ptr(w1), _ptr(w2), float(eps), _ptr(rows), n, W,
                                  _stream()), "le_rmsnorm_pair")


def residual_add(resid, a=None, f=None, bias=None, copy=None) -> None:
    """resid += a + f + bias (each optional; a and f as _addend() takes them,
    bias float32 [W]); ``copy`` receives the new rows in its own type."""
    _need_cuda(resid, a, f, bias, copy)
    T, W = resid.shape
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == W)
    assert copy is None or (copy.is_contiguous() and copy.shape == resid.shape)
    ap, ac, an, as_ = _addend(a, T, W)
    fp, fc, fn, fs = _addend(f, T, W)
    _check(core().le_residual_add(_ptr(resid), _ptr(copy), dtype_code(copy.dtype) if copy is not None else F32, ap, ac, an,
                                  as_, fp, fc, fn, fs, _ptr(bias), T, W, _stream()), "le_residual_add")


def gate_rows(out, z, table, col, ids, status) -> None:
    """out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col + j]."""
    _need_cuda(out, z, table, ids)
    T, D = z.shape
    assert out.shape == z.shape and out.dtype == z.dtype and out.is_contiguous() and z.is_contiguous()
    assert table.stride(1) == 1 and 0 <= col and col + D <= table.shape[1] and ids.dtype == torch.int32
    _check(core().le_gate_rows(_ptr(out), _ptr(z), dtype_code(z.dtype), _ptr(table), dtype_code(table.dtype), table.stride(0),
                               col, _ptr(ids), table.shape[0], T, D, _ptr(status), _stream()), "le_gate_rows")


def stream_entry(resid, table, ids, vec, status) -> None:
    """resid[t] += table[ids[t]] + vec (either may be None)."""
    _need_cuda(resid, table, ids, vec)
    T, W = resid.shape
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    assert table is None or (table.is_contiguous() and table.shape[1] == W)
    assert vec is None or (vec.dtype == torch.float32 and vec.is_contiguous() and vec.numel() == W)
    _check(core().le_stream_entry(_ptr(resid), _ptr(table), dtype_code(table.dtype) if table is not None else F32, _ptr(ids),
                                  table.shape[0] if table is not None else 0, _ptr(vec), T, W, _ptr(status), _stream()),
           "le_stream_entry")


# -------------------------------------------------------------------------- gates, state-space scans, matrix memory
def sigmoid_gate(out, x, gate, scale: float = 1.0) -> None:
    """out = x * sigmoid(gate) * scale, entry by entry; all three [T, W] in
    the activations' type, each a column range of wider rows if need be
    (``out`` may be ``x``)."""
    _need_cuda(out, x, gate)
    T, W = x.shape
    assert out.shape == x.shape == gate.shape and out.dtype == x.dtype == gate.dtype
    assert out.stride(1) == 1 and x.stride(1) == 1 and gate.stride(1) == 1
    _check(core().le_sigmoid_gate(_ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(gate), gate.stride(0),
                                  dtype_code(x.dtype), T, W, float(scale), _stream()), "le_sigmoid_gate")


SSM_MAX_STATE = 512


def ssm_scan(out, x, bc, b_col: int, c_col: int, dt, z, dt_bias, a_log, d_skip, state, state_slots, cu_q, num_requests: int,
             n_state: int, rows_per_head: int, rows_per_group: int, per_row: bool, out_scale: float = 1.0) -> None:
    """A diagonal state-space recurrence over the step's tokens, request by
    request, from each request's state row and back into it.  Per row r
    (channel) with N = ``n_state`` numbers of state, per token:
        dt = softplus(dt_raw + dt_bias);  S <- exp(dt * A) S + dt * x_r * B;  y = S . C + D * x_r
        out = y * silu(z_r) * out_scale        (``z`` None: no gate)
    with A = -exp(a_log).  ``per_row`` False: dt, dt_bias, D and a_log have
    one entry per head of ``rows_per_head`` rows; True: one per row, and
    ``a_log`` is [rows, N].  ``bc``: rows that hold B [groups, N] at column
    ``b_col`` and C at ``c_col``; the rows of a group (``rows_per_group``
    consecutive ones) share them.  ``x``, ``bc``, ``dt``, ``z`` are column
    ranges of rows in the activations' type; ``out`` that type or float32;
    ``state`` float32 [state rows, rows, N]."""
    _need_cuda(out, x, bc, dt, z, dt_bias, a_log, d_skip, state, state_slots, cu_q)
    T, rows = x.shape
    assert out.shape == (T, rows) and out.stride(1) == 1 and x.stride(1) == 1 and bc.stride(1) == 1 and dt.stride(1) == 1
    assert x.dtype == bc.dtype == dt.dtype and (z is None or (z.dtype == x.dtype and z.stride(1) == 1 and z.shape == x.shape))
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (rows, n_state)
    entries = rows if per_row else rows // rows_per_head
    assert dt_bias.dtype == torch.float32 and dt_bias.numel() == entries and dt.shape[1] >= entries
    assert a_log.dtype == torch.float32 and a_log.is_contiguous() and a_log.numel() == (rows * n_state if per_row else entries)
    assert d_skip is None or (d_skip.dtype == torch.float32 and d_skip.numel() == entries)
    _check(core().le_ssm_scan(_ptr(out), dtype_code(out.dtype), out.stride(0), _ptr(x), x.stride(0), _ptr(bc), bc.stride(0),
                              int(b_col), int(c_col), _ptr(dt), dt.stride(0), _ptr(z), z.stride(0) if z is not None else 0,
                              dtype_code(x.dtype), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(state), state.shape[0],
                              _ptr(state_slots), _ptr(cu_q), int(num_requests), T, rows, int(n_state), int(rows_per_head),
                              int(rows_per_group), 1 if per_row else 0, float(out_scale), _stream()), "le_ssm_scan")


def mlstm_rows(dim: int, vdim: int) -> int:
    """The columns of a head's matrix memory that one block of ``mlstm_scan``
    takes (a divisor of ``vdim``); the state's layout follows it."""
    return int(core().le_mlstm_rows(int(dim), int(vdim)))


def mlstm_state_shape(heads: int, dim: int, vdim: int) -> tuple:
    """The shape of a request's state for ``mlstm_scan``: per head and block
    the block's columns of S, its copy of n, and a row whose first entry is m."""
    r = mlstm_rows(dim, vdim)
    return (heads, vdim // r, r + 2, dim)


def mlstm_scan(out, rows, q_col: int, k_col: int, v_col: int, i_col: int, f_col: int, i_bias, f_bias, state, state_slots, cu_q,
               num_requests: int, heads: int, dim: int, vdim: int, cap: float, q_scale: float) -> None:
    """The mLSTM's matrix memory over the step's tokens, request by request.
    ``rows``: per token q, k [heads, dim], v [heads, vdim] and one gate
    pre-activation per head for the input and the forget gate, at the given
    columns.  With i = cap tanh((a_i + b_i) / cap), f = logsigmoid(cap
    tanh((a_f + b_f) / cap)) and a running maximum m (from 0):
        m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k
        out = S^T (q * q_scale) / (max(|n . q * q_scale|, e^(-m')) + 1e-6)
    ``out`` float32 [T, heads * vdim]; ``state`` float32 [state rows,
    *mlstm_state_shape()]."""
    _need_cuda(out, rows, i_bias, f_bias, state, state_slots, cu_q)
    T = rows.shape[0]
    assert out.dtype == torch.float32 and out.shape == (T, heads * vdim) and out.stride(1) == 1 and rows.stride(1) == 1
    assert i_bias.dtype == torch.float32 and f_bias.dtype == torch.float32 and i_bias.numel() == heads and f_bias.numel() == heads
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == mlstm_state_shape(heads, dim, vdim)
    _check(core().le_mlstm_scan(_ptr(out), out.stride(0), _ptr(rows), rows.stride(0), int(q_col), int(k_col), int(v_col),
                                int(i_col), int(f_col), dtype_code(rows.dtype), _ptr(i_bias), _ptr(f_bias), _ptr(state),
                                state.shape[0], _ptr(state_slots), _ptr(cu_q), int(num_requests), int(heads), int(dim), int(vdim),
                                float(cap), float(q_scale), _stream()), "le_mlstm_scan")


def rope_qknorm_store(rows, bias, w_q, w_k, eps, q_count, k_count, rates, rot, magnitude, k_cache, v_cache, positions,
                      request_of_token, block_table, heads, kv_heads, head_dim, page_size, write_kv, status) -> None:
    """Rows hold q [heads, head_dim] | k [kv_heads, head_dim] | v [kv_heads,
    head_dim].  ``bias`` (float32, the rows' width, or None) is added; q as a
    whole (and k as a whole) is divided by sqrt(sum of squares / ``q_count`` +
    eps) and multiplied by ``w_q`` (``w_k``), float32, both None for no norm;
    in every head of q and k entry i < rot / 2 turns with entry i + rot / 2 by
    position * rates[i] (``rates`` float64: the angle is taken in 64 bits),
    cosine and sine times ``magnitude``.  Queries are
    rewritten in place; keys and values go to the caches' pages when
    ``write_kv``."""
    _need_cuda(rows, bias, w_q, w_k, rates, k_cache, v_cache, positions, block_table)
    T = rows.shape[0]
    width = (heads + 2 * kv_heads) * head_dim
    assert rows.stride(1) == 1 and rows.shape[1] >= width
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == width)
    assert (w_q is None) == (w_k is None)
    assert w_q is None or (w_q.dtype == torch.float32 and w_q.numel() == heads * head_dim and w_k.dtype == torch.float32
                           and w_k.numel() == kv_heads * head_dim and w_q.is_contiguous() and w_k.is_contiguous())
    assert rates.dtype == torch.float64 and rates.is_contiguous() and rates.numel() >= rot // 2
    pages = 0
    if write_kv:
        assert k_cache.dtype == rows.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (kv_heads, page_size, head_dim) and v_cache.shape == k_cache.shape
        pages = k_cache.shape[0]
    _check(core().le_rope_qknorm_store(_ptr(rows), rows.stride(0), dtype_code(rows.dtype), _ptr(bias), _ptr(w_q), _ptr(w_k),
                                       float(eps), int(q_count), int(k_count), _ptr(rates), int(rot), float(magnitude),
                                       _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None,
                                       _ptr(positions), _ptr(request_of_token), _ptr(block_table), block_table.shape[1], T,
                                       heads, kv_heads, head_dim, page_size, pages, 1 if write_kv else 0, _ptr(status),
                                       _stream()), "le_rope_qknorm_store")
