"""ctypes binding of libfluxb200.so (declared in include/fluxb200.h).

The library is the only compute path: if it has not been built the import of any kernel
wrapper raises, and tensors that are not on a CUDA device are rejected — there is no CPU or
PyTorch fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p, POINTER
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libfluxb200.so"

F32, BF16 = 0, 1
EPI_NONE, EPI_GELU, EPI_GATE_RESID = 0, 1, 2
ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT = -1, -2, -3, -4

# name -> (restype, argtypes); mirrors include/fluxb200.h one to one.
_P, _I, _L, _F = c_void_p, c_int, c_int64, c_float


class LinearProblem(ctypes.Structure):
    """fluxb_linear_problem of include/fluxb200.h."""

    _fields_ = [
        ("x", _P), ("w", _P), ("bias", _P), ("y", _P),
        ("M", _L), ("ldx", _L), ("ldw", _L), ("ldy", _L),
        ("y2", _P), ("ldy2", _L), ("resid", _P), ("ldr", _L),
        ("gate", _P), ("gate_stride", _L), ("rows_per_batch", _L),
    ]


class QkvStream(ctypes.Structure):
    """fluxb_qkv_stream of include/fluxb200.h."""

    _fields_ = [("pe", _P), ("q_scale", _P), ("k_scale", _P), ("row_offset", _L)]


SIGNATURES = {
    "fluxb_version": (_I, []),
    "fluxb_last_error": (c_char_p, []),
    "fluxb_device_status_read": (_I, [POINTER(c_int)]),
    "fluxb_linear": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _I, _P, _L, _L, _I, _P, _L, _P, _L, _L, _I, _P]),
    "fluxb_linear_grouped": (_I, [POINTER(LinearProblem), _I, _L, _L, _I, _L, _I, _I, _P]),
    "fluxb_linear_qkv_grouped": (_I, [POINTER(LinearProblem), POINTER(QkvStream), _I, _L, _L, _L, _L, _L, _P, _F, _L, _I, _I, _P]),
    "fluxb_linear_qkv_grouped_scatter": (_I, [POINTER(LinearProblem), POINTER(QkvStream), _I, _L, _L, _L, _L, _L,
                                              POINTER(c_void_p), _I, _L, _L, _L, _L, _L, _F, _L, _I, _I, _P]),
    "fluxb_modulation_gemv": (_I, [_P, _P, _P, _P, _L, _L, _L, _I, _P]),
    "fluxb_modulation_gemv_rows": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _I, _I, _P]),
    "fluxb_attention": (_I, [_P, _P, _P, _P] + [_L] * 5 + [_L] * 12 + [_F, _P]),
    "fluxb_layer_norm_modulation": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _F, _I, _P]),
    "fluxb_rms_norm": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _F, _I, _P]),
    "fluxb_rms_norm_bwd_partial_rows": (_L, [_L]),
    "fluxb_rms_norm_bwd": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _I, _P]),
    "fluxb_rms_norm_bwd_static_max_floats": (_I, []),
    "fluxb_rms_norm_bwd_static": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _I, _P]),
    "fluxb_rope": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _I, _P]),
    "fluxb_qkv_prep": (_I, [_P, _L, _L, _P, _P, _P, _L, _L, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _F, _P]),
    "fluxb_modulation_scale_shift": (_I, [_P, _P, _P, _L, _L, _L, _L, _I, _I, _P]),
    "fluxb_modulation_gate_proj": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _I, _I, _P]),
    "fluxb_silu": (_I, [_P, _P, _L, _I, _P]),
    "fluxb_peer_header_bytes": (_I, []),
    "fluxb_peer_alloc": (_I, [_L, POINTER(c_void_p)]),
    "fluxb_peer_free": (_I, [_P]),
    "fluxb_peer_export": (_I, [_P, _P]),
    "fluxb_peer_open": (_I, [_P, POINTER(c_void_p)]),
    "fluxb_peer_close": (_I, [_P]),
    "fluxb_peer_signal": (_I, [POINTER(c_void_p), _I, _I, _I, _P]),
    "fluxb_peer_wait": (_I, [POINTER(c_void_p), _I, _I, _I, _P]),
    "fluxb_qkv_prep_scatter": (_I, [_P, _L, _L, _P, _P, _P, _L, _L, _P, _P, _P, POINTER(c_void_p), _I, _L, _L,
                                    _L, _L, _L, _L, _L, _L, _L, _F, _P]),
    "fluxb_attention_split": (_I, [_P, _P, _P, _P, POINTER(c_void_p), _I, _L] + [_L] * 5 + [_L] * 12 + [_F, _I, _P, _P, _P]),
    "fluxb_attention_scatter": (_I, [_P, _P, _P, POINTER(c_void_p), _I, _L] + [_L] * 5 + [_L] * 12 + [_F, _P]),
}

_lib = None
kernel_calls = 0  # C-ABI compute calls that returned success (each launches at least one kernel)


class FluxbError(RuntimeError):
    """A C-ABI call returned a CUDA / timeout error code."""


def load() -> ctypes.CDLL:
    """Loads the shared library once and declares every signature."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m triton_kernels_b200.build` "
                "(there is no fallback path)"
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(rc: int, launches: bool = True) -> None:
    """Turns a status code into the Python exception the reference API would raise.  Setup calls
    that launch nothing pass launches=False so that `kernel_calls` counts kernels only."""
    global kernel_calls
    if rc == 0:
        if launches:
            kernel_calls += 1
        return
    msg = load().fluxb_last_error().decode()
    if rc == ERR_BAD_ARG:
        raise ValueError(msg)
    if rc == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise FluxbError(f"fluxb200 error {rc}: {msg}")


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float32:
        return F32
    raise NotImplementedError(f"fluxb200 kernels take float32 or bfloat16 tensors, got {t.dtype}")


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "fluxb200 kernels run on CUDA tensors only (no CPU fallback); got a tensor on " f"{t.device}"
            )


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_handle() -> int:
    return torch.cuda.current_stream().cuda_stream


def device_status() -> tuple[int, int]:
    """Reads (and clears) the device status word: (code, where).  Synchronises the device."""
    out = (c_int * 2)()
    check(load().fluxb_device_status_read(out))
    return out[0], out[1]
