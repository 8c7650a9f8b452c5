"""ctypes binding of libevoattn.so (the C ABI declared in include/evoattn.h).

There is no fallback: if the library is missing or a call fails, this module
raises.  Build the library with `python megakernel-exploration_b200/build.py`.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libevoattn.so")

ABI_VERSION = 103


class EvoDims(C.Structure):
    _fields_ = [("B", C.c_int32), ("S", C.c_int32), ("N", C.c_int32),
                ("H", C.c_int32), ("D", C.c_int32)]


class EvoStrides(C.Structure):
    """Element strides of the activation tensors along B, N_SEQ, N_CTX, H (D is contiguous)."""
    _fields_ = [("b", C.c_int64), ("s", C.c_int64), ("n", C.c_int64), ("h", C.c_int64)]


class EvoAttnError(RuntimeError):
    def __init__(self, code: int, what: str, detail: str = ""):
        self.code = code
        super().__init__(f"libevoattn: {what} failed with {code}: {detail}")


# name -> (restype, argtypes); every symbol include/evoattn.h declares
SYMBOLS = {
    "evo_version": (C.c_int, []),
    "evo_strerror": (C.c_char_p, [C.c_int]),
    "evo_last_cuda_error": (C.c_int, []),
    "evo_last_error_detail": (C.c_char_p, []),
    "evo_fwd": (C.c_int, [C.POINTER(EvoDims)] + [C.c_void_p] * 8 + [C.c_float, C.c_void_p]),
    "evo_fwd_strided": (C.c_int, [C.POINTER(EvoDims), C.POINTER(EvoStrides)] + [C.c_void_p] * 8 + [C.c_float, C.c_void_p]),
    "evo_bwd_strided": (C.c_int, [C.POINTER(EvoDims), C.POINTER(EvoStrides)] + [C.c_void_p] * 14
                        + [C.c_size_t, C.c_float, C.c_void_p]),
    "evo_bwd_phased": (C.c_int, [C.POINTER(EvoDims), C.POINTER(EvoStrides)] + [C.c_void_p] * 14
                       + [C.c_size_t, C.c_float, C.c_uint, C.c_int, C.c_void_p]),
    "evo_fwd_gated": (C.c_int, [C.POINTER(EvoDims), C.POINTER(EvoStrides)] + [C.c_void_p] * 10 + [C.c_float, C.c_void_p]),
    "evo_fwd_views": (C.c_int, [C.POINTER(EvoDims), C.POINTER(EvoStrides), C.POINTER(EvoStrides)] + [C.c_void_p] * 10
                      + [C.c_float, C.c_void_p]),
    "evo_bwd_views": (C.c_int, [C.POINTER(EvoDims)] + [C.POINTER(EvoStrides)] * 3 + [C.c_void_p] * 16
                      + [C.c_size_t, C.c_float, C.c_uint, C.c_int, C.c_void_p]),
    "evo_bwd_gated": (C.c_int, [C.POINTER(EvoDims), C.POINTER(EvoStrides)] + [C.c_void_p] * 16
                      + [C.c_size_t, C.c_float, C.c_uint, C.c_int, C.c_void_p]),
    "evo_bwd_gated_workspace_bytes": (C.c_size_t, [C.POINTER(EvoDims)]),
    "evo_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(EvoDims)]),
    "evo_bwd": (C.c_int, [C.POINTER(EvoDims)] + [C.c_void_p] * 14 + [C.c_size_t, C.c_float, C.c_void_p]),
    "evo_bwd_static_scratch_capacity": (C.c_size_t, []),
    "evo_bwd_static_scratch": (C.c_int, [C.POINTER(EvoDims)] + [C.c_void_p] * 13 + [C.c_float, C.c_void_p]),
    "evo_device_status": (C.c_int, [C.POINTER(C.c_uint32)]),
    "evo_selftest_mma": (C.c_int, [C.c_int] + [C.c_void_p] * 8),
    "evo_selftest_mma_extra": (C.c_int, [C.c_int] + [C.c_void_p] * 6),
    "evo_selftest_wait_timeout": (C.c_int, [C.c_ulonglong, C.c_void_p, C.c_void_p]),
    "evo_profile_enable": (C.c_int, [C.c_int]),
    "evo_profile_read": (C.c_int, [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_int)]),
}

_lib = None
_lock = threading.Lock()


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise ImportError(
                    f"{LIB_PATH} not found: build it with "
                    f"`python {os.path.join(HERE, 'build.py')}` (needs nvcc, sm_100a)")
            h = C.CDLL(LIB_PATH)
            for name, (res, args) in SYMBOLS.items():
                fn = getattr(h, name)   # AttributeError if the symbol is not exported
                fn.restype = res
                fn.argtypes = args
            v = h.evo_version()
            if v // 100 != ABI_VERSION // 100:
                raise ImportError(f"libevoattn ABI {v} does not match binding {ABI_VERSION}")
            _lib = h
    return _lib


def strerror(code: int) -> str:
    return lib().evo_strerror(code).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        detail = strerror(code)
        if code == -7:
            detail += f" (cudaError {lib().evo_last_cuda_error()})"
        if code == -6:
            detail += f" ({lib().evo_last_error_detail().decode()})"
        raise EvoAttnError(code, what, detail)


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def fwd(dims: EvoDims, q, k, v, bias, mask, o, o_resid, lse, scale: float, stream: int) -> None:
    check(lib().evo_fwd(C.byref(dims), _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask),
                        _ptr(o), _ptr(o_resid), _ptr(lse), float(scale), stream), "evo_fwd")


def fwd_strided(dims: EvoDims, strides: EvoStrides, q, k, v, bias, mask, o, o_resid, lse, scale: float,
                stream: int) -> None:
    """evo_fwd on activation views that share the element strides `strides`."""
    check(lib().evo_fwd_strided(C.byref(dims), C.byref(strides), _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask),
                                _ptr(o), _ptr(o_resid), _ptr(lse), float(scale), stream), "evo_fwd_strided")


def bwd_strided(dims: EvoDims, strides: EvoStrides, q, k, v, bias, mask, o, o_resid, lse, d_o, dq, dk, dv, dbias,
                workspace, scale: float, stream: int) -> None:
    check(lib().evo_bwd_strided(C.byref(dims), C.byref(strides), _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask),
                                _ptr(o), _ptr(o_resid), _ptr(lse), _ptr(d_o), _ptr(dq), _ptr(dk), _ptr(dv),
                                _ptr(dbias), _ptr(workspace), workspace.numel() * workspace.element_size(),
                                float(scale), stream), "evo_bwd_strided")


BWD_PHASE_DBIAS, BWD_PHASE_DQKV = 1, 2


def bwd_phased(dims: EvoDims, strides, q, k, v, bias, mask, o, o_resid, lse, d_o, dq, dk, dv, dbias, workspace,
               scale: float, phases: int, reserved_sms: int, stream: int) -> None:
    """One or both phases of the backward (see evo_bwd_phased); strides may be None (contiguous)."""
    check(lib().evo_bwd_phased(C.byref(dims), C.byref(strides) if strides is not None else None,
                               _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask), _ptr(o), _ptr(o_resid),
                               _ptr(lse), _ptr(d_o), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dbias), _ptr(workspace),
                               workspace.numel() * workspace.element_size(), float(scale), int(phases),
                               int(reserved_sms), stream), "evo_bwd_phased")


def fwd_gated(dims: EvoDims, strides, q, k, v, bias, mask, gate, o, o_gated, o_resid, lse, scale: float,
              stream: int) -> None:
    """evo_fwd_strided with the sigmoid gate fused in: o receives the attention output, o_gated
    sigmoid(gate) * O.  strides may be None (contiguous)."""
    check(lib().evo_fwd_gated(C.byref(dims), C.byref(strides) if strides is not None else None,
                              _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask), _ptr(gate), _ptr(o), _ptr(o_gated),
                              _ptr(o_resid), _ptr(lse), float(scale), stream), "evo_fwd_gated")


def bwd_gated_workspace_bytes(dims: EvoDims) -> int:
    return int(lib().evo_bwd_gated_workspace_bytes(C.byref(dims)))


def bwd_gated(dims: EvoDims, strides, q, k, v, bias, mask, gate, o, o_resid, lse, d_out, dq, dk, dv, d_gate, dbias,
              workspace, scale: float, phases: int, reserved_sms: int, stream: int) -> None:
    """Backward of fwd_gated: d_out is the gradient of the gated output; d_gate receives the gate's."""
    check(lib().evo_bwd_gated(C.byref(dims), C.byref(strides) if strides is not None else None,
                              _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask), _ptr(gate), _ptr(o), _ptr(o_resid),
                              _ptr(lse), _ptr(d_out), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(d_gate), _ptr(dbias),
                              _ptr(workspace), workspace.numel() * workspace.element_size(), float(scale),
                              int(phases), int(reserved_sms), stream), "evo_bwd_gated")


def _sref(strides):
    return C.byref(strides) if strides is not None else None


def fwd_views(dims: EvoDims, s_qkv, s_out, q, k, v, bias, mask, gate, o, o_gated, o_resid, lse, scale: float,
              stream: int) -> None:
    """evo_fwd_gated with separate views for q/k/v (s_qkv) and the output side (s_out); None = contiguous."""
    check(lib().evo_fwd_views(C.byref(dims), _sref(s_qkv), _sref(s_out), _ptr(q), _ptr(k), _ptr(v), _ptr(bias),
                              _ptr(mask), _ptr(gate), _ptr(o), _ptr(o_gated), _ptr(o_resid), _ptr(lse), float(scale),
                              stream), "evo_fwd_views")


def bwd_views(dims: EvoDims, s_qkv, s_out, s_grad, q, k, v, bias, mask, gate, o, o_resid, lse, d_out, dq, dk, dv,
              d_gate, dbias, workspace, scale: float, phases: int, reserved_sms: int, stream: int) -> None:
    """evo_bwd_gated with separate views for q/k/v (s_qkv), o/d_out/gate/d_gate (s_out) and dq/dk/dv (s_grad)."""
    check(lib().evo_bwd_views(C.byref(dims), _sref(s_qkv), _sref(s_out), _sref(s_grad), _ptr(q), _ptr(k), _ptr(v),
                              _ptr(bias), _ptr(mask), _ptr(gate), _ptr(o), _ptr(o_resid), _ptr(lse), _ptr(d_out),
                              _ptr(dq), _ptr(dk), _ptr(dv), _ptr(d_gate), _ptr(dbias), _ptr(workspace),
                              workspace.numel() * workspace.element_size(), float(scale), int(phases),
                              int(reserved_sms), stream), "evo_bwd_views")


def bwd_workspace_bytes(dims: EvoDims) -> int:
    return int(lib().evo_bwd_workspace_bytes(C.byref(dims)))


def bwd(dims: EvoDims, q, k, v, bias, mask, o, o_resid, lse, d_o, dq, dk, dv, dbias, workspace,
        scale: float, stream: int) -> None:
    check(lib().evo_bwd(C.byref(dims), _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask),
                        _ptr(o), _ptr(o_resid), _ptr(lse), _ptr(d_o), _ptr(dq), _ptr(dk), _ptr(dv),
                        _ptr(dbias), _ptr(workspace),
                        workspace.numel() * workspace.element_size(), float(scale), stream),
          "evo_bwd")


def bwd_static_scratch(dims: EvoDims, q, k, v, bias, mask, o, o_resid, lse, d_o, dq, dk, dv, dbias,
                       scale: float, stream: int) -> None:
    """evo_bwd with the library's built-in scratch array instead of a caller workspace."""
    check(lib().evo_bwd_static_scratch(C.byref(dims), _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask),
                                       _ptr(o), _ptr(o_resid), _ptr(lse), _ptr(d_o), _ptr(dq), _ptr(dk),
                                       _ptr(dv), _ptr(dbias), float(scale), stream),
          "evo_bwd_static_scratch")


def device_status() -> int:
    """Synchronises the device; raises if a kernel reported a timed-out wait."""
    raw = C.c_uint32(0)
    code = lib().evo_device_status(C.byref(raw))
    if code != 0:
        raise EvoAttnError(code, "evo_device_status",
                           f"{strerror(code)} (status word 0x{raw.value:08x})")
    return 0


def profile_enable(on: bool) -> None:
    check(lib().evo_profile_enable(1 if on else 0), "evo_profile_enable")


def profile_read(kernel: int):
    """(total milliseconds, launches) of kernel 0 (forward) / 1 (backward dQ,dK,dV) / 2 (backward dBias)."""
    ms, n = C.c_float(0.0), C.c_int(0)
    check(lib().evo_profile_read(kernel, C.byref(ms), C.byref(n)), "evo_profile_read")
    return ms.value, n.value


def selftest_mma_extra(D: int, y, z, a, b, out, stream: int) -> None:
    check(lib().evo_selftest_mma_extra(int(D), _ptr(y), _ptr(z), _ptr(a), _ptr(b), _ptr(out), stream),
          "evo_selftest_mma_extra")


def selftest_wait_timeout(limit_ns: int, released, stream: int) -> None:
    """Launches the one-CTA kernel whose wait runs out after `limit_ns` (see evo_selftest_wait_timeout)."""
    check(lib().evo_selftest_wait_timeout(int(limit_ns), _ptr(released), stream), "evo_selftest_wait_timeout")


def selftest_mma(D: int, x, y, z, out_yzt, out_xy, out_xty, out_ts, stream: int) -> None:
    check(lib().evo_selftest_mma(int(D), _ptr(x), _ptr(y), _ptr(z), _ptr(out_yzt), _ptr(out_xy),
                                 _ptr(out_xty), _ptr(out_ts), stream), "evo_selftest_mma")
