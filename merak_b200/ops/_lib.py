"""ctypes bindings of the sm_100a kernel library (``_mrk_kernels.so``) and of the host-only
native library (``_mrk_native.so``).

The kernel library is mandatory on a machine with a GPU: :func:`kernels` raises instead of
letting callers fall back silently to eager PyTorch.  On a CPU-only machine the ops in this
package run their PyTorch reference implementations, which is what the CPU test-suite checks.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_KERNEL_LIB_PATH = os.path.join(_PKG_DIR, "_mrk_kernels.so")
_NATIVE_LIB_PATH = os.path.join(_PKG_DIR, "_mrk_native.so")

_lock = threading.Lock()
_kernels = None
_native = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


class KernelError(RuntimeError):
    """A native entry point returned a non-zero code."""


def _maybe_build():
    if os.environ.get("MERAK_B200_NO_BUILD") == "1":
        return
    try:
        from .. import build as _build

        _build.build()
    except Exception as exc:  # pragma: no cover - surfaced by the caller
        raise RuntimeError("building the native libraries failed: %s" % exc) from exc


def _declare(lib):
    def sig(name, restype, *argtypes):
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.restype = restype
            fn.argtypes = list(argtypes)

    sig("mrk_last_error", ctypes.c_char_p)
    sig("mrk_status_read", ctypes.c_uint, c_int)
    sig("mrk_abi_version", c_int)
    sig("mrk_launch_count", ctypes.c_ulonglong)
    sig("mrk_gemm_bf16", c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_ll,
        c_void_p, c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_int, c_float, c_int, c_void_p)
    c_ull = ctypes.c_ulonglong
    P = c_void_p
    sig("mrk_attn_fwd", c_int, *([P] * 6 + [c_int] * 6 + [c_ll] * 12 + [c_int, c_float, P]))
    sig("mrk_attn_bwd", c_int, *([P] * 12 + [c_int] * 6 + [P, c_int, c_float, P]))
    sig("mrk_attn_fwd_drop", c_int, *([P] * 6 + [c_int] * 6 + [c_ll] * 12 + [c_int, c_float, c_float, P, c_ull, P]))
    sig("mrk_attn_bwd_drop", c_int, *([P] * 12 + [c_int] * 6 + [P, c_int, c_float, c_float, P, c_ull, P]))
    sig("mrk_norm_fwd", c_int, P, P, P, P, P, P, P, P, P, c_ull, c_float, c_float, c_ll, c_int, c_int, c_int, P)
    sig("mrk_norm_bwd", c_int, P, P, P, P, P, P, P, P, P, P, P, P, c_ull, c_float, c_ll, c_int, c_int, c_int, P)
    sig("mrk_norm_bwd_workspace_rows", c_int)
    sig("mrk_ce_stats", c_int, P, P, P, c_ll, c_int, c_ll, c_int, c_int, c_int, P)
    sig("mrk_ce_finalize", c_int, P, c_int, c_ll, P, P, P, P, P, c_ll, c_int, P)
    sig("mrk_ce_grad", c_int, P, P, P, P, P, c_ll, c_int, c_ll, c_ll, c_int, c_int, c_int, P)
    sig("mrk_adamw", c_int, P, P, P, P, P, P, P, P, c_ll, c_int, c_int, P)
    sig("mrk_sumsq", c_int, P, c_ll, P, c_int, P)
    sig("mrk_clip_coef", c_int, P, c_float, c_float, P, P, P, P)
    sig("mrk_embedding_fwd", c_int, P, P, P, P, c_int, P, c_ll, c_int, P)
    sig("mrk_embedding_bwd", c_int, P, P, P, c_ll, c_int, c_int, c_int, c_int, P)
    sig("mrk_rope", c_int, P, P, P, P, P, c_ll, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_int, P)
    sig("mrk_swiglu_fwd", c_int, P, P, c_ll, c_int, c_ll, P)
    sig("mrk_act_fwd", c_int, P, P, c_ll, c_int, P)
    sig("mrk_act_bwd", c_int, P, P, P, P, c_ll, c_int, c_ll, c_int, P)
    sig("mrk_swiglu_bwd", c_int, P, P, P, c_ll, c_int, c_ll, P)
    sig("mrk_colsum", c_int, P, P, c_ll, c_int, c_ll, P)
    sig("mrk_dropout", c_int, P, P, c_ll, c_float, P, c_ull, P)
    sig("mrk_scaled_cast", c_int, P, P, c_ll, P, c_float, c_int, c_int, c_int, P)
    c_uint = ctypes.c_uint
    sig("mrk_symm_alloc", c_int, c_ull, P)
    sig("mrk_symm_free", c_int, P)
    sig("mrk_symm_ctrl_bytes", c_int)
    sig("mrk_ipc_handle_bytes", c_int)
    sig("mrk_ipc_get_handle", c_int, P, P)
    sig("mrk_ipc_open", c_int, P, P)
    sig("mrk_ipc_close", c_int, P)
    sig("mrk_dp_reduce_scatter", c_int, P, P, c_int, c_int, c_ll, c_ll, P, c_uint, c_int, c_int, P)
    sig("mrk_dp_adamw_allgather", c_int, P, P, c_int, c_int, c_ll, c_ll, P, P, P, P, P, P, c_float, c_float,
        P, P, P, c_uint, c_int, c_int, c_int, P)
    sig("mrk_sample_topk_topp", c_int, P, c_int, c_ll, c_int, c_ll, c_int, c_float, c_float, c_int, P,
        ctypes.c_ulonglong, ctypes.c_ulonglong, P, P, P)
    sig("mrk_memcpy_d2d_async", c_int, P, P, ctypes.c_ulonglong, P)
    sig("mrk_dp_norm_gather", c_int, P, c_int, c_int, P, c_uint, c_int, c_int, P)
    sig("mrk_tp_reduce_pull", c_int, P, P, c_int, c_int, P, c_ll, c_int, c_int, P, c_uint, c_int, c_int, P)
    sig("mrk_tp_gather_rows", c_int, P, P, c_int, c_int, P, c_ll, c_int, c_int, c_uint, c_int, c_int, P)
    sig("mrk_gemm_bf16_rs_units", c_int, c_int, c_int)
    sig("mrk_gemm_bf16_rs", c_int, P, P, P, P, P, P, c_int, c_int, c_int, c_ll, c_ll, c_int, c_int, c_int, c_int,
        c_uint, c_int, c_int, P, c_int, P)
    sig("mrk_gemm_bf16_ag", c_int, P, P, P, P, c_int, c_int, c_int, c_ll, c_ll, P, P, c_ll, c_int, c_int, c_float,
        P, P, c_uint, c_int, c_int, c_int, c_int, c_uint, c_int, P)
    sig("mrk_moe_alltoall_push", c_int, P, P, c_int, c_int, P, P, P, c_int, c_int, c_uint, c_int, c_int, P)
    sig("mrk_symm_barrier", c_int, P, c_int, c_int, c_int, c_uint, c_int, c_int, P)
    return lib


def kernels():
    """Returns the loaded kernel library, building it first if the shared object is missing."""
    global _kernels
    if _kernels is not None:
        return _kernels
    with _lock:
        if _kernels is None:
            if not os.path.exists(_KERNEL_LIB_PATH):
                _maybe_build()
            if not os.path.exists(_KERNEL_LIB_PATH):
                raise RuntimeError(
                    "merak_b200: %s is missing; run `python -m merak_b200.build`" % _KERNEL_LIB_PATH)
            _kernels = _declare(ctypes.CDLL(_KERNEL_LIB_PATH))
    return _kernels


def native():
    """Returns the host-only native library (AutoPipe partitioner, schedule simulator)."""
    global _native
    if _native is not None:
        return _native
    with _lock:
        if _native is None:
            if not os.path.exists(_NATIVE_LIB_PATH):
                _maybe_build()
            if not os.path.exists(_NATIVE_LIB_PATH):
                raise RuntimeError(
                    "merak_b200: %s is missing; run `python -m merak_b200.build`" % _NATIVE_LIB_PATH)
            _native = ctypes.CDLL(_NATIVE_LIB_PATH)
    return _native


def use_kernels(*tensors) -> bool:
    """True when the inputs live on a CUDA device, i.e. the sm_100a kernels must run."""
    return len(tensors) > 0 and all(t is None or t.is_cuda for t in tensors) and any(
        t is not None for t in tensors)


_FALLBACK_SEEN = set()


def note_library_fallback(op: str, x) -> None:
    """A CUDA tensor reached an op whose sm_100a kernel does not take its dtype / shape (the kernels
    are bf16), so a PyTorch library op runs instead.  Said once per (op, dtype) so it is never
    silent; ``MERAK_STRICT_KERNELS=1`` turns it into an error."""
    if x is None or not getattr(x, "is_cuda", False):
        return                                        # CPU tensors: the PyTorch formulation is the path
    key = (op, str(x.dtype), tuple(x.shape[-1:]))
    if key in _FALLBACK_SEEN:
        return
    _FALLBACK_SEEN.add(key)
    msg = ("%s: no sm_100a kernel for dtype %s / last dim %d on a CUDA tensor; running the PyTorch library op"
           % (op, x.dtype, x.shape[-1]))
    if os.environ.get("MERAK_STRICT_KERNELS", "0") == "1":
        raise KernelError(msg)
    import warnings
    warnings.warn(msg, RuntimeWarning, stacklevel=3)


def check(rc: int, what: str):
    if rc != 0:
        msg = kernels().mrk_last_error()
        raise KernelError("%s failed (code %d): %s" % (what, rc, msg.decode() if msg else "?"))


def status(clear: bool = False) -> int:
    """Status word of the current device: non-zero after a device-side bounded wait gave up."""
    return int(kernels().mrk_status_read(1 if clear else 0))


def assert_status_ok(what: str = ""):
    s = status(clear=True)
    if s != 0:
        raise KernelError("device status word is 0x%x after %s (1=mbarrier timeout, 2=peer-flag "
                          "timeout, 4=bad argument)" % (s, what or "kernel"))


def launch_count() -> int:
    """Kernels launched by the library so far in this process."""
    return int(kernels().mrk_launch_count())


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream
