"""ctypes binding of the C ABI declared in ``include/fp8w8a16_b200.h``.

The shared library is the product: there is no Python or CPU fallback.  If it is
missing, importing this module raises, and so does every op.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_int32, c_int64, c_size_t, c_void_p, c_char_p, POINTER
from pathlib import Path

import os

# FP8W8A16_LIBRARY names another build of the library (a debug or instrumented build, say); default: the in-tree one.
LIB_PATH = Path(os.environ.get("FP8W8A16_LIBRARY") or (Path(__file__).resolve().parent / "lib" / "libfp8w8a16_b200.so"))

OK = 0
ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_DEVICE = -1, -2, -3, -4, -5
SCALE_F16, SCALE_F32 = 0, 1
DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
ALGO_AUTO, ALGO_GEMV, ALGO_TC = 0, 1, 2
ACT_SILU, ACT_GELU = 1, 2
COMM_HANDLE_BYTES = 64
VARIANT_NAMES = ("gemv", "tc_cluster", "tc_streamk", "tc_tiles", "grouped", "grouped_paired", "fused_allreduce", "dequant")

# name -> (restype, argtypes); mirrors include/fp8w8a16_b200.h one to one
PROTOTYPES = {
    "fp8w8a16_version": (c_int, []),
    "fp8w8a16_last_error": (c_char_p, []),
    "fp8w8a16_launch_count": (ctypes.c_uint64, []),
    "fp8w8a16_device_status": (c_int, [POINTER(c_int), c_int]),
    "fp8w8a16_variant_counts": (c_int, [POINTER(ctypes.c_uint64), c_int]),
    "fp8w8a16_e4m3_to_fp16": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "fp8w8a16_e4m3_to_fp16_scaled": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "fp8w8a16_dequant_block_scaled": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "fp8w8a16_linear_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "fp8w8a16_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_void_p, c_size_t, c_void_p]),
    "fp8w8a16_linear_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "fp8w8a16_comm_create": (c_int, [c_int, c_int, c_int64, ctypes.c_uint, POINTER(c_void_p)]),
    "fp8w8a16_comm_export": (c_int, [c_void_p, c_void_p]),
    "fp8w8a16_comm_attach": (c_int, [c_void_p, c_int, c_void_p]),
    "fp8w8a16_comm_attach_ptr": (c_int, [c_void_p, c_int, c_void_p]),
    "fp8w8a16_comm_base": (c_void_p, [c_void_p]),
    "fp8w8a16_comm_bytes": (c_size_t, [c_void_p]),
    "fp8w8a16_comm_reset": (c_int, [c_void_p, c_void_p]),
    "fp8w8a16_comm_destroy": (c_int, [c_void_p]),
    "fp8w8a16_linear_allreduce": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int, c_void_p, c_size_t, c_void_p]),
    "fp8w8a16_linear_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p, c_size_t, c_void_p]),
    "fp8w8a16_linear_allreduce_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                                   c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "fp8w8a16_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_float, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "fp8w8a16_moe_topk_softmax": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "fp8w8a16_moe_router_topk": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, ctypes.c_float,
                                         c_void_p, c_void_p, c_void_p, c_void_p]),
    "fp8w8a16_moe_align": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p]),
    "fp8w8a16_moe_token_tile": (c_int, [c_int, c_int]),
    "fp8w8a16_moe_grouped_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "fp8w8a16_moe_grouped_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "fp8w8a16_moe_forward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                     c_size_t, c_void_p]),
    "fp8w8a16_moe_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "fp8w8a16_moe_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "fp8w8a16_moe_combine": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "fp8w8a16_ep_create": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, ctypes.c_uint, POINTER(c_void_p)]),
    "fp8w8a16_ep_export": (c_int, [c_void_p, c_void_p]),
    "fp8w8a16_ep_attach": (c_int, [c_void_p, c_int, c_void_p]),
    "fp8w8a16_ep_attach_ptr": (c_int, [c_void_p, c_int, c_void_p]),
    "fp8w8a16_ep_base": (c_void_p, [c_void_p]),
    "fp8w8a16_ep_bytes": (c_size_t, [c_void_p]),
    "fp8w8a16_ep_reset": (c_int, [c_void_p, c_void_p]),
    "fp8w8a16_ep_destroy": (c_int, [c_void_p]),
    "fp8w8a16_ep_workspace_bytes": (c_size_t, [c_void_p, c_int, c_int, c_int, c_int]),
    "fp8w8a16_ep_dispatch": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "fp8w8a16_ep_experts": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                    c_void_p, c_size_t, c_void_p]),
    "fp8w8a16_ep_combine": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "fp8w8a16_ep_moe_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library (once).  Raises RuntimeError if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m vllm_fp8_w8a16_sm70_b200.build` "
                "(there is no fallback path)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    msg = load().fp8w8a16_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, what: str) -> None:
    """Non-zero status -> RuntimeError, the way the reference's TORCH_CHECK surfaces in Python
    (src/fp8_w8a16_sm70/fp8_dequant.cu:1518-1537)."""
    if rc != OK:
        raise RuntimeError(f"{what} failed (code {rc}): {last_error()}")


def device_status(reset: bool = True) -> int:
    st = c_int(0)
    check(load().fp8w8a16_device_status(ctypes.byref(st), 1 if reset else 0), "fp8w8a16_device_status")
    return st.value


def variant_counts() -> dict:
    """Calls served so far in this process, by kernel variant (FP8W8A16_VARIANT_* order)."""
    buf = (ctypes.c_uint64 * len(VARIANT_NAMES))()
    n = load().fp8w8a16_variant_counts(buf, len(VARIANT_NAMES))
    if n != len(VARIANT_NAMES):
        raise RuntimeError(f"library reports {n} kernel variants, this binding knows {len(VARIANT_NAMES)}")
    return dict(zip(VARIANT_NAMES, (int(v) for v in buf)))
