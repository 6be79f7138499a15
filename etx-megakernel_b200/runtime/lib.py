"""ctypes binding of libetxb200.so (include/etxb200.h) and the nvcc recipe that builds it.

There is no CPU fallback: if the shared library is missing or a symbol does not resolve, loading raises; every call
that returns a non-zero status raises EtxbError with the library's message.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parents[1]
CSRC = PKG / "csrc"
LIB_PATH = PKG / "libetxb200.so"
SOURCES = ["etxb.cu"]
HEADERS = ["etxb_abi.h", "etxb_prims.cuh", "etxb_gemv.cuh", "etxb_gemv_nb.cuh", "etxb_attn.cuh", "etxb_attn_fused.cuh", "etxb_attn_gq.cuh", "etxb_batch.cuh", "etxb_tc.cuh", "etxb_mla.cuh", "etxb_kernel.cuh"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
              "-shared", "-Xcompiler", "-fPIC"]

STATUS = {0: "OK", 1: "E_ARG", 2: "E_PLAN", 3: "E_CUDA", 4: "E_RESIDENCY", 5: "E_TIMEOUT", 6: "E_ABORTED", 7: "E_UNSUPPORTED"}
BODY = {"nop": 0, "prologue": 1, "argmax": 2, "gemv": 3, "moe_up": 4, "moe_down": 5, "topk": 6, "attnprep": 7, "attn": 8,
        "attn_reduce": 9, "splitk_part": 10, "splitk_sum": 11, "attn_fused": 12, "norm_col": 13, "gemv_nb": 14, "route": 15,
        "moe_up_g": 16, "moe_down_g": 17, "prologue_nb": 18, "argmax_nb": 19, "gemv_tc": 20, "moe_up_tc": 21, "moe_down_tc": 22, "mla_attn": 23}

# every symbol include/etxb200.h declares
SYMBOLS = ["etxb_version", "etxb_last_error", "etxb_device_info", "etxb_create", "etxb_bind", "etxb_set_step", "etxb_set_option",
           "etxb_launch", "etxb_launch_unfused", "etxb_wait", "etxb_step", "etxb_status", "etxb_trace", "etxb_exec_counts", "etxb_destroy",
           "etxb_decode_host", "etxb_op_launch", "etxb_attn_fused_static", "etxb_exchange_alloc", "etxb_exchange_free", "etxb_exchange_open",
           "etxb_exchange_close", "etxb_set_exchange"]
IPC_HANDLE_BYTES = 64


class EtxbError(RuntimeError):
    def __init__(self, code: int, message: str):
        self.code, self.status = code, STATUS.get(code, str(code))
        super().__init__(f"{self.status}: {message}")


class StepParams(C.Structure):
    _fields_ = [("tok", C.c_int32), ("pos", C.c_int32), ("write_next", C.c_int32), ("H", C.c_int32), ("V", C.c_int32), ("nrep", C.c_int32),
                ("embed", C.c_void_p), ("resid", C.c_void_p), ("positions", C.c_void_p), ("seq_lens", C.c_void_p),
                ("slot_mapping", C.c_void_p), ("logits", C.c_void_p), ("token_in", C.c_void_p), ("token_out", C.c_void_p),
                ("token_time", C.c_void_p)]


class Status(C.Structure):
    _fields_ = [("ctrl", C.c_int32), ("stuck_task", C.c_int32), ("stuck_event", C.c_int32), ("stuck_value", C.c_int32),
                ("stuck_target", C.c_int32), ("tasks_run", C.c_int32), ("epoch", C.c_uint32), ("last_ms", C.c_float), ("kernel_variant", C.c_int32)]


class DeviceInfo(C.Structure):
    _fields_ = [("sm_count", C.c_int32), ("smem_per_block_optin", C.c_int32), ("l2_bytes", C.c_int32), ("cc_major", C.c_int32),
                ("cc_minor", C.c_int32), ("workers", C.c_int32), ("threads", C.c_int32), ("smem_bytes", C.c_int32), ("hbm_bytes", C.c_uint64)]


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any((CSRC / f).stat().st_mtime > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA library for sm_100a in-tree (nvcc cross-compiles without a GPU)."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIB_PATH), *[str(CSRC / s) for s in SOURCES]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stderr)
    return LIB_PATH


_lib = None


def load():
    """The loaded library with argument types set; raises if it is missing (no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise FileNotFoundError(f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()'); "
                                "there is no CPU path")
    lib = C.CDLL(str(LIB_PATH))
    missing = [s for s in SYMBOLS if not hasattr(lib, s)]
    if missing:
        raise ImportError(f"{LIB_PATH} does not export {missing}")
    vp, i32, sz = C.c_void_p, C.c_int32, C.c_size_t
    lib.etxb_version.restype = i32
    lib.etxb_last_error.restype = C.c_char_p
    proto = {
        "etxb_device_info": [C.c_int, C.POINTER(DeviceInfo)], "etxb_create": [vp, sz, C.c_int, C.POINTER(vp)],
        "etxb_bind": [vp, C.c_char_p, vp, sz], "etxb_set_step": [vp, C.POINTER(StepParams)], "etxb_set_option": [vp, C.c_char_p, C.c_int64],
        "etxb_launch": [vp, vp], "etxb_launch_unfused": [vp, vp], "etxb_wait": [vp, C.c_double], "etxb_step": [vp, vp, C.c_double], "etxb_status": [vp, C.POINTER(Status)],
        "etxb_trace": [vp, vp, sz], "etxb_exec_counts": [vp, vp, sz], "etxb_destroy": [vp],
        "etxb_decode_host": [vp, vp, i32, i32, i32, vp, vp], "etxb_op_launch": [C.c_int, i32, vp, sz, i32, C.POINTER(StepParams), vp],
        "etxb_attn_fused_static": [C.c_int, vp, sz, vp],
        "etxb_exchange_alloc": [C.c_int, sz, C.POINTER(vp), vp], "etxb_exchange_free": [C.c_int, vp],
        "etxb_exchange_open": [C.c_int, vp, C.POINTER(vp)], "etxb_exchange_close": [C.c_int, vp],
        "etxb_set_exchange": [vp, i32, i32, vp, sz, C.POINTER(vp)],
    }
    for name, args in proto.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, i32
    _lib = lib
    return lib


def check(code: int):
    if code != 0:
        raise EtxbError(code, load().etxb_last_error().decode(errors="replace"))


def device_info(device: int = 0) -> DeviceInfo:
    info = DeviceInfo()
    check(load().etxb_device_info(device, C.byref(info)))
    return info
