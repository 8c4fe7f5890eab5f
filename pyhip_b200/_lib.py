"""ctypes binding of libb200moe.so (the C ABI declared in include/b200moe.h).

Mirrors how the reference reaches its kernels: a lazily loaded, cached ``ctypes.CDLL`` handle,
raw device pointers and the current torch stream passed as ``void*``
(src/core/hiptools.py:10-35,82-100 of tingqli/pyhip); a non-zero status becomes a Python
exception, as the reference's ``HIP error`` exceptions do (hiptools.py:37-39).

There is no fallback: if the shared library is missing or fails to load, importing callers
get an ImportError / RuntimeError that says how to build it.
"""
from __future__ import annotations

import ctypes
import functools
import pathlib
import subprocess

PKG_DIR = pathlib.Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libb200moe.so"
SOURCES = ["api.cu", "moe_aux.cu", "moe_gemm_sm100.cu", "moe_gemm_fp8_sm100.cu", "moe_gemm_bf16_sm100.cu",
           "moe_batch1.cu", "forward_static.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]

W_MXFP4, W_FP8_128, W_FP8_ROW, W_BF16 = 0, 1, 2, 3
ACT_SILU, ACT_SWIGLU = 0, 1
COMBINE_GATHER, COMBINE_FUSED = 0, 1
ACTQ_TERMS, ACTQ_1X128 = 0, 1
ABI_VERSION = 3


class Shape(ctypes.Structure):
    _fields_ = [("T", ctypes.c_int32), ("K", ctypes.c_int32), ("E", ctypes.c_int32),
                ("E_route", ctypes.c_int32), ("H", ctypes.c_int32), ("I", ctypes.c_int32),
                ("B", ctypes.c_int32), ("weight_format", ctypes.c_int32),
                ("activation", ctypes.c_int32), ("swiglu_limit", ctypes.c_float),
                ("act_terms", ctypes.c_int32), ("combine_mode", ctypes.c_int32),
                ("act_quant", ctypes.c_int32), ("doweight_stage1", ctypes.c_int32), ("cta_pairs", ctypes.c_int32)]


_WS_FIELDS = ["total_bytes", "max_rows", "off_sorted_ids", "off_sorted_w", "off_sorted_e",
              "off_num_valid", "off_loc", "off_status", "off_xq", "off_xsf", "off_hq", "off_hsf", "off_out2",
              "off_sort_scratch"]


class Workspace(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in _WS_FIELDS]


class Io(ctypes.Structure):
    """b200moe_io: every tensor of one layer call (optional ones may be None)."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("x_bf16", "topk_ids", "topk_weight", "expert_mask", "num_local_tokens",
                                               "w1_q", "w1_scale_prepared", "w2_q", "w2_scale_prepared", "bias1",
                                               "bias2", "y_bf16")]


EXPORTS = ["b200moe_version", "b200moe_last_error", "b200moe_workspace_layout",
           "b200moe_prepared_scale_bytes", "b200moe_prepare_scales", "b200moe_sort_align",
           "b200moe_quant_rows", "b200moe_quant_rows_e4m3", "b200moe_gateup", "b200moe_down", "b200moe_combine",
           "b200moe_forward", "b200moe_forward_dyn", "b200moe_sort_align_dyn", "b200moe_sort_align_ws",
           "b200moe_sort_scratch_bytes", "b200moe_route_topk", "b200moe_forward_static", "b200moe_gather_sum", "b200moe_debug_probe",
           "b200moe_forward_ex", "b200moe_static_status", "b200moe_ep_plan", "b200moe_quant_rows_fp8_1x128",
           "b200moe_forward_batch1", "b200moe_batch1_scratch_bytes"]


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile the CUDA sources for sm_100a into pyhip_b200/libb200moe.so (nvcc cross-compiles
    without a GPU)."""
    srcs = [CSRC / s for s in SOURCES]
    deps = srcs + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "b200moe.h"]
    if not force and LIB_PATH.exists() and all(LIB_PATH.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return LIB_PATH
    cmd = ["nvcc", *NVCC_FLAGS, "-o", str(LIB_PATH), *map(str, srcs)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


@functools.cache
def lib() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                          "(needs nvcc); this package has no CPU or eager fallback")
    L = ctypes.CDLL(str(LIB_PATH))
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    sp, wp = ctypes.POINTER(Shape), ctypes.POINTER(Workspace)
    L.b200moe_version.restype = ctypes.c_int
    L.b200moe_last_error.restype = ctypes.c_char_p
    L.b200moe_workspace_layout.argtypes = [sp, wp]
    L.b200moe_prepared_scale_bytes.argtypes = [sp, ctypes.c_int, ctypes.POINTER(i64)]
    L.b200moe_prepare_scales.argtypes = [sp, ctypes.c_int, vp, vp, vp]
    L.b200moe_sort_align.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp]
    L.b200moe_quant_rows.argtypes = [vp, i32, vp, vp, i32, i32, i32, i32, i32, i64, vp, vp, vp]
    L.b200moe_quant_rows_e4m3.argtypes = [vp, i32, vp, vp, i32, i32, i32, i32, i64, vp, vp, vp]
    L.b200moe_quant_rows_fp8_1x128.argtypes = [vp, i32, vp, vp, i32, i32, i32, i32, i64, vp, vp, vp]
    L.b200moe_gateup.argtypes = [sp, wp, vp, vp, vp, vp, vp, vp]
    L.b200moe_down.argtypes = [sp, wp, vp, vp, vp, vp, vp, vp]
    L.b200moe_forward_ex.argtypes = [sp, wp, vp, ctypes.POINTER(Io), vp]
    L.b200moe_static_status.argtypes = [sp, vp, vp]
    L.b200moe_combine.argtypes = [sp, wp, vp, vp, vp, vp]
    L.b200moe_forward.argtypes = [sp, wp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    L.b200moe_forward_dyn.argtypes = [sp, wp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    L.b200moe_sort_align_dyn.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp]
    L.b200moe_sort_align_ws.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i64, vp]
    L.b200moe_sort_scratch_bytes.argtypes = [i32, ctypes.POINTER(i64)]
    L.b200moe_route_topk.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp]
    L.b200moe_forward_static.argtypes = [sp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    L.b200moe_forward_batch1.argtypes = [sp] + [vp] * 14
    L.b200moe_batch1_scratch_bytes.argtypes = [sp, ctypes.POINTER(ctypes.c_int64)]
    L.b200moe_gather_sum.argtypes = [vp, vp, i32, i32, i32, vp, vp]
    L.b200moe_ep_plan.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    L.b200moe_debug_probe.argtypes = [ctypes.c_int, vp, vp, vp]
    for name in EXPORTS:
        if name not in ("b200moe_version", "b200moe_last_error"):
            getattr(L, name).restype = ctypes.c_int
    if L.b200moe_version() != ABI_VERSION:
        raise RuntimeError("libb200moe.so version mismatch; rebuild it")
    return L


class B200MoEError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().b200moe_last_error().decode(errors="replace")
        kind = "argument error" if rc < 0 else f"CUDA error {rc}"
        raise B200MoEError(f"{what}: {kind}: {msg}")


def workspace_layout(shape: Shape) -> Workspace:
    ws = Workspace()
    check(lib().b200moe_workspace_layout(ctypes.byref(shape), ctypes.byref(ws)), "workspace_layout")
    return ws
