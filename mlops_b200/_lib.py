"""ctypes binding of `libb200moe.so` (the C ABI declared in `include/b200moe.h`).

The library is the only compute path of this package: when it is missing, importing
this module raises. There is no fallback."""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int32, c_longlong, c_void_p
from pathlib import Path

# B200MOE_LIBRARY names another build of the same library (an instrumented or experimental
# one: `python -m mlops_b200.build --define NAME=VALUE --output path`); the ABI is the same.
LIBRARY_PATH = Path(os.environ.get("B200MOE_LIBRARY") or Path(__file__).resolve().parent / "libb200moe.so")

ERROR_NAMES = {
    0: "ok",
    -1: "bad argument",
    -2: "alignment requirement not met",
    -3: "TMA tensor map refused",
    -4: "kernel launch failed",
    -5: "driver entry point unavailable",
    -6: "size beyond a documented maximum",
}

P = c_void_p
LL = c_longlong
I = c_int
F = c_float

# name -> (restype, argtypes); one entry per declaration in include/b200moe.h
SIGNATURES = {
    "b200moe_route_topk": (I, [P, LL, I, I, I, I, P, I, I, F, P, P, P]),
    "b200moe_routing_probability_sum_workspace_bytes": (LL, [LL, I]),
    "b200moe_routing_probability_sum": (I, [P, LL, LL, I, I, P, P, P]),
    "b200moe_routing_gradient": (I, [P, LL, LL, I, I, I, P, P, P, P, P, F, P, P, LL, P]),
    "b200moe_sort_assignments_workspace_bytes": (LL, [LL, I]),
    "b200moe_sort_assignments": (I, [P, LL, I, P, P, P, P, P, P, P]),
    "b200moe_sort_assignments_static": (I, [P, LL, I, P, P, P, P, P, P]),
    "b200moe_quantize_rows": (I, [P, LL, LL, P, I, LL, I, P, LL, P, LL, LL, I, P, LL, P, P]),
    "b200moe_quantize_rows_scatter": (I, [P, LL, LL, P, I, LL, I, P, LL, P, LL, LL, P, LL, P, P]),
    "b200moe_swiglu_quantize": (I, [P, LL, LL, I, P, LL, P, LL, LL, P, LL, F, I, P]),
    "b200moe_dswiglu_routed": (
        I,
        [P, LL, P, LL, P, LL, P, LL, I, P, P, LL, P, LL, LL, P, LL, P, LL, F, I, P, P],
    ),
    "b200moe_quantize_blocks": (I, [P, I, I, I, I, P, P, P]),
    "b200moe_grouped_gemm_fp8": (
        I,
        [P, LL, P, LL, LL, P, P, P, LL, P, LL, P, I, I, LL, I, I, I, I, P, P],
    ),
    "b200moe_grouped_gemm_fp8_scatter": (
        I,
        [P, LL, P, LL, LL, P, P, P, LL, P, P, LL, P, I, I, LL, I, I, I, I, P, P],
    ),
    "b200moe_grouped_gemm_fp8_swiglu": (
        I,
        [P, LL, P, LL, LL, P, P, P, LL, P, LL, P, LL, LL, P, I, I, LL, I, I, F, I, P, P],
    ),
    "b200moe_grouped_gemm_fp8_combine": (
        I,
        [P, LL, P, LL, LL, P, P, P, LL, LL, P, P, P, LL, P, I, I, LL, I, I, I, P, P],
    ),
    "b200moe_finish_combine": (I, [P, LL, P, LL, P, LL, LL, I, P]),
    "b200moe_grouped_wgrad_bf16": (I, [P, LL, P, LL, P, I, I, LL, I, I, P, I, P, P]),
    "b200moe_grouped_wgrad_bf16_accumulate": (I, [P, LL, P, LL, P, I, I, LL, I, I, P, I, F, P, P]),
    "b200moe_grouped_gemm_bf16": (I, [P, LL, P, P, LL, P, LL, P, I, I, LL, I, I, I, F, P, P]),
    "b200moe_quantize_columns": (I, [P, LL, LL, I, P, I, I, P, LL, P, P]),
    "b200moe_grouped_wgrad_fp8": (I, [P, LL, P, P, LL, P, P, I, I, LL, I, I, P, I, F, I, P, P]),
    "b200moe_set_cta_limit": (I, [I]),
    "b200moe_set_gemm_pair": (I, [I]),
    "b200moe_lora_project": (I, [P, LL, P, I, P, I, LL, I, I, P, LL, P]),
    "b200moe_lora_expand": (I, [P, LL, P, I, P, I, LL, I, I, F, P, LL, P]),
    "b200moe_combine": (I, [P, LL, LL, P, P, P, LL, P, LL, LL, I, I, P]),
    "b200moe_gather_rows": (I, [P, LL, LL, P, I, LL, I, P, LL, P, P]),
    "b200moe_peer_dispatch_rows": (I, [P, LL, LL, P, LL, I, P, LL, LL, P, P, I, P, P]),
    "b200moe_build_copies": (I, [P, P, I, I, I, I, P, P, P, P, P, P]),
    "b200moe_gather_scalar": (I, [P, LL, P, LL, P, P, P]),
}


class NativeLibraryMissing(ImportError):
    pass


def _load() -> ctypes.CDLL:
    if not LIBRARY_PATH.exists():
        raise NativeLibraryMissing(
            f"{LIBRARY_PATH} is missing: build it with `python -m mlops_b200.build` "
            "(nvcc, sm_100a). This package has no other compute path."
        )
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


class NativeError(RuntimeError):
    pass


def check(code: int, what: str) -> None:
    if code != 0:
        raise NativeError(f"{what}: {ERROR_NAMES.get(code, 'error')} (code {code})")
