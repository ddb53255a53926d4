"""The C-ABI library loads and exports exactly what `include/b200moe.h` declares."""

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    header = (ROOT / "include" / "b200moe.h").read_text()
    return sorted(set(re.findall(r"\b(b200moe_\w+)\s*\(", header)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "b200moe_grouped_gemm_fp8" in names and "b200moe_route_topk" in names
    assert len(names) >= 12


def test_library_exports_every_declared_symbol():
    from mlops_b200 import _lib

    handle = ctypes.CDLL(str(_lib.LIBRARY_PATH))
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"


def test_binding_covers_every_declared_symbol():
    from mlops_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_argument_validation_needs_no_gpu():
    """Entry points reject null pointers and bad sizes before touching the device."""
    from mlops_b200._lib import lib

    assert lib.b200moe_route_topk(None, 0, 1, 8, 2, 1, None, 1, 1, 1.0, None, None, None) == -1
    assert lib.b200moe_sort_assignments_workspace_bytes(4096 * 3 + 1, 8) == 4 * 8 * 4
    assert lib.b200moe_sort_assignments_workspace_bytes(-1, 8) == -1
    assert lib.b200moe_grouped_gemm_fp8(None, 0, None, 0, 0, None, None, None, 0, None, 0, None, 1, 1, 0, 8, 16, 0,
                                        128,
                                        None, None) == -1
    assert lib.b200moe_combine(None, 0, 0, None, None, None, 0, None, 0, 0, 8, 1, None) == -1


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch

    from mlops_b200 import ops
    from mlops_b200._lib import NativeError

    with pytest.raises(NativeError):
        ops.route_topk(torch.zeros(4, 8), 2, "softmax_then_topk")
    with pytest.raises(NativeError):
        ops.quantize_rows(torch.zeros(4, 128, dtype=torch.bfloat16))


def test_device_probes_compile_for_sm_100a():
    """The stand-alone probes beside the kernels build with nvcc (nothing runs without a GPU)."""
    from mlops_b200 import probes

    names = sorted(p.stem for p in probes.PROBES.glob("*.cu"))
    assert "handshake" in names
    for name in names:
        assert probes.build(name).exists()
