"""The allocation-free sort entry point (`b200moe_sort_assignments_static`), for hosts that
cannot call the CUDA allocator: it must give exactly what `b200moe_sort_assignments` gives,
call after call, although every call reuses the same built-in scratch array. The comparator,
the workspace sort, is itself pinned: `tests/test_gpu_routing.py` holds it bit-exact against
the stored outputs of the reference's `sort_assignments` and against the CPU restatement.

Collected last on purpose (file name), so a failure here cannot hide another test's."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _compare(ids, experts):
    from mlops_b200 import ops

    n = ids.numel()
    order = torch.empty(n, dtype=torch.int32, device=DEV)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
    slots = torch.empty(n, dtype=torch.int32, device=DEV)
    counts = torch.empty(experts, dtype=torch.int64, device=DEV)
    # status block is created (allocated) by the wrapper on first use: do that before the call
    ops.status_block(DEV)
    ops.sort_assignments_static(ids, experts, order, offsets, slots, counts)
    o_ref, f_ref, s_ref, c_ref = ops.sort_assignments(ids, experts)
    assert torch.equal(order, o_ref)
    assert torch.equal(offsets, f_ref)
    assert torch.equal(slots, s_ref.reshape(-1))
    assert torch.equal(counts, c_ref)
    ops.check_status(DEV)


def test_static_scratch_sort_matches_workspace_sort_twice_in_a_row():
    g = torch.Generator().manual_seed(21)
    # first call: large, fills much of the scratch; second call: small and with other experts,
    # so stale histogram entries of the first call would show up if they were ever read
    first = torch.randint(0, 256, (32768, 8), generator=g).to(torch.int32).to(DEV)
    second = torch.randint(0, 8, (700, 2), generator=g).to(torch.int32).to(DEV)
    _compare(first, 256)
    _compare(second, 8)
    _compare(first, 256)


def test_static_scratch_sort_rejects_sizes_beyond_its_array():
    from mlops_b200._lib import lib

    ids = torch.zeros(8, dtype=torch.int32, device=DEV)
    out = torch.empty(8, dtype=torch.int32, device=DEV)
    offs = torch.empty(1025, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    # 1024 experts allow 256 chunks = 1048576 assignments; one more chunk must be refused
    too_many = 256 * 4096 + 1
    code = lib.b200moe_sort_assignments_static(ids.data_ptr(), too_many, 1024, out.data_ptr(), offs.data_ptr(),
                                               out.data_ptr(), None, status.data_ptr(), None)
    assert code == -6
