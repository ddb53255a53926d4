"""The expert-parallel dispatch kernel (`b200moe_peer_dispatch_rows`) on one GPU: the "peers'"
arenas are local buffers here, so the addressing (destination rank by send segment, one fixed
segment per source rank in an arena) is checked without a second device; the real thing, over
NVLink between processes, is covered by tests/test_gpu_ep.py (2 GPUs) and by `bench.py`'s
`ep_check`."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("world,tokens,width,counts", [(3, 200, 512, [70, 0, 130]), (2, 64, 7168, [64, 64]),
                                                       (8, 300, 256, [40, 31, 0, 300, 7, 1, 64, 100])])
def test_rows_land_in_the_destinations_segments(world, tokens, width, counts):
    from mlops_b200 import ops

    g = torch.Generator().manual_seed(world * 10 + tokens)
    src = torch.randn(tokens, width, generator=g).bfloat16().to(DEV)
    # send rows grouped by destination: counts[r] rows for rank r, each one some token of this rank
    gather = torch.cat([torch.randperm(tokens, generator=g)[:n] for n in counts]).to(torch.int32).to(DEV)
    capacity, me = max(counts) + 3, 1
    arenas = [torch.full((world * capacity, width), -1.0, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    starts = [0]
    for n in counts:
        starts.append(starts[-1] + n)
    ops.peer_dispatch_rows(src, gather, [a.data_ptr() for a in arenas], width, world * capacity, starts,
                           [me * capacity] * world)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    for r in range(world):
        mine = arenas[r][me * capacity: me * capacity + counts[r]]
        assert torch.equal(mine, src[gather[starts[r]:starts[r + 1]].long()])
        untouched = torch.ones(world * capacity, dtype=torch.bool)
        untouched[me * capacity: me * capacity + counts[r]] = False
        assert bool((arenas[r][untouched.to(DEV)] == -1.0).all())   # nothing outside this sender's segment


def test_a_bad_row_or_destination_is_reported_and_skipped():
    from mlops_b200 import ops
    from mlops_b200._lib import NativeError

    src = torch.ones(8, 256, dtype=torch.bfloat16, device=DEV)
    arena = torch.zeros(4, 256, dtype=torch.bfloat16, device=DEV)
    gather = torch.tensor([0, 99, 1, 2, 3, 4], dtype=torch.int32, device=DEV)   # 99: no such token
    ops.peer_dispatch_rows(src, gather, [arena.data_ptr()], 256, 4, [0, 6], [0])  # rows 4, 5 fall outside the arena
    torch.cuda.synchronize()
    with pytest.raises(NativeError):
        ops.check_status(DEV)
    assert bool((arena[0] == 1).all()) and bool((arena[1] == 0).all()) and bool((arena[2:4] == 1).all())
