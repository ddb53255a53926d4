"""Receive arenas in NVLink peer memory for the expert-parallel dispatch.

Every rank owns a ring of arena slots in symmetric memory (`torch.distributed._symmetric_memory`:
one allocation per rank, mapped into every process of the group). A dispatch is ONE kernel per
rank (`b200moe_peer_dispatch_rows`): it gathers the token rows a rank sends and writes them
straight into the destinations' arenas over NVLink -- no send buffer, no library all-to-all for
the payload. An arena slot holds one fixed segment of `capacity` rows per source rank, so a
sender needs to know nothing about the other senders: its rows start at `rank * capacity`.

Ordering, all on a communication stream and without a device-side wait of our own:
  * the kernel of exchange n starts after everything the caller had queued on its stream (the
    rows exist) and after the previous exchange's rendezvous completed on this rank;
  * a tiny NCCL all-reduce follows the kernel: when it completes on a rank, every rank's kernel
    of exchange n has finished, so the rank may read its slot (`Ticket.wait`);
  * slot n % 3 is written again at exchange n + 3. A writer gets there only after the rendezvous
    of exchange n + 2 completed, which the slot's owner entered only after the work it had
    queued by then -- its reads of exchange n among it -- was done. (The caller must have queued
    the consumer of exchange n before it starts exchange n + 2; the expert-parallel layer's
    pipeline -- send c + 1, then process c -- does.)

The reference's transport is a third-party library (MoonEP,
`src/mlops/expert_parallel/quack/communication.py`); its contract -- one copy of a token per
destination rank, received grouped by source rank -- is what this provides.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops

SLOTS = 3


class Ticket:
    """One exchange in flight: `wait()` makes the current stream wait until every rank's rows have
    landed in this rank's slot; `rows` is the slot as `[world * capacity, width]` bf16."""

    def __init__(self, work, rows, capacity):
        self.work, self.rows, self.capacity = work, rows, capacity

    def wait(self):
        self.work.wait()


class PeerArena:
    def __init__(self, group, device, capacity: int, width: int):
        """Collective over `group`: every rank allocates `SLOTS` slots of `world * capacity` bf16
        rows of `width` and maps its peers' arenas."""
        import torch.distributed._symmetric_memory as symmetric_memory

        self.group, self.device = group, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.capacity, self.width = int(capacity), int(width)
        self.slot_rows = self.world * self.capacity
        self.buffer = symmetric_memory.empty((SLOTS, self.slot_rows, self.width), dtype=torch.bfloat16,
                                             device=self.device)
        self.handle = symmetric_memory.rendezvous(self.buffer, group=group.group_name)
        self.base = [int(p) for p in self.handle.buffer_ptrs]
        self.slot_bytes = self.slot_rows * self.width * 2
        self.stream = torch.cuda.Stream(self.device, priority=-1)  # ahead of the GEMMs' CTAs when SMs free up
        self.flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.exchanges = 0
        self.previous = None
        self.bytes_moved = 0

    def fits(self, rows_per_peer: int, width: int) -> bool:
        return rows_per_peer <= self.capacity and width == self.width

    def dispatch(self, src: torch.Tensor, gather: torch.Tensor, send_counts) -> Ticket:
        """Send row i = `src[gather[i]]`; the first `send_counts[0]` send rows go to rank 0, the
        next `send_counts[1]` to rank 1, ... Returns the ticket of this exchange; after
        `ticket.wait()` the rows received from rank s are `ticket.rows[s * capacity : s * capacity
        + (what s sent here)]`, in s's order."""
        counts = [int(v) for v in send_counts]
        if max(counts, default=0) > self.capacity or src.shape[1] != self.width:
            raise ValueError("the dispatch does not fit the arena it was created for")
        current = torch.cuda.current_stream(self.device)
        slot = self.exchanges % SLOTS
        self.exchanges += 1
        starts = [0]
        for v in counts:
            starts.append(starts[-1] + v)
        self.stream.wait_stream(current)  # the rows and the index exist; earlier readers of this ring are queued
        with torch.cuda.stream(self.stream):
            if self.previous is not None:
                self.previous.wait()  # this rank has passed the previous rendezvous
            ops.peer_dispatch_rows(src, gather, [b + slot * self.slot_bytes for b in self.base], self.width,
                                   self.slot_rows, starts, [self.rank * self.capacity] * self.world,
                                   stream=self.stream)
            work = dist.all_reduce(self.flag, group=self.group, async_op=True)
        for tensor in (src, gather):
            tensor.record_stream(self.stream)
        self.previous = work
        self.bytes_moved += starts[-1] * self.width * 2
        return Ticket(work, self.buffer[slot], self.capacity)

    def received_index(self, recv_counts: torch.Tensor, total: int) -> torch.Tensor:
        """int64 `[total]`: the arena row of every received row, in `[source][arrival]` order (the
        position a dense all-to-all would have delivered it at). `recv_counts`: int64 device tensor
        `[world]`, rows received from each rank; `total` their sum (known to the host: no copy)."""
        source = torch.repeat_interleave(torch.arange(self.world, device=self.device), recv_counts,
                                         output_size=total)
        first = torch.cumsum(recv_counts, 0) - recv_counts
        return source * self.capacity + (torch.arange(total, device=self.device) - first[source])

    def close(self):
        if self.previous is not None:
            self.previous.wait()
            self.previous = None
        self.buffer = self.handle = None
