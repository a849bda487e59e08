"""Sharing the quantisation of a replicated activation between the ranks of one node.

With the weight split along N every rank multiplies the WHOLE activation X by its weight shard, so every rank needs
all of X quantised, and quantising it is HBM-bound work that does not shrink with the number of GPUs (the reference
has no distributed code at all: src/deepwell/__init__.py:45-83 is a placeholder).  Here each rank quantises only its
1/world slice of the rows (whole 128-row scale tiles, so a slice is one contiguous piece of the payload and one of the
tiled scale buffer) and writes that slice into every peer's operand buffer over NVLink with plain device-to-device copies.
Those copies are executed by the copy engines, which, unlike any kernel, run while a GEMM's thread blocks hold every SM
(measured between two ranks: a 256 MB copy into a peer's buffer issued behind the start of a 1.33 ms GEMM is done after 0.39 ms), so
the exchange for the next step hides under this step's GEMMs.

    ex = QuantizedRowExchange([(M, K0), (M, K1), ...], group)      # once; allocates and maps the operand buffers
    step s:   ex.quantise_and_push(xs, slot=(s + 1) % 2)          # own slices -> every rank's buffers, asynchronously
              ... GEMMs of step s on ex.operand(slot=s % 2, i) ...
              ex.fence((s + 1) % 2)                                # all slices of the next slot have landed everywhere

The operand buffers live in memory every rank of the node can address (torch symmetric memory; CUDA IPC handles of ordinary
allocations as a slow last resort).  The fence is one 4-byte all-reduce per step: when it completes on a
rank, every rank has passed the point behind its own pushes and behind its GEMMs of the step, so the next slot is complete
everywhere and the slot just used may be overwritten.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _native as nv


def _map_on_all_ranks(nbytes: int, device: torch.device, group) -> Tuple[List[torch.Tensor], str]:
    """One uint8 buffer of `nbytes` per rank, each addressable from every rank: ([view of rank 0's, rank 1's, ...], how)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    errors = []
    try:
        # symmetric memory: every rank's buffer is mapped into this process's address space on ITS OWN device; a copy into a
        # peer's view is a device-to-device copy that the copy engines carry over NVLink (measured on B200: 256 MB in
        # 0.36 ms = 750 GB/s, 16 us of host time, and it runs while a GEMM holds the SMs)
        import torch.distributed._symmetric_memory as symm_mem
        local = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        handle = symm_mem.rendezvous(local, group=group if group is not None else dist.group.WORLD)
        views = [local if r == rank else handle.get_buffer(r, (nbytes,), torch.uint8) for r in range(world)]
        return views, "symmetric memory"
    except Exception as e:                      # no symmetric-memory support in this build / on this box
        errors.append(f"symmetric memory: {type(e).__name__}: {str(e)[:160]}")
    try:
        # CUDA IPC handles of an ordinary allocation: works everywhere, but the peers' views are tensors on the peers'
        # devices and the copies into them were staged through host memory on the box measured (25 GB/s): a last resort
        from torch.multiprocessing.reductions import reduce_tensor
        local = torch.empty(nbytes, dtype=torch.uint8, device=device)
        torch.cuda.synchronize(device)
        shared = [None] * world
        dist.all_gather_object(shared, reduce_tensor(local), group=group)
        views = [local if r == rank else shared[r][0](*shared[r][1]) for r in range(world)]
        return views, "CUDA IPC handles"
    except Exception as e:
        errors.append(f"CUDA IPC: {type(e).__name__}: {str(e)[:160]}")
    raise RuntimeError("no way to map peer memory: " + "; ".join(errors))


class QuantizedRowExchange:
    """Row-wise MXFP8 operands (codes [rows, cols] + tiled scales) of replicated activations, each rank quantising
    rows [rank * rows / world, (rank + 1) * rows / world) and copying them into every peer's buffer."""

    def __init__(self, shapes: Sequence[Tuple[int, int]], group=None, device: Optional[torch.device] = None, slots: int = 2,
                 scale_rule: int = nv.RULE_OCP_FLOOR, push: str = "graph"):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.shapes = [(int(r), int(c)) for r, c in shapes]
        self.slots, self.rule = slots, scale_rule
        for rows, cols in self.shapes:
            if rows % (128 * self.world) or cols % 32:
                raise ValueError(f"activation {rows} x {cols}: rows must be a multiple of 128 x world ({128 * self.world}), "
                                 "cols of 32, so that every rank's slice is whole scale tiles")
        # layout of one slot: per activation, payload then tiled scales, each 256-byte aligned
        self._offsets, off = [], 0
        for rows, cols in self.shapes:
            code_bytes, sf_bytes = rows * cols, nv.scale_bytes(rows, cols, nv.SF_TILED)
            self._offsets.append((off, code_bytes, off + -(-code_bytes // 256) * 256, sf_bytes))
            off = self._offsets[-1][2] + -(-sf_bytes // 256) * 256
        self.slot_bytes = off
        self.views, self.how = _map_on_all_ranks(self.slot_bytes * slots, self.device, group)
        self.copy_stream = torch.cuda.Stream(self.device)
        self._quantised = [torch.cuda.Event() for _ in range(slots)]
        self._pushed = [torch.cuda.Event() for _ in range(slots)]
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.bytes_pushed_per_call = sum((cb + sb) // self.world for _, cb, _, sb in self._offsets) * (self.world - 1)
        # The copies of one slot always run between the same addresses: 2 x activations x (world - 1) of them.  Issued one
        # by one they cost the host about 16 us each, more than a step's GEMMs last on 8 GPUs, so each slot's copies are
        # recorded once as a CUDA graph of memcpy nodes and replayed with a single launch.
        if push not in ("graph", "stream"):
            raise ValueError("push must be 'graph' or 'stream'")
        self.push = push
        self._graphs = [self._capture_copies(slot) for slot in range(slots)] if push == "graph" and self.world > 1 else None

    def _region(self, view: torch.Tensor, slot: int, i: int):
        c_off, c_bytes, s_off, s_bytes = self._offsets[i]
        base = slot * self.slot_bytes
        return view[base + c_off: base + c_off + c_bytes], view[base + s_off: base + s_off + s_bytes]

    def operand(self, slot: int, i: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(codes uint8 [rows, cols], tiled scales uint8) of activation i in `slot`, in this rank's own buffer."""
        codes, scales = self._region(self.views[self.rank], slot, i)
        return codes.view(self.shapes[i]), scales

    def _slice(self, i: int) -> Tuple[int, int, int, int]:
        """Byte ranges [c_lo, c_hi) of the payload and [s_lo, s_hi) of the tiled scales that hold this rank's rows of activation i."""
        rows, cols = self.shapes[i]
        r0, r1 = self.rank * rows // self.world, (self.rank + 1) * rows // self.world
        sf_per_row_tile = self._offsets[i][3] // (rows // 128)
        return r0 * cols, r1 * cols, (r0 // 128) * sf_per_row_tile, (r1 // 128) * sf_per_row_tile

    def _issue_copies(self, slot: int) -> None:
        for step in range(1, self.world):                         # every rank starts with a different peer
            peer = (self.rank + step) % self.world
            for i in range(len(self.shapes)):
                c_lo, c_hi, s_lo, s_hi = self._slice(i)
                src_c, src_s = self._region(self.views[self.rank], slot, i)
                dst_c, dst_s = self._region(self.views[peer], slot, i)
                dst_c[c_lo:c_hi].copy_(src_c[c_lo:c_hi], non_blocking=True)
                dst_s[s_lo:s_hi].copy_(src_s[s_lo:s_hi], non_blocking=True)

    def _capture_copies(self, slot: int) -> "torch.cuda.CUDAGraph":
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self.copy_stream, capture_error_mode="thread_local"):
            self._issue_copies(slot)
        return graph

    def quantise_and_push(self, xs: Sequence[torch.Tensor], slot: int) -> None:
        """Quantises this rank's row slice of every activation into `slot` (current stream) and copies the slices into
        every peer's buffer (copy stream: copy engines over NVLink, asynchronous to the current stream)."""
        if len(xs) != len(self.shapes):
            raise ValueError("one tensor per registered activation")
        for i, x in enumerate(xs):
            rows, cols = self.shapes[i]
            if tuple(x.shape) != (rows, cols) or x.dtype != torch.bfloat16 or not x.is_contiguous():
                raise ValueError(f"activation {i} must be a contiguous bfloat16 [{rows}, {cols}] tensor")
            r0, r1 = self.rank * rows // self.world, (self.rank + 1) * rows // self.world
            codes, scales = self._region(self.views[self.rank], slot, i)
            c_lo, c_hi, s_lo, s_hi = self._slice(i)
            nv.quantize_into(x[r0:r1], codes[c_lo:c_hi], scales[s_lo:s_hi], nv.DIR_ROW, self.rule, nv.SF_TILED)
        self._quantised[slot].record()
        self.copy_stream.wait_event(self._quantised[slot])
        with torch.cuda.stream(self.copy_stream):
            if self._graphs is not None:
                self._graphs[slot].replay()
            else:
                self._issue_copies(slot)
            self._pushed[slot].record()

    def fence(self, slot: int) -> None:
        """After this returns (stream-wise), every rank's slices of `slot` are in this rank's buffer, and every rank has
        finished the work it issued before its own fence (so the other slot may be refilled)."""
        torch.cuda.current_stream(self.device).wait_event(self._pushed[slot])
        dist.all_reduce(self._token, group=self.group)
