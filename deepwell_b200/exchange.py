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
    ex.set_shared_rows([M, M // 2, ...])                           # optional: how many rows of each activation are shared
    step s:   ex.quantise_and_push(xs, slot=(s + 1) % 2)          # own slices -> every rank's buffers, asynchronously
              ... GEMMs of step s on ex.operand(slot=s % 2, i) ...
              ex.fence((s + 1) % 2)                                # all slices of the next slot have landed everywhere

The operand buffers live in memory every rank of the node can address (torch symmetric memory; CUDA IPC handles of ordinary
allocations as a slow last resort).  The fence is one 4-byte all-reduce per step: when it completes on a
rank, every rank has passed the point behind its own pushes and behind its GEMMs of the step, so the next slot is complete
everywhere and the slot just used may be overwritten.

What a rank receives per step crosses its NVLink ports at ~750 GB/s; where the GEMMs of a step are shorter than that transfer
(eight ranks on the Llama-3-8B shapes) only the first `shared_rows[i]` rows of an activation are shared and every rank
quantises the remaining rows itself, so that the transfer still ends before the step does.

ColumnGather (below) moves the OUTPUT of an N-sharded layer the same way: every rank's column shard into every rank's
gathered result, by copy engines, while the next layer's GEMM runs.
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


class SlotLayout:
    """Where the row-wise operands of several activations sit in one slot of the exchange buffer, and which bytes of them
    belong to which rows.  Pure arithmetic (no device): per activation the payload [rows, cols] then its tiled scales, each
    256-byte aligned.  Rows come in whole 128-row scale tiles, so rows [r0, r1) are one contiguous byte range of the payload
    and one of the scale buffer."""

    def __init__(self, shapes: Sequence[Tuple[int, int]], world: int):
        self.world = int(world)
        self.shapes = [(int(r), int(c)) for r, c in shapes]
        for rows, cols in self.shapes:
            if rows % (128 * self.world) or cols % 32:
                raise ValueError(f"activation {rows} x {cols}: rows must be a multiple of 128 x world ({128 * self.world}), "
                                 "cols of 32, so that every rank's slice is whole scale tiles")
        self.offsets, off = [], 0           # (payload offset, payload bytes, scale offset, scale bytes) per activation
        for rows, cols in self.shapes:
            code_bytes, sf_bytes = rows * cols, (rows // 128) * (-(-(cols // 32) // 4)) * 512
            self.offsets.append((off, code_bytes, off + -(-code_bytes // 256) * 256, sf_bytes))
            off = self.offsets[-1][2] + -(-sf_bytes // 256) * 256
        self.slot_bytes = off

    def check_shared_rows(self, shared_rows: Optional[Sequence[int]]) -> List[int]:
        rows = [r for r, _ in self.shapes]
        wanted = rows if shared_rows is None else [int(r) for r in shared_rows]
        if len(wanted) != len(rows) or any(w < 0 or w > r or w % (128 * self.world) for w, r in zip(wanted, rows)):
            raise ValueError(f"shared_rows must be one multiple of {128 * self.world} in [0, rows] per activation")
        return wanted

    def rows_of(self, shared: int, rank: int) -> Tuple[int, int]:
        """The part [r0, r1) of the shared rows [0, shared) that `rank` quantises."""
        return rank * shared // self.world, (rank + 1) * shared // self.world

    def byte_ranges(self, i: int, r0: int, r1: int) -> Tuple[int, int, int, int]:
        """[c_lo, c_hi) of the payload and [s_lo, s_hi) of the tiled scales of activation i that hold rows [r0, r1)."""
        rows, cols = self.shapes[i]
        sf_per_row_tile = self.offsets[i][3] // (rows // 128)
        return r0 * cols, r1 * cols, (r0 // 128) * sf_per_row_tile, (r1 // 128) * sf_per_row_tile


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
        self.layout = SlotLayout(shapes, self.world)
        self.shapes, self._offsets, self.slot_bytes = self.layout.shapes, self.layout.offsets, self.layout.slot_bytes
        self.slots, self.rule = slots, scale_rule
        for (rows, cols), (_, _, _, sf_bytes) in zip(self.shapes, self._offsets):
            assert sf_bytes == nv.scale_bytes(rows, cols, nv.SF_TILED)       # the library's tiled layout is the one assumed here
        self.views, self.how = _map_on_all_ranks(self.slot_bytes * slots, self.device, group)
        self.copy_stream = torch.cuda.Stream(self.device)
        self._quantised = [torch.cuda.Event() for _ in range(slots)]
        self._pushed = [torch.cuda.Event() for _ in range(slots)]
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        # The copies of one slot always run between the same addresses: 2 x activations x (world - 1) of them.  Issued one
        # by one they cost the host about 16 us each, more than a step's GEMMs last on 8 GPUs, so each slot's copies are
        # recorded once as a CUDA graph of memcpy nodes and replayed with a single launch.
        if push not in ("graph", "stream"):
            raise ValueError("push must be 'graph' or 'stream'")
        self.push_mode = push
        self._graphs = None
        self.shared_rows: List[int] = []
        self.set_shared_rows(None)

    def set_shared_rows(self, shared_rows: Optional[Sequence[int]]) -> None:
        """Collective: rows [0, shared_rows[i]) of activation i are quantised once (1/world of them per rank) and exchanged,
        rows from shared_rows[i] on by every rank itself.  None = all rows shared.  Each count must be a multiple of
        128 x world (0 = not shared at all).  The operand buffers hold stale data afterwards until the next
        quantise_and_push of each slot."""
        wanted = self.layout.check_shared_rows(shared_rows)
        torch.cuda.synchronize(self.device)          # no copy of the old plan in flight on this rank ...
        dist.barrier(group=self.group)               # ... or on any other
        self.shared_rows = wanted
        self.bytes_pushed_per_call = sum(self._slice_bytes(i) for i in range(len(self.shapes))) * (self.world - 1)
        self._graphs = None
        if self.push_mode == "graph" and self.world > 1 and self.bytes_pushed_per_call > 0:
            self._graphs = [self._capture_copies(slot) for slot in range(self.slots)]
        dist.barrier(group=self.group)

    def _region(self, view: torch.Tensor, slot: int, i: int):
        c_off, c_bytes, s_off, s_bytes = self._offsets[i]
        base = slot * self.slot_bytes
        return view[base + c_off: base + c_off + c_bytes], view[base + s_off: base + s_off + s_bytes]

    def operand(self, slot: int, i: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(codes uint8 [rows, cols], tiled scales uint8) of activation i in `slot`, in this rank's own buffer."""
        codes, scales = self._region(self.views[self.rank], slot, i)
        return codes.view(self.shapes[i]), scales

    def _rows_of(self, i: int, rank: int) -> Tuple[int, int]:
        return self.layout.rows_of(self.shared_rows[i], rank)

    def _byte_ranges(self, i: int, r0: int, r1: int) -> Tuple[int, int, int, int]:
        return self.layout.byte_ranges(i, r0, r1)

    def _slice(self, i: int) -> Tuple[int, int, int, int]:
        return self._byte_ranges(i, *self._rows_of(i, self.rank))

    def _slice_bytes(self, i: int) -> int:
        c_lo, c_hi, s_lo, s_hi = self._slice(i)
        return (c_hi - c_lo) + (s_hi - s_lo)

    def _issue_copies(self, slot: int) -> None:
        """On the copy stream (current): this rank's slices of `slot` to every peer, one branch per peer."""
        def to_peer(k: int) -> None:
            peer = (self.rank + 1 + k) % self.world               # every rank starts with a different peer
            for i in range(len(self.shapes)):
                c_lo, c_hi, s_lo, s_hi = self._slice(i)
                if c_hi == c_lo:
                    continue
                src_c, src_s = self._region(self.views[self.rank], slot, i)
                dst_c, dst_s = self._region(self.views[peer], slot, i)
                dst_c[c_lo:c_hi].copy_(src_c[c_lo:c_hi], non_blocking=True)
                dst_s[s_lo:s_hi].copy_(src_s[s_lo:s_hi], non_blocking=True)

        for k in range(self.world - 1):              # one after the other: measured on 4 B200s, a rank's copies to its three
            to_peer(k)                               # peers reach 749 GB/s in a row and 736 GB/s as parallel branches

    def _capture_copies(self, slot: int) -> "torch.cuda.CUDAGraph":
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self.copy_stream, capture_error_mode="thread_local"):
            self._issue_copies(slot)
        return graph

    def pieces(self, xs: Sequence[torch.Tensor], slot: int):
        """(shared, local): the (input rows, codes, scales) triples that fill `slot` on this rank — `shared`: this rank's part
        of the shared rows of every activation (what push() sends to the peers); `local`: per activation the rows every rank
        quantises itself (a list of lists, in the order of the activations).  A caller that wants the local rows quantised
        elsewhere in its step (behind a GEMM, say) quantises `shared`, calls push(slot), and issues `local` when it likes,
        before fence(slot)."""
        if len(xs) != len(self.shapes):
            raise ValueError("one tensor per registered activation")
        shared, local = [], []
        for i, x in enumerate(xs):
            rows, cols = self.shapes[i]
            if tuple(x.shape) != (rows, cols) or x.dtype != torch.bfloat16 or not x.is_contiguous():
                raise ValueError(f"activation {i} must be a contiguous bfloat16 [{rows}, {cols}] tensor")
            codes, scales = self._region(self.views[self.rank], slot, i)

            def triple(p0, p1):
                c_lo, c_hi, s_lo, s_hi = self._byte_ranges(i, p0, p1)
                return (x[p0:p1], codes[c_lo:c_hi], scales[s_lo:s_hi])

            r0, r1 = self._rows_of(i, self.rank)
            if r1 > r0:
                shared.append(triple(r0, r1))
            local.append([triple(self.shared_rows[i], rows)] if self.shared_rows[i] < rows else [])
        return shared, local

    def quantise(self, jobs) -> int:
        """Row-wise quantisation of (input, codes, tiled scales) triples on the current stream, in one launch per eight where
        the shapes allow.  Returns the number of launches."""
        jobs = list(jobs)
        if not jobs:
            return 0
        if all(j[0].shape[0] % 128 == 0 and j[0].shape[1] % 128 == 0 and j[0].data_ptr() % 16 == 0 and j[1].data_ptr() % 16 == 0
               for j in jobs):
            return nv.quantize_rows_batch_into([j[0] for j in jobs], [j[1] for j in jobs], [j[2] for j in jobs],
                                               self.rule, nv.SF_TILED)
        for x, codes, scales in jobs:                              # shapes the batched launch does not take
            nv.quantize_into(x, codes, scales, nv.DIR_ROW, self.rule, nv.SF_TILED)
        return len(jobs)

    def push(self, slot: int) -> None:
        """Behind the work issued so far on the current stream: this rank's shared slices of `slot` into every peer's buffer
        (copy stream: copy engines over NVLink, asynchronous to the current stream)."""
        if self.bytes_pushed_per_call == 0:
            return
        self._quantised[slot].record()
        self.copy_stream.wait_event(self._quantised[slot])
        with torch.cuda.stream(self.copy_stream):
            if self._graphs is not None:
                self._graphs[slot].replay()
            else:
                self._issue_copies(slot)
            self._pushed[slot].record()

    def quantise_and_push(self, xs: Sequence[torch.Tensor], slot: int,
                          extra: Sequence[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = ()) -> int:
        """Quantises this rank's row slice of every activation (and the rows that are not shared) into `slot` on the current
        stream and copies the slices into every peer's buffer.  `extra`: further (input, codes, tiled scales) triples
        quantised row-wise in the same launches, e.g. the rank's weight shards: the pieces of a sharded step are small, and
        one launch for all of them saves each its own ramp and tail.  Returns the number of quantiser launches."""
        shared, local = self.pieces(xs, slot)
        launches = self.quantise(shared + [j for per in local for j in per] + list(extra))
        self.push(slot)
        return launches

    def fence(self, slot: int) -> None:
        """After this returns (stream-wise), every rank's slices of `slot` are in this rank's buffer, and every rank has
        finished the work it issued before its own fence (so the other slot may be refilled)."""
        if self.bytes_pushed_per_call == 0:          # nothing is shared: every rank filled its own buffer, no rank waits for another
            return
        torch.cuda.current_stream(self.device).wait_event(self._pushed[slot])
        dist.all_reduce(self._token, group=self.group)

class ColumnGather:
    """The column shards Y_r = Y[:, n0_r:n1_r] that the ranks of an N-sharded layer compute, brought to every rank by the
    copy engines instead of an NCCL all-gather, whose kernels wait for the GEMM's thread blocks like any other kernel.

    layout "blocked" (default): rank-major blocks [world, M, n_local], the layout an all-gather delivers.  A shard is one
    contiguous piece, so each destination takes one plain device-to-device copy: copy-engine traffic over NVLink at
    ~750 GB/s that runs while the next layer's GEMM holds the SMs.  The GEMM writes its shard straight into block `rank`
    of this rank's buffer; the copies of one output are recorded once as a CUDA graph and replayed.
    layout "row_major": the full row-major [M, N]; every destination takes one pitched copy (dw_mxfp8_copy_2d_async).
    Measured on B200, pitched copies with rows of 4-28 KB do not overlap the GEMMs and are no faster than the NCCL
    gather followed by a strided pass, so this form only saves that pass.

        cg = ColumnGather([(M, N0), (M, N1), ...], group)          # once
        y_shard = cg.shard(i)                                       # [M, n_local] bf16: the GEMM's output buffer
        ... GEMM of layer i writes y_shard ...
        done = cg.push(i)                                           # asynchronous: copy stream; shard(i) is free after `done`
                                                                    # (slots > 1: shard(i, slot), push(i, slot), full(i, slot))
        cg.fence()                                                  # all shards of everything pushed so far have landed
        y_all = cg.full(i)                                          # [world, M, n_local] (blocked) or [M, N] (row_major)
    """

    def __init__(self, shapes: Sequence[Tuple[int, int]], group=None, device: Optional[torch.device] = None,
                 layout: str = "blocked", slots: int = 1):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        if layout not in ("blocked", "row_major"):
            raise ValueError("layout must be 'blocked' or 'row_major'")
        self.group, self.layout, self.slots = group, layout, int(slots)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.shapes = [(int(m), int(n)) for m, n in shapes]
        for m, n in self.shapes:
            if n % (8 * self.world):
                raise ValueError(f"output {m} x {n}: N must be a multiple of 8 x world so that every shard's rows are 16-byte pieces")
        # this rank's buffer: the gathered outputs one after the other; row_major keeps the shards (what the GEMMs
        # write) behind them, blocked has them inside (block `rank` of each output)
        self._full_off, self._shard_off, off = [], [], 0
        for m, n in self.shapes:
            self._full_off.append(off)
            off += -(-m * n * 2 // 256) * 256
        for i, (m, n) in enumerate(self.shapes):
            if layout == "blocked":
                self._shard_off.append(self._full_off[i] + self.rank * m * (n // self.world) * 2)
            else:
                self._shard_off.append(off)
                off += -(-m * (n // self.world) * 2 // 256) * 256
        self.slot_bytes = off                     # with several slots a layer's GEMM of one step fills a slot while the copies
        self.views, self.how = _map_on_all_ranks(off * self.slots, self.device, group)    # of the step before still read another
        self.copy_stream = torch.cuda.Stream(self.device)
        self._ready = [torch.cuda.Event() for _ in self.shapes]
        self._done = [[torch.cuda.Event() for _ in self.shapes] for _ in range(self.slots)]   # pushes of (slot, i) executed
        self._pushed = torch.cuda.Event()
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.bytes_pushed = [m * (n // self.world) * 2 * (self.world - 1) for m, n in self.shapes]
        self._graphs = None
        if layout == "blocked" and self.world > 1:
            torch.cuda.synchronize(self.device)
            self._graphs = []
            for slot in range(self.slots):
                self._graphs.append([])
                for i in range(len(self.shapes)):
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=self.copy_stream, capture_error_mode="thread_local"):
                        self._issue(i, slot)
                    self._graphs[slot].append(graph)

    def _bytes(self, i: int) -> int:
        m, n = self.shapes[i]
        return m * (n // self.world) * 2

    def shard(self, i: int, slot: int = 0) -> torch.Tensor:
        m, n = self.shapes[i]
        at = slot * self.slot_bytes + self._shard_off[i]
        return self.views[self.rank][at: at + self._bytes(i)].view(torch.bfloat16).view(m, n // self.world)

    def full(self, i: int, slot: int = 0) -> torch.Tensor:
        m, n = self.shapes[i]
        at = slot * self.slot_bytes + self._full_off[i]
        flat = self.views[self.rank][at: at + m * n * 2].view(torch.bfloat16)
        return flat.view(self.world, m, n // self.world) if self.layout == "blocked" else flat.view(m, n)

    def _issue(self, i: int, slot: int) -> None:
        """On the copy stream (current): shard i of `slot` to every destination, one after the other."""
        m, n = self.shapes[i]
        nl, nbytes = n // self.world, self._bytes(i)
        base = slot * self.slot_bytes
        src = self.views[self.rank][base + self._shard_off[i]: base + self._shard_off[i] + nbytes]
        first = 1 if self.layout == "blocked" else 0             # blocked: the shard already sits in this rank's own block

        def to_peer(k: int) -> None:
            peer = (self.rank + first + k) % self.world          # every rank starts with a different destination
            if self.layout == "blocked":
                at = base + self._full_off[i] + self.rank * nbytes
                self.views[peer][at: at + nbytes].copy_(src, non_blocking=True)
            else:
                dst = self.views[peer].data_ptr() + base + self._full_off[i] + self.rank * nl * 2
                nv.copy_2d_async(dst, n * 2, src.data_ptr(), nl * 2, nl * 2, m, self.device)

        for k in range(self.world - first):
            to_peer(k)

    def push(self, i: int, slot: int = 0) -> "torch.cuda.Event":
        """Behind the work issued so far on the current stream (the GEMM that writes shard(i, slot)): this rank's shard into
        its place in output i of `slot` on every rank.  Returns the event that follows the copies: shard(i, slot) may be
        overwritten once it has happened."""
        self._ready[i].record()
        self.copy_stream.wait_event(self._ready[i])
        with torch.cuda.stream(self.copy_stream):
            if self._graphs is not None:
                self._graphs[slot][i].replay()
            else:
                self._issue(i, slot)
            self._done[slot][i].record()
            self._pushed.record()
        return self._done[slot][i]

    def fence(self) -> None:
        """Stream-wise: after this, every rank's shards of all outputs pushed so far are in this rank's buffers (and this
        rank's in every other's).  One 4-byte all-reduce."""
        torch.cuda.current_stream(self.device).wait_event(self._pushed)
        dist.all_reduce(self._token, group=self.group)
