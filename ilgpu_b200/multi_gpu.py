"""Radix sort, scan, reduce and histogram over the GPUs of one box.

One process per GPU.  On GPUs the whole of it runs inside the native multi-GPU library
(``include/b200alg_mg.h``: local kernels, NCCL for the few words each primitive exchanges,
peer stores for the buckets of the sort); ``torch.distributed`` only carries the rendezvous
token.  The same algorithms are also written out here over ``torch.distributed`` with a
pluggable local engine; that path serves engines without the native library (the CPU
engine of the tests over ``gloo``):

* reduce, histogram - local kernel, then an all-reduce of one element / of the bins;
* scan - local reduce, all-gather of the per-rank totals, fold of the lower ranks' totals,
  local scan seeded with that value;
* sort - sample sort: sampled (key, global index) splitters, stable partition of the shard
  into one bucket per rank, all-to-all of the buckets, stable local radix sort.  Rank r
  ends up with the r-th slice of the globally sorted sequence.

The reference has no multi-device algorithms (its only multi-GPU facility is peer access,
Src/ILGPU/Runtime/PeerAccess.cs), so this is new surface.  The local work goes through a
small "engine" interface; the product engine is :class:`NativeEngine` (CUDA).  Tests of
the host logic substitute a CPU engine and run the same code over ``gloo``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _native as N
from .algorithms import (Accelerator, ArgumentOutOfRangeException, B200AlgException, NotSupportedException, RadixSortOperation, ScanKind,
                         ScanReduceOperation, _ptr, _stream_ptr, dtype_code)

_SIGNED_VIEW = {1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}
_UNSIGNED = (torch.uint8, torch.uint16, torch.uint32, torch.uint64)


def _stride_of(t: torch.Tensor) -> int:
    return int(t.stride(0)) if t.dim() == 1 and t.numel() > 1 else 1


def _signed_view(t: torch.Tensor) -> torch.Tensor:
    """Same bits as a signed integer tensor (collectives and indexing know these types)."""
    target = _SIGNED_VIEW[t.dtype.itemsize]
    return t if t.dtype == target else t.view(target)


class NativeEngine:
    """Local work on one B200 through the C ABI."""

    def __init__(self, accelerator: Accelerator):
        self.acc = accelerator
        self.device = accelerator.device
        self._temps: dict[str, torch.Tensor] = {}

    def _temp(self, tag: str, ints: int) -> torch.Tensor:
        t = self._temps.get(tag)
        if t is None or t.numel() < ints:
            t = self.acc.Allocate1D(max(ints, 64), torch.int32)
            self._temps[tag] = t
        return t

    def empty(self, n: int, dtype: torch.dtype) -> torch.Tensor:
        return torch.empty(int(n), dtype=dtype, device=self.device)

    def reduce(self, view: torch.Tensor, op: ScanReduceOperation) -> torch.Tensor:
        out = self.empty(1, op.dtype)
        self.acc.CreateReduction(op)(None, view, out)
        return out

    def scan(self, src, dst, op: ScanReduceOperation, kind: ScanKind, carry) -> None:
        temp = self._temp("scan", self.acc.ComputeScanTempStorageSize(op.dtype, src.numel()))
        self.acc.CreateScan(op, kind)(None, src, dst, temp, carry_in=carry)

    def histogram(self, view, bins, overflow, locator) -> None:
        self.acc.CreateHistogram(locator, checked=overflow is not None)(None, view, bins, overflow)

    def sort(self, keys, values, op: RadixSortOperation) -> None:
        n = keys.numel()
        if values is None:
            temp = self._temp("sort", self.acc.ComputeRadixSortTempStorageSize(op, n))
            self.acc.CreateRadixSort(op)(None, keys, temp)
        else:
            temp = self._temp("sort", self.acc.ComputeRadixSortPairsTempStorageSize(op, values.dtype, n))
            self.acc.CreateRadixSortPairs(op)(None, keys, values, temp)

    def partition(self, keys, values, op: RadixSortOperation, splitter_keys, splitter_index, index_base: int):
        n = keys.numel()
        L = self.acc.L
        need = ctypes.c_int64(0)
        B200AlgException.ThrowIfFailed(L.b200alg_bucket_partition_temp_bytes(dtype_code(keys.dtype), n, ctypes.byref(need)))
        temp = self._temp("partition", (need.value + 3) // 4)
        out_keys = torch.empty_like(keys)
        out_values = None if values is None else torch.empty_like(values)
        num_splitters = splitter_keys.numel()
        counts = self.empty(num_splitters + 1, torch.int64)
        with self.acc.Bind():
            B200AlgException.ThrowIfFailed(L.b200alg_bucket_partition(
                _stream_ptr(None), _ptr(keys), _ptr(values), n, dtype_code(keys.dtype),
                0 if values is None else values.dtype.itemsize, N.SORT_DESCENDING if op.descending else 0,
                _ptr(splitter_keys), _ptr(splitter_index), num_splitters, int(index_base),
                _ptr(out_keys), _ptr(out_values), _ptr(counts), _ptr(temp), temp.numel() * 4))
        return out_keys, out_values, counts

    # -- the partition in two steps, with the exchange fused into the second one --
    supports_peer_scatter = True

    def _partition_temp(self, keys) -> torch.Tensor:
        need = ctypes.c_int64(0)
        B200AlgException.ThrowIfFailed(self.acc.L.b200alg_bucket_partition_temp_bytes(
            dtype_code(keys.dtype), keys.numel(), ctypes.byref(need)))
        return self._temp("partition", (need.value + 3) // 4)

    def bucket_count(self, keys, op: RadixSortOperation, splitter_keys, splitter_index, index_base: int) -> torch.Tensor:
        temp = self._partition_temp(keys)
        counts = self.empty(splitter_keys.numel() + 1, torch.int64)
        with self.acc.Bind():
            B200AlgException.ThrowIfFailed(self.acc.L.b200alg_bucket_count(
                _stream_ptr(None), _ptr(keys), keys.numel(), dtype_code(keys.dtype),
                N.SORT_DESCENDING if op.descending else 0, _ptr(splitter_keys), _ptr(splitter_index),
                splitter_keys.numel(), int(index_base), _ptr(counts), _ptr(temp), temp.numel() * 4))
        return counts

    def select_splitters(self, sample_keys, sample_index, count, op: RadixSortOperation, num_picks: int):
        """The pairs of ranks (j + 1) * count / (num_picks + 1) among the first `count` (a device
        int64) samples, in the order a stable sort of the keys would give, without sorting."""
        max_m = sample_keys.numel()
        out_keys = self.empty(num_picks, sample_keys.dtype)
        out_index = self.empty(num_picks, torch.int64)
        temp = self._temp("select", max_m)
        with self.acc.Bind():
            B200AlgException.ThrowIfFailed(self.acc.L.b200alg_select_splitters(
                _stream_ptr(None), _ptr(sample_keys), _ptr(sample_index), max_m, _ptr(count),
                dtype_code(sample_keys.dtype), N.SORT_DESCENDING if op.descending else 0, int(num_picks),
                _ptr(out_keys), _ptr(out_index), _ptr(temp), temp.numel() * 4))
        return out_keys, out_index

    def bucket_scatter(self, keys, values, op: RadixSortOperation, splitter_keys, splitter_index, index_base: int,
                       key_pointers: list[int], value_pointers: list[int] | None) -> None:
        """Stores bucket b of this shard at key_pointers[b] (an address that may lie in a peer
        GPU's receive buffer): partition and exchange in one kernel."""
        temp = self._partition_temp(keys)
        table = torch.tensor(key_pointers + (value_pointers or []), dtype=torch.int64).to(self.device, non_blocking=True)
        nb = len(key_pointers)
        vtable = table[nb:] if value_pointers else None
        with self.acc.Bind():
            B200AlgException.ThrowIfFailed(self.acc.L.b200alg_bucket_scatter(
                _stream_ptr(None), _ptr(keys), _ptr(values), keys.numel(), dtype_code(keys.dtype),
                0 if values is None else values.dtype.itemsize, N.SORT_DESCENDING if op.descending else 0,
                _ptr(splitter_keys), _ptr(splitter_index), splitter_keys.numel(), int(index_base),
                _ptr(table), _ptr(vtable), _ptr(temp), temp.numel() * 4))
        self._keepalive = table   # the kernel reads the table asynchronously

    def peer_buffers(self, group, capacity: int) -> "PeerBuffers":
        pb = getattr(self, "_peer_buffers", None)
        if pb is None or pb.capacity < capacity:
            pb = PeerBuffers(group, self.device, max(capacity, 1 << 16))
            self._peer_buffers = pb
        return pb


class PeerBuffers:
    """Receive buffers that every rank of the group can store into: one symmetric-memory
    allocation per rank, mapped into all processes of the node (NVLink peer access).  The
    first half takes keys, the second half values; `capacity` is in elements of 8 bytes."""

    def __init__(self, group, device, capacity: int):
        import torch.distributed._symmetric_memory as symm
        self.capacity = int(capacity)
        self.buffer = symm.empty(self.capacity * 16, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buffer, group)
        self.pointers = [int(p) for p in self.handle.buffer_ptrs]

    def key_pointer(self, rank: int) -> int:
        return self.pointers[rank]

    def value_pointer(self, rank: int) -> int:
        return self.pointers[rank] + self.capacity * 8

    def local_keys(self, count: int, dtype: torch.dtype) -> torch.Tensor:
        return self.buffer[: count * dtype.itemsize].view(dtype)

    def local_values(self, count: int, dtype: torch.dtype) -> torch.Tensor:
        start = self.capacity * 8
        return self.buffer[start: start + count * dtype.itemsize].view(dtype)

    def barrier(self, channel: int) -> None:
        """Device-side barrier over the group, enqueued on the current stream."""
        self.handle.barrier(channel=channel)


def _identity_tensor(op: ScanReduceOperation, device) -> torch.Tensor:
    """One element holding the operation's Identity (0, MinValue or MaxValue)."""
    dt = op.dtype
    if op.op == N.ADD:
        return torch.zeros(1, dtype=_SIGNED_VIEW[dt.itemsize] if dt in _UNSIGNED else dt, device=device).view(dt)
    if dt.is_floating_point:
        info = torch.finfo(dt)
        return torch.full((1,), info.min if op.op == N.MAX else info.max, dtype=dt, device=device)
    if dt in _UNSIGNED:   # MinValue = all zero bits, MaxValue = all one bits
        return torch.full((1,), 0 if op.op == N.MAX else -1, dtype=_SIGNED_VIEW[dt.itemsize], device=device).view(dt)
    info = torch.iinfo(dt)
    return torch.full((1,), info.min if op.op == N.MAX else info.max, dtype=dt, device=device)


def _fold_lower_ranks(totals: torch.Tensor, rank: int, op: ScanReduceOperation) -> torch.Tensor | None:
    """Combines the totals of ranks < rank in rank order; None for rank 0 (= Identity)."""
    if rank == 0:
        return None
    lower = totals[:rank]
    dt = op.dtype
    if op.op == N.ADD:
        if dt.is_floating_point:
            return lower.to(torch.float64).sum().to(dt).reshape(1)
        s = _signed_view(lower).to(torch.int64).sum()          # wraps like unchecked C# arithmetic
        if dt.itemsize == 4:
            s = ((s + 2 ** 31) % 2 ** 32) - 2 ** 31
        return s.to(_SIGNED_VIEW[dt.itemsize]).reshape(1).view(dt)
    pick = torch.max if op.op == N.MAX else torch.min
    if dt in _UNSIGNED:
        flip = -(2 ** (dt.itemsize * 8 - 1))
        return (pick(_signed_view(lower) ^ flip) ^ flip).reshape(1).view(dt)
    return pick(lower).reshape(1)


class NativeComm:
    """A communicator of the native multi-GPU library for this rank of a process group
    (b200alg_comm_create_rank).  The process group only hands the rendezvous token round."""

    def __init__(self, accelerator: Accelerator, group, sort_capacity: int):
        self.acc = accelerator
        self.M = N.mg_lib()
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.sort_capacity = int(sort_capacity)
        token = [None]
        if self.rank == 0:
            buf = ctypes.create_string_buffer(N.UNIQUE_ID_BYTES)
            B200AlgException.ThrowIfFailed(self.M.b200alg_comm_unique_id(buf))
            token[0] = buf.raw
        dist.broadcast_object_list(token, src=dist.get_global_rank(group, 0), group=group)
        handle = ctypes.c_void_p()
        with self.acc.Bind():
            self._check(self.M.b200alg_comm_create_rank(token[0], self.world, self.rank, self.sort_capacity, ctypes.byref(handle)))
        self.handle = handle

    def _check(self, status: int) -> None:
        if status == N.NCCL_ERROR:
            raise B200AlgException(status)
        B200AlgException.ThrowIfFailed(status)

    def status(self, stream=None) -> None:
        """Synchronises; raises when a bounded wait between GPUs ran out or a receive buffer was too small."""
        with self.acc.Bind():
            self._check(self.M.b200alg_comm_status(self.handle, _stream_ptr(stream)))

    def destroy(self) -> None:
        if self.handle is not None:
            self.M.b200alg_comm_destroy(self.handle)
            self.handle = None


class ShardedAlgorithms:
    """The primitives over all ranks of a process group (one rank per GPU)."""

    SAMPLES_PER_RANK = 2048
    use_peer_scatter = True   # False: exchange the buckets with an NCCL all-to-all instead
    use_native = True         # False: the torch.distributed formulation also on GPUs

    def __init__(self, engine, group=None, sort_capacity: int | None = None):
        self.engine = NativeEngine(engine) if isinstance(engine, Accelerator) else engine
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self._sort_capacity = sort_capacity
        self._comm: NativeComm | None = None

    # -- native path --
    def _native(self) -> bool:
        return self.use_native and isinstance(self.engine, NativeEngine) and dist.get_backend(self.group) == "nccl"

    def _communicator(self, sort_elements: int | None = None) -> NativeComm:
        """The native communicator; (re)built collectively when the sort first needs a receive
        buffer (its capacity: 1.3 x the largest shard, unless given at construction)."""
        need_sort = sort_elements is not None and (self._comm is None or self._comm.sort_capacity == 0)
        if self._comm is None or need_sort:
            capacity = 0
            if sort_elements is not None:
                capacity = self._sort_capacity
                if capacity is None:
                    t = torch.tensor([sort_elements], dtype=torch.int64, device=self.engine.device)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
                    capacity = int(int(t.item()) * 1.3) + (1 << 16)
            if self._comm is not None:
                self._comm.destroy()
            self._comm = NativeComm(self.engine.acc, self.group, capacity)
        return self._comm

    def CheckStatus(self) -> None:
        if self._comm is not None:
            self._comm.status()

    # -- collectives on bit patterns --
    def _all_gather(self, t: torch.Tensor) -> torch.Tensor:
        s = _signed_view(t.contiguous())
        parts = [torch.empty_like(s) for _ in range(self.world)]
        dist.all_gather(parts, s, group=self.group)
        return torch.cat(parts).view(t.dtype)

    def _all_reduce(self, t: torch.Tensor, op_code: int) -> None:
        if op_code == N.ADD:
            dist.all_reduce(t if t.dtype.is_floating_point else _signed_view(t), op=dist.ReduceOp.SUM, group=self.group)
            return
        red = dist.ReduceOp.MAX if op_code == N.MAX else dist.ReduceOp.MIN
        if t.dtype in _UNSIGNED:
            s = _signed_view(t)
            flip = -(2 ** (t.dtype.itemsize * 8 - 1))
            s ^= flip
            dist.all_reduce(s, op=red, group=self.group)
            s ^= flip
        else:
            dist.all_reduce(t, op=red, group=self.group)

    # -- reduce --
    def Reduce(self, view: torch.Tensor, operation: ScanReduceOperation) -> torch.Tensor:
        """Every rank gets the fold over all shards (one element)."""
        if self._native():
            c = self._communicator()
            out = self.engine.empty(1, operation.dtype)
            with self.engine.acc.Bind():
                c._check(c.M.b200alg_reduce_mg(c.handle, _stream_ptr(None), _ptr(view), _stride_of(view), view.numel(),
                                               dtype_code(operation.dtype), operation.op, _ptr(out)))
            return out
        out = self.engine.reduce(view, operation)
        self._all_reduce(out, operation.op)
        return out

    # -- histogram --
    def Histogram(self, view, histogram, histogramOverflow, locator) -> None:
        """Adds the counts of all shards to every rank's ``histogram`` (replicas must agree
        on entry); ``histogramOverflow`` may be None (unchecked)."""
        if self._native():
            c = self._communicator()
            with self.engine.acc.Bind():
                c._check(c.M.b200alg_histogram_mg(c.handle, _stream_ptr(None), _ptr(view), _stride_of(view), view.numel(),
                                                  dtype_code(view.dtype), locator.code, float(locator.lo), float(locator.hi),
                                                  _ptr(histogram), histogram.numel(), dtype_code(histogram.dtype),
                                                  _ptr(histogramOverflow)))
            return
        local = torch.zeros_like(histogram)
        self.engine.histogram(view, local, None, locator)
        self._all_reduce(local, N.ADD)
        if histogramOverflow is not None and not histogram.dtype.is_floating_point:
            # an increment started from MaxValue iff the distance up to MaxValue is below the count
            bits = histogram.dtype.itemsize * 8
            h, c = _signed_view(histogram).to(torch.int64), _signed_view(local).to(torch.int64)
            if bits == 32:
                top = (2 ** 32 - 1) if histogram.dtype in _UNSIGNED else (2 ** 31 - 1)
                dist_to_max = (top - h) % 2 ** 32
                crossed = dist_to_max < (c % 2 ** 32)
            else:
                # 64-bit bins: compare in the unsigned order via the sign-flip trick
                top = -1 if histogram.dtype in _UNSIGNED else (2 ** 63 - 1)
                flip = -(2 ** 63)
                crossed = ((top - h) ^ flip) < (c ^ flip)
            histogramOverflow |= crossed.any().to(histogramOverflow.dtype)
        sh, sl = (histogram, local) if histogram.dtype.is_floating_point else (_signed_view(histogram), _signed_view(local))
        sh += sl

    # -- scan --
    def Scan(self, input: torch.Tensor, output: torch.Tensor, operation: ScanReduceOperation, kind: ScanKind) -> None:
        """Scan of the concatenation of all ranks' inputs (rank order); each rank writes its slice."""
        if self._native() and _stride_of(input) == 1 and _stride_of(output) == 1:
            c = self._communicator()
            n = input.numel()
            acc = self.engine.acc
            temp = self.engine._temp("scan", acc.ComputeScanTempStorageSize(operation.dtype, max(n, 1)))
            with acc.Bind():
                c._check(c.M.b200alg_scan_mg(c.handle, _stream_ptr(None), _ptr(input), _ptr(output), n,
                                             dtype_code(operation.dtype), operation.op, int(kind == ScanKind.Inclusive),
                                             _ptr(temp), temp.numel() * 4))
            return
        if input.numel() == 0:
            total = _identity_tensor(operation, input.device)
        else:
            total = self.engine.reduce(input, operation)
        totals = self._all_gather(total)
        carry = _fold_lower_ranks(totals, self.rank, operation)
        if input.numel():
            self.engine.scan(input, output, operation, kind, carry)

    # -- sort --
    # Global position of element i of rank r, as used for tie-breaking: r * 2^40 + i.  It only
    # has to be monotone in (rank, position), so no prefix sum of the shard sizes is needed.
    _RANK_SHIFT = 40

    def _sort(self, keys: torch.Tensor, values: torch.Tensor | None, operation: RadixSortOperation):
        eng, G, r = self.engine, self.world, self.rank
        n = keys.numel()
        device = keys.device
        s = self.SAMPLES_PER_RANK
        kview = _SIGNED_VIEW[keys.dtype.itemsize]
        base = r << self._RANK_SHIFT

        # 1. samples: evenly spaced (key, global position) pairs of this shard (with repeats
        #    when the shard is short), gathered together with the shard size in one message
        msg = torch.zeros(2 * s + 1, dtype=torch.int64, device=device)
        msg[0] = n
        if n:
            pos = (torch.arange(s, dtype=torch.int64, device=device) * n) // s
            msg[1:1 + s] = _signed_view(keys)[pos].to(torch.int64)
            msg[1 + s:] = pos + base
        table = self._all_gather(msg).view(G, 2 * s + 1)
        sizes = table[:, 0]
        # a rank without data has no samples: it borrows the block of the first rank that has some
        has = sizes > 0
        donor = torch.argmax(has.to(torch.int64))
        block = torch.where(has, torch.arange(G, device=device), donor)
        table = table[block]
        all_keys = table[:, 1:1 + s].reshape(-1).to(kview).view(keys.dtype).contiguous()
        all_index = table[:, 1 + s:].reshape(-1).contiguous()
        # blocks lie in rank order and positions ascend inside a block, so a stable sort by key
        # orders the (key, position) pairs
        eng.sort(all_keys, all_index, operation)
        cut = (torch.arange(1, G, dtype=torch.int64, device=device) * (G * s)) // G
        splitter_keys = _signed_view(all_keys)[cut].view(keys.dtype).contiguous()
        splitter_index = all_index[cut].contiguous()

        if G > 1 and getattr(eng, "supports_peer_scatter", False) and self.use_peer_scatter:
            return self._exchange_by_peer_stores(keys, values, operation, splitter_keys, splitter_index, base)

        # 2. stable partition of the shard into one bucket per rank
        if n:
            out_keys, out_values, counts = eng.partition(keys, values, operation, splitter_keys, splitter_index, base)
        else:
            out_keys, out_values, counts = keys, values, torch.zeros(G, dtype=torch.int64, device=device)

        # 3. exchange (the split sizes have to reach the host: the one synchronisation of the sort)
        matrix = self._all_gather(counts).view(G, G).tolist()      # matrix[src][dst]
        send = [int(c) for c in matrix[r]]
        recv = [int(matrix[src][r]) for src in range(G)]
        recv_keys = eng.empty(sum(recv), keys.dtype)
        dist.all_to_all_single(_signed_view(recv_keys), _signed_view(out_keys), recv, send, group=self.group)
        recv_values = None
        if values is not None:
            recv_values = eng.empty(sum(recv), values.dtype)
            dist.all_to_all_single(_signed_view(recv_values), _signed_view(out_values), recv, send, group=self.group)

        # 4. received runs lie in source-rank order; a stable local sort finishes the job
        if recv_keys.numel():
            eng.sort(recv_keys, recv_values, operation)
        return recv_keys, recv_values

    def _exchange_by_peer_stores(self, keys, values, operation, splitter_keys, splitter_index, base):
        """Steps 2-4 with the exchange fused into the partition: the partition kernel stores
        every bucket straight into its owner's receive buffer (peer memory over NVLink), so
        the data is written once and no separate all-to-all runs."""
        eng, G, r = self.engine, self.world, self.rank
        n = keys.numel()
        device = keys.device
        if n:
            counts = eng.bucket_count(keys, operation, splitter_keys, splitter_index, base)
        else:
            counts = torch.zeros(G, dtype=torch.int64, device=device)
        matrix = self._all_gather(counts).view(G, G).tolist()      # matrix[src][dst]; the one host sync
        column = [sum(matrix[src][dst] for src in range(G)) for dst in range(G)]
        peers = eng.peer_buffers(self.group, 2 * max(column))      # same decision on every rank
        kb = keys.dtype.itemsize
        # my block inside rank b's buffer starts after the blocks of the lower ranks
        start = [sum(matrix[src][b] for src in range(r)) for b in range(G)]
        key_pointers = [peers.key_pointer(b) + start[b] * kb for b in range(G)]
        value_pointers = None
        if values is not None:
            vb = values.dtype.itemsize
            value_pointers = [peers.value_pointer(b) + start[b] * vb for b in range(G)]
        peers.barrier(channel=0)      # every rank is done with what the previous call left in its buffer
        if n:
            eng.bucket_scatter(keys, values, operation, splitter_keys, splitter_index, base, key_pointers, value_pointers)
        peers.barrier(channel=1)      # every rank's stores have landed
        total = column[r]
        recv_keys = peers.local_keys(total, keys.dtype).clone()
        recv_values = None if values is None else peers.local_values(total, values.dtype).clone()
        if total:
            eng.sort(recv_keys, recv_values, operation)
        return recv_keys, recv_values

    def SortAsync(self, keys: torch.Tensor, values: torch.Tensor | None, operation: RadixSortOperation):
        """Enqueues the whole sort without a host synchronisation (native path only) and returns
        ``(out_keys, out_values, count)``: buffers of the communicator's capacity whose first
        ``count[0]`` elements (an int64 on the device) are rank r's slice of the sorted whole."""
        if keys.dtype != operation.dtype:
            raise NotSupportedException(f"keys are {keys.dtype}, operation sorts {operation.dtype}")
        if values is not None and values.dtype.itemsize not in (4, 8):
            raise NotSupportedException("values of 4 or 8 bytes")
        if not self._native():
            raise NotSupportedException("the asynchronous sort needs the native multi-GPU library")
        c = self._communicator(sort_elements=keys.numel())
        if keys.numel() > c.sort_capacity:
            raise ArgumentOutOfRangeException("the shard is larger than the communicator's sort capacity")
        cap = c.sort_capacity
        out_keys = self.engine.empty(cap, keys.dtype)
        out_values = None if values is None else self.engine.empty(cap, values.dtype)
        count = self.engine.empty(1, torch.int64)
        with self.engine.acc.Bind():
            c._check(c.M.b200alg_sort_mg(c.handle, _stream_ptr(None), _ptr(keys), _ptr(values), keys.numel(),
                                         dtype_code(keys.dtype), 0 if values is None else values.dtype.itemsize,
                                         N.SORT_DESCENDING if operation.descending else 0, _ptr(out_keys), _ptr(out_values),
                                         cap, _ptr(count)))
        return out_keys, out_values, count

    def SortKeys(self, keys: torch.Tensor, operation: RadixSortOperation):
        """Returns ``(sorted_slice, count)``: rank r holds the r-th slice of the sorted whole."""
        if keys.dtype != operation.dtype:
            raise NotSupportedException(f"keys are {keys.dtype}, operation sorts {operation.dtype}")
        if self._native():
            out, _, count = self.SortAsync(keys, None, operation)
            self.CheckStatus()                      # synchronises: the slice length is needed on the host now
            m = int(count.item())
            return out[:m], m
        out, _ = self._sort(keys, None, operation)
        return out, out.numel()

    def SortPairs(self, keys: torch.Tensor, values: torch.Tensor, operation: RadixSortOperation):
        """Stable: equal keys keep the order (rank, position) they had on entry."""
        if keys.dtype != operation.dtype:
            raise NotSupportedException(f"keys are {keys.dtype}, operation sorts {operation.dtype}")
        if values.dtype.itemsize not in (4, 8):
            raise NotSupportedException("values of 4 or 8 bytes")
        if self._native():
            out, outv, count = self.SortAsync(keys, values, operation)
            self.CheckStatus()
            m = int(count.item())
            return out[:m], outv[:m]
        return self._sort(keys, values, operation)

    def sort_launches_per_step(self, operation: RadixSortOperation) -> int:
        """Kernels of the library launched by one SortKeys call: the sample sort and the final
        sort (histogram, offsets, one pass per key byte, copy-back each) and the partition
        (bucket histogram, offsets, count export, one pass)."""
        passes = operation.dtype.itemsize
        if self._native():
            # samples, collect, rank + pick of the splitters, row of the size matrix, plan, 3 barriers;
            # the final sort (histogram, offsets, passes, copy-back); bucket sizes (3) and the partition (2)
            return 9 + (3 + passes) + 5
        return 2 * (3 + passes) + 4
