"""Host logic of the multi-GPU primitives on CPU: two `gloo` ranks run
ilgpu_b200.multi_gpu.ShardedAlgorithms with the CPU oracle as the local engine (the
product engine is CUDA only), and every rank's result is compared with the single-array
answer."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleEngine:
    """CPU stand-in for NativeEngine built on the oracle (tests only)."""

    def __init__(self):
        from oracle import cpu_oracle
        self.o = cpu_oracle
        self.device = torch.device("cpu")

    def empty(self, n, dtype):
        return torch.empty(int(n), dtype=dtype)

    @staticmethod
    def _opname(op):
        return {0: "add", 1: "max", 2: "min"}[op.op]

    def reduce(self, view, op):
        return torch.from_numpy(np.asarray([self.o.reduce(view.numpy(), self._opname(op))], dtype=view.numpy().dtype))

    def scan(self, src, dst, op, kind, carry):
        from ilgpu_b200 import ScanKind
        x = src.numpy()
        inclusive = kind == ScanKind.Inclusive
        res = self.o.scan(x, self._opname(op), inclusive)
        if carry is not None:
            c = carry.numpy()[0]
            with np.errstate(over="ignore"):
                res = {"add": lambda: (res + c).astype(x.dtype), "max": lambda: np.maximum(res, c),
                       "min": lambda: np.minimum(res, c)}[self._opname(op)]()
        dst.numpy()[:] = res

    def histogram(self, view, bins, overflow, locator):
        name = "modulo" if locator.code == 1 else "equal_width_clamp"
        self.o.histogram(view.numpy(), bins.numpy(), name, locator.lo, locator.hi,
                         None if overflow is None else overflow.numpy())

    def sort(self, keys, values, op):
        k, v = self.o.radix_sort(keys.numpy(), None if values is None else values.numpy(), descending=op.descending)
        keys.numpy()[:] = k
        if values is not None:
            values.numpy()[:] = v

    def partition(self, keys, values, op, splitter_keys, splitter_index, index_base):
        name = {v: k for k, v in self.o.NP_DTYPES.items()}[keys.numpy().dtype.type]
        flip = (1 << 64) - 1 if op.descending else 0
        tk = np.asarray([self.o.key_bits(name, int(b)) ^ flip for b in keys.numpy().view(f"u{keys.dtype.itemsize}")], dtype=np.uint64)
        sk = [self.o.key_bits(name, int(b)) ^ flip for b in splitter_keys.numpy().view(f"u{keys.dtype.itemsize}")]
        si = splitter_index.numpy()
        gi = index_base + np.arange(keys.numel(), dtype=np.int64)
        bucket = np.zeros(keys.numel(), dtype=np.int64)
        for s_key, s_idx in zip(sk, si):
            bucket += ((np.uint64(s_key) < tk) | ((np.uint64(s_key) == tk) & (s_idx <= gi))).astype(np.int64)
        order = np.argsort(bucket, kind="stable")
        counts = torch.from_numpy(np.bincount(bucket, minlength=len(sk) + 1).astype(np.int64))
        out_k = torch.from_numpy(keys.numpy()[order].copy())
        out_v = None if values is None else torch.from_numpy(values.numpy()[order].copy())
        return out_k, out_v, counts


def _shard(a, rank, world, uneven=True):
    cuts = [0] + [int(len(a) * (i + 1) / world * (0.8 if uneven and i == 0 else 1.0)) for i in range(world)]
    cuts[-1] = len(a)
    return a[cuts[rank]:cuts[rank + 1]].copy()


def _worker(rank, world, port):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import ilgpu_b200 as ib
        from ilgpu_b200.multi_gpu import ShardedAlgorithms
        sh = ShardedAlgorithms(OracleEngine())
        sh.SAMPLES_PER_RANK = 64
        rng = np.random.default_rng(5)
        Ops, Sorts = ib.ScanReduceOperations, ib.RadixSortOperations

        # reduce and scan: int32 add (wrapping), uint32 max, float32 add, int64 min
        cases = [(rng.integers(-2 ** 31, 2 ** 31, 5001).astype(np.int32), Ops.AddInt32, "add"),
                 (rng.integers(0, 2 ** 32, 4000).astype(np.uint32), Ops.MaxUInt32, "max"),
                 (rng.integers(-2 ** 62, 2 ** 62, 3000).astype(np.int64), Ops.MinInt64, "min"),
                 (rng.random(6000).astype(np.float32), Ops.AddFloat, "add")]
        for full, op, name in cases:
            mine = torch.from_numpy(_shard(full, rank, world))
            got = sh.Reduce(mine, op).numpy()[0]
            with np.errstate(over="ignore"):
                ref = {"add": full.sum(dtype=full.dtype), "max": full.max(), "min": full.min()}[name]
            if full.dtype.kind == "f":
                assert abs(float(got) - float(ref)) <= 1e-5 * np.log2(full.size) * float(np.abs(full).sum())
            else:
                assert got == ref, (name, got, ref)
            for kind in (ib.ScanKind.Inclusive, ib.ScanKind.Exclusive):
                out = torch.empty_like(mine)
                sh.Scan(mine, out, op, kind)
                with np.errstate(over="ignore"):
                    incl = {"add": np.cumsum(full, dtype=full.dtype), "max": np.maximum.accumulate(full),
                            "min": np.minimum.accumulate(full)}[name]
                ident = np.asarray([op.Identity]).astype(full.dtype) if full.dtype.kind != "u" or name != "min" else np.asarray([np.iinfo(full.dtype).max], full.dtype)
                ref_full = incl if kind == ib.ScanKind.Inclusive else np.concatenate([ident, incl[:-1]])
                ref_mine = _shard(ref_full, rank, world)
                if full.dtype.kind == "f":
                    assert np.max(np.abs(out.numpy().astype(np.float64) - ref_mine)) <= 1e-5 * np.log2(full.size) * float(np.abs(full).sum())
                else:
                    np.testing.assert_array_equal(out.numpy(), ref_mine)

        # histogram with overflow flag: replicas agree before and after
        x = rng.standard_normal(7000).astype(np.float32)
        bins = torch.zeros(64, dtype=torch.int32)
        bins[10] = 2 ** 31 - 5           # close to MaxValue: the global count pushes it over
        ref_bins, ref_ov = bins.numpy().copy(), np.zeros(1, np.int32)
        from oracle import cpu_oracle
        cpu_oracle.histogram(x, ref_bins, "equal_width_clamp", -3.0, 3.0, ref_ov)
        ov = torch.zeros(1, dtype=torch.int32)
        sh.Histogram(torch.from_numpy(_shard(x, rank, world)), bins, ov, ib.EqualWidthClampLocator(-3.0, 3.0))
        np.testing.assert_array_equal(bins.numpy(), ref_bins)
        np.testing.assert_array_equal(ov.numpy(), ref_ov)

        # sort: keys (uniform), pairs with heavy duplicates (stability across ranks), descending signed
        keys = rng.integers(0, 2 ** 32, 9001).astype(np.uint32)
        out, count = sh.SortKeys(torch.from_numpy(_shard(keys, rank, world)), Sorts.AscendingUInt32)
        gathered = [None] * world
        dist.all_gather_object(gathered, out.numpy())
        np.testing.assert_array_equal(np.concatenate(gathered), np.sort(keys, kind="stable"))
        assert all(len(g) > 0.25 * len(keys) / world for g in gathered)     # balanced

        dup = rng.integers(0, 7, 8000).astype(np.uint64)                  # 7 distinct keys
        payload = np.arange(dup.size, dtype=np.uint32)
        k, v = sh.SortPairs(torch.from_numpy(_shard(dup, rank, world)), torch.from_numpy(_shard(payload, rank, world)),
                            Sorts.AscendingUInt64)
        dist.all_gather_object(gathered, (k.numpy(), v.numpy()))
        gk = np.concatenate([g[0] for g in gathered]); gv = np.concatenate([g[1] for g in gathered])
        order = np.argsort(dup, kind="stable")
        np.testing.assert_array_equal(gk, dup[order])
        np.testing.assert_array_equal(gv, payload[order])
        assert all(len(g[0]) > 0.25 * len(dup) / world for g in gathered)   # ties are split by position

        neg = rng.integers(-1000, 1000, 5000).astype(np.int32)
        k, v = sh.SortPairs(torch.from_numpy(_shard(neg, rank, world)),
                            torch.from_numpy(_shard(np.arange(neg.size, dtype=np.int64), rank, world)), Sorts.DescendingInt32)
        dist.all_gather_object(gathered, (k.numpy(), v.numpy()))
        order = np.argsort(-neg.astype(np.int64), kind="stable")
        np.testing.assert_array_equal(np.concatenate([g[0] for g in gathered]), neg[order])
        np.testing.assert_array_equal(np.concatenate([g[1] for g in gathered]), order)

        # a rank without data
        part = keys[:1000] if rank == 0 else keys[:0]
        out, _ = sh.SortKeys(torch.from_numpy(part.copy()), Sorts.AscendingUInt32)
        dist.all_gather_object(gathered, out.numpy())
        np.testing.assert_array_equal(np.concatenate(gathered), np.sort(keys[:1000]))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_algorithms_over_gloo(world):
    mp.spawn(_worker, args=(world, _free_port()), nprocs=world, join=True)
