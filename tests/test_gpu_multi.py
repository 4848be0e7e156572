"""The multi-GPU primitives on real GPUs (NCCL, one process per GPU).  Needs at least two
devices; on a single-GPU box the test is skipped (the host logic is covered over gloo by
test_multi_gpu_gloo.py)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _shard(a, rank, world):
    return a[len(a) * rank // world: len(a) * (rank + 1) // world].copy()


def _worker(rank, world, port):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import ilgpu_b200 as ib
        from ilgpu_b200 import synthetic
        from ilgpu_b200.multi_gpu import ShardedAlgorithms
        sh = ShardedAlgorithms(ib.Accelerator(rank))
        Ops, Sorts = ib.ScanReduceOperations, ib.RadixSortOperations
        dev = lambda a: torch.from_numpy(a).cuda()

        n = 1 << 21
        x = synthetic.uniform_int32(n, seed=1)
        mine = dev(_shard(x, rank, world))
        assert int(sh.Reduce(mine, Ops.AddInt32).cpu()[0]) == int(x.sum(dtype=np.int32))
        out = torch.empty_like(mine)
        sh.Scan(mine, out, Ops.AddInt32, ib.ScanKind.Exclusive)
        ref = np.concatenate([[0], np.cumsum(x, dtype=np.int32)[:-1]]).astype(np.int32)
        np.testing.assert_array_equal(out.cpu().numpy(), _shard(ref, rank, world))

        f = synthetic.uniform_float32(n, seed=5)
        mine = dev(_shard(f, rank, world))
        tol = 1e-5 * np.log2(n) * float(np.abs(f.astype(np.float64)).sum())
        assert abs(float(sh.Reduce(mine, Ops.AddFloat).cpu()[0]) - float(f.astype(np.float64).sum())) <= tol
        out = torch.empty_like(mine)
        sh.Scan(mine, out, Ops.AddFloat, ib.ScanKind.Inclusive)
        ref = np.cumsum(f.astype(np.float64))
        assert np.max(np.abs(out.cpu().numpy().astype(np.float64) - _shard(ref, rank, world))) <= tol

        g = synthetic.normal_float32(n, seed=3)
        bins = torch.zeros(256, dtype=torch.int32, device="cuda")
        ov = torch.zeros(1, dtype=torch.int32, device="cuda")
        sh.Histogram(dev(_shard(g, rank, world)), bins, ov, ib.EqualWidthClampLocator(-4.0, 4.0))
        t = (g - np.float32(-4.0)) * np.float32(32.0)
        ref_bins = np.bincount(np.clip(np.floor(t), 0, 255).astype(np.int64), minlength=256).astype(np.int32)
        np.testing.assert_array_equal(bins.cpu().numpy(), ref_bins)
        assert int(ov.cpu()[0]) == 0

        keys = synthetic.uniform_uint32(n, seed=2)
        out, _ = sh.SortKeys(dev(_shard(keys, rank, world)), Sorts.AscendingUInt32)
        gathered = [None] * world
        dist.all_gather_object(gathered, out.cpu().numpy())
        np.testing.assert_array_equal(np.concatenate(gathered), np.sort(keys))

        zk = synthetic.zipf_uint64(n, seed=4)
        zv = np.arange(n, dtype=np.uint32)
        k, v = sh.SortPairs(dev(_shard(zk, rank, world)), dev(_shard(zv, rank, world)), Sorts.AscendingUInt64)
        dist.all_gather_object(gathered, (k.cpu().numpy(), v.cpu().numpy()))
        order = np.argsort(zk, kind="stable")
        np.testing.assert_array_equal(np.concatenate([p[0] for p in gathered]), zk[order])
        np.testing.assert_array_equal(np.concatenate([p[1] for p in gathered]), zv[order])
        sizes = [len(p[0]) for p in gathered]
        assert min(sizes) > 0.5 * n / world, sizes        # duplicates are split by position: balanced

        # uneven shards, one of them empty; descending signed keys with duplicates
        dk = synthetic.uniform_int32(n, seed=7, lo=-5000, hi=5000)
        cuts = [0, 0] + [n * r // world + 17 * r for r in range(2, world)] + [n]      # rank 0 holds nothing
        part = dk[cuts[rank]:cuts[rank + 1]].copy()
        uneven = ShardedAlgorithms(ib.Accelerator(rank), sort_capacity=n + 1024)      # a shard may be the whole input
        out, m = uneven.SortKeys(dev(part), Sorts.DescendingInt32)
        dist.all_gather_object(gathered, out.cpu().numpy())
        np.testing.assert_array_equal(np.concatenate(gathered), np.sort(dk)[::-1])

        # the measurement hook: the same sort with events where its phases meet
        import ctypes
        from ilgpu_b200.algorithms import dtype_code
        c = sh._communicator(sort_elements=n)
        fn = c.M.b200alg_testing_time_sort_mg
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                               ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]
        mine = dev(_shard(keys, rank, world))
        res = torch.empty(c.sort_capacity, dtype=torch.uint32, device="cuda")
        cnt = torch.zeros(1, dtype=torch.int64, device="cuda")
        ms = (ctypes.c_float * 6)()
        rc = fn(c.handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.c_void_p(mine.data_ptr()), None,
                mine.numel(), dtype_code(mine.dtype), 0, 0, ctypes.c_void_p(res.data_ptr()), None, c.sort_capacity,
                ctypes.c_void_p(cnt.data_ptr()), ms)
        assert rc == 0, rc
        assert all(0.0 <= x < 1000.0 for x in ms), list(ms)
        sh.CheckStatus()
        dist.all_gather_object(gathered, res[:int(cnt.item())].cpu().numpy())
        np.testing.assert_array_equal(np.concatenate(gathered), np.sort(keys))
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


def test_sharded_algorithms_over_nccl():
    world = torch.cuda.device_count()
    if world < 2:
        pytest.skip("needs at least two GPUs")
    world = min(world, 8)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port), nprocs=world, join=True)
