"""GPU parity of the bucket partition entry points on one GPU (the multi-GPU sort's
partition + exchange step: b200alg_bucket_partition, b200alg_bucket_count,
b200alg_bucket_scatter), against a numpy restatement.

The reference has no multi-GPU sort; these entry points are checked against their own
definition: element i of a shard (global position base + i) goes to bucket
b = #{splitters (sk, si) : (sk, si) <= (key, base + i)} in the sort order of the operation,
and the partition is stable.  Everything is bit-exact.
"""
import numpy as np
import pytest
import torch

from ilgpu_b200 import RadixSortOperations as Ops
from ilgpu_b200.multi_gpu import NativeEngine
from oracle import cpu_oracle as oracle

pytestmark = pytest.mark.gpu


def _ordinal(keys: np.ndarray, descending: bool) -> np.ndarray:
    """Position of every key in the operation's order (ties share it), via the oracle's sort."""
    order, _ = oracle.radix_sort(keys, np.arange(keys.size, dtype=np.uint32), descending=descending)
    bits = keys.view({4: np.uint32, 8: np.uint64}[keys.dtype.itemsize])
    sorted_bits = order.view(bits.dtype)
    # rank of the first occurrence of each distinct bit pattern in the sorted sequence
    first = {}
    for pos, b in enumerate(sorted_bits.tolist()):
        first.setdefault(b, pos)
    return np.array([first[b] for b in bits.tolist()], dtype=np.int64)


def _expected(keys, descending, splitter_pos, base):
    """Buckets, given splitters that are elements of `keys` at positions splitter_pos."""
    ordinal = _ordinal(keys, descending)
    idx = np.arange(keys.size, dtype=np.int64) + base
    sp = sorted((int(ordinal[p]), int(idx[p])) for p in splitter_pos)
    bucket = np.zeros(keys.size, dtype=np.int64)
    for so, si in sp:
        bucket += (so < ordinal) | ((so == ordinal) & (si <= idx))
    return bucket, sp


CASES = [
    ("UInt32", np.uint32, 1), ("UInt32", np.uint32, 3), ("UInt32", np.uint32, 7), ("UInt32", np.uint32, 12),
    ("Int32", np.int32, 3), ("Float", np.float32, 5), ("UInt64", np.uint64, 7), ("Int64", np.int64, 2),
    ("Double", np.float64, 9),
]


@pytest.mark.parametrize("tname,np_t,num_splitters", CASES)
@pytest.mark.parametrize("direction", ["Ascending", "Descending"])
@pytest.mark.parametrize("n,distinct", [(5000, 0), (20011, 50), (70001, 3)])
def test_partition_count_scatter(accelerator, tname, np_t, num_splitters, direction, n, distinct):
    op = getattr(Ops, direction + tname)
    rng = np.random.default_rng(n + num_splitters)
    if distinct:
        pool = rng.integers(-1000, 1000, size=distinct).astype(np_t) if np.dtype(np_t).kind != "u" else \
            rng.integers(0, 2000, size=distinct).astype(np_t)
        keys = pool[rng.integers(0, distinct, size=n)]
    elif np.dtype(np_t).kind == "f":
        keys = rng.standard_normal(n).astype(np_t)
    else:
        info = np.iinfo(np_t)
        keys = rng.integers(info.min, info.max, size=n, dtype=np_t, endpoint=True)
    values = np.arange(n, dtype=np.uint32)
    base = 3 << 40
    splitter_pos = np.sort(rng.choice(n, size=num_splitters, replace=False))
    bucket, sp = _expected(keys, op.descending, splitter_pos, base)
    # splitters in ascending (key order, index) order, as the sample sort produces them
    by_index = {int(p) + base: int(p) for p in splitter_pos}
    ordered_pos = [by_index[si] for _, si in sp]
    splitter_keys = torch.from_numpy(keys[ordered_pos].copy().view(
        {4: np.int32, 8: np.int64}[keys.dtype.itemsize])).cuda().view(op.dtype)
    splitter_index = torch.tensor([si for _, si in sp], dtype=torch.int64, device="cuda")

    stable = np.argsort(bucket, kind="stable")
    want_keys, want_values = keys[stable], values[stable]
    want_counts = np.bincount(bucket, minlength=num_splitters + 1)

    eng = NativeEngine(accelerator)
    dkeys = torch.from_numpy(keys.view({4: np.int32, 8: np.int64}[keys.dtype.itemsize]).copy()).cuda().view(op.dtype)
    dvalues = torch.from_numpy(values.view(np.int32).copy()).cuda().view(torch.uint32)

    def bits(t):
        return t.view({4: torch.int32, 8: torch.int64}[t.dtype.itemsize]).cpu().numpy()
    want_bits = want_keys.view({4: np.int32, 8: np.int64}[keys.dtype.itemsize])

    # partition into one output array
    out_keys, out_values, counts = eng.partition(dkeys, dvalues, op, splitter_keys, splitter_index, base)
    assert counts.cpu().numpy().tolist() == want_counts.tolist()
    assert np.array_equal(bits(out_keys), want_bits)
    assert np.array_equal(bits(out_values).view(np.uint32), want_values)

    # sizes only
    counts2 = eng.bucket_count(dkeys, op, splitter_keys, splitter_index, base)
    assert counts2.cpu().numpy().tolist() == want_counts.tolist()

    # one destination per bucket (here: slices of local buffers, in reverse bucket order)
    recv_keys = torch.zeros(n, dtype=dkeys.dtype, device="cuda")
    recv_values = torch.zeros(n, dtype=torch.uint32, device="cuda")
    starts = np.concatenate([[0], np.cumsum(want_counts[::-1])])[:-1][::-1]   # bucket b starts here
    kp = [recv_keys.data_ptr() + int(starts[b]) * keys.dtype.itemsize for b in range(num_splitters + 1)]
    vp = [recv_values.data_ptr() + int(starts[b]) * 4 for b in range(num_splitters + 1)]
    eng.bucket_scatter(dkeys, dvalues, op, splitter_keys, splitter_index, base, kp, vp)
    torch.cuda.synchronize()
    got_k, got_v = bits(recv_keys), bits(recv_values).view(np.uint32)
    offs = np.concatenate([[0], np.cumsum(want_counts)])
    for b in range(num_splitters + 1):
        lo, hi = int(offs[b]), int(offs[b + 1])
        s = int(starts[b])
        assert np.array_equal(got_k[s:s + hi - lo], want_bits[lo:hi]), f"bucket {b} keys"
        assert np.array_equal(got_v[s:s + hi - lo], want_values[lo:hi]), f"bucket {b} values"

    # keys only
    out_keys, _, counts = eng.partition(dkeys, None, op, splitter_keys, splitter_index, base)
    assert np.array_equal(bits(out_keys), want_bits)


@pytest.mark.parametrize("tname,np_t", [("UInt32", np.uint32), ("Int32", np.int32), ("Float", np.float32),
                                         ("UInt64", np.uint64), ("Double", np.float64)])
@pytest.mark.parametrize("direction", ["Ascending", "Descending"])
@pytest.mark.parametrize("slots,count,picks,distinct", [(4096, 4096, 1, 0), (4096, 4096, 7, 5), (6144, 4100, 3, 0),
                                                        (2048, 5, 7, 2), (2048, 0, 3, 0), (16384, 16384, 7, 40)])
def test_select_splitters(accelerator, tname, np_t, direction, slots, count, picks, distinct):
    """b200alg_select_splitters against a stable sort of the first `count` samples."""
    op = getattr(Ops, direction + tname)
    rng = np.random.default_rng(slots + count + picks)
    if distinct:
        keys = rng.integers(0, distinct, size=slots).astype(np_t)
        if np.dtype(np_t).kind != "u":
            keys = keys - np_t(distinct // 2)
    elif np.dtype(np_t).kind == "f":
        keys = rng.standard_normal(slots).astype(np_t)
    else:
        info = np.iinfo(np_t)
        keys = rng.integers(info.min, info.max, size=slots, dtype=np_t, endpoint=True)
    index = rng.integers(0, 1 << 50, size=slots, dtype=np.int64)
    raw = {4: np.int32, 8: np.int64}[keys.dtype.itemsize]
    eng = NativeEngine(accelerator)
    dkeys = torch.from_numpy(keys.view(raw).copy()).cuda().view(op.dtype)
    dindex = torch.from_numpy(index).cuda()
    dcount = torch.tensor([count], dtype=torch.int64, device="cuda")
    got_keys, got_index = eng.select_splitters(dkeys, dindex, dcount, op, picks)
    torch.cuda.synchronize()
    got_k = got_keys.view({4: torch.int32, 8: torch.int64}[keys.dtype.itemsize]).cpu().numpy()
    got_i = got_index.cpu().numpy()
    if count == 0:
        assert not got_k.any() and not got_i.any()
        return
    ordinal = _ordinal(keys[:count], op.descending)
    by_rank = np.argsort(ordinal, kind="stable")      # slot order breaks ties
    want = [int(by_rank[((j + 1) * count) // (picks + 1)]) for j in range(picks)]
    assert np.array_equal(got_k, keys.view(raw)[want])
    assert np.array_equal(got_i, index[want])
