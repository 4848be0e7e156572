"""Writes tests/golden/reference_kats.npz: the known-answer cases of the reference's own
unit tests for this path, with the expected values computed the way those tests compute
them on the host (serial loops).  Nothing from the CPU oracle or the CUDA library is used.

  sort     RadixSortExtensionTests.tt:37-131, :144-365 - ramps from the test sequencers
           (Generic/AlgorithmsTestData.tt:74-96), worst case (inverted ramp), best case,
           constants 0 / 1 / -1, ascending and descending, pairs with keys = values.
  scan     ScanExtensionTests.tt:40-118 and CalcValues :286-305.
  reduce   ReductionExtensionTests.tt and CalcValue :205-212.
  hist     HistogramTests.tt:42-94 (inputs 1..1024, modulo bins, 64 / 256 bins) and the
           overflow scenario :146-203.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np

SIZES = [1, 31, 33, 127, 1027]                      # Generic/ConfigurationBase.tt:80
TYPES = {"Int32": np.int32, "Int64": np.int64, "UInt32": np.uint32, "UInt64": np.uint64,
         "Float": np.float32, "Double": np.float64}  # AtomicNumericTypes
SIGNED = ["Int32", "Int64", "Float", "Double"]


def sequence(t, start, step, length):
    seq = np.empty(length, dtype=t)
    seq[0] = t(start)
    with np.errstate(over="ignore"):
        for i in range(1, length):
            seq[i] = seq[i - 1] + t(step)
    return seq


def inverted_sequence(t, start, step, length):
    seq = np.empty(length, dtype=t)
    seq[length - 1] = t(start)
    with np.errstate(over="ignore"):
        for i in range(length - 2, -1, -1):
            seq[i] = seq[i + 1] + t(step)
    return seq


def identity(t, op):
    if op == "Add":
        return t(0)
    info = np.finfo(t) if np.dtype(t).kind == "f" else np.iinfo(t)
    return t(info.min) if op == "Max" else t(info.max)


def apply(t, op, a, b):
    with np.errstate(over="ignore"):
        if op == "Add":
            return t(a + b)
    return max(a, b) if op == "Max" else min(a, b)


def calc_values(t, values, op, inclusive):
    result = np.empty_like(values)
    result[0] = values[0]
    for i in range(1, len(values)):
        result[i] = apply(t, op, result[i - 1], values[i])
    if not inclusive:
        result = np.concatenate([np.asarray([identity(t, op)], dtype=t), result[:-1]])
    return result


def calc_value(t, values, op):
    r = values[0]
    for v in values[1:]:
        r = apply(t, op, r, v)
    return np.asarray([r], dtype=t)


def modulo_bin(tname, value, num_bins):
    if tname in ("Float", "Double"):
        return int(abs(np.fmod(value, TYPES[tname](num_bins))))
    return abs(int(np.fmod(int(value), num_bins)))     # C# % truncates toward zero


def apply_histogram(tname, bin_t, hist, values):
    info_max = np.finfo(bin_t).max if np.dtype(bin_t).kind == "f" else np.iinfo(bin_t).max
    overflow = False
    with np.errstate(over="ignore"):
        for v in values:
            b = modulo_bin(tname, v, len(hist))
            overflow |= bool(hist[b] == info_max)
            hist[b] = hist[b] + bin_t(1)
    return np.asarray([1 if overflow else 0], dtype=np.int32)


def main():
    out = {}
    for tname, t in TYPES.items():
        for size in SIZES:
            ramp = sequence(t, 0, 1, size)
            inv = inverted_sequence(t, 0, 1, size)
            for direction, expected in (("asc", ramp), ("desc", inv)):
                out[f"sort/{tname}/{direction}/worst/{size}/in"] = inv if direction == "asc" else ramp
                out[f"sort/{tname}/{direction}/worst/{size}/out"] = expected
                out[f"sort/{tname}/{direction}/best/{size}/in"] = expected
                out[f"sort/{tname}/{direction}/best/{size}/out"] = expected
            for c in [0, 1] + ([-1] if tname in SIGNED else []):
                const = sequence(t, c, 0, size)
                out[f"sort/{tname}/asc/const{c}/{size}/in"] = const
                out[f"sort/{tname}/asc/const{c}/{size}/out"] = const
            # The reference's pairs theory draws its sizes from ArraySizes.Skip(7), which is empty for
            # the five sizes above, so it never runs; these cases are built the way it would build them.
            if size in (127, 1027):
                out[f"pairs/{tname}/asc/{size}/in"] = inv
                out[f"pairs/{tname}/asc/{size}/out"] = ramp
            for op in ("Add", "Max", "Min"):
                cases = [("ascending", sequence(t, 0, 1, size))]
                if tname in SIGNED:
                    cases += [("descending", sequence(t, 0, -1, size)), ("const0", sequence(t, 0, 0, size)),
                              ("const1", sequence(t, 1, 0, size)), ("const-1", sequence(t, -1, 0, size))]
                for label, seq in cases:
                    if tname == "Float" and size > 1000:
                        continue
                    out[f"scan/{tname}/{op}/{label}/{size}/in"] = seq
                    out[f"scan/{tname}/{op}/{label}/{size}/incl"] = calc_values(t, seq, op, True)
                    out[f"scan/{tname}/{op}/{label}/{size}/excl"] = calc_values(t, seq, op, False)
                    out[f"reduce/{tname}/{op}/{label}/{size}/in"] = seq
                    out[f"reduce/{tname}/{op}/{label}/{size}/out"] = calc_value(t, seq, op)
    for in_name, in_t in TYPES.items():
        x = np.arange(1, 1025).astype(in_t)
        for bin_name, bin_t in TYPES.items():
            for num_bins in (64, 256):
                hist = np.zeros(num_bins, dtype=bin_t)
                ov = apply_histogram(in_name, bin_t, hist, x)
                out[f"hist/{in_name}/{bin_name}/{num_bins}/bins"] = hist
                out[f"hist/{in_name}/{bin_name}/{num_bins}/overflow"] = ov
            if np.dtype(bin_t).kind != "f":
                x32 = np.arange(1, 33).astype(in_t)
                hist = np.asarray([np.iinfo(bin_t).max - 32 - 1], dtype=bin_t)
                ov1 = apply_histogram(in_name, bin_t, hist, x32)
                out[f"histoverflow/{in_name}/{bin_name}/start"] = np.asarray([np.iinfo(bin_t).max - 32 - 1], dtype=bin_t)
                out[f"histoverflow/{in_name}/{bin_name}/after1"] = hist.copy()
                out[f"histoverflow/{in_name}/{bin_name}/overflow1"] = ov1
                ov2 = apply_histogram(in_name, bin_t, hist, x32)
                out[f"histoverflow/{in_name}/{bin_name}/after2"] = hist.copy()
                out[f"histoverflow/{in_name}/{bin_name}/overflow2"] = ov2
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kats.npz")
    np.savez_compressed(path, **out)
    print(f"{len(out)} arrays -> {path} ({os.path.getsize(path)} bytes)")


if __name__ == "__main__":
    main()
