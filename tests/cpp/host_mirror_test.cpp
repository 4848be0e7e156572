// Exercises the C++ host mirror (include/ilgpu_algorithms.hpp) the way the reference's xunit
// suites exercise ILGPU.Algorithms: ramps of the sizes 1/31/33/127/1027 from the test
// sequencers, worst / best / constant sort cases, inclusive and exclusive scans with Add / Max /
// Min, reductions with and without an output view, modulo-bin histograms of 1..1024 and the
// overflow scenario, provider objects, and the argument errors
// (Src/ILGPU.Algorithms.Tests/RadixSortExtensionTests.tt, ScanExtensionTests.tt,
// ReductionExtensionTests.tt, HistogramTests.tt).  Expected values are computed on the host with
// serial loops, as those tests do.  Exit code 0 = all checks passed.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <vector>

#include "ilgpu_algorithms.hpp"

using namespace ILGPU;
using namespace ILGPU::Algorithms;

static int g_checks = 0, g_failures = 0;
#define CHECK(cond)                                                                 \
    do {                                                                            \
        ++g_checks;                                                                 \
        if (!(cond)) { ++g_failures; std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)

template <typename T> std::vector<T> ComputeSequence(T start, T step, int length) {
    std::vector<T> s(length);
    s[0] = start;
    for (int i = 1; i < length; ++i) s[i] = (T)(s[i - 1] + step);
    return s;
}
template <typename T> std::vector<T> ComputeInvertedSequence(T start, T step, int length) {
    std::vector<T> s(length);
    s[length - 1] = start;
    for (int i = length - 2; i >= 0; --i) s[i] = (T)(s[i + 1] + step);
    return s;
}

template <typename T> std::vector<T> Download(const MemoryBuffer1D<T> &b) {
    std::vector<T> h(b.Length());
    b.CopyToCPU(h.data());
    return h;
}

static const int kSizes[] = {1, 31, 33, 127, 1027};

template <typename T, typename Asc, typename Desc> void SortTests(const Accelerator &acc) {
    AcceleratorStream stream;
    for (int size : kSizes) {
        auto ramp = ComputeSequence<T>(0, 1, size);
        auto inverted = ComputeInvertedSequence<T>(0, 1, size);
        auto buf = acc.Allocate1D<T>(size);
        auto temp = acc.Allocate1D<int>(ComputeRadixSortTempStorageSize<T, Asc>(acc, size));
        auto asc = CreateRadixSort<T, Stride1D::Dense, Asc>(acc);
        auto desc = CreateRadixSort<T, Stride1D::Dense, Desc>(acc);
        for (const auto &input : {inverted, ramp}) {  // worst case, best case
            buf->CopyFromCPU(input.data());
            asc(stream, buf->View(), temp->View());
            acc.Synchronize();
            CHECK(Download(*buf) == ramp);
            buf->CopyFromCPU(input.data());
            desc(stream, buf->View(), temp->View());
            acc.Synchronize();
            CHECK(Download(*buf) == inverted);
        }
        for (int c : {0, 1, -1}) {
            if (c < 0 && !std::numeric_limits<T>::is_signed) continue;
            auto constant = ComputeSequence<T>((T)c, 0, size);
            buf->CopyFromCPU(constant.data());
            asc(stream, buf->View(), temp->View());
            acc.Synchronize();
            CHECK(Download(*buf) == constant);
        }
        // provider API
        auto provider = CreateRadixSortProvider<T, Asc>(acc, size);
        auto buffered = provider.template CreateRadixSort<T, Stride1D::Dense, Asc>();
        buf->CopyFromCPU(inverted.data());
        buffered(stream, buf->View());
        acc.Synchronize();
        CHECK(Download(*buf) == ramp);
        // pairs: keys = values = inverted ramp
        if (size >= 127) {
            auto keys = acc.Allocate1D<T>(size);
            auto values = acc.Allocate1D<T>(size);
            keys->CopyFromCPU(inverted.data());
            values->CopyFromCPU(inverted.data());
            auto pairs_provider = CreateRadixSortPairsProvider<T, T, Asc>(acc, size);
            pairs_provider.template CreateRadixSortPairs<T, T, Asc>()(stream, keys->View(), values->View());
            acc.Synchronize();
            CHECK(Download(*keys) == ramp);
            CHECK(Download(*values) == ramp);
        }
    }
}

template <typename Op> typename Op::T Apply(typename Op::T a, typename Op::T b) {
    using T = typename Op::T;
    if (Op::Op == B200ALG_ADD) return (T)(a + b);
    return Op::Op == B200ALG_MAX ? std::max(a, b) : std::min(a, b);
}

template <typename Op> void ScanReduceTests(const Accelerator &acc) {
    using T = typename Op::T;
    AcceleratorStream stream;
    for (int size : kSizes) {
        if (std::is_same<T, float>::value && size > 1000) continue;  // the reference skips these
        std::vector<std::vector<T>> sequences = {ComputeSequence<T>(0, 1, size), ComputeSequence<T>(0, 0, size),
                                                 ComputeSequence<T>(1, 0, size)};
        if (std::numeric_limits<T>::is_signed) {
            sequences.push_back(ComputeSequence<T>(0, (T)-1, size));
            sequences.push_back(ComputeSequence<T>((T)-1, 0, size));
        }
        auto input = acc.Allocate1D<T>(size);
        auto output = acc.Allocate1D<T>(size);
        auto temp = acc.Allocate1D<int>(ComputeScanTempStorageSize<T>(acc, size));
        for (const auto &seq : sequences) {
            input->CopyFromCPU(seq.data());
            // CalcValues (ScanExtensionTests.tt:286-305)
            std::vector<T> inclusive(size);
            inclusive[0] = seq[0];
            for (int i = 1; i < size; ++i) inclusive[i] = Apply<Op>(inclusive[i - 1], seq[i]);
            std::vector<T> exclusive(size);
            exclusive[0] = Op::Identity();
            for (int i = 1; i < size; ++i) exclusive[i] = inclusive[i - 1];
            CreateScan<T, Stride1D::Dense, Stride1D::Dense, Op>(acc, ScanKind::Inclusive)(stream, input->View(), output->View(), temp->View());
            acc.Synchronize();
            CHECK(Download(*output) == inclusive);
            auto provider = CreateScanProvider<T>(acc, size);
            provider.template CreateScan<T, Stride1D::Dense, Stride1D::Dense, Op>(ScanKind::Exclusive)(stream, input->View(), output->View());
            acc.Synchronize();
            CHECK(Download(*output) == exclusive);
            // CalcValue (ReductionExtensionTests.tt:205-212)
            const T expected = inclusive[size - 1];
            CHECK((Reduce<T, Stride1D::Dense, Op>(acc, stream, ArrayView1D<T>(input->View())) == expected));
            auto cell = acc.Allocate1D<T>(1);
            Reduce<T, Stride1D::Dense, Op>(acc, stream, ArrayView1D<T>(input->View()), cell->View());
            acc.Synchronize();
            CHECK(Download(*cell)[0] == expected);
        }
    }
}

template <typename T, typename TBin> void HistogramTests(const Accelerator &acc) {
    AcceleratorStream stream;
    const int length = 1024;
    std::vector<T> values(length);
    for (int i = 0; i < length; ++i) values[i] = (T)(i + 1);
    auto input = acc.Allocate1D<T>(length);
    input->CopyFromCPU(values.data());
    for (int numBins : {64, 256}) {
        std::vector<TBin> expected(numBins, TBin(0));
        for (T v : values) expected[(int)std::fabs(std::fmod((double)v, (double)numBins))] += TBin(1);
        auto histogram = acc.Allocate1D<TBin>(numBins);
        histogram->MemSetToZero();
        auto overflow = acc.Allocate1D<int>(1);
        overflow->MemSetToZero();
        Histogram<T, Stride1D::Dense, TBin>(acc, stream, ArrayView1D<T>(input->View()), histogram->View(), overflow->View(), ModuloBinOperation());
        acc.Synchronize();
        CHECK(Download(*histogram) == expected);
        CHECK(Download(*overflow)[0] == 0);
    }
    if (std::numeric_limits<TBin>::is_integer) {
        // HistogramTests.tt:146-203: one bin just below MaxValue, 32 inputs, applied twice
        const int n = 32;
        auto small = acc.Allocate1D<T>(n);
        small->CopyFromCPU(values.data());
        TBin bin = (TBin)(std::numeric_limits<TBin>::max() - (TBin)n - 1);
        auto histogram = acc.Allocate1D<TBin>(1);
        histogram->CopyFromCPU(&bin);
        auto overflow = acc.Allocate1D<int>(1);
        overflow->MemSetToZero();
        Histogram<T, Stride1D::Dense, TBin>(acc, stream, ArrayView1D<T>(small->View()), histogram->View(), overflow->View(), ModuloBinOperation());
        acc.Synchronize();
        CHECK(Download(*overflow)[0] == 0);
        CHECK(Download(*histogram)[0] == (TBin)(std::numeric_limits<TBin>::max() - 1));
        Histogram<T, Stride1D::Dense, TBin>(acc, stream, ArrayView1D<T>(small->View()), histogram->View(), overflow->View(), ModuloBinOperation());
        acc.Synchronize();
        CHECK(Download(*overflow)[0] == 1);
    }
}

template <typename E, typename F> bool Throws(F f) {
    try { f(); } catch (const E &) { return true; } catch (...) { return false; }
    return false;
}

void ArgumentTests(const Accelerator &acc) {
    AcceleratorStream stream;
    auto data = acc.Allocate1D<int32_t>(64);
    auto temp = acc.Allocate1D<int>(1 << 16);
    using Add = ScanReduceOperations::AddInt32;
    auto scan = CreateScan<int32_t, Stride1D::Dense, Stride1D::Dense, Add>(acc, ScanKind::Inclusive);
    CHECK(Throws<ArgumentNullException>([&] { scan(stream, ArrayView1D<int32_t>(), data->View(), temp->View()); }));
    CHECK(Throws<ArgumentOutOfRangeException>([&] { scan(stream, data->View(), data->View().SubView(0, 8), temp->View()); }));
    CHECK(Throws<ArgumentOutOfRangeException>([&] { scan(stream, data->View(), data->View(), temp->View().SubView(0, 2)); }));
    auto reduce = CreateReduction<int32_t, Stride1D::Dense, Add>(acc);
    CHECK(Throws<ArgumentOutOfRangeException>([&] { reduce(stream, ArrayView1D<int32_t>(data->View().SubView(0, 0)), data->View()); }));
    CHECK(Throws<ArgumentNullException>([&] { reduce(stream, data->View(), ArrayView<int32_t>()); }));
    auto sort = CreateRadixSort<int32_t, Stride1D::Dense, RadixSortOperations::AscendingInt32>(acc);
    CHECK(Throws<ArgumentOutOfRangeException>([&] { sort(stream, data->View(), temp->View().SubView(0, 2)); }));
    // strided view: every third element is sorted, the others stay
    std::vector<int32_t> host(64);
    for (int i = 0; i < 64; ++i) host[i] = 1000 - i;
    data->CopyFromCPU(host.data());
    auto strided_sort = CreateRadixSort<int32_t, Stride1D::General, RadixSortOperations::AscendingInt32>(acc);
    strided_sort(stream, AsGeneral(data->View(), 3), temp->View());
    acc.Synchronize();
    auto got = Download(*data);
    bool ok = true;
    for (int i = 0; i < 64; ++i) {
        if (i % 3) ok = ok && got[i] == host[i];
        else if (i >= 3) ok = ok && got[i] >= got[i - 3];
    }
    CHECK(ok);
}

int main() {
    try {
        Accelerator acc(0);
        namespace S = RadixSortOperations;
        SortTests<int32_t, S::AscendingInt32, S::DescendingInt32>(acc);
        SortTests<int64_t, S::AscendingInt64, S::DescendingInt64>(acc);
        SortTests<uint32_t, S::AscendingUInt32, S::DescendingUInt32>(acc);
        SortTests<uint64_t, S::AscendingUInt64, S::DescendingUInt64>(acc);
        SortTests<float, S::AscendingFloat, S::DescendingFloat>(acc);
        SortTests<double, S::AscendingDouble, S::DescendingDouble>(acc);
        namespace R = ScanReduceOperations;
        ScanReduceTests<R::AddInt32>(acc); ScanReduceTests<R::MaxInt32>(acc); ScanReduceTests<R::MinInt32>(acc);
        ScanReduceTests<R::AddInt64>(acc); ScanReduceTests<R::MaxInt64>(acc); ScanReduceTests<R::MinInt64>(acc);
        ScanReduceTests<R::AddUInt32>(acc); ScanReduceTests<R::MaxUInt32>(acc); ScanReduceTests<R::MinUInt32>(acc);
        ScanReduceTests<R::AddUInt64>(acc); ScanReduceTests<R::MaxUInt64>(acc); ScanReduceTests<R::MinUInt64>(acc);
        ScanReduceTests<R::AddFloat>(acc); ScanReduceTests<R::MaxFloat>(acc); ScanReduceTests<R::MinFloat>(acc);
        ScanReduceTests<R::AddDouble>(acc); ScanReduceTests<R::MaxDouble>(acc); ScanReduceTests<R::MinDouble>(acc);
        HistogramTests<int32_t, int32_t>(acc); HistogramTests<int64_t, uint32_t>(acc); HistogramTests<uint32_t, int64_t>(acc);
        HistogramTests<uint64_t, uint64_t>(acc); HistogramTests<float, float>(acc); HistogramTests<double, double>(acc);
        HistogramTests<float, int32_t>(acc);
        ArgumentTests(acc);
    } catch (const std::exception &e) {
        std::printf("EXCEPTION: %s\n", e.what());
        return 2;
    }
    std::printf("%d checks, %d failures\n", g_checks, g_failures);
    return g_failures == 0 ? 0 : 1;
}
