// Tile descriptors of the chained (decoupled look-back) kernels: scan and unique.
#pragma once

#include "common.cuh"

namespace b200alg {

enum : unsigned int { kInvalid = 0u, kAggregate = 1u, kInclusive = 2u };

// Tile descriptors, one record of kDescStride bytes per tile.  Records are spread out so that
// the polls of many successor tiles do not all land on one L2 line.  4-byte types pack
// {flag, value} into one 64-bit word that is read and written with single (relaxed)
// accesses.  8-byte types keep the two partial results in separate slots of the record and
// publish the flag with release / acquire.
constexpr int kDescStride = 128;
static_assert(kDescStride >= 32 && kDescStride % 32 == 0, "a record holds flag + two 8-byte values");

template <typename T, int BYTES = sizeof(T)> struct TileState;

template <typename T> struct TileState<T, 4> {
    unsigned char *base;
    __host__ __device__ TileState(void *b, int) : base((unsigned char *)b) {}
    __device__ __forceinline__ unsigned long long *word(int tile) const {
        return (unsigned long long *)(base + (size_t)tile * kDescStride);
    }
    __device__ __forceinline__ void publish(int tile, unsigned int flag, T v) {
        unsigned int bits;
        memcpy(&bits, &v, 4);
        st_relaxed_u64(word(tile), ((unsigned long long)flag << 32) | bits);
    }
    __device__ __forceinline__ unsigned int poll(int tile, T &v) {
        unsigned long long w = ld_relaxed_u64(word(tile));
        unsigned int bits = (unsigned int)w;
        memcpy(&v, &bits, 4);
        return (unsigned int)(w >> 32);
    }
};

template <typename T> struct TileState<T, 8> {
    unsigned char *base;   // record: flag (4 bytes) at 0, aggregate at 8, inclusive at 16
    __host__ __device__ TileState(void *b, int) : base((unsigned char *)b) {}
    __device__ __forceinline__ void publish(int tile, unsigned int flag, T v) {
        unsigned char *rec = base + (size_t)tile * kDescStride;
        unsigned long long bits;
        memcpy(&bits, &v, 8);
        st_relaxed_u64((unsigned long long *)(rec + (flag == kInclusive ? 16 : 8)), bits);
        st_release_u32((unsigned int *)rec, flag);
    }
    __device__ __forceinline__ unsigned int poll(int tile, T &v) {
        unsigned char *rec = base + (size_t)tile * kDescStride;
        unsigned int f = ld_acquire_u32((const unsigned int *)rec);
        if (f != kInvalid) {
            unsigned long long bits = ld_relaxed_u64((const unsigned long long *)(rec + (f == kInclusive ? 16 : 8)));
            memcpy(&v, &bits, 8);
        }
        return f;
    }
};

}  // namespace b200alg
