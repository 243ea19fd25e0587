// Device helpers shared by the top-k kernels: sortable 64-bit keys, a block-wide bitonic sort and a
// block-wide radix select.
#pragma once

#include <stdint.h>

namespace tqtopk {

static __device__ __forceinline__ uint32_t ordered_bits(float s) {
    // negative: all bits flipped, otherwise the sign bit set -- as one shift and one three-input logic operation
    const uint32_t u = __float_as_uint(s);
    return u ^ ((uint32_t)((int32_t)u >> 31) | 0x80000000u);
}
static __device__ __forceinline__ unsigned long long make_key(float s, uint32_t row) {
    return ((unsigned long long)ordered_bits(s) << 32) | (unsigned long long)(0xffffffffu - row);
}
static __device__ void block_sort_desc(unsigned long long* a, int n2) {
    for (int k = 2; k <= n2; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < n2; i += blockDim.x) {
                const int l = i ^ j;
                if (l > i) {
                    const unsigned long long x = a[i], y = a[l];
                    const bool desc = (i & k) == 0;
                    if (desc ? (x < y) : (x > y)) { a[i] = y; a[l] = x; }
                }
            }
        }
    __syncthreads();
}

constexpr int kSelThreads = 256;
constexpr int kSelPerThread = 8;
constexpr int kSelBatch = kSelPerThread * kSelThreads;   // scores examined between two looks at the buffer
constexpr int kSelCap = 4096;                            // candidate buffer (64-bit keys) per block

// Keep the `k` largest of the `c` distinct keys in buf[0..c) (c <= kSelCap), unsorted, in buf[0..k); returns
// the k-th largest key or a lower bound of it that no other key of the buffer reaches.  Radix select, 8 bits per pass from the top, with a 256-bin histogram in shared
// memory; far cheaper than sorting the buffer.  Whole block; c and k are uniform, k <= c.
static __device__ unsigned long long block_select_topk(unsigned long long* buf, int c, int k, int* hist /*[256]*/,
                                                int* scratch /*[4]*/) {
    unsigned long long prefix = 0ull, mask = 0ull;
    int remaining = k;
    for (int shift = 56; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < c; i += blockDim.x) {
            const unsigned long long key = buf[i];
            if ((key & mask) == prefix) atomicAdd(&hist[(int)((key >> shift) & 255ull)], 1);
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // lane l owns bins 255-8l .. 248-8l (descending); find where the running count reaches `remaining`
            const int lane = threadIdx.x;
            int mine = 0;
#pragma unroll
            for (int b = 0; b < 8; ++b) mine += hist[255 - 8 * lane - b];
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            const int before = incl - mine;  // keys in strictly higher bins of higher lanes
            if (before < remaining && incl >= remaining) {
                int acc = before;
                for (int b = 0; b < 8; ++b) {
                    const int bin = 255 - 8 * lane - b;
                    if (acc + hist[bin] >= remaining) {
                        scratch[0] = bin;
                        scratch[1] = remaining - acc;
                        scratch[3] = acc + hist[bin] == remaining;   // the whole bin belongs to the k largest
                        break;
                    }
                    acc += hist[bin];
                }
            }
        }
        __syncthreads();
        prefix |= (unsigned long long)scratch[0] << shift;
        mask |= 255ull << shift;
        remaining = scratch[1];
        const bool whole_bin = scratch[3] != 0;
        __syncthreads();
        if (whole_bin) break;   // every key with this prefix is in: the lower bits need no passes (usual after four)
    }
    // prefix is now the k-th largest key, or its leading bytes with zeros behind them when the selection stopped at a
    // bin that is taken whole; gather the keys >= prefix (exactly k, keys are distinct)
    unsigned long long keep[kSelCap / kSelThreads];
    int nkeep = 0;
    for (int i = threadIdx.x, j = 0; j < kSelCap / kSelThreads; i += blockDim.x, ++j) {
        keep[j] = 0ull;
        if (i < c) { const unsigned long long key = buf[i]; if (key >= prefix) { keep[j] = key; ++nkeep; } }
    }
    if (threadIdx.x == 0) scratch[2] = 0;
    __syncthreads();
    int pos = nkeep ? atomicAdd(&scratch[2], nkeep) : 0;
#pragma unroll
    for (int j = 0; j < kSelCap / kSelThreads; ++j)
        if (keep[j] != 0ull) buf[pos++] = keep[j];
    __syncthreads();
    return prefix;
}


static __device__ __forceinline__ float unordered_bits(uint32_t o) {
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}

}  // namespace tqtopk
