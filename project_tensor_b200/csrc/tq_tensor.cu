// Tensor-core quantizers for B200 (sm_100a): TMA in, tcgen05.mma with TMEM accumulators, SIMT epilogue.
//
// One persistent CTA per SM walks over tiles of 128 rows.  Per tile:
//
//   TMA (1 thread)      x tile, four 128-row x 32-float boxes with the 128-byte swizzle  -> smem ring
//   converters (8 warps) one thread per half row: sum of squares, scale to unit length * 2^10,
//                        split every value into fp16 hi + fp16 lo, tcgen05.st both as the A operand
//                        straight into tensor memory (lane = row) -- A never touches shared memory
//   MMA (1 thread)      acc = A_hi*B_hi + A_hi*B_lo + A_lo*B_hi with kind::f16, fp32 accumulate in
//                        TMEM; B = 2^10 * R split the same way, resident in smem for the whole kernel.
//                        The dropped lo*lo term is 2^-24 relative.
//   epilogue (4 warps)   one thread per row: tcgen05.ld 32 columns at a time, locate each value among
//                        the codebook boundaries through a 32-cell lookup table held in the lanes of
//                        the warp (one shuffle per table), pack codes, and flag the row if any value
//                        lies inside a guard band around a boundary.
//   TurboQuantProd adds: rho = value - centroid (still in the rotated basis), |rho|, rho split to
//                        fp16 hi/lo and stored back into the tile's A columns, a second MMA against
//                        B2 = 16 * (R S^T), and a sign/guard epilogue on that accumulator.
//                        residual S^T == rho (R S^T) because the residual is rho R.
//
// Flagged rows (about 1% of them) are recomputed afterwards by the exact kernel in the reference's
// own float32 operation order, so the packed output equals the reference's wherever the reference's
// own arithmetic decides, while 99% of the rows only ever see the tensor-core pass.
//
// Every wait is bounded: on a timeout the kernel records a status word, all roles leave their loops,
// tensor memory is released and the kernel returns.
#include "tq_common.cuh"
#include "tq_ptx.cuh"

#include <cuda.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

namespace {

using namespace tqptx;

constexpr int kTileRows = 128;
// Warps: TMA, MMA, then the workers.  UNI (the kernels that run): 16 workers, four per row, each owning 32 columns of
// its row through every phase of a tile -- conversion, first-accumulator epilogue and (TurboQuantProd) sign epilogue.
// All workers walk the same code, so whichever phase the tensor pipe has finished finds warps to run it; with the
// phases given to different warps (!UNI: converter warps and 8 epilogue warps, two per row; kept for comparison)
// the issue slots were idle 44 % of the time although every warp had a backlog, because each role waited for the other.
template <bool PROD, bool UNI> struct Threads {
    static constexpr int kEpiPerRow = UNI ? 0 : 2;
    static constexpr int kConvWarps = UNI ? 16 : (PROD ? 8 : 16);
    static constexpr int kFirstEpiWarp = 2 + kConvWarps;
    static constexpr int kThreads = (2 + kConvWarps + 4 * kEpiPerRow) * 32;
};
constexpr int kFirstConvWarp = 2;
constexpr int kBoxBytes = 128 * 128;     // 128 rows x 32 floats
constexpr float kScaleA = 1024.f;        // unit vector -> A operand
constexpr float kScaleB = 1024.f;        // rotation    -> B operand
constexpr float kAccScale = kScaleA * kScaleB;  // accumulator = 2^20 * rotated coordinate
constexpr float kScaleRho = 1.f / 1024.f;       // accumulator units -> 2^10 * rho for the second A operand
constexpr float kScaleM = 16.f;                 // R S^T -> second B operand
constexpr int kCells = 32;
constexpr int kPendCap = 32;               // second-stage entries staged per warp and list (a ballot adds up to 32)
constexpr float kCellMul = 31.99998f;

struct TensorArgs {
    const __half* bmat;      // [R_hi | R_lo | M_hi | M_lo], each d*d halves in the interleaved layout
    const float2* cell_lut;  // [32] per cell: boundary (x 2^20, +inf if none), boundaries below the cell (as int bits)
    const float* code_ncent; // [32] entry l: -centroid(l mod levels) * 2^10
    float cell_scale, cell_offset;
    float code_guard, sign_guard;  // in accumulator units
    int64_t n;
    int64_t ntiles;
    uint32_t* codes;
    uint32_t* signs;
    float* norms;
    float* rnorms;
    TqRecheck lists;
    unsigned long long* status;  // [0]: set to a non-zero code when a wait timed out
    int wait_kcycles;            // limit of one bounded wait, in units of 1024 cycles
#ifdef TQ_PROF
    long long* prof;             // cycle counters per role (measurement builds only)
#endif
};

// ---------------------------------------------------------------------------------------------
// Shared-memory plan
// ---------------------------------------------------------------------------------------------
constexpr int kW = 128;   // width of the operand layouts in tensor and shared memory; d = 64 is zero-padded to it
template <int D, bool PROD, bool UNI>
struct Smem {
    static constexpr int kBoxesPerTile = D / 32;
    static constexpr int kBBytes = kW * kW * 2;                     // one fp16 operand matrix (padded)
    static constexpr int kNumB = PROD ? 4 : 2;
    static constexpr int kRingBoxes = PROD ? 5 : 8;
    static constexpr int off_b = 0;
    static constexpr int off_ring = off_b + kNumB * kBBytes;
    static constexpr int off_misc = off_ring + kRingBoxes * kBoxBytes;  // sumsq exchange, force flags, barriers
    static constexpr int kPendWarps = Threads<PROD, UNI>::kConvWarps + 4 * Threads<PROD, UNI>::kEpiPerRow;   // every worker warp
                                                                // stages entries: a 64-bit and a 32-bit list each
    static constexpr int kPendBytes = kPendWarps * kPendCap * (8 + 4);
    static constexpr int kRsSlots = UNI ? 3 : 4;                 // tiles whose |rho|^2 partial sums are alive at once
    static constexpr int kRsParts = UNI ? 4 : 2;                 // threads per row in the first epilogue
    static constexpr int kRsBytes = kRsSlots * kRsParts * kTileRows * 4;
    static constexpr int kMiscBytes = 8 * kTileRows * 4 + 4 * kTileRows + 512 + kRsBytes + kCells * 16 + kPendBytes;
    static constexpr int total = off_misc + kMiscBytes + 1024;      // + slack to align the base to 1024
    static_assert(total <= 227 * 1024, "shared memory plan");
};

// barrier indices inside the barrier block
enum {
    BAR_FULL = 0,                 // [8]  ring slot filled by TMA
    BAR_EMPTY = 8,                // [8]  ring slot drained by the converters
    BAR_A_FULL = 16,              // [2]
    BAR_A_EMPTY = 18,             // [2]
    BAR_ACC_FULL = 20,            // [2]
    BAR_ACC_EMPTY = 22,           // [2]
    BAR_RHO_FULL = 24,            // [2]
    BAR_ACC2_FULL = 26,           // [2]
    BAR_COUNT = 28
};

// Work for the exact second stage is rare (about one row in a hundred), but a global atomic per entry
// would stall the epilogue warp for a memory round trip each time.  Every epilogue warp therefore
// collects its entries in a private shared-memory buffer and reserves space in the global lists
// once per batch.
struct WarpPending {
    unsigned long long* codes;  // [kPendCap]
    unsigned int* rows;         // [kPendCap]
    int n_codes, n_rows;        // warp-uniform
};

__device__ __noinline__ void flush_pending_codes(const TqRecheck& l, WarpPending& w, int lane) {
    __syncwarp();
    unsigned int base = 0;
    if (lane == 0) base = atomicAdd(&l.hdr->n_codes, (unsigned int)w.n_codes);
    base = __shfl_sync(0xffffffffu, base, 0);
    for (int i = lane; i < w.n_codes; i += 32) {
        if (base + i < l.code_cap) l.code_entries[base + i] = w.codes[i];
        else l.hdr->overflow = 1u;
    }
    __syncwarp();
    w.n_codes = 0;
}
__device__ __noinline__ void flush_pending_rows(const TqRecheck& l, WarpPending& w, int lane) {
    __syncwarp();
    unsigned int base = 0;
    if (lane == 0) base = atomicAdd(&l.hdr->n_rows, (unsigned int)w.n_rows);
    base = __shfl_sync(0xffffffffu, base, 0);
    for (int i = lane; i < w.n_rows; i += 32) {
        if (base + i < l.row_cap) l.row_entries[base + i] = w.rows[i];
        else l.hdr->overflow = 1u;
    }
    __syncwarp();
    w.n_rows = 0;
}
// Whole warp: every lane with `want` appends its row.
__device__ __forceinline__ void pend_rows(const TqRecheck& l, WarpPending& w, bool want, int64_t row, int lane) {
    const uint32_t votes = __ballot_sync(0xffffffffu, want);
    if (votes == 0u) return;
    if (w.n_rows + __popc(votes) > kPendCap) flush_pending_rows(l, w, lane);
    if (want) w.rows[w.n_rows + __popc(votes & ((1u << lane) - 1u))] = (unsigned int)row;
    w.n_rows += __popc(votes);
}

// One 32-column chunk of the first accumulator for one row: codes (packed into w), guard-band test,
// and for TurboQuantProd the scaled residual split into fp16 hi/lo pairs;
// the lookup tables live in the lanes of the warp: lut_bnd / lut_base1 (boundaries below the cell) by cell, lut_ncent by code.
// (One shuffle instead of two -- the count packed into the low mantissa bits of the boundary, taken apart with an AND --
// was slower: 217 -> 226 us for TurboQuantProd, 162 -> 183 us for TurboQuantMSE; the integer pipe is the scarcer one.)
template <int BITS, bool PROD>
__device__ __forceinline__ uint32_t process_chunk(const uint32_t (&v)[32], float lut_bnd, int lut_base1, float lut_ncent,
                                              float cell_scale, float cell_offset, float guard, uint32_t (&w)[BITS + 1],
                                              uint32_t (&rhi)[16], uint32_t (&rlo)[16], float& rs) {
    // Elements go through the steps in groups of kGroup, step by step, so that the shuffles of a group
    // are in flight together instead of one element's chain after the other.
    constexpr int kGroup = 8;
    uint32_t nearmask = 0;  // bit e: element e lies inside the guard band of its boundary
#pragma unroll
    for (int k = 0; k <= BITS; ++k) w[k] = 0;
#pragma unroll
    for (int g = 0; g < 32; g += kGroup) {
        int cell[kGroup];
        float bnd[kGroup];
        int base1[kGroup];
        uint32_t code[kGroup];
#pragma unroll
        for (int t = 0; t < kGroup; ++t) {
            const float u = fma_sat(__uint_as_float(v[g + t]), cell_scale, cell_offset);
            cell[t] = __float_as_int(fma_rm(u, kCellMul, 8388608.f));
        }
#pragma unroll
        for (int t = 0; t < kGroup; ++t) {
            bnd[t] = __shfl_sync(0xffffffffu, lut_bnd, cell[t]);
            base1[t] = __shfl_sync(0xffffffffu, lut_base1, cell[t]);
        }
        float dlt[kGroup];
        float nearest = 3.0e38f;   // smallest |boundary - value| of the group
#pragma unroll
        for (int t = 0; t < kGroup; ++t) {
            const int e = g + t;
            // boundary - value is negative exactly when the value lies above the boundary: its sign bit is the step from
            // "boundaries below the cell" to the code (a value equal to the boundary is inside the guard band)
            dlt[t] = bnd[t] - __uint_as_float(v[e]);
            code[t] = (uint32_t)base1[t] + (__float_as_uint(dlt[t]) >> 31);
            const int bit = e * BITS, wi = bit >> 5, sh = bit & 31;
            w[wi] += code[t] << sh;
            if (sh + BITS > 32) w[wi + 1] += code[t] >> (32 - sh);
        }
#pragma unroll
        for (int t = 0; t < kGroup; t += 2) nearest = min3_abs(nearest, dlt[t], dlt[t + 1]);
        if (nearest < guard) {   // about one group in five thousand
#pragma unroll
            for (int t = 0; t < kGroup; ++t)
                if (fabsf(dlt[t]) < guard) nearmask |= 1u << (g + t);
        }
        if (PROD) {
            float r[kGroup];
#pragma unroll
            for (int t = 0; t < kGroup; ++t) {
                const float ncent = __shfl_sync(0xffffffffu, lut_ncent, (int)code[t]);
                r[t] = fmaf(__uint_as_float(v[g + t]), kScaleRho, ncent);  // 2^10 * (value - centroid)
            }
            // (packed fp32x2 arithmetic here made the kernel slower: the pairs have to be moved into adjacent registers)
#pragma unroll
            for (int t = 0; t < kGroup; t += 2) {
                rs = fmaf(r[t], r[t], rs);
                rs = fmaf(r[t + 1], r[t + 1], rs);
                const __half2 h = __floats2half2_rn(r[t], r[t + 1]);
                const float2 hf = __half22float2(h);
                rhi[(g + t) >> 1] = *reinterpret_cast<const uint32_t*>(&h);
                rlo[(g + t) >> 1] = pack_half2(r[t] - hf.x, r[t + 1] - hf.y);
            }
        }
    }
    return nearmask;
}

// Whole warp: every lane appends one (row, coordinate) entry per bit of its mask.  Called after the
// accumulator has been handed back, so it never delays the tensor pipe.
__device__ __noinline__ void pend_codes(const TqRecheck& l, WarpPending& w, uint32_t mask, int64_t row, int first_coord,
                                        int lane) {
    for (;;) {
        const uint32_t votes = __ballot_sync(0xffffffffu, mask != 0u);
        if (votes == 0u) break;
        if (w.n_codes + __popc(votes) > kPendCap) flush_pending_codes(l, w, lane);
        if (mask != 0u) {
            const int e = __ffs(mask) - 1;
            mask &= mask - 1;
            w.codes[w.n_codes + __popc(votes & ((1u << lane) - 1u))] =
                ((unsigned long long)row << 8) | (unsigned long long)(first_coord + e);
        }
        w.n_codes += __popc(votes);
    }
}

template <int D, int BITS, bool PROD, bool UNI>
__global__ void __launch_bounds__(Threads<PROD, UNI>::kThreads, 1)
tensor_quantize_kernel(const __grid_constant__ CUtensorMap tmap_x, const TensorArgs a) {
    static_assert(D == 128 || D == 64, "this kernel is written for d = 128 and d = 64");
    // d = 64 runs in the layouts of d = 128 with the upper half of every row absent: the converter warps
    // and the epilogue warps of that half stay idle, the contractions stop after d / 16 k-blocks and cover
    // N = d output coordinates.
    constexpr int kThreads = Threads<PROD, UNI>::kThreads;
    constexpr int kFirstEpiWarp = Threads<PROD, UNI>::kFirstEpiWarp;
    constexpr int kConvParts = Threads<PROD, UNI>::kConvWarps / 4;   // converter threads per row
    constexpr int kXs = kW / kConvParts;                        // values a converter thread handles (64 or 32)
    constexpr int kActiveParts = D / kXs;                       // parts that have data (d = 64: half of them)
    using L = Smem<D, PROD, UNI>;
    constexpr int kEpiChunks = UNI ? 1 : 2;                     // 32-column chunks a thread owns in the first epilogue
    constexpr int kEpiParts = D / (32 * kEpiChunks);            // first-epilogue threads per row that have data
    constexpr int kSignChunks = kXs / 32;                       // chunks a thread owns in the sign epilogue
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t smem_base = smem_u32(smem);

    float* ssq_all = reinterpret_cast<float*>(smem + L::off_misc);                      // [2 tiles][4 parts][128]
    unsigned char* force = smem + L::off_misc + 8 * kTileRows * 4;                      // [4][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::off_misc + 8 * kTileRows * 4 + 4 * kTileRows);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
    float* rs_part = reinterpret_cast<float*>(smem + L::off_misc + L::kMiscBytes - L::kPendBytes - L::kRsBytes - kCells * 16);  // [kRsSlots][kRsParts][128]
    float2* cell_lut = reinterpret_cast<float2*>(smem + L::off_misc + L::kMiscBytes - L::kPendBytes - kCells * 16);  // [32]
    unsigned char* pend_base = smem + L::off_misc + L::kMiscBytes - L::kPendBytes;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    TQ_PROF_CODE(const long long prof_t0 = clock64(); long long prof_acc[21] = {0};)   // per-thread sums, written out once at the end

    // ---- one-time set-up ------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; ++i) { mbar_init(BAR(BAR_FULL + i), 1); mbar_init(BAR(BAR_EMPTY + i), 4); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(BAR_A_FULL + i), 4 * kActiveParts);              // the converter warps that have data
            mbar_init(BAR(BAR_A_EMPTY + i), PROD ? 4 * kActiveParts : 1);  // Prod: freed by the sign epilogue
            mbar_init(BAR(BAR_ACC_FULL + i), 1);
            mbar_init(BAR(BAR_ACC_EMPTY + i), PROD ? 1 : 4 * kEpiParts);   // Prod: freed when MMA 2 has read rho
            mbar_init(BAR(BAR_RHO_FULL + i), 4 * kEpiParts);
        }
        mbar_init(BAR(BAR_ACC2_FULL), 1);
        mbar_init(BAR(BAR_ACC2_FULL + 1), 1);
        abort_flag[0] = 0;
        abort_flag[1] = a.wait_kcycles;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < kCells) cell_lut[threadIdx.x] = a.cell_lut[threadIdx.x];
    {   // operand matrices: global -> smem, once per CTA
        const uint4* src = reinterpret_cast<const uint4*>(a.bmat);
        uint4* dst = reinterpret_cast<uint4*>(smem + L::off_b);
        for (int i = threadIdx.x; i < L::kNumB * L::kBBytes / 16; i += kThreads) dst[i] = __ldg(src + i);
        fence_async_smem();  // make these generic-proxy writes visible to the tensor core's reads
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    TQ_PROF_CODE(const long long prof_t1 = clock64();)

    const int64_t my_tiles = a.ntiles > (int64_t)blockIdx.x ? (a.ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);
    constexpr int kABlock = kW / 2;  // TMEM columns of one fp16 A block (two halves per column)
    // TMEM column map
    auto A_COL = [&](int b) { return (uint32_t)(b * 2 * kABlock); };
    // TMEM: two tile buffers, each an A block (x split; for Prod later the second accumulator) and an
    // accumulator block (for Prod later rho, split and stored in place chunk by chunk)
    auto ACC_COL = [&](int b) { return (uint32_t)(4 * kABlock + b * kW); };

    if (warp == 0) {
        // ---- TMA producer ----------------------------------------------------------------------
        if (lane == 0) {
            int64_t g = 0;
            for (int64_t i = 0; i < my_tiles; ++i) {
                const int64_t tile = blockIdx.x + i * gridDim.x;
                bool ok = true;
                for (int bx = 0; bx < L::kBoxesPerTile; ++bx, ++g) {
                    const int slot = (int)(g % L::kRingBoxes);
                    const uint32_t par = (uint32_t)((g / L::kRingBoxes) & 1);
                    if (!mbar_wait(BAR(BAR_EMPTY + slot), par ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(BAR(BAR_FULL + slot), kBoxBytes);
                    tma_load_box(smem_base + L::off_ring + slot * kBoxBytes, &tmap_x, bx * 32, (int)(tile * kTileRows),
                                 BAR(BAR_FULL + slot));
                }
                if (!ok) break;
            }
            if (*abort_flag) {
                // copies armed above may still be on their way into this block's shared memory
                for (int64_t gg = g > L::kRingBoxes ? g - L::kRingBoxes : 0; gg < g; ++gg)
                    mbar_drain(BAR(BAR_FULL + (int)(gg % L::kRingBoxes)), (uint32_t)((gg / L::kRingBoxes) & 1));
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ------------------------------------------------------------------------
        // The whole warp walks the loop and waits; one elected lane issues.  Everything an instruction takes
        // (tensor-memory addresses, descriptors) is computed from warp-uniform values, so it sits in uniform
        // registers and an issue costs a few cycles; issued from a single lane of a diverged warp the same
        // instructions cost about 64 cycles each, more when the other warps of the scheduler are busy.
        {
            const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
            const uint32_t sbo = (kW / 8) * 128, lbo = 128;
            const uint32_t b_rhi = smem_base + L::off_b, b_rlo = b_rhi + L::kBBytes;
            const uint32_t b_mhi = b_rlo + L::kBBytes, b_mlo = b_mhi + L::kBBytes;
            // descriptors of k-block 0; the start-address field counts 16-byte units, so k-block kb
            // (two core matrices further) is the same descriptor + kb * 2 * lbo / 16
            const uint64_t d_rhi = make_smem_desc(b_rhi, lbo, sbo), d_rlo = make_smem_desc(b_rlo, lbo, sbo);
            const uint64_t d_mhi = make_smem_desc(b_mhi, lbo, sbo), d_mlo = make_smem_desc(b_mlo, lbo, sbo);
            (void)d_mhi; (void)d_mlo; (void)b_mlo;
            // Prod runs one tile ahead with the first contraction: MMA1(i), then MMA2(i-1), so that the
            // residual epilogue of a tile overlaps tensor work of its neighbour.
            const int64_t iters = PROD ? my_tiles + 1 : my_tiles;
            for (int64_t i = 0; i < iters; ++i) {
                TQ_PROF_CODE(const bool pr = a.prof && blockIdx.x == 0 && lane == 0;)
                if (i < my_tiles) {
                    const int b = (int)(i & 1);
                    const uint32_t par2 = (uint32_t)((i >> 1) & 1);
                    TQ_PROF_CODE(long long c0 = clock64();)
                    if (!warp_wait(BAR(BAR_A_FULL + b), par2, abort_flag)) break;
                    TQ_PROF_CODE(long long c1 = clock64();)
                    if (!warp_wait(BAR(BAR_ACC_EMPTY + b), par2 ^ 1u, abort_flag)) break;
                    tc_fence_after();
                    TQ_PROF_CODE(long long c2 = clock64(); if (pr) { prof_acc[8] += c1 - c0; prof_acc[9] += c2 - c1; })
                    const uint32_t acc = tm + ACC_COL(b);
                    const uint32_t a_hi = tm + A_COL(b), a_lo = a_hi + kABlock;
                    if (elect_one()) {
                        mma_ts_first(acc, a_hi, d_rhi, kIdesc);
                        mma_ts_acc(acc, a_hi, d_rlo, kIdesc);
                        mma_ts_acc(acc, a_lo, d_rhi, kIdesc);
#pragma unroll 1
                        for (int kb = 1; kb < D / 16; ++kb) {
                            const uint64_t dh = d_rhi + (uint64_t)(kb * 2 * lbo >> 4);
                            const uint64_t dl = d_rlo + (uint64_t)(kb * 2 * lbo >> 4);
                            mma_ts_acc(acc, a_hi + kb * 8, dh, kIdesc);
                            mma_ts_acc(acc, a_hi + kb * 8, dl, kIdesc);
                            mma_ts_acc(acc, a_lo + kb * 8, dh, kIdesc);
                        }
                        mma_commit(BAR(BAR_ACC_FULL + b));
                        if (!PROD) mma_commit(BAR(BAR_A_EMPTY + b));
                    }
                    __syncwarp();
                    TQ_PROF_CODE(if (pr) prof_acc[10] += clock64() - c2;)
                }
                if (PROD && i >= 1) {
                    const int64_t j = i - 1;
                    const int b = (int)(j & 1);
                    const uint32_t par2 = (uint32_t)((j >> 1) & 1);
                    TQ_PROF_CODE(long long c0 = clock64();)
                    if (!warp_wait(BAR(BAR_RHO_FULL + b), par2, abort_flag)) break;
                    tc_fence_after();
                    TQ_PROF_CODE(long long c1 = clock64(); if (pr) prof_acc[11] += c1 - c0;)
                    // The second accumulator goes to the A block of the OTHER buffer: MMA 1 of tile j + 1, issued
                    // above, was its last reader, and using it (rather than this tile's own A block) lets the
                    // converters refill a block one tile earlier.  The last tile has no successor whose
                    // converter waited for the previous sign epilogue to leave that block, so wait here.
                    if (i == my_tiles && j >= 1 &&
                        !warp_wait(BAR(BAR_A_EMPTY + (b ^ 1)), (uint32_t)((((j + 1) >> 1) & 1) ^ 1), abort_flag))
                        break;
                    const uint32_t acc2 = tm + A_COL(b ^ 1);
                    const uint32_t rho = tm + ACC_COL(b);     // rho hi / lo pairs, 16 + 16 columns per 32 coordinates
                    if (elect_one()) {
                        mma_ts_first(acc2, rho, d_mhi, kIdesc);
                        mma_ts_acc(acc2, rho, d_mlo, kIdesc);
                        mma_ts_acc(acc2, rho + 16, d_mhi, kIdesc);
#pragma unroll 1
                        for (int kb = 1; kb < D / 16; ++kb) {
                            const uint64_t dh = d_mhi + (uint64_t)(kb * 2 * lbo >> 4);
                            const uint64_t dl = d_mlo + (uint64_t)(kb * 2 * lbo >> 4);
                            const uint32_t r_hi = rho + (kb >> 1) * 32 + (kb & 1) * 8, r_lo = r_hi + 16;
                            mma_ts_acc(acc2, r_hi, dh, kIdesc);
                            mma_ts_acc(acc2, r_hi, dl, kIdesc);
                            mma_ts_acc(acc2, r_lo, dh, kIdesc);
                        }
                        mma_commit(BAR(BAR_ACC2_FULL + b));
                        mma_commit(BAR(BAR_ACC_EMPTY + b));         // rho has been read: the accumulator block is free
                    }
                    __syncwarp();
                    TQ_PROF_CODE(if (pr) prof_acc[12] += clock64() - c1;)
                }
            }
        }
    } else {
        // ---- workers ------------------------------------------------------------------------------
        // Roles of this warp: UNI: every role, on the 32 columns [32 * half, 32 * half + 32) of its rows; otherwise a
        // converter warp (which also runs the sign epilogue of TurboQuantProd) or a first-epilogue warp.
        const bool conv_role = UNI || warp < kFirstEpiWarp;
        const bool epi_role = UNI || warp >= kFirstEpiWarp;
        const int cw = warp - kFirstConvWarp;      // 0 .. workers-1
        const int half = cw >> 2;                  // converter: which kXs floats of the row
        const int quarter = warp & 3;              // TMEM lane quarter this warp may touch
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        constexpr int kCodeWords = D * BITS / 32;  // words per packed row
        const int colgroup = UNI ? half : (warp - kFirstEpiWarp) >> 2;   // first epilogue: which kEpiChunks chunks of the row
        const int chunk0 = colgroup * kEpiChunks;
        const bool conv_active = conv_role && half < kActiveParts;      // d = 64: the warps of the absent columns idle
        const bool epi_active = epi_role && colgroup < kEpiParts;
        // lookup tables held in the lanes of the warp: per cell (boundary, boundaries below), per code (- centroid * 2^10)
        const float lut_bnd = cell_lut[lane].x;
        const int lut_base1 = __float_as_int(cell_lut[lane].y);   // boundaries below the cell = code of a value below its boundary
        const float lut_ncent = a.code_ncent[lane];
        WarpPending pend;
        pend.codes = reinterpret_cast<unsigned long long*>(pend_base) + cw * kPendCap;
        pend.rows = reinterpret_cast<unsigned int*>(pend_base + L::kPendWarps * kPendCap * 8) + cw * kPendCap;
        pend.n_codes = 0;
        pend.n_rows = 0;
        int64_t g_base = 0;

        // -- sign epilogue of tile j (TurboQuantProd): second accumulator -> sign bits, residual norm, rows for the exact
        // stage.  The second accumulator of tile j sits in the A block that the conversion of tile j + 3 refills, so
        // "sign epilogue of tile i - 3, then conversion of tile i" is the order the data allows anyway.
        auto sign_epilogue = [&](int64_t j) {
            const int sc0 = half * kSignChunks;
            const int64_t tile = blockIdx.x + j * gridDim.x;
            const int b = (int)(j & 1);
            const uint32_t par2 = (uint32_t)((j >> 1) & 1);
            const int64_t grow = tile * kTileRows + row;
            TQ_PROF_CODE(const bool pr = a.prof && blockIdx.x == 0 && threadIdx.x == kFirstConvWarp * 32; long long c0 = clock64(), c1;)
            bool redo_row = sc0 == 0 && force[(j & 3) * kTileRows + row] != 0;
            const bool live = mbar_wait(BAR(BAR_ACC2_FULL + b), par2, abort_flag) && grow < a.n;   // no stores after a give-up
            tc_fence_after();
            TQ_PROF_CODE(c1 = clock64(); if (pr) prof_acc[18] += c1 - c0;)
            const uint32_t acc2 = tmem + lane_addr + A_COL(b ^ 1);
            if (sc0 == 0 && live) {   // rs is in 2^10 units
                const float* rp = rs_part + (int)(j % L::kRsSlots) * L::kRsParts * kTileRows + row;
                float rs_all = rp[0];
#pragma unroll
                for (int pt = 1; pt < kEpiParts; ++pt) rs_all += rp[pt * kTileRows];
                a.rnorms[grow] = sqrtf(rs_all) * kScaleRho;
            }
            uint32_t va[32];
            uint32_t sw0 = 0, sw1 = 0;
#pragma unroll 1
            for (int ch = 0; ch < kSignChunks; ++ch) {
                TQ_PROF_CODE(const long long l0 = clock64();)
                tmem_ld32(acc2 + (sc0 + ch) * 32, va);
                tmem_wait_ld();
                TQ_PROF_CODE(if (pr) prof_acc[15] += clock64() - l0;)
                // Word layout: coordinate e of the chunk sits at bit (e >> 1) + 16 * (e & 1), bit = 1 for a non-negative
                // projection (-0.0 counts as negative here; such a row is inside the guard band and recomputed anyway).
                // One funnel shift per coordinate pushes its sign bit into a chain: four chains of eight (even / odd
                // coordinates, lower / upper half), filled from the highest coordinate down, inverted at the end.
                uint32_t wd[4] = {0u, 0u, 0u, 0u};
                float am[4] = {3.0e38f, 3.0e38f, 3.0e38f, 3.0e38f};
#pragma unroll
                for (int i = 7; i >= 0; --i) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int e = (c >> 1) * 16 + 2 * i + (c & 1);     // chain c: parity c & 1, half c >> 1
                        wd[c] = __funnelshift_l(va[e], wd[c], 1);          // (chain << 1) | sign bit
                    }
                }
#pragma unroll
                for (int e = 0; e < 32; e += 8) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        am[c] = min3_abs(am[c], __uint_as_float(va[e + 2 * c]), __uint_as_float(va[e + 2 * c + 1]));
                }
                // chains 0 / 1: even / odd coordinates 0..15 -> bits 0..7 / 16..23; chains 2 / 3: coordinates 16..31 -> 8..15 / 24..31
                const uint32_t word = ~((wd[0] | (wd[2] << 8)) | ((wd[1] | (wd[3] << 8)) << 16));
                const float amin = fminf(fminf(am[0], am[1]), fminf(am[2], am[3]));
                if (ch == 0) sw0 = word; else sw1 = word;
                redo_row = redo_row || (amin < a.sign_guard);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(BAR_A_EMPTY + (b ^ 1)));  // that A block may be refilled
            if (live) {
                if (kSignChunks == 2) *reinterpret_cast<uint2*>(a.signs + grow * (D / 32) + sc0) = make_uint2(sw0, sw1);
                else a.signs[grow * (D / 32) + sc0] = sw0;
            }
            pend_rows(a.lists, pend, redo_row && live, grow, lane);
            TQ_PROF_CODE(if (pr) prof_acc[19] += clock64() - c1;)
        };

        // -- conversion of tile i: fp32 rows -> unit length, fp16 hi/lo, into tensor memory
        auto convert = [&](int64_t i) {
            const int64_t tile = blockIdx.x + i * gridDim.x;
            const int b = (int)(i & 1);
            const uint32_t par2 = (uint32_t)((i >> 1) & 1);
            float x[kXs];
            bool fail = false;
            TQ_PROF_CODE(const bool pr = a.prof && blockIdx.x == 0 && threadIdx.x == kFirstConvWarp * 32; long long c0 = clock64(), c1;)
#pragma unroll
            for (int bb = 0; bb < kXs / 32; ++bb) {
                const int64_t g = g_base + half * (kXs / 32) + bb;
                const int slot = (int)(g % L::kRingBoxes);
                const uint32_t par = (uint32_t)((g / L::kRingBoxes) & 1);
                TQ_PROF_CODE(long long cw0 = clock64();)
                if (!fail && !mbar_wait(BAR(BAR_FULL + slot), par, abort_flag)) fail = true;
                TQ_PROF_CODE(if (pr) prof_acc[6] += clock64() - cw0;)
                const unsigned char* box = smem + L::off_ring + slot * kBoxBytes + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 v = fail ? make_float4(0.f, 0.f, 0.f, 0.f)
                                          : lds_once_f4(box + ((c ^ (row & 7)) << 4));
                    x[bb * 32 + c * 4 + 0] = v.x;
                    x[bb * 32 + c * 4 + 1] = v.y;
                    x[bb * 32 + c * 4 + 2] = v.z;
                    x[bb * 32 + c * 4 + 3] = v.w;
                }
                __threadfence_block();   // every lane's loads from the stage are performed before the stage is released
                __syncwarp();
                if (lane == 0 && !fail) mbar_arrive(BAR(BAR_EMPTY + slot));
            }
            // 32 values per thread: two values per instruction (fma / mul / add .f32x2), 3 % faster; 64 values per
            // thread: scalar, the packed form is 7 % slower there (register pairs)
            constexpr bool kPacked = kXs == 32;
            float ss;
            if (kPacked) {
                float2 s2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                for (int k = 0; k < kXs; k += 2) {
                    const float2 xx = make_float2(x[k], x[k + 1]);
                    s2[(k >> 1) & 1] = __ffma2_rn(xx, xx, s2[(k >> 1) & 1]);
                }
                ss = (s2[0].x + s2[0].y) + (s2[1].x + s2[1].y);
            } else {
                float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int k = 0; k < kXs; ++k) s4[k & 3] = fmaf(x[k], x[k], s4[k & 3]);
                ss = (s4[0] + s4[1]) + (s4[2] + s4[3]);
            }
            // partial sums of a tile go to the buffer of its parity: a fast warp writes the next tile's sums
            // before the barrier of that tile, while a slow partner may still be reading this tile's
            float* ssq = ssq_all + b * 4 * kTileRows;
            ssq[half * kTileRows + row] = ss;
            TQ_PROF_CODE(c1 = clock64(); if (pr) prof_acc[0] += c1 - c0;)
            if (kActiveParts > 1) bar_sync(1 + quarter, 32 * kActiveParts);  // the warps that share these 32 rows
            else __syncwarp();
            TQ_PROF_CODE(c0 = clock64(); if (pr) prof_acc[1] += c0 - c1;)
            float tot = ssq[row];
#pragma unroll
            for (int pt = 1; pt < kActiveParts; ++pt) tot += ssq[pt * kTileRows + row];
            const float nrm = sqrtf(tot);
            const bool ok = nrm > 0.f;
            // rows the tensor-core pass cannot represent go to the exact kernel: overflowed or
            // denormal-range norms
            const bool odd = !(tot < 3.0e38f) || (ok && tot < 1.0e-30f);
            // scale 0 for rows that go to the exact kernel anyway (zero, overflowed or denormal-range norms): their
            // products are 0, or NaN for rows that hold Inf / NaN, which stay in their own accumulator rows
            const float sc = (ok && !odd) ? kScaleA / nrm : 0.f;
            if (half == 0) {
                const int64_t grow = tile * kTileRows + row;
                if (grow < a.n && !fail) a.norms[grow] = nrm;
                force[(i & 3) * kTileRows + row] = odd ? 1 : 0;
            }
            if (!mbar_wait(BAR(BAR_A_EMPTY + b), par2 ^ 1u, abort_flag)) fail = true;
            tc_fence_after();
            TQ_PROF_CODE(c1 = clock64(); if (pr) prof_acc[2] += c1 - c0;)
            const uint32_t a_hi = tmem + lane_addr + A_COL(b) + half * (kXs / 2);
#pragma unroll
            for (int s = 0; s < kXs / 32; ++s) {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int p = 0; p < 16; ++p) {
                    float l0, l1;
                    __half2 h;
                    if (kPacked) {
                        const float2 u = __fmul2_rn(make_float2(x[s * 32 + 2 * p], x[s * 32 + 2 * p + 1]), make_float2(sc, sc));
                        h = __floats2half2_rn(u.x, u.y);
                        const float2 hf = __half22float2(h);
                        const float2 l = __fadd2_rn(u, make_float2(-hf.x, -hf.y));
                        l0 = l.x; l1 = l.y;
                    } else {
                        const float u0 = x[s * 32 + 2 * p] * sc;
                        const float u1 = x[s * 32 + 2 * p + 1] * sc;
                        h = __floats2half2_rn(u0, u1);
                        const float2 hf = __half22float2(h);
                        l0 = u0 - hf.x; l1 = u1 - hf.y;
                    }
                    hi[p] = *reinterpret_cast<const uint32_t*>(&h);
                    lo[p] = pack_half2(l0, l1);
                }
                tmem_st16(a_hi + s * 16, hi);
                tmem_st16(a_hi + kABlock + s * 16, lo);
            }
            TQ_PROF_CODE(c0 = clock64(); if (pr) prof_acc[3] += c0 - c1;)
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(BAR_A_FULL + b));
            TQ_PROF_CODE(if (pr) { prof_acc[4] += clock64() - c0; prof_acc[5] += 1; })
            g_base += L::kBoxesPerTile;
        };

        // -- first-accumulator epilogue of tile i: codes (+ rho for TurboQuantProd)
        auto epilogue1 = [&](int64_t i) {
            const int64_t tile = blockIdx.x + i * gridDim.x;
            const int b = (int)(i & 1);
            const uint32_t par2 = (uint32_t)((i >> 1) & 1);
            const int64_t grow = tile * kTileRows + row;
            const bool live_row = grow < a.n;
            TQ_PROF_CODE(const bool pr = a.prof && blockIdx.x == 0 && threadIdx.x == (UNI ? kFirstConvWarp : kFirstEpiWarp) * 32; long long c0 = clock64(), c1;)
            const bool got = mbar_wait(BAR(BAR_ACC_FULL + b), par2, abort_flag);   // false: some role gave up, the
            const bool live = live_row && got;                                      // accumulator is not to be trusted
            tc_fence_after();
            TQ_PROF_CODE(c1 = clock64(); if (pr) prof_acc[16] += c1 - c0;)
            const bool redo_row = force[(i & 3) * kTileRows + row] != 0;  // whole row to the exact stage
            float rs = 0.f;
            const uint32_t acc = tmem + lane_addr + ACC_COL(b);
            uint32_t nm[kEpiChunks];
            auto store_codes = [&](int ch, const uint32_t (&w)[BITS + 1]) {
                if (live) {  // this chunk's packed codes: BITS words at a BITS*4-byte aligned offset of the row
                    uint32_t* dst = a.codes + grow * kCodeWords + (chunk0 + ch) * BITS;
                    if (BITS == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                    else if (BITS == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
                    else {
#pragma unroll
                        for (int k = 0; k < BITS; ++k) dst[k] = w[k];
                    }
                }
            };
            if (PROD) {
                // a real loop over the chunks: half the code of the unrolled form, which matters for the
                // instruction cache more than the loop overhead does
                uint32_t nm0 = 0, nm1 = 0;
#pragma unroll 1
                for (int ch = 0; ch < kEpiChunks; ++ch) {
                    uint32_t va[32];
                    TQ_PROF_CODE(const long long l0 = clock64();)
                    tmem_ld32(acc + (chunk0 + ch) * 32, va);
                    tmem_wait_ld();
                    TQ_PROF_CODE(if (pr) prof_acc[13] += clock64() - l0;)
                    uint32_t w[BITS + 1], rhi[16], rlo[16];
                    const uint32_t m = process_chunk<BITS, PROD>(va, lut_bnd, lut_base1, lut_ncent, a.cell_scale, a.cell_offset,
                                                                 a.code_guard, w, rhi, rlo, rs);
                    if (ch == 0) nm0 = m; else nm1 = m;
                    store_codes(ch, w);
                    // rho replaces the chunk it was computed from: 16 columns of hi pairs, 16 of lo pairs
                    tmem_st16(acc + (chunk0 + ch) * 32, rhi);
                    tmem_st16(acc + (chunk0 + ch) * 32 + 16, rlo);
                }
                nm[0] = nm0;
                nm[kEpiChunks - 1] = kEpiChunks == 1 ? nm0 : nm1;
            } else {
                uint32_t va[32], vb[32];
                tmem_ld32(acc + chunk0 * 32, va);
                tmem_wait_ld();
#pragma unroll
                for (int ch = 0; ch < kEpiChunks; ++ch) {
                    // fetch the next chunk while this one is processed
                    if (ch + 1 < kEpiChunks) {
                        if (ch & 1) tmem_ld32(acc + (chunk0 + ch + 1) * 32, va); else tmem_ld32(acc + (chunk0 + ch + 1) * 32, vb);
                    }
                    uint32_t w[BITS + 1], rhi[16], rlo[16];
                    nm[ch] = (ch & 1)
                        ? process_chunk<BITS, PROD>(vb, lut_bnd, lut_base1, lut_ncent, a.cell_scale, a.cell_offset, a.code_guard, w, rhi, rlo, rs)
                        : process_chunk<BITS, PROD>(va, lut_bnd, lut_base1, lut_ncent, a.cell_scale, a.cell_offset, a.code_guard, w, rhi, rlo, rs);
                    store_codes(ch, w);
                    if (ch + 1 < kEpiChunks) tmem_wait_ld();
                }
            }
            if (PROD) {
                TQ_PROF_CODE(const long long l0 = clock64();)
                tmem_wait_st();
                TQ_PROF_CODE(if (pr) prof_acc[14] += clock64() - l0;)
                // this thread's share of |rho|^2; summed in the sign epilogue of the same tile, which every worker reaches
                // only after all of them have arrived on RHO_FULL below.  A slot is written again kRsSlots tiles later.
                // !UNI, four slots: the warp of the other half may run ahead of this one (it needs MMA 1 of a later tile,
                // not this warp's progress), but its first epilogue of tile i + 4 cannot start before every warp has
                // finished the first epilogue of tile i + 2, which follows the sign epilogue of tile i.  UNI, three slots:
                // the first epilogue of tile i + 3 follows the conversion of tile i + 4, which waits for the sign epilogue
                // of tile i + 1 of every worker, and each worker runs that one after its sign epilogue of tile i.
                rs_part[((int)(i % L::kRsSlots) * L::kRsParts + colgroup) * kTileRows + row] = rs;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(PROD ? BAR_RHO_FULL + b : BAR_ACC_EMPTY + b));
            // second-stage work is recorded after the accumulator went back to the tensor pipe
            uint32_t any_nm = 0;
#pragma unroll
            for (int ch = 0; ch < kEpiChunks; ++ch) {
                if (!live || redo_row) nm[ch] = 0;
                any_nm |= nm[ch];
            }
            if (__any_sync(0xffffffffu, any_nm != 0u)) {
#pragma unroll
                for (int ch = 0; ch < kEpiChunks; ++ch) pend_codes(a.lists, pend, nm[ch], grow, (chunk0 + ch) * 32, lane);
            }
            if (!PROD) pend_rows(a.lists, pend, redo_row && live && chunk0 == 0, grow, lane);
            TQ_PROF_CODE(if (pr) prof_acc[17] += clock64() - c1;)
        };

        if (UNI) {
            // Per iteration: sign epilogue of tile it - 3, conversion of tile it, first epilogue of tile it - 1.  The tensor
            // pipe runs the first contraction of tile it during the first epilogue of tile it - 1 and the second
            // contraction of tile it - 1 during the next iteration's sign epilogue and conversion, so in steady state
            // no phase finds its barrier unfinished.
            const int64_t tiles = conv_active ? my_tiles : 0;
            const int64_t iters = tiles > 0 ? tiles + (PROD ? 3 : 1) : 0;
            for (int64_t it = 0; it < iters; ++it) {
                if (PROD) {
                    if (it >= 3) {
                        sign_epilogue(it - 3);
                    } else if (it == 2) {
                        // A block 0 carries no second accumulator before tile 2 refills it; MMA 1 of tile 0 must have read it
                        mbar_wait(BAR(BAR_ACC_FULL + 0), 0u, abort_flag);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(BAR(BAR_A_EMPTY + 0));
                    }
                }
                if (it < tiles) convert(it);
                if (it >= 1 && it - 1 < tiles) epilogue1(it - 1);
            }
        } else if (conv_role) {
            // TurboQuantProd: the converter warps also run the sign epilogue: they wait about half of every tile for a
            // free A block, while the epilogue warps are the longest chain of this variant.
            const int64_t conv_tiles = conv_active ? my_tiles : 0;
            const int64_t conv_iters = PROD ? (conv_tiles > 0 ? conv_tiles + 3 : 0) : conv_tiles;
            for (int64_t i = 0; i < conv_iters; ++i) {
                if (PROD) {
                    if (i >= 3) {
                        sign_epilogue(i - 3);
                    } else if (i == 2) {
                        mbar_wait(BAR(BAR_ACC_FULL + 0), 0u, abort_flag);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(BAR(BAR_A_EMPTY + 0));
                    }
                    if (i >= conv_tiles) continue;
                }
                convert(i);
            }
        } else {
            const int64_t epi_tiles = epi_active ? my_tiles : 0;
            for (int64_t i = 0; i < epi_tiles; ++i) epilogue1(i);
        }
        if (pend.n_codes > 0) flush_pending_codes(a.lists, pend, lane);
        if (pend.n_rows > 0) flush_pending_rows(a.lists, pend, lane);
    }

    // ---- teardown -----------------------------------------------------------------------------------
    if (*abort_flag) __nanosleep(20000);   // tensor instructions issued before the give-up may still be running
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.status, 1ull);
#ifdef TQ_PROF
    if (a.prof && blockIdx.x == 0) {
#pragma unroll
        for (int k = 0; k < 21; ++k)
            if (prof_acc[k]) atomicAdd(reinterpret_cast<unsigned long long*>(a.prof + k), (unsigned long long)prof_acc[k]);
    }
    if (a.prof && threadIdx.x == 0) {
        const long long t2 = clock64();
        atomicMax(reinterpret_cast<unsigned long long*>(a.prof + 21), (unsigned long long)(t2 - prof_t0));
        atomicMax(reinterpret_cast<unsigned long long*>(a.prof + 22), (unsigned long long)(prof_t1 - prof_t0));
        if (blockIdx.x == 0) a.prof[23] = t2 - prof_t0;
    }
#endif
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ---------------------------------------------------------------------------------------------
// d = 256 (TurboQuantMSE): the split rotation is 2 x 128 KB and cannot stay in shared memory, so it streams
// ---------------------------------------------------------------------------------------------
// A tile is 128 rows x 256 columns.  The unit rows, split into fp16 hi / lo, fill both A blocks of tensor memory
// (K half I in block I); the two accumulator blocks take the two halves J of the output columns.  The rotation is
// stored as 32 chunks of 8 KB -- chunk ((J * 2 + I) * 8 + kb) holds R_hi and R_lo for output columns [128 J, 128 J + 128)
// and input coordinates [128 I + 16 kb, + 16) as K-major 8 x 8 core matrices -- and every CTA pulls the 256 KB through a
// ring of 8 chunks once per tile (from L2), three tensor instructions per chunk.  Tensor memory is full with one tile
// (A 256 + accumulators 256 columns), so the conversion of a tile cannot overlap the contractions of its predecessor;
// the epilogue of output half 0 runs beside the contractions of half 1.  96 tensor instructions (6.1 K cycles) per tile
// stand against 6.4 K cycles of HBM time for its 148 KB.
// Warps: TMA for the rows, MMA, bulk copies of the rotation, 16 converters (64 values per thread), 8 epilogue warps.
namespace d256 {
constexpr int kD = 256;
constexpr int kBoxesPerTile = kD / 32;           // 8
constexpr int kXRing = 8;                    // one tile: a converter must not meet a slot's second use before its first
                                            // (its wait on the later parity would pass at once while the first copy is still on its way)
constexpr int kChunkBytes = 8192;                // R_hi and R_lo of one (J, I, kb): 128 x 16 halves each
constexpr int kChunksPerMatrix = 32;          // per tile: the rotation, and for TurboQuantProd 16 (R S^T) behind it
constexpr int kBRing = 8;                    // (10 chunks, which is what shared memory leaves room for, were slower: 582 against 542 us)
constexpr int kConvWarps = 16, kEpiWarps = 8;
constexpr int kFirstConv = 3, kFirstEpi = kFirstConv + kConvWarps;
constexpr int kThreads = (3 + kConvWarps + kEpiWarps) * 32;      // 864
constexpr int off_b = 0;
constexpr int off_x = off_b + kBRing * kChunkBytes;              // 128 KB
constexpr int off_ssq = off_x + kXRing * kBoxBytes;              // [2 tiles][4 parts][128] floats
constexpr int off_force = off_ssq + 2 * 4 * kTileRows * 4;       // [4][128] bytes
constexpr int off_bars = off_force + 4 * kTileRows;
enum { X_FULL = 0, X_EMPTY = 8, B_FULL = 16, B_EMPTY = 24, A_FULL = 32, A_EMPTY = 33, ACC_FULL = 34, ACC_EMPTY = 36, RHO_FULL = 38, ACC2_FULL = 40, N_BARS = 42 };
constexpr int off_lut = off_bars + 512;                          // barriers, tensor-memory slot, give-up flag; then the cell table
constexpr int off_rs = off_lut + 512;                            // |rho|^2 partial sums [4 column groups][128] (TurboQuantProd)
constexpr int off_pend = off_rs + 4 * kTileRows * 4;
constexpr int kPendBytes = kEpiWarps * kPendCap * (8 + 4) + kConvWarps * kPendCap * 4;   // epilogue warps: both lists; converters: rows
constexpr int total = off_pend + kPendBytes + 1024;
static_assert(total <= 227 * 1024, "shared memory plan");
}  // namespace d256

template <int BITS, bool PROD>
__global__ void __launch_bounds__(d256::kThreads, 1)
tensor_quantize256_kernel(const __grid_constant__ CUtensorMap tmap_x, const TensorArgs a) {
    using namespace d256;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t smem_base = smem_u32(smem);
    float* ssq_all = reinterpret_cast<float*>(smem + off_ssq);
    unsigned char* force = smem + off_force;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off_bars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float2* cell_lut = reinterpret_cast<float2*>(smem + off_lut);
    float* rs_part = reinterpret_cast<float*>(smem + off_rs);
    unsigned char* pend_base = smem + off_pend;
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kXRing; ++i) { mbar_init(BAR(X_FULL + i), 1); mbar_init(BAR(X_EMPTY + i), 4); }
        for (int i = 0; i < kBRing; ++i) { mbar_init(BAR(B_FULL + i), 1); mbar_init(BAR(B_EMPTY + i), 1); }
        mbar_init(BAR(A_FULL), kConvWarps);
        mbar_init(BAR(A_EMPTY), 1);
        for (int j = 0; j < 2; ++j) {
            mbar_init(BAR(ACC_FULL + j), 1);
            mbar_init(BAR(ACC_EMPTY + j), PROD ? 1 : kEpiWarps);      // Prod: freed when the second contraction has read rho
            mbar_init(BAR(RHO_FULL + j), kEpiWarps);
            mbar_init(BAR(ACC2_FULL + j), 1);
        }
        abort_flag[0] = 0;
        abort_flag[1] = a.wait_kcycles;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < kCells) cell_lut[threadIdx.x] = a.cell_lut[threadIdx.x];
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int64_t my_tiles = a.ntiles > (int64_t)blockIdx.x ? (a.ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);
    constexpr int kABlock = 64;                                  // columns of one fp16 operand block (128 values)
    auto A_COL = [&](int i) { return (uint32_t)(i * 2 * kABlock); };
    auto ACC_COL = [&](int j) { return (uint32_t)(4 * kABlock + j * 128); };

    if (warp == 0) {
        // ---- rows: TMA boxes of 32 columns x 128 rows ------------------------------------------------
        if (lane == 0) {
            int64_t g = 0;
            bool ok = true;
            for (int64_t i = 0; i < my_tiles && ok; ++i) {
                const int64_t tile = blockIdx.x + i * gridDim.x;
                for (int bx = 0; bx < kBoxesPerTile; ++bx, ++g) {
                    const int slot = (int)(g % kXRing);
                    if (!mbar_wait(BAR(X_EMPTY + slot), (uint32_t)(((g / kXRing) & 1) ^ 1), abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(BAR(X_FULL + slot), kBoxBytes);
                    tma_load_box(smem_base + off_x + slot * kBoxBytes, &tmap_x, bx * 32, (int)(tile * kTileRows), BAR(X_FULL + slot));
                }
            }
            if (*abort_flag)
                for (int64_t gg = g > kXRing ? g - kXRing : 0; gg < g; ++gg)
                    mbar_drain(BAR(X_FULL + (int)(gg % kXRing)), (uint32_t)((gg / kXRing) & 1));
        }
    } else if (warp == 2) {
        // ---- rotation: one bulk copy per chunk, the same 32 chunks for every tile ------------------------
        if (lane == 0) {
            int64_t g = 0;
            bool ok = true;
            const unsigned char* src = reinterpret_cast<const unsigned char*>(a.bmat);
            for (int64_t i = 0; i < my_tiles && ok; ++i) {
                for (int c = 0; c < (PROD ? 2 : 1) * kChunksPerMatrix; ++c, ++g) {
                    const int slot = (int)(g % kBRing);
                    if (!mbar_wait(BAR(B_EMPTY + slot), (uint32_t)(((g / kBRing) & 1) ^ 1), abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(BAR(B_FULL + slot), kChunkBytes);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(smem_base + off_b + slot * kChunkBytes), "l"(src + (size_t)c * kChunkBytes), "r"(kChunkBytes),
                                   "r"(BAR(B_FULL + slot))
                                 : "memory");
                }
            }
            if (*abort_flag)
                for (int64_t gg = g > kBRing ? g - kBRing : 0; gg < g; ++gg)
                    mbar_drain(BAR(B_FULL + (int)(gg % kBRing)), (uint32_t)((gg / kBRing) & 1));
        }
    } else if (warp == 1) {
        // ---- MMA issuer: the whole warp walks the loop, one elected lane issues -------------------------
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
        int64_t g = 0;
        bool ok = true;
        for (int64_t i = 0; i < my_tiles && ok; ++i) {
            const uint32_t par = (uint32_t)(i & 1);
            if (!warp_wait(BAR(A_FULL), par, abort_flag)) break;
            for (int j = 0; j < 2 && ok; ++j) {
                if (!warp_wait(BAR(ACC_EMPTY + j), par ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t acc = tm + ACC_COL(j);
                for (int c = 0; c < 16; ++c, ++g) {          // c = I * 8 + kb
                    const int slot = (int)(g % kBRing);
                    if (!warp_wait(BAR(B_FULL + slot), (uint32_t)((g / kBRing) & 1), abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t chunk = smem_base + off_b + slot * kChunkBytes;
                    const uint64_t d_hi = make_smem_desc(chunk, 128, 256), d_lo = make_smem_desc(chunk + kChunkBytes / 2, 128, 256);
                    const uint32_t a_hi = tm + A_COL(c >> 3) + (uint32_t)(c & 7) * 8, a_lo = a_hi + kABlock;
                    if (elect_one()) {
                        if (c == 0) mma_ts_first(acc, a_hi, d_hi, kIdesc);
                        else mma_ts_acc(acc, a_hi, d_hi, kIdesc);
                        mma_ts_acc(acc, a_hi, d_lo, kIdesc);
                        mma_ts_acc(acc, a_lo, d_hi, kIdesc);
                        mma_commit(BAR(B_EMPTY + slot));
                        if (c == 15) mma_commit(BAR(ACC_FULL + j));
                    }
                    __syncwarp();
                }
            }
            if (!ok) break;
            if (!PROD) {
                if (elect_one()) mma_commit(BAR(A_EMPTY));       // both operand blocks have been read
                __syncwarp();
                continue;
            }
            // TurboQuantProd: rho (split, in place of the accumulators: K half I in accumulator block I) times the chunks of
            // 16 (R S^T); output half J goes to operand block J, which the first contraction has finished reading.
            if (!warp_wait(BAR(RHO_FULL + 0), par, abort_flag) || !warp_wait(BAR(RHO_FULL + 1), par, abort_flag)) break;
            tc_fence_after();
            for (int j = 0; j < 2 && ok; ++j) {
                const uint32_t acc2 = tm + A_COL(j);
                for (int c = 0; c < 16; ++c, ++g) {
                    const int slot = (int)(g % kBRing);
                    if (!warp_wait(BAR(B_FULL + slot), (uint32_t)((g / kBRing) & 1), abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t chunk = smem_base + off_b + slot * kChunkBytes;
                    const uint64_t d_hi = make_smem_desc(chunk, 128, 256), d_lo = make_smem_desc(chunk + kChunkBytes / 2, 128, 256);
                    const int kb = c & 7;
                    // rho of 32 coordinates: 16 columns of hi pairs, then 16 of lo pairs
                    const uint32_t r_hi = tm + ACC_COL(c >> 3) + (uint32_t)(kb >> 1) * 32 + (uint32_t)(kb & 1) * 8, r_lo = r_hi + 16;
                    if (elect_one()) {
                        if (c == 0) mma_ts_first(acc2, r_hi, d_hi, kIdesc);
                        else mma_ts_acc(acc2, r_hi, d_hi, kIdesc);
                        mma_ts_acc(acc2, r_hi, d_lo, kIdesc);
                        mma_ts_acc(acc2, r_lo, d_hi, kIdesc);
                        mma_commit(BAR(B_EMPTY + slot));
                        if (c == 15) mma_commit(BAR(ACC2_FULL + j));
                    }
                    __syncwarp();
                }
            }
            if (!ok) break;
            if (elect_one()) { mma_commit(BAR(ACC_EMPTY + 0)); mma_commit(BAR(ACC_EMPTY + 1)); }   // rho has been read
            __syncwarp();
        }
    } else if (warp < kFirstEpi) {
        // ---- converters: one thread per quarter row (64 values, two boxes) -------------------------------
        const int cw = warp - kFirstConv;
        const int part = cw >> 2;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        WarpPending cpend;           // rows for the exact stage found by the sign epilogue
        cpend.codes = nullptr;
        cpend.rows = reinterpret_cast<unsigned int*>(pend_base + kEpiWarps * kPendCap * 12) + cw * kPendCap;
        cpend.n_codes = 0;
        cpend.n_rows = 0;
        for (int64_t i = 0; i < my_tiles; ++i) {
            const int64_t tile = blockIdx.x + i * gridDim.x;
            const uint32_t par = (uint32_t)(i & 1);
            float x[64];
            bool fail = false;
#pragma unroll
            for (int bb = 0; bb < 2; ++bb) {
                const int64_t g = i * kBoxesPerTile + part * 2 + bb;
                const int slot = (int)(g % kXRing);
                if (!fail && !mbar_wait(BAR(X_FULL + slot), (uint32_t)((g / kXRing) & 1), abort_flag)) fail = true;
                const unsigned char* box = smem + off_x + slot * kBoxBytes + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 v = fail ? make_float4(0.f, 0.f, 0.f, 0.f) : lds_once_f4(box + ((c ^ (row & 7)) << 4));
                    x[bb * 32 + c * 4 + 0] = v.x;
                    x[bb * 32 + c * 4 + 1] = v.y;
                    x[bb * 32 + c * 4 + 2] = v.z;
                    x[bb * 32 + c * 4 + 3] = v.w;
                }
                __threadfence_block();   // every lane's loads from the stage are performed before the stage is released
                __syncwarp();
                if (lane == 0 && !fail) mbar_arrive(BAR(X_EMPTY + slot));
            }
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < 64; ++k) s4[k & 3] = fmaf(x[k], x[k], s4[k & 3]);
            float* ssq = ssq_all + (int)par * 4 * kTileRows;     // by tile parity: a fast warp may write the next tile's sums early
            ssq[part * kTileRows + row] = (s4[0] + s4[1]) + (s4[2] + s4[3]);
            bar_sync(1 + quarter, 128);                           // the four warps that share these 32 rows
            const float tot = (ssq[row] + ssq[kTileRows + row]) + (ssq[2 * kTileRows + row] + ssq[3 * kTileRows + row]);
            const float nrm = sqrtf(tot);
            const bool okn = nrm > 0.f;
            const bool odd = !(tot < 3.0e38f) || (okn && tot < 1.0e-30f);   // rows for the exact kernel: overflowed or denormal-range norms
            const float sc = (okn && !odd) ? kScaleA / nrm : 0.f;
            if (part == 0) {
                const int64_t grow = tile * kTileRows + row;
                if (grow < a.n && !fail) a.norms[grow] = nrm;
                force[(i & 3) * kTileRows + row] = odd ? 1 : 0;
            }
            // TurboQuantProd: this thread itself was the last reader of its cells (sign epilogue of the previous tile, below)
            if (!PROD && !mbar_wait(BAR(A_EMPTY), par ^ 1u, abort_flag)) fail = true;
            tc_fence_after();
            const uint32_t a_hi = tmem + lane_addr + A_COL(part >> 1) + (uint32_t)(part & 1) * 32;
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int p = 0; p < 16; ++p) {
                    const float u0 = x[s * 32 + 2 * p] * sc, u1 = x[s * 32 + 2 * p + 1] * sc;
                    const __half2 h = __floats2half2_rn(u0, u1);
                    const float2 hf = __half22float2(h);
                    hi[p] = *reinterpret_cast<const uint32_t*>(&h);
                    lo[p] = pack_half2(u0 - hf.x, u1 - hf.y);
                }
                tmem_st16(a_hi + s * 16, hi);
                tmem_st16(a_hi + kABlock + s * 16, lo);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(A_FULL));
            if (PROD) {
                // ---- sign epilogue of the same tile: the second accumulator of output half J sits in operand block J.  A
                // thread reads exactly the cells it fills again for the next tile (columns [32 h, 32 h + 32) and
                // [64 + 32 h, 64 + 32 h + 32) with h = part & 1: two sign words of the row), so no other warp's
                // progress matters to it.
                const int j = part >> 1, hcol = part & 1;
                const int64_t grow = tile * kTileRows + row;
                bool redo_row = part == 0 && force[(i & 3) * kTileRows + row] != 0;
                const bool live = mbar_wait(BAR(ACC2_FULL + j), par, abort_flag) && grow < a.n;   // no stores after a give-up
                tc_fence_after();
                if (part == 0 && live) {      // |rho|^2 in 2^10 units: the four partial sums of the first epilogue
                    const float rs_all = (rs_part[row] + rs_part[kTileRows + row]) + (rs_part[2 * kTileRows + row] + rs_part[3 * kTileRows + row]);
                    a.rnorms[grow] = sqrtf(rs_all) * kScaleRho;
                }
                const uint32_t acc2 = tmem + lane_addr + A_COL(j);
                uint32_t sw[2] = {0u, 0u};
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t va[32];
                    tmem_ld32(acc2 + (hcol + 2 * ch) * 32, va);
                    tmem_wait_ld();
                    uint32_t wd[4] = {0u, 0u, 0u, 0u};
                    float am[4] = {3.0e38f, 3.0e38f, 3.0e38f, 3.0e38f};
#pragma unroll
                    for (int k = 7; k >= 0; --k) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) wd[c] = __funnelshift_l(va[(c >> 1) * 16 + 2 * k + (c & 1)], wd[c], 1);
                    }
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            am[c] = min3_abs(am[c], __uint_as_float(va[e + 2 * c]), __uint_as_float(va[e + 2 * c + 1]));
                    }
                    const uint32_t word = ~((wd[0] | (wd[2] << 8)) | ((wd[1] | (wd[3] << 8)) << 16));
                    if (ch == 0) sw[0] = word; else sw[1] = word;
                    redo_row = redo_row || (fminf(fminf(am[0], am[1]), fminf(am[2], am[3])) < a.sign_guard);
                }
                tc_fence_before();
                if (live) {
                    a.signs[grow * (kD / 32) + j * 4 + hcol] = sw[0];
                    a.signs[grow * (kD / 32) + j * 4 + 2 + hcol] = sw[1];
                }
                pend_rows(a.lists, cpend, redo_row && live, grow, lane);
            }
        }
        if (PROD && cpend.n_rows > 0) flush_pending_rows(a.lists, cpend, lane);
    } else {
        // ---- epilogue: two threads per row, 64 columns of each output half -------------------------------
        const int ew = warp - kFirstEpi;
        const int quarter = warp & 3;
        const int colgroup = ew >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        constexpr int kCodeWords = kD * BITS / 32;
        const float lut_bnd = cell_lut[lane].x;
        const int lut_base1 = __float_as_int(cell_lut[lane].y);
        const float lut_ncent = PROD ? a.code_ncent[lane] : 0.f;
        WarpPending pend;
        pend.codes = reinterpret_cast<unsigned long long*>(pend_base) + ew * kPendCap;
        pend.rows = reinterpret_cast<unsigned int*>(pend_base + kEpiWarps * kPendCap * 8) + ew * kPendCap;
        pend.n_codes = 0;
        pend.n_rows = 0;
        for (int64_t i = 0; i < my_tiles; ++i) {
            const int64_t tile = blockIdx.x + i * gridDim.x;
            const uint32_t par = (uint32_t)(i & 1);
            const int64_t grow = tile * kTileRows + row;
#pragma unroll 1
            for (int j = 0; j < 2; ++j) {
                const bool got = mbar_wait(BAR(ACC_FULL + j), par, abort_flag);
                const bool live = got && grow < a.n;
                const bool redo_row = force[(i & 3) * kTileRows + row] != 0;   // written before this tile's A_FULL, which precedes ACC_FULL
                tc_fence_after();
                const uint32_t acc = tmem + lane_addr + ACC_COL(j);
                uint32_t nm0 = 0, nm1 = 0;
                float rs = 0.f;
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    const int chunk = colgroup * 2 + ch;                 // 32-column chunk of this output half
                    uint32_t va[32];
                    tmem_ld32(acc + chunk * 32, va);
                    tmem_wait_ld();
                    uint32_t w[BITS + 1], rhi[16], rlo[16];
                    const uint32_t m = process_chunk<BITS, PROD>(va, lut_bnd, lut_base1, lut_ncent, a.cell_scale, a.cell_offset, a.code_guard, w, rhi, rlo, rs);
                    if (ch == 0) nm0 = m; else nm1 = m;
                    if (PROD) {      // rho replaces the chunk it was computed from: 16 columns of hi pairs, 16 of lo pairs
                        tmem_st16(acc + chunk * 32, rhi);
                        tmem_st16(acc + chunk * 32 + 16, rlo);
                    }
                    if (live) {
                        uint32_t* dst = a.codes + grow * kCodeWords + (j * 4 + chunk) * BITS;
                        if (BITS == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                        else if (BITS == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
                        else {
#pragma unroll
                            for (int k = 0; k < BITS; ++k) dst[k] = w[k];
                        }
                    }
                }
                if (PROD) {
                    tmem_wait_st();
                    // this thread's share of |rho|^2; one tile is in flight per block, and the sign epilogue that reads the
                    // sums comes after the second contraction, which waits for every epilogue warp's arrival below
                    rs_part[(j * 2 + colgroup) * kTileRows + row] = rs;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(PROD ? RHO_FULL + j : ACC_EMPTY + j));
                if (!live || redo_row) { nm0 = 0; nm1 = 0; }
                if (__any_sync(0xffffffffu, (nm0 | nm1) != 0u)) {
                    pend_codes(a.lists, pend, nm0, grow, j * 128 + (colgroup * 2) * 32, lane);
                    pend_codes(a.lists, pend, nm1, grow, j * 128 + (colgroup * 2 + 1) * 32, lane);
                }
                if (!PROD && j == 0) pend_rows(a.lists, pend, redo_row && live && colgroup == 0, grow, lane);
            }
        }
        if (pend.n_codes > 0) flush_pending_codes(a.lists, pend, lane);
        if (pend.n_rows > 0) flush_pending_rows(a.lists, pend, lane);
    }

    if (*abort_flag) __nanosleep(20000);   // tensor instructions issued before the give-up may still be running
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.status, 1ull);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// fp16 bits of a float, round to nearest even (host)
uint16_t host_half_bits(float f) {
    const __half h = __float2half_rn(f);
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}
float host_half_value(uint16_t b) {
    __half h;
    memcpy(&h, &b, 2);
    return __half2float(h);
}

// Split scale*M[n][k] into hi + lo fp16 and lay both out as 8x8 core matrices, K-major.
// m is d x d; the operand is laid out kW x kW (the caller zero-fills hi / lo, so d < kW is padded with zeros)
void split_operand(const std::vector<double>& m, int d, double scale, uint16_t* hi, uint16_t* lo) {
    const size_t sbo = (size_t)(kW / 8) * 128, lbo = 128;
    for (int n = 0; n < d; ++n)
        for (int k = 0; k < d; ++k) {
            const float v = (float)(m[(size_t)n * d + k] * scale);
            const uint16_t h = host_half_bits(v);
            const uint16_t l = host_half_bits((float)((double)v - (double)host_half_value(h)));
            const size_t off = ((size_t)(n / 8) * sbo + (size_t)(k / 8) * lbo + (size_t)(n % 8) * 16 + (size_t)(k % 8) * 2) / 2;
            hi[off] = h;
            lo[off] = l;
        }
}

// d = 256: chunk ((J * 2 + I) * 8 + kb) = [hi | lo], each 128 (n) x 16 (k) halves as K-major core matrices:
// 8-row groups 256 bytes apart, the two core matrices of a group 128 bytes apart.
void split_operand_chunks(const double* m, double scale, uint16_t* out) {
    const int d = 256;
    for (int n = 0; n < d; ++n)
        for (int k = 0; k < d; ++k) {
            const float v = (float)(m[(size_t)n * d + k] * scale);      // B[n][k]
            const uint16_t h = host_half_bits(v);
            const uint16_t l = host_half_bits((float)((double)v - (double)host_half_value(h)));
            const int J = n / 128, I = k / 128, kb = (k % 128) / 16, nn = n % 128, kk = k % 16;
            const size_t chunk = (size_t)((J * 2 + I) * 8 + kb) * 8192;
            const size_t off = (size_t)(nn / 8) * 256 + (size_t)(kk / 8) * 128 + (size_t)(nn % 8) * 16 + (size_t)(kk % 8) * 2;
            out[(chunk + off) / 2] = h;
            out[(chunk + 4096 + off) / 2] = l;
        }
}

int host_cell(float v, float scale, float offset) {
    float u = fmaf(v, scale, offset);
    u = u < 0.f ? 0.f : (u > 1.f ? 1.f : u);
    if (!(u == u)) u = 0.f;
    return (int)floor((double)u * (double)kCellMul);
}

// Find a 32-cell uniform grid over the (scaled) boundaries such that every cell holds at most one
// boundary and every boundary keeps its cell within +-margin.  Returns false if none is found.
bool build_cell_lut(const float* bnd_scaled, int nb, float margin, float* scale, float* offset, float* lut_bnd,
                    int* lut_base) {
    const float bmin = bnd_scaled[0], bmax = bnd_scaled[nb - 1];
    // cells must be much wider than the margin, also when there is a single boundary
    const float span = fmaxf(bmax - bmin, 1024.f * margin);
    for (int ta = 1; ta <= 24; ++ta)
        for (int tb = 1; tb <= 24; ++tb) {
            const float lo = bmin - span * 0.013f * ta, hi = bmax + span * 0.013f * tb;
            const float sc = 1.f / (hi - lo), of = -lo * sc;
            int cells[256];
            bool ok = true;
            for (int k = 0; k < nb && ok; ++k) {
                const int c = host_cell(bnd_scaled[k], sc, of);
                if (host_cell(bnd_scaled[k] - margin, sc, of) != c || host_cell(bnd_scaled[k] + margin, sc, of) != c) ok = false;
                if (c <= 0 || c >= kCells - 1) ok = false;  // keep the end cells free of boundaries
                if (k > 0 && c == cells[k - 1]) ok = false;
                cells[k] = c;
            }
            if (!ok) continue;
            int k = 0;
            for (int c = 0; c < kCells; ++c) {
                lut_base[c] = k;
                if (k < nb && cells[k] == c) {
                    lut_bnd[c] = bnd_scaled[k];
                    ++k;
                } else {
                    lut_bnd[c] = INFINITY;
                }
            }
            *scale = sc;
            *offset = of;
            return true;
        }
    return false;
}

}  // namespace

TqEncodeTiledFn tq_encode_tiled_fn() {
    static TqEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TqEncodeTiledFn>(p);
    }
    return fn;
}

struct TensorConsts {
    void* dev = nullptr;   // one allocation: operand matrices + lookup tables
    TensorArgs args{};     // pointers into `dev` and the scalar parameters
};

bool tq_tensor_supported(int d, int bits) { return (d == 128 || d == 64) && bits >= 1 && bits <= 4; }
// The quantize kernels alone also cover d = 256, with the operand matrices streamed.
bool tq_tensor_quantize_supported(int d, int bits, bool has_projection) {
    (void)has_projection;
    return tq_tensor_supported(d, bits) || (d == 256 && bits >= 1 && bits <= 4);
}

int tq_tensor_plan_init(tq_plan* p, const float* rotation, const float* codebook, const float* projection) {
    const int d = p->dev.d, levels = p->dev.levels, nb = levels - 1;
    // boundaries exactly as the plan holds them
    std::vector<float> bnd(nb), bnd_s(nb);
    for (int k = 0; k < nb; ++k) {
        volatile float s = codebook[k] + codebook[k + 1];
        bnd[k] = 0.5f * s;
        bnd_s[k] = bnd[k] * kAccScale;
    }
    for (int k = 1; k < nb; ++k)
        if (!(bnd_s[k] > bnd_s[k - 1])) return TQ_OK;  // degenerate codebook: leave tensor_ok false
    for (int k = 0; k < nb; ++k)
        if (!(fabsf(bnd[k]) < 4.f)) return TQ_OK;
    float lut_bnd[kCells], lut_cent[kCells], cs = 0.f, co = 0.f;
    int lut_base[kCells];
    const float guard = TQ_CODE_GUARD * kAccScale;
    if (!build_cell_lut(bnd_s.data(), nb, 4.f * guard, &cs, &co, lut_bnd, lut_base)) return TQ_OK;
    float lut2[kCells * 2];
    for (int c = 0; c < kCells; ++c) {
        lut2[2 * c] = lut_bnd[c];
        memcpy(&lut2[2 * c + 1], &lut_base[c], 4);       // boundaries in lower cells = code of a value below this cell's boundary
    }
    for (int l = 0; l < kCells; ++l) lut_cent[l] = -codebook[l % levels] * kScaleA;

    const size_t dd = (size_t)kW * kW;   // operand matrices are stored padded to kW x kW
    const int nmat = projection ? 4 : 2;
    std::vector<uint16_t> mats(d == 256 ? (size_t)d * d * nmat : dd * nmat, 0);
    std::vector<double> m((size_t)d * d);
    if (d == 256) {
        for (size_t i = 0; i < (size_t)d * d; ++i) m[i] = rotation[i];  // B1[n=j][k] = R[j][k]
        split_operand_chunks(m.data(), kScaleB, mats.data());
    } else {
        for (size_t i = 0; i < (size_t)d * d; ++i) m[i] = rotation[i];  // B1[n=j][k] = R[j][k]
        split_operand(m, d, kScaleB, mats.data(), mats.data() + dd);
    }
    if (projection) {
        // B2[n=j][k] = (R S^T)[k][j] = sum_i R[k][i] S[j][i]
        for (int j = 0; j < d; ++j)
            for (int k = 0; k < d; ++k) {
                double acc = 0.0;
                for (int i = 0; i < d; ++i) acc += (double)rotation[(size_t)k * d + i] * (double)projection[(size_t)j * d + i];
                m[(size_t)j * d + k] = acc;
            }
        if (d == 256) split_operand_chunks(m.data(), kScaleM, mats.data() + (size_t)d * d * 2);   // the second 256 KB of chunks
        else split_operand(m, d, kScaleM, mats.data() + 2 * dd, mats.data() + 3 * dd);
    }
    const size_t mat_bytes = mats.size() * 2;
    const size_t total = mat_bytes + 5 * kCells * 4;
    TensorConsts* t = new TensorConsts();
    cudaError_t e = cudaMalloc(&t->dev, total);
    if (e != cudaSuccess) {
        delete t;
        return tq_fail(TQ_ERR_CUDA, "cudaMalloc(%zu) failed: %s", total, cudaGetErrorString(e));
    }
    unsigned char* base = static_cast<unsigned char*>(t->dev);
    bool ok = cudaMemcpy(base, mats.data(), mat_bytes, cudaMemcpyHostToDevice) == cudaSuccess &&
              cudaMemcpy(base + mat_bytes, lut2, sizeof(lut2), cudaMemcpyHostToDevice) == cudaSuccess &&
              cudaMemcpy(base + mat_bytes + kCells * 16, lut_cent, kCells * 4, cudaMemcpyHostToDevice) == cudaSuccess;
    if (!ok || !tq_encode_tiled_fn()) {
        cudaFree(t->dev);
        delete t;
        return tq_fail(TQ_ERR_CUDA, "upload of tensor-path constants failed");
    }
    t->args.bmat = reinterpret_cast<const __half*>(base);
    t->args.cell_lut = reinterpret_cast<const float2*>(base + mat_bytes);
    t->args.code_ncent = reinterpret_cast<const float*>(base + mat_bytes + kCells * 16);
    t->args.cell_scale = cs;
    t->args.cell_offset = co;
    t->args.code_guard = guard;
    // accumulator 2 holds 2^10 * 16 * (residual . S row)
    t->args.sign_guard = TQ_SIGN_GUARD * 1024.f * kScaleM;
    p->tensor = t;
    p->tensor_ok = true;
    return TQ_OK;
}

void tq_tensor_plan_free(tq_plan* p) {
    if (p->tensor) {
        if (p->tensor->dev) cudaFree(p->tensor->dev);
        delete p->tensor;
        p->tensor = nullptr;
    }
}

#ifndef TQ_UNI_PROD
#define TQ_UNI_PROD false
#endif
#ifndef TQ_UNI_MSE
#define TQ_UNI_MSE false
#endif
template <int D, int BITS, bool PROD>
static int launch_one(const CUtensorMap& map, const TensorArgs& args, int grid, cudaStream_t st) {
    constexpr bool UNI = PROD ? TQ_UNI_PROD : TQ_UNI_MSE;
    const int sm = Smem<D, PROD, UNI>::total;
    TQ_CUDA_TRY(cudaFuncSetAttribute(tensor_quantize_kernel<D, BITS, PROD, UNI>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm));
    tensor_quantize_kernel<D, BITS, PROD, UNI><<<grid, Threads<PROD, UNI>::kThreads, sm, st>>>(map, args); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

template <int BITS, bool PROD>
static int launch_256(const CUtensorMap& map, const TensorArgs& args, int grid, cudaStream_t st) {
    TQ_CUDA_TRY(cudaFuncSetAttribute(tensor_quantize256_kernel<BITS, PROD>, cudaFuncAttributeMaxDynamicSharedMemorySize, d256::total));
    tensor_quantize256_kernel<BITS, PROD><<<grid, d256::kThreads, d256::total, st>>>(map, args); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

int tq_launch_tensor_quantize(const tq_plan* p, bool prod, const float* x, int64_t n, uint32_t* codes,
                              uint32_t* signs, float* rnorms, float* norms, const TqRecheck* lists, cudaStream_t st) {
    TqRange range("tq.quantize.tensor_core");
    if (!p->tensor) return tq_fail(TQ_ERR_UNSUPPORTED, "no tensor-core kernel for this plan");
    const int d = p->dev.d;
    if (n > (int64_t)0x7fffff00) return tq_fail(TQ_ERR_UNSUPPORTED, "n above 2^31 rows per call");
    TensorArgs args = p->tensor->args;
    args.n = n;
    args.ntiles = (n + kTileRows - 1) / kTileRows;
    args.codes = codes;
    args.signs = signs;
    args.norms = norms;
    args.rnorms = rnorms;
    args.lists = *lists;
    args.status = p->counters + 1;
    args.wait_kcycles = p->wait_kcycles;
#ifdef TQ_PROF
    args.prof = reinterpret_cast<long long*>(p->counters + 8);   // cycle counters per role, measurement builds only
#endif

    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)d, (cuuint64_t)n};
    const cuuint64_t gstride[1] = {(cuuint64_t)d * 4};
    const cuuint32_t box[2] = {32, (cuuint32_t)kTileRows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = tq_encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(x), gdim, gstride,
                                         box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return tq_fail(TQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);

    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->device);
    const int grid = (int)(args.ntiles < sms ? args.ntiles : sms);
    const int bits = p->dev.bits;
    tq_timer_mark(p, 0, 0, st);
    int rc = TQ_ERR_UNSUPPORTED;
    if (d == 256) {
        switch (bits) {
            case 1: rc = prod ? launch_256<1, true>(map, args, grid, st) : launch_256<1, false>(map, args, grid, st); break;
            case 2: rc = prod ? launch_256<2, true>(map, args, grid, st) : launch_256<2, false>(map, args, grid, st); break;
            case 3: rc = prod ? launch_256<3, true>(map, args, grid, st) : launch_256<3, false>(map, args, grid, st); break;
            case 4: rc = prod ? launch_256<4, true>(map, args, grid, st) : launch_256<4, false>(map, args, grid, st); break;
        }
        tq_timer_mark(p, 0, 1, st);
        if (rc != TQ_ERR_UNSUPPORTED) return rc;
        return tq_fail(TQ_ERR_UNSUPPORTED, "no tensor-core kernel for bits=%d", bits);
    }
#define TQ_DISPATCH(B)                                                                                     \
    case B:                                                                                                \
        if (d == 64) rc = prod ? launch_one<64, B, true>(map, args, grid, st) : launch_one<64, B, false>(map, args, grid, st); \
        else rc = prod ? launch_one<128, B, true>(map, args, grid, st) : launch_one<128, B, false>(map, args, grid, st);      \
        break;
    switch (bits) {
        TQ_DISPATCH(1)
        TQ_DISPATCH(2)
        TQ_DISPATCH(3)
        TQ_DISPATCH(4)
    }
#undef TQ_DISPATCH
    tq_timer_mark(p, 0, 1, st);
    if (rc != TQ_ERR_UNSUPPORTED) return rc;
    return tq_fail(TQ_ERR_UNSUPPORTED, "no tensor-core kernel for bits=%d", bits);
}
