// Tensor-core scoring of TurboQuantProd keys (d = 128, 1..4 code bits) on B200.
//
//   score(q, key) = norm * ( (R q) . codebook[codes]  +  alpha * rnorm * ((S q) . signs) )
//
// is a small GEMM per tile of 128 keys: the keys are the M side, the (at most 32) queries the N side
// and the 128 coordinates the K side.  Per tile:
//
//   bulk copy (1 thread)   packed codes and sign words of 128 keys -> smem ring (plain 1-D bulk copies)
//   expanders (8 warps)    one thread per half key: turn packed codes into fp16 operands and store
//                          them into tensor memory with tcgen05.st (lane = key).  Two codes at a time
//                          index a lookup table of (hi pair, lo pair) half2 values -- centroid * 2^10
//                          split into fp16 hi + lo -- replicated per lane in smem so the lookups are
//                          free of bank conflicts; two sign bits become one half2 of +-1 with a shift
//                          and a logic op (the sign layout keeps them 16 bits apart for that).
//   MMA (1 thread)         D1 = C_hi Q_hi + C_lo Q_hi + C_hi Q_lo,  D2 = Sg P_hi + Sg P_lo  (kind::f16,
//                          fp32 accumulators in TMEM); Q = R q and P = S q are rotated / projected,
//                          scaled by a power of two and split into fp16 hi + lo once per call by a
//                          small preparation kernel, and live in smem as the B operand.
//   epilogue (4 warps)     one thread per key: tcgen05.ld both accumulators, apply the per-query
//                          descale, alpha * rnorm and norm, store one coalesced 128-byte line per query.
//
// A second kernel selects the per-query top-k from a score matrix with a rising threshold and a
// bitonic prune (the same scheme as the general kernel in tq_score.cu), one block per row segment.
#include "tq_common.cuh"
#include "tq_ptx.cuh"
#include "tq_topk.cuh"

#include <cuda.h>
#include <math.h>
#include <math_constants.h>
#include <stdlib.h>
#include <string.h>

namespace {

using namespace tqptx;
using namespace tqtopk;

constexpr int D = 128;
constexpr int kTileKeys = 128;
// Warps: bulk copy, MMA, 16 expanders (one thread per quarter key), then 4 epilogue warps per 16 queries of the pass.
// A pass of 64 queries has 16 epilogue warps and, a block being limited to 32 warps, 8 expanders (one thread per
// half key): what its tile waits for is the way of the single accumulator through the epilogue, which is as short with
// one block of 16 queries per thread as in the smaller passes.
template <int QPAD> struct ScoreThreads {
    static constexpr int kExpWarps = QPAD == 64 ? 8 : 16;
    static constexpr int kEpiPerRow = QPAD / 16;
    static constexpr int kEpiThreads = 4 * kEpiPerRow * 32;
    static constexpr int kThreads = (2 + kExpWarps) * 32 + kEpiThreads;
    static constexpr int kFirstEpiWarp = 2 + kExpWarps;
};
constexpr int kFirstExpWarp = 2;
constexpr int kMaxStages = 8;
constexpr float kCentScale = 1024.f;
constexpr int kRowBytesB = D * 2;  // one query row of one fp16 operand matrix
constexpr int kPrepSmemBytes = 2 * D * D * 4;  // rotation and projection matrices staged by the preparation kernel
constexpr int kEpiBarrier = 1;     // named barrier of the epilogue warps

// Prepared queries of one group: per half of the coordinates (two halves of 128 for d = 256, one otherwise) the four
// fp16 operand matrices q_hi, q_lo, p_hi, p_lo, then one (1 / scale) pair per query.
__host__ __device__ constexpr int prep_group_bytes(int qpad, int halves = 1) { return halves * 4 * qpad * kRowBytesB + 2 * qpad * 4; }

struct ScoreTcArgs {
    const uint32_t* codes;
    const uint32_t* signs;
    const float* rnorms;
    const float* norms;
    const unsigned char* prep;    // [groups][prep_group_bytes]
    const float* codebook;
    int64_t keys_per_group;       // rows between the first keys of consecutive groups
    int64_t key_off;              // first key of every group handled by this launch
    int64_t key_cnt;              // keys per group handled by this launch
    int64_t tiles_per_group, total_tiles;
    int nq;                       // live queries (<= QPAD)
    int64_t out_group_stride;     // floats between groups in `scores`
    int64_t out_row_stride;       // floats between query rows
    float* scores;                // points at (group 0, first query of this pass, key_off)
    int tile_store;               // 1: score tiles leave through shared memory and a bulk tensor store (tmap_out)
    int norms_bulk;               // 1: norms and residual norms travel with the packed rows through the key ring
    int tile_stride;              // tile kt of a group covers keys [kt * tile_stride * 128, +128): > 1 scores a sample of the tiles
    // Top-k without a score matrix (candidate mode): a score that reaches its query's threshold is appended to that
    // query's candidate list (sortable key: score bits | row) instead of being written anywhere else.
    int fused;                    // 0: score matrix; 1: candidates through a staging list; 2: the sampled pass (every score, fixed slots)
    int qpg_total, q0;            // queries per group over all passes, first query of this pass
    const float* thr;             // [groups][qpg_total] lower bound of the k-th best score so far (-inf: none)
    unsigned int* cnt;            // [groups][qpg_total] entries appended to each list
    unsigned long long* cand;     // [groups][qpg_total][cand_cap]
    int64_t cand_cap;
    float alpha;
    unsigned long long* status;
    int wait_kcycles;             // limit of one bounded wait, in units of 1024 cycles
#ifdef TQ_PROF
    long long* prof;              // per-role cycle counters (measurement builds only)
#endif
};

enum {
    SB_K_FULL = 0,      // [8]
    SB_K_EMPTY = 8,     // [8]
    SB_A_FULL = 16,     // [4]: per A buffer; in a pass of 64 queries per chunk of 32 coordinates of the single buffer
    SB_A_EMPTY = 20,    // [4]
    SB_D_FULL = 24,     // [2]
    SB_D_EMPTY = 26,    // [2]
    SB_B_FULL = 28,     // [2]
    SB_B_EMPTY = 30,    // [2]
    SB_COUNT = 32
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// Shared memory -> global, one box of a 3-D tensor map (keys, queries of the pass, groups); parts of the box
// outside the tensor are not written.
__device__ __forceinline__ void tensor_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until all but the newest `N` bulk groups of this thread have finished reading shared memory.
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// DR is the dimension of the vectors.  The operand layouts are those of d = 128 in every case: for d = 64 the upper
// half of every key is absent (its expander warps idle, the contractions stop after DR / 16 k-blocks); for d = 256 a
// tile of keys passes through the operand buffers as two halves of 128 coordinates, one after the other, whose
// contractions add up in the same accumulators (the prepared queries of a group then fill 64 KB, so that only one
// group's are resident).
template <int BITS, int QPAD, int DR>
struct ScoreSmem {
    static_assert(QPAD <= 32 || DR <= 128, "a pass of 64 queries exists for d <= 128");
    static constexpr int kHalves = DR == 256 ? 2 : 1;
    static constexpr int kBBufs = (DR == 256 || QPAD == 64) ? 1 : 2;     // 64 KB of prepared queries: one group resident
    static constexpr int kPrepBytes = prep_group_bytes(QPAD, kHalves);
    static constexpr int kLutEntries = 1 << (2 * BITS);
    static constexpr int kLutBytes = kLutEntries * 32 * 8;
    static constexpr int kCodeRowBytes = DR * BITS / 8;
    static constexpr int kSignRowBytes = DR / 8;
    static constexpr int kNormOff = kTileKeys * (kCodeRowBytes + kSignRowBytes);   // norms, then residual norms, of the tile's keys
    static constexpr int kStageBytes = kNormOff + 2 * kTileKeys * 4;
    static constexpr int kBBytes = (kPrepBytes + 127) & ~127;
    static constexpr int kOutBytes = QPAD * kTileKeys * 4;          // one staged tile of scores [query][key]
    static constexpr int kFixed = kLutBytes + kBBufs * kBBytes + 2 * kOutBytes + 640 + 128 + 128;
    static constexpr int kFit = (227 * 1024 - kFixed) / kStageBytes;
    static constexpr int kStages = kFit < kMaxStages ? kFit : kMaxStages;
    static_assert(kStages >= 3, "key ring too short");
    static constexpr int off_lut = 0;
    static constexpr int off_b = off_lut + kLutBytes;
    static constexpr int off_out = off_b + kBBufs * kBBytes;
    static constexpr int off_ring = off_out + 2 * kOutBytes;
    static constexpr int off_misc = off_ring + kStages * kStageBytes;
    static constexpr int total = off_misc + 640 + 128;
};

// CAND: candidate mode (top-k without a score matrix) is a kernel of its own, so that the matrix kernel carries none
// of its registers and code.
template <int BITS, int QPAD, int DR, bool CAND>
__global__ void __launch_bounds__(ScoreThreads<QPAD>::kThreads, 1)
score_tc_kernel(const __grid_constant__ CUtensorMap tmap_out, const ScoreTcArgs a) {
    static_assert(DR == 256 || DR == 128 || DR == 64, "written for d = 256, 128 and 64");
    using L = ScoreSmem<BITS, QPAD, DR>;
    constexpr int kHalves = L::kHalves;          // passes of a key tile through the operand buffers
    constexpr int kBBufs = L::kBBufs;
    constexpr int kDH = DR / kHalves;            // coordinates per pass
    constexpr int kChunks = kDH / 32;            // chunks of 32 coordinates per pass of a key through the buffers
    constexpr int kSub = kChunks * 4 > ScoreThreads<QPAD>::kExpWarps ? kChunks * 4 / ScoreThreads<QPAD>::kExpWarps : 1;   // chunks per expander thread (2 in a pass of 64 queries at d = 128)
    constexpr int kParts = kChunks / kSub;       // expander warps per lane quarter that have data
    constexpr int kFirstEpiWarp = ScoreThreads<QPAD>::kFirstEpiWarp;
    // A pass of 64 queries runs its single A buffer as a ring of chunks: the contractions of a tile take the chunks in
    // order (two k-blocks each) and hand every chunk back as soon as they are through with it, so the expanders fill
    // chunk c of the next tile while the contractions of this one are at chunk c + 1.
    constexpr bool kChunkRing = QPAD == 64;
    constexpr int kStages = L::kStages;
    constexpr int kThreads = ScoreThreads<QPAD>::kThreads;
    constexpr int kEpiPerRow = ScoreThreads<QPAD>::kEpiPerRow;
    constexpr int kEpiThreads = ScoreThreads<QPAD>::kEpiThreads;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const uint32_t smem_base = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::off_misc);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + SB_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    TQ_PROF_CODE(const long long prof_t0 = clock64();)

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(BAR(SB_K_FULL + i), 1);
            mbar_init(BAR(SB_K_EMPTY + i), 4 * kParts + (a.norms_bulk ? 4 * kEpiPerRow : 0));   // expanders (+ epilogue warps)
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(BAR(SB_A_FULL + i), kChunkRing ? 4 : 4 * kParts);
            mbar_init(BAR(SB_A_EMPTY + i), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(SB_D_FULL + i), 1);
            mbar_init(BAR(SB_D_EMPTY + i), 4 * kEpiPerRow);
            mbar_init(BAR(SB_B_FULL + i), 1);
            mbar_init(BAR(SB_B_EMPTY + i), 1 + 4 * kEpiPerRow);  // last MMA of the group + every epilogue warp
        }
        abort_flag[0] = 0;
        abort_flag[1] = a.wait_kcycles;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {   // pair lookup table: entry e = (code0 | code1 << BITS) -> (half2 hi(c0), hi(c1)), (half2 lo(c0), lo(c1))
        uint2* lut = reinterpret_cast<uint2*>(smem + L::off_lut);
        for (int i = threadIdx.x; i < L::kLutEntries * 32; i += kThreads) {
            const int e = i >> 5;
            const float c0 = __ldg(a.codebook + (e & ((1 << BITS) - 1))) * kCentScale;
            const float c1 = __ldg(a.codebook + (e >> BITS)) * kCentScale;
            const __half2 h = __floats2half2_rn(c0, c1);
            const float2 hf = __half22float2(h);
            uint2 v;
            v.x = *reinterpret_cast<const uint32_t*>(&h);
            v.y = pack_half2(c0 - hf.x, c1 - hf.y);
            lut[i] = v;
        }
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

    // contiguous tile range of this CTA, so that it rarely changes group
    const int64_t t0 = a.total_tiles * (int64_t)blockIdx.x / gridDim.x;
    const int64_t t1 = a.total_tiles * (int64_t)(blockIdx.x + 1) / gridDim.x;
    // Instruction descriptors for N = QPAD and N = 2*QPAD (hi and lo query halves side by side).
    constexpr uint32_t kIdesc1 = (1u << 4) | ((uint32_t)(QPAD >> 3) << 17) | ((uint32_t)(kTileKeys >> 4) << 24);
    constexpr uint32_t kIdesc2 = (1u << 4) | ((uint32_t)(2 * QPAD >> 3) << 17) | ((uint32_t)(kTileKeys >> 4) << 24);
    // TMEM: two A buffers of 192 columns (C_hi | C_lo | Sg), then the accumulators D1 = [C q_hi | C_hi q_lo]
    // and D2 = [Sg p_hi | Sg p_lo], 2*QPAD columns each; double-buffered when they fit (QPAD = 16).
    constexpr uint32_t kBufCols = 192;
    constexpr uint32_t kColHi = 0, kColLo = 64, kColSg = 128;
    // A pass of 64 queries has 256 accumulator columns and room for one A buffer only (run as a ring of chunks, below).
    // Measured alternatives per 64 x 1,048,576 scores / per 1,048,576 keys in candidate mode: 16 expander and 8 epilogue
    // warps with two blocks of 16 queries per epilogue thread 176 / 258 us (the accumulator stays with the epilogue twice
    // as long); the same with both A buffers and the hi and lo products added inside 128 accumulator columns (40
    // instructions of N = 64 per tile) 173 / 245 us; 8 expander and 16 epilogue warps with the A buffer handed over
    // whole 174 / 175 us; as a ring of chunks 171 / 178 us.
    constexpr int kABufs = QPAD == 64 ? 1 : 2;
    constexpr int kDBufs = QPAD == 16 ? 2 : 1;
    constexpr uint32_t kColD = kABufs * kBufCols, kDCols = 4 * QPAD;

    if (warp == 0) {
        if (lane == 0) {
            int64_t prev_g = -1, gcount = 0, issued = 0;
            int64_t g = t0 / a.tiles_per_group, kt = t0 - g * a.tiles_per_group;
            for (int64_t t = t0; t < t1; ++t, ++kt) {
                if (kt == a.tiles_per_group) { kt = 0; ++g; }
                if (g != prev_g) {
                    const int bb = (kBBufs == 2 ? (int)(gcount & 1) : 0);
                    if (!mbar_wait(BAR(SB_B_EMPTY + bb), (uint32_t)((kBBufs == 2 ? gcount >> 1 : gcount) & 1) ^ 1u, abort_flag)) break;
                    mbar_arrive_expect_tx(BAR(SB_B_FULL + bb), L::kPrepBytes);
                    bulk_load(smem_base + L::off_b + bb * L::kBBytes, a.prep + g * L::kPrepBytes, L::kPrepBytes, BAR(SB_B_FULL + bb));
                    prev_g = g;
                    ++gcount;
                }
                const int64_t i = t - t0;
                const int s = (int)(i % kStages);
                if (!mbar_wait(BAR(SB_K_EMPTY + s), (uint32_t)((i / kStages) & 1) ^ 1u, abort_flag)) break;
                const int64_t k0 = kt * a.tile_stride * kTileKeys;      // first key of the tile within this launch's range
                int64_t valid = a.key_cnt - k0;
                if (valid > kTileKeys) valid = kTileKeys;
                const int64_t row0 = g * a.keys_per_group + a.key_off + k0;
                const uint32_t cb = (uint32_t)valid * L::kCodeRowBytes, sb = (uint32_t)valid * L::kSignRowBytes;
                const unsigned char* csrc = reinterpret_cast<const unsigned char*>(a.codes) + row0 * L::kCodeRowBytes;
                const unsigned char* ssrc = reinterpret_cast<const unsigned char*>(a.signs) + row0 * L::kSignRowBytes;
                unsigned char* stage = smem + L::off_ring + s * L::kStageBytes;
                // a ragged last tile of 8- or 24-byte rows need not end on a 16-byte multiple: the bulk copies take
                // the multiple, plain loads the few bytes behind it
                copy_tail_words(stage, csrc, cb);
                copy_tail_words(stage + kTileKeys * L::kCodeRowBytes, ssrc, sb);
                const uint32_t nb = a.norms_bulk ? (uint32_t)valid * 4u : 0u;
                if (nb) {
                    copy_tail_words(stage + L::kNormOff, reinterpret_cast<const unsigned char*>(a.norms + row0), nb);
                    copy_tail_words(stage + L::kNormOff + kTileKeys * 4, reinterpret_cast<const unsigned char*>(a.rnorms + row0), nb);
                }
                mbar_arrive_expect_tx(BAR(SB_K_FULL + s), (cb & ~15u) + (sb & ~15u) + 2 * (nb & ~15u));
                const uint32_t dst = smem_base + L::off_ring + s * L::kStageBytes;
                if (cb & ~15u) bulk_load(dst, csrc, cb & ~15u, BAR(SB_K_FULL + s));
                if (sb & ~15u) bulk_load(dst + kTileKeys * L::kCodeRowBytes, ssrc, sb & ~15u, BAR(SB_K_FULL + s));
                if (nb & ~15u) {
                    bulk_load(dst + L::kNormOff, a.norms + row0, nb & ~15u, BAR(SB_K_FULL + s));
                    bulk_load(dst + L::kNormOff + kTileKeys * 4, a.rnorms + row0, nb & ~15u, BAR(SB_K_FULL + s));
                }
                issued = i + 1;
            }
            if (*abort_flag) {
                // copies armed above may still be on their way into this block's shared memory
                for (int64_t ii = issued > kStages ? issued - kStages : 0; ii < issued; ++ii)
                    mbar_drain(BAR(SB_K_FULL + (int)(ii % kStages)), (uint32_t)((ii / kStages) & 1));
                for (int64_t gg = gcount > kBBufs ? gcount - kBBufs : 0; gg < gcount; ++gg)
                    mbar_drain(BAR(SB_B_FULL + (kBBufs == 2 ? (int)(gg & 1) : 0)), (uint32_t)((kBBufs == 2 ? gg >> 1 : gg) & 1));
            }
        }
    } else if (warp == 1) {
        // The whole warp walks the tiles and waits; one elected lane issues, with every operand computed from
        // warp-uniform values (a single lane of a diverged warp pays about 64 cycles per instruction).
        {
            const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
            const uint32_t lbo = 128, sbo = (D / 8) * 128;
            int64_t prev_g = -1, gcount = 0;
            int bb = 0;
            int64_t g = t0 / a.tiles_per_group, kt = t0 - g * a.tiles_per_group;
            uint64_t dq_hi = 0, dp_hi = 0;
            if constexpr (kChunkRing) {
                bool gave_up = false;
                for (int64_t t = t0; t < t1 && !gave_up; ++t, ++kt) {
                    if (kt == a.tiles_per_group) { kt = 0; ++g; }
                    const int64_t i = t - t0;
                    const uint32_t par = (uint32_t)(i & 1);
                    if (g != prev_g) {
                        bb = 0;
                        if (!warp_wait(BAR(SB_B_FULL), (uint32_t)(gcount & 1), abort_flag)) break;
                        prev_g = g;
                        ++gcount;
                        const uint32_t bq = smem_base + L::off_b;
                        dq_hi = make_smem_desc(bq + 0 * QPAD * kRowBytesB, lbo, sbo);
                        dp_hi = make_smem_desc(bq + 2 * QPAD * kRowBytesB, lbo, sbo);
                    }
                    const uint32_t d1 = tm + kColD, d2 = d1 + 2 * QPAD;
                    const bool last_of_group = (t + 1 == t1) || (kt + 1 == a.tiles_per_group);
#pragma unroll 1
                    for (int c = 0; c < kChunks; ++c) {
                        if (!warp_wait(BAR(SB_A_FULL + c), par, abort_flag)) { gave_up = true; break; }
                        if (c == 0 && !warp_wait(BAR(SB_D_EMPTY), par ^ 1u, abort_flag)) { gave_up = true; break; }
                        tc_fence_after();
                        if (elect_one()) {
#pragma unroll 1
                            for (int kb = 2 * c; kb < 2 * c + 2; ++kb) {
                                const uint64_t step = (uint64_t)(kb * 2 * lbo >> 4);
                                const uint64_t qh = dq_hi + step, ph = dp_hi + step;
                                if (kb == 0) {
                                    mma_ts_first(d1, tm + kColHi, qh, kIdesc2);
                                    mma_ts_acc(d1, tm + kColLo, qh, kIdesc1);
                                    mma_ts_first(d2, tm + kColSg, ph, kIdesc2);
                                } else {
                                    mma_ts_acc(d1, tm + kColHi + kb * 8, qh, kIdesc2);
                                    mma_ts_acc(d1, tm + kColLo + kb * 8, qh, kIdesc1);
                                    mma_ts_acc(d2, tm + kColSg + kb * 8, ph, kIdesc2);
                                }
                            }
                            mma_commit(BAR(SB_A_EMPTY + c));     // this chunk's slot may be filled for the next tile
                            if (c == kChunks - 1) {
                                mma_commit(BAR(SB_D_FULL));
                                if (last_of_group) mma_commit(BAR(SB_B_EMPTY));
                            }
                        }
                        __syncwarp();
                    }
                }
            } else if constexpr (kHalves == 1) {
                for (int64_t t = t0; t < t1; ++t, ++kt) {
                    if (kt == a.tiles_per_group) { kt = 0; ++g; }
                    const int64_t i = t - t0;
                    const int b = kABufs == 2 ? (int)(i & 1) : 0;
                    const uint32_t par2 = (uint32_t)((kABufs == 2 ? i >> 1 : i) & 1);
                    if (g != prev_g) {
                        bb = (kBBufs == 2 ? (int)(gcount & 1) : 0);
                        if (!warp_wait(BAR(SB_B_FULL + bb), (uint32_t)((kBBufs == 2 ? gcount >> 1 : gcount) & 1), abort_flag)) break;
                        prev_g = g;
                        ++gcount;
                        const uint32_t bq = smem_base + L::off_b + bb * L::kBBytes;
                        dq_hi = make_smem_desc(bq + 0 * QPAD * kRowBytesB, lbo, sbo);
                        dp_hi = make_smem_desc(bq + 2 * QPAD * kRowBytesB, lbo, sbo);
                    }
                    TQ_PROF_CODE(long long c0 = clock64();)
                    if (!warp_wait(BAR(SB_A_FULL + b), par2, abort_flag)) break;
                    TQ_PROF_CODE(long long c1 = clock64();)
                    const int db = kDBufs == 2 ? (int)(i & 1) : 0;
                    const uint32_t dpar = (uint32_t)((kDBufs == 2 ? i >> 1 : i) & 1);
                    if (!warp_wait(BAR(SB_D_EMPTY + db), dpar ^ 1u, abort_flag)) break;
                    tc_fence_after();
                    TQ_PROF_CODE(long long c2 = clock64(); if (a.prof && blockIdx.x == 0 && lane == 0) { a.prof[8] += c1 - c0; a.prof[9] += c2 - c1; })
                    const uint32_t base = tm + b * kBufCols;
                    const uint32_t d1 = tm + kColD + db * kDCols, d2 = d1 + 2 * QPAD;
                    const bool last_of_group = (t + 1 == t1) || (kt + 1 == a.tiles_per_group);
                    if (elect_one()) {
                        // q_hi and q_lo (p_hi and p_lo) are adjacent row blocks of one operand: N = 2*QPAD
                        mma_ts_first(d1, base + kColHi, dq_hi, kIdesc2);
                        mma_ts_acc(d1, base + kColLo, dq_hi, kIdesc1);
                        mma_ts_first(d2, base + kColSg, dp_hi, kIdesc2);
#pragma unroll 1
                        for (int kb = 1; kb < DR / 16; ++kb) {
                            // the start-address field counts 16-byte units: one k-block (two core matrices) further
                            const uint64_t step = (uint64_t)(kb * 2 * lbo >> 4);
                            const uint64_t qh = dq_hi + step, ph = dp_hi + step;
                            mma_ts_acc(d1, base + kColHi + kb * 8, qh, kIdesc2);
                            mma_ts_acc(d1, base + kColLo + kb * 8, qh, kIdesc1);
                            mma_ts_acc(d2, base + kColSg + kb * 8, ph, kIdesc2);
                        }
                        mma_commit(BAR(SB_D_FULL + db));
                        mma_commit(BAR(SB_A_EMPTY + b));
                        if (last_of_group) mma_commit(BAR(SB_B_EMPTY + bb));
                    }
                    __syncwarp();
                    TQ_PROF_CODE(if (a.prof && blockIdx.x == 0 && lane == 0) a.prof[10] += clock64() - c2;)
                }
            } else {
                // d = 256: every tile passes through the operand buffers twice (coordinates 0..127, then 128..255)
                bool gave_up = false;
                for (int64_t t = t0; t < t1 && !gave_up; ++t, ++kt) {
                    if (kt == a.tiles_per_group) { kt = 0; ++g; }
                    const int64_t i = t - t0;
                    if (g != prev_g) {
                        bb = (kBBufs == 2 ? (int)(gcount & 1) : 0);
                        if (!warp_wait(BAR(SB_B_FULL + bb), (uint32_t)((kBBufs == 2 ? gcount >> 1 : gcount) & 1), abort_flag)) break;
                        prev_g = g;
                        ++gcount;
                        const uint32_t bq = smem_base + L::off_b + bb * L::kBBytes;
                        dq_hi = make_smem_desc(bq + 0 * QPAD * kRowBytesB, lbo, sbo);
                        dp_hi = make_smem_desc(bq + 2 * QPAD * kRowBytesB, lbo, sbo);
                    }
                    const int db = kDBufs == 2 ? (int)(i & 1) : 0;
                    const uint32_t dpar = kDBufs == 2 ? (uint32_t)((i >> 1) & 1) : (uint32_t)(i & 1);
                    const uint32_t d1 = tm + kColD + db * kDCols, d2 = d1 + 2 * QPAD;
                    const bool last_of_group = (t + 1 == t1) || (kt + 1 == a.tiles_per_group);
#pragma unroll 1
                    for (int h = 0; h < kHalves; ++h) {
                        const int64_t j = i * kHalves + h;       // passes through the operand buffers since the start
                        const int b = (int)(j & 1);
                        const uint32_t par2 = (uint32_t)((j >> 1) & 1);
                        TQ_PROF_CODE(long long c0 = clock64();)
                        if (!warp_wait(BAR(SB_A_FULL + b), par2, abort_flag)) { gave_up = true; break; }
                        TQ_PROF_CODE(long long c1 = clock64();)
                        if (h == 0 && !warp_wait(BAR(SB_D_EMPTY + db), dpar ^ 1u, abort_flag)) { gave_up = true; break; }
                        tc_fence_after();
                        TQ_PROF_CODE(long long c2 = clock64(); if (a.prof && blockIdx.x == 0 && lane == 0) { a.prof[8] += c1 - c0; a.prof[9] += c2 - c1; })
                        const uint32_t base = tm + b * kBufCols;
                        if (elect_one()) {
                            // the operand matrices of the second half of the coordinates follow those of the first
                            const uint64_t half_step = (uint64_t)((uint32_t)h * 4u * QPAD * kRowBytesB >> 4);
                            const uint64_t q0d = dq_hi + half_step, p0d = dp_hi + half_step;
                            // q_hi and q_lo (p_hi and p_lo) are adjacent row blocks of one operand: N = 2*QPAD
                            if (h == 0) {
                                mma_ts_first(d1, base + kColHi, q0d, kIdesc2);
                                mma_ts_acc(d1, base + kColLo, q0d, kIdesc1);
                                mma_ts_first(d2, base + kColSg, p0d, kIdesc2);
                            } else {
                                mma_ts_acc(d1, base + kColHi, q0d, kIdesc2);
                                mma_ts_acc(d1, base + kColLo, q0d, kIdesc1);
                                mma_ts_acc(d2, base + kColSg, p0d, kIdesc2);
                            }
#pragma unroll 1
                            for (int kb = 1; kb < kDH / 16; ++kb) {
                                // the start-address field counts 16-byte units: one k-block (two core matrices) further
                                const uint64_t step = (uint64_t)(kb * 2 * lbo >> 4);
                                const uint64_t qh = q0d + step, ph = p0d + step;
                                mma_ts_acc(d1, base + kColHi + kb * 8, qh, kIdesc2);
                                mma_ts_acc(d1, base + kColLo + kb * 8, qh, kIdesc1);
                                mma_ts_acc(d2, base + kColSg + kb * 8, ph, kIdesc2);
                            }
                            if (h == kHalves - 1) mma_commit(BAR(SB_D_FULL + db));
                            mma_commit(BAR(SB_A_EMPTY + b));
                            if (h == kHalves - 1 && last_of_group) mma_commit(BAR(SB_B_EMPTY + bb));
                        }
                        __syncwarp();
                        TQ_PROF_CODE(if (a.prof && blockIdx.x == 0 && lane == 0) a.prof[10] += clock64() - c2;)
                    }
                }
            }
        }
    } else if (warp < kFirstEpiWarp) {
        // ---- expanders: one thread per quarter key (32 coordinates) ---------------------------------
        const int part = (warp - kFirstExpWarp) >> 2;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint2* lut_lane = reinterpret_cast<const uint2*>(smem + L::off_lut) + lane;
        constexpr uint32_t kPairMask = (1u << (2 * BITS)) - 1u;
        TQ_PROF_CODE(long long pc[5] = {0, 0, 0, 0, 0};)
        if constexpr (kChunkRing) {
            // a pass of 64 queries: the thread's chunks one after the other, each into its slot of the single A buffer
            for (int64_t t = t0; t < (part < kParts ? t1 : t0); ++t) {
                const int64_t i = t - t0;
                const int s = (int)(i % kStages);
                const uint32_t par = (uint32_t)(i & 1);
                bool fail = !mbar_wait(BAR(SB_K_FULL + s), (uint32_t)((i / kStages) & 1), abort_flag);
#pragma unroll 1
                for (int sp = 0; sp < kSub; ++sp) {
                    const int chunk = part * kSub + sp;
                    uint32_t w[BITS + 1], sw;
                    {
                        const unsigned char* stage = smem + L::off_ring + s * L::kStageBytes;
                        const volatile uint32_t* cw = reinterpret_cast<const volatile uint32_t*>(stage + row * L::kCodeRowBytes) + chunk * BITS;
                        const volatile uint32_t* sg = reinterpret_cast<const volatile uint32_t*>(stage + kTileKeys * L::kCodeRowBytes + row * L::kSignRowBytes) + chunk;
#pragma unroll
                        for (int k = 0; k < BITS; ++k) w[k] = fail ? 0u : cw[k];
                        w[BITS] = 0;
                        sw = fail ? 0u : ~sg[0];
                    }
                    __threadfence_block();   // every lane's loads from the stage are performed before the stage is released
                    __syncwarp();
                    if (sp == kSub - 1 && lane == 0 && !fail) mbar_arrive(BAR(SB_K_EMPTY + s));
                    uint32_t hi[16], lo[16], sg[16];
#pragma unroll
                    for (int p = 0; p < 16; ++p) {
                        const int bit = p * 2 * BITS, wi = bit >> 5, sh = bit & 31;
                        uint32_t e;
                        if (sh + 2 * BITS <= 32) e = (w[wi] >> sh) & kPairMask;
                        else e = __funnelshift_r(w[wi], w[wi + 1], sh) & kPairMask;
                        const uint2 v = lut_lane[e * 32];
                        hi[p] = v.x;
                        lo[p] = v.y;
                        sg[p] = ((sw << (15 - p)) & 0x80008000u) | 0x3c003c00u;
                    }
                    if (!mbar_wait(BAR(SB_A_EMPTY + chunk), par ^ 1u, abort_flag)) fail = true;
                    tc_fence_after();
                    const uint32_t abase = tmem + lane_addr + chunk * 16;
                    tmem_st16(abase + kColHi, hi);
                    tmem_st16(abase + kColLo, lo);
                    tmem_st16(abase + kColSg, sg);
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(SB_A_FULL + chunk));
                }
            }
        } else if constexpr (kHalves == 1) {
            for (int64_t t = t0; t < (part < kParts ? t1 : t0); ++t) {
                const int64_t i = t - t0;
                const int s = (int)(i % kStages);
                const int b = kABufs == 2 ? (int)(i & 1) : 0;
                const uint32_t par2 = (uint32_t)((kABufs == 2 ? i >> 1 : i) & 1);
                TQ_PROF_CODE(long long c0 = clock64();)
                bool fail = !mbar_wait(BAR(SB_K_FULL + s), (uint32_t)((i / kStages) & 1), abort_flag);
                TQ_PROF_CODE(long long c1 = clock64(); pc[0] += c1 - c0;)
                uint32_t w[BITS + 1], sw;
                {
                    const unsigned char* stage = smem + L::off_ring + s * L::kStageBytes;
                    const volatile uint32_t* cw = reinterpret_cast<const volatile uint32_t*>(stage + row * L::kCodeRowBytes) + part * BITS;
                    const volatile uint32_t* sg = reinterpret_cast<const volatile uint32_t*>(stage + kTileKeys * L::kCodeRowBytes + row * L::kSignRowBytes) + part;
#pragma unroll
                    for (int k = 0; k < BITS; ++k) w[k] = fail ? 0u : cw[k];
                    w[BITS] = 0;
                    sw = fail ? 0u : ~sg[0];
                }
                __threadfence_block();   // every lane's loads from the stage are performed before the stage is released
                __syncwarp();
                if (lane == 0 && !fail) mbar_arrive(BAR(SB_K_EMPTY + s));
                TQ_PROF_CODE(c0 = clock64(); pc[1] += c0 - c1;)
                // expand while the A buffer may still be in use; only the stores wait for it
                uint32_t hi[16], lo[16], sg[16];
#pragma unroll
                for (int p = 0; p < 16; ++p) {
                    const int bit = p * 2 * BITS, wi = bit >> 5, sh = bit & 31;
                    uint32_t e;
                    if (sh + 2 * BITS <= 32) e = (w[wi] >> sh) & kPairMask;
                    else e = __funnelshift_r(w[wi], w[wi + 1], sh) & kPairMask;
                    const uint2 v = lut_lane[e * 32];
                    hi[p] = v.x;
                    lo[p] = v.y;
                    // the sign word covers the 32 coordinates of this part; pair p: bits p, 16+p
                    sg[p] = ((sw << (15 - p)) & 0x80008000u) | 0x3c003c00u;
                }
                TQ_PROF_CODE(c1 = clock64(); pc[4] += c1 - c0;)
                if (!mbar_wait(BAR(SB_A_EMPTY + b), par2 ^ 1u, abort_flag)) fail = true;
                TQ_PROF_CODE(c0 = clock64(); pc[2] += c0 - c1;)
                tc_fence_after();
                const uint32_t abase = tmem + lane_addr + b * kBufCols + part * 16;
                tmem_st16(abase + kColHi, hi);
                tmem_st16(abase + kColLo, lo);
                tmem_st16(abase + kColSg, sg);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(SB_A_FULL + b));
                TQ_PROF_CODE(c1 = clock64(); pc[3] += c1 - c0;)
#ifdef TQ_PROF
                if (a.prof && blockIdx.x == 0 && threadIdx.x == kFirstExpWarp * 32 && t + 1 == t1) {
                    for (int k = 0; k < 5; ++k) a.prof[k] = pc[k];
                    a.prof[6] = t1 - t0;
                }
#endif
            }
        } else {
            for (int64_t t = t0; t < (part < kParts ? t1 : t0); ++t) {
                const int64_t i = t - t0;
                const int s = (int)(i % kStages);
                TQ_PROF_CODE(long long c0 = clock64();)
                bool fail = !mbar_wait(BAR(SB_K_FULL + s), (uint32_t)((i / kStages) & 1), abort_flag);
                TQ_PROF_CODE(long long c1 = clock64(); pc[0] += c1 - c0;)
#pragma unroll 1
                for (int h = 0; h < kHalves; ++h) {
                    const int64_t j = i * kHalves + h;       // passes through the operand buffers since the start
                    const int b = (int)(j & 1);
                    const uint32_t par2 = (uint32_t)((j >> 1) & 1);
                    TQ_PROF_CODE(if (h) c1 = clock64();)
                    uint32_t w[BITS + 1], sw;
                    {
                        const int chunk = h * 4 + part;      // this thread's 32 coordinates of the key
                        const unsigned char* stage = smem + L::off_ring + s * L::kStageBytes;
                        const volatile uint32_t* cw = reinterpret_cast<const volatile uint32_t*>(stage + row * L::kCodeRowBytes) + chunk * BITS;
                        const volatile uint32_t* sg = reinterpret_cast<const volatile uint32_t*>(stage + kTileKeys * L::kCodeRowBytes + row * L::kSignRowBytes) + chunk;
#pragma unroll
                        for (int k = 0; k < BITS; ++k) w[k] = fail ? 0u : cw[k];
                        w[BITS] = 0;
                        sw = fail ? 0u : ~sg[0];
                    }
                    __threadfence_block();   // every lane's loads from the stage are performed before the stage is released
                    __syncwarp();
                    if (h == kHalves - 1 && lane == 0 && !fail) mbar_arrive(BAR(SB_K_EMPTY + s));
                    TQ_PROF_CODE(c0 = clock64(); pc[1] += c0 - c1;)
                    // expand while the A buffer may still be in use; only the stores wait for it
                    uint32_t hi[16], lo[16], sg[16];
#pragma unroll
                    for (int p = 0; p < 16; ++p) {
                        const int bit = p * 2 * BITS, wi = bit >> 5, sh = bit & 31;
                        uint32_t e;
                        if (sh + 2 * BITS <= 32) e = (w[wi] >> sh) & kPairMask;
                        else e = __funnelshift_r(w[wi], w[wi + 1], sh) & kPairMask;
                        const uint2 v = lut_lane[e * 32];
                        hi[p] = v.x;
                        lo[p] = v.y;
                        // the sign word covers the 32 coordinates of this part; pair p: bits p, 16+p
                        sg[p] = ((sw << (15 - p)) & 0x80008000u) | 0x3c003c00u;
                    }
                    TQ_PROF_CODE(c1 = clock64(); pc[4] += c1 - c0;)
                    if (!mbar_wait(BAR(SB_A_EMPTY + b), par2 ^ 1u, abort_flag)) fail = true;
                    TQ_PROF_CODE(c0 = clock64(); pc[2] += c0 - c1;)
                    tc_fence_after();
                    const uint32_t abase = tmem + lane_addr + b * kBufCols + part * 16;
                    tmem_st16(abase + kColHi, hi);
                    tmem_st16(abase + kColLo, lo);
                    tmem_st16(abase + kColSg, sg);
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(SB_A_FULL + b));
                    TQ_PROF_CODE(c1 = clock64(); pc[3] += c1 - c0;)
                }
#ifdef TQ_PROF
                if (a.prof && blockIdx.x == 0 && threadIdx.x == kFirstExpWarp * 32 && t + 1 == t1) {
                    for (int k = 0; k < 5; ++k) a.prof[k] = pc[k];
                    a.prof[6] = t1 - t0;
                }
#endif
            }
        }
    } else {
        // ---- epilogue -----------------------------------------------------------------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int q16 = ((warp - kFirstEpiWarp) >> 2) * 16;   // this thread's 16 queries of the pass
        const bool store_leader = threadIdx.x == kFirstEpiWarp * 32;
        int64_t prev_g = -1, gcount = 0;
        int bb = 0;
        int64_t g = t0 / a.tiles_per_group, kt = t0 - g * a.tiles_per_group;
        // norm and residual norm of this thread's key, fetched one tile ahead of their use (a load issued
        // in the tile that needs it would stall the stores for a full trip to memory)
        auto fetch_norms = [&](int64_t gg, int64_t kk, float& n_out, float& r_out) {
            const int64_t key_n = kk * a.tile_stride * kTileKeys + row;
            const bool live_n = key_n < a.key_cnt;
            const int64_t grow_n = gg * a.keys_per_group + a.key_off + key_n;
            n_out = live_n ? __ldg(a.norms + grow_n) : 0.f;
            r_out = live_n ? __ldg(a.rnorms + grow_n) : 0.f;
        };
        // candidate mode: thresholds of the current group, and in place of the score tile buffers a staging list of
        // survivors (keys, then the numbers of their lists) and 16 x 32 parked scores per warp
        int64_t thr_g = -1;
        float* thr_s = reinterpret_cast<float*>(bars + SB_COUNT + 2);   // [QPAD]
        int* st_count = reinterpret_cast<int*>(thr_s + QPAD);
        constexpr int kStageCap = (2 * L::kOutBytes - 4 * kEpiPerRow * 16 * 32 * 4) / 12 / 128 * 128;    // 1,280 entries (32 queries), 640 (16), 2,688 (64)
        static_assert(kStageCap >= 512, "candidate staging must fit the score tile buffers");
        unsigned long long* st_keys = reinterpret_cast<unsigned long long*>(smem + L::off_out);
        uint32_t* st_list = reinterpret_cast<uint32_t*>(smem + L::off_out + kStageCap * 8);
        float* warp_scores = reinterpret_cast<float*>(smem + L::off_out + kStageCap * 12) + (warp - kFirstEpiWarp) * 16 * 32;
        const int epi_t = threadIdx.x - kFirstEpiWarp * 32;
        auto flush_staging = [&]() {      // all epilogue threads, after a barrier that made every append visible
            int n = *st_count;
            if (n > kStageCap) n = kStageCap;
            for (int i = epi_t; i < n; i += kEpiThreads) {
                const int64_t l = st_list[i];
                const int64_t gp = (int64_t)atomicAdd(a.cnt + l, 1u);
                if (gp < a.cand_cap) a.cand[l * a.cand_cap + gp] = st_keys[i];
            }
            bar_sync(kEpiBarrier, kEpiThreads);
            if (epi_t == 0) *st_count = 0;
            bar_sync(kEpiBarrier, kEpiThreads);
        };
        if (CAND) {
            if (epi_t == 0) *st_count = 0;
            bar_sync(kEpiBarrier, kEpiThreads);
        }
        float nrm_next = 0.f, rn_next = 0.f;
        if (t0 < t1 && !a.norms_bulk) fetch_norms(g, kt, nrm_next, rn_next);
        TQ_PROF_CODE(long long ep[8] = {0, 0, 0, 0, 0, 0, 0, 0};)
        for (int64_t t = t0; t < t1; ++t, ++kt) {
            TQ_PROF_CODE(const long long ctop = clock64();)
            if (kt == a.tiles_per_group) { kt = 0; ++g; }
            const int64_t i = t - t0;
            const int b = (int)(i & 1);        // staging buffer and accumulators of this tile
            const uint32_t par2 = (uint32_t)((i >> 1) & 1);
            if (g != prev_g) { bb = (kBBufs == 2 ? (int)(gcount & 1) : 0); prev_g = g; ++gcount; }
            const int64_t key = kt * a.tile_stride * kTileKeys + row;          // within this launch's key range
            const bool live = key < a.key_cnt;
            float nrm, arn;
            if (a.norms_bulk) {
                // norms ride in the key ring (a load from global memory here costs a full trip to HBM per tile,
                // which one tile of lookahead does not hide once a tile takes less than a microsecond)
                const int s = (int)(i % kStages);
                mbar_wait(BAR(SB_K_FULL + s), (uint32_t)((i / kStages) & 1), abort_flag);
                // volatile: the values stay in registers through the whole tile, and a plain load may be executed again where
                // the value is used (cheaper than keeping or spilling a register) -- after the arrival below, when the
                // stage may already hold another tile.  That happened: in candidate mode, where warps that lag behind
                // their tile for microseconds exist, about one score in 10^9 came out with the norm of a key eight tiles on.
                const volatile float* nr = reinterpret_cast<const volatile float*>(smem + L::off_ring + s * L::kStageBytes + L::kNormOff);
                nrm = live ? nr[row] : 0.f;
                arn = live ? a.alpha * nr[kTileKeys + row] : 0.f;
                __threadfence_block();   // every lane's loads from the stage are performed before the stage is released
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(SB_K_EMPTY + s));
            } else {
                nrm = nrm_next;
                arn = a.alpha * rn_next;
                if (t + 1 < t1) {
                    const bool wrap = kt + 1 == a.tiles_per_group;
                    fetch_norms(wrap ? g + 1 : g, wrap ? 0 : kt + 1, nrm_next, rn_next);
                }
            }
            TQ_PROF_CODE(long long c0 = clock64();)
            const int db = kDBufs == 2 ? b : 0;
            const uint32_t dpar = kDBufs == 2 ? par2 : (uint32_t)(i & 1);
            const bool got = mbar_wait(BAR(SB_D_FULL + db), dpar, abort_flag);   // false: some role gave up
            tc_fence_after();
            TQ_PROF_CODE(long long c1 = clock64();)
            TQ_PROF_CODE(long long c2 = c1;)
            const uint32_t rowid = (uint32_t)(g * a.keys_per_group + a.key_off + key);   // row of the key arrays (candidate mode)
            uint32_t pm = 0;      // candidate mode: bit k = this key's score for query q16 + k reaches the query's threshold
            const uint32_t dbase = tmem + lane_addr + kColD + db * kDCols + q16;
            const float2* ds = reinterpret_cast<const float2*>(smem + L::off_b + bb * L::kBBytes + kHalves * 4 * QPAD * kRowBytesB) + q16;
            float sc[16];
            {
                uint32_t ua[16], ub[16];
                tmem_ld16(dbase, ua);                  // C q_hi   (+ C_lo q_hi)
                tmem_ld16(dbase + QPAD, ub);           // C_hi q_lo
                tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < 16; ++k) sc[k] = (__uint_as_float(ua[k]) + __uint_as_float(ub[k])) * ds[k].x;
                tmem_ld16(dbase + 2 * QPAD, ua);       // Sg p_hi
                tmem_ld16(dbase + 3 * QPAD, ub);       // Sg p_lo
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(SB_D_EMPTY + db));   // the accumulators are free again
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const float s2 = (__uint_as_float(ua[k]) + __uint_as_float(ub[k])) * ds[k].y;
                    sc[k] = nrm * fmaf(arn, s2, sc[k]);
                }
            }
            TQ_PROF_CODE(c2 = clock64();)
            // After a give-up (`got` false) nothing is written for the tile, but every epilogue warp still walks through the
            // named barriers below: the warps learn of the give-up at different tiles, and a barrier that some of them
            // skipped would never complete.
            if (CAND) {
                if (g != thr_g) {      // thresholds of this group's queries (constant during the launch) into shared memory
                    thr_g = g;
                    bar_sync(kEpiBarrier, kEpiThreads);      // everybody is done with the previous group's
                    if (epi_t < QPAD) thr_s[epi_t] = epi_t < a.nq ? __ldg(a.thr + g * a.qpg_total + a.q0 + epi_t) : CUDART_INF_F;
                    bar_sync(kEpiBarrier, kEpiThreads);
                }
                const int64_t q_first = g * a.qpg_total + a.q0 + q16;
                if (a.fused == 2) {
                    // The sampled pass (thresholds at -inf, every score is a candidate): the slot of a score is known
                    // without a counter (tile of the sample x 128 + row); the host presets the lists' lengths.
                    // A key beyond the end of the group leaves an empty slot.
#pragma unroll
                    for (int k = 0; k < 16; ++k)
                        if (q16 + k < a.nq)
                            a.cand[(q_first + k) * a.cand_cap + kt * kTileKeys + row] = live && got ? make_key(sc[k], rowid) : 0ull;
                } else {
                    // This thread's scores against their thresholds: a mask, and -- when any of the warp's 32 keys has
                    // a survivor -- the scores parked in shared memory, so that the loop below can pick them by a
                    // run-time index.
                    float* mine = warp_scores + lane;
                    uint32_t m = 0;
#pragma unroll
                    for (int k = 0; k < 16; ++k) m |= (live && got && sc[k] >= thr_s[q16 + k]) ? (1u << k) : 0u;
                    if (__any_sync(0xffffffffu, m != 0u)) {
#pragma unroll
                        for (int k = 0; k < 16; ++k) mine[k * 32] = sc[k];
                    }
                    pm = m;
                }
            } else if (a.tile_store) {
                // The tile leaves as one box [queries of the pass][128 keys]: staged in shared memory (lanes hold
                // consecutive keys, so the stores are free of bank conflicts) and written by one bulk tensor store,
                // which clips the keys and queries beyond the matrix.  Two staging buffers: the store of tile
                // i - 2 must have read its buffer before tile i overwrites it.  (A box per warp -- 32 keys x 16 queries from
                // a slice of its own, no barrier between the epilogue warps -- was slower: 115 against 109 us.)
                float* stage = reinterpret_cast<float*>(smem + L::off_out + b * L::kOutBytes);
                TQ_PROF_CODE(const long long s0 = clock64();)
                if (store_leader) bulk_wait_read<1>();
                bar_sync(kEpiBarrier, kEpiThreads);
                TQ_PROF_CODE(const long long s1 = clock64();)
#pragma unroll
                for (int k = 0; k < 16; ++k) stage[(q16 + k) * kTileKeys + row] = sc[k];
                fence_async_smem();
                TQ_PROF_CODE(const long long s2 = clock64();)
                bar_sync(kEpiBarrier, kEpiThreads);
                TQ_PROF_CODE(const long long s3 = clock64();)
                if (store_leader && got) {
                    tensor_store_3d(&tmap_out, smem_base + L::off_out + b * L::kOutBytes, (int)(kt * kTileKeys), 0, (int)g);
                    bulk_commit();
                }
                TQ_PROF_CODE(ep[4] += s1 - s0; ep[5] += s2 - s1; ep[6] += s3 - s2; ep[7] += clock64() - s3;)
            } else if (live && got) {
                float* out = a.scores + g * a.out_group_stride + key + (int64_t)q16 * a.out_row_stride;
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    if (q16 + k < a.nq) {
                        __stcs(out, sc[k]);
                        out += a.out_row_stride;
                    }
                }
            }
            if (CAND && a.fused != 2) {
                // The loop runs once per query that has a survivor among the warp's 32 keys and is kept rolled: the candidate
                // path must stay small, this kernel lives on its instruction cache (the same logic unrolled over the
                // queries doubled the kernel's time without a single survivor).
                // Survivors go to a staging list in shared memory (a global counter update per survivor would put a
                // trip to L2 on this warp's path every tile); the list is emptied into the global lists, all its
                // entries at once, when it is half full (looked at every eighth tile: the barrier couples the warps).
                const float* mine = warp_scores + lane;
                const int64_t q_first = g * a.qpg_total + a.q0 + q16;
                if ((i & 7) == 0 && bar_or(kEpiBarrier, kEpiThreads, *st_count > kStageCap / 2)) flush_staging();
                uint32_t wm = __reduce_or_sync(0xffffffffu, pm);
#pragma unroll 1
                while (wm != 0u) {
                    const int k = __ffs(wm) - 1;
                    wm &= wm - 1u;
                    const bool pass = (pm >> k) & 1u;
                    const uint32_t votes = __ballot_sync(0xffffffffu, pass);
                    const int leader = __ffs(votes) - 1;
                    uint32_t base = 0;
                    if (lane == leader) base = (uint32_t)atomicAdd(st_count, (int)__popc(votes));
                    base = __shfl_sync(0xffffffffu, base, leader);
                    if (pass) {
                        const uint32_t pos = base + __popc(votes & ((1u << lane) - 1u));
                        const unsigned long long ck = make_key(mine[k * 32], rowid);
                        if (pos < (uint32_t)kStageCap) {
                            st_keys[pos] = ck;
                            st_list[pos] = (uint32_t)(q_first + k);
                        } else {      // the staging list is full (nearly every score passes): straight to the global list
                            const int64_t gp = (int64_t)atomicAdd(a.cnt + q_first + k, 1u);
                            if (gp < a.cand_cap) a.cand[(q_first + k) * a.cand_cap + gp] = ck;
                        }
                    }
                }
            }
            TQ_PROF_CODE(ep[0] += c0 - ctop; ep[1] += c1 - c0; ep[2] += c2 - c1; ep[3] += clock64() - c2;)
            const bool last_of_group = (t + 1 == t1) || (kt + 1 == a.tiles_per_group);
            if (last_of_group) {
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(SB_B_EMPTY + bb));
            }
        }
        if (CAND) {
            bar_sync(kEpiBarrier, kEpiThreads);
            flush_staging();
        }
#ifdef TQ_PROF
        if (a.prof && blockIdx.x == 0 && threadIdx.x == kFirstEpiWarp * 32 + 32) {      // a thread that is not the store leader's warp
            a.prof[18] = ep[0]; a.prof[12] = ep[1]; a.prof[13] = ep[2]; a.prof[14] = ep[3];
            a.prof[19] = ep[4]; a.prof[20] = ep[5]; a.prof[21] = ep[6]; a.prof[22] = ep[7];
        }
#endif
        if (store_leader) bulk_wait_all();   // the staged tiles must have left before the block's shared memory goes away
    }

    if (*abort_flag) __nanosleep(20000);   // tensor instructions issued before the give-up may still be running
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.status, 2ull);
    TQ_PROF_CODE(if (a.prof && blockIdx.x == 0 && threadIdx.x == 0) { a.prof[16] = clock64() - prof_t0; a.prof[17] = prof_t1 - prof_t0; })
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// Rotate / project the queries of one pass and lay them out as fp16 hi/lo B operands.
// grid (QPAD, groups), block 128 (thread = coordinate).
__global__ void __launch_bounds__(128)
score_prep_kernel(TqDev p, const float* __restrict__ q, int qpg, int q0, int nq, int qpad, unsigned char* __restrict__ prep) {
    __shared__ float qs[D];
    __shared__ float red[2][4];
    const int slot = blockIdx.x, g = blockIdx.y, j = threadIdx.x;
    unsigned char* base = prep + (size_t)g * prep_group_bytes(qpad);
    const size_t off = (size_t)(slot / 8) * ((D / 8) * 128) + (size_t)(j / 8) * 128 + (size_t)(slot % 8) * 16 + (size_t)(j % 8) * 2;
    __half* m0 = reinterpret_cast<__half*>(base + 0 * (size_t)qpad * kRowBytesB + off);
    __half* m1 = reinterpret_cast<__half*>(base + 1 * (size_t)qpad * kRowBytesB + off);
    __half* m2 = reinterpret_cast<__half*>(base + 2 * (size_t)qpad * kRowBytesB + off);
    __half* m3 = reinterpret_cast<__half*>(base + 3 * (size_t)qpad * kRowBytesB + off);
    float2* ds = reinterpret_cast<float2*>(base + 4 * (size_t)qpad * kRowBytesB);
    if (slot >= nq) {
        *m0 = *m1 = *m2 = *m3 = __float2half_rn(0.f);
        if (j == 0) ds[slot] = make_float2(0.f, 0.f);
        return;
    }
    const int d = p.d;   // 128, or 64 with the upper half of every operand row left unused
    qs[j] = j < d ? q[((size_t)g * qpg + q0 + slot) * d + j] : 0.f;
    __syncthreads();
    float r = 0.f, s = 0.f;
    // The matrices are usually cold (the keys streamed through L2 since the last call), so the time would
    // go into memory latency if the loads trickled in between the arithmetic: bring both matrices into
    // shared memory with all copies in flight at once, then run the two chains in order from there.
    extern __shared__ __align__(16) float mats[];   // [2][D][D]: R^T, S^T
    {
        const uint32_t dst0 = (uint32_t)__cvta_generic_to_shared(mats);
        const int kChunks = d * d / 4;              // 16-byte chunks per matrix
        for (int c = j; c < kChunks; c += 128) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + c * 16), "l"(p.Rt + (size_t)c * 4) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + (kChunks + c) * 16), "l"(p.St + (size_t)c * 4) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }
    const float* Rs = mats;
    const float* Ss = mats + d * d;
    if (j < d) {
#pragma unroll 16
        for (int k = 0; k < d; ++k) {
            r = fmaf(qs[k], Rs[k * d + j], r);
            s = fmaf(qs[k], Ss[k * d + j], s);
        }
    }
    float mr = fabsf(r), ms = fabsf(s);
    for (int o = 16; o > 0; o >>= 1) {
        mr = fmaxf(mr, __shfl_xor_sync(0xffffffffu, mr, o));
        ms = fmaxf(ms, __shfl_xor_sync(0xffffffffu, ms, o));
    }
    if ((j & 31) == 0) { red[0][j >> 5] = mr; red[1][j >> 5] = ms; }
    __syncthreads();
    mr = fmaxf(fmaxf(red[0][0], red[0][1]), fmaxf(red[0][2], red[0][3]));
    ms = fmaxf(fmaxf(red[1][0], red[1][1]), fmaxf(red[1][2], red[1][3]));
    // power-of-two scales that bring the largest magnitude into [512, 1024): safe in fp16, exact to undo
    const bool okr = mr > 0.f && mr < 3.0e38f, oks = ms > 0.f && ms < 3.0e38f;
    const float e1 = okr ? ldexpf(1.f, 9 - ilogbf(mr)) : 1.f;
    const float e2 = oks ? ldexpf(1.f, 9 - ilogbf(ms)) : 1.f;
    const float rs = r * e1, ss = s * e2;
    const __half rh = __float2half_rn(rs), sh = __float2half_rn(ss);
    *m0 = rh;
    *m1 = __float2half_rn(rs - __half2float(rh));
    *m2 = sh;
    *m3 = __float2half_rn(ss - __half2float(sh));
    if (j == 0) ds[slot] = make_float2(1.f / (e1 * kCentScale), 1.f / e2);
}

// The same for d = 256: the matrices do not fit shared memory and are read from global memory (usually cold), so the
// kernel lives on the number of loads in flight: block 1024, thread = (coordinate, quarter of the sum), 16 loads per
// matrix in flight per thread (39 us with 256 threads and four: a third of the scoring of 1,048,576 keys it precedes).
// The operands are written as two halves of 128 coordinates, each in the layout of d = 128.
__global__ void __launch_bounds__(1024)
score_prep256_kernel(TqDev p, const float* __restrict__ q, int qpg, int q0, int nq, int qpad, unsigned char* __restrict__ prep) {
    constexpr int kD = 256, kParts = 4, kSteps = kD / kParts;
    __shared__ float qs[kD];
    __shared__ float part[2][kParts][kD];
    __shared__ float red[2][8];
    const int slot = blockIdx.x, g = blockIdx.y, j = threadIdx.x & (kD - 1), kq = threadIdx.x >> 8;
    unsigned char* base = prep + (size_t)g * prep_group_bytes(qpad, 2);
    const int jh = j & 127;
    const size_t off = (size_t)(j >> 7) * (4 * (size_t)qpad * kRowBytesB) + (size_t)(slot / 8) * ((D / 8) * 128) +
                       (size_t)(jh / 8) * 128 + (size_t)(slot % 8) * 16 + (size_t)(jh % 8) * 2;
    __half* m0 = reinterpret_cast<__half*>(base + 0 * (size_t)qpad * kRowBytesB + off);
    __half* m1 = reinterpret_cast<__half*>(base + 1 * (size_t)qpad * kRowBytesB + off);
    __half* m2 = reinterpret_cast<__half*>(base + 2 * (size_t)qpad * kRowBytesB + off);
    __half* m3 = reinterpret_cast<__half*>(base + 3 * (size_t)qpad * kRowBytesB + off);
    float2* ds = reinterpret_cast<float2*>(base + 8 * (size_t)qpad * kRowBytesB);
    if (slot >= nq) {
        if (kq == 0) {
            *m0 = *m1 = *m2 = *m3 = __float2half_rn(0.f);
            if (j == 0) ds[slot] = make_float2(0.f, 0.f);
        }
        return;
    }
    if (kq == 0) qs[j] = q[((size_t)g * qpg + q0 + slot) * kD + j];
    __syncthreads();
    // four independent chains per matrix; the order of the sums differs from the general kernel's, which the fp32
    // tolerance of the scores covers
    float r[4] = {0.f, 0.f, 0.f, 0.f}, s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* Rt = p.Rt + (size_t)kq * kSteps * kD + j;
    const float* St = p.St + (size_t)kq * kSteps * kD + j;
    const float* qk = qs + kq * kSteps;
#pragma unroll 16
    for (int k = 0; k < kSteps; ++k) {
        r[k & 3] = fmaf(qk[k], __ldg(Rt + (size_t)k * kD), r[k & 3]);
        s[k & 3] = fmaf(qk[k], __ldg(St + (size_t)k * kD), s[k & 3]);
    }
    part[0][kq][j] = (r[0] + r[1]) + (r[2] + r[3]);
    part[1][kq][j] = (s[0] + s[1]) + (s[2] + s[3]);
    __syncthreads();
    if (kq != 0) return;      // threads 0..255 (warps 0..7) finish the coordinate
    const float rr = (part[0][0][j] + part[0][1][j]) + (part[0][2][j] + part[0][3][j]);
    const float sv = (part[1][0][j] + part[1][1][j]) + (part[1][2][j] + part[1][3][j]);
    float mr = fabsf(rr), ms = fabsf(sv);
    for (int o = 16; o > 0; o >>= 1) {
        mr = fmaxf(mr, __shfl_xor_sync(0xffffffffu, mr, o));
        ms = fmaxf(ms, __shfl_xor_sync(0xffffffffu, ms, o));
    }
    if ((j & 31) == 0) { red[0][j >> 5] = mr; red[1][j >> 5] = ms; }
    asm volatile("bar.sync 1, 256;" ::: "memory");      // the 256 threads that are left
    mr = ms = 0.f;
    for (int w = 0; w < 8; ++w) { mr = fmaxf(mr, red[0][w]); ms = fmaxf(ms, red[1][w]); }
    const bool okr = mr > 0.f && mr < 3.0e38f, oks = ms > 0.f && ms < 3.0e38f;
    const float e1 = okr ? ldexpf(1.f, 9 - ilogbf(mr)) : 1.f;
    const float e2 = oks ? ldexpf(1.f, 9 - ilogbf(ms)) : 1.f;
    const float rs = rr * e1, ss = sv * e2;
    const __half rh = __float2half_rn(rs), sh = __float2half_rn(ss);
    *m0 = rh;
    *m1 = __float2half_rn(rs - __half2float(rh));
    *m2 = sh;
    *m3 = __float2half_rn(ss - __half2float(sh));
    if (j == 0) ds[slot] = make_float2(1.f / (e1 * kCentScale), 1.f / e2);
}

// grid (segments, rows): block scans scores[row][seg*seg_len ...) and writes its k best as sortable keys
// to part[((group*lists_per_group + list_base + seg) * qpg + qi) * topk ...].  Candidates above the
// running threshold are collected in shared memory; when the buffer could overflow in the next batch
// it is cut back to the k best, which also raises the threshold.
__global__ void __launch_bounds__(kSelThreads)
topk_rows_kernel(const float* __restrict__ scores, int64_t row_stride, int64_t group_stride, int qpg, int64_t n,
                 int64_t seg_len, int64_t first_row_of_group_stride, int64_t key_off, int topk, int k2,
                 int lists_per_group, int list_base, unsigned long long* __restrict__ part) {
    __shared__ __align__(16) unsigned long long buf[kSelCap];
    __shared__ int hist[256];
    __shared__ int scratch[4];
    __shared__ int cnt;
    __shared__ unsigned long long thr;
    const int seg = blockIdx.x, r = blockIdx.y, g = r / qpg, qi = r - g * qpg;
    const float* src = scores + g * group_stride + qi * row_stride;
    const uint32_t row0 = (uint32_t)(g * first_row_of_group_stride + key_off);
    const int64_t k0 = (int64_t)seg * seg_len;
    int64_t k1 = k0 + seg_len;
    if (k1 > n) k1 = n;
    if (threadIdx.x == 0) { cnt = 0; thr = 0ull; }
    __syncthreads();
    // First threshold without filling the buffer: every thread takes the best of 32 scores from the head of the segment
    // (8,192 in all); the k-th best of those 256 maxima is a score that at least k scores of the segment reach, and on
    // data without order about 3 % of all scores do, so the candidates of the whole segment fit the buffer and the one
    // selection at the end is all there is (without it the first 4,096 scores all pass, each through the shared counter,
    // and a selection is needed as soon as they have).  Data that defeats the estimate only brings the cut-backs back.
    constexpr int kPre = 4 * kSelPerThread;
    if (topk <= kSelThreads && k1 - k0 >= (int64_t)kPre * kSelThreads) {
        uint32_t best = 0u;
#pragma unroll
        for (int j = 0; j < kPre; ++j) {
            const uint32_t o = ordered_bits(__ldg(src + k0 + j * kSelThreads + threadIdx.x));
            best = o > best ? o : best;
        }
        buf[threadIdx.x] = (unsigned long long)best;
        block_sort_desc(buf, kSelThreads);
        const unsigned long long t0 = buf[topk - 1] << 32;   // below every key that carries this score
        __syncthreads();
        if (threadIdx.x == 0) thr = t0;
        __syncthreads();
    }
    // The scores of the next batch are already on their way while this one is filtered, and the common
    // case (nothing to prune) costs one barrier per batch.
    float nxt[kSelPerThread];
#pragma unroll
    for (int j = 0; j < kSelPerThread; ++j) {
        const int64_t key = k0 + j * kSelThreads + threadIdx.x;
        nxt[j] = key < k1 ? __ldcs(src + key) : 0.f;
    }
    for (int64_t kb = k0; kb < k1; kb += kSelBatch) {
        float v[kSelPerThread];
#pragma unroll
        for (int j = 0; j < kSelPerThread; ++j) v[j] = nxt[j];
        if (kb + kSelBatch < k1) {
#pragma unroll
            for (int j = 0; j < kSelPerThread; ++j) {
                const int64_t key = kb + kSelBatch + j * kSelThreads + threadIdx.x;
                nxt[j] = key < k1 ? __ldcs(src + key) : 0.f;
            }
        }
        // The test that nearly every score fails is one 32-bit compare of the score's sortable bits with the upper half
        // of the threshold; the 64-bit key, the bound check and the append are behind it.
        const unsigned long long t = thr;
        const uint32_t t_hi = (uint32_t)(t >> 32);
#pragma unroll
        for (int j = 0; j < kSelPerThread; ++j) {
            const uint32_t o = ordered_bits(v[j]);
            if (o >= t_hi) {
                const int64_t key = kb + j * kSelThreads + threadIdx.x;
                const unsigned long long ck = ((unsigned long long)o << 32) | (unsigned long long)(0xffffffffu - (row0 + (uint32_t)key));
                if (key < k1 && ck > t) buf[atomicAdd(&cnt, 1)] = ck;
            }
        }
        // Each thread tests the count it sees after its own appends; the thread that appended last sees the
        // final count, so the OR over the block is the test on the final count and is the same for everyone.
        if (__syncthreads_or(cnt + kSelBatch > kSelCap)) {
            const int c = cnt;  // stable: every thread is in this branch
            if (c > topk) {
                const unsigned long long kth = block_select_topk(buf, c, topk, hist, scratch);
                if (threadIdx.x == 0) { cnt = topk; thr = kth; }
            }
            __syncthreads();
        }
    }
    __syncthreads();
    int c = cnt;
    if (c > topk) { block_select_topk(buf, c, topk, hist, scratch); c = topk; }
    __syncthreads();
    for (int i = c + threadIdx.x; i < k2; i += kSelThreads) buf[i] = 0ull;
    block_sort_desc(buf, k2);
    unsigned long long* dst = part + (((size_t)g * lists_per_group + list_base + seg) * qpg + qi) * topk;
    for (int i = threadIdx.x; i < topk; i += kSelThreads) dst[i] = buf[i];
}

// Candidate mode, after a scoring pass: one block per (query, group) takes the query's candidate list (and, mode 0,
// its best list so far), keeps the k best as sorted keys in best[group][query][topk], raises the query's threshold
// to the k-th best score (once there are k) and empties the list.  Mode 1 (the sampled pass that only finds a
// first threshold) leaves the best list alone: its keys will be scored again by the full pass.
__global__ void __launch_bounds__(256)
select_candidates_kernel(const unsigned long long* __restrict__ cand, unsigned int* __restrict__ cnt, int64_t cap,
                         unsigned long long* __restrict__ best, float* __restrict__ thr, int qpg, int topk, int k2, int mode) {
    __shared__ __align__(16) unsigned long long a[kSelCap];
    __shared__ int hist[256];
    __shared__ int scratch[4];
    __shared__ int count;
    __shared__ unsigned long long cut;   // keys at or below it cannot be among the k best any more
    const int64_t q = (int64_t)blockIdx.y * qpg + blockIdx.x;
    const unsigned long long* list = cand + q * cap;
    unsigned long long* mine = best + q * topk;
    const int64_t n = min((int64_t)cnt[q], cap);
    if (threadIdx.x == 0) { count = 0; cut = 0ull; }
    __syncthreads();
    if (mode == 0) {
        for (int i = threadIdx.x; i < topk; i += blockDim.x) {
            const unsigned long long v = mine[i];
            if (v != 0ull) a[atomicAdd(&count, 1)] = v;
        }
        __syncthreads();
    }
    constexpr int kBatch = 2048;
    for (int64_t base = 0; base < n; base += kBatch) {
        if (count + kBatch > kSelCap) {  // uniform: count only changes between barriers
            const int c = count;
            __syncthreads();
            if (c > topk) {
                const unsigned long long kth = block_select_topk(a, c, topk, hist, scratch);
                if (threadIdx.x == 0) { count = topk; cut = kth; }
            }
            __syncthreads();
        }
        const unsigned long long t = cut;
        const int64_t end = base + kBatch < n ? base + kBatch : n;
        for (int64_t i = base + threadIdx.x; i < end; i += blockDim.x) {
            const unsigned long long v = __ldcs(list + i);
            if (v > t) a[atomicAdd(&count, 1)] = v;      // also drops the empty slots
        }
        __syncthreads();
    }
    const int c = count;
    const int keep = c < topk ? c : topk;
    if (keep < c) block_select_topk(a, c, keep, hist, scratch);
    __syncthreads();
    for (int i = keep + threadIdx.x; i < k2; i += blockDim.x) a[i] = 0ull;
    block_sort_desc(a, k2);
    if (mode == 0)
        for (int i = threadIdx.x; i < topk; i += blockDim.x) mine[i] = a[i];
    if (threadIdx.x == 0) {
        if (keep == topk) thr[q] = unordered_bits((uint32_t)(a[topk - 1] >> 32));
        cnt[q] = 0u;
    }
}

// thresholds to -inf, best lists to empty, list lengths to `first_count` (what the sampled pass will leave in them; 0 without one)
__global__ void init_candidates_kernel(float* thr, unsigned int* cnt, unsigned long long* best, int64_t lists, int topk,
                                       unsigned int first_count) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < lists) { thr[i] = -CUDART_INF_F; cnt[i] = first_count; }
    if (i < lists * topk) best[i] = 0ull;
}

int pow2_at_least(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

template <int BITS, int QPAD, int DR>
int launch_score(const CUtensorMap& map, const ScoreTcArgs& args, int grid, cudaStream_t st) {
    const int sm = ScoreSmem<BITS, QPAD, DR>::total;
    if (args.fused) {
        TQ_CUDA_TRY(cudaFuncSetAttribute(score_tc_kernel<BITS, QPAD, DR, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm));
        score_tc_kernel<BITS, QPAD, DR, true><<<grid, ScoreThreads<QPAD>::kThreads, sm, st>>>(map, args); tq_count_launch();
        TQ_CUDA_TRY(cudaGetLastError());
        return TQ_OK;
    }
    TQ_CUDA_TRY(cudaFuncSetAttribute(score_tc_kernel<BITS, QPAD, DR, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm));
    score_tc_kernel<BITS, QPAD, DR, false><<<grid, ScoreThreads<QPAD>::kThreads, sm, st>>>(map, args); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

}  // namespace

#ifndef TQ_SCORE_PASS
#define TQ_SCORE_PASS 64     // queries per scoring launch at d <= 128 (32: the measurement build without passes of 64)
#endif

// ---- host-side planning ---------------------------------------------------------------------------
constexpr int64_t kChunkKeys = 1 << 22;     // keys per group scored into scratch at a time when only top-k is wanted
                                            // (2^20: 221 us per 1M keys and 32 queries, 2^21: 198, 2^23: 185; scratch 16 B x queries per key)
constexpr int64_t kSegLen = 65536;          // scores per selection block (top-100 call at 1,048,576 keys: 32,768 -> 214 us, 65,536 -> 204, 131,072 -> 213, 262,144 -> 241)

// prepared queries of one group in the scratch block: the largest of the passes (64 queries; 32 queries of d = 256)
constexpr size_t kPrepGroupMax = prep_group_bytes(64, 1) > prep_group_bytes(32, 2) ? prep_group_bytes(64, 1) : prep_group_bytes(32, 2);

struct ScoreTcPlan {
    int64_t chunk, nchunks, segs_per_chunk, lists_per_group;
    size_t prep_bytes, part_bytes, matrix_bytes, total;
    size_t off_prep, off_part, off_matrix;
};

static ScoreTcPlan plan_score(int groups, int qpg, int64_t keys_per_group, int topk, bool need_scratch_matrix) {
    ScoreTcPlan s{};
    s.chunk = keys_per_group < kChunkKeys ? keys_per_group : kChunkKeys;
    if (s.chunk < 1) s.chunk = 1;
    s.nchunks = (keys_per_group + s.chunk - 1) / s.chunk;
    if (s.nchunks < 1) s.nchunks = 1;
    s.segs_per_chunk = (s.chunk + kSegLen - 1) / kSegLen;
    s.lists_per_group = s.nchunks * s.segs_per_chunk;
    s.prep_bytes = ((size_t)groups * kPrepGroupMax + 255) & ~size_t(255);
    s.part_bytes = topk > 0 ? (((size_t)groups * s.lists_per_group * qpg * topk * 8) + 255) & ~size_t(255) : 0;
    s.matrix_bytes = (topk > 0 && need_scratch_matrix) ? (((size_t)groups * qpg * s.chunk * 4) + 255) & ~size_t(255) : 0;
    s.off_prep = 0;
    s.off_part = s.prep_bytes;
    s.off_matrix = s.off_part + s.part_bytes;
    s.total = s.off_matrix + s.matrix_bytes;
    return s;
}

// Candidate mode (top-k without any score matrix) for key sets of several chunks: per query a threshold, a counter,
// a best-k list and a candidate list that can hold every key of one chunk (so no list can overflow, whatever the data).
constexpr int64_t kCandChunk = 1 << 21;     // keys per group per scoring launch
constexpr int64_t kSampleEvery = 64;        // the first threshold comes from every 64th tile of the first chunk

struct CandPlan {
    int64_t chunk, nchunks, cand_cap, lists;
    size_t off_thr, off_cnt, off_best, off_cand, total;
};

static CandPlan plan_candidates(int groups, int qpg, int64_t keys_per_group, int topk) {
    CandPlan s{};
    auto pad = [](size_t b) { return (b + 255) & ~size_t(255); };
    s.chunk = kCandChunk;
    s.nchunks = (keys_per_group + s.chunk - 1) / s.chunk;
    s.cand_cap = s.chunk;
    s.lists = (int64_t)groups * qpg;
    s.off_thr = pad((size_t)groups * kPrepGroupMax);
    s.off_cnt = s.off_thr + pad((size_t)s.lists * 4);
    s.off_best = s.off_cnt + pad((size_t)s.lists * 4);
    s.off_cand = s.off_best + pad((size_t)s.lists * (topk > 0 ? topk : 1) * 8);
    s.total = s.off_cand + pad((size_t)s.lists * s.cand_cap * 8);
    return s;
}

// Candidate mode pays a sampled pass and two selections up front; it wins once a key set spans several chunks
// (measured: 8,388,608 keys x 32 queries 158 us per 1,048,576 keys against 188 us through a scratch matrix; a single
// chunk of 1,048,576 keys 307 us against 224 us).
static bool use_candidates(const float* scores, int topk, int64_t keys_per_group) {
    return scores == nullptr && topk > 0 && keys_per_group > 2 * kCandChunk;
}

int64_t tq_score_tc_scratch(int groups, int qpg, int64_t keys_per_group, int topk) {
    const size_t a = plan_score(groups, qpg, keys_per_group, topk, true).total;
    const size_t b = use_candidates(nullptr, topk, keys_per_group) ? plan_candidates(groups, qpg, keys_per_group, topk).total : 0;
    return (int64_t)(a > b ? a : b);
}

int tq_merge_keys_launch(const unsigned long long* part, int lists, int qpg, int groups, int topk, int64_t idx_base,
                         float* top_scores, int64_t* top_idx, cudaStream_t st);

int tq_launch_score_tc(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes,
                       const uint32_t* signs, const float* rnorms, const float* norms, int64_t keys_per_group,
                       float* scores, int topk, float* top_scores, int64_t* top_idx, int64_t idx_base, void* scratch,
                       size_t scratch_bytes, cudaStream_t st, int64_t group_rows) {
    TqRange range("tq.score.tensor_core");
    if (group_rows <= 0) group_rows = keys_per_group;
    const bool candidates = use_candidates(scores, topk, keys_per_group);
    const ScoreTcPlan sp = plan_score(groups, qpg, keys_per_group, topk, scores == nullptr);
    const CandPlan cp = plan_candidates(groups, qpg, keys_per_group, topk);
    const size_t need = candidates ? cp.total : sp.total;
    if (!scratch || scratch_bytes < need)
        return tq_fail(TQ_ERR_SCRATCH_TOO_SMALL, "score scratch: need %zu bytes, got %zu", need, scratch_bytes);
    unsigned char* sc = static_cast<unsigned char*>(scratch);
    unsigned char* prep = sc;     // both layouts start with the prepared queries
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->device);
    const int bits = p->dev.bits;
    float* thr = reinterpret_cast<float*>(sc + cp.off_thr);
    unsigned int* cnt = reinterpret_cast<unsigned int*>(sc + cp.off_cnt);
    unsigned long long* best = reinterpret_cast<unsigned long long*>(sc + cp.off_best);
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(sc + cp.off_cand);

    // One scoring launch per pass of at most 64 queries (32 at d = 256) over keys [key_off, key_off + key_cnt) of every group (every
    // tile_stride-th tile of them), into a matrix (mat != null) or into the candidate lists.
    // `prepared`: the scratch block still holds the prepared queries of the only pass (a call of several launches
    // over the same queries prepares them once).
    auto score_passes = [&](int64_t key_off, int64_t key_cnt, int tile_stride, float* mat, int64_t row_stride, bool prepared) -> int {
        const int64_t group_stride = (int64_t)qpg * row_stride;
        // A pass of 64 expands the keys once for queries that would otherwise take two passes (64 queries x 1,048,576
        // keys: 171 us against 219 us in two passes of 32; 33 queries: 168 against 205 us in passes of 32 and 16).
        const int pass = p->dev.d == 256 ? 32 : TQ_SCORE_PASS;
        for (int q0 = 0; q0 < qpg; q0 += pass) {
            const int nq = qpg - q0 < pass ? qpg - q0 : pass;
            const int qpad = nq <= 16 ? 16 : nq <= 32 ? 32 : 64;
            if (prepared && qpg <= pass) {
                // nothing to do
            } else if (p->dev.d == 256) {
                score_prep256_kernel<<<dim3(qpad, groups), 1024, 0, st>>>(p->dev, q, qpg, q0, nq, qpad, prep); tq_count_launch();
            } else {
                TQ_CUDA_TRY(cudaFuncSetAttribute(score_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmemBytes));
                score_prep_kernel<<<dim3(qpad, groups), 128, kPrepSmemBytes, st>>>(p->dev, q, qpg, q0, nq, qpad, prep); tq_count_launch();
            }
            TQ_CUDA_TRY(cudaGetLastError());
            ScoreTcArgs a{};
            a.codes = codes; a.signs = signs; a.rnorms = rnorms; a.norms = norms;
            a.prep = prep; a.codebook = p->dev.codebook;
            a.keys_per_group = group_rows; a.key_off = key_off; a.key_cnt = key_cnt;
            a.tile_stride = tile_stride;
            const int64_t tiles = (key_cnt + kTileKeys - 1) / kTileKeys;
            a.tiles_per_group = (tiles + tile_stride - 1) / tile_stride;
            a.total_tiles = a.tiles_per_group * groups;
            a.nq = nq;
            a.out_group_stride = group_stride; a.out_row_stride = row_stride;
            a.scores = mat ? mat + (int64_t)q0 * row_stride : nullptr;
            a.alpha = p->dev.alpha;
            a.norms_bulk = (groups == 1 || group_rows % 4 == 0) && key_off % 4 == 0 ? 1 : 0;   // 16-byte aligned tile starts
            a.fused = mat ? 0 : (tile_stride > 1 ? 2 : 1);    // 2: the sampled pass
            a.qpg_total = qpg; a.q0 = q0;
            a.thr = thr; a.cnt = cnt; a.cand = cand; a.cand_cap = cp.cand_cap;
            a.status = p->counters + 1;
            a.wait_kcycles = p->wait_kcycles;
#ifdef TQ_PROF
            a.prof = reinterpret_cast<long long*>(p->counters + 8);
#endif
            if (a.total_tiles == 0) continue;
            const int grid = (int)(a.total_tiles < sms ? a.total_tiles : sms);
            // Score tiles leave through a bulk tensor store when the matrix allows one: 16-byte aligned base and
            // row pitch.  Box = 128 keys x the queries of the pass x one group; extents clip ragged edges.
            CUtensorMap map;
            memset(&map, 0, sizeof(map));
            a.tile_store = 0;
            if (mat && (reinterpret_cast<uintptr_t>(a.scores) & 15u) == 0 && row_stride % 4 == 0 && key_cnt > 0 && tq_encode_tiled_fn()) {
                const cuuint64_t gdim[3] = {(cuuint64_t)key_cnt, (cuuint64_t)nq, (cuuint64_t)groups};
                const cuuint64_t gstride[2] = {(cuuint64_t)row_stride * 4, (cuuint64_t)group_stride * 4};
                const cuuint32_t box[3] = {(cuuint32_t)kTileKeys, (cuuint32_t)qpad, 1};
                const cuuint32_t estr[3] = {1, 1, 1};
                const CUresult cr = tq_encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, a.scores, gdim, gstride, box, estr,
                                                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (cr == CUDA_SUCCESS) a.tile_store = 1;
            }
            int r = TQ_ERR_UNSUPPORTED;
            tq_timer_mark(p, 1, 0, st);
#define TQ_SC(B)                                                                                             \
    case B:                                                                                                  \
        if (p->dev.d == 64) r = qpad == 16 ? launch_score<B, 16, 64>(map, a, grid, st) : qpad == 32 ? launch_score<B, 32, 64>(map, a, grid, st)       \
                                                                                                   : launch_score<B, 64, 64>(map, a, grid, st);      \
        else if (p->dev.d == 256) r = qpad == 16 ? launch_score<B, 16, 256>(map, a, grid, st) : launch_score<B, 32, 256>(map, a, grid, st);          \
        else r = qpad == 16 ? launch_score<B, 16, 128>(map, a, grid, st) : qpad == 32 ? launch_score<B, 32, 128>(map, a, grid, st)                   \
                                                                                      : launch_score<B, 64, 128>(map, a, grid, st);                  \
        break;
            switch (bits) { TQ_SC(1) TQ_SC(2) TQ_SC(3) TQ_SC(4) }
#undef TQ_SC
            tq_timer_mark(p, 1, 1, st);
            if (r != TQ_OK) return r == TQ_ERR_UNSUPPORTED ? tq_fail(r, "no tensor-core scoring kernel for bits=%d", bits) : r;
        }
        return TQ_OK;
    };

    if (!candidates) {
        // A score matrix exists: the caller's (everything scored in one go) or, when only the top-k is wanted, a scratch
        // matrix per chunk of keys; the top-k is selected from it segment by segment and the lists are merged at the end.
        unsigned long long* part = reinterpret_cast<unsigned long long*>(sc + sp.off_part);
        float* tmp = reinterpret_cast<float*>(sc + sp.off_matrix);
        if (topk > 0) TQ_CUDA_TRY(cudaMemsetAsync(part, 0, sp.part_bytes, st));  // zero = empty slot
        const int64_t nchunks = scores ? 1 : sp.nchunks;
        for (int64_t c = 0; c < nchunks; ++c) {
            const int64_t key_off = scores ? 0 : c * sp.chunk;
            int64_t key_cnt = scores ? keys_per_group : keys_per_group - key_off;
            if (!scores && key_cnt > sp.chunk) key_cnt = sp.chunk;
            float* mat = scores ? scores : tmp;
            const int64_t row_stride = scores ? keys_per_group : sp.chunk;
            const int rc = score_passes(key_off, key_cnt, 1, mat, row_stride, c > 0);
            if (rc != TQ_OK) return rc;
            if (topk > 0) {
                const int64_t segs = (key_cnt + kSegLen - 1) / kSegLen;
                // lists of chunk c occupy slots [c*segs_per_chunk, ...); unused slots stay zero (= empty)
                topk_rows_kernel<<<dim3((unsigned)segs, (unsigned)(groups * qpg)), kSelThreads, 0, st>>>(
                    mat, row_stride, (int64_t)qpg * row_stride, qpg, key_cnt, kSegLen, group_rows, key_off, topk, pow2_at_least(topk),
                    (int)sp.lists_per_group, (int)(c * sp.segs_per_chunk), part); tq_count_launch();
                TQ_CUDA_TRY(cudaGetLastError());
            }
        }
        if (topk > 0)
            return tq_merge_keys_launch(part, (int)sp.lists_per_group, qpg, groups, topk, idx_base, top_scores, top_idx, st);
        return TQ_OK;
    }

    // Top-k only over several chunks.  Every query keeps a threshold (a lower bound of its k-th best score so far); the
    // scoring kernel appends the scores that reach it to the query's candidate list and nothing else leaves the kernel;
    // after every launch the lists are folded into the running best-k lists, which raises the thresholds for the next
    // chunk.  The first threshold comes from scoring every 64th tile of the first chunk with the threshold at -inf: the
    // k-th best of a subset is a lower bound of the k-th best of the whole, so the full pass that follows loses nothing
    // and appends only about 64 k scores per query.
    const int k2 = pow2_at_least(topk);
    const int64_t cells = cp.lists * topk;
    const int64_t tiles0 = (cp.chunk + kTileKeys - 1) / kTileKeys;
    const int64_t sample_tiles = (tiles0 + kSampleEvery - 1) / kSampleEvery;
    init_candidates_kernel<<<(unsigned)((cells + 255) / 256), 256, 0, st>>>(thr, cnt, best, cp.lists, topk,
                                                                            (unsigned int)(sample_tiles * kTileKeys)); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    auto select = [&](int mode) -> int {
        select_candidates_kernel<<<dim3((unsigned)qpg, (unsigned)groups), 256, 0, st>>>(cand, cnt, cp.cand_cap, best, thr, qpg, topk, k2, mode);
        tq_count_launch();
        TQ_CUDA_TRY(cudaGetLastError());
        return TQ_OK;
    };
    for (int64_t c = 0; c < cp.nchunks; ++c) {
        const int64_t key_off = c * cp.chunk;
        int64_t key_cnt = keys_per_group - key_off;
        if (key_cnt > cp.chunk) key_cnt = cp.chunk;
        if (c == 0) {
            int rc = score_passes(key_off, key_cnt, (int)kSampleEvery, nullptr, 0, false);
            if (rc != TQ_OK) return rc;
            rc = select(1);
            if (rc != TQ_OK) return rc;
        }
        int rc = score_passes(key_off, key_cnt, 1, nullptr, 0, true);
        if (rc != TQ_OK) return rc;
        rc = select(0);
        if (rc != TQ_OK) return rc;
    }
    return tq_merge_keys_launch(best, 1, qpg, groups, topk, idx_base, top_scores, top_idx, st);
}
