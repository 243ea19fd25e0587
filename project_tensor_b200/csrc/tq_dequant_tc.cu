// Tensor-core dequantize for d = 128 on B200: TurboQuantMSE.dequantize and TurboQuantProd.dequantize
// (_quant.py:238-242,251-254 and 317-332).
//
//   MSE :  x~ = norm * ( codebook[codes] . R )
//   Prod:  x~ = norm * ( codebook[codes] . R  +  alpha * rnorm * (signs . S) ),  alpha = sqrt(pi/2) / d
//
// Both are contractions over the 128 coordinates with the 128 keys of a tile on the M side and the 128
// output coordinates on the N side.  Operands are fp16 hi + lo pairs (three products per contraction, fp32
// accumulate), which keeps the result within about 1e-7 relative of the float32 reference arithmetic.
// For Prod the per-key factor alpha * rnorm is folded into the sign operand (+-beta, split hi/lo, exact),
// so that both contractions add into one accumulator.  Per tile:
//
//   bulk copy (1 thread)   packed codes (and sign words) of 128 keys -> smem ring
//   expanders (8 warps)    one thread per half key: codes -> (hi, lo) half2 pairs through a lane-replicated
//                          pair lookup table, signs -> +-beta pairs; tcgen05.st into a ring of four
//                          64-column operand slots in tensor memory (C_hi, C_lo [, B_hi, B_lo] of
//                          successive tiles)
//   MMA (1 thread)         operand by operand: C_hi x (Rt_hi, Rt_lo), C_lo x Rt_hi [, B_hi x (St_hi, St_lo),
//                          B_lo x St_hi], N = 128, accumulators double-buffered
//   epilogue (8 warps)     two threads per key: tcgen05.ld, times norm * 2^-20, then through a staging block in
//                          shared memory so that every global store instruction writes whole 128-byte lines
//
// Every wait is bounded; a wait that runs out sets the plan's status word and the kernel drains.
#include "tq_common.cuh"
#include "tq_ptx.cuh"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <vector>

namespace {

using namespace tqptx;

constexpr int D = 128;   // width of the operand layouts; vectors of d = 64 use their lower half
constexpr int kTileKeys = 128;
constexpr int kFirstExpWarp = 2;
constexpr int kFirstEpiWarp = 10;
constexpr int kThreads = 18 * 32;
constexpr int kSlots = 4;
constexpr float kCentScale = 1024.f;   // centroids  -> A operand
constexpr float kRotScale = 1024.f;    // rotation   -> B operand
constexpr float kBetaScale = 65536.f;  // alpha * rnorm -> A operand
constexpr float kProjScale = 16.f;     // projection -> B operand (kBetaScale * kProjScale = kCentScale * kRotScale)
constexpr float kOutScale = 1.f / (kCentScale * kRotScale);
constexpr int kMatBytes = D * D * 2;   // one fp16 operand matrix

struct DequantArgs {
    const uint32_t* codes;
    const uint32_t* signs;
    const float* rnorms;
    const float* norms;
    const unsigned char* bmat;   // [Rt_hi | Rt_lo | St_hi | St_lo], interleaved core-matrix layout
    const float* codebook;
    float alpha;
    int64_t n, ntiles;
    float* out;                  // reconstructions [n][d]; or, in pair mode, scores [n]
    const float* pair_q;         // pair mode: one query row per key, [n][d]
    unsigned long long* status;
    int wait_kcycles;            // limit of one bounded wait, in units of 1024 cycles
};

enum {
    DB_K_FULL = 0,     // [8]
    DB_K_EMPTY = 8,    // [8]
    DB_A_FULL = 16,    // [4]
    DB_A_EMPTY = 20,   // [4]
    DB_D_FULL = 24,    // [2]
    DB_D_EMPTY = 26,   // [2]
    DB_COUNT = 28
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld32_(uint32_t taddr, uint32_t (&v)[32]) { tmem_ld32(taddr, v); }

template <int BITS, bool PROD, int DR>
struct DqSmem {
    static constexpr int kLutEntries = 1 << (2 * BITS);
    static constexpr int kLutBytes = kLutEntries * 32 * 8;
    static constexpr int kCodeRowBytes = DR * BITS / 8;
    static constexpr int kSignRowBytes = DR / 8;
    static constexpr int kRowExtra = PROD ? kSignRowBytes : 0;   // sign words
    static constexpr int kStageBytes = kTileKeys * (kCodeRowBytes + kRowExtra);
    static constexpr int kNumB = PROD ? 4 : 2;
    static constexpr int kStages = PROD ? 4 : 6;
    static constexpr int kOutRowBytes = 36 * 4;                   // 32 floats of a row + padding against bank conflicts
    static constexpr int kOutWarpBytes = 32 * kOutRowBytes;       // staging block of one epilogue warp
    static constexpr int off_lut = 0;
    static constexpr int off_b = off_lut + kLutBytes;
    static constexpr int off_ring = off_b + kNumB * kMatBytes;
    static constexpr int off_out = off_ring + kStages * kStageBytes;
    static constexpr int off_misc = off_out + 8 * kOutWarpBytes;
    static constexpr int off_pair = off_misc + 512 + 128;           // pair mode: partial dot products [2 tiles][128]
    static constexpr int total = off_pair + 2 * kTileKeys * 4;
    static_assert(total <= 227 * 1024, "shared memory plan");
};

// PAIR: instead of storing the reconstruction, every key's row is multiplied with the query row of the same
// index and summed: attention_score with one query per key (_quant.py:342-358), which equals q . dequantize(key).
template <int BITS, bool PROD, int DR, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
dequant_tc_kernel(const DequantArgs a) {
    static_assert(DR == 128 || DR == 64, "written for d = 128 and d = 64");
    // d = 64: the expander warps and the epilogue warps of the upper half idle, the contractions stop after
    // DR / 16 k-blocks and cover N = DR output coordinates
    constexpr int kHalves = DR / 64;
    using L = DqSmem<BITS, PROD, DR>;
    constexpr int kStages = L::kStages;
    constexpr int kOps = PROD ? 4 : 2;   // operands per tile: C_hi, C_lo [, B_hi, B_lo]
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const uint32_t smem_base = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::off_misc);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + DB_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; ++i) { mbar_init(BAR(DB_K_FULL + i), 1); mbar_init(BAR(DB_K_EMPTY + i), 4 * kHalves); }
        for (int i = 0; i < kSlots; ++i) { mbar_init(BAR(DB_A_FULL + i), 4 * kHalves); mbar_init(BAR(DB_A_EMPTY + i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(BAR(DB_D_FULL + i), 1); mbar_init(BAR(DB_D_EMPTY + i), 4 * kHalves); }
        abort_flag[0] = 0;
        abort_flag[1] = a.wait_kcycles;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {   // pair lookup table: entry e = (code0 | code1 << BITS) -> (half2 hi(c0), hi(c1)), (half2 lo(c0), lo(c1)),
        // one copy per lane so that the lookups of a warp never collide on a bank
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
    {   // operand matrices: global -> smem, once per CTA
        const uint4* src = reinterpret_cast<const uint4*>(a.bmat);
        uint4* dst = reinterpret_cast<uint4*>(smem + L::off_b);
        for (int i = threadIdx.x; i < L::kNumB * kMatBytes / 16; i += kThreads) dst[i] = __ldg(src + i);
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

    const int64_t my_tiles = a.ntiles > (int64_t)blockIdx.x ? (a.ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(DR >> 3) << 17) | ((uint32_t)(kTileKeys >> 4) << 24);
    constexpr uint32_t kSlotCols = 64;
    constexpr uint32_t kColD = kSlots * kSlotCols;   // two accumulators of 128 columns behind the operand ring

    if (warp == 0) {
        // ---- bulk-copy producer -----------------------------------------------------------------
        if (lane == 0) {
            int64_t issued = 0;
            for (int64_t i = 0; i < my_tiles; ++i) {
                const int64_t tile = blockIdx.x + i * gridDim.x;
                const int s = (int)(i % kStages);
                if (!mbar_wait(BAR(DB_K_EMPTY + s), (uint32_t)((i / kStages) & 1) ^ 1u, abort_flag)) break;
                int64_t valid = a.n - tile * kTileKeys;
                if (valid > kTileKeys) valid = kTileKeys;
                const int64_t row0 = tile * kTileKeys;
                const uint32_t cb = (uint32_t)valid * L::kCodeRowBytes;
                const uint32_t dst = smem_base + L::off_ring + s * L::kStageBytes;
                unsigned char* stage = smem + L::off_ring + s * L::kStageBytes;
                const unsigned char* csrc = reinterpret_cast<const unsigned char*>(a.codes) + row0 * L::kCodeRowBytes;
                // a ragged last tile of 8- or 24-byte rows need not end on a 16-byte multiple: the bulk copies take
                // the multiple, plain loads the few bytes behind it
                copy_tail_words(stage, csrc, cb);
                if (PROD) {
                    const uint32_t sb = (uint32_t)valid * L::kSignRowBytes;
                    const unsigned char* ssrc = reinterpret_cast<const unsigned char*>(a.signs) + row0 * L::kSignRowBytes;
                    copy_tail_words(stage + kTileKeys * L::kCodeRowBytes, ssrc, sb);
                    mbar_arrive_expect_tx(BAR(DB_K_FULL + s), (cb & ~15u) + (sb & ~15u));
                    if (cb & ~15u) bulk_load(dst, csrc, cb & ~15u, BAR(DB_K_FULL + s));
                    if (sb & ~15u) bulk_load(dst + kTileKeys * L::kCodeRowBytes, ssrc, sb & ~15u, BAR(DB_K_FULL + s));
                } else {
                    mbar_arrive_expect_tx(BAR(DB_K_FULL + s), cb & ~15u);
                    if (cb & ~15u) bulk_load(dst, csrc, cb & ~15u, BAR(DB_K_FULL + s));
                }
                issued = i + 1;
            }
            if (*abort_flag) {
                // copies armed above may still be on their way into this block's shared memory
                for (int64_t ii = issued > kStages ? issued - kStages : 0; ii < issued; ++ii)
                    mbar_drain(BAR(DB_K_FULL + (int)(ii % kStages)), (uint32_t)((ii / kStages) & 1));
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer --------------------------------------------------------------------------
        // The whole warp walks the loop and waits; one elected lane issues from warp-uniform operands.
        {
            const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
            const uint32_t lbo = 128, sbo = (D / 8) * 128;
            const uint32_t b0 = smem_base + L::off_b;
            const uint64_t d_rhi = make_smem_desc(b0, lbo, sbo), d_rlo = make_smem_desc(b0 + kMatBytes, lbo, sbo);
            const uint64_t d_shi = make_smem_desc(b0 + 2 * kMatBytes, lbo, sbo), d_slo = make_smem_desc(b0 + 3 * kMatBytes, lbo, sbo);
            (void)d_shi; (void)d_slo;
            for (int64_t i = 0; i < my_tiles; ++i) {
                const int b = (int)(i & 1);
                const uint32_t par2 = (uint32_t)((i >> 1) & 1);
                if (!warp_wait(BAR(DB_D_EMPTY + b), par2 ^ 1u, abort_flag)) break;
                const uint32_t acc = tm + kColD + b * D;
                bool ok = true;
#pragma unroll
                for (int op = 0; op < kOps; ++op) {              // 0: C_hi, 1: C_lo, 2: B_hi, 3: B_lo
                    const int64_t n = (int64_t)kOps * i + op;
                    const int slot = (int)(n & (kSlots - 1));
                    if (!warp_wait(BAR(DB_A_FULL + slot), (uint32_t)((n / kSlots) & 1), abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t aop = tm + slot * kSlotCols;
                    const uint64_t bh = op < 2 ? d_rhi : d_shi, bl = op < 2 ? d_rlo : d_slo;
                    if (elect_one()) {
                        if (op == 0) mma_ts_first(acc, aop, bh, kIdesc); else mma_ts_acc(acc, aop, bh, kIdesc);
                        if ((op & 1) == 0) mma_ts_acc(acc, aop, bl, kIdesc);   // hi operand also meets the lo matrix
#pragma unroll 1
                        for (int kb = 1; kb < DR / 16; ++kb) {
                            // the start-address field counts 16-byte units: one k-block (two core matrices) further
                            const uint64_t step = (uint64_t)(kb * 2 * lbo >> 4);
                            mma_ts_acc(acc, aop + kb * 8, bh + step, kIdesc);
                            if ((op & 1) == 0) mma_ts_acc(acc, aop + kb * 8, bl + step, kIdesc);
                        }
                        mma_commit(BAR(DB_A_EMPTY + slot));
                    }
                    __syncwarp();
                }
                if (!ok) break;
                if (elect_one()) mma_commit(BAR(DB_D_FULL + b));
                __syncwarp();
            }
        }
    } else if (warp < kFirstEpiWarp) {
        // ---- expanders ----------------------------------------------------------------------------
        const int half = (warp - kFirstExpWarp) >> 2;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint2* lut_lane = reinterpret_cast<const uint2*>(smem + L::off_lut) + lane;
        constexpr int kHalfWords = 2 * BITS;  // code words of 64 coordinates
        constexpr uint32_t kPairMask = (1u << (2 * BITS)) - 1u;
        // residual norm of this thread's key, fetched a tile ahead of its use (Prod)
        float rn_next = 0.f;
        if (PROD && my_tiles > 0) {
            const int64_t r0 = (int64_t)blockIdx.x * kTileKeys + row;
            rn_next = r0 < a.n ? __ldg(a.rnorms + r0) : 0.f;
        }
        for (int64_t i = 0; i < (half < kHalves ? my_tiles : 0); ++i) {
            const int s = (int)(i % kStages);
            const float rn = rn_next;
            if (PROD && i + 1 < my_tiles) {
                const int64_t r1 = (blockIdx.x + (i + 1) * gridDim.x) * kTileKeys + row;
                rn_next = r1 < a.n ? __ldg(a.rnorms + r1) : 0.f;
            }
            bool fail = !mbar_wait(BAR(DB_K_FULL + s), (uint32_t)((i / kStages) & 1), abort_flag);
            uint32_t w[kHalfWords + 1], sw[2] = {0u, 0u};
            {
                const unsigned char* stage = smem + L::off_ring + s * L::kStageBytes;
                const volatile uint32_t* cw = reinterpret_cast<const volatile uint32_t*>(stage + row * L::kCodeRowBytes) + half * kHalfWords;
#pragma unroll
                for (int k = 0; k < kHalfWords; ++k) w[k] = fail ? 0u : cw[k];
                w[kHalfWords] = 0;
                if (PROD) {
                    const volatile uint32_t* sg = reinterpret_cast<const volatile uint32_t*>(stage + kTileKeys * L::kCodeRowBytes + row * L::kSignRowBytes) + half * 2;
                    sw[0] = fail ? 0u : ~sg[0];   // a set bit now means a negative sign
                    sw[1] = fail ? 0u : ~sg[1];
                }
            }
            __threadfence_block();   // every lane's loads from the stage are performed before the stage is released
            __syncwarp();
            if (lane == 0 && !fail) mbar_arrive(BAR(DB_K_EMPTY + s));
            uint32_t hi[2][16], lo[2][16];
#pragma unroll
            for (int sb = 0; sb < 2; ++sb)
#pragma unroll
                for (int p = 0; p < 16; ++p) {
                    const int pair = sb * 16 + p;
                    const int bit = pair * 2 * BITS, wi = bit >> 5, sh = bit & 31;
                    uint32_t e;
                    if (sh + 2 * BITS <= 32) e = (w[wi] >> sh) & kPairMask;
                    else e = __funnelshift_r(w[wi], w[wi + 1], sh) & kPairMask;
                    const uint2 v = lut_lane[e * 32];
                    hi[sb][p] = v.x;
                    lo[sb][p] = v.y;
                }
            // beta = alpha * rnorm as fp16 hi + lo, both halves of a pair alike; the signs flip bit 15 / 31
            uint32_t bh2 = 0u, bl2 = 0u;
            if (PROD) {
                const float beta = a.alpha * rn * kBetaScale;
                const __half bh = __float2half_rn(beta);
                const __half bl = __float2half_rn(beta - __half2float(bh));
                const uint32_t bhu = (uint32_t)__half_as_ushort(bh), blu = (uint32_t)__half_as_ushort(bl);
                bh2 = bhu | (bhu << 16);
                bl2 = blu | (blu << 16);
            }
#pragma unroll
            for (int op = 0; op < kOps; ++op) {
                const int64_t n = (int64_t)kOps * i + op;
                const int slot = (int)(n & (kSlots - 1));
                if (!mbar_wait(BAR(DB_A_EMPTY + slot), (uint32_t)((n / kSlots) & 1) ^ 1u, abort_flag)) fail = true;
                tc_fence_after();
                const uint32_t abase = tmem + lane_addr + slot * kSlotCols + half * 32;
#pragma unroll
                for (int sb = 0; sb < 2; ++sb) {
                    if (op == 0) tmem_st16(abase + sb * 16, hi[sb]);
                    else if (op == 1) tmem_st16(abase + sb * 16, lo[sb]);
                    else {
                        // sign word sb covers coordinates 32*sb .. 32*sb+31 of this half; pair p: bits p, 16+p
                        uint32_t sg[16];
                        const uint32_t pat = op == 2 ? bh2 : bl2;
#pragma unroll
                        for (int p = 0; p < 16; ++p) sg[p] = pat ^ ((sw[sb] << (15 - p)) & 0x80008000u);
                        tmem_st16(abase + sb * 16, sg);
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(DB_A_FULL + slot));
            }
        }
    } else {
        // ---- epilogue: two threads per key, each one half of the output coordinates -----------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int colhalf = (warp - kFirstEpiWarp) >> 2;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        float nrm_next = 0.f;
        if (my_tiles > 0) {
            const int64_t r0 = (int64_t)blockIdx.x * kTileKeys + row;
            nrm_next = r0 < a.n ? __ldg(a.norms + r0) : 0.f;
        }
        for (int64_t i = 0; i < (colhalf < kHalves ? my_tiles : 0); ++i) {
            const int64_t tile = blockIdx.x + i * gridDim.x;
            const int b = (int)(i & 1);
            const uint32_t par2 = (uint32_t)((i >> 1) & 1);
            const float sc = nrm_next * kOutScale;
            if (i + 1 < my_tiles) {   // the norm of the next tile's key is fetched a tile ahead of its use
                const int64_t rn = (tile + gridDim.x) * kTileKeys + row;
                nrm_next = rn < a.n ? __ldg(a.norms + rn) : 0.f;
            }
            unsigned char* stg = smem + L::off_out + (warp - kFirstEpiWarp) * L::kOutWarpBytes;
            const int64_t row0 = tile * kTileKeys + quarter * 32;
            // pair mode: the warp's 32 x 32 block of query values, four rows x 128 bytes per load instruction;
            // the first block is requested before the wait for the accumulator
            float4 qv[8];
            auto fetch_q = [&](int ch) {
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int r = it * 4 + (lane >> 3), c4 = lane & 7;
                    qv[it] = row0 + r < a.n ? __ldg(reinterpret_cast<const float4*>(a.pair_q + (row0 + r) * DR + colhalf * 64 + ch * 32) + c4)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            };
            if (PAIR) fetch_q(0);
            // after a give-up nothing is written: the accumulator cannot be trusted
            const int64_t n_live = mbar_wait(BAR(DB_D_FULL + b), par2, abort_flag) ? a.n : 0;
            tc_fence_after();
            const uint32_t acc = tmem + lane_addr + kColD + b * D + colhalf * 64;
            uint32_t va[32], vb[32];
            tmem_ld32_(acc, va);
            tmem_ld32_(acc + 32, vb);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(DB_D_EMPTY + b));   // the accumulator is free again
            if (PAIR) {
                float dot = 0.f;
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int r = it * 4 + (lane >> 3), c4 = lane & 7;
                        *reinterpret_cast<float4*>(stg + r * L::kOutRowBytes + c4 * 16) = qv[it];
                    }
                    __syncwarp();
                    if (ch == 0) fetch_q(1);
                    const float4* mine = reinterpret_cast<const float4*>(stg + lane * L::kOutRowBytes);
                    const uint32_t* v = ch == 0 ? va : vb;
#pragma unroll
                    for (int m = 0; m < 8; ++m) {
                        const float4 qq = mine[m];
                        dot = fmaf(__uint_as_float(v[4 * m]), qq.x, dot);
                        dot = fmaf(__uint_as_float(v[4 * m + 1]), qq.y, dot);
                        dot = fmaf(__uint_as_float(v[4 * m + 2]), qq.z, dot);
                        dot = fmaf(__uint_as_float(v[4 * m + 3]), qq.w, dot);
                    }
                    __syncwarp();
                }
                // the two threads of a row add their halves through shared memory (buffer by tile parity)
                float* part = reinterpret_cast<float*>(smem + L::off_pair) + b * kTileKeys;
                if (kHalves == 2) {
                    if (colhalf == 1) part[row] = dot;
                    bar_sync(1 + quarter, 64);
                    if (colhalf == 0) dot += part[row];
                }
                const int64_t grow = tile * kTileKeys + row;
                if (colhalf == 0 && grow < n_live) a.out[grow] = dot * sc;
                continue;
            }
            // Through a per-warp staging block in shared memory, so that the global stores of a warp cover
            // whole 128-byte lines (four rows x 32 floats per instruction) instead of 16 bytes of 32 rows.
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                float4* mine = reinterpret_cast<float4*>(stg + lane * L::kOutRowBytes);
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    const uint32_t* v = ch == 0 ? va : vb;
                    mine[m] = make_float4(__uint_as_float(v[4 * m]) * sc, __uint_as_float(v[4 * m + 1]) * sc,
                                          __uint_as_float(v[4 * m + 2]) * sc, __uint_as_float(v[4 * m + 3]) * sc);
                }
                __syncwarp();
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int r = it * 4 + (lane >> 3), c4 = lane & 7;
                    const float4 val = *reinterpret_cast<const float4*>(stg + r * L::kOutRowBytes + c4 * 16);
                    if (row0 + r < n_live)
                        __stcs(reinterpret_cast<float4*>(a.out + (row0 + r) * DR + colhalf * 64 + ch * 32) + c4, val);
                }
                __syncwarp();
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------------------------
    if (*abort_flag) __nanosleep(20000);   // tensor instructions issued before the give-up may still be running
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.status, 3ull);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ---------------------------------------------------------------------------------------------
// d = 256: the transposed matrices (2 x 128 KB each) stream from L2
// ---------------------------------------------------------------------------------------------
// A tile is 128 keys.  The expanded centroids (fp16 hi / lo) fill both operand blocks of tensor memory (coordinates
// [128 I, 128 I + 128) in block I), the two accumulator blocks take the two halves J of the output coordinates, and the
// split transposed rotation comes as 32 chunks of 8 KB (chunk (J * 2 + I) * 8 + kb: 128 output coordinates x 16 input
// coordinates, hi then lo, K-major core matrices) through a ring, three tensor instructions per chunk.  TurboQuantProd
// runs a second phase on the same tile: the expanders overwrite the operand blocks with +-beta (beta = alpha * rnorm
// * 2^16, hi / lo), 32 chunks of the transposed projection follow, and the products add into the same accumulators.
// Warps: bulk copies of the packed keys, MMA, bulk copies of the chunks, 16 expanders (64 coordinates per thread),
// 8 epilogue warps (two threads per key and output half).
namespace dq256 {
constexpr int kD = 256;
constexpr int kChunkBytes = 8192;
constexpr int kBRing = 8;
constexpr int kKStages = 2;
constexpr int kExpWarps = 16, kEpiWarps = 8;
constexpr int kFirstExp = 3, kFirstEpi = kFirstExp + kExpWarps;
constexpr int kThreads256 = (3 + kExpWarps + kEpiWarps) * 32;
enum { K_FULL = 0, K_EMPTY = 2, B_FULL = 4, B_EMPTY = 12, A_FULL = 20, A_EMPTY = 21, D_FULL = 22, D_EMPTY = 24, N_BARS = 26 };
template <int BITS, bool PROD>
struct Smem {
    static constexpr int kLutBytes = (1 << (2 * BITS)) * 32 * 8;
    static constexpr int kCodeRowBytes = kD * BITS / 8;
    static constexpr int kSignRowBytes = kD / 8;
    static constexpr int kStageBytes = kTileKeys * (kCodeRowBytes + (PROD ? kSignRowBytes : 0));
    static constexpr int kOutRowBytes = 36 * 4;
    static constexpr int kOutWarpBytes = 32 * kOutRowBytes;
    static constexpr int off_lut = 0;
    static constexpr int off_b = off_lut + kLutBytes;
    static constexpr int off_ring = off_b + kBRing * kChunkBytes;
    static constexpr int off_out = off_ring + kKStages * kStageBytes;
    static constexpr int off_misc = off_out + kEpiWarps * kOutWarpBytes;
    static constexpr int total = off_misc + 512 + 128 + 128;    // + slack to align the base
    static_assert(total <= 227 * 1024, "shared memory plan");
};
}  // namespace dq256

template <int BITS, bool PROD>
__global__ void __launch_bounds__(dq256::kThreads256, 1)
dequant256_kernel(const DequantArgs a) {
    using namespace dq256;
    using L = dq256::Smem<BITS, PROD>;
    constexpr int kPhases = PROD ? 2 : 1;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const uint32_t smem_base = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::off_misc);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kKStages; ++i) { mbar_init(BAR(K_FULL + i), 1); mbar_init(BAR(K_EMPTY + i), kExpWarps); }
        for (int i = 0; i < kBRing; ++i) { mbar_init(BAR(B_FULL + i), 1); mbar_init(BAR(B_EMPTY + i), 1); }
        mbar_init(BAR(A_FULL), kExpWarps);
        mbar_init(BAR(A_EMPTY), 1);
        for (int j = 0; j < 2; ++j) { mbar_init(BAR(D_FULL + j), 1); mbar_init(BAR(D_EMPTY + j), kEpiWarps); }
        abort_flag[0] = 0;
        abort_flag[1] = a.wait_kcycles;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {   // pair lookup table, one copy per lane (see the d = 128 kernel)
        uint2* lut = reinterpret_cast<uint2*>(smem + L::off_lut);
        for (int i = threadIdx.x; i < (1 << (2 * BITS)) * 32; i += kThreads256) {
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
    const int64_t my_tiles = a.ntiles > (int64_t)blockIdx.x ? (a.ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(kTileKeys >> 4) << 24);
    constexpr int kABlock = 64;
    auto A_COL = [&](int i) { return (uint32_t)(i * 2 * kABlock); };
    auto ACC_COL = [&](int j) { return (uint32_t)(4 * kABlock + j * 128); };

    if (warp == 0) {
        // ---- packed keys -----------------------------------------------------------------------------
        if (lane == 0) {
            int64_t issued = 0;
            for (int64_t i = 0; i < my_tiles; ++i) {
                const int64_t tile = blockIdx.x + i * gridDim.x;
                const int s = (int)(i % kKStages);
                if (!mbar_wait(BAR(K_EMPTY + s), (uint32_t)((i / kKStages) & 1) ^ 1u, abort_flag)) break;
                int64_t valid = a.n - tile * kTileKeys;
                if (valid > kTileKeys) valid = kTileKeys;
                const int64_t row0 = tile * kTileKeys;
                const uint32_t cb = (uint32_t)valid * L::kCodeRowBytes;     // rows are multiples of 16 bytes at d = 256
                const uint32_t dst = smem_base + L::off_ring + s * L::kStageBytes;
                const unsigned char* csrc = reinterpret_cast<const unsigned char*>(a.codes) + row0 * L::kCodeRowBytes;
                if (PROD) {
                    const uint32_t sb = (uint32_t)valid * L::kSignRowBytes;
                    const unsigned char* ssrc = reinterpret_cast<const unsigned char*>(a.signs) + row0 * L::kSignRowBytes;
                    mbar_arrive_expect_tx(BAR(K_FULL + s), cb + sb);
                    bulk_load(dst, csrc, cb, BAR(K_FULL + s));
                    bulk_load(dst + kTileKeys * L::kCodeRowBytes, ssrc, sb, BAR(K_FULL + s));
                } else {
                    mbar_arrive_expect_tx(BAR(K_FULL + s), cb);
                    bulk_load(dst, csrc, cb, BAR(K_FULL + s));
                }
                issued = i + 1;
            }
            if (*abort_flag)
                for (int64_t ii = issued > kKStages ? issued - kKStages : 0; ii < issued; ++ii)
                    mbar_drain(BAR(K_FULL + (int)(ii % kKStages)), (uint32_t)((ii / kKStages) & 1));
        }
    } else if (warp == 2) {
        // ---- operand chunks: the same 32 (64) chunks for every tile -------------------------------------
        if (lane == 0) {
            int64_t g = 0;
            bool ok = true;
            for (int64_t i = 0; i < my_tiles && ok; ++i) {
                for (int c = 0; c < kPhases * 32; ++c, ++g) {
                    const int slot = (int)(g % kBRing);
                    if (!mbar_wait(BAR(B_EMPTY + slot), (uint32_t)(((g / kBRing) & 1) ^ 1), abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(BAR(B_FULL + slot), kChunkBytes);
                    bulk_load(smem_base + L::off_b + slot * kChunkBytes, a.bmat + (size_t)c * kChunkBytes, kChunkBytes, BAR(B_FULL + slot));
                }
            }
            if (*abort_flag)
                for (int64_t gg = g > kBRing ? g - kBRing : 0; gg < g; ++gg)
                    mbar_drain(BAR(B_FULL + (int)(gg % kBRing)), (uint32_t)((gg / kBRing) & 1));
        }
    } else if (warp == 1) {
        // ---- MMA issuer ---------------------------------------------------------------------------------
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
        int64_t g = 0, phase_n = 0;
        bool ok = true;
        for (int64_t i = 0; i < my_tiles && ok; ++i) {
            const uint32_t par = (uint32_t)(i & 1);
            for (int ph = 0; ph < kPhases && ok; ++ph, ++phase_n) {
                if (!warp_wait(BAR(A_FULL), (uint32_t)(phase_n & 1), abort_flag)) { ok = false; break; }
                for (int j = 0; j < 2 && ok; ++j) {
                    if (ph == 0 && !warp_wait(BAR(D_EMPTY + j), par ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t acc = tm + ACC_COL(j);
                    for (int c = 0; c < 16; ++c, ++g) {          // c = I * 8 + kb
                        const int slot = (int)(g % kBRing);
                        if (!warp_wait(BAR(B_FULL + slot), (uint32_t)((g / kBRing) & 1), abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t chunk = smem_base + L::off_b + slot * kChunkBytes;
                        const uint64_t d_hi = make_smem_desc(chunk, 128, 256), d_lo = make_smem_desc(chunk + kChunkBytes / 2, 128, 256);
                        const uint32_t a_hi = tm + A_COL(c >> 3) + (uint32_t)(c & 7) * 8, a_lo = a_hi + kABlock;
                        if (elect_one()) {
                            if (ph == 0 && c == 0) mma_ts_first(acc, a_hi, d_hi, kIdesc);
                            else mma_ts_acc(acc, a_hi, d_hi, kIdesc);
                            mma_ts_acc(acc, a_hi, d_lo, kIdesc);
                            mma_ts_acc(acc, a_lo, d_hi, kIdesc);
                            mma_commit(BAR(B_EMPTY + slot));
                            if (c == 15 && ph == kPhases - 1) mma_commit(BAR(D_FULL + j));
                        }
                        __syncwarp();
                    }
                }
                if (!ok) break;
                if (elect_one()) mma_commit(BAR(A_EMPTY));       // the operand blocks have been read
                __syncwarp();
            }
        }
    } else if (warp < kFirstEpi) {
        // ---- expanders: one thread per quarter key (64 coordinates) ---------------------------------------
        const int part = (warp - kFirstExp) >> 2;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint2* lut_lane = reinterpret_cast<const uint2*>(smem + L::off_lut) + lane;
        constexpr int kHalfWords = 2 * BITS;  // code words of 64 coordinates
        constexpr uint32_t kPairMask = (1u << (2 * BITS)) - 1u;
        int64_t phase_n = 0;
        for (int64_t i = 0; i < my_tiles; ++i) {
            const int64_t tile = blockIdx.x + i * gridDim.x;
            const int s = (int)(i % kKStages);
            float rn = 0.f;
            if (PROD) {
                const int64_t r0 = tile * kTileKeys + row;
                rn = r0 < a.n ? __ldg(a.rnorms + r0) : 0.f;
            }
            bool fail = !mbar_wait(BAR(K_FULL + s), (uint32_t)((i / kKStages) & 1), abort_flag);
            uint32_t w[kHalfWords + 1], sw[2] = {0u, 0u};
            {
                const unsigned char* stage = smem + L::off_ring + s * L::kStageBytes;
                const volatile uint32_t* cw = reinterpret_cast<const volatile uint32_t*>(stage + row * L::kCodeRowBytes) + part * kHalfWords;
#pragma unroll
                for (int k = 0; k < kHalfWords; ++k) w[k] = fail ? 0u : cw[k];
                w[kHalfWords] = 0;
                if (PROD) {
                    const volatile uint32_t* sg = reinterpret_cast<const volatile uint32_t*>(stage + kTileKeys * L::kCodeRowBytes + row * L::kSignRowBytes) + part * 2;
                    sw[0] = fail ? 0u : ~sg[0];   // a set bit now means a negative sign
                    sw[1] = fail ? 0u : ~sg[1];
                }
            }
            __threadfence_block();   // every lane's loads from the stage are performed before the stage is released
            __syncwarp();
            if (lane == 0 && !fail) mbar_arrive(BAR(K_EMPTY + s));
            const uint32_t abase = tmem + lane_addr + A_COL(part >> 1) + (uint32_t)(part & 1) * 32;
            {   // phase 0: centroids
                uint32_t hi[2][16], lo[2][16];
#pragma unroll
                for (int sb = 0; sb < 2; ++sb)
#pragma unroll
                    for (int p = 0; p < 16; ++p) {
                        const int pair = sb * 16 + p;
                        const int bit = pair * 2 * BITS, wi = bit >> 5, sh = bit & 31;
                        uint32_t e;
                        if (sh + 2 * BITS <= 32) e = (w[wi] >> sh) & kPairMask;
                        else e = __funnelshift_r(w[wi], w[wi + 1], sh) & kPairMask;
                        const uint2 v = lut_lane[e * 32];
                        hi[sb][p] = v.x;
                        lo[sb][p] = v.y;
                    }
                if (!mbar_wait(BAR(A_EMPTY), (uint32_t)(phase_n & 1) ^ 1u, abort_flag)) fail = true;
                tc_fence_after();
#pragma unroll
                for (int sb = 0; sb < 2; ++sb) {
                    tmem_st16(abase + sb * 16, hi[sb]);
                    tmem_st16(abase + kABlock + sb * 16, lo[sb]);
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(A_FULL));
                ++phase_n;
            }
            if (PROD) {   // phase 1: +-beta, both halves of a pair alike; the signs flip bit 15 / 31
                const float beta = a.alpha * rn * kBetaScale;
                const __half bh = __float2half_rn(beta);
                const __half bl = __float2half_rn(beta - __half2float(bh));
                const uint32_t bhu = (uint32_t)__half_as_ushort(bh), blu = (uint32_t)__half_as_ushort(bl);
                const uint32_t bh2 = bhu | (bhu << 16), bl2 = blu | (blu << 16);
                if (!mbar_wait(BAR(A_EMPTY), (uint32_t)(phase_n & 1) ^ 1u, abort_flag)) fail = true;
                tc_fence_after();
#pragma unroll
                for (int sb = 0; sb < 2; ++sb) {
                    uint32_t sgh[16], sgl[16];
#pragma unroll
                    for (int p = 0; p < 16; ++p) {
                        const uint32_t flip = (sw[sb] << (15 - p)) & 0x80008000u;   // sign word sb: pair p = bits p, 16 + p
                        sgh[p] = bh2 ^ flip;
                        sgl[p] = bl2 ^ flip;
                    }
                    tmem_st16(abase + sb * 16, sgh);
                    tmem_st16(abase + kABlock + sb * 16, sgl);
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(A_FULL));
                ++phase_n;
            }
        }
    } else {
        // ---- epilogue: two threads per key and output half -------------------------------------------------
        const int ew = warp - kFirstEpi;
        const int quarter = warp & 3;
        const int colgroup = ew >> 2;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        unsigned char* stg = smem + L::off_out + ew * L::kOutWarpBytes;
        for (int64_t i = 0; i < my_tiles; ++i) {
            const int64_t tile = blockIdx.x + i * gridDim.x;
            const uint32_t par = (uint32_t)(i & 1);
            const int64_t row0 = tile * kTileKeys + quarter * 32;
            const float sc = (row0 + lane < a.n ? __ldg(a.norms + row0 + lane) : 0.f) * kOutScale;
#pragma unroll 1
            for (int j = 0; j < 2; ++j) {
                const int64_t n_live = mbar_wait(BAR(D_FULL + j), par, abort_flag) ? a.n : 0;   // after a give-up nothing is written
                tc_fence_after();
                const uint32_t acc = tmem + lane_addr + ACC_COL(j) + colgroup * 64;
                uint32_t va[32], vb[32];
                tmem_ld32(acc, va);
                tmem_ld32(acc + 32, vb);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(D_EMPTY + j));   // the accumulator is free again
                // through the warp's staging block, so that its global stores cover whole 128-byte lines
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    float4* mine = reinterpret_cast<float4*>(stg + lane * L::kOutRowBytes);
#pragma unroll
                    for (int m = 0; m < 8; ++m) {
                        const uint32_t* v = ch == 0 ? va : vb;
                        mine[m] = make_float4(__uint_as_float(v[4 * m]) * sc, __uint_as_float(v[4 * m + 1]) * sc,
                                              __uint_as_float(v[4 * m + 2]) * sc, __uint_as_float(v[4 * m + 3]) * sc);
                    }
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int r = it * 4 + (lane >> 3), c4 = lane & 7;
                        const float4 val = *reinterpret_cast<const float4*>(stg + r * L::kOutRowBytes + c4 * 16);
                        if (row0 + r < n_live)
                            __stcs(reinterpret_cast<float4*>(a.out + (row0 + r) * kD + j * 128 + colgroup * 64 + ch * 32) + c4, val);
                    }
                    __syncwarp();
                }
            }
        }
    }

    if (*abort_flag) __nanosleep(20000);   // tensor instructions issued before the give-up may still be running
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.status, 3ull);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ---- host side ------------------------------------------------------------------------------------
uint16_t half_bits(float v) {
    const __half h = __float2half_rn(v);
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}
float half_value(uint16_t b) {
    __half h;
    memcpy(&h, &b, 2);
    return __half2float(h);
}

// B[n][k] = m[k][n] * scale as fp16 hi + lo in the K-major 8x8 core-matrix layout the tensor core reads.
void split_transposed(const float* m, int d, float scale, uint16_t* hi, uint16_t* lo) {
    const size_t sbo = (size_t)(D / 8) * 128, lbo = 128;   // laid out D x D; the caller zero-fills, so d < D is padded
    for (int n = 0; n < d; ++n)
        for (int k = 0; k < d; ++k) {
            const float v = m[(size_t)k * d + n] * scale;
            const uint16_t h = half_bits(v);
            const uint16_t l = half_bits(v - half_value(h));
            const size_t off = ((size_t)(n / 8) * sbo + (size_t)(k / 8) * lbo + (size_t)(n % 8) * 16 + (size_t)(k % 8) * 2) / 2;
            hi[off] = h;
            lo[off] = l;
        }
}

// d = 256: B[n][k] = m[k][n] * scale in chunks ((J * 2 + I) * 8 + kb) = [hi | lo] of 128 (n) x 16 (k) halves each, K-major
// core matrices (8-row groups 256 bytes apart, the two core matrices of a group 128 bytes apart)
void split_transposed_chunks(const float* m, float scale, uint16_t* out) {
    const int d = 256;
    for (int n = 0; n < d; ++n)
        for (int k = 0; k < d; ++k) {
            const float v = m[(size_t)k * d + n] * scale;
            const uint16_t h = half_bits(v);
            const uint16_t l = half_bits(v - half_value(h));
            const int J = n / 128, I = k / 128, kb = (k % 128) / 16, nn = n % 128, kk = k % 16;
            const size_t chunk = (size_t)((J * 2 + I) * 8 + kb) * 8192;
            const size_t off = (size_t)(nn / 8) * 256 + (size_t)(kk / 8) * 128 + (size_t)(nn % 8) * 16 + (size_t)(kk % 8) * 2;
            out[(chunk + off) / 2] = h;
            out[(chunk + 4096 + off) / 2] = l;
        }
}

template <int BITS, bool PROD>
int launch_256(const DequantArgs& args, int grid, cudaStream_t st) {
    const int sm = dq256::Smem<BITS, PROD>::total;
    TQ_CUDA_TRY(cudaFuncSetAttribute(dequant256_kernel<BITS, PROD>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm));
    dequant256_kernel<BITS, PROD><<<grid, dq256::kThreads256, sm, st>>>(args); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

template <int BITS, bool PROD, int DR, bool PAIR = false>
int launch_one(const DequantArgs& args, int grid, cudaStream_t st) {
    const int sm = DqSmem<BITS, PROD, DR>::total;
    TQ_CUDA_TRY(cudaFuncSetAttribute(dequant_tc_kernel<BITS, PROD, DR, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm));
    dequant_tc_kernel<BITS, PROD, DR, PAIR><<<grid, kThreads, sm, st>>>(args); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

}  // namespace

struct DequantConsts {
    void* dev = nullptr;   // [Rt_hi | Rt_lo | St_hi | St_lo]
};

bool tq_dequant_tc_supported(int d, int bits_mse, bool prod) {
    // the pair lookup table of a 4-bit code and four operand matrices do not fit side by side
    return (d == 128 || d == 64 || d == 256) && bits_mse >= 1 && bits_mse <= (prod ? 3 : 4);
}

int tq_dequant_tc_plan_init(tq_plan* p, const float* rotation, const float* projection) {
    const int d = p->dev.d;
    if (d != 128 && d != 64 && d != 256) return TQ_OK;
    const size_t dd = (size_t)D * D;
    const int nmat = projection ? 4 : 2;
    std::vector<uint16_t> mats(d == 256 ? (size_t)d * d * nmat : dd * nmat, 0);
    if (d == 256) {
        split_transposed_chunks(rotation, kRotScale, mats.data());
        if (projection) split_transposed_chunks(projection, kProjScale, mats.data() + (size_t)d * d * 2);
    } else {
        split_transposed(rotation, d, kRotScale, mats.data(), mats.data() + dd);
        if (projection) split_transposed(projection, d, kProjScale, mats.data() + 2 * dd, mats.data() + 3 * dd);
    }
    DequantConsts* c = new DequantConsts();
    cudaError_t e = cudaMalloc(&c->dev, mats.size() * 2);
    if (e == cudaSuccess) e = cudaMemcpy(c->dev, mats.data(), mats.size() * 2, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        if (c->dev) cudaFree(c->dev);
        delete c;
        return tq_fail(TQ_ERR_CUDA, "upload of dequantize operand matrices failed: %s", cudaGetErrorString(e));
    }
    p->dequant = c;
    return TQ_OK;
}

void tq_dequant_tc_plan_free(tq_plan* p) {
    if (p->dequant) {
        if (p->dequant->dev) cudaFree(p->dequant->dev);
        delete p->dequant;
        p->dequant = nullptr;
    }
}

int tq_launch_dequant_tc(const tq_plan* p, bool prod, const uint32_t* codes, const uint32_t* signs, const float* rnorms,
                         const float* norms, int64_t n, float* out, cudaStream_t st) {
    TqRange range("tq.dequantize.tensor_core");
    if (n == 0) return TQ_OK;
    if (!p->dequant) return tq_fail(TQ_ERR_UNSUPPORTED, "no tensor-core dequantize constants in this plan");
    DequantArgs a{};
    a.codes = codes; a.signs = signs; a.rnorms = rnorms; a.norms = norms;
    a.bmat = static_cast<const unsigned char*>(p->dequant->dev);
    a.codebook = p->dev.codebook;
    a.alpha = p->dev.alpha;
    a.n = n;
    a.ntiles = (n + kTileKeys - 1) / kTileKeys;
    a.out = out;
    a.status = p->counters + 1;
    a.wait_kcycles = p->wait_kcycles;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->device);
    const int grid = (int)(a.ntiles < sms ? a.ntiles : sms);
    const int bits = p->dev.bits;
    int r = TQ_ERR_UNSUPPORTED;
#define TQ_DQ(B, P)                                                                                  \
    case B:                                                                                          \
        r = p->dev.d == 64 ? launch_one<B, P, 64>(a, grid, st) : launch_one<B, P, 128>(a, grid, st); \
        break;
    if (p->dev.d == 256) {
        if (prod) {
            switch (bits) {
                case 1: r = launch_256<1, true>(a, grid, st); break;
                case 2: r = launch_256<2, true>(a, grid, st); break;
                case 3: r = launch_256<3, true>(a, grid, st); break;
                default: break;
            }
        } else {
            switch (bits) {
                case 1: r = launch_256<1, false>(a, grid, st); break;
                case 2: r = launch_256<2, false>(a, grid, st); break;
                case 3: r = launch_256<3, false>(a, grid, st); break;
                case 4: r = launch_256<4, false>(a, grid, st); break;
                default: break;
            }
        }
    } else if (prod) {
        switch (bits) { TQ_DQ(1, true) TQ_DQ(2, true) TQ_DQ(3, true) default: break; }
    } else {
        switch (bits) { TQ_DQ(1, false) TQ_DQ(2, false) TQ_DQ(3, false) TQ_DQ(4, false) default: break; }
    }
#undef TQ_DQ
    if (r == TQ_ERR_UNSUPPORTED) return tq_fail(r, "no tensor-core dequantize kernel for bits=%d", bits);
    return r;
}

// attention_score with one query row per key on the dequantize kernel: scores[i] = q[i] . dequantize(key i).
int tq_launch_pairwise_tc(const tq_plan* p, const float* q, const uint32_t* codes, const uint32_t* signs, const float* rnorms,
                          const float* norms, int64_t n, float* scores, cudaStream_t st) {
    TqRange range("tq.score.pairwise.tensor_core");
    if (n == 0) return TQ_OK;
    if (!p->dequant || !p->has_projection) return tq_fail(TQ_ERR_UNSUPPORTED, "no tensor-core dequantize constants in this plan");
    DequantArgs a{};
    a.codes = codes; a.signs = signs; a.rnorms = rnorms; a.norms = norms;
    a.bmat = static_cast<const unsigned char*>(p->dequant->dev);
    a.codebook = p->dev.codebook;
    a.alpha = p->dev.alpha;
    a.n = n;
    a.ntiles = (n + kTileKeys - 1) / kTileKeys;
    a.out = scores;
    a.pair_q = q;
    a.status = p->counters + 1;
    a.wait_kcycles = p->wait_kcycles;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->device);
    const int grid = (int)(a.ntiles < sms ? a.ntiles : sms);
    int r = TQ_ERR_UNSUPPORTED;
#define TQ_PW(B)                                                                                                   \
    case B:                                                                                                        \
        r = p->dev.d == 64 ? launch_one<B, true, 64, true>(a, grid, st) : launch_one<B, true, 128, true>(a, grid, st); \
        break;
    switch (p->dev.bits) { TQ_PW(1) TQ_PW(2) TQ_PW(3) default: break; }
#undef TQ_PW
    if (r == TQ_ERR_UNSUPPORTED) return tq_fail(r, "no tensor-core pairwise kernel for bits=%d", p->dev.bits);
    return r;
}
