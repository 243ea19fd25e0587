// attention_score for three or four queries per group of keys with the score matrix as the result -- the decode
// step of grouped-query attention over a quantized key cache: every KV head is scored by its 4 query heads
// (TurboQuantProd.attention_score, _quant.py:334-358, called once per query head by the reference's users).
// d = 128 or 64, 1..3 code bits.
//
// Like tq_score_few.cu the kernel turns the rotated and projected queries into lookup tables -- a pair table
// [d/2][4^bits] and a sign-byte table [d/8][256] -- here with the (up to) four queries of the group interleaved,
// so that one 16-byte load serves all of them, and laid out by lane: eight lanes share a key, lane l walks pairs
// PPL*l .. PPL*l+PPL-1 and sign bytes BPL*l .., and entry (i, e) of lane l sits at ((i * entries + e) * 8 + l) * 4
// floats.  The eight lanes of a key therefore read eight different 16-byte bank groups whatever their codes are
// (one thread per key, as in the one-query kernel, loses 2.7x to bank conflicts with 16-byte entries).  The
// partial sums of the eight lanes meet in a reduce-scatter of four shuffles.  Measured against the tensor-core kernel (whose
// cost does not shrink below 16 queries): 156 vs 191 us for 64 groups x 4 queries x 32,768 keys at d = 128.
#include "tq_common.cuh"

#include <stdint.h>

namespace {

constexpr int kThreads = 512;
constexpr int kTile = 512;
constexpr int kWarps = kThreads / 32;
constexpr int QP = 4;

template <int KB, int DR>
constexpr size_t lut_smem_floats() {
    return (size_t)((DR / 2) * (1 << (2 * KB)) + (DR / 8) * 256) * QP + 2 * QP * kTile + 3 * QP * DR;
}

// grid (blocks over the tiles of a group, 1, groups); qpg <= 4
template <int KB, int DR>
__global__ void __launch_bounds__(kThreads)
score_lut_kernel(TqDev p, const float* __restrict__ q, const uint32_t* __restrict__ codes,
                 const uint32_t* __restrict__ signs, const float* __restrict__ rnorms, const float* __restrict__ norms,
                 int64_t n, int64_t group_rows, int qpg, float* __restrict__ scores) {
    constexpr int kPairs = DR / 2, kEntries = 1 << (2 * KB), kBytes = DR / 8;
    constexpr int kCodeWords = DR * KB / 32, kSignWords = DR / 32;
    constexpr uint32_t kMask = kEntries - 1;
    constexpr int PPL = kPairs / 8, BPL = kBytes / 8;
    constexpr int kLaneBits = PPL * 2 * KB;             // bits of the code row one lane looks at (<= 48)
    constexpr int kSteps = kTile / (kWarps * 4);        // a warp takes 4 keys per step
    constexpr bool kNeedW1 = 32 % kLaneBits != 0;       // a lane's bits can lie across two words
    extern __shared__ __align__(16) float smf[];
    float* pair_t = smf;                                // [PPL][kEntries][8 lanes][QP]
    float* byte_t = pair_t + kPairs * kEntries * QP;    // [BPL][256][8 lanes][QP]
    float* sbuf = byte_t + kBytes * 256 * QP;           // [2][QP][kTile] scores of a tile, double-buffered
    float* qin = sbuf + 2 * QP * kTile;                 // [QP][DR]
    float* qr = qin + QP * DR;                          // rotated queries
    float* ps = qr + QP * DR;                           // projected queries

    const int g = blockIdx.z, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    for (int i = t; i < QP * DR; i += kThreads) {
        const int qq = i / DR, k = i - qq * DR;
        qin[i] = qq < qpg ? __ldg(q + ((size_t)g * qpg + qq) * DR + k) : 0.f;
    }
    __syncthreads();
    // rotated[j] = sum_k q[k] R[j][k], projected[j] = sum_k q[k] S[j][k]: one FMA per k, k ascending, as in
    // the reference's matrix products
    for (int i = t; i < QP * DR; i += kThreads) {
        const int qq = i / DR, j = i - qq * DR;
        const float* qv = qin + qq * DR;
        float r = 0.f, sacc = 0.f;
        for (int k0 = 0; k0 < DR; k0 += 16) {
            float mr[16], ms[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                mr[u] = __ldg(p.Rt + (size_t)(k0 + u) * DR + j);
                ms[u] = __ldg(p.St + (size_t)(k0 + u) * DR + j);
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                r = fmaf(qv[k0 + u], mr[u], r);
                sacc = fmaf(qv[k0 + u], ms[u], sacc);
            }
        }
        qr[i] = r;
        ps[i] = sacc;
    }
    __syncthreads();
    for (int idx = t; idx < kPairs * kEntries; idx += kThreads) {
        const int l = idx & 7, e = (idx >> 3) & (kEntries - 1), i = idx / (8 * kEntries);
        const int pp = PPL * l + i;
        const float c0 = __ldg(p.codebook + (e & ((1 << KB) - 1))), c1 = __ldg(p.codebook + (e >> KB));
#pragma unroll
        for (int qq = 0; qq < QP; ++qq) pair_t[idx * QP + qq] = fmaf(c1, qr[qq * DR + 2 * pp + 1], c0 * qr[qq * DR + 2 * pp]);
    }
    for (int idx = t; idx < kBytes * 256; idx += kThreads) {
        const int l = idx & 7, v = (idx >> 3) & 255, i = idx >> 11;
        const int pos = BPL * l + i, w = pos >> 2, b = pos & 3;
#pragma unroll
        for (int qq = 0; qq < QP; ++qq) {
            float acc = 0.f;
#pragma unroll
            for (int bit = 0; bit < 8; ++bit) {
                // stored order of the sign words: even coordinates in bits 0..15, odd ones in bits 16..31
                const int bp = 8 * b + bit;
                const int coord = 32 * w + (bp < 16 ? 2 * bp : 2 * (bp - 16) + 1);
                const float x = ps[qq * DR + coord];
                acc += (v >> bit) & 1 ? x : -x;
            }
            byte_t[idx * QP + qq] = acc;
        }
    }

    // lane l8 of the 8 that share key (warp * 32 + step * 4 + lane / 8) of a tile
    const int l8 = lane & 7, ksc = warp * 32 + (lane >> 3);
    constexpr int kLastWord = kCodeWords - 1;
    const int cw_i = (kLaneBits * l8) >> 5, cw_sh = (kLaneBits * l8) & 31;
    const int cw_i2 = cw_i + 1 < kLastWord ? cw_i + 1 : kLastWord;
    const int sw_i = (BPL * l8) >> 2, sw_sh = ((BPL * l8) & 3) * 8;
    const bool b0 = l8 & 1, b1 = l8 & 2;
    const int qsel = 2 * (l8 & 1) + ((l8 >> 1) & 1);   // the query whose sum this lane holds after the exchange
    const float* pair_l = pair_t + l8 * QP;
    const float* byte_l = byte_t + l8 * QP;
    const float alpha = p.alpha;
    const int64_t tiles = (n + kTile - 1) / kTile;
    const int64_t gbase = (int64_t)g * group_rows;

    uint32_t pw0[kSteps], pw1[kSteps], psg[kSteps];
    float pnr[kSteps], prn[kSteps];
    auto fetch_step = [&](int64_t tile, int st) {
        const int64_t key = tile * kTile + ksc + st * 4;
        pw0[st] = 0u; pw1[st] = 0u; psg[st] = 0u; pnr[st] = 0.f; prn[st] = 0.f;
        if (tile < tiles && key < n) {
            const int64_t row = gbase + key;
            const uint32_t* crow = codes + row * kCodeWords;
            pw0[st] = __ldg(crow + cw_i);
            if (kNeedW1) pw1[st] = __ldg(crow + cw_i2);
            psg[st] = __ldg(signs + row * kSignWords + sw_i);
            pnr[st] = __ldg(norms + row);
            prn[st] = __ldg(rnorms + row);
        }
    };
    int64_t tile = blockIdx.x;
#pragma unroll
    for (int st = 0; st < kSteps; ++st) fetch_step(tile, st);
    __syncthreads();   // tables complete

    int buf = 0;
    for (; tile < tiles; tile += gridDim.x) {
        const int64_t k0 = tile * kTile;
        float* sb = sbuf + buf * QP * kTile;
#pragma unroll
        for (int st = 0; st < kSteps; ++st) {
            const uint32_t lo = __funnelshift_r(pw0[st], pw1[st], cw_sh);
            const uint64_t z = kLaneBits > 32 ? ((uint64_t)(pw1[st] >> cw_sh) << 32) | lo : (uint64_t)lo;
            const uint32_t sg = psg[st] >> sw_sh;
            const float ar = alpha * prn[st], nr = pnr[st];
            // the registers of this step are free: the same step of the block's next tile is fetched into them
            fetch_step(tile + gridDim.x, st);
            float a1[QP], a2[QP];
#pragma unroll
            for (int qq = 0; qq < QP; ++qq) { a1[qq] = 0.f; a2[qq] = 0.f; }
#pragma unroll
            for (int i = 0; i < PPL; ++i) {
                const uint32_t e = (uint32_t)(z >> (i * 2 * KB)) & kMask;
                const float4 x = *reinterpret_cast<const float4*>(pair_l + (i * kEntries + e) * 8 * QP);
                a1[0] += x.x; a1[1] += x.y; a1[2] += x.z; a1[3] += x.w;
            }
#pragma unroll
            for (int i = 0; i < BPL; ++i) {
                const float4 x = *reinterpret_cast<const float4*>(byte_l + (i * 256 + ((sg >> (8 * i)) & 255u)) * 8 * QP);
                a2[0] += x.x; a2[1] += x.y; a2[2] += x.z; a2[3] += x.w;
            }
            // The eight partial sums of each of the four queries meet in a reduce-scatter: lanes trade the half of
            // their values the partner keeps (2 shuffles, then 1), and one more exchange joins the two groups of
            // four lanes: 4 shuffles instead of the 12 of four butterflies.  Lane l8 ends with query qsel.
            float v[QP];
#pragma unroll
            for (int qq = 0; qq < QP; ++qq) v[qq] = fmaf(ar, a2[qq], a1[qq]);
            const float rx = __shfl_xor_sync(0xffffffffu, b0 ? v[0] : v[2], 1);
            const float ry = __shfl_xor_sync(0xffffffffu, b0 ? v[1] : v[3], 1);
            const float ax = (b0 ? v[2] : v[0]) + rx, ay = (b0 ? v[3] : v[1]) + ry;
            float s = (b1 ? ay : ax) + __shfl_xor_sync(0xffffffffu, b1 ? ax : ay, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (l8 < 4) sb[qsel * kTile + ksc + st * 4] = nr * s;
        }
        __syncthreads();   // the tile's scores are in shared memory; the other buffer's readers are done
        if (k0 + t < n) {
            for (int qq = 0; qq < qpg; ++qq) scores[((size_t)g * qpg + qq) * n + k0 + t] = sb[qq * kTile + t];
        }
        buf ^= 1;
    }
}

template <int KB, int DR>
int launch_lut(const tq_plan* p, const float* q, const uint32_t* codes, const uint32_t* signs, const float* rnorms,
               const float* norms, int64_t n, int64_t group_rows, int groups, int qpg, float* scores, cudaStream_t st) {
    const size_t sm = lut_smem_floats<KB, DR>() * 4;
    TQ_CUDA_TRY(cudaFuncSetAttribute(score_lut_kernel<KB, DR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->device);
    int per_sm = 1;                                   // resident blocks per SM (shared memory and registers)
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, score_lut_kernel<KB, DR>, kThreads, sm);
    if (per_sm < 1) per_sm = 1;
    const int64_t tiles = (n + kTile - 1) / kTile;
    // every block builds the tables of its group (a few microseconds): as many blocks per group as are resident
    // at once, the tiles of the group dealt round-robin among them
    int64_t blocks = (int64_t)sms * per_sm / groups;   // rounded down: a second wave would double the time
    if (blocks > tiles) blocks = tiles;
    if (blocks < 1) blocks = 1;
    score_lut_kernel<KB, DR><<<dim3((unsigned)blocks, 1, (unsigned)groups), kThreads, sm, st>>>(
        p->dev, q, codes, signs, rnorms, norms, n, group_rows, qpg, scores); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

}  // namespace

bool tq_score_lut_supported(const tq_plan* p, int qpg) {
    // d = 64 is compiled and correct, but the tensor-core kernel is a little faster there (130 vs 135 us for
    // 64 groups x 4 queries x 32,768 keys; at d = 128: 191 vs 156 us)
    return p->has_projection && p->dev.d == 128 && p->dev.bits >= 1 && p->dev.bits <= 3 && qpg >= 3 && qpg <= 4;
}

// scores: [groups][qpg][keys_per_group]
int tq_launch_score_lut(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes, const uint32_t* signs,
                        const float* rnorms, const float* norms, int64_t keys_per_group, float* scores, cudaStream_t st,
                        int64_t group_rows) {
    TqRange range("tq.score.lookup_tables");
    if (group_rows <= 0) group_rows = keys_per_group;
    const int d = p->dev.d, bits = p->dev.bits;
    int r = TQ_ERR_UNSUPPORTED;
#define TQ_LUT(B)                                                                                                        \
    case B:                                                                                                             \
        r = d == 64 ? launch_lut<B, 64>(p, q, codes, signs, rnorms, norms, keys_per_group, group_rows, groups, qpg, scores, st)     \
                    : launch_lut<B, 128>(p, q, codes, signs, rnorms, norms, keys_per_group, group_rows, groups, qpg, scores, st);   \
        break;
    switch (bits) { TQ_LUT(1) TQ_LUT(2) TQ_LUT(3) }
#undef TQ_LUT
    if (r == TQ_ERR_UNSUPPORTED) return tq_fail(r, "no lookup-table scoring kernel for d=%d bits=%d", d, bits);
    return r;
}
