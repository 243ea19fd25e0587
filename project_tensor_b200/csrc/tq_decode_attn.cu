// Decode attention over a quantized key/value cache, d = 128 or 64:
//
//   out[g][a] = softmax_i( scale * score(q[g][a], key[g][i]) ) . value[g][i]
//
// with keys held as TurboQuantProd encodings (score = TurboQuantProd.attention_score, _quant.py:334-358) and
// values as TurboQuantMSE encodings (value = TurboQuantMSE.dequantize, _quant.py:238-254).  It is the caller
// side of attention_score -- scale, softmax, weighted sum of values: scaled_dot_product_attention,
// _core.py:1606-1683 -- done without ever writing the scores or the dequantized values to memory: per key
// the kernel reads the packed key (d*b/8 + d/8 + 8 bytes) and the packed value (d*b/8 + 4 bytes) once.
//
// Two facts shape it:
//   * scores for a few queries per group come from lookup tables (as in tq_score_few.cu): per query a pair
//     table [d/2][4^bits] and a byte table [d/8][256], here interleaved by query so that one vector load
//     serves all queries of a pass;
//   * dequantize is linear after the centroid gather: sum_i p_i * norm_i * (c[idx_i] R) = (sum_i p_i norm_i
//     c[idx_i]) R, so the block accumulates in the rotated domain (one multiply-add per coordinate, key and
//     query) and the d x d rotation is applied once per query in the combine kernel.
//
// A block of 512 threads walks tiles of 512 keys of one group: thread t scores key t of the tile for the QP
// queries of the pass, the block agrees on the running maximum (online softmax), then the same threads
// regroup as (8 consecutive coordinates, key t / (d/8) of every batch of 512 / (d/8) keys) and add the tile's
// values, staged in shared memory by cp.async, into their 8 x QP accumulators: one load of packed codes, one
// of the weights and eight codebook lookups feed 8 x QP multiply-adds.  Key ranges are split over blocks; every block leaves (max, sum,
// accumulator) per query in scratch and decode_combine_kernel merges the splits and rotates.
#include "tq_common.cuh"

#include <math_constants.h>
#include <stdint.h>

namespace {

constexpr int kThreads = 512;
constexpr int kTile = 512;
constexpr int kMaxSplits = 64;
constexpr int kWarps = kThreads / 32;

struct DecodeArgs {
    const float* q;              // [groups][qpg][d]
    const uint32_t* kcodes;
    const uint32_t* ksigns;
    const float* krnorms;
    const float* knorms;
    const uint32_t* vcodes;
    const float* vnorms;
    const float* vcodebook;      // codebook of the value quantizer
    int vbits, vwords;           // bits per value code, 32-bit words per packed value row
    int qpg;
    int64_t keys_per_group, group_rows;
    const int64_t* length;       // optional device-side number of keys per group (capped by keys_per_group)
    float scale_log2e;           // scale * log2(e): the softmax runs in base 2
    int splits;
    int vbufs;                   // value tiles in shared memory: 2 = the next tile is copied while this one is used
    float* part;                 // [groups][qpg][splits][d + 2]: accumulator, running max, running sum
};

template <int QP>
__device__ __forceinline__ void ld_vec(const float* p, float (&v)[QP]) {
    if constexpr (QP == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else if constexpr (QP == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p);
        v[0] = t.x; v[1] = t.y;
    } else {
        v[0] = *p;
    }
}
template <int QP>
__device__ __forceinline__ void st_vec(float* p, const float (&v)[QP]) {
    if constexpr (QP == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else if constexpr (QP == 2) *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
    else *p = v[0];
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int DR, int QP>
__host__ __device__ constexpr int pbuf_floats() { return kTile * QP > kWarps * DR ? kTile * QP : kWarps * DR; }

// floats of shared memory in front of the value tiles
template <int KB, int DR, int QP>
constexpr size_t decode_smem_floats() {
    return (size_t)((DR / 2) * (1 << (2 * KB)) + (DR / 8) * 256) * QP + pbuf_floats<DR, QP>() + kTile * QP + 3 * QP * DR +
           kWarps * QP + 8 + 16;
}

// grid (splits, passes over the queries of a group, groups)
// VSTRADDLE: the 8 codes of a thread may lie across two 32-bit words (3-bit values only)
template <int KB, int DR, int QP, bool VSTRADDLE>
__global__ void __launch_bounds__(kThreads, 1)
decode_partial_kernel(TqDev kp, DecodeArgs a) {
    constexpr int kPairs = DR / 2, kEntries = 1 << (2 * KB), kBytes = DR / 8;
    constexpr int kCodeWords = DR * KB / 32, kSignWords = DR / 32;
    constexpr uint32_t kMask = kEntries - 1;
    // scoring: 8 lanes share a key; lane l walks pairs PPL*l .. PPL*l + PPL-1 and sign bytes BPL*l .. of the row
    constexpr int PPL = kPairs / 8, BPL = kBytes / 8;
    constexpr int kLaneBits = PPL * 2 * KB;             // bits of the code row one lane looks at (<= 64)
    constexpr int kSteps = kTile / (kWarps * 4);        // a warp takes 4 keys per step
    // value phase: 8 coordinates per thread
    constexpr int kCT = DR / 8;                         // threads that share a key
    constexpr int kIterKeys = kThreads / kCT;           // keys the block takes per step
    extern __shared__ __align__(16) unsigned char smraw[];
    float* pair_t = reinterpret_cast<float*>(smraw);   // [PPL][kEntries][8 lanes][QP]
    float* byte_t = pair_t + kPairs * kEntries * QP;    // [BPL][256][8 lanes][QP]
    float* pbuf = byte_t + kBytes * 256 * QP;           // [kTile][QP] weight * value norm; at the end [kWarps][DR]
    float* sbuf = pbuf + pbuf_floats<DR, QP>();         // [kTile][QP] scaled scores of the tile
    float* qin = sbuf + kTile * QP;                     // [QP][DR]
    float* qr = qin + QP * DR;                          // rotated queries
    float* ps = qr + QP * DR;                           // projected queries
    float* red = ps + QP * DR;                          // [kWarps][QP]
    float* sm_m = red + kWarps * QP;                    // [4] running maximum per query
    float* sm_f = sm_m + 4;                             // [4] factor that brings older sums to the new maximum
    float* vcb = sm_f + 4;                              // [16] value codebook
    uint32_t* vt = reinterpret_cast<uint32_t*>(vcb + 16);   // [vbufs][kTile][vwords] packed value rows

    const int g = blockIdx.z, q0 = blockIdx.y * QP, split = blockIdx.x;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    int64_t n = a.keys_per_group;
    if (a.length) {
        const int64_t len = *a.length;
        n = len < n ? len : n;
        if (n < 0) n = 0;
    }

    for (int i = t; i < QP * DR; i += kThreads) {
        const int qq = i / DR, k = i - qq * DR;
        qin[i] = q0 + qq < a.qpg ? __ldg(a.q + ((size_t)g * a.qpg + q0 + qq) * DR + k) : 0.f;
    }
    if (t < 16) vcb[t] = t < (1 << a.vbits) ? __ldg(a.vcodebook + t) : 0.f;
    if (t < 4) sm_m[t] = -CUDART_INF_F;
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
                mr[u] = __ldg(kp.Rt + (size_t)(k0 + u) * DR + j);
                ms[u] = __ldg(kp.St + (size_t)(k0 + u) * DR + j);
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
    // Tables.  Entry (i, e) of lane l sits at ((i * entries + e) * 8 + l) * QP floats: with QP = 4 the eight
    // lanes of a key read eight different 16-byte bank groups whatever their codes are.
    for (int idx = t; idx < kPairs * kEntries; idx += kThreads) {
        const int l = idx & 7, e = (idx >> 3) & (kEntries - 1), i = idx / (8 * kEntries);
        const int pp = PPL * l + i;
        const float c0 = __ldg(kp.codebook + (e & ((1 << KB) - 1))), c1 = __ldg(kp.codebook + (e >> KB));
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

    const int64_t tiles_total = (n + kTile - 1) / kTile;
    const int64_t tps = (tiles_total + a.splits - 1) / a.splits;
    const int64_t tile0 = (int64_t)split * tps;
    int64_t tile1 = tile0 + tps;
    if (tile1 > tiles_total) tile1 = tiles_total;

    // scoring role: lane l8 of the 8 that share key (warp * 32 + step * 4 + lane / 8) of the tile
    const int l8 = lane & 7, ksc = warp * 32 + (lane >> 3);
    constexpr int kLastWord = kCodeWords - 1;
    const int cw_i = (kLaneBits * l8) >> 5, cw_sh = (kLaneBits * l8) & 31;
    const int cw_i2 = cw_i + 1 < kLastWord ? cw_i + 1 : kLastWord;
    const int sw_i = (BPL * l8) >> 2, sw_sh = ((BPL * l8) & 3) * 8;
    const bool b0 = l8 & 1, b1 = l8 & 2;
    // the query whose sum the lane holds after the exchange among the eight lanes of a key
    const int qsel = QP == 4 ? 2 * (l8 & 1) + ((l8 >> 1) & 1) : QP == 2 ? (l8 & 1) : 0;
    const float* pair_l = pair_t + l8 * QP;
    const float* byte_l = byte_t + l8 * QP;
    // value role: coordinates 8c .. 8c+7 of key `ksub` of every batch of kIterKeys keys; their codes are the
    // 8 * vbits bits that start at byte vbits * c of the packed row
    const int c = t & (kCT - 1), ksub = t / kCT;
    const int vbyte = a.vbits * c, vw = vbyte >> 2, vsh = (vbyte & 3) * 8;
    const int vw2 = vw + 1 < a.vwords ? vw + 1 : vw;
    const int vbits = a.vbits;
    const uint32_t vmask = (1u << a.vbits) - 1u;
    const int vwords = a.vwords;
    const float alpha = kp.alpha;
    const int vstride = a.vbufs > 1 ? kTile * vwords : 0;   // words between the two value buffers

    float l_part[QP], acc[QP][8];
#pragma unroll
    for (int qq = 0; qq < QP; ++qq) {
        l_part[qq] = 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[qq][u] = 0.f;
    }
    // packed key words and norms of the next tile, fetched one tile ahead
    uint32_t pw0[kSteps], pw1[kSteps], psg[kSteps];
    float pnr[kSteps], prn[kSteps], vn = 0.f;
    auto fetch_keys = [&](int64_t tile) {
        const int64_t k0 = tile * kTile;
#pragma unroll
        for (int st = 0; st < kSteps; ++st) {
            const int64_t key = k0 + ksc + st * 4;
            pw0[st] = 0u; pw1[st] = 0u; psg[st] = 0u; pnr[st] = 0.f; prn[st] = 0.f;
            if (key < n) {
                const int64_t row = (int64_t)g * a.group_rows + key;
                const uint32_t* crow = a.kcodes + row * kCodeWords;
                pw0[st] = __ldg(crow + cw_i);
                pw1[st] = __ldg(crow + cw_i2);
                psg[st] = __ldg(a.ksigns + row * kSignWords + sw_i);
                pnr[st] = __ldg(a.knorms + row);
                prn[st] = __ldg(a.krnorms + row);
            }
        }
        vn = k0 + t < n ? __ldg(a.vnorms + (int64_t)g * a.group_rows + k0 + t) : 0.f;
    };
    // packed value rows of a tile -> shared memory (rows beyond n are not read from memory; what shared memory
    // holds for them meets a weight of zero)
    auto fetch_values = [&](int64_t tile, uint32_t* dst) {
        const int64_t k0 = tile * kTile;
        int64_t rows = n - k0;
        if (rows > kTile) rows = kTile;
        const int nwords = (int)rows * vwords;
        const uint32_t* src = a.vcodes + ((int64_t)g * a.group_rows + k0) * vwords;
        if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
            const int n16 = nwords >> 2;
            for (int i = t; i < n16; i += kThreads) cp_async16(dst + 4 * i, src + 4 * i);
            for (int i = 4 * n16 + t; i < nwords; i += kThreads) cp_async4(dst + i, src + i);
        } else {
            for (int i = t; i < nwords; i += kThreads) cp_async4(dst + i, src + i);
        }
        cp_async_commit();
    };
    if (tile0 < tile1) {
        fetch_keys(tile0);
        if (a.vbufs > 1) fetch_values(tile0, vt);
    }
    __syncthreads();   // tables complete

    // scoring phase of a tile: its scaled scores go to sbuf, the warp's maximum per query to red
    auto score_tile = [&](int64_t tile) {
        const int64_t k0 = tile * kTile;
        float mrun = -CUDART_INF_F;    // running maximum of this lane's query (qsel) over its keys of the tile
#pragma unroll
        for (int st = 0; st < kSteps; ++st) {
            float v[QP];
            const uint32_t lo = __funnelshift_r(pw0[st], pw1[st], cw_sh);
            const uint64_t z = kLaneBits > 32 ? ((uint64_t)(pw1[st] >> cw_sh) << 32) | lo : (uint64_t)lo;
            const uint32_t sg = psg[st] >> sw_sh;
            float a1[QP], a2[QP];
#pragma unroll
            for (int qq = 0; qq < QP; ++qq) { a1[qq] = 0.f; a2[qq] = 0.f; }
#pragma unroll
            for (int i = 0; i < PPL; ++i) {
                const uint32_t e = (uint32_t)(z >> (i * 2 * KB)) & kMask;
                float x[QP];
                ld_vec<QP>(pair_l + (i * kEntries + e) * 8 * QP, x);
#pragma unroll
                for (int qq = 0; qq < QP; ++qq) a1[qq] += x[qq];
            }
#pragma unroll
            for (int i = 0; i < BPL; ++i) {
                float x[QP];
                ld_vec<QP>(byte_l + (i * 256 + ((sg >> (8 * i)) & 255u)) * 8 * QP, x);
#pragma unroll
                for (int qq = 0; qq < QP; ++qq) a2[qq] += x[qq];
            }
            const float ar = alpha * prn[st];
#pragma unroll
            for (int qq = 0; qq < QP; ++qq) v[qq] = fmaf(ar, a2[qq], a1[qq]);
            // The eight partial sums of every query meet in a reduce-scatter: lanes trade the values their partner
            // keeps, so QP = 4 takes 2 + 1 + 1 shuffles instead of the 12 of four butterflies (shuffles share the
            // pipe of the lookups).  The lane ends with the sum of query qsel.
            float s;
            if constexpr (QP == 4) {
                const float rx = __shfl_xor_sync(0xffffffffu, b0 ? v[0] : v[2], 1);
                const float ry = __shfl_xor_sync(0xffffffffu, b0 ? v[1] : v[3], 1);
                const float ax = (b0 ? v[2] : v[0]) + rx, ay = (b0 ? v[3] : v[1]) + ry;
                s = (b1 ? ay : ax) + __shfl_xor_sync(0xffffffffu, b1 ? ax : ay, 2);
            } else if constexpr (QP == 2) {
                s = (b0 ? v[1] : v[0]) + __shfl_xor_sync(0xffffffffu, b0 ? v[0] : v[1], 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
            } else {
                s = v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
            }
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            const bool valid = k0 + ksc + st * 4 < n;
            s = valid ? s * (pnr[st] * a.scale_log2e) : -CUDART_INF_F;
            mrun = fmaxf(mrun, s);
            if (l8 < QP) sbuf[(ksc + st * 4) * QP + qsel] = s;
        }
        {
            // lanes 0..QP-1 of the warp end with the maximum of their query over the warp's 32 keys
            float m = mrun;
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
            if (lane < QP) red[warp * QP + qsel] = m;
        }
    };
    // value phase of a tile: weights (pbuf) times centroid values, added to the accumulators
    auto value_tile = [&](const uint32_t* vcur) {
#pragma unroll 4
        for (int it = 0; it < kTile / kIterKeys; ++it) {
            const int kk = it * kIterKeys + ksub;
            uint32_t cbits = vcur[kk * vwords + vw];
            if (VSTRADDLE) cbits = __funnelshift_r(cbits, vcur[kk * vwords + vw2], vsh);
            else cbits >>= vsh;
            float pq[QP];
            ld_vec<QP>(pbuf + kk * QP, pq);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float cv = vcb[cbits & vmask];
                cbits >>= vbits;
#pragma unroll
                for (int qq = 0; qq < QP; ++qq) acc[qq][u] = fmaf(pq[qq], cv, acc[qq][u]);
            }
        }
    };
    if (tile0 < tile1) score_tile(tile0);

    int buf = 0;
    for (int64_t tile = tile0; tile < tile1; ++tile) {
        const float vn_tile = vn;
        __syncthreads();   // scores and tile maxima visible; the value phase of the previous tile is over
        if (a.vbufs == 1) fetch_values(tile, vt);
        if (t < ((kWarps * QP + 31) & ~31)) {   // whole warps, so that the shuffles have all their lanes
            // 16 lanes per query: each takes one warp's maximum, a butterfly leaves the tile maximum in all of them
            const int qq = t / kWarps, w = t & (kWarps - 1);
            float mt = qq < QP ? red[w * QP + qq] : -CUDART_INF_F;
#pragma unroll
            for (int o = kWarps / 2; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
            if (w == 0 && qq < QP) {
                const float mo = sm_m[qq], mn = fmaxf(mo, mt);
                sm_f[qq] = mn == -CUDART_INF_F ? 1.f : exp2f(mo - mn);
                sm_m[qq] = mn;
            }
        }
        __syncthreads();
        {
            float s[QP], pv[QP];
            ld_vec<QP>(sbuf + t * QP, s);
#pragma unroll
            for (int qq = 0; qq < QP; ++qq) {
                const float mn = sm_m[qq], f = sm_f[qq];
                const float p = exp2f(s[qq] - (mn == -CUDART_INF_F ? 0.f : mn));   // masked keys: exp2(-inf) = 0
                l_part[qq] = fmaf(l_part[qq], f, p);
#pragma unroll
                for (int u = 0; u < 8; ++u) acc[qq][u] *= f;
                pv[qq] = p * vn_tile;
            }
            st_vec<QP>(pbuf + t * QP, pv);
        }
        cp_async_wait_all();
        __syncthreads();
        const uint32_t* vcur = vt + buf * vstride;
        if (tile + 1 < tile1) {
            fetch_keys(tile + 1);
            if (a.vbufs > 1) fetch_values(tile + 1, vt + (buf ^ 1) * vstride);
        }
        // Between here and the next barrier every warp owes the value phase of this tile and the scoring phase of
        // the next one.  Even warps take them in that order, odd warps in the other, so that at any time half of
        // the SM's warps walk the tables (16-byte shared-memory loads) while the other half multiply and add.
        const bool more = tile + 1 < tile1;
        for (int ph = 0; ph < 2; ++ph) {
            if (((ph ^ warp) & 1) == 0) value_tile(vcur);
            else if (more) score_tile(tile + 1);
        }
        if (a.vbufs > 1) buf ^= 1;
    }

    __syncthreads();   // last value phase over: pbuf and red are free
#pragma unroll
    for (int qq = 0; qq < QP; ++qq) {
        float v = l_part[qq];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) red[warp * QP + qq] = v;
    }
    // accumulators: lanes c, c + kCT, ... of a warp hold the same coordinates; warps are added through pbuf
    float res[QP];
#pragma unroll
    for (int qq = 0; qq < QP; ++qq) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            float v = acc[qq][u];
#pragma unroll
            for (int o = kCT; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane < kCT) pbuf[warp * DR + lane * 8 + u] = v;
        }
        __syncthreads();
        float sum = 0.f;
        if (t < DR) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) sum += pbuf[w * DR + t];
        }
        res[qq] = sum;
        __syncthreads();
    }
    if (t < DR) {
#pragma unroll
        for (int qq = 0; qq < QP; ++qq) {
            if (q0 + qq >= a.qpg) continue;
            float* dst = a.part + (((size_t)g * a.qpg + q0 + qq) * a.splits + split) * (DR + 2);
            dst[t] = res[qq];
            if (t == 0) {
                float l = 0.f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) l += red[w * QP + qq];
                dst[DR] = sm_m[qq];
                dst[DR + 1] = l;
            }
        }
    }
}

// One block per (group, query): merge the splits (weights 2^(m_s - M)), divide by the sum, and apply the value
// quantizer's rotation: out[j] = sum_k a[k] R[k][j] (the `@ self.rotation` of _quant.py:241).
__global__ void decode_combine_kernel(const float* __restrict__ part, int splits, int d, const float* __restrict__ Rv,
                                      float* __restrict__ out) {
    extern __shared__ float avec[];
    const int t = threadIdx.x;
    const float* pr = part + (size_t)blockIdx.x * splits * (d + 2);
    float M = -CUDART_INF_F;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, pr[(size_t)s * (d + 2) + d]);
    float L = 0.f, av = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float m = pr[(size_t)s * (d + 2) + d];
        const float w = m == -CUDART_INF_F ? 0.f : exp2f(m - M);
        L = fmaf(w, pr[(size_t)s * (d + 2) + d + 1], L);
        if (t < d) av = fmaf(w, pr[(size_t)s * (d + 2) + t], av);
    }
    if (t < d) avec[t] = L > 0.f ? av / L : 0.f;   // no keys at all: zeros
    __syncthreads();
    if (t < d) {
        float o = 0.f;
        for (int k0 = 0; k0 < d; k0 += 32) {   // d is 64 or 128; 32 matrix elements in flight
            float m[32];
#pragma unroll
            for (int u = 0; u < 32; ++u) m[u] = __ldg(Rv + (size_t)(k0 + u) * d + t);
#pragma unroll
            for (int u = 0; u < 32; ++u) o = fmaf(avec[k0 + u], m[u], o);
        }
        out[(size_t)blockIdx.x * d + t] = o;
    }
}

int queries_per_pass(int kbits, int qpg) { return qpg == 1 ? 1 : (kbits <= 3 ? 4 : 2); }

// One block is resident per SM, so blocks run in waves of `sms`.  Among the split counts that fill 1..4 waves,
// take the one with the fewest tile times per SM (a block's set-up counted as one tile).
int splits_for(int sms, int groups, int passes, int64_t keys_per_group) {
    const int64_t tiles = (keys_per_group + kTile - 1) / kTile;
    const int64_t gq = (int64_t)groups * passes;
    if (tiles <= 1 || gq <= 0) return 1;
    int64_t best = 1, best_cost = -1;
    for (int w = 1; w <= 4; ++w) {
        int64_t s = (int64_t)sms * w / gq;
        if (s < 1) s = 1;
        if (s > tiles) s = tiles;
        if (s > kMaxSplits) s = kMaxSplits;
        const int64_t waves = (gq * s + sms - 1) / sms;
        const int64_t cost = waves * ((tiles + s - 1) / s + 1);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
    }
    return (int)best;
}

int sm_count(int device) {
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms > 0 ? sms : 148;
}

template <int KB, int DR, int QP>
int launch_partial(const tq_plan* kp, DecodeArgs a, int groups, int passes, cudaStream_t st) {
    const size_t fixed = decode_smem_floats<KB, DR, QP>() * 4, vtile = (size_t)kTile * a.vwords * 4;
    a.vbufs = fixed + 2 * vtile <= 227 * 1024 ? 2 : 1;
    const size_t sm = fixed + a.vbufs * vtile;
    const dim3 grid((unsigned)a.splits, (unsigned)passes, (unsigned)groups);
    if (a.vbits == 3) {
        TQ_CUDA_TRY(cudaFuncSetAttribute(decode_partial_kernel<KB, DR, QP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        decode_partial_kernel<KB, DR, QP, true><<<grid, kThreads, sm, st>>>(kp->dev, a); tq_count_launch();
    } else {
        TQ_CUDA_TRY(cudaFuncSetAttribute(decode_partial_kernel<KB, DR, QP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        decode_partial_kernel<KB, DR, QP, false><<<grid, kThreads, sm, st>>>(kp->dev, a); tq_count_launch();
    }
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

template <int KB, int DR>
int launch_partial_qp(const tq_plan* kp, const DecodeArgs& a, int groups, int passes, int qp, cudaStream_t st) {
    if (qp == 1) return launch_partial<KB, DR, 1>(kp, a, groups, passes, st);
    if constexpr (KB <= 3) return launch_partial<KB, DR, 4>(kp, a, groups, passes, st);
    else return launch_partial<KB, DR, 2>(kp, a, groups, passes, st);
}

}  // namespace

bool tq_decode_attention_supported(const tq_plan* kp, const tq_plan* vp) {
    const int d = kp->dev.d;
    return kp->has_projection && vp->dev.d == d && (d == 128 || d == 64) && kp->dev.bits >= 1 && kp->dev.bits <= 4 &&
           vp->dev.bits >= 1 && vp->dev.bits <= 4;
}

int64_t tq_decode_attention_scratch(const tq_plan* kp, int groups, int qpg, int64_t keys_per_group) {
    const int qp = queries_per_pass(kp->dev.bits, qpg);
    const int passes = (qpg + qp - 1) / qp;
    const int splits = splits_for(sm_count(kp->device), groups, passes, keys_per_group);
    return (int64_t)groups * qpg * splits * (kp->dev.d + 2) * (int64_t)sizeof(float);
}

int tq_launch_decode_attention(const tq_plan* kp, const tq_plan* vp, const float* q, int groups, int qpg,
                               const uint32_t* kcodes, const uint32_t* ksigns, const float* krnorms, const float* knorms,
                               const uint32_t* vcodes, const float* vnorms, int64_t keys_per_group, int64_t group_rows,
                               const int64_t* length, float scale, float* out, void* scratch, size_t scratch_bytes,
                               cudaStream_t st) {
    TqRange range("tq.decode_attention");
    const int d = kp->dev.d, kb = kp->dev.bits;
    const int qp = queries_per_pass(kb, qpg);
    const int passes = (qpg + qp - 1) / qp;
    DecodeArgs a{};
    a.q = q; a.kcodes = kcodes; a.ksigns = ksigns; a.krnorms = krnorms; a.knorms = knorms;
    a.vcodes = vcodes; a.vnorms = vnorms; a.vcodebook = vp->dev.codebook;
    a.vbits = vp->dev.bits; a.vwords = vp->dev.code_words;
    a.qpg = qpg; a.keys_per_group = keys_per_group; a.group_rows = group_rows; a.length = length;
    a.scale_log2e = scale * 1.4426950408889634f;
    a.splits = splits_for(sm_count(kp->device), groups, passes, keys_per_group);
    a.part = static_cast<float*>(scratch);
    const size_t need = (size_t)groups * qpg * a.splits * (d + 2) * sizeof(float);
    if (!scratch || scratch_bytes < need)
        return tq_fail(TQ_ERR_SCRATCH_TOO_SMALL, "decode attention scratch: need %zu bytes, got %zu", need, scratch_bytes);
    int r = TQ_ERR_UNSUPPORTED;
#define TQ_DEC(B)                                                                                     \
    case B:                                                                                           \
        r = d == 64 ? launch_partial_qp<B, 64>(kp, a, groups, passes, qp, st)                          \
                    : launch_partial_qp<B, 128>(kp, a, groups, passes, qp, st);                        \
        break;
    switch (kb) { TQ_DEC(1) TQ_DEC(2) TQ_DEC(3) TQ_DEC(4) }
#undef TQ_DEC
    if (r != TQ_OK) return r;
    decode_combine_kernel<<<(unsigned)(groups * qpg), (d + 31) & ~31, d * sizeof(float), st>>>(a.part, a.splits, d, vp->dev.R, out); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}
