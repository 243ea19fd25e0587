// attention_score for one or two queries per group of keys (the reference's own call pattern: one query broadcast
// over all keys, _quant.py:334-358), d = 128, 64 or 256, 1..4 code bits.
//
//   score(q, key) = norm * ( (R q) . codebook[codes]  +  alpha * rnorm * ((S q) . signs) )
//
// With so few queries the tensor-core kernel would idle most of each instruction (its cost does not shrink
// with the number of queries below 16), and the arithmetic is tiny: the call is bound by reading 72 bytes per
// key.  So this is a plain streaming kernel: per (group, query) the rotated and projected query are turned
// into two lookup tables in shared memory,
//
//   pair table   [d/2 positions][4^bits entries]   c[code0] * (R q)[2p] + c[code1] * (R q)[2p+1]
//   byte table   [d/8 positions][256 entries]      sum over the 8 sign bits of the byte of +-(S q)[coordinate]
//
// and every thread walks the packed codes and sign words of one key: d/2 + d/8 lookups and additions, no
// unpacking.  The sums run in another order than the reference's (table entries are pairs / octets of
// products), which keeps the scores within about 1e-6 relative of the float32 reference, inside the 1e-4 bound.
#include "tq_common.cuh"

#include <stdint.h>

namespace {

constexpr int kFewThreads = 256;

// grid (blocks over keys, queries per group, groups)
template <int BITS, int DR>
__global__ void __launch_bounds__(kFewThreads)
score_few_kernel(TqDev p, const float* __restrict__ q, const uint32_t* __restrict__ codes,
                 const uint32_t* __restrict__ signs, const float* __restrict__ rnorms, const float* __restrict__ norms,
                 int64_t keys_per_group, int64_t group_rows, int qpg, float* __restrict__ scores) {
    constexpr int kPairs = DR / 2, kEntries = 1 << (2 * BITS), kBytes = DR / 8;
    constexpr int kCodeWords = DR * BITS / 32, kSignWords = DR / 32;
    constexpr uint32_t kMask = kEntries - 1;
    extern __shared__ float tables[];
    float* pair_t = tables;                       // [kPairs][kEntries]
    float* byte_t = tables + kPairs * kEntries;   // [kBytes][256]
    const int g = blockIdx.z, qi = blockIdx.y;
    // Every block rotates and projects its query itself (2 d^2 FMAs, the matrices come from L2): rotated[j] =
    // sum_k q[k] R[j][k], projected[j] = sum_k q[k] S[j][k], one FMA per k, k ascending as in the reference's
    // matrix products.  That costs a few microseconds per block and saves a launch and a scratch buffer.
    __shared__ float qs[DR], qr[DR], ps[DR];
    if (threadIdx.x < DR) qs[threadIdx.x] = __ldg(q + ((size_t)g * qpg + qi) * DR + threadIdx.x);
    __syncthreads();
    if (threadIdx.x < DR) {
        const int j = threadIdx.x;
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
                r = fmaf(qs[k0 + u], mr[u], r);
                sacc = fmaf(qs[k0 + u], ms[u], sacc);
            }
        }
        qr[j] = r;
        ps[j] = sacc;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kPairs * kEntries; i += kFewThreads) {
        const int pp = i / kEntries, e = i - pp * kEntries;
        const float c0 = __ldg(p.codebook + (e & ((1 << BITS) - 1))), c1 = __ldg(p.codebook + (e >> BITS));
        pair_t[i] = fmaf(c1, qr[2 * pp + 1], c0 * qr[2 * pp]);
    }
    for (int i = threadIdx.x; i < kBytes * 256; i += kFewThreads) {
        const int pos = i >> 8, v = i & 255, w = pos >> 2, b = pos & 3;
        float acc = 0.f;
#pragma unroll
        for (int bit = 0; bit < 8; ++bit) {
            // stored order of the sign words: even coordinates in bits 0..15, odd ones in bits 16..31
            const int bp = 8 * b + bit;
            const int coord = 32 * w + (bp < 16 ? 2 * bp : 2 * (bp - 16) + 1);
            const float x = ps[coord];
            acc += (v >> bit) & 1 ? x : -x;
        }
        byte_t[i] = acc;
    }
    __syncthreads();

    const float alpha = p.alpha;
    float* out = scores + ((size_t)g * qpg + qi) * keys_per_group;
    for (int64_t key = (int64_t)blockIdx.x * kFewThreads + threadIdx.x; key < keys_per_group;
         key += (int64_t)gridDim.x * kFewThreads) {
        const int64_t row = (int64_t)g * group_rows + key;
        uint32_t cw[kCodeWords + 1], sw[kSignWords];
        const uint32_t* crow = codes + row * kCodeWords;
        const uint32_t* srow = signs + row * kSignWords;
        if (kCodeWords % 4 == 0) {
#pragma unroll
            for (int k = 0; k < kCodeWords; k += 4) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(crow + k));
                cw[k] = v.x; cw[k + 1] = v.y; cw[k + 2] = v.z; cw[k + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int k = 0; k < kCodeWords; k += 2) {
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(crow + k));
                cw[k] = v.x; cw[k + 1] = v.y;
            }
        }
        cw[kCodeWords] = 0u;
#pragma unroll
        for (int k = 0; k < kSignWords; k += 2) {
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(srow + k));
            sw[k] = v.x; sw[k + 1] = v.y;
        }
        const float nrm = __ldg(norms + row), rn = __ldg(rnorms + row);
        float s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[2] = {0.f, 0.f};
#pragma unroll
        for (int pp = 0; pp < kPairs; ++pp) {
            const int bit = pp * 2 * BITS, wi = bit >> 5, sh = bit & 31;
            uint32_t e;
            if (sh + 2 * BITS <= 32) e = (cw[wi] >> sh) & kMask;
            else e = __funnelshift_r(cw[wi], cw[wi + 1], sh) & kMask;
            s1[pp & 3] += pair_t[pp * kEntries + e];
        }
#pragma unroll
        for (int pos = 0; pos < kBytes; ++pos) s2[pos & 1] += byte_t[pos * 256 + ((sw[pos >> 2] >> (8 * (pos & 3))) & 255u)];
        const float a1 = (s1[0] + s1[1]) + (s1[2] + s1[3]);
        out[key] = nrm * fmaf(alpha * rn, s2[0] + s2[1], a1);
    }
}

template <int BITS, int DR>
int launch_few(const tq_plan* p, const float* q, const uint32_t* codes, const uint32_t* signs, const float* rnorms,
               const float* norms, int64_t keys_per_group, int64_t group_rows, int groups, int qpg, float* scores,
               cudaStream_t st) {
    const int sm = ((DR / 2) * (1 << (2 * BITS)) + (DR / 8) * 256) * 4;
    TQ_CUDA_TRY(cudaFuncSetAttribute(score_few_kernel<BITS, DR>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm));
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->device);
    int64_t blocks = (keys_per_group + kFewThreads - 1) / kFewThreads;
    const int64_t cap = (int64_t)sms * 4;   // the tables cost a few microseconds per block: a few blocks per SM, grid-stride
    if (blocks > cap) blocks = cap;
    score_few_kernel<BITS, DR><<<dim3((unsigned)blocks, (unsigned)qpg, (unsigned)groups), kFewThreads, sm, st>>>(
        p->dev, q, codes, signs, rnorms, norms, keys_per_group, group_rows, qpg, scores); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

}  // namespace

// d = 128 and 64: one or two queries (from three on, the lookup-table kernel for four and the tensor-core kernel are
// faster).  d = 256: one query (a pass over the packed keys per query; against 1,048,576 keys one query takes 145 us here
// and 201 us on the tensor-core kernel, two 228 and 200, four 394 and 194).
bool tq_score_few_supported(const tq_plan* p, int qpg) {
    if (!p->has_projection || p->dev.bits < 1 || p->dev.bits > 4 || qpg < 1) return false;
    if (p->dev.d == 256) return qpg == 1;
    return (p->dev.d == 128 || p->dev.d == 64) && qpg <= 2;
}

// scores: [groups][qpg][keys_per_group]
int tq_launch_score_few(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes, const uint32_t* signs,
                        const float* rnorms, const float* norms, int64_t keys_per_group, float* scores, cudaStream_t st,
                        int64_t group_rows) {
    TqRange range("tq.score.one_or_two_queries");
    if (group_rows <= 0) group_rows = keys_per_group;
    const int d = p->dev.d, bits = p->dev.bits;
    int r = TQ_ERR_UNSUPPORTED;
#define TQ_FEW(B)                                                                                                        \
    case B:                                                                                                             \
        r = d == 64 ? launch_few<B, 64>(p, q, codes, signs, rnorms, norms, keys_per_group, group_rows, groups, qpg, scores, st)     \
            : d == 256 ? launch_few<B, 256>(p, q, codes, signs, rnorms, norms, keys_per_group, group_rows, groups, qpg, scores, st) \
                       : launch_few<B, 128>(p, q, codes, signs, rnorms, norms, keys_per_group, group_rows, groups, qpg, scores, st); \
        break;
    switch (bits) { TQ_FEW(1) TQ_FEW(2) TQ_FEW(3) TQ_FEW(4) }
#undef TQ_FEW
    if (r == TQ_ERR_UNSUPPORTED) return tq_fail(r, "no few-query scoring kernel for d=%d bits=%d", d, bits);
    return r;
}
