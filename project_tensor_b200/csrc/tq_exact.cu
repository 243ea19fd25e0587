// Exact kernels: float32 arithmetic carried out in the same order as the reference's NumPy path
// (tensor_gpu_v2/_quant.py), so that decisions taken on a knife edge -- a rotated coordinate that
// sits on a codebook boundary, a QJL projection that is almost zero -- come out the same way.
//
// Order of operations that is reproduced here:
//   * row reductions (np.linalg.norm, np.sum(axis=1)) use NumPy's pairwise scheme: blocks of at
//     most 128 elements are summed with 8 interleaved accumulators combined as
//     ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)); longer rows are split recursively at n/2 rounded
//     down to a multiple of 8;
//   * matrix products (`@`, BLAS sgemm) accumulate each output element with one fused
//     multiply-add per k, k ascending, starting from zero;
//   * every other elementwise step is a separately rounded float32 operation (no contraction).
//
// One warp owns one row.  These kernels serve arbitrary (d <= 1024, bits <= 8); they are also the
// second stage of the tensor-core quantizers, which hand over lists of coordinates and rows to re-decide.
#include "tq_common.cuh"

namespace {

constexpr int kWarps = 4;

__device__ float np_pairwise_sum(const float* s, int n, int lane) {
    if (n < 8) {
        float r = 0.f;
        for (int i = 0; i < n; ++i) r = __fadd_rn(r, s[i]);
        return r;
    }
    if (n <= 128) {
        const int nb = n - (n & 7);
        float r = 0.f;
        if (lane < 8) {
            r = s[lane];
            for (int i = 8 + lane; i < nb; i += 8) r = __fadd_rn(r, s[i]);
        }
        r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 1));
        r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 2));
        r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 4));
        r = __shfl_sync(0xffffffffu, r, 0);
        for (int i = nb; i < n; ++i) r = __fadd_rn(r, s[i]);
        return r;
    }
    int h = n >> 1;
    h -= h & 7;
    const float a = np_pairwise_sum(s, h, lane);
    const float b = np_pairwise_sum(s + h, n - h, lane);
    return __fadd_rn(a, b);
}

// np.searchsorted(boundaries, v, side="left"): boundaries strictly below v; NaN sorts last.
__device__ __forceinline__ int count_below(const float* __restrict__ b, int nb, float v) {
    if (v != v) return nb;
    int lo = 0, hi = nb;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(b + mid) < v) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// out[j] = sum_k vec[k] * M[k*d + j] for the four columns j0+lane+{0,32,64,96}; FMA chain, k ascending.
__device__ __forceinline__ void chain4(const float* vec, const float* __restrict__ M, int d, int j0, int lane,
                                       float acc[4]) {
    int j[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        j[c] = j0 + lane + 32 * c;
        if (j[c] >= d) j[c] = d - 1;  // keep the load in bounds; the caller ignores the value
        acc[c] = 0.f;
    }
#pragma unroll 4
    for (int k = 0; k < d; ++k) {
        const float v = vec[k];
        const float* m = M + (size_t)k * d;
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[c] = __fmaf_rn(v, __ldg(m + j[c]), acc[c]);
    }
}

__device__ __forceinline__ void store_packed_codes(const uint8_t* cs, int d, int bits, int words, int lane,
                                                   uint32_t* out) {
    for (int w = lane; w < words; w += 32) {
        const int lo_bit = w * 32;
        uint32_t v = 0;
        for (int j = lo_bit / bits; j < d && j * bits < lo_bit + 32; ++j) {
            const int sh = j * bits - lo_bit;
            v |= sh >= 0 ? ((uint32_t)cs[j] << sh) : ((uint32_t)cs[j] >> (-sh));
        }
        out[w] = v;
    }
}

// TurboQuantMSE.quantize / TurboQuantProd.quantize, array part (_quant.py:224-236, 300-308).
// One block works on kRB rows at a time with one thread per output coordinate, so that every matrix
// element fetched from L1/L2 feeds kRB chains; the vectors sit in shared memory transposed ([k][row])
// and are read as broadcast float4s.
constexpr int kRB = 8;

struct RowsSmem {
    float* vt;      // [d][kRB]   unit vectors, later residuals (transposed)
    float* ct;      // [d][kRB]   centroid values (transposed)
    float* sq;      // [kRB][dp]  squares, row-major for the pairwise sums
    uint8_t* cs;    // [kRB][dp]  codes
    float* nrm;     // [kRB]
};
__host__ __device__ inline size_t rows_smem_bytes(int d) {
    const int dp = (d + 31) & ~31;
    return (size_t)(2 * d * kRB + kRB * dp + kRB) * sizeof(float) + (size_t)kRB * dp + 64;
}

// acc[r] = sum_k vt[k][r] * M[k * d + tj] for the kRB rows of a block: one FMA per k, k ascending.  The U matrix
// elements of a batch are fetched before the first of them is used -- written out as two loops because the
// chains wait on L2 latency, and whether the compiler hoists the loads of a single loop by itself changed the
// kernel's time by a factor of two from one build to the next.
template <int U>
__device__ __forceinline__ void rows_chain(const float* __restrict__ M, int d, int tj, const float* vt, float (&acc)[kRB]) {
#pragma unroll
    for (int r = 0; r < kRB; ++r) acc[r] = 0.f;
    int k0 = 0;
    for (; k0 + U <= d; k0 += U) {
        float m[U];
#pragma unroll
        for (int u = 0; u < U; ++u) m[u] = __ldg(M + (size_t)(k0 + u) * d + tj);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float4 a = *reinterpret_cast<const float4*>(vt + (k0 + u) * kRB);
            const float4 b = *reinterpret_cast<const float4*>(vt + (k0 + u) * kRB + 4);
            acc[0] = __fmaf_rn(a.x, m[u], acc[0]); acc[1] = __fmaf_rn(a.y, m[u], acc[1]);
            acc[2] = __fmaf_rn(a.z, m[u], acc[2]); acc[3] = __fmaf_rn(a.w, m[u], acc[3]);
            acc[4] = __fmaf_rn(b.x, m[u], acc[4]); acc[5] = __fmaf_rn(b.y, m[u], acc[5]);
            acc[6] = __fmaf_rn(b.z, m[u], acc[6]); acc[7] = __fmaf_rn(b.w, m[u], acc[7]);
        }
    }
    for (; k0 < d; ++k0) {
        const float m = __ldg(M + (size_t)k0 * d + tj);
        const float4 a = *reinterpret_cast<const float4*>(vt + k0 * kRB);
        const float4 b = *reinterpret_cast<const float4*>(vt + k0 * kRB + 4);
        acc[0] = __fmaf_rn(a.x, m, acc[0]); acc[1] = __fmaf_rn(a.y, m, acc[1]);
        acc[2] = __fmaf_rn(a.z, m, acc[2]); acc[3] = __fmaf_rn(a.w, m, acc[3]);
        acc[4] = __fmaf_rn(b.x, m, acc[4]); acc[5] = __fmaf_rn(b.y, m, acc[5]);
        acc[6] = __fmaf_rn(b.z, m, acc[6]); acc[7] = __fmaf_rn(b.w, m, acc[7]);
    }
}

// MAPPED: results go to the rows the append map names (a cache) instead of the input's own row numbers; a
// separate instantiation, so that the plain quantizer carries none of it.
// MAXT: the largest block the instantiation is launched with (d rounded up to 32).  The small one may use up to
// 255 registers and keeps 32 matrix elements in flight per thread (rows_chain).
template <bool PROD, bool MAPPED, int MAXT>
__global__ void __launch_bounds__(MAXT)
exact_quantize_kernel(TqDev p, const float* __restrict__ x, int64_t n, uint32_t* __restrict__ codes,
                      uint32_t* __restrict__ signs, float* __restrict__ rnorms, float* __restrict__ norms,
                      TqRecheck lists, unsigned long long* redo_counter, TqRowMap map) {
    extern __shared__ float smem[];
    const int d = p.d, dp = (d + 31) & ~31;
    const int64_t len0 = MAPPED ? *map.length : 0;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = blockDim.x >> 5;
    RowsSmem sm;
    sm.vt = smem;
    sm.ct = sm.vt + (size_t)d * kRB;
    sm.sq = sm.ct + (size_t)d * kRB;
    sm.nrm = sm.sq + (size_t)kRB * dp;
    sm.cs = reinterpret_cast<uint8_t*>(sm.nrm + kRB);
    const int tj = t < d ? t : d - 1;  // coordinate this thread computes (threads beyond d mirror the last one)

    // all rows, or the rows of the list (every row again if a list overflowed)
    const bool listed = lists.hdr != nullptr && lists.hdr->overflow == 0;
    const int64_t limit = listed ? (int64_t)min(lists.hdr->n_rows, lists.row_cap) : n;
    if (lists.hdr != nullptr && redo_counter && blockIdx.x == 0 && t == 0)
        *redo_counter = (unsigned long long)limit;     // rows redone by this call (a plain store: no clearing launch needed)

    for (int64_t g0 = (int64_t)blockIdx.x * kRB; g0 < limit; g0 += (int64_t)gridDim.x * kRB) {
        int64_t rows[kRB];                    // input rows (-1: none)
        int64_t mapped[MAPPED ? kRB : 1];     // MAPPED: the rows their results go to
#pragma unroll
        for (int r = 0; r < kRB; ++r) {
            const int64_t idx = g0 + r;
            int64_t row = idx < limit ? (listed ? (int64_t)lists.row_entries[idx] : idx) : -1;
            if (row >= n) row = -1;
            rows[r] = row;
            if (MAPPED) {
                mapped[r] = row;
                if (row >= 0) {
                    const int64_t grp = row / map.tokens, pos = len0 + (row - grp * map.tokens);
                    mapped[r] = pos < map.capacity ? grp * map.capacity + pos : -1;   // a full cache takes no more rows
                }
            }
        }
        const int64_t* orow = MAPPED ? mapped : rows;
        __syncthreads();  // previous group fully written out
#pragma unroll
        for (int r = 0; r < kRB; ++r) {
            const float v = (rows[r] >= 0 && t < d) ? x[rows[r] * d + t] : 0.f;
            if (t < dp) sm.sq[r * dp + t] = __fmul_rn(v, v);
            if (t < d) sm.vt[t * kRB + r] = v;
        }
        __syncthreads();
        for (int r = warp; r < kRB; r += nwarps) {
            const float nr = __fsqrt_rn(np_pairwise_sum(sm.sq + r * dp, d, lane));
            if (lane == 0) sm.nrm[r] = nr;
        }
        __syncthreads();
        if (t < d) {
#pragma unroll
            for (int r = 0; r < kRB; ++r) {
                const float nr = sm.nrm[r];
                sm.vt[t * kRB + r] = nr > 0.f ? __fdiv_rn(sm.vt[t * kRB + r], nr) : 0.f;
            }
        }
        __syncthreads();

        float acc[kRB];
        constexpr int kU = MAXT <= 256 ? 32 : 16;   // matrix elements in flight per thread (64 and 128 were slower: 50 and 62 us
                                                    // against 33 us for the listed rows of 1,048,576 keys)
        // rotated[j] = sum_k unit[k] * R[j][k]
        rows_chain<kU>(p.Rt, d, tj, sm.vt, acc);
        if (t < d) {
#pragma unroll
            for (int r = 0; r < kRB; ++r) {
                const int code = count_below(p.boundaries, p.levels - 1, acc[r]);
                sm.cs[r * dp + t] = (uint8_t)code;
                if (PROD) sm.ct[t * kRB + r] = __ldg(p.codebook + code);
            }
        }
        __syncthreads();
        for (int r = warp; r < kRB; r += nwarps) {
            if (orow[r] < 0) continue;
            store_packed_codes(sm.cs + r * dp, d, p.bits, p.code_words, lane, codes + orow[r] * p.code_words);
            if (lane == 0) norms[orow[r]] = sm.nrm[r];
        }

        if (PROD) {
            // recon[j] = sum_k centroid[k] * R[k][j];  residual = unit - recon
            rows_chain<kU>(p.R, d, tj, sm.ct, acc);
            __syncthreads();  // nobody reads unit[k] of other coordinates any more
#pragma unroll
            for (int r = 0; r < kRB; ++r) {
                const float res = t < d ? __fsub_rn(sm.vt[t * kRB + r], acc[r]) : 0.f;
                if (t < d) sm.vt[t * kRB + r] = res;
                if (t < dp) sm.sq[r * dp + t] = __fmul_rn(res, res);
            }
            __syncthreads();
            for (int r = warp; r < kRB; r += nwarps) {
                const float rn = __fsqrt_rn(np_pairwise_sum(sm.sq + r * dp, d, lane));
                if (lane == 0 && orow[r] >= 0) rnorms[orow[r]] = rn;
            }
            // projected[j] = sum_k residual[k] * S[j][k]
            rows_chain<kU>(p.St, d, tj, sm.vt, acc);
#pragma unroll
            for (int r = 0; r < kRB; ++r) {
                const uint32_t word = __ballot_sync(0xffffffffu, t < d && acc[r] >= 0.f);
                if (lane == 0 && orow[r] >= 0 && warp * 32 < d)
                    signs[orow[r] * p.sign_words + warp] = tq_sign_word_from_natural(word);
            }
        }
    }
}


// Second stage of the tensor-core quantizers, part 1: one thread per listed (row, coordinate).
// The coordinate's rotated value is recomputed exactly as the reference does (norm by pairwise sum,
// IEEE division, one FMA per k, k ascending) and its code re-decided.  If the stored code differs it is
// patched in place (MSE); for TurboQuantProd the residual of the whole row depends on it, so the
// row goes to the row list instead.  A list holds some ten thousand entries per million rows and a dependent access
// to global memory costs about a microsecond, so the kernel is as long as its chain of such accesses: header, entry,
// then the whole row into registers (D / 4 loads of 16 bytes in flight at once) together with the first half of the
// matrix row.  D is 64, 128 or 256 (the tensor-core geometries): the row sum is one block of NumPy's pairwise scheme
// (eight interleaved sums) per 128 values.
// Sum of squares of Q * 4 consecutive values as NumPy sums a block of its pairwise scheme (eight interleaved sums);
// the values stay in xv.
template <int Q>
__device__ __forceinline__ float block_sumsq(const float4* __restrict__ xr, float4 (&xv)[Q]) {
#pragma unroll
    for (int i = 0; i < Q; ++i) xv[i] = xr[i];
    float r8[8] = {__fmul_rn(xv[0].x, xv[0].x), __fmul_rn(xv[0].y, xv[0].y), __fmul_rn(xv[0].z, xv[0].z), __fmul_rn(xv[0].w, xv[0].w),
                   __fmul_rn(xv[1].x, xv[1].x), __fmul_rn(xv[1].y, xv[1].y), __fmul_rn(xv[1].z, xv[1].z), __fmul_rn(xv[1].w, xv[1].w)};
#pragma unroll
    for (int i = 2; i < Q; i += 2) {
        const float4 a = xv[i], b = xv[i + 1];
        r8[0] = __fadd_rn(r8[0], __fmul_rn(a.x, a.x)); r8[1] = __fadd_rn(r8[1], __fmul_rn(a.y, a.y));
        r8[2] = __fadd_rn(r8[2], __fmul_rn(a.z, a.z)); r8[3] = __fadd_rn(r8[3], __fmul_rn(a.w, a.w));
        r8[4] = __fadd_rn(r8[4], __fmul_rn(b.x, b.x)); r8[5] = __fadd_rn(r8[5], __fmul_rn(b.y, b.y));
        r8[6] = __fadd_rn(r8[6], __fmul_rn(b.z, b.z)); r8[7] = __fadd_rn(r8[7], __fmul_rn(b.w, b.w));
    }
    return __fadd_rn(__fadd_rn(__fadd_rn(r8[0], r8[1]), __fadd_rn(r8[2], r8[3])),
                     __fadd_rn(__fadd_rn(r8[4], r8[5]), __fadd_rn(r8[6], r8[7])));
}
// acc += sum over the Q * 4 values in xv of (value / nrm) * matrix value, one FMA per value, in order; the matrix row
// part comes in two batches of loads.
template <int Q>
__device__ __forceinline__ float block_chain(const float4 (&xv)[Q], const float4* __restrict__ rj, float nrm, bool ok, float acc) {
    float4 rv[Q / 2];
#pragma unroll
    for (int i = 0; i < Q / 2; ++i) rv[i] = __ldg(rj + i);
#pragma unroll
    for (int i = 0; i < Q; ++i) {
        if (i == Q / 2) {
#pragma unroll
            for (int u = 0; u < Q / 2; ++u) rv[u] = __ldg(rj + Q / 2 + u);
        }
        const float4 v = xv[i], m = rv[i % (Q / 2)];
        acc = __fmaf_rn(ok ? __fdiv_rn(v.x, nrm) : 0.f, m.x, acc);
        acc = __fmaf_rn(ok ? __fdiv_rn(v.y, nrm) : 0.f, m.y, acc);
        acc = __fmaf_rn(ok ? __fdiv_rn(v.z, nrm) : 0.f, m.z, acc);
        acc = __fmaf_rn(ok ? __fdiv_rn(v.w, nrm) : 0.f, m.w, acc);
    }
    return acc;
}

template <int D>
__global__ void __launch_bounds__(128)
exact_code_check_kernel(TqDev p, bool prod, const float* __restrict__ x, int64_t n, uint32_t* __restrict__ codes,
                        TqRecheck lists) {
    // D = 256: two neighbouring lanes share an entry, each with one half of the row in its registers (the halves are
    // also the two blocks of NumPy's pairwise sum for n = 256).  The chain runs over the first half in the even lane,
    // then over the second half in the odd lane, which decides.
    constexpr int LANES = D > 128 ? 2 : 1;                 // lanes per entry
    constexpr int H = D / LANES, Q = H / 4;
    const unsigned int t0 = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned int e0 = t0 / LANES;
    const int half = LANES == 2 ? (int)(threadIdx.x & 1u) : 0;
    // asked for before the header is known to allow it (the list's capacity bounds the index)
    unsigned long long ent = e0 < lists.code_cap ? lists.code_entries[e0] : 0ull;
    if (lists.hdr->overflow) return;  // the row pass will redo everything
    const unsigned int count = min(lists.hdr->n_codes, lists.code_cap);
    const unsigned int stride = gridDim.x * blockDim.x / LANES;
    // both lanes of a pair run the same number of passes (their e is the same), so the shuffles below are whole-warp
    for (unsigned int e = e0; e < ((count + 31u) & ~31u) + stride; e += stride) {
        if (__all_sync(0xffffffffu, e >= count)) break;
        const bool have = e < count;
        if (e != e0 && have) ent = lists.code_entries[e];
        const int64_t row = (int64_t)(ent >> 8);
        const int j = (int)(ent & 255u);
        const bool valid = have && row < n && j < D;
        const float4* xr = reinterpret_cast<const float4*>(x + (valid ? row : 0) * D) + half * Q;
        const float4* rj = reinterpret_cast<const float4*>(p.R + (size_t)(valid ? j : 0) * D) + half * Q;
        uint32_t* crow = codes + (valid ? row : 0) * p.code_words;
        const uint32_t old = tq_get_code(crow, valid ? j : 0, p.bits);
        float4 xv[Q];
        float acc;
        const float mine = block_sumsq<Q>(xr, xv);
        if (LANES == 1) {
            const float nrm = __fsqrt_rn(mine);
            acc = block_chain<Q>(xv, rj, nrm, nrm > 0.f, 0.f);
        } else {
            const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
            const float nrm = __fsqrt_rn(half == 0 ? __fadd_rn(mine, other) : __fadd_rn(other, mine));   // first half + second half
            const bool ok = nrm > 0.f;
            const float first = block_chain<Q>(xv, rj, nrm, ok, 0.f);                 // meaningful in the even lane
            const float carry = __shfl_xor_sync(0xffffffffu, first, 1);               // odd lane: the first half's sum
            acc = block_chain<Q>(xv, rj, nrm, ok, carry);                             // meaningful in the odd lane
            if (half == 0) continue;                                                  // the odd lane decides
        }
        if (!valid) continue;
        const uint32_t code = (uint32_t)count_below(p.boundaries, p.levels - 1, acc);
        if (old == code) continue;
        if (prod) {
            const unsigned int pos = atomicAdd(&lists.hdr->n_rows, 1u);
            if (pos < lists.row_cap) lists.row_entries[pos] = (unsigned int)row;
            else lists.hdr->overflow = 1u;
        } else {
            const uint32_t delta = old ^ code;
            const int bit = j * p.bits, w = bit >> 5, sh = bit & 31;
            atomicXor(crow + w, delta << sh);
            if (sh + p.bits > 32) atomicXor(crow + w + 1, delta >> (32 - sh));
        }
        atomicAdd(&lists.hdr->pad[0], 1u);  // diagnostic: codes the exact arithmetic decided differently
    }
}

// TurboQuantMSE.dequantize / TurboQuantProd.dequantize (_quant.py:238-242,251-254,317-332).
// Same block shape as the quantizer above: kRB rows per pass, one thread per output coordinate.
template <bool PROD>
__global__ void __launch_bounds__(1024)
exact_dequantize_kernel(TqDev p, const uint32_t* __restrict__ codes, const uint32_t* __restrict__ signs,
                        const float* __restrict__ rnorms, const float* __restrict__ norms, int64_t n,
                        float* __restrict__ out) {
    extern __shared__ float smem[];
    const int d = p.d, t = threadIdx.x;
    float* ct = smem;                        // [d][kRB] centroid values (transposed)
    float* st = ct + (size_t)d * kRB;        // [d][kRB] +-1 signs (transposed), Prod only
    const int tj = t < d ? t : d - 1;
    for (int64_t g0 = (int64_t)blockIdx.x * kRB; g0 < n; g0 += (int64_t)gridDim.x * kRB) {
        __syncthreads();
        if (t < d) {
#pragma unroll
            for (int r = 0; r < kRB; ++r) {
                const int64_t row = g0 + r;
                float c = 0.f, sg = 0.f;
                if (row < n) {
                    c = __ldg(p.codebook + tq_get_code(codes + row * p.code_words, t, p.bits));
                    if (PROD) sg = ((signs[row * p.sign_words + (t >> 5)] >> tq_sign_bitpos(t)) & 1u) ? 1.f : -1.f;
                }
                ct[t * kRB + r] = c;
                if (PROD) st[t * kRB + r] = sg;
            }
        }
        __syncthreads();
        float acc[kRB], acs[kRB];
#pragma unroll
        for (int r = 0; r < kRB; ++r) { acc[r] = 0.f; acs[r] = 0.f; }
#pragma unroll 8
        for (int k = 0; k < d; ++k) {
            const float m = __ldg(p.R + (size_t)k * d + tj);
            const float4 a = *reinterpret_cast<const float4*>(ct + k * kRB);
            const float4 b = *reinterpret_cast<const float4*>(ct + k * kRB + 4);
            acc[0] = __fmaf_rn(a.x, m, acc[0]); acc[1] = __fmaf_rn(a.y, m, acc[1]);
            acc[2] = __fmaf_rn(a.z, m, acc[2]); acc[3] = __fmaf_rn(a.w, m, acc[3]);
            acc[4] = __fmaf_rn(b.x, m, acc[4]); acc[5] = __fmaf_rn(b.y, m, acc[5]);
            acc[6] = __fmaf_rn(b.z, m, acc[6]); acc[7] = __fmaf_rn(b.w, m, acc[7]);
            if (PROD) {
                const float ms = __ldg(p.S + (size_t)k * d + tj);
                const float4 e = *reinterpret_cast<const float4*>(st + k * kRB);
                const float4 f = *reinterpret_cast<const float4*>(st + k * kRB + 4);
                acs[0] = __fmaf_rn(e.x, ms, acs[0]); acs[1] = __fmaf_rn(e.y, ms, acs[1]);
                acs[2] = __fmaf_rn(e.z, ms, acs[2]); acs[3] = __fmaf_rn(e.w, ms, acs[3]);
                acs[4] = __fmaf_rn(f.x, ms, acs[4]); acs[5] = __fmaf_rn(f.y, ms, acs[5]);
                acs[6] = __fmaf_rn(f.z, ms, acs[6]); acs[7] = __fmaf_rn(f.w, ms, acs[7]);
            }
        }
        if (t < d) {
#pragma unroll
            for (int r = 0; r < kRB; ++r) {
                const int64_t row = g0 + r;
                if (row < n) {
                    float u = acc[r];
                    if (PROD) u = __fadd_rn(u, __fmul_rn(__fmul_rn(acs[r], p.alpha), rnorms[row]));
                    out[row * d + t] = __fmul_rn(u, norms[row]);
                }
            }
        }
    }
}

// TurboQuantProd.attention_score with one query row per key (_quant.py:342-358), in the
// reference's own order: de-rotate the key, multiply by the query, pairwise-sum.
__global__ void __launch_bounds__(kWarps * 32)
exact_pairwise_score_kernel(TqDev p, const float* __restrict__ q, const uint32_t* __restrict__ codes,
                            const uint32_t* __restrict__ signs, const float* __restrict__ rnorms,
                            const float* __restrict__ norms, int64_t n, float* __restrict__ scores) {
    extern __shared__ float smem[];
    const int d = p.d, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int dp = (d + 31) & ~31;
    float* qa = smem + (size_t)warp * 3 * dp;  // query row
    float* ca = qa + dp;                       // centroid values, then products
    float* pa = ca + dp;                       // products of the second stage
    for (int64_t row = (int64_t)blockIdx.x * kWarps + warp; row < n; row += (int64_t)gridDim.x * kWarps) {
        const uint32_t* crow = codes + row * p.code_words;
        const uint32_t* srow = signs + row * p.sign_words;
        for (int k = lane; k < d; k += 32) {
            qa[k] = q[row * d + k];
            ca[k] = __ldg(p.codebook + tq_get_code(crow, k, p.bits));
        }
        __syncwarp();
        float t1[32], t2[32];  // d <= 1024 -> at most 32 columns per lane
        int cnt = 0;
        for (int j0 = 0; j0 < d; j0 += 128) {
            float r[4], s[4];
            chain4(ca, p.R, d, j0, lane, r);
            chain4(qa, p.St, d, j0, lane, s);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = j0 + lane + 32 * c;
                float a = 0.f, b = 0.f;
                if (j < d) {
                    a = __fmul_rn(qa[j], r[c]);
                    b = ((srow[j >> 5] >> tq_sign_bitpos(j)) & 1u) ? s[c] : -s[c];
                }
                t1[cnt] = a;
                t2[cnt] = b;
                ++cnt;
            }
        }
        __syncwarp();
        cnt = 0;
        for (int j0 = 0; j0 < d; j0 += 128) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = j0 + lane + 32 * c;
                if (j < d) { ca[j] = t1[cnt]; pa[j] = t2[cnt]; }
                ++cnt;
            }
        }
        __syncwarp();
        const float s1 = np_pairwise_sum(ca, d, lane);
        const float s2 = np_pairwise_sum(pa, d, lane);
        if (lane == 0) {
            const float st2 = __fmul_rn(__fmul_rn(p.alpha, rnorms[row]), s2);
            scores[row] = __fmul_rn(norms[row], __fadd_rn(s1, st2));
        }
        __syncwarp();
    }
}

int grid_for(int64_t work_items, int per_block) {
    int64_t g = (work_items + per_block - 1) / per_block;
    const int64_t cap = 148 * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace

int tq_launch_exact_code_check(const tq_plan* p, bool prod, const float* x, int64_t n, uint32_t* codes,
                               const TqRecheck* lists, cudaStream_t st) {
    TqRange range("tq.quantize.recheck_coordinates");
    if (n == 0) return TQ_OK;
    // as many threads as a list of typical length has entries (about 1 in 50 rows of 128 coordinates at 4 bits, in
    // proportion to the coordinates); longer lists take more passes
    int64_t blocks = (n * p->dev.d / 128 / 48 * (p->dev.d > 128 ? 2 : 1) + 127) / 128;   // d = 256: two lanes per entry
    blocks = blocks < 8 ? 8 : (blocks > 148 * 8 ? 148 * 8 : blocks);
    if (p->dev.d == 128) exact_code_check_kernel<128><<<(int)blocks, 128, 0, st>>>(p->dev, prod, x, n, codes, *lists);
    else if (p->dev.d == 64) exact_code_check_kernel<64><<<(int)blocks, 128, 0, st>>>(p->dev, prod, x, n, codes, *lists);
    else if (p->dev.d == 256) exact_code_check_kernel<256><<<(int)blocks, 128, 0, st>>>(p->dev, prod, x, n, codes, *lists);
    else return tq_fail(TQ_ERR_UNSUPPORTED, "the coordinate re-check is written for d = 64, 128 and 256");
    tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

int tq_launch_exact_quantize(const tq_plan* p, bool prod, const float* x, int64_t n, uint32_t* codes,
                             uint32_t* signs, float* rnorms, float* norms, const TqRecheck* lists_in,
                             unsigned long long* redo_counter, cudaStream_t st, const TqRowMap* map_in) {
    TqRange range("tq.quantize.exact_rows");
    if (n == 0) return TQ_OK;
    const size_t sm = rows_smem_bytes(p->dev.d);
    const TqRowMap map = map_in ? *map_in : TqRowMap{0, 0, nullptr};
    TqRecheck none{};
    const TqRecheck lists = lists_in ? *lists_in : none;
    // the listed pass does not know its size on the host: a fixed grid strides over the list
    const int grid = lists_in ? 148 * 4 : grid_for(n, kRB);
    const int threads = (p->dev.d + 31) & ~31;
#define TQ_LAUNCH_EXACT(P, M, T)                                                                                           \
    do {                                                                                                                  \
        TQ_CUDA_TRY(cudaFuncSetAttribute(exact_quantize_kernel<P, M, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)); \
        exact_quantize_kernel<P, M, T><<<grid, threads, sm, st>>>(p->dev, x, n, codes, signs, rnorms, norms, lists, redo_counter, map); tq_count_launch(); \
    } while (0)
#define TQ_LAUNCH_EXACT_T(P, M)                  \
    do {                                         \
        if (threads <= 256) TQ_LAUNCH_EXACT(P, M, 256); \
        else TQ_LAUNCH_EXACT(P, M, 1024);        \
    } while (0)
    const bool mapped = map.tokens > 0;
    if (prod) {
        if (mapped) TQ_LAUNCH_EXACT_T(true, true);
        else TQ_LAUNCH_EXACT_T(true, false);
    } else {
        if (mapped) TQ_LAUNCH_EXACT_T(false, true);
        else TQ_LAUNCH_EXACT_T(false, false);
    }
#undef TQ_LAUNCH_EXACT_T
#undef TQ_LAUNCH_EXACT
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

__global__ void append_advance_kernel(int64_t* length, int64_t tokens, int64_t capacity) {
    const int64_t v = *length + tokens;
    *length = v < capacity ? v : capacity;
}

int tq_launch_append_advance(int64_t* length, int64_t tokens, int64_t capacity, cudaStream_t st) {
    append_advance_kernel<<<1, 1, 0, st>>>(length, tokens, capacity); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

int tq_launch_exact_dequantize(const tq_plan* p, bool prod, const uint32_t* codes, const uint32_t* signs,
                               const float* rnorms, const float* norms, int64_t n, float* out,
                               cudaStream_t st) {
    TqRange range("tq.dequantize.exact");
    if (n == 0) return TQ_OK;
    const int d = p->dev.d;
    const size_t sm = (size_t)2 * d * kRB * sizeof(float);
    const int grid = grid_for(n, kRB);
    const int threads = (d + 31) & ~31;
    if (prod) {
        TQ_CUDA_TRY(cudaFuncSetAttribute(exact_dequantize_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        exact_dequantize_kernel<true><<<grid, threads, sm, st>>>(p->dev, codes, signs, rnorms, norms, n, out); tq_count_launch();
    } else {
        TQ_CUDA_TRY(cudaFuncSetAttribute(exact_dequantize_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        exact_dequantize_kernel<false><<<grid, threads, sm, st>>>(p->dev, codes, signs, rnorms, norms, n, out); tq_count_launch();
    }
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

int tq_launch_exact_pairwise(const tq_plan* p, const float* q, const uint32_t* codes, const uint32_t* signs,
                             const float* rnorms, const float* norms, int64_t n, float* scores,
                             cudaStream_t st) {
    TqRange range("tq.score.pairwise.exact");
    if (n == 0) return TQ_OK;
    const int dp = (p->dev.d + 31) & ~31;
    const size_t sm = (size_t)kWarps * 3 * dp * sizeof(float);
    TQ_CUDA_TRY(cudaFuncSetAttribute(exact_pairwise_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    exact_pairwise_score_kernel<<<grid_for(n, kWarps), kWarps * 32, sm, st>>>(p->dev, q, codes, signs, rnorms, norms, n, scores); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}
