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
// second stage of the tensor-core quantizers, which hand over the rows they flagged (`rowmask`).
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

struct WarpBufs {
    float* a;
    float* b;
    uint8_t* c;
};

__device__ __forceinline__ WarpBufs warp_bufs(float* smem, int d, int warp) {
    const int dp = (d + 31) & ~31;
    float* base = smem + (size_t)warp * (2 * dp + dp / 4);
    WarpBufs w;
    w.a = base;
    w.b = base + dp;
    w.c = reinterpret_cast<uint8_t*>(base + 2 * dp);
    return w;
}

size_t smem_bytes(int d) {
    const int dp = (d + 31) & ~31;
    return (size_t)kWarps * (2 * dp + dp / 4) * sizeof(float);
}

// TurboQuantMSE.quantize / TurboQuantProd.quantize, array part (_quant.py:224-236, 300-308).
template <bool PROD>
__global__ void __launch_bounds__(kWarps * 32)
exact_quantize_kernel(TqDev p, const float* __restrict__ x, int64_t n, uint32_t* __restrict__ codes,
                      uint32_t* __restrict__ signs, float* __restrict__ rnorms, float* __restrict__ norms,
                      const uint32_t* __restrict__ rowmask, unsigned long long* redo_counter) {
    extern __shared__ float smem[];
    const int d = p.d, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const WarpBufs wb = warp_bufs(smem, d, warp);
    const int64_t nwords = (n + 31) >> 5;
    const int64_t wstride = (int64_t)gridDim.x * kWarps;

    for (int64_t wi = (int64_t)blockIdx.x * kWarps + warp; wi < nwords; wi += wstride) {
        uint32_t m = rowmask ? rowmask[wi] : 0xffffffffu;
        if (rowmask && m && lane == 0 && redo_counter) atomicAdd(redo_counter, (unsigned long long)__popc(m));
        while (m) {
            const int bit = __ffs(m) - 1;
            m &= m - 1;
            const int64_t row = wi * 32 + bit;
            if (row >= n) break;
            const float* xr = x + row * d;

            for (int k = lane; k < d; k += 32) {
                const float v = xr[k];
                wb.a[k] = v;
                wb.b[k] = __fmul_rn(v, v);
            }
            __syncwarp();
            const float nrm = __fsqrt_rn(np_pairwise_sum(wb.b, d, lane));
            const bool ok = nrm > 0.f;
            for (int k = lane; k < d; k += 32) wb.a[k] = ok ? __fdiv_rn(wb.a[k], nrm) : 0.f;
            __syncwarp();

            for (int j0 = 0; j0 < d; j0 += 128) {
                float acc[4];
                chain4(wb.a, p.Rt, d, j0, lane, acc);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int j = j0 + lane + 32 * c;
                    if (j < d) {
                        const int code = count_below(p.boundaries, p.levels - 1, acc[c]);
                        wb.c[j] = (uint8_t)code;
                        if (PROD) wb.b[j] = __ldg(p.codebook + code);
                    }
                }
            }
            __syncwarp();
            store_packed_codes(wb.c, d, p.bits, p.code_words, lane, codes + row * p.code_words);
            if (lane == 0) norms[row] = nrm;

            if (PROD) {
                for (int j0 = 0; j0 < d; j0 += 128) {
                    float acc[4];
                    chain4(wb.b, p.R, d, j0, lane, acc);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = j0 + lane + 32 * c;
                        if (j < d) wb.a[j] = __fsub_rn(wb.a[j], acc[c]);  // residual replaces unit
                    }
                }
                __syncwarp();
                for (int k = lane; k < d; k += 32) wb.b[k] = __fmul_rn(wb.a[k], wb.a[k]);
                __syncwarp();
                const float rn = __fsqrt_rn(np_pairwise_sum(wb.b, d, lane));
                if (lane == 0) rnorms[row] = rn;
                uint32_t* srow = signs + row * p.sign_words;
                for (int j0 = 0; j0 < d; j0 += 128) {
                    float acc[4];
                    chain4(wb.a, p.St, d, j0, lane, acc);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = j0 + lane + 32 * c;
                        const uint32_t word = __ballot_sync(0xffffffffu, j < d && acc[c] >= 0.f);
                        if (lane == 0 && j0 + 32 * c < d) srow[(j0 >> 5) + c] = tq_sign_word_from_natural(word);
                    }
                }
            }
            __syncwarp();
        }
    }
}

// TurboQuantMSE.dequantize / TurboQuantProd.dequantize (_quant.py:238-242,251-254,317-332).
template <bool PROD>
__global__ void __launch_bounds__(kWarps * 32)
exact_dequantize_kernel(TqDev p, const uint32_t* __restrict__ codes, const uint32_t* __restrict__ signs,
                        const float* __restrict__ rnorms, const float* __restrict__ norms, int64_t n,
                        float* __restrict__ out) {
    extern __shared__ float smem[];
    const int d = p.d, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const WarpBufs wb = warp_bufs(smem, d, warp);
    for (int64_t row = (int64_t)blockIdx.x * kWarps + warp; row < n; row += (int64_t)gridDim.x * kWarps) {
        const uint32_t* crow = codes + row * p.code_words;
        for (int k = lane; k < d; k += 32) {
            wb.a[k] = __ldg(p.codebook + tq_get_code(crow, k, p.bits));
            if (PROD) wb.b[k] = ((signs[row * p.sign_words + (k >> 5)] >> tq_sign_bitpos(k)) & 1u) ? 1.f : -1.f;
        }
        __syncwarp();
        const float nrm = norms[row];
        const float rn = PROD ? rnorms[row] : 0.f;
        for (int j0 = 0; j0 < d; j0 += 128) {
            float r[4], s[4];
            chain4(wb.a, p.R, d, j0, lane, r);
            if (PROD) chain4(wb.b, p.S, d, j0, lane, s);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = j0 + lane + 32 * c;
                if (j < d) {
                    float u = r[c];
                    if (PROD) u = __fadd_rn(u, __fmul_rn(__fmul_rn(s[c], p.alpha), rn));
                    out[row * d + j] = __fmul_rn(u, nrm);
                }
            }
        }
        __syncwarp();
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

int tq_launch_exact_quantize(const tq_plan* p, bool prod, const float* x, int64_t n, uint32_t* codes,
                             uint32_t* signs, float* rnorms, float* norms, const uint32_t* rowmask,
                             unsigned long long* redo_counter, cudaStream_t st) {
    if (n == 0) return TQ_OK;
    const size_t sm = smem_bytes(p->dev.d);
    const int grid = grid_for((n + 31) / 32, kWarps);
    if (prod) {
        TQ_CUDA_TRY(cudaFuncSetAttribute(exact_quantize_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        exact_quantize_kernel<true><<<grid, kWarps * 32, sm, st>>>(p->dev, x, n, codes, signs, rnorms, norms, rowmask, redo_counter);
    } else {
        TQ_CUDA_TRY(cudaFuncSetAttribute(exact_quantize_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        exact_quantize_kernel<false><<<grid, kWarps * 32, sm, st>>>(p->dev, x, n, codes, signs, rnorms, norms, rowmask, redo_counter);
    }
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

int tq_launch_exact_dequantize(const tq_plan* p, bool prod, const uint32_t* codes, const uint32_t* signs,
                               const float* rnorms, const float* norms, int64_t n, float* out,
                               cudaStream_t st) {
    if (n == 0) return TQ_OK;
    const size_t sm = smem_bytes(p->dev.d);
    const int grid = grid_for(n, kWarps);
    if (prod) {
        TQ_CUDA_TRY(cudaFuncSetAttribute(exact_dequantize_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        exact_dequantize_kernel<true><<<grid, kWarps * 32, sm, st>>>(p->dev, codes, signs, rnorms, norms, n, out);
    } else {
        TQ_CUDA_TRY(cudaFuncSetAttribute(exact_dequantize_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        exact_dequantize_kernel<false><<<grid, kWarps * 32, sm, st>>>(p->dev, codes, signs, rnorms, norms, n, out);
    }
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

int tq_launch_exact_pairwise(const tq_plan* p, const float* q, const uint32_t* codes, const uint32_t* signs,
                             const float* rnorms, const float* norms, int64_t n, float* scores,
                             cudaStream_t st) {
    if (n == 0) return TQ_OK;
    const int dp = (p->dev.d + 31) & ~31;
    const size_t sm = (size_t)kWarps * 3 * dp * sizeof(float);
    TQ_CUDA_TRY(cudaFuncSetAttribute(exact_pairwise_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    exact_pairwise_score_kernel<<<grid_for(n, kWarps), kWarps * 32, sm, st>>>(p->dev, q, codes, signs, rnorms, norms, n, scores);
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}
