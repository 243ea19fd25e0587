// Scoring kernels for TurboQuantProd encodings (any d <= 1024, bits <= 8).
//
// score(q, key i) = norms[i] * ( (R q) . codebook[codes_i]  +  alpha * residual_norms[i] * ((S q) . qjl_i) )
//
// which is TurboQuantProd.attention_score (_quant.py:347-357) with the inverse rotation moved from
// the keys to the query: q . (codebook[codes] R) == (R q) . codebook[codes].  The reference
// de-rotates every key on every call; here the query is rotated and projected once per block into
// shared memory and the packed keys are streamed once.
//
// Optional fused per-query top-k: every block keeps, per query, a candidate buffer in shared
// memory with a rising threshold, prunes it with a bitonic sort when it fills, and writes its k
// best (score, row) pairs as 64-bit sortable keys; a second kernel merges the per-block lists.
#include "tq_common.cuh"
#include "tq_topk.cuh"

#include <math.h>

namespace {

constexpr int kThreads = 128;
constexpr int kQT = 8;  // queries scored together per pass over a block's keys

using namespace tqtopk;

__global__ void __launch_bounds__(kThreads)
score_kernel(TqDev p, const float* __restrict__ q, int qpg, const uint32_t* __restrict__ codes,
             const uint32_t* __restrict__ signs, const float* __restrict__ rnorms,
             const float* __restrict__ norms, int64_t keys_per_group, int64_t group_rows, int64_t keys_per_block,
             float* __restrict__ scores, int topk, int cap2, unsigned long long* __restrict__ part) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int d = p.d;
    float* qraw = reinterpret_cast<float*>(smraw);       // [kQT][d]   raw queries
    float* qs = qraw + kQT * d;                           // [kQT][2][d] rotated | projected
    float* cb = qs + kQT * 2 * d;                         // [256] codebook
    unsigned long long* buf = reinterpret_cast<unsigned long long*>(cb + 256);  // [kQT][cap2]
    __shared__ int cnt[kQT];
    __shared__ unsigned long long thr[kQT];
    __shared__ int need_prune;

    const int g = blockIdx.y;
    const int64_t k0 = (int64_t)blockIdx.x * keys_per_block;
    int64_t k1 = k0 + keys_per_block;
    if (k1 > keys_per_group) k1 = keys_per_group;
    const int64_t gbase = (int64_t)g * group_rows;  // first row of this group in the key arrays

    for (int i = threadIdx.x; i < 256; i += kThreads) cb[i] = i < p.levels ? p.codebook[i] : 0.f;

    for (int q0 = 0; q0 < qpg; q0 += kQT) {
        const int nq = min(kQT, qpg - q0);
        __syncthreads();
        for (int i = threadIdx.x; i < kQT * d; i += kThreads) {
            const int t = i / d;
            qraw[i] = t < nq ? q[((int64_t)g * qpg + q0 + t) * d + (i - t * d)] : 0.f;
        }
        if (threadIdx.x < kQT) { cnt[threadIdx.x] = 0; thr[threadIdx.x] = 0ull; }
        if (threadIdx.x == 0) need_prune = 0;
        __syncthreads();
        // rotated / projected queries: qs[t][0][j] = sum_k R[j][k] q[k],  qs[t][1][j] = sum_k S[j][k] q[k]
        for (int i = threadIdx.x; i < kQT * 2 * d; i += kThreads) {
            const int t = i / (2 * d), r = i - t * 2 * d, which = r / d, j = r - which * d;
            const float* M = which ? p.St : p.Rt;
            const float* qv = qraw + t * d;
            float acc = 0.f;
            for (int k = 0; k < d; ++k) acc = fmaf(qv[k], __ldg(M + (size_t)k * d + j), acc);
            qs[i] = acc;
        }
        __syncthreads();

        for (int64_t kb = k0; kb < k1; kb += kThreads) {
            const int64_t key = kb + threadIdx.x;
            const bool live = key < k1;
            float a1[kQT], a2[kQT];
#pragma unroll
            for (int t = 0; t < kQT; ++t) { a1[t] = 0.f; a2[t] = 0.f; }
            if (live) {
                const uint32_t* crow = codes + (gbase + key) * p.code_words;
                const uint32_t* srow = signs + (gbase + key) * p.sign_words;
                uint32_t sw = 0;
                for (int j = 0; j < d; ++j) {
                    if ((j & 31) == 0) sw = srow[j >> 5];
                    const float c = cb[tq_get_code(crow, j, p.bits)];
                    const float s = (sw >> tq_sign_bitpos(j)) & 1u ? 1.f : -1.f;
#pragma unroll
                    for (int t = 0; t < kQT; ++t) {
                        a1[t] = fmaf(c, qs[(t * 2) * d + j], a1[t]);
                        a2[t] = fmaf(s, qs[(t * 2 + 1) * d + j], a2[t]);
                    }
                }
                const float nrm = norms[gbase + key];
                const float arn = p.alpha * rnorms[gbase + key];
#pragma unroll
                for (int t = 0; t < kQT; ++t) {
                    if (t < nq) {
                        const float s = nrm * (a1[t] + arn * a2[t]);
                        if (scores) scores[((int64_t)g * qpg + q0 + t) * keys_per_group + key] = s;
                        if (topk > 0) {
                            const unsigned long long ck = make_key(s, (uint32_t)(gbase + key));
                            if (ck > thr[t]) {
                                const int pos = atomicAdd(&cnt[t], 1);
                                buf[(size_t)t * cap2 + pos] = ck;  // capacity is guaranteed by the prune rule
                            }
                        }
                    }
                }
            }
            if (topk > 0) {
                __syncthreads();
                if (threadIdx.x < nq && cnt[threadIdx.x] + kThreads > cap2) need_prune = 1;
                __syncthreads();
                if (need_prune) {
                    for (int t = 0; t < nq; ++t) {
                        const int c = cnt[t];
                        if (c + kThreads > cap2) {
                            unsigned long long* b = buf + (size_t)t * cap2;
                            for (int i = c + threadIdx.x; i < cap2; i += kThreads) b[i] = 0ull;
                            block_sort_desc(b, cap2);
                            if (threadIdx.x == 0) { cnt[t] = topk; thr[t] = b[topk - 1]; }
                        }
                    }
                    __syncthreads();
                    if (threadIdx.x == 0) need_prune = 0;
                    __syncthreads();
                }
            }
        }
        if (topk > 0) {
            __syncthreads();
            for (int t = 0; t < nq; ++t) {
                const int c = cnt[t];
                unsigned long long* b = buf + (size_t)t * cap2;
                for (int i = c + threadIdx.x; i < cap2; i += kThreads) b[i] = 0ull;
                block_sort_desc(b, cap2);
                unsigned long long* dst = part + (((size_t)g * gridDim.x + blockIdx.x) * qpg + q0 + t) * topk;
                for (int i = threadIdx.x; i < topk; i += kThreads) dst[i] = b[i];
            }
        }
    }
}

// Merge `lists` lists of `topk` sortable keys per query into the final top-k.
// part: [groups][lists][qpg][topk]; one block per (query, group).  Lists are loaded in batches into a
// shared buffer that is cut back to the k best by radix select whenever it fills; one final sort.
__global__ void __launch_bounds__(256)
merge_keys_kernel(const unsigned long long* __restrict__ part, int lists, int qpg, int topk, int k2,
                  int64_t idx_base, float* __restrict__ top_scores, int64_t* __restrict__ top_idx) {
    __shared__ __align__(16) unsigned long long a[kSelCap];
    __shared__ int hist[256];
    __shared__ int scratch[4];
    __shared__ int count;
    __shared__ unsigned long long thr;   // keys at or below it cannot be among the k best any more
    const int qi = blockIdx.x, g = blockIdx.y;
    if (threadIdx.x == 0) { count = 0; thr = 0ull; }
    __syncthreads();
    // all slots of all lists in batches, whatever the number of lists (some callers bring hundreds of short
    // ones, mostly empty)
    const int total = lists * topk;
    constexpr int kBatch = 2048;
    for (int base = 0; base < total; base += kBatch) {
        if (count + kBatch > kSelCap) {  // uniform: count only changes between barriers
            const int c = count;
            __syncthreads();
            if (c > topk) {
                const unsigned long long kth = block_select_topk(a, c, topk, hist, scratch);
                if (threadIdx.x == 0) { count = topk; thr = kth; }
            }
            __syncthreads();
        }
        const unsigned long long t = thr;
        const int end = base + kBatch < total ? base + kBatch : total;
        // empty slots (0) are left out, so every key in the buffer is distinct
        for (int i = base + threadIdx.x; i < end; i += blockDim.x) {
            const int l = i / topk, j = i - l * topk;
            const unsigned long long v = part[(((size_t)g * lists + l) * qpg + qi) * topk + j];
            if (v > t) a[atomicAdd(&count, 1)] = v;   // also drops the empty slots
        }
        __syncthreads();
    }
    const int c = count;
    const int keep = c < topk ? c : topk;
    if (keep < c) block_select_topk(a, c, keep, hist, scratch);
    __syncthreads();
    for (int i = keep + threadIdx.x; i < k2; i += blockDim.x) a[i] = 0ull;
    block_sort_desc(a, k2);
    for (int i = threadIdx.x; i < topk; i += blockDim.x) {
        const unsigned long long ck = a[i];
        const size_t o = ((size_t)g * qpg + qi) * topk + i;
        if (ck == 0ull) {
            top_scores[o] = -INFINITY;
            top_idx[o] = -1;
        } else {
            top_scores[o] = unordered_bits((uint32_t)(ck >> 32));
            top_idx[o] = idx_base + (int64_t)(0xffffffffu - (uint32_t)ck);
        }
    }
}

// Merge (score, index) lists gathered from several shards: [lists][queries][topk] -> [queries][topk].
__global__ void __launch_bounds__(256)
merge_pairs_kernel(const float* __restrict__ in_scores, const int64_t* __restrict__ in_idx, int lists,
                   size_t score_list_stride, size_t idx_list_stride, int queries, int topk, int k2,
                   float* __restrict__ out_scores, int64_t* __restrict__ out_idx) {
    extern __shared__ __align__(16) unsigned char smraw[];
    unsigned long long* a = reinterpret_cast<unsigned long long*>(smraw);  // [2*k2]
    const int qi = blockIdx.x;
    for (int i = threadIdx.x; i < 2 * k2; i += blockDim.x) a[i] = 0ull;
    __syncthreads();
    for (int l = 0; l < lists; ++l) {
        const size_t row = (size_t)qi * topk;   // lists may lie apart (one block per rank after an all-gather)
        for (int i = threadIdx.x; i < k2; i += blockDim.x) {
            unsigned long long ck = 0ull;
            // position in the concatenation of all lists stands in for the index: earlier list and
            // earlier slot win ties, which is ascending row order for contiguous shards
            if (i < topk && in_idx[l * idx_list_stride + row + i] >= 0)
                ck = make_key(in_scores[l * score_list_stride + row + i], (uint32_t)(l * topk + i));
            a[k2 + i] = ck;
        }
        block_sort_desc(a, 2 * k2);
    }
    for (int i = threadIdx.x; i < topk; i += blockDim.x) {
        const unsigned long long ck = a[i];
        const size_t o = (size_t)qi * topk + i;
        if (ck == 0ull) {
            out_scores[o] = -INFINITY;
            out_idx[o] = -1;
        } else {
            const uint32_t pos = 0xffffffffu - (uint32_t)ck;
            const size_t l = pos / topk, src = (size_t)qi * topk + (pos % topk);
            out_scores[o] = in_scores[l * score_list_stride + src];
            out_idx[o] = in_idx[l * idx_list_stride + src];
        }
    }
}

int pow2_at_least(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

struct ScoreGeometry {
    int nblk;
    int64_t keys_per_block;
    int cap2;
};

ScoreGeometry geometry(int groups, int64_t keys_per_group, int topk) {
    ScoreGeometry s;
    int64_t want = (148 * 8 + groups - 1) / groups;  // about 8 blocks per SM over all groups
    int64_t maxb = (keys_per_group + kThreads - 1) / kThreads;
    if (want > maxb) want = maxb;
    if (want < 1) want = 1;
    int64_t kpb = (keys_per_group + want - 1) / want;
    kpb = (kpb + kThreads - 1) / kThreads * kThreads;
    if (kpb < kThreads) kpb = kThreads;
    s.keys_per_block = kpb;
    s.nblk = (int)((keys_per_group + kpb - 1) / kpb);
    if (s.nblk < 1) s.nblk = 1;
    s.cap2 = topk > 0 ? pow2_at_least(topk + kThreads) : 0;
    return s;
}

}  // namespace

int64_t tq_score_tc_scratch(int groups, int qpg, int64_t keys_per_group, int topk);
int tq_launch_score_tc(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes,
                       const uint32_t* signs, const float* rnorms, const float* norms, int64_t keys_per_group,
                       float* scores, int topk, float* top_scores, int64_t* top_idx, int64_t idx_base, void* scratch,
                       size_t scratch_bytes, cudaStream_t st, int64_t group_rows);

static bool use_tensor_scoring(const tq_plan* p) {
    return p->path != TQ_PATH_EXACT && p->has_projection && tq_tensor_quantize_supported(p->dev.d, p->dev.bits, true);
}

static int64_t general_topk_scratch(int groups, int qpg, int64_t keys_per_group, int topk) {
    if (topk <= 0) return 0;
    const ScoreGeometry s = geometry(groups, keys_per_group, topk);
    return (int64_t)groups * s.nblk * qpg * topk * (int64_t)sizeof(unsigned long long);
}

int64_t tq_score_topk_scratch(const tq_plan* p, int groups, int qpg, int64_t keys_per_group, int topk) {
    const int64_t a = general_topk_scratch(groups, qpg, keys_per_group, topk);
    const int64_t b = tq_tensor_quantize_supported(p->dev.d, p->dev.bits, true) ? tq_score_tc_scratch(groups, qpg, keys_per_group, topk) : 0;
    return a > b ? a : b;
}

int tq_merge_keys_launch(const unsigned long long* part, int lists, int qpg, int groups, int topk, int64_t idx_base,
                         float* top_scores, int64_t* top_idx, cudaStream_t st) {
    const int k2 = pow2_at_least(topk);
    merge_keys_kernel<<<dim3(qpg, groups), 256, 0, st>>>(part, lists, qpg, topk, k2,
                                                                                           idx_base, top_scores, top_idx); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}

int tq_launch_score_batched(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes,
                            const uint32_t* signs, const float* rnorms, const float* norms,
                            int64_t keys_per_group, float* scores, int topk, float* top_scores,
                            int64_t* top_idx, int64_t idx_base, void* scratch, size_t scratch_bytes,
                            cudaStream_t st, int64_t group_rows) {
    if (group_rows <= 0) group_rows = keys_per_group;
    // One or two queries per group and the matrix wanted (the reference's own call): the streaming kernel.
    if (p->path == TQ_PATH_AUTO && topk == 0 && scores && tq_score_few_supported(p, qpg) && keys_per_group > 0 && groups > 0)
        return tq_launch_score_few(p, q, groups, qpg, codes, signs, rnorms, norms, keys_per_group, scores, st, group_rows);
    // Three or four queries per group (grouped-query decode): the lane-interleaved lookup-table kernel.
    if (p->path == TQ_PATH_AUTO && topk == 0 && scores && tq_score_lut_supported(p, qpg) && keys_per_group > 0 && groups > 0)
        return tq_launch_score_lut(p, q, groups, qpg, codes, signs, rnorms, norms, keys_per_group, scores, st, group_rows);
    // d = 64 has 8-byte sign rows (and 8- or 24-byte code rows): a group must start on a 16-byte boundary
    // for the bulk copies of the tensor-core kernel
    const bool aligned_groups = p->dev.d >= 128 || groups == 1 || group_rows % 2 == 0;
    if (use_tensor_scoring(p) && aligned_groups && keys_per_group > 0 && groups > 0 && qpg > 0)
        return tq_launch_score_tc(p, q, groups, qpg, codes, signs, rnorms, norms, keys_per_group, scores, topk, top_scores,
                                  top_idx, idx_base, scratch, scratch_bytes, st, group_rows);
    return tq_launch_score_general(p, q, groups, qpg, codes, signs, rnorms, norms, keys_per_group, scores, topk,
                                   top_scores, top_idx, idx_base, scratch, scratch_bytes, st, group_rows);
}

int tq_launch_score_general(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes,
                            const uint32_t* signs, const float* rnorms, const float* norms,
                            int64_t keys_per_group, float* scores, int topk, float* top_scores,
                            int64_t* top_idx, int64_t idx_base, void* scratch, size_t scratch_bytes,
                            cudaStream_t st, int64_t group_rows) {
    TqRange range("tq.score.general");
    if (group_rows <= 0) group_rows = keys_per_group;
    const ScoreGeometry s = geometry(groups, keys_per_group, topk);
    if (topk > 0) {
        const int64_t need = general_topk_scratch(groups, qpg, keys_per_group, topk);
        if (!scratch || (int64_t)scratch_bytes < need)
            return tq_fail(TQ_ERR_SCRATCH_TOO_SMALL, "top-k scratch: need %lld bytes, got %zu", (long long)need, scratch_bytes);
    }
    if (keys_per_group == 0 || groups == 0 || qpg == 0) {
        if (topk > 0 && groups > 0 && qpg > 0) {
            // no keys: every slot is empty
            const size_t cnt = (size_t)groups * qpg * topk;
            TQ_CUDA_TRY(cudaMemsetAsync(scratch, 0, cnt * sizeof(unsigned long long), st));
            merge_keys_kernel<<<dim3(qpg, groups), 256, 0, st>>>(
                static_cast<unsigned long long*>(scratch), 1, qpg, topk, pow2_at_least(topk), idx_base, top_scores, top_idx); tq_count_launch();
            TQ_CUDA_TRY(cudaGetLastError());
        }
        return TQ_OK;
    }
    const int d = p->dev.d;
    const size_t sm = (size_t)(kQT * d + kQT * 2 * d + 256) * sizeof(float) + (size_t)kQT * s.cap2 * sizeof(unsigned long long);
    if (sm > 200 * 1024) return tq_fail(TQ_ERR_UNSUPPORTED, "score kernel needs %zu bytes of shared memory", sm);
    TQ_CUDA_TRY(cudaFuncSetAttribute(score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    score_kernel<<<dim3(s.nblk, groups), kThreads, sm, st>>>(p->dev, q, qpg, codes, signs, rnorms, norms,
                                                             keys_per_group, group_rows, s.keys_per_block, scores, topk, s.cap2,
                                                             static_cast<unsigned long long*>(scratch)); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    if (topk > 0) {
        const int k2 = pow2_at_least(topk);
        merge_keys_kernel<<<dim3(qpg, groups), 256, 0, st>>>(
            static_cast<unsigned long long*>(scratch), s.nblk, qpg, topk, k2, idx_base, top_scores, top_idx); tq_count_launch();
        TQ_CUDA_TRY(cudaGetLastError());
    }
    return TQ_OK;
}

int tq_launch_topk_merge(const float* in_scores, const int64_t* in_idx, int lists, int queries, int topk,
                         float* out_scores, int64_t* out_idx, cudaStream_t st, int64_t score_list_stride,
                         int64_t idx_list_stride) {
    TqRange range("tq.topk.merge");
    if (queries == 0) return TQ_OK;
    const int k2 = pow2_at_least(topk);
    if (score_list_stride <= 0) score_list_stride = (int64_t)queries * topk;
    if (idx_list_stride <= 0) idx_list_stride = (int64_t)queries * topk;
    merge_pairs_kernel<<<queries, 256, 2 * k2 * sizeof(unsigned long long), st>>>(in_scores, in_idx, lists, (size_t)score_list_stride,
                                                                                  (size_t)idx_list_stride, queries, topk, k2, out_scores, out_idx); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}
