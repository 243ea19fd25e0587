// Shared declarations for libtq_sm100.so (TurboQuant on B200).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#include <cuda.h>

#include "../../include/tq_b200.h"

#define TQ_MAX_DIM 1024
#define TQ_MAX_BITS 8
#define TQ_MAX_TOPK 1024

// Guard band (in units of a rotated unit-vector coordinate) inside which the tensor-core kernels
// do not trust their own comparison against a decision boundary and hand the row to the exact
// kernel.  The tensor-core rotation is accurate to ~1e-7; the band leaves a wide margin.
#define TQ_CODE_GUARD 2.0e-6f
// Same idea for the QJL projection, whose sign is taken at zero.
#define TQ_SIGN_GUARD 4.0e-6f

// Work lists that the tensor-core quantizers leave in the caller's scratch buffer for the exact
// second stage.  Layout of the scratch: this header (64 bytes), then `code_cap` 64-bit entries
// (row << 8 | coordinate: a rotated coordinate inside the guard band of a boundary), then `row_cap`
// 32-bit row numbers (rows to recompute completely).  If a list overflows, `overflow` is set and
// the second stage recomputes every row instead.
struct TqRecheckHeader {
    unsigned int n_codes;    // entries appended to the coordinate list (may exceed code_cap)
    unsigned int n_rows;     // entries appended to the row list (may exceed row_cap)
    unsigned int overflow;
    unsigned int pad[13];
};
struct TqRecheck {
    TqRecheckHeader* hdr;
    unsigned long long* code_entries;
    unsigned int* row_entries;
    unsigned int code_cap, row_cap;
};
// Where the rows of a quantize call land when they are appended to a cache of `capacity` rows per group:
// input row r is token r % tokens of group r / tokens and goes to row group * capacity + *length + token.
// `length` lives on the device (one value for all groups), so a captured launch stays valid while the cache
// grows.  tokens == 0: output row = input row.
struct TqRowMap {
    int64_t tokens, capacity;
    const int64_t* length;
};
__host__ __device__ __forceinline__ unsigned int tq_recheck_code_cap(int64_t n) { return (unsigned int)(n / 2 + 4096); }
__host__ __device__ __forceinline__ unsigned int tq_recheck_row_cap(int64_t n) { return (unsigned int)(n / 8 + 4096); }

// Device-side view of a plan: plain pointers, passed to kernels by value.
struct TqDev {
    int d;             // vector dimension
    int bits;          // bits per coordinate of the MSE stage
    int levels;        // 1 << bits
    int code_words;    // 32-bit words per packed code row
    int sign_words;    // 32-bit words per packed sign row
    float alpha;       // float32(sqrt(pi/2) / d), _quant.py:322-324,351-353
    const float* R;    // rotation, row-major [j][k]
    const float* Rt;   // its transpose [k][j]
    const float* S;    // projection, row-major [j][k] (null for MSE-only plans)
    const float* St;   // its transpose
    const float* codebook;    // [levels]
    const float* boundaries;  // [levels-1]
};

// Optional timing of the main kernel of a quantize (kind 0) or batched scoring (kind 1) call: a ring of event pairs,
// one pair per launch, read back by tq_plan_kernel_ms after the stream has been synchronised.
constexpr int kTimerSlots = 1024;
constexpr int kTimerKinds = 4;   // 0 quantize kernel, 1 scoring kernel, 2 coordinate re-check, 3 row re-computation
struct TqKernelTimer {
    cudaEvent_t ev[kTimerKinds][kTimerSlots][2];
    long long count[kTimerKinds];
    int kinds;   // bit k: launches of kind k are timed
};
inline void tq_timer_mark(const struct tq_plan* p, int kind, int edge, cudaStream_t st);   // defined below the plan

struct TensorConsts;  // defined in tq_tensor.cu
struct DequantConsts; // defined in tq_dequant_tc.cu

struct tq_plan {
    TqDev dev;
    int device;
    int path;
    bool has_projection;
    bool tensor_ok;          // tensor-core kernels cover this (d, bits)
    void* slab;              // one device allocation holding every constant
    TensorConsts* tensor;    // host-side bookkeeping for the tensor-core kernels (may be null)
    DequantConsts* dequant;  // operand matrices of the tensor-core dequantize kernels (may be null)
    unsigned long long* counters;  // device: [0] rows re-done by the exact kernel in the last quantize, [1] status word
                                   // (non-zero once a tensor-core kernel gave up on a bounded wait; sticky until read)
    int wait_kcycles;              // limit of a bounded wait inside the tensor-core kernels, in units of 1024 cycles
    struct TqKernelTimer* timer;   // event pairs around the main kernels while tq_plan_time_kernels is on (else null)
};

inline void tq_timer_mark(const tq_plan* p, int kind, int edge, cudaStream_t st) {
    TqKernelTimer* t = p->timer;
    if (!t || !((t->kinds >> kind) & 1)) return;
    cudaEventRecord(t->ev[kind][t->count[kind] % kTimerSlots][edge], st);
    if (edge == 1) ++t->count[kind];
}

// ---- error plumbing (tq_api.cu) -------------------------------------------------------------
int tq_fail(int code, const char* fmt, ...);
#define TQ_CUDA_TRY(expr)                                                                   \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess)                                                             \
            return tq_fail(TQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));   \
    } while (0)

// A named NVTX range around the launches of one step of a call (a profiler shows the library's kernels grouped by it;
// without a profiler attached the calls do nothing).
#include <nvtx3/nvToolsExt.h>
struct TqRange {
    explicit TqRange(const char* name) { nvtxRangePushA(name); }
    ~TqRange() { nvtxRangePop(); }
    TqRange(const TqRange&) = delete;
    TqRange& operator=(const TqRange&) = delete;
};

// Every kernel launch of the library is counted (tq_kernel_launches reports the total).
void tq_count_launch();

// ---- launchers implemented in the kernel files -----------------------------------------------
// Exact (reference-order float32) kernels.  With `lists` null every row is computed; otherwise
// first the listed coordinates are re-decided (tq_launch_exact_code_check), then the listed rows
// are recomputed.
int tq_launch_exact_quantize(const tq_plan* p, bool prod, const float* x, int64_t n, uint32_t* codes,
                             uint32_t* signs, float* rnorms, float* norms, const TqRecheck* lists,
                             unsigned long long* redo_counter, cudaStream_t st, const TqRowMap* map = nullptr);
int tq_launch_append_advance(int64_t* length, int64_t tokens, int64_t capacity, cudaStream_t st);
int tq_launch_exact_code_check(const tq_plan* p, bool prod, const float* x, int64_t n, uint32_t* codes,
                               const TqRecheck* lists, cudaStream_t st);
int tq_launch_exact_dequantize(const tq_plan* p, bool prod, const uint32_t* codes, const uint32_t* signs,
                               const float* rnorms, const float* norms, int64_t n, float* out,
                               cudaStream_t st);
int tq_launch_exact_pairwise(const tq_plan* p, const float* q, const uint32_t* codes, const uint32_t* signs,
                             const float* rnorms, const float* norms, int64_t n, float* scores,
                             cudaStream_t st);

// Tensor-core (tcgen05) kernels.
bool tq_tensor_supported(int d, int bits);
bool tq_tensor_quantize_supported(int d, int bits, bool has_projection);
int tq_tensor_plan_init(tq_plan* p, const float* rotation, const float* codebook, const float* projection);
void tq_tensor_plan_free(tq_plan* p);
int tq_launch_tensor_quantize(const tq_plan* p, bool prod, const float* x, int64_t n, uint32_t* codes,
                              uint32_t* signs, float* rnorms, float* norms, const TqRecheck* lists,
                              cudaStream_t st);

// Tensor-core dequantize (d = 128): operand matrices per plan, then one launch per call.
bool tq_dequant_tc_supported(int d, int bits_mse, bool prod);
int tq_dequant_tc_plan_init(tq_plan* p, const float* rotation, const float* projection);
void tq_dequant_tc_plan_free(tq_plan* p);
int tq_launch_dequant_tc(const tq_plan* p, bool prod, const uint32_t* codes, const uint32_t* signs, const float* rnorms,
                         const float* norms, int64_t n, float* out, cudaStream_t st);

int tq_launch_pairwise_tc(const tq_plan* p, const float* q, const uint32_t* codes, const uint32_t* signs, const float* rnorms,
                          const float* norms, int64_t n, float* scores, cudaStream_t st);

// Streaming scoring kernel for one or two queries per group (d = 128 / 64, 1..4 code bits).
bool tq_score_few_supported(const tq_plan* p, int qpg);
int tq_launch_score_few(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes, const uint32_t* signs,
                        const float* rnorms, const float* norms, int64_t keys_per_group, float* scores, cudaStream_t st,
                        int64_t group_rows = 0);

// Lookup-table scoring kernel for three or four queries per group (d = 128 / 64, 1..3 code bits), tq_score_lut.cu.
bool tq_score_lut_supported(const tq_plan* p, int qpg);
int tq_launch_score_lut(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes, const uint32_t* signs,
                        const float* rnorms, const float* norms, int64_t keys_per_group, float* scores, cudaStream_t st,
                        int64_t group_rows = 0);

// Scoring kernels.  `group_rows`: rows between the first keys of consecutive groups in the key arrays (0 = the
// groups follow one another, keys_per_group rows each); top-k indices count rows of the arrays.
int tq_launch_score_batched(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes,
                            const uint32_t* signs, const float* rnorms, const float* norms,
                            int64_t keys_per_group, float* scores, int topk, float* top_scores,
                            int64_t* top_idx, int64_t idx_base, void* scratch, size_t scratch_bytes,
                            cudaStream_t st, int64_t group_rows = 0);
int tq_launch_score_general(const tq_plan* p, const float* q, int groups, int qpg, const uint32_t* codes,
                            const uint32_t* signs, const float* rnorms, const float* norms,
                            int64_t keys_per_group, float* scores, int topk, float* top_scores,
                            int64_t* top_idx, int64_t idx_base, void* scratch, size_t scratch_bytes,
                            cudaStream_t st, int64_t group_rows = 0);
// Decode attention over packed keys (Prod plan) and packed values (MSE plan), tq_decode_attn.cu.
bool tq_decode_attention_supported(const tq_plan* kp, const tq_plan* vp);
int64_t tq_decode_attention_scratch(const tq_plan* kp, int groups, int qpg, int64_t keys_per_group);
int tq_launch_decode_attention(const tq_plan* kp, const tq_plan* vp, const float* q, int groups, int qpg,
                               const uint32_t* kcodes, const uint32_t* ksigns, const float* krnorms, const float* knorms,
                               const uint32_t* vcodes, const float* vnorms, int64_t keys_per_group, int64_t group_rows,
                               const int64_t* length, float scale, float* out, void* scratch, size_t scratch_bytes,
                               cudaStream_t st);
int64_t tq_score_topk_scratch(const tq_plan* p, int groups, int qpg, int64_t keys_per_group, int topk);
// list strides in elements (floats / int64s); 0 = the lists follow one another, queries * topk entries each
int tq_launch_topk_merge(const float* in_scores, const int64_t* in_idx, int lists, int queries, int topk,
                         float* out_scores, int64_t* out_idx, cudaStream_t st, int64_t score_list_stride = 0,
                         int64_t idx_list_stride = 0);

// Packing helpers.
int tq_launch_unpack_codes(const tq_plan* p, const uint32_t* codes, int64_t n, uint8_t* out, cudaStream_t st);
int tq_launch_pack_codes(const tq_plan* p, const uint8_t* in, int64_t n, uint32_t* codes, cudaStream_t st);
int tq_launch_unpack_signs(const tq_plan* p, const uint32_t* signs, int64_t n, int8_t* out, cudaStream_t st);
int tq_launch_pack_signs(const tq_plan* p, const int8_t* in, int64_t n, uint32_t* signs, cudaStream_t st);

// cuTensorMapEncodeTiled through the runtime's driver entry point table (the library does not link libcuda).
typedef CUresult (*TqEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TqEncodeTiledFn tq_encode_tiled_fn();   // tq_tensor.cu; null if the driver does not offer the entry point

// ---- small device helpers ---------------------------------------------------------------------
// Bit position of coordinate j's QJL sign inside its 32-bit word: the even coordinates of a group of
// 32 fill bits 0..15 and the odd ones bits 16..31, so coordinates (2i, 2i+1) sit exactly 16 bits
// apart -- the two halves of one half2 operand of the scoring kernel.
__host__ __device__ __forceinline__ int tq_sign_bitpos(int j) { return ((j & 31) >> 1) + ((j & 1) << 4); }

// Re-order a word whose bit i belongs to coordinate i (e.g. a ballot) into the stored order above.
__device__ __forceinline__ uint32_t tq_sign_word_from_natural(uint32_t w) {
    uint32_t e = w & 0x55555555u, o = (w >> 1) & 0x55555555u;
    e = (e | (e >> 1)) & 0x33333333u; o = (o | (o >> 1)) & 0x33333333u;
    e = (e | (e >> 2)) & 0x0f0f0f0fu; o = (o | (o >> 2)) & 0x0f0f0f0fu;
    e = (e | (e >> 4)) & 0x00ff00ffu; o = (o | (o >> 4)) & 0x00ff00ffu;
    e = (e | (e >> 8)) & 0x0000ffffu; o = (o | (o >> 8)) & 0x0000ffffu;
    return e | (o << 16);
}

// Code of coordinate j in a packed row (little-endian bit stream, `bits` <= 8).
__device__ __forceinline__ uint32_t tq_get_code(const uint32_t* row, int j, int bits) {
    const int bit = j * bits;
    const int w = bit >> 5, s = bit & 31;
    uint32_t v = row[w] >> s;
    if (s + bits > 32) v |= row[w + 1] << (32 - s);
    return v & ((1u << bits) - 1u);
}
