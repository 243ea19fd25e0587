/*
 * tq_b200.h -- C ABI of libtq_sm100.so: TurboQuant vector quantisation on NVIDIA B200 (sm_100a).
 *
 * The library replaces the array arithmetic of Project-Tensor's
 * tensor_gpu_v2/_quant.py (TurboQuantMSE / TurboQuantProd).  That file has no FFI of its own:
 * its boundary is a handful of NumPy/CuPy array expressions inside Python methods.  Each entry
 * point below names the reference lines whose arithmetic it takes over; the Python classes in
 * project_tensor_b200/turboquant.py keep the reference's names and signatures and call these
 * functions through ctypes.
 *
 * Conventions
 *   - Every function returns 0 (TQ_OK) or a negative TQ_ERR_* code, never throws, never aborts.
 *     tq_last_error() gives a human-readable message for the calling thread's last failure.
 *   - Arguments are validated on the host before anything is launched.
 *   - All data pointers are DEVICE pointers (on the plan's device) unless a parameter is marked
 *     "host".  The caller owns every buffer.  The library allocates device memory only in
 *     tq_plan_create (the constants of one quantizer) and frees it in tq_plan_destroy.
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued asynchronously on it.
 *   - `x`, `out`, `scores`, `q` are dense row-major float32.  Pointers must be 16-byte aligned.
 *
 * Packed layouts (row = one vector / key)
 *   codes : row stride tq_code_row_bytes() = 4*ceil(d*bits/32) bytes; coordinate j occupies bits
 *           [j*bits, (j+1)*bits) of the row read as a little-endian bit stream; padding bits are 0.
 *   signs : row stride tq_sign_row_bytes() = 4*ceil(d/32) bytes, one 32-bit word per 32 coordinates;
 *           inside a word the even coordinates take bits 0..15 and the odd ones bits 16..31
 *           (coordinate j -> bit ((j%32)>>1) + 16*(j&1)); a bit is 1 when the QJL sign is +1
 *           (the reference stores +1/-1 int8, _quant.py:67-70).
 */
#ifndef TQ_B200_H
#define TQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQ_VERSION 100

#define TQ_OK 0
#define TQ_ERR_INVALID_ARGUMENT (-1)  /* null pointer, bad size, misaligned pointer */
#define TQ_ERR_UNSUPPORTED (-2)       /* dimension / bit width outside what the kernels cover */
#define TQ_ERR_CUDA (-3)              /* a CUDA runtime or driver call failed */
#define TQ_ERR_SCRATCH_TOO_SMALL (-4) /* scratch buffer smaller than the matching *_scratch_bytes query says */
#define TQ_ERR_NO_DEVICE (-5)         /* no sm_100 device, or the requested device is absent */

/* Which arithmetic tq_*_quantize / tq_*_dequantize / tq_score_batched use. */
#define TQ_PATH_AUTO 0    /* tensor-core kernels where they exist for (d, bits), else exact kernels */
#define TQ_PATH_EXACT 1   /* float32 kernels that accumulate in the reference's order */
#define TQ_PATH_TENSOR 2  /* tensor-core kernels; TQ_ERR_UNSUPPORTED if (d, bits) has none */

typedef struct tq_plan tq_plan;

int tq_version(void);
const char* tq_last_error(void);

/* Number of CUDA devices this process can see, or a negative TQ_ERR_*. */
int tq_device_count(void);

/* Kernels launched by this library in this process so far, all devices and streams (a running total; take
 * the difference around a region).  No reference counterpart: the reference launches whatever CuPy launches. */
int64_t tq_kernel_launches(void);

/*
 * Upload the constants of one quantizer to `device`.
 * Replaces the per-call `xp.asarray(self.rotation / codebook / boundaries / projection)` of
 * _quant.py:215-222,294-295.  rotation: host float32[d*d] row-major (TurboQuantMSE.rotation,
 * _quant.py:193-201); codebook: host float32[2^bits_mse], sorted (:203-211); projection: host
 * float32[d*d] or NULL for an MSE-only plan (TurboQuantProd.projection, :283-292).
 * Boundaries are derived as 0.5f*(c[k]+c[k+1]) in float32 exactly as _quant.py:212 does.
 * Limits: 2 <= d <= 1024, 1 <= bits_mse <= 8.
 */
int tq_plan_create(int d, int bits_mse, const float* rotation, const float* codebook,
                   const float* projection, int device, tq_plan** out);
void tq_plan_destroy(tq_plan* plan);
int tq_plan_set_path(tq_plan* plan, int path);
/* 1 when tensor-core kernels exist for this plan's (d, bits_mse), else 0. */
int tq_plan_has_tensor_path(const tq_plan* plan);

int64_t tq_code_row_bytes(const tq_plan* plan);
int64_t tq_sign_row_bytes(const tq_plan* plan);
/* Scratch bytes tq_mse_quantize / tq_prod_quantize need for n rows (may be 0). */
int64_t tq_quantize_scratch_bytes(const tq_plan* plan, int64_t n);
/* Scratch bytes tq_score_batched needs for these sizes (prepared queries, and for topk > 0 the
 * candidate lists and, when no score matrix is requested, a chunk of scores).  May be > 0 for topk == 0. */
int64_t tq_topk_scratch_bytes(const tq_plan* plan, int groups, int q_per_group,
                              int64_t keys_per_group, int topk);

/*
 * TurboQuantMSE.quantize, array part (_quant.py:224-236 called from :244-249):
 * norms[i] = ||x_i||_2; unit = x_i / norm (rows whose norm is not > 0 become 0);
 * codes[i][j] = number of boundaries strictly below (unit R^T)[j]  (searchsorted side="left").
 */
int tq_mse_quantize(const tq_plan* plan, const float* x, int64_t n, void* codes, float* norms,
                    void* scratch, size_t scratch_bytes, void* stream);

/*
 * tq_mse_quantize for callers that must not allocate.  No counterpart in the reference (NumPy/CuPy
 * allocate freely); it exists for hosts that cannot hand over a scratch buffer at call time: a
 * serving loop whose device memory was carved up at start-up and is frozen afterwards, a binding
 * from a runtime that can only pass through buffers it registered in advance, or a region where a
 * device allocation would stall every stream of the process.  Inputs and outputs are still the
 * caller's; only the work lists of the second stage live in an array inside the library's device
 * image (about 1.2 MB, held by every GPU that loads the library until the process exits).
 *
 *   - n must not exceed TQ_NOALLOC_MAX_ROWS; larger batches are refused with TQ_ERR_UNSUPPORTED
 *     (split them, or use tq_mse_quantize).
 *   - The first call on each device looks the array's device address up (cudaGetSymbolAddress); make
 *     that first call before any stream capture starts.  No call allocates or frees device memory.
 *   - All calls on one device share the one array.  Each call resets the list counters itself, so
 *     calls in sequence on a stream are fine; calls that overlap on the GPU (different streams,
 *     different threads) race on the lists and may corrupt each other's output.
 * Same results as tq_mse_quantize.
 */
#define TQ_NOALLOC_MAX_ROWS 262144
int tq_mse_quantize_noalloc(const tq_plan* plan, const float* x, int64_t n, void* codes, float* norms,
                            void* stream);

/* TurboQuantMSE.dequantize (_quant.py:238-242,251-254): out_i = (codebook[codes_i] R) * norms[i]. */
int tq_mse_dequantize(const tq_plan* plan, const void* codes, const float* norms, int64_t n,
                      float* out, void* stream);

/*
 * TurboQuantProd.quantize, array part (_quant.py:300-308): the MSE stage above, then
 * residual = unit - codebook[codes] R, residual_norms = ||residual||_2,
 * signs = (residual S^T >= 0).
 */
int tq_prod_quantize(const tq_plan* plan, const float* x, int64_t n, void* codes, void* signs,
                     float* residual_norms, float* norms, void* scratch, size_t scratch_bytes,
                     void* stream);

/*
 * TurboQuantProd.dequantize (_quant.py:317-332):
 * out_i = (codebook[codes_i] R + sqrt(pi/2)/d * residual_norms[i] * (qjl_i S)) * norms[i].
 */
int tq_prod_dequantize(const tq_plan* plan, const void* codes, const void* signs,
                       const float* residual_norms, const float* norms, int64_t n, float* out,
                       void* stream);

/*
 * TurboQuantProd.attention_score with one query row broadcast over n keys
 * (_quant.py:338-341,347-358): scores[i] = norms[i] * ( q . (codebook[codes_i] R)
 *   + sqrt(pi/2)/d * residual_norms[i] * ((S q) . qjl_i) ).   q: float32[d].
 */
int tq_score_broadcast(const tq_plan* plan, const float* q, const void* codes, const void* signs,
                       const float* residual_norms, const float* norms, int64_t n, float* scores,
                       void* stream);

/* Same formula with one query row per key (_quant.py:342-358).  q: float32[n*d]. */
int tq_score_pairwise(const tq_plan* plan, const float* q, const void* codes, const void* signs,
                      const float* residual_norms, const float* norms, int64_t n, float* scores,
                      void* stream);

/*
 * Many queries against shared keys in one pass.  The reference has no such call: its users loop
 * attention_score over query rows and stack the results (validate_turboquant.py:92-95,
 * test_turboquant.py:117-118); this computes the same numbers without re-reading the keys.
 * Keys are split into `groups` consecutive blocks of keys_per_group rows; queries are
 * float32[groups][q_per_group][d]; query (g, a) is scored against the keys of block g only.
 *   scores     : float32[groups][q_per_group][keys_per_group], or NULL to skip the matrix.
 *   topk > 0   : also return, per query, the topk largest scores in descending order
 *                (ties: lower key index first) as top_scores float32[groups][q_per_group][topk]
 *                and top_idx int64[...] = idx_base + row index within the whole key array.
 *                Slots beyond keys_per_group hold -inf / -1.  1 <= topk <= 1024.
 */
int tq_score_batched(const tq_plan* plan, const float* q, int groups, int q_per_group,
                     const void* codes, const void* signs, const float* residual_norms,
                     const float* norms, int64_t keys_per_group, float* scores, int topk,
                     float* top_scores, int64_t* top_idx, int64_t idx_base, void* scratch,
                     size_t scratch_bytes, void* stream);

/*
 * tq_score_batched over a cache whose groups are `group_rows` rows apart in the key arrays and hold
 * keys_per_group <= group_rows keys each (the layout tq_prod_append fills: group_rows = capacity,
 * keys_per_group = current length).  scores stays dense, float32[groups][q_per_group][keys_per_group];
 * top_idx = idx_base + row within the key arrays (group * group_rows + position).  The scratch size is
 * that of tq_topk_scratch_bytes for the same groups, q_per_group, keys_per_group and topk.
 * No reference counterpart: the reference has no cache type (its encodings are immutable dataclasses,
 * _quant.py:156-169).
 */
int tq_score_cache(const tq_plan* plan, const float* q, int groups, int q_per_group, const void* codes,
                   const void* signs, const float* residual_norms, const float* norms,
                   int64_t keys_per_group, int64_t group_rows, float* scores, int topk, float* top_scores,
                   int64_t* top_idx, int64_t idx_base, void* scratch, size_t scratch_bytes, void* stream);

/*
 * Append path: quantize `tokens` new vectors for each of `groups` sequences/heads straight into a packed
 * cache.  x: float32[groups][tokens][d].  The cache arrays hold `capacity` rows per group; every group
 * holds the same number of rows already, kept in DEVICE memory at `length` (one int64), so the call needs
 * no host-side length and a CUDA graph that captured it stays valid as the cache grows.  Token j of
 * group g is written to row g * capacity + *length + j, with the same numbers tq_*_quantize gives
 * (the arithmetic of _quant.py:224-236, 300-308 in the reference's order of operations); rows that would
 * land beyond `capacity` are dropped.  advance != 0: afterwards *length = min(*length + tokens, capacity),
 * in stream order.  One kernel launch (two with advance), no scratch, any d and bits.
 * No reference counterpart (TurboQuantProd.quantize, _quant.py:297-315, always builds a new encoding).
 */
int tq_mse_append(const tq_plan* plan, const float* x, int groups, int tokens, void* codes, float* norms,
                  int64_t capacity, int64_t* length, int advance, void* stream);
int tq_prod_append(const tq_plan* plan, const float* x, int groups, int tokens, void* codes, void* signs,
                   float* residual_norms, float* norms, int64_t capacity, int64_t* length, int advance,
                   void* stream);

/*
 * Decode attention over a quantized key/value cache, without writing scores or dequantized values:
 *
 *   out[g][a][:] = sum_i softmax_i( scale * score(q[g][a], key[g][i]) ) * value[g][i][:]
 *
 * score = TurboQuantProd.attention_score (_quant.py:334-358) on keys packed by tq_prod_quantize / tq_prod_append
 * with `kplan`; value = TurboQuantMSE.dequantize (_quant.py:238-254) of rows packed by tq_mse_quantize /
 * tq_mse_append with `vplan` (an MSE plan of the same d; its rotation and codebook may differ from the keys').
 * Scale, softmax and the weighted sum follow scaled_dot_product_attention (_core.py:1606-1683) without mask or
 * dropout; scale == 0 selects d^-1/2 as `scale or D ** -0.5` does there.
 * q: float32[groups][q_per_group][d]; out: the same shape.  Keys and values of group g occupy rows
 * [g * group_rows, g * group_rows + keys_per_group) of their arrays (group_rows >= keys_per_group).
 * length: null, or a device pointer to one int64 holding the number of keys per group (the counter
 * tq_prod_append advances); the kernel then attends over min(*length, keys_per_group) keys, so a captured
 * launch keeps working while the cache grows up to keys_per_group.  No keys: out = 0.
 * d = 64 or 128, 1..4 code bits for keys and values, else TQ_ERR_UNSUPPORTED.
 * scratch: tq_decode_attention_scratch_bytes(kplan, groups, q_per_group, keys_per_group) bytes, 16-byte aligned.
 */
int64_t tq_decode_attention_scratch_bytes(const tq_plan* kplan, int groups, int q_per_group, int64_t keys_per_group);
int tq_decode_attention(const tq_plan* kplan, const tq_plan* vplan, const float* q, int groups, int q_per_group,
                        const void* k_codes, const void* k_signs, const float* k_residual_norms, const float* k_norms,
                        const void* v_codes, const float* v_norms, int64_t keys_per_group, int64_t group_rows,
                        const int64_t* length, float scale, float* out, void* scratch, size_t scratch_bytes,
                        void* stream);

/*
 * Merge `lists` candidate lists per query (e.g. one per GPU after an all-gather) into one
 * descending top-k.  in_scores/in_idx: [lists][queries][topk]; out: [queries][topk].
 * No reference counterpart (the reference is single-device).
 */
int tq_topk_merge(const float* in_scores, const int64_t* in_idx, int lists, int queries, int topk,
                  float* out_scores, int64_t* out_idx, void* stream);

/*
 * The same merge over the result of ONE all-gather: every rank sends one block of `list_bytes` bytes that
 * holds its float32 [queries][topk] scores at offset 0 and its int64 [queries][topk] indices at offset
 * `idx_offset_bytes`; `gathered` is the `lists` blocks back to back, as the collective leaves them.  Nothing is
 * repacked between the scoring call (which writes scores and indices straight into the send block), the
 * collective and this merge.  list_bytes: a multiple of 8; idx_offset_bytes: a multiple of 16, at least
 * 4*queries*topk.  No reference counterpart (the reference is single-device).
 */
int tq_topk_merge_gathered(const void* gathered, int64_t list_bytes, int64_t idx_offset_bytes, int lists, int queries,
                           int topk, float* out_scores, int64_t* out_idx, void* stream);

/*
 * Conversions between the packed layouts and the reference's array fields
 * (TurboQuantMSEEncoding.indices uint8[n][d], TurboQuantProdEncoding.qjl int8[n][d] of +1/-1,
 * _quant.py:156-169).
 */
int tq_unpack_codes(const tq_plan* plan, const void* codes, int64_t n, uint8_t* indices, void* stream);
int tq_pack_codes(const tq_plan* plan, const uint8_t* indices, int64_t n, void* codes, void* stream);
int tq_unpack_signs(const tq_plan* plan, const void* signs, int64_t n, int8_t* qjl, void* stream);
int tq_pack_signs(const tq_plan* plan, const int8_t* qjl, int64_t n, void* signs, void* stream);

/*
 * Counters of the last tq_*_quantize call on this plan, read back from the device (synchronises
 * `stream`): rows the tensor-core kernel handed to the exact kernel because a coordinate fell
 * within the guard band of a decision boundary.  Diagnostic only.
 */
int tq_plan_last_recheck_rows(const tq_plan* plan, void* stream, int64_t* rows);

/*
 * Bounded waits.  Inside the tensor-core kernels every wait on a barrier has a limit; when one runs out the
 * kernel stops storing results, lets the copies and tensor instructions it has in flight finish, sets the plan's
 * status word and returns -- the context stays usable, the outputs of that call are incomplete.
 * tq_plan_status reads the word back (synchronises `stream`): 0 = no kernel of this plan has given up since the
 * last query; 1 / 2 / 3 = a quantize / scoring / dequantize kernel has (the word is cleared by the query).  The
 * Python classes query it wherever they synchronise anyway and raise instead of handing out such results.
 * tq_plan_set_wait_limit changes the limit (cycles; default about 2 s) for later launches of this plan; 0 makes a
 * kernel give up at the first barrier it finds unfinished, which is how the tests walk this path without a fault.
 * No reference counterpart (NumPy has nothing to wait for).
 */
int tq_plan_status(const tq_plan* plan, void* stream, int64_t* status);

/*
 * Device time of the main kernel of each call, for benchmarks: with timing on (bit 0 of `on`), every tq_*_quantize call on the
 * tensor-core path records a CUDA event before and after its tensor-core kernel (kind 0; the exact second stage
 * lies outside the pair) and every tq_score_batched / tq_score_cache call around each launch of the tensor-core
 * scoring kernel (kind 1); the two kernels of the quantizers' exact second stage have pairs of their own (kind 2: the
 * re-check of listed coordinates, kind 3: the re-computation of listed rows; recorded when bit 1 of `on` is set).  tq_plan_kernel_ms returns how many of the most recent launches of `kind` it wrote to
 * ms[] (at most max_count, at most 1,024), oldest first, in milliseconds; synchronise the stream before.  Turning
 * timing on or off resets the record.  No reference counterpart.
 */
int tq_plan_time_kernels(tq_plan* plan, int on);
int tq_plan_kernel_ms(const tq_plan* plan, int kind, float* ms, int max_count);
int tq_plan_set_wait_limit(tq_plan* plan, int64_t cycles);

#ifdef __cplusplus
}
#endif
#endif /* TQ_B200_H */
