// C ABI of libtq_sm100.so: argument checking, plan life cycle and dispatch to the kernels.
#include "tq_common.cuh"

#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <new>
#include <vector>

// Scratch of tq_mse_quantize_noalloc: lives in the library's device image, so every GPU that loads the
// library holds these bytes until the process exits.  Sized for TQ_NOALLOC_MAX_ROWS rows.
#define TQ_NOALLOC_SCRATCH_BYTES \
    (sizeof(TqRecheckHeader) + 8 * (size_t)(TQ_NOALLOC_MAX_ROWS / 2 + 4096) + 4 * (size_t)(TQ_NOALLOC_MAX_ROWS / 8 + 4096) + 16)
static __device__ __align__(256) unsigned char g_noalloc_scratch[TQ_NOALLOC_SCRATCH_BYTES];

namespace {
thread_local char g_err[512] = "";

// Device address of g_noalloc_scratch per GPU.  In host code the array's name is only a handle for the
// runtime, not an address a kernel could use; the address has to be asked for, once per device, with
// that device current.
constexpr int kMaxDevices = 64;
void* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct DeviceScope {
    int prev = -1;
    bool ok = true;
    explicit DeviceScope(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~DeviceScope() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

int check_plan(const tq_plan* p, bool need_proj) {
    if (!p) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "plan is null");
    if (need_proj && !p->has_projection)
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "this plan was created without a projection matrix");
    return TQ_OK;
}

int check_ptr(const void* p, const char* name) {
    if (!p) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "%s is null", name);
    if (!aligned16(p)) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "%s is not 16-byte aligned", name);
    return TQ_OK;
}

#define TQ_TRY(expr)             \
    do {                         \
        int r__ = (expr);        \
        if (r__ != TQ_OK) return r__; \
    } while (0)

bool use_tensor(const tq_plan* p, int* err) {
    *err = TQ_OK;
    if (p->path == TQ_PATH_EXACT) return false;
    if (p->path == TQ_PATH_TENSOR && !p->tensor_ok) {
        *err = tq_fail(TQ_ERR_UNSUPPORTED, "no tensor-core kernel for d=%d bits=%d", p->dev.d, p->dev.bits);
        return false;
    }
    return p->tensor_ok;
}
}  // namespace

static std::atomic<long long> g_launches{0};
void tq_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int tq_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

extern "C" {

int tq_version(void) { return TQ_VERSION; }
const char* tq_last_error(void) { return g_err; }

int64_t tq_kernel_launches(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }

int tq_device_count(void) {
    int n = 0;
    const cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return tq_fail(TQ_ERR_NO_DEVICE, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
    return n;
}

int tq_plan_create(int d, int bits_mse, const float* rotation, const float* codebook, const float* projection,
                   int device, tq_plan** out) {
    if (!out) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!rotation || !codebook) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "rotation/codebook is null");
    if (d < 2 || d > TQ_MAX_DIM) return tq_fail(TQ_ERR_UNSUPPORTED, "dimension %d outside [2, %d]", d, TQ_MAX_DIM);
    if (bits_mse < 1 || bits_mse > TQ_MAX_BITS)
        return tq_fail(TQ_ERR_UNSUPPORTED, "bits %d outside [1, %d]", bits_mse, TQ_MAX_BITS);
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return tq_fail(TQ_ERR_NO_DEVICE, "no CUDA device visible");
    if (device < 0 || device >= ndev) return tq_fail(TQ_ERR_NO_DEVICE, "device %d not present (%d visible)", device, ndev);
    cudaDeviceProp prop;
    TQ_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return tq_fail(TQ_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    DeviceScope scope(device);
    if (!scope.ok) return tq_fail(TQ_ERR_CUDA, "cannot select device %d", device);

    tq_plan* p = new (std::nothrow) tq_plan();
    if (!p) return tq_fail(TQ_ERR_CUDA, "out of host memory");
    memset(p, 0, sizeof(*p));
    p->device = device;
    p->path = TQ_PATH_AUTO;
    p->wait_kcycles = 4000000;   // ~2 s at 2 GHz
    p->has_projection = projection != nullptr;
    const int levels = 1 << bits_mse;
    const size_t dd = (size_t)d * d;

    // host staging: R, Rt, S, St, codebook, boundaries, counters (padded to 256 B each)
    auto pad = [](size_t bytes) { return (bytes + 255) & ~size_t(255); };
    const size_t o_R = 0, o_Rt = o_R + pad(dd * 4), o_S = o_Rt + pad(dd * 4), o_St = o_S + pad(dd * 4),
                 o_cb = o_St + pad(dd * 4), o_bd = o_cb + pad(levels * 4), o_cnt = o_bd + pad(levels * 4),
                 total = o_cnt + 256;
    std::vector<unsigned char> host(total, 0);
    float* hR = reinterpret_cast<float*>(host.data() + o_R);
    float* hRt = reinterpret_cast<float*>(host.data() + o_Rt);
    float* hS = reinterpret_cast<float*>(host.data() + o_S);
    float* hSt = reinterpret_cast<float*>(host.data() + o_St);
    float* hcb = reinterpret_cast<float*>(host.data() + o_cb);
    float* hbd = reinterpret_cast<float*>(host.data() + o_bd);
    memcpy(hR, rotation, dd * 4);
    for (int j = 0; j < d; ++j)
        for (int k = 0; k < d; ++k) hRt[(size_t)k * d + j] = rotation[(size_t)j * d + k];
    if (projection) {
        memcpy(hS, projection, dd * 4);
        for (int j = 0; j < d; ++j)
            for (int k = 0; k < d; ++k) hSt[(size_t)k * d + j] = projection[(size_t)j * d + k];
    }
    memcpy(hcb, codebook, levels * 4);
    for (int k = 0; k + 1 < levels; ++k) {
        volatile float s = codebook[k] + codebook[k + 1];  // float32 sum, then float32 product
        hbd[k] = 0.5f * s;
    }

    cudaError_t e = cudaMalloc(&p->slab, total);
    if (e != cudaSuccess) {
        delete p;
        return tq_fail(TQ_ERR_CUDA, "cudaMalloc(%zu) failed: %s", total, cudaGetErrorString(e));
    }
    e = cudaMemcpy(p->slab, host.data(), total, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(p->slab);
        delete p;
        return tq_fail(TQ_ERR_CUDA, "upload of plan constants failed: %s", cudaGetErrorString(e));
    }
    unsigned char* base = static_cast<unsigned char*>(p->slab);
    TqDev& v = p->dev;
    v.d = d;
    v.bits = bits_mse;
    v.levels = levels;
    v.code_words = (d * bits_mse + 31) / 32;
    v.sign_words = (d + 31) / 32;
    v.alpha = (float)(sqrt(M_PI / 2.0) / (double)d);
    v.R = reinterpret_cast<float*>(base + o_R);
    v.Rt = reinterpret_cast<float*>(base + o_Rt);
    v.S = projection ? reinterpret_cast<float*>(base + o_S) : nullptr;
    v.St = projection ? reinterpret_cast<float*>(base + o_St) : nullptr;
    v.codebook = reinterpret_cast<float*>(base + o_cb);
    v.boundaries = reinterpret_cast<float*>(base + o_bd);
    p->counters = reinterpret_cast<unsigned long long*>(base + o_cnt);

    p->tensor_ok = false;
    if (tq_tensor_quantize_supported(d, bits_mse, projection != nullptr)) {
        const int r = tq_tensor_plan_init(p, rotation, codebook, projection);
        if (r != TQ_OK) {
            cudaFree(p->slab);
            delete p;
            return r;
        }
        p->tensor_ok = p->tensor != nullptr;
    }
    if (p->tensor_ok && tq_dequant_tc_supported(d, bits_mse, projection != nullptr)) {
        const int r = tq_dequant_tc_plan_init(p, rotation, projection);
        if (r != TQ_OK) {
            tq_tensor_plan_free(p);
            cudaFree(p->slab);
            delete p;
            return r;
        }
    }
    *out = p;
    return TQ_OK;
}

void tq_plan_destroy(tq_plan* p) {
    if (!p) return;
    DeviceScope scope(p->device);
    if (p->timer) {
        for (int k = 0; k < kTimerKinds; ++k)
            for (int i = 0; i < kTimerSlots; ++i) { cudaEventDestroy(p->timer->ev[k][i][0]); cudaEventDestroy(p->timer->ev[k][i][1]); }
        delete p->timer;
    }
    tq_tensor_plan_free(p);
    tq_dequant_tc_plan_free(p);
    if (p->slab) cudaFree(p->slab);
    delete p;
}

int tq_plan_set_path(tq_plan* p, int path) {
    TQ_TRY(check_plan(p, false));
    if (path != TQ_PATH_AUTO && path != TQ_PATH_EXACT && path != TQ_PATH_TENSOR)
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "unknown path %d", path);
    if (path == TQ_PATH_TENSOR && !p->tensor_ok)
        return tq_fail(TQ_ERR_UNSUPPORTED, "no tensor-core kernel for d=%d bits=%d", p->dev.d, p->dev.bits);
    p->path = path;
    return TQ_OK;
}

int tq_plan_has_tensor_path(const tq_plan* p) { return p && p->tensor_ok ? 1 : 0; }
int64_t tq_code_row_bytes(const tq_plan* p) { return p ? 4 * (int64_t)p->dev.code_words : 0; }
int64_t tq_sign_row_bytes(const tq_plan* p) { return p ? 4 * (int64_t)p->dev.sign_words : 0; }

int64_t tq_quantize_scratch_bytes(const tq_plan* p, int64_t n) {
    if (!p || n < 0) return 0;
    // header + list of (row, coordinate) entries + list of rows for the exact second stage
    return (int64_t)sizeof(TqRecheckHeader) + 8 * (int64_t)tq_recheck_code_cap(n) + 4 * (int64_t)tq_recheck_row_cap(n) + 16;
}

int64_t tq_topk_scratch_bytes(const tq_plan* p, int groups, int q_per_group, int64_t keys_per_group, int topk) {
    if (!p || groups < 0 || q_per_group < 0 || keys_per_group < 0) return 0;
    return tq_score_topk_scratch(p, groups, q_per_group, keys_per_group, topk);
}

static int quantize_common(const tq_plan* p, bool prod, const float* x, int64_t n, void* codes, void* signs,
                           float* rnorms, float* norms, void* scratch, size_t scratch_bytes, void* stream) {
    TQ_TRY(check_plan(p, prod));
    if (n < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n is negative");
    if (n == 0) return TQ_OK;
    TQ_TRY(check_ptr(x, "x"));
    TQ_TRY(check_ptr(codes, "codes"));
    TQ_TRY(check_ptr(norms, "norms"));
    if (prod) {
        TQ_TRY(check_ptr(signs, "signs"));
        TQ_TRY(check_ptr(rnorms, "residual_norms"));
    }
    DeviceScope scope(p->device);
    if (!scope.ok) return tq_fail(TQ_ERR_CUDA, "cannot select device %d", p->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int err;
    if (use_tensor(p, &err)) {
        const int64_t need = tq_quantize_scratch_bytes(p, n);
        if (!scratch || (int64_t)scratch_bytes < need)
            return tq_fail(TQ_ERR_SCRATCH_TOO_SMALL, "quantize scratch: need %lld bytes, got %zu", (long long)need, scratch_bytes);
        TQ_TRY(check_ptr(scratch, "scratch"));
        TqRecheck lists;
        unsigned char* sc = static_cast<unsigned char*>(scratch);
        lists.hdr = reinterpret_cast<TqRecheckHeader*>(sc);
        lists.code_cap = tq_recheck_code_cap(n);
        lists.row_cap = tq_recheck_row_cap(n);
        lists.code_entries = reinterpret_cast<unsigned long long*>(sc + sizeof(TqRecheckHeader));
        lists.row_entries = reinterpret_cast<unsigned int*>(sc + sizeof(TqRecheckHeader) + 8 * (size_t)lists.code_cap);
        TQ_CUDA_TRY(cudaMemsetAsync(lists.hdr, 0, sizeof(TqRecheckHeader), st));
        TQ_TRY(tq_launch_tensor_quantize(p, prod, x, n, static_cast<uint32_t*>(codes), static_cast<uint32_t*>(signs),
                                         rnorms, norms, &lists, st));
        tq_timer_mark(p, 2, 0, st);
        TQ_TRY(tq_launch_exact_code_check(p, prod, x, n, static_cast<uint32_t*>(codes), &lists, st));
        tq_timer_mark(p, 2, 1, st);
        tq_timer_mark(p, 3, 0, st);
        const int rc = tq_launch_exact_quantize(p, prod, x, n, static_cast<uint32_t*>(codes), static_cast<uint32_t*>(signs),
                                                rnorms, norms, &lists, p->counters, st);
        tq_timer_mark(p, 3, 1, st);
        return rc;
    }
    if (err != TQ_OK) return err;
    return tq_launch_exact_quantize(p, prod, x, n, static_cast<uint32_t*>(codes), static_cast<uint32_t*>(signs), rnorms,
                                    norms, nullptr, nullptr, st);
}

int tq_mse_quantize(const tq_plan* p, const float* x, int64_t n, void* codes, float* norms, void* scratch,
                    size_t scratch_bytes, void* stream) {
    return quantize_common(p, false, x, n, codes, nullptr, nullptr, norms, scratch, scratch_bytes, stream);
}

int tq_prod_quantize(const tq_plan* p, const float* x, int64_t n, void* codes, void* signs, float* residual_norms,
                     float* norms, void* scratch, size_t scratch_bytes, void* stream) {
    return quantize_common(p, true, x, n, codes, signs, residual_norms, norms, scratch, scratch_bytes, stream);
}

// Append path: groups * tokens new vectors go behind the `*length` rows every group of a cache already holds.
// One launch of the reference-order kernel (any d, any bits; the batches are small: one or a few tokens per
// sequence and head), no scratch, no host knowledge of the length.
static int append_common(const tq_plan* p, bool prod, const float* x, int groups, int tokens, void* codes, void* signs,
                         float* rnorms, float* norms, int64_t capacity, int64_t* length, int advance, void* stream) {
    TQ_TRY(check_plan(p, prod));
    if (groups < 0 || tokens < 0 || capacity < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "negative size");
    if (tokens > capacity) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "tokens (%d) exceed the capacity (%lld)", tokens, (long long)capacity);
    if ((double)groups * (double)capacity >= 4294967296.0)
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "groups * capacity must stay below 2^32");
    if (groups == 0 || tokens == 0) return TQ_OK;
    TQ_TRY(check_ptr(x, "x"));
    TQ_TRY(check_ptr(codes, "codes"));
    TQ_TRY(check_ptr(norms, "norms"));
    TQ_TRY(check_ptr(length, "length"));
    if (prod) {
        TQ_TRY(check_ptr(signs, "signs"));
        TQ_TRY(check_ptr(rnorms, "residual_norms"));
    }
    DeviceScope scope(p->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const TqRowMap map{tokens, capacity, length};
    TQ_TRY(tq_launch_exact_quantize(p, prod, x, (int64_t)groups * tokens, static_cast<uint32_t*>(codes),
                                    static_cast<uint32_t*>(signs), rnorms, norms, nullptr, nullptr, st, &map));
    if (advance) TQ_TRY(tq_launch_append_advance(length, tokens, capacity, st));
    return TQ_OK;
}

int tq_mse_append(const tq_plan* p, const float* x, int groups, int tokens, void* codes, float* norms, int64_t capacity,
                  int64_t* length, int advance, void* stream) {
    return append_common(p, false, x, groups, tokens, codes, nullptr, nullptr, norms, capacity, length, advance, stream);
}

int tq_prod_append(const tq_plan* p, const float* x, int groups, int tokens, void* codes, void* signs,
                   float* residual_norms, float* norms, int64_t capacity, int64_t* length, int advance, void* stream) {
    return append_common(p, true, x, groups, tokens, codes, signs, residual_norms, norms, capacity, length, advance, stream);
}

int tq_mse_quantize_noalloc(const tq_plan* p, const float* x, int64_t n, void* codes, float* norms, void* stream) {
    TQ_TRY(check_plan(p, false));
    if (n < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n is negative");
    if (n > TQ_NOALLOC_MAX_ROWS)
        return tq_fail(TQ_ERR_UNSUPPORTED, "tq_mse_quantize_noalloc handles at most %d rows per call, got %lld; "
                       "split the batch or use tq_mse_quantize with caller scratch", TQ_NOALLOC_MAX_ROWS, (long long)n);
    if (p->device < 0 || p->device >= kMaxDevices) return tq_fail(TQ_ERR_NO_DEVICE, "device index %d out of range", p->device);
    void* scratch = nullptr;
    {
        DeviceScope scope(p->device);
        if (!scope.ok) return tq_fail(TQ_ERR_CUDA, "cannot select device %d", p->device);
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_ptr[p->device]) {
            void* ptr = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
            if (e != cudaSuccess || !ptr)
                return tq_fail(TQ_ERR_CUDA, "cudaGetSymbolAddress(g_noalloc_scratch) failed: %s", cudaGetErrorString(e));
            g_noalloc_ptr[p->device] = ptr;
        }
        scratch = g_noalloc_ptr[p->device];
    }
    // quantize_common clears the list header at the start of every call (cudaMemsetAsync, no allocation);
    // the entries behind it are only read up to the counts written by the same call.
    return quantize_common(p, false, x, n, codes, nullptr, nullptr, norms, scratch, TQ_NOALLOC_SCRATCH_BYTES, stream);
}

int tq_mse_dequantize(const tq_plan* p, const void* codes, const float* norms, int64_t n, float* out, void* stream) {
    TQ_TRY(check_plan(p, false));
    if (n < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n is negative");
    if (n == 0) return TQ_OK;
    TQ_TRY(check_ptr(codes, "codes"));
    TQ_TRY(check_ptr(norms, "norms"));
    TQ_TRY(check_ptr(out, "out"));
    DeviceScope scope(p->device);
    // the tensor-core kernel when the plan has one (within ~1e-7 relative of the reference arithmetic); the
    // exact kernel reproduces the reference bit for bit and serves every other geometry and the EXACT path
    if (p->path != TQ_PATH_EXACT && p->dequant)
        return tq_launch_dequant_tc(p, false, static_cast<const uint32_t*>(codes), nullptr, nullptr, norms, n, out,
                                    static_cast<cudaStream_t>(stream));
    return tq_launch_exact_dequantize(p, false, static_cast<const uint32_t*>(codes), nullptr, nullptr, norms, n, out,
                                      static_cast<cudaStream_t>(stream));
}

int tq_prod_dequantize(const tq_plan* p, const void* codes, const void* signs, const float* residual_norms,
                       const float* norms, int64_t n, float* out, void* stream) {
    TQ_TRY(check_plan(p, true));
    if (n < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n is negative");
    if (n == 0) return TQ_OK;
    TQ_TRY(check_ptr(codes, "codes"));
    TQ_TRY(check_ptr(signs, "signs"));
    TQ_TRY(check_ptr(residual_norms, "residual_norms"));
    TQ_TRY(check_ptr(norms, "norms"));
    TQ_TRY(check_ptr(out, "out"));
    DeviceScope scope(p->device);
    if (p->path != TQ_PATH_EXACT && p->dequant)
        return tq_launch_dequant_tc(p, true, static_cast<const uint32_t*>(codes), static_cast<const uint32_t*>(signs),
                                    residual_norms, norms, n, out, static_cast<cudaStream_t>(stream));
    return tq_launch_exact_dequantize(p, true, static_cast<const uint32_t*>(codes), static_cast<const uint32_t*>(signs),
                                      residual_norms, norms, n, out, static_cast<cudaStream_t>(stream));
}

static int check_encoding(const void* codes, const void* signs, const float* rn, const float* norms) {
    TQ_TRY(check_ptr(codes, "codes"));
    TQ_TRY(check_ptr(signs, "signs"));
    TQ_TRY(check_ptr(rn, "residual_norms"));
    TQ_TRY(check_ptr(norms, "norms"));
    return TQ_OK;
}

int tq_score_broadcast(const tq_plan* p, const float* q, const void* codes, const void* signs,
                       const float* residual_norms, const float* norms, int64_t n, float* scores, void* stream) {
    TQ_TRY(check_plan(p, true));
    if (n < 0 || n >= (int64_t)1 << 32) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n outside [0, 2^32)");
    if (n == 0) return TQ_OK;
    TQ_TRY(check_ptr(q, "q"));
    TQ_TRY(check_encoding(codes, signs, residual_norms, norms));
    TQ_TRY(check_ptr(scores, "scores"));
    DeviceScope scope(p->device);
    if (p->path == TQ_PATH_AUTO && tq_score_few_supported(p, 1))
        return tq_launch_score_few(p, q, 1, 1, static_cast<const uint32_t*>(codes), static_cast<const uint32_t*>(signs),
                                   residual_norms, norms, n, scores, static_cast<cudaStream_t>(stream));
    return tq_launch_score_general(p, q, 1, 1, static_cast<const uint32_t*>(codes), static_cast<const uint32_t*>(signs),
                                   residual_norms, norms, n, scores, 0, nullptr, nullptr, 0, nullptr, 0,
                                   static_cast<cudaStream_t>(stream));
}

int tq_score_pairwise(const tq_plan* p, const float* q, const void* codes, const void* signs,
                      const float* residual_norms, const float* norms, int64_t n, float* scores, void* stream) {
    TQ_TRY(check_plan(p, true));
    if (n < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n is negative");
    if (n == 0) return TQ_OK;
    TQ_TRY(check_ptr(q, "q"));
    TQ_TRY(check_encoding(codes, signs, residual_norms, norms));
    TQ_TRY(check_ptr(scores, "scores"));
    DeviceScope scope(p->device);
    // q[i] . dequantize(key i) on the tensor-core dequantize kernel where the plan has one; the exact kernel
    // (reference order of operations) otherwise and on the EXACT path
    if (p->path != TQ_PATH_EXACT && p->dequant && p->dev.d != 256)      // d = 256: no pair form of the streaming kernel
        return tq_launch_pairwise_tc(p, q, static_cast<const uint32_t*>(codes), static_cast<const uint32_t*>(signs),
                                     residual_norms, norms, n, scores, static_cast<cudaStream_t>(stream));
    return tq_launch_exact_pairwise(p, q, static_cast<const uint32_t*>(codes), static_cast<const uint32_t*>(signs),
                                    residual_norms, norms, n, scores, static_cast<cudaStream_t>(stream));
}

int tq_score_batched(const tq_plan* p, const float* q, int groups, int q_per_group, const void* codes,
                     const void* signs, const float* residual_norms, const float* norms, int64_t keys_per_group,
                     float* scores, int topk, float* top_scores, int64_t* top_idx, int64_t idx_base, void* scratch,
                     size_t scratch_bytes, void* stream) {
    return tq_score_cache(p, q, groups, q_per_group, codes, signs, residual_norms, norms, keys_per_group, keys_per_group,
                          scores, topk, top_scores, top_idx, idx_base, scratch, scratch_bytes, stream);
}

int tq_score_cache(const tq_plan* p, const float* q, int groups, int q_per_group, const void* codes,
                   const void* signs, const float* residual_norms, const float* norms, int64_t keys_per_group,
                   int64_t group_rows, float* scores, int topk, float* top_scores, int64_t* top_idx, int64_t idx_base,
                   void* scratch, size_t scratch_bytes, void* stream) {
    TQ_TRY(check_plan(p, true));
    if (groups < 0 || q_per_group < 0 || keys_per_group < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "negative size");
    if (group_rows < keys_per_group) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "group_rows is smaller than keys_per_group");
    if (groups > 65535) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "groups > 65535");
    if ((double)groups * (double)group_rows >= 4294967296.0)
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "groups * keys_per_group must stay below 2^32");
    if (topk < 0 || topk > TQ_MAX_TOPK) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "topk outside [0, %d]", TQ_MAX_TOPK);
    // the selection kernels run one grid row per (group, query)
    if (topk > 0 && (int64_t)groups * q_per_group > 65535)
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "top-k over %d groups x %d queries: groups * q_per_group must stay below 65536",
                       groups, q_per_group);
    if (q_per_group > 65535) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "q_per_group > 65535");
    if (!scores && topk == 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "nothing to compute: scores is null and topk is 0");
    if (groups == 0 || q_per_group == 0) return TQ_OK;
    TQ_TRY(check_ptr(q, "q"));
    if (keys_per_group > 0) TQ_TRY(check_encoding(codes, signs, residual_norms, norms));
    if (scores) TQ_TRY(check_ptr(scores, "scores"));
    if (topk > 0) {
        TQ_TRY(check_ptr(top_scores, "top_scores"));
        TQ_TRY(check_ptr(top_idx, "top_idx"));
    }
    DeviceScope scope(p->device);
    return tq_launch_score_batched(p, q, groups, q_per_group, static_cast<const uint32_t*>(codes),
                                   static_cast<const uint32_t*>(signs), residual_norms, norms, keys_per_group, scores,
                                   topk, top_scores, top_idx, idx_base, scratch, scratch_bytes,
                                   static_cast<cudaStream_t>(stream), group_rows);
}

int64_t tq_decode_attention_scratch_bytes(const tq_plan* kp, int groups, int q_per_group, int64_t keys_per_group) {
    if (!kp || groups < 0 || q_per_group < 0 || keys_per_group < 0) return 0;
    return tq_decode_attention_scratch(kp, groups, q_per_group, keys_per_group);
}

int tq_decode_attention(const tq_plan* kp, const tq_plan* vp, const float* q, int groups, int q_per_group,
                        const void* k_codes, const void* k_signs, const float* k_residual_norms, const float* k_norms,
                        const void* v_codes, const float* v_norms, int64_t keys_per_group, int64_t group_rows,
                        const int64_t* length, float scale, float* out, void* scratch, size_t scratch_bytes, void* stream) {
    TQ_TRY(check_plan(kp, true));
    TQ_TRY(check_plan(vp, false));
    if (kp->device != vp->device) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "key and value plans live on different devices");
    if (!tq_decode_attention_supported(kp, vp))
        return tq_fail(TQ_ERR_UNSUPPORTED, "decode attention covers d = 64 or 128 (same for keys and values) and 1..4 code bits; "
                       "got d = %d / %d, key code bits %d, value bits %d", kp->dev.d, vp->dev.d, kp->dev.bits, vp->dev.bits);
    if (groups < 0 || q_per_group < 0 || keys_per_group < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "negative size");
    if (group_rows < keys_per_group) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "group_rows is smaller than keys_per_group");
    if (groups > 65535) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "groups > 65535");
    if (q_per_group > 65535) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "q_per_group > 65535 (one grid row per pass of queries)");
    if ((double)groups * (double)group_rows >= 4294967296.0)
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "groups * group_rows must stay below 2^32");
    if (!(scale == scale) || scale < 0.f) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "scale must be a number >= 0 (0 selects d^-1/2)");
    if (groups == 0 || q_per_group == 0) return TQ_OK;
    TQ_TRY(check_ptr(q, "q"));
    TQ_TRY(check_ptr(out, "out"));
    if (keys_per_group > 0) {
        TQ_TRY(check_encoding(k_codes, k_signs, k_residual_norms, k_norms));
        TQ_TRY(check_ptr(v_codes, "v_codes"));
        TQ_TRY(check_ptr(v_norms, "v_norms"));
    }
    if (scale == 0.f) scale = 1.0f / sqrtf((float)kp->dev.d);   // `scale or D ** -0.5`, _core.py:1652
    DeviceScope scope(kp->device);
    return tq_launch_decode_attention(kp, vp, q, groups, q_per_group, static_cast<const uint32_t*>(k_codes),
                                      static_cast<const uint32_t*>(k_signs), k_residual_norms, k_norms,
                                      static_cast<const uint32_t*>(v_codes), v_norms, keys_per_group, group_rows, length,
                                      scale, out, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

int tq_topk_merge(const float* in_scores, const int64_t* in_idx, int lists, int queries, int topk, float* out_scores,
                  int64_t* out_idx, void* stream) {
    if (lists < 1 || queries < 0 || topk < 1 || topk > TQ_MAX_TOPK)
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "bad merge sizes lists=%d queries=%d topk=%d", lists, queries, topk);
    if ((double)lists * topk >= 4294967295.0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "lists * topk too large");
    if (queries == 0) return TQ_OK;
    TQ_TRY(check_ptr(in_scores, "in_scores"));
    TQ_TRY(check_ptr(in_idx, "in_idx"));
    TQ_TRY(check_ptr(out_scores, "out_scores"));
    TQ_TRY(check_ptr(out_idx, "out_idx"));
    return tq_launch_topk_merge(in_scores, in_idx, lists, queries, topk, out_scores, out_idx,
                                static_cast<cudaStream_t>(stream));
}

int tq_topk_merge_gathered(const void* gathered, int64_t list_bytes, int64_t idx_offset_bytes, int lists, int queries,
                           int topk, float* out_scores, int64_t* out_idx, void* stream) {
    if (lists < 1 || queries < 0 || topk < 1 || topk > TQ_MAX_TOPK)
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "bad merge sizes lists=%d queries=%d topk=%d", lists, queries, topk);
    if ((double)lists * topk >= 4294967295.0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "lists * topk too large");
    if (queries == 0) return TQ_OK;
    const int64_t cnt = (int64_t)queries * topk;
    if (list_bytes % 8 != 0 || idx_offset_bytes % 16 != 0 || idx_offset_bytes < 4 * cnt || list_bytes < idx_offset_bytes + 8 * cnt)
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "block of %lld bytes with indices at %lld does not hold %lld scores and indices",
                       (long long)list_bytes, (long long)idx_offset_bytes, (long long)cnt);
    TQ_TRY(check_ptr(gathered, "gathered"));
    TQ_TRY(check_ptr(out_scores, "out_scores"));
    TQ_TRY(check_ptr(out_idx, "out_idx"));
    const unsigned char* base = static_cast<const unsigned char*>(gathered);
    return tq_launch_topk_merge(reinterpret_cast<const float*>(base), reinterpret_cast<const int64_t*>(base + idx_offset_bytes),
                                lists, queries, topk, out_scores, out_idx, static_cast<cudaStream_t>(stream), list_bytes / 4,
                                list_bytes / 8);
}

int tq_unpack_codes(const tq_plan* p, const void* codes, int64_t n, uint8_t* indices, void* stream) {
    TQ_TRY(check_plan(p, false));
    if (n < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n is negative");
    if (n == 0) return TQ_OK;
    TQ_TRY(check_ptr(codes, "codes"));
    if (!indices) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "indices is null");
    DeviceScope scope(p->device);
    return tq_launch_unpack_codes(p, static_cast<const uint32_t*>(codes), n, indices, static_cast<cudaStream_t>(stream));
}
int tq_pack_codes(const tq_plan* p, const uint8_t* indices, int64_t n, void* codes, void* stream) {
    TQ_TRY(check_plan(p, false));
    if (n < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n is negative");
    if (n == 0) return TQ_OK;
    TQ_TRY(check_ptr(codes, "codes"));
    if (!indices) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "indices is null");
    DeviceScope scope(p->device);
    return tq_launch_pack_codes(p, indices, n, static_cast<uint32_t*>(codes), static_cast<cudaStream_t>(stream));
}
int tq_unpack_signs(const tq_plan* p, const void* signs, int64_t n, int8_t* qjl, void* stream) {
    TQ_TRY(check_plan(p, false));
    if (n < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n is negative");
    if (n == 0) return TQ_OK;
    TQ_TRY(check_ptr(signs, "signs"));
    if (!qjl) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "qjl is null");
    DeviceScope scope(p->device);
    return tq_launch_unpack_signs(p, static_cast<const uint32_t*>(signs), n, qjl, static_cast<cudaStream_t>(stream));
}
int tq_pack_signs(const tq_plan* p, const int8_t* qjl, int64_t n, void* signs, void* stream) {
    TQ_TRY(check_plan(p, false));
    if (n < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "n is negative");
    if (n == 0) return TQ_OK;
    TQ_TRY(check_ptr(signs, "signs"));
    if (!qjl) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "qjl is null");
    DeviceScope scope(p->device);
    return tq_launch_pack_signs(p, qjl, n, static_cast<uint32_t*>(signs), static_cast<cudaStream_t>(stream));
}

int tq_plan_time_kernels(tq_plan* p, int on) {
    TQ_TRY(check_plan(p, false));
    DeviceScope scope(p->device);
    if (on && !p->timer) {
        TqKernelTimer* t = new (std::nothrow) TqKernelTimer();
        if (!t) return tq_fail(TQ_ERR_CUDA, "out of host memory");
        for (int k = 0; k < kTimerKinds; ++k) t->count[k] = 0;
        for (int k = 0; k < kTimerKinds; ++k)
            for (int i = 0; i < kTimerSlots; ++i)
                for (int e = 0; e < 2; ++e) TQ_CUDA_TRY(cudaEventCreate(&t->ev[k][i][e]));
        p->timer = t;
    }
    if (p->timer) {
        for (int k = 0; k < kTimerKinds; ++k) p->timer->count[k] = 0;
        p->timer->kinds = (on & 1 ? 0x3 : 0) | (on & 2 ? 0xc : 0);   // bit 0: the main kernels, bit 1: the second-stage kernels
    }
    if (!on && p->timer) {
        for (int k = 0; k < kTimerKinds; ++k)
            for (int i = 0; i < kTimerSlots; ++i) { cudaEventDestroy(p->timer->ev[k][i][0]); cudaEventDestroy(p->timer->ev[k][i][1]); }
        delete p->timer;
        p->timer = nullptr;
    }
    return TQ_OK;
}

int tq_plan_kernel_ms(const tq_plan* p, int kind, float* ms, int max_count) {
    if (!p || kind < 0 || kind >= kTimerKinds || !ms || max_count < 0) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "bad arguments");
    if (!p->timer) return 0;
    DeviceScope scope(p->device);
    long long n = p->timer->count[kind];
    if (n > kTimerSlots) n = kTimerSlots;      // the ring keeps the most recent launches
    if (n > max_count) n = max_count;
    for (long long i = 0; i < n; ++i) {
        const long long slot = (p->timer->count[kind] - n + i) % kTimerSlots;
        if (cudaEventElapsedTime(&ms[i], p->timer->ev[kind][slot][0], p->timer->ev[kind][slot][1]) != cudaSuccess)
            return tq_fail(TQ_ERR_CUDA, "an event of launch %lld has not completed; synchronise the stream first", i);
    }
    return (int)n;
}

int tq_plan_set_wait_limit(tq_plan* p, int64_t cycles) {
    TQ_TRY(check_plan(p, false));
    if (cycles != 0 && (cycles < 1024 || cycles > (int64_t)1 << 40))
        return tq_fail(TQ_ERR_INVALID_ARGUMENT, "wait limit outside [2^10, 2^40] cycles (0: give up at the first wait)");
    p->wait_kcycles = (int)(cycles >> 10);
    return TQ_OK;
}

int tq_plan_status(const tq_plan* p, void* stream, int64_t* status) {
    TQ_TRY(check_plan(p, false));
    if (!status) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "status is null");
    DeviceScope scope(p->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned long long v = 0;
    TQ_CUDA_TRY(cudaMemcpyAsync(&v, p->counters + 1, sizeof(v), cudaMemcpyDeviceToHost, st));
    TQ_CUDA_TRY(cudaStreamSynchronize(st));
    *status = (int64_t)v;
    if (v != 0) TQ_CUDA_TRY(cudaMemsetAsync(p->counters + 1, 0, sizeof(v), st));   // reported once
    return TQ_OK;
}

int tq_plan_last_recheck_rows(const tq_plan* p, void* stream, int64_t* rows) {
    TQ_TRY(check_plan(p, false));
    if (!rows) return tq_fail(TQ_ERR_INVALID_ARGUMENT, "rows is null");
    DeviceScope scope(p->device);
    unsigned long long v[2] = {0, 0};
    TQ_CUDA_TRY(cudaMemcpyAsync(v, p->counters, sizeof(v), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    TQ_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    *rows = (int64_t)v[0];
    if (v[1] != 0) return tq_fail(TQ_ERR_CUDA, "a tensor-core kernel gave up on a bounded wait (status %llu)", v[1]);
    return TQ_OK;
}

#ifdef TQ_PROF
// Measurement builds only: raw access to the plan's counter block (per-role cycle counters).
int tq_debug_read_counters(const tq_plan* p, long long* out, int n) {
    if (!p || n > 32) return -1;
    return cudaMemcpy(out, p->counters, n * sizeof(long long), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -3;
}
int tq_debug_zero_counters(const tq_plan* p) {
    if (!p) return -1;
    return cudaMemset(p->counters, 0, 256) == cudaSuccess ? 0 : -3;
}

#endif

}  // extern "C"
