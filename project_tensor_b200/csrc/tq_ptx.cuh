// Inline-PTX wrappers shared by the tensor-core kernels (sm_100a): mbarriers with bounded waits,
// TMA / bulk copies, tensor-memory allocation, tcgen05.mma / ld / st / commit and descriptor helpers.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Cycle counters per role exist only in measurement builds (-DTQ_PROF).
#ifdef TQ_PROF
#define TQ_PROF_CODE(...) __VA_ARGS__
#else
#define TQ_PROF_CODE(...)
#endif

namespace tqptx {

// Limit of one bounded wait in units of 1024 cycles: ~2 s at 2 GHz by default.  Every kernel keeps two words in shared
// memory: [0] the give-up flag that all roles watch, [1] the limit for this launch (from the plan).
constexpr int kDefaultWaitKcycles = 4000000;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// Loads of data that a ring stage holds only until this thread's warp arrives on the stage's "empty" barrier.  A plain
// load may be executed again at the place where its value is used (instead of keeping a register alive), which can lie
// behind the arrival, when the stage may already hold the next tile; a volatile load is executed once, where it stands.
__device__ __forceinline__ float4 lds_once_f4(const void* p) {
    float4 v;
    asm volatile("ld.volatile.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out or another thread has already given up.  Every answer "not yet"
// costs the waiting warp a dozen instructions on the scheduler it shares with working warps (a profile of the quantize
// kernel showed a quarter of all executed instructions in these loops), hence the short loop body.  (A suspend-time hint
// on the try_wait -- 8 us, 1 ms -- changed no kernel's time, and it lets a wait outlive a limit shorter than the hint.)
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (*abort_flag) return false;  // somebody already gave up: do not block again
    if (abort_flag[1] == 0) {       // limit 0: give up at the first wait that would have to wait (how the path is tested)
        *abort_flag = 1;
        return false;
    }
    const long long deadline = clock64() + ((long long)abort_flag[1] << 10);
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;   // blocks inside the hardware for a while before it answers
        if (clock64() > deadline) {
            *abort_flag = 1;
            return false;
        }
        if (*abort_flag) return false;
    }
}
// Has the phase completed?  Answers at once (try_wait may keep the thread suspended for a while first).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_test_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag);
}

// After a give-up: wait, bounded and without looking at the flag, for a phase that this thread armed itself (bulk
// copies in flight towards this block's shared memory, tensor instructions still writing tensor memory), so that
// nothing lands in memory the block has already left.  ~0.5 ms at most.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < (1 << 14); ++it) {
        if (mbar_try_wait(bar, parity)) return;
        __nanosleep(32);
    }
}

// The same wait executed by every lane of a converged warp; the answer is the same for all of them.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    const bool ok = mbar_wait(bar, parity, abort_flag);
    return __all_sync(0xffffffffu, ok);
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// Bytes of a row block that a bulk copy may not take (it moves multiples of 16 bytes): the last `bytes % 16`
// bytes, copied here with plain 4-byte loads by the calling thread.  Call before the arrive on the mbarrier
// that publishes the block, so that its release covers these stores.  `bytes` is a multiple of 4.
__device__ __forceinline__ void copy_tail_words(unsigned char* dst, const unsigned char* src, uint32_t bytes) {
    const uint32_t bulk = bytes & ~15u;
    for (uint32_t o = bulk; o < bytes; o += 4)
        *reinterpret_cast<uint32_t*>(dst + o) = __ldg(reinterpret_cast<const uint32_t*>(src + o));
}

// Named barrier over `count` threads that also ORs a predicate across them.
__device__ __forceinline__ bool bar_or(int id, int count, bool pred) {
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %3, 0;\n\t"
        "barrier.cta.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(out)
        : "r"(id), "r"(count), "r"((uint32_t)pred)
        : "memory");
    return out != 0;
}

// Plain named barrier over `count` threads (a multiple of 32).
// min(m, |a|, |b|) as one three-input minimum (sm_100)
__device__ __forceinline__ float min3_abs(float m, float a, float b) {
    float r;
    asm("{\n\t.reg .f32 ta, tb;\n\tabs.f32 ta, %2;\n\tabs.f32 tb, %3;\n\tmin.f32 %0, %1, ta, tb;\n\t}" : "=f"(r) : "f"(m), "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void bar_sync(int id, int count) {
    asm volatile("barrier.cta.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem descriptor]^T, 128 x N x 16, fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same instruction with the accumulate flag fixed at compile time: `first` overwrites the accumulator.
__device__ __forceinline__ void mma_ts_first(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void mma_ts_acc(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
        : "memory");
}
// mbarrier arrive once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

__device__ __forceinline__ float fma_sat(float a, float b, float c) {
    float r;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float fma_rm(float a, float b, float c) {
    float r;
    asm("fma.rm.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ uint32_t pack_half2(float lo_elem, float hi_elem) {
    const __half2 h = __floats2half2_rn(lo_elem, hi_elem);  // .x (low 16 bits) = first argument
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Shared-memory matrix descriptor of a K-major operand stored without swizzle as 8x8 fp16 core
// matrices (8 rows x 16 bytes, contiguous): lbo = bytes between core matrices along K, sbo = bytes
// between 8-row groups.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version for sm_100
    return d;                // layout type 0: no swizzle
}


}  // namespace tqptx
