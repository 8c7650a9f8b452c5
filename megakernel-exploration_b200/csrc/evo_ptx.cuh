// Thin inline-PTX layer for sm_100a: mbarrier, TMA (bulk tensor copies), tcgen05
// (tensor-memory allocation, UMMA issue/commit, tensor-memory loads) and the
// shared-memory / instruction descriptors that tcgen05.mma consumes.
//
// Every wait in here is bounded: a wait that runs out of iterations records a
// code in the device status word, raises the CTA-wide abort flag and returns
// false, so that callers can unwind, free tensor memory and return.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace evo {

// ---- device status word ---------------------------------------------------
// A 32-bit word in global memory, passed to every kernel.  0 = ok.  Otherwise
// (code << 16) | site, written by the first failing wait.

enum : uint32_t {
    ST_OK = 0,
    ST_WAIT_TIMEOUT = 1,   // a bounded mbarrier wait gave up
};

__device__ __forceinline__ void report(unsigned int* status, uint32_t code, uint32_t site) {
    atomicCAS(status, 0u, (code << 16) | (site & 0xffffu));
}

// What a bounded wait needs to give up cleanly: the CTA-shared abort word
// (once any thread gives up, every other wait of the CTA returns false soon
// after) and the global status word.
struct WaitCtx {
    volatile uint32_t* abort_flag;
    unsigned int* status;
};

// ---- small helpers ----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders generic-proxy writes to shared memory before later async-proxy
// (TMA / tcgen05.mma) reads of the same locations.
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking probe of phase `parity`.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Optional cycle accounting (builds with -DEVO_TRACE only): per wait site / code
// region, summed over warps and CTAs, in the words that follow the status word.
#if defined(EVO_TRACE) && defined(EVO_TL_ONLY)
__device__ __forceinline__ void trace_add(unsigned int*, uint32_t, long long) {}
__device__ __forceinline__ void trace_init() {}
__device__ __forceinline__ void trace_flush(unsigned int*) {}
#elif defined(EVO_TRACE)
// accumulators live in shared memory during the kernel and are added to the global
// words once at the end, so that tracing perturbs the timing as little as possible
__device__ __forceinline__ unsigned long long* trace_smem() {
    __shared__ unsigned long long t[512];
    return t;
}
__device__ __forceinline__ void trace_add(unsigned int*, uint32_t site, long long dt) {
    if ((threadIdx.x & 31u) == 0u) {
        unsigned long long* t = trace_smem();
        atomicAdd(&t[(site & 255u) * 2], static_cast<unsigned long long>(dt));
        atomicAdd(&t[(site & 255u) * 2 + 1], 1ull);
    }
}
// all threads, before the first and after the last traced region (with __syncthreads around)
__device__ __forceinline__ void trace_init() {
    unsigned long long* t = trace_smem();
    for (int i = threadIdx.x; i < 512; i += blockDim.x) t[i] = 0ull;
}
__device__ __forceinline__ void trace_flush(unsigned int* status) {
    unsigned long long* t = trace_smem();
    unsigned long long* g = reinterpret_cast<unsigned long long*>(status + 2);
    for (int i = threadIdx.x; i < 512; i += blockDim.x)
        if (t[i]) atomicAdd(&g[i], t[i]);
}
#endif
#ifdef EVO_TRACE
// timeline of CTA 0 (trace builds): clock at (role, step, event), plain stores to global memory
__device__ __forceinline__ void timeline(unsigned int* status, int role, int step, int evt) {
    if (blockIdx.x == 0 && (threadIdx.x & 31u) == 0u && step < 64) {
        unsigned long long* g = reinterpret_cast<unsigned long long*>(status + 2) + 512;
        g[(role * 64 + step) * 8 + evt] = static_cast<unsigned long long>(clock64());
    }
}
#define EVO_TL(status, role, step, evt) timeline((status), (role), (step), (evt))
#define EVO_TRACE_INIT() trace_init()
#define EVO_TRACE_FLUSH(status) trace_flush(status)
#define EVO_T0() const long long evo_t0_ = clock64()
#define EVO_T1(status, site) trace_add((status), (site), clock64() - evo_t0_)
#define EVO_TS(var) const long long var = clock64()
#define EVO_TE(var, status, site) trace_add((status), (site), clock64() - var)
#else
#define EVO_TL(status, role, step, evt) do {} while (0)
#define EVO_TRACE_INIT() do {} while (0)
#define EVO_TRACE_FLUSH(status) do {} while (0)
#define EVO_T0() do {} while (0)
#define EVO_T1(status, site) do {} while (0)
#define EVO_TS(var) do {} while (0)
#define EVO_TE(var, status, site) do {} while (0)
#endif

// Budget of one wait: an iteration limit and a wall-clock limit (try_wait may
// itself block for a hardware-defined interval), whichever comes first.
#ifndef EVO_WAIT_LIMIT
#define EVO_WAIT_LIMIT (1u << 24)
#endif
#ifndef EVO_WAIT_NS
#define EVO_WAIT_NS 2000000000ull   // 2 s
#endif

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait on phase `parity` of `bar` with explicit limits (iterations, nanoseconds).
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, uint32_t parity, const WaitCtx& w,
                                                  uint32_t site, uint32_t max_iters, uint64_t max_ns) {
    EVO_T0();
    if (mbar_try_wait(bar, parity)) {
        EVO_T1(w.status, site);
        return true;
    }
    uint64_t t0 = 0;
    for (uint32_t it = 0; it < max_iters; ++it) {
        if (mbar_try_wait(bar, parity)) {
            EVO_T1(w.status, site);
            return true;
        }
#ifdef EVO_WAIT_BACKOFF_NS
        __nanosleep(EVO_WAIT_BACKOFF_NS);
#endif
        if ((it & 63u) == 63u) {
            if (*w.abort_flag) return false;
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > max_ns) break;
            if (it > 4096u) __nanosleep(64);
        }
    }
    report(w.status, ST_WAIT_TIMEOUT, site);
    *w.abort_flag = 1u;
    return false;
}

// Bounded wait on phase `parity` of `bar` (the limits every kernel of the library uses).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& w,
                                          uint32_t site) {
    return mbar_wait_limited(bar, parity, w, site, EVO_WAIT_LIMIT, EVO_WAIT_NS);
}

// Makes a per-thread flag uniform across the warp (true only if true everywhere),
// so that .sync.aligned instructions after a bounded wait stay convergent.
__device__ __forceinline__ bool warp_all(bool ok) { return __all_sync(0xffffffffu, ok) != 0; }

// Hands a shared-memory buffer that this (converged) warp has READ with ordinary
// loads back to the producer that will overwrite it through TMA.  An arrive does
// not wait for the warp's earlier shared-memory loads to return: measured on
// B200, a warp's loads queued behind heavy barrier polling were still pending
// when its arrive let the producer refill the buffer, and they returned the new
// tile.  The fence makes lane 0 wait for the warp's outstanding loads (a load
// instruction completes for all lanes together) before the arrive.
__device__ __forceinline__ void mbar_release_after_reads(uint64_t* bar) {
    __syncwarp();
    if ((threadIdx.x & 31u) == 0u) {
        __threadfence_block();
        mbar_arrive(bar);
    }
}

// The same hand-back without a fence.  `dep` must be computed FROM the values the last
// loads of the buffer returned (any cheap combination of one register per load
// instruction).  Lane 0 stores it to a scratch word before the arrive: the store
// cannot issue before those loads have written their registers (a load instruction
// completes for all lanes of the warp together), instructions issue in order, and the
// arrive's release semantics keep it behind the store.  Costs a few logic operations
// and one store instead of a membar (which also waits for every other outstanding
// access of the thread).  `scratch` is the shared address of any word nobody reads.
__device__ __forceinline__ void mbar_release_after_loads(uint64_t* bar, uint32_t dep, uint32_t scratch) {
    __syncwarp();
    if ((threadIdx.x & 31u) == 0u) {
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(scratch), "r"(dep) : "memory");
        mbar_arrive(bar);
    }
}

// ---- explicit shared-memory accesses ----------------------------------------------
// Pointers into the dynamic shared-memory block are formed through integer arithmetic
// (alignment), after which the compiler no longer knows their address space and emits
// generic loads; these take the 32-bit shared address directly.
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t saddr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
    return v;
}
__device__ __forceinline__ float lds32f(uint32_t saddr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t saddr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts128f(uint32_t saddr, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// ---- TMA --------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar,
                                            int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1)
        : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* src,
                                             int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* src,
                                                  int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group"
        " [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_commit_group() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until at most N committed bulk groups still READ their shared source.
template <int N>
__device__ __forceinline__ void tma_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Wait until at most N committed bulk groups are incomplete (writes visible).
template <int N>
__device__ __forceinline__ void tma_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tcgen05: tensor memory --------------------------------------------------
// One full warp allocates `ncols` (power of two >= 32) columns; the base
// address lands in the shared word `dst`.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 bit, 32 consecutive columns: thread i of the warp receives
// lane (addr.lane + i), columns addr.col .. addr.col+31.
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(addr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(addr)
        : "memory");
}
// Store 16 consecutive 32-bit columns of this thread's lane.
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// Store 32 consecutive 32-bit columns of this thread's lane (counterpart of tmem_ld32).
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// N consecutive fp32 columns (N = 8, 16 or 32) of this thread's lane into dst[].
template <int N>
__device__ __forceinline__ void tmem_ld_f32(uint32_t addr, float* dst) {
    static_assert(N == 8 || N == 16 || N == 32, "8, 16 or 32 columns");
    if constexpr (N == 8) {
        uint32_t r[8];
        tmem_ld8(addr, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = __uint_as_float(r[i]);
    } else if constexpr (N == 32) {
        uint32_t r[32];
        tmem_ld32(addr, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[i] = __uint_as_float(r[i]);
    } else {
        uint32_t r[16];
        tmem_ld16(addr, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = __uint_as_float(r[i]);
    }
}

// ---- tcgen05: UMMA ------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit):
//   [0,14)  start address >> 4        [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4   [46,48) version = 1 on sm_100
//   [49,52) base offset = 0           [61,64) swizzle: 0 none, 2 128B, 4 64B, 6 32B
enum : uint32_t { SWZ_NONE = 0, SWZ_128B = 2, SWZ_64B = 4, SWZ_32B = 6 };

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t swz) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(swz & 7u) << 61;
    return d;
}
// Moving a descriptor by a byte offset only touches the start-address field.
__device__ __forceinline__ uint64_t desc_advance(uint64_t d, uint32_t bytes) {
    return d + static_cast<uint64_t>(bytes >> 4);
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulation:
//   [4,6) D format (1 = f32)  [7,10) A format (1 = bf16)  [10,13) B format (1 = bf16)
//   [15] A major (0 = K, 1 = MN)  [16] B major  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16(uint32_t M, uint32_t N, uint32_t a_mn,
                                                       uint32_t b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (a_mn << 15) | (b_mn << 16) | ((N >> 3) << 17) |
           ((M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A is bf16 in tensor memory, row m in lane m, two
// consecutive k per 32-bit column (8 columns per K = 16 block); issued by ONE thread.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier receives one arrival once every MMA issued so far by this
// thread has completed (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}

// ---- numerics helpers -----------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 2^x for x <= 0 (any magnitude, -inf included) on the fused-multiply-add pipe instead of
// the special-function unit, two values at a time: x = n + f with n = round(x), f in
// [-0.5, 0.5]; 2^f by a cubic (minimax, relative error 7.5e-5, far below the bf16 rounding
// the result goes through); 2^n by adding n to the exponent field.  Adding 1.5 * 2^23
// rounds to the nearest integer and leaves it in the low mantissa bits.  A loop that is
// bound by the special-function unit can hand every k-th column pair to this routine so that
// both pipes work at the same time.  Measured at B=1, S=512, N=384, H=8, D=32: the dBias kernel,
// whose arithmetic is little more than the exp2, gains 8 % with every fourth pair (0.218 ->
// 0.200 ms); the forward and the dQ/dK/dV kernel, which are not bound by that unit, gain nothing
// (every third pair) or lose (every second: 0.441 -> 0.478 ms and 0.480 -> 0.533 ms).
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
    x.x = fmaxf(x.x, -126.0f);
    x.y = fmaxf(x.y, -126.0f);
    const float2 xf = __fadd2_rn(x, make_float2(12582912.0f, 12582912.0f));
    const float2 n = __fadd2_rn(xf, make_float2(-12582912.0f, -12582912.0f));
    const float2 f = __ffma2_rn(n, make_float2(-1.0f, -1.0f), x);
    float2 p = __ffma2_rn(f, make_float2(0.0551714588f, 0.0551714588f), make_float2(0.242610862f, 0.242610862f));
    p = __ffma2_rn(p, f, make_float2(0.693260992f, 0.693260992f));
    p = __ffma2_rn(p, f, make_float2(0.99992809f, 0.99992809f));
    float2 r;
    r.x = __uint_as_float(__float_as_uint(p.x) + (__float_as_uint(xf.x) << 23));
    r.y = __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(xf.y) << 23));
    return r;
}
// Column pair `c` goes to the polynomial when c % EVERY == EVERY - 1 (EVERY = 0: never).
template <int EVERY>
__device__ __forceinline__ constexpr bool use_poly(int c) {
    return EVERY > 0 && (c % (EVERY > 0 ? EVERY : 1)) == EVERY - 1;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// Packed fp32 pairs (one instruction, two lanes of work) and the three-input maximum.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float2 bf16x2_f2(uint32_t w) { return make_float2(bf16_lo(w), bf16_hi(w)); }
__device__ __forceinline__ float2 u2f2(uint32_t lo, uint32_t hi) {
    return make_float2(__uint_as_float(lo), __uint_as_float(hi));
}

// Named barrier over `nthreads` threads (ids 1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Register reallocation between warpgroups (all four warps of the warpgroup
// execute it): the producer/mma warpgroup gives registers back, the compute
// warpgroups take them.
template <int N>
__device__ __forceinline__ void reg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// Byte offset of 16-byte chunk c of row r in a TMA-swizzled tile whose rows are
// ROW_BYTES (32, 64 or 128) long: the swizzle XORs the chunk index with address
// bits 7.. (row >> 2, row >> 1, row for 32/64/128-byte rows).
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t swz_off(int r, int c) {
    static_assert(ROW_BYTES == 16 || ROW_BYTES == 32 || ROW_BYTES == 64 || ROW_BYTES == 128, "tile row");
    if constexpr (ROW_BYTES == 16) {
        return r * 16;                  // one chunk per row: nothing to swizzle
    } else {
        constexpr int SH = (ROW_BYTES == 128) ? 0 : (ROW_BYTES == 64 ? 1 : 2);
        constexpr int MASK = ROW_BYTES / 16 - 1;
        return r * ROW_BYTES + ((c ^ ((r >> SH) & MASK)) << 4);
    }
}

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

}  // namespace evo
