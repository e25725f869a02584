// tcgen05 building blocks shared by the tensor-core MEX kernels: bounded mbarrier waits, shared-memory matrix
// descriptors, the TF32 MMA and its commit, tensor-memory allocation and loads, the split-TF32 main loop.
#pragma once
#include <type_traits>
#include "mex_common.cuh"

namespace simnets {
namespace {

constexpr int kTcThreads = 256;
constexpr int kTcKT = 16;                 // taps per stage (two MMA k-steps of 8)
constexpr int kTcPos = 128;               // positions per tile = MMA M
constexpr uint32_t kWaitTries = 1u << 21; // x ~1 us suspend hint: about two seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Bounded wait for the phase with the given parity to complete; false if it never did.  A try that fails is
// followed by a short sleep: a sleeping warp issues nothing, whereas a tight retry loop takes issue slots from
// the warps that do the work (retries made up 40 % of the instructions executed before the sleep was added).
__device__ __forceinline__ bool mbar_try(uint32_t addr, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity), "r"(1000u) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    if (mbar_try(addr, parity)) return true;
    uint32_t ns = 32;
    for (uint32_t it = 0; it < kWaitTries; ++it) {
        __nanosleep(ns);
        if (mbar_try(addr, parity)) return true;
        if (ns < 256) ns *= 2;                      // back off: polling competes with the working warps for issue slots
    }
    return false;
}

// Shared-memory matrix descriptor: K-major, no swizzle.  Element (row, k) of a tile lives at
//   (row / 8) * sbo + (k / 4) * lbo + (row % 8) * 16 + (k % 4) * 4   bytes from the start address.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= uint64_t((saddr >> 4) & 0x3FFFu);
    d |= uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= uint64_t(1) << 46;                    // descriptor version of this architecture
    return d;                                   // base offset 0, layout type 0 = no swizzle
}

// Instruction descriptor: D = F32, A = B = TF32, both K-major, M = 128, N = nt.
__host__ __device__ constexpr uint32_t umma_idesc(int nt) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(nt >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ float tf32_hi(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// byte offset of element (row, k) inside a [rows x KT] K-major core-matrix tile with leading byte offset LBO
// (distance between 16-byte chunks along k) and stride byte offset (KT / 4) * LBO (distance between 8-row groups)
template <int KT, int LBO>
__host__ __device__ constexpr int core_off(int row, int k) { return (row >> 3) * ((KT / 4) * LBO) + (k >> 2) * LBO + (row & 7) * 16 + (k & 3) * 4; }
__host__ __device__ constexpr int core_offset(int row, int k) { return core_off<16, 128>(row, k); }

// Shared state of one tensor-core tile computation.
struct TcShared {
    uint64_t bar_free[2];
    uint64_t bar_done;
    uint32_t tmem;
    int failed;
};

// Set-up common to the three kernels: barriers, tensor-memory allocation of `cols` columns (power of two >= 32).
__device__ __forceinline__ uint32_t tc_begin(TcShared& sh, uint32_t cols) {
    if (threadIdx.x == 0) {
        mbar_init(&sh.bar_free[0], 1); mbar_init(&sh.bar_free[1], 1); mbar_init(&sh.bar_done, 1);
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if ((threadIdx.x >> 5) == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem)), "r"(cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    return sh.tmem;
}

// Frees the tensor memory; every thread of the CTA must call it, after its last tensor-memory load.
__device__ __forceinline__ void tc_end(uint32_t tmem, uint32_t cols) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if ((threadIdx.x >> 5) == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(cols) : "memory");
}

// Main loop: D[128 x NT] = sum over nchunks chunks of KT reduction elements of A[128 x KT] * B[NT x KT]^T with split-TF32
// operands, STAGES shared-memory stages.  Per chunk c every thread calls store(c, a_hi, a_lo, b_hi, b_lo), which writes
// the stage from registers filled earlier (plain stores and / or cp.async), then load(c + 1), which only ISSUES the
// global loads of the next chunk into registers: they are in flight across the fence, the barrier, the MMA issue
// and the wait for the stage.  Returns true on every thread if all MMAs completed, false if a bounded wait expired.
template <int NT, int KT, int LBO, int STAGES, class Load, class Store>
__device__ __forceinline__ bool tc_mainloop(TcShared& sh, unsigned char* dsm, uint32_t tmem_d, int nchunks, Load load, Store store) {
    constexpr int SBO = (KT / 4) * LBO;
    constexpr int A_BYTES = (128 / 8) * SBO, B_BYTES = (NT / 8) * SBO;
    constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
    constexpr uint32_t idesc = umma_idesc(NT);
    bool ok = true;
    if (nchunks > 0) load(0);
    for (int c = 0; c < nchunks; ++c) {
        const int stage = c % STAGES, use = c / STAGES;
        unsigned char* sA = dsm + stage * STAGE_BYTES;
        unsigned char* sB = sA + 2 * A_BYTES;
        if (use >= 1 && ok) ok = mbar_wait(&sh.bar_free[stage], uint32_t(use - 1) & 1u);   // the MMAs that last read this stage are done
        store(c, sA, sA + A_BYTES, sB, sB + B_BYTES);
        if (c + 1 < nchunks) load(c + 1);
        cp_async_wait_all();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA's async proxy
        __syncthreads();
        if (threadIdx.x == 0 && ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(sA), a_lo = a_hi + A_BYTES, b_hi = smem_u32(sB), b_lo = b_hi + B_BYTES;
#pragma unroll
            for (int ks = 0; ks < KT / 8; ++ks) {                       // a k-step of 8 = two 16-byte chunks
                const uint32_t o = ks * 2 * LBO;
                const uint64_t dah = umma_desc(a_hi + o, LBO, SBO), dal = umma_desc(a_lo + o, LBO, SBO);
                const uint64_t dbh = umma_desc(b_hi + o, LBO, SBO), dbl = umma_desc(b_lo + o, LBO, SBO);
                umma_tf32(tmem_d, dal, dbh, idesc, (c | ks) != 0);
                umma_tf32(tmem_d, dah, dbl, idesc, 1);
                umma_tf32(tmem_d, dah, dbh, idesc, 1);
            }
            umma_commit(c + 1 < nchunks ? &sh.bar_free[stage] : &sh.bar_done);
        }
    }
    if (ok && nchunks > 0) ok = mbar_wait(&sh.bar_done, 0);
    if (!ok) sh.failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    return sh.failed == 0;
}

// The same loop with deeper prefetching, for kernels whose B operand is copied verbatim from global memory:
//  * the global loads of the A operand are issued TWO chunks ahead: load(c, parity) fills register set c % 2 and
//    store(c, parity, a_hi, a_lo) consumes it, so that a thread always has the loads of a whole chunk in flight (the
//    parity is a compile-time tag, std::integral_constant, so both register sets stay in registers);
//  * bcopy(c, b_hi) issues the cp.async copies of chunk c's B tile ONE chunk ahead, into the other stage, so that their
//    latency is not waited for between store(c) and the MMAs of chunk c.
// Two stages.
template <int NT, int KT, int LBO, class Load, class Store, class BCopy>
__device__ __forceinline__ bool tc_mainloop_ahead2(TcShared& sh, unsigned char* dsm, uint32_t tmem_d, int nchunks, Load load, Store store, BCopy bcopy) {
    constexpr int SBO = (KT / 4) * LBO;
    constexpr int A_BYTES = (128 / 8) * SBO, B_BYTES = (NT / 8) * SBO;
    constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
    constexpr uint32_t idesc = umma_idesc(NT);
    using Even = std::integral_constant<int, 0>;
    using Odd = std::integral_constant<int, 1>;
    bool ok = true;
    if (nchunks > 0) {
        load(0, Even{});
        bcopy(0, dsm + 2 * A_BYTES);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (nchunks > 1) load(1, Odd{});
    auto step = [&](int c, auto parity) {
        const int stage = c & 1;
        unsigned char* sA = dsm + stage * STAGE_BYTES;
        unsigned char* sB = sA + 2 * A_BYTES;
        store(c, parity, sA, sA + A_BYTES);              // this stage was found free one step ago (or is used for the first time)
        if (c + 2 < nchunks) load(c + 2, parity);        // into the register set that store(c) just emptied
        if (c + 1 < nchunks) {
            // the other stage is free once the MMAs of chunk c - 1 are done
            if (c >= 1 && ok) ok = mbar_wait(&sh.bar_free[stage ^ 1], uint32_t((c - 1) >> 1) & 1u);
            bcopy(c + 1, dsm + (stage ^ 1) * STAGE_BYTES + 2 * A_BYTES);
            asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 1;" ::: "memory");      // chunk c's tile has landed
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA's async proxy
        __syncthreads();
        if (threadIdx.x == 0 && ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(sA), a_lo = a_hi + A_BYTES, b_hi = smem_u32(sB), b_lo = b_hi + B_BYTES;
#pragma unroll
            for (int ks = 0; ks < KT / 8; ++ks) {
                const uint32_t o = ks * 2 * LBO;
                const uint64_t dah = umma_desc(a_hi + o, LBO, SBO), dal = umma_desc(a_lo + o, LBO, SBO);
                const uint64_t dbh = umma_desc(b_hi + o, LBO, SBO), dbl = umma_desc(b_lo + o, LBO, SBO);
                umma_tf32(tmem_d, dal, dbh, idesc, (c | ks) != 0);
                umma_tf32(tmem_d, dah, dbl, idesc, 1);
                umma_tf32(tmem_d, dah, dbh, idesc, 1);
            }
            umma_commit(c + 1 < nchunks ? &sh.bar_free[stage] : &sh.bar_done);
        }
    };
    for (int c = 0; c < nchunks; c += 2) {
        step(c, Even{});
        if (c + 1 < nchunks) step(c + 1, Odd{});
    }
    if (ok && nchunks > 0) ok = mbar_wait(&sh.bar_done, 0);
    if (!ok) sh.failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    return sh.failed == 0;
}

template <int NT, int KT, int LBO, int STAGES>
__host__ __device__ constexpr int tc_smem_bytes() { return STAGES * (2 * (128 / 8) * (KT / 4) * LBO + 2 * (NT / 8) * (KT / 4) * LBO); }

// 32 consecutive tensor-memory columns of this thread's lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Read-only global load that the compiler keeps in program order with the other loads of this kind: the epilogue
// below wants eight of them in flight per batch, not all thirty-two hoisted to the top (which spills).
__device__ __forceinline__ float ld_nc_ordered(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// 2^v and log2(v) on the special-function unit, denormals flushed (operands here are sums and ratios of
// exponentials that stay far above the denormal range)
__device__ __forceinline__ float ex2_ftz(float v) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v)); return r; }
__device__ __forceinline__ float lg2_ftz(float v) { float r; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v)); return r; }

// hi = v rounded to TF32, lo = the exact remainder v - hi (at most 13 significant bits; the tensor core reads its
// top 10, so the pair carries v to about 2^-21)
__device__ __forceinline__ void split_tf32_trunc(float v, float& hi, float& lo) { hi = tf32_hi(v); lo = v - hi; }

// split v into TF32 hi and the exact remainder
// (the remainder is rounded to TF32 here, to nearest, rather than left to the tensor core's truncation)
__device__ __forceinline__ void split_tf32(float v, float& hi, float& lo) { hi = tf32_hi(v); lo = tf32_hi(v - hi); }

}  // namespace
}  // namespace simnets
