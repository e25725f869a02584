// Pair-tile tensor-core MEX kernels: forward, input gradient and offsets gradient for layers whose offsets alternate
// between two unshared regions along the width (unshared_offset_region = [.., 2] with 1x1 spatial blocks, unit stride,
// no padding).
//
// In such a layer the horizontally adjacent output positions (w, w + 1), w even, belong to the sibling regions 2p and
// 2p + 1 and read adjacent input pixels.  The kernels of mex_tc_ws.cu give a CTA the positions of ONE region, so every
// thread reads every other float: half of each 32-byte sector is fetched for nothing, and a thread has 4 bytes in
// flight per load.  Here a work item is a PAIR of tiles, 128 positions of region 2p and their right-hand neighbours in
// region 2p + 1: each thread owns one pixel pair, every global access is an aligned 8-byte load or store of both
// pixels, whole sectors are used once, and the bytes in flight per thread double.  The two tiles of a pair are two
// independent GEMMs (different offsets operand, separate accumulators in tensor memory) that share their loads.
//
// Same GEMM formulation, operand layouts, split-TF32 scheme and role structure as mex_tc_ws.cu (producers -> MMA ->
// epilogue over mbarrier rings, accumulators double buffered in tensor memory); what differs:
//   * all eight producer warps fill every stage (a thread converts half of the stage's 16 reduction elements for its
//     pixel pair) and keep the raw loads of the next DEPTH stages in flight in registers;
//   * the offsets gradient is persistent too: a CTA owns (region pair, instance tiles, tap tile), walks its share of
//     the positions in chunks of 16 pixel pairs and keeps its accumulators in tensor memory until the end, so that the
//     per-CTA partial sums are written once.
// Every mbarrier wait is bounded and also gives up as soon as another role has failed: a wait that runs out raises the
// CTA's failure flag, every role leaves its loop, copies in flight are waited for, tensor memory is freed and word 1
// of the workspace flags reports it (the exact kernels launched behind then redo the work).
#include <cstring>
#include <cuda.h>          // CUtensorMap and the enums of cuTensorMapEncodeTiled (types only: the entry point is looked up at run time)

#include "ws.cuh"

namespace simnets {

namespace {

constexpr int kPairProducerWarps = 8;
constexpr int kPairProducers = kPairProducerWarps * 32;       // 256: thread % 128 = pixel-pair row, thread / 128 = half of the chunk
constexpr int kPairEpilogueWarps = 8;
constexpr int kPairMmaWarp = kPairProducerWarps + kPairEpilogueWarps;
constexpr int kPairLoaderWarp = kPairMmaWarp + 1;
constexpr int kPairThreads = (kPairLoaderWarp + 1) * 32;      // 576

template <int STAGES>
struct PairShared {
    uint64_t full[STAGES];       // producers -> MMA (256 arrivals)
    uint64_t bfull[STAGES];      // loader -> MMA (1 arrival + bytes)
    uint64_t empty[STAGES];      // MMA -> producers, loader
    uint64_t acc_full[2];        // MMA -> epilogue
    uint64_t acc_empty[2];       // epilogue -> MMA (256 arrivals)
    uint64_t drain;              // MMA warp: every MMA it issued has completed
    uint32_t tmem;
    volatile int failed;
};

// Bounded wait that also ends when another role of the CTA has given up.  A failed try is followed by a sleep that
// doubles up to `cap_ns`: a polling warp takes issue slots from the warps that do the work (with a fixed 64 ns sleep
// the polling loops of the ten waiting warps were half of all instructions executed), so roles that can afford a
// late wake-up (the epilogue behind a double-buffered accumulator) pass a long cap, the MMA warp a short one.
__device__ __forceinline__ bool pair_wait(volatile int& failed, uint64_t* bar, uint32_t parity, uint32_t tries, uint32_t cap_ns = 256) {
    const uint32_t addr = smem_u32(bar);
    if (mbar_try(addr, parity)) return true;
    uint32_t ns = 32;
    for (uint32_t it = 0; it < tries; ++it) {
        if (failed) return false;
        __nanosleep(ns);
        if (mbar_try(addr, parity)) return true;
        ns = ns < cap_ns ? ns * 2 : cap_ns;
    }
    return false;
}

// Warp-wide form for the places where a warp-synchronous instruction follows the wait (tcgen05.ld, __syncwarp, the MMA
// warp's elected issue): the verdict is made uniform by a vote, so that a wait that ran out in one lane takes the whole
// warp out of its loop together.  (Arrivals stay one per thread: one arrival per warp behind a __syncwarp measured
// 1 to 5 % slower on the three kernels.)
__device__ __forceinline__ bool pair_wait_warp(volatile int& failed, uint64_t* bar, uint32_t parity, uint32_t tries, uint32_t cap_ns = 256,
                                               bool need = true) {
    const bool ok = !failed && (!need || pair_wait(failed, bar, parity, tries, cap_ns));
    return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void bulk_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_raw(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// 16 consecutive tensor-memory columns of this thread's lane (no wait: pair it with tmem_ld_wait)
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Asynchronous global -> shared copy of 8 (or 4) bytes by this thread, zero fill when `valid` is false; copies are
// grouped with pair_async_commit and awaited with pair_async_wait<N> (at most N groups still pending).
__device__ __forceinline__ void pair_async8(uint32_t sdst, const void* gsrc, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(sdst), "l"(gsrc), "r"(valid ? 8u : 0u) : "memory");
}
__device__ __forceinline__ void pair_async4(uint32_t sdst, const void* gsrc, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(sdst), "l"(gsrc), "r"(valid ? 4u : 0u) : "memory");
}
__device__ __forceinline__ void pair_async16(uint32_t sdst, const void* gsrc, bool valid) {      // L2 only: streamed once
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sdst), "l"(gsrc), "r"(valid ? 16u : 0u) : "memory");
}
__device__ __forceinline__ void pair_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void pair_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float2 ldg2(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }
__device__ __forceinline__ float2 ldcs2(const float* p) { return __ldcs(reinterpret_cast<const float2*>(p)); }

// A pixel pair: the position jl of region 2 * pair and its right-hand neighbour in region 2 * pair + 1.
struct PairColumn {
    long long base;     // offset of y[n, 0, pos] for the left pixel (the right one is base + 1); -1: outside the output grid
    long long gbase;    // offset of dy[n, 0, .] for the left pixel
    size_t xbase;       // offset of x[n, c0, h0, w0] for the left pixel
    float mx0, mx1;
};

__device__ __forceinline__ PairColumn pair_column_of(const MexGeo& g, int pair, long long jl, long long P, const float* __restrict__ mx) {
    PairColumn p;
    const Column c = column_of(g, 2 * pair, jl, P, nullptr);
    p.base = c.base; p.gbase = c.gbase; p.xbase = 0; p.mx0 = p.mx1 = 0.f;
    if (c.base >= 0) {
        p.xbase = (((size_t)c.n * g.C + c.c0) * g.H + c.h0) * g.W + c.w0;
        const float2 m = ldg2(mx + (c.base - (long long)c.n * (g.M - 1) * g.N));      // n * N + pos
        p.mx0 = m.x; p.mx1 = m.y;
    }
    return p;
}

template <int STAGES>
__device__ __forceinline__ uint32_t pair_setup(PairShared<STAGES>& sh, uint32_t tmem_cols) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full[s], kPairProducers); mbar_init(&sh.bfull[s], 1); mbar_init(&sh.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh.acc_full[b], 1); mbar_init(&sh.acc_empty[b], kPairEpilogueWarps * 32); }
        mbar_init(&sh.drain, 1);
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if ((threadIdx.x >> 5) == kPairMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    return sh.tmem;
}

template <int STAGES>
__device__ __forceinline__ void pair_teardown(PairShared<STAGES>& sh, uint32_t tmem, uint32_t tmem_cols, int* __restrict__ flag) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if ((threadIdx.x >> 5) == kPairMmaWarp)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
    if (threadIdx.x == 0 && sh.failed) atomicExch(&flag[1], 1);
}

// Stage of the forward and input-gradient kernels: [tile 0: A hi, A lo][tile 1: A hi, A lo][tile 0: B hi, B lo][tile 1: B hi, B lo]
constexpr int kPairA = kTcPos * kTcKT * 4;                     // one plane of the position operand
template <int NT> __host__ __device__ constexpr int pair_b_bytes() { return NT * kTcKT * 4; }
template <int NT> __host__ __device__ constexpr int pair_stage_bytes() { return 4 * kPairA + 4 * pair_b_bytes<NT>(); }
template <int NT> __host__ __device__ constexpr int pair_stages() { return NT == 128 ? 2 : 3; }
// bytes of the producers' raw slot ring: DEPTH steps of SLOTS float2 per producer thread
template <int DEPTH, int SLOTS> __host__ __device__ constexpr int pair_raw_bytes() { return DEPTH * SLOTS * kPairProducers * 8; }

// Loader role: per stage the pre-split offsets tiles of both regions of the pair (two bulk copies on one barrier).
// `tiles`: [region][row tile][chunk][2 planes][NT x 16].
template <int NT, int STAGES>
__device__ __forceinline__ void pair_loader_role(PairShared<STAGES>& sh, unsigned char* dsm, const float* __restrict__ tiles, const WsPlan& plan,
                                                 int my_items, int row_tiles, int chunks, uint32_t tries) {
    constexpr int B2 = 2 * pair_b_bytes<NT>(), STAGE_BYTES = pair_stage_bytes<NT>();
    if ((threadIdx.x & 31) == 0) {
        WsRing<STAGES> ring = {0, 0u};
        int issued = 0;
        for (int li = 0; li < my_items && !sh.failed; ++li) {
            const WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));       // it.r = region pair
            const size_t per_region = (size_t)row_tiles * chunks * 2 * NT * kTcKT;
            const float* src0 = tiles + (size_t)(2 * it.r) * per_region + (size_t)it.mt * chunks * 2 * NT * kTcKT;
            const float* src1 = src0 + per_region;
            bool ok = true;
            for (int c = 0; c < chunks; ++c, src0 += 2 * NT * kTcKT, src1 += 2 * NT * kTcKT) {
                if (ring.fill >= 1 && !pair_wait(sh.failed, &sh.empty[ring.stage], (ring.fill - 1) & 1u, tries, 512)) { ok = false; break; }
                unsigned char* dst = dsm + ring.stage * STAGE_BYTES + 4 * kPairA;
                bulk_expect(&sh.bfull[ring.stage], 2 * B2);
                bulk_copy_raw(dst, src0, B2, &sh.bfull[ring.stage]);
                bulk_copy_raw(dst + B2, src1, B2, &sh.bfull[ring.stage]);
                ring.advance(1);
                if (issued < STAGES) ++issued;
            }
            if (!ok) { sh.failed = 1; break; }
        }
        // copies still in flight must land before the CTA may exit: walk back over the last `issued` stages
        // (plain bounded waits: the failure flag must not cut these short)
        for (int d = 0; d < issued; ++d) {
            if (ring.stage == 0) { ring.stage = STAGES; --ring.fill; }
            --ring.stage;
            if (!mbar_wait(&sh.bfull[ring.stage], ring.fill & 1u)) sh.failed = 1;
        }
    }
    __syncwarp();
}

// MMA role: both tiles of the pair per stage; accumulators of item li at columns (li % 2) * 2 NT + tile * NT.
// skip_commit >= 0 (test hook): the accumulator of that local item is never published.
template <int NT, int STAGES>
__device__ __forceinline__ void pair_mma_role(PairShared<STAGES>& sh, unsigned char* dsm, uint32_t tmem, int my_items, int chunks,
                                              uint32_t tries, int skip_commit) {
    constexpr int B_BYTES = pair_b_bytes<NT>(), STAGE_BYTES = pair_stage_bytes<NT>();
    constexpr uint32_t idesc = umma_idesc(NT);
    constexpr int SBO = (kTcKT / 4) * 128;
    const int lane = threadIdx.x & 31;
    WsRing<STAGES> ring = {0, 0u};
    for (int li = 0; li < my_items; ++li) {
        const int buf = li & 1;
        const uint32_t round = uint32_t(li) >> 1;
        if (!pair_wait_warp(sh.failed, &sh.acc_empty[buf], (round - 1) & 1u, tries, 256, round >= 1)) { sh.failed = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        bool ok = true;
        for (int c = 0; c < chunks; ++c) {
            const int stage = ring.stage;
            if (!pair_wait_warp(sh.failed, &sh.full[stage], ring.fill & 1u, tries, 64) || !pair_wait_warp(sh.failed, &sh.bfull[stage], ring.fill & 1u, tries, 64)) { ok = false; break; }
            ring.advance(1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint32_t base = smem_u32(dsm + stage * STAGE_BYTES);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const uint32_t a_hi = base + t * 2 * kPairA, a_lo = a_hi + kPairA;
                    const uint32_t b_hi = base + 4 * kPairA + t * 2 * B_BYTES, b_lo = b_hi + B_BYTES;
                    const uint32_t tmem_d = tmem + uint32_t((buf * 2 + t) * NT);
#pragma unroll
                    for (int ks = 0; ks < kTcKT / 8; ++ks) {
                        const uint32_t o = ks * 2 * 128;
                        const uint64_t dah = umma_desc(a_hi + o, 128, SBO), dal = umma_desc(a_lo + o, 128, SBO);
                        const uint64_t dbh = umma_desc(b_hi + o, 128, SBO), dbl = umma_desc(b_lo + o, 128, SBO);
                        umma_tf32(tmem_d, dal, dbh, idesc, (c | ks) != 0);
                        umma_tf32(tmem_d, dah, dbl, idesc, 1);
                        umma_tf32(tmem_d, dah, dbh, idesc, 1);
                    }
                }
                umma_commit(&sh.empty[stage]);
            }
            __syncwarp();
        }
        if (!ok) { sh.failed = 1; break; }
        if (lane == 0 && li != skip_commit) umma_commit(&sh.acc_full[buf]);
        __syncwarp();
    }
    // whatever ended the loop, the tensor memory may be freed only after the MMAs in flight have completed
    if (lane == 0) umma_commit(&sh.drain);
    __syncwarp();
    if (!mbar_wait(&sh.drain, 0)) sh.failed = 1;
}

// TF32 split without a conversion: the hi plane may hold v itself (the tensor core reads the sign, the exponent and the top
// 10 mantissa bits and ignores the rest); lo = v minus that truncation, exactly.
__device__ __forceinline__ float tf32_lo(float v) { return v - __uint_as_float(__float_as_uint(v) & 0xffffe000u); }

// split 8 values into TF32 hi / lo and store them as the two 16-byte groups (k0, k0 + 4) of row `row`
__device__ __forceinline__ void store_split8(unsigned char* a_hi, unsigned char* a_lo, int row, int k0, const float (&e)[8]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        // hi plane: the values themselves (the tensor core reads their top 19 bits); lo plane: what that drops
        const float4 hi = make_float4(e[4 * h], e[4 * h + 1], e[4 * h + 2], e[4 * h + 3]);
        const float4 lo = make_float4(tf32_lo(hi.x), tf32_lo(hi.y), tf32_lo(hi.z), tf32_lo(hi.w));
        const int off = core_offset(row, k0 + 4 * h);
        *reinterpret_cast<float4*>(a_hi + off) = hi;
        *reinterpret_cast<float4*>(a_lo + off) = lo;
    }
}

// Walks a CTA's sequence of (item, chunk) steps for the producers' prefetch cursor.
struct StepCursor {
    int li, c;
    __device__ __forceinline__ bool advance(int chunks) { if (++c == chunks) { c = 0; ++li; return true; } return false; }
};

// ---- forward ---------------------------------------------------------------------------------------------------
// item = (region pair, instance tile of NT, tile of 128 pixel pairs); a stage holds 16 taps.
template <int NT, int DEPTH>
__global__ void __launch_bounds__(kPairThreads, 1) mex_fwd_pair(MexGeo g, const float* __restrict__ x, const float* __restrict__ tiles,
                                                               const float* __restrict__ mo, const float* __restrict__ mx,
                                                               float* __restrict__ y, float* __restrict__ pooled, WsPlan plan,
                                                               int* __restrict__ flag, int test_expire) {
    constexpr int STAGES = pair_stages<NT>();
    constexpr int STAGE_BYTES = pair_stage_bytes<NT>();
    constexpr uint32_t TMEM_COLS = 4 * NT;
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ PairShared<STAGES> sh;
    __shared__ __align__(16) float mo_w[kPairEpilogueWarps][2][NT / 2];
    if (flag[0]) return;                                // factorisation unsafe: the exact kernels run instead

    const long long P = (long long)g.B * g.rs;
    const int mtiles = (g.M + NT - 1) / NT, kchunks = (g.K + kTcKT - 1) / kTcKT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int my_items = plan.items > int(blockIdx.x) ? (plan.items - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const uint32_t tries = test_expire ? 256u : kWaitTries;
    const uint32_t tmem = pair_setup(sh, TMEM_COLS);

    if (warp < kPairProducerWarps) {
        // ---------------- producers: thread % 128 = pixel-pair row, thread / 128 = which 8 of the stage's 16 taps
        const int prow = threadIdx.x % kTcPos, khalf = threadIdx.x / kTcPos;
        const float a = float(g.eps) * 1.4426950408889634f;
        const unsigned hw = unsigned(g.H) * unsigned(g.W);
        const int K = g.K, total = my_items * kchunks;
        // Raw pixel pairs travel global -> shared by per-thread asynchronous copies, DEPTH stages ahead, into a private
        // slot ring behind the operand stages ([DEPTH][8 taps][256 threads] float2): no registers are held by loads in
        // flight, and a thread only ever reads back what it copied itself.
        float2* raw = reinterpret_cast<float2*>(dsm + STAGES * STAGE_BYTES) + threadIdx.x;
        struct Meta { float mx0, mx1; int kleft; };          // kleft: taps of this thread's eight that exist (<= 0: dead row)
        Meta meta[DEPTH];
        StepCursor cur = {0, 0};
        PairColumn col;
        if (my_items > 0) {
            const WsItem it = ws_item(plan, int(blockIdx.x));
            col = pair_column_of(g, it.r, (long long)it.jt * kTcPos + prow, P, mx);
        }
        auto issue = [&](Meta& m, int d) {       // the chunk under the cursor, then move the cursor
            const int k0 = cur.c * kTcKT + khalf * 8;
            m.kleft = col.base >= 0 ? K - k0 : 0;
            m.mx0 = col.mx0; m.mx1 = col.mx1;
            const float* xp = x + col.xbase + (size_t)k0 * hw;
            const uint32_t dst = smem_u32(raw + d * 8 * kPairProducers);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool in = u < m.kleft;
                pair_async8(dst + u * kPairProducers * 8, in ? xp + u * hw : x, in);
            }
            if (cur.advance(kchunks) && cur.li < my_items) {
                const WsItem it = ws_item(plan, int(blockIdx.x) + cur.li * int(gridDim.x));
                col = pair_column_of(g, it.r, (long long)it.jt * kTcPos + prow, P, mx);
            }
        };
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) { if (d < total) issue(meta[d], d); pair_async_commit(); }
        WsRing<STAGES> ring = {0, 0u};
        bool alive = true;
        for (int s0 = 0; s0 < total && alive; s0 += DEPTH) {
#pragma unroll
            for (int d = 0; d < DEPTH; ++d) {
                const int step = s0 + d;
                if (step >= total || !alive) break;
                pair_async_wait<DEPTH - 1>();                        // this step's copies have landed
                const Meta m = meta[d];
                float e0[8], e1[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    // x - mx first: both may be far from zero while their difference is small
                    const float2 v = raw[(d * 8 + u) * kPairProducers];
                    e0[u] = u < m.kleft ? ex2_ftz(a * (v.x - m.mx0)) : 0.f;
                    e1[u] = u < m.kleft ? ex2_ftz(a * (v.y - m.mx1)) : 0.f;
                }
                if (step + DEPTH < total) issue(meta[d], d);          // reuses the slot just read; lands DEPTH stages later
                pair_async_commit();
                const int stage = ring.stage;
                if (sh.failed || (ring.fill >= 1 && !pair_wait(sh.failed, &sh.empty[stage], (ring.fill - 1) & 1u, tries))) { sh.failed = 1; alive = false; break; }
                unsigned char* sA = dsm + stage * STAGE_BYTES;
                store_split8(sA, sA + kPairA, prow, khalf * 8, e0);
                store_split8(sA + 2 * kPairA, sA + 3 * kPairA, prow, khalf * 8, e1);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&sh.full[stage]);
                ring.advance(1);
            }
        }
        pair_async_wait<0>();
    } else if (warp == kPairLoaderWarp) {
        pair_loader_role<NT, STAGES>(sh, dsm, tiles, plan, my_items, mtiles, kchunks, tries);
    } else if (warp == kPairMmaWarp) {
        pair_mma_role<NT, STAGES>(sh, dsm, tmem, my_items, kchunks, tries, test_expire ? 0 : -1);
    } else {
        // ---------------- epilogue: lane = pixel pair, registers = instances of both tiles
        const int ew = warp - kPairProducerWarps, quarter = warp & 3, half = ew >> 2;
        float* mow0 = mo_w[ew][0];
        float* mow1 = mo_w[ew][1];
        const float inv_eps = 1.f / float(g.eps), k_log = 0.69314718056f * inv_eps, c_add = float(g.cst) * inv_eps;
        const unsigned Nu = unsigned(g.N);
        for (int li = 0; li < my_items; ++li) {
            const int buf = li & 1;
            if (__any_sync(0xffffffffu, sh.failed)) break;
            const WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
            const int m0 = it.mt * NT + half * (NT / 2);
            for (int i = lane; i < NT / 2; i += 32) {
                const bool in = m0 + i < g.M;
                mow0[i] = in ? __ldg(mo + (2 * it.r) * g.M + m0 + i) : 0.f;
                mow1[i] = in ? __ldg(mo + (2 * it.r + 1) * g.M + m0 + i) : 0.f;
            }
            __syncwarp();
            const PairColumn col = pair_column_of(g, it.r, (long long)it.jt * kTcPos + quarter * 32 + lane, P, mx);
            const float cadd0 = col.mx0 + c_add, cadd1 = col.mx1 + c_add;
            float* yb = y + (col.base >= 0 ? col.base : 0) + (long long)m0 * g.N;
            // 2x2 sum pooling of the output, fused: a pixel pair is the upper or the lower half of a pooling window, and the
            // other half belongs to the sibling region pair (another work item).  Each half is added to a zeroed tensor by
            // one reduction: 0 + a + b with two addends is the same number in either order, so the sum is deterministic.
            float* pb = nullptr;
            if (pooled != nullptr && col.base >= 0) {
                const long long mn = (long long)g.M * g.N;
                const int n = int(col.base / mn), pos = int(col.base - (long long)n * mn);
                const int w = pos % g.Wo, hc = pos / g.Wo, h = hc % g.Ho, cc = hc / g.Ho;
                const int Ng = g.N >> 2;
                pb = pooled + (long long)n * g.M * Ng + (cc * (g.Ho >> 1) + (h >> 1)) * (g.Wo >> 1) + (w >> 1) + (long long)m0 * Ng;
            }
            if (!pair_wait_warp(sh.failed, &sh.acc_full[buf], (uint32_t(li) >> 1) & 1u, tries, 1024)) { sh.failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < NT / 2; c0 += 16) {
                uint32_t v0[16], v1[16];
                const uint32_t taddr = tmem + uint32_t(buf * 2 * NT + half * (NT / 2) + c0) + (uint32_t(quarter * 32) << 16);
                tmem_ld16_issue(taddr, v0);
                tmem_ld16_issue(taddr + NT, v1);
                tmem_ld_wait();
                if (col.base >= 0) {
                    float* yp = yb + (size_t)c0 * Nu;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        if (m0 + c0 + i < g.M) {
                            float2 o;
                            o.x = fmaf(lg2_ftz(__uint_as_float(v0[i])), k_log, cadd0 + mow0[c0 + i]);
                            o.y = fmaf(lg2_ftz(__uint_as_float(v1[i])), k_log, cadd1 + mow1[c0 + i]);
                            __stcs(reinterpret_cast<float2*>(yp + i * Nu), o);
                            if (pb != nullptr) atomicAdd(pb + (size_t)(c0 + i) * (Nu >> 2), o.x + o.y);
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&sh.acc_empty[buf]);
            __syncwarp();
        }
    }
    pair_teardown(sh, tmem, TMEM_COLS, flag);
}

// ---- input gradient ----------------------------------------------------------------------------------------------
// item = (region pair, tap tile of NT, tile of 128 pixel pairs); a stage holds 16 instances.  Q[j, m] = dy * 2^(a ((mx_j
// - y) + mo_m) + c'); T = Q Eo; dx = Ex * T.  dy may be given pooled 2x2: both pixels of a pair then read one value.
//
// Roles: 4 raw-loader warps (thread = pixel-pair row) issue the asynchronous copies of y and dy, DEPTH stages ahead, into a
// slot ring ([DEPTH][y, dy][16 instances][128 rows] float2) and publish a slot through an mbarrier that their copies
// arrive on; 8 converter warps turn a slot into the split-TF32 position operand of a stage; 1 thread issues the MMAs;
// 1 thread copies the offsets operand; 8 epilogue warps finish dx.  Loading has warps of its own because a warp that
// issues copies faster than memory takes them stalls in the load/store unit: measured on the converters of an earlier
// version, 38 % of their time went into issuing copies, during which they converted nothing, and while they converted
// nothing was being requested from memory.
constexpr int kDxRawWarps = 4;
constexpr int kDxFirstRawWarp = kPairLoaderWarp + 1;
constexpr int kDxThreads = (kDxFirstRawWarp + kDxRawWarps) * 32;      // 704
// a slot: y as [16 instances][128 rows] float2, then dy likewise, or as [16][128] float when dy is given pooled (one value per pair)
// y and dy of 16 instances x 128 pixel pairs, then the offset maxima of those instances in both regions (2 x 16 floats)
template <bool POOLED> __host__ __device__ constexpr int dx_mo_off() { return kTcKT * kTcPos * (POOLED ? 12 : 16); }
template <bool POOLED> __host__ __device__ constexpr int dx_slot_bytes() { return dx_mo_off<POOLED>() + 2 * kTcKT * 4; }
template <bool POOLED> __host__ __device__ constexpr int dx_depth() { return POOLED ? 3 : 2; }      // slots: all but one can be in flight

__device__ __forceinline__ void async_arrive_noinc(uint64_t* bar) {   // arrives once this thread's earlier asynchronous copies have landed
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 8 consecutive tensor-memory columns of this thread's lane (no wait: pair it with tmem_ld_wait)
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr) : "memory");
}

// WIDE: every tensor is 16-byte aligned and the map width is a multiple of 4, so two neighbouring pixel pairs of a tile are
// 16 contiguous bytes: a raw loader then copies two rows at a time (half the copy instructions).
template <int NT, bool POOLED, bool WIDE>
__global__ void __launch_bounds__(kDxThreads, 1) mex_dx_pair(MexGeo g, const float* __restrict__ x, const float* __restrict__ tiles,
                                                            const float* __restrict__ mo, const float* __restrict__ mx,
                                                            const float* __restrict__ y, const float* __restrict__ dy,
                                                            float* __restrict__ dx, WsPlan plan, int* __restrict__ flag) {
    constexpr int STAGES = pair_stages<NT>(), DEPTH = dx_depth<POOLED>(), kDxSlotBytes = dx_slot_bytes<POOLED>();
    constexpr int STAGE_BYTES = pair_stage_bytes<NT>();
    constexpr uint32_t TMEM_COLS = 4 * NT;
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ PairShared<STAGES> sh;
    __shared__ uint64_t raw_full[DEPTH], raw_empty[DEPTH];
    if (flag[0]) return;

    const long long P = (long long)g.B * g.rs;
    const int ktiles = (g.K + NT - 1) / NT, mchunks = (g.M + kTcKT - 1) / kTcKT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int my_items = plan.items > int(blockIdx.x) ? (plan.items - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const int total = my_items * mchunks;
    const uint32_t tries = kWaitTries;
    if (threadIdx.x == 0)
        for (int d = 0; d < DEPTH; ++d) { mbar_init(&raw_full[d], kDxRawWarps * 32); mbar_init(&raw_empty[d], kPairProducers); }
    const uint32_t tmem = pair_setup(sh, TMEM_COLS);          // (its fence and barrier publish the two rings above as well)
    const float a = float(g.eps) * 1.4426950408889634f, c2 = float(g.cst) * 1.4426950408889634f;
    unsigned char* rawbase = dsm + STAGES * STAGE_BYTES;

    if (warp < kPairProducerWarps) {
        // ---------------- converters: thread % 128 = pixel-pair row, thread / 128 = which 8 of the stage's 16 instances
        const int prow = threadIdx.x % kTcPos, mhalf = threadIdx.x / kTcPos;
        const int M = g.M;
        WsRing<STAGES> ring = {0, 0u};
        WsRing<DEPTH> slot = {0, 0u};
        for (int li = 0; li < my_items && !sh.failed; ++li) {
            const WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
            const PairColumn col = pair_column_of(g, it.r, (long long)it.jt * kTcPos + prow, P, mx);
            bool ok = true;
            for (int c = 0; c < mchunks; ++c) {
                const int mleft = col.base >= 0 ? M - c * kTcKT - mhalf * 8 : 0;     // a dead row contributes nothing
                if (!pair_wait(sh.failed, &raw_full[slot.stage], slot.fill & 1u, tries)) { ok = false; break; }
                const float2* ry = reinterpret_cast<const float2*>(rawbase + slot.stage * kDxSlotBytes) + (mhalf * 8) * kTcPos + prow;
                const float2* rg = ry + kTcKT * kTcPos;                                   // dy as pairs
                const float* rgp = reinterpret_cast<const float*>(rawbase + slot.stage * kDxSlotBytes + kTcKT * kTcPos * 8) + (mhalf * 8) * kTcPos + prow;   // dy pooled
                // the offset maxima of this thread's 8 instances in both regions (same addresses in every lane: broadcasts)
                const float4* ms = reinterpret_cast<const float4*>(rawbase + slot.stage * kDxSlotBytes + dx_mo_off<POOLED>()) + mhalf * 2;
                const float4 ma0 = ms[0], ma1 = ms[1], mb0 = ms[4], mb1 = ms[5];
                const float mo0v[8] = {ma0.x, ma0.y, ma0.z, ma0.w, ma1.x, ma1.y, ma1.z, ma1.w};
                const float mo1v[8] = {mb0.x, mb0.y, mb0.z, mb0.w, mb1.x, mb1.y, mb1.z, mb1.w};
                float q0[8], q1[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const bool in = u < mleft;
                    const float2 yv = ry[u * kTcPos];
                    float2 gv;
                    if (POOLED) { gv.x = rgp[u * kTcPos]; gv.y = gv.x; }
                    else gv = rg[u * kTcPos];
                    q0[u] = in ? gv.x * ex2_ftz(fmaf(a, (col.mx0 - yv.x) + mo0v[u], c2)) : 0.f;
                    q1[u] = in ? gv.y * ex2_ftz(fmaf(a, (col.mx1 - yv.y) + mo1v[u], c2)) : 0.f;
                }
                mbar_arrive(&raw_empty[slot.stage]);                          // the slot may be refilled
                slot.advance(1);
                const int stage = ring.stage;
                if (ring.fill >= 1 && !pair_wait(sh.failed, &sh.empty[stage], (ring.fill - 1) & 1u, tries)) { ok = false; break; }
                unsigned char* sA = dsm + stage * STAGE_BYTES;
                store_split8(sA, sA + kPairA, prow, mhalf * 8, q0);
                store_split8(sA + 2 * kPairA, sA + 3 * kPairA, prow, mhalf * 8, q1);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&sh.full[stage]);
                ring.advance(1);
            }
            if (!ok) { sh.failed = 1; break; }
        }
    } else if (warp == kPairLoaderWarp) {
        pair_loader_role<NT, STAGES>(sh, dsm, tiles, plan, my_items, ktiles, mchunks, tries);
    } else if (warp == kPairMmaWarp) {
        pair_mma_role<NT, STAGES>(sh, dsm, tmem, my_items, mchunks, tries, -1);
    } else if (warp >= kDxFirstRawWarp) {
        // ---------------- raw loaders.  8-byte copies: thread = pixel-pair row, all 16 instances of a stage.  WIDE: thread =
        // (two neighbouring rows, half of the instances), 16-byte copies.
        const int lt = int(threadIdx.x) - kDxFirstRawWarp * 32;
        const int row = WIDE ? 2 * (lt & 63) : lt, mfirst = WIDE ? 8 * (lt >> 6) : 0;
        constexpr int NM = WIDE ? 8 : 16;
        const int M = g.M;
        const unsigned Nu = unsigned(g.N), Ngu = unsigned(g.Ng);
        WsRing<DEPTH> slot = {0, 0u};
        for (int li = 0; li < my_items && !sh.failed; ++li) {
            const WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
            const Column col = column_of(g, 2 * it.r, (long long)it.jt * kTcPos + row, P, nullptr);
            const bool live = col.base >= 0;
            const float* yp = y + (live ? col.base : 0) + (size_t)mfirst * Nu;
            const float* gp = dy + (live ? col.gbase : 0) + (size_t)mfirst * Ngu;
            bool ok = true;
            for (int c = 0; c < mchunks; ++c, yp += (size_t)kTcKT * Nu, gp += (size_t)kTcKT * Ngu) {
                if (slot.fill >= 1 && !pair_wait(sh.failed, &raw_empty[slot.stage], (slot.fill - 1) & 1u, tries)) { ok = false; break; }
                const uint32_t dsty = smem_u32(rawbase + slot.stage * kDxSlotBytes) + (mfirst * kTcPos + row) * 8;
                const uint32_t dstg = smem_u32(rawbase + slot.stage * kDxSlotBytes) + kTcKT * kTcPos * 8 + (mfirst * kTcPos + row) * (POOLED ? 4 : 8);
                constexpr int GP = kTcPos * (POOLED ? 4 : 8);                 // bytes between instances in the dy part
                const int mleft = live ? M - c * kTcKT - mfirst : 0;         // a dead row must not read a stranger's y: zero fill
                if (mleft >= NM) {
#pragma unroll
                    for (int u = 0; u < NM; ++u) {
                        if (WIDE) {
                            pair_async16(dsty + u * kTcPos * 8, yp + u * Nu, true);
                            if (POOLED) pair_async8(dstg + u * GP, gp + u * Ngu, true);          // the pooled values of two neighbouring pairs
                            else pair_async16(dstg + u * GP, gp + u * Ngu, true);
                        } else {
                            pair_async8(dsty + u * kTcPos * 8, yp + u * Nu, true);
                            if (POOLED) pair_async4(dstg + u * GP, gp + u * Ngu, true);
                            else pair_async8(dstg + u * GP, gp + u * Ngu, true);
                        }
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < NM; ++u) {
                        const bool in = u < mleft;
                        if (WIDE) {
                            pair_async16(dsty + u * kTcPos * 8, in ? yp + u * Nu : y, in);
                            if (POOLED) pair_async8(dstg + u * GP, in ? gp + u * Ngu : dy, in);
                            else pair_async16(dstg + u * GP, in ? gp + u * Ngu : dy, in);
                        } else {
                            pair_async8(dsty + u * kTcPos * 8, in ? yp + u * Nu : y, in);
                            if (POOLED) pair_async4(dstg + u * GP, in ? gp + u * Ngu : dy, in);
                            else pair_async8(dstg + u * GP, in ? gp + u * Ngu : dy, in);
                        }
                    }
                }
                if (lt < 2 * kTcKT) {                                         // offset maxima of the stage's instances: region lt / 16, instance lt % 16
                    const int mi = c * kTcKT + (lt & (kTcKT - 1));
                    const bool in = mi < M;
                    pair_async4(smem_u32(rawbase + slot.stage * kDxSlotBytes + dx_mo_off<POOLED>()) + lt * 4,
                                in ? mo + (2 * it.r + (lt >> 4)) * M + mi : mo, in);
                }
                async_arrive_noinc(&raw_full[slot.stage]);
                slot.advance(1);
            }
            if (!ok) { sh.failed = 1; break; }
        }
        pair_async_commit();
        pair_async_wait<0>();                                  // nothing of this thread's may still be in flight at exit
    } else {
        // ---------------- epilogue: lane = pixel pair, registers = taps of both tiles, 8 taps at a time
        const int ew = warp - kPairProducerWarps, quarter = warp & 3, half = ew >> 2;
        const unsigned hw = unsigned(g.H) * unsigned(g.W);
        for (int li = 0; li < my_items; ++li) {
            const int buf = li & 1;
            if (__any_sync(0xffffffffu, sh.failed)) break;
            const WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));        // it.mt = tap tile
            const PairColumn col = pair_column_of(g, it.r, (long long)it.jt * kTcPos + quarter * 32 + lane, P, mx);
            const int k_first = it.mt * NT + half * (NT / 2);
            const float* xb = x + col.xbase + (size_t)k_first * hw;
            float* db = dx + col.xbase + (size_t)k_first * hw;
            int kleft = col.base >= 0 ? g.K - k_first : 0;
            float2 xr[8], xn[8];                                    // x of the block at hand and of the next one, in flight
#pragma unroll
            for (int i = 0; i < 8; ++i) xr[i] = i < kleft ? ldg2(xb + (size_t)i * hw) : make_float2(0.f, 0.f);
            if (!pair_wait_warp(sh.failed, &sh.acc_full[buf], (uint32_t(li) >> 1) & 1u, tries, 1024)) { sh.failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < NT / 2; c0 += 8) {
                uint32_t v0[8], v1[8];
                const uint32_t taddr = tmem + uint32_t(buf * 2 * NT + half * (NT / 2) + c0) + (uint32_t(quarter * 32) << 16);
                tmem_ld8_issue(taddr, v0);
                tmem_ld8_issue(taddr + NT, v1);
                if (c0 + 8 < NT / 2) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) xn[i] = 8 + i < kleft ? ldg2(xb + (size_t)(c0 + 8 + i) * hw) : make_float2(0.f, 0.f);
                }
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (i < kleft) {
                        float2 o;
                        o.x = ex2_ftz(a * (xr[i].x - col.mx0)) * __uint_as_float(v0[i]);
                        o.y = ex2_ftz(a * (xr[i].y - col.mx1)) * __uint_as_float(v1[i]);
                        *reinterpret_cast<float2*>(db + (size_t)(c0 + i) * hw) = o;
                    }
                }
                kleft -= 8;
#pragma unroll
                for (int i = 0; i < 8; ++i) xr[i] = xn[i];
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&sh.acc_empty[buf]);
        }
    }
    pair_teardown(sh, tmem, TMEM_COLS, flag);
}

// ---- offsets gradient --------------------------------------------------------------------------------------------
// U[m, k] = sum over positions j of Q[m, j] * Ex[k, j] per region.  A CTA owns (region pair, MT tiles of 128 instances, one
// tile of NT taps) and a contiguous share of the pair's positions, walked in chunks of CP pixel pairs (CP / 8 MMA k-steps);
// its 2 * MT accumulators (128 lanes x NT columns each) stay in tensor memory until the last chunk.  Both operands are
// computed: A = Q^T (rows = instances), B = Ex^T (rows = taps), reduction along positions, stored one float at a time in
// the K-major core-matrix layout with a leading byte offset of 144, which spreads the positions of a row and the rows a
// warp stores at once over all 32 banks.  (MT, NT, CP) = (1, 64, 16) for layers up to 128 instances and 64 taps, else CP = 8
// with up to two instance tiles and 128 taps, so that larger layers read y, dy and x once too.
// Roles: 4 raw-loader warps copy a chunk's y, dy, x pairs and per-position maxima into a slot ring ([DEPTH][y rows, dy rows,
// x rows, mx][CP pairs] float2), 16 converter warps turn a slot into the operands of a stage, one thread issues the MMAs;
// the converters write the partial sums out at the end.
constexpr int kDoLBO = 144;
constexpr int kDoConvWarps = 16, kDoConv = kDoConvWarps * 32;                                    // 512 converters
constexpr int kDoMmaWarp = kDoConvWarps, kDoFirstRawWarp = kDoMmaWarp + 1, kDoRawWarps = 8;
constexpr int kDoPairThreads = (kDoFirstRawWarp + kDoRawWarps) * 32;                             // 672
constexpr int kDoStages = 2;

template <int MT, int NT, int CP, bool POOLED>
struct DoCfg {
    static constexpr int DEPTH = POOLED ? 3 : 2;                                 // slots of the raw ring: all but one can be in flight
    static constexpr int SBO = (CP / 4) * kDoLBO;
    static constexpr int A_PLANE = (128 / 8) * SBO, B_PLANE = (NT / 8) * SBO;
    static constexpr int TILE_BYTES = 2 * MT * A_PLANE + 2 * B_PLANE;            // one tile of the pair: MT x (A hi, A lo), B hi, B lo
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int QR = MT * 128, XR = NT;                                 // rows of y (and of dy) and of x in a slot
    static constexpr int G_OFF = QR * CP * 8, X_OFF = G_OFF + QR * CP * (POOLED ? 4 : 8), MX_OFF = X_OFF + XR * CP * 8;   // dy pooled: one float per pair
    static constexpr int SLOT_DATA = MX_OFF + CP * 8;                             // bytes one chunk brings in
    static constexpr int SLOT_BYTES = (SLOT_DATA + 127) & ~127;                   // slots start on 128-byte boundaries (tensor-map copies)
    static constexpr int SMEM = kDoStages * STAGE_BYTES + DEPTH * SLOT_BYTES;
    static constexpr int ROWSLOTS = kDoConv / CP;                                // 32 (CP = 16) or 64 (CP = 8) rows converted at once
    static constexpr int QROWS = QR / ROWSLOTS, XROWS = XR / ROWSLOTS;
    static_assert(SMEM <= 227 * 1024, "stages and slot ring must fit the shared memory of one CTA");
    static_assert(2 * MT * NT <= 512, "accumulators must fit the tensor memory");
};

struct DoPairShared {
    uint64_t full[kDoStages];        // converters -> MMA (512 arrivals)
    uint64_t empty[kDoStages];       // MMA -> converters
    uint64_t raw_full[3];            // raw loaders' copies -> converters (128 arrivals)
    uint64_t raw_empty[3];           // converters -> raw loaders (512 arrivals)
    uint64_t acc_full;               // MMA -> converters, after the last chunk
    uint32_t tmem;
    volatile int failed;
};

struct DoPairPlan { int units, mgroups, ktiles, splits; };

// Tensor maps of the offsets-gradient kernel's raw loader (LOAD == 2): y, dy, x and the per-position maxima seen as
// (w, row parity class, row within the class, instance or channel, sample), so that the pixel pairs of one chunk -- a run
// of one image row, or a few whole rows, of the region pair's rows -- times all instances are ONE box.  Plain per-CTA
// tiled copies from this GPU's own tensors; each CTA fetches its own boxes, nothing is shared between CTAs.
struct DoMaps { CUtensorMap y, dy, x, mx; };

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3, int c4) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// LOAD: how the raw loaders fetch a chunk.  0: 8-byte asynchronous copies, one pixel pair per thread; 1: 16-byte copies,
// two neighbouring pairs per thread; 2: four tensor-map box copies per chunk issued by one thread (see DoMaps).
constexpr int do_pair_threads(int load) { return load == 2 ? (kDoFirstRawWarp + 1) * 32 : kDoPairThreads; }      // one loader warp suffices for box copies

template <int MT, int NT, int CP, bool POOLED, int LOAD>
__global__ void __launch_bounds__(do_pair_threads(LOAD), 1) mex_doff_pair(MexGeo g, const float* __restrict__ x, const float* __restrict__ mo,
                                                                  const float* __restrict__ mx, const float* __restrict__ y,
                                                                  const float* __restrict__ dy, float* __restrict__ part,
                                                                  DoPairPlan plan, int* __restrict__ flag,
                                                                  const __grid_constant__ DoMaps maps) {
    constexpr bool WIDE = LOAD == 1;
    using Cfg = DoCfg<MT, NT, CP, POOLED>;
    constexpr int kDoDepth = Cfg::DEPTH;
    constexpr uint32_t TMEM_COLS = 2 * MT * NT;
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ DoPairShared sh;
    if (flag[0]) return;

    const long long P = (long long)g.B * g.rs;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = int(blockIdx.x) % plan.units, split = int(blockIdx.x) / plan.units;
    const int kt = unit % plan.ktiles, mg = (unit / plan.ktiles) % plan.mgroups, pair = unit / (plan.ktiles * plan.mgroups);
    const long long chunks = (P + CP - 1) / CP;
    const long long c_begin = chunks * split / plan.splits, c_end = chunks * (split + 1) / plan.splits;
    const int nchunks = int(c_end - c_begin);
    const uint32_t tries = kWaitTries;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDoStages; ++s) { mbar_init(&sh.full[s], kDoConv); mbar_init(&sh.empty[s], 1); }
        for (int d = 0; d < kDoDepth; ++d) { mbar_init(&sh.raw_full[d], LOAD == 2 ? 1 : kDoRawWarps * 32); mbar_init(&sh.raw_empty[d], kDoConv); }
        mbar_init(&sh.acc_full, 1);
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kDoMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sh.tmem;

    const int M = g.M, K = g.K;
    const int m_first = mg * MT * 128, k_first = kt * NT;
    unsigned char* rawbase = dsm + kDoStages * Cfg::STAGE_BYTES;

    if (warp < kDoConvWarps) {
        // ---------------- converters: the lanes of a warp cover the CP pairs of the chunk and 32 / CP rows of a block of ROWSLOTS
        // rows, chosen 4 (CP = 16) or 2 (CP = 8) apart so that their one-float stores fall into different banks
        const int j = lane & (CP - 1);
        const int rb = CP == 16 ? (warp & 3) + 4 * (lane >> 4) + 8 * (warp >> 2) : (warp & 1) + 2 * (lane >> 3) + 8 * (warp >> 1);
        const float a = float(g.eps) * 1.4426950408889634f, c2 = float(g.cst) * 1.4426950408889634f;
        float mo0[Cfg::QROWS], mo1[Cfg::QROWS];      // offset maxima of this thread's instances, both regions
#pragma unroll
        for (int i = 0; i < Cfg::QROWS; ++i) {
            const int m = m_first + Cfg::ROWSLOTS * i + rb;
            mo0[i] = m < M ? __ldg(mo + (2 * pair) * M + m) : 0.f;
            mo1[i] = m < M ? __ldg(mo + (2 * pair + 1) * M + m) : 0.f;
        }
        WsRing<kDoStages> ring = {0, 0u};
        WsRing<kDoDepth> slot = {0, 0u};
        bool alive = true;
        for (int c = 0; c < nchunks; ++c) {
            if (sh.failed || !pair_wait(sh.failed, &sh.raw_full[slot.stage], slot.fill & 1u, tries)) { alive = false; break; }
            const unsigned char* sb = rawbase + slot.stage * Cfg::SLOT_BYTES;
            const float2* rs = reinterpret_cast<const float2*>(sb) + j;
            const float2* rgf = reinterpret_cast<const float2*>(sb + Cfg::G_OFF) + j;
            const float* rgp = reinterpret_cast<const float*>(sb + Cfg::G_OFF) + j;
            const float2* rx = reinterpret_cast<const float2*>(sb + Cfg::X_OFF) + j;
            const float2 mxv = reinterpret_cast<const float2*>(sb + Cfg::MX_OFF)[j];
            float2 yv[Cfg::QROWS], gv[Cfg::QROWS], xv[Cfg::XROWS];
#pragma unroll
            for (int i = 0; i < Cfg::QROWS; ++i) {
                yv[i] = rs[(Cfg::ROWSLOTS * i + rb) * CP];
                if (POOLED) { gv[i].x = rgp[(Cfg::ROWSLOTS * i + rb) * CP]; gv[i].y = gv[i].x; }
                else gv[i] = rgf[(Cfg::ROWSLOTS * i + rb) * CP];
            }
#pragma unroll
            for (int i = 0; i < Cfg::XROWS; ++i) xv[i] = rx[(Cfg::ROWSLOTS * i + rb) * CP];
            // Rows past M or K and dead positions hold zeros (zero-filled copies): they give Q = 0 or are never stored.  An
            // instance row past M may turn into 0 * inf = NaN; it feeds only accumulator rows that are never written out.
            float qa[Cfg::QROWS], qb[Cfg::QROWS], ea[Cfg::XROWS], eb[Cfg::XROWS];
#pragma unroll
            for (int i = 0; i < Cfg::QROWS; ++i) {
                qa[i] = gv[i].x * ex2_ftz(fmaf(a, (mxv.x - yv[i].x) + mo0[i], c2));
                qb[i] = gv[i].y * ex2_ftz(fmaf(a, (mxv.y - yv[i].y) + mo1[i], c2));
            }
#pragma unroll
            for (int i = 0; i < Cfg::XROWS; ++i) {
                ea[i] = ex2_ftz(a * (xv[i].x - mxv.x));
                eb[i] = ex2_ftz(a * (xv[i].y - mxv.y));
            }
            mbar_arrive(&sh.raw_empty[slot.stage]);
            slot.advance(1);
            const int stage = ring.stage;
            if (ring.fill >= 1 && !pair_wait(sh.failed, &sh.empty[stage], (ring.fill - 1) & 1u, tries)) { alive = false; break; }
            unsigned char* t0 = dsm + stage * Cfg::STAGE_BYTES;
            unsigned char* t1 = t0 + Cfg::TILE_BYTES;
#pragma unroll
            for (int i = 0; i < Cfg::QROWS; ++i) {                              // A: Q^T, per instance tile planes hi, lo
                const int row = Cfg::ROWSLOTS * i + rb;
                const int off = (row >> 7) * 2 * Cfg::A_PLANE + core_off<CP, kDoLBO>(row & 127, j);
                *reinterpret_cast<float*>(t0 + off) = qa[i];
                *reinterpret_cast<float*>(t0 + off + Cfg::A_PLANE) = tf32_lo(qa[i]);
                *reinterpret_cast<float*>(t1 + off) = qb[i];
                *reinterpret_cast<float*>(t1 + off + Cfg::A_PLANE) = tf32_lo(qb[i]);
            }
#pragma unroll
            for (int i = 0; i < Cfg::XROWS; ++i) {                              // B: Ex^T, planes hi, lo
                const int off = 2 * MT * Cfg::A_PLANE + core_off<CP, kDoLBO>(Cfg::ROWSLOTS * i + rb, j);
                *reinterpret_cast<float*>(t0 + off) = ea[i];
                *reinterpret_cast<float*>(t0 + off + Cfg::B_PLANE) = tf32_lo(ea[i]);
                *reinterpret_cast<float*>(t1 + off) = eb[i];
                *reinterpret_cast<float*>(t1 + off + Cfg::B_PLANE) = tf32_lo(eb[i]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&sh.full[stage]);
            ring.advance(1);
        }
        // ---------------- the partial sums: lane = instance row, registers = taps
        bool good = alive && !sh.failed;
        if (good && nchunks > 0) good = pair_wait(sh.failed, &sh.acc_full, 0, tries);
        good = __all_sync(0xffffffffu, good);                                   // the warp-wide loads and syncs below need one verdict
        if (!good) sh.failed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (good) {
            // lane = instance row in tensor memory; a warp turns each 32 x 32 block through shared memory (the operand
            // stages are free by now) so that a store instruction writes 32 consecutive taps of ONE row: whole 128-byte
            // lines instead of 32 scattered floats (the scattered form cost more than the main loop at small batches)
            const int quarter = warp & 3, t = (warp >> 2) & 1, chalf = warp >> 3;      // lane quarter, tile of the pair, half of the columns
            float* tb = reinterpret_cast<float*>(dsm) + warp * (32 * 33);
#pragma unroll 1
            for (int mt = 0; mt < MT; ++mt) {
                const int m0 = m_first + mt * 128 + quarter * 32;
                float* dst = part + (((size_t)split * g.R + (2 * pair + t)) * M + m0) * K + k_first;
#pragma unroll 1
                for (int c0 = chalf * (NT / 2); c0 < (chalf + 1) * (NT / 2); c0 += 32) {
                    uint32_t v[32];
                    if (nchunks > 0) tmem_ld32(tmem + uint32_t((t * MT + mt) * NT + c0) + (uint32_t(quarter * 32) << 16), v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) tb[lane * 33 + i] = nchunks > 0 ? __uint_as_float(v[i]) : 0.f;
                    __syncwarp();
                    const bool kin = k_first + c0 + lane < K;
#pragma unroll 4
                    for (int r = 0; r < 32; ++r)
                        if (kin && m0 + r < M) dst[(size_t)r * K + c0 + lane] = tb[r * 33 + lane];
                    __syncwarp();
                }
            }
        }
    } else if (warp == kDoMmaWarp) {
        constexpr uint32_t idesc = umma_idesc(NT);
        WsRing<kDoStages> ring = {0, 0u};
        bool ok = true;
        for (int c = 0; c < nchunks; ++c) {
            const int stage = ring.stage;
            if (!pair_wait_warp(sh.failed, &sh.full[stage], ring.fill & 1u, tries, 64)) { ok = false; break; }
            ring.advance(1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint32_t base = smem_u32(dsm + stage * Cfg::STAGE_BYTES);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const uint32_t tb = base + t * Cfg::TILE_BYTES;
                    const uint32_t b_hi = tb + 2 * MT * Cfg::A_PLANE, b_lo = b_hi + Cfg::B_PLANE;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint32_t a_hi = tb + mt * 2 * Cfg::A_PLANE, a_lo = a_hi + Cfg::A_PLANE;
                        const uint32_t tmem_d = tmem + uint32_t((t * MT + mt) * NT);
#pragma unroll
                        for (int ks = 0; ks < CP / 8; ++ks) {
                            const uint32_t o = ks * 2 * kDoLBO;
                            const uint64_t dah = umma_desc(a_hi + o, kDoLBO, Cfg::SBO), dal = umma_desc(a_lo + o, kDoLBO, Cfg::SBO);
                            const uint64_t dbh = umma_desc(b_hi + o, kDoLBO, Cfg::SBO), dbl = umma_desc(b_lo + o, kDoLBO, Cfg::SBO);
                            umma_tf32(tmem_d, dal, dbh, idesc, (c | ks) != 0);
                            umma_tf32(tmem_d, dah, dbl, idesc, 1);
                            umma_tf32(tmem_d, dah, dbh, idesc, 1);
                        }
                    }
                }
                umma_commit(&sh.empty[stage]);
            }
            __syncwarp();
        }
        if (!ok) sh.failed = 1;
        // published even after a failure: the tensor memory may be freed only after the MMAs in flight have completed
        if (lane == 0 && nchunks > 0) umma_commit(&sh.acc_full);
        __syncwarp();
        if (nchunks > 0 && !mbar_wait(&sh.acc_full, 0)) sh.failed = 1;
    } else if (LOAD == 2) {
        // ---------------- raw loader, tensor-map form: one thread, four box copies per chunk onto the slot's barrier.  Rows
        // past M, channels past K and samples past the batch lie outside the maps' extents and arrive as zeros.
        if (threadIdx.x == kDoFirstRawWarp * 32) {
            const int rh = pair % g.oh;                                           // row class of this region pair (regions 2 pair, 2 pair + 1)
            const int rw = g.rw;                                                  // pixel pairs per image row
            WsRing<kDoDepth> slot = {0, 0u};
            int issued = 0;
            for (int c = 0; c < nchunks; ++c) {
                if (sh.failed) break;
                if (slot.fill >= 1 && !pair_wait(sh.failed, &sh.raw_empty[slot.stage], (slot.fill - 1) & 1u, tries)) { sh.failed = 1; break; }
                const long long j0 = (c_begin + c) * CP;                          // first pixel pair of the chunk (whole rows or a run inside one)
                const int n = int(j0 / g.rs), l = int(j0 % g.rs);
                const int lh = l / rw, lw = l - lh * rw;
                uint64_t* bar = &sh.raw_full[slot.stage];
                const uint32_t sbase = smem_u32(rawbase + slot.stage * Cfg::SLOT_BYTES);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(uint32_t(Cfg::SLOT_DATA)) : "memory");
                tma_load_5d(sbase, &maps.y, bar, 2 * lw, rh, lh, m_first, n);
                if (POOLED) tma_load_4d(sbase + Cfg::G_OFF, &maps.dy, bar, lw, lh, m_first, n);
                else tma_load_5d(sbase + Cfg::G_OFF, &maps.dy, bar, 2 * lw, rh, lh, m_first, n);
                tma_load_5d(sbase + Cfg::X_OFF, &maps.x, bar, 2 * lw, rh, lh, k_first, n);
                tma_load_4d(sbase + Cfg::MX_OFF, &maps.mx, bar, 2 * lw, rh, lh, n);
                slot.advance(1);
                if (issued < kDoDepth) ++issued;
            }
            // copies still in flight must land before the CTA may exit (they have, on the normal path): walk back over
            // the last `issued` slots
            for (int d = 0; d < issued; ++d) {
                if (slot.stage == 0) { slot.stage = kDoDepth; --slot.fill; }
                --slot.stage;
                if (!mbar_wait(&sh.raw_full[slot.stage], slot.fill & 1u)) sh.failed = 1;
            }
        }
    } else {
        // ---------------- raw loaders; zero fill past M, K and for dead pairs.  8-byte copies: one pixel pair per thread;
        // WIDE: two neighbouring pairs per thread, 16-byte copies.  The 128 threads cover CP pairs x RS row slots.
        const int lt = int(threadIdx.x) - kDoFirstRawWarp * 32;
        constexpr int PT = WIDE ? CP / 2 : CP;                                 // threads along the pairs of the chunk
        constexpr int RS = kDoRawWarps * 32 / PT;                              // row slots: rows rsl, rsl + RS, ...
        const int j = WIDE ? 2 * (lt % PT) : (lt % PT), rsl = lt / PT;
        const unsigned Nu = unsigned(g.N), Ngu = unsigned(g.Ng), hw = unsigned(g.H) * unsigned(g.W);
        WsRing<kDoDepth> slot = {0, 0u};
        for (int c = 0; c < nchunks; ++c) {
            if (sh.failed) break;
            if (slot.fill >= 1 && !pair_wait(sh.failed, &sh.raw_empty[slot.stage], (slot.fill - 1) & 1u, tries)) { sh.failed = 1; break; }
            const Column col = column_of(g, 2 * pair, (c_begin + c) * CP + j, P, nullptr);
            const bool live = col.base >= 0;
            const float* yp = y + (live ? col.base : 0) + (size_t)(m_first + rsl) * Nu;
            const float* gp = dy + (live ? col.gbase : 0) + (size_t)(m_first + rsl) * Ngu;
            const float* xp = x + (live ? (((size_t)col.n * g.C + col.c0 + k_first + rsl) * g.H + col.h0) * g.W + col.w0 : 0);
            const uint32_t sbase = smem_u32(rawbase + slot.stage * Cfg::SLOT_BYTES);
            const uint32_t dst = sbase + (rsl * CP + j) * 8;
            const uint32_t dstg = sbase + Cfg::G_OFF + (rsl * CP + j) * (POOLED ? 4 : 8), dstx = sbase + Cfg::X_OFF + (rsl * CP + j) * 8;
            constexpr int GB = POOLED ? 4 : 8;                                  // bytes per pair in the dy part
            const bool full = live && m_first + Cfg::QR <= M && k_first + NT <= K;
#pragma unroll
            for (int i = 0; i < Cfg::QR / RS; ++i) {
                const bool in = full || (live && m_first + rsl + RS * i < M);
                const float* ys = in ? yp + (size_t)(RS * i) * Nu : y;
                const float* gs = in ? gp + (size_t)(RS * i) * Ngu : dy;
                const uint32_t dy_ = dst + (RS * i) * CP * 8, dg_ = dstg + (RS * i) * CP * GB;
                if (WIDE) {
                    pair_async16(dy_, ys, in);
                    if (POOLED) pair_async8(dg_, gs, in);                       // the pooled values of two neighbouring pairs
                    else pair_async16(dg_, gs, in);
                } else {
                    pair_async8(dy_, ys, in);
                    if (POOLED) pair_async4(dg_, gs, in);
                    else pair_async8(dg_, gs, in);
                }
            }
#pragma unroll
            for (int i = 0; i < Cfg::XR / RS; ++i) {
                const bool in = full || (live && k_first + rsl + RS * i < K);
                const float* xs = in ? xp + (size_t)(RS * i) * hw : x;
                if (WIDE) pair_async16(dstx + (RS * i) * CP * 8, xs, in);
                else pair_async8(dstx + (RS * i) * CP * 8, xs, in);
            }
            if (rsl == 0) {                                                     // the per-position maxima of the pairs
                const float* ms = live ? mx + (col.base - (long long)col.n * (M - 1) * g.N) : mx;
                if (WIDE) pair_async16(sbase + Cfg::MX_OFF + j * 8, ms, live);
                else pair_async8(sbase + Cfg::MX_OFF + j * 8, ms, live);
            }
            async_arrive_noinc(&sh.raw_full[slot.stage]);
            slot.advance(1);
        }
        pair_async_commit();
        pair_async_wait<0>();
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kDoMmaWarp)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    if (threadIdx.x == 0 && sh.failed) atomicExch(&flag[1], 1);
}

#define PAIR_RUN(KERNEL, THREADS, SMEM, GRID, ...)                               \
    do {                                                                        \
        static bool attr_done = false;                                          \
        const cudaError_t e_ = ws_set_smem(KERNEL, SMEM, attr_done);            \
        if (e_ != cudaSuccess) return e_;                                       \
        KERNEL<<<GRID, THREADS, SMEM, s>>>(__VA_ARGS__);                         \
    } while (0)

// two neighbouring pixel pairs of a tile are 16 contiguous, 16-byte aligned bytes in every tensor
inline bool mex_pair_wide(const MexGeo& g, const void* a, const void* b, const void* c, const void* d) {
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(d);
    return g.W % 4 == 0 && (bits & 15u) == 0;
}

inline int pair_nt(int n) { return n > 64 ? 128 : 64; }

template <int NT>
cudaError_t launch_fwd_pair_nt(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, float* y, float* pooled,
                               int* flag, int test_expire, cudaStream_t s) {
    const long long P = (long long)g.B * g.rs;
    const int mtiles = (g.M + NT - 1) / NT, pairs = g.R / 2;
    const long long items = ((P + kTcPos - 1) / kTcPos) * mtiles * pairs;
    if (items >= 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const WsPlan plan = {int(items), make_fastdiv(pairs), make_fastdiv(mtiles)};
    const int grid = int(std::min<long long>(items, ws_sm_count()));
    constexpr int smem = pair_stages<NT>() * pair_stage_bytes<NT>() + pair_raw_bytes<3, 8>();
    PAIR_RUN((mex_fwd_pair<NT, 3>), kPairThreads, smem, grid, g, x, tiles, mo, mx, y, pooled, plan, flag, test_expire);
    count_launch();
    return cudaGetLastError();
}

template <int NT, bool POOLED>
cudaError_t launch_dx_pair_nt(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, const float* y,
                              const float* dy, float* dx, int* flag, cudaStream_t s) {
    const long long P = (long long)g.B * g.rs;
    const int ktiles = (g.K + NT - 1) / NT, pairs = g.R / 2;
    const long long items = ((P + kTcPos - 1) / kTcPos) * ktiles * pairs;
    if (items >= 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const WsPlan plan = {int(items), make_fastdiv(pairs), make_fastdiv(ktiles)};
    const int grid = int(std::min<long long>(items, ws_sm_count()));
    constexpr int smem = pair_stages<NT>() * pair_stage_bytes<NT>() + dx_depth<POOLED>() * dx_slot_bytes<POOLED>();
    static_assert(smem <= 227 * 1024, "stages and slot ring must fit the shared memory of one CTA");
    if (mex_pair_wide(g, x, y, dy, dx)) PAIR_RUN((mex_dx_pair<NT, POOLED, true>), kDxThreads, smem, grid, g, x, tiles, mo, mx, y, dy, dx, plan, flag);
    else PAIR_RUN((mex_dx_pair<NT, POOLED, false>), kDxThreads, smem, grid, g, x, tiles, mo, mx, y, dy, dx, plan, flag);
    count_launch();
    return cudaGetLastError();
}

// tiling of the offsets gradient: instance tiles per CTA, tap tile width and pairs per chunk
inline void dopair_tiling(const MexGeo& g, int& mt, int& nt, int& cp) {
    mt = g.M > 128 ? 2 : 1;
    nt = g.K > 64 ? 128 : 64;
    cp = (mt == 1 && nt == 64) ? 16 : 8;
}

inline DoPairPlan dopair_plan(const MexGeo& g) {
    int mt, nt, cp;
    dopair_tiling(g, mt, nt, cp);
    DoPairPlan p;
    p.mgroups = ((g.M + 127) / 128 + mt - 1) / mt;
    p.ktiles = (g.K + nt - 1) / nt;
    p.units = (g.R / 2) * p.mgroups * p.ktiles;
    const long long chunks = ((long long)g.B * g.rs + cp - 1) / cp;
    long long s = ws_sm_count() / p.units;
    if (s > chunks) s = chunks;
    if (s < 1) s = 1;
    p.splits = int(s);
    return p;
}

// cuTensorMapEncodeTiled of the driver, looked up once (the library links no driver stub); nullptr if unavailable
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) != cudaSuccess || st != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// A float32 tensor seen as rank-4 or rank-5 (dims fastest first, strides in floats for dims 1..), one box per copy
inline bool encode_f32_map(CUtensorMap* map, const float* base, int rank, const long long* dims, const long long* strides, const int* box) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t gd[5], gs[4];
    cuuint32_t bd[5], es[5];
    for (int i = 0; i < rank; ++i) { gd[i] = cuuint64_t(dims[i]); bd[i] = cuuint32_t(box[i]); es[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) gs[i] = cuuint64_t(strides[i]) * 4;
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, cuuint32_t(rank), const_cast<float*>(base), gd, gs, bd, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The box copies need: one channel block and one region along the channels; rows of the region pair a fixed number of rows
// apart with the height a multiple of it; every global stride a multiple of 16 bytes (width a multiple of 4, of 8 for a
// pooled dy) and 16-byte aligned tensors; chunks that are runs of one row or whole rows and never straddle two samples.
template <int MT, int NT, int CP, bool POOLED>
bool doff_tma_maps(const MexGeo& g, const float* x, const float* mx, const float* y, const float* dy, DoMaps* maps) {
    const int rw = g.rw;                                     // pixel pairs per row
    if (g.Co != 1 || g.oc != 1 || g.rc != 1 || g.H % g.oh != 0 || g.rh * g.oh != g.H || g.W % 4 != 0 || g.rs % CP != 0) return false;
    if (!(rw % CP == 0 || CP % rw == 0)) return false;
    if (POOLED && (g.oh != 2 || g.W % 8 != 0)) return false;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(mx) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(dy)) & 15u) return false;
    const int cols = rw >= CP ? CP : rw, rows = rw >= CP ? 1 : CP / rw;      // pixel pairs per box row, box rows
    const long long W = g.W, H = g.H, N = g.N;
    {   // y[B][M][H][W] as (w, row class, row in class, instance, sample)
        const long long dims[5] = {W, g.oh, H / g.oh, g.M, g.B}, strides[4] = {W, W * g.oh, N, (long long)g.M * N};
        const int box[5] = {2 * cols, 1, rows, MT * 128, 1};
        if (!encode_f32_map(&maps->y, y, 5, dims, strides, box)) return false;
        if (!POOLED && !encode_f32_map(&maps->dy, dy, 5, dims, strides, box)) return false;
    }
    if (POOLED) {   // dy[B][M][H/2][W/2] as (w / 2, h / 2, instance, sample): one value per pixel pair and row pair
        const long long dims[4] = {W / 2, H / 2, g.M, g.B}, strides[3] = {W / 2, g.Ng, (long long)g.M * g.Ng};
        const int box[4] = {cols, rows, MT * 128, 1};
        if (!encode_f32_map(&maps->dy, dy, 4, dims, strides, box)) return false;
    }
    {   // x[B][C][H][W], channels of the block only
        const long long dims[5] = {W, g.oh, H / g.oh, g.K, g.B}, strides[4] = {W, W * g.oh, H * W, (long long)g.C * H * W};
        const int box[5] = {2 * cols, 1, rows, NT, 1};
        if (!encode_f32_map(&maps->x, x, 5, dims, strides, box)) return false;
    }
    {   // mx[B][H][W]
        const long long dims[4] = {W, g.oh, H / g.oh, g.B}, strides[3] = {W, W * g.oh, N};
        const int box[4] = {2 * cols, 1, rows, 1};
        if (!encode_f32_map(&maps->mx, mx, 4, dims, strides, box)) return false;
    }
    return true;
}

template <int MT, int NT, int CP, bool POOLED>
cudaError_t launch_doff_pair_p(const MexGeo& g, const DoPairPlan& plan, bool wide, const float* x, const float* mo, const float* mx,
                               const float* y, const float* dy, float* part, int* flag, cudaStream_t s) {
    constexpr int smem = DoCfg<MT, NT, CP, POOLED>::SMEM;
    const long long grid = (long long)plan.units * plan.splits;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    DoMaps maps;
    memset(&maps, 0, sizeof(maps));
    if (doff_tma_maps<MT, NT, CP, POOLED>(g, x, mx, y, dy, &maps))
        PAIR_RUN((mex_doff_pair<MT, NT, CP, POOLED, 2>), do_pair_threads(2), smem, int(grid), g, x, mo, mx, y, dy, part, plan, flag, maps);
    else if (wide) PAIR_RUN((mex_doff_pair<MT, NT, CP, POOLED, 1>), kDoPairThreads, smem, int(grid), g, x, mo, mx, y, dy, part, plan, flag, maps);
    else PAIR_RUN((mex_doff_pair<MT, NT, CP, POOLED, 0>), kDoPairThreads, smem, int(grid), g, x, mo, mx, y, dy, part, plan, flag, maps);
    count_launch();
    return cudaGetLastError();
}

template <int MT, int NT, int CP>
cudaError_t launch_doff_pair_t(const MexGeo& g, const DoPairPlan& plan, bool wide, const float* x, const float* mo, const float* mx,
                               const float* y, const float* dy, float* part, int* flag, cudaStream_t s) {
    return g.gp == 2 ? launch_doff_pair_p<MT, NT, CP, true>(g, plan, wide, x, mo, mx, y, dy, part, flag, s)
                     : launch_doff_pair_p<MT, NT, CP, false>(g, plan, wide, x, mo, mx, y, dy, part, flag, s);
}

}  // namespace

// Pair tiles serve a layer whose sibling regions alternate along the width (see the head of this file); pointers must
// allow 8-byte accesses of pixel pairs.
bool mex_pair_shape(const MexGeo& g) {
    return g.bh == 1 && g.bw == 1 && g.sh == 1 && g.sw == 1 && g.ph == 0 && g.pw == 0 && g.pc == 0 &&
           (g.Co - 1) * g.sc + g.bc <= g.C && g.Ho == g.H && g.Wo == g.W && g.unshared && g.ow == 2 && g.W % 2 == 0 &&
           g.R % 2 == 0 && g.rw * 2 == g.Wo && (g.gp == 1 || g.gp == 2);
}

bool mex_pair_aligned(const void* a, const void* b, const void* c, const void* d) {
    return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(d)) & 7u) == 0;
}

int mex_pair_nt_fwd(const MexGeo& g) { return pair_nt(g.M); }
int mex_pair_nt_dx(const MexGeo& g) { return pair_nt(g.K); }
int mex_pair_doff_splits(const MexGeo& g) { return dopair_plan(g).splits; }

size_t mex_pair_tile_floats(const MexGeo& g) {
    const int ntf = pair_nt(g.M), ntd = pair_nt(g.K);
    const size_t fwd = (size_t)g.R * ((g.M + ntf - 1) / ntf) * ((g.K + kTcKT - 1) / kTcKT) * 2 * ntf * kTcKT;
    const size_t dxf = (size_t)g.R * ((g.K + ntd - 1) / ntd) * ((g.M + kTcKT - 1) / kTcKT) * 2 * ntd * kTcKT;
    return fwd > dxf ? fwd : dxf;
}

cudaError_t launch_mex_fwd_pair(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, float* y,
                                float* pooled, int* flag, int test_expire, cudaStream_t s) {
    if (pooled != nullptr) {           // the epilogue adds the two halves of every pooling window onto zeros
        const cudaError_t e = cudaMemsetAsync(pooled, 0, sizeof(float) * (size_t)g.B * g.M * (g.N >> 2), s);
        if (e != cudaSuccess) return e;
    }
    if (pair_nt(g.M) == 128) return launch_fwd_pair_nt<128>(g, x, tiles, mo, mx, y, pooled, flag, test_expire, s);
    return launch_fwd_pair_nt<64>(g, x, tiles, mo, mx, y, pooled, flag, test_expire, s);
}

cudaError_t launch_mex_dx_pair(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, const float* y,
                               const float* dy, float* dx, int* flag, cudaStream_t s) {
    if (g.gp == 2) return pair_nt(g.K) == 128 ? launch_dx_pair_nt<128, true>(g, x, tiles, mo, mx, y, dy, dx, flag, s)
                                              : launch_dx_pair_nt<64, true>(g, x, tiles, mo, mx, y, dy, dx, flag, s);
    return pair_nt(g.K) == 128 ? launch_dx_pair_nt<128, false>(g, x, tiles, mo, mx, y, dy, dx, flag, s)
                               : launch_dx_pair_nt<64, false>(g, x, tiles, mo, mx, y, dy, dx, flag, s);
}

cudaError_t launch_mex_doff_pair(const MexGeo& g, const float* x, const float* mo, const float* mx, const float* y, const float* dy,
                                 float* part, int* splits_out, int* flag, cudaStream_t s) {
    const DoPairPlan plan = dopair_plan(g);
    *splits_out = plan.splits;
    int mt, nt, cp;
    dopair_tiling(g, mt, nt, cp);
    const bool wide = mex_pair_wide(g, x, y, dy, mx);
    if (mt == 1 && nt == 64) return launch_doff_pair_t<1, 64, 16>(g, plan, wide, x, mo, mx, y, dy, part, flag, s);
    if (mt == 1) return launch_doff_pair_t<1, 128, 8>(g, plan, wide, x, mo, mx, y, dy, part, flag, s);
    if (nt == 64) return launch_doff_pair_t<2, 64, 8>(g, plan, wide, x, mo, mx, y, dy, part, flag, s);
    return launch_doff_pair_t<2, 128, 8>(g, plan, wide, x, mo, mx, y, dy, part, flag, s);
}

}  // namespace simnets
