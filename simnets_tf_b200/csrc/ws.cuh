// Shared by the persistent, warp-specialised tensor-core MEX kernels: role layout of a CTA, the mbarrier ring that
// connects the roles, the bulk-copy loader of the pre-split offsets operand and the MMA issue loop.
#pragma once
#include "tc.cuh"

namespace simnets {
namespace {

constexpr int kWsGroups = 2;                        // producer groups; group i fills the stages of chunks i, i + 2, ...
constexpr int kWsProducerWarps = 4 * kWsGroups;     // warps 0..7: thread % 128 = position row of the tile
constexpr int kWsEpilogueWarps = 8;                 // warps 8..15: lane quarter = warp % 4, column half = (warp - 8) / 4
constexpr int kWsMmaWarp = kWsProducerWarps + kWsEpilogueWarps;
constexpr int kWsLoaderWarp = kWsMmaWarp + 1;
constexpr int kWsThreads = (kWsLoaderWarp + 1) * 32;   // 576

template <int STAGES>
struct WsShared {
    uint64_t full[STAGES];       // producers -> MMA: position operand of the stage stored (128 arrivals)
    uint64_t bfull[STAGES];      // loader -> MMA: offsets operand of the stage has landed (1 arrival + its bytes)
    uint64_t empty[STAGES];      // MMA -> producers, loader: the MMAs that read the stage are done
    uint64_t acc_full[2];        // MMA -> epilogue: accumulator complete
    uint64_t acc_empty[2];       // epilogue -> MMA: accumulator read out (256 arrivals)
    uint32_t tmem;
    volatile int failed;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One contiguous global -> shared copy of `bytes` (multiple of 16, both addresses 16-byte aligned) by the copy engine;
// the barrier's current phase completes once this thread's arrival and all the bytes are in.
__device__ __forceinline__ void bulk_copy_to_smem(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int NT>
__host__ __device__ constexpr int ws_stage_bytes() { return 2 * kTcPos * kTcKT * 4 + 2 * NT * kTcKT * 4; }

template <int NT>
__host__ __device__ constexpr int ws_stages() { return NT == 256 ? 3 : 4; }

// Everything a role needs to walk the item list without a division: the list (fewer than 2^31 items) and exact
// multiply-shift dividers for the number of regions and of instance tiles.
struct WsPlan { int items; FastDiv f_R, f_mt; };

// work item -> (region, instance tile, position tile); consecutive items share their x tile
struct WsItem { int r, mt, jt; };
__device__ __forceinline__ WsItem ws_item(const WsPlan& p, int item) {
    WsItem w;
    const uint32_t q = fast_div(uint32_t(item), p.f_R);
    w.r = item - int(q * p.f_R.d);
    w.jt = int(fast_div(q, p.f_mt));
    w.mt = int(q) - w.jt * int(p.f_mt.d);
    return w;
}

// Position in the ring of shared-memory stages: the stage and how many times it has been filled before.
template <int STAGES>
struct WsRing {
    int stage;
    uint32_t fill;
    __device__ __forceinline__ void advance(int by) { stage += by; if (stage >= STAGES) { stage -= STAGES; ++fill; } }
};

// Barriers and tensor memory of a persistent CTA; returns the tensor-memory base address.
template <int STAGES>
__device__ __forceinline__ uint32_t ws_setup(WsShared<STAGES>& sh, uint32_t tmem_cols) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full[s], 128); mbar_init(&sh.bfull[s], 1); mbar_init(&sh.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh.acc_full[b], 1); mbar_init(&sh.acc_empty[b], kWsEpilogueWarps * 32); }
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if ((threadIdx.x >> 5) == kWsMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    return sh.tmem;
}

// Every role ends here: frees the tensor memory and reports a wait that expired.
template <int STAGES>
__device__ __forceinline__ void ws_teardown(WsShared<STAGES>& sh, uint32_t tmem, uint32_t tmem_cols, int* __restrict__ flag) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if ((threadIdx.x >> 5) == kWsMmaWarp)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
    if (threadIdx.x == 0 && sh.failed) atomicExch(&flag[1], 1);     // results of this launch are invalid
}

// Loader role: the pre-split offsets operand of every stage, one bulk copy each (hi plane then lo plane).  `tiles` is
// laid out [region][row tile][chunk][2 planes][NT x 16] as mex_tc_prep writes it; an item's row tile is its `mt`.
template <int NT, int STAGES>
__device__ __forceinline__ void ws_loader_role(WsShared<STAGES>& sh, unsigned char* dsm, const float* __restrict__ tiles, const WsPlan& plan,
                                               int my_items, int row_tiles, int chunks) {
    constexpr int A_BYTES = kTcPos * kTcKT * 4, B_BYTES = NT * kTcKT * 4, STAGE_BYTES = ws_stage_bytes<NT>();
    if ((threadIdx.x & 31) == 0) {
        WsRing<STAGES> ring = {0, 0u};
        int issued = 0;                                            // copies issued, saturating at STAGES
        for (int li = 0; li < my_items && !sh.failed; ++li) {
            const WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
            const float* src = tiles + ((size_t)it.r * row_tiles + it.mt) * chunks * 2 * NT * kTcKT;
            bool ok = true;
            for (int c = 0; c < chunks; ++c, src += 2 * NT * kTcKT) {
                if (ring.fill >= 1 && !mbar_wait(&sh.empty[ring.stage], (ring.fill - 1) & 1u)) { ok = false; break; }
                bulk_copy_to_smem(dsm + ring.stage * STAGE_BYTES + 2 * A_BYTES, src, 2 * B_BYTES, &sh.bfull[ring.stage]);
                ring.advance(1);
                if (issued < STAGES) ++issued;
            }
            if (!ok) { sh.failed = 1; break; }
        }
        // copies still in flight must land before the CTA may exit (they have, on the normal path): walk back
        // over the last `issued` stages
        for (int d = 0; d < issued; ++d) {
            if (ring.stage == 0) { ring.stage = STAGES; --ring.fill; }
            --ring.stage;
            if (!mbar_wait(&sh.bfull[ring.stage], ring.fill & 1u)) sh.failed = 1;
        }
    }
    __syncwarp();
}

// MMA role: the warp walks the items together, lane 0 issues.  D[128 x NT] of item li goes to accumulator li % 2.
template <int NT, int STAGES>
__device__ __forceinline__ void ws_mma_role(WsShared<STAGES>& sh, unsigned char* dsm, uint32_t tmem, int my_items, int chunks) {
    constexpr int A_BYTES = kTcPos * kTcKT * 4, B_BYTES = NT * kTcKT * 4, STAGE_BYTES = ws_stage_bytes<NT>();
    constexpr uint32_t idesc = umma_idesc(NT);
    constexpr int SBO = (kTcKT / 4) * 128;
    const int lane = threadIdx.x & 31;
    WsRing<STAGES> ring = {0, 0u};
    for (int li = 0; li < my_items; ++li) {
        const int buf = li & 1;
        const uint32_t round = uint32_t(li) >> 1;
        if (sh.failed) break;
        if (round >= 1 && !mbar_wait(&sh.acc_empty[buf], (round - 1) & 1u)) { sh.failed = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem + uint32_t(buf * NT);
        bool ok = true;
        for (int c = 0; c < chunks; ++c) {
            const int stage = ring.stage;
            if (!mbar_wait(&sh.full[stage], ring.fill & 1u) || !mbar_wait(&sh.bfull[stage], ring.fill & 1u)) { ok = false; break; }
            ring.advance(1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint32_t a_hi = smem_u32(dsm + stage * STAGE_BYTES), a_lo = a_hi + A_BYTES, b_hi = a_hi + 2 * A_BYTES, b_lo = b_hi + B_BYTES;
#pragma unroll
                for (int ks = 0; ks < kTcKT / 8; ++ks) {
                    const uint32_t o = ks * 2 * 128;
                    const uint64_t dah = umma_desc(a_hi + o, 128, SBO), dal = umma_desc(a_lo + o, 128, SBO);
                    const uint64_t dbh = umma_desc(b_hi + o, 128, SBO), dbl = umma_desc(b_lo + o, 128, SBO);
                    umma_tf32(tmem_d, dal, dbh, idesc, (c | ks) != 0);
                    umma_tf32(tmem_d, dah, dbl, idesc, 1);
                    umma_tf32(tmem_d, dah, dbh, idesc, 1);
                }
                umma_commit(&sh.empty[stage]);
            }
            __syncwarp();
        }
        if (!ok) { sh.failed = 1; break; }
        if (lane == 0) umma_commit(&sh.acc_full[buf]);
        __syncwarp();
    }
}

inline int ws_sm_count() { return device_sm_count(); }

template <class Kernel>
cudaError_t ws_set_smem(Kernel kernel, int smem, bool& done) {
    if (done) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) done = true;
    return e;
}

#define WS_RUN(KERNEL, SMEM, GRID, ...)                                         \
    do {                                                                        \
        static bool attr_done = false;                                          \
        const cudaError_t e_ = ws_set_smem(KERNEL, SMEM, attr_done);            \
        if (e_ != cudaSuccess) return e_;                                       \
        KERNEL<<<GRID, kWsThreads, SMEM, s>>>(__VA_ARGS__);                      \
    } while (0)


}  // namespace
}  // namespace simnets
