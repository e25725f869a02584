// Persistent, warp-specialised tensor-core MEX kernels.
//
// Same GEMM formulation, operand layouts and split-TF32 scheme as mex_tc.cu, but one CTA per SM that walks a list of
// work items, with its warps split into three roles that run concurrently and hand tiles to one another through
// mbarriers:
//   producers   two groups of four warps, each filling every other stage of a shared-memory ring: load x (or y, dy),
//               evaluate the exponentials, split them into TF32 hi / lo and store the position operand;
//   loader      one thread copies the pre-split offsets tile of each stage with a bulk asynchronous copy that
//               completes on the stage's own mbarrier (it runs up to a whole ring ahead);
//   one thread  issues the tcgen05 MMAs of each full stage; tcgen05.commit releases the stage back to the
//               producers and the loader and, after an item's last stage, publishes the accumulator;
//   epilogue    warps read the accumulator from tensor memory, finish the arithmetic and store.
// The accumulator is double buffered in tensor memory, so the epilogue of item i overlaps the loads and MMAs of
// item i + 1: global-memory latency, MMA latency and the epilogue's stores no longer add up per tile as they do in
// the one-tile-per-CTA kernels.  Every mbarrier wait is bounded; a wait that expires raises the CTA's failure flag,
// every role leaves its loop at the next check, the tensor memory is freed and flag[1] tells the host.
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

// ---- forward ---------------------------------------------------------------------------------------------------
template <int NT, bool SPATIAL1, bool INTERIOR>
__global__ void __launch_bounds__(kWsThreads, 1) mex_fwd_ws(MexGeo g, const float* __restrict__ x, const float* __restrict__ tiles,
                                                           const float* __restrict__ mo, const float* __restrict__ mx,
                                                           float* __restrict__ y, WsPlan plan, int* __restrict__ flag) {
    constexpr int STAGES = ws_stages<NT>();
    constexpr int A_BYTES = kTcPos * kTcKT * 4, STAGE_BYTES = ws_stage_bytes<NT>();
    constexpr uint32_t TMEM_COLS = 2 * NT < 32 ? 32 : 2 * NT;
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ WsShared<STAGES> sh;
    __shared__ __align__(16) float mo_w[kWsEpilogueWarps][NT / 2];
    __shared__ int tap_tab[SPATIAL1 ? 1 : kTapTable];
    if (flag[0]) return;                                // factorisation unsafe: the exact kernels run instead
    if (!SPATIAL1) fill_tap_table(g, tap_tab);          // (published by the barrier inside ws_setup)
    const bool tab_ok = tap_table_ok(g);

    const long long P = (long long)g.B * g.rs;
    const int mtiles = (g.M + NT - 1) / NT, kchunks = (g.K + kTcKT - 1) / kTcKT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int my_items = plan.items > int(blockIdx.x) ? (plan.items - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;

    const uint32_t tmem = ws_setup(sh, TMEM_COLS);

    if (warp < kWsProducerWarps) {
        // ---------------- producers: thread % 128 = position row; 16 taps per stage; group = every other chunk
        const int prow = threadIdx.x % kTcPos, group = threadIdx.x / kTcPos;
        const float a = float(g.eps) * 1.4426950408889634f, oob = float(g.oob);     // exp(eps * (x - mx)) = 2^(a * x - a * mx)
        int li = group / kchunks, c = group % kchunks;                // item (local index) and chunk held in xv
        WsRing<STAGES> ring = {group, 0u};                            // kWsGroups <= STAGES
        WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
        Column col = column_of(g, it.r, (long long)it.jt * kTcPos + prow, P, mx);
        float xv[kTcKT];
        const int K = g.K;
        const unsigned hw = unsigned(g.H) * unsigned(g.W);
        auto load = [&](int c) {
            const bool live = col.base >= 0;
            if (SPATIAL1 && INTERIOR) {
                // 1x1 blocks that never leave the input: tap u of the chunk is channel c0 + 16 c + u of one pixel,
                // consecutive taps are one plane (H * W floats) apart
                const float* xp = x + ((size_t)col.n * g.C + col.c0 + c * kTcKT) * hw + (size_t)col.h0 * g.W + col.w0;
                if (live && (c + 1) * kTcKT <= K) {
#pragma unroll
                    for (int u = 0; u < kTcKT; ++u) xv[u] = __ldg(xp + (size_t)u * hw);
                } else {
#pragma unroll
                    for (int u = 0; u < kTcKT; ++u) xv[u] = (live && c * kTcKT + u < K) ? __ldg(xp + (size_t)u * hw) : 0.f;
                }
            } else {
                const float* xs = x + (size_t)col.n * g.C * hw;
#pragma unroll
                for (int u = 0; u < kTcKT; ++u) {
                    const int k = c * kTcKT + u;
                    xv[u] = 0.f;
                    if (live && k < K)
                    {
                        const Tap tp = tap_get<SPATIAL1>(g, tap_tab, tab_ok, k);
                        xv[u] = INTERIOR ? __ldg(xs + ((col.c0 + tp.c) * g.H + col.h0 + tp.h) * g.W + col.w0 + tp.w)
                                         : patch_value_at(g, xs, col.c0, col.h0, col.w0, tp, oob);
                    }
                }
            }
        };
        if (li < my_items) load(c);
        for (; li < my_items;) {
            const int stage = ring.stage;
            unsigned char* sA = dsm + stage * STAGE_BYTES;
            if (sh.failed) break;
            float e[kTcKT];
            {
                // x - mx first: both may be far from zero while their difference is small.  A dead row holds x = 0 and
                // gets an infinite maximum of the sign that makes a * (x - mx) = -inf, i.e. every tap 0
                const float mxd = col.base >= 0 ? col.mx : (a > 0.f ? INFINITY : -INFINITY);
#pragma unroll
                for (int u = 0; u < kTcKT; ++u) e[u] = ex2_ftz(a * (xv[u] - mxd));
                if ((c + 1) * kTcKT > K) {
#pragma unroll
                    for (int u = 0; u < kTcKT; ++u) if (c * kTcKT + u >= K) e[u] = 0.f;
                }
            }
            // this group's next chunk goes in flight now; it lands while this one is split, stored and handed over
            c += kWsGroups;
            if (c >= kchunks) {
                do { c -= kchunks; ++li; } while (c >= kchunks);
                if (li < my_items) {
                    it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
                    col = column_of(g, it.r, (long long)it.jt * kTcPos + prow, P, mx);
                }
            }
            if (li < my_items) load(c);
            if (ring.fill >= 1 && !mbar_wait(&sh.empty[stage], (ring.fill - 1) & 1u)) { sh.failed = 1; break; }
#pragma unroll
            for (int h = 0; h < kTcKT / 4; ++h) {
                float4 hi, lo;
                split_tf32_trunc(e[4 * h], hi.x, lo.x); split_tf32_trunc(e[4 * h + 1], hi.y, lo.y);
                split_tf32_trunc(e[4 * h + 2], hi.z, lo.z); split_tf32_trunc(e[4 * h + 3], hi.w, lo.w);
                const int off = core_offset(prow, 4 * h);
                *reinterpret_cast<float4*>(sA + off) = hi;
                *reinterpret_cast<float4*>(sA + A_BYTES + off) = lo;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&sh.full[stage]);
            ring.advance(kWsGroups);
        }
    } else if (warp == kWsLoaderWarp) {
        ws_loader_role<NT, STAGES>(sh, dsm, tiles, plan, my_items, mtiles, kchunks);
    } else if (warp == kWsMmaWarp) {
        ws_mma_role<NT, STAGES>(sh, dsm, tmem, my_items, kchunks);
    } else {
        // ---------------- epilogue: lane = position, registers = instances
        const int quarter = warp & 3, half = (warp - kWsProducerWarps) >> 2;     // 8 % 4 == 0: warp % 4 is the lane quarter this warp may read
        float* mow = mo_w[warp - kWsProducerWarps];                              // this warp's slice of the item's offset maxima
        const float inv_eps = 1.f / float(g.eps), k_log = 0.69314718056f * inv_eps, c_add = float(g.cst) * inv_eps;
        const unsigned Nu = unsigned(g.N);                                       // distance between instances in y (32 N < 2^31)
        for (int li = 0; li < my_items; ++li) {
            const int buf = li & 1;
            if (sh.failed) break;
            const WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
            const int m0 = it.mt * NT + half * (NT / 2);
            for (int i = lane; i < NT / 2; i += 32) mow[i] = m0 + i < g.M ? __ldg(mo + it.r * g.M + m0 + i) : 0.f;
            __syncwarp();
            const Column col = column_of(g, it.r, (long long)it.jt * kTcPos + quarter * 32 + lane, P, mx);
            const float cadd = col.mx + c_add;
            float* yb = y + (col.base >= 0 ? col.base : 0) + (long long)m0 * g.N;
            const bool full = m0 + NT / 2 <= g.M;
            if (!mbar_wait(&sh.acc_full[buf], (uint32_t(li) >> 1) & 1u)) { sh.failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < NT / 2; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + uint32_t(buf * NT + half * (NT / 2) + c0) + (uint32_t(quarter * 32) << 16), v);
                if (col.base >= 0) {
                    float* yp = yb + (size_t)c0 * Nu;                   // the 32 instances of the block: 32-bit offsets i * N
                    if (full) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const float4 o4 = *reinterpret_cast<const float4*>(mow + c0 + i);
                            __stcs(yp + (i + 0) * Nu, fmaf(lg2_ftz(__uint_as_float(v[i + 0])), k_log, cadd + o4.x));
                            __stcs(yp + (i + 1) * Nu, fmaf(lg2_ftz(__uint_as_float(v[i + 1])), k_log, cadd + o4.y));
                            __stcs(yp + (i + 2) * Nu, fmaf(lg2_ftz(__uint_as_float(v[i + 2])), k_log, cadd + o4.z));
                            __stcs(yp + (i + 3) * Nu, fmaf(lg2_ftz(__uint_as_float(v[i + 3])), k_log, cadd + o4.w));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (m0 + c0 + i < g.M) __stcs(yp + i * Nu, fmaf(lg2_ftz(__uint_as_float(v[i])), k_log, cadd + mow[c0 + i]));
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&sh.acc_empty[buf]);
            __syncwarp();                                   // every lane is done with this item's mow
        }
    }

    ws_teardown(sh, tmem, TMEM_COLS, flag);
}

// ---- input gradient ----------------------------------------------------------------------------------------------
// T[j (position, lane), k (tap, column)] = sum_m Q[j, m] * Eo[m, k];  dx[tap k of position j] = Ex[j, k] * T[j, k], with
// Q[j, m] = dy * 2^(a mx_j + (a mo_m + c') - a y).  Item = (region, tap tile of NT, position tile of 128); a stage holds
// 16 instances.  Blocks must not overlap.  tiles: Eo^T pre-split by mex_tc_prep (rows = taps).
template <int NT, bool SPATIAL1, bool INTERIOR>
__global__ void __launch_bounds__(kWsThreads, 1) mex_dx_ws(MexGeo g, const float* __restrict__ x, const float* __restrict__ tiles,
                                                          const float* __restrict__ mo, const float* __restrict__ mx,
                                                          const float* __restrict__ y, const float* __restrict__ dy,
                                                          float* __restrict__ dx, WsPlan plan, int* __restrict__ flag) {
    constexpr int STAGES = ws_stages<NT>();
    constexpr int A_BYTES = kTcPos * kTcKT * 4, STAGE_BYTES = ws_stage_bytes<NT>();
    constexpr uint32_t TMEM_COLS = 2 * NT < 32 ? 32 : 2 * NT;
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ WsShared<STAGES> sh;
    __shared__ int tap_tab[SPATIAL1 ? 1 : kTapTable];
    if (flag[0]) return;
    if (!SPATIAL1) fill_tap_table(g, tap_tab);          // (published by the barrier inside ws_setup)
    const bool tab_ok = tap_table_ok(g);

    const long long P = (long long)g.B * g.rs;
    const int ktiles = (g.K + NT - 1) / NT, mchunks = (g.M + kTcKT - 1) / kTcKT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int my_items = plan.items > int(blockIdx.x) ? (plan.items - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const uint32_t tmem = ws_setup(sh, TMEM_COLS);
    const float a = float(g.eps) * 1.4426950408889634f, c2 = float(g.cst) * 1.4426950408889634f;

    if (warp < kWsProducerWarps) {
        // ---------------- producers: thread % 128 = position row; 16 instances per stage; group = every other chunk
        const int prow = threadIdx.x % kTcPos, group = threadIdx.x / kTcPos;
        const int M = g.M;
        const unsigned Nu = unsigned(g.N), Ngu = unsigned(g.Ng);            // 32-bit offsets u * N: 16 N < 2^31
        int li = group / mchunks, c = group % mchunks;
        WsRing<STAGES> ring = {group, 0u};
        WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
        Column col = column_of(g, it.r, (long long)it.jt * kTcPos + prow, P, mx);
        float yv[kTcKT], gv[kTcKT];
        auto load = [&](int c) {
            const bool live = col.base >= 0;
            const int m0 = c * kTcKT;
            const float* yp = y + (live ? col.base : 0) + (size_t)m0 * Nu;
            const float* gp = dy + (live ? col.gbase : 0) + (size_t)m0 * Ngu;
            if (m0 + kTcKT <= M) {
#pragma unroll
                for (int u = 0; u < kTcKT; ++u) {
                    yv[u] = live ? __ldcs(yp + u * Nu) : 0.f;               // a dead row must not read a stranger's y: 0 * 2^(big) = NaN
                    gv[u] = live ? __ldcs(gp + u * Ngu) : 0.f;                // dy = 0: no contribution
                }
            } else {
#pragma unroll
                for (int u = 0; u < kTcKT; ++u) {
                    const bool in = m0 + u < M;
                    yv[u] = (in && live) ? __ldcs(yp + u * Nu) : 0.f;
                    gv[u] = (in && live) ? __ldcs(gp + u * Ngu) : 0.f;
                }
            }
        };
        if (li < my_items) load(c);
        for (; li < my_items;) {
            const int stage = ring.stage;
            unsigned char* sA = dsm + stage * STAGE_BYTES;
            if (sh.failed) break;
            float q[kTcKT];
            {
                const float mxv = col.mx;
                const float* mor = mo + it.r * M + c * kTcKT;               // offset maxima of this chunk's instances (cached, same for all lanes)
#pragma unroll
                for (int u = 0; u < kTcKT; ++u) {
                    const float mv = c * kTcKT + u < M ? __ldg(mor + u) : 0.f;
                    q[u] = gv[u] * ex2_ftz(fmaf(a, (mxv - yv[u]) + mv, c2));
                }
            }
            c += kWsGroups;
            if (c >= mchunks) {
                do { c -= mchunks; ++li; } while (c >= mchunks);
                if (li < my_items) {
                    it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
                    col = column_of(g, it.r, (long long)it.jt * kTcPos + prow, P, mx);
                }
            }
            if (li < my_items) load(c);
            if (ring.fill >= 1 && !mbar_wait(&sh.empty[stage], (ring.fill - 1) & 1u)) { sh.failed = 1; break; }
#pragma unroll
            for (int h = 0; h < kTcKT / 4; ++h) {
                float4 hi, lo;
                split_tf32_trunc(q[4 * h], hi.x, lo.x); split_tf32_trunc(q[4 * h + 1], hi.y, lo.y);
                split_tf32_trunc(q[4 * h + 2], hi.z, lo.z); split_tf32_trunc(q[4 * h + 3], hi.w, lo.w);
                const int off = core_offset(prow, 4 * h);
                *reinterpret_cast<float4*>(sA + off) = hi;
                *reinterpret_cast<float4*>(sA + A_BYTES + off) = lo;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&sh.full[stage]);
            ring.advance(kWsGroups);
        }
    } else if (warp == kWsLoaderWarp) {
        ws_loader_role<NT, STAGES>(sh, dsm, tiles, plan, my_items, ktiles, mchunks);
    } else if (warp == kWsMmaWarp) {
        ws_mma_role<NT, STAGES>(sh, dsm, tmem, my_items, mchunks);
    } else {
        // ---------------- epilogue: lane = position, registers = taps
        const int quarter = warp & 3, half = (warp - kWsProducerWarps) >> 2;
        const unsigned hw = unsigned(g.H) * unsigned(g.W);                   // 32 H W < 2^31 (checked by the shape predicate)
        for (int li = 0; li < my_items; ++li) {
            const int buf = li & 1;
            if (sh.failed) break;
            const WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));        // it.mt = tap tile
            const Column col = column_of(g, it.r, (long long)it.jt * kTcPos + quarter * 32 + lane, P, mx);
            const float emx = col.mx;                                        // Ex = 2^(a (x - mx))
            const int k_first = it.mt * NT + half * (NT / 2);
            if (!mbar_wait(&sh.acc_full[buf], (uint32_t(li) >> 1) & 1u)) { sh.failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (SPATIAL1 && INTERIOR) {
                // tap k of a 1x1 block that never leaves the input: channel c0 + k of one pixel, planes H * W floats apart
                const size_t first = (((size_t)col.n * g.C + col.c0 + k_first) * g.H + col.h0) * g.W + col.w0;
#pragma unroll 1
                for (int c0 = 0; c0 < NT / 2; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem + uint32_t(buf * NT + half * (NT / 2) + c0) + (uint32_t(quarter * 32) << 16), v);
                    if (col.base >= 0) {
                        const float* xb = x + first + (size_t)c0 * hw;
                        float* db = dx + first + (size_t)c0 * hw;
                        const int kleft = g.K - k_first - c0;
#pragma unroll
                        for (int i0 = 0; i0 < 32; i0 += 8) {             // eight loads in flight, then their eight stores
                            float xr[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) xr[i] = (i0 + i < kleft) ? ld_nc_ordered(xb + (i0 + i) * hw) : 0.f;
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if (i0 + i < kleft) db[(i0 + i) * hw] = ex2_ftz(a * (xr[i] - emx)) * __uint_as_float(v[i0 + i]);
                        }
                    }
                }
            } else {
                const size_t sample = (size_t)col.n * g.C * g.H * g.W;
#pragma unroll 1
                for (int c0 = 0; c0 < NT / 2; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem + uint32_t(buf * NT + half * (NT / 2) + c0) + (uint32_t(quarter * 32) << 16), v);
                    if (col.base >= 0) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int k = k_first + c0 + i;
                            if (k >= g.K) continue;
                            const Tap tp = tap_get<SPATIAL1>(g, tap_tab, tab_ok, k);
                            const int cc = col.c0 + tp.c, hh = col.h0 + tp.h, ww = col.w0 + tp.w;
                            if (cc < 0 || cc >= g.C || hh < 0 || hh >= g.H || ww < 0 || ww >= g.W) continue;
                            const size_t ad = sample + ((size_t)cc * g.H + hh) * g.W + ww;
                            dx[ad] = ex2_ftz(a * (__ldg(x + ad) - emx)) * __uint_as_float(v[i]);
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&sh.acc_empty[buf]);
        }
    }
    ws_teardown(sh, tmem, TMEM_COLS, flag);
}

int ws_sm_count() {
    static int sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    return sms[dev];
}

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

template <int NT>
cudaError_t launch_fwd_ws_nt(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, float* y, int* flag,
                             bool sp1, bool interior, cudaStream_t s) {
    const long long P = (long long)g.B * g.rs;
    const int mtiles = (g.M + NT - 1) / NT;
    const long long items = ((P + kTcPos - 1) / kTcPos) * mtiles * g.R;
    if (items >= 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const WsPlan plan = {int(items), make_fastdiv(g.R), make_fastdiv(mtiles)};
    const int grid = int(std::min<long long>(items, ws_sm_count()));
    constexpr int smem = ws_stages<NT>() * ws_stage_bytes<NT>();
    if (sp1) {
        if (interior) WS_RUN((mex_fwd_ws<NT, true, true>), smem, grid, g, x, tiles, mo, mx, y, plan, flag);
        else WS_RUN((mex_fwd_ws<NT, true, false>), smem, grid, g, x, tiles, mo, mx, y, plan, flag);
    } else {
        if (interior) WS_RUN((mex_fwd_ws<NT, false, true>), smem, grid, g, x, tiles, mo, mx, y, plan, flag);
        else WS_RUN((mex_fwd_ws<NT, false, false>), smem, grid, g, x, tiles, mo, mx, y, plan, flag);
    }
    count_launch();
    return cudaGetLastError();
}

template <int NT>
cudaError_t launch_dx_ws_nt(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, const float* y,
                            const float* dy, float* dx, int* flag, cudaStream_t s) {
    const long long P = (long long)g.B * g.rs;
    const int ktiles = (g.K + NT - 1) / NT;
    const long long items = ((P + kTcPos - 1) / kTcPos) * ktiles * g.R;
    if (items >= 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const WsPlan plan = {int(items), make_fastdiv(g.R), make_fastdiv(ktiles)};
    const int grid = int(std::min<long long>(items, ws_sm_count()));
    constexpr int smem = ws_stages<NT>() * ws_stage_bytes<NT>();
    if (g.bh == 1 && g.bw == 1) {
        if (patches_inside_input(g)) WS_RUN((mex_dx_ws<NT, true, true>), smem, grid, g, x, tiles, mo, mx, y, dy, dx, plan, flag);
        else WS_RUN((mex_dx_ws<NT, true, false>), smem, grid, g, x, tiles, mo, mx, y, dy, dx, plan, flag);
    } else {
        WS_RUN((mex_dx_ws<NT, false, false>), smem, grid, g, x, tiles, mo, mx, y, dy, dx, plan, flag);
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace

// tiles: Eo^T pre-split by launch_mex_tc_prep(g, true, ...) (NT = tile width picked for K, as mex_dx_tc).
cudaError_t launch_mex_dx_ws(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, const float* y,
                             const float* dy, float* dx, int* flag, cudaStream_t s) {
    const int nt = g.K > 128 ? 256 : (g.K > 64 ? 128 : 64);
    switch (nt) {
    case 256: return launch_dx_ws_nt<256>(g, x, tiles, mo, mx, y, dy, dx, flag, s);
    case 128: return launch_dx_ws_nt<128>(g, x, tiles, mo, mx, y, dy, dx, flag, s);
    default: return launch_dx_ws_nt<64>(g, x, tiles, mo, mx, y, dy, dx, flag, s);
    }
}

// tiles: Eo pre-split by launch_mex_tc_prep(g, false, ...) (same tiling as mex_fwd_tc: NT = mex_tc_nt(g)).
cudaError_t launch_mex_fwd_ws(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, float* y,
                              int* flag, bool interior, cudaStream_t s) {
    const bool sp1 = g.bh == 1 && g.bw == 1;
    switch (mex_tc_nt(g)) {
    case 256: return launch_fwd_ws_nt<256>(g, x, tiles, mo, mx, y, flag, sp1, interior, s);
    case 128: return launch_fwd_ws_nt<128>(g, x, tiles, mo, mx, y, flag, sp1, interior, s);
    default: return launch_fwd_ws_nt<64>(g, x, tiles, mo, mx, y, flag, sp1, interior, s);
    }
}

}  // namespace simnets
