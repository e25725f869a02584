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
#include "ws.cuh"

namespace simnets {

namespace {

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
        // This warp's column of the first item; from then on the column of item li + 1 (an index division and a load of the
        // position's maximum) is requested before the arithmetic of item li, so that its latency is not paid per item.
        WsItem it = ws_item(plan, int(blockIdx.x));
        Column col;
        col.base = -1; col.mx = 0.f;
        if (my_items > 0) col = column_of(g, it.r, (long long)it.jt * kTcPos + quarter * 32 + lane, P, mx);
        int held_r = -1, held_mt = -1;                                           // whose offset maxima mow holds
        for (int li = 0; li < my_items; ++li) {
            const int buf = li & 1;
            if (sh.failed) break;
            const int m0 = it.mt * NT + half * (NT / 2);
            if (it.r != held_r || it.mt != held_mt) {
                __syncwarp();                                   // every lane is done with the previous contents
                for (int i = lane; i < NT / 2; i += 32) mow[i] = m0 + i < g.M ? __ldg(mo + it.r * g.M + m0 + i) : 0.f;
                __syncwarp();
                held_r = it.r; held_mt = it.mt;
            }
            const float cadd = col.mx + c_add;
            const bool live = col.base >= 0;
            float* yb = y + (live ? col.base : 0) + (long long)m0 * g.N;
            const bool full = m0 + NT / 2 <= g.M;
            WsItem nit = it;
            Column ncol = col;
            if (li + 1 < my_items) {
                nit = ws_item(plan, int(blockIdx.x) + (li + 1) * int(gridDim.x));
                ncol = column_of(g, nit.r, (long long)nit.jt * kTcPos + quarter * 32 + lane, P, mx);
            }
            if (!mbar_wait(&sh.acc_full[buf], (uint32_t(li) >> 1) & 1u)) { sh.failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < NT / 2; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + uint32_t(buf * NT + half * (NT / 2) + c0) + (uint32_t(quarter * 32) << 16), v);
                if (live) {
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
            it = nit;
            col = ncol;
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
