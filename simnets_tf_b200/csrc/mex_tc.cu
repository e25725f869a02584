// MEX forward, input gradient and offsets gradient on the 5th-generation tensor cores (tcgen05, accumulators
// in tensor memory).
//
// After the factorisation of mex_tiled.cu all three passes are plain GEMMs over operands derived from x, y, dy
// and the offsets:  forward  S[j, m] = sum_k Ex[j, k] * Eo[m, k];  input gradient  T[j, k] = sum_m Q[j, m] * Eo[m, k]
// (dx = Ex * T);  offsets gradient  U[m, k] = sum_j Q[m, j] * Ex[k, j]  (dO = Eo * U), with Q = dy * G.
// FP32 accuracy is kept with the split-TF32 scheme: every operand is written to
// shared memory as hi = round-to-TF32(v) and lo = v - hi, and each k-step issues three MMAs
// (hi*hi + hi*lo + lo*hi); the dropped lo*lo term and the truncation of lo are below 3 * 2^-21 of a product, and
// all products are positive, so S keeps ~6 significant digits (tests compare y at 1e-5 of tensor scale).
//
// Tile: 128 positions (the MMA's M, one per tensor-memory lane) x NT instances (the MMA's N, NT = 64/128/256,
// one per tensor-memory column).  Positions are the lane dimension on purpose: in the epilogue lane = position,
// so for every instance the 32 lanes of a warp store to 32 neighbouring positions (coalesced), exactly as the
// CUDA-core kernels do.  256 threads: each stage (16 taps) they compute Ex = exp(eps*(x - mx)) for 128 x 16 values,
// split them and store them in the canonical K-major core-matrix layout (8 rows x 16 bytes, no swizzle), copy the
// matching pre-split Eo tile with cp.async, fence to the async proxy, and one thread issues the six MMAs of the
// stage; tcgen05.commit arrives on an mbarrier that frees the stage (two stages).  Every mbarrier wait is bounded:
// on expiry the kernel records an error word, still waits for its copies, frees its tensor memory and returns.
#include "tc.cuh"

namespace simnets {

namespace {

// ---- prepass: a [rows x red] matrix split into hi / lo, laid out tile by tile exactly as the MMA reads it -------
// tiles[r][row tile of NT][chunk of 16 along red][plane][NT * 16 floats]; out-of-range entries are zero.
// Forward: rows = instances, red = taps (source Eo[r][m][ld]); input gradient: rows = taps, red = instances (Eo^T).
__global__ void __launch_bounds__(256) mex_tc_prep(int R, int rows, int red, int ld, int NT, const float* __restrict__ src, float* __restrict__ tiles) {
    const int chunks = (red + kTcKT - 1) / kTcKT, rtiles = (rows + NT - 1) / NT;
    const long long total = (long long)R * rtiles * chunks * NT * kTcKT;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int kk = int(i % kTcKT);
        long long q = i / kTcKT;
        const int row = int(q % NT); q /= NT;
        const int kc = int(q % chunks); q /= chunks;
        const int rt = int(q % rtiles), r = int(q / rtiles);
        const int gr = rt * NT + row, gk = kc * kTcKT + kk;
        const float v = (gr < rows && gk < red) ? src[((size_t)r * rows + gr) * ld + gk] : 0.f;
        float hi, lo;
        split_tf32(v, hi, lo);
        float* tile = tiles + (((size_t)r * rtiles + rt) * chunks + kc) * 2 * NT * kTcKT;
        tile[core_offset(row, kk) / 4] = hi;
        tile[NT * kTcKT + core_offset(row, kk) / 4] = lo;
    }
}

// ---- forward ---------------------------------------------------------------------------------------------------
template <int NT, bool SPATIAL1, bool INTERIOR>
__global__ void __launch_bounds__(kTcThreads) mex_fwd_tc(MexGeo g, const float* __restrict__ x, const float* __restrict__ tiles,
                                                        const float* __restrict__ mo, const float* __restrict__ mx,
                                                        float* __restrict__ y, int* __restrict__ flag) {
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ TcShared sh;
    __shared__ float mo_s[NT];
    if (flag[0]) return;                                // factorisation unsafe: the exact kernels run instead

    const long long P = (long long)g.B * g.rs;
    const int mtiles = (g.M + NT - 1) / NT, kchunks = (g.K + kTcKT - 1) / kTcKT;
    int bid = blockIdx.x;
    const int r = bid % g.R; bid /= g.R;
    const int mt = bid % mtiles;
    const long long jt = bid / mtiles;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < NT; i += kTcThreads) mo_s[i] = (mt * NT + i < g.M) ? mo[r * g.M + mt * NT + i] : 0.f;
    const uint32_t tmem_d = tc_begin(sh, NT);

    // staging role: position row = tid % 128, taps (tid / 128) * 8 .. + 7 of every stage
    const int prow = threadIdx.x % kTcPos, khalf = threadIdx.x / kTcPos;
    const Column sc = column_of(g, r, jt * kTcPos + prow, P, mx);
    const bool live = sc.base >= 0;
    const float* xs = x + (size_t)sc.n * g.C * g.H * g.W;
    const float eps = float(g.eps), oob = float(g.oob);
    const float* btiles = tiles + ((size_t)r * mtiles + mt) * kchunks * 2 * NT * kTcKT;

    float xv[8];                                             // raw taps of the chunk being prefetched
    auto load = [&](int c) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int k = c * kTcKT + khalf * 8 + u;
            xv[u] = 0.f;
            if (live && k < g.K)
                xv[u] = INTERIOR ? __ldg(xs + interior_index<SPATIAL1>(g, sc.c0, sc.h0, sc.w0, k))
                                 : patch_value<SPATIAL1>(g, xs, sc.c0, sc.h0, sc.w0, k, oob);
        }
    };
    auto store = [&](int c, unsigned char* a_hi, unsigned char* a_lo, unsigned char* b_hi, unsigned char*) {
        // instance operand: verbatim copy of the pre-split tile (hi plane then lo plane, contiguous)
        const float* src = btiles + (size_t)c * 2 * NT * kTcKT;
        for (int v = threadIdx.x; v < 2 * NT * kTcKT / 4; v += kTcThreads) cp_async16(reinterpret_cast<float*>(b_hi) + v * 4, src + v * 4, 16);
        // position operand: 8 taps of this thread's position
        float e[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) e[u] = (live && c * kTcKT + khalf * 8 + u < g.K) ? fast_exp(eps * (xv[u] - sc.mx)) : 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {                            // two 16-byte groups of 4 taps
            float4 hi, lo;
            split_tf32(e[4 * h], hi.x, lo.x); split_tf32(e[4 * h + 1], hi.y, lo.y);
            split_tf32(e[4 * h + 2], hi.z, lo.z); split_tf32(e[4 * h + 3], hi.w, lo.w);
            const int off = core_offset(prow, khalf * 8 + 4 * h);
            *reinterpret_cast<float4*>(a_hi + off) = hi;
            *reinterpret_cast<float4*>(a_lo + off) = lo;
        }
    };
    const bool good = tc_mainloop<NT, kTcKT, 128, 2>(sh, dsm, tmem_d, kchunks, load, store);

    // epilogue: lane = position, registers = instances.  Warps w and w + 4 share a lane quarter and split the columns.
    if (good) {
        const int quarter = warp & 3, half = warp >> 2;
        const Column col = column_of(g, r, jt * kTcPos + quarter * 32 + lane, P, mx);
        const float inv_eps = 1.f / eps, k_log = 0.69314718056f * inv_eps;
        const float cadd = col.mx + float(g.cst) * inv_eps;
        float* yb = y + (col.base >= 0 ? col.base : 0);
#pragma unroll 1
        for (int c0 = half * (NT / 2); c0 < (half + 1) * (NT / 2); c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_d + (uint32_t(quarter * 32) << 16) + uint32_t(c0), v);
            if (col.base >= 0) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int m = mt * NT + c0 + i;
                    if (m < g.M) __stcs(yb + (long long)m * g.N, fmaf(__log2f(__uint_as_float(v[i])), k_log, cadd + mo_s[c0 + i]));
                }
            }
        }
    } else if (threadIdx.x == 0) {
        atomicExch(&flag[1], 1);                                 // a wait expired: results of this launch are invalid
    }
    tc_end(tmem_d, NT);
}

// ---- input gradient ----------------------------------------------------------------------------------------------
// T[j (position, lane), k (tap, column)] = sum_m Q[j, m] * Eo[m, k];  dx[tap k of position j] = Ex[j, k] * T[j, k].
// A = Q computed from y, dy (reads coalesced along positions), B = pre-split Eo^T tiles.  Blocks must not overlap.
constexpr int kDxMaxM = 2048;      // instances whose a * mo + c' fit the kernel's shared-memory table (larger M: CUDA-core kernels)

template <int NT, bool SPATIAL1, bool INTERIOR>
__global__ void __launch_bounds__(kTcThreads, NT == 256 ? 2 : 3) mex_dx_tc(MexGeo g, const float* __restrict__ x, const float* __restrict__ tiles,
                                                       const float* __restrict__ mo, const float* __restrict__ mx,
                                                       const float* __restrict__ y, const float* __restrict__ dy,
                                                       float* __restrict__ dx, int* __restrict__ flag) {
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ TcShared sh;
    __shared__ int tap_tab[SPATIAL1 ? 1 : kTapTable];
    if (flag[0]) return;
    if (!SPATIAL1) fill_tap_table(g, tap_tab);            // (published by the barrier inside tc_begin)
    const bool tab_ok = tap_table_ok(g);
    const long long P = (long long)g.B * g.rs;
    const int ktiles = (g.K + NT - 1) / NT, mchunks = (g.M + kTcKT - 1) / kTcKT;
    // mo of every instance of the region, rounded up to a whole chunk, behind the operand stages (sized by the launcher:
    // a fixed table for the largest M would cost the fourth CTA per multiprocessor)
    constexpr int kStages = tc_smem_bytes<NT, kTcKT, 128, 2>();
    float* amo_s = reinterpret_cast<float*>(dsm + kStages);
    int bid = blockIdx.x;
    const int r = bid % g.R; bid /= g.R;
    const int kt = bid % ktiles;
    const long long jt = bid / ktiles;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Q[j, m] = dy * exp(eps * (mx_j + mo_m - y) + c) = dy * 2^(a * ((mx_j - y) + mo_m) + c'),  a = eps * log2(e).  The
    // difference mx - y is taken first: both can be hundreds of units from zero while their difference is small.
    const float a = float(g.eps) * 1.4426950408889634f, c2 = float(g.cst) * 1.4426950408889634f;
    for (int i = threadIdx.x; i < mchunks * kTcKT; i += kTcThreads) amo_s[i] = i < g.M ? mo[r * g.M + i] : 0.f;
    const uint32_t tmem_d = tc_begin(sh, NT);             // (its barrier also publishes amo_s)

    const int prow = threadIdx.x % kTcPos, mhalf = threadIdx.x / kTcPos;
    const Column sc = column_of(g, r, jt * kTcPos + prow, P, mx);
    const bool live = sc.base >= 0;
    const float mxv = sc.mx;
    // Running pointers to (this thread's first instance of the next chunk to load, its position); the eight instances
    // of a chunk are addressed with 32-bit element offsets u * N from them (the launcher checks 16 * N < 2^31).
    const unsigned Nu = unsigned(g.N), Ngu = unsigned(g.Ng);
    const float* yp = y + (live ? sc.base : 0) + (size_t)(mhalf * 8) * Nu;
    const float* gp = dy + (live ? sc.gbase : 0) + (size_t)(mhalf * 8) * Ngu;
    const float* btiles = tiles + ((size_t)r * ktiles + kt) * mchunks * 2 * NT * kTcKT;
    const int M = g.M;

    // two register sets of raw y / dy values: the loads of chunk c + 2 are issued as soon as chunk c has been consumed
    float yv[2][8], gv[2][8];
    auto load = [&](int c, auto parity) {
        constexpr int S = decltype(parity)::value;
        const int m0 = c * kTcKT + mhalf * 8;
        if (m0 + 8 <= M) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                yv[S][u] = live ? __ldcs(yp + u * Nu) : 0.f;            // a dead row must not read a stranger's y: 0 * 2^(big) = NaN
                gv[S][u] = live ? __ldcs(gp + u * Ngu) : 0.f;
            }
        } else {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool in = m0 + u < M;
                yv[S][u] = (in && live) ? __ldcs(yp + u * Nu) : 0.f;
                gv[S][u] = (in && live) ? __ldcs(gp + u * Ngu) : 0.f;   // dy = 0: no contribution
            }
        }
        yp += (size_t)kTcKT * Nu;
        gp += (size_t)kTcKT * Ngu;
    };
    auto bcopy = [&](int c, unsigned char* b_hi) {
        const float* src = btiles + (size_t)c * 2 * NT * kTcKT;
        for (int v = threadIdx.x; v < 2 * NT * kTcKT / 4; v += kTcThreads) cp_async16(reinterpret_cast<float*>(b_hi) + v * 4, src + v * 4, 16);
    };
    auto store = [&](int c, auto parity, unsigned char* a_hi, unsigned char* a_lo) {
        constexpr int S = decltype(parity)::value;
        const float* mv = amo_s + c * kTcKT + mhalf * 8;                // (padded with zeros up to a whole chunk)
        float q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) q[u] = gv[S][u] * ex2_ftz(fmaf(a, (mxv - yv[S][u]) + mv[u], c2));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float4 hi, lo;
            split_tf32_trunc(q[4 * h], hi.x, lo.x); split_tf32_trunc(q[4 * h + 1], hi.y, lo.y);
            split_tf32_trunc(q[4 * h + 2], hi.z, lo.z); split_tf32_trunc(q[4 * h + 3], hi.w, lo.w);
            const int off = core_offset(prow, mhalf * 8 + 4 * h);
            *reinterpret_cast<float4*>(a_hi + off) = hi;
            *reinterpret_cast<float4*>(a_lo + off) = lo;
        }
    };
    const bool good = tc_mainloop_ahead2<NT, kTcKT, 128>(sh, dsm, tmem_d, mchunks, load, store, bcopy);

    if (good) {
        const int quarter = warp & 3, half = warp >> 2;
        const Column col = column_of(g, r, jt * kTcPos + quarter * 32 + lane, P, mx);
        const float emx = col.mx;                                      // Ex = 2^(a * (x - mx))
        if (SPATIAL1 && INTERIOR) {
            // tap k of a 1x1 block that never leaves the input: channel c0 + k of one pixel, planes H * W floats apart
            const unsigned hw = unsigned(g.H) * unsigned(g.W);           // the launcher takes this path only if NT * H * W < 2^31
            const size_t first = (((size_t)col.n * g.C + col.c0 + kt * NT) * g.H + col.h0) * g.W + col.w0;
            const float* xb = x + first;
            float* db = dx + first;
#pragma unroll 1
            for (int c0 = half * (NT / 2); c0 < (half + 1) * (NT / 2); c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_d + (uint32_t(quarter * 32) << 16) + uint32_t(c0), v);
                if (col.base >= 0) {
                    const int kleft = g.K - kt * NT - c0;
                    unsigned off = unsigned(c0) * hw;
#pragma unroll
                    for (int i0 = 0; i0 < 32; i0 += 8) {                 // eight loads in flight, then their eight stores
                        float xr[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) xr[i] = (i0 + i < kleft) ? ld_nc_ordered(xb + (off + i * hw)) : 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (i0 + i < kleft) db[off + i * hw] = ex2_ftz(a * (xr[i] - emx)) * __uint_as_float(v[i0 + i]);
                        off += 8 * hw;
                    }
                }
            }
        } else {
            const size_t sample = (size_t)col.n * g.C * g.H * g.W;
#pragma unroll 1
            for (int c0 = half * (NT / 2); c0 < (half + 1) * (NT / 2); c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_d + (uint32_t(quarter * 32) << 16) + uint32_t(c0), v);
                if (col.base >= 0) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int k = kt * NT + c0 + i;
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
    } else if (threadIdx.x == 0) {
        atomicExch(&flag[1], 1);
    }
    tc_end(tmem_d, NT);
}

// ---- offsets gradient --------------------------------------------------------------------------------------------
// U[m (instance, lane), k (tap, column)] = sum over this split's positions j of Q[m, j] * Ex[k, j]; both operands are
// computed on the fly with lanes running along positions (coalesced reads of y, dy, x) and stored one float at a
// time; a leading byte offset of 144 spreads the eight 16-byte chunks of a row over all banks.
constexpr int kDoKT = 32, kDoLBO = 144;

template <int NT, bool SPATIAL1, bool INTERIOR>
__global__ void __launch_bounds__(kTcThreads, NT == 64 ? 3 : 2) mex_doff_tc(MexGeo g, const float* __restrict__ x, const float* __restrict__ mo,
                                                         const float* __restrict__ mx, const float* __restrict__ y,
                                                         const float* __restrict__ dy, float* __restrict__ part, int splits,
                                                         int* __restrict__ flag) {
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ TcShared sh;
    __shared__ float amo_s[128];                        // mo of this CTA's instances
    __shared__ int tap_tab[SPATIAL1 ? 1 : kTapTable];
    if (flag[0]) return;
    if (!SPATIAL1) fill_tap_table(g, tap_tab);          // (published by the barrier inside tc_begin)
    const bool tab_ok = tap_table_ok(g);
    const long long P = (long long)g.B * g.rs;
    const int mtiles = (g.M + 127) / 128, ktiles = (g.K + NT - 1) / NT;
    int bid = blockIdx.x;
    const int kt = bid % ktiles; bid /= ktiles;
    const int mt = bid % mtiles; bid /= mtiles;
    const int r = bid % g.R;
    const int split = bid / g.R;
    const long long chunks = (P + kDoKT - 1) / kDoKT;
    const long long c_begin = chunks * split / splits, c_end = chunks * (split + 1) / splits;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Q = dy * 2^(a * ((mx - y) + mo) + c'),  Ex = 2^(a * (x - mx)),  a = eps * log2(e); differences first (see mex_dx_tc)
    const float a = float(g.eps) * 1.4426950408889634f, c2 = float(g.cst) * 1.4426950408889634f, oob = float(g.oob);
    if (threadIdx.x < 128) amo_s[threadIdx.x] = (mt * 128 + threadIdx.x < g.M) ? mo[r * g.M + mt * 128 + threadIdx.x] : 0.f;
    const uint32_t tmem_d = tc_begin(sh, NT);

    const int M = g.M, K = g.K;
    const int m0 = mt * 128 + warp * 16;                 // this warp's 16 instances
    const int k0 = kt * NT + warp * (NT / 8);            // and its NT / 8 taps
    const unsigned Nu = unsigned(g.N), Ngu = unsigned(g.Ng);        // 32-bit element offsets u * N below: 16 * N < 2^31
    const unsigned hw = unsigned(g.H) * unsigned(g.W);
    const bool m_full = m0 + 16 <= M, k_full = k0 + NT / 8 <= K;

    // registers of the chunk being prefetched: lane = position of the chunk, this warp's 16 instances and NT / 8 taps
    Column col;
    float yv[16], gv[16], xv[NT / 8];
    auto load = [&](int c) {
        col = column_of(g, r, (c_begin + c) * kDoKT + lane, P, mx);
        const bool live = col.base >= 0;
        const float* yp = y + (live ? col.base : 0) + (size_t)m0 * Nu;
        const float* gp = dy + (live ? col.gbase : 0) + (size_t)m0 * Ngu;
        if (m_full) {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                yv[u] = live ? __ldcs(yp + u * Nu) : 0.f;               // a dead row must not read a stranger's y: 0 * 2^(big) = NaN
                gv[u] = live ? __ldcs(gp + u * Ngu) : 0.f;               // dy = 0: no contribution
            }
        } else {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const bool in = m0 + u < M;
                yv[u] = (in && live) ? __ldcs(yp + u * Nu) : 0.f;
                gv[u] = (in && live) ? __ldcs(gp + u * Ngu) : 0.f;
            }
        }
        if (SPATIAL1 && INTERIOR) {
            const float* xp = x + (((size_t)col.n * g.C + col.c0 + k0) * g.H + col.h0) * g.W + col.w0;
#pragma unroll
            for (int u = 0; u < NT / 8; ++u) xv[u] = (live && (k_full || k0 + u < K)) ? __ldg(xp + u * hw) : 0.f;
        } else {
            const float* xs = x + (size_t)col.n * g.C * g.H * g.W;
#pragma unroll
            for (int u = 0; u < NT / 8; ++u)
                xv[u] = (live && k0 + u < K) ? patch_value_at(g, xs, col.c0, col.h0, col.w0, tap_get<SPATIAL1>(g, tap_tab, tab_ok, k0 + u), oob) : 0.f;
        }
    };
    auto store = [&](int, unsigned char* a_hi, unsigned char* a_lo, unsigned char* b_hi, unsigned char* b_lo) {
        const bool live = col.base >= 0;
        const float mxv = col.mx;
        const float mxd = live ? mxv : (a > 0.f ? INFINITY : -INFINITY);     // dead column: x = 0, so a * (x - mxd) = -inf and Ex = 0
#pragma unroll
        for (int u = 0; u < 16; ++u) {                           // A: Q[m, j]
            const int row = warp * 16 + u;
            float hi, lo;
            split_tf32_trunc(gv[u] * ex2_ftz(fmaf(a, (mxv - yv[u]) + amo_s[row], c2)), hi, lo);
            const int off = core_off<kDoKT, kDoLBO>(row, lane);
            *reinterpret_cast<float*>(a_hi + off) = hi;
            *reinterpret_cast<float*>(a_lo + off) = lo;
        }
#pragma unroll
        for (int u = 0; u < NT / 8; ++u) {                       // B: Ex[k, j]
            const int row = warp * (NT / 8) + u;
            float hi, lo;
            split_tf32_trunc((k_full || k0 + u < K) ? ex2_ftz(a * (xv[u] - mxd)) : 0.f, hi, lo);
            const int off = core_off<kDoKT, kDoLBO>(row, lane);
            *reinterpret_cast<float*>(b_hi + off) = hi;
            *reinterpret_cast<float*>(b_lo + off) = lo;
        }
    };
    const bool good = tc_mainloop<NT, kDoKT, kDoLBO, 1>(sh, dsm, tmem_d, int(c_end - c_begin), load, store);

    if (good) {
        const int quarter = warp & 3, half = warp >> 2;
        const int m = mt * 128 + quarter * 32 + lane;
        float* dst = part + (((size_t)split * g.R + r) * g.M + (m < g.M ? m : 0)) * g.K;
#pragma unroll 1
        for (int c0 = half * (NT / 2); c0 < (half + 1) * (NT / 2); c0 += 32) {
            uint32_t v[32];
            if (c_end > c_begin) tmem_ld32(tmem_d + (uint32_t(quarter * 32) << 16) + uint32_t(c0), v);
            if (m < g.M) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int k = kt * NT + c0 + i;
                    if (k < g.K) dst[k] = c_end > c_begin ? __uint_as_float(v[i]) : 0.f;
                }
            }
        }
    } else if (threadIdx.x == 0) {
        atomicExch(&flag[1], 1);
    }
    tc_end(tmem_d, NT);
}

template <class Kernel>
cudaError_t set_smem_once(Kernel kernel, int smem, bool& done) {
    if (done) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) done = true;
    return e;
}

#define TC_RUN(KERNEL, SMEM, GRID, ...)                                        \
    do {                                                                       \
        static bool attr_done = false;                                         \
        const cudaError_t e_ = set_smem_once(KERNEL, SMEM, attr_done);          \
        if (e_ != cudaSuccess) return e_;                                      \
        KERNEL<<<GRID, kTcThreads, SMEM, s>>>(__VA_ARGS__);                     \
    } while (0)

template <int NT>
cudaError_t launch_fwd_nt(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, float* y, int* flag,
                          bool sp1, bool interior, cudaStream_t s) {
    const long long P = (long long)g.B * g.rs;
    const long long blocks = ((P + kTcPos - 1) / kTcPos) * ((g.M + NT - 1) / NT) * g.R;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    constexpr int smem = tc_smem_bytes<NT, kTcKT, 128, 2>();
    if (sp1) {
        if (interior) TC_RUN((mex_fwd_tc<NT, true, true>), smem, int(blocks), g, x, tiles, mo, mx, y, flag);
        else TC_RUN((mex_fwd_tc<NT, true, false>), smem, int(blocks), g, x, tiles, mo, mx, y, flag);
    } else {
        if (interior) TC_RUN((mex_fwd_tc<NT, false, true>), smem, int(blocks), g, x, tiles, mo, mx, y, flag);
        else TC_RUN((mex_fwd_tc<NT, false, false>), smem, int(blocks), g, x, tiles, mo, mx, y, flag);
    }
    count_launch();
    return cudaGetLastError();
}

template <int NT>
cudaError_t launch_dx_nt(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, const float* y,
                         const float* dy, float* dx, int* flag, cudaStream_t s) {
    const long long P = (long long)g.B * g.rs;
    const long long blocks = ((P + kTcPos - 1) / kTcPos) * ((g.K + NT - 1) / NT) * g.R;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    if (g.M > kDxMaxM) return cudaErrorInvalidConfiguration;
    constexpr int smem_max = tc_smem_bytes<NT, kTcKT, 128, 2>() + kDxMaxM * 4;
    const int smem = tc_smem_bytes<NT, kTcKT, 128, 2>() + ((g.M + kTcKT - 1) / kTcKT) * kTcKT * 4;
#define DX_RUN(KERNEL)                                                                              \
    do {                                                                                            \
        static bool attr_done = false;                                                              \
        const cudaError_t e_ = set_smem_once(KERNEL, smem_max, attr_done);                          \
        if (e_ != cudaSuccess) return e_;                                                           \
        KERNEL<<<int(blocks), kTcThreads, smem, s>>>(g, x, tiles, mo, mx, y, dy, dx, flag);         \
    } while (0)
    if (g.bh == 1 && g.bw == 1) {
        if (patches_inside_input(g) && (long long)NT * g.H * g.W < 0x7fffffffLL) DX_RUN((mex_dx_tc<NT, true, true>));
        else DX_RUN((mex_dx_tc<NT, true, false>));
    } else {
        DX_RUN((mex_dx_tc<NT, false, false>));
    }
#undef DX_RUN
    count_launch();
    return cudaGetLastError();
}

template <int NT>
cudaError_t launch_doff_nt(const MexGeo& g, const float* x, const float* mo, const float* mx, const float* y, const float* dy,
                           float* part, int splits, int* flag, cudaStream_t s) {
    const long long blocks = (long long)((g.M + 127) / 128) * ((g.K + NT - 1) / NT) * g.R * splits;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    constexpr int smem = tc_smem_bytes<NT, kDoKT, kDoLBO, 1>();
    if (g.bh == 1 && g.bw == 1) {
        if (patches_inside_input(g)) TC_RUN((mex_doff_tc<NT, true, true>), smem, int(blocks), g, x, mo, mx, y, dy, part, splits, flag);
        else TC_RUN((mex_doff_tc<NT, true, false>), smem, int(blocks), g, x, mo, mx, y, dy, part, splits, flag);
    } else {
        TC_RUN((mex_doff_tc<NT, false, false>), smem, int(blocks), g, x, mo, mx, y, dy, part, splits, flag);
    }
    count_launch();
    return cudaGetLastError();
}

inline int pick_nt(int n) { return n > 128 ? 256 : (n > 64 ? 128 : 64); }

}  // namespace

int mex_tc_nt(const MexGeo& g) { return pick_nt(g.M); }

// floats of the pre-split tiles: forward (rows = instances) and input gradient (rows = taps) side by side
size_t mex_tc_tile_floats(const MexGeo& g) {
    const int ntf = pick_nt(g.M), ntd = pick_nt(g.K);
    const size_t fwd = (size_t)g.R * ((g.M + ntf - 1) / ntf) * ((g.K + kTcKT - 1) / kTcKT) * 2 * ntf * kTcKT;
    const size_t dxf = (size_t)g.R * ((g.K + ntd - 1) / ntd) * ((g.M + kTcKT - 1) / kTcKT) * 2 * ntd * kTcKT;
    return fwd > dxf ? fwd : dxf;
}

// number of position splits of the tensor-core offsets gradient (each CTA: 128 instances x NT taps)
int mex_tc_doff_splits(const MexGeo& g) {
    const int nt = pick_nt(g.K);
    const long long P = (long long)g.B * g.rs, chunks = (P + kDoKT - 1) / kDoKT;
    const long long tiles = (long long)((g.M + 127) / 128) * ((g.K + nt - 1) / nt) * g.R;
    const int per_sm = nt == 64 ? 3 : 2;                         // CTAs per SM that the register budget allows
    long long s = ((long long)device_sm_count() * per_sm) / tiles;                      // one full wave: measured against a half, two and four (the partial sums are 128 x NT floats per CTA)
    if (s > chunks) s = chunks;
    if (s < 1) s = 1;
    if (s > 512) s = 512;
    return int(s);
}

cudaError_t launch_mex_tc_prep(const MexGeo& g, bool transposed, const float* src, float* tiles, cudaStream_t s, int nt) {
    const int rows = transposed ? g.K : g.M, red = transposed ? g.M : g.K, NT = nt > 0 ? nt : pick_nt(rows);
    const long long total = (long long)g.R * ((rows + NT - 1) / NT) * ((red + kTcKT - 1) / kTcKT) * NT * kTcKT;
    mex_tc_prep<<<int(std::min<long long>((total + 255) / 256, (long long)device_sm_count() * 8)), 256, 0, s>>>(g.R, rows, red, pad4(red), NT, src, tiles);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_fwd_tc(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, float* y,
                              int* flag, bool interior, cudaStream_t s) {
    const bool sp1 = g.bh == 1 && g.bw == 1;
    switch (pick_nt(g.M)) {
    case 256: return launch_fwd_nt<256>(g, x, tiles, mo, mx, y, flag, sp1, interior, s);
    case 128: return launch_fwd_nt<128>(g, x, tiles, mo, mx, y, flag, sp1, interior, s);
    default: return launch_fwd_nt<64>(g, x, tiles, mo, mx, y, flag, sp1, interior, s);
    }
}

cudaError_t launch_mex_dx_tc(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, const float* y,
                             const float* dy, float* dx, int* flag, cudaStream_t s) {
    switch (pick_nt(g.K)) {
    case 256: return launch_dx_nt<256>(g, x, tiles, mo, mx, y, dy, dx, flag, s);
    case 128: return launch_dx_nt<128>(g, x, tiles, mo, mx, y, dy, dx, flag, s);
    default: return launch_dx_nt<64>(g, x, tiles, mo, mx, y, dy, dx, flag, s);
    }
}

cudaError_t launch_mex_doff_tc(const MexGeo& g, const float* x, const float* mo, const float* mx, const float* y, const float* dy,
                               float* part, int splits, int* flag, cudaStream_t s) {
    switch (pick_nt(g.K)) {
    case 256: return launch_doff_nt<256>(g, x, mo, mx, y, dy, part, splits, flag, s);
    case 128: return launch_doff_nt<128>(g, x, mo, mx, y, dy, part, splits, flag, s);
    default: return launch_doff_nt<64>(g, x, mo, mx, y, dy, part, splits, flag, s);
    }
}

}  // namespace simnets
