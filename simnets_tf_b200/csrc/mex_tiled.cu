// MEX forward / input-gradient / offsets-gradient as factorised generalized GEMMs (float32).
//
// The reference evaluates y[m,j] = mx + log(sum_k exp(eps*(x[k,j] + o[m,k] - mx)) + c)/eps with one
// exp per (m, k, j) term (HUJI-Deep/simnets-tf src/kernels/mex_kernel_cpu.cpp:11-38,
// include/utils/mex_utils.hpp:10-29): M*N*K exponentials per sample, which binds the kernel to the
// special-function unit, not to memory.  Here the exponent is split per operand:
//
//     exp(eps*(x[k,j] + o[m,k])) = exp(eps*(x[k,j] - mx[j])) * exp(eps*(o[m,k] - mo[m])) * exp(eps*(mx[j] + mo[m]))
//          Ex[k,j] in (0,1]  ^                 Eo[m,k] in (0,1]  ^
//
// with mx[j] = max_k x[k,j] and mo[m] = max_k o[m,k] (min for eps < 0), so that
//     S[m,j] = sum_k Eo[m,k] * Ex[k,j]          -- a plain FP32 GEMM, K*N + M*K exponentials in total
//     y[m,j] = mx[j] + mo[m] + (log S[m,j] + c)/eps
// and, with the softmax weight p = Eo*Ex*G,  G[m,j] = exp(eps*(mx[j] + mo[m] - y[m,j]) + c)
// (mex_utils.hpp:31-56 computes p = exp(eps*(x + o - y) + c) directly),
//     dX patch[k,j] = Ex[k,j] * sum_m Eo[m,k] * (dy*G)[m,j]
//     dO[m,k]       = Eo[m,k] * sum_j (dy*G)[m,j] * Ex[k,j].
// S >= exp(-|eps| * (max_k o - min_k o)) whenever the offsets are finite, so the factorisation cannot
// underflow if |eps| * spread(o) <= 60; a prepass checks exactly that and raises a device flag
// otherwise, in which case these kernels return at once and the exact one-exp-per-term kernels
// (direct_kernels.cu), launched right behind them and gated on the same flag, do the work.
//
// Offset regions (shared / unshared) never move data: a CTA works on the positions of ONE region,
// enumerated in the region-local order of the reference's split_patches (mex_utils.hpp:69-116).
#include <mutex>
#include "kernels.cuh"
#include "tile.cuh"
#include "mex_common.cuh"

namespace simnets {

namespace {

// ------------------------------------------------------------------ prepasses
// One block per (region, instance): stabiliser mo, Eo in both layouts, and the safety flag.  With tile pointers the block
// also writes its part of the tensor-core operand tiles (Eo split into TF32 hi / lo, laid out as the MMA reads it: what
// mex_tc_prep produces in a launch of its own): tf = forward tiles, rows = instances in tiles of ntf, reduction = taps;
// td = input-gradient tiles, rows = taps in tiles of ntd, reduction = instances.  The grid then also covers the rows that
// pad the last instance tile or chunk (gridDim.x = R * Mp, Mp >= M): those blocks write zeros only.
__device__ __forceinline__ float prep_tf32_hi(float v) { uint32_t r; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v)); return __uint_as_float(r); }
__device__ __forceinline__ int prep_core_offset(int row, int k) { return (row >> 3) * 128 + (k >> 2) * 32 + (row & 7) * 4 + (k & 3); }   // floats, 16-wide chunks

__global__ void __launch_bounds__(512) mex_prep_offsets(MexGeo g, int Mp, const float* __restrict__ off, float* __restrict__ mo,
                                                        float* __restrict__ eo, float* __restrict__ eot, int* __restrict__ flag,
                                                        float* __restrict__ tf, int ntf, float* __restrict__ td, int ntd,
                                                        float* __restrict__ offn, float* __restrict__ lse_out) {
    __shared__ float s_hi[512], s_lo[512];
    __shared__ int s_bad[512];
    const int nt = blockDim.x;                       // 128, or 512 for long rows
    const int r = blockIdx.x / Mp, m = blockIdx.x % Mp;
    const bool real = m < g.M;
    const int rm = r * g.M + m;
    const float* o = off + (size_t)rm * g.K;
    float hi = -CUDART_INF_F, lo = CUDART_INF_F;
    int bad = 0;
    if (real) {
        for (int k = threadIdx.x; k < g.K; k += nt) {
            const float v = o[k];
            if (!isfinite(v)) bad = 1;
            hi = fmaxf(hi, v); lo = fminf(lo, v);
        }
    }
    s_hi[threadIdx.x] = hi; s_lo[threadIdx.x] = lo; s_bad[threadIdx.x] = bad;
    __syncthreads();
    for (int s = nt / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            s_hi[threadIdx.x] = fmaxf(s_hi[threadIdx.x], s_hi[threadIdx.x + s]);
            s_lo[threadIdx.x] = fminf(s_lo[threadIdx.x], s_lo[threadIdx.x + s]);
            s_bad[threadIdx.x] |= s_bad[threadIdx.x + s];
        }
        __syncthreads();
    }
    hi = s_hi[0]; lo = s_lo[0]; bad = s_bad[0];
    const float eps = float(g.eps);
    const float ref = eps > 0.f ? hi : lo;
    // SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS: the op works on offsets minus the log-sum-exp of their row.  Eo = exp(eps (o - ref))
    // does not change; the row's reference value does, and the shifted row is kept for the exact kernels.
    float lse = 0.f;
    if (offn != nullptr) {
        __syncthreads();
        const float base = (hi == CUDART_INF_F || hi == -CUDART_INF_F) ? 0.f : hi;      // as a stable log-sum-exp treats infinite maxima
        float sum = 0.f;
        if (real) for (int k = threadIdx.x; k < g.K; k += nt) sum += expf(o[k] - base);
        s_hi[threadIdx.x] = sum;
        __syncthreads();
        for (int s = nt / 2; s > 0; s >>= 1) {
            if (threadIdx.x < s) s_hi[threadIdx.x] += s_hi[threadIdx.x + s];
            __syncthreads();
        }
        lse = base + logf(s_hi[0]);
        if (real) {
            for (int k = threadIdx.x; k < g.K; k += nt) offn[(size_t)rm * g.K + k] = o[k] - lse;
            if (threadIdx.x == 0) lse_out[rm] = lse;
        }
    }
    if (real && threadIdx.x == 0) {
        mo[rm] = ref - lse;
        if (bad || !(fabsf(eps) * (hi - lo) <= kSafeSpread)) atomicOr(flag, 1);
    }
    // taps up to the padding of the tiles: chunks of 16 for the forward tiles, whole tap tiles for the input-gradient tiles
    const int kchunks = (g.K + 15) / 16, mchunks = (g.M + 15) / 16;
    const int mtiles = tf ? (g.M + ntf - 1) / ntf : 0, ktiles = td ? (g.K + ntd - 1) / ntd : 0;
    int kend = g.K;
    if (tf && m < mtiles * ntf) kend = max(kend, kchunks * 16);
    if (td && m < mchunks * 16) kend = max(kend, ktiles * ntd);
    for (int k = threadIdx.x; k < kend; k += nt) {
        const float e = (real && k < g.K) ? fast_exp(eps * (o[k] - ref)) : 0.f;
        if (real && k < g.K) {
            eo[(size_t)rm * pad4(g.K) + k] = e;
            eot[((size_t)r * g.K + k) * pad4(g.M) + m] = e;
        }
        const float eh = prep_tf32_hi(e), el = prep_tf32_hi(e - eh);
        if (tf && m < mtiles * ntf && k < kchunks * 16) {
            float* tile = tf + (((size_t)r * mtiles + m / ntf) * kchunks + k / 16) * 2 * ntf * 16;
            const int q = prep_core_offset(m % ntf, k % 16);
            tile[q] = eh; tile[ntf * 16 + q] = el;
        }
        if (td && m < mchunks * 16 && k < ktiles * ntd) {
            float* tile = td + (((size_t)r * ktiles + k / ntd) * mchunks + m / 16) * 2 * ntd * 16;
            const int q = prep_core_offset(k % ntd, m % 16);
            tile[q] = eh; tile[ntd * 16 + q] = el;
        }
    }
}

// mx[n][pos] = max (eps > 0) or min (eps < 0) over the K taps of the patch at pos; NaN taps are ignored,
// as the reference's max pass ignores them (std::max(acc, NaN) keeps acc).
template <bool SPATIAL1>
__global__ void __launch_bounds__(256) mex_colmax(MexGeo g, const float* __restrict__ x, float* __restrict__ mx, const int* __restrict__ flag,
                                                  int interior) {
    if (*flag) return;
    const long long total = (long long)g.B * g.N;
    const bool up = g.eps > 0;
    const float oob = float(g.oob);
    const size_t hw = (size_t)g.H * g.W;
    for (long long idx = blockIdx.x * 256LL + threadIdx.x; idx < total; idx += (long long)gridDim.x * 256) {
        const int pos = int(idx % g.N), n = int(idx / g.N);
        const int w = pos % g.Wo, h = (pos / g.Wo) % g.Ho, c = pos / (g.Wo * g.Ho);
        const float* xs = x + (size_t)n * g.C * g.H * g.W;
        const int c0 = c * g.sc - g.pc, h0 = h * g.sh - g.ph, w0 = w * g.sw - g.pw;
        float v = up ? -CUDART_INF_F : CUDART_INF_F;
        if (SPATIAL1 && interior) {
            // 1x1 blocks inside the input: tap k is channel c0 + k of one pixel; eight independent loads at a time
            const float* p = xs + ((size_t)c0 * g.H + h0) * g.W + w0;
#pragma unroll 8
            for (int k = 0; k < g.K; ++k) {
                const float t = __ldg(p + k * hw);
                v = up ? fmaxf(v, t) : fminf(v, t);
            }
        } else {
            for (int k = 0; k < g.K; ++k) {
                const float t = patch_value<SPATIAL1>(g, xs, c0, h0, w0, k, oob);
                v = up ? fmaxf(v, t) : fminf(v, t);
            }
        }
        mx[idx] = v;
    }
}

// Short spatial blocks that tile the rows of the input (block width = stride along w, 2 or 4 wide, no padding, no patch
// leaving the input): the taps of one block row are one aligned vector, consecutive positions read consecutive vectors,
// and the bc * bh row loads of a position do not depend on one another, so they are issued together instead of tap by
// tap with a division each.  Same values: max and min are associative and skip NaN taps either way.
template <int BW>
__global__ void __launch_bounds__(256) mex_colmax_rows(MexGeo g, const float* __restrict__ x, float* __restrict__ mx, const int* __restrict__ flag) {
    if (*flag) return;
    const long long total = (long long)g.B * g.N;
    const bool up = g.eps > 0;
    const int rows = g.bc * g.bh;
    const size_t plane_step = (size_t)(g.H - g.bh + 1) * g.W;            // from the last row of a channel's block to the first of the next
    for (long long idx = blockIdx.x * 256LL + threadIdx.x; idx < total; idx += (long long)gridDim.x * 256) {
        const int pos = int(idx % g.N), n = int(idx / g.N);
        const int w = pos % g.Wo, h = (pos / g.Wo) % g.Ho, c = pos / (g.Wo * g.Ho);
        const float* rp = x + (size_t)n * g.C * g.H * g.W + ((size_t)(c * g.sc) * g.H + h * g.sh) * g.W + w * BW;
        float v = up ? -CUDART_INF_F : CUDART_INF_F;
        int kh = 0;
#pragma unroll 8
        for (int rr = 0; rr < rows; ++rr) {
            float t;
            if (BW == 2) {
                const float2 q = __ldg(reinterpret_cast<const float2*>(rp));
                t = up ? fmaxf(q.x, q.y) : fminf(q.x, q.y);
            } else {
                const float4 q = __ldg(reinterpret_cast<const float4*>(rp));
                t = up ? fmaxf(fmaxf(q.x, q.y), fmaxf(q.z, q.w)) : fminf(fminf(q.x, q.y), fminf(q.z, q.w));
            }
            v = up ? fmaxf(v, t) : fminf(v, t);
            if (++kh == g.bh) { kh = 0; rp += plane_step; } else rp += g.W;
        }
        mx[idx] = v;
    }
}

// The same maxima with eight threads per position (warp w of a CTA takes taps w, w + 8, ...): layers with few
// positions and long patches (8x8 maps under 256 channels) otherwise leave most of the GPU idle while each
// thread walks its patch alone.  max and min are associative and NaN taps are skipped either way: same values.
template <bool SPATIAL1>
__global__ void __launch_bounds__(256) mex_colmax_sliced(MexGeo g, const float* __restrict__ x, float* __restrict__ mx, const int* __restrict__ flag,
                                                         int interior) {
    __shared__ float part[8][32];
    if (*flag) return;
    const long long total = (long long)g.B * g.N;
    const bool up = g.eps > 0;
    const float oob = float(g.oob);
    const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
    for (long long first = blockIdx.x * 32LL; first < total; first += (long long)gridDim.x * 32) {
        const long long idx = first + lane;
        float v = up ? -CUDART_INF_F : CUDART_INF_F;
        if (idx < total) {
            const int pos = int(idx % g.N), n = int(idx / g.N);
            const int w = pos % g.Wo, h = (pos / g.Wo) % g.Ho, c = pos / (g.Wo * g.Ho);
            const float* xs = x + (size_t)n * g.C * g.H * g.W;
            const int c0 = c * g.sc - g.pc, h0 = h * g.sh - g.ph, w0 = w * g.sw - g.pw;
            if (SPATIAL1 && interior) {
                const size_t hw = (size_t)g.H * g.W;
                const float* p = xs + ((size_t)c0 * g.H + h0) * g.W + w0;
#pragma unroll 8
                for (int k = slice; k < g.K; k += 8) {
                    const float t = __ldg(p + k * hw);
                    v = up ? fmaxf(v, t) : fminf(v, t);
                }
            } else {
#pragma unroll 4
                for (int k = slice; k < g.K; k += 8) {
                    const float t = patch_value<SPATIAL1>(g, xs, c0, h0, w0, k, oob);
                    v = up ? fmaxf(v, t) : fminf(v, t);
                }
            }
        }
        part[slice][lane] = v;
        __syncthreads();
        if (slice == 0 && idx < total) {
#pragma unroll
            for (int q = 1; q < 8; ++q) v = up ? fmaxf(v, part[q][lane]) : fminf(v, part[q][lane]);
            mx[idx] = v;
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------- forward
// C[i = m, j = position] = sum_{q = k} EoT[k][m] * Ex[k][j]
// INTERIOR: no patch of this geometry leaves the input, so taps need no bounds test.
template <int TM, bool SPATIAL1, bool INTERIOR>
__global__ void __launch_bounds__(256) mex_fwd_tiled(MexGeo g, const float* __restrict__ x, const float* __restrict__ eot,
                                                     const float* __restrict__ mo, const float* __restrict__ mx,
                                                     float* __restrict__ y, const int* __restrict__ flag) {
    using Cfg = TileCfg<TM, 128, 8, TM / 16, 8, 1, 1>;
    static_assert(Cfg::THREADS == 256, "256 threads");
    if (*flag) return;
    __shared__ __align__(16) float smem[Cfg::SMEM_FLOATS];
    __shared__ long long col_base[Cfg::TN];
    __shared__ float col_mx[Cfg::TN];
    const long long P = (long long)g.B * g.rs;                 // positions of one region over the batch
    const int mtiles = (g.M + TM - 1) / TM;
    int bid = blockIdx.x;
    const int r = bid % g.R; bid /= g.R;
    const int mt = bid % mtiles;
    const long long jt = bid / mtiles;
    const int i0 = mt * TM;
    const long long j0 = jt * Cfg::TN;

    // staging role: this thread stages column s_lane, rows s_k, s_k + 2, ... of every chunk
    const int s_lane = threadIdx.x % 128, s_k = threadIdx.x / 128;
    const Column sc = column_of(g, r, j0 + s_lane, P, mx);
    if (s_k == 0) { col_base[s_lane] = sc.base; col_mx[s_lane] = sc.mx; }
    const float* xs = x + (size_t)sc.n * g.C * g.H * g.W;
    const bool live = sc.base >= 0;
    const float eps = float(g.eps), oob = float(g.oob);
    const float dead = eps > 0 ? -CUDART_INF_F : CUDART_INF_F;  // exp(eps * (dead - mx)) == 0
    const float* arow = eot + (size_t)r * g.K * pad4(g.M);
    const int ldm = pad4(g.M);
    const TileThread<Cfg> t;
    float rb[Cfg::B_PER];

    float2 acc[Cfg::RM][Cfg::RN / 2];
#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_)
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN / 2; ++c_) acc[r_][c_] = make_float2(0.f, 0.f);

    auto fetchA = [&](int chunk, float* As) { stage_copy_async<Cfg, TM>(As, arow, ldm, chunk * Cfg::KC, g.K, i0, g.M); };
    auto fetchB = [&](int chunk, float*) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) {
            const int k = chunk * Cfg::KC + s_k + s * 2;
            if (!live || k >= g.K) rb[s] = dead;
            else if (INTERIOR) rb[s] = __ldg(xs + interior_index<SPATIAL1>(g, sc.c0, sc.h0, sc.w0, k));
            else rb[s] = patch_value<SPATIAL1>(g, xs, sc.c0, sc.h0, sc.w0, k, oob);
        }
    };
    auto commitA = [&](float*) { cp_async_wait_all(); };
    auto commitB = [&](float* Bs) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) Bs[(s_k + s * 2) * Cfg::TN + s_lane] = live ? fast_exp(eps * (rb[s] - sc.mx)) : 0.f;
    };
    auto comb = [&](int r_, int cp, const float2 (&a)[1], const float2 (&b)[1]) { acc[r_][cp] = fma2(a[0], b[0], acc[r_][cp]); };
    tile_mainloop<Cfg, false, false>(smem, (g.K + Cfg::KC - 1) / Cfg::KC, t, fetchA, fetchB, commitA, commitB, comb);

    // y = mx + mo + (log S + c)/eps, with log S = log2 S * ln 2
    const float inv_eps = 1.f / eps, k_log = 0.69314718056f * inv_eps, k_cst = float(g.cst) * inv_eps;
    long long cb[Cfg::RN];
    float cm_[Cfg::RN];
#pragma unroll
    for (int c_ = 0; c_ < Cfg::RN; ++c_) { cb[c_] = col_base[t.col(c_)]; cm_[c_] = col_mx[t.col(c_)] + k_cst; }
#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_) {
        const int m = i0 + t.row(r_);
        if (m >= g.M) continue;
        const float mom = mo[r * g.M + m];
        float* yrow = y + (long long)m * g.N;
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN; ++c_) {
            if (cb[c_] < 0) continue;
            const float sacc = (c_ & 1) ? acc[r_][c_ >> 1].y : acc[r_][c_ >> 1].x;
            __stcs(yrow + cb[c_], fmaf(__log2f(sacc), k_log, cm_[c_] + mom));
        }
    }
}

// ------------------------------------------------------------ input gradient
// C[i = k, j = position] = sum_{q = m} Eo[m][k] * (dy*G)[m][j];  dx[tap k of position j] = Ex[k][j] * C
// (taps of different positions never coincide: the host only takes this kernel when blocks do not overlap).
template <int TM, bool SPATIAL1>
__global__ void __launch_bounds__(256) mex_dx_tiled(MexGeo g, const float* __restrict__ x, const float* __restrict__ eo,
                                                    const float* __restrict__ mo, const float* __restrict__ mx,
                                                    const float* __restrict__ y, const float* __restrict__ dy,
                                                    float* __restrict__ dx, const int* __restrict__ flag) {
    using Cfg = TileCfg<TM, 128, 8, TM / 16, 8, 1, 1>;
    if (*flag) return;
    __shared__ __align__(16) float smem[Cfg::SMEM_FLOATS];
    __shared__ Column cols[Cfg::TN];
    const long long P = (long long)g.B * g.rs;
    const int ktiles = (g.K + TM - 1) / TM;
    int bid = blockIdx.x;
    const int r = bid % g.R; bid /= g.R;
    const int kt = bid % ktiles;
    const long long jt = bid / ktiles;
    const int i0 = kt * TM;
    const long long j0 = jt * Cfg::TN;

    const int s_lane = threadIdx.x % 128, s_k = threadIdx.x / 128;
    const Column sc = column_of(g, r, j0 + s_lane, P, mx);
    if (s_k == 0) cols[s_lane] = sc;
    const bool live = sc.base >= 0;
    const TileThread<Cfg> t;
    const float eps = float(g.eps), cst = float(g.cst);
    const float* arow = eo + (size_t)r * g.M * pad4(g.K);
    const int ldk = pad4(g.K);
    const float* mor = mo + r * g.M;
    float rby[Cfg::B_PER], rbg[Cfg::B_PER], rbm[Cfg::B_PER];

    float2 acc[Cfg::RM][Cfg::RN / 2];
#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_)
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN / 2; ++c_) acc[r_][c_] = make_float2(0.f, 0.f);

    auto fetchA = [&](int chunk, float* As) { stage_copy_async<Cfg, TM>(As, arow, ldk, chunk * Cfg::KC, g.M, i0, g.K); };
    auto fetchB = [&](int chunk, float*) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) {
            const int m = chunk * Cfg::KC + s_k + s * 2;
            const bool ok = m < g.M && live;
            rby[s] = ok ? __ldcs(y + sc.base + (long long)m * g.N) : 0.f;
            rbg[s] = ok ? __ldcs(dy + sc.gbase + (long long)m * g.Ng) : 0.f;
            rbm[s] = ok ? __ldg(mor + m) : 0.f;
        }
    };
    auto commitA = [&](float*) { cp_async_wait_all(); };
    auto commitB = [&](float* Bs) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s)       // rows past M and dead columns carry dy = 0
            Bs[(s_k + s * 2) * Cfg::TN + s_lane] = rbg[s] * fast_exp(eps * (sc.mx + rbm[s] - rby[s]) + cst);
    };
    auto comb = [&](int r_, int cp, const float2 (&a)[1], const float2 (&b)[1]) { acc[r_][cp] = fma2(a[0], b[0], acc[r_][cp]); };
    tile_mainloop<Cfg, false, false>(smem, (g.M + Cfg::KC - 1) / Cfg::KC, t, fetchA, fetchB, commitA, commitB, comb);

#pragma unroll
    for (int c_ = 0; c_ < Cfg::RN; ++c_) {
        const Column col = cols[t.col(c_)];
        if (col.base < 0) continue;
        const size_t sample = (size_t)col.n * g.C * g.H * g.W;
#pragma unroll
        for (int r_ = 0; r_ < Cfg::RM; ++r_) {
            const int k = i0 + t.row(r_);
            if (k >= g.K) continue;
            const Tap tp = tap_of<SPATIAL1>(g, k);
            const int cc = col.c0 + tp.c, hh = col.h0 + tp.h, ww = col.w0 + tp.w;
            if (cc < 0 || cc >= g.C || hh < 0 || hh >= g.H || ww < 0 || ww >= g.W) continue;
            const size_t a = sample + ((size_t)cc * g.H + hh) * g.W + ww;
            const float sacc = (c_ & 1) ? acc[r_][c_ >> 1].y : acc[r_][c_ >> 1].x;
            dx[a] = fast_exp(eps * (__ldg(x + a) - col.mx)) * sacc;
        }
    }
}

// ---------------------------------------------------------- offsets gradient
// C[i = m, j = k] = sum_{q = positions of region r in this split} (dy*G)[m][q] * Ex[k][q]; both operands
// are contiguous along q in memory, so they are stored transposed (swizzled stages).
template <int TILE, int KC, bool SPATIAL1>
__global__ void __launch_bounds__(256) mex_doff_tiled(MexGeo g, const float* __restrict__ x, const float* __restrict__ mo,
                                                      const float* __restrict__ mx, const float* __restrict__ y,
                                                      const float* __restrict__ dy, float* __restrict__ part, int splits,
                                                      const int* __restrict__ flag) {
    using Cfg = TileCfg<TILE, TILE, KC, TILE / 16, TILE / 16, 1, 1>;
    static_assert(Cfg::THREADS == 256, "256 threads");
    constexpr int ROWS = 256 / KC;                                  // tile rows one staging pass covers
    if (*flag) return;
    __shared__ __align__(16) float smem[Cfg::SMEM_FLOATS];
    const long long P = (long long)g.B * g.rs;
    const int mtiles = (g.M + TILE - 1) / TILE, ktiles = (g.K + TILE - 1) / TILE;
    int bid = blockIdx.x;
    const int kt = bid % ktiles; bid /= ktiles;
    const int mt = bid % mtiles; bid /= mtiles;
    const int r = bid % g.R;
    const int split = bid / g.R;
    const int i0 = mt * TILE, jk0 = kt * TILE;
    const long long chunks = (P + KC - 1) / KC;
    const long long c_begin = chunks * split / splits, c_end = chunks * (split + 1) / splits;

    const TileThread<Cfg> t;
    const float eps = float(g.eps), cst = float(g.cst), oob = float(g.oob);
    const int qq = threadIdx.x % KC, e0 = threadIdx.x / KC;         // this thread stages q = qq, rows e0 + ROWS*s
    const float* mor = mo + r * g.M;
    float mom[Cfg::A_PER];
#pragma unroll
    for (int s = 0; s < Cfg::A_PER; ++s) mom[s] = (i0 + e0 + ROWS * s < g.M) ? mor[i0 + e0 + ROWS * s] : 0.f;
    Column cur;                                                     // the position this thread stages in the fetched chunk
    float ray[Cfg::A_PER], rag[Cfg::A_PER], rbx[Cfg::B_PER];

    float2 acc[Cfg::RM][Cfg::RN / 2];
#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_)
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN / 2; ++c_) acc[r_][c_] = make_float2(0.f, 0.f);

    auto fetchA = [&](int chunk, float*) {
        cur = column_of(g, r, (c_begin + chunk) * KC + qq, P, mx);
#pragma unroll
        for (int s = 0; s < Cfg::A_PER; ++s) {
            const int m = i0 + e0 + ROWS * s;
            const bool ok = cur.base >= 0 && m < g.M;
            ray[s] = ok ? __ldcs(y + cur.base + (long long)m * g.N) : 0.f;
            rag[s] = ok ? __ldcs(dy + cur.gbase + (long long)m * g.Ng) : 0.f;
        }
    };
    auto fetchB = [&](int, float*) {
        const float* xs = x + (size_t)cur.n * g.C * g.H * g.W;
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) {
            const int k = jk0 + e0 + ROWS * s;
            rbx[s] = (cur.base >= 0 && k < g.K) ? patch_value<SPATIAL1>(g, xs, cur.c0, cur.h0, cur.w0, k, oob) : 0.f;
        }
    };
    auto commitA = [&](float* As) {
#pragma unroll
        for (int s = 0; s < Cfg::A_PER; ++s)
            As[stage_offset<TILE, true>(qq, e0 + ROWS * s)] = rag[s] * fast_exp(eps * (cur.mx + mom[s] - ray[s]) + cst);
    };
    auto commitB = [&](float* Bs) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) {
            const int e = e0 + ROWS * s;
            Bs[stage_offset<TILE, true>(qq, e)] = (cur.base >= 0 && jk0 + e < g.K) ? fast_exp(eps * (rbx[s] - cur.mx)) : 0.f;
        }
    };
    auto comb = [&](int r_, int cp, const float2 (&a)[1], const float2 (&b)[1]) { acc[r_][cp] = fma2(a[0], b[0], acc[r_][cp]); };
    tile_mainloop<Cfg, true, true>(smem, int(c_end - c_begin), t, fetchA, fetchB, commitA, commitB, comb);

    float* dst = part + ((size_t)split * g.R + r) * g.M * g.K;
#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_) {
        const int m = i0 + t.row(r_);
        if (m >= g.M) continue;
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN; ++c_) {
            const int k = jk0 + t.col(c_);
            if (k < g.K) dst[(size_t)m * g.K + k] = (c_ & 1) ? acc[r_][c_ >> 1].y : acc[r_][c_ >> 1].x;
        }
    }
}

// doff[r][m][k] (+)= Eo[r][m][k] * sum over splits, in split order (deterministic)
__global__ void __launch_bounds__(256) mex_doff_reduce(long long n, int K, int splits, const float* __restrict__ part, const float* __restrict__ eo,
                                                       float* __restrict__ doff, int accumulate, const int* __restrict__ flag) {
    if (flag[0] | flag[1]) return;               // unsafe spread, or a tensor-core launch gave up on a wait: the exact kernel behind does the work
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
        float s = 0.f;
        for (int p = 0; p < splits; ++p) s += part[(size_t)p * n + i];
        s *= eo[(i / K) * pad4(K) + i % K];
        doff[i] = accumulate ? doff[i] + s : s;
    }
}

// The same reduction for offsets given raw (SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS).  s[k] is the gradient with respect to the
// normalised row (the split sums times Eo, or, when a status word is set, what the exact kernel left in the first R M K
// floats of `part`); the gradient with respect to the raw row is s[k] - softmax(raw)[k] * sum_k s[k], with
// softmax(raw)[k] = exp(raw[k] - lse).  Rows of up to 1024 taps: one CTA per (region, instance) row, every thread keeps its
// EPT values of s in registers between the row sum and the final pass (the partial sums are read once).
template <int EPT>
__global__ void __launch_bounds__(128) mex_doff_reduce_norm(int K, int splits, long long n, const float* __restrict__ part, const float* __restrict__ eo,
                                                            const float* __restrict__ raw, const float* __restrict__ lse,
                                                            float* __restrict__ doff, int accumulate, const int* __restrict__ flag) {
    __shared__ float red[128];
    const bool exact = (flag[0] | flag[1]) != 0;
    const long long row = blockIdx.x;
    float sk[EPT];
    float gs = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
        const int k = threadIdx.x + 128 * e;
        sk[e] = 0.f;
        if (k < K) {
            const long long i = row * K + k;
            if (exact) sk[e] = part[i];
            else {
                float a = 0.f;
                for (int p = 0; p < splits; ++p) a += part[(size_t)p * n + i];
                sk[e] = a * eo[row * pad4(K) + k];
            }
        }
        gs += sk[e];
    }
    red[threadIdx.x] = gs;
    __syncthreads();
    for (int s = 64; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    gs = red[0];
    const float l = lse[row];
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
        const int k = threadIdx.x + 128 * e;
        if (k < K) {
            const long long i = row * K + k;
            const float v = sk[e] - expf(raw[i] - l) * gs;
            doff[i] = accumulate ? doff[i] + v : v;
        }
    }
}

// Longer rows (the classifier head: 10 rows of 8192 taps): the element-parallel reduction into a scratch row set, then the
// row pass.  `tmp` = gradient with respect to the normalised rows.
__global__ void __launch_bounds__(256) mex_doff_reduce_tmp(long long n, int K, int splits, const float* __restrict__ part, const float* __restrict__ eo,
                                                           float* __restrict__ tmp, const int* __restrict__ flag) {
    const bool exact = (flag[0] | flag[1]) != 0;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
        if (exact) { tmp[i] = part[i]; continue; }
        float s = 0.f;
        for (int p = 0; p < splits; ++p) s += part[(size_t)p * n + i];
        tmp[i] = s * eo[(i / K) * pad4(K) + i % K];
    }
}

__global__ void __launch_bounds__(256) mex_doff_norm_rows(int K, const float* __restrict__ tmp, const float* __restrict__ raw, const float* __restrict__ lse,
                                                          float* __restrict__ doff, int accumulate) {
    __shared__ float red[256];
    const long long row = blockIdx.x;
    const float* t = tmp + row * K;
    float gs = 0.f;
    for (int k = threadIdx.x; k < K; k += 256) gs += t[k];
    red[threadIdx.x] = gs;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    gs = red[0];
    const float l = lse[row];
    for (int k = threadIdx.x; k < K; k += 256) {
        const long long i = row * K + k;
        const float v = t[k] - expf(raw[i] - l) * gs;
        doff[i] = accumulate ? doff[i] + v : v;
    }
}

inline bool mex_norm(uint32_t flags) { return (flags & SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS) != 0; }

// The tail of every offsets-gradient path: the split partial sums become doff, and the exact kernel behind acts only when a
// status word is set.  With raw offsets the exact kernel goes first, into `part`, and one launch reduces and normalises.
cudaError_t finish_doff(const MexGeo& g, const MexWs& w, int splits, const float* x, const float* off, const float* y, const float* dy,
                        float* doff, bool accumulate, uint32_t flags, cudaStream_t s) {
    const long long n = (long long)g.R * g.M * g.K;
    if (mex_norm(flags)) {
        cudaError_t e = launch_mex_doff_direct(g, false, x, w.offn, y, dy, w.part, false, s, w.flag);
        if (e != cudaSuccess) return e;
        const int rows = g.R * g.M;
        if (g.K <= 128) mex_doff_reduce_norm<1><<<rows, 128, 0, s>>>(g.K, splits, n, w.part, w.eo, off, w.lse, doff, accumulate, w.flag);
        else if (g.K <= 256) mex_doff_reduce_norm<2><<<rows, 128, 0, s>>>(g.K, splits, n, w.part, w.eo, off, w.lse, doff, accumulate, w.flag);
        else if (g.K <= 512) mex_doff_reduce_norm<4><<<rows, 128, 0, s>>>(g.K, splits, n, w.part, w.eo, off, w.lse, doff, accumulate, w.flag);
        else if (g.K <= 1024) mex_doff_reduce_norm<8><<<rows, 128, 0, s>>>(g.K, splits, n, w.part, w.eo, off, w.lse, doff, accumulate, w.flag);
        else {
            mex_doff_reduce_tmp<<<int(std::min<long long>((n + 255) / 256, (long long)device_sm_count() * 8)), 256, 0, s>>>(n, g.K, splits, w.part, w.eo, w.dtmp, w.flag);
            mex_doff_norm_rows<<<rows, 256, 0, s>>>(g.K, w.dtmp, off, w.lse, doff, accumulate);
            count_launch();
        }
        count_launch();
        return cudaGetLastError();
    }
    mex_doff_reduce<<<int(std::min<long long>((n + 255) / 256, (long long)device_sm_count() * 8)), 256, 0, s>>>(n, g.K, splits, w.part, w.eo, doff, accumulate, w.flag);
    count_launch();
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return launch_mex_doff_direct(g, false, x, off, y, dy, doff, accumulate, s, w.flag);
}

// Pair tiles: sibling regions alternate along the width and every tensor allows 8-byte accesses of pixel pairs.
bool use_pair_kernels(const MexGeo& g, uint32_t flags, const void* a, const void* b, const void* c, const void* d) {
    return !(flags & (SIMNETS_FLAG_MEX_NO_PAIR_TILES | SIMNETS_FLAG_MEX_TC_ONE_TILE)) && mex_pair_shape(g) && mex_pair_aligned(a, b, c, d);
}

// The prepass also writes the pair-tile kernels' operand tiles: decided by shape and flags alone (not by pointer
// alignment), so that a gradient call on a primed workspace knows what the forward call left there.
bool pair_prep(const MexGeo& g, uint32_t flags) {
    return use_tc_kernels(g, flags) && !(flags & (SIMNETS_FLAG_MEX_NO_PAIR_TILES | SIMNETS_FLAG_MEX_TC_ONE_TILE)) && mex_pair_shape(g);
}

bool blocks_disjoint(const MexGeo& g) { return g.sc >= g.bc && g.sh >= g.bh && g.sw >= g.bw; }

bool blocks_cover_input(const MexGeo& g) {
    auto full = [](int dim, int block, int stride, int pad) { return stride == block && pad == 0 && dim % block == 0; };
    return full(g.C, g.bc, g.sc, g.pc) && full(g.H, g.bh, g.sh, g.ph) && full(g.W, g.bw, g.sw, g.pw);
}

cudaError_t run_prepasses(const MexGeo& g, const MexWs& w, const float* x, const float* off, cudaStream_t s, bool need_mx = true,
                          bool pair_tiles = false, bool normalize = false) {
    cudaError_t e = cudaMemsetAsync(w.flag, 0, 16, s);
    if (e != cudaSuccess) return e;
    if (pair_tiles) {
        // the pair-tile kernels' operand tiles (forward and input gradient) come out of the same launch
        const int ntf = mex_pair_nt_fwd(g), ntd = mex_pair_nt_dx(g);
        const int Mp = std::max(((g.M + ntf - 1) / ntf) * ntf, ((g.M + 15) / 16) * 16);
        mex_prep_offsets<<<g.R * Mp, g.K >= 2048 ? 512 : 128, 0, s>>>(g, Mp, off, w.mo, w.eo, w.eot, w.flag, w.tc_tiles, ntf, w.tc_tiles_dx, ntd,
                                                                      normalize ? w.offn : nullptr, w.lse);
    } else {
        mex_prep_offsets<<<g.R * g.M, g.K >= 2048 ? 512 : 128, 0, s>>>(g, g.M, off, w.mo, w.eo, w.eot, w.flag, nullptr, 0, nullptr, 0,
                                                                       normalize ? w.offn : nullptr, w.lse);
    }
    if (!need_mx) { count_launch(); return cudaGetLastError(); }
    // long patches over few positions are contiguous per position: reduce them with one CTA each
    if (g.K >= 256 && g.N <= 16) { count_launch(); return launch_mex_colmax_wide(g, x, w.mx, w.flag, s); }
    const long long total = (long long)g.B * g.N;
    const int inside = patches_inside_input(g) ? 1 : 0;
    // (measured on 32x32x64, 16x16x128 and 8x8x256 maps at batches 256 and 2048: eight threads per position win for
    // long patches while one thread per position would not fill the GPU's thread slots: 2048 per multiprocessor)
    if (g.K >= 128 && total < (long long)device_sm_count() * 2048) {
        const int grid = int(std::min<long long>((total + 31) / 32, (long long)device_sm_count() * 32));
        if (g.bh == 1 && g.bw == 1) mex_colmax_sliced<true><<<grid, 256, 0, s>>>(g, x, w.mx, w.flag, inside);
        else mex_colmax_sliced<false><<<grid, 256, 0, s>>>(g, x, w.mx, w.flag, inside);
    } else if ((g.bw == 2 || g.bw == 4) && g.sw == g.bw && g.W % g.bw == 0 && inside &&
               (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        // every vector load is aligned: rows start at multiples of W floats, W and the sample stride are multiples of bw
        const int grid = int(std::min<long long>((total + 255) / 256, (long long)device_sm_count() * 16));
        if (g.bw == 2) mex_colmax_rows<2><<<grid, 256, 0, s>>>(g, x, w.mx, w.flag);
        else mex_colmax_rows<4><<<grid, 256, 0, s>>>(g, x, w.mx, w.flag);
    } else {
        const int grid = int(std::min<long long>((total + 255) / 256, (long long)device_sm_count() * 16));
        if (g.bh == 1 && g.bw == 1) mex_colmax<true><<<grid, 256, 0, s>>>(g, x, w.mx, w.flag, inside);
        else mex_colmax<false><<<grid, 256, 0, s>>>(g, x, w.mx, w.flag, inside);
    }
    count_launch(2);
    return cudaGetLastError();
}

// The forward pass of this layer leaves in the workspace everything run_prepasses() would write for the gradients
// (the short-patch and few-instance forward kernels skip the per-position maxima, which their gradients need).
bool forward_primes_workspace(MexGeo g, uint32_t flags) {
    if (!(flags & SIMNETS_FLAG_MEX_WORKSPACE_PRIMED)) return false;
    g.gp = 1; g.Ng = g.N;        // the forward pass never sees a pooled dy
    return (!smallm_shape(g) || mex_head_shape(g)) && !use_smallk_kernels(g, flags);
}

}  // namespace

// where the forward pass of this shape reads the per-position extrema from, or nullptr if it computes them on the fly
float* mex_workspace_maxima(const MexGeo& g, void* ws, uint32_t flags) {
    if (use_smallk_kernels(g, flags) || smallm_shape(g)) return nullptr;
    return carve(g, ws).mx;
}

bool mex_use_tiled(const MexGeo& g, bool f64, uint32_t flags) {
    if (f64 || !g.finite || g.B == 0) return false;
    if (flags & (SIMNETS_FLAG_FORCE_DIRECT | SIMNETS_FLAG_MEX_EXACT)) return false;
    return true;
}

size_t mex_workspace_bytes(const MexGeo& g, bool f64, uint32_t flags) {
    if (!mex_use_tiled(g, f64, flags)) return 256;
    return carve(g, nullptr).bytes;
}

static cudaError_t mex_fwd_tiled_body(const MexGeo& g, const float* x, const float* off, float* y, void* ws, uint32_t flags, cudaStream_t s,
                                      float* pooled, bool* pooled_done);

cudaError_t launch_mex_fwd_tiled(const MexGeo& g, const float* x, const float* off, float* y, void* ws, uint32_t flags, cudaStream_t s,
                                 float* pooled) {
    bool pooled_done = false;
    const cudaError_t e = mex_fwd_tiled_body(g, x, off, y, ws, flags, s, pooled, &pooled_done);
    if (e != cudaSuccess || pooled == nullptr || pooled_done) return e;
    return launch_sum_pool2((long long)g.B * g.M * g.Co, g.Ho, g.Wo, y, pooled, s);
}

static cudaError_t mex_fwd_tiled_body(const MexGeo& g, const float* x, const float* off, float* y, void* ws, uint32_t flags, cudaStream_t s,
                                      float* pooled, bool* pooled_done) {
    const MexWs w = carve(g, ws);
    if (use_smallk_kernels(g, flags)) {
        cudaError_t e = run_prepasses(g, w, x, off, s, false, false, mex_norm(flags));
        if (e != cudaSuccess) return e;
        e = launch_mex_fwd_smallk(g, x, w.eo, w.mo, y, w.flag, s);
        if (e != cudaSuccess) return e;
        return launch_mex_fwd_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, s, w.flag);
    }
    if (smallm_shape(g)) {
        cudaError_t e = run_prepasses(g, w, x, off, s, false, false, mex_norm(flags));
        if (e != cudaSuccess) return e;
        e = mex_head_shape(g) ? launch_mex_fwd_head(g, x, w.eo, w.eot, w.mo, w.mx, y, w.part, w.flag, s)        // (also leaves the maxima for the gradients)
                              : launch_mex_fwd_smallm(g, x, w.eot, w.mo, y, w.flag, s);
        if (e != cudaSuccess) return e;
        return launch_mex_fwd_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, s, w.flag);
    }
    // (the caller may have had the layer in front leave the per-position extrema in the workspace: SIMNETS_FLAG_MEX_MAXIMA_GIVEN)
    cudaError_t e = run_prepasses(g, w, x, off, s, !(flags & SIMNETS_FLAG_MEX_MAXIMA_GIVEN), pair_prep(g, flags), mex_norm(flags));
    if (e != cudaSuccess) return e;
    if (use_tc_kernels(g, flags)) {
        if (use_pair_kernels(g, flags, x, y, y, y)) {
            const bool fuse = pooled != nullptr && (reinterpret_cast<uintptr_t>(pooled) & 3u) == 0;
            e = launch_mex_fwd_pair(g, x, w.tc_tiles, w.mo, w.mx, y, fuse ? pooled : nullptr, w.flag,
                                    (flags & SIMNETS_FLAG_MEX_TEST_EXPIRE_WAIT) != 0, s);
            if (e != cudaSuccess) return e;
            e = launch_mex_fwd_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, s, w.flag);
            if (e != cudaSuccess || !fuse) return e;
            *pooled_done = true;
            // if the exact kernel had to recompute y (a status word is set), the pooling is redone from y as well
            return launch_sum_pool2((long long)g.B * g.M * g.Co, g.Ho, g.Wo, y, pooled, s, w.flag);
        }
        e = launch_mex_tc_prep(g, false, w.eo, w.tc_tiles, s);
        if (e != cudaSuccess) return e;
        e = (flags & SIMNETS_FLAG_MEX_TC_ONE_TILE) ? launch_mex_fwd_tc(g, x, w.tc_tiles, w.mo, w.mx, y, w.flag, patches_inside_input(g), s)
                                                   : launch_mex_fwd_ws(g, x, w.tc_tiles, w.mo, w.mx, y, w.flag, patches_inside_input(g), s);
        if (e != cudaSuccess) return e;
        return launch_mex_fwd_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, s, w.flag);
    }
    const long long P = (long long)g.B * g.rs;
    const bool sp1 = g.bh == 1 && g.bw == 1;
    const bool wide = g.M > 64;
    const long long jtiles = (P + 127) / 128;
    const long long blocks = jtiles * ((g.M + (wide ? 127 : 63)) / (wide ? 128 : 64)) * g.R;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const bool interior = patches_inside_input(g);
#define FWD(TM, SP, IN) mex_fwd_tiled<TM, SP, IN><<<int(blocks), 256, 0, s>>>(g, x, w.eot, w.mo, w.mx, y, w.flag)
#define FWD_TM(TM)                                                                         \
    if (sp1) { if (interior) FWD(TM, true, true); else FWD(TM, true, false); }            \
    else { if (interior) FWD(TM, false, true); else FWD(TM, false, false); }
    if (wide) { FWD_TM(128) } else { FWD_TM(64) }
#undef FWD_TM
#undef FWD
    count_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return launch_mex_fwd_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, s, w.flag);       // runs only if the flag was raised
}

// --------------------------------------------- forward on library-owned scratch
// Scratch for simnets_mex_forward_static_scratch(): a fixed device array that every GPU loading this
// library carries until the process exits.  In host code the name below is only a handle for the
// runtime, not a device address; the address a kernel may use comes from cudaGetSymbolAddress, taken
// once per device with that device current.
static __device__ __align__(256) unsigned char g_mex_static_scratch[SIMNETS_MEX_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};
}  // namespace

int launch_mex_fwd_static(const MexGeo& g, const float* x, const float* off, float* y, uint32_t flags, cudaStream_t s) {
    if (carve(g, nullptr).fwd_bytes > size_t(SIMNETS_MEX_STATIC_SCRATCH_BYTES)) return SIMNETS_E_TOO_LARGE;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return int(e);
    if (dev < 0 || dev >= kMaxDevices) return SIMNETS_E_UNSUPPORTED;
    void* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        if (!g_static_ptr[dev]) {
            e = cudaGetSymbolAddress(&ptr, g_mex_static_scratch);      // address on the CURRENT device
            if (e != cudaSuccess) return int(e);
            g_static_ptr[dev] = ptr;
        }
        ptr = g_static_ptr[dev];
    }
    // launch_mex_fwd_tiled clears the one word that must start at zero (the safety flag) on every call;
    // everything else in the scratch is fully rewritten by the prepasses before it is read.
    // The caller's flags stay in force; the tensor-core route is switched off on top of them, because the capacity
    // check above counts the CUDA-core route's scratch only (no operand tiles).
    e = launch_mex_fwd_tiled(g, x, off, y, ptr, (flags | SIMNETS_FLAG_MEX_NO_TENSORCORE) & ~uint32_t(SIMNETS_FLAG_MEX_MAXIMA_GIVEN), s);
    return e == cudaSuccess ? SIMNETS_OK : int(e);
}

cudaError_t launch_mex_dx_tiled(const MexGeo& g, const float* x, const float* off, const float* y, const float* dy, float* dx,
                                void* ws, uint32_t flags, cudaStream_t s, bool prepped) {
    const MexWs w = carve(g, ws);
    if (!blocks_disjoint(g)) {           // overlapping blocks: the exact kernel (on the normalised rows, if the offsets came raw)
        if (mex_norm(flags) && !(prepped || forward_primes_workspace(g, flags))) {
            const cudaError_t e0 = run_prepasses(g, w, x, off, s, false, false, true);
            if (e0 != cudaSuccess) return e0;
        }
        return launch_mex_dx_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, dy, dx, s, nullptr);
    }
    const bool small = smallm_shape(g) || use_smallk_kernels(g, flags);
    cudaError_t e = (prepped || forward_primes_workspace(g, flags)) ? cudaSuccess : run_prepasses(g, w, x, off, s, !small, pair_prep(g, flags), mex_norm(flags));
    if (e != cudaSuccess) return e;
    if (!blocks_cover_input(g)) {
        e = cudaMemsetAsync(dx, 0, sizeof(float) * (size_t)g.B * g.C * g.H * g.W, s);
        if (e != cudaSuccess) return e;
    }
    if (use_smallk_kernels(g, flags)) {
        e = launch_mex_dx_smallk(g, x, w.eo, w.mo, y, dy, dx, w.flag, s);
        if (e != cudaSuccess) return e;
        return launch_mex_dx_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, dy, dx, s, w.flag);
    }
    if (use_tc_kernels(g, flags) && use_pair_kernels(g, flags, x, y, dy, dx)) {
        e = launch_mex_dx_pair(g, x, w.tc_tiles_dx, w.mo, w.mx, y, dy, dx, w.flag, s);
        if (e != cudaSuccess) return e;
        return launch_mex_dx_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, dy, dx, s, w.flag);
    }
    if (use_tc_kernels(g, flags)) {
        e = launch_mex_tc_prep(g, true, w.eot, w.tc_tiles, s);
        if (e != cudaSuccess) return e;
        // long patches (wide tap tiles, heavy epilogue): the persistent kernel; otherwise several one-tile CTAs per SM,
        // all of whose warps evaluate the exponentials, are faster (measured on the three MEX layers of the 3x32x32 net)
        e = ((flags & SIMNETS_FLAG_MEX_TC_ONE_TILE) || g.K <= 128) ? launch_mex_dx_tc(g, x, w.tc_tiles, w.mo, w.mx, y, dy, dx, w.flag, s)
                                                                   : launch_mex_dx_ws(g, x, w.tc_tiles, w.mo, w.mx, y, dy, dx, w.flag, s);
        if (e != cudaSuccess) return e;
        return launch_mex_dx_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, dy, dx, s, w.flag);
    }
    if (small && smallm_shape(g) && mex_head_shape(g)) {
        if (!(prepped || forward_primes_workspace(g, flags))) {              // run_prepasses skipped the maxima for this family
            e = launch_mex_colmax_wide(g, x, w.mx, w.flag, s);
            if (e != cudaSuccess) return e;
        }
        e = launch_mex_bwd_head(g, true, false, x, w.eo, w.mo, w.mx, y, dy, dx, nullptr, 1, w.flag, s);
        if (e != cudaSuccess) return e;
        return launch_mex_dx_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, dy, dx, s, w.flag);
    }
    if (small) {
        e = launch_mex_dx_smallm(g, x, w.eo, w.mo, y, dy, dx, w.flag, s);
        if (e != cudaSuccess) return e;
        return launch_mex_dx_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, dy, dx, s, w.flag);
    }
    const long long P = (long long)g.B * g.rs;
    const bool sp1 = g.bh == 1 && g.bw == 1;
    const bool wide = g.K > 64;
    const long long blocks = ((P + 127) / 128) * ((g.K + (wide ? 127 : 63)) / (wide ? 128 : 64)) * g.R;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
#define DX(TM, SP) mex_dx_tiled<TM, SP><<<int(blocks), 256, 0, s>>>(g, x, w.eo, w.mo, w.mx, y, dy, dx, w.flag)
    if (wide) { if (sp1) DX(128, true); else DX(128, false); }
    else { if (sp1) DX(64, true); else DX(64, false); }
#undef DX
    count_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return launch_mex_dx_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, dy, dx, s, w.flag);
}

cudaError_t launch_mex_doff_tiled(const MexGeo& g, const float* x, const float* off, const float* y, const float* dy, float* doff,
                                  bool accumulate, void* ws, uint32_t flags, cudaStream_t s, bool prepped) {
    const MexWs w = carve(g, ws);
    cudaError_t e = (prepped || forward_primes_workspace(g, flags)) ? cudaSuccess : run_prepasses(g, w, x, off, s, !use_smallk_kernels(g, flags), pair_prep(g, flags), mex_norm(flags));
    if (e != cudaSuccess) return e;
    if (use_tc_kernels(g, flags)) {
        int tsplits = mex_tc_doff_splits(g);
        e = use_pair_kernels(g, flags, x, y, dy, dy) ? launch_mex_doff_pair(g, x, w.mo, w.mx, y, dy, w.part, &tsplits, w.flag, s)
                                                     : launch_mex_doff_tc(g, x, w.mo, w.mx, y, dy, w.part, tsplits, w.flag, s);
        if (e != cudaSuccess) return e;
        return finish_doff(g, w, tsplits, x, off, y, dy, doff, accumulate, flags, s);
    }
    const int splits = doff_splits(g);
    if (use_smallk_kernels(g, flags)) {
        e = launch_mex_doff_smallk(g, x, w.mo, y, dy, w.part, splits, w.flag, s);
        if (e != cudaSuccess) return e;
        return finish_doff(g, w, splits, x, off, y, dy, doff, accumulate, flags, s);
    }
    if (smallm_shape(g) && mex_head_shape(g)) {
        const int hs = mex_head_splits(g);
        e = launch_mex_bwd_head(g, false, true, x, w.eo, w.mo, w.mx, y, dy, nullptr, w.part, hs, w.flag, s);
        if (e != cudaSuccess) return e;
        return finish_doff(g, w, hs, x, off, y, dy, doff, accumulate, flags, s);
    }
    if (smallm_shape(g)) {
        e = launch_mex_doff_smallm(g, x, w.mo, w.mx, y, dy, w.part, splits, w.flag, s);
        if (e != cudaSuccess) return e;
        return finish_doff(g, w, splits, x, off, y, dy, doff, accumulate, flags, s);
    }
    const int tile = doff_big(g) ? 128 : 64;
    const long long blocks = (long long)((g.M + tile - 1) / tile) * ((g.K + tile - 1) / tile) * g.R * splits;
    const bool sp1 = g.bh == 1 && g.bw == 1;
#define DOFF(T, KC, SP) mex_doff_tiled<T, KC, SP><<<int(blocks), 256, 0, s>>>(g, x, w.mo, w.mx, y, dy, w.part, splits, w.flag)
    if (doff_big(g)) { if (sp1) DOFF(128, 16, true); else DOFF(128, 16, false); }
    else { if (sp1) DOFF(64, 32, true); else DOFF(64, 32, false); }
#undef DOFF
    count_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return finish_doff(g, w, splits, x, off, y, dy, doff, accumulate, flags, s);
}

// Both gradients of one layer in one call: the offsets prepass and the per-position maxima are computed once.
cudaError_t launch_mex_backward_tiled(const MexGeo& g, const float* x, const float* off, const float* y, const float* dy, float* dx,
                                      float* doff, bool accumulate, void* ws, uint32_t flags, cudaStream_t s) {
    const MexWs w = carve(g, ws);
    cudaError_t e = forward_primes_workspace(g, flags) ? cudaSuccess : run_prepasses(g, w, x, off, s, !use_smallk_kernels(g, flags), pair_prep(g, flags), mex_norm(flags));
    if (e != cudaSuccess) return e;
    if (smallm_shape(g) && mex_head_shape(g) && blocks_disjoint(g)) {
        // the head: input gradient and the partial sums of the offsets gradient from one read of x
        const int hs = mex_head_splits(g);
        if (!blocks_cover_input(g)) {
            e = cudaMemsetAsync(dx, 0, sizeof(float) * (size_t)g.B * g.C * g.H * g.W, s);
            if (e != cudaSuccess) return e;
        }
        e = launch_mex_bwd_head(g, true, true, x, w.eo, w.mo, w.mx, y, dy, dx, w.part, hs, w.flag, s);
        if (e != cudaSuccess) return e;
        e = launch_mex_dx_direct(g, false, x, mex_norm(flags) ? w.offn : off, y, dy, dx, s, w.flag);
        if (e != cudaSuccess) return e;
        return finish_doff(g, w, hs, x, off, y, dy, doff, accumulate, flags, s);
    }
    e = launch_mex_dx_tiled(g, x, off, y, dy, dx, ws, flags, s, true);
    if (e != cudaSuccess) return e;
    return launch_mex_doff_tiled(g, x, off, y, dy, doff, accumulate, ws, flags, s, true);
}

}  // namespace simnets
