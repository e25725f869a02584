// Similarity forward and parameter gradients as implicit-im2col generalized GEMMs (float32).
//
//   forward   y[n, m, pos]   = sum_k f(t[m,k], w[m,k], patch[k, (n,pos)])              i = m, j = position, q = tap
//   params    (dT, dW)[m, k] = sum_{n,pos} g(dy[n,m,pos], patch[k,(n,pos)], t, w)      i = m, j = tap,      q = position
//
// with the reference's element functors (HUJI-Deep/simnets-tf include/utils/similarity_utils.hpp:17-119).
// The patch matrix of the reference (src/utils/im2col.cpp:247-280) is never built: a tap table gives, for
// each k = (c, kh, kw), its offset inside a sample and its (kh, kw); a position gives its patch corner.
// NaN handling costs no branch in the inner loop: while an input value is staged into shared memory a NaN
// becomes (value 0, mask 0) and the mask multiplies the term (ignore_nan_input modes); in the other modes
// the NaN itself is staged and propagates through the arithmetic exactly as in the reference.
// Per-(m,k) constants (0.5*log(w + fudge) - 0.5*log(2*pi), -w, -0.5*w) are computed once by a prepass,
// which also lays the parameters out tap-major so that the forward kernel's loads are contiguous.
#include "kernels.cuh"
#include "tile.cuh"

namespace simnets {

namespace {

constexpr double kLog2Pi = 1.8378770664093454835606594728112;
constexpr int kDpTile = 64, kDpKC = 32;

struct SimWs {
    int* flag;       // [2]: word 1 = a bounded wait of the tensor-core forward kernel ran out (its output is redone)
    float* planes;   // [3][K][Mp]: t, scale (-w or -0.5w), per-term constant; Mp = M rounded up to 4 floats
    float* cm;       // [M] per-instance constant added once per output
    int2* taps;      // [K]: {offset of tap inside a sample, (kh << 16) | kw}
    float* part;     // [S][3][M][K] split partial sums of the parameter gradients
    float* dxp;      // [2][bh*bw*M][Cp]: t and s*w (s = 2 for plain L2, else 1), channel-contiguous, for the input gradient
    float* tc_tiles; // pre-split parameter tiles of the tensor-core forward kernel
    float* tc_bias;  // [M] its per-instance constant
    size_t bytes;
};

__host__ inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }
__host__ __device__ inline int pad4(int v) { return (v + 3) & ~3; }

// taps per parameter-gradient tile: 32 when the patch is that short (cfg5: K = 27), else 64
__host__ inline int dp_tn(const SimGeo& g) { return g.K <= 32 ? 32 : 64; }

__host__ int dp_splits(const SimGeo& g) {
    const long long P = (long long)g.B * g.N;
    const long long chunks = (P + kDpKC - 1) / kDpKC;
    const long long tiles = (long long)((g.M + kDpTile - 1) / kDpTile) * ((g.K + dp_tn(g) - 1) / dp_tn(g));
    // the narrow tile runs four CTAs of 128 threads per SM (128 registers per thread): two waves of those
    const int ctas = device_sm_count() * (dp_tn(g) == 32 ? 8 : 4);                  // (the wide tile: two CTAs of 256 threads per SM)
    long long s = (ctas + tiles - 1) / tiles;
    // every split costs one set of partial sums (3 M K floats written and read again): at small batches a split keeps
    // at least 1024 positions, or the partial sums outweigh the operands
    const long long by_work = std::max<long long>(1, P / 1024);
    if (s > by_work) s = by_work;
    if (s > chunks) s = chunks;
    if (s < 1) s = 1;
    if (s > 2048) s = 2048;
    return int(s);
}

__host__ SimWs carve(const SimGeo& g, void* base) {
    SimWs w;
    char* p = static_cast<char*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { char* r = p ? p + off : nullptr; off += align256(bytes); return r; };
    w.flag = reinterpret_cast<int*>(take(sizeof(int) * 2));
    w.planes = reinterpret_cast<float*>(take(sizeof(float) * 3 * (size_t)g.K * pad4(g.M)));
    w.cm = reinterpret_cast<float*>(take(sizeof(float) * g.M));
    w.taps = reinterpret_cast<int2*>(take(sizeof(int2) * g.K));
    w.part = reinterpret_cast<float*>(take(sizeof(float) * 3 * (size_t)dp_splits(g) * g.M * g.K));
    w.dxp = reinterpret_cast<float*>(take(sizeof(float) * 2 * (size_t)g.bh * g.bw * g.M * pad4(g.C)));
    w.tc_tiles = reinterpret_cast<float*>(take(sizeof(float) * sim_tc_tile_floats(g)));
    w.tc_bias = reinterpret_cast<float*>(take(sizeof(float) * g.M));
    w.bytes = off;
    return w;
}

// One block per instance m: tap-major parameter planes, the per-instance constant, and (block 0) the tap table.
__global__ void __launch_bounds__(128) sim_prep(SimGeo g, const float* __restrict__ tm, const float* __restrict__ wt,
                                                float* __restrict__ planes, float* __restrict__ cm, int2* __restrict__ taps,
                                                float* __restrict__ dxp, int* __restrict__ flag) {
    __shared__ float red[128];
    const int m = blockIdx.x;
    if (m == 0 && threadIdx.x < 2) flag[threadIdx.x] = 0;
    const float fudge = float(g.fudge);
    const int ldm = pad4(g.M);
    const size_t plane = (size_t)g.K * ldm;
    float csum = 0.f;
    for (int k = threadIdx.x; k < g.K; k += 128) {
        const float t = tm[(size_t)m * g.K + k], w = g.absw ? fabsf(wt[(size_t)m * g.K + k]) : wt[(size_t)m * g.K + k];
        float scale = -w, c = 0.f;
        if (g.mode == SIM_L2N) { scale = -0.5f * w; csum += 0.5f * logf(w + fudge); }
        if (g.mode == SIM_L2N_NAN) { scale = -0.5f * w; c = float(0.5 * (double(logf(w + fudge)) - kLog2Pi)); }
        planes[(size_t)k * ldm + m] = t;
        planes[plane + (size_t)k * ldm + m] = scale;
        planes[2 * plane + (size_t)k * ldm + m] = c;
        const int kw = k % g.bw, kh = (k / g.bw) % g.bh, c_ = k / (g.bw * g.bh);
        if (m == 0) taps[k] = make_int2((c_ * g.H + kh) * g.W + kw, (kh << 16) | kw);
        const size_t q = (size_t)(kh * g.bw + kw) * g.M + m, dplane = (size_t)g.bh * g.bw * g.M * pad4(g.C);
        dxp[q * pad4(g.C) + c_] = t;
        dxp[dplane + q * pad4(g.C) + c_] = (g.mode == SIM_L2 ? 2.f : 1.f) * w;
    }
    red[threadIdx.x] = csum;
    __syncthreads();
    for (int s = 64; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) cm[m] = g.mode == SIM_L2N ? red[0] + float(-0.5 * double(g.K) * kLog2Pi) : 0.f;
}

struct SimColumn {
    long long base;     // n*M*N + pos, or -1 past the end
    int n, h0, w0;      // sample, patch corner
};

__device__ __forceinline__ SimColumn sim_column(const SimGeo& g, long long j, long long P) {
    SimColumn c;
    c.base = -1; c.n = 0; c.h0 = c.w0 = 0;
    if (j >= P) return c;
    const int n = int(j / g.N), pos = int(j % g.N);
    c.n = n;
    c.h0 = (pos / g.ow) * g.sh - g.ph;
    c.w0 = (pos % g.ow) * g.sw - g.pw;
    c.base = (long long)n * g.M * g.N + pos;
    return c;
}

__device__ __forceinline__ float sim_tap_value(const SimGeo& g, const float* __restrict__ xs, const SimColumn& col, int2 tap, float oob) {
    const int hh = col.h0 + (tap.y >> 16), ww = col.w0 + (tap.y & 0xffff);
    if (hh >= 0 && hh < g.H && ww >= 0 && ww < g.W) return __ldg(xs + tap.x + col.h0 * g.W + col.w0);
    return oob;
}

// ------------------------------------------------------------------- forward
// MODE is a SimMode; NA = parameter planes used, NB = input planes (value [, mask]).
template <int MODE> struct FwdPlanes {
    static constexpr int NA = MODE == SIM_L2N_NAN ? 3 : 2;
    static constexpr int NB = (MODE == SIM_L2N_NAN || MODE == SIM_L1_SKIP) ? 2 : 1;
};

__device__ __forceinline__ float2 abs2(float2 v) { return make_float2(fabsf(v.x), fabsf(v.y)); }

template <int TM, int MODE>
__global__ void __launch_bounds__(256, TM == 128 ? 2 : 1) sim_fwd_tiled(SimGeo g, const float* __restrict__ x, const float* __restrict__ planes,
                                                     const float* __restrict__ cm, const int2* __restrict__ taps, float* __restrict__ y) {
    constexpr int NA = FwdPlanes<MODE>::NA, NB = FwdPlanes<MODE>::NB;
    using Cfg = TileCfg<TM, 128, 8, TM / 16, 8, NA, NB>;
    static_assert(Cfg::THREADS == 256, "256 threads");
    __shared__ __align__(16) float smem[Cfg::SMEM_FLOATS];
    __shared__ long long col_base[Cfg::TN];
    const long long P = (long long)g.B * g.N;
    const int mtiles = (g.M + TM - 1) / TM;
    const int mt = blockIdx.x % mtiles;
    const long long jt = blockIdx.x / mtiles;
    const int i0 = mt * TM;
    const long long j0 = jt * Cfg::TN;

    const TileThread<Cfg> t;
    const float oob = float(g.oob);
    const int ldm = pad4(g.M);
    const size_t plane = (size_t)g.K * ldm;
    const int s_lane = threadIdx.x % 128, s_k = threadIdx.x / 128;
    const SimColumn sc = sim_column(g, j0 + s_lane, P);
    if (s_k == 0) col_base[s_lane] = sc.base;
    const bool live = sc.base >= 0;
    // a patch that lies entirely inside the image needs no per-tap bounds test
    const bool inside = live && sc.h0 >= 0 && sc.w0 >= 0 && sc.h0 + g.bh <= g.H && sc.w0 + g.bw <= g.W;
    const float* xs = x + (size_t)sc.n * g.C * g.H * g.W;
    const float* xc = xs + sc.h0 * g.W + sc.w0;
    float rb[Cfg::B_PER];

    float2 acc[Cfg::RM][Cfg::RN / 2];
#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_)
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN / 2; ++c_) acc[r_][c_] = make_float2(0.f, 0.f);

    auto fetchA = [&](int chunk, float* As) {
#pragma unroll
        for (int p = 0; p < NA; ++p)
            stage_copy_async<Cfg, TM>(As + p * Cfg::KC * TM, planes + p * plane, ldm, chunk * Cfg::KC, g.K, i0, g.M);
    };
    auto fetchB = [&](int chunk, float*) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) {
            const int k = chunk * Cfg::KC + s_k + s * 2;
            // rows past K pair a zero scale / zero constant with a finite value: the term is exactly 0
            if (k >= g.K || !live) rb[s] = 0.f;
            else if (inside) rb[s] = __ldg(xc + __ldg(taps + k).x);
            else rb[s] = sim_tap_value(g, xs, sc, __ldg(taps + k), oob);
        }
    };
    auto commitA = [&](float*) { cp_async_wait_all(); };
    auto commitB = [&](float* Bs) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) {
            const int o = (s_k + s * 2) * Cfg::TN + s_lane;
            if (NB == 2) {
                const bool nan = rb[s] != rb[s];
                Bs[o] = nan ? 0.f : rb[s];
                Bs[Cfg::KC * Cfg::TN + o] = nan ? 0.f : 1.f;
            } else {
                Bs[o] = rb[s];
            }
        }
    };
    auto comb = [&](int r_, int cp, const float2 (&a)[NA], const float2 (&b)[NB]) {
        const float2 d = add2(a[0], neg2(b[0]));
        if (MODE == SIM_L1) acc[r_][cp] = fma2(a[1], abs2(d), acc[r_][cp]);
        else if (MODE == SIM_L1_SKIP) acc[r_][cp] = fma2(a[1], mul2(abs2(d), b[NB - 1]), acc[r_][cp]);
        else if (MODE == SIM_L2N_NAN) acc[r_][cp] = fma2(b[NB - 1], fma2(mul2(a[1], d), d, a[NA - 1]), acc[r_][cp]);
        else acc[r_][cp] = fma2(mul2(a[1], d), d, acc[r_][cp]);
    };
    tile_mainloop<Cfg, false, false>(smem, (g.K + Cfg::KC - 1) / Cfg::KC, t, fetchA, fetchB, commitA, commitB, comb);

    long long cb[Cfg::RN];
#pragma unroll
    for (int c_ = 0; c_ < Cfg::RN; ++c_) cb[c_] = col_base[t.col(c_)];
    const float quirk_c = float(-0.5 * double(g.K) * kLog2Pi);
#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_) {
        const int m = i0 + t.row(r_);
        if (m >= g.M) continue;
        const float cmm = cm[m];
        float* yrow = y + (long long)m * g.N;
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN; ++c_) {
            if (cb[c_] < 0) continue;
            float v = (c_ & 1) ? acc[r_][c_ >> 1].y : acc[r_][c_ >> 1].x;
            if (MODE == SIM_L2N) {
                v += cmm;
                if (g.batch_quirk) v += quirk_c * float(g.B - 1 - int(cb[c_] / ((long long)g.M * g.N)));
            }
            __stcs(yrow + cb[c_], v);
        }
    }
}

// -------------------------------------------------------- parameter gradients
// Accumulators per output (m, k): sT = sum a*d, sW = sum a*d*d (L1: a*sign(d), a*|d|), sN = sum a*mask,
// with a = dy and d = mask*(x - t).  Both operands are contiguous along q (positions) in memory.
template <int MODE, int TN>
__global__ void __launch_bounds__(TN * 4, TN == 32 ? 4 : 2) sim_dparams_tiled(SimGeo g, const float* __restrict__ x, const float* __restrict__ tm,
                                                         const float* __restrict__ dy, const int2* __restrict__ taps,
                                                         float* __restrict__ part, int splits) {
    constexpr bool MASKED = MODE == SIM_L2N_NAN || MODE == SIM_L1_SKIP;
    constexpr bool NORM = MODE == SIM_L2N || MODE == SIM_L2N_NAN;
    constexpr bool L1 = MODE == SIM_L1 || MODE == SIM_L1_SKIP;
    constexpr int NB = MASKED ? 2 : 1;
    using Cfg = TileCfg<kDpTile, TN, kDpKC, 4, 4, 1, NB>;
    static_assert(Cfg::THREADS == TN * 4, "64 x TN outputs, 4 x 4 per thread");
    constexpr int ROWS = Cfg::THREADS / 32;          // tile rows one staging pass covers
    __shared__ __align__(16) float smem[Cfg::SMEM_FLOATS];
    const long long P = (long long)g.B * g.N;
    const int ktiles = (g.K + TN - 1) / TN, mtiles = (g.M + kDpTile - 1) / kDpTile;
    int bid = blockIdx.x;
    const int kt = bid % ktiles; bid /= ktiles;
    const int mt = bid % mtiles;
    const int split = bid / mtiles;
    const int i0 = mt * kDpTile, jk0 = kt * TN;
    const long long chunks = (P + kDpKC - 1) / kDpKC;
    const long long c_begin = chunks * split / splits, c_end = chunks * (split + 1) / splits;

    const TileThread<Cfg> t;
    const float oob = float(g.oob);
    const int qq = threadIdx.x % 32, e0 = threadIdx.x / 32;
    SimColumn cur;
    float ra[Cfg::A_PER], rb[Cfg::B_PER];
    int2 mytaps[Cfg::B_PER];
#pragma unroll
    for (int s = 0; s < Cfg::B_PER; ++s) {
        const int k = jk0 + e0 + ROWS * s;
        mytaps[s] = k < g.K ? taps[k] : make_int2(0, 0);
    }
    float2 tt[4][2];
#pragma unroll
    for (int r_ = 0; r_ < 4; ++r_)
#pragma unroll
        for (int c_ = 0; c_ < 4; ++c_) {
            const int m = i0 + t.row(r_), k = jk0 + t.col(c_);
            const float v = (m < g.M && k < g.K) ? tm[(size_t)m * g.K + k] : 0.f;
            if (c_ & 1) tt[r_][c_ >> 1].y = v; else tt[r_][c_ >> 1].x = v;
        }
    float2 sT[4][2], sW[4][2], sN[4][2];
#pragma unroll
    for (int r_ = 0; r_ < 4; ++r_)
#pragma unroll
        for (int c_ = 0; c_ < 2; ++c_) { sT[r_][c_] = make_float2(0.f, 0.f); sW[r_][c_] = sT[r_][c_]; sN[r_][c_] = sT[r_][c_]; }

    auto fetchA = [&](int chunk, float*) {
        cur = sim_column(g, (c_begin + chunk) * kDpKC + qq, P);
#pragma unroll
        for (int s = 0; s < Cfg::A_PER; ++s) {
            const int m = i0 + e0 + ROWS * s;
            ra[s] = (cur.base >= 0 && m < g.M) ? __ldcs(dy + cur.base + (long long)m * g.N) : 0.f;
        }
    };
    auto fetchB = [&](int, float*) {
        const float* xs = x + (size_t)cur.n * g.C * g.H * g.W;
        const bool inside = cur.base >= 0 && cur.h0 >= 0 && cur.w0 >= 0 && cur.h0 + g.bh <= g.H && cur.w0 + g.bw <= g.W;
        const float* xc = xs + cur.h0 * g.W + cur.w0;
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) {
            const int k = jk0 + e0 + ROWS * s;
            // dead positions carry dy = 0 and a finite value, so every term they touch is exactly 0
            if (cur.base < 0 || k >= g.K) rb[s] = 0.f;
            else if (inside) rb[s] = __ldg(xc + mytaps[s].x);
            else rb[s] = sim_tap_value(g, xs, cur, mytaps[s], oob);
        }
    };
    auto commitA = [&](float* As) {
#pragma unroll
        for (int s = 0; s < Cfg::A_PER; ++s) As[stage_offset<kDpTile, true>(qq, e0 + ROWS * s)] = ra[s];
    };
    auto commitB = [&](float* Bs) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) {
            const int o = stage_offset<TN, true>(qq, e0 + ROWS * s);
            if (MASKED) {
                const bool nan = rb[s] != rb[s];
                Bs[o] = nan ? 0.f : rb[s];
                Bs[Cfg::KC * Cfg::TN + o] = (nan || cur.base < 0) ? 0.f : 1.f;
            } else {
                Bs[o] = rb[s];
            }
        }
    };
    auto comb = [&](int r_, int cp, const float2 (&a)[1], const float2 (&b)[NB]) {
        const float2 d = MASKED ? fma2(neg2(tt[r_][cp]), b[NB - 1], b[0]) : add2(b[0], neg2(tt[r_][cp]));
        if (L1) {
            const float2 sg = make_float2(float((0.f < d.x) - (d.x < 0.f)), float((0.f < d.y) - (d.y < 0.f)));
            sT[r_][cp] = fma2(a[0], sg, sT[r_][cp]);
            sW[r_][cp] = fma2(a[0], abs2(d), sW[r_][cp]);
        } else {
            const float2 u = mul2(a[0], d);
            sT[r_][cp] = add2(sT[r_][cp], u);
            sW[r_][cp] = fma2(u, d, sW[r_][cp]);
            if (NORM) sN[r_][cp] = MASKED ? fma2(a[0], b[NB - 1], sN[r_][cp]) : add2(sN[r_][cp], a[0]);
        }
    };
    tile_mainloop<Cfg, true, true>(smem, int(c_end - c_begin), t, fetchA, fetchB, commitA, commitB, comb);

    const size_t mk = (size_t)g.M * g.K;
    float* dst = part + (size_t)split * 3 * mk;
#pragma unroll
    for (int r_ = 0; r_ < 4; ++r_) {
        const int m = i0 + t.row(r_);
        if (m >= g.M) continue;
#pragma unroll
        for (int c_ = 0; c_ < 4; ++c_) {
            const int k = jk0 + t.col(c_);
            if (k >= g.K) continue;
            const bool hi = c_ & 1;
            dst[(size_t)m * g.K + k] = hi ? sT[r_][c_ >> 1].y : sT[r_][c_ >> 1].x;
            dst[mk + (size_t)m * g.K + k] = hi ? sW[r_][c_ >> 1].y : sW[r_][c_ >> 1].x;
            if (NORM) dst[2 * mk + (size_t)m * g.K + k] = hi ? sN[r_][c_ >> 1].y : sN[r_][c_ >> 1].x;
        }
    }
}

// -------------------------------------------------------------- input gradient
// dx[n, c, h, w] = sum over the taps (kh, kw) whose patch covers the pixel and over m of  s*w * dy * (t - x)   (L1: sign(t - x))
// as a generalized GEMM with i = c, j = pixel, q = (kh, kw, m): the reference's column gradient followed by col2im
// (HUJI-Deep/simnets-tf src/kernels/similarity_grad_kernel_cpu.cpp:205-268) becomes one gather, nothing is scattered.
// A = (t, s*w)[q][c] from the prepass, B[q][j] = dy at the output position that tap (kh, kw) maps the pixel to (0 if none),
// and the pixel's own x value sits in registers.  NaN pixels give 0 in the ignore_nan_input modes (epilogue select).
// Known deviation: a pixel holding +-inf whose coverage is partial (taps cut off by padding or stride) yields NaN where
// the reference yields +-inf, because a cut-off tap contributes 0 * (t - inf).
struct DxColumn { long long base; int n, h, w; };   // base = n*C*H*W + h*W + w, or -1 past the end

template <int TM, int MODE>
__global__ void __launch_bounds__(256) sim_dx_tiled(SimGeo g, const float* __restrict__ x, const float* __restrict__ dxp,
                                                    const float* __restrict__ dy, float* __restrict__ dx) {
    constexpr bool L1 = MODE == SIM_L1 || MODE == SIM_L1_SKIP;
    constexpr bool SKIP_NAN = MODE == SIM_L2N_NAN || MODE == SIM_L1_SKIP;
    using Cfg = TileCfg<TM, 128, 8, TM / 16, 8, 2, 1>;
    static_assert(Cfg::THREADS == 256, "256 threads");
    __shared__ __align__(16) float smem[Cfg::SMEM_FLOATS];
    __shared__ long long col_base[Cfg::TN];
    const long long P = (long long)g.B * g.H * g.W;
    const int ctiles = (g.C + TM - 1) / TM;
    const int ct = blockIdx.x % ctiles;
    const long long jt = blockIdx.x / ctiles;
    const int i0 = ct * TM;
    const long long j0 = jt * Cfg::TN;
    const int Q = g.bh * g.bw * g.M, ldc = pad4(g.C);
    const size_t dplane = (size_t)Q * ldc;

    const TileThread<Cfg> t;
    const int s_lane = threadIdx.x % 128, s_k = threadIdx.x / 128;
    DxColumn sc;
    {
        const long long j = j0 + s_lane;
        sc.base = -1; sc.n = sc.h = sc.w = 0;
        if (j < P) {
            const int hw = g.H * g.W;
            sc.n = int(j / hw);
            const int p = int(j - (long long)sc.n * hw);
            sc.h = p / g.W; sc.w = p % g.W;
            sc.base = (long long)sc.n * g.C * hw + p;
        }
    }
    if (s_k == 0) col_base[s_lane] = sc.base;
    const float* dyn = dy + (size_t)sc.n * g.M * g.N;
    // staging cursor over q = (tap, m): element s of a chunk is q = chunk*8 + s_k + 2*s
    float rb[Cfg::B_PER];

    float2 acc[Cfg::RM][Cfg::RN / 2];
#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_)
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN / 2; ++c_) acc[r_][c_] = make_float2(0.f, 0.f);

    auto fetchA = [&](int chunk, float* As) {
#pragma unroll
        for (int p = 0; p < 2; ++p) stage_copy_async<Cfg, TM>(As + p * Cfg::KC * TM, dxp + p * dplane, ldc, chunk * Cfg::KC, Q, i0, g.C);
    };
    auto fetchB = [&](int chunk, float*) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) {
            const int q = chunk * Cfg::KC + s_k + s * 2;
            float v = 0.f;
            if (q < Q && sc.base >= 0) {
                const int tap = q / g.M, m = q - tap * g.M;
                const int kh = tap / g.bw, kw = tap - kh * g.bw;
                const int hp = sc.h + g.ph - kh, wp = sc.w + g.pw - kw;
                if (hp >= 0 && wp >= 0) {
                    const int ho = hp / g.sh, wo = wp / g.sw;
                    if (ho * g.sh == hp && wo * g.sw == wp && ho < g.oh && wo < g.ow) v = __ldg(dyn + (size_t)m * g.N + ho * g.ow + wo);
                }
            }
            rb[s] = v;
        }
    };
    auto commitA = [&](float*) { cp_async_wait_all(); };
    auto commitB = [&](float* Bs) {
#pragma unroll
        for (int s = 0; s < Cfg::B_PER; ++s) Bs[(s_k + s * 2) * Cfg::TN + s_lane] = rb[s];
    };

    // wait for col_base, then this thread's own x values (one per output)
    __syncthreads();
    long long cb[Cfg::RN];
#pragma unroll
    for (int c_ = 0; c_ < Cfg::RN; ++c_) cb[c_] = col_base[t.col(c_)];
    float2 xx[Cfg::RM][Cfg::RN / 2];
    const size_t chw = (size_t)g.H * g.W;
#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_) {
        const int c = i0 + t.row(r_);
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN; ++c_) {
            const float v = (c < g.C && cb[c_] >= 0) ? __ldg(x + cb[c_] + (size_t)c * chw) : 0.f;
            if (c_ & 1) xx[r_][c_ >> 1].y = v; else xx[r_][c_ >> 1].x = v;
        }
    }
    auto comb = [&](int r_, int cp, const float2 (&a)[2], const float2 (&b)[1]) {
        const float2 d = add2(a[0], neg2(xx[r_][cp]));
        const float2 e = mul2(a[1], b[0]);
        if (L1) {
            const float2 sg = make_float2(float((0.f < d.x) - (d.x < 0.f)), float((0.f < d.y) - (d.y < 0.f)));
            acc[r_][cp] = fma2(e, sg, acc[r_][cp]);
        } else {
            acc[r_][cp] = fma2(e, d, acc[r_][cp]);
        }
    };
    tile_mainloop<Cfg, false, false>(smem, (Q + Cfg::KC - 1) / Cfg::KC, t, fetchA, fetchB, commitA, commitB, comb);

#pragma unroll
    for (int r_ = 0; r_ < Cfg::RM; ++r_) {
        const int c = i0 + t.row(r_);
        if (c >= g.C) continue;
#pragma unroll
        for (int c_ = 0; c_ < Cfg::RN; ++c_) {
            if (cb[c_] < 0) continue;
            float v = (c_ & 1) ? acc[r_][c_ >> 1].y : acc[r_][c_ >> 1].x;
            const float xv = (c_ & 1) ? xx[r_][c_ >> 1].y : xx[r_][c_ >> 1].x;
            if (SKIP_NAN && xv != xv) v = 0.f;
            dx[cb[c_] + (size_t)c * chw] = v;
        }
    }
}

// Sums the split partials in split order and applies the per-parameter factors of the backward functors.
// 32 outputs x 16 slices of the splits per CTA; the slices are added in a fixed order (same sums on every run)
__global__ void __launch_bounds__(512) sim_dparams_reduce(SimGeo g, int splits, const float* __restrict__ part,
                                                          const float* __restrict__ wt, float* __restrict__ dt, float* __restrict__ dw,
                                                          int accumulate) {
    // a CTA sums 8 consecutive outputs (one 32-byte sector per split) over all splits: 64 slices of the splits in
    // parallel, then the slices in a fixed order (deterministic).  Few outputs per CTA so that the short patches of a
    // first layer (M K = 1728) still spread over a couple of hundred CTAs.
    __shared__ float red[3][64][8];
    const int mk = g.M * g.K;
    const float fudge = float(g.fudge);
    const bool third = g.mode == SIM_L2N || g.mode == SIM_L2N_NAN;
    const int lane = threadIdx.x & 7, slice = threadIdx.x >> 3;
    for (int first = blockIdx.x * 8; first < mk; first += gridDim.x * 8) {
        const int i = first + lane;
        float a = 0.f, b = 0.f, c = 0.f;
        if (i < mk) {
#pragma unroll 4
            for (int s = slice; s < splits; s += 64) {
                const float* p = part + (size_t)s * 3 * mk;
                a += p[i]; b += p[mk + i];
                if (third) c += p[2 * mk + i];
            }
        }
        red[0][slice][lane] = a; red[1][slice][lane] = b; red[2][slice][lane] = c;
        __syncthreads();
        if (slice == 0 && i < mk) {
#pragma unroll 8
            for (int q = 1; q < 64; ++q) { a += red[0][q][lane]; b += red[1][q][lane]; c += red[2][q][lane]; }
            const float wraw = wt[i], w = g.absw ? fabsf(wraw) : wraw;
            float gt, gw;
            if (g.mode == SIM_L1 || g.mode == SIM_L1_SKIP) { gt = w * a; gw = -b; }
            else if (g.mode == SIM_L2) { gt = 2.f * w * a; gw = -b; }
            else { gt = w * a; gw = 0.5f * (c / (w + fudge) - b); }
            if (g.absw) gw *= wraw > 0.f ? 1.f : (wraw < 0.f ? -1.f : 0.f);          // d|w|/dw, 0 at w = 0
            dt[i] = accumulate ? dt[i] + gt : gt;
            dw[i] = accumulate ? dw[i] + gw : gw;
        }
        __syncthreads();
    }
}

void launch_prep(const SimGeo& g, const SimWs& w, const float* t, const float* wt, cudaStream_t s) {
    sim_prep<<<g.M, 128, 0, s>>>(g, t, wt, w.planes, w.cm, w.taps, w.dxp, w.flag);
    count_launch();
}

}  // namespace

bool sim_use_tiled(const SimGeo& g, bool f64, uint32_t flags) {
    if (f64 || g.B == 0) return false;
    if (flags & SIMNETS_FLAG_FORCE_DIRECT) return false;
    if (g.bh >= 32768 || g.bw >= 32768) return false;
    return true;
}

size_t sim_workspace_bytes(const SimGeo& g, bool f64, uint32_t flags) {
    if (!sim_use_tiled(g, f64, flags)) return 256;
    return carve(g, nullptr).bytes;
}

static cudaError_t sim_fwd_tiled_body(const SimGeo& g, const float* x, const float* t, const float* w, float* y, void* ws, uint32_t flags,
                                      cudaStream_t s, float* ch_max, float* ch_min, bool* extrema_done);

cudaError_t launch_sim_fwd_tiled(const SimGeo& g, const float* x, const float* t, const float* w, float* y, void* ws, uint32_t flags,
                                 cudaStream_t s, float* ch_max, float* ch_min) {
    bool done = false;
    const cudaError_t e = sim_fwd_tiled_body(g, x, t, w, y, ws, flags, s, ch_max, ch_min, &done);
    if (e != cudaSuccess || done) return e;
    return launch_sim_extrema(g, y, ch_max, ch_min, s);
}

static cudaError_t sim_fwd_tiled_body(const SimGeo& g, const float* x, const float* t, const float* w, float* y, void* ws, uint32_t flags,
                                      cudaStream_t s, float* ch_max, float* ch_min, bool* extrema_done) {
    const SimWs W = carve(g, ws);
    launch_prep(g, W, t, w, s);
    if (sim_tc_shape(g, flags)) {
        // opt-in: the expanded square on the tensor cores; behind it the term-by-term kernel, which runs only if a
        // bounded wait of the tensor-core kernel ran out (word 1 of the flags)
        const cudaError_t e = launch_sim_fwd_tc(g, x, W.planes, W.cm, W.taps, W.tc_tiles, W.tc_bias, W.flag, y, s);
        if (e != cudaSuccess) return e;
        return launch_sim_fwd_direct(g, false, x, t, w, y, s, W.flag);
    }
    if (sim_smallk_shape(g)) { *extrema_done = true; return launch_sim_fwd_smallk(g, x, W.planes, W.cm, W.taps, y, ch_max, ch_min, s); }
    const long long P = (long long)g.B * g.N;
    const bool wide = g.M > 64;
    const long long blocks = ((P + 127) / 128) * ((g.M + (wide ? 127 : 63)) / (wide ? 128 : 64));
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
#define FWD(TM, MODE) sim_fwd_tiled<TM, MODE><<<int(blocks), 256, 0, s>>>(g, x, W.planes, W.cm, W.taps, y)
#define FWD_MODES(TM)                                        \
    switch (g.mode) {                                        \
    case SIM_L1: FWD(TM, SIM_L1); break;                     \
    case SIM_L1_SKIP: FWD(TM, SIM_L1_SKIP); break;           \
    case SIM_L2: FWD(TM, SIM_L2); break;                     \
    case SIM_L2N: FWD(TM, SIM_L2N); break;                   \
    default: FWD(TM, SIM_L2N_NAN); break;                    \
    }
    if (wide) { FWD_MODES(128) } else { FWD_MODES(64) }
#undef FWD_MODES
#undef FWD
    count_launch();
    return cudaGetLastError();
}

// every pixel is covered by at least one tap (otherwise an uncovered NaN pixel would have to come out as 0)
static bool every_pixel_covered(const SimGeo& g) {
    auto axis = [](int dim, int block, int stride, int pad, int out) {
        if (stride > block) return false;                        // gaps between patches
        return pad >= 0 && (out - 1) * stride + block - pad >= dim;   // last patch reaches the end; first starts at <= 0
    };
    return axis(g.H, g.bh, g.sh, g.ph, g.oh) && axis(g.W, g.bw, g.sw, g.pw, g.ow);
}

cudaError_t launch_sim_dx_tiled(const SimGeo& g, const float* x, const float* t, const float* w, const float* dy, float* dx, void* ws, cudaStream_t s) {
    // few channels: the gather kernel is memory bound there and needs no staging; also when some pixel has no tap at all
    if (g.C < 16 || !every_pixel_covered(g)) return launch_sim_dx_direct(g, false, x, t, w, dy, dx, s);
    const SimWs W = carve(g, ws);
    launch_prep(g, W, t, w, s);
    const long long P = (long long)g.B * g.H * g.W;
    const bool wide = g.C > 64;
    const long long blocks = ((P + 127) / 128) * ((g.C + (wide ? 127 : 63)) / (wide ? 128 : 64));
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
#define DX(TM, MODE) sim_dx_tiled<TM, MODE><<<int(blocks), 256, 0, s>>>(g, x, W.dxp, dy, dx)
#define DX_MODES(TM)                                         \
    switch (g.mode) {                                        \
    case SIM_L1: DX(TM, SIM_L1); break;                      \
    case SIM_L1_SKIP: DX(TM, SIM_L1_SKIP); break;            \
    case SIM_L2: DX(TM, SIM_L2); break;                      \
    case SIM_L2N: DX(TM, SIM_L2N); break;                    \
    default: DX(TM, SIM_L2N_NAN); break;                     \
    }
    if (wide) { DX_MODES(128) } else { DX_MODES(64) }
#undef DX_MODES
#undef DX
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_sim_dparams_tiled(const SimGeo& g, const float* x, const float* t, const float* w, const float* dy,
                                     float* dt, float* dw, bool accumulate, void* ws, cudaStream_t s) {
    const SimWs W = carve(g, ws);
    launch_prep(g, W, t, w, s);
    const int splits = dp_splits(g);
    const int tn = dp_tn(g);
    const int blocks = ((g.M + kDpTile - 1) / kDpTile) * ((g.K + tn - 1) / tn) * splits;
#define DP(MODE)                                                                                              \
    do {                                                                                                      \
        if (tn == 32) sim_dparams_tiled<MODE, 32><<<blocks, 128, 0, s>>>(g, x, t, dy, W.taps, W.part, splits); \
        else sim_dparams_tiled<MODE, 64><<<blocks, 256, 0, s>>>(g, x, t, dy, W.taps, W.part, splits);          \
    } while (0)
    switch (g.mode) {
    case SIM_L1: DP(SIM_L1); break;
    case SIM_L1_SKIP: DP(SIM_L1_SKIP); break;
    case SIM_L2: DP(SIM_L2); break;
    case SIM_L2N: DP(SIM_L2N); break;
    default: DP(SIM_L2N_NAN); break;
    }
#undef DP
    const int mk = g.M * g.K;
    sim_dparams_reduce<<<std::min((mk + 7) / 8, device_sm_count() * 8), 512, 0, s>>>(g, splits, W.part, w, dt, dw, accumulate);
    count_launch(2);
    return cudaGetLastError();
}

}  // namespace simnets
