// Similarity forward for short patches (K = C * bh * bw <= 32: a first layer over a few image channels).
//
// As a generalized GEMM this shape is all epilogue: 27 taps under 64 templates leave the 128 x 128 tile kernel of
// sim_tiled.cu half empty along the reduction and it spends its time staging.  Here the patch lives in registers: a
// thread owns TWO output positions (so that every arithmetic instruction is the packed two-lane form), loads their K
// taps once, and walks the templates two at a time; the (template, weight) pairs of a tap come from shared memory as
// one 16-byte broadcast read per four terms.  The inner product is the same three operations per term as everywhere
// else (difference, scale, fused multiply-add), so results equal the tile kernel's up to summation order.
// All five modes of the forward functor (include/utils/similarity_utils.hpp:17-60 of the reference) are covered; NaN
// taps of the ignore-NaN modes become a per-position bit mask (K <= 32 bits).
#include "kernels.cuh"
#include "tile.cuh"

namespace simnets {

namespace {

constexpr int kSkThreads = 128;
constexpr int kSkBlocksPerSm = 4;      // 128 registers per thread: four CTAs (16 warps) per SM measured 6 % faster than three at 168

struct SkColumn { long long base; int n, h0, w0; };

__device__ __forceinline__ SkColumn sk_column(const SimGeo& g, long long j, long long P) {
    SkColumn c;
    c.base = -1; c.n = 0; c.h0 = c.w0 = 0;
    if (j >= P) return c;
    const int n = int(j / g.N), pos = int(j % g.N);
    c.n = n;
    c.h0 = (pos / g.ow) * g.sh - g.ph;
    c.w0 = (pos % g.ow) * g.sw - g.pw;
    c.base = (long long)n * g.M * g.N + pos;
    return c;
}

// planes: [3][K][ldm] (template, scale, per-term constant) as sim_prep writes them; taps: [K] {offset inside a sample, (kh << 16) | kw}
// KT = the patch length at compile time (the tap loops are fully unrolled, the patches are register arrays).
template <int MODE, int KT>
__global__ void __launch_bounds__(kSkThreads, kSkBlocksPerSm) sim_fwd_smallk(SimGeo g, const float* __restrict__ x, const float* __restrict__ planes,
                                                               const float* __restrict__ cm, const int2* __restrict__ taps,
                                                               float* __restrict__ y, float* __restrict__ ch_max, float* __restrict__ ch_min) {
    constexpr bool MASKED = MODE == SIM_L2N_NAN || MODE == SIM_L1_SKIP;
    constexpr bool L1 = MODE == SIM_L1 || MODE == SIM_L1_SKIP;
    constexpr int MQ = 4;                                   // templates walked together: four independent accumulator chains
    extern __shared__ __align__(16) float sm[];
    const int M = g.M, ldm = (g.M + 3) & ~3, Mq = (M + MQ - 1) / MQ * MQ;
    // shared: ts[k][m] = {t, t, s, s}: both lanes of the packed operands come out of one 16-byte broadcast read;
    // cs[k][m] = {c, c} for the NaN-aware L2; tp[k] = tap table
    float4* ts = reinterpret_cast<float4*>(sm);
    float2* cs = reinterpret_cast<float2*>(sm + (size_t)KT * Mq * 4);
    __shared__ int2 tp[KT];
    const size_t plane = (size_t)KT * ldm;
    for (int i = threadIdx.x; i < KT * Mq; i += kSkThreads) {
        const int k = i / Mq, m = i % Mq;
        const bool in = m < M;
        const float t = in ? planes[(size_t)k * ldm + m] : 0.f, sc = in ? planes[plane + (size_t)k * ldm + m] : 0.f;
        ts[i] = make_float4(t, t, sc, sc);
        if (MODE == SIM_L2N_NAN) { const float c = in ? planes[2 * plane + (size_t)k * ldm + m] : 0.f; cs[i] = make_float2(c, c); }
    }
    if (threadIdx.x < KT) tp[threadIdx.x] = taps[threadIdx.x];
    __syncthreads();

    const long long P = (long long)g.B * g.N;
    const float oob = float(g.oob);
    const float quirk_c = float(-0.5 * double(KT) * 1.8378770664093453);      // -0.5 K log(2 pi)
    for (long long j0 = (blockIdx.x * (long long)kSkThreads + threadIdx.x) * 2; j0 < P; j0 += (long long)gridDim.x * kSkThreads * 2) {
        const SkColumn c0 = sk_column(g, j0, P), c1 = sk_column(g, j0 + 1, P);
        // the two patches, tap by tap, NEGATED, in registers: d = t + (-x)
        float2 nx[KT];
        unsigned mask0 = 0u, mask1 = 0u;
        const float* xs0 = x + (size_t)c0.n * g.C * g.H * g.W + c0.h0 * g.W + c0.w0;
        const float* xs1 = x + (size_t)c1.n * g.C * g.H * g.W + c1.h0 * g.W + c1.w0;
        const bool in0 = c0.h0 >= 0 && c0.w0 >= 0 && c0.h0 + g.bh <= g.H && c0.w0 + g.bw <= g.W;
        const bool in1 = c1.base >= 0 && c1.h0 >= 0 && c1.w0 >= 0 && c1.h0 + g.bh <= g.H && c1.w0 + g.bw <= g.W;
#pragma unroll
        for (int k = 0; k < KT; ++k) {
            const int2 t2 = tp[k];
            const int kh = t2.y >> 16, kw = t2.y & 0xffff;
            float a = oob, b = oob;
            if (in0 || (c0.h0 + kh >= 0 && c0.h0 + kh < g.H && c0.w0 + kw >= 0 && c0.w0 + kw < g.W)) a = __ldg(xs0 + t2.x);
            if (in1 || (c1.base >= 0 && c1.h0 + kh >= 0 && c1.h0 + kh < g.H && c1.w0 + kw >= 0 && c1.w0 + kw < g.W)) b = __ldg(xs1 + t2.x);
            if (MASKED) {
                if (a == a) mask0 |= 1u << k; else a = 0.f;
                if (b == b) mask1 |= 1u << k; else b = 0.f;
            }
            nx[k] = make_float2(-a, -b);
        }
        const bool pair_store = c1.base == c0.base + 1 && ((c0.base & 1) == 0) && ((((long long)g.N) & 1) == 0);
        // per-pixel extrema over the instances, for a consumer that stabilises a log-sum-exp over them (NaN ignored)
        float2 vmax = make_float2(-CUDART_INF_F, -CUDART_INF_F), vmin = make_float2(CUDART_INF_F, CUDART_INF_F);
#pragma unroll 1
        for (int m0 = 0; m0 < Mq; m0 += MQ) {
            float2 acc[MQ];
#pragma unroll
            for (int q = 0; q < MQ; ++q) acc[q] = make_float2(0.f, 0.f);
#pragma unroll
            for (int k = 0; k < KT; ++k) {
                float2 k0;
                if (MASKED) k0 = make_float2((mask0 >> k) & 1u ? 1.f : 0.f, (mask1 >> k) & 1u ? 1.f : 0.f);
#pragma unroll
                for (int q = 0; q < MQ; ++q) {
                    const float4 p = ts[k * Mq + m0 + q];
                    const float2 tt = make_float2(p.x, p.y), ss = make_float2(p.z, p.w);
                    const float2 d = add2(tt, nx[k]);
                    if (!MASKED) {
                        if (L1) acc[q] = fma2(ss, make_float2(fabsf(d.x), fabsf(d.y)), acc[q]);
                        else acc[q] = fma2(mul2(ss, d), d, acc[q]);
                    } else if (L1) {
                        acc[q] = fma2(ss, mul2(make_float2(fabsf(d.x), fabsf(d.y)), k0), acc[q]);
                    } else {
                        acc[q] = fma2(k0, fma2(mul2(ss, d), d, cs[k * Mq + m0 + q]), acc[q]);
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < MQ; ++q) {
                const int m = m0 + q;
                if (m >= M) break;
                float2 v = acc[q];
                if (MODE == SIM_L2N) {
                    const float cmm = cm[m];
                    v.x += cmm; v.y += cmm;
                    if (g.batch_quirk) { v.x += quirk_c * float(g.B - 1 - c0.n); v.y += quirk_c * float(g.B - 1 - c1.n); }
                }
                vmax = make_float2(fmaxf(vmax.x, v.x), fmaxf(vmax.y, v.y));
                vmin = make_float2(fminf(vmin.x, v.x), fminf(vmin.y, v.y));
                if (c0.base >= 0) {
                    float* dst = y + c0.base + (long long)m * g.N;
                    if (pair_store) __stcs(reinterpret_cast<float2*>(dst), v);
                    else {
                        __stcs(dst, v.x);
                        if (c1.base >= 0) __stcs(y + c1.base + (long long)m * g.N, v.y);
                    }
                }
            }
        }
        if (ch_max != nullptr || ch_min != nullptr) {
            const long long q0 = c0.base - (long long)c0.n * (g.M - 1) * g.N, q1 = c1.base - (long long)c1.n * (g.M - 1) * g.N;      // n * N + pos
            if (c0.base >= 0) { if (ch_max) ch_max[q0] = vmax.x; if (ch_min) ch_min[q0] = vmin.x; }
            if (c1.base >= 0) { if (ch_max) ch_max[q1] = vmax.y; if (ch_min) ch_min[q1] = vmin.y; }
        }
    }
}

// The same extrema from a finished output tensor, for the forward kernels that do not produce them on the way
__global__ void __launch_bounds__(256) sim_extrema(long long P, int M, int N, const float* __restrict__ y, float* __restrict__ ch_max, float* __restrict__ ch_min) {
    for (long long q = blockIdx.x * 256LL + threadIdx.x; q < P; q += (long long)gridDim.x * 256) {
        const long long n = q / N;
        const float* p = y + n * (long long)M * N + (q - n * N);
        float hi = -CUDART_INF_F, lo = CUDART_INF_F;
        for (int m = 0; m < M; ++m) { const float v = __ldg(p + (long long)m * N); hi = fmaxf(hi, v); lo = fminf(lo, v); }
        if (ch_max) ch_max[q] = hi;
        if (ch_min) ch_min[q] = lo;
    }
}

size_t sk_smem_bytes(const SimGeo& g) { return (size_t)g.K * ((g.M + 3) / 4 * 4) * (16 + (g.mode == SIM_L2N_NAN ? 8 : 0)); }

template <int KT>
cudaError_t launch_sk(const SimGeo& g, const float* x, const float* planes, const float* cm, const int2* taps, float* y, float* ch_max,
                      float* ch_min, cudaStream_t s) {
    const long long P = (long long)g.B * g.N;
    const size_t smem = sk_smem_bytes(g);
    const long long want = (P / 2 + kSkThreads - 1) / kSkThreads;
    const int grid = int(std::max<long long>(1, std::min<long long>(want, (long long)kSkBlocksPerSm * device_sm_count())));
#define SK(MODE)                                                                                                       \
    do {                                                                                                               \
        static bool attr_done = false;                                                                                 \
        if (!attr_done) {                                                                                              \
            const cudaError_t e_ = cudaFuncSetAttribute(sim_fwd_smallk<MODE, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024); \
            if (e_ != cudaSuccess) return e_;                                                                          \
            attr_done = true;                                                                                          \
        }                                                                                                              \
        sim_fwd_smallk<MODE, KT><<<grid, kSkThreads, smem, s>>>(g, x, planes, cm, taps, y, ch_max, ch_min);              \
    } while (0)
    switch (g.mode) {
    case SIM_L1: SK(SIM_L1); break;
    case SIM_L1_SKIP: SK(SIM_L1_SKIP); break;
    case SIM_L2: SK(SIM_L2); break;
    case SIM_L2N: SK(SIM_L2N); break;
    default: SK(SIM_L2N_NAN); break;
    }
#undef SK
    count_launch();
    return cudaGetLastError();
}

}  // namespace

// patch lengths with a compiled kernel (2x2 and 3x3 blocks over one or three channels) and parameters that fit shared memory
bool sim_smallk_shape(const SimGeo& g) {
    return (g.K == 4 || g.K == 9 || g.K == 12 || g.K == 27) && sk_smem_bytes(g) <= 64 * 1024;
}

// planes, cm, taps: as sim_prep leaves them in the workspace
cudaError_t launch_sim_fwd_smallk(const SimGeo& g, const float* x, const float* planes, const float* cm, const int2* taps, float* y,
                                  float* ch_max, float* ch_min, cudaStream_t s) {
    switch (g.K) {
    case 4: return launch_sk<4>(g, x, planes, cm, taps, y, ch_max, ch_min, s);
    case 9: return launch_sk<9>(g, x, planes, cm, taps, y, ch_max, ch_min, s);
    case 12: return launch_sk<12>(g, x, planes, cm, taps, y, ch_max, ch_min, s);
    default: return launch_sk<27>(g, x, planes, cm, taps, y, ch_max, ch_min, s);
    }
}

cudaError_t launch_sim_extrema(const SimGeo& g, const float* y, float* ch_max, float* ch_min, cudaStream_t s) {
    const long long P = (long long)g.B * g.N;
    if (P == 0 || (ch_max == nullptr && ch_min == nullptr)) return cudaSuccess;
    sim_extrema<<<int(std::min<long long>((P + 255) / 256, (long long)device_sm_count() * 16)), 256, 0, s>>>(P, g.M, g.N, y, ch_max, ch_min);
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
