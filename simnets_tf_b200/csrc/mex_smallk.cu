// MEX for short patches (K <= 32 taps, e.g. 4x2x2 blocks): the streaming regime.
//
// With K = 16 and M = 256 every input value feeds 256 outputs and every output is 16 multiply-adds: the
// work is dominated by writing y (forward) or reading y and dy (backward), i.e. by HBM.  GEMM tiles would
// stage each y / dy element through shared memory for only K uses, so here a THREAD owns whole positions:
// it keeps the K factors Ex[k] = exp(eps*(x[k] - mx)) of its positions in registers (the patch maximum mx
// falls out of the same K values, no prepass over x), walks the instances m, and reads Eo[m][0..K) as
// 16-byte shared-memory broadcasts.  For a fixed m consecutive threads hold consecutive positions, so every
// global access to y / dy is a full 128-byte line per warp.  Same factorised arithmetic and safety flag as
// mex_tiled.cu (see the derivation there).
#include "mex_common.cuh"

namespace simnets {

namespace {

constexpr int kT = 256;          // threads per CTA
constexpr int kMC = 256;         // instances whose Eo rows sit in shared memory at a time

// Loads the K taps of one position, returns their extreme (max for eps > 0) and leaves the raw values in v[].
template <int KP, bool SPATIAL1>
__device__ __forceinline__ float load_patch(const MexGeo& g, const float* __restrict__ x, const Column& col, float (&v)[KP]) {
    const bool up = g.eps > 0;
    const float oob = float(g.oob), dead = up ? -CUDART_INF_F : CUDART_INF_F;
    float ext = dead;
    const float* xs = x + (size_t)col.n * g.C * g.H * g.W;
#pragma unroll
    for (int k = 0; k < KP; ++k) {
        v[k] = (k < g.K && col.base >= 0) ? patch_value<SPATIAL1>(g, xs, col.c0, col.h0, col.w0, k, oob) : dead;
        ext = up ? fmaxf(ext, v[k]) : fminf(ext, v[k]);
    }
    return ext;
}

// Eo rows m0 .. m0+kMC-1 of region r (zero beyond M / K) and their stabilisers into shared memory.
template <int KP>
__device__ __forceinline__ void load_offsets_chunk(const MexGeo& g, const float* __restrict__ eo, const float* __restrict__ mo,
                                                   int r, int m0, float* eo_s, float* mo_s) {
    const int ldk = pad4(g.K);
    for (int i = threadIdx.x; i < kMC * KP; i += kT) {
        const int mm = i / KP, k = i % KP, m = m0 + mm;
        eo_s[i] = (m < g.M && k < g.K) ? __ldg(eo + ((size_t)r * g.M + m) * ldk + k) : 0.f;
    }
    for (int i = threadIdx.x; i < kMC; i += kT) mo_s[i] = (m0 + i < g.M) ? __ldg(mo + r * g.M + m0 + i) : 0.f;
}

// ------------------------------------------------------------------- forward
template <int KP, int C, bool SPATIAL1>
__global__ void __launch_bounds__(kT, 2) mex_fwd_smallk(MexGeo g, const float* __restrict__ x, const float* __restrict__ eo,
                                                     const float* __restrict__ mo, float* __restrict__ y, const int* __restrict__ flag) {
    __shared__ __align__(16) float eo_s[kMC * KP];
    __shared__ float mo_s[kMC];
    if (*flag) return;
    const long long P = (long long)g.B * g.rs;
    const int r = blockIdx.x % g.R;
    const long long j0 = (long long)(blockIdx.x / g.R) * (kT * C);
    const float eps = float(g.eps);
    float2 ex[C][KP / 2];
    float cadd[C];
    float* yb[C];                             // walks down the instances: y[n, m, pos] for m = 0, 1, ...
    bool live[C];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const Column col = column_of(g, r, j0 + c * kT + threadIdx.x, P, nullptr);
        float v[KP];
        const float mxv = load_patch<KP, SPATIAL1>(g, x, col, v);
#pragma unroll
        for (int k = 0; k < KP / 2; ++k) ex[c][k] = make_float2(fast_exp(eps * (v[2 * k] - mxv)), fast_exp(eps * (v[2 * k + 1] - mxv)));
        cadd[c] = mxv + float(g.cst) / eps;
        live[c] = col.base >= 0;
        yb[c] = y + (live[c] ? col.base : 0);
    }
    const float k_log = 0.69314718056f / eps;
    for (int m0 = 0; m0 < g.M; m0 += kMC) {
        __syncthreads();
        load_offsets_chunk<KP>(g, eo, mo, r, m0, eo_s, mo_s);
        __syncthreads();
        const int mend = min(kMC, g.M - m0);
#pragma unroll 4
        for (int mm = 0; mm < mend; ++mm) {
            float2 e[KP / 2];
#pragma unroll
            for (int q = 0; q < KP / 4; ++q) {
                const float4 t = *reinterpret_cast<const float4*>(eo_s + mm * KP + q * 4);
                e[2 * q] = make_float2(t.x, t.y); e[2 * q + 1] = make_float2(t.z, t.w);
            }
            const float mom = mo_s[mm];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                // two independent chains halve the dependent-FMA depth of one output
                float2 s2 = mul2(e[0], ex[c][0]), s3 = mul2(e[1], ex[c][1]);
#pragma unroll
                for (int k = 2; k < KP / 2; k += 2) { s2 = fma2(e[k], ex[c][k], s2); s3 = fma2(e[k + 1], ex[c][k + 1], s3); }
                s2 = add2(s2, s3);
                float lg;                                  // S >= exp(-60): never denormal, the flush-to-zero form is exact enough
                asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(lg) : "f"(s2.x + s2.y));
                if (live[c]) __stcs(yb[c], fmaf(lg, k_log, cadd[c] + mom));
                yb[c] += g.N;
            }
        }
    }
}

// ------------------------------------------------------------ input gradient
// acc[k] = sum_m Eo[m][k] * (dy*G)[m];  dx[tap k] = Ex[k] * acc[k]   (blocks must not overlap)
template <int KP, int C, bool SPATIAL1>
__global__ void __launch_bounds__(kT, 2) mex_dx_smallk(MexGeo g, const float* __restrict__ x, const float* __restrict__ eo,
                                                    const float* __restrict__ mo, const float* __restrict__ y, const float* __restrict__ dy,
                                                    float* __restrict__ dx, const int* __restrict__ flag) {
    __shared__ __align__(16) float eo_s[kMC * KP];
    __shared__ float mo_s[kMC];
    if (*flag) return;
    const long long P = (long long)g.B * g.rs;
    const int r = blockIdx.x % g.R;
    const long long j0 = (long long)(blockIdx.x / g.R) * (kT * C);
    const float eps = float(g.eps), cst = float(g.cst);
    constexpr int U = 4;                       // instances per load batch
    Column cols[C];
    float xv[C][KP], mxv[C], livef[C];
    long long sbase[C];                        // a position past the end reads position 0 and is masked by livef = 0
    float2 acc[C][KP / 2];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        cols[c] = column_of(g, r, j0 + c * kT + threadIdx.x, P, nullptr);
        mxv[c] = load_patch<KP, SPATIAL1>(g, x, cols[c], xv[c]);
        livef[c] = cols[c].base >= 0 ? 1.f : 0.f;
        sbase[c] = cols[c].base >= 0 ? cols[c].base : 0;
        if (cols[c].base < 0) mxv[c] = 0.f;
#pragma unroll
        for (int k = 0; k < KP / 2; ++k) acc[c][k] = make_float2(0.f, 0.f);
    }
    for (int m0 = 0; m0 < g.M; m0 += kMC) {
        __syncthreads();
        load_offsets_chunk<KP>(g, eo, mo, r, m0, eo_s, mo_s);
        __syncthreads();
        const int mend = min(kMC, g.M - m0);
        for (int mb = 0; mb < mend; mb += U) {
            // issue the whole batch of loads before the first use: U*C*2 independent 128-byte warp requests in flight
            float yv[U][C], gv[U][C];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool ok = mb + u < mend;
                const long long row = (long long)(m0 + mb + u) * g.N;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    yv[u][c] = (ok && livef[c] != 0.f) ? __ldcs(y + sbase[c] + row) : 0.f;     // a dead position must not read a stranger's y (0 * exp(big) = NaN)
                    gv[u][c] = ok ? __ldcs(dy + sbase[c] + row) : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int mm = min(mb + u, kMC - 1);
                float q[C];
#pragma unroll
                for (int c = 0; c < C; ++c) q[c] = livef[c] * gv[u][c] * fast_exp(eps * (mxv[c] + mo_s[mm] - yv[u][c]) + cst);
#pragma unroll
                for (int k4 = 0; k4 < KP / 4; ++k4) {
                    const float4 t = *reinterpret_cast<const float4*>(eo_s + mm * KP + k4 * 4);
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        acc[c][2 * k4] = fma2(make_float2(t.x, t.y), splat2(q[c]), acc[c][2 * k4]);
                        acc[c][2 * k4 + 1] = fma2(make_float2(t.z, t.w), splat2(q[c]), acc[c][2 * k4 + 1]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < C; ++c) {
        if (cols[c].base < 0) continue;
        const size_t sample = (size_t)cols[c].n * g.C * g.H * g.W;
#pragma unroll
        for (int k = 0; k < KP; ++k) {
            if (k >= g.K) continue;
            const Tap tp = tap_of<SPATIAL1>(g, k);
            const int cc = cols[c].c0 + tp.c, hh = cols[c].h0 + tp.h, ww = cols[c].w0 + tp.w;
            if (cc < 0 || cc >= g.C || hh < 0 || hh >= g.H || ww < 0 || ww >= g.W) continue;
            const float a = (k & 1) ? acc[c][k >> 1].y : acc[c][k >> 1].x;
            dx[sample + ((size_t)cc * g.H + hh) * g.W + ww] = fast_exp(eps * (xv[c][k] - mxv[c])) * a;
        }
    }
}

// ---------------------------------------------------------- offsets gradient
// Thread m of the CTA accumulates dO[m][0..K) over a slab of positions.  Tiles of 32 positions: y / dy are read
// coalesced along positions (lane = position), turned into Q = dy*G, transposed through shared memory so that
// thread m then reads Q[j][m] conflict free, and multiplied with the tile's Ex[j][0..K) (shared-memory broadcast).
constexpr int kPT = 32;          // positions per tile

template <int KP, bool SPATIAL1>
__global__ void __launch_bounds__(kT, 2) mex_doff_smallk(MexGeo g, const float* __restrict__ x, const float* __restrict__ mo,
                                                      const float* __restrict__ y, const float* __restrict__ dy,
                                                      float* __restrict__ part, int slabs, const int* __restrict__ flag) {
    constexpr int SUP = KP <= 16 ? 128 : 64;                 // positions whose Ex are prepared together
    __shared__ float q_s[kPT][kT + 1];
    __shared__ __align__(16) float ex_s[SUP][KP];
    __shared__ float mx_s[SUP];
    __shared__ long long base_s[SUP];
    __shared__ float mo_s[kT];
    if (*flag) return;
    const long long P = (long long)g.B * g.rs;
    const int mchunks = (g.M + kT - 1) / kT;
    int bid = blockIdx.x;
    const int mc = bid % mchunks; bid /= mchunks;
    const int r = bid % g.R;
    const int slab = bid / g.R;
    const int m0 = mc * kT;
    const long long sups = (P + SUP - 1) / SUP;
    const long long s_begin = sups * slab / slabs, s_end = sups * (slab + 1) / slabs;
    const float eps = float(g.eps), cst = float(g.cst);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int my_m = m0 + threadIdx.x;
    mo_s[threadIdx.x] = my_m < g.M ? mo[r * g.M + my_m] : 0.f;
    float2 acc[KP / 2];
#pragma unroll
    for (int k = 0; k < KP / 2; ++k) acc[k] = make_float2(0.f, 0.f);

    for (long long sup = s_begin; sup < s_end; ++sup) {
        __syncthreads();
        if (threadIdx.x < SUP) {
            const Column col = column_of(g, r, sup * SUP + threadIdx.x, P, nullptr);
            float v[KP];
            const float mxv = load_patch<KP, SPATIAL1>(g, x, col, v);
#pragma unroll
            for (int k = 0; k < KP; ++k) ex_s[threadIdx.x][k] = col.base >= 0 ? fast_exp(eps * (v[k] - mxv)) : 0.f;
            mx_s[threadIdx.x] = col.base >= 0 ? mxv : 0.f;
            base_s[threadIdx.x] = col.base;
        }
        __syncthreads();
#pragma unroll 1
        for (int sub = 0; sub < SUP / kPT; ++sub) {
            {
                const long long base = base_s[sub * kPT + lane];
                const bool live = base >= 0;
                const long long sb = live ? base : 0;
                const float mxv = mx_s[sub * kPT + lane];
                constexpr int U = 8;
#pragma unroll 1
                for (int i0 = 0; i0 < kT / 8; i0 += U) {             // this warp's 32 instances, U rows of loads in flight
                    float yv[U], gv[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int m = min(m0 + warp * (kT / 8) + i0 + u, g.M - 1);
                        yv[u] = __ldcs(y + sb + (long long)m * g.N);
                        gv[u] = __ldcs(dy + sb + (long long)m * g.N);
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int mm = warp * (kT / 8) + i0 + u;
                        const bool ok = live && m0 + mm < g.M;
                        q_s[lane][mm] = ok ? gv[u] * fast_exp(eps * (mxv + mo_s[mm] - yv[u]) + cst) : 0.f;
                    }
                }
            }
            __syncthreads();
#pragma unroll 4
            for (int j = 0; j < kPT; ++j) {
                const float2 q2 = splat2(q_s[j][threadIdx.x]);
#pragma unroll
                for (int k4 = 0; k4 < KP / 4; ++k4) {
                    const float4 t = *reinterpret_cast<const float4*>(&ex_s[sub * kPT + j][k4 * 4]);
                    acc[2 * k4] = fma2(make_float2(t.x, t.y), q2, acc[2 * k4]);
                    acc[2 * k4 + 1] = fma2(make_float2(t.z, t.w), q2, acc[2 * k4 + 1]);
                }
            }
            __syncthreads();
        }
    }
    if (my_m < g.M) {
        float* dst = part + (((size_t)slab * g.R + r) * g.M + my_m) * g.K;
#pragma unroll
        for (int k = 0; k < KP; ++k)
            if (k < g.K) dst[k] = (k & 1) ? acc[k >> 1].y : acc[k >> 1].x;
    }
}

}  // namespace

#define SMALLK_DISPATCH(KERNEL, C_, ...)                                                            \
    do {                                                                                            \
        const bool sp1 = g.bh == 1 && g.bw == 1;                                                    \
        if (g.K <= 8) { if (sp1) KERNEL<8, C_, true> __VA_ARGS__; else KERNEL<8, C_, false> __VA_ARGS__; }          \
        else if (g.K <= 16) { if (sp1) KERNEL<16, C_, true> __VA_ARGS__; else KERNEL<16, C_, false> __VA_ARGS__; }  \
        else { if (sp1) KERNEL<32, C_, true> __VA_ARGS__; else KERNEL<32, C_, false> __VA_ARGS__; }                 \
    } while (0)

cudaError_t launch_mex_fwd_smallk(const MexGeo& g, const float* x, const float* eo, const float* mo, float* y, const int* flag, cudaStream_t s) {
    const long long P = (long long)g.B * g.rs;
    if (g.K <= 16) {
        const long long blocks = ((P + kT * 4 - 1) / (kT * 4)) * g.R;
        if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
        SMALLK_DISPATCH(mex_fwd_smallk, 4, <<<int(blocks), kT, 0, s>>>(g, x, eo, mo, y, flag));
    } else {
        const long long blocks = ((P + kT * 2 - 1) / (kT * 2)) * g.R;
        if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
        SMALLK_DISPATCH(mex_fwd_smallk, 2, <<<int(blocks), kT, 0, s>>>(g, x, eo, mo, y, flag));
    }
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_dx_smallk(const MexGeo& g, const float* x, const float* eo, const float* mo, const float* y, const float* dy,
                                 float* dx, const int* flag, cudaStream_t s) {
    const long long P = (long long)g.B * g.rs;
    if (g.K <= 16) {
        const long long blocks = ((P + kT * 2 - 1) / (kT * 2)) * g.R;
        if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
        SMALLK_DISPATCH(mex_dx_smallk, 2, <<<int(blocks), kT, 0, s>>>(g, x, eo, mo, y, dy, dx, flag));
    } else {
        const long long blocks = ((P + kT - 1) / kT) * g.R;
        if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
        SMALLK_DISPATCH(mex_dx_smallk, 1, <<<int(blocks), kT, 0, s>>>(g, x, eo, mo, y, dy, dx, flag));
    }
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_doff_smallk(const MexGeo& g, const float* x, const float* mo, const float* y, const float* dy,
                                   float* part, int slabs, const int* flag, cudaStream_t s) {
    const int blocks = ((g.M + kT - 1) / kT) * g.R * slabs;
    const bool sp1 = g.bh == 1 && g.bw == 1;
#define DOFFK(KP) do { if (sp1) mex_doff_smallk<KP, true><<<blocks, kT, 0, s>>>(g, x, mo, y, dy, part, slabs, flag); \
                       else mex_doff_smallk<KP, false><<<blocks, kT, 0, s>>>(g, x, mo, y, dy, part, slabs, flag); } while (0)
    if (g.K <= 8) DOFFK(8); else if (g.K <= 16) DOFFK(16); else DOFFK(32);
#undef DOFFK
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
