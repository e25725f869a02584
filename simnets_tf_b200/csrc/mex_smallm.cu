// MEX for few instances over long patches (M <= 16, K >= 256; e.g. the 10-way head over a whole 512x4x4
// sample).  As a GEMM this shape is a sliver: 10 x 8192 x batch.  Tiling it leaves most of the machine
// idle, so here one CTA owns one output position: its 256 threads stride over the K taps (contiguous in
// memory for such blocks, hence coalesced), the patch maximum is a block reduction, and the M sums are
// reduced with warp shuffles.  Same factorised arithmetic and same safety flag as mex_tiled.cu.
#include "mex_common.cuh"

namespace simnets {

namespace {

constexpr int kT = 256;
constexpr int kMaxM = 16;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// A block that spans whole rows and whole planes (the head over a complete 512 x 4 x 4 sample) is one contiguous run of
// K floats: tap k sits at c0 * H * W + k, no decoding (two divisions and two modulos per tap otherwise) and no bounds test.
__device__ __forceinline__ bool patches_contiguous(const MexGeo& g) {
    return g.bw == g.W && g.pw == 0 && g.bh == g.H && g.ph == 0 && g.pc == 0 && (g.Co - 1) * g.sc + g.bc <= g.C;
}
template <bool SPATIAL1>
__device__ __forceinline__ float tap_value(const MexGeo& g, const float* __restrict__ xs, const Column& col, int k, float oob, bool contig) {
    if (contig) return __ldg(xs + (size_t)col.c0 * g.H * g.W + k);
    return patch_value<SPATIAL1>(g, xs, col.c0, col.h0, col.w0, k, oob);
}

// max (eps > 0) or min over the K taps of one patch, over the whole block; NaN taps are ignored
template <bool SPATIAL1>
__device__ __forceinline__ float block_patch_extreme(const MexGeo& g, const float* __restrict__ xs, const Column& col, float oob, float* red) {
    const bool up = g.eps > 0, contig = patches_contiguous(g);
    float v = up ? -CUDART_INF_F : CUDART_INF_F;
    for (int k = threadIdx.x; k < g.K; k += kT) {
        const float t = tap_value<SPATIAL1>(g, xs, col, k, oob, contig);
        v = up ? fmaxf(v, t) : fminf(v, t);
    }
    v = up ? warp_max(v) : warp_min(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < kT / 32; ++w) r = up ? fmaxf(r, red[w]) : fminf(r, red[w]);
    __syncthreads();
    return r;
}

template <bool SPATIAL1>
__global__ void __launch_bounds__(kT) mex_colmax_wide(MexGeo g, const float* __restrict__ x, float* __restrict__ mx, const int* __restrict__ flag) {
    __shared__ float red[kT / 32];
    if (*flag) return;
    const long long idx = blockIdx.x;
    const int pos = int(idx % g.N), n = int(idx / g.N);
    Column col;
    col.c0 = (pos / (g.Wo * g.Ho)) * g.sc - g.pc;
    col.h0 = ((pos / g.Wo) % g.Ho) * g.sh - g.ph;
    col.w0 = (pos % g.Wo) * g.sw - g.pw;
    const float v = block_patch_extreme<SPATIAL1>(g, x + (size_t)n * g.C * g.H * g.W, col, float(g.oob), red);
    if (threadIdx.x == 0) mx[idx] = v;
}

template <bool SPATIAL1>
__global__ void __launch_bounds__(kT) mex_fwd_smallm(MexGeo g, const float* __restrict__ x, const float* __restrict__ eot,
                                                     const float* __restrict__ mo, float* __restrict__ y, const int* __restrict__ flag) {
    __shared__ float red[kT / 32];
    __shared__ float racc[kT / 32][kMaxM];
    if (*flag) return;
    const long long P = (long long)g.B * g.rs;
    const int r = blockIdx.x % g.R;
    const Column col = column_of(g, r, blockIdx.x / g.R, P, nullptr);
    if (col.base < 0) return;
    const float* xs = x + (size_t)col.n * g.C * g.H * g.W;
    const float eps = float(g.eps), oob = float(g.oob);
    const float mxv = block_patch_extreme<SPATIAL1>(g, xs, col, oob, red);
    const int ldm = pad4(g.M);
    const bool contig = patches_contiguous(g);
    float acc[kMaxM];
#pragma unroll
    for (int m = 0; m < kMaxM; ++m) acc[m] = 0.f;
    for (int k = threadIdx.x; k < g.K; k += kT) {
        const float e = fast_exp(eps * (tap_value<SPATIAL1>(g, xs, col, k, oob, contig) - mxv));
        const float4* row = reinterpret_cast<const float4*>(eot + ((size_t)r * g.K + k) * ldm);
#pragma unroll
        for (int q = 0; q < kMaxM / 4; ++q)
            if (q * 4 < ldm) {
                const float4 v = __ldg(row + q);     // columns past M hold stale workspace bytes; they are never stored
                acc[q * 4 + 0] = fmaf(e, v.x, acc[q * 4 + 0]); acc[q * 4 + 1] = fmaf(e, v.y, acc[q * 4 + 1]);
                acc[q * 4 + 2] = fmaf(e, v.z, acc[q * 4 + 2]); acc[q * 4 + 3] = fmaf(e, v.w, acc[q * 4 + 3]);
            }
    }
#pragma unroll
    for (int m = 0; m < kMaxM; ++m) {
        const float v = warp_sum(acc[m]);
        if ((threadIdx.x & 31) == 0) racc[threadIdx.x >> 5][m] = v;
    }
    __syncthreads();
    if (threadIdx.x < g.M) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kT / 32; ++w) s += racc[w][threadIdx.x];
        y[col.base + (long long)threadIdx.x * g.N] = mxv + mo[r * g.M + threadIdx.x] + (fast_log(s) + float(g.cst)) / eps;
    }
}

template <bool SPATIAL1>
__global__ void __launch_bounds__(kT) mex_dx_smallm(MexGeo g, const float* __restrict__ x, const float* __restrict__ eo,
                                                    const float* __restrict__ mo, const float* __restrict__ y, const float* __restrict__ dy,
                                                    float* __restrict__ dx, const int* __restrict__ flag) {
    __shared__ float red[kT / 32];
    __shared__ float Q[kMaxM];
    if (*flag) return;
    const long long P = (long long)g.B * g.rs;
    const int r = blockIdx.x % g.R;
    const Column col = column_of(g, r, blockIdx.x / g.R, P, nullptr);
    if (col.base < 0) return;
    const size_t sample = (size_t)col.n * g.C * g.H * g.W;
    const float eps = float(g.eps), oob = float(g.oob);
    const float mxv = block_patch_extreme<SPATIAL1>(g, x + sample, col, oob, red);
    if (threadIdx.x < kMaxM) {
        const int m = threadIdx.x;
        Q[m] = m < g.M ? dy[col.base + (long long)m * g.N] * fast_exp(eps * (mxv + mo[r * g.M + m] - y[col.base + (long long)m * g.N]) + float(g.cst)) : 0.f;
    }
    __syncthreads();
    const int ldk = pad4(g.K);
    const float* eor = eo + (size_t)r * g.M * ldk;
    const bool contig = patches_contiguous(g);
    for (int k = threadIdx.x; k < g.K; k += kT) {
        size_t a;
        if (contig) {
            a = sample + (size_t)col.c0 * g.H * g.W + k;
        } else {
            const Tap tp = tap_of<SPATIAL1>(g, k);
            const int cc = col.c0 + tp.c, hh = col.h0 + tp.h, ww = col.w0 + tp.w;
            if (cc < 0 || cc >= g.C || hh < 0 || hh >= g.H || ww < 0 || ww >= g.W) continue;
            a = sample + ((size_t)cc * g.H + hh) * g.W + ww;
        }
        float s = 0.f;
        for (int m = 0; m < g.M; ++m) s = fmaf(__ldg(eor + (size_t)m * ldk + k), Q[m], s);
        dx[a] = fast_exp(eps * (x[a] - mxv)) * s;
    }
}

constexpr int kGroup = 16;     // positions whose dy*G values are staged together

template <bool SPATIAL1>
__global__ void __launch_bounds__(kT) mex_doff_smallm(MexGeo g, const float* __restrict__ x, const float* __restrict__ mo,
                                                      const float* __restrict__ mx, const float* __restrict__ y, const float* __restrict__ dy,
                                                      float* __restrict__ part, int splits, const int* __restrict__ flag) {
    __shared__ Column cols[kGroup];
    __shared__ float Qs[kGroup][kMaxM];
    if (*flag) return;
    const long long P = (long long)g.B * g.rs;
    const int ktiles = (g.K + kT - 1) / kT;
    int bid = blockIdx.x;
    const int kt = bid % ktiles; bid /= ktiles;
    const int r = bid % g.R;
    const int split = bid / g.R;
    const int k = kt * kT + threadIdx.x;
    const long long groups = (P + kGroup - 1) / kGroup;
    const long long g_begin = groups * split / splits, g_end = groups * (split + 1) / splits;
    const float eps = float(g.eps), oob = float(g.oob), cst = float(g.cst);
    const bool contig = patches_contiguous(g);
    float acc[kMaxM];
#pragma unroll
    for (int m = 0; m < kMaxM; ++m) acc[m] = 0.f;
    for (long long gi = g_begin; gi < g_end; ++gi) {
        if (threadIdx.x < kGroup) cols[threadIdx.x] = column_of(g, r, gi * kGroup + threadIdx.x, P, mx);
        __syncthreads();
        {
            const int p = threadIdx.x / kMaxM, m = threadIdx.x % kMaxM;      // 256 threads = 16 positions x 16 instances
            const Column& c = cols[p];
            float q = 0.f;
            if (c.base >= 0 && m < g.M)
                q = dy[c.base + (long long)m * g.N] * fast_exp(eps * (c.mx + mo[r * g.M + m] - y[c.base + (long long)m * g.N]) + cst);
            Qs[p][m] = q;
        }
        __syncthreads();
        if (k < g.K) {
#pragma unroll 4
            for (int p = 0; p < kGroup; ++p) {
                const Column& c = cols[p];
                if (c.base < 0) continue;
                const float v = tap_value<SPATIAL1>(g, x + (size_t)c.n * g.C * g.H * g.W, c, k, oob, contig);
                const float e = fast_exp(eps * (v - c.mx));
#pragma unroll
                for (int m = 0; m < kMaxM; ++m) acc[m] = fmaf(Qs[p][m], e, acc[m]);
            }
        }
        __syncthreads();
    }
    if (k < g.K) {
        float* dst = part + ((size_t)split * g.R + r) * g.M * g.K;
#pragma unroll
        for (int m = 0; m < kMaxM; ++m)
            if (m < g.M) dst[(size_t)m * g.K + k] = acc[m];
    }
}

}  // namespace

cudaError_t launch_mex_colmax_wide(const MexGeo& g, const float* x, float* mx, const int* flag, cudaStream_t s) {
    const long long total = (long long)g.B * g.N;
    if (total > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    if (g.bh == 1 && g.bw == 1) mex_colmax_wide<true><<<int(total), kT, 0, s>>>(g, x, mx, flag);
    else mex_colmax_wide<false><<<int(total), kT, 0, s>>>(g, x, mx, flag);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_fwd_smallm(const MexGeo& g, const float* x, const float* eot, const float* mo, float* y, const int* flag, cudaStream_t s) {
    const long long blocks = (long long)g.B * g.rs * g.R;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    if (g.bh == 1 && g.bw == 1) mex_fwd_smallm<true><<<int(blocks), kT, 0, s>>>(g, x, eot, mo, y, flag);
    else mex_fwd_smallm<false><<<int(blocks), kT, 0, s>>>(g, x, eot, mo, y, flag);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_dx_smallm(const MexGeo& g, const float* x, const float* eo, const float* mo, const float* y, const float* dy,
                                 float* dx, const int* flag, cudaStream_t s) {
    const long long blocks = (long long)g.B * g.rs * g.R;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    if (g.bh == 1 && g.bw == 1) mex_dx_smallm<true><<<int(blocks), kT, 0, s>>>(g, x, eo, mo, y, dy, dx, flag);
    else mex_dx_smallm<false><<<int(blocks), kT, 0, s>>>(g, x, eo, mo, y, dy, dx, flag);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_doff_smallm(const MexGeo& g, const float* x, const float* mo, const float* mx, const float* y, const float* dy,
                                   float* part, int splits, const int* flag, cudaStream_t s) {
    const int blocks = ((g.K + kT - 1) / kT) * g.R * splits;
    if (g.bh == 1 && g.bw == 1) mex_doff_smallm<true><<<blocks, kT, 0, s>>>(g, x, mo, mx, y, dy, part, splits, flag);
    else mex_doff_smallm<false><<<blocks, kT, 0, s>>>(g, x, mo, mx, y, dy, part, splits, flag);
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
