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
__device__ __forceinline__ float ex2_approx(float v) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v)); return r; }
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


// ---- contiguous patches: the classifier head over whole samples -----------------------------------------------------
// When every patch is one contiguous run of K floats (patches_contiguous) and there is a single offsets region, the op
// is a sliver GEMM [positions x K] x [K x M <= 16] whose cost is reading x.  One CTA per position (above) re-reads the
// whole offsets table (M K floats) for every position; here a CTA takes several positions, so that the table is read
// once per group, and the backward pass produces the input gradient and the offsets-gradient partial sums from ONE read
// of x.  The forward kernel stores the per-position maxima, which primes the workspace for the gradients.
constexpr int kHeadPB = 8;         // positions per CTA in the forward pass
constexpr int kHeadSlices = 8;     // tap slices: a CTA takes one slice of the patches of its positions

// Forward: CTA = (group of up to 8 positions, slice of the taps).  Each CTA stabilises with the maximum of ITS slice (the
// slice of x is 32 KiB at most and stays in L1 for the second pass, so x is read from memory once and no separate maximum
// pass exists), leaves per-position partial sums S_s[m] and maxima mx_s in the workspace, and the CTA that finishes a
// group last combines them: mx = max_s mx_s, S[m] = sum_s S_s[m] * exp(eps (mx_s - mx)) -- the same value as with one
// global maximum, up to rounding.  It then writes y and the per-position maxima (which prime the gradients).
template <int MP>
__global__ void __launch_bounds__(kT) mex_fwd_head(MexGeo g, int pb, int slices, const float* __restrict__ x, const float* __restrict__ eot,
                                                   const float* __restrict__ mo, float* __restrict__ mx, float* __restrict__ y,
                                                   float* __restrict__ partial, int* __restrict__ tickets, const int* __restrict__ flag) {
    __shared__ float red[kT / 32][kHeadPB];
    __shared__ float racc[kT / 32][kHeadPB][MP];
    __shared__ float mxs[kHeadPB];
    __shared__ int last;
    if (*flag) return;
    const long long P = (long long)g.B * g.N;                      // positions (one region)
    const int group = blockIdx.x / slices, slice = blockIdx.x % slices;
    const long long p0 = (long long)group * pb;
    const int np = int(min((long long)pb, P - p0));
    const int K = g.K, M = g.M, ldm = pad4(g.M);
    const int kper = ((K + slices - 1) / slices + 3) & ~3, k_begin = slice * kper, k_end = min(K, k_begin + kper);
    const bool up = g.eps > 0;
    const float a = float(g.eps) * 1.4426950408889634f;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // position p of the group: sample n = p / N, patch = channels [c0, c0 + bc) of that sample, contiguous
    const float* xp[kHeadPB];
#pragma unroll
    for (int p = 0; p < kHeadPB; ++p) {
        const long long q = p0 + (p < np ? p : 0);
        const int n = int(q / g.N), pos = int(q % g.N);
        xp[p] = x + ((size_t)n * g.C + (size_t)(pos / (g.Wo * g.Ho)) * g.sc) * g.H * g.W;
    }
    // pass 1: maxima of the slice (NaN taps ignored, as fmaxf / fminf do)
    float v[kHeadPB];
#pragma unroll
    for (int p = 0; p < kHeadPB; ++p) v[p] = up ? -CUDART_INF_F : CUDART_INF_F;
    for (int k = k_begin + threadIdx.x; k < k_end; k += kT) {
#pragma unroll
        for (int p = 0; p < kHeadPB; ++p) {
            if (p >= np) break;
            const float t = __ldg(xp[p] + k);
            v[p] = up ? fmaxf(v[p], t) : fminf(v[p], t);
        }
    }
#pragma unroll
    for (int p = 0; p < kHeadPB; ++p) {
        v[p] = up ? warp_max(v[p]) : warp_min(v[p]);
        if (lane == 0) red[warp][p] = v[p];
    }
    __syncthreads();
    if (threadIdx.x < kHeadPB) {
        float r = red[0][threadIdx.x];
        for (int w = 1; w < kT / 32; ++w) r = up ? fmaxf(r, red[w][threadIdx.x]) : fminf(r, red[w][threadIdx.x]);
        mxs[threadIdx.x] = r;
    }
    __syncthreads();
    float mxv[kHeadPB];
#pragma unroll
    for (int p = 0; p < kHeadPB; ++p) mxv[p] = mxs[p];
    // pass 2 (x comes from L1 now): sums over the slice's taps for every instance
    float acc[kHeadPB][MP];
#pragma unroll
    for (int p = 0; p < kHeadPB; ++p)
#pragma unroll
        for (int m = 0; m < MP; ++m) acc[p][m] = 0.f;
    for (int k = k_begin + threadIdx.x; k < k_end; k += kT) {
        float eo[MP];
        const float4* row = reinterpret_cast<const float4*>(eot + (size_t)k * ldm);
#pragma unroll
        for (int q = 0; q < MP / 4; ++q) {
            const float4 t = __ldg(row + q);                      // MP = ldm; columns past M hold stale bytes and are never stored
            eo[q * 4] = t.x; eo[q * 4 + 1] = t.y; eo[q * 4 + 2] = t.z; eo[q * 4 + 3] = t.w;
        }
#pragma unroll
        for (int p = 0; p < kHeadPB; ++p) {
            if (p >= np) break;
            const float e = ex2_approx(a * (__ldg(xp[p] + k) - mxv[p]));      // (an empty slice never gets here: its -inf maximum is unused)
#pragma unroll
            for (int m = 0; m < MP; ++m) acc[p][m] = fmaf(e, eo[m], acc[p][m]);
        }
    }
#pragma unroll
    for (int p = 0; p < kHeadPB; ++p)
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            const float t = warp_sum(acc[p][m]);
            if (lane == 0) racc[warp][p][m] = t;
        }
    __syncthreads();
    // this slice's partial sums and maxima: partial[group][slice][p < pb][MP + 1]
    float* mine = partial + ((size_t)group * slices + slice) * pb * (MP + 1);
    for (int i = threadIdx.x; i < pb * (MP + 1); i += kT) {
        const int p = i / (MP + 1), m = i % (MP + 1);
        float sum = mxs[p];
        if (m < MP) {
            sum = 0.f;
#pragma unroll
            for (int w = 0; w < kT / 32; ++w) sum += racc[w][p][m];
        }
        mine[i] = sum;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(tickets + group, 1) == slices - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    // the last CTA of the group: combine the slices in slice order (deterministic)
    const float* all = partial + (size_t)group * slices * pb * (MP + 1);
    for (int i = threadIdx.x; i < np * MP; i += kT) {
        const int p = i / MP, m = i % MP;
        float gm = up ? -CUDART_INF_F : CUDART_INF_F;
        for (int s2 = 0; s2 < slices; ++s2) {
            const float t = __ldcg(all + ((size_t)s2 * pb + p) * (MP + 1) + MP);
            gm = up ? fmaxf(gm, t) : fminf(gm, t);
        }
        float sum = 0.f;
        for (int s2 = 0; s2 < slices; ++s2) {
            const float* ps = all + ((size_t)s2 * pb + p) * (MP + 1);
            const float ms = __ldcg(ps + MP);
            const float part_sum = __ldcg(ps + m);
            if (part_sum != 0.f) sum = fmaf(part_sum, ex2_approx(a * (ms - gm)), sum);      // (skips empty slices, whose maximum is infinite)
        }
        const long long q = p0 + p;
        if (m == 0) mx[q] = gm;
        if (m < M) {
            const int n = int(q / g.N), pos = int(q % g.N);
            y[((long long)n * M + m) * g.N + pos] = gm + mo[m] + (fast_log(sum) + float(g.cst)) / float(g.eps);
        }
    }
}

// Forward for aligned patches (K and the patch starts multiples of four floats): CTA = (16 positions, slice of 1024 taps),
// warp = two positions.  A lane owns taps 4 (lane + 32 i) .. + 3, i < 8, of both positions: sixteen 16-byte loads per
// thread are issued before anything waits (64 KiB of x in flight per CTA), the slice of the offsets table is staged in
// shared memory meanwhile (instance-major, so that a lane's 16-byte reads are conflict free), the slice's maximum is a
// warp reduction, and the sums of a position never leave its warp.  Partial sums, ticket and the combining CTA are the
// ones of mex_fwd_head.  x is read from memory exactly once.
constexpr int kWidePB = 16, kWideSlice = 1024;

template <int MP>
__global__ void __launch_bounds__(kT, 2) mex_fwd_head_wide(MexGeo g, int slices, const float* __restrict__ x, const float* __restrict__ eo,
                                                           const float* __restrict__ mo, float* __restrict__ mx, float* __restrict__ y,
                                                           float* __restrict__ partial, int* __restrict__ tickets, const int* __restrict__ flag) {
    extern __shared__ __align__(16) float seo[];                   // [MP][kWideSlice]
    __shared__ int last;
    if (*flag) return;
    const long long P = (long long)g.B * g.N;
    const int group = blockIdx.x / slices, slice = blockIdx.x % slices;
    const long long p0 = (long long)group * kWidePB;
    const int np = int(min((long long)kWidePB, P - p0));
    const int K = g.K, M = g.M, ldk = pad4(g.K);
    const int k_begin = slice * kWideSlice, klen = min(kWideSlice, K - k_begin);
    const bool up = g.eps > 0;
    const float a = float(g.eps) * 1.4426950408889634f;
    const float fill = up ? -CUDART_INF_F : CUDART_INF_F;          // absent taps: never the extremum, exp gives 0
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float4 xv[2][8];
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
        const int p = 2 * warp + pp;
        const long long q = p0 + (p < np ? p : 0);
        const int n = int(q / g.N), pos = int(q % g.N);
        const float4* xp = reinterpret_cast<const float4*>(x + ((size_t)n * g.C + (size_t)pos * g.sc) * g.H * g.W + k_begin);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int t = 4 * (lane + 32 * i);
            xv[pp][i] = (p < np && t < klen) ? __ldcs(xp + lane + 32 * i) : make_float4(fill, fill, fill, fill);
        }
    }
    // the slice of exp(eps (offsets - mo)): rows past M and taps past the slice hold zeros
    for (int i = threadIdx.x; i < MP * (kWideSlice / 4); i += kT) {
        const int m = i / (kWideSlice / 4), t = 4 * (i % (kWideSlice / 4));
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < M && t < klen) v = __ldg(reinterpret_cast<const float4*>(eo + (size_t)m * ldk + k_begin + t));
        reinterpret_cast<float4*>(seo)[i] = v;
    }
    float mxw[2];
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
        float v = fill;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 t = xv[pp][i];
            v = up ? fmaxf(fmaxf(v, t.x), fmaxf(fmaxf(t.y, t.z), t.w)) : fminf(fminf(v, t.x), fminf(fminf(t.y, t.z), t.w));
        }
        mxw[pp] = up ? warp_max(v) : warp_min(v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float4& t = xv[pp][i];
            t.x = ex2_approx(a * (t.x - mxw[pp])); t.y = ex2_approx(a * (t.y - mxw[pp]));
            t.z = ex2_approx(a * (t.z - mxw[pp])); t.w = ex2_approx(a * (t.w - mxw[pp]));
        }
    }
    __syncthreads();
    float acc[2][MP];
#pragma unroll
    for (int m = 0; m < MP; ++m) acc[0][m] = acc[1][m] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 e0 = xv[0][i], e1 = xv[1][i];
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            const float4 w = reinterpret_cast<const float4*>(seo + m * kWideSlice)[lane + 32 * i];
            acc[0][m] = fmaf(e0.x, w.x, fmaf(e0.y, w.y, fmaf(e0.z, w.z, fmaf(e0.w, w.w, acc[0][m]))));
            acc[1][m] = fmaf(e1.x, w.x, fmaf(e1.y, w.y, fmaf(e1.z, w.z, fmaf(e1.w, w.w, acc[1][m]))));
        }
    }
    // this slice's partial sums and maxima: partial[group][slice][p < 16][MP + 1]
    float* mine = partial + ((size_t)group * slices + slice) * kWidePB * (MP + 1);
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
        float keep = mxw[pp];                                       // lane MP keeps the maximum, lane m < MP the sum of instance m
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            const float t = warp_sum(acc[pp][m]);
            if (lane == m) keep = t;
        }
        if (lane <= MP) mine[(2 * warp + pp) * (MP + 1) + lane] = keep;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(tickets + group, 1) == slices - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    // the last CTA of the group: combine the slices in slice order (deterministic)
    const float* all = partial + (size_t)group * slices * kWidePB * (MP + 1);
    for (int i = threadIdx.x; i < np * MP; i += kT) {
        const int p = i / MP, m = i % MP;
        float gm = fill;
        for (int s2 = 0; s2 < slices; ++s2) {
            const float t = __ldcg(all + ((size_t)s2 * kWidePB + p) * (MP + 1) + MP);
            gm = up ? fmaxf(gm, t) : fminf(gm, t);
        }
        float sum = 0.f;
        for (int s2 = 0; s2 < slices; ++s2) {
            const float* ps = all + ((size_t)s2 * kWidePB + p) * (MP + 1);
            const float ms = __ldcg(ps + MP);
            const float part_sum = __ldcg(ps + m);
            if (part_sum != 0.f) sum = fmaf(part_sum, ex2_approx(a * (ms - gm)), sum);
        }
        const long long q = p0 + p;
        if (m == 0) mx[q] = gm;
        if (m < M) {
            const int n = int(q / g.N), pos = int(q % g.N);
            y[((long long)n * M + m) * g.N + pos] = gm + mo[m] + (fast_log(sum) + float(g.cst)) / float(g.eps);
        }
    }
}

// Backward: CTA = (tile of kT * KPT taps, split of the positions).  Per position: Q[m] = dy * exp(eps (mx + mo - y) + c);
// per tap of the tile: Ex once, then dx = Ex * sum_m Eo[m, k] Q[m] and U[m, k] += Q[m] * Ex.
constexpr int kHeadKPT = 4;        // taps per thread

template <int MP, bool DX, bool DOFF>
__global__ void __launch_bounds__(kT) mex_bwd_head(MexGeo g, const float* __restrict__ x, const float* __restrict__ eo,
                                                   const float* __restrict__ mo, const float* __restrict__ mx,
                                                   const float* __restrict__ y, const float* __restrict__ dy,
                                                   float* __restrict__ dx, float* __restrict__ part, int splits,
                                                   const int* __restrict__ flag) {
    constexpr int GP = 8;                                           // positions staged together
    __shared__ float Qs[2][GP][kMaxM + 1];                          // Q of a group's positions and, in the last column, their maxima
    if (*flag) return;
    const long long P = (long long)g.B * g.N;
    const int K = g.K, M = g.M, ldk = pad4(g.K);
    const int ktiles = (K + kT * kHeadKPT - 1) / (kT * kHeadKPT);
    const int kt = blockIdx.x % ktiles, split = blockIdx.x / ktiles;
    const long long p_begin = P * split / splits, p_end = P * (split + 1) / splits;
    const float a = float(g.eps) * 1.4426950408889634f, c2 = float(g.cst) * 1.4426950408889634f;
    const int kbase = kt * kT * kHeadKPT + threadIdx.x;            // this thread's taps: kbase + i * kT
    const size_t hwc = (size_t)g.H * g.W;
    float eor[MP][kHeadKPT];                                        // Eo of this thread's taps
#pragma unroll
    for (int m = 0; m < MP; ++m)
#pragma unroll
        for (int i = 0; i < kHeadKPT; ++i)
            eor[m][i] = (DX && m < M && kbase + i * kT < K) ? __ldg(eo + (size_t)m * ldk + kbase + i * kT) : 0.f;
    float acc[MP][kHeadKPT];
#pragma unroll
    for (int m = 0; m < MP; ++m)
#pragma unroll
        for (int i = 0; i < kHeadKPT; ++i) acc[m][i] = 0.f;
    int buf = 0;
    for (long long q0 = p_begin; q0 < p_end; q0 += GP, buf ^= 1) {
        // the group's Q values: GP x 16 threads, one (position, instance) each; all their loads are in flight together
        if (threadIdx.x < GP * kMaxM) {
            const int p = threadIdx.x / kMaxM, m = threadIdx.x % kMaxM;
            const long long q = q0 + p;
            float qv = 0.f;
            if (q < p_end && m < M) {
                const int n = int(q / g.N), pos = int(q % g.N);
                const long long o = ((long long)n * M + m) * g.N + pos;
                qv = __ldg(dy + o) * ex2_approx(fmaf(a, (__ldg(mx + q) - __ldg(y + o)) + mo[m], c2));
            }
            Qs[buf][p][m] = qv;
            if (m == 0) Qs[buf][p][kMaxM] = q < p_end ? __ldg(mx + q) : 0.f;
        }
        // x of the whole group goes in flight before the barrier
        float xv[GP][kHeadKPT];
        size_t base[GP];
#pragma unroll
        for (int p = 0; p < GP; ++p) {
            const long long q = q0 + p < p_end ? q0 + p : p_end - 1;
            const int n = int(q / g.N), pos = int(q % g.N);
            base[p] = ((size_t)n * g.C + (size_t)(pos / (g.Wo * g.Ho)) * g.sc) * hwc;
#pragma unroll
            for (int i = 0; i < kHeadKPT; ++i) xv[p][i] = kbase + i * kT < K ? __ldg(x + base[p] + kbase + i * kT) : 0.f;
        }
        __syncthreads();                                           // (double buffered: one barrier per group)
#pragma unroll
        for (int p = 0; p < GP; ++p) {
            if (q0 + p >= p_end) break;
            const float mxv = Qs[buf][p][kMaxM];
            float e[kHeadKPT];
#pragma unroll
            for (int i = 0; i < kHeadKPT; ++i) e[i] = kbase + i * kT < K ? ex2_approx(a * (xv[p][i] - mxv)) : 0.f;
            float qm[MP];
#pragma unroll
            for (int m = 0; m < MP; ++m) qm[m] = Qs[buf][p][m];
            if (DX) {
#pragma unroll
                for (int i = 0; i < kHeadKPT; ++i) {
                    float s = 0.f;
#pragma unroll
                    for (int m = 0; m < MP; ++m) s = fmaf(eor[m][i], qm[m], s);
                    if (kbase + i * kT < K) dx[base[p] + kbase + i * kT] = e[i] * s;
                }
            }
            if (DOFF) {
#pragma unroll
                for (int m = 0; m < MP; ++m)
#pragma unroll
                    for (int i = 0; i < kHeadKPT; ++i) acc[m][i] = fmaf(qm[m], e[i], acc[m][i]);
            }
        }
    }
    if (DOFF) {
        float* dst = part + (size_t)split * M * K;
#pragma unroll
        for (int m = 0; m < MP; ++m)
            if (m < M)
#pragma unroll
                for (int i = 0; i < kHeadKPT; ++i)
                    if (kbase + i * kT < K) dst[(size_t)m * K + kbase + i * kT] = acc[m][i];
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

// ---- the contiguous-patch head
bool mex_head_shape(const MexGeo& g) {
    return smallm_shape(g) && g.R == 1 && g.bw == g.W && g.pw == 0 && g.bh == g.H && g.ph == 0 && g.pc == 0 &&
           (g.Co - 1) * g.sc + g.bc <= g.C && g.Ho == 1 && g.Wo == 1;
}

int mex_head_splits(const MexGeo& g) {
    const int ktiles = (g.K + kT * kHeadKPT - 1) / (kT * kHeadKPT);
    const long long P = (long long)g.B * g.N;
    long long s = (2LL * device_sm_count() + ktiles - 1) / ktiles;
    if (s > P) s = P;
    if (s < 1) s = 1;
    return int(s);
}

// patches and patch starts on 16-byte boundaries (given a 16-byte aligned x)
static bool head_wide_shape(const MexGeo& g, const float* x) {
    const long long hw = (long long)g.H * g.W;
    return g.K % 4 == 0 && g.K >= kWideSlice / 2 && (g.C * hw) % 4 == 0 && (g.sc * hw) % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
}
static int head_slices_max(const MexGeo& g) { return std::max(kHeadSlices, (g.K + kWideSlice - 1) / kWideSlice); }

// scratch of the forward head kernels behind `part`-sized storage: partial sums then tickets
size_t mex_head_fwd_scratch_floats(const MexGeo& g) {
    const long long P = (long long)g.B * g.N;
    return size_t(P + kWidePB) * head_slices_max(g) * (pad4(g.M) + 1) + size_t(P + 1);       // groups of at least one position each
}

cudaError_t launch_mex_fwd_head(const MexGeo& g, const float* x, const float* eo, const float* eot, const float* mo, float* mx, float* y,
                                float* scratch, const int* flag, cudaStream_t s) {
    const long long P = (long long)g.B * g.N;
    if (head_wide_shape(g, x)) {
        const long long groups = (P + kWidePB - 1) / kWidePB;
        const int slices = (g.K + kWideSlice - 1) / kWideSlice;
        if (groups * slices > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
        float* partial = scratch;
        int* tickets = reinterpret_cast<int*>(scratch + size_t(P + kWidePB) * head_slices_max(g) * (pad4(g.M) + 1));
        cudaError_t e = cudaMemsetAsync(tickets, 0, sizeof(int) * size_t(groups), s);
        if (e != cudaSuccess) return e;
        const int blocks = int(groups * slices);
#define HEAD_WIDE(MP)                                                                                                   \
        do {                                                                                                            \
            static bool attr_done = false;                                                                              \
            constexpr int smem = MP * kWideSlice * 4;                                                                   \
            if (!attr_done) {                                                                                           \
                e = cudaFuncSetAttribute(mex_fwd_head_wide<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);     \
                if (e != cudaSuccess) return e;                                                                         \
                attr_done = true;                                                                                       \
            }                                                                                                           \
            mex_fwd_head_wide<MP><<<blocks, kT, smem, s>>>(g, slices, x, eo, mo, mx, y, partial, tickets, flag);        \
        } while (0)
        switch (pad4(g.M)) {
        case 4: HEAD_WIDE(4); break;
        case 8: HEAD_WIDE(8); break;
        case 12: HEAD_WIDE(12); break;
        default: HEAD_WIDE(16); break;
        }
#undef HEAD_WIDE
        count_launch();
        return cudaGetLastError();
    }
    // Large batches: 8 positions per CTA over whole patches (measured fastest: the offsets table is read once per 8
    // positions and nothing is combined).  Small batches, where that leaves most SMs idle: smaller groups and tap slices.
    int pb = kHeadPB;
    while (pb > 2 && ((P + pb - 1) / pb) * kHeadSlices < device_sm_count()) pb >>= 1;
    const long long groups = (P + pb - 1) / pb;
    const int slices = (g.K >= kHeadSlices * 64 && 2 * groups < device_sm_count()) ? kHeadSlices : 1;
    if (groups * slices > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    float* partial = scratch;
    int* tickets = reinterpret_cast<int*>(scratch + size_t(P + kWidePB) * head_slices_max(g) * (pad4(g.M) + 1));
    cudaError_t e = cudaMemsetAsync(tickets, 0, sizeof(int) * size_t(groups), s);
    if (e != cudaSuccess) return e;
    const int blocks = int(groups * slices);
    switch (pad4(g.M)) {
    case 4: mex_fwd_head<4><<<blocks, kT, 0, s>>>(g, pb, slices, x, eot, mo, mx, y, partial, tickets, flag); break;
    case 8: mex_fwd_head<8><<<blocks, kT, 0, s>>>(g, pb, slices, x, eot, mo, mx, y, partial, tickets, flag); break;
    case 12: mex_fwd_head<12><<<blocks, kT, 0, s>>>(g, pb, slices, x, eot, mo, mx, y, partial, tickets, flag); break;
    default: mex_fwd_head<16><<<blocks, kT, 0, s>>>(g, pb, slices, x, eot, mo, mx, y, partial, tickets, flag); break;
    }
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_bwd_head(const MexGeo& g, bool want_dx, bool want_doff, const float* x, const float* eo, const float* mo,
                                const float* mx, const float* y, const float* dy, float* dx, float* part, int splits,
                                const int* flag, cudaStream_t s) {
    const int ktiles = (g.K + kT * kHeadKPT - 1) / (kT * kHeadKPT);
    const int blocks = ktiles * splits;
#define HEAD_BWD(MP)                                                                                                          \
    do {                                                                                                                      \
        if (want_dx && want_doff) mex_bwd_head<MP, true, true><<<blocks, kT, 0, s>>>(g, x, eo, mo, mx, y, dy, dx, part, splits, flag); \
        else if (want_dx) mex_bwd_head<MP, true, false><<<blocks, kT, 0, s>>>(g, x, eo, mo, mx, y, dy, dx, part, splits, flag);        \
        else mex_bwd_head<MP, false, true><<<blocks, kT, 0, s>>>(g, x, eo, mo, mx, y, dy, dx, part, splits, flag);                     \
    } while (0)
    switch (pad4(g.M)) {
    case 4: HEAD_BWD(4); break;
    case 8: HEAD_BWD(8); break;
    case 12: HEAD_BWD(12); break;
    default: HEAD_BWD(16); break;
    }
#undef HEAD_BWD
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
