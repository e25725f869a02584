// Shape-agnostic kernels: one thread per output element (or one block per reduced parameter).
// They accept every geometry and both dtypes, serve float64, unusual shapes and the
// SIMNETS_FLAG_FORCE_DIRECT switch, and give the tiled kernels a second GPU implementation to be
// compared with.  Tap addresses come from the geometry structs; no patch matrix is built.
//
// Arithmetic follows the reference's element functors (HUJI-Deep/simnets-tf,
// include/utils/similarity_utils.hpp:17-150 and include/utils/mex_utils.hpp:10-56), accumulation
// order follows its CPU kernels where a thread owns the whole sum.
#include "kernels.cuh"

namespace simnets {

namespace {

constexpr int kThreads = 256;

template <typename T> __device__ __forceinline__ bool is_nan(T v) { return v != v; }
template <typename T> __device__ __forceinline__ T sign_of(T v) { return T((T(0) < v) - (v < T(0))); }

__device__ __forceinline__ float dev_exp(float v) { return expf(v); }
__device__ __forceinline__ double dev_exp(double v) { return exp(v); }
__device__ __forceinline__ float dev_log(float v) { return logf(v); }
__device__ __forceinline__ double dev_log(double v) { return log(v); }
__device__ __forceinline__ float dev_abs(float v) { return fabsf(v); }
__device__ __forceinline__ double dev_abs(double v) { return fabs(v); }
template <typename T> __device__ __forceinline__ T pos_inf() { return T(CUDART_INF); }

constexpr double kLog2Pi = 1.8378770664093454835606594728112;

// Deterministic block-wide sum (fixed tree), result valid in thread 0.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T* smem) {
    smem[threadIdx.x] = v;
    __syncthreads();
    for (int s = kThreads / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) smem[threadIdx.x] += smem[threadIdx.x + s];
        __syncthreads();
    }
    const T r = smem[0];
    __syncthreads();
    return r;
}

// ------------------------------------------------------------------ Similarity
template <typename T>
__global__ void __launch_bounds__(kThreads) sim_fwd_direct(SimGeo g, const T* __restrict__ x, const T* __restrict__ tm,
                                                           const T* __restrict__ wt, T* __restrict__ y, const int* __restrict__ gate) {
    if (gate && gate[1] == 0) return;
    const long long total = (long long)g.B * g.M * g.N;
    const T oob = T(g.oob), fudge = T(g.fudge);
    for (long long idx = blockIdx.x * (long long)kThreads + threadIdx.x; idx < total; idx += (long long)gridDim.x * kThreads) {
        const int j = int(idx % g.N);
        const long long q = idx / g.N;
        const int m = int(q % g.M), n = int(q / g.M);
        const int ho = j / g.ow, wo = j % g.ow;
        const T* xs = x + (size_t)n * g.C * g.H * g.W;
        const T* tp = tm + (size_t)m * g.K;
        const T* wp = wt + (size_t)m * g.K;
        T sum = T(0);
        int k = 0;
        for (int c = 0; c < g.C; ++c)
            for (int kh = 0; kh < g.bh; ++kh)
                for (int kw = 0; kw < g.bw; ++kw, ++k) {
                    const int hh = ho * g.sh - g.ph + kh, ww = wo * g.sw - g.pw + kw;
                    const T v = (hh >= 0 && hh < g.H && ww >= 0 && ww < g.W) ? xs[((size_t)c * g.H + hh) * g.W + ww] : oob;
                    const T t = tp[k], w = g.absw ? dev_abs(wp[k]) : wp[k], d = t - v;
                    switch (g.mode) {
                    case SIM_L1: sum += -w * dev_abs(d); break;
                    case SIM_L1_SKIP: if (!is_nan(v)) sum += -w * dev_abs(d); break;
                    case SIM_L2: sum += -w * d * d; break;
                    case SIM_L2N: sum += T(0.5) * (-w * d * d + dev_log(w + fudge)); break;
                    default: if (!is_nan(v)) sum += T(0.5) * (-w * d * d - T(kLog2Pi) + dev_log(w + fudge)); break;
                    }
                }
        if (g.mode == SIM_L2N) {
            const T c = T(-0.5 * double(g.K) * kLog2Pi);
            const int reps = g.batch_quirk ? g.B - n : 1;
            for (int i = 0; i < reps; ++i) sum += c;
        }
        y[idx] = sum;
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) sim_dx_direct(SimGeo g, const T* __restrict__ x, const T* __restrict__ tm,
                                                          const T* __restrict__ wt, const T* __restrict__ dy, T* __restrict__ dx) {
    const long long total = (long long)g.B * g.C * g.H * g.W;
    for (long long idx = blockIdx.x * (long long)kThreads + threadIdx.x; idx < total; idx += (long long)gridDim.x * kThreads) {
        const int w0 = int(idx % g.W);
        long long q = idx / g.W;
        const int h0 = int(q % g.H); q /= g.H;
        const int c = int(q % g.C), n = int(q / g.C);
        const T v = x[idx];
        const T* g_n = dy + (size_t)n * g.M * g.N;
        T total_sum = T(0);
        for (int kh = 0; kh < g.bh; ++kh) {
            const int hp = h0 + g.ph - kh;
            if (hp < 0 || hp % g.sh != 0) continue;
            const int ho = hp / g.sh;
            if (ho >= g.oh) continue;
            for (int kw = 0; kw < g.bw; ++kw) {
                const int wp_ = w0 + g.pw - kw;
                if (wp_ < 0 || wp_ % g.sw != 0) continue;
                const int wo = wp_ / g.sw;
                if (wo >= g.ow) continue;
                const int k = (c * g.bh + kh) * g.bw + kw;
                const int j = ho * g.ow + wo;
                T sum = T(0);
                for (int m = 0; m < g.M; ++m) {
                    const T wr = wt[(size_t)m * g.K + k];
                    const T t = tm[(size_t)m * g.K + k], w = g.absw ? dev_abs(wr) : wr, err = g_n[(size_t)m * g.N + j];
                    switch (g.mode) {
                    case SIM_L1: sum += err * w * sign_of(t - v); break;
                    case SIM_L1_SKIP: if (!is_nan(v)) sum += err * w * sign_of(t - v); break;
                    case SIM_L2: sum += T(2) * err * w * (t - v); break;
                    case SIM_L2N: sum += T(0.5) * (T(2) * err * w * (t - v)); break;
                    default: if (!is_nan(v)) sum += T(0.5) * (T(2) * err * w * (t - v)); break;
                    }
                }
                total_sum += sum;
            }
        }
        dx[idx] = total_sum;
    }
}

// One block per (instance m, tap k): reduces over batch and output positions.
template <typename T>
__global__ void __launch_bounds__(kThreads) sim_dparams_direct(SimGeo g, const T* __restrict__ x, const T* __restrict__ tm,
                                                               const T* __restrict__ wt, const T* __restrict__ dy,
                                                               T* __restrict__ dt, T* __restrict__ dw, int accumulate) {
    __shared__ T smem[kThreads];
    const int mk = blockIdx.x;
    const int m = mk / g.K, k = mk % g.K;
    const int kw = k % g.bw, kh = (k / g.bw) % g.bh, c = k / (g.bw * g.bh);
    const T wraw = wt[mk];
    const T t = tm[mk], w = g.absw ? dev_abs(wraw) : wraw, oob = T(g.oob), fudge = T(g.fudge);
    T st = T(0), sw_ = T(0);
    const long long total = (long long)g.B * g.N;
    for (long long i = threadIdx.x; i < total; i += kThreads) {
        const int j = int(i % g.N), n = int(i / g.N);
        const int ho = j / g.ow, wo = j % g.ow;
        const int hh = ho * g.sh - g.ph + kh, ww = wo * g.sw - g.pw + kw;
        const T v = (hh >= 0 && hh < g.H && ww >= 0 && ww < g.W) ? x[(((size_t)n * g.C + c) * g.H + hh) * g.W + ww] : oob;
        const T err = dy[((size_t)n * g.M + m) * g.N + j];
        const T d = v - t;
        switch (g.mode) {
        case SIM_L1: st += err * w * sign_of(d); sw_ += -err * dev_abs(d); break;
        case SIM_L1_SKIP: if (!is_nan(v)) { st += err * w * sign_of(d); sw_ += -err * dev_abs(d); } break;
        case SIM_L2: st += T(2) * err * w * d; sw_ += -err * d * d; break;
        case SIM_L2N: st += err * w * d; sw_ += T(0.5) * (-err * d * d + err / (w + fudge)); break;
        default: if (!is_nan(v)) { st += err * w * d; sw_ += T(0.5) * (-err * d * d + err / (w + fudge)); } break;
        }
    }
    const T rt = block_sum(st, smem);
    T rw = block_sum(sw_, smem);
    if (g.absw) rw *= sign_of(wraw);                   // d|w|/dw, 0 at w = 0
    if (threadIdx.x == 0) {
        dt[mk] = accumulate ? dt[mk] + rt : rt;
        dw[mk] = accumulate ? dw[mk] + rw : rw;
    }
}

// ------------------------------------------------------------------------- MEX
template <typename T>
__device__ __forceinline__ T mex_tap(const MexGeo& g, const T* __restrict__ xs, int c, int h, int w, int k, T oob) {
    const int kw = k % g.bw, kh = (k / g.bw) % g.bh, kc = k / (g.bw * g.bh);
    const int cc = c * g.sc - g.pc + kc, hh = h * g.sh - g.ph + kh, ww = w * g.sw - g.pw + kw;
    return (cc >= 0 && cc < g.C && hh >= 0 && hh < g.H && ww >= 0 && ww < g.W) ? xs[((size_t)cc * g.H + hh) * g.W + ww] : oob;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) mex_fwd_direct(MexGeo g, const T* __restrict__ x, const T* __restrict__ off, T* __restrict__ y, const int* __restrict__ gate) {
    if (gate && (gate[0] | gate[1]) == 0) return;
    const long long total = (long long)g.B * g.M * g.N;
    const T oob = T(g.oob), eps = T(g.eps), cst = T(g.cst);
    for (long long idx = blockIdx.x * (long long)kThreads + threadIdx.x; idx < total; idx += (long long)gridDim.x * kThreads) {
        const int j = int(idx % g.N);
        const long long q = idx / g.N;
        const int m = int(q % g.M), n = int(q / g.M);
        const int w = j % g.Wo, h = (j / g.Wo) % g.Ho, c = j / (g.Wo * g.Ho);
        const T* xs = x + (size_t)n * g.C * g.H * g.W;
        const T* o = off + ((size_t)mex_region_of(g, c, h, w) * g.M + m) * g.K;
        T mx = eps > T(0) ? -pos_inf<T>() : pos_inf<T>();
        for (int k = 0; k < g.K; ++k) {
            const T v = o[k] + mex_tap(g, xs, c, h, w, k, oob);
            // comparisons written as the host library's max/min: a NaN operand never replaces mx
            if (eps > T(0)) { if (mx < v) mx = v; } else { if (v < mx) mx = v; }
        }
        T out = mx;
        if (g.finite) {
            T sum = T(0);
            for (int k = 0; k < g.K; ++k) sum += dev_exp(eps * (mex_tap(g, xs, c, h, w, k, oob) + o[k] - mx) + cst);
            out = mx + dev_log(sum) / eps;
        }
        y[idx] = out;
    }
}

template <typename T>
__device__ __forceinline__ T mex_weight(const MexGeo& g, T eps, T cst, T data, T offset, T top, T top_diff) {
    if (g.finite) return top_diff * dev_exp(eps * (data + offset - top) + cst);
    return top_diff * T((data + offset) == top);
}

template <typename T>
__global__ void __launch_bounds__(kThreads) mex_dx_direct(MexGeo g, const T* __restrict__ x, const T* __restrict__ off,
                                                          const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, const int* __restrict__ gate) {
    if (gate && (gate[0] | gate[1]) == 0) return;
    const long long total = (long long)g.B * g.C * g.H * g.W;
    const T eps = T(g.eps), cst = T(g.cst);
    for (long long idx = blockIdx.x * (long long)kThreads + threadIdx.x; idx < total; idx += (long long)gridDim.x * kThreads) {
        const int w0 = int(idx % g.W);
        long long q = idx / g.W;
        const int h0 = int(q % g.H); q /= g.H;
        const int c0 = int(q % g.C), n = int(q / g.C);
        const T v = x[idx];
        const T* y_n = y + (size_t)n * g.M * g.N;
        T total_sum = T(0);
        for (int kc = 0; kc < g.bc; ++kc) {
            const int cp = c0 + g.pc - kc;
            if (cp < 0 || cp % g.sc != 0 || cp / g.sc >= g.Co) continue;
            for (int kh = 0; kh < g.bh; ++kh) {
                const int hp = h0 + g.ph - kh;
                if (hp < 0 || hp % g.sh != 0 || hp / g.sh >= g.Ho) continue;
                for (int kw = 0; kw < g.bw; ++kw) {
                    const int wp_ = w0 + g.pw - kw;
                    if (wp_ < 0 || wp_ % g.sw != 0 || wp_ / g.sw >= g.Wo) continue;
                    const int c = cp / g.sc, h = hp / g.sh, w = wp_ / g.sw;
                    const int k = (kc * g.bh + kh) * g.bw + kw;
                    const int j = (c * g.Ho + h) * g.Wo + w;
                    const T* o = off + (size_t)mex_region_of(g, c, h, w) * g.M * g.K + k;
                    const T* g_j = dy + mex_dy_base(g, n, j);
                    T sum = T(0);
                    for (int m = 0; m < g.M; ++m)
                        sum += mex_weight(g, eps, cst, v, o[(size_t)m * g.K], y_n[(size_t)m * g.N + j], g_j[(size_t)m * g.Ng]);
                    total_sum += sum;
                }
            }
        }
        dx[idx] = total_sum;
    }
}

// One block at a time per (region r, instance m, tap k): reduces over batch and the region's positions.
// The grid is capped and strides over the (r, m, k) triples, so that a gated-off launch costs a few
// hundred blocks, not one per parameter.
template <typename T>
__global__ void __launch_bounds__(kThreads) mex_doff_direct(MexGeo g, const T* __restrict__ x, const T* __restrict__ off,
                                                            const T* __restrict__ y, const T* __restrict__ dy,
                                                            T* __restrict__ doff, int accumulate, const int* __restrict__ gate) {
    __shared__ T smem[kThreads];
    if (gate && (gate[0] | gate[1]) == 0) return;
    const T oob = T(g.oob), eps = T(g.eps), cst = T(g.cst);
    const long long triples = (long long)g.R * g.M * g.K;
    for (long long rmk = blockIdx.x; rmk < triples; rmk += gridDim.x) {
        const int k = int(rmk % g.K), m = int((rmk / g.K) % g.M), r = int(rmk / ((long long)g.K * g.M));
        const T o = off[rmk];
        T sum = T(0);
        const long long total = (long long)g.B * g.rs;
        for (long long i = threadIdx.x; i < total; i += kThreads) {
            const int l = int(i % g.rs), n = int(i / g.rs);
            const int j = mex_region_position(g, r, l);
            if (j < 0) continue;
            const int w = j % g.Wo, h = (j / g.Wo) % g.Ho, c = j / (g.Wo * g.Ho);
            const T v = mex_tap(g, x + (size_t)n * g.C * g.H * g.W, c, h, w, k, oob);
            const size_t oi = ((size_t)n * g.M + m) * g.N + j;
            sum += mex_weight(g, eps, cst, v, o, y[oi], dy[mex_dy_base(g, n, j) + (long long)m * g.Ng]);
        }
        const T rsum = block_sum(sum, smem);
        if (threadIdx.x == 0) doff[rmk] = accumulate ? doff[rmk] + rsum : rsum;
    }
}

// gated: the launch follows a factorised kernel and does work only if that one raised the safety flag; a grid that
// just fills the GPU keeps the usual case (every CTA reads the flag and returns) at a few microseconds
inline int grid_for(long long total, bool gated = false) {
    const long long blocks = (total + kThreads - 1) / kThreads;
    const long long cap = (long long)device_sm_count() * (gated ? 8 : 32);
    return int(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

#define SIMNETS_DTYPE_SWITCH(is_f64, CALL32, CALL64) do { if (is_f64) { CALL64; } else { CALL32; } } while (0)

cudaError_t launch_sim_fwd_direct(const SimGeo& g, bool f64, const void* x, const void* t, const void* w, void* y, cudaStream_t s,
                                  const int* gate) {
    const long long total = (long long)g.B * g.M * g.N;
    if (total == 0) return cudaSuccess;
    SIMNETS_DTYPE_SWITCH(f64,
        (sim_fwd_direct<float><<<grid_for(total), kThreads, 0, s>>>(g, (const float*)x, (const float*)t, (const float*)w, (float*)y, gate)),
        (sim_fwd_direct<double><<<grid_for(total), kThreads, 0, s>>>(g, (const double*)x, (const double*)t, (const double*)w, (double*)y, gate)));
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_sim_dx_direct(const SimGeo& g, bool f64, const void* x, const void* t, const void* w, const void* dy, void* dx, cudaStream_t s) {
    const long long total = (long long)g.B * g.C * g.H * g.W;
    if (total == 0) return cudaSuccess;
    SIMNETS_DTYPE_SWITCH(f64,
        (sim_dx_direct<float><<<grid_for(total), kThreads, 0, s>>>(g, (const float*)x, (const float*)t, (const float*)w, (const float*)dy, (float*)dx)),
        (sim_dx_direct<double><<<grid_for(total), kThreads, 0, s>>>(g, (const double*)x, (const double*)t, (const double*)w, (const double*)dy, (double*)dx)));
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_sim_dparams_direct(const SimGeo& g, bool f64, const void* x, const void* t, const void* w, const void* dy,
                                      void* dt, void* dw, bool accumulate, cudaStream_t s) {
    const int blocks = g.M * g.K;
    SIMNETS_DTYPE_SWITCH(f64,
        (sim_dparams_direct<float><<<blocks, kThreads, 0, s>>>(g, (const float*)x, (const float*)t, (const float*)w, (const float*)dy, (float*)dt, (float*)dw, accumulate)),
        (sim_dparams_direct<double><<<blocks, kThreads, 0, s>>>(g, (const double*)x, (const double*)t, (const double*)w, (const double*)dy, (double*)dt, (double*)dw, accumulate)));
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_fwd_direct(const MexGeo& g, bool f64, const void* x, const void* off, void* y, cudaStream_t s, const int* gate) {
    const long long total = (long long)g.B * g.M * g.N;
    if (total == 0) return cudaSuccess;
    SIMNETS_DTYPE_SWITCH(f64,
        (mex_fwd_direct<float><<<grid_for(total, gate != nullptr), kThreads, 0, s>>>(g, (const float*)x, (const float*)off, (float*)y, gate)),
        (mex_fwd_direct<double><<<grid_for(total), kThreads, 0, s>>>(g, (const double*)x, (const double*)off, (double*)y, gate)));
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_dx_direct(const MexGeo& g, bool f64, const void* x, const void* off, const void* y, const void* dy, void* dx, cudaStream_t s, const int* gate) {
    const long long total = (long long)g.B * g.C * g.H * g.W;
    if (total == 0) return cudaSuccess;
    SIMNETS_DTYPE_SWITCH(f64,
        (mex_dx_direct<float><<<grid_for(total, gate != nullptr), kThreads, 0, s>>>(g, (const float*)x, (const float*)off, (const float*)y, (const float*)dy, (float*)dx, gate)),
        (mex_dx_direct<double><<<grid_for(total), kThreads, 0, s>>>(g, (const double*)x, (const double*)off, (const double*)y, (const double*)dy, (double*)dx, gate)));
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_doff_direct(const MexGeo& g, bool f64, const void* x, const void* off, const void* y, const void* dy,
                                   void* doff, bool accumulate, cudaStream_t s, const int* gate) {
    const long long triples = (long long)g.R * g.M * g.K;
    const long long cap = (long long)device_sm_count() * 16;
    const int blocks = int(triples < cap ? triples : cap);
    SIMNETS_DTYPE_SWITCH(f64,
        (mex_doff_direct<float><<<blocks, kThreads, 0, s>>>(g, (const float*)x, (const float*)off, (const float*)y, (const float*)dy, (float*)doff, accumulate, gate)),
        (mex_doff_direct<double><<<blocks, kThreads, 0, s>>>(g, (const double*)x, (const double*)off, (const double*)y, (const double*)dy, (double*)doff, accumulate, gate)));
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
