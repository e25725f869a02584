// Device-side geometry shared by all kernels: how an output position maps to input taps
// (the implicit patch matrix), and how MEX output positions map to offset regions.
// Nothing here materialises a patch ("im2col") buffer: every kernel derives tap addresses
// from these structs on the fly.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace simnets {

enum SimMode : int { SIM_L1 = 0, SIM_L1_SKIP = 1, SIM_L2 = 2, SIM_L2N = 3, SIM_L2N_NAN = 4 };

struct SimGeo {
    int B, C, H, W, M;
    int bh, bw, sh, sw, ph, pw;
    int oh, ow;            // output height / width
    int K, N;              // K = C*bh*bw taps per patch, N = oh*ow positions per sample
    int mode;              // SimMode
    int batch_quirk;       // add the L2N constant (B - n) times to sample n
    int absw;              // the weights tensor holds raw values: the op uses |w| and returns dL/dw_raw = sign(w_raw) dL/d|w|
    double fudge, oob;
};

// Division of 0 <= n < 2^31 by a positive constant known on the host: n / d = (n * mul) >> shift, exactly
// (mul = ceil(2^shift / d), shift = 31 + ceil(log2 d)).  One wide multiply and a shift instead of a division loop.
struct FastDiv { uint32_t d, mul, shift; };
__host__ inline FastDiv make_fastdiv(int d) {
    FastDiv f;
    f.d = uint32_t(d < 1 ? 1 : d);
    uint32_t l = 0;
    while ((1ull << l) < f.d) ++l;
    f.shift = 31 + l;
    f.mul = uint32_t(((1ull << f.shift) + f.d - 1) / f.d);
    return f;
}
__host__ __device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f) { return uint32_t(((unsigned long long)n * f.mul) >> f.shift); }

struct MexGeo {
    int B, C, H, W, M;
    int bc, bh, bw, sc, sh, sw, pc, ph, pw;
    int Co, Ho, Wo;        // output grid per instance
    int rc, rh, rw;        // extent of one offsets region (positions)
    int oc, oh, ow;        // number of regions along each axis
    int R, rs;             // num_regions, region_size
    int K, N;              // K = bc*bh*bw, N = Co*Ho*Wo
    FastDiv f_rs, f_rw, f_rh, f_ow, f_oh;   // dividers for region_size, rw, rh, ow, oh
    int gp, Ng;            // dy is given pooled gp x gp over (h, w) (1 = full resolution); Ng = positions per instance in dy
    int unshared;
    int finite;            // epsilon is finite
    int softmax;
    double eps, cst, oob;  // cst = 0 (softmax_mode) or -log(K)
};

__host__ __device__ __forceinline__ int mex_region_of(const MexGeo& g, int c, int h, int w) {
    const int rc = g.unshared ? c % g.oc : c / g.rc;
    const int rh = g.unshared ? h % g.oh : h / g.rh;
    const int rw = g.unshared ? w % g.ow : w / g.rw;
    return (rc * g.oh + rh) * g.ow + rw;
}

// Offset of dy[n, instance 0, output position pos]; consecutive instances are g.Ng apart.  With gp > 1 the
// caller's dy holds one value per gp x gp window of output positions (the gradient of a sum pooling that
// consumed the output), and every position of a window reads that value.
__host__ __device__ __forceinline__ long long mex_dy_base(const MexGeo& g, int n, int pos) {
    if (g.gp == 1) return (long long)n * g.M * g.N + pos;
    const int w = pos % g.Wo, h = (pos / g.Wo) % g.Ho, c = pos / (g.Wo * g.Ho);
    return (long long)n * g.M * g.Ng + (c * (g.Ho >> 1) + (h >> 1)) * (g.Wo >> 1) + (w >> 1);     // gp is 1 or 2
}

// Position l (0 <= l < region_size) of region r -> output coordinates; false when the region's footprint hangs
// over the edge of the output grid there.
__host__ __device__ __forceinline__ bool mex_region_chw(const MexGeo& g, int r, int l, int& c, int& h, int& w) {
    const uint32_t q0 = fast_div(uint32_t(r), g.f_ow), rw = uint32_t(r) - q0 * g.ow;
    const uint32_t rc = fast_div(q0, g.f_oh), rh = q0 - rc * g.oh;
    const uint32_t q1 = fast_div(uint32_t(l), g.f_rw), lw = uint32_t(l) - q1 * g.rw;
    const uint32_t lc = fast_div(q1, g.f_rh), lh = q1 - lc * g.rh;
    c = g.unshared ? int(lc) * g.oc + int(rc) : int(rc) * g.rc + int(lc);
    h = g.unshared ? int(lh) * g.oh + int(rh) : int(rh) * g.rh + int(lh);
    w = g.unshared ? int(lw) * g.ow + int(rw) : int(rw) * g.rw + int(lw);
    return c < g.Co && h < g.Ho && w < g.Wo;
}

// Position l (0 <= l < region_size) of region r -> flat output position (c*Ho + h)*Wo + w, or -1
// when the region's footprint hangs over the edge of the output grid there.
__host__ __device__ __forceinline__ int mex_region_position(const MexGeo& g, int r, int l) {
    const int rw = r % g.ow, rh = (r / g.ow) % g.oh, rc = r / (g.ow * g.oh);
    const int lw = l % g.rw, lh = (l / g.rw) % g.rh, lc = l / (g.rw * g.rh);
    const int c = g.unshared ? lc * g.oc + rc : rc * g.rc + lc;
    const int h = g.unshared ? lh * g.oh + rh : rh * g.rh + lh;
    const int w = g.unshared ? lw * g.ow + rw : rw * g.rw + lw;
    if (c >= g.Co || h >= g.Ho || w >= g.Wo) return -1;
    return (c * g.Ho + h) * g.Wo + w;
}

}  // namespace simnets
