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
    double fudge, oob;
};

struct MexGeo {
    int B, C, H, W, M;
    int bc, bh, bw, sc, sh, sw, pc, ph, pw;
    int Co, Ho, Wo;        // output grid per instance
    int rc, rh, rw;        // extent of one offsets region (positions)
    int oc, oh, ow;        // number of regions along each axis
    int R, rs;             // num_regions, region_size
    int K, N;              // K = bc*bh*bw, N = Co*Ho*Wo
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
    return (long long)n * g.M * g.Ng + (c * (g.Ho / g.gp) + h / g.gp) * (g.Wo / g.gp) + w / g.gp;
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
