// Measurement probe: the rate at which this GPU issues dependent-free FP32 fused multiply-adds from registers, the
// denominator of "fraction of the FP32 pipe" figures.  Not part of the operators.
#include "kernels.cuh"

namespace simnets {

namespace {

// Every thread runs `iters` rounds of 16 independent FMA chains (8 registers x 2), scalar or as the packed
// two-lane instruction; nothing touches memory inside the loop.
template <bool PACKED>
__global__ void __launch_bounds__(1024) fp32_fma_probe(int iters, float seed, float* __restrict__ out) {
    float2 a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = make_float2(seed + j, seed - j);
    const float2 b = make_float2(1.0000001f, 0.9999999f), c = make_float2(1e-7f, -1e-7f);
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (PACKED) a[j] = __ffma2_rn(a[j], b, c);
            else { a[j].x = fmaf(a[j].x, b.x, c.x); a[j].y = fmaf(a[j].y, b.y, c.y); }
        }
    }
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += a[j].x + a[j].y;
    if (s == 123.456f) out[0] = s;                      // never true: keeps the chains alive
}

}  // namespace

cudaError_t launch_fp32_probe(bool packed, int blocks, int iters, float* out, cudaStream_t s) {
    if (packed) fp32_fma_probe<true><<<blocks, 1024, 0, s>>>(iters, 1.f, out);
    else fp32_fma_probe<false><<<blocks, 1024, 0, s>>>(iters, 1.f, out);
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
