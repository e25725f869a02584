// 2x2 / stride-2 sum pooling over the two innermost dimensions of a dense [planes, H, W] float32 tensor: the pooling
// SimNets put behind every MEX layer but the last.  Pure HBM stream: a thread reads two 16-byte pieces (rows 2h and
// 2h + 1) and writes two outputs, so a warp moves whole 128-byte lines in both directions.
#include "kernels.cuh"

namespace simnets {

namespace {

// the four addends are summed in window order, ((a + b) + c) + d, like a sequential pooling loop
__global__ void __launch_bounds__(256) sum_pool2_vec4(long long total, int Ho, int W4, int W, const float* __restrict__ x, float* __restrict__ y,
                                                      const int* __restrict__ gate) {
    if (gate && (gate[0] | gate[1]) == 0) return;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int w4 = int(i % W4);
        const long long ph = i / W4;                          // plane * Ho + h
        const float* r0 = x + (2 * ph) * W + 4 * w4;          // rows 2h and 2h + 1 of the same plane are adjacent
        const float4 a = *reinterpret_cast<const float4*>(r0), b = *reinterpret_cast<const float4*>(r0 + W);
        float2 o;
        o.x = ((a.x + a.y) + b.x) + b.y;
        o.y = ((a.z + a.w) + b.z) + b.w;
        *reinterpret_cast<float2*>(y + ph * (W / 2) + 2 * w4) = o;
    }
    (void)Ho;
}

__global__ void __launch_bounds__(256) sum_pool2_scalar(long long total, int Wo, int W, const float* __restrict__ x, float* __restrict__ y,
                                                        const int* __restrict__ gate) {
    if (gate && (gate[0] | gate[1]) == 0) return;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int w = int(i % Wo);
        const long long ph = i / Wo;
        const float* r0 = x + (2 * ph) * W + 2 * w;
        y[i] = ((r0[0] + r0[1]) + r0[W]) + r0[W + 1];
    }
}

}  // namespace

// planes * H * W inputs, H and W even
cudaError_t launch_sum_pool2(long long planes, int H, int W, const float* x, float* y, cudaStream_t s, const int* gate) {
    const int Ho = H / 2, Wo = W / 2;
    if (planes == 0 || Ho == 0 || Wo == 0) return cudaSuccess;
    const bool vec = W % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 7) == 0;
    const long long total = vec ? planes * Ho * (W / 4) : planes * Ho * Wo;
    // (a gated launch almost always returns at once: one wave of CTAs is enough)
    const int grid = int(std::min<long long>((total + 255) / 256, (long long)device_sm_count() * (gate ? 4 : 16)));
    if (vec) sum_pool2_vec4<<<grid, 256, 0, s>>>(total, Ho, W / 4, W, x, y, gate);
    else sum_pool2_scalar<<<grid, 256, 0, s>>>(total, Wo, W, x, y, gate);
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
