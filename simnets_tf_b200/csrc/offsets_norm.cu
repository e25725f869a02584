// normalize_offsets of the MEX layer (reference python/simnets/keras.py:155-160): every row of K offsets (one per
// region and instance) minus its log-sum-exp, and the gradient of that map.  One launch each instead of the dozen small
// tensor-library kernels a composed logsumexp costs, which matters when a data-parallel rank's step is a millisecond.
#include "kernels.cuh"

namespace simnets {

namespace {

constexpr int kNormThreads = 128;

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, u) : v + u;
    }
    __syncthreads();                                   // red may still be read from a previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < kNormThreads / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

// out[row][k] = off[row][k] - logsumexp_k(off[row][:])
__global__ void __launch_bounds__(kNormThreads) normalize_offsets_fwd(int K, const float* __restrict__ off, float* __restrict__ out) {
    __shared__ float red[kNormThreads / 32];
    const float* o = off + (size_t)blockIdx.x * K;
    float mx = -CUDART_INF_F;
    for (int k = threadIdx.x; k < K; k += kNormThreads) mx = fmaxf(mx, o[k]);
    mx = block_reduce(mx, true, red);
    const float ref = (mx == CUDART_INF_F || mx == -CUDART_INF_F) ? 0.f : mx;      // as a stable logsumexp treats infinite maxima
    float sum = 0.f;
    for (int k = threadIdx.x; k < K; k += kNormThreads) sum += expf(o[k] - ref);
    sum = block_reduce(sum, false, red);
    const float lse = ref + logf(sum);
    float* y = out + (size_t)blockIdx.x * K;
    for (int k = threadIdx.x; k < K; k += kNormThreads) y[k] = o[k] - lse;
}

// doff[row][k] = dout[row][k] - softmax(off[row][:])[k] * sum_k dout[row][:]
__global__ void __launch_bounds__(kNormThreads) normalize_offsets_bwd(int K, const float* __restrict__ off, const float* __restrict__ dout,
                                                                      float* __restrict__ doff) {
    __shared__ float red[kNormThreads / 32];
    const float* o = off + (size_t)blockIdx.x * K;
    const float* g = dout + (size_t)blockIdx.x * K;
    float mx = -CUDART_INF_F;
    for (int k = threadIdx.x; k < K; k += kNormThreads) mx = fmaxf(mx, o[k]);
    mx = block_reduce(mx, true, red);
    const float ref = (mx == CUDART_INF_F || mx == -CUDART_INF_F) ? 0.f : mx;
    float sum = 0.f, gs = 0.f;
    for (int k = threadIdx.x; k < K; k += kNormThreads) { sum += expf(o[k] - ref); gs += g[k]; }
    sum = block_reduce(sum, false, red);
    gs = block_reduce(gs, false, red);
    const float scale = gs / sum;
    float* d = doff + (size_t)blockIdx.x * K;
    for (int k = threadIdx.x; k < K; k += kNormThreads) d[k] = g[k] - expf(o[k] - ref) * scale;
}

}  // namespace

cudaError_t launch_normalize_offsets_fwd(long long rows, int K, const float* off, float* out, cudaStream_t s) {
    if (rows == 0 || K == 0) return cudaSuccess;
    if (rows > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    normalize_offsets_fwd<<<int(rows), kNormThreads, 0, s>>>(K, off, out);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_normalize_offsets_bwd(long long rows, int K, const float* off, const float* dout, float* doff, cudaStream_t s) {
    if (rows == 0 || K == 0) return cudaSuccess;
    if (rows > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    normalize_offsets_bwd<<<int(rows), kNormThreads, 0, s>>>(K, off, dout, doff);
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
