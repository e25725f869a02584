// Softmax cross-entropy of a batch of logit rows and its gradient, in one launch: the loss the reference's example
// networks train with (HUJI-Deep/simnets-tf README.md:108-111, keras `categorical_crossentropy` behind a softmax; in
// TensorFlow a chain of softmax, log, multiply and reduce kernels and their gradients).
//   loss    = scale * sum_b (logsumexp(logits[b, :]) - logits[b, label_b])
//   dlogits = scale * (softmax(logits[b, :]) - onehot(label_b))
// One warp per row; per-CTA sums are combined in CTA order by the CTA that finishes last (same sum on every run).
#include "kernels.cuh"

namespace simnets {

namespace {

constexpr int kLossThreads = 256, kLossRows = kLossThreads / 32;

__device__ __forceinline__ float loss_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float loss_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(kLossThreads) softmax_xent(int batch, int classes, float scale, const float* __restrict__ logits,
                                                            const long long* __restrict__ labels, float* __restrict__ loss,
                                                            float* __restrict__ dlogits, float* __restrict__ partial, unsigned* __restrict__ ticket) {
    __shared__ float rows[kLossRows];
    __shared__ bool last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float mine = 0.f;                                              // lane 0: sum of this warp's rows
    for (long long b = (long long)blockIdx.x * kLossRows + warp; b < batch; b += (long long)gridDim.x * kLossRows) {
        const float* row = logits + b * classes;
        const long long label = labels[b];
        float mx = -CUDART_INF_F;
        for (int c = lane; c < classes; c += 32) mx = fmaxf(mx, row[c]);
        mx = loss_warp_max(mx);
        float sum = 0.f;
        for (int c = lane; c < classes; c += 32) sum += __expf(row[c] - mx);
        sum = loss_warp_sum(sum);
        const float lse = mx + __logf(sum);
        const bool labelled = label >= 0 && label < classes;       // a label outside [0, classes) contributes nothing
        if (dlogits) {
            float* drow = dlogits + b * classes;
            for (int c = lane; c < classes; c += 32)
                drow[c] = labelled ? scale * (__expf(row[c] - lse) - (c == label ? 1.f : 0.f)) : 0.f;
        }
        if (lane == 0 && labelled) mine += lse - row[label];
    }
    if (lane == 0) rows[warp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int w = 0; w < kLossRows; ++w) s += rows[w];
        partial[blockIdx.x] = s;
        __threadfence();
        last = atomicInc(ticket, gridDim.x - 1) == gridDim.x - 1;   // wraps to 0: the counter is clean for the next call
        if (last) {
            __threadfence();
            float total = 0.f;
            for (unsigned i = 0; i < gridDim.x; ++i) total += __ldcg(partial + i);
            *loss = scale * total;
        }
    }
}

int loss_grid(int batch) {
    const long long want = (batch + kLossRows - 1) / kLossRows;
    return int(std::max<long long>(1, std::min<long long>(want, 2LL * device_sm_count())));
}

}  // namespace

size_t softmax_xent_workspace_bytes(int batch) { return 256 + sizeof(float) * size_t(loss_grid(batch)); }

cudaError_t launch_softmax_xent(int batch, int classes, float scale, const float* logits, const long long* labels, float* loss,
                                float* dlogits, void* ws, cudaStream_t s) {
    unsigned* ticket = static_cast<unsigned*>(ws);
    float* partial = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
    const cudaError_t e = cudaMemsetAsync(ticket, 0, sizeof(unsigned), s);
    if (e != cudaSuccess) return e;
    softmax_xent<<<loss_grid(batch), kLossThreads, 0, s>>>(batch, classes, scale, logits, labels, loss, dlogits, partial, ticket);
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
