// Opt-in tensor-core evaluation of the L2 Similarity forward pass (SIMNETS_FLAG_SIM_L2_TENSORCORE).
//
// The reference evaluates  y[n, m, pos] = sum_k s[m,k] * (x[k,(n,pos)] - t[m,k])^2 + c[m]  term by term
// (HUJI-Deep/simnets-tf include/utils/similarity_utils.hpp:26-36, with s = -w for plain L2 and -w/2 with the
// normalisation term, whose constants are c[m]).  Expanding the square turns the sum into one GEMM over a doubled
// reduction axis,
//     y = [x^2 | x] . [s | -2 s t]^T + (sum_k s t^2 + c[m]),
// which runs on the tcgen05 tensor cores with split-TF32 operands (hi*hi + hi*lo + lo*hi, FP32 accumulation), in the
// persistent warp-specialised form of the MEX forward kernel: producer warps gather the patches (tap table, padding
// value outside the image), square, split and store the position operand; one thread bulk-copies the pre-split parameter
// tiles; one thread issues the MMAs; the epilogue adds the per-instance constant and stores.  A stage holds 8 taps:
// reduction entries 0..7 are the squares, 8..15 the values.
//
// The expansion cancels where the term-by-term form does not (x close to t with both far from zero), so this path is
// not the default: results agree with the term-by-term kernels to 1e-3 of the largest output magnitude, not 1e-5.
// Inputs must be finite (an infinite x gives inf - inf = NaN here, -inf in the reference); NaN propagates as there.
#include "ws.cuh"

namespace simnets {

namespace {

constexpr int kSimTcTaps = 8;

struct SimTcColumn {
    long long base;     // n*M*N + pos, or -1 past the end
    int n, h0, w0;
};

__device__ __forceinline__ SimTcColumn sim_tc_column(const SimGeo& g, long long j, long long P) {
    SimTcColumn c;
    c.base = -1; c.n = 0; c.h0 = c.w0 = 0;
    if (j >= P) return c;
    const int n = int(j / g.N), pos = int(j % g.N);
    c.n = n;
    c.h0 = (pos / g.ow) * g.sh - g.ph;
    c.w0 = (pos % g.ow) * g.sw - g.pw;
    c.base = (long long)n * g.M * g.N + pos;
    return c;
}

__device__ __forceinline__ float sim_tc_hi(float v) { uint32_t r; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v)); return __uint_as_float(r); }
// float index of element (row, k) inside one [NT x 16] plane of a parameter tile (K-major core matrices, no swizzle)
__device__ __forceinline__ int sim_tc_core(int row, int k) { return (row >> 3) * 128 + (k >> 2) * 32 + (row & 7) * 4 + (k & 3); }

// One block per row of the parameter tiles (instance m, or a padding row of the last tile, which is zeroed):
// tiles[mt][chunk][hi, lo][NT x 16] and bias[m] = sum_k s t^2 + c[m].  planes, cm: as sim_prep leaves them.
__global__ void __launch_bounds__(128) sim_tc_prep(SimGeo g, int NT, const float* __restrict__ planes, const float* __restrict__ cm,
                                                   float* __restrict__ tiles, float* __restrict__ bias) {
    __shared__ float red[128];
    const int m = blockIdx.x, ldm = (g.M + 3) & ~3;
    const int kchunks = (g.K + kSimTcTaps - 1) / kSimTcTaps;
    const size_t plane = (size_t)g.K * ldm;
    float* mine = tiles + (size_t)(m / NT) * kchunks * 2 * NT * 16;
    const int row = m % NT;
    float bsum = 0.f;
    for (int k = threadIdx.x; k < kchunks * kSimTcTaps; k += 128) {
        float s = 0.f, t = 0.f;
        if (m < g.M && k < g.K) { t = planes[(size_t)k * ldm + m]; s = planes[plane + (size_t)k * ldm + m]; }
        const float b0 = s, b1 = -2.f * s * t;
        bsum = fmaf(s * t, t, bsum);
        float* tile = mine + (size_t)(k / kSimTcTaps) * 2 * NT * 16;
        const int q0 = sim_tc_core(row, k % kSimTcTaps), q1 = sim_tc_core(row, kSimTcTaps + k % kSimTcTaps);
        const float h0 = sim_tc_hi(b0), h1 = sim_tc_hi(b1);
        tile[q0] = h0; tile[NT * 16 + q0] = sim_tc_hi(b0 - h0);
        tile[q1] = h1; tile[NT * 16 + q1] = sim_tc_hi(b1 - h1);
    }
    red[threadIdx.x] = bsum;
    __syncthreads();
    for (int s = 64; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0 && m < g.M) bias[m] = red[0] + cm[m];
}

template <int NT>
__global__ void __launch_bounds__(kWsThreads, 1) sim_fwd_tc(SimGeo g, const float* __restrict__ x, const float* __restrict__ tiles,
                                                           const float* __restrict__ bias, const int2* __restrict__ taps,
                                                           float* __restrict__ y, WsPlan plan, int* __restrict__ flag) {
    constexpr int STAGES = ws_stages<NT>();
    constexpr int A_BYTES = kTcPos * kTcKT * 4, STAGE_BYTES = ws_stage_bytes<NT>();
    constexpr uint32_t TMEM_COLS = 2 * NT < 32 ? 32 : 2 * NT;
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ WsShared<STAGES> sh;
    __shared__ __align__(16) float bias_w[kWsEpilogueWarps][NT / 2];

    const long long P = (long long)g.B * g.N;
    const int mtiles = (g.M + NT - 1) / NT, kchunks = (g.K + kSimTcTaps - 1) / kSimTcTaps;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int my_items = plan.items > int(blockIdx.x) ? (plan.items - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;

    const uint32_t tmem = ws_setup(sh, TMEM_COLS);

    if (warp < kWsProducerWarps) {
        // ---------------- producers: thread % 128 = position row; 8 taps per stage; group = every other chunk
        const int prow = threadIdx.x % kTcPos, group = threadIdx.x / kTcPos;
        const float oob = float(g.oob);
        const int K = g.K;
        int li = group / kchunks, c = group % kchunks;
        WsRing<STAGES> ring = {group, 0u};
        WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
        SimTcColumn col = sim_tc_column(g, (long long)it.jt * kTcPos + prow, P);
        float xv[kSimTcTaps];
        auto load = [&](int c) {
            const float* xs = x + (size_t)col.n * g.C * g.H * g.W + col.h0 * g.W + col.w0;
#pragma unroll
            for (int u = 0; u < kSimTcTaps; ++u) {
                const int k = c * kSimTcTaps + u;
                xv[u] = 0.f;                                              // dead rows and taps past K add nothing
                if (col.base >= 0 && k < K) {
                    const int2 tap = __ldg(taps + k);
                    const int hh = col.h0 + (tap.y >> 16), ww = col.w0 + (tap.y & 0xffff);
                    xv[u] = (hh >= 0 && hh < g.H && ww >= 0 && ww < g.W) ? __ldg(xs + tap.x) : oob;
                }
            }
        };
        if (li < my_items) load(c);
        for (; li < my_items;) {
            const int stage = ring.stage;
            unsigned char* sA = dsm + stage * STAGE_BYTES;
            if (sh.failed) break;
            float e[kTcKT];
#pragma unroll
            for (int u = 0; u < kSimTcTaps; ++u) { e[u] = xv[u] * xv[u]; e[kSimTcTaps + u] = xv[u]; }
            c += kWsGroups;
            if (c >= kchunks) {
                do { c -= kchunks; ++li; } while (c >= kchunks);
                if (li < my_items) {
                    it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
                    col = sim_tc_column(g, (long long)it.jt * kTcPos + prow, P);
                }
            }
            if (li < my_items) load(c);
            if (ring.fill >= 1 && !mbar_wait(&sh.empty[stage], (ring.fill - 1) & 1u)) { sh.failed = 1; break; }
#pragma unroll
            for (int h = 0; h < kTcKT / 4; ++h) {
                float4 hi, lo;
                split_tf32_trunc(e[4 * h], hi.x, lo.x); split_tf32_trunc(e[4 * h + 1], hi.y, lo.y);
                split_tf32_trunc(e[4 * h + 2], hi.z, lo.z); split_tf32_trunc(e[4 * h + 3], hi.w, lo.w);
                const int off = core_offset(prow, 4 * h);
                *reinterpret_cast<float4*>(sA + off) = hi;
                *reinterpret_cast<float4*>(sA + A_BYTES + off) = lo;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&sh.full[stage]);
            ring.advance(kWsGroups);
        }
    } else if (warp == kWsLoaderWarp) {
        ws_loader_role<NT, STAGES>(sh, dsm, tiles, plan, my_items, mtiles, kchunks);
    } else if (warp == kWsMmaWarp) {
        ws_mma_role<NT, STAGES>(sh, dsm, tmem, my_items, kchunks);
    } else {
        // ---------------- epilogue: lane = position, registers = instances
        const int quarter = warp & 3, half = (warp - kWsProducerWarps) >> 2;
        float* bw = bias_w[warp - kWsProducerWarps];
        const unsigned Nu = unsigned(g.N);
        for (int li = 0; li < my_items; ++li) {
            const int buf = li & 1;
            if (__any_sync(0xffffffffu, sh.failed)) break;
            const WsItem it = ws_item(plan, int(blockIdx.x) + li * int(gridDim.x));
            const int m0 = it.mt * NT + half * (NT / 2);
            for (int i = lane; i < NT / 2; i += 32) bw[i] = m0 + i < g.M ? __ldg(bias + m0 + i) : 0.f;
            __syncwarp();
            const SimTcColumn col = sim_tc_column(g, (long long)it.jt * kTcPos + quarter * 32 + lane, P);
            float* yb = y + (col.base >= 0 ? col.base : 0) + (long long)m0 * g.N;
            const bool ok = mbar_wait(&sh.acc_full[buf], (uint32_t(li) >> 1) & 1u);
            if (!__all_sync(0xffffffffu, ok)) { sh.failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < NT / 2; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + uint32_t(buf * NT + half * (NT / 2) + c0) + (uint32_t(quarter * 32) << 16), v);
                if (col.base >= 0) {
                    float* yp = yb + (size_t)c0 * Nu;
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (m0 + c0 + i < g.M) __stcs(yp + i * Nu, __uint_as_float(v[i]) + bw[c0 + i]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&sh.acc_empty[buf]);
            __syncwarp();                                   // every lane is done with this item's constants
        }
    }

    ws_teardown(sh, tmem, TMEM_COLS, flag);
}

}  // namespace

bool sim_tc_shape(const SimGeo& g, uint32_t flags) {
    if (!(flags & SIMNETS_FLAG_SIM_L2_TENSORCORE)) return false;
    if (g.mode != SIM_L2 && g.mode != SIM_L2N) return false;       // L1 and the NaN-skipping modes have no such expansion
    if (g.batch_quirk) return false;
    return g.bh < 32768 && g.bw < 32768;
}

int sim_tc_nt(const SimGeo& g) { return g.M > 64 ? 128 : 64; }

size_t sim_tc_tile_floats(const SimGeo& g) {
    const int NT = sim_tc_nt(g);
    return (size_t)((g.M + NT - 1) / NT) * ((g.K + kSimTcTaps - 1) / kSimTcTaps) * 2 * NT * 16;
}

cudaError_t launch_sim_fwd_tc(const SimGeo& g, const float* x, const float* planes, const float* cm, const int2* taps, float* tiles,
                              float* bias, int* flag, float* y, cudaStream_t s) {
    const int NT = sim_tc_nt(g), mtiles = (g.M + NT - 1) / NT;
    sim_tc_prep<<<mtiles * NT, 128, 0, s>>>(g, NT, planes, cm, tiles, bias);      // (sim_prep has cleared the flag words)
    count_launch();
    const long long P = (long long)g.B * g.N;
    const long long items = ((P + kTcPos - 1) / kTcPos) * mtiles;
    if (items >= 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const WsPlan plan = {int(items), make_fastdiv(1), make_fastdiv(mtiles)};
    const int grid = int(std::min<long long>(items, ws_sm_count()));
    if (NT == 128) WS_RUN(sim_fwd_tc<128>, ws_stages<128>() * ws_stage_bytes<128>(), grid, g, x, tiles, bias, taps, y, plan, flag);
    else WS_RUN(sim_fwd_tc<64>, ws_stages<64>() * ws_stage_bytes<64>(), grid, g, x, tiles, bias, taps, y, plan, flag);
    count_launch();
    return cudaGetLastError();
}

}  // namespace simnets
