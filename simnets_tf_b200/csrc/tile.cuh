// Register-blocked generalized-GEMM tile engine for sm_100a CUDA cores.
//
//   C[i, j]  (op)=  reduce_q  comb(A[i, q], B[q, j])
//
// One CTA owns a TM x TN tile of C; each thread owns RM x RN outputs (RM, RN in {4, 8}) as 4-wide
// groups so that every shared-memory read is a 16-byte vector and a warp's reads of one operand
// coalesce into one or two wavefronts (lanes: 4 along i x 8 along j).  The reduction index q is
// walked in chunks of KC through double-buffered shared memory, laid out q-major ([q][i] / [q][j])
// with NA / NB float planes per operand.  Operands are not copied verbatim: a kernel supplies
//   fetchA/fetchB(chunk)   global -> registers, issued BEFORE the math of the current chunk so the
//                          loads are in flight while the FP32 pipe works, and
//   commitA/commitB(buf)   registers -> shared, applying the element transform (exp, NaN mask, ...)
// so implicit patch gathers, masks and exponentials cost nothing inside the inner loop.
// An operand whose global layout is contiguous along q is stored transposed; its 4-float groups
// are XOR-swizzled by (q >> 2) & 7 and rotated by q & 3 inside the group, so that 32 lanes storing
// 32 consecutive q of one row hit 32 different banks (template flags ASWZ / BSWZ; the read side
// applies the same XOR and undoes the rotation at compile time, q being an unrolled loop index).
#pragma once
#include <cuda_runtime.h>

namespace simnets {

template <int TM_, int TN_, int KC_, int RM_, int RN_, int NA_, int NB_>
struct TileCfg {
    static constexpr int TM = TM_, TN = TN_, KC = KC_, RM = RM_, RN = RN_, NA = NA_, NB = NB_;
    static constexpr int TI = TM / RM, TJ = TN / RN;          // threads along i / j
    static constexpr int THREADS = TI * TJ;
    static constexpr int A_STAGE = NA * KC * TM, B_STAGE = NB * KC * TN;   // floats per buffer
    static constexpr int SMEM_FLOATS = 2 * (A_STAGE + B_STAGE);
    static constexpr int A_PER = KC * TM / THREADS, B_PER = KC * TN / THREADS;  // staged elements / thread / chunk
    static_assert(RM == 4 || RM == 8, "RM must be 4 or 8");
    static_assert(RN == 4 || RN == 8, "RN must be 4 or 8");
    static_assert(TI % 4 == 0 && TJ % 8 == 0, "a warp spans 4 threads along i and 8 along j");
    static_assert((KC * TM) % THREADS == 0 && (KC * TN) % THREADS == 0, "staging must divide evenly");
};

// Thread coordinates inside the CTA tile.
template <class Cfg>
struct TileThread {
    int ti, tj;
    __device__ __forceinline__ TileThread() {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        constexpr int WJ = Cfg::TJ / 8;                       // warps along j
        ti = (warp / WJ) * 4 + (lane >> 3);
        tj = (warp % WJ) * 8 + (lane & 7);
    }
    // local row of output r (0 <= r < RM): two groups of 4, half a tile apart, when RM == 8
    __device__ __forceinline__ int row(int r) const { return (r >> 2) * (Cfg::TM / 2) + ti * 4 + (r & 3); }
    __device__ __forceinline__ int col(int c) const { return (c >> 2) * (Cfg::TN / 2) + tj * 4 + (c & 3); }
};

// Physical float offset of element (q, e) of one plane in a [KC][T] stage, optionally swizzled.
template <int T, bool SWZ>
__device__ __forceinline__ int stage_offset(int q, int e) {
    if (SWZ) return q * T + ((((e >> 2) ^ ((q >> 2) & 7)) << 2) | ((e + q) & 3));
    return q * T + e;
}

// Float offset of the 16-byte group that holds elements e .. e+3 (e a multiple of 4) at step q.
template <int T, bool SWZ>
__device__ __forceinline__ int stage_group_offset(int q, int e) {
    if (SWZ) return q * T + (((e >> 2) ^ ((q >> 2) & 7)) << 2);
    return q * T + e;
}

// The math of one chunk: KC steps, each a rank-1 generalized update of the RM x RN register tile.
template <class Cfg, bool ASWZ, bool BSWZ, class Comb>
__device__ __forceinline__ void tile_compute(const float* __restrict__ As, const float* __restrict__ Bs,
                                             const TileThread<Cfg>& t, Comb comb) {
#pragma unroll
    for (int q = 0; q < Cfg::KC; ++q) {
        float a[Cfg::NA][Cfg::RM], b[Cfg::NB][Cfg::RN];
#pragma unroll
        for (int p = 0; p < Cfg::NA; ++p)
#pragma unroll
            for (int g = 0; g < Cfg::RM / 4; ++g) {
                const float4 v = *reinterpret_cast<const float4*>(As + p * Cfg::KC * Cfg::TM +
                                                                  stage_group_offset<Cfg::TM, ASWZ>(q, g * (Cfg::TM / 2) + t.ti * 4));
                const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) a[p][g * 4 + u] = vv[ASWZ ? ((u + q) & 3) : u];
            }
#pragma unroll
        for (int p = 0; p < Cfg::NB; ++p)
#pragma unroll
            for (int g = 0; g < Cfg::RN / 4; ++g) {
                const float4 v = *reinterpret_cast<const float4*>(Bs + p * Cfg::KC * Cfg::TN +
                                                                  stage_group_offset<Cfg::TN, BSWZ>(q, g * (Cfg::TN / 2) + t.tj * 4));
                const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) b[p][g * 4 + u] = vv[BSWZ ? ((u + q) & 3) : u];
            }
#pragma unroll
        for (int r = 0; r < Cfg::RM; ++r)
#pragma unroll
            for (int c = 0; c < Cfg::RN; ++c) {
                float av[Cfg::NA], bv[Cfg::NB];
#pragma unroll
                for (int p = 0; p < Cfg::NA; ++p) av[p] = a[p][r];
#pragma unroll
                for (int p = 0; p < Cfg::NB; ++p) bv[p] = b[p][c];
                comb(r, c, av, bv);
            }
    }
}

// Double-buffered main loop over `nchunks` chunks of the reduction index.
template <class Cfg, bool ASWZ, bool BSWZ, class FetchA, class FetchB, class CommitA, class CommitB, class Comb>
__device__ __forceinline__ void tile_mainloop(float* smem, int nchunks, const TileThread<Cfg>& t, FetchA fetchA, FetchB fetchB,
                                              CommitA commitA, CommitB commitB, Comb comb) {
    float* As0 = smem;
    float* As1 = smem + Cfg::A_STAGE;
    float* Bs0 = smem + 2 * Cfg::A_STAGE;
    float* Bs1 = Bs0 + Cfg::B_STAGE;
    if (nchunks <= 0) return;
    fetchA(0); fetchB(0);
    commitA(As0); commitB(Bs0);
    __syncthreads();
    for (int c = 0; c < nchunks; ++c) {
        const bool more = c + 1 < nchunks;
        if (more) { fetchA(c + 1); fetchB(c + 1); }
        tile_compute<Cfg, ASWZ, BSWZ>((c & 1) ? As1 : As0, (c & 1) ? Bs1 : Bs0, t, comb);
        if (more) { commitA((c & 1) ? As0 : As1); commitB((c & 1) ? Bs0 : Bs1); }
        __syncthreads();
    }
}

__device__ __forceinline__ float fast_exp(float v) { return __expf(v); }
__device__ __forceinline__ float fast_log(float v) { return __logf(v); }

}  // namespace simnets
