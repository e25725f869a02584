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
        // 4 x 8 lane grid, rows interleaved in pairs: any 8 consecutive lanes span 2 rows x 4 columns, so a
        // quarter-warp's 16-byte reads touch 2 distinct A vectors and 4 distinct B vectors
        const int li = ((lane >> 4) << 1) | (lane & 1), lj = (lane & 15) >> 1;
        ti = (warp / WJ) * 4 + li;
        tj = (warp % WJ) * 8 + lj;
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

// sm_100 packed FP32 math: one instruction performs two FMAs / adds / multiplies on a register pair,
// halving the issue slots the FP32 work needs.  The register tile is therefore kept as float2 pairs
// along j, and a kernel's `comb` receives the A value splatted into both halves.
__device__ __forceinline__ float2 splat2(float v) { return make_float2(v, v); }
__device__ __forceinline__ float2 neg2(float2 v) { return make_float2(-v.x, -v.y); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }

// The math of one chunk: KC steps, each a rank-1 generalized update of the RM x RN register tile.
// comb(r, cp, a[NA], b[NB]) updates outputs (r, 2*cp) and (r, 2*cp + 1).
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
            for (int cp = 0; cp < Cfg::RN / 2; ++cp) {
                float2 av[Cfg::NA], bv[Cfg::NB];
#pragma unroll
                for (int p = 0; p < Cfg::NA; ++p) av[p] = splat2(a[p][r]);
#pragma unroll
                for (int p = 0; p < Cfg::NB; ++p) bv[p] = make_float2(b[p][2 * cp], b[p][2 * cp + 1]);
                comb(r, cp, av, bv);
            }
    }
}

// Double-buffered main loop over `nchunks` chunks of the reduction index.  fetchX(chunk, dst) may either
// load into registers (to be transformed and stored by commitX(dst)) or start asynchronous copies straight
// into the destination stage (commitX then only waits for them).
template <class Cfg, bool ASWZ, bool BSWZ, class FetchA, class FetchB, class CommitA, class CommitB, class Comb>
__device__ __forceinline__ void tile_mainloop(float* smem, int nchunks, const TileThread<Cfg>& t, FetchA fetchA, FetchB fetchB,
                                              CommitA commitA, CommitB commitB, Comb comb) {
    float* As0 = smem;
    float* As1 = smem + Cfg::A_STAGE;
    float* Bs0 = smem + 2 * Cfg::A_STAGE;
    float* Bs1 = Bs0 + Cfg::B_STAGE;
    if (nchunks <= 0) return;
    fetchA(0, As0); fetchB(0, Bs0);
    commitA(As0); commitB(Bs0);
    __syncthreads();
    for (int c = 0; c < nchunks; ++c) {
        const bool more = c + 1 < nchunks;
        float* An = (c & 1) ? As0 : As1;
        float* Bn = (c & 1) ? Bs0 : Bs1;
        if (more) { fetchA(c + 1, An); fetchB(c + 1, Bn); }
        tile_compute<Cfg, ASWZ, BSWZ>((c & 1) ? As1 : As0, (c & 1) ? Bs1 : Bs0, t, comb);
        if (more) { commitA(An); commitB(Bn); }
        __syncthreads();
    }
}

// 16-byte asynchronous global -> shared copy; bytes beyond `valid_bytes` (0..16) are zero-filled.
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gsrc, int valid_bytes) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gsrc), "r"(valid_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Copies one [KC][T] stage plane verbatim from a row-major global matrix whose rows are 16-byte aligned
// (leading dimension `ld` a multiple of 4 floats): rows q0 .. q0+KC-1 (zero past `rows`), columns
// e0 .. e0+T-1 (zero past `cols`).  Every thread issues KC*T/4/THREADS copies.
template <class Cfg, int T>
__device__ __forceinline__ void stage_copy_async(float* dst, const float* __restrict__ src, int ld, int q0, int rows, int e0, int cols) {
    constexpr int VEC = Cfg::KC * T / 4;
    static_assert(VEC % Cfg::THREADS == 0 || VEC < Cfg::THREADS, "stage copy shape");
#pragma unroll
    for (int v = threadIdx.x; v < VEC; v += Cfg::THREADS) {
        const int q = v / (T / 4), e = (v % (T / 4)) * 4;
        const int left = (q0 + q < rows) ? (cols - (e0 + e)) : 0;
        const int bytes = left >= 4 ? 16 : (left > 0 ? left * 4 : 0);
        cp_async16(dst + q * T + e, bytes > 0 ? src + (size_t)(q0 + q) * ld + e0 + e : src, bytes);
    }
}

__device__ __forceinline__ float fast_exp(float v) { return __expf(v); }
__device__ __forceinline__ float fast_log(float v) { return __logf(v); }

}  // namespace simnets
