// MEX forward on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// After the factorisation of mex_tiled.cu the forward pass is a plain GEMM  S[j, m] = sum_k Ex[j, k] * Eo[m, k]
// with both operands in (0, 1].  FP32 accuracy is kept with the split-TF32 scheme: every operand is written to
// shared memory as hi = round-to-TF32(v) and lo = v - hi, and each k-step issues three MMAs
// (hi*hi + hi*lo + lo*hi); the dropped lo*lo term and the truncation of lo are below 3 * 2^-21 of a product, and
// all products are positive, so S keeps ~6 significant digits (tests compare y at 1e-5 of tensor scale).
//
// Tile: 128 positions (the MMA's M, one per tensor-memory lane) x NT instances (the MMA's N, NT = 64/128/256,
// one per tensor-memory column).  Positions are the lane dimension on purpose: in the epilogue lane = position,
// so for every instance the 32 lanes of a warp store to 32 neighbouring positions (coalesced), exactly as the
// CUDA-core kernels do.  256 threads: each stage (16 taps) they compute Ex = exp(eps*(x - mx)) for 128 x 16 values,
// split them and store them in the canonical K-major core-matrix layout (8 rows x 16 bytes, no swizzle), copy the
// matching pre-split Eo tile with cp.async, fence to the async proxy, and one thread issues the six MMAs of the
// stage; tcgen05.commit arrives on an mbarrier that frees the stage (two stages).  Every mbarrier wait is bounded:
// on expiry the kernel records an error word, still waits for its copies, frees its tensor memory and returns.
#include "mex_common.cuh"

namespace simnets {

namespace {

constexpr int kTcThreads = 256;
constexpr int kTcKT = 16;                 // taps per stage (two MMA k-steps of 8)
constexpr int kTcPos = 128;               // positions per tile = MMA M
constexpr uint32_t kWaitTries = 1u << 21; // x ~1 us suspend hint: about two seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Bounded wait for the phase with the given parity to complete; false if it never did.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < kWaitTries; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(addr), "r"(parity), "r"(1000u) : "memory");
        if (ok) return true;
    }
    return false;
}

// Shared-memory matrix descriptor: K-major, no swizzle.  Element (row, k) of a tile lives at
//   (row / 8) * sbo + (k / 4) * lbo + (row % 8) * 16 + (k % 4) * 4   bytes from the start address.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= uint64_t((saddr >> 4) & 0x3FFFu);
    d |= uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= uint64_t(1) << 46;                    // descriptor version of this architecture
    return d;                                   // base offset 0, layout type 0 = no swizzle
}

// Instruction descriptor: D = F32, A = B = TF32, both K-major, M = 128, N = nt.
__host__ __device__ constexpr uint32_t umma_idesc(int nt) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(nt >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ float tf32_hi(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// byte offset of element (row, k) inside a [rows x 16] K-major core-matrix tile (lbo = 128, sbo = 512)
__host__ __device__ constexpr int core_offset(int row, int k) { return (row >> 3) * 512 + (k >> 2) * 128 + (row & 7) * 16 + (k & 3) * 4; }

// ---- prepass: Eo split into hi / lo, laid out tile by tile exactly as the MMA reads it -------------------------
// tiles[r][mt][kc][plane][NT * 16 floats]; rows past M and taps past K are zero.
__global__ void __launch_bounds__(256) mex_tc_prep(MexGeo g, int NT, const float* __restrict__ eo, float* __restrict__ tiles) {
    const int kchunks = (g.K + kTcKT - 1) / kTcKT, mtiles = (g.M + NT - 1) / NT;
    const int ldk = pad4(g.K);
    const long long total = (long long)g.R * mtiles * kchunks * NT * kTcKT;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int kk = int(i % kTcKT);
        long long q = i / kTcKT;
        const int row = int(q % NT); q /= NT;
        const int kc = int(q % kchunks); q /= kchunks;
        const int mt = int(q % mtiles), r = int(q / mtiles);
        const int m = mt * NT + row, k = kc * kTcKT + kk;
        const float v = (m < g.M && k < g.K) ? eo[((size_t)r * g.M + m) * ldk + k] : 0.f;
        const float hi = tf32_hi(v);
        float* tile = tiles + (((size_t)r * mtiles + mt) * kchunks + kc) * 2 * NT * kTcKT;
        tile[core_offset(row, kk) / 4] = hi;
        tile[NT * kTcKT + core_offset(row, kk) / 4] = v - hi;
    }
}

// ---- forward ---------------------------------------------------------------------------------------------------
template <int NT, bool SPATIAL1, bool INTERIOR>
__global__ void __launch_bounds__(kTcThreads) mex_fwd_tc(MexGeo g, const float* __restrict__ x, const float* __restrict__ tiles,
                                                        const float* __restrict__ mo, const float* __restrict__ mx,
                                                        float* __restrict__ y, int* __restrict__ flag) {
    constexpr int A_BYTES = kTcPos * kTcKT * 4;        // one plane of the position operand, one stage
    constexpr int B_BYTES = NT * kTcKT * 4;            // one plane of the instance operand, one stage
    constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ uint64_t bar_free[2];
    __shared__ uint64_t bar_done;
    __shared__ uint32_t tmem_holder;
    __shared__ float mo_s[NT];
    __shared__ int failed;
    if (flag[0]) return;                                // factorisation unsafe: the exact kernels run instead

    const long long P = (long long)g.B * g.rs;
    const int mtiles = (g.M + NT - 1) / NT, kchunks = (g.K + kTcKT - 1) / kTcKT;
    int bid = blockIdx.x;
    const int r = bid % g.R; bid /= g.R;
    const int mt = bid % mtiles;
    const long long jt = bid / mtiles;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(&bar_free[0], 1); mbar_init(&bar_free[1], 1); mbar_init(&bar_done, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_holder)), "r"(uint32_t(NT)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = threadIdx.x; i < NT; i += kTcThreads) mo_s[i] = (mt * NT + i < g.M) ? mo[r * g.M + mt * NT + i] : 0.f;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_holder;

    // staging role: position row = tid % 128, taps (tid / 128) * 8 .. + 7 of every stage
    const int prow = threadIdx.x % kTcPos, khalf = threadIdx.x / kTcPos;
    const Column sc = column_of(g, r, jt * kTcPos + prow, P, mx);
    const bool live = sc.base >= 0;
    const float* xs = x + (size_t)sc.n * g.C * g.H * g.W;
    const float eps = float(g.eps), oob = float(g.oob);
    const float* btiles = tiles + ((size_t)r * mtiles + mt) * kchunks * 2 * NT * kTcKT;
    constexpr uint32_t idesc = umma_idesc(NT);
    bool ok = true;

    for (int c = 0; c < kchunks; ++c) {
        const int stage = c & 1;
        unsigned char* sA = dsm + stage * STAGE_BYTES;           // [hi | lo] position operand
        unsigned char* sB = sA + 2 * A_BYTES;                    // [hi | lo] instance operand
        // the MMAs that last read this stage (chunk c - 2) must have completed
        if (c >= 2 && ok) ok = mbar_wait(&bar_free[stage], uint32_t((c >> 1) - 1) & 1u);
        // instance operand: verbatim copy of the pre-split tile (hi plane then lo plane, contiguous)
        {
            const float* src = btiles + (size_t)c * 2 * NT * kTcKT;
            for (int v = threadIdx.x; v < 2 * B_BYTES / 16; v += kTcThreads)
                cp_async16(reinterpret_cast<float*>(sB) + v * 4, src + v * 4, 16);
        }
        // position operand: 8 taps of this thread's position
        {
            float e[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = c * kTcKT + khalf * 8 + u;
                float v = 0.f;
                if (live && k < g.K) {
                    const float xv = INTERIOR ? __ldg(xs + interior_index<SPATIAL1>(g, sc.c0, sc.h0, sc.w0, k))
                                              : patch_value<SPATIAL1>(g, xs, sc.c0, sc.h0, sc.w0, k, oob);
                    v = fast_exp(eps * (xv - sc.mx));
                }
                e[u] = v;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {                        // two 16-byte groups of 4 taps
                float4 hi, lo;
                hi.x = tf32_hi(e[4 * h]); hi.y = tf32_hi(e[4 * h + 1]); hi.z = tf32_hi(e[4 * h + 2]); hi.w = tf32_hi(e[4 * h + 3]);
                lo.x = e[4 * h] - hi.x; lo.y = e[4 * h + 1] - hi.y; lo.z = e[4 * h + 2] - hi.z; lo.w = e[4 * h + 3] - hi.w;
                const int off = core_offset(prow, khalf * 8 + 4 * h);
                *reinterpret_cast<float4*>(sA + off) = hi;
                *reinterpret_cast<float4*>(sA + A_BYTES + off) = lo;
            }
        }
        cp_async_wait_all();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA's async proxy
        __syncthreads();
        if (threadIdx.x == 0 && ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(sA), a_lo = a_hi + A_BYTES, b_hi = smem_u32(sB), b_lo = b_hi + B_BYTES;
#pragma unroll
            for (int ks = 0; ks < kTcKT / 8; ++ks) {                  // k-step of 8 = two 16-byte chunks = 256 bytes further
                const uint32_t o = ks * 256;
                const uint64_t dah = umma_desc(a_hi + o, 128, 512), dal = umma_desc(a_lo + o, 128, 512);
                const uint64_t dbh = umma_desc(b_hi + o, 128, 512), dbl = umma_desc(b_lo + o, 128, 512);
                umma_tf32(tmem_d, dal, dbh, idesc, (c | ks) != 0);
                umma_tf32(tmem_d, dah, dbl, idesc, 1);
                umma_tf32(tmem_d, dah, dbh, idesc, 1);
            }
            umma_commit(c + 1 < kchunks ? &bar_free[stage] : &bar_done);
        }
    }
    if (ok) ok = mbar_wait(&bar_done, 0);
    if (!ok) failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool good = failed == 0;

    // epilogue: lane = position, registers = instances.  Warps w and w + 4 share a lane quarter and split the columns.
    if (good) {
        const int quarter = warp & 3, half = warp >> 2;
        const Column col = column_of(g, r, jt * kTcPos + quarter * 32 + lane, P, mx);
        const float inv_eps = 1.f / eps, k_log = 0.69314718056f * inv_eps;
        const float cadd = col.mx + float(g.cst) * inv_eps;
        float* yb = y + (col.base >= 0 ? col.base : 0);
#pragma unroll 1
        for (int c0 = half * (NT / 2); c0 < (half + 1) * (NT / 2); c0 += 32) {
            uint32_t v[32];
            const uint32_t taddr = tmem_d + (uint32_t(quarter * 32) << 16) + uint32_t(c0);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                  "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                  "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                  "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(taddr) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (col.base >= 0) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int m = mt * NT + c0 + i;
                    if (m < g.M) __stcs(yb + (long long)m * g.N, fmaf(__log2f(__uint_as_float(v[i])), k_log, cadd + mo_s[c0 + i]));
                }
            }
        }
    } else if (threadIdx.x == 0) {
        atomicExch(&flag[1], 1);                                 // a wait expired: results of this launch are invalid
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(uint32_t(NT)) : "memory");
}

template <int NT>
cudaError_t launch_nt(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, float* y, int* flag,
                      bool sp1, bool interior, cudaStream_t s) {
    const long long P = (long long)g.B * g.rs;
    const long long blocks = ((P + kTcPos - 1) / kTcPos) * ((g.M + NT - 1) / NT) * g.R;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    constexpr int smem = 2 * (2 * kTcPos * kTcKT * 4 + 2 * NT * kTcKT * 4);
#define TC_LAUNCH(SP, IN)                                                                                               \
    do {                                                                                                                \
        static bool attr_set = false;                                                                                   \
        if (!attr_set) {                                                                                                \
            cudaError_t e = cudaFuncSetAttribute(mex_fwd_tc<NT, SP, IN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            if (e != cudaSuccess) return e;                                                                             \
            attr_set = true;                                                                                            \
        }                                                                                                               \
        mex_fwd_tc<NT, SP, IN><<<int(blocks), kTcThreads, smem, s>>>(g, x, tiles, mo, mx, y, flag);                      \
    } while (0)
    if (sp1) { if (interior) TC_LAUNCH(true, true); else TC_LAUNCH(true, false); }
    else { if (interior) TC_LAUNCH(false, true); else TC_LAUNCH(false, false); }
#undef TC_LAUNCH
    count_launch();
    return cudaGetLastError();
}

}  // namespace

int mex_tc_nt(const MexGeo& g) { return g.M > 128 ? 256 : (g.M > 64 ? 128 : 64); }

size_t mex_tc_tile_floats(const MexGeo& g) {
    const int NT = mex_tc_nt(g);
    return (size_t)g.R * ((g.M + NT - 1) / NT) * ((g.K + kTcKT - 1) / kTcKT) * 2 * NT * kTcKT;
}

cudaError_t launch_mex_tc_prep(const MexGeo& g, const float* eo, float* tiles, cudaStream_t s) {
    const int NT = mex_tc_nt(g);
    const long long total = (long long)mex_tc_tile_floats(g) / 2;
    mex_tc_prep<<<int(std::min<long long>((total + 255) / 256, 148LL * 8)), 256, 0, s>>>(g, NT, eo, tiles);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mex_fwd_tc(const MexGeo& g, const float* x, const float* tiles, const float* mo, const float* mx, float* y,
                              int* flag, bool interior, cudaStream_t s) {
    const bool sp1 = g.bh == 1 && g.bw == 1;
    switch (mex_tc_nt(g)) {
    case 256: return launch_nt<256>(g, x, tiles, mo, mx, y, flag, sp1, interior, s);
    case 128: return launch_nt<128>(g, x, tiles, mo, mx, y, flag, sp1, interior, s);
    default: return launch_nt<64>(g, x, tiles, mo, mx, y, flag, sp1, interior, s);
    }
}

}  // namespace simnets
