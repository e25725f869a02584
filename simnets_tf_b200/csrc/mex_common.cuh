// Shared by the MEX kernel files: workspace carve-up, tap decoding, per-position bookkeeping.
#pragma once
#include <algorithm>
#include "kernels.cuh"
#include "tile.cuh"

namespace simnets {
namespace {

constexpr float kSafeSpread = 60.0f;

struct MexWs {           // workspace carve-up, every part 256-byte aligned
    int* flag;           // != 0: factorisation unsafe, take the exact kernels
    float* mo;           // [R][M]
    float* eo;           // [R][M][Kp]  Eo, offsets layout, rows padded to a multiple of 4 floats
    float* eot;          // [R][K][Mp]  Eo transposed, rows padded likewise (16-byte aligned rows for async copies)
    float* mx;           // [B][N]
    float* part;         // [S][R][M][K] split-q partial sums of the offsets gradient
    float* tc_tiles;     // Eo split into TF32 hi / lo planes, tile by tile in the tensor-core operand layout
    float* tc_tiles_dx;  // the same for the input gradient of the pair-tile kernels (rows = taps), written together with tc_tiles
    float* offn;         // [R][M][K] offsets minus their row's log-sum-exp, when the caller passes raw offsets
    float* lse;          // [R][M] that log-sum-exp
    float* dtmp;         // [R][M][K] offsets gradient with respect to the normalised rows (rows longer than 1024 taps only)
    size_t bytes;
    size_t fwd_bytes;    // bytes the forward pass touches (everything before `part`)
};

__host__ inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }
__host__ __device__ inline int pad4(int v) { return (v + 3) & ~3; }

// offsets-gradient tiling: 128 x 128 outputs (chunks of 16 positions) when both M and K fill it, else 64 x 64 (chunks of 32)
__host__ inline bool doff_big(const MexGeo& g) { return g.M >= 96 && g.K >= 96; }

// (The two specialised families below read dy at full resolution only; a pooled dy takes the general tiles.)
// Few instances over long patches (a classifier head: M = 10, K = 8192): one CTA per position instead of GEMM tiles.
__host__ inline bool smallm_shape(const MexGeo& g) { return g.gp == 1 && g.M <= 16 && g.K >= 256; }

// Short patches (K <= 32): the streaming kernels of mex_smallk.cu.
__host__ inline bool smallk_shape(const MexGeo& g) { return g.gp == 1 && g.K <= 32; }

// GEMM-sized layers (many instances, mid to long patches): the tensor-core forward of mex_tc.cu.
// (M and N bounds: the kernels keep one value per instance in shared memory and address the instances of a chunk
// with 32-bit offsets of up to 16 N elements; the same for 32 H W input elements.)
__host__ inline bool tc_shape(const MexGeo& g) {
    return !smallk_shape(g) && !smallm_shape(g) && g.M >= 48 && g.K >= 48 && g.M <= 2048 && g.N < (1 << 26) &&
           (long long)g.H * g.W < (1 << 25);
}

// Short patches under many instances: the passes are dominated by writing y or reading y and dy, one exp or log per
// element; on the tensor cores the K multiply-adds per element disappear from the instruction stream, which the
// streaming kernels of mex_smallk.cu cannot match (measured on a 4x2x2-block, 256-instance layer).
__host__ inline bool tc_smallk_shape(const MexGeo& g) {
    return smallk_shape(g) && g.K >= 8 && g.M >= 48 && g.M <= 2048 && g.N < (1 << 26) && (long long)g.H * g.W < (1 << 25);
}

// no patch reaches outside the input: no padding, and the last patch along each axis ends inside
__host__ inline bool patches_inside_input(const MexGeo& g) {
    auto inside = [](int dim, int block, int stride, int pad, int out) { return pad == 0 && (out - 1) * stride + block <= dim; };
    return inside(g.C, g.bc, g.sc, g.pc, g.Co) && inside(g.H, g.bh, g.sh, g.ph, g.Ho) && inside(g.W, g.bw, g.sw, g.pw, g.Wo);
}

__host__ inline int doff_splits(const MexGeo& g) {
    if (smallk_shape(g)) {
        const long long P = (long long)g.B * g.rs, tiles = (P + 31) / 32, ctas = (long long)((g.M + 255) / 256) * g.R;
        long long s = (device_sm_count() * 3 + ctas - 1) / ctas;
        if (s > tiles) s = tiles;
        if (s < 1) s = 1;
        if (s > 512) s = 512;
        return int(s);
    }
    if (smallm_shape(g)) {
        const long long P = (long long)g.B * g.rs, ktiles = (g.K + 255) / 256;
        long long s = (device_sm_count() * 4 + ktiles * g.R - 1) / (ktiles * g.R);
        if (s > (P + 15) / 16) s = (P + 15) / 16;
        if (s < 1) s = 1;
        if (s > 64) s = 64;
        return int(s);
    }
    const int tile = doff_big(g) ? 128 : 64, kc = doff_big(g) ? 16 : 32;
    const long long P = (long long)g.B * g.rs;
    const long long chunks = (P + kc - 1) / kc;
    const long long tiles = (long long)((g.M + tile - 1) / tile) * ((g.K + tile - 1) / tile) * g.R;
    long long s = (device_sm_count() * 2 + tiles - 1) / tiles;
    if (s > chunks) s = chunks;
    if (s < 1) s = 1;
    if (s > 64) s = 64;
    return int(s);
}

// which family a launch takes
__host__ inline bool use_tc_kernels(const MexGeo& g, uint32_t flags) {
    return !(flags & SIMNETS_FLAG_MEX_NO_TENSORCORE) && (tc_shape(g) || tc_smallk_shape(g));
}
__host__ inline bool use_smallk_kernels(const MexGeo& g, uint32_t flags) { return smallk_shape(g) && !use_tc_kernels(g, flags); }

// The layout must not depend on whether dy comes pooled: a forward call (full resolution) and the gradient calls that
// reuse its workspace (possibly with a pooled dy, for which some kernel families are not used) must find every part in
// the same place.  Sizes are therefore the larger of the two variants.
__host__ inline MexWs carve(const MexGeo& g_in, void* base) {
    MexWs w;
    char* p = static_cast<char*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { char* r = p ? p + off : nullptr; off += align256(bytes); return r; };
    MexGeo g = g_in;                      // dy at full resolution
    g.gp = 1; g.Ng = g.N;
    MexGeo gq = g;                        // dy pooled 2 x 2, where the output size allows it
    const bool poolable = g.Ho % 2 == 0 && g.Wo % 2 == 0;
    if (poolable) { gq.gp = 2; gq.Ng = g.N / 4; }
    w.flag = reinterpret_cast<int*>(take(16));
    w.mo = reinterpret_cast<float*>(take(sizeof(float) * g.R * g.M));
    w.eo = reinterpret_cast<float*>(take(sizeof(float) * (size_t)g.R * g.M * pad4(g.K)));
    w.eot = reinterpret_cast<float*>(take(sizeof(float) * (size_t)g.R * g.K * pad4(g.M)));
    w.mx = reinterpret_cast<float*>(take(sizeof(float) * (size_t)g.B * g.N));
    w.fwd_bytes = off;
    auto splits_of = [](const MexGeo& q) {
        int s = (tc_shape(q) || tc_smallk_shape(q)) ? std::max(doff_splits(q), mex_tc_doff_splits(q)) : doff_splits(q);
        if ((tc_shape(q) || tc_smallk_shape(q)) && mex_pair_shape(q)) s = std::max(s, mex_pair_doff_splits(q));
        if (mex_head_shape(q)) s = std::max(s, mex_head_splits(q));
        return s;
    };
    const int max_splits = std::max(splits_of(g), splits_of(gq));
    size_t part_floats = (size_t)max_splits * g.R * g.M * g.K;
    if (mex_head_shape(g)) part_floats = std::max(part_floats, mex_head_fwd_scratch_floats(g));      // the head's forward pass parks its slice sums here
    w.part = reinterpret_cast<float*>(take(sizeof(float) * part_floats));
    if (mex_head_shape(g)) w.fwd_bytes = off;                      // (so the forward pass of that shape reaches this far)
    // (the pair-tile kernels tile with 64 or 128 rows where the one-region kernels may use 32: room for the larger of the two)
    auto tiles_of = [](const MexGeo& q, bool* pair) {
        const bool tc = tc_shape(q) || tc_smallk_shape(q);
        *pair = *pair || (tc && mex_pair_shape(q));
        return tc ? std::max(mex_tc_tile_floats(q), mex_pair_shape(q) ? mex_pair_tile_floats(q) : size_t(0)) : size_t(0);
    };
    bool pair = false;
    const size_t tile_floats = std::max(tiles_of(g, &pair), tiles_of(gq, &pair));
    w.tc_tiles = reinterpret_cast<float*>(take(sizeof(float) * tile_floats));
    w.tc_tiles_dx = reinterpret_cast<float*>(take(pair ? sizeof(float) * tile_floats : 0));
    // raw offsets (SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS): the normalised rows for the exact kernels and each row's log-sum-exp
    w.offn = reinterpret_cast<float*>(take(sizeof(float) * (size_t)g.R * g.M * g.K));
    w.lse = reinterpret_cast<float*>(take(sizeof(float) * g.R * g.M));
    w.dtmp = reinterpret_cast<float*>(take(g.K > 1024 ? sizeof(float) * (size_t)g.R * g.M * g.K : 0));
    w.bytes = off;
    return w;
}

struct Tap { int c, h, w; };

template <bool SPATIAL1>
__device__ __forceinline__ Tap tap_of(const MexGeo& g, int k) {
    Tap t;
    if (SPATIAL1) { t.c = k; t.h = 0; t.w = 0; }
    else { t.w = k % g.bw; const int q = k / g.bw; t.h = q % g.bh; t.c = q / g.bh; }
    return t;
}

// value of tap k of the patch whose corner is (c0, h0, w0) in sample xs
template <bool SPATIAL1>
__device__ __forceinline__ float patch_value(const MexGeo& g, const float* __restrict__ xs, int c0, int h0, int w0, int k, float oob) {
    const Tap t = tap_of<SPATIAL1>(g, k);
    const int cc = c0 + t.c, hh = h0 + t.h, ww = w0 + t.w;
    if (cc >= 0 && cc < g.C && hh >= 0 && hh < g.H && ww >= 0 && ww < g.W) return __ldg(xs + ((size_t)cc * g.H + hh) * g.W + ww);
    return oob;
}

// Index of tap k of the patch at (c0, h0, w0) inside its sample, for geometries in which no patch leaves the input.
template <bool SPATIAL1>
__device__ __forceinline__ int interior_index(const MexGeo& g, int c0, int h0, int w0, int k) {
    const Tap t = tap_of<SPATIAL1>(g, k);
    return ((c0 + t.c) * g.H + h0 + t.h) * g.W + w0 + t.w;
}

// Decoded taps of a block in shared memory: decoding tap k of a c x h x w block costs two divisions and two modulos,
// which at short patches (4x2x2 blocks) was most of the instructions of the kernels that gather x tap by tap.
// Entry = (c << 16) | (h << 8) | w; usable when tap_table_ok(g), filled once per CTA before its first barrier.
constexpr int kTapTable = 1024;
__device__ __forceinline__ bool tap_table_ok(const MexGeo& g) { return g.K <= kTapTable && g.bh <= 256 && g.bw <= 256 && g.bc <= 32768; }
__device__ __forceinline__ void fill_tap_table(const MexGeo& g, int* tab) {
    if (!tap_table_ok(g)) return;
    for (int k = threadIdx.x; k < g.K; k += blockDim.x) {
        const Tap t = tap_of<false>(g, k);
        tab[k] = (t.c << 16) | (t.h << 8) | t.w;
    }
}
template <bool SPATIAL1>
__device__ __forceinline__ Tap tap_get(const MexGeo& g, const int* tab, bool tab_ok, int k) {
    if (SPATIAL1 || !tab_ok) return tap_of<SPATIAL1>(g, k);
    const int v = tab[k];
    Tap t; t.c = v >> 16; t.h = (v >> 8) & 255; t.w = v & 255;
    return t;
}
// value of a decoded tap of the patch whose corner is (c0, h0, w0) in sample xs
__device__ __forceinline__ float patch_value_at(const MexGeo& g, const float* __restrict__ xs, int c0, int h0, int w0, Tap t, float oob) {
    const int cc = c0 + t.c, hh = h0 + t.h, ww = w0 + t.w;
    if (cc >= 0 && cc < g.C && hh >= 0 && hh < g.H && ww >= 0 && ww < g.W) return __ldg(xs + ((size_t)cc * g.H + hh) * g.W + ww);
    return oob;
}

// Per-column (= one output position of one sample) bookkeeping shared by the tile kernels.
struct Column {
    long long base;      // n*M*N + pos : offset of y[n, 0, pos]; -1 for a position outside the output grid
    long long gbase;     // offset of dy[n, 0, pos] (instances g.Ng apart): equals base unless dy is given pooled
    int n, c0, h0, w0;   // sample and patch corner in the input
    float mx;
};

// j-th position (over the whole batch) of region r -> Column
__device__ __forceinline__ Column column_of(const MexGeo& g, int r, long long jl, long long P, const float* __restrict__ mx) {
    Column c;
    c.base = -1; c.gbase = 0; c.n = 0; c.c0 = c.h0 = c.w0 = 0; c.mx = 0.f;
    if (jl >= P) return c;
    int n, l;
    if (P <= 0x7fffffffLL) { const uint32_t j32 = uint32_t(jl); n = int(fast_div(j32, g.f_rs)); l = int(j32 - uint32_t(n) * uint32_t(g.rs)); }
    else { n = int(jl / g.rs); l = int(jl % g.rs); }
    int cc, h, w;
    if (!mex_region_chw(g, r, l, cc, h, w)) return c;
    const int pos = (cc * g.Ho + h) * g.Wo + w;
    c.n = n; c.c0 = cc * g.sc - g.pc; c.h0 = h * g.sh - g.ph; c.w0 = w * g.sw - g.pw;
    c.base = (long long)n * g.M * g.N + pos;
    c.gbase = c.base;
    if (g.gp == 2) c.gbase = (long long)n * g.M * g.Ng + (cc * (g.Ho >> 1) + (h >> 1)) * (g.Wo >> 1) + (w >> 1);     // gp is 1 or 2
    c.mx = mx ? mx[(long long)n * g.N + pos] : 0.f;
    return c;
}


}  // namespace
}  // namespace simnets
