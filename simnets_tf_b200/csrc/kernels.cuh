// Internal launch interface between the C ABI layer (api.cu) and the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include "simnets_b200.h"
#include "geometry.cuh"

namespace simnets {

void count_launch(int n = 1);

// offsets_norm.cu
cudaError_t launch_normalize_offsets_fwd(long long rows, int K, const float* off, float* out, cudaStream_t);
cudaError_t launch_normalize_offsets_bwd(long long rows, int K, const float* off, const float* dout, float* doff, cudaStream_t);

// probe.cu
cudaError_t launch_fp32_probe(bool packed, int blocks, int iters, float* out, cudaStream_t);

// pool.cu
// gate: when given, the kernel runs only if gate[0] | gate[1] is non-zero (the pooling behind a recomputed forward pass)
cudaError_t launch_sum_pool2(long long planes, int H, int W, const float* x, float* y, cudaStream_t, const int* gate = nullptr);

// direct_kernels.cu -- any shape, float32 and float64
// gate: when given, the kernel runs only if gate[1] is non-zero (the redo behind the tensor-core forward kernel)
cudaError_t launch_sim_fwd_direct(const SimGeo&, bool f64, const void* x, const void* t, const void* w, void* y, cudaStream_t,
                                  const int* gate = nullptr);
cudaError_t launch_sim_dx_direct(const SimGeo&, bool f64, const void* x, const void* t, const void* w, const void* dy, void* dx, cudaStream_t);
cudaError_t launch_sim_dparams_direct(const SimGeo&, bool f64, const void* x, const void* t, const void* w, const void* dy,
                                      void* dt, void* dw, bool accumulate, cudaStream_t);
// MEX launchers take an optional device flag: with `gate` non-null the kernel runs only if *gate != 0
cudaError_t launch_mex_fwd_direct(const MexGeo&, bool f64, const void* x, const void* off, void* y, cudaStream_t, const int* gate = nullptr);
cudaError_t launch_mex_dx_direct(const MexGeo&, bool f64, const void* x, const void* off, const void* y, const void* dy, void* dx, cudaStream_t,
                                 const int* gate = nullptr);
cudaError_t launch_mex_doff_direct(const MexGeo&, bool f64, const void* x, const void* off, const void* y, const void* dy,
                                   void* doff, bool accumulate, cudaStream_t, const int* gate = nullptr);

}  // namespace simnets

namespace simnets {
// tiled_*.cu -- float32 generalized-GEMM tile kernels for the hot shapes
bool sim_use_tiled(const SimGeo&, bool f64, uint32_t flags);
size_t sim_workspace_bytes(const SimGeo&, bool f64, uint32_t flags);
// ch_max / ch_min: when given, also the per-pixel extrema of y over the instances ([B][N] each)
cudaError_t launch_sim_fwd_tiled(const SimGeo&, const float* x, const float* t, const float* w, float* y, void* ws, uint32_t flags, cudaStream_t,
                                 float* ch_max = nullptr, float* ch_min = nullptr);
bool sim_tc_shape(const SimGeo&, uint32_t flags);
float* mex_workspace_maxima(const MexGeo&, void* ws, uint32_t flags);
// per-pixel maximum and minimum over the instances of a Similarity output y[B][M][N] (NaN entries ignored); either may be null
cudaError_t launch_sim_extrema(const SimGeo&, const float* y, float* ch_max, float* ch_min, cudaStream_t);
size_t sim_tc_tile_floats(const SimGeo&);
cudaError_t launch_sim_fwd_tc(const SimGeo&, const float* x, const float* planes, const float* cm, const int2* taps, float* tiles,
                              float* bias, int* flag, float* y, cudaStream_t);
cudaError_t launch_sim_dx_tiled(const SimGeo&, const float* x, const float* t, const float* w, const float* dy, float* dx, void* ws, cudaStream_t);
cudaError_t launch_sim_dparams_tiled(const SimGeo&, const float* x, const float* t, const float* w, const float* dy,
                                     float* dt, float* dw, bool accumulate, void* ws, cudaStream_t);
// sim_smallk.cu -- forward for short patches (K <= 32): patches in registers, two positions per thread
bool sim_smallk_shape(const SimGeo&);
cudaError_t launch_sim_fwd_smallk(const SimGeo&, const float* x, const float* planes, const float* cm, const int2* taps, float* y,
                                  float* ch_max, float* ch_min, cudaStream_t);
bool mex_use_tiled(const MexGeo&, bool f64, uint32_t flags);
size_t mex_workspace_bytes(const MexGeo&, bool f64, uint32_t flags);
// pooled: when given, the 2x2 sum pooling of y is produced as well (fused into the pair-tile kernel, a pooling launch behind the others)
cudaError_t launch_mex_fwd_tiled(const MexGeo&, const float* x, const float* off, float* y, void* ws, uint32_t flags, cudaStream_t,
                                 float* pooled = nullptr);
// mex_smallm.cu -- one CTA per position, for M <= 16 and K >= 256
cudaError_t launch_mex_colmax_wide(const MexGeo&, const float* x, float* mx, const int* flag, cudaStream_t);
cudaError_t launch_mex_fwd_smallm(const MexGeo&, const float* x, const float* eot, const float* mo, float* y, const int* flag, cudaStream_t);
cudaError_t launch_mex_dx_smallm(const MexGeo&, const float* x, const float* eo, const float* mo, const float* y, const float* dy,
                                 float* dx, const int* flag, cudaStream_t);
cudaError_t launch_mex_doff_smallm(const MexGeo&, const float* x, const float* mo, const float* mx, const float* y, const float* dy,
                                   float* part, int splits, const int* flag, cudaStream_t);
// the head: a single region of contiguous patches (whole samples), several positions per CTA, both gradients from one read of x
bool mex_head_shape(const MexGeo&);
int mex_head_splits(const MexGeo&);
size_t mex_head_fwd_scratch_floats(const MexGeo&);
cudaError_t launch_mex_fwd_head(const MexGeo&, const float* x, const float* eo, const float* eot, const float* mo, float* mx, float* y,
                                float* scratch, const int* flag, cudaStream_t);
cudaError_t launch_mex_bwd_head(const MexGeo&, bool want_dx, bool want_doff, const float* x, const float* eo, const float* mo,
                                const float* mx, const float* y, const float* dy, float* dx, float* part, int splits,
                                const int* flag, cudaStream_t);
// mex_smallk.cu -- one thread per position, for K <= 32 (HBM-bound streaming regime)
cudaError_t launch_mex_fwd_smallk(const MexGeo&, const float* x, const float* eo, const float* mo, float* y, const int* flag, cudaStream_t);
cudaError_t launch_mex_dx_smallk(const MexGeo&, const float* x, const float* eo, const float* mo, const float* y, const float* dy,
                                 float* dx, const int* flag, cudaStream_t);
cudaError_t launch_mex_doff_smallk(const MexGeo&, const float* x, const float* mo, const float* y, const float* dy,
                                   float* part, int slabs, const int* flag, cudaStream_t);
// mex_tc.cu -- the three MEX GEMMs on tcgen05 tensor cores (split-TF32), for GEMM-sized layers
int mex_tc_nt(const MexGeo&);
size_t mex_tc_tile_floats(const MexGeo&);
int mex_tc_doff_splits(const MexGeo&);
// nt: tile width along the rows (0: the width the one-region kernels use for this shape)
cudaError_t launch_mex_tc_prep(const MexGeo&, bool transposed, const float* src, float* tiles, cudaStream_t, int nt = 0);
cudaError_t launch_mex_fwd_tc(const MexGeo&, const float* x, const float* tiles, const float* mo, const float* mx, float* y,
                              int* flag, bool interior, cudaStream_t);
cudaError_t launch_mex_dx_tc(const MexGeo&, const float* x, const float* tiles, const float* mo, const float* mx, const float* y,
                             const float* dy, float* dx, int* flag, cudaStream_t);
cudaError_t launch_mex_doff_tc(const MexGeo&, const float* x, const float* mo, const float* mx, const float* y, const float* dy,
                               float* part, int splits, int* flag, cudaStream_t);
// mex_tc_ws.cu -- persistent, warp-specialised versions (producer / MMA / epilogue roles, double-buffered accumulator)
cudaError_t launch_mex_fwd_ws(const MexGeo&, const float* x, const float* tiles, const float* mo, const float* mx, float* y,
                              int* flag, bool interior, cudaStream_t);
cudaError_t launch_mex_dx_ws(const MexGeo&, const float* x, const float* tiles, const float* mo, const float* mx, const float* y,
                             const float* dy, float* dx, int* flag, cudaStream_t);
// mex_tc_pair.cu -- the same three passes on PAIRS of tiles of sibling regions (8-byte accesses of pixel pairs)
bool mex_pair_shape(const MexGeo&);
bool mex_pair_aligned(const void*, const void*, const void*, const void*);
int mex_pair_nt_fwd(const MexGeo&);
int mex_pair_nt_dx(const MexGeo&);
int mex_pair_doff_splits(const MexGeo&);
size_t mex_pair_tile_floats(const MexGeo&);      // floats of one set of pre-split operand tiles as the pair-tile prepass writes them
// pooled: when given, also the 2x2 sum pooling of y ([B, M * Co, Ho / 2, Wo / 2]; Ho and Wo even), added up by the epilogue
cudaError_t launch_mex_fwd_pair(const MexGeo&, const float* x, const float* tiles, const float* mo, const float* mx, float* y,
                                float* pooled, int* flag, int test_expire, cudaStream_t);
cudaError_t launch_mex_dx_pair(const MexGeo&, const float* x, const float* tiles, const float* mo, const float* mx, const float* y,
                               const float* dy, float* dx, int* flag, cudaStream_t);
cudaError_t launch_mex_doff_pair(const MexGeo&, const float* x, const float* mo, const float* mx, const float* y, const float* dy,
                                 float* part, int* splits_out, int* flag, cudaStream_t);
// number of multiprocessors of the current device (148 when no device answers)
int device_sm_count();

size_t softmax_xent_workspace_bytes(int batch);
cudaError_t launch_softmax_xent(int batch, int classes, float scale, const float* logits, const long long* labels, float* loss,
                                float* dlogits, void* ws, cudaStream_t);
// forward on the library's fixed device scratch; returns a status code of simnets_b200.h
int launch_mex_fwd_static(const MexGeo&, const float* x, const float* off, float* y, uint32_t flags, cudaStream_t);
cudaError_t launch_mex_dx_tiled(const MexGeo&, const float* x, const float* off, const float* y, const float* dy, float* dx,
                                void* ws, uint32_t flags, cudaStream_t, bool prepped = false);
cudaError_t launch_mex_backward_tiled(const MexGeo&, const float* x, const float* off, const float* y, const float* dy, float* dx,
                                      float* doff, bool accumulate, void* ws, uint32_t flags, cudaStream_t);
cudaError_t launch_mex_doff_tiled(const MexGeo&, const float* x, const float* off, const float* y, const float* dy, float* doff,
                                  bool accumulate, void* ws, uint32_t flags, cudaStream_t, bool prepped = false);
}  // namespace simnets
