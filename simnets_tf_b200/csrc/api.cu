// C ABI of the library (include/simnets_b200.h): validates descriptors, picks a kernel family and
// enqueues it on the caller's stream.  No entry point here allocates, frees or synchronises.
#include <atomic>
#include <cmath>
#include <cstdio>
#include "simnets_b200.h"
#include "host_dims.hpp"
#include "kernels.cuh"

namespace simnets {
static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(uint64_t(n), std::memory_order_relaxed); }
int device_sm_count() {
    static std::atomic<int> sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = sms[dev].load(std::memory_order_relaxed);
    if (!n) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}
}  // namespace simnets

using namespace simnets;

namespace {
inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }
inline int from_cuda(cudaError_t e) { return e == cudaSuccess ? SIMNETS_OK : int(e); }
}  // namespace

extern "C" {

int simnets_abi_version(void) { return 1; }
uint64_t simnets_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* simnets_status_string(int status) {
    switch (status) {
    case SIMNETS_OK: return "ok";
    case SIMNETS_E_NULL: return "a required pointer is NULL";
    case SIMNETS_E_DESC: return "invalid descriptor (fails the operator's attribute / shape validation)";
    case SIMNETS_E_DTYPE: return "dtype must be float32 (0) or float64 (1)";
    case SIMNETS_E_WORKSPACE: return "workspace missing or smaller than the *_workspace_bytes query";
    case SIMNETS_E_UNSUPPORTED: return "valid descriptor outside the supported index range";
    case SIMNETS_E_TOO_LARGE: return "problem exceeds the fixed capacity of this entry point";
    default: break;
    }
    if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
    return "unknown status";
}

/* ------------------------------------------------------------- Similarity */
int simnets_similarity_output_dims(const simnets_sim_desc* d, int32_t* out_h, int32_t* out_w) {
    SimGeo g;
    const int rc = sim_geometry(d, &g);
    if (rc) return rc;
    if (!out_h || !out_w) return SIMNETS_E_NULL;
    *out_h = g.oh; *out_w = g.ow;
    return SIMNETS_OK;
}

size_t simnets_similarity_workspace_bytes(const simnets_sim_desc* d) {
    SimGeo g;
    if (sim_geometry(d, &g)) return 0;
    return sim_workspace_bytes(g, d->dtype == SIMNETS_F64, d->flags);
}

int simnets_similarity_forward(const simnets_sim_desc* d, const void* x, const void* t, const void* w, void* y,
                               void* ws, size_t ws_bytes, void* stream) {
    SimGeo g;
    const int rc = sim_geometry(d, &g);
    if (rc) return rc;
    if (!t || !w || (g.B > 0 && (!x || !y))) return SIMNETS_E_NULL;   // batch-sized tensors may be NULL when batch == 0
    const bool f64 = d->dtype == SIMNETS_F64;
    if (sim_use_tiled(g, f64, d->flags)) {
        if (!ws || ws_bytes < sim_workspace_bytes(g, f64, d->flags)) return SIMNETS_E_WORKSPACE;
        return from_cuda(launch_sim_fwd_tiled(g, (const float*)x, (const float*)t, (const float*)w, (float*)y, ws, d->flags, as_stream(stream)));
    }
    return from_cuda(launch_sim_fwd_direct(g, f64, x, t, w, y, as_stream(stream)));
}

int simnets_similarity_forward_extrema(const simnets_sim_desc* d, const void* x, const void* t, const void* w, void* y, void* ch_max, void* ch_min,
                                       void* ws, size_t ws_bytes, void* stream) {
    SimGeo g;
    const int rc = sim_geometry(d, &g);
    if (rc) return rc;
    if (d->dtype != SIMNETS_F32) return SIMNETS_E_UNSUPPORTED;
    if (!t || !w || (g.B > 0 && (!x || !y))) return SIMNETS_E_NULL;
    if (g.B == 0) return SIMNETS_OK;
    if (sim_use_tiled(g, false, d->flags)) {
        if (!ws || ws_bytes < sim_workspace_bytes(g, false, d->flags)) return SIMNETS_E_WORKSPACE;
        return from_cuda(launch_sim_fwd_tiled(g, (const float*)x, (const float*)t, (const float*)w, (float*)y, ws, d->flags, as_stream(stream),
                                              (float*)ch_max, (float*)ch_min));
    }
    const cudaError_t e = launch_sim_fwd_direct(g, false, x, t, w, y, as_stream(stream));
    if (e != cudaSuccess) return from_cuda(e);
    return from_cuda(launch_sim_extrema(g, (const float*)y, (float*)ch_max, (float*)ch_min, as_stream(stream)));
}

void* simnets_mex_workspace_maxima(const simnets_mex_desc* d, void* workspace) {
    MexGeo g;
    if (!d || !workspace || mex_geometry(d, nullptr, &g)) return nullptr;
    if (!mex_use_tiled(g, d->dtype == SIMNETS_F64, d->flags)) return nullptr;
    return mex_workspace_maxima(g, workspace, d->flags);
}

int simnets_similarity_input_grad(const simnets_sim_desc* d, const void* x, const void* t, const void* w, const void* dy,
                                  void* dx, void* ws, size_t ws_bytes, void* stream) {
    SimGeo g;
    const int rc = sim_geometry(d, &g);
    if (rc) return rc;
    if (!t || !w || (g.B > 0 && (!x || !dy || !dx))) return SIMNETS_E_NULL;
    const bool f64 = d->dtype == SIMNETS_F64;
    if (sim_use_tiled(g, f64, d->flags)) {
        if (!ws || ws_bytes < sim_workspace_bytes(g, f64, d->flags)) return SIMNETS_E_WORKSPACE;
        return from_cuda(launch_sim_dx_tiled(g, (const float*)x, (const float*)t, (const float*)w, (const float*)dy, (float*)dx, ws, as_stream(stream)));
    }
    return from_cuda(launch_sim_dx_direct(g, f64, x, t, w, dy, dx, as_stream(stream)));
}

int simnets_similarity_params_grad(const simnets_sim_desc* d, const void* x, const void* t, const void* w, const void* dy,
                                   void* dt, void* dw, void* ws, size_t ws_bytes, void* stream) {
    SimGeo g;
    const int rc = sim_geometry(d, &g);
    if (rc) return rc;
    if (!t || !w || !dt || !dw || (g.B > 0 && (!x || !dy))) return SIMNETS_E_NULL;
    const bool f64 = d->dtype == SIMNETS_F64;
    const bool acc = (d->flags & SIMNETS_FLAG_ACCUMULATE) != 0;
    if (sim_use_tiled(g, f64, d->flags)) {
        if (!ws || ws_bytes < sim_workspace_bytes(g, f64, d->flags)) return SIMNETS_E_WORKSPACE;
        return from_cuda(launch_sim_dparams_tiled(g, (const float*)x, (const float*)t, (const float*)w, (const float*)dy,
                                                  (float*)dt, (float*)dw, acc, ws, as_stream(stream)));
    }
    return from_cuda(launch_sim_dparams_direct(g, f64, x, t, w, dy, dt, dw, acc, as_stream(stream)));
}

/* -------------------------------------------------------------------- MEX */
int simnets_mex_dims(const simnets_mex_desc* d, simnets_mex_geometry* out) {
    if (!out) return SIMNETS_E_NULL;
    return mex_geometry(d, out, nullptr);
}

int get_mex_offsets_nregions(int n_input_dim, const int* input_dim, int n_padding, const int* padding, int n_strides,
                             const int* strides, int num_instances, int blocks_round_down, int use_unshared_regions,
                             int n_blocks, const int* blocks, int n_shared, const int* shared, int n_unshared,
                             const int* unshared) {
    if (!input_dim || !padding || !strides || !blocks || !shared || !unshared) return -1;
    if (n_input_dim != 3 || n_blocks != 3) return -1;
    if (n_shared < 1 || n_unshared < 1) return -1;
    simnets_mex_desc d = {};
    d.dtype = SIMNETS_F32;
    d.batch = 1; d.channels = input_dim[0]; d.height = input_dim[1]; d.width = input_dim[2];
    d.num_instances = num_instances;
    auto three = [](int n, const int* v, int32_t* dst) {
        if (n == 1) { dst[0] = dst[1] = dst[2] = v[0]; return true; }          // broadcast
        if (n == 2) { dst[0] = -1; dst[1] = v[0]; dst[2] = v[1]; return true; } // as ExpandDimSpec prepends -1
        if (n == 3) { dst[0] = v[0]; dst[1] = v[1]; dst[2] = v[2]; return true; }
        return false;
    };
    if (!three(n_padding, padding, d.padding) || !three(n_strides, strides, d.strides)) return -1;
    for (int a = 0; a < 3; ++a) d.blocks[a] = blocks[a];
    d.epsilon = 1.0f;
    d.blocks_round_down = blocks_round_down > 0;
    d.use_unshared_regions = use_unshared_regions > 0;
    // A region list that is not three long stands for its first entry applied to height and width, as
    // MexDimensionsData::CalculateDimensions reads it (src/kernels/mex_kernel_common.cpp:86-93, 113-120); the op itself
    // accepts one or three entries only (mex_kernel_common.cpp:51-54), this helper any length, like the reference's.
    auto region = [](int n, const int* v, int32_t* dst, int32_t* n_dst) {
        if (n == 3) { dst[0] = v[0]; dst[1] = v[1]; dst[2] = v[2]; *n_dst = 3; }
        else { dst[0] = v[0]; *n_dst = 1; }
    };
    region(n_shared, shared, d.shared_offset_region, &d.n_shared_offset_region);
    region(n_unshared, unshared, d.unshared_offset_region, &d.n_unshared_offset_region);
    simnets_mex_geometry g;
    if (mex_geometry(&d, &g, nullptr)) return -1;
    return g.num_regions;
}

size_t simnets_mex_workspace_bytes(const simnets_mex_desc* d) {
    MexGeo g;
    if (mex_geometry(d, nullptr, &g)) return 0;
    return mex_workspace_bytes(g, d->dtype == SIMNETS_F64, d->flags);
}

int simnets_mex_forward(const simnets_mex_desc* d, const void* x, const void* off, void* y, void* ws, size_t ws_bytes, void* stream) {
    MexGeo g;
    const int rc = mex_geometry(d, nullptr, &g);
    if (rc) return rc;
    if (!off || (g.B > 0 && (!x || !y))) return SIMNETS_E_NULL;
    const bool f64 = d->dtype == SIMNETS_F64;
    if ((d->flags & SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS) && g.B > 0 && !mex_use_tiled(g, f64, d->flags)) return SIMNETS_E_UNSUPPORTED;
    if (mex_use_tiled(g, f64, d->flags)) {
        if (!ws || ws_bytes < mex_workspace_bytes(g, f64, d->flags)) return SIMNETS_E_WORKSPACE;
        return from_cuda(launch_mex_fwd_tiled(g, (const float*)x, (const float*)off, (float*)y, ws, d->flags, as_stream(stream)));
    }
    return from_cuda(launch_mex_fwd_direct(g, f64, x, off, y, as_stream(stream)));
}

size_t simnets_softmax_cross_entropy_workspace_bytes(int32_t batch) { return softmax_xent_workspace_bytes(batch < 0 ? 0 : batch); }

int simnets_softmax_cross_entropy(int32_t batch, int32_t classes, float scale, const float* logits, const int64_t* labels, float* loss,
                                  float* dlogits, void* ws, size_t ws_bytes, void* stream) {
    if (batch < 0 || classes < 1) return SIMNETS_E_DESC;
    if (!loss || (batch > 0 && (!logits || !labels))) return SIMNETS_E_NULL;
    if (!ws || ws_bytes < softmax_xent_workspace_bytes(batch)) return SIMNETS_E_WORKSPACE;
    return from_cuda(launch_softmax_xent(batch, classes, scale, logits, reinterpret_cast<const long long*>(labels), loss, dlogits, ws,
                                         as_stream(stream)));
}

int simnets_mex_forward_pool2x2(const simnets_mex_desc* d, const void* x, const void* off, void* y, void* y_pooled, void* ws, size_t ws_bytes,
                                void* stream) {
    MexGeo g;
    const int rc = mex_geometry(d, nullptr, &g);
    if (rc) return rc;
    if (d->dtype != SIMNETS_F32 || g.Ho % 2 || g.Wo % 2) return SIMNETS_E_UNSUPPORTED;
    if (!off || (g.B > 0 && (!x || !y || !y_pooled))) return SIMNETS_E_NULL;
    if (g.B == 0) return SIMNETS_OK;
    if (mex_use_tiled(g, false, d->flags)) {
        if (!ws || ws_bytes < mex_workspace_bytes(g, false, d->flags)) return SIMNETS_E_WORKSPACE;
        return from_cuda(launch_mex_fwd_tiled(g, (const float*)x, (const float*)off, (float*)y, ws, d->flags, as_stream(stream), (float*)y_pooled));
    }
    if (d->flags & SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS) return SIMNETS_E_UNSUPPORTED;
    const cudaError_t e = launch_mex_fwd_direct(g, false, x, off, y, as_stream(stream));
    if (e != cudaSuccess) return from_cuda(e);
    return from_cuda(launch_sum_pool2((long long)g.B * g.M * g.Co, g.Ho, g.Wo, (const float*)y, (float*)y_pooled, as_stream(stream)));
}

int simnets_similarity_workspace_status(const void* ws, void* stream, int32_t* host_out) {
    if (!ws || !host_out) return SIMNETS_E_NULL;
    return from_cuda(cudaMemcpyAsync(host_out, ws, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, as_stream(stream)));
}

int simnets_mex_workspace_status(const void* ws, void* stream, int32_t* host_out) {
    if (!ws || !host_out) return SIMNETS_E_NULL;
    return from_cuda(cudaMemcpyAsync(host_out, ws, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, as_stream(stream)));
}

int simnets_mex_forward_static_scratch(const simnets_mex_desc* d, const void* x, const void* off, void* y, void* stream) {
    MexGeo g;
    const int rc = mex_geometry(d, nullptr, &g);
    if (rc) return rc;
    if (!off || (g.B > 0 && (!x || !y))) return SIMNETS_E_NULL;
    if (d->flags & SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS) return SIMNETS_E_UNSUPPORTED;
    const bool f64 = d->dtype == SIMNETS_F64;
    if (!mex_use_tiled(g, f64, d->flags))        // these shapes run on kernels that need no scratch at all
        return from_cuda(launch_mex_fwd_direct(g, f64, x, off, y, as_stream(stream)));
    return launch_mex_fwd_static(g, (const float*)x, (const float*)off, (float*)y, d->flags, as_stream(stream));
}

int simnets_mex_input_grad(const simnets_mex_desc* d, const void* x, const void* off, const void* y, const void* dy, void* dx,
                           void* ws, size_t ws_bytes, void* stream) {
    MexGeo g;
    const int rc = mex_geometry(d, nullptr, &g);
    if (rc) return rc;
    if (!off || (g.B > 0 && (!x || !y || !dy || !dx))) return SIMNETS_E_NULL;
    const bool f64 = d->dtype == SIMNETS_F64;
    if ((d->flags & SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS) && g.B > 0 && !mex_use_tiled(g, f64, d->flags)) return SIMNETS_E_UNSUPPORTED;
    if (mex_use_tiled(g, f64, d->flags)) {
        if (!ws || ws_bytes < mex_workspace_bytes(g, f64, d->flags)) return SIMNETS_E_WORKSPACE;
        return from_cuda(launch_mex_dx_tiled(g, (const float*)x, (const float*)off, (const float*)y, (const float*)dy, (float*)dx,
                                             ws, d->flags, as_stream(stream)));
    }
    return from_cuda(launch_mex_dx_direct(g, f64, x, off, y, dy, dx, as_stream(stream)));
}

int simnets_mex_offsets_grad(const simnets_mex_desc* d, const void* x, const void* off, const void* y, const void* dy,
                             void* doff, void* ws, size_t ws_bytes, void* stream) {
    MexGeo g;
    const int rc = mex_geometry(d, nullptr, &g);
    if (rc) return rc;
    if (!off || !doff || (g.B > 0 && (!x || !y || !dy))) return SIMNETS_E_NULL;
    const bool f64 = d->dtype == SIMNETS_F64;
    if ((d->flags & SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS) && g.B > 0 && !mex_use_tiled(g, f64, d->flags)) return SIMNETS_E_UNSUPPORTED;
    const bool acc = (d->flags & SIMNETS_FLAG_ACCUMULATE) != 0;
    if (mex_use_tiled(g, f64, d->flags)) {
        if (!ws || ws_bytes < mex_workspace_bytes(g, f64, d->flags)) return SIMNETS_E_WORKSPACE;
        return from_cuda(launch_mex_doff_tiled(g, (const float*)x, (const float*)off, (const float*)y, (const float*)dy,
                                               (float*)doff, acc, ws, d->flags, as_stream(stream)));
    }
    return from_cuda(launch_mex_doff_direct(g, f64, x, off, y, dy, doff, acc, as_stream(stream)));
}

int simnets_mex_backward(const simnets_mex_desc* d, const void* x, const void* off, const void* y, const void* dy,
                         void* dx, void* doff, void* ws, size_t ws_bytes, void* stream) {
    MexGeo g;
    const int rc = mex_geometry(d, nullptr, &g);
    if (rc) return rc;
    if (!off || !doff || (g.B > 0 && (!x || !y || !dy || !dx))) return SIMNETS_E_NULL;
    const bool f64 = d->dtype == SIMNETS_F64;
    if ((d->flags & SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS) && g.B > 0 && !mex_use_tiled(g, f64, d->flags)) return SIMNETS_E_UNSUPPORTED;
    const bool acc = (d->flags & SIMNETS_FLAG_ACCUMULATE) != 0;
    if (mex_use_tiled(g, f64, d->flags)) {
        if (!ws || ws_bytes < mex_workspace_bytes(g, f64, d->flags)) return SIMNETS_E_WORKSPACE;
        return from_cuda(launch_mex_backward_tiled(g, (const float*)x, (const float*)off, (const float*)y, (const float*)dy,
                                                   (float*)dx, (float*)doff, acc, ws, d->flags, as_stream(stream)));
    }
    const int r1 = from_cuda(launch_mex_dx_direct(g, f64, x, off, y, dy, dx, as_stream(stream)));
    if (r1) return r1;
    return from_cuda(launch_mex_doff_direct(g, f64, x, off, y, dy, doff, acc, as_stream(stream)));
}

int simnets_normalize_offsets_forward(int64_t rows, int32_t k, const void* off, void* out, void* stream) {
    if (rows < 0 || k < 0) return SIMNETS_E_DESC;
    if (rows > 0 && k > 0 && (!off || !out)) return SIMNETS_E_NULL;
    return from_cuda(launch_normalize_offsets_fwd(rows, k, (const float*)off, (float*)out, as_stream(stream)));
}

int simnets_normalize_offsets_backward(int64_t rows, int32_t k, const void* off, const void* dout, void* doff, void* stream) {
    if (rows < 0 || k < 0) return SIMNETS_E_DESC;
    if (rows > 0 && k > 0 && (!off || !dout || !doff)) return SIMNETS_E_NULL;
    return from_cuda(launch_normalize_offsets_bwd(rows, k, (const float*)off, (const float*)dout, (float*)doff, as_stream(stream)));
}

int64_t simnets_fp32_fma_probe(int32_t packed, int32_t iters, void* scratch, void* stream) {
    if (iters < 1 || !scratch) return SIMNETS_E_DESC;
    const int blocks = device_sm_count() * 2;                       // two CTAs of 1024 threads fill an SM
    const cudaError_t e = launch_fp32_probe(packed != 0, blocks, iters, (float*)scratch, as_stream(stream));
    if (e != cudaSuccess) return -int64_t(e) - 1000;
    return int64_t(blocks) * 1024 * 16 * iters;
}

int simnets_sum_pool2x2_forward(int64_t planes, int32_t height, int32_t width, const void* x, void* y, void* stream) {
    if (planes < 0 || height < 0 || width < 0) return SIMNETS_E_DESC;
    if (height % 2 || width % 2) return SIMNETS_E_UNSUPPORTED;
    if (planes > 0 && height > 0 && width > 0 && (!x || !y)) return SIMNETS_E_NULL;
    return from_cuda(launch_sum_pool2(planes, height, width, (const float*)x, (float*)y, as_stream(stream)));
}

}  // extern "C"
