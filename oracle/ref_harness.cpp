// ref_harness.cpp -- TEST INFRASTRUCTURE, not product code.
//
// Drives the reference's OWN CPU math -- its templates ggemm_cpu / ggemm_readc_cpu, its element
// functors, im2col_3d_cpu / col2im_3d_cpu, split_patches_cpu, interlace_cpu and
// MexDimensionsData::CalculateDimensions -- over raw pointers, without TensorFlow.  The reference
// sources are compiled where they lie (oracle/Makefile points the compiler at the reference
// checkout; nothing is copied), against the small TensorFlow test double in oracle/tf_stub.
// Only the host orchestration of the reference's OpKernel::Compute bodies is restated here, each
// function naming the body it follows; every template is instantiated with the reference's own
// template arguments.  The result, oracle/_ref/libsimnets_ref.so, exports the same entry points
// as simnets_oracle.cpp and is used to pin that restatement and to generate tests/golden/.
//
// Known, deliberate consequence of being the reference as written: for L2 + normalization_term
// without ignore_nan_input the -0.5*K*log(2*pi) constant is added to the whole output tensor on
// every batch iteration (src/kernels/similarity_kernel_cpu.cpp:118-120), whatever the flags say.
#include <cstdint>
#include <cmath>
#include <cstring>
#include <vector>
#include <algorithm>

#include "kernels/mex_kernel_common.hpp"
#include "utils/im2col.hpp"
#include "utils/ggemm_cpu.hpp"
#include "utils/similarity_utils.hpp"
#include "utils/mex_utils.hpp"

#include "simnets_b200.h"

#define ORACLE_API extern "C" __attribute__((visibility("default")))

namespace {

struct SimGeom { int B, C, H, W, M, bh, bw, sh, sw, ph, pw, oh, ow, K, N; bool is_1x1; };

// include/kernels/similarity_kernel_common.hpp:84-110,113-164
int sim_geom(const simnets_sim_desc* d, SimGeom* s) {
    if (!d) return SIMNETS_E_NULL;
    if (d->similarity_function != SIMNETS_SIM_L1 && d->similarity_function != SIMNETS_SIM_L2) return SIMNETS_E_DESC;
    if (d->normalization_term && d->similarity_function != SIMNETS_SIM_L2) return SIMNETS_E_DESC;
    if (d->ignore_nan_input && !d->normalization_term) return SIMNETS_E_DESC;
    if (d->flags & SIMNETS_FLAG_SIM_L1_SKIP_NAN) return SIMNETS_E_UNSUPPORTED;   // not a reference mode
    s->B = d->batch; s->C = d->channels; s->H = d->height; s->W = d->width; s->M = d->num_instances;
    s->bh = d->block_h; s->bw = d->block_w; s->sh = d->stride_h; s->sw = d->stride_w; s->ph = d->pad_h; s->pw = d->pad_w;
    s->oh = simnets_tf::dimension_out_size(s->H, s->ph, s->bh, s->sh, true);
    s->ow = simnets_tf::dimension_out_size(s->W, s->pw, s->bw, s->sw, true);
    s->K = s->C * s->bh * s->bw; s->N = s->oh * s->ow;
    s->is_1x1 = s->bh == 1 && s->bw == 1 && s->sh == 1 && s->sw == 1 && s->ph == 0 && s->pw == 0;
    return SIMNETS_OK;
}

template <typename T> using V2 = typename vec<T>::vec2;

// Follows SimilarityKernelCPU<T>::Compute, src/kernels/similarity_kernel_cpu.cpp:19-122
template <typename T>
int sim_fwd(const simnets_sim_desc* d, const T* x, const T* tmpl, const T* wts, T* y) {
    SimGeom s; int rc = sim_geom(d, &s); if (rc) return rc;
    std::vector<T> col(size_t(s.K) * s.N);
    std::vector<V2<T>> params(size_t(s.M) * s.K);
    interlace_cpu<T>(s.M * s.K, tmpl, wts, params.data());
    const size_t in_sz = size_t(s.C) * s.H * s.W, out_sz = size_t(s.M) * s.N;
    const T fudge = d->normalization_term_fudge;
    for (int n = 0; n < s.B; ++n) {
        const T* cb;
        if (!s.is_1x1) {
            simnets_tf::im2col_3d_cpu<T>(x + n * in_sz, s.C, s.H, s.W, s.C, s.bh, s.bw, 0, s.ph, s.pw, s.C, s.sh, s.sw,
                                         col.data(), true, d->out_of_bounds_value);
            cb = col.data();
        } else cb = x + n * in_sz;
        T* top = y + n * out_sz;
        if (d->similarity_function == SIMNETS_SIM_L1) {
            ggemm_cpu<V2<T>, T, T, uint8_t, sim_l1_forward<T>, ggemm_add<T>, false>(s.M, s.N, s.K, params.data(), cb, top, 0, 0);
        } else if (d->normalization_term) {
            if (d->ignore_nan_input)
                ggemm_cpu<V2<T>, T, T, T, sim_l2_normalized_forward<T, false, true>, ggemm_add<T>, false>(s.M, s.N, s.K, params.data(), cb, top, 0, fudge);
            else
                ggemm_cpu<V2<T>, T, T, T, sim_l2_normalized_forward<T, false, false>, ggemm_add<T>, false>(s.M, s.N, s.K, params.data(), cb, top, 0, fudge);
        } else {
            ggemm_cpu<V2<T>, T, T, uint8_t, sim_l2_forward<T, false>, ggemm_add<T>, false>(s.M, s.N, s.K, params.data(), cb, top, 0, 0);
        }
        if (d->similarity_function == SIMNETS_SIM_L2 && d->normalization_term && !d->ignore_nan_input) {
            const T c = T(-0.5) * T(s.K) * std::log(2.0 * M_PI);
            for (size_t i = 0; i < size_t(s.B) * out_sz; ++i) y[i] += c;     // whole tensor, every iteration
        }
    }
    return SIMNETS_OK;
}

// Follows SimilarityInputGradKernelCPU<T>::Compute, src/kernels/similarity_grad_kernel_cpu.cpp:158-270
template <typename T>
int sim_dx(const simnets_sim_desc* d, const T* x, const T* tmpl, const T* wts, const T* dy, T* dx) {
    SimGeom s; int rc = sim_geom(d, &s); if (rc) return rc;
    std::vector<T> col(size_t(s.K) * s.N), dcol(size_t(s.K) * s.N, T(0));
    std::vector<V2<T>> params(size_t(s.M) * s.K);
    interlace_cpu<T>(s.M * s.K, tmpl, wts, params.data());
    const size_t in_sz = size_t(s.C) * s.H * s.W, out_sz = size_t(s.M) * s.N;
    const T fudge = d->normalization_term_fudge;
    std::fill(dx, dx + size_t(s.B) * in_sz, T(0));
    for (int n = 0; n < s.B; ++n) {
        const T* cb; T* db;
        if (!s.is_1x1) {
            simnets_tf::im2col_3d_cpu<T>(x + n * in_sz, s.C, s.H, s.W, s.C, s.bh, s.bw, 0, s.ph, s.pw, s.C, s.sh, s.sw,
                                         col.data(), true, d->out_of_bounds_value);
            cb = col.data(); db = dcol.data();
        } else { cb = x + n * in_sz; db = dx + n * in_sz; }
        const T* top = dy + n * out_sz;
        if (d->similarity_function == SIMNETS_SIM_L1) {
            ggemm_readc_cpu<true, false, V2<T>, T, T, uint8_t, sim_l1_backward_bottom<T>, ggemm_add<T>, false, no_op<T>, false>(
                s.K, s.N, s.M, params.data(), top, cb, db, 0, 0);
        } else if (d->normalization_term) {
            if (d->ignore_nan_input)
                ggemm_readc_cpu<true, false, V2<T>, T, T, T, sim_l2_normalized_backward_bottom<T, false, true>, ggemm_add<T>, false, no_op<T>, false>(
                    s.K, s.N, s.M, params.data(), top, cb, db, 0, fudge);
            else
                ggemm_readc_cpu<true, false, V2<T>, T, T, T, sim_l2_normalized_backward_bottom<T, false, false>, ggemm_add<T>, false, no_op<T>, false>(
                    s.K, s.N, s.M, params.data(), top, cb, db, 0, fudge);
        } else {
            ggemm_readc_cpu<true, false, V2<T>, T, T, uint8_t, sim_l2_backward_bottom<T, false>, ggemm_add<T>, false, no_op<T>, false>(
                s.K, s.N, s.M, params.data(), top, cb, db, 0, 0);
        }
        if (!s.is_1x1)
            simnets_tf::col2im_3d_cpu<T>(db, s.C, s.H, s.W, s.C, s.bh, s.bw, 0, s.ph, s.pw, s.C, s.sh, s.sw, dx + n * in_sz, true);
    }
    return SIMNETS_OK;
}

// Follows SimilarityParametersGradKernelCPU<T>::Compute, src/kernels/similarity_grad_kernel_cpu.cpp:23-146
template <typename T>
int sim_dp(const simnets_sim_desc* d, const T* x, const T* tmpl, const T* wts, const T* dy, T* dt, T* dw) {
    SimGeom s; int rc = sim_geom(d, &s); if (rc) return rc;
    std::vector<T> col(size_t(s.K) * s.N), row(size_t(s.K) * s.N);
    std::vector<V2<T>> params(size_t(s.M) * s.K), grad(size_t(s.M) * s.K, make_vec2<T>(0, 0));
    interlace_cpu<T>(s.M * s.K, tmpl, wts, params.data());
    const size_t in_sz = size_t(s.C) * s.H * s.W, out_sz = size_t(s.M) * s.N;
    const T fudge = d->normalization_term_fudge;
    for (int n = 0; n < s.B; ++n) {
        const T* cb;
        if (!s.is_1x1) {
            simnets_tf::im2col_3d_cpu<T>(x + n * in_sz, s.C, s.H, s.W, s.C, s.bh, s.bw, 0, s.ph, s.pw, s.C, s.sh, s.sw,
                                         col.data(), true, d->out_of_bounds_value);
            cb = col.data();
        } else cb = x + n * in_sz;
        for (int k = 0; k < s.K; ++k)               // the Eigen shuffle({1,0}) of :100-103
            for (int j = 0; j < s.N; ++j) row[size_t(j) * s.K + k] = cb[size_t(k) * s.N + j];
        const T* top = dy + n * out_sz;
        if (d->similarity_function == SIMNETS_SIM_L1) {
            ggemm_readc_cpu<false, false, T, T, V2<T>, uint8_t, sim_l1_backward_weights<T>, add_vec2<T>, true, no_op<V2<T>>, false>(
                s.M, s.K, s.N, top, row.data(), params.data(), grad.data(), make_vec2<T>(0, 0), 0);
        } else if (d->normalization_term) {
            if (d->ignore_nan_input)
                ggemm_readc_cpu<false, false, T, T, V2<T>, T, sim_l2_normalized_backward_weights<T, false, true>, add_vec2<T>, true, no_op<V2<T>>, false>(
                    s.M, s.K, s.N, top, row.data(), params.data(), grad.data(), make_vec2<T>(0, 0), fudge);
            else
                ggemm_readc_cpu<false, false, T, T, V2<T>, T, sim_l2_normalized_backward_weights<T, false, false>, add_vec2<T>, true, no_op<V2<T>>, false>(
                    s.M, s.K, s.N, top, row.data(), params.data(), grad.data(), make_vec2<T>(0, 0), fudge);
        } else {
            ggemm_readc_cpu<false, false, T, T, V2<T>, uint8_t, sim_l2_backward_weights<T, false>, add_vec2<T>, true, no_op<V2<T>>, false>(
                s.M, s.K, s.N, top, row.data(), params.data(), grad.data(), make_vec2<T>(0, 0), 0);
        }
    }
    deinterlace_cpu<T>(s.M * s.K, grad.data(), dt, dw);
    return SIMNETS_OK;
}

// ------------------------------------------------------------------------- MEX
// The reference's own geometry code (src/kernels/mex_kernel_common.cpp:63-158), fed like
// get_mex_offsets_nregions feeds it (src/kernels/mex_dims_helper.cpp:16-42).
int mex_geom(const simnets_mex_desc* d, MexDimensionsData* m) {
    if (!d) return SIMNETS_E_NULL;
    if (d->num_instances <= 0) return SIMNETS_E_DESC;
    if ((d->n_shared_offset_region != 1 && d->n_shared_offset_region != 3) ||
        (d->n_unshared_offset_region != 1 && d->n_unshared_offset_region != 3)) return SIMNETS_E_DESC;
    m->padding_.assign(d->padding, d->padding + 3);
    m->strides_.assign(d->strides, d->strides + 3);
    m->blocks_.assign(d->blocks, d->blocks + 3);
    m->shared_offset_region_.assign(d->shared_offset_region, d->shared_offset_region + d->n_shared_offset_region);
    m->unshared_offset_region_.assign(d->unshared_offset_region, d->unshared_offset_region + d->n_unshared_offset_region);
    m->batch_ = d->batch; m->channels_ = d->channels; m->height_ = d->height; m->width_ = d->width;
    m->num_instances_ = d->num_instances;
    m->blocks_round_down_ = d->blocks_round_down != 0;
    m->use_unshared_regions_ = d->use_unshared_regions != 0;
    m->softmax_mode_ = d->softmax_mode != 0;
    m->epsilon_ = d->epsilon;
    m->blocks_out_of_bounds_value_ = d->blocks_out_of_bounds_value;
    m->CalculateDimensions();
    if (m->block_c_ > m->channels_) return SIMNETS_E_DESC;      // mex_kernel_common.cpp:169
    return SIMNETS_OK;
}

// mex_forward_cpu of src/kernels/mex_kernel_cpu.cpp:11-38, same template arguments
template <typename T>
void ref_mex_forward(int M, int N, int K, bool softmax_mode, T epsilon, const T* offsets, const T* in, T* out, int batch) {
    const T init_value = epsilon > 0 ? -INFINITY : INFINITY;
    if (epsilon > 0)
        ggemm_cpu<T, T, T, uint8_t, ggemm_add<T, uint8_t>, ggemm_max<T>, false, true, true, true>(M, N, K, offsets, in, out, init_value, 0, batch);
    else
        ggemm_cpu<T, T, T, uint8_t, ggemm_add<T, uint8_t>, ggemm_min<T>, false, true, true, true>(M, N, K, offsets, in, out, init_value, 0, batch);
    if (std::isfinite(epsilon))
        ggemm_readc_cpu<false, false, T, T, T, V2<T>, mex_forward_exp<T>, ggemm_add<T>, true, mex_forward_out<T>, true, true, true, true>(
            M, N, K, offsets, in, out, out, 0, make_vec2<T>(epsilon, softmax_mode ? T(0) : (T)-std::log(K)), batch);
}

template <typename T, bool REV>
void split(const MexDimensionsData& m, int dim, typename std::conditional<REV, T*, const T*>::type in, T* out) {
    split_patches_cpu<T, REV>(m.N_, dim, m.width_out_, m.height_out_, m.channels_out_, m.offsets_w_, m.offsets_h_, m.offsets_c_,
                              m.shared_offsets_region_w_, m.shared_offsets_region_h_, m.shared_offsets_region_c_, in, out,
                              m.use_unshared_regions_);
}

template <typename T>
const T* mex_col(const MexDimensionsData& m, const T* xin, std::vector<T>& col) {
    if (m.is_1x1_) return xin;
    simnets_tf::im2col_3d_cpu<T>(xin, m.channels_, m.height_, m.width_, m.block_c_, m.block_h_, m.block_w_, m.pad_c_, m.pad_h_, m.pad_w_,
                                 m.stride_c_, m.stride_h_, m.stride_w_, col.data(), m.blocks_round_down_, m.blocks_out_of_bounds_value_);
    return col.data();
}

// Follows MEXKernelCPU<T>::Compute, src/kernels/mex_kernel_cpu.cpp:60-159
template <typename T>
int mex_fwd(const simnets_mex_desc* d, const T* x, const T* off, T* y) {
    MexDimensionsData m; int rc = mex_geom(d, &m); if (rc) return rc;
    std::vector<T> col(size_t(m.K_) * m.N_), sin(size_t(m.num_regions_) * m.K_ * m.region_size_, T(0)),
        sout(size_t(m.num_regions_) * m.M_ * m.region_size_, T(0));
    const size_t in_sz = size_t(m.channels_) * m.height_ * m.width_, out_sz = size_t(m.M_) * m.N_;
    for (int n = 0; n < m.batch_; ++n) {
        const T* cb = mex_col<T>(m, x + n * in_sz, col);
        T* top = y + n * out_sz;
        if (m.num_regions_ > 1) {
            split<T, false>(m, m.K_, cb, sin.data());
            ref_mex_forward<T>(m.M_, m.region_size_, m.K_, m.softmax_mode_, T(m.epsilon_), off, sin.data(), sout.data(), m.num_regions_);
            split<T, true>(m, m.M_, top, sout.data());
        } else {
            ref_mex_forward<T>(m.M_, m.region_size_, m.K_, m.softmax_mode_, T(m.epsilon_), off, cb, top, m.num_regions_);
        }
    }
    return SIMNETS_OK;
}

// Follows MEXGradInputKernelCPU<T>::Compute, src/kernels/mex_grad_kernel_cpu.cpp:23-209
template <typename T>
int mex_dx(const simnets_mex_desc* d, const T* x, const T* off, const T* y, const T* dy, T* dx) {
    MexDimensionsData m; int rc = mex_geom(d, &m); if (rc) return rc;
    const int R = m.num_regions_, rs = m.region_size_;
    std::vector<T> col(size_t(m.K_) * m.N_), dcol(size_t(m.K_) * m.N_, T(0)), sin(size_t(R) * m.K_ * rs, T(0)), dsin(size_t(R) * m.K_ * rs, T(0)),
        sout(size_t(R) * m.M_ * rs, T(0)), dsout(size_t(R) * m.M_ * rs, T(0)), offT(size_t(R) * m.M_ * m.K_);
    std::vector<V2<T>> inter(size_t(R) * m.M_ * rs);
    for (int r = 0; r < R; ++r)                      // the Eigen shuffle({0,2,1}) of :89-94
        for (int i = 0; i < m.M_; ++i)
            for (int k = 0; k < m.K_; ++k) offT[(size_t(r) * m.K_ + k) * m.M_ + i] = off[(size_t(r) * m.M_ + i) * m.K_ + k];
    const size_t in_sz = size_t(m.channels_) * m.height_ * m.width_, out_sz = size_t(m.M_) * m.N_;
    for (int n = 0; n < m.batch_; ++n) {
        const T* cb = mex_col<T>(m, x + n * in_sz, col);
        T* cd = m.is_1x1_ ? dx + n * in_sz : dcol.data();
        const T* top = y + n * out_sz; const T* dtop = dy + n * out_sz;
        const T *pin, *pout, *pdout; T* pdin;
        if (R > 1) {
            split<T, false>(m, m.K_, cb, sin.data());
            split<T, false>(m, m.M_, top, sout.data());
            split<T, false>(m, m.M_, dtop, dsout.data());
            pin = sin.data(); pdin = dsin.data(); pout = sout.data(); pdout = dsout.data();
        } else { pin = cb; pdin = cd; pout = top; pdout = dtop; }
        interlace_cpu<T>(R * m.M_ * rs, pout, pdout, inter.data());
        if (std::isfinite(m.epsilon_))
            ggemm_readc_cpu<false, false, T, V2<T>, T, V2<T>, mex_backward_bottom_finite<T>, ggemm_add<T>, false, no_op<T, V2<T>>, false, true, true, true>(
                m.K_, rs, m.M_, offT.data(), inter.data(), pin, pdin, 0,
                make_vec2<T>(m.epsilon_, m.softmax_mode_ ? T(0) : (T)-std::log(m.K_)), R);
        else
            ggemm_readc_cpu<false, false, T, V2<T>, T, uint8_t, mex_backward_bottom_infinite<T>, ggemm_add<T>, false, no_op<T, uint8_t>, false, true, true, true>(
                m.K_, rs, m.M_, offT.data(), inter.data(), pin, pdin, 0, 0, R);
        if (R > 1) split<T, true>(m, m.K_, cd, dsin.data());
        if (!m.is_1x1_)
            simnets_tf::col2im_3d_cpu<T>(cd, m.channels_, m.height_, m.width_, m.block_c_, m.block_h_, m.block_w_, m.pad_c_, m.pad_h_, m.pad_w_,
                                         m.stride_c_, m.stride_h_, m.stride_w_, dx + n * in_sz, m.blocks_round_down_);
    }
    return SIMNETS_OK;
}

// Follows MEXGradOffsetsKernelCPU<T>::Compute, src/kernels/mex_grad_kernel_cpu.cpp:211-370
template <typename T>
int mex_doff(const simnets_mex_desc* d, const T* x, const T* off, const T* y, const T* dy, T* doff) {
    MexDimensionsData m; int rc = mex_geom(d, &m); if (rc) return rc;
    const int R = m.num_regions_, rs = m.region_size_;
    std::vector<T> col(size_t(m.K_) * m.N_, T(0)), sin(size_t(R) * m.K_ * rs, T(0)), sinT(size_t(R) * m.K_ * rs, T(0)),
        sout(size_t(R) * m.M_ * rs, T(0)), dsout(size_t(R) * m.M_ * rs, T(0));
    std::vector<V2<T>> inter(size_t(R) * m.M_ * rs);
    std::fill(doff, doff + size_t(R) * m.M_ * m.K_, T(0));
    const size_t in_sz = size_t(m.channels_) * m.height_ * m.width_, out_sz = size_t(m.M_) * m.N_;
    for (int n = 0; n < m.batch_; ++n) {
        const T* cb = mex_col<T>(m, x + n * in_sz, col);
        const T* top = y + n * out_sz; const T* dtop = dy + n * out_sz;
        const T *pin, *pout, *pdout;
        if (R > 1) {
            split<T, false>(m, m.K_, cb, sin.data());
            split<T, false>(m, m.M_, top, sout.data());
            split<T, false>(m, m.M_, dtop, dsout.data());
            pin = sin.data(); pout = sout.data(); pdout = dsout.data();
        } else { pin = cb; pout = top; pdout = dtop; }
        interlace_cpu<T>(R * m.M_ * rs, pout, pdout, inter.data());
        for (int r = 0; r < R; ++r)                  // the Eigen shuffle({0,2,1}) of :351-357
            for (int k = 0; k < m.K_; ++k)
                for (int l = 0; l < rs; ++l) sinT[(size_t(r) * rs + l) * m.K_ + k] = pin[(size_t(r) * m.K_ + k) * rs + l];
        if (std::isfinite(m.epsilon_))
            ggemm_readc_cpu<false, false, V2<T>, T, T, V2<T>, mex_backward_offsets_finite<T>, ggemm_add<T>, true, no_op<T, V2<T>>, false, true, true, true>(
                m.M_, m.K_, rs, inter.data(), sinT.data(), off, doff, 0,
                make_vec2<T>(m.epsilon_, m.softmax_mode_ ? T(0) : (T)-std::log(m.K_)), R);
        else
            ggemm_readc_cpu<false, false, V2<T>, T, T, uint8_t, mex_backward_offsets_infinite<T>, ggemm_add<T>, true, no_op<T, uint8_t>, false, true, true, true>(
                m.M_, m.K_, rs, inter.data(), sinT.data(), off, doff, 0, 0, R);
    }
    return SIMNETS_OK;
}

}  // namespace

#define CP(T, p) static_cast<const T*>(p)
#define MP(T, p) static_cast<T*>(p)
#define BY_DTYPE(d, F32, F64)                          \
    if (!(d)) return SIMNETS_E_NULL;                   \
    if ((d)->dtype == SIMNETS_F32) return F32;         \
    if ((d)->dtype == SIMNETS_F64) return F64;         \
    return SIMNETS_E_DTYPE;

ORACLE_API const char* oracle_kind(void) { return "reference"; }

ORACLE_API int oracle_similarity_output_dims(const simnets_sim_desc* d, int32_t* oh, int32_t* ow) {
    SimGeom s; int rc = sim_geom(d, &s); if (rc) return rc;
    *oh = s.oh; *ow = s.ow; return SIMNETS_OK;
}
ORACLE_API int oracle_similarity_forward(const simnets_sim_desc* d, const void* x, const void* t, const void* w, void* y) {
    BY_DTYPE(d, sim_fwd<float>(d, CP(float, x), CP(float, t), CP(float, w), MP(float, y)),
             sim_fwd<double>(d, CP(double, x), CP(double, t), CP(double, w), MP(double, y)))
}
ORACLE_API int oracle_similarity_input_grad(const simnets_sim_desc* d, const void* x, const void* t, const void* w, const void* dy, void* dx) {
    BY_DTYPE(d, sim_dx<float>(d, CP(float, x), CP(float, t), CP(float, w), CP(float, dy), MP(float, dx)),
             sim_dx<double>(d, CP(double, x), CP(double, t), CP(double, w), CP(double, dy), MP(double, dx)))
}
ORACLE_API int oracle_similarity_params_grad(const simnets_sim_desc* d, const void* x, const void* t, const void* w, const void* dy, void* dt, void* dw) {
    BY_DTYPE(d, sim_dp<float>(d, CP(float, x), CP(float, t), CP(float, w), CP(float, dy), MP(float, dt), MP(float, dw)),
             sim_dp<double>(d, CP(double, x), CP(double, t), CP(double, w), CP(double, dy), MP(double, dt), MP(double, dw)))
}
ORACLE_API int oracle_mex_dims(const simnets_mex_desc* d, simnets_mex_geometry* g) {
    MexDimensionsData m; int rc = mex_geom(d, &m); if (rc) return rc;
    if (!g) return SIMNETS_E_NULL;
    g->block_c = m.block_c_; g->block_h = m.block_h_; g->block_w = m.block_w_;
    g->stride_c = m.stride_c_; g->stride_h = m.stride_h_; g->stride_w = m.stride_w_;
    g->pad_c = m.pad_c_; g->pad_h = m.pad_h_; g->pad_w = m.pad_w_;
    g->channels_out = m.channels_out_; g->height_out = m.height_out_; g->width_out = m.width_out_;
    g->channels_out_total = m.channels_out_total_;
    g->region_c = m.shared_offsets_region_c_; g->region_h = m.shared_offsets_region_h_; g->region_w = m.shared_offsets_region_w_;
    g->offsets_c = m.offsets_c_; g->offsets_h = m.offsets_h_; g->offsets_w = m.offsets_w_;
    g->num_regions = m.num_regions_; g->region_size = m.region_size_;
    g->M = m.M_; g->K = m.K_; g->N = m.N_; g->is_1x1 = m.is_1x1_;
    return SIMNETS_OK;
}
ORACLE_API int oracle_mex_forward(const simnets_mex_desc* d, const void* x, const void* off, void* y) {
    BY_DTYPE(d, mex_fwd<float>(d, CP(float, x), CP(float, off), MP(float, y)),
             mex_fwd<double>(d, CP(double, x), CP(double, off), MP(double, y)))
}
ORACLE_API int oracle_mex_input_grad(const simnets_mex_desc* d, const void* x, const void* off, const void* y, const void* dy, void* dx) {
    BY_DTYPE(d, mex_dx<float>(d, CP(float, x), CP(float, off), CP(float, y), CP(float, dy), MP(float, dx)),
             mex_dx<double>(d, CP(double, x), CP(double, off), CP(double, y), CP(double, dy), MP(double, dx)))
}
ORACLE_API int oracle_mex_offsets_grad(const simnets_mex_desc* d, const void* x, const void* off, const void* y, const void* dy, void* doff) {
    BY_DTYPE(d, mex_doff<float>(d, CP(float, x), CP(float, off), CP(float, y), CP(float, dy), MP(float, doff)),
             mex_doff<double>(d, CP(double, x), CP(double, off), CP(double, y), CP(double, dy), MP(double, doff)))
}
