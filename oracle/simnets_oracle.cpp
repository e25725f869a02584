// simnets_oracle.cpp -- TEST INFRASTRUCTURE, not product code.
//
// A CPU restatement, in plain loops, of the arithmetic of the Similarity and MEX
// operators of HUJI-Deep/simnets-tf (paths below are relative to that project).
// It exists so that the CUDA library can be checked against an independent
// implementation; only tests, the smoke check and the benchmark's CPU-baseline
// leg may load it.  The product never calls into it.
//
// The loops keep the reference's order of floating-point operations (sequential
// accumulation over the patch index, per-sample accumulation of parameter
// gradients in batch order, col2im accumulation in patch-offset order), so that
// on the same machine the results agree bit for bit with the reference's own
// templates compiled by oracle/Makefile into oracle/_ref (tests/test_oracle_pin.py
// checks this, and checks both against the committed vectors in tests/golden/).
// Build with -ffp-contract=off and without -ffast-math: NaN tests are `x != x`.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#include <algorithm>

#include "simnets_b200.h"

#define ORACLE_API extern "C" __attribute__((visibility("default")))

namespace {

// include/utils/im2col.hpp:101-108
int out_size(int image, int pad, int patch, int stride, bool round_down) {
    if (round_down) return (image + 2 * pad - patch) / stride + 1;
    return static_cast<int>(std::ceil(static_cast<float>(image + 2 * pad - patch) / stride)) + 1;
}

int ceil_div(int a, int b) { return a / b + ((a % b) > 0); }   // include/utils/ggemm_cpu.hpp:451-454

// include/utils/ggemm_cpu.hpp:638-640
template <typename T> int sgn(T v) { return (T(0) < v) - (v < T(0)); }

// src/utils/im2col.cpp:247-280 : patch matrix col[p][c_out][h_out][w_out]
template <typename T>
void patches(const T* im, int C, int H, int W, int pc, int ph, int pw, int padc, int padh, int padw,
             int sc, int sh, int sw, bool round_down, T oob, T* col) {
    const int Hc = out_size(H, padh, ph, sh, round_down);
    const int Wc = out_size(W, padw, pw, sw, round_down);
    const int Cc = out_size(C, padc, pc, sc, round_down);
    const int P = pc * ph * pw;
    for (int p = 0; p < P; ++p) {
        const int wo = p % pw, ho = (p / pw) % ph, co = p / ph / pw;
        for (int c = 0; c < Cc; ++c)
            for (int h = 0; h < Hc; ++h)
                for (int w = 0; w < Wc; ++w) {
                    const int hh = h * sh - padh + ho, ww = w * sw - padw + wo, cc = c * sc - padc + co;
                    const bool in = hh >= 0 && hh < H && ww >= 0 && ww < W && cc >= 0 && cc < C;
                    col[((size_t(p) * Cc + c) * Hc + h) * Wc + w] = in ? im[(size_t(cc) * H + hh) * W + ww] : oob;
                }
    }
}

// src/utils/im2col.cpp:297-328 : accumulate the patch-matrix gradient back, p outermost
template <typename T>
void unpatches(const T* col, int C, int H, int W, int pc, int ph, int pw, int padc, int padh, int padw,
               int sc, int sh, int sw, bool round_down, T* im) {
    for (size_t i = 0; i < size_t(C) * H * W; ++i) im[i] = T(0);
    const int Hc = out_size(H, padh, ph, sh, round_down);
    const int Wc = out_size(W, padw, pw, sw, round_down);
    const int Cc = out_size(C, padc, pc, sc, round_down);
    const int P = pc * ph * pw;
    for (int p = 0; p < P; ++p) {
        const int wo = p % pw, ho = (p / pw) % ph, co = p / ph / pw;
        for (int c = 0; c < Cc; ++c)
            for (int h = 0; h < Hc; ++h)
                for (int w = 0; w < Wc; ++w) {
                    const int hh = h * sh - padh + ho, ww = w * sw - padw + wo, cc = c * sc - padc + co;
                    if (hh >= 0 && hh < H && ww >= 0 && ww < W && cc >= 0 && cc < C)
                        im[(size_t(cc) * H + hh) * W + ww] += col[((size_t(p) * Cc + c) * Hc + h) * Wc + w];
                }
    }
}

// ------------------------------------------------------------------ Similarity
struct SimDims { int B, C, H, W, M, bh, bw, sh, sw, ph, pw, oh, ow, K, N; bool one_by_one; };

// include/kernels/similarity_kernel_common.hpp:84-110 (validation), :113-164 (dimensions)
int sim_dims(const simnets_sim_desc* d, SimDims* s) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype != SIMNETS_F32 && d->dtype != SIMNETS_F64) return SIMNETS_E_DTYPE;
    if (d->similarity_function != SIMNETS_SIM_L1 && d->similarity_function != SIMNETS_SIM_L2) return SIMNETS_E_DESC;
    const bool l1_skip = (d->flags & SIMNETS_FLAG_SIM_L1_SKIP_NAN) != 0;
    if (d->normalization_term && d->similarity_function != SIMNETS_SIM_L2) return SIMNETS_E_DESC;
    if (d->ignore_nan_input && !d->normalization_term) return SIMNETS_E_DESC;
    if (l1_skip && d->similarity_function != SIMNETS_SIM_L1) return SIMNETS_E_DESC;
    if (d->batch < 0 || d->channels <= 0 || d->height <= 0 || d->width <= 0 || d->num_instances <= 0) return SIMNETS_E_DESC;
    if (d->block_h <= 0 || d->block_w <= 0 || d->stride_h <= 0 || d->stride_w <= 0 || d->pad_h < 0 || d->pad_w < 0) return SIMNETS_E_DESC;
    s->B = d->batch; s->C = d->channels; s->H = d->height; s->W = d->width; s->M = d->num_instances;
    s->bh = d->block_h; s->bw = d->block_w; s->sh = d->stride_h; s->sw = d->stride_w; s->ph = d->pad_h; s->pw = d->pad_w;
    if (s->H + 2 * s->ph < s->bh || s->W + 2 * s->pw < s->bw) return SIMNETS_E_DESC;
    s->oh = out_size(s->H, s->ph, s->bh, s->sh, true);
    s->ow = out_size(s->W, s->pw, s->bw, s->sw, true);
    s->K = s->C * s->bh * s->bw;
    s->N = s->oh * s->ow;
    s->one_by_one = s->bh == 1 && s->bw == 1 && s->sh == 1 && s->sw == 1 && s->ph == 0 && s->pw == 0;
    return SIMNETS_OK;
}

enum SimMode { L1, L1_SKIP, L2, L2N, L2N_NAN };
SimMode sim_mode(const simnets_sim_desc* d) {
    if (d->similarity_function == SIMNETS_SIM_L1) return (d->flags & SIMNETS_FLAG_SIM_L1_SKIP_NAN) ? L1_SKIP : L1;
    if (!d->normalization_term) return L2;
    return d->ignore_nan_input ? L2N_NAN : L2N;
}

// include/utils/similarity_utils.hpp:17-80
template <typename T> T sim_term(SimMode mode, T t, T w, T x, T fudge) {
    switch (mode) {
    case L1: return -w * std::abs(t - x);
    case L1_SKIP: if (x != x) return T(0); return -w * std::abs(t - x);   // extension, no reference counterpart
    case L2: return -w * (t - x) * (t - x);
    case L2N: return T(0.5) * (-w * (t - x) * (t - x) + std::log(w + fudge));
    case L2N_NAN:
        if (x != x) return T(0);
        return T(0.5) * (-w * (t - x) * (t - x) - std::log(2.0 * M_PI) + std::log(w + fudge));
    }
    return T(0);
}

// src/kernels/similarity_kernel_cpu.cpp:69-121 with ggemm_cpu (include/utils/ggemm_cpu.hpp:485-499)
template <typename T>
int sim_forward(const simnets_sim_desc* d, const T* x, const T* tmpl, const T* wts, T* y) {
    SimDims s; int rc = sim_dims(d, &s); if (rc) return rc;
    if (!x || !tmpl || !wts || !y) return SIMNETS_E_NULL;
    const SimMode mode = sim_mode(d);
    const T fudge = T(d->normalization_term_fudge);
    std::vector<T> col(size_t(s.K) * s.N);
    const size_t in_sz = size_t(s.C) * s.H * s.W, out_sz = size_t(s.M) * s.N;
    const bool quirk = (d->flags & SIMNETS_FLAG_SIM_BATCH_CONST_QUIRK) != 0;
    const T norm_const = T(T(-0.5) * T(s.K) * std::log(2.0 * M_PI));
    for (int n = 0; n < s.B; ++n) {
        patches<T>(x + n * in_sz, s.C, s.H, s.W, s.C, s.bh, s.bw, 0, s.ph, s.pw, s.C, s.sh, s.sw, true,
                   T(d->out_of_bounds_value), col.data());
        T* out = y + n * out_sz;
        for (int m = 0; m < s.M; ++m)
            for (int j = 0; j < s.N; ++j) {
                T sum = T(0);
                for (int k = 0; k < s.K; ++k)
                    sum = sum + sim_term<T>(mode, tmpl[size_t(m) * s.K + k], wts[size_t(m) * s.K + k], col[size_t(k) * s.N + j], fudge);
                out[size_t(m) * s.N + j] = sum;
            }
        if (mode == L2N) {
            // src/kernels/similarity_kernel_cpu.cpp:118-120 adds the constant to the WHOLE output tensor
            // on every batch iteration; SimilarityRef adds it once (similarity_ref_kernel_cpu.cpp:89-93).
            if (quirk) { for (size_t i = 0; i < size_t(s.B) * out_sz; ++i) y[i] += norm_const; }
            else       { for (size_t i = 0; i < out_sz; ++i) out[i] += norm_const; }
        }
    }
    return SIMNETS_OK;
}

// include/utils/similarity_utils.hpp:122-150 through ggemm_readc_cpu<TRANSPOSE_A> and col2im_3d_cpu
// (src/kernels/similarity_grad_kernel_cpu.cpp:205-268)
template <typename T>
int sim_input_grad(const simnets_sim_desc* d, const T* x, const T* tmpl, const T* wts, const T* dy, T* dx) {
    SimDims s; int rc = sim_dims(d, &s); if (rc) return rc;
    if (!x || !tmpl || !wts || !dy || !dx) return SIMNETS_E_NULL;
    const SimMode mode = sim_mode(d);
    std::vector<T> col(size_t(s.K) * s.N), dcol(size_t(s.K) * s.N);
    const size_t in_sz = size_t(s.C) * s.H * s.W, out_sz = size_t(s.M) * s.N;
    for (int n = 0; n < s.B; ++n) {
        patches<T>(x + n * in_sz, s.C, s.H, s.W, s.C, s.bh, s.bw, 0, s.ph, s.pw, s.C, s.sh, s.sw, true,
                   T(d->out_of_bounds_value), col.data());
        const T* g = dy + n * out_sz;
        for (int k = 0; k < s.K; ++k)
            for (int j = 0; j < s.N; ++j) {
                const T data = col[size_t(k) * s.N + j];
                T sum = T(0);
                for (int m = 0; m < s.M; ++m) {
                    const T t = tmpl[size_t(m) * s.K + k], w = wts[size_t(m) * s.K + k], err = g[size_t(m) * s.N + j];
                    T v;
                    switch (mode) {
                    case L1: v = err * w * sgn<T>(t - data); break;
                    case L1_SKIP: v = (data != data) ? T(0) : err * w * sgn<T>(t - data); break;
                    case L2: v = T(2) * err * w * (t - data); break;
                    case L2N: v = T(0.5) * (T(2) * err * w * (t - data)); break;
                    default: v = (data != data) ? T(0) : T(0.5) * (T(2) * err * w * (t - data)); break;
                    }
                    sum = sum + v;
                }
                dcol[size_t(k) * s.N + j] = sum;
            }
        unpatches<T>(dcol.data(), s.C, s.H, s.W, s.C, s.bh, s.bw, 0, s.ph, s.pw, s.C, s.sh, s.sw, true, dx + n * in_sz);
    }
    return SIMNETS_OK;
}

// include/utils/similarity_utils.hpp:83-119 through ggemm_readc_cpu<ADD_TO_C>
// (src/kernels/similarity_grad_kernel_cpu.cpp:84-144)
template <typename T>
int sim_params_grad(const simnets_sim_desc* d, const T* x, const T* tmpl, const T* wts, const T* dy, T* dt, T* dw) {
    SimDims s; int rc = sim_dims(d, &s); if (rc) return rc;
    if (!x || !tmpl || !wts || !dy || !dt || !dw) return SIMNETS_E_NULL;
    const SimMode mode = sim_mode(d);
    const T fudge = T(d->normalization_term_fudge);
    std::vector<T> col(size_t(s.K) * s.N);
    const size_t in_sz = size_t(s.C) * s.H * s.W, out_sz = size_t(s.M) * s.N;
    for (size_t i = 0; i < size_t(s.M) * s.K; ++i) { dt[i] = T(0); dw[i] = T(0); }
    for (int n = 0; n < s.B; ++n) {
        patches<T>(x + n * in_sz, s.C, s.H, s.W, s.C, s.bh, s.bw, 0, s.ph, s.pw, s.C, s.sh, s.sw, true,
                   T(d->out_of_bounds_value), col.data());
        const T* g = dy + n * out_sz;
        for (int m = 0; m < s.M; ++m)
            for (int k = 0; k < s.K; ++k) {
                const T t = tmpl[size_t(m) * s.K + k], w = wts[size_t(m) * s.K + k];
                T st = T(0), sw_ = T(0);
                for (int j = 0; j < s.N; ++j) {
                    const T err = g[size_t(m) * s.N + j], xv = col[size_t(k) * s.N + j];
                    T vt, vw;
                    switch (mode) {
                    case L1: vt = err * w * sgn<T>(xv - t); vw = -err * std::abs(xv - t); break;
                    case L1_SKIP:
                        if (xv != xv) { vt = T(0); vw = T(0); }
                        else { vt = err * w * sgn<T>(xv - t); vw = -err * std::abs(xv - t); }
                        break;
                    case L2: vt = T(2) * err * w * (xv - t); vw = -err * (xv - t) * (xv - t); break;
                    default:
                        if (mode == L2N_NAN && xv != xv) { vt = T(0); vw = T(0); break; }
                        vt = T(2) * err * w * (xv - t); vw = -err * (xv - t) * (xv - t);
                        vt *= T(0.5);
                        vw = T(0.5) * (vw + err / (w + fudge));
                        break;
                    }
                    st = st + vt; sw_ = sw_ + vw;
                }
                dt[size_t(m) * s.K + k] = dt[size_t(m) * s.K + k] + st;
                dw[size_t(m) * s.K + k] = dw[size_t(m) * s.K + k] + sw_;
            }
    }
    return SIMNETS_OK;
}

// src/kernels/similarity_ref_kernel_cpu.cpp:61-102 : the reference's naive second opinion
template <typename T>
int sim_naive(const simnets_sim_desc* d, const T* x, const T* tmpl, const T* wts, T* y) {
    SimDims s; int rc = sim_dims(d, &s); if (rc) return rc;
    for (int n = 0; n < s.B; ++n)
        for (int o = 0; o < s.M; ++o)
            for (int yy = 0; yy < s.oh; ++yy)
                for (int xx = 0; xx < s.ow; ++xx) {
                    T acc = T(0);
                    for (int k = 0; k < s.C; ++k)
                        for (int p = 0; p < s.bh; ++p)
                            for (int q = 0; q < s.bw; ++q) {
                                const size_t pi = ((size_t(o) * s.C + k) * s.bh + p) * s.bw + q;
                                const T u = wts[pi], z = tmpl[pi];
                                const int iy = yy * s.sh - s.ph + p, ix = xx * s.sw - s.pw + q;
                                T pixel = T(d->out_of_bounds_value);
                                if (iy >= 0 && iy < s.H && ix >= 0 && ix < s.W)
                                    pixel = x[((size_t(n) * s.C + k) * s.H + iy) * s.W + ix];
                                if (d->ignore_nan_input && std::isnan(pixel)) continue;
                                const T diff = pixel - z;
                                T value = u * (d->similarity_function == SIMNETS_SIM_L1 ? -std::abs(diff) : -(diff * diff));
                                if (d->normalization_term) {
                                    value *= 0.5;
                                    value += 0.5 * std::log(u + d->normalization_term_fudge) - 0.5 * std::log(2.0 * M_PI);
                                }
                                acc += value;
                            }
                    y[((size_t(n) * s.M + o) * s.oh + yy) * s.ow + xx] = acc;
                }
    return SIMNETS_OK;
}

// ------------------------------------------------------------------------- MEX
// src/kernels/mex_kernel_common.cpp:8-27
bool expand_spec(const int32_t* spec, const int img[3], int out[3]) {
    for (int i = 0; i < 3; ++i) out[i] = spec[i] == -1 ? img[i] : spec[i];
    return true;
}

// src/kernels/mex_kernel_common.cpp:29-58 (validation), :63-158 (geometry), :161-170
int mex_geometry(const simnets_mex_desc* d, simnets_mex_geometry* g) {
    if (!d || !g) return SIMNETS_E_NULL;
    if (d->dtype != SIMNETS_F32 && d->dtype != SIMNETS_F64) return SIMNETS_E_DTYPE;
    if (d->num_instances <= 0) return SIMNETS_E_DESC;
    if (d->batch < 0 || d->channels <= 0 || d->height <= 0 || d->width <= 0) return SIMNETS_E_DESC;
    if ((d->n_shared_offset_region != 1 && d->n_shared_offset_region != 3) ||
        (d->n_unshared_offset_region != 1 && d->n_unshared_offset_region != 3)) return SIMNETS_E_DESC;
    if (d->epsilon != d->epsilon || d->epsilon == 0.0f) return SIMNETS_E_DESC;
    const int img[3] = {d->channels, d->height, d->width};
    int pad[3], str[3];
    expand_spec(d->padding, img, pad);
    expand_spec(d->strides, img, str);
    for (int i = 0; i < 3; ++i)
        if (d->blocks[i] <= 0 || str[i] <= 0 || pad[i] < 0 || img[i] + 2 * pad[i] < d->blocks[i]) return SIMNETS_E_DESC;
    if (d->blocks[0] > d->channels) return SIMNETS_E_DESC;
    g->block_c = d->blocks[0]; g->block_h = d->blocks[1]; g->block_w = d->blocks[2];
    g->pad_c = pad[0]; g->pad_h = pad[1]; g->pad_w = pad[2];
    g->stride_c = str[0]; g->stride_h = str[1]; g->stride_w = str[2];
    const bool rd = d->blocks_round_down != 0;
    g->height_out = out_size(d->height, g->pad_h, g->block_h, g->stride_h, rd);
    g->width_out = out_size(d->width, g->pad_w, g->block_w, g->stride_w, rd);
    g->channels_out = out_size(d->channels, g->pad_c, g->block_c, g->stride_c, rd);
    const int32_t* reg = d->use_unshared_regions ? d->unshared_offset_region : d->shared_offset_region;
    const int nreg = d->use_unshared_regions ? d->n_unshared_offset_region : d->n_shared_offset_region;
    int rc_, rh_, rw_;
    if (nreg == 3) { rc_ = reg[0]; rh_ = reg[1]; rw_ = reg[2]; } else { rc_ = -1; rh_ = rw_ = reg[0]; }
    if (rh_ < 0) rh_ = g->height_out;
    rh_ = std::min(rh_, g->height_out);
    if (rw_ < 0) rw_ = g->width_out;
    rw_ = std::min(rw_, g->width_out);
    if (rc_ < 0) rc_ = g->channels_out;
    rc_ = std::min(rc_, g->channels_out);
    if (rc_ <= 0 || rh_ <= 0 || rw_ <= 0) return SIMNETS_E_DESC;
    if (!d->use_unshared_regions) {
        g->region_c = rc_; g->region_h = rh_; g->region_w = rw_;
        g->offsets_c = ceil_div(g->channels_out, rc_);
        g->offsets_h = ceil_div(g->height_out, rh_);
        g->offsets_w = ceil_div(g->width_out, rw_);
    } else {
        g->offsets_c = rc_; g->offsets_h = rh_; g->offsets_w = rw_;
        g->region_c = ceil_div(g->channels_out, rc_);
        g->region_h = ceil_div(g->height_out, rh_);
        g->region_w = ceil_div(g->width_out, rw_);
    }
    g->num_regions = g->offsets_c * g->offsets_h * g->offsets_w;
    g->region_size = g->region_c * g->region_h * g->region_w;
    g->channels_out_total = g->channels_out * d->num_instances;
    g->M = d->num_instances;
    g->K = g->block_c * g->block_h * g->block_w;
    g->N = g->channels_out * g->height_out * g->width_out;
    g->is_1x1 = (g->block_c == d->channels || (g->block_c == 1 && g->stride_c == 1)) && g->block_w == 1 && g->block_h == 1 &&
                g->stride_h == 1 && g->stride_w == 1 && g->pad_c == 0 && g->pad_h == 0 && g->pad_w == 0;
    return SIMNETS_OK;
}

// Region geometry of split_patches_cpu (include/utils/mex_utils.hpp:69-116): region index and the
// position inside the region (in the order the split buffer lists them) of output position (c,h,w).
struct RegionMap {
    const simnets_mex_geometry& g; bool unshared;
    int region_of(int c, int h, int w) const {
        const int rc = unshared ? c % g.offsets_c : c / g.region_c;
        const int rh = unshared ? h % g.offsets_h : h / g.region_h;
        const int rw = unshared ? w % g.offsets_w : w / g.region_w;
        return (rc * g.offsets_h + rh) * g.offsets_w + rw;
    }
    // position l of region r -> flat output position, or -1 when it falls outside the output
    int position(int r, int l) const {
        const int rw = r % g.offsets_w, rh = (r / g.offsets_w) % g.offsets_h, rc = r / (g.offsets_w * g.offsets_h);
        const int lw = l % g.region_w, lh = (l / g.region_w) % g.region_h, lc = l / (g.region_w * g.region_h);
        const int c = unshared ? lc * g.offsets_c + rc : rc * g.region_c + lc;
        const int h = unshared ? lh * g.offsets_h + rh : rh * g.region_h + lh;
        const int w = unshared ? lw * g.offsets_w + rw : rw * g.region_w + lw;
        if (c >= g.channels_out || h >= g.height_out || w >= g.width_out) return -1;
        return (c * g.height_out + h) * g.width_out + w;
    }
};

template <typename T> void region_table(const simnets_mex_geometry& g, bool unshared, std::vector<int>& reg) {
    RegionMap rm{g, unshared};
    reg.resize(g.N);
    for (int c = 0; c < g.channels_out; ++c)
        for (int h = 0; h < g.height_out; ++h)
            for (int w = 0; w < g.width_out; ++w)
                reg[(c * g.height_out + h) * g.width_out + w] = rm.region_of(c, h, w);
}

// src/kernels/mex_kernel_cpu.cpp:11-38 (two passes) inside the per-sample loop of :117-158
template <typename T>
int mex_forward(const simnets_mex_desc* d, const T* x, const T* off, T* y) {
    simnets_mex_geometry g; int rc = mex_geometry(d, &g); if (rc) return rc;
    if (!x || !off || !y) return SIMNETS_E_NULL;
    const T eps = T(d->epsilon);
    const T cst = d->softmax_mode ? T(0) : T(-std::log(g.K));
    const T init = eps > 0 ? -std::numeric_limits<T>::infinity() : std::numeric_limits<T>::infinity();
    std::vector<int> reg; region_table<T>(g, d->use_unshared_regions != 0, reg);
    std::vector<T> col(size_t(g.K) * g.N);
    const size_t in_sz = size_t(d->channels) * d->height * d->width, out_sz = size_t(g.M) * g.N;
    for (int n = 0; n < d->batch; ++n) {
        patches<T>(x + n * in_sz, d->channels, d->height, d->width, g.block_c, g.block_h, g.block_w, g.pad_c, g.pad_h,
                   g.pad_w, g.stride_c, g.stride_h, g.stride_w, d->blocks_round_down != 0,
                   T(d->blocks_out_of_bounds_value), col.data());
        for (int m = 0; m < g.M; ++m)
            for (int j = 0; j < g.N; ++j) {
                const T* o = off + (size_t(reg[j]) * g.M + m) * g.K;
                T mx = init;
                for (int k = 0; k < g.K; ++k) {
                    const T v = o[k] + col[size_t(k) * g.N + j];
                    mx = eps > 0 ? std::max(mx, v) : std::min(mx, v);
                }
                T out = mx;
                if (std::isfinite(eps)) {
                    T sum = T(0);
                    for (int k = 0; k < g.K; ++k)
                        sum = sum + std::exp(eps * (col[size_t(k) * g.N + j] + o[k] - mx) + cst);
                    out = mx + std::log(sum) / eps;
                }
                y[n * out_sz + size_t(m) * g.N + j] = out;
            }
    }
    return SIMNETS_OK;
}

// include/utils/mex_utils.hpp:31-45
template <typename T> T mex_weight(bool finite, T eps, T cst, T data, T offset, T top, T top_diff) {
    if (finite) return top_diff * std::exp(eps * (data + offset - top) + cst);
    return top_diff * ((data + offset) == top);
}

// src/kernels/mex_grad_kernel_cpu.cpp:117-207
template <typename T>
int mex_input_grad(const simnets_mex_desc* d, const T* x, const T* off, const T* y, const T* dy, T* dx) {
    simnets_mex_geometry g; int rc = mex_geometry(d, &g); if (rc) return rc;
    if (!x || !off || !y || !dy || !dx) return SIMNETS_E_NULL;
    const T eps = T(d->epsilon);
    const T cst = d->softmax_mode ? T(0) : T(-std::log(g.K));
    const bool finite = std::isfinite(d->epsilon);
    std::vector<int> reg; region_table<T>(g, d->use_unshared_regions != 0, reg);
    std::vector<T> col(size_t(g.K) * g.N), dcol(size_t(g.K) * g.N);
    const size_t in_sz = size_t(d->channels) * d->height * d->width, out_sz = size_t(g.M) * g.N;
    for (int n = 0; n < d->batch; ++n) {
        patches<T>(x + n * in_sz, d->channels, d->height, d->width, g.block_c, g.block_h, g.block_w, g.pad_c, g.pad_h,
                   g.pad_w, g.stride_c, g.stride_h, g.stride_w, d->blocks_round_down != 0,
                   T(d->blocks_out_of_bounds_value), col.data());
        for (int k = 0; k < g.K; ++k)
            for (int j = 0; j < g.N; ++j) {
                const T data = col[size_t(k) * g.N + j];
                T sum = T(0);
                for (int m = 0; m < g.M; ++m)
                    sum = sum + mex_weight<T>(finite, eps, cst, data, off[(size_t(reg[j]) * g.M + m) * g.K + k],
                                              y[n * out_sz + size_t(m) * g.N + j], dy[n * out_sz + size_t(m) * g.N + j]);
                dcol[size_t(k) * g.N + j] = sum;
            }
        unpatches<T>(dcol.data(), d->channels, d->height, d->width, g.block_c, g.block_h, g.block_w, g.pad_c, g.pad_h,
                     g.pad_w, g.stride_c, g.stride_h, g.stride_w, d->blocks_round_down != 0, dx + n * in_sz);
    }
    return SIMNETS_OK;
}

// src/kernels/mex_grad_kernel_cpu.cpp:298-368 : per sample, per region, positions in split-buffer order
template <typename T>
int mex_offsets_grad(const simnets_mex_desc* d, const T* x, const T* off, const T* y, const T* dy, T* doff) {
    simnets_mex_geometry g; int rc = mex_geometry(d, &g); if (rc) return rc;
    if (!x || !off || !y || !dy || !doff) return SIMNETS_E_NULL;
    const T eps = T(d->epsilon);
    const T cst = d->softmax_mode ? T(0) : T(-std::log(g.K));
    const bool finite = std::isfinite(d->epsilon);
    RegionMap rm{g, d->use_unshared_regions != 0};
    std::vector<T> col(size_t(g.K) * g.N);
    const size_t in_sz = size_t(d->channels) * d->height * d->width, out_sz = size_t(g.M) * g.N;
    for (size_t i = 0; i < size_t(g.num_regions) * g.M * g.K; ++i) doff[i] = T(0);
    std::vector<int> pos(size_t(g.num_regions) * g.region_size);
    for (int r = 0; r < g.num_regions; ++r)
        for (int l = 0; l < g.region_size; ++l) pos[size_t(r) * g.region_size + l] = rm.position(r, l);
    for (int n = 0; n < d->batch; ++n) {
        patches<T>(x + n * in_sz, d->channels, d->height, d->width, g.block_c, g.block_h, g.block_w, g.pad_c, g.pad_h,
                   g.pad_w, g.stride_c, g.stride_h, g.stride_w, d->blocks_round_down != 0,
                   T(d->blocks_out_of_bounds_value), col.data());
        for (int r = 0; r < g.num_regions; ++r)
            for (int m = 0; m < g.M; ++m)
                for (int k = 0; k < g.K; ++k) {
                    const T o = off[(size_t(r) * g.M + m) * g.K + k];
                    T sum = T(0);
                    for (int l = 0; l < g.region_size; ++l) {
                        const int j = pos[size_t(r) * g.region_size + l];
                        if (j < 0) continue;   // the reference feeds zeroed (y, dy, x) here: an exact +0 term
                        sum = sum + mex_weight<T>(finite, eps, cst, col[size_t(k) * g.N + j], o,
                                                  y[n * out_sz + size_t(m) * g.N + j], dy[n * out_sz + size_t(m) * g.N + j]);
                    }
                    T& dst = doff[(size_t(r) * g.M + m) * g.K + k];
                    dst = dst + sum;
                }
    }
    return SIMNETS_OK;
}

// src/kernels/mex_kernel_cpu.cpp:162-207,256-286 : the reference's naive second opinion (MexRef)
template <typename T>
int mex_naive(const simnets_mex_desc* d, const T* x, const T* off, T* y) {
    simnets_mex_geometry g; int rc = mex_geometry(d, &g); if (rc) return rc;
    RegionMap rm{g, d->use_unshared_regions != 0};
    const T eps = T(d->epsilon);
    for (int n = 0; n < d->batch; ++n)
        for (int m = 0; m < g.M; ++m)
            for (int c = 0; c < g.channels_out; ++c)
                for (int h = 0; h < g.height_out; ++h)
                    for (int w = 0; w < g.width_out; ++w) {
                        const int r = rm.region_of(c, h, w);
                        std::vector<T> v(g.K);
                        for (int k = 0; k < g.K; ++k) {
                            const int kw = k % g.block_w, kh = (k / g.block_w) % g.block_h, kc = k / (g.block_w * g.block_h);
                            const int cc = c * g.stride_c - g.pad_c + kc, hh = h * g.stride_h - g.pad_h + kh,
                                      ww = w * g.stride_w - g.pad_w + kw;
                            T val = T(d->blocks_out_of_bounds_value);
                            if (cc >= 0 && cc < d->channels && hh >= 0 && hh < d->height && ww >= 0 && ww < d->width)
                                val = x[((size_t(n) * d->channels + cc) * d->height + hh) * d->width + ww];
                            v[k] = val + off[(size_t(r) * g.M + m) * g.K + k];
                        }
                        T mm = v[0];
                        for (int k = 0; k < g.K; ++k) mm = eps > 0 ? std::max(mm, v[k]) : std::min(mm, v[k]);
                        T out = mm;
                        if (std::isfinite(eps)) {
                            T sum = 0;
                            for (int k = 0; k < g.K; ++k) sum += std::exp(eps * (v[k] - mm));
                            out = std::log(sum / (d->softmax_mode ? 1 : g.K)) / eps + mm;
                        }
                        y[((size_t(n) * g.M + m) * g.channels_out + c) * g.height_out * g.width_out + size_t(h) * g.width_out + w] = out;
                    }
    return SIMNETS_OK;
}

}  // namespace

#define CP(T, p) static_cast<const T*>(p)
#define MP(T, p) static_cast<T*>(p)

ORACLE_API const char* oracle_kind(void) { return "port"; }

ORACLE_API int oracle_similarity_output_dims(const simnets_sim_desc* d, int32_t* oh, int32_t* ow) {
    SimDims s; int rc = sim_dims(d, &s); if (rc) return rc;
    *oh = s.oh; *ow = s.ow; return SIMNETS_OK;
}
ORACLE_API int oracle_similarity_forward(const simnets_sim_desc* d, const void* x, const void* t, const void* w, void* y) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype == SIMNETS_F32) return sim_forward<float>(d, CP(float, x), CP(float, t), CP(float, w), MP(float, y));
    if (d->dtype == SIMNETS_F64) return sim_forward<double>(d, CP(double, x), CP(double, t), CP(double, w), MP(double, y));
    return SIMNETS_E_DTYPE;
}
ORACLE_API int oracle_similarity_naive(const simnets_sim_desc* d, const void* x, const void* t, const void* w, void* y) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype == SIMNETS_F32) return sim_naive<float>(d, CP(float, x), CP(float, t), CP(float, w), MP(float, y));
    if (d->dtype == SIMNETS_F64) return sim_naive<double>(d, CP(double, x), CP(double, t), CP(double, w), MP(double, y));
    return SIMNETS_E_DTYPE;
}
ORACLE_API int oracle_similarity_input_grad(const simnets_sim_desc* d, const void* x, const void* t, const void* w,
                                            const void* dy, void* dx) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype == SIMNETS_F32) return sim_input_grad<float>(d, CP(float, x), CP(float, t), CP(float, w), CP(float, dy), MP(float, dx));
    if (d->dtype == SIMNETS_F64) return sim_input_grad<double>(d, CP(double, x), CP(double, t), CP(double, w), CP(double, dy), MP(double, dx));
    return SIMNETS_E_DTYPE;
}
ORACLE_API int oracle_similarity_params_grad(const simnets_sim_desc* d, const void* x, const void* t, const void* w,
                                             const void* dy, void* dt, void* dw) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype == SIMNETS_F32) return sim_params_grad<float>(d, CP(float, x), CP(float, t), CP(float, w), CP(float, dy), MP(float, dt), MP(float, dw));
    if (d->dtype == SIMNETS_F64) return sim_params_grad<double>(d, CP(double, x), CP(double, t), CP(double, w), CP(double, dy), MP(double, dt), MP(double, dw));
    return SIMNETS_E_DTYPE;
}
ORACLE_API int oracle_mex_dims(const simnets_mex_desc* d, simnets_mex_geometry* g) { return mex_geometry(d, g); }
ORACLE_API int oracle_mex_forward(const simnets_mex_desc* d, const void* x, const void* off, void* y) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype == SIMNETS_F32) return mex_forward<float>(d, CP(float, x), CP(float, off), MP(float, y));
    if (d->dtype == SIMNETS_F64) return mex_forward<double>(d, CP(double, x), CP(double, off), MP(double, y));
    return SIMNETS_E_DTYPE;
}
ORACLE_API int oracle_mex_naive(const simnets_mex_desc* d, const void* x, const void* off, void* y) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype == SIMNETS_F32) return mex_naive<float>(d, CP(float, x), CP(float, off), MP(float, y));
    if (d->dtype == SIMNETS_F64) return mex_naive<double>(d, CP(double, x), CP(double, off), MP(double, y));
    return SIMNETS_E_DTYPE;
}
ORACLE_API int oracle_mex_input_grad(const simnets_mex_desc* d, const void* x, const void* off, const void* y,
                                     const void* dy, void* dx) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype == SIMNETS_F32) return mex_input_grad<float>(d, CP(float, x), CP(float, off), CP(float, y), CP(float, dy), MP(float, dx));
    if (d->dtype == SIMNETS_F64) return mex_input_grad<double>(d, CP(double, x), CP(double, off), CP(double, y), CP(double, dy), MP(double, dx));
    return SIMNETS_E_DTYPE;
}
ORACLE_API int oracle_mex_offsets_grad(const simnets_mex_desc* d, const void* x, const void* off, const void* y,
                                       const void* dy, void* doff) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype == SIMNETS_F32) return mex_offsets_grad<float>(d, CP(float, x), CP(float, off), CP(float, y), CP(float, dy), MP(float, doff));
    if (d->dtype == SIMNETS_F64) return mex_offsets_grad<double>(d, CP(double, x), CP(double, off), CP(double, y), CP(double, dy), MP(double, doff));
    return SIMNETS_E_DTYPE;
}
