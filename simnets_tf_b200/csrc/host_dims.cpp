// Descriptor validation and dimension arithmetic (host only, no CUDA calls).
//
// Similarity: the attr checks of SimilarityKernelCommon's constructor and the sizes of
// CalculateDimensions (reference include/kernels/similarity_kernel_common.hpp:84-110, 113-164).
// MEX: the attr checks of MEXKernelCommon's constructor and the region geometry of
// MexDimensionsData::CalculateDimensions (reference src/kernels/mex_kernel_common.cpp:29-58, 63-170).
#include "host_dims.hpp"
#include <cmath>

namespace simnets {

namespace {

// reference include/utils/im2col.hpp:101-108
int conv_out(int image, int pad, int patch, int stride, bool round_down) {
    const int span = image + 2 * pad - patch;
    if (round_down) return span / stride + 1;
    return static_cast<int>(std::ceil(static_cast<float>(span) / stride)) + 1;
}

int div_up(int a, int b) { return (a + b - 1) / b; }

}  // namespace

int sim_geometry(const simnets_sim_desc* d, SimGeo* g) {
    if (!d || !g) return SIMNETS_E_NULL;
    if (d->dtype != SIMNETS_F32 && d->dtype != SIMNETS_F64) return SIMNETS_E_DTYPE;
    const bool l1 = d->similarity_function == SIMNETS_SIM_L1;
    if (!l1 && d->similarity_function != SIMNETS_SIM_L2) return SIMNETS_E_DESC;
    // "normalization_term is relevant only if similarity_function is L2"
    if (d->normalization_term && l1) return SIMNETS_E_DESC;
    // "ignore_nan is relevant only if normalization_term is true"
    if (d->ignore_nan_input && !d->normalization_term) return SIMNETS_E_DESC;
    const bool l1_skip = (d->flags & SIMNETS_FLAG_SIM_L1_SKIP_NAN) != 0;
    if (l1_skip && !l1) return SIMNETS_E_DESC;
    if (d->batch < 0 || d->channels < 1 || d->height < 1 || d->width < 1 || d->num_instances < 1) return SIMNETS_E_DESC;
    if (d->block_h < 1 || d->block_w < 1 || d->stride_h < 1 || d->stride_w < 1 || d->pad_h < 0 || d->pad_w < 0) return SIMNETS_E_DESC;
    if (d->height + 2 * d->pad_h < d->block_h || d->width + 2 * d->pad_w < d->block_w) return SIMNETS_E_DESC;
    g->B = d->batch; g->C = d->channels; g->H = d->height; g->W = d->width; g->M = d->num_instances;
    g->bh = d->block_h; g->bw = d->block_w; g->sh = d->stride_h; g->sw = d->stride_w; g->ph = d->pad_h; g->pw = d->pad_w;
    g->oh = conv_out(g->H, g->ph, g->bh, g->sh, true);
    g->ow = conv_out(g->W, g->pw, g->bw, g->sw, true);
    const long long K = 1LL * g->C * g->bh * g->bw, N = 1LL * g->oh * g->ow;
    if (K > (1 << 24) || N > (1 << 28) || K * g->M > (1LL << 30)) return SIMNETS_E_UNSUPPORTED;
    g->K = int(K); g->N = int(N);
    g->mode = l1 ? (l1_skip ? SIM_L1_SKIP : SIM_L1) : (!d->normalization_term ? SIM_L2 : (d->ignore_nan_input ? SIM_L2N_NAN : SIM_L2N));
    g->batch_quirk = (d->flags & SIMNETS_FLAG_SIM_BATCH_CONST_QUIRK) != 0;
    g->absw = (d->flags & SIMNETS_FLAG_SIM_ABS_WEIGHTS) != 0;
    g->fudge = d->normalization_term_fudge;
    g->oob = d->out_of_bounds_value;
    return SIMNETS_OK;
}

int mex_geometry(const simnets_mex_desc* d, simnets_mex_geometry* o, MexGeo* g) {
    if (!d) return SIMNETS_E_NULL;
    if (d->dtype != SIMNETS_F32 && d->dtype != SIMNETS_F64) return SIMNETS_E_DTYPE;
    if (d->num_instances < 1) return SIMNETS_E_DESC;                       // "num_instances must be positive"
    if (d->batch < 0 || d->channels < 1 || d->height < 1 || d->width < 1) return SIMNETS_E_DESC;
    if (d->n_shared_offset_region != 1 && d->n_shared_offset_region != 3) return SIMNETS_E_DESC;
    if (d->n_unshared_offset_region != 1 && d->n_unshared_offset_region != 3) return SIMNETS_E_DESC;
    if (std::isnan(d->epsilon) || d->epsilon == 0.0f) return SIMNETS_E_DESC;
    const int image[3] = {d->channels, d->height, d->width};
    int pad[3], stride[3], block[3], out[3];
    for (int a = 0; a < 3; ++a) {
        pad[a] = d->padding[a] == -1 ? image[a] : d->padding[a];          // -1 stands for the image dimension
        stride[a] = d->strides[a] == -1 ? image[a] : d->strides[a];
        block[a] = d->blocks[a];
        if (block[a] < 1 || stride[a] < 1 || pad[a] < 0 || image[a] + 2 * pad[a] < block[a]) return SIMNETS_E_DESC;
        out[a] = conv_out(image[a], pad[a], block[a], stride[a], d->blocks_round_down != 0);
        if (out[a] < 1) return SIMNETS_E_DESC;
    }
    if (block[0] > d->channels) return SIMNETS_E_DESC;                     // "block depth must be smaller than input depth"

    // A region list of length 1, [d], means [-1, d, d]; -1 means the whole output extent; all clamped.
    const bool unshared = d->use_unshared_regions != 0;
    const int32_t* spec = unshared ? d->unshared_offset_region : d->shared_offset_region;
    const int nspec = unshared ? d->n_unshared_offset_region : d->n_shared_offset_region;
    int want[3];
    if (nspec == 3) { want[0] = spec[0]; want[1] = spec[1]; want[2] = spec[2]; }
    else { want[0] = -1; want[1] = want[2] = spec[0]; }
    int extent[3], count[3];
    for (int a = 0; a < 3; ++a) {
        int v = want[a] < 0 ? out[a] : want[a];
        if (v > out[a]) v = out[a];
        if (v < 1) return SIMNETS_E_DESC;
        if (unshared) { count[a] = v; extent[a] = div_up(out[a], v); }      // v distinct offset sets, interleaved
        else { extent[a] = v; count[a] = div_up(out[a], v); }               // contiguous v-wide regions
    }
    const long long K = 1LL * block[0] * block[1] * block[2], N = 1LL * out[0] * out[1] * out[2];
    const long long R = 1LL * count[0] * count[1] * count[2];
    if (K > (1 << 24) || N > (1 << 28) || R * d->num_instances * K > (1LL << 30) || N * d->num_instances > (1LL << 31) - 1)
        return SIMNETS_E_UNSUPPORTED;
    const bool one_by_one = (block[0] == d->channels || (block[0] == 1 && stride[0] == 1)) && block[1] == 1 && block[2] == 1 &&
                            stride[1] == 1 && stride[2] == 1 && pad[0] == 0 && pad[1] == 0 && pad[2] == 0;
    if (o) {
        o->block_c = block[0]; o->block_h = block[1]; o->block_w = block[2];
        o->stride_c = stride[0]; o->stride_h = stride[1]; o->stride_w = stride[2];
        o->pad_c = pad[0]; o->pad_h = pad[1]; o->pad_w = pad[2];
        o->channels_out = out[0]; o->height_out = out[1]; o->width_out = out[2];
        o->channels_out_total = out[0] * d->num_instances;
        o->region_c = extent[0]; o->region_h = extent[1]; o->region_w = extent[2];
        o->offsets_c = count[0]; o->offsets_h = count[1]; o->offsets_w = count[2];
        o->num_regions = int(R); o->region_size = extent[0] * extent[1] * extent[2];
        o->M = d->num_instances; o->K = int(K); o->N = int(N); o->is_1x1 = one_by_one;
    }
    if (g) {
        g->B = d->batch; g->C = d->channels; g->H = d->height; g->W = d->width; g->M = d->num_instances;
        g->bc = block[0]; g->bh = block[1]; g->bw = block[2];
        g->sc = stride[0]; g->sh = stride[1]; g->sw = stride[2];
        g->pc = pad[0]; g->ph = pad[1]; g->pw = pad[2];
        g->Co = out[0]; g->Ho = out[1]; g->Wo = out[2];
        g->rc = extent[0]; g->rh = extent[1]; g->rw = extent[2];
        g->oc = count[0]; g->oh = count[1]; g->ow = count[2];
        g->R = int(R); g->rs = extent[0] * extent[1] * extent[2];
        g->K = int(K); g->N = int(N);
        g->f_rs = make_fastdiv(g->rs); g->f_rw = make_fastdiv(g->rw); g->f_rh = make_fastdiv(g->rh);
        g->f_ow = make_fastdiv(g->ow); g->f_oh = make_fastdiv(g->oh);
        g->gp = (d->flags & SIMNETS_FLAG_MEX_DY_POOLED2) ? 2 : 1;
        if (out[1] % g->gp || out[2] % g->gp) return SIMNETS_E_UNSUPPORTED;
        g->Ng = out[0] * (out[1] / g->gp) * (out[2] / g->gp);
        g->unshared = unshared;
        g->finite = std::isfinite(d->epsilon);
        g->softmax = d->softmax_mode != 0;
        g->eps = d->epsilon;
        g->cst = d->softmax_mode ? 0.0 : -std::log(double(K));
        g->oob = d->blocks_out_of_bounds_value;
    }
    return SIMNETS_OK;
}

}  // namespace simnets
