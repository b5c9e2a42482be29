// C-ABI entry points of the standalone deep-learning kernels and the variant
// descriptions.  The fused pairs live in dl_pair_*.cu.
#include "dl_host.cuh"

namespace {
__global__ void bn_finalize_kernel(const double* mom, int C, float eps, float* mean, float* invstd) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const double n = mom[3 * c], mu = mom[3 * c + 1] / n;
    double var = mom[3 * c + 2] / n - mu * mu;
    if (var < 0.0) var = 0.0;
    mean[c] = (float)mu;
    invstd[c] = (float)(1.0 / sqrt(var + (double)eps));
}

}  // namespace

// ------------------------------------------------------------------ exported symbols

extern "C" {

int hfuse_im2col_f32(HFUSE_IM2COL_PARAMS(), hfuse_stream_t stream) {
    Im2colArgs a;
    if (int rc = prep_im2col(IM2COL_NAMES(), a)) return rc;
    return dispatch_solo<Im2colRole>("im2col", kDefaultSolo_im2col, a, S_(stream));
}
int hfuse_maxpool2d_f32(HFUSE_MAXPOOL_PARAMS(), hfuse_stream_t stream) {
    MaxPoolArgs a;
    if (int rc = prep_maxpool(MAXPOOL_NAMES(), a)) return rc;
    return dispatch_solo<MaxPoolRole>("maxpool", kDefaultSolo_maxpool, a, S_(stream));
}
int hfuse_bnstats_f32(HFUSE_BNSTATS_PARAMS(), hfuse_stream_t stream) {
    BnStatsArgs a;
    if (int rc = prep_bnstats(BNSTATS_NAMES(), a)) return rc;
    return dispatch_solo<BnStatsRole>("bnstats", kDefaultSolo_bnstats, a, S_(stream));
}
int hfuse_upsample_bilinear2d_f32(HFUSE_UPSAMPLE_PARAMS(), hfuse_stream_t stream) {
    UpsampleArgs a;
    if (int rc = prep_upsample(UPSAMPLE_NAMES(), a)) return rc;
    return dispatch_solo<UpsampleRole>("upsample", kDefaultSolo_upsample, a, S_(stream));
}
int hfuse_histc_f32(HFUSE_HISTC_PARAMS(), hfuse_stream_t stream) {
    HistcArgs a;
    if (int rc = prep_histc(HISTC_NAMES(), a)) return rc;
    return dispatch_solo<HistcRole>("histc", kDefaultSolo_histc, a, S_(stream));
}

size_t hfuse_bnstats_workspace_bytes(int N, int C, int HW) {
    (void)N; (void)HW;
    return C > 0 ? bn_workspace_bytes(C) : 0;
}

int hfuse_bnstats_finalize_f64(const double* moments, int C, float eps, float* mean, float* invstd,
                               hfuse_stream_t stream) {
    if (!moments || !mean || !invstd || C <= 0) return HFUSE_ERR_BAD_ARG;
    bn_finalize_kernel<<<(C + 127) / 128, 128, 0, S_(stream)>>>(moments, C, eps, mean, invstd);
    return check_launch();
}

}  // extern "C"

namespace hfuse {
// used by the tuning entry points in host_util.cu
int dl_describe(const char* name, int variant, char* buf, size_t n) {
    static const char* solos[] = {"im2col", "maxpool", "bnstats", "upsample", "histc"};
    static const char* pairs[] = {"im2col_maxpool", "im2col_bnstats", "im2col_histc", "im2col_upsample",
                                  "maxpool_bnstats", "maxpool_upsample", "histc_maxpool", "histc_upsample",
                                  "upsample_bnstats", "histc_bnstats", "upsample_bnstats_allreduce"};
    for (const char* s : solos)
        if (!strcmp(s, name)) return describe_dl_solo(variant, buf, n);
    for (const char* p : pairs)
        if (!strcmp(p, name)) return describe_dl_pair(variant, buf, n);
    return HFUSE_ERR_UNKNOWN_PAIR;
}
// compiled default variant of a DL kernel or pair (for the exchange pair: of its cursor form when that is the default form)
int dl_default_variant(const char* name) {
#define D(kind, n) if (!strcmp(name, #n)) return kDefault##kind##_##n;
    D(Solo, im2col) D(Solo, maxpool) D(Solo, bnstats) D(Solo, upsample) D(Solo, histc)
    D(Pair, im2col_maxpool) D(Pair, im2col_bnstats) D(Pair, im2col_histc) D(Pair, im2col_upsample)
    D(Pair, maxpool_bnstats) D(Pair, maxpool_upsample) D(Pair, histc_maxpool) D(Pair, histc_upsample)
    D(Pair, upsample_bnstats) D(Pair, histc_bnstats)
#undef D
    if (!strcmp(name, "upsample_bnstats_allreduce"))
        return kDefaultPool_upsample_bnstats_allreduce == 1 ? kDefaultPoolPair_upsample_bnstats_allreduce
                                                            : kDefaultPair_upsample_bnstats_allreduce;
    if (!strcmp(name, "upsample_bnstats_allreduce_wide"))      // what the exchange pair runs with more than four ranks
        return kDefaultPool_upsample_bnstats_allreduce == 1 ? kDefaultPoolPair_upsample_bnstats_allreduce_wide
                                                            : kDefaultPair_upsample_bnstats_allreduce_wide;
    return HFUSE_ERR_UNKNOWN_PAIR;
}
}  // namespace hfuse
