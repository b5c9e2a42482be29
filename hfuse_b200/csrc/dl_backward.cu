// C-ABI entry points of the two backward kernels and of their fused pair.
#include "dl_backward.cuh"
#include "dl_host.cuh"

namespace {

int prep_maxpool_bwd(const float* grad_out, const int64_t* idx, int N, int C, int H, int W, int pH, int pW, int kh,
                     int kw, int sh, int sw, int ph, int pw, int dh, int dw, float* grad_in, MaxPoolBwdArgs& a) {
    if (!grad_out || !idx || !grad_in) return HFUSE_ERR_BAD_ARG;
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || pH <= 0 || pW <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 ||
        ph < 0 || pw < 0 || dh <= 0 || dw <= 0)
        return HFUSE_ERR_BAD_ARG;
    if ((long long)N * C * H * W > kMaxItems) return HFUSE_ERR_TOO_LARGE;
    if (!aligned16(grad_out) || !aligned16(idx) || !aligned16(grad_in)) return HFUSE_ERR_ALIGNMENT;
    a.grad_out = grad_out; a.idx = reinterpret_cast<const long long*>(idx); a.grad_in = grad_in;
    a.N = N; a.C = C; a.H = H; a.W = W; a.pH = pH; a.pW = pW;
    a.kh = kh; a.kw = kw; a.sh = sh; a.sw = sw; a.ph = ph; a.pw = pw; a.dh = dh; a.dw = dw;
    a.div_w = make_fastdiv((uint32_t)W); a.div_h = make_fastdiv((uint32_t)H);
    return HFUSE_OK;
}

int prep_bn_bwd(const float* x, const float* dy, int N, int C, int HW, const float* weight, const float* mean,
                const float* invstd, float* dx, float* grad_weight, float* grad_bias, BnBwdArgs& a) {
    if (!x || !dy || !mean || !invstd) return HFUSE_ERR_BAD_ARG;
    if (N <= 0 || C <= 0 || HW <= 0) return HFUSE_ERR_BAD_ARG;
    if ((long long)N * HW > kMaxItems) return HFUSE_ERR_TOO_LARGE;
    if (!aligned16(x) || !aligned16(dy) || (dx && !aligned16(dx))) return HFUSE_ERR_ALIGNMENT;
    a.x = x; a.dy = dy; a.weight = weight; a.mean = mean; a.invstd = invstd;
    a.dx = dx; a.grad_weight = grad_weight; a.grad_bias = grad_bias;
    a.N = N; a.C = C; a.HW = HW;
    a.inv_m = (float)(1.0 / ((double)N * (double)HW));
    a.vec = (HW % 4) == 0;
    a.per_img = (unsigned)(a.vec ? HW / 4 : HW);
    a.per_channel = (unsigned)N * a.per_img;
    a.div_img = make_fastdiv(a.per_img);
    return HFUSE_OK;
}

}  // namespace

extern "C" {

int hfuse_maxpool2d_backward_f32(const float* grad_out, const int64_t* idx, int N, int C, int H, int W, int pH, int pW,
                                 int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw, float* grad_in,
                                 hfuse_stream_t stream) {
    MaxPoolBwdArgs a;
    if (int rc = prep_maxpool_bwd(grad_out, idx, N, C, H, W, pH, pW, kh, kw, sh, sw, ph, pw, dh, dw, grad_in, a)) return rc;
    return launch_solo<MaxPoolBwdRole, 256, 4>(a, 0, S_(stream));
}

int hfuse_bn_backward_f32(const float* x, const float* grad_out, int N, int C, int HW, const float* weight,
                          const float* mean, const float* invstd, float* grad_in, float* grad_weight, float* grad_bias,
                          hfuse_stream_t stream) {
    BnBwdArgs a;
    if (int rc = prep_bn_bwd(x, grad_out, N, C, HW, weight, mean, invstd, grad_in, grad_weight, grad_bias, a)) return rc;
    return launch_solo<BnBwdRole, 512, 2>(a, 0, S_(stream));
}

int hfuse_maxpool_backward_bn_backward_f32(const float* p_grad_out, const int64_t* p_idx, int pN, int pC, int pHin,
                                           int pWin, int pH, int pW, int kh, int kw, int sh, int sw, int ph, int pw,
                                           int dh, int dw, float* p_grad_in, const float* x, const float* grad_out, int N,
                                           int C, int HW, const float* weight, const float* mean, const float* invstd,
                                           float* grad_in, float* grad_weight, float* grad_bias, hfuse_stream_t stream) {
    MaxPoolBwdArgs a;
    BnBwdArgs b;
    if (int rc = prep_maxpool_bwd(p_grad_out, p_idx, pN, pC, pHin, pWin, pH, pW, kh, kw, sh, sw, ph, pw, dh, dw, p_grad_in, a))
        return rc;
    if (int rc = prep_bn_bwd(x, grad_out, N, C, HW, weight, mean, invstd, grad_in, grad_weight, grad_bias, b)) return rc;
    return launch_pair<MaxPoolBwdRole, BnBwdRole, 256, 256, 2>(a, b, 0, S_(stream));
}

}  // extern "C"
