// PyTorch extension: torch.ops.hfuse_b200.* for the five DL kernels and their ten fused pairs.
//
// Stands in for the torch C++ extension the reference's Python harness calls
// (TorchKernel's build.sh / call_{1080,v100}.py, README.md:68,84-95 of aoli-al/HFuse).  It only
// checks tensors, allocates the outputs and forwards raw pointers plus the current stream to the C
// ABI in include/hfuse_b200.h; all device code lives in libhfuse_b200.so.  CUDA tensors only.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <map>
#include <mutex>
#include <tuple>

#include "../../include/hfuse_b200.h"

namespace {

using at::Tensor;
using IntList = at::IntArrayRef;

void check_in(const Tensor& t, const char* what, int dims = -1) {
    TORCH_CHECK(t.is_cuda(), what, " must be a CUDA tensor: hfuse_b200 has no CPU path");
    TORCH_CHECK(t.scalar_type() == at::kFloat, what, " must be float32");
    TORCH_CHECK(t.is_contiguous(), what, " must be contiguous (NCHW)");
    TORCH_CHECK(dims < 0 || t.dim() == dims, what, " must be ", dims, "-D");
}
void ok(int rc, const char* fn) { TORCH_CHECK(rc == HFUSE_OK, fn, ": ", hfuse_error_string(rc), " (", rc, ")"); }
void* stream() { return c10::cuda::getCurrentCUDAStream().stream(); }
int i32(int64_t v) { return static_cast<int>(v); }

// ---- one descriptor per operator: shapes, outputs, and the C-ABI argument values -------------------
struct Im2col {
    Tensor x, col;
    int N, C, H, W, kh, kw, ph, pw, sh, sw, dh, dw;
    Im2col(const Tensor& x_, IntList k, IntList p, IntList s, IntList d) : x(x_) {
        check_in(x, "im2col input", 4);
        TORCH_CHECK(k.size() == 2 && p.size() == 2 && s.size() == 2 && d.size() == 2, "im2col: 2-element lists expected");
        N = i32(x.size(0)); C = i32(x.size(1)); H = i32(x.size(2)); W = i32(x.size(3));
        kh = i32(k[0]); kw = i32(k[1]); ph = i32(p[0]); pw = i32(p[1]); sh = i32(s[0]); sw = i32(s[1]); dh = i32(d[0]); dw = i32(d[1]);
        TORCH_CHECK(sh > 0 && sw > 0 && dh > 0 && dw > 0 && kh > 0 && kw > 0, "im2col: bad kernel/stride/dilation");
        const int64_t Hc = (H + 2 * ph - (dh * (kh - 1) + 1)) / sh + 1, Wc = (W + 2 * pw - (dw * (kw - 1) + 1)) / sw + 1;
        TORCH_CHECK(Hc > 0 && Wc > 0, "im2col: kernel does not fit the padded input");
        col = at::empty({N, (int64_t)C * kh * kw, Hc * Wc}, x.options());
    }
};
#define IM2COL_ARGS(o) (o).x.data_ptr<float>(), (o).N, (o).C, (o).H, (o).W, (o).kh, (o).kw, (o).ph, (o).pw, (o).sh, (o).sw, (o).dh, (o).dw, (o).col.data_ptr<float>()

struct MaxPool {
    Tensor x, out, idx;
    int N, C, H, W, pH, pW, kh, kw, sh, sw, ph, pw, dh, dw;
    MaxPool(const Tensor& x_, IntList k, IntList s, IntList p, IntList d) : x(x_) {
        check_in(x, "max_pool input", 4);
        TORCH_CHECK(k.size() == 2 && p.size() == 2 && s.size() == 2 && d.size() == 2, "max_pool: 2-element lists expected");
        N = i32(x.size(0)); C = i32(x.size(1)); H = i32(x.size(2)); W = i32(x.size(3));
        kh = i32(k[0]); kw = i32(k[1]); sh = i32(s[0]); sw = i32(s[1]); ph = i32(p[0]); pw = i32(p[1]); dh = i32(d[0]); dw = i32(d[1]);
        TORCH_CHECK(sh > 0 && sw > 0 && dh > 0 && dw > 0 && kh > 0 && kw > 0, "max_pool: bad kernel/stride/dilation");
        pH = (H + 2 * ph - dh * (kh - 1) - 1) / sh + 1; pW = (W + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
        TORCH_CHECK(pH > 0 && pW > 0, "max_pool: window does not fit the padded input");
        out = at::empty({N, C, pH, pW}, x.options());
        idx = at::empty({N, C, pH, pW}, x.options().dtype(at::kLong));
    }
};
#define MAXPOOL_ARGS(o) (o).x.data_ptr<float>(), (o).N, (o).C, (o).H, (o).W, (o).pH, (o).pW, (o).kh, (o).kw, (o).sh, (o).sw, (o).ph, (o).pw, (o).dh, (o).dw, (o).out.data_ptr<float>(), (o).idx.data_ptr<int64_t>()

// zero-initialised scratch for the statistics kernel, one per (device, stream, channels)
Tensor bn_workspace(const Tensor& like, int C) {
    static std::mutex mu;
    static std::map<std::tuple<int, void*, int>, Tensor> cache;
    std::lock_guard<std::mutex> lk(mu);
    auto key = std::make_tuple((int)like.get_device(), stream(), C);
    auto it = cache.find(key);
    if (it == cache.end())
        it = cache.emplace(key, at::zeros({(int64_t)hfuse_bnstats_workspace_bytes(1, C, 1)}, like.options().dtype(at::kByte))).first;
    return it->second;
}
struct BnStats {
    Tensor x, mean, invstd, ws;
    int N, C, HW;
    float eps;
    BnStats(const Tensor& x_, double eps_) : x(x_), eps((float)eps_) {
        check_in(x, "batch_norm input");
        TORCH_CHECK(x.dim() >= 2 && x.numel() > 0, "batch_norm input must have at least 2 dimensions and be non-empty");
        N = i32(x.size(0)); C = i32(x.size(1)); HW = i32(x.numel() / ((int64_t)N * C));
        mean = at::empty({C}, x.options()); invstd = at::empty({C}, x.options());
        ws = bn_workspace(x, C);
    }
};
#define BNSTATS_ARGS(o) (o).x.data_ptr<float>(), (o).N, (o).C, (o).HW, (o).eps, (o).mean.data_ptr<float>(), (o).invstd.data_ptr<float>(), (double*)nullptr, (o).ws.data_ptr(), (size_t)(o).ws.numel()

struct Upsample {
    Tensor x, out;
    int N, C, H, W, oH, oW, align;
    Upsample(const Tensor& x_, IntList size, bool align_corners) : x(x_), align(align_corners) {
        check_in(x, "upsample input", 4);
        TORCH_CHECK(size.size() == 2 && size[0] > 0 && size[1] > 0, "upsample: output size must be two positive ints");
        N = i32(x.size(0)); C = i32(x.size(1)); H = i32(x.size(2)); W = i32(x.size(3)); oH = i32(size[0]); oW = i32(size[1]);
        out = at::empty({N, C, oH, oW}, x.options());
    }
};
#define UPSAMPLE_ARGS(o) (o).x.data_ptr<float>(), (o).N, (o).C, (o).H, (o).W, (o).oH, (o).oW, (o).align, (o).out.data_ptr<float>()

struct Histc {
    Tensor x, counts;
    int64_t n;
    int bins;
    float lo, hi;
    Histc(const Tensor& x_, int64_t bins_, double lo_, double hi_) : x(x_), n(x_.numel()), bins(i32(bins_)), lo((float)lo_), hi((float)hi_) {
        check_in(x, "histc input");
        TORCH_CHECK(bins > 0, "histc: bins must be positive");
        TORCH_CHECK(lo < hi, "histc: max must be larger than min");
        counts = at::empty({bins}, x.options().dtype(at::kInt));      // uint32 counts in int32 storage
    }
};
#define HISTC_ARGS(o) (o).n ? (o).x.data_ptr<float>() : nullptr, (o).n, (o).bins, (o).lo, (o).hi, (uint32_t*)(o).counts.data_ptr<int>()

// ---- standalone operators -----------------------------------------------------------------------------
Tensor im2col(const Tensor& x, IntList k, IntList p, IntList s, IntList d) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Im2col a(x, k, p, s, d);
    ok(hfuse_im2col_f32(IM2COL_ARGS(a), stream()), "hfuse_im2col_f32");
    return a.col;
}
std::tuple<Tensor, Tensor> max_pool2d_with_indices(const Tensor& x, IntList k, IntList s, IntList p, IntList d) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    MaxPool a(x, k, s, p, d);
    ok(hfuse_maxpool2d_f32(MAXPOOL_ARGS(a), stream()), "hfuse_maxpool2d_f32");
    return {a.out, a.idx};
}
std::tuple<Tensor, Tensor> batch_norm_stats(const Tensor& x, double eps) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    BnStats a(x, eps);
    ok(hfuse_bnstats_f32(BNSTATS_ARGS(a), stream()), "hfuse_bnstats_f32");
    return {a.mean, a.invstd};
}
Tensor upsample_bilinear2d(const Tensor& x, IntList size, bool align_corners) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Upsample a(x, size, align_corners);
    ok(hfuse_upsample_bilinear2d_f32(UPSAMPLE_ARGS(a), stream()), "hfuse_upsample_bilinear2d_f32");
    return a.out;
}
Tensor histc(const Tensor& x, int64_t bins, double lo, double hi) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Histc a(x, bins, lo, hi);
    ok(hfuse_histc_f32(HISTC_ARGS(a), stream()), "hfuse_histc_f32");
    return a.counts;
}

// ---- fused pairs: K1's arguments, then K2's; outputs in the same order ---------------------------------
std::tuple<Tensor, Tensor, Tensor> im2col_maxpool(const Tensor& x, IntList k, IntList p, IntList s, IntList d,
                                                  const Tensor& y, IntList k2, IntList s2, IntList p2, IntList d2) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Im2col a(x, k, p, s, d); MaxPool b(y, k2, s2, p2, d2);
    ok(hfuse_im2col_maxpool_f32(IM2COL_ARGS(a), MAXPOOL_ARGS(b), stream()), "hfuse_im2col_maxpool_f32");
    return {a.col, b.out, b.idx};
}
std::tuple<Tensor, Tensor, Tensor> im2col_bnstats(const Tensor& x, IntList k, IntList p, IntList s, IntList d,
                                                  const Tensor& y, double eps) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Im2col a(x, k, p, s, d); BnStats b(y, eps);
    ok(hfuse_im2col_bnstats_f32(IM2COL_ARGS(a), BNSTATS_ARGS(b), stream()), "hfuse_im2col_bnstats_f32");
    return {a.col, b.mean, b.invstd};
}
std::tuple<Tensor, Tensor> im2col_histc(const Tensor& x, IntList k, IntList p, IntList s, IntList d, const Tensor& y,
                                        int64_t bins, double lo, double hi) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Im2col a(x, k, p, s, d); Histc b(y, bins, lo, hi);
    ok(hfuse_im2col_histc_f32(IM2COL_ARGS(a), HISTC_ARGS(b), stream()), "hfuse_im2col_histc_f32");
    return {a.col, b.counts};
}
std::tuple<Tensor, Tensor> im2col_upsample(const Tensor& x, IntList k, IntList p, IntList s, IntList d, const Tensor& y,
                                           IntList size, bool align_corners) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Im2col a(x, k, p, s, d); Upsample b(y, size, align_corners);
    ok(hfuse_im2col_upsample_f32(IM2COL_ARGS(a), UPSAMPLE_ARGS(b), stream()), "hfuse_im2col_upsample_f32");
    return {a.col, b.out};
}
std::tuple<Tensor, Tensor, Tensor, Tensor> maxpool_bnstats(const Tensor& x, IntList k, IntList s, IntList p, IntList d,
                                                           const Tensor& y, double eps) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    MaxPool a(x, k, s, p, d); BnStats b(y, eps);
    ok(hfuse_maxpool_bnstats_f32(MAXPOOL_ARGS(a), BNSTATS_ARGS(b), stream()), "hfuse_maxpool_bnstats_f32");
    return {a.out, a.idx, b.mean, b.invstd};
}
std::tuple<Tensor, Tensor, Tensor> maxpool_upsample(const Tensor& x, IntList k, IntList s, IntList p, IntList d,
                                                    const Tensor& y, IntList size, bool align_corners) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    MaxPool a(x, k, s, p, d); Upsample b(y, size, align_corners);
    ok(hfuse_maxpool_upsample_f32(MAXPOOL_ARGS(a), UPSAMPLE_ARGS(b), stream()), "hfuse_maxpool_upsample_f32");
    return {a.out, a.idx, b.out};
}
std::tuple<Tensor, Tensor, Tensor> histc_maxpool(const Tensor& x, int64_t bins, double lo, double hi, const Tensor& y,
                                                 IntList k, IntList s, IntList p, IntList d) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Histc a(x, bins, lo, hi); MaxPool b(y, k, s, p, d);
    ok(hfuse_histc_maxpool_f32(HISTC_ARGS(a), MAXPOOL_ARGS(b), stream()), "hfuse_histc_maxpool_f32");
    return {a.counts, b.out, b.idx};
}
std::tuple<Tensor, Tensor> histc_upsample(const Tensor& x, int64_t bins, double lo, double hi, const Tensor& y, IntList size,
                                          bool align_corners) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Histc a(x, bins, lo, hi); Upsample b(y, size, align_corners);
    ok(hfuse_histc_upsample_f32(HISTC_ARGS(a), UPSAMPLE_ARGS(b), stream()), "hfuse_histc_upsample_f32");
    return {a.counts, b.out};
}
std::tuple<Tensor, Tensor, Tensor> upsample_bnstats(const Tensor& x, IntList size, bool align_corners, const Tensor& y,
                                                    double eps) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Upsample a(x, size, align_corners); BnStats b(y, eps);
    ok(hfuse_upsample_bnstats_f32(UPSAMPLE_ARGS(a), BNSTATS_ARGS(b), stream()), "hfuse_upsample_bnstats_f32");
    return {a.out, b.mean, b.invstd};
}
std::tuple<Tensor, Tensor, Tensor> histc_bnstats(const Tensor& x, int64_t bins, double lo, double hi, const Tensor& y,
                                                 double eps) {
    check_in(x, "first input");
    c10::cuda::CUDAGuard g(x.device());
    Histc a(x, bins, lo, hi); BnStats b(y, eps);
    ok(hfuse_histc_bnstats_f32(HISTC_ARGS(a), BNSTATS_ARGS(b), stream()), "hfuse_histc_bnstats_f32");
    return {a.counts, b.mean, b.invstd};
}

}  // namespace

TORCH_LIBRARY(hfuse_b200, m) {
    m.def("im2col(Tensor x, int[2] kernel_size, int[2] padding, int[2] stride, int[2] dilation) -> Tensor", &im2col);
    m.def("max_pool2d_with_indices(Tensor x, int[2] kernel_size, int[2] stride, int[2] padding, int[2] dilation) -> (Tensor, Tensor)", &max_pool2d_with_indices);
    m.def("batch_norm_stats(Tensor x, float eps) -> (Tensor, Tensor)", &batch_norm_stats);
    m.def("upsample_bilinear2d(Tensor x, int[2] output_size, bool align_corners) -> Tensor", &upsample_bilinear2d);
    m.def("histc(Tensor x, int bins, float min, float max) -> Tensor", &histc);
    m.def("im2col_maxpool(Tensor x, int[2] kernel_size, int[2] padding, int[2] stride, int[2] dilation, Tensor y, int[2] pool_kernel, int[2] pool_stride, int[2] pool_padding, int[2] pool_dilation) -> (Tensor, Tensor, Tensor)", &im2col_maxpool);
    m.def("im2col_bnstats(Tensor x, int[2] kernel_size, int[2] padding, int[2] stride, int[2] dilation, Tensor y, float eps) -> (Tensor, Tensor, Tensor)", &im2col_bnstats);
    m.def("im2col_histc(Tensor x, int[2] kernel_size, int[2] padding, int[2] stride, int[2] dilation, Tensor y, int bins, float min, float max) -> (Tensor, Tensor)", &im2col_histc);
    m.def("im2col_upsample(Tensor x, int[2] kernel_size, int[2] padding, int[2] stride, int[2] dilation, Tensor y, int[2] output_size, bool align_corners) -> (Tensor, Tensor)", &im2col_upsample);
    m.def("maxpool_bnstats(Tensor x, int[2] kernel_size, int[2] stride, int[2] padding, int[2] dilation, Tensor y, float eps) -> (Tensor, Tensor, Tensor, Tensor)", &maxpool_bnstats);
    m.def("maxpool_upsample(Tensor x, int[2] kernel_size, int[2] stride, int[2] padding, int[2] dilation, Tensor y, int[2] output_size, bool align_corners) -> (Tensor, Tensor, Tensor)", &maxpool_upsample);
    m.def("histc_maxpool(Tensor x, int bins, float min, float max, Tensor y, int[2] kernel_size, int[2] stride, int[2] padding, int[2] dilation) -> (Tensor, Tensor, Tensor)", &histc_maxpool);
    m.def("histc_upsample(Tensor x, int bins, float min, float max, Tensor y, int[2] output_size, bool align_corners) -> (Tensor, Tensor)", &histc_upsample);
    m.def("upsample_bnstats(Tensor x, int[2] output_size, bool align_corners, Tensor y, float eps) -> (Tensor, Tensor, Tensor)", &upsample_bnstats);
    m.def("histc_bnstats(Tensor x, int bins, float min, float max, Tensor y, float eps) -> (Tensor, Tensor, Tensor)", &histc_bnstats);
}
