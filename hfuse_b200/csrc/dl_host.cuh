// Host side shared by the deep-learning entry points: argument checking and
// variant dispatch.  Included by dl_api.cu (standalone kernels) and by one small
// translation unit per fused pair, so that the pairs compile in parallel.  The
// device code is in dl_roles.cuh and fused.cuh.
#pragma once
#include "dl_roles.cuh"
#include "launch.cuh"

using namespace hfuse;

// ---- argument-name lists matching the HFUSE_*_PARAMS macros of the public header ----------
#define IM2COL_NAMES(P) P##im, P##N, P##C, P##H, P##W, P##kh, P##kw, P##ph, P##pw, P##sh, P##sw, P##dh, P##dw, P##col
#define MAXPOOL_NAMES(P)                                                                                  \
    P##in, P##N, P##C, P##H, P##W, P##pH, P##pW, P##kh, P##kw, P##sh, P##sw, P##ph, P##pw, P##dh, P##dw, \
        P##out, P##idx
#define BNSTATS_NAMES(P) P##x, P##N, P##C, P##HW, P##eps, P##mean, P##invstd, P##moments, P##workspace, P##workspace_bytes
#define UPSAMPLE_NAMES(P) P##in, P##N, P##C, P##H, P##W, P##outH, P##outW, P##align_corners, P##out
#define HISTC_NAMES(P) P##x, P##n, P##nbins, P##lo, P##hi, P##counts

namespace {

constexpr long long kMaxItems = (1LL << 31) - 1;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

// ------------------------------------------------------------------ argument checking
int prep_im2col(HFUSE_IM2COL_PARAMS(), Im2colArgs& a) {
    if (!im || !col) return HFUSE_ERR_BAD_ARG;
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || ph < 0 || pw < 0 || sh <= 0 || sw <= 0 ||
        dh <= 0 || dw <= 0)
        return HFUSE_ERR_BAD_ARG;
    const long long eh = (long long)H + 2LL * ph - ((long long)dh * (kh - 1) + 1);
    const long long ew = (long long)W + 2LL * pw - ((long long)dw * (kw - 1) + 1);
    if (eh < 0 || ew < 0) return HFUSE_ERR_BAD_ARG;           // kernel larger than the padded image
    const long long Hc = eh / sh + 1, Wc = ew / sw + 1;
    if ((long long)H * W > kMaxItems || Hc * Wc > kMaxItems) return HFUSE_ERR_TOO_LARGE;
    if (!aligned16(im) || !aligned16(col)) return HFUSE_ERR_ALIGNMENT;
    a.im = im; a.col = col;
    a.N = N; a.C = C; a.H = H; a.W = W;
    a.kh = kh; a.kw = kw; a.ph = ph; a.pw = pw; a.sh = sh; a.sw = sw; a.dh = dh; a.dw = dw;
    a.Hc = (int)Hc; a.Wc = (int)Wc;
    const long long items = (long long)N * C * Hc * (Wc / 4);
    a.mode = (kh == 3 && kw == 3 && sh == 1 && sw == 1 && dh == 1 && dw == 1 && (Wc % 4) == 0 && items > 0 &&
              items <= kMaxItems)
                 ? 1 : 0;
    // tap planes start at multiples of Hc*Wc floats: with Wc % 8 == 0 every row start is 32-byte aligned
    if (a.mode == 1 && ph == 1 && pw == 1 && (Wc % 8) == 0 && (W % 4) == 0 && aligned32(col)) a.mode = 2;
    a.band = 0; a.bands = 1; a.bulk_ok = 0;
    if (a.mode >= 1 && ph == 1 && pw == 1 && (W % 4) == 0) {
        // shared-memory tile + bulk stores are possible: as many rows per unit as fit 20 KB per buffer
        const long long fit = (20 * 1024) / (12LL * Wc) - 2;
        if (fit >= 1) {
            a.band = (int)(fit < Hc ? fit : Hc);
            a.bands = (int)((Hc + a.band - 1) / a.band);
            a.bulk_ok = ((long long)N * C * a.bands <= kMaxItems) ? 1 : 0;
        }
    }
    a.div_bands = make_fastdiv((uint32_t)a.bands);
    a.div_w4 = make_fastdiv(a.mode == 2 ? (uint32_t)(Wc / 8) : a.mode == 1 ? (uint32_t)(Wc / 4) : 1u);
    a.div_hc = make_fastdiv((uint32_t)Hc);
    a.div_wc = make_fastdiv((uint32_t)Wc);
    a.div_taps = make_fastdiv((uint32_t)(kh * kw));
    a.div_kw = make_fastdiv((uint32_t)kw);
    a.small = ((long long)N * C * kh * kw * Hc * Wc <= kMaxItems) ? 1 : 0;
    return HFUSE_OK;
}

int prep_maxpool(HFUSE_MAXPOOL_PARAMS(), MaxPoolArgs& a) {
    if (!in || !out || !idx) return HFUSE_ERR_BAD_ARG;
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || pH <= 0 || pW <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 ||
        ph < 0 || pw < 0 || dh <= 0 || dw <= 0)
        return HFUSE_ERR_BAD_ARG;
    if (ph > kh / 2 || pw > kw / 2) return HFUSE_ERR_BAD_ARG;                 // same rule as the operator
    // every window must start inside the image (rules out pooled sizes the shape cannot give)
    if ((long long)(pH - 1) * sh - ph >= H || (long long)(pW - 1) * sw - pw >= W) return HFUSE_ERR_BAD_ARG;
    if ((long long)H * W > kMaxItems) return HFUSE_ERR_TOO_LARGE;
    if (!aligned16(in) || !aligned16(out) || !aligned16(idx)) return HFUSE_ERR_ALIGNMENT;
    a.in = in; a.out = out; a.idx = reinterpret_cast<long long*>(idx);
    a.N = N; a.C = C; a.H = H; a.W = W; a.pH = pH; a.pW = pW;
    a.kh = kh; a.kw = kw; a.sh = sh; a.sw = sw; a.ph = ph; a.pw = pw; a.dh = dh; a.dw = dw;
    const long long items = (long long)N * C * pH * (pW / 4);
    a.mode = (kh == 2 && kw == 2 && sh == 2 && sw == 2 && ph == 0 && pw == 0 && dh == 1 && dw == 1 &&
              (pW % 4) == 0 && (W % 4) == 0 && 2LL * pH <= H && 2LL * pW <= W && items <= kMaxItems)
                 ? 1 : 0;
    a.wide = aligned32(idx) ? 1 : 0;
    a.div_p4 = make_fastdiv(a.mode == 1 ? (uint32_t)(pW / 4) : 1u);
    a.div_ph = make_fastdiv((uint32_t)pH);
    a.div_pw = make_fastdiv((uint32_t)pW);
    a.small = ((long long)N * C * pH * pW <= kMaxItems) ? 1 : 0;
    return HFUSE_OK;
}

int prep_bnstats(HFUSE_BNSTATS_PARAMS(), BnStatsArgs& a) {
    if (!x || !mean || !invstd) return HFUSE_ERR_BAD_ARG;
    if (N <= 0 || C <= 0 || HW <= 0 || !(eps >= 0.f)) return HFUSE_ERR_BAD_ARG;
    if ((long long)N * HW > kMaxItems) return HFUSE_ERR_TOO_LARGE;
    if (!aligned16(x)) return HFUSE_ERR_ALIGNMENT;
    if (workspace && !aligned16(workspace)) return HFUSE_ERR_ALIGNMENT;
    a.x = x; a.N = N; a.C = C; a.HW = HW; a.eps = eps;
    a.total = (float)((double)N * (double)HW);
    a.mean = mean; a.invstd = invstd; a.moments = moments;
    a.partial = nullptr; a.tickets = nullptr;
    a.S = 1; a.chunk = 0; a.per_channel = 0; a.per_img = 1; a.div_img = make_fastdiv(1);
    a.vec = (HW % 4) == 0;
    a.ws = workspace; a.ws_bytes = workspace_bytes;
    a.xchg = BnXchg{};
    // bulk-load path: rows of 1 to 25 KB that are 16-byte multiples; three buffers, each holding as many rows
    // as fit 25 KB, all fills of a channel equally long (measured on B200: two to four buffers of 12.5 or 25 KB
    // are within 0.3 us of each other; alone or with a large statistics range the register path is faster)
    a.bulk = 0; a.bulk_ok = 0; a.bulk_rows = 1; a.bulk_bufs = 3;
    const long long row_bytes = (long long)HW * 4;
    if (a.vec && row_bytes >= 1024 && row_bytes <= 25600) {
        const int rmax = (int)(25600 / row_bytes);
        const int fills = (N + rmax - 1) / rmax;
        a.bulk_rows = (unsigned)((N + fills - 1) / fills);
        a.bulk_ok = 1;
    }
    return HFUSE_OK;
}

float scale_of(int in_size, int out_size, int align_corners) {
    if (align_corners) return out_size > 1 ? (float)(in_size - 1) / (float)(out_size - 1) : 0.f;
    return (float)in_size / (float)out_size;
}

int prep_upsample(HFUSE_UPSAMPLE_PARAMS(), UpsampleArgs& a) {
    if (!in || !out) return HFUSE_ERR_BAD_ARG;
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || outH <= 0 || outW <= 0) return HFUSE_ERR_BAD_ARG;
    if ((long long)H * W > kMaxItems || (long long)outH * outW > kMaxItems) return HFUSE_ERR_TOO_LARGE;
    if (!aligned16(in) || !aligned16(out)) return HFUSE_ERR_ALIGNMENT;
    a.in = in; a.out = out; a.N = N; a.C = C; a.H = H; a.W = W; a.outH = outH; a.outW = outW;
    a.rheight = scale_of(H, outH, align_corners);
    a.rwidth = scale_of(W, outW, align_corners);
    a.align_corners = align_corners ? 1 : 0;
    const long long items = (long long)N * C * outH * (outW / 4);
    a.mode = ((outW % 4) == 0 && items <= kMaxItems) ? 1 : 0;
    const long long strips = (long long)N * C * (H + 1LL) * (W / 4);
    if (!align_corners && outH == 2LL * H && outW == 2LL * W && (W % 4) == 0 && strips <= kMaxItems) a.mode = 2;
    a.wide = aligned32(out) ? 1 : 0;
    a.div_w4 = make_fastdiv(a.mode == 2 ? (uint32_t)(W / 4) : 1u);
    a.div_j = make_fastdiv((uint32_t)H + 1u);
    a.div_ow4 = make_fastdiv(a.mode == 1 ? (uint32_t)(outW / 4) : 1u);
    a.div_oh = make_fastdiv((uint32_t)outH);
    a.div_ow = make_fastdiv((uint32_t)outW);
    a.small = ((long long)N * C * outH * outW <= kMaxItems) ? 1 : 0;
    return HFUSE_OK;
}

int prep_histc(HFUSE_HISTC_PARAMS(), HistcArgs& a) {
    if (!counts || n < 0 || (n > 0 && !x)) return HFUSE_ERR_BAD_ARG;
    if (nbins <= 0 || !(lo < hi) || !(lo > -INFINITY) || !(hi < INFINITY)) return HFUSE_ERR_BAD_ARG;    // also rejects NaN bounds
    if (nbins > (1 << 24)) return HFUSE_ERR_TOO_LARGE;         // bins must stay exact in fp32
    if (x && !aligned16(x)) return HFUSE_ERR_ALIGNMENT;
    a.x = x; a.n = n; a.nbins = nbins; a.lo = lo; a.hi = hi; a.counts = counts;
    a.fbins = (float)nbins;
    a.fast = (n >> 2) < (1LL << 31) ? 1 : 0;
    a.range = hi - lo;
    int e = 0;
    const float mant = frexpf(a.range, &e);
    a.range_pow2 = (mant == 0.5f) && (e > -100) && (e < 100);
    a.inv_range = a.range_pow2 ? 1.f / a.range : 0.f;
    a.copies = 0;
    a.lane_private = 0;
    // bulk-load sweep: the [bin][lane] histogram (up to 256 bins) and fewer than 2^31 16-byte items
    a.bulk = 0;
    a.bulk_ok = (a.fast && nbins <= 256 && x) ? 1 : 0;
    return HFUSE_OK;
}

// The histogram kernels add to `counts`, so it is cleared first: by a small kernel that lets its
// successor start at once (`griddepcontrol.launch_dependents`); the histogram kernel is launched
// as its programmatic dependent and waits for it only before its flush.  A memset node in the
// same place delays the histogram kernel by 3.6 us on B200, this form by about 0.5 us.
__global__ void clear_counts_kernel(unsigned* counts, int n) {
    asm volatile("griddepcontrol.launch_dependents;");
    for (int i = (int)(blockIdx.x * blockDim.x + threadIdx.x); i < n; i += (int)(gridDim.x * blockDim.x)) counts[i] = 0u;
}
int clear_counts(const HistcArgs& a, cudaStream_t s) {
    const int blocks = a.nbins <= 4096 ? 1 : (a.nbins < (1 << 20) ? (a.nbins + 4095) / 4096 : 256);
    clear_counts_kernel<<<blocks, 256, 0, s>>>(a.counts, a.nbins);
    return check_launch();
}
// Which store path the im2col role takes in the kernel or pair `name`: the option
// "im2col_store_path" if it was set (0 or 1), else the compiled default of that kernel or pair.
int default_im2col_bulk(const char* name);
void choose_path(Im2colArgs& a, const char* name) {
    if (!a.bulk_ok) return;
    const int opt = option_get("im2col_store_path", -1);
    if (opt >= 0 ? opt == 1 : default_im2col_bulk(name) == 1) a.mode = 3;
}
// The same for the statistics role's load path (option "bnstats_load_path").
int default_bnstats_bulk(const char* name);
void choose_path(BnStatsArgs& a, const char* name) {
    if (!a.bulk_ok) return;
    const int opt = option_get("bnstats_load_path", -1);
    a.bulk = (opt >= 0 ? opt == 1 : default_bnstats_bulk(name) == 1) ? 1 : 0;
}
// And for the histogram role's load path (option "histc_load_path").
int default_histc_bulk(const char* name);
void choose_path(HistcArgs& a, const char* name) {
    if (!a.bulk_ok) return;
    const int opt = option_get("histc_load_path", -1);
    a.bulk = (opt >= 0 ? opt == 1 : default_histc_bulk(name) == 1) ? 1 : 0;
}
template <class A> void choose_path(A&, const char*) {}

// pre_launch returns a negative error, 0, or 1 when the main kernel must be launched as the
// programmatic dependent of what pre_launch queued
int pre_launch(const HistcArgs& a, cudaStream_t s) {
    if (int rc = clear_counts(a, s)) return rc;
    return 1;
}
template <class A> int pre_launch(const A&, cudaStream_t) { return HFUSE_OK; }

// ------------------------------------------------------------------ variants
// (index, T1, T2, minBlocks/SM).  Splits move in 128-thread steps like the reference's sweep
// (tools/llvm-smart-fuser/main.cpp:215-227); minBlocks is the register cap of its `_lb`
// presets (lib/KernelFuser/KernelPrinter.cpp:44-65) expressed as blocks per SM.
#define DL_PAIR_VARIANTS(X)                                                                         \
    X(0, 256, 256, 2) X(1, 384, 128, 2) X(2, 128, 384, 2) X(3, 256, 256, 3) X(4, 512, 512, 1)       \
    X(5, 768, 256, 1) X(6, 256, 768, 1) X(7, 640, 384, 1) X(8, 384, 640, 1) X(9, 512, 256, 1)       \
    X(10, 256, 512, 1) X(11, 128, 128, 4) X(12, 128, 128, 6) X(13, 896, 128, 1) X(14, 128, 896, 1)  \
    X(15, 512, 256, 2) X(16, 256, 512, 2) X(20, 384, 256, 2) X(21, 256, 384, 2)
// vertical fusion (the reference's vfuse presets): (index, T, minBlocks/SM), described as "T:0:minBlocks"
#define DL_VPAIR_VARIANTS(X) X(17, 512, 2) X(18, 1024, 1) X(19, 256, 4)
constexpr int kDlPairVariants = 22;

#define DL_SOLO_VARIANTS(X) \
    X(0, 256, 4) X(1, 256, 8) X(2, 512, 2) X(3, 128, 8) X(4, 512, 4) X(5, 1024, 1) X(6, 128, 16) X(7, 768, 1) X(8, 768, 2) X(9, 384, 4)
constexpr int kDlSoloVariants = 10;

template <class RA, class RB>
int dispatch_pair(const char* name, int default_variant, typename RA::Args a, typename RB::Args b, cudaStream_t s) {
    const Tune t = tune_get(name);
    const int v = t.variant >= 0 ? t.variant : default_variant;
    choose_path(a, name);
    choose_path(b, name);
    const int pa = pre_launch(a, s), pb = pre_launch(b, s);
    if (pa < 0) return pa;
    if (pb < 0) return pb;
    const bool dep = pa > 0 || pb > 0;
    switch (v) {
#define X(I, TA, TB, MB) \
    case I: return launch_pair<RA, RB, TA, TB, MB>(a, b, t.blocks_per_sm, s, dep);
        DL_PAIR_VARIANTS(X)
#undef X
#define X(I, T, MB) \
    case I: return launch_vpair<RA, RB, T, MB>(a, b, t.blocks_per_sm, s, dep);
        DL_VPAIR_VARIANTS(X)
#undef X
    }
    return HFUSE_ERR_BAD_ARG;
}

// pairs whose second role takes over a share of the first role's items (launch_pair_share)
template <class RA, class RB>
int dispatch_pair_share(const char* name, int default_variant, int default_share, typename RA::Args a,
                        typename RB::Args b, cudaStream_t s) {
    const Tune t = tune_get(name);
    const int v = t.variant >= 0 ? t.variant : default_variant;
    const int share = t.share_permille >= 0 ? t.share_permille : default_share;
    choose_path(a, name);
    choose_path(b, name);
    const int pa = pre_launch(a, s), pb = pre_launch(b, s);
    if (pa < 0) return pa;
    if (pb < 0) return pb;
    const bool dep = pa > 0 || pb > 0;
    switch (v) {
#define X(I, TA, TB, MB) \
    case I: return launch_pair_share<RA, RB, TA, TB, MB>(a, b, t.blocks_per_sm, share, s, dep);
        DL_PAIR_VARIANTS(X)
#undef X
#define X(I, T, MB) \
    case I: return launch_vpair<RA, RB, T, MB>(a, b, t.blocks_per_sm, s, dep);
        DL_VPAIR_VARIANTS(X)
#undef X
    }
    return HFUSE_ERR_BAD_ARG;
}

// pairs whose first role's items are drawn from a cursor by both thread ranges (launch_pair_pool)
template <class RA, class RB>
int dispatch_pair_pool(const char* name, int default_variant, typename RA::Args a, typename RB::Args b, cudaStream_t s) {
    const Tune t = tune_get(name);
    const int v = t.variant >= 0 ? t.variant : default_variant;
    choose_path(a, name);
    choose_path(b, name);
    const int pa = pre_launch(a, s), pb = pre_launch(b, s);
    if (pa < 0) return pa;
    if (pb < 0) return pb;
    const bool dep = pa > 0 || pb > 0;
    switch (v) {
#define X(I, TA, TB, MB) \
    case I: return launch_pair_pool<RA, RB, TA, TB, MB>(a, b, t.blocks_per_sm, s, dep);
        DL_PAIR_VARIANTS(X)
#undef X
#define X(I, T, MB) \
    case I: return launch_vpair<RA, RB, T, MB>(a, b, t.blocks_per_sm, s, dep);
        DL_VPAIR_VARIANTS(X)
#undef X
    }
    return HFUSE_ERR_BAD_ARG;
}

template <class R>
int dispatch_solo(const char* name, int default_variant, typename R::Args a, cudaStream_t s) {
    const Tune t = tune_get(name);
    const int v = t.variant >= 0 ? t.variant : default_variant;
    choose_path(a, name);
    const int pa = pre_launch(a, s);
    if (pa < 0) return pa;
    switch (v) {
#define X(I, T, MB) \
    case I: return launch_solo<R, T, MB>(a, t.blocks_per_sm, s, pa > 0);
        DL_SOLO_VARIANTS(X)
#undef X
    }
    return HFUSE_ERR_BAD_ARG;
}

int describe_dl_pair(int v, char* buf, size_t n) {
    switch (v) {
#define X(I, TA, TB, MB) \
    case I: snprintf(buf, n, "%d:%d:%d", TA, TB, MB); return kDlPairVariants;
        DL_PAIR_VARIANTS(X)
#undef X
#define X(I, T, MB) \
    case I: snprintf(buf, n, "%d:0:%d", T, MB); return kDlPairVariants;
        DL_VPAIR_VARIANTS(X)
#undef X
    }
    return HFUSE_ERR_BAD_ARG;
}
int describe_dl_solo(int v, char* buf, size_t n) {
    switch (v) {
#define X(I, T, MB) \
    case I: snprintf(buf, n, "%d:0:%d", T, MB); return kDlSoloVariants;
        DL_SOLO_VARIANTS(X)
#undef X
    }
    return HFUSE_ERR_BAD_ARG;
}

// default variant per kernel / pair (index into the lists above), chosen by the sweep
// in bench.py --tune on a B200
#include "dl_tuned.inc"

int default_bnstats_bulk(const char* name) {
    if (!strcmp(name, "bnstats")) return kBnStatsBulk_bnstats;
    if (!strcmp(name, "im2col_bnstats")) return kBnStatsBulk_im2col_bnstats;
    if (!strcmp(name, "maxpool_bnstats")) return kBnStatsBulk_maxpool_bnstats;
    if (!strcmp(name, "upsample_bnstats")) return kBnStatsBulk_upsample_bnstats;
    if (!strcmp(name, "histc_bnstats")) return kBnStatsBulk_histc_bnstats;
    if (!strcmp(name, "upsample_bnstats_allreduce")) return kBnStatsBulk_upsample_bnstats_allreduce;
    return 0;
}

int default_histc_bulk(const char* name) {
    if (!strcmp(name, "histc")) return kHistcBulk_histc;
    if (!strcmp(name, "im2col_histc")) return kHistcBulk_im2col_histc;
    if (!strcmp(name, "histc_maxpool")) return kHistcBulk_histc_maxpool;
    if (!strcmp(name, "histc_upsample")) return kHistcBulk_histc_upsample;
    if (!strcmp(name, "histc_bnstats")) return kHistcBulk_histc_bnstats;
    return 0;
}

int default_im2col_bulk(const char* name) {
    if (!strcmp(name, "im2col")) return kIm2colBulk_im2col;
    if (!strcmp(name, "im2col_maxpool")) return kIm2colBulk_im2col_maxpool;
    if (!strcmp(name, "im2col_bnstats")) return kIm2colBulk_im2col_bnstats;
    if (!strcmp(name, "im2col_histc")) return kIm2colBulk_im2col_histc;
    if (!strcmp(name, "im2col_upsample")) return kIm2colBulk_im2col_upsample;
    return 0;
}

}  // namespace

#define S_(x) static_cast<cudaStream_t>(x)

#define DEFINE_PAIR(NAME, RA, PA, NA, prepA, ArgsA, RB, PB, NB, prepB, ArgsB)                          \
    extern "C" int hfuse_##NAME##_f32(PA(a_), PB(b_), hfuse_stream_t stream) {                                   \
        ArgsA a;                                                                                       \
        ArgsB b;                                                                                       \
        if (int rc = prepA(NA(a_), a)) return rc;                                                      \
        if (int rc = prepB(NB(b_), b)) return rc;                                                      \
        return dispatch_pair<RA, RB>(#NAME, kDefaultPair_##NAME, a, b, S_(stream));                    \
    }

#define IM2COL_ Im2colRole, HFUSE_IM2COL_PARAMS, IM2COL_NAMES, prep_im2col, Im2colArgs
#define MAXPOOL_ MaxPoolRole, HFUSE_MAXPOOL_PARAMS, MAXPOOL_NAMES, prep_maxpool, MaxPoolArgs
#define BNSTATS_ BnStatsRole, HFUSE_BNSTATS_PARAMS, BNSTATS_NAMES, prep_bnstats, BnStatsArgs
#define UPSAMPLE_ UpsampleRole, HFUSE_UPSAMPLE_PARAMS, UPSAMPLE_NAMES, prep_upsample, UpsampleArgs
#define HISTC_ HistcRole, HFUSE_HISTC_PARAMS, HISTC_NAMES, prep_histc, HistcArgs
#define DEFINE_PAIR_(NAME, A, B) DEFINE_PAIR_X(NAME, A, B)
#define DEFINE_PAIR_X(NAME, ...) DEFINE_PAIR(NAME, __VA_ARGS__)

