// Role bodies of the five deep-learning kernels on the fused path.
//
// Each role is written once as `Role::run<T, BAR>(args, ctx)` where T is the
// size of the thread range that executes it and BAR its named-barrier id.
// A standalone kernel runs one role over the whole block; a fused kernel runs
// two roles side by side (fused.cuh).  Because both use the same body, a
// fused pair and its two standalone kernels produce identical bytes.
//
// Reference kernels these replace (signatures recovered from the reference's
// profiler traces; block shapes from configs/ml_kernels.yaml):
//   im2col_kernel<float>                         ml_kernels.yaml:28-36, scripts/data/ml-event.csv:17
//   MaxPoolForward<float,float>                  ml_kernels.yaml:37-45, scripts/data/ml-event.csv:5
//   batch_norm_collect_statistics_kernel<InvStd> ml_kernels.yaml:19-27, scripts/data/ml-event.csv:14
//   upsample_bilinear2d_out_frame<float,float>   ml_kernels.yaml:1-9,   scripts/data/ml-event.csv:32
//   kernelHistogram1D<..., SHARED, ...>          ml_kernels.yaml:10-18, scripts/data/ml-event.csv:33
#pragma once
#include "common.cuh"
#include <math_constants.h>

namespace hfuse {

// =============================================================================
// im2col (unfold).  col[n][(c*kh+i)*kw+j][h*Wc+w] = im[n][c][h*sh-ph+i*dh][w*sw-pw+j*dw]
// =============================================================================
struct Im2colArgs {
    const float* im;
    float* col;
    int N, C, H, W;
    int kh, kw, ph, pw, sh, sw, dh, dw;
    int Hc, Wc;
    int mode;   // 0 = generic (one output element per item), 1 = 3x3 stride-1 tile path
};

struct Im2colRole {
    using Args = Im2colArgs;
    static int smem_bytes(const Args&, int) { return 0; }
    static int plan(Args&, int /*T*/, int /*grid*/) { return 0; }

    // 3x3 / stride 1 / dilation 1, Wc % 4 == 0: one item = four adjacent
    // output columns of one (plane, row).  The thread reads the 3 x 6 input
    // patch once and writes all nine taps as aligned 16-byte streaming stores,
    // so every input element is fetched from L1/L2 three times instead of nine
    // and 90 % of the traffic (the stores) is fully coalesced.
    template <int T>
    static __device__ __forceinline__ void run_k3s1(const Args& a, const RoleCtx& ctx) {
        constexpr int KH = 3, KW = 3;
        const unsigned W4 = (unsigned)a.Wc >> 2;
        const unsigned Hc = (unsigned)a.Hc;
        const unsigned total = (unsigned)a.N * a.C * Hc * W4;     // host guarantees < 2^31
        const size_t tap_stride = (size_t)a.Hc * a.Wc;
        const bool vec_mid = (a.pw == 1) && ((a.W & 3) == 0);
        for (unsigned it = (unsigned)ctx.block * T + ctx.tid; it < total; it += (unsigned)ctx.nblocks * T) {
            const unsigned w4 = it % W4;
            const unsigned r = it / W4;
            const unsigned h = r % Hc;
            const unsigned plane = r / Hc;
            const float* src = a.im + (size_t)plane * a.H * a.W;
            float* dst = a.col + (size_t)plane * (KH * KW) * tap_stride + (size_t)h * a.Wc + w4 * 4;
            const int wi0 = (int)(w4 * 4) - a.pw;
            float v[KH][4 + KW - 1];
#pragma unroll
            for (int i = 0; i < KH; ++i) {
                const int hi = (int)h - a.ph + i;
                const bool row_ok = (hi >= 0) && (hi < a.H);
                const float* row = src + (size_t)(row_ok ? hi : 0) * a.W;
                if (vec_mid && (wi0 + 1 + 3 < a.W)) {
                    // columns wi0+1 .. wi0+4 start on a 16-byte boundary
                    float4 m = row_ok ? __ldg(reinterpret_cast<const float4*>(row + wi0 + 1))
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
                    v[i][1] = m.x; v[i][2] = m.y; v[i][3] = m.z; v[i][4] = m.w;
                    v[i][0] = (row_ok && wi0 >= 0) ? __ldg(row + wi0) : 0.f;
                    v[i][5] = (row_ok && wi0 + 5 < a.W) ? __ldg(row + wi0 + 5) : 0.f;
                } else {
#pragma unroll
                    for (int x = 0; x < 4 + KW - 1; ++x) {
                        const int wi = wi0 + x;
                        v[i][x] = (row_ok && wi >= 0 && wi < a.W) ? __ldg(row + wi) : 0.f;
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < KH; ++i)
#pragma unroll
                for (int j = 0; j < KW; ++j)
                    stg_stream4(dst + (size_t)(i * KW + j) * tap_stride,
                                make_float4(v[i][j], v[i][j + 1], v[i][j + 2], v[i][j + 3]));
        }
    }

    template <int T>
    static __device__ __forceinline__ void run_generic(const Args& a, const RoleCtx& ctx) {
        const unsigned long long plane_out = (unsigned long long)a.Hc * a.Wc;
        const unsigned long long taps = (unsigned long long)a.kh * a.kw;
        const unsigned long long total = (unsigned long long)a.N * a.C * taps * plane_out;
        for (unsigned long long e = (unsigned long long)ctx.block * T + ctx.tid; e < total;
             e += (unsigned long long)ctx.nblocks * T) {
            const unsigned w = (unsigned)(e % a.Wc);
            unsigned long long r = e / a.Wc;
            const unsigned h = (unsigned)(r % a.Hc);
            r /= a.Hc;
            const unsigned tap = (unsigned)(r % taps);
            const unsigned long long plane = r / taps;
            const int i = tap / a.kw, j = tap % a.kw;
            const int hi = (int)h * a.sh - a.ph + i * a.dh;
            const int wi = (int)w * a.sw - a.pw + j * a.dw;
            float v = 0.f;
            if (hi >= 0 && hi < a.H && wi >= 0 && wi < a.W)
                v = __ldg(a.im + (size_t)plane * a.H * a.W + (size_t)hi * a.W + wi);
            stg_stream1(a.col + e, v);
        }
    }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        if (a.mode == 1) run_k3s1<T>(a, ctx);
        else run_generic<T>(a, ctx);
    }
};

// =============================================================================
// max_pool2d_with_indices forward
// =============================================================================
struct MaxPoolArgs {
    const float* in;
    float* out;
    long long* idx;
    int N, C, H, W, pH, pW;
    int kh, kw, sh, sw, ph, pw, dh, dw;
    int mode;   // 0 = generic, 1 = 2x2 stride 2 without padding, pW % 4 == 0, W % 4 == 0
};

__device__ __forceinline__ void pool_take(float v, int at, float& best, int& best_at) {
    // strictly greater, or NaN: the first maximum in scan order is kept and NaN wins
    if ((v > best) || (v != v)) { best = v; best_at = at; }
}

struct MaxPoolRole {
    using Args = MaxPoolArgs;
    static int smem_bytes(const Args&, int) { return 0; }
    static int plan(Args&, int, int) { return 0; }

    // four adjacent outputs per item: 2 rows x 8 columns in (four 16-byte loads),
    // one 16-byte value store and two 16-byte index stores out
    template <int T>
    static __device__ __forceinline__ void run_k2s2(const Args& a, const RoleCtx& ctx) {
        const unsigned P4 = (unsigned)a.pW >> 2;
        const unsigned pH = (unsigned)a.pH;
        const unsigned total = (unsigned)a.N * a.C * pH * P4;      // host guarantees < 2^31
        for (unsigned it = (unsigned)ctx.block * T + ctx.tid; it < total; it += (unsigned)ctx.nblocks * T) {
            const unsigned p4 = it % P4;
            const unsigned r = it / P4;
            const unsigned oh = r % pH;
            const unsigned plane = r / pH;
            const float* row0 = a.in + (size_t)plane * a.H * a.W + (size_t)(2 * oh) * a.W + 8 * p4;
            const float4 t0 = ldg_stream4(row0), t1 = ldg_stream4(row0 + 4);
            const float4 b0 = ldg_stream4(row0 + a.W), b1 = ldg_stream4(row0 + a.W + 4);
            const float top[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
            const float bot[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            const int base = (int)(2 * oh) * a.W + (int)(8 * p4);
            float best[4];
            int at[4];
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                best[o] = -CUDART_INF_F;
                at[o] = base + 2 * o;
                pool_take(top[2 * o], base + 2 * o, best[o], at[o]);
                pool_take(top[2 * o + 1], base + 2 * o + 1, best[o], at[o]);
                pool_take(bot[2 * o], base + a.W + 2 * o, best[o], at[o]);
                pool_take(bot[2 * o + 1], base + a.W + 2 * o + 1, best[o], at[o]);
            }
            const size_t o_off = ((size_t)plane * pH + oh) * a.pW + 4 * p4;
            stg_stream4(a.out + o_off, make_float4(best[0], best[1], best[2], best[3]));
            stg_stream_2xi64(a.idx + o_off, at[0], at[1]);
            stg_stream_2xi64(a.idx + o_off + 2, at[2], at[3]);
        }
    }

    template <int T>
    static __device__ __forceinline__ void run_generic(const Args& a, const RoleCtx& ctx) {
        const unsigned long long total = (unsigned long long)a.N * a.C * a.pH * a.pW;
        for (unsigned long long e = (unsigned long long)ctx.block * T + ctx.tid; e < total;
             e += (unsigned long long)ctx.nblocks * T) {
            const int ow = (int)(e % a.pW);
            unsigned long long r = e / a.pW;
            const int oh = (int)(r % a.pH);
            const unsigned long long plane = r / a.pH;
            int hstart = oh * a.sh - a.ph;
            int wstart = ow * a.sw - a.pw;
            const int hend = min(hstart + (a.kh - 1) * a.dh + 1, a.H);
            const int wend = min(wstart + (a.kw - 1) * a.dw + 1, a.W);
            while (hstart < 0) hstart += a.dh;
            while (wstart < 0) wstart += a.dw;
            const float* src = a.in + (size_t)plane * a.H * a.W;
            float best = -CUDART_INF_F;
            int at = hstart * a.W + wstart;
            for (int h = hstart; h < hend; h += a.dh)
                for (int w = wstart; w < wend; w += a.dw) pool_take(__ldg(src + h * a.W + w), h * a.W + w, best, at);
            a.out[e] = best;
            a.idx[e] = at;
        }
    }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        if (a.mode == 1) run_k2s2<T>(a, ctx);
        else run_generic<T>(a, ctx);
    }
};

// =============================================================================
// upsample_bilinear2d forward
// =============================================================================
struct UpsampleArgs {
    const float* in;
    float* out;
    int N, C, H, W, outH, outW;
    float rheight, rwidth;
    int align_corners;
    int mode;   // 0 = one output per item, 1 = four adjacent outputs per item (outW % 4 == 0)
};

__device__ __forceinline__ void bilinear_src(float scale, int dst, int align, int in_size, int& i1, int& i1p,
                                             float& lam0, float& lam1) {
    float src;
    if (align) {
        src = __fmul_rn(scale, (float)dst);
    } else {
        src = __fsub_rn(__fmul_rn(scale, __fadd_rn((float)dst, 0.5f)), 0.5f);
        src = src < 0.f ? 0.f : src;
    }
    i1 = (int)src;
    i1p = (i1 < in_size - 1) ? 1 : 0;
    lam1 = __fsub_rn(src, (float)i1);
    lam0 = __fsub_rn(1.f, lam1);
}

// every product and sum rounded on its own (no FMA contraction), in the
// association h0*(w0*a + w1*b) + h1*(w0*c + w1*d)
__device__ __forceinline__ float bilinear_blend(float h0, float h1, float w0, float w1, float a, float b,
                                                float c, float d) {
    const float top = __fadd_rn(__fmul_rn(w0, a), __fmul_rn(w1, b));
    const float bot = __fadd_rn(__fmul_rn(w0, c), __fmul_rn(w1, d));
    return __fadd_rn(__fmul_rn(h0, top), __fmul_rn(h1, bot));
}

struct UpsampleRole {
    using Args = UpsampleArgs;
    static int smem_bytes(const Args&, int) { return 0; }
    static int plan(Args&, int, int) { return 0; }

    template <int T>
    static __device__ __forceinline__ void run_vec4(const Args& a, const RoleCtx& ctx) {
        const unsigned W4 = (unsigned)a.outW >> 2;
        const unsigned oH = (unsigned)a.outH;
        const unsigned total = (unsigned)a.N * a.C * oH * W4;      // host guarantees < 2^31
        for (unsigned it = (unsigned)ctx.block * T + ctx.tid; it < total; it += (unsigned)ctx.nblocks * T) {
            const unsigned w4 = it % W4;
            const unsigned r = it / W4;
            const unsigned h2 = r % oH;
            const unsigned plane = r / oH;
            int h1, h1p;
            float h0l, h1l;
            bilinear_src(a.rheight, (int)h2, a.align_corners, a.H, h1, h1p, h0l, h1l);
            const float* r0 = a.in + (size_t)plane * a.H * a.W + (size_t)h1 * a.W;
            const float* r1 = r0 + (size_t)h1p * a.W;
            float o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                int w1, w1p;
                float w0l, w1l;
                bilinear_src(a.rwidth, (int)(w4 * 4) + k, a.align_corners, a.W, w1, w1p, w0l, w1l);
                o[k] = bilinear_blend(h0l, h1l, w0l, w1l, __ldg(r0 + w1), __ldg(r0 + w1 + w1p), __ldg(r1 + w1),
                                      __ldg(r1 + w1 + w1p));
            }
            stg_stream4(a.out + ((size_t)plane * oH + h2) * a.outW + w4 * 4, make_float4(o[0], o[1], o[2], o[3]));
        }
    }

    template <int T>
    static __device__ __forceinline__ void run_scalar(const Args& a, const RoleCtx& ctx) {
        const unsigned long long total = (unsigned long long)a.N * a.C * a.outH * a.outW;
        for (unsigned long long e = (unsigned long long)ctx.block * T + ctx.tid; e < total;
             e += (unsigned long long)ctx.nblocks * T) {
            const int w2 = (int)(e % a.outW);
            unsigned long long r = e / a.outW;
            const int h2 = (int)(r % a.outH);
            const unsigned long long plane = r / a.outH;
            int h1, h1p, w1, w1p;
            float h0l, h1l, w0l, w1l;
            bilinear_src(a.rheight, h2, a.align_corners, a.H, h1, h1p, h0l, h1l);
            bilinear_src(a.rwidth, w2, a.align_corners, a.W, w1, w1p, w0l, w1l);
            const float* r0 = a.in + (size_t)plane * a.H * a.W + (size_t)h1 * a.W;
            const float* r1 = r0 + (size_t)h1p * a.W;
            a.out[e] = bilinear_blend(h0l, h1l, w0l, w1l, __ldg(r0 + w1), __ldg(r0 + w1 + w1p), __ldg(r1 + w1),
                                      __ldg(r1 + w1 + w1p));
        }
    }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        if (a.mode == 1) run_vec4<T>(a, ctx);
        else run_scalar<T>(a, ctx);
    }
};

// =============================================================================
// histc: fixed-width bins over [lo, hi]
// =============================================================================
struct HistcArgs {
    const float* x;
    long long n;
    int nbins;
    float lo, hi;
    float range;        // hi - lo, rounded to fp32
    float inv_range;    // 1 / range, only meaningful when range_pow2
    int range_pow2;     // range is a power of two: multiplying by inv_range equals dividing by range
    unsigned* counts;   // zeroed by the caller (the entry point clears it on the stream)
    int copies;         // private shared-memory histograms per role (0 = global atomics only)
};

struct HistcRole {
    using Args = HistcArgs;
    static int smem_bytes(const Args& a, int) { return a.copies * a.nbins * (int)sizeof(unsigned); }
    // one private histogram per warp while that fits in 16 KB of shared memory,
    // fewer (shared between warps) beyond that, none when a single copy would not fit
    static int plan(Args& a, int T, int) {
        const int budget = 16 * 1024;
        int copies = budget / (a.nbins * (int)sizeof(unsigned));
        if (copies > T / 32) copies = T / 32;
        a.copies = copies;
        return 0;
    }

    static __device__ __forceinline__ void tally(const Args& a, float v, unsigned* hist) {
        if (v >= a.lo && v <= a.hi) {
            const float t = __fmul_rn(__fsub_rn(v, a.lo), (float)a.nbins);
            const float q = a.range_pow2 ? __fmul_rn(t, a.inv_range) : __fdiv_rn(t, a.range);
            int b = (int)q;
            if (b == a.nbins) b -= 1;
            atomicAdd(hist + b, 1u);
        }
    }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        unsigned* sh = reinterpret_cast<unsigned*>(ctx.smem);
        unsigned* hist = a.counts;
        if (a.copies > 0) {
            for (int i = ctx.tid; i < a.copies * a.nbins; i += T) sh[i] = 0u;
            role_sync<BAR, T>();
            hist = sh + ((ctx.tid >> 5) % a.copies) * a.nbins;
        }
        const long long n4 = a.n >> 2;
        for (long long i = (long long)ctx.block * T + ctx.tid; i < n4; i += (long long)ctx.nblocks * T) {
            const float4 v = ldg_stream4(a.x + 4 * i);
            tally(a, v.x, hist); tally(a, v.y, hist); tally(a, v.z, hist); tally(a, v.w, hist);
        }
        if (ctx.block == 0) {   // ragged tail (n % 4 values)
            for (long long i = 4 * n4 + ctx.tid; i < a.n; i += T) tally(a, __ldg(a.x + i), hist);
        }
        if (a.copies > 0) {
            role_sync<BAR, T>();
            for (int b = ctx.tid; b < a.nbins; b += T) {
                unsigned s = 0;
                for (int c = 0; c < a.copies; ++c) s += sh[c * a.nbins + b];
                if (s) atomicAdd(a.counts + b, s);
            }
        }
    }
};

// =============================================================================
// batch_norm_collect_statistics: per-channel mean and 1/sqrt(biased var + eps)
// =============================================================================
struct BnStatsArgs {
    const float* x;       // [N][C][HW]
    int N, C, HW;
    float eps;
    float total;          // N*HW as float
    float* mean;          // [C]
    float* invstd;        // [C]
    double* moments;      // optional [C][3]: n, n*mean, M2 + n*mean^2 (summable across GPUs), or null
    float* partial;       // scratch [C][S][3], used when S > 1
    unsigned* tickets;    // scratch [C], zero before the first call; every call leaves it zero
    int S;                // batch slices per channel (<= 32)
    int ips;              // images per slice
    int vec;              // HW % 4 == 0: 16-byte loads
    size_t ws_bytes;      // size of the caller's scratch buffer (host-side check only)
    void* ws;             // the caller's scratch buffer
};

constexpr int kBnMaxSlices = 32;
inline size_t bn_ticket_bytes(int C) { return (((size_t)C * sizeof(unsigned)) + 255) & ~(size_t)255; }
inline size_t bn_workspace_bytes(int C) {
    return bn_ticket_bytes(C) + (size_t)C * kBnMaxSlices * 3 * sizeof(float);
}

struct Moments { float n, mean, m2; };

__device__ __forceinline__ Moments chan_merge(Moments a, Moments b) {
    const float n = a.n + b.n;
    if (n == 0.f) return a;
    const float delta = b.mean - a.mean;
    const float fb = b.n / n;
    Moments r;
    r.n = n;
    r.mean = a.mean + delta * fb;
    r.m2 = a.m2 + b.m2 + delta * delta * a.n * fb;
    return r;
}

__device__ __forceinline__ Moments warp_merge(Moments m) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        Moments o;
        o.n = __shfl_xor_sync(0xffffffffu, m.n, off);
        o.mean = __shfl_xor_sync(0xffffffffu, m.mean, off);
        o.m2 = __shfl_xor_sync(0xffffffffu, m.m2, off);
        // both lanes of a pair must compute the same bits: merge in lane order
        const bool low = ((threadIdx.x & off) == 0);
        m = low ? chan_merge(m, o) : chan_merge(o, m);
    }
    return m;
}

struct BnStatsRole {
    using Args = BnStatsArgs;
    // two parity buffers of per-warp moments
    static int smem_bytes(const Args&, int T) { return 2 * 3 * (T / 32) * (int)sizeof(float); }
    // Split each channel's batch into S slices so that the grid has a few units
    // per block, without making a unit smaller than two loads per thread.
    static int plan(Args& a, int T, int grid) {
        const long long per_img = a.vec ? a.HW / 4 : a.HW;
        long long s_small = ((long long)a.N * per_img) / (2LL * T);
        if (s_small < 1) s_small = 1;
        if (s_small > a.N) s_small = a.N;
        if (s_small > kBnMaxSlices) s_small = kBnMaxSlices;
        long long s_want = (4LL * grid + a.C - 1) / a.C;
        if (s_want < 1) s_want = 1;
        long long S = s_want < s_small ? s_want : s_small;
        a.ips = (int)((a.N + S - 1) / S);
        a.S = (a.N + a.ips - 1) / a.ips;
        if (a.S > 1) {
            if (a.ws == nullptr || a.ws_bytes < bn_workspace_bytes(a.C)) return -4;   // HFUSE_ERR_WORKSPACE
            a.tickets = reinterpret_cast<unsigned*>(a.ws);
            a.partial = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(a.ws) + bn_ticket_bytes(a.C));
        }
        return 0;
    }

    static __device__ __forceinline__ void finish(const Args& a, int c, Moments m) {
        const float var = m.m2 / a.total;
        a.mean[c] = m.mean;
        a.invstd[c] = 1.f / sqrtf(var + a.eps);
        if (a.moments) {
            const double n = (double)a.N * (double)a.HW, mu = (double)m.mean;
            a.moments[3 * c + 0] = n;
            a.moments[3 * c + 1] = n * mu;
            a.moments[3 * c + 2] = (double)m.m2 + n * mu * mu;
        }
    }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        constexpr int NW = T / 32;
        static_assert(NW <= 32, "one warp merges the per-warp moments");
        float* sh = reinterpret_cast<float*>(ctx.smem);
        const int lane = ctx.tid & 31, warp = ctx.tid >> 5;
        const int units = a.C * a.S;
        int parity = 0;
        for (int u = ctx.block; u < units; u += ctx.nblocks, parity ^= 1) {
            const int c = u / a.S, s = u % a.S;
            const int n0 = s * a.ips, n1 = min(a.N, n0 + a.ips);
            // ---- per-thread Welford, four independent lanes sharing one count
            float cnt = 0.f;
            float mu[4] = {0.f, 0.f, 0.f, 0.f}, m2[4] = {0.f, 0.f, 0.f, 0.f};
            float tail_n = 0.f;
            if (a.vec) {
                const int hw4 = a.HW >> 2;
                const int total = (n1 - n0) * hw4;
                for (int k = ctx.tid; k < total; k += T) {
                    const int n = n0 + k / hw4, off = k % hw4;
                    const float4 v = ldg_stream4(a.x + ((size_t)n * a.C + c) * a.HW + 4 * off);
                    cnt += 1.f;
                    const float r = __frcp_rn(cnt);
                    const float xs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float d = xs[j] - mu[j];
                        mu[j] += d * r;
                        m2[j] += d * (xs[j] - mu[j]);
                    }
                }
            } else {
                const int total = (n1 - n0) * a.HW;
                for (int k = ctx.tid; k < total; k += T) {
                    const int n = n0 + k / a.HW, off = k % a.HW;
                    const float xv = __ldg(a.x + ((size_t)n * a.C + c) * a.HW + off);
                    tail_n += 1.f;
                    const float d = xv - mu[0];
                    mu[0] += d * __frcp_rn(tail_n);
                    m2[0] += d * (xv - mu[0]);
                }
            }
            Moments m;
            if (a.vec) {
                Moments q0{cnt, mu[0], m2[0]}, q1{cnt, mu[1], m2[1]}, q2{cnt, mu[2], m2[2]}, q3{cnt, mu[3], m2[3]};
                m = chan_merge(chan_merge(q0, q1), chan_merge(q2, q3));
            } else {
                m = Moments{tail_n, mu[0], m2[0]};
            }
            // ---- warp, then role-wide merge through shared memory and the role's barrier
            m = warp_merge(m);
            float* buf = sh + parity * 3 * NW;
            if (lane == 0) { buf[warp] = m.n; buf[NW + warp] = m.mean; buf[2 * NW + warp] = m.m2; }
            role_sync<BAR, T>();
            if (warp == 0) {
                Moments w = (lane < NW) ? Moments{buf[lane], buf[NW + lane], buf[2 * NW + lane]}
                                        : Moments{0.f, 0.f, 0.f};
                w = warp_merge(w);
                if (a.S == 1) {
                    if (lane == 0) finish(a, c, w);
                } else {
                    // publish this slice, then the last slice to arrive folds all of
                    // them in slice order (so the result does not depend on timing)
                    unsigned ticket = 0;
                    if (lane == 0) {
                        float* p = a.partial + ((size_t)c * a.S + s) * 3;
                        __stcg(p, w.n); __stcg(p + 1, w.mean); __stcg(p + 2, w.m2);
                        __threadfence();
                        ticket = atomicAdd(a.tickets + c, 1u);
                    }
                    ticket = __shfl_sync(0xffffffffu, ticket, 0);
                    if (ticket == (unsigned)(a.S - 1)) {
                        __threadfence();
                        Moments q{0.f, 0.f, 0.f};
                        if (lane < a.S) {
                            const float* p = a.partial + ((size_t)c * a.S + lane) * 3;
                            q = Moments{__ldcg(p), __ldcg(p + 1), __ldcg(p + 2)};
                        }
                        q = warp_merge(q);
                        if (lane == 0) {
                            finish(a, c, q);
                            a.tickets[c] = 0u;     // ready for the next call
                        }
                    }
                }
            }
            // the parity buffer keeps warp 0's reads of this unit apart from
            // the next unit's writes; the unit after that is fenced by the
            // next role barrier
        }
    }
};

}  // namespace hfuse
