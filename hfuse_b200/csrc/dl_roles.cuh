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
    int mode;   // 0 = generic (one output element per item), 1 = 3x3 stride-1 tile path (4 columns per item),
                // 2 = the same with 8 columns per item and 256-bit stores (pad 1, Wc % 8 == 0, col 32-byte aligned),
                // 3 = 3x3 stride-1 pad-1 through a shared-memory tile and bulk (TMA) stores (run_bulk)
    int band, bands;          // mode 3: output rows per work unit, units per plane
    int bulk_ok;              // the shape allows mode 3 (the host picks the mode per kernel or pair)
    FastDiv div_bands;        // mode 3: by bands
    FastDiv div_w4, div_hc;   // tile paths: by Wc/4 (mode 1) or Wc/8 (mode 2), and by Hc
    FastDiv div_wc, div_taps, div_kw;   // generic path with fewer than 2^31 outputs (small != 0)
    int small;
};

struct Im2colRole {
    using Args = Im2colArgs;
    // mode 3: two buffers of three column-shifted copies of band + 2 input rows
    static int smem_bytes(const Args& a, int) { return a.mode == 3 ? 2 * 3 * (a.band + 2) * a.Wc * (int)sizeof(float) : 0; }
    static int plan(Args&, int /*T*/, int /*grid*/) { return 0; }

    // 3x3 / stride 1 / pad 1 / dilation 1 (so Wc == W, Hc == H), W % 4 == 0, through shared memory.
    // Work unit = (plane, band of `band` output rows).  The role loads the band's band + 2 input
    // rows once (16-byte loads) and lays them down three times in shared memory (16-byte stores),
    // shifted by one column to the right, not at all, and one to the left, with the zero padding written in:
    // copy j, row r, column w holds im[h0 - 1 + r][w - 1 + j].  Tap (i, j) of the band is then the
    // CONTIGUOUS block of rows i .. i + band - 1 of copy j, and its place in `col` is contiguous
    // too (rows h0 .. h0 + band - 1 of one tap plane), so each of the nine taps leaves as one bulk
    // copy of band * Wc * 4 bytes issued by one thread.  Two buffers: the copies of one unit drain
    // while the next unit is loaded.
    template <int T, int BAR>
    static __device__ __forceinline__ void run_bulk(const Args& a, const RoleCtx& ctx) {
        const int Wc = a.Wc, W4 = a.W >> 2;
        const unsigned copy_elems = (unsigned)(a.band + 2) * Wc;
        float* sm = reinterpret_cast<float*>(ctx.smem);
        const unsigned units = (unsigned)a.N * a.C * a.bands;
        const size_t tap_stride = (size_t)a.Hc * a.Wc;
        int buf = 0;
        for (unsigned u = ctx.block; u < units; u += ctx.nblocks, buf ^= 1) {
            unsigned bi;
            const unsigned plane = fast_divmod(u, a.div_bands, bi);
            const int h0 = (int)bi * a.band;
            const int nrows = min(a.band, a.Hc - h0);
            float* tile = sm + (size_t)buf * 3 * copy_elems;
            // the copies that read this buffer two units ago must have finished reading it
            if (ctx.tid == 0) bulk_wait_read<1>();
            role_sync<BAR, T>();
            const float* src = a.im + (size_t)plane * a.H * a.W;
            // One 16-byte load per item (row r, columns 4m .. 4m+3); the columns just outside come
            // from the neighbouring lanes (a warp walks along the rows), so each of the three copies
            // is written with one aligned 16-byte shared-memory store.  Warp-uniform trip count:
            // every lane takes part in the shuffles.
            const int total = (nrows + 2) * W4;
            const int lane = ctx.tid & 31;
            for (int base = ctx.tid & ~31; base < total; base += T) {
                const int it = base + lane;
                const bool live = it < total;
                const int r = live ? it / W4 : 0, m = live ? it - r * W4 : 0;
                const int hi = h0 - 1 + r;
                const bool row_ok = live && hi >= 0 && hi < a.H;
                const float* p = src + (size_t)(row_ok ? hi : 0) * a.W + 4 * m;
                const float4 v = row_ok ? __ldg(reinterpret_cast<const float4*>(p)) : make_float4(0.f, 0.f, 0.f, 0.f);
                float left = __shfl_up_sync(0xffffffffu, v.w, 1), right = __shfl_down_sync(0xffffffffu, v.x, 1);
                if (lane == 0 && m > 0) left = row_ok ? __ldg(p - 1) : 0.f;            // the neighbour sits in another warp
                if (lane == 31 && m + 1 < W4) right = row_ok ? __ldg(p + 4) : 0.f;
                if (m == 0) left = 0.f;                                                 // zero padding at the row ends
                if (m + 1 == W4) right = 0.f;
                if (!live) continue;
                float* row = tile + r * Wc + 4 * m;
                *reinterpret_cast<float4*>(row) = make_float4(left, v.x, v.y, v.z);                      // j = 0: im[w - 1]
                *reinterpret_cast<float4*>(row + copy_elems) = v;                                        // j = 1
                *reinterpret_cast<float4*>(row + 2 * copy_elems) = make_float4(v.y, v.z, v.w, right);    // j = 2: im[w + 1]
            }
            fence_proxy_async_shared();
            role_sync<BAR, T>();
            if (ctx.tid == 0) {
                float* dst = a.col + (size_t)plane * 9 * tap_stride + (size_t)h0 * Wc;
                const uint32_t bytes = (uint32_t)nrows * Wc * (uint32_t)sizeof(float);
#pragma unroll
                for (int i = 0; i < 3; ++i)
#pragma unroll
                    for (int j = 0; j < 3; ++j)
                        bulk_store(dst + (size_t)(i * 3 + j) * tap_stride, tile + j * copy_elems + i * Wc, bytes);
                bulk_commit();
            }
        }
        if (ctx.tid == 0) bulk_wait<0>();      // shared memory must outlive the copies that read it
    }

    // 3x3 / stride 1 / dilation 1, Wc % 4 == 0: one item = four adjacent
    // output columns of one (plane, row).  The thread reads the 3 x 6 input
    // patch once and writes all nine taps as aligned 16-byte streaming stores,
    // so every input element is fetched from L1/L2 three times instead of nine
    // and 90 % of the traffic (the stores) is fully coalesced.
    template <int T>
    static __device__ __forceinline__ void run_k3s1(const Args& a, const RoleCtx& ctx) {
        constexpr int KH = 3, KW = 3;
        const unsigned total = (unsigned)a.N * a.C * a.Hc * (a.Wc >> 2);     // host guarantees < 2^31
        const size_t tap_stride = (size_t)a.Hc * a.Wc;
        // pad 1 and W % 4 == 0: the four centre columns are one aligned 16-byte load and the two
        // outer columns are the neighbouring lanes' centre values (a warp walks along a row)
        const bool vec_mid = (a.pw == 1) && ((a.W & 3) == 0);
        const unsigned lane = ctx.tid & 31;
        // warp-uniform trip count: every lane takes part in the shuffles
        for (unsigned base = (unsigned)ctx.block * T + (ctx.tid & ~31); base < total;
             base += (unsigned)ctx.nblocks * T) {
            const bool live = base + lane < total;
            const unsigned it = live ? base + lane : total - 1;
            unsigned w4, h;
            const unsigned r = fast_divmod(it, a.div_w4, w4);
            const unsigned plane = fast_divmod(r, a.div_hc, h);
            const float* src = a.im + (size_t)plane * a.H * a.W;
            float* dst = a.col + (size_t)plane * (KH * KW) * tap_stride + h * a.Wc + w4 * 4;
            const int wi0 = (int)(w4 * 4) - a.pw;
            float v[KH][4 + KW - 1];
            if (vec_mid) {
                // neighbours in the same row sit in lanes +-1 unless the row (or the warp) ends there
                const bool has_l = w4 > 0, has_r = (int)(w4 * 4) + 4 < a.W;
#pragma unroll
                for (int i = 0; i < KH; ++i) {
                    const int hi = (int)h - a.ph + i;
                    const bool row_ok = (hi >= 0) && (hi < a.H);
                    const float* row = src + (size_t)(row_ok ? hi : 0) * a.W + w4 * 4;
                    const float4 m = row_ok ? __ldg(reinterpret_cast<const float4*>(row))
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
                    float left = __shfl_up_sync(0xffffffffu, m.w, 1);
                    float right = __shfl_down_sync(0xffffffffu, m.x, 1);
                    if (lane == 0 && has_l) left = row_ok ? __ldg(row - 1) : 0.f;
                    if (lane == 31 && has_r) right = row_ok ? __ldg(row + 4) : 0.f;
                    v[i][0] = has_l ? left : 0.f;
                    v[i][1] = m.x; v[i][2] = m.y; v[i][3] = m.z; v[i][4] = m.w;
                    v[i][5] = has_r ? right : 0.f;
                }
            } else {
#pragma unroll
                for (int i = 0; i < KH; ++i) {
                    const int hi = (int)h - a.ph + i;
                    const bool row_ok = (hi >= 0) && (hi < a.H);
                    const float* row = src + (size_t)(row_ok ? hi : 0) * a.W;
#pragma unroll
                    for (int x = 0; x < 4 + KW - 1; ++x) {
                        const int wi = wi0 + x;
                        v[i][x] = (row_ok && wi >= 0 && wi < a.W) ? __ldg(row + wi) : 0.f;
                    }
                }
            }
            if (!live) continue;
#pragma unroll
            for (int i = 0; i < KH; ++i)
#pragma unroll
                for (int j = 0; j < KW; ++j)
                    stg_stream4(dst + (size_t)(i * KW + j) * tap_stride,
                                make_float4(v[i][j], v[i][j + 1], v[i][j + 2], v[i][j + 3]));
        }
    }

    // 3x3 / stride 1 / pad 1, Wc % 8 == 0: eight adjacent output columns per item, two aligned
    // 16-byte loads per input row, outer columns from the neighbouring lanes, nine 32-byte stores.
    template <int T>
    static __device__ __forceinline__ void run_k3s1_wide(const Args& a, const RoleCtx& ctx) {
        const unsigned W8 = (unsigned)a.Wc >> 3;
        const unsigned total = (unsigned)a.N * a.C * a.Hc * W8;     // host guarantees < 2^31
        const size_t tap_stride = (size_t)a.Hc * a.Wc;
        const unsigned lane = ctx.tid & 31;
        for (unsigned base = (unsigned)ctx.block * T + (ctx.tid & ~31); base < total;
             base += (unsigned)ctx.nblocks * T) {
            const bool live = base + lane < total;
            const unsigned it = live ? base + lane : total - 1;
            unsigned w8, h;
            const unsigned r = fast_divmod(it, a.div_w4, w8);
            const unsigned plane = fast_divmod(r, a.div_hc, h);
            const float* src = a.im + (size_t)plane * a.H * a.W;
            float* dst = a.col + (size_t)plane * 9 * tap_stride + h * a.Wc + w8 * 8;
            const bool has_l = w8 > 0, has_r = w8 + 1 < W8;
            float v[3][10];
#pragma unroll
            for (int i = 0; i < 3; ++i) {
                const int hi = (int)h - 1 + i;
                const bool row_ok = (hi >= 0) && (hi < a.H);
                const float* row = src + (size_t)(row_ok ? hi : 0) * a.W + w8 * 8;
                const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 m0 = row_ok ? __ldg(reinterpret_cast<const float4*>(row)) : z;
                const float4 m1 = row_ok ? __ldg(reinterpret_cast<const float4*>(row + 4)) : z;
                float left = __shfl_up_sync(0xffffffffu, m1.w, 1);
                float right = __shfl_down_sync(0xffffffffu, m0.x, 1);
                if (lane == 0 && has_l) left = row_ok ? __ldg(row - 1) : 0.f;
                if (lane == 31 && has_r) right = row_ok ? __ldg(row + 8) : 0.f;
                v[i][0] = has_l ? left : 0.f;
                v[i][1] = m0.x; v[i][2] = m0.y; v[i][3] = m0.z; v[i][4] = m0.w;
                v[i][5] = m1.x; v[i][6] = m1.y; v[i][7] = m1.z; v[i][8] = m1.w;
                v[i][9] = has_r ? right : 0.f;
            }
            if (!live) continue;
#pragma unroll
            for (int i = 0; i < 3; ++i)
#pragma unroll
                for (int j = 0; j < 3; ++j) stg_stream8(dst + (size_t)(i * 3 + j) * tap_stride, &v[i][j]);
        }
    }

    template <int T>
    static __device__ __forceinline__ void run_generic(const Args& a, const RoleCtx& ctx) {
        if (a.small) {      // every index fits 31 bits: multiply-high divisions only
            const unsigned total = (unsigned)a.N * a.C * a.kh * a.kw * a.Hc * a.Wc;
            for (unsigned e = (unsigned)ctx.block * T + ctx.tid; e < total; e += (unsigned)ctx.nblocks * T) {
                unsigned w, h, tap, j;
                unsigned r = fast_divmod(e, a.div_wc, w);
                r = fast_divmod(r, a.div_hc, h);
                const unsigned plane = fast_divmod(r, a.div_taps, tap);
                const unsigned i = fast_divmod(tap, a.div_kw, j);
                const int hi = (int)h * a.sh - a.ph + (int)i * a.dh;
                const int wi = (int)w * a.sw - a.pw + (int)j * a.dw;
                float v = 0.f;
                if (hi >= 0 && hi < a.H && wi >= 0 && wi < a.W)
                    v = __ldg(a.im + (size_t)plane * a.H * a.W + (size_t)hi * a.W + wi);
                stg_stream1(a.col + e, v);
            }
            return;
        }
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
        if (a.mode == 3) run_bulk<T, BAR>(a, ctx);
        else if (a.mode == 2) run_k3s1_wide<T>(a, ctx);
        else if (a.mode == 1) run_k3s1<T>(a, ctx);
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
    FastDiv div_p4, div_ph;   // 2x2 path: by pW/4 and by pH
    int wide;                 // idx is 32-byte aligned: one 256-bit store for the four indices
    FastDiv div_pw;           // generic path with fewer than 2^31 outputs (small != 0): by pW (and div_ph by pH)
    int small;
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
            unsigned p4, oh;
            const unsigned r = fast_divmod(it, a.div_p4, p4);
            const unsigned plane = fast_divmod(r, a.div_ph, oh);
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
            if (a.wide) stg_stream_4xi64(a.idx + o_off, at[0], at[1], at[2], at[3]);
            else { stg_stream_2xi64(a.idx + o_off, at[0], at[1]); stg_stream_2xi64(a.idx + o_off + 2, at[2], at[3]); }
        }
    }

    template <int T>
    static __device__ __forceinline__ void run_generic(const Args& a, const RoleCtx& ctx) {
        const unsigned long long total = (unsigned long long)a.N * a.C * a.pH * a.pW;
        for (unsigned long long e = (unsigned long long)ctx.block * T + ctx.tid; e < total;
             e += (unsigned long long)ctx.nblocks * T) {
            int ow, oh;
            unsigned long long plane;
            if (a.small) {
                unsigned uw, uh;
                const unsigned r = fast_divmod((unsigned)e, a.div_pw, uw);
                plane = fast_divmod(r, a.div_ph, uh);
                ow = (int)uw; oh = (int)uh;
            } else {
                ow = (int)(e % a.pW);
                const unsigned long long r = e / a.pW;
                oh = (int)(r % a.pH);
                plane = r / a.pH;
            }
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
    int mode;   // 0 = one output per item, 1 = four adjacent outputs per item (outW % 4 == 0),
                // 2 = exact x2 strip path (run_x2)
    FastDiv div_w4, div_j;   // x2 path: by W/4 and by H+1
    int wide;                // output is 32-byte aligned: 256-bit stores
    FastDiv div_ow4, div_oh, div_ow;   // 4-wide path: by outW/4 and outH; scalar path (small != 0): by outW and outH
    int small;
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

    // Items of the vector paths (the scalar path counts in 64 bits and is never split):
    // the 4-wide path works on N*C*outH*(outW/4) items, the x2 strip path on N*C*(H+1)*(W/4).
    static __host__ __device__ __forceinline__ unsigned vec_items(const Args& a) {
        return a.mode == 2 ? (unsigned)a.N * a.C * ((unsigned)a.H + 1) * ((unsigned)a.W >> 2)
                           : (unsigned)a.N * a.C * (unsigned)a.outH * ((unsigned)a.outW >> 2);
    }
    // only the vector paths can hand part of their items to another thread range
    static __host__ __device__ __forceinline__ bool splittable(const Args& a) { return a.mode != 0; }
    // A range of items handed to another thread range must start on a row boundary (the x2
    // path reads its left and right neighbours' columns from the adjacent lanes).
    static __host__ __device__ __forceinline__ unsigned vec_row_items(const Args& a) {
        return a.mode == 2 ? (unsigned)a.W >> 2 : (unsigned)a.outW >> 2;
    }

    // four adjacent outputs of one output row (item `it` of the 4-wide path)
    static __device__ __forceinline__ void vec4_item(const Args& a, unsigned it) {
        const unsigned oH = (unsigned)a.outH;
        unsigned w4, h2;
        const unsigned r = fast_divmod(it, a.div_ow4, w4);
        const unsigned plane = fast_divmod(r, a.div_oh, h2);
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

    template <int T>
    static __device__ __forceinline__ void run_vec4(const Args& a, const RoleCtx& ctx, unsigned begin, unsigned end) {
        for (unsigned it = begin + (unsigned)ctx.block * T + ctx.tid; it < end; it += (unsigned)ctx.nblocks * T)
            vec4_item(a, it);
    }

    // Exact x2, align_corners = false, W % 4 == 0.  The source weights are
    // then exactly {0.25, 0.75} (1 and 0 on the clamped first row / column), so
    // the generic formula can be evaluated from registers: one item = input
    // columns 4m-1 .. 4m+4 of two neighbouring input rows (two 16-byte loads
    // and four scalars) -> an 8-wide strip of the two output rows between them
    // (four 16-byte stores).  Every product and sum is the one the generic
    // path computes, so both paths give the same bits.
    // One warp's chunk of the x2 strip path: items base .. base + 31 (base a multiple of 32 below
    // `total`), one item per lane; every lane of the warp takes part in the shuffles, lanes beyond
    // `total` re-run the last item and store nothing.
    static __device__ __forceinline__ void x2_chunk(const Args& a, unsigned base, unsigned total, unsigned lane) {
        const unsigned W4 = (unsigned)a.W >> 2;
        const bool live = base + lane < total;
        const unsigned it = live ? base + lane : total - 1;
        unsigned m, ju;
        const unsigned r = fast_divmod(it, a.div_w4, m);
        const unsigned plane = fast_divmod(r, a.div_j, ju);
        const int j = (int)ju;
        // output rows 2j-1 (if j >= 1) and 2j (if j <= H-1) blend input rows ra and rb
        const int ra = j > 0 ? j - 1 : 0;
        const int rb = j == 0 ? (a.H > 1 ? 1 : 0) : (j < a.H ? j : a.H - 1);
        const float* pa = a.in + (size_t)plane * a.H * a.W + ra * a.W + 4 * m;
        const float* pb = a.in + (size_t)plane * a.H * a.W + rb * a.W + 4 * m;
        const bool has_l = m > 0, has_r = m + 1 < W4;
        const float4 qa = __ldg(reinterpret_cast<const float4*>(pa));
        const float4 qb = __ldg(reinterpret_cast<const float4*>(pb));
        // columns 4m-1 and 4m+4 are the neighbouring lanes' values unless the row (or the warp) ends
        float la = __shfl_up_sync(0xffffffffu, qa.w, 1), lb = __shfl_up_sync(0xffffffffu, qb.w, 1);
        float ra_ = __shfl_down_sync(0xffffffffu, qa.x, 1), rb_ = __shfl_down_sync(0xffffffffu, qb.x, 1);
        if (lane == 0 && has_l) { la = __ldg(pa - 1); lb = __ldg(pb - 1); }
        if (lane == 31 && has_r) { ra_ = __ldg(pa + 4); rb_ = __ldg(pb + 4); }
        if (!live) return;
        float ca[6], cb[6];          // columns 4m-1 .. 4m+4
        ca[1] = qa.x; ca[2] = qa.y; ca[3] = qa.z; ca[4] = qa.w;
        cb[1] = qb.x; cb[2] = qb.y; cb[3] = qb.z; cb[4] = qb.w;
        ca[0] = has_l ? la : 0.f;  cb[0] = has_l ? lb : 0.f;
        ca[5] = has_r ? ra_ : ca[4]; cb[5] = has_r ? rb_ : cb[4];   // w1p = 0 at the edge
        // horizontal blends of both input rows for output columns 8m .. 8m+7
        float ta[8], tb[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            // even column 8m+2k: source 4m+k-0.25 -> (4m+k-1, 4m+k) with weights (0.25, 0.75);
            // the very first column clamps to source 0 -> weights (1, 0) on columns (0, 1)
            if (k == 0 && !has_l) {
                ta[0] = __fadd_rn(__fmul_rn(1.f, ca[1]), __fmul_rn(0.f, a.W > 1 ? ca[2] : ca[1]));
                tb[0] = __fadd_rn(__fmul_rn(1.f, cb[1]), __fmul_rn(0.f, a.W > 1 ? cb[2] : cb[1]));
            } else {
                ta[2 * k] = __fadd_rn(__fmul_rn(0.25f, ca[k]), __fmul_rn(0.75f, ca[k + 1]));
                tb[2 * k] = __fadd_rn(__fmul_rn(0.25f, cb[k]), __fmul_rn(0.75f, cb[k + 1]));
            }
            // odd column 8m+2k+1: source 4m+k+0.25 -> (4m+k, 4m+k+1) with weights (0.75, 0.25)
            ta[2 * k + 1] = __fadd_rn(__fmul_rn(0.75f, ca[k + 1]), __fmul_rn(0.25f, ca[k + 2]));
            tb[2 * k + 1] = __fadd_rn(__fmul_rn(0.75f, cb[k + 1]), __fmul_rn(0.25f, cb[k + 2]));
        }
        float* orow = a.out + (size_t)plane * a.outH * a.outW + 8 * m;
        if (j > 0) {        // odd output row 2j-1: weights (0.75, 0.25)
            float o[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = __fadd_rn(__fmul_rn(0.75f, ta[k]), __fmul_rn(0.25f, tb[k]));
            float* p = orow + (size_t)(2 * j - 1) * a.outW;
            if (a.wide) stg_stream8(p, o);
            else { stg_stream4(p, make_float4(o[0], o[1], o[2], o[3])); stg_stream4(p + 4, make_float4(o[4], o[5], o[6], o[7])); }
        }
        if (j < a.H) {      // even output row 2j: weights (0.25, 0.75), or (1, 0) on the clamped row 0
            const float h0 = j == 0 ? 1.f : 0.25f, h1 = j == 0 ? 0.f : 0.75f;
            float o[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = __fadd_rn(__fmul_rn(h0, ta[k]), __fmul_rn(h1, tb[k]));
            float* p = orow + (size_t)(2 * j) * a.outW;
            if (a.wide) stg_stream8(p, o);
            else { stg_stream4(p, make_float4(o[0], o[1], o[2], o[3])); stg_stream4(p + 4, make_float4(o[4], o[5], o[6], o[7])); }
        }
    }

    template <int T>
    static __device__ __forceinline__ void run_x2(const Args& a, const RoleCtx& ctx, unsigned begin, unsigned total) {
        const unsigned lane = ctx.tid & 31;
        // items [begin, total) (the host guarantees fewer than 2^31 in all); warp-uniform trip count
        for (unsigned base = begin + (unsigned)ctx.block * T + (ctx.tid & ~31); base < total;
             base += (unsigned)ctx.nblocks * T)
            x2_chunk(a, base, total, lane);
    }

    // Items of a vector path drawn from a cursor that all warps of the block share (any thread
    // range may call this, at any time): warp chunk c of block b covers items (c * nblocks + b) * 32
    // onward, so the chunks in flight across the grid are neighbours in memory whichever warp
    // takes them.  The next chunk number is asked for before the current chunk is worked on.
    static __device__ __forceinline__ void run_pool(const Args& a, int block, int nblocks, unsigned* cursor, unsigned lane) {
        const unsigned total = vec_items(a);
        unsigned c = 0;
        if (lane == 0) c = atomicAdd(cursor, 1u);
        for (;;) {
            c = __shfl_sync(0xffffffffu, c, 0);
            const unsigned long long base = ((unsigned long long)c * (unsigned)nblocks + (unsigned)block) * 32ull;
            if (base >= total) break;          // every warp overshoots the cursor once
            if (lane == 0) c = atomicAdd(cursor, 1u);
            if (a.mode == 2) x2_chunk(a, (unsigned)base, total, lane);
            else if ((unsigned)base + lane < total) vec4_item(a, (unsigned)base + lane);
        }
    }

    template <int T>
    static __device__ __forceinline__ void run_scalar(const Args& a, const RoleCtx& ctx) {
        const unsigned long long total = (unsigned long long)a.N * a.C * a.outH * a.outW;
        for (unsigned long long e = (unsigned long long)ctx.block * T + ctx.tid; e < total;
             e += (unsigned long long)ctx.nblocks * T) {
            int w2, h2;
            unsigned long long plane;
            if (a.small) {
                unsigned uw, uh;
                const unsigned r = fast_divmod((unsigned)e, a.div_ow, uw);
                plane = fast_divmod(r, a.div_oh, uh);
                w2 = (int)uw; h2 = (int)uh;
            } else {
                w2 = (int)(e % a.outW);
                const unsigned long long r = e / a.outW;
                h2 = (int)(r % a.outH);
                plane = r / a.outH;
            }
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
        if (a.mode == 2) run_x2<T>(a, ctx, 0u, vec_items(a));
        else if (a.mode == 1) run_vec4<T>(a, ctx, 0u, vec_items(a));
        else run_scalar<T>(a, ctx);
    }

    // Items [begin, end) of a vector path, for a kernel that hands part of the work to another
    // thread range (begin and end on row boundaries).  The scalar path is not split: the
    // caller passes begin = 0 to the range that owns it and an empty range to the other.
    template <int T>
    static __device__ __forceinline__ void run_range(const Args& a, const RoleCtx& ctx, unsigned begin, unsigned end) {
        if (a.mode == 2) { if (begin < end) run_x2<T>(a, ctx, begin, end); }
        else if (a.mode == 1) run_vec4<T>(a, ctx, begin, end);
        else if (begin == 0u && end != 0u) run_scalar<T>(a, ctx);
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
    float fbins;        // nbins as fp32 (exact: nbins <= 2^24)
    float range;        // hi - lo, rounded to fp32
    float inv_range;    // 1 / range, only meaningful when range_pow2
    int range_pow2;     // range is a power of two: multiplying by inv_range equals dividing by range
    unsigned* counts;   // zeroed on the stream before the kernel's flush (see the entry points)
    int copies;         // private shared-memory histograms per role (0 = global atomics only)
    int lane_private;   // shared histogram laid out [bin][32 lanes]: lane l only ever touches bank l
    int fast;           // fewer than 2^31 16-byte items: 32-bit indices and the peeled loop
    int bulk_ok;        // the shape allows the bulk-load sweep (the host picks per kernel or pair)
    int bulk;           // 1: the values come through bulk (TMA) copies into a shared-memory ring (sweep_bulk)
};

struct HistcRole {
    using Args = HistcArgs;
    // bulk-load sweep: a ring of kBulkBufs buffers of kBulkU 16-byte items per thread behind the histogram,
    // with a "full" and an "empty" mbarrier per buffer in front of it
    static constexpr int kBulkU = 2, kBulkBufs = 4;
    static __host__ __device__ __forceinline__ int bulk_chunk_bytes(int T) { return T * kBulkU * 16; }
    static int smem_bytes(const Args& a, int T) {
        return (a.lane_private ? 32 : a.copies) * a.nbins * (int)sizeof(unsigned) +
               (a.bulk ? 64 + kBulkBufs * bulk_chunk_bytes(T) : 0);
    }
    // Up to 256 bins: one counter per (bin, lane) = 32 KB at most.  Lane l of every warp
    // only touches word bin*32 + l, i.e. bank l, so a warp's 32 increments never meet in a
    // bank or an address whatever the data looks like.  Beyond that: one private histogram
    // per warp while that fits in 16 KB, fewer (shared between warps) for more bins, global
    // atomics only when a single copy would not fit.
    static int plan(Args& a, int T, int) {
        if (a.nbins <= 256) {
            a.lane_private = 1;
            a.copies = 1;
            return 0;
        }
        a.lane_private = 0;
        a.bulk = 0;          // the ring sits behind the [bin][lane] histogram only
        const int budget = 16 * 1024;
        int copies = budget / (a.nbins * (int)sizeof(unsigned));
        if (copies > T / 32) copies = T / 32;
        a.copies = copies;
        return 0;
    }

    static __device__ __forceinline__ void red_shared_inc(uint32_t saddr) {
        asm volatile("red.shared.add.u32 [%0], 1;" ::"r"(saddr) : "memory");
    }

    // bin of v, or -1 when v is outside [lo, hi] or NaN
    static __device__ __forceinline__ int bin_of(const Args& a, float v) {
        if (!(v >= a.lo && v <= a.hi)) return -1;
        const float t = __fmul_rn(__fsub_rn(v, a.lo), a.fbins);
        const float q = a.range_pow2 ? __fmul_rn(t, a.inv_range) : __fdiv_rn(t, a.range);
        const int b = (int)q;
        return b == a.nbins ? b - 1 : b;
    }

    // The same bin with as few instructions as the arithmetic allows (the sweep is bound by
    // instruction issue, not by memory, when it spends thirty instructions on a value):
    // d = v - lo is computed anyway and is >= 0 exactly when v >= lo (a difference of two
    // floats is zero only if they are equal, and NaN compares false), so the range test costs
    // one more compare (v <= hi); the products and the quotient are rounded one by one in the
    // order above, so the bin is the same; q (at most nbins, and a shared-memory histogram has
    // at most a few thousand bins) truncates by adding 2^23 towards zero and reading the
    // mantissa; the top edge (v == hi gives q == nbins) is a min.  The reduction is predicated,
    // so whatever an out-of-range value produced as a bin is never used.
    template <int SHIFT, bool POW2>
    static __device__ __forceinline__ void count(const Args& a, float v, uint32_t sbase, int last) {
        const float d = __fsub_rn(v, a.lo);
        const float t = __fmul_rn(d, a.fbins);
        const float q = POW2 ? __fmul_rn(t, a.inv_range) : __fdiv_rn(t, a.range);
        const int b = min(__float_as_int(__fadd_rz(q, 8388608.f)) & 0x7fffff, last);
        if ((d >= 0.f) && (v <= a.hi)) red_shared_inc(sbase + ((uint32_t)b << SHIFT));
    }

    // Sweep over fewer than 2^31 16-byte items into a shared-memory histogram.  The items of a
    // thread are i0 + k * stride; the first `full` groups of U items are in range for every
    // thread, so the main loop carries no bounds checks, and the loads of group k + 1 are issued
    // before group k is counted (every warp keeps loads in flight while its reductions drain).
    template <int T, int SHIFT, bool POW2>
    static __device__ __forceinline__ void sweep_fast(const Args& a, const RoleCtx& ctx, uint32_t sbase) {
        constexpr int U = 4;
        const int last = a.nbins - 1;
        const uint32_t n4 = (uint32_t)(a.n >> 2);
        const uint32_t stride = (uint32_t)ctx.nblocks * T;
        const uint32_t full = n4 / (stride * U);
        uint32_t i = (uint32_t)ctx.block * T + ctx.tid;
        auto count4 = [&](const float4& v) {
            count<SHIFT, POW2>(a, v.x, sbase, last); count<SHIFT, POW2>(a, v.y, sbase, last);
            count<SHIFT, POW2>(a, v.z, sbase, last); count<SHIFT, POW2>(a, v.w, sbase, last);
        };
        if (full > 0) {
            float4 nxt[U];
#pragma unroll
            for (int u = 0; u < U; ++u) nxt[u] = ldg_stream4(a.x + 4ull * (i + u * stride));
            for (uint32_t k = 1; k < full; ++k) {
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) v[u] = nxt[u];
                i += U * stride;
#pragma unroll
                for (int u = 0; u < U; ++u) nxt[u] = ldg_stream4(a.x + 4ull * (i + u * stride));
#pragma unroll
                for (int u = 0; u < U; ++u) count4(v[u]);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) count4(nxt[u]);
            i += U * stride;
        }
        for (; i < n4; i += stride) count4(ldg_stream4(a.x + 4ull * i));     // ragged end: fewer than U items per thread
        if (ctx.block == 0)      // n % 4 values
            for (long long j = 4ll * n4 + ctx.tid; j < a.n; j += T) count<SHIFT, POW2>(a, __ldg(a.x + j), sbase, last);
    }

    // Bulk-load sweep ([bin][lane] histogram, fewer than 2^31 items).  The input is cut into chunks of
    // T * kBulkU 16-byte items; block b takes chunks b, b + blocks, ...  Thread 0 brings a chunk into
    // the ring with ONE bulk (TMA) copy that signals the buffer's "full" mbarrier with its bytes; every
    // warp waits for "full", reads its items (thread t: items t, t + T, ...: no bank conflicts), says so
    // on the buffer's "empty" mbarrier (one arrival per warp) and counts; thread 0 refills a buffer once
    // its "empty" phase is complete, one chunk behind its own reading so that it rarely has to wait.
    // The loads then cost the sweep no issue slots, no registers and no long-latency stalls: what is
    // left are shared-memory reads.  The ragged end (fewer items than a chunk) goes through plain loads.
    // Returns false when a wait ran out of time (the counts are then incomplete).  The mbarriers at the
    // head of the ring must have been initialised (bulk_init) and a barrier of the role passed since.
    static __device__ __forceinline__ void bulk_init(unsigned char* ring, int warps) {
        unsigned long long* full = reinterpret_cast<unsigned long long*>(ring);
        for (int b = 0; b < kBulkBufs; ++b) { mbar_init(full + b, 1u); mbar_init(full + kBulkBufs + b, (uint32_t)warps); }
        fence_mbar_init();
    }
    static __device__ __forceinline__ void bulk_done(unsigned char* ring) {
        unsigned long long* full = reinterpret_cast<unsigned long long*>(ring);
        for (int b = 0; b < 2 * kBulkBufs; ++b) mbar_inval(full + b);
    }
    // Kept inline: out of line (`__noinline__`) the role's arguments are re-read from memory for every value
    // and the pairs that use this path take 35 and 49 us instead of 27 and 35.
    template <int T, int SHIFT, bool POW2>
    static __device__ __forceinline__ bool sweep_bulk(const Args& a, const RoleCtx& ctx, uint32_t sbase, unsigned char* ring) {
        constexpr int U = kBulkU, NB = kBulkBufs;
        constexpr uint32_t CI = (uint32_t)T * U;              // 16-byte items per chunk
        constexpr unsigned long long kTimeoutNs = 2000000000ull;
        unsigned long long* full = reinterpret_cast<unsigned long long*>(ring);
        unsigned long long* empty = full + NB;
        const float4* tiles = reinterpret_cast<const float4*>(ring + 64);
        const int last = a.nbins - 1;
        const uint32_t n4 = (uint32_t)(a.n >> 2);
        const uint32_t nchunks = n4 / CI, blk = (uint32_t)ctx.block, nblk = (uint32_t)ctx.nblocks;
        const uint32_t mine = blk < nchunks ? (nchunks - blk + nblk - 1u) / nblk : 0u;
        const int lane = ctx.tid & 31;
        auto count4 = [&](const float4& v) {
            count<SHIFT, POW2>(a, v.x, sbase, last); count<SHIFT, POW2>(a, v.y, sbase, last);
            count<SHIFT, POW2>(a, v.z, sbase, last); count<SHIFT, POW2>(a, v.w, sbase, last);
        };
        auto issue = [&](uint32_t g) {                       // chunk blk + g * nblk as fill number g
            const uint32_t slot = g % NB;
            mbar_expect_tx(full + slot, CI * 16u);
            bulk_load(const_cast<float4*>(tiles) + (size_t)slot * CI, a.x + 4ull * CI * (blk + g * nblk), CI * 16u, full + slot);
        };
        if (ctx.tid == 0)
            for (uint32_t g = 0; g < (uint32_t)NB && g < mine; ++g) issue(g);
        bool ok = true;
        for (uint32_t g = 0; g < mine; ++g) {
            const uint32_t slot = g % NB, par = (g / NB) & 1u;
            // a wait that ran out of time ends the sweep for the whole warp (the other warps follow within their own limit)
            ok = __all_sync(0xffffffffu, ok && mbar_wait(full + slot, par, kTimeoutNs));
            if (!ok) break;
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = tiles[(size_t)slot * CI + (uint32_t)ctx.tid + (uint32_t)u * T];
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + slot);
            // refill the buffer of the chunk before this one: its readers have had a whole chunk's time
            if (ctx.tid == 0 && g >= 1u && g - 1u + NB < mine) {
                if (mbar_wait(empty + (g - 1u) % NB, ((g - 1u) / NB) & 1u, kTimeoutNs)) issue(g - 1u + NB);
                else ok = false;          // nothing more is issued; every warp's next wait runs out and ends its sweep
            }
#pragma unroll
            for (int u = 0; u < U; ++u) count4(v[u]);
        }
        if (blk == nblk - 1u)      // fewer items than a chunk
            for (uint32_t i = nchunks * CI + (uint32_t)ctx.tid; i < n4; i += T) count4(ldg_stream4(a.x + 4ull * i));
        if (ctx.block == 0)        // n % 4 values
            for (long long j = 4ll * n4 + ctx.tid; j < a.n; j += T) count<SHIFT, POW2>(a, __ldg(a.x + j), sbase, last);
        return ok;
    }

    // General sweep: 64-bit indices, any histogram placement.  SHARED selects the address space at
    // compile time: the shared-memory histogram is updated with `red.shared` (no return value, no
    // generic-address atomics).  Used for 2^31 or more items and for the global-atomics layout.
    template <int T, bool SHARED>
    static __device__ __forceinline__ void sweep(const Args& a, const RoleCtx& ctx, unsigned* hist) {
        const long long n4 = a.n >> 2;
        // shared address of bin b is sbase + 4 * (b << shift): shift = 5 spreads a bin over 32 lanes
        const int shift = (SHARED && a.lane_private) ? 5 : 0;
        const uint32_t sbase = SHARED ? (uint32_t)__cvta_generic_to_shared(hist) + (a.lane_private ? 4u * (ctx.tid & 31) : 0u)
                                      : 0u;
        constexpr int U = 4;
        const long long stride = (long long)ctx.nblocks * T;
        long long i = (long long)ctx.block * T + ctx.tid;
        float4 nxt[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (i + u * stride < n4) nxt[u] = ldg_stream4(a.x + 4 * (i + u * stride));
        for (; i < n4; i += U * stride) {
            float4 v[U];
            bool ok[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                ok[u] = i + u * stride < n4;
                v[u] = nxt[u];
            }
            const long long j = i + U * stride;
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (j + u * stride < n4) nxt[u] = ldg_stream4(a.x + 4 * (j + u * stride));
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (!ok[u]) continue;
                const int b0 = bin_of(a, v[u].x), b1 = bin_of(a, v[u].y), b2 = bin_of(a, v[u].z), b3 = bin_of(a, v[u].w);
                if (SHARED) {
                    if (b0 >= 0) red_shared_inc(sbase + (4u * b0 << shift));
                    if (b1 >= 0) red_shared_inc(sbase + (4u * b1 << shift));
                    if (b2 >= 0) red_shared_inc(sbase + (4u * b2 << shift));
                    if (b3 >= 0) red_shared_inc(sbase + (4u * b3 << shift));
                } else {
                    if (b0 >= 0) atomicAdd(hist + b0, 1u);
                    if (b1 >= 0) atomicAdd(hist + b1, 1u);
                    if (b2 >= 0) atomicAdd(hist + b2, 1u);
                    if (b3 >= 0) atomicAdd(hist + b3, 1u);
                }
            }
        }
        if (ctx.block == 0) {   // ragged tail (n % 4 values)
            for (long long i = 4 * n4 + ctx.tid; i < a.n; i += T) {
                const int b = bin_of(a, __ldg(a.x + i));
                if (b >= 0) {
                    if (SHARED) red_shared_inc(sbase + (4u * b << shift));
                    else atomicAdd(hist + b, 1u);
                }
            }
        }
    }

    template <int T, int SHIFT>
    static __device__ __forceinline__ void sweep_fast_pick(const Args& a, const RoleCtx& ctx, uint32_t sbase) {
        if (a.range_pow2) sweep_fast<T, SHIFT, true>(a, ctx, sbase);
        else sweep_fast<T, SHIFT, false>(a, ctx, sbase);
    }

    // The counts are cleared by a small kernel launched just before this one, and this kernel is
    // launched as its programmatic dependent: it starts while the clearing kernel runs and only
    // waits for it here, before its first access to the counts.  Launched without that attribute
    // the instruction returns at once (stream order has already done the waiting).
    static __device__ __forceinline__ void wait_for_cleared_counts() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        if (a.copies == 0) {
            wait_for_cleared_counts();
            sweep<T, false>(a, ctx, a.counts);
            return;
        }
        unsigned* sh = reinterpret_cast<unsigned*>(ctx.smem);
        const int words = (a.lane_private ? 32 : a.copies) * a.nbins;
        for (int i = ctx.tid; i < words; i += T) sh[i] = 0u;
        unsigned char* ring = ctx.smem + words * (int)sizeof(unsigned);      // bulk-load sweep only
        if (a.bulk && ctx.tid == 0) bulk_init(ring, T / 32);
        role_sync<BAR, T>();
        unsigned* hist = a.lane_private ? sh : sh + ((ctx.tid >> 5) % a.copies) * a.nbins;
        bool ok = true;
        if (a.fast) {
            const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(hist) + (a.lane_private ? 4u * (ctx.tid & 31) : 0u);
            if (a.bulk) {          // only with the [bin][lane] histogram (plan)
                if (a.range_pow2) ok = sweep_bulk<T, 7, true>(a, ctx, sbase, ring);
                else ok = sweep_bulk<T, 7, false>(a, ctx, sbase, ring);
            } else if (a.lane_private) sweep_fast_pick<T, 7>(a, ctx, sbase);
            else sweep_fast_pick<T, 2>(a, ctx, sbase);
        } else {
            sweep<T, true>(a, ctx, hist);
        }
        role_sync<BAR, T>();
        if (a.bulk && ctx.tid == 0) bulk_done(ring);     // nobody waits any more: the memory may be reused
        wait_for_cleared_counts();
        // a wait of the bulk-load sweep that ran out of time: the counts are incomplete; bin 0 says so
        if (!ok) atomicMax(a.counts, 0xffffffffu);
        for (int b = ctx.tid; b < a.nbins; b += T) {
            unsigned s = 0;
            if (a.lane_private) {
                // rotate the start so that the threads of a warp read different banks
                for (int l = 0; l < 32; ++l) s += sh[b * 32 + ((l + ctx.tid) & 31)];
            } else {
                for (int c = 0; c < a.copies; ++c) s += sh[c * a.nbins + b];
            }
            if (s) atomicAdd(a.counts + b, s);
        }
    }
};

// =============================================================================
// batch_norm_collect_statistics: per-channel mean and 1/sqrt(biased var + eps)
// =============================================================================
// Work unit = (channel, slice): the channel's N*HW values, taken in (n, hw)
// order, are cut into S equal slices and the whole role (T threads) reduces
// one slice: each thread accumulates shifted sums over its 16-byte loads and
// turns them into Welford moments (count, mean, M2); a warp folds them with a
// shuffle tree of Chan merges; the per-warp moments meet in shared memory
// behind the role's named barrier and warp 0 folds them.  S = 1 (a whole
// channel per unit) whenever there are at least about as many channels as
// blocks; otherwise the slice moments go to scratch and the block that takes
// the last ticket of a channel folds all S of them in slice order, so the
// result does not depend on arrival order.
// ---- cross-GPU exchange of the per-channel moments over peer memory -------------------------
// Every rank owns one exchange buffer and holds peer pointers to all of them.  The warp that
// has finished channel c sends the channel's (n, sum, sum of squares) to EVERY rank's buffer
// (row [slot][its rank][c]) as six 8-byte words (three 16-byte stores), each word carrying 4 payload
// bytes and the 4-byte epoch of this use of the slot.  An aligned 8-byte store arrives whole, so a word whose epoch
// matches holds valid payload: no fence, no counter, no atomic.  The same warp then polls the
// rows of all ranks for channel c in its OWN buffer (one lane per rank, bounded in time) and
// folds them in rank order, so all ranks compute the same bits.  Slots rotate and epochs only
// grow; a rank can run at most one call ahead of the slowest one (its next kernel cannot end
// before every rank has delivered), so a slot is never overwritten before it has been read.
// Slot and epoch of a call come from a call counter kept in the buffer's header ON THE DEVICE.
// The header holds one 64-bit word: the number of completed exchange launches in its upper half, the
// number of blocks of the running launch that have checked in in its lower half.  One thread per
// block adds 1 to it when the block starts: the value it gets back carries the call count (the same
// for every block of the launch, since the count only moves once all of them have checked in) and
// the block's ticket.  The block that drew the last ticket moves the word on to the next call
// (count + 1, tickets back to 0) before it ends.  The add is issued at the start of the block and
// its result is first needed when the block sends, so it costs no wait.  The host passes nothing
// that changes from call to call: a launch replayed from a CUDA graph moves on to the next slot
// and epoch like a direct launch does, and a launch that failed on the host leaves the counter
// where the other ranks' counters are.
constexpr int kXchgMaxRanks = 8;
constexpr int kXchgSlots = 4;
constexpr int kXchgRowWords = 6;      // 48 bytes: five words with payload, the sixth carries the tag only
struct XchgLayout {                   // header of an exchange buffer
    unsigned status;                  // set to 1 when a wait ran out of time
    unsigned pad0;
    unsigned long long ticket;        // (completed launches << 32) | blocks of the running launch that checked in
    unsigned pad[60];
    // followed by unsigned long long rows[kXchgSlots][kXchgMaxRanks][C][kXchgRowWords]
};
struct BnXchg {
    int world;                // 0: exchange disabled
    int rank;
    unsigned long long timeout_ns;
    unsigned char* peer[kXchgMaxRanks];   // exchange buffers of all ranks (peer[rank] is the local one)
};
struct XchgUse {              // which slot a launch writes, and the tag its words carry
    unsigned slot;
    unsigned epoch;           // use count of the slot, never 0 (the buffer starts zeroed)
};
// one thread per block, when the block starts; returns the word as it was before this block's ticket
__device__ __forceinline__ unsigned long long xchg_check_in(const BnXchg& x) {
    return atomicAdd(&reinterpret_cast<XchgLayout*>(x.peer[x.rank])->ticket, 1ull);
}
__device__ __forceinline__ XchgUse xchg_use(unsigned long long word) {
    const unsigned n = (unsigned)(word >> 32);
    return XchgUse{n % kXchgSlots, n / kXchgSlots + 1u};
}
// the same thread, after the block's last exchange access: the block with the last ticket moves
// the word on to the next call
__device__ __forceinline__ void xchg_check_out(const BnXchg& x, unsigned long long word, unsigned nblocks) {
    if ((unsigned)word == nblocks - 1u)
        atomicAdd(&reinterpret_cast<XchgLayout*>(x.peer[x.rank])->ticket, (1ull << 32) - (unsigned long long)nblocks);
}
// 16-byte accesses to an exchange row (this GPU's or a peer's), never cached in L1
__device__ __forceinline__ void st_peer_2x64(unsigned long long* p, unsigned long long a, unsigned long long b) {
    asm volatile("st.volatile.global.v2.u64 [%0], {%1,%2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_peer_2x64(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
    asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ volatile unsigned long long* xchg_row(unsigned char* base, int C, unsigned slot, int src,
                                                                 int c) {
    unsigned long long* rows = reinterpret_cast<unsigned long long*>(base + sizeof(XchgLayout));
    return rows + (((size_t)slot * kXchgMaxRanks + src) * C + c) * kXchgRowWords;
}

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
    int S;                // slices per channel (<= kBnMaxSlices)
    unsigned chunk;       // vector (or scalar) items per slice
    unsigned per_channel; // vector (or scalar) items per channel = N * HW / (vec ? 4 : 1)
    unsigned per_img;     // vector (or scalar) items per image
    FastDiv div_img;      // by per_img
    int vec;              // HW % 4 == 0: 16-byte loads
    size_t ws_bytes;      // size of the caller's scratch buffer (host-side check only)
    void* ws;             // the caller's scratch buffer
    BnXchg xchg;          // world == 0 unless launched through an exchange entry point
    int bulk_ok;          // the shape allows the bulk-load path (16-byte rows of 1 to 24 KB)
    int bulk;             // 1: channels are brought into shared memory by bulk (TMA) copies (run_bulk)
    unsigned bulk_rows;   // image rows of one channel per shared-memory buffer on that path
    unsigned bulk_bufs;   // buffers in the ring (2 .. kBnBulkMaxBufs)
};

constexpr int kBnMaxSlices = 256;
constexpr int kBnBulkMaxBufs = 4;
inline size_t bn_ticket_bytes(int C) { return (((size_t)C * sizeof(unsigned)) + 255) & ~(size_t)255; }
inline size_t bn_workspace_bytes(int C) {
    return bn_ticket_bytes(C) + (size_t)C * kBnMaxSlices * 3 * sizeof(float);
}

struct Moments { float n, mean, m2; };

__device__ __forceinline__ Moments chan_merge(Moments a, Moments b) {
    const float n = a.n + b.n;
    if (n == 0.f) return a;
    const float delta = b.mean - a.mean;
    const float fb = __fdividef(b.n, n);
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
    // two parity buffers of per-warp moments; on the bulk-load path two mbarriers and two tile buffers behind them
    static __host__ __device__ __forceinline__ int moments_bytes(int T) { return (2 * 3 * (T / 32) * (int)sizeof(float) + 15) & ~15; }
    static int smem_bytes(const Args& a, int T) {
        return moments_bytes(T) + (a.bulk ? kBnBulkMaxBufs * 8 + (int)a.bulk_bufs * (int)a.bulk_rows * a.HW * (int)sizeof(float) : 0);
    }

    // One channel per unit when the channels alone give every block work;
    // otherwise S slices per channel, but never fewer than two loads per thread in a slice.
    static int plan(Args& a, int T, int grid) {
        const long long per_channel = (long long)a.N * a.HW / (a.vec ? 4 : 1);
        long long s_small = per_channel / (2LL * T);
        if (s_small < 1) s_small = 1;
        if (s_small > kBnMaxSlices) s_small = kBnMaxSlices;
        long long s_want = (2LL * a.C >= grid) ? 1 : (grid + a.C - 1) / a.C;
        const long long S = s_want < s_small ? s_want : s_small;
        a.per_channel = (unsigned)per_channel;
        a.per_img = (unsigned)(a.vec ? a.HW / 4 : a.HW);
        a.div_img = make_fastdiv(a.per_img);
        a.chunk = (unsigned)((per_channel + S - 1) / S);
        a.S = (int)((per_channel + a.chunk - 1) / a.chunk);
        if (a.S != 1) a.bulk = 0;      // the bulk-load path works on whole channels
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

    // Exchange form of finish(), in two halves, each run by all 32 lanes of one warp.
    // xchg_send: the channel's local moments are in lane 0; lane r stores them into rank r's buffer.
    static __device__ __forceinline__ void xchg_send(const Args& a, XchgUse use, int c, Moments m, int lane) {
        const BnXchg& x = a.xchg;
        const float mean_l = __shfl_sync(0xffffffffu, m.mean, 0);
        const float m2_l = __shfl_sync(0xffffffffu, m.m2, 0);
        const double n = (double)a.N * (double)a.HW, mu = (double)mean_l;
        const unsigned long long s1 = (unsigned long long)__double_as_longlong(n * mu);
        const unsigned long long s2 = (unsigned long long)__double_as_longlong((double)m2_l + n * mu * mu);
        const unsigned long long tag = (unsigned long long)use.epoch << 32;
        if (lane < x.world) {          // lane r sends to rank r: the stores of all ranks go out side by side
            // three 16-byte stores instead of six 8-byte ones (fewer packets on the link); each 8-byte
            // half still carries its own tag, so it does not matter whether a store arrives in one piece
            unsigned long long* row = const_cast<unsigned long long*>(xchg_row(x.peer[lane], a.C, use.slot, x.rank, c));
            st_peer_2x64(row, tag | (s1 & 0xffffffffull), tag | (s1 >> 32));
            st_peer_2x64(row + 2, tag | (s2 & 0xffffffffull), tag | (s2 >> 32));
            st_peer_2x64(row + 4, tag | (unsigned long long)(unsigned)((long long)a.N * a.HW), tag);
        }
    }

    // xchg_collect: lane r waits (bounded) for rank r's row of channel c in the local buffer; the
    // rows are folded in rank order and lane 0 writes the channel's global statistics.
    static __device__ __forceinline__ void xchg_collect(const Args& a, XchgUse use, int c, int lane) {
        const BnXchg& x = a.xchg;
        double rs1 = 0.0, rs2 = 0.0, rn = 0.0;
        bool ok = true;
        if (lane < x.world) {
            const unsigned long long* row = const_cast<const unsigned long long*>(xchg_row(x.peer[x.rank], a.C, use.slot, lane, c));
            unsigned long long t0 = 0, t1, w[6];
            for (bool first = true;; first = false) {
                ld_peer_2x64(row, w[0], w[1]);
                ld_peer_2x64(row + 2, w[2], w[3]);
                ld_peer_2x64(row + 4, w[4], w[5]);
                bool all = true;
#pragma unroll
                for (int k = 0; k < 6; ++k) all &= (unsigned)(w[k] >> 32) == use.epoch;
                if (all) break;
                // the clock is only read once a poll has failed (the row is usually there already)
                if (first) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
                __nanosleep(64);
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                if (t1 - t0 > x.timeout_ns) { ok = false; break; }
            }
            rs1 = __longlong_as_double((long long)((w[0] & 0xffffffffull) | (w[1] << 32)));
            rs2 = __longlong_as_double((long long)((w[2] & 0xffffffffull) | (w[3] << 32)));
            rn = (double)(unsigned)(w[4] & 0xffffffffull);
        }
        ok = __all_sync(0xffffffffu, ok);
        double tn = 0.0, t1s = 0.0, t2s = 0.0;
        for (int r = 0; r < x.world; ++r) {       // rank order: identical bits on every rank
            tn += __shfl_sync(0xffffffffu, rn, r);
            t1s += __shfl_sync(0xffffffffu, rs1, r);
            t2s += __shfl_sync(0xffffffffu, rs2, r);
        }
        if (lane == 0) {
            if (!ok) atomicExch(&reinterpret_cast<XchgLayout*>(x.peer[x.rank])->status, 1u);   // results invalid
            const double mean = t1s / tn;
            double var = t2s / tn - mean * mean;
            if (var < 0.0) var = 0.0;
            a.mean[c] = (float)mean;
            a.invstd[c] = (float)(1.0 / sqrt(var + (double)a.eps));
            if (a.moments) { a.moments[3 * c] = tn; a.moments[3 * c + 1] = t1s; a.moments[3 * c + 2] = t2s; }
        }
    }

    // called by all 32 lanes of warp 0 with the channel's folded moments in lane 0.  DEFER: send
    // now, collect later (collect_deferred), so that the wait for the peers overlaps other work.
    template <bool XCHG, bool DEFER>
    static __device__ __forceinline__ void complete(const Args& a, XchgUse use, int c, Moments m, int lane) {
        if (XCHG) {
            xchg_send(a, use, c, m, lane);
            if (!DEFER) xchg_collect(a, use, c, lane);
        } else if (lane == 0) {
            finish(a, c, m);
        }
    }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        run_impl<T, BAR, false, false>(a, ctx);
    }

    // The second half of run_impl<.., XCHG = true, DEFER = true>: warp 0 collects the channels whose
    // moments this block sent.  Only the one-slice-per-channel plan defers (the block that owns a
    // unit is then the one that sent it); with slices the exchange already happened in run_impl.
    template <int T>
    static __device__ __forceinline__ void collect_deferred(const Args& a, const RoleCtx& ctx, unsigned long long word) {
        if (a.S != 1 || (ctx.tid >> 5) != 0) return;
        const XchgUse use = xchg_use(__shfl_sync(0xffffffffu, word, 0));      // thread 0 holds the block's check-in word
        for (unsigned u = ctx.block; u < (unsigned)a.C; u += ctx.nblocks) xchg_collect(a, use, (int)u, ctx.tid & 31);
    }

    // The end of a unit, entered by all T threads with their shifted sums: per-thread moments, warp
    // fold, the role-wide fold through shared memory behind the role's barrier, then warp 0 finishes
    // the channel (or publishes the slice and, on the last ticket, folds all slices).
    template <int T, int BAR, bool XCHG, bool DEFER>
    static __device__ __forceinline__ void fold_unit(const Args& a, const RoleCtx& ctx, unsigned long long word, int parity,
                                                     unsigned c, unsigned s, float cnt, float sum, float sq, float shift) {
        constexpr int NW = T / 32;
        static_assert(NW <= 32, "one warp folds the per-warp moments");
        float* sh = reinterpret_cast<float*>(ctx.smem);
        const int lane = ctx.tid & 31, warp = ctx.tid >> 5;
        Moments m{0.f, 0.f, 0.f};
        if (cnt > 0.f) {
            const float dm = sum / cnt;
            m = Moments{cnt, shift + dm, fmaxf(sq - sum * dm, 0.f)};
        }
        m = warp_merge(m);
        float* buf = sh + parity * 3 * NW;
        if (lane == 0) { buf[warp] = m.n; buf[NW + warp] = m.mean; buf[2 * NW + warp] = m.m2; }
        role_sync<BAR, T>();
        // The parity buffer keeps warp 0's reads of this unit apart from the next unit's
        // writes; the unit after that is fenced by the next barrier.
        if (warp != 0) return;
        Moments w = (lane < NW) ? Moments{buf[lane], buf[NW + lane], buf[2 * NW + lane]} : Moments{0.f, 0.f, 0.f};
        w = warp_merge(w);
        XchgUse use{0u, 0u};
        if (XCHG) use = xchg_use(__shfl_sync(0xffffffffu, word, 0));     // warp 0: thread 0 holds the word
        if (a.S == 1) {
            complete<XCHG, DEFER>(a, use, (int)c, w, lane);
            return;
        }
        // publish this slice; the block that takes the last ticket folds all slices
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
            for (int i = lane; i < a.S; i += 32) {      // fixed order: lane, lane+32, ...
                const float* p = a.partial + ((size_t)c * a.S + i) * 3;
                q = chan_merge(q, Moments{__ldcg(p), __ldcg(p + 1), __ldcg(p + 2)});
            }
            q = warp_merge(q);
            if (lane == 0) a.tickets[c] = 0u;     // ready for the next call
            complete<XCHG, false>(a, use, (int)c, q, lane);
        }
    }

    // Bulk-load path (one slice per channel, rows of HW floats that are 16-byte multiples): the
    // channel's N rows come into shared memory through bulk (TMA) copies, `bulk_rows` rows per
    // buffer, a ring of `bulk_bufs` buffers, each with an mbarrier that counts the bytes landed.
    // One thread issues the copies, so the loads in flight cost no registers and do not depend on
    // how many threads the role has; all T threads then sum a buffer from shared memory while the
    // others are on their way.  A buffer is refilled after the role's barrier that follows its
    // last reader.
    template <int T, int BAR, bool XCHG, bool DEFER>
    static __device__ __forceinline__ void run_bulk(const Args& a, const RoleCtx& ctx, unsigned long long word) {
        unsigned char* base = ctx.smem + moments_bytes(T);
        unsigned long long* full = reinterpret_cast<unsigned long long*>(base);      // one barrier per buffer
        unsigned char* tiles = base + kBnBulkMaxBufs * 8;
        const unsigned row_bytes = (unsigned)a.HW * (unsigned)sizeof(float), row4 = (unsigned)a.HW >> 2;
        const unsigned R = a.bulk_rows, rows = (unsigned)a.N, NB = a.bulk_bufs;
        const unsigned buf_bytes = R * row_bytes;
        const unsigned nfill = (rows + R - 1) / R;         // buffer fills per channel
        const size_t img_stride = (size_t)a.C * a.HW;
        constexpr unsigned long long kTimeoutNs = 2000000000ull;
        if (ctx.tid == 0) {
            for (unsigned b = 0; b < NB; ++b) mbar_init(full + b, 1u);
            fence_mbar_init();
        }
        role_sync<BAR, T>();
        // The fills of all of this block's channels form one sequence: fill g belongs to channel
        // block + (g / nfill) * nblocks and holds its rows [(g % nfill) * R, ...); it goes to buffer
        // g % NB.  NB fills are in flight ahead of the reader, across channel boundaries too, so the
        // second channel of a block does not start with an empty ring.
        const unsigned blk = (unsigned)ctx.block, nblk = (unsigned)ctx.nblocks;
        const unsigned nunits = blk < (unsigned)a.C ? ((unsigned)a.C - blk + nblk - 1u) / nblk : 0u;
        const unsigned total = nunits * nfill;
        auto issue = [&](unsigned g) {
            const unsigned u = blk + (g / nfill) * nblk, k = g % nfill;
            const unsigned n = min(R, rows - k * R), slot = g % NB;
            const float* src = a.x + (size_t)u * a.HW + (size_t)(k * R) * img_stride;
            mbar_expect_tx(full + slot, n * row_bytes);
            unsigned char* dst = tiles + (size_t)slot * buf_bytes;
            for (unsigned r = 0; r < n; ++r)
                bulk_load(dst + (size_t)r * row_bytes, src + (size_t)r * img_stride, row_bytes, full + slot);
        };
        if (ctx.tid == 0)
            for (unsigned g = 0; g < NB && g < total; ++g) issue(g);
        int parity = 0;
        bool ok = true;
        float cnt = 0.f, sum = 0.f, sq = 0.f, shift = 0.f;
        for (unsigned g = 0; g < total; ++g) {
            const unsigned slot = g % NB, k = g % nfill;
            ok &= mbar_wait(full + slot, (g / NB) & 1u, kTimeoutNs);
            const unsigned items = min(R, rows - k * R) * row4;
            const float4* t = reinterpret_cast<const float4*>(tiles + (size_t)slot * buf_bytes);
            for (unsigned i = ctx.tid; i < items; i += T) {
                const float4 v = t[i];
                if (cnt == 0.f) shift = v.x;
                const float d0 = v.x - shift, d1 = v.y - shift, d2 = v.z - shift, d3 = v.w - shift;
                sum += (d0 + d1) + (d2 + d3);
                sq = fmaf(d0, d0, fmaf(d1, d1, fmaf(d2, d2, fmaf(d3, d3, sq))));
                cnt += 4.f;
            }
            if (g + NB < total) {          // the buffer is refilled once every thread has read it
                role_sync<BAR, T>();
                if (ctx.tid == 0) issue(g + NB);
            }
            if (k + 1u == nfill) {         // the channel is complete
                // a wait that ran out of time: the statistics of this channel come out as NaN
                if (!__all_sync(0xffffffffu, ok)) sum = __int_as_float(0x7fc00000);
                fold_unit<T, BAR, XCHG, DEFER>(a, ctx, word, parity, blk + (g / nfill) * nblk, 0u, cnt, sum, sq, shift);
                parity ^= 1;
                cnt = 0.f; sum = 0.f; sq = 0.f; shift = 0.f;
            }
        }
        // thread 0 is past the last fold's barrier, so nobody waits on the barriers any more: give
        // their shared memory back (a vertically fused partner reuses it)
        if (ctx.tid == 0)
            for (unsigned b = 0; b < NB; ++b) mbar_inval(full + b);
    }

    // `word`: the block's check-in word (XCHG only; held by thread 0, see xchg_check_in)
    template <int T, int BAR, bool XCHG, bool DEFER>
    static __device__ __forceinline__ void run_impl(const Args& a, const RoleCtx& ctx, unsigned long long word = 0ull) {
        if (a.bulk) {
            run_bulk<T, BAR, XCHG, DEFER>(a, ctx, word);
            return;
        }
        constexpr int UNROLL = 4;      // 16-byte loads in flight per thread and trip (8 was measured: 0.4 us off the standalone kernel, spills in the 40-register pair shapes)
        const unsigned units = (unsigned)a.C * (unsigned)a.S;
        int parity = 0;
        for (unsigned u = ctx.block; u < units; u += ctx.nblocks, parity ^= 1) {
            const unsigned c = u / a.S, s = u - c * a.S;
            const unsigned k0 = s * a.chunk;
            const unsigned k1 = min(k0 + a.chunk, a.per_channel);
            const float* xc = a.x + (size_t)c * a.HW;
            const size_t img_stride = (size_t)a.C * a.HW;
            // ---- per-thread sums of (x - shift) and (x - shift)^2; shift = the thread's first value
            float cnt = 0.f, sum = 0.f, sq = 0.f, shift = 0.f;
            for (unsigned k = k0 + ctx.tid; k < k1; k += T * UNROLL) {
                if (a.vec) {
                    float4 v[UNROLL];
                    bool ok[UNROLL];
#pragma unroll
                    for (int j = 0; j < UNROLL; ++j) {
                        const unsigned kk = k + T * j;
                        ok[j] = kk < k1;
                        if (ok[j]) {
                            unsigned off;
                            const unsigned n = fast_divmod(kk, a.div_img, off);
                            v[j] = ldg_stream4(xc + n * img_stride + 4 * off);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < UNROLL; ++j) {
                        if (!ok[j]) continue;
                        if (cnt == 0.f) shift = v[j].x;
                        const float d0 = v[j].x - shift, d1 = v[j].y - shift, d2 = v[j].z - shift, d3 = v[j].w - shift;
                        sum += (d0 + d1) + (d2 + d3);
                        sq = fmaf(d0, d0, fmaf(d1, d1, fmaf(d2, d2, fmaf(d3, d3, sq))));
                        cnt += 4.f;
                    }
                } else {
                    float v[UNROLL];
                    bool ok[UNROLL];
#pragma unroll
                    for (int j = 0; j < UNROLL; ++j) {
                        const unsigned kk = k + T * j;
                        ok[j] = kk < k1;
                        if (ok[j]) {
                            unsigned off;
                            const unsigned n = fast_divmod(kk, a.div_img, off);
                            v[j] = __ldg(xc + n * img_stride + off);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < UNROLL; ++j) {
                        if (!ok[j]) continue;
                        if (cnt == 0.f) shift = v[j];
                        const float d = v[j] - shift;
                        sum += d;
                        sq = fmaf(d, d, sq);
                        cnt += 1.f;
                    }
                }
            }
            fold_unit<T, BAR, XCHG, DEFER>(a, ctx, word, parity, c, s, cnt, sum, sq, shift);
        }
    }
};

// The same role with the cross-GPU exchange switched on (fused compute + collective).
struct BnStatsXchgRole : BnStatsRole {
    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        unsigned long long word = 0ull;
        if (ctx.tid == 0) word = xchg_check_in(a.xchg);
        BnStatsRole::run_impl<T, BAR, true, false>(a, ctx, word);
        if (ctx.tid == 0) xchg_check_out(a.xchg, word, (unsigned)ctx.nblocks);   // warp 0 did this block's exchange
    }
    // The two halves for a kernel that puts other work between sending and collecting; run_early
    // returns the block's check-in word (in thread 0), which run_late takes back.
    template <int T, int BAR>
    static __device__ __forceinline__ unsigned long long run_early(const Args& a, const RoleCtx& ctx) {
        unsigned long long word = 0ull;
        if (ctx.tid == 0) word = xchg_check_in(a.xchg);
        BnStatsRole::run_impl<T, BAR, true, true>(a, ctx, word);
        return word;
    }
    template <int T, int BAR>
    static __device__ __forceinline__ void run_late(const Args& a, const RoleCtx& ctx, unsigned long long word) {
        BnStatsRole::collect_deferred<T>(a, ctx, word);
        if (ctx.tid == 0) xchg_check_out(a.xchg, word, (unsigned)ctx.nblocks);
    }
};

}  // namespace hfuse
