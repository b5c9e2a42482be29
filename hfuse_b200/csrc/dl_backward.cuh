// Role bodies of the two backward kernels the reference lists next to the forward ones
// (configs/ml_kernels.yaml:46-63): max_pool_backward_nchw and batch_norm_backward_kernel, the
// only kernel there that declares barriers.  Written as roles like the forward kernels, so
// they run standalone or side by side in a fused block.
#pragma once
#include "common.cuh"

namespace hfuse {

// =============================================================================
// max_pool2d backward: grad_in[n,c,h,w] = sum of grad_out over the outputs whose
// recorded index is h*W+w.  Gather form (one input element per item, the candidate
// outputs scanned in (ph, pw) order): no atomics, deterministic.
// =============================================================================
struct MaxPoolBwdArgs {
    const float* grad_out;
    const long long* idx;
    float* grad_in;
    int N, C, H, W, pH, pW;
    int kh, kw, sh, sw, ph, pw, dh, dw;
    FastDiv div_w, div_h;
};

struct MaxPoolBwdRole {
    using Args = MaxPoolBwdArgs;
    static int smem_bytes(const Args&, int) { return 0; }
    static int plan(Args&, int, int) { return 0; }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        const unsigned total = (unsigned)a.N * a.C * a.H * a.W;            // host guarantees < 2^31
        const int ext_h = (a.kh - 1) * a.dh + 1, ext_w = (a.kw - 1) * a.dw + 1;
        for (unsigned it = (unsigned)ctx.block * T + ctx.tid; it < total; it += (unsigned)ctx.nblocks * T) {
            unsigned w, h;
            const unsigned r = fast_divmod(it, a.div_w, w);
            const unsigned plane = fast_divmod(r, a.div_h, h);
            // outputs whose window can contain (h, w)
            const int hp = (int)h + a.ph, wp = (int)w + a.pw;
            const int ph0 = hp < ext_h ? 0 : (hp - ext_h) / a.sh + 1;
            const int pw0 = wp < ext_w ? 0 : (wp - ext_w) / a.sw + 1;
            const int ph1 = min(hp / a.sh + 1, a.pH), pw1 = min(wp / a.sw + 1, a.pW);
            const long long me = (long long)h * a.W + w;
            const size_t obase = (size_t)plane * a.pH * a.pW;
            float g = 0.f;
            for (int p = ph0; p < ph1; ++p)
                for (int q = pw0; q < pw1; ++q) {
                    const size_t o = obase + (size_t)p * a.pW + q;
                    if (__ldg(a.idx + o) == me) g += __ldg(a.grad_out + o);
                }
            stg_stream1(a.grad_in + it, g);
        }
    }
};

// =============================================================================
// batch_norm backward (training mode):
//   sum_dy = sum(dy), dot = sum(dy * (x - mean))                 per channel
//   grad_bias = sum_dy, grad_weight = dot * invstd
//   grad_in = (dy - sum_dy/M - (x - mean) * invstd^2 * dot/M) * invstd * weight
// One channel per unit and role: pass 1 reduces the two sums (per-thread partials over
// 16-byte loads, warp shuffles, per-warp partials in shared memory behind the role's named
// barrier), pass 2 re-reads the channel (it is still in L2) and writes grad_in.
// =============================================================================
struct BnBwdArgs {
    const float* x;         // [N][C][HW]
    const float* dy;        // [N][C][HW]
    const float* weight;    // [C] or null (= 1)
    const float* mean;      // [C] saved mean
    const float* invstd;    // [C] saved 1/sqrt(var + eps)
    float* dx;              // [N][C][HW] or null
    float* grad_weight;     // [C] or null
    float* grad_bias;       // [C] or null
    int N, C, HW;
    float inv_m;            // 1 / (N*HW)
    unsigned per_channel, per_img;
    FastDiv div_img;
    int vec;                // HW % 4 == 0
};

struct BnBwdRole {
    using Args = BnBwdArgs;
    static int smem_bytes(const Args&, int T) { return 2 * 2 * (T / 32) * (int)sizeof(float); }
    static int plan(Args&, int, int) { return 0; }

    template <int T, int BAR>
    static __device__ __forceinline__ void run(const Args& a, const RoleCtx& ctx) {
        constexpr int NW = T / 32;
        float* sh = reinterpret_cast<float*>(ctx.smem);
        const int lane = ctx.tid & 31, warp = ctx.tid >> 5;
        const size_t img_stride = (size_t)a.C * a.HW;
        int parity = 0;
        for (int c = ctx.block; c < a.C; c += ctx.nblocks, parity ^= 1) {
            const float mu = __ldg(a.mean + c), is = __ldg(a.invstd + c);
            const float* xc = a.x + (size_t)c * a.HW;
            const float* dc = a.dy + (size_t)c * a.HW;
            // ---- pass 1: sum(dy) and sum(dy * (x - mean))
            float s = 0.f, d = 0.f;
            for (unsigned k = ctx.tid; k < a.per_channel; k += T) {
                unsigned off;
                const unsigned n = fast_divmod(k, a.div_img, off);
                if (a.vec) {
                    const float4 xv = __ldg(reinterpret_cast<const float4*>(xc + n * img_stride) + off);
                    const float4 gv = __ldg(reinterpret_cast<const float4*>(dc + n * img_stride) + off);
                    s += (gv.x + gv.y) + (gv.z + gv.w);
                    d = fmaf(gv.x, xv.x - mu, fmaf(gv.y, xv.y - mu, fmaf(gv.z, xv.z - mu, fmaf(gv.w, xv.w - mu, d))));
                } else {
                    const float xv = __ldg(xc + n * img_stride + off), gv = __ldg(dc + n * img_stride + off);
                    s += gv;
                    d = fmaf(gv, xv - mu, d);
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                s += __shfl_xor_sync(0xffffffffu, s, o);
                d += __shfl_xor_sync(0xffffffffu, d, o);
            }
            float* buf = sh + parity * 2 * NW;
            if (lane == 0) { buf[warp] = s; buf[NW + warp] = d; }
            role_sync<BAR, T>();
            // every warp folds the per-warp partials in the same order: identical sums everywhere
            float ts = 0.f, td = 0.f;
            for (int wv = 0; wv < NW; ++wv) { ts += buf[wv]; td += buf[NW + wv]; }
            if (ctx.tid == 0) {
                if (a.grad_bias) a.grad_bias[c] = ts;
                if (a.grad_weight) a.grad_weight[c] = td * is;
            }
            // ---- pass 2: grad_in
            if (a.dx) {
                const float wgt = a.weight ? __ldg(a.weight + c) : 1.f;
                const float k_mean = ts * a.inv_m, k_dot = td * a.inv_m * is * is, scale = is * wgt;
                float* oc = a.dx + (size_t)c * a.HW;
                for (unsigned k = ctx.tid; k < a.per_channel; k += T) {
                    unsigned off;
                    const unsigned n = fast_divmod(k, a.div_img, off);
                    if (a.vec) {
                        const float4 xv = __ldg(reinterpret_cast<const float4*>(xc + n * img_stride) + off);
                        const float4 gv = __ldg(reinterpret_cast<const float4*>(dc + n * img_stride) + off);
                        float4 o;
                        o.x = (gv.x - k_mean - (xv.x - mu) * k_dot) * scale;
                        o.y = (gv.y - k_mean - (xv.y - mu) * k_dot) * scale;
                        o.z = (gv.z - k_mean - (xv.z - mu) * k_dot) * scale;
                        o.w = (gv.w - k_mean - (xv.w - mu) * k_dot) * scale;
                        stg_stream4(oc + n * img_stride + 4 * off, o);
                    } else {
                        const float xv = __ldg(xc + n * img_stride + off), gv = __ldg(dc + n * img_stride + off);
                        stg_stream1(oc + n * img_stride + off, (gv - k_mean - (xv - mu) * k_dot) * scale);
                    }
                }
            }
            // parity buffers: the next channel's partials go to the other half; the one after is
            // fenced by the next barrier
        }
    }
};

}  // namespace hfuse
