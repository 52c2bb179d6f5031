// Input gradient of the adder convolution on NCHW tensors, with implicit col2im by gathering:
//   gx[n,ci,y,x] = sum over (co,kh,kw) with (y+pad-kh, x+pad-kw) = S*(ho,wo), 0<=ho<Ho, 0<=wo<Wo of
//                  clamp(w[co,ci,kh,kw] - x[n,ci,y,x], -1, 1) * g[n,co,ho,wo]
// This is CONV_BACKWARD's grad_i (adder_cuda/adder.cu:245-246, :266) followed by the col2im that
// autograd applies for F.unfold (adder.py:32-33), folded into one pass: every input pixel sums
// the taps that read it, so nothing is accumulated with atomics and the result is deterministic.
// Taps that fall into the padding are never gathered, which is what col2im's cropping does.
//
// Work decomposition.  A CTA owns TCI = CGI*RC input channels and a tile of TI images x TH input
// rows; a thread owns RC channels x RW input pixels of one row (for stride S > 1 the RW pixels are
// S apart and share one column parity, so the set of valid taps is the same for all of them, and the
// segments of a CTA are ordered by (row, column) phase so that a warp runs one compile-time tap list).  The
// thread keeps its RC*RW input values in registers for the whole kernel.  Output channels are
// streamed in chunks of CKO through a double-buffered shared-memory stage holding the zero-filled
// patch of g [CKO][TI*G_ROWS][PITCH] and the weights [CKO*k*k][TCI+4] (input channel innermost).
//
// FAST variant: clamp(d,-1,1) = 2*sat(d/2 + 1/2) - 1, so with w' = w/2 + 1/2 staged in shared
// memory and x' = -x/2 in registers a term costs one saturating add and one fused multiply-add;
// the correction sum(g) over the same taps is the box sum of the channel-summed g patch, which
// the CTA accumulates on the side.  The exact variant evaluates the formula as written.
#include <type_traits>
#include "common.cuh"
#include "kernels.h"
#include "patch_fill.cuh"
#include <cstdio>

#ifndef GX_PACKED
#define GX_PACKED 1
#endif
namespace adder {

template <bool FAST>
__device__ __forceinline__ float gx_term(float wv, float xv) {
    if (FAST) return __saturatef(wv + xv);                 // wv = w/2+1/2, xv = -x/2
    return fminf(fmaxf(wv - xv, -1.f), 1.f);
}

// Stride-2 taps of one output channel for a thread whose pixels have row phase PH = (y+pad) mod 2 and
// column phase PW = (x+pad) mod 2: only the taps kh = PH, PH+2, ... and kw = PW, PW+2, ... reach an
// output pixel, so the loops are compile-time and nothing is predicated.  row0/col0 locate the tap
// (PH, PW) in the shared-memory patch of g; later taps sit one row / one column before it.
template <int KS, int RW, int RC, bool FAST, int PH, int PW>
__device__ __forceinline__ void gx_taps_stride2(float (&acc)[RC][RW], const float (&xv)[RC][RW], const float* gch,
                                                const float* wch, int row0, int col0, int pitch) {
    constexpr int NKW = (KS - PW + 1) / 2;      // taps of this class along a row: kw = PW, PW + 2, ...
#pragma unroll
    for (int kh = PH; kh < KS; kh += 2) {
        // the NKW taps of a row read runs that overlap in all but one value: load their union once
        const float* gr = gch + (row0 - (kh - PH) / 2) * pitch + col0 - (NKW - 1);
        float gv[RW + NKW - 1];
#pragma unroll
        for (int j = 0; j < RW + NKW - 1; ++j) gv[j] = gr[j];
#pragma unroll
        for (int t = 0; t < NKW; ++t) {
            const int kw = PW + 2 * t;
            const float4 wq = *reinterpret_cast<const float4*>(wch + (kh * KS + kw) * RC);
            const float wv[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
            for (int cc = 0; cc < RC; ++cc)
#pragma unroll
                for (int j = 0; j < RW; ++j)
                    acc[cc][j] = fmaf(gx_term<FAST>(wv[cc], xv[cc][j]), gv[NKW - 1 - t + j], acc[cc][j]);
        }
    }
}

// Weight slab of one output-channel chunk -> shared memory as [col][input-channel quad][tap][4]: a thread's four
// input channels of one tap are one 128-bit load, and the taps of a column sit at compile-time offsets from it
// (no index arithmetic in the tap loops).  WCOL = TCI*KS*KS floats per column.
// 3x3: thread (wgrp, wpr) owns the (input channel, tap) pairs wpr, wpr + WPP, ... and walks the output
// channels wgrp, wgrp + wgroups, ...: the index arithmetic is done once per pair, and consecutive pairs
// are consecutive in global memory.  1x1: the slab is [CKO][TCI]; a flat element loop measured faster.
template <int KS>
__device__ __forceinline__ void gx_stage_weights(const GxArgs& a, float* wt, int coc0, int ci0, int wgrp, int wpr,
                                                 int tid, int nthreads) {
    constexpr int KK = KS * KS;
    if constexpr (KS == 1) {
        for (int e = tid; e < a.CKO * a.TCI; e += nthreads) {
            uint32_t col, cil;
            a.d_tci.divmod(e, col, cil);
            const int co = coc0 + col, ci = ci0 + cil;
            const bool ok = (co < a.g.Co) & (ci < a.g.Ci);
            cp_async4(wt + col * a.WCOL + cil, ok ? a.w + ((size_t)co * a.g.Ci + ci) : a.w, ok);
        }
    } else if (wgrp < a.wgroups) {
        const int ncol = min(a.CKO, a.g.Co - coc0);
        for (int pr = wpr; pr < a.TCI * KK; pr += a.WPP) {
            uint32_t cil, tap;
            a.d_kk.divmod(pr, cil, tap);
            const int ci = ci0 + cil;
            const bool okc = ci < a.g.Ci;
            const float* src = a.w + ((size_t)coc0 * a.g.Ci + (okc ? ci : 0)) * KK + tap;
            float* dst = wt + ((cil >> 2) * KK + tap) * 4 + (cil & 3);
            for (int col = wgrp; col < a.CKO; col += a.wgroups) {
                const bool ok = okc & (col < ncol);
                cp_async4(dst + col * a.WCOL, ok ? src + (size_t)col * a.g.Ci * KK : a.w, ok);
            }
        }
    }
}

// FAST form: every thread turns the weights IT copied into w/2 + 1/2 once its copies have landed
// (same element-to-thread map as gx_stage_weights, so no barrier is needed in between).
template <int KS>
__device__ __forceinline__ void gx_scale_weights(const GxArgs& a, float* wt, int wgrp, int wpr, int tid, int nthreads) {
    constexpr int KK = KS * KS;
    if constexpr (KS == 1) {
        for (int e = tid; e < a.CKO * a.TCI; e += nthreads) {
            uint32_t col, cil;
            a.d_tci.divmod(e, col, cil);
            float* p = wt + col * a.WCOL + cil;
            *p = fmaf(*p, 0.5f, 0.5f);
        }
    } else if (wgrp < a.wgroups) {
        for (int pr = wpr; pr < a.TCI * KK; pr += a.WPP) {
            uint32_t cil, tap;
            a.d_kk.divmod(pr, cil, tap);
            float* p = wt + ((cil >> 2) * KK + tap) * 4 + (cil & 3);
            for (int col = wgrp; col < a.CKO; col += a.wgroups) p[col * a.WCOL] = fmaf(p[col * a.WCOL], 0.5f, 0.5f);
        }
    }
}

// MB = CTAs per SM the register budget is cut for.  A layer whose output channels fit one chunk needs one
// stage of shared memory only, and with 4-pixel segments few enough registers for three CTAs per SM: the
// third CTA's loads and stores then run under the other two's arithmetic (16->16 32x32: 69 -> 66 us).
template <int KS, int S, int RW, int RC, bool FAST, int MB = 2>
__global__ void __launch_bounds__(256, MB) adder_gx_kernel(const GxArgs a) {
    constexpr int KK = KS * KS;
    extern __shared__ __align__(16) float smem[];
    float* const Gs = smem;
    float* const Wt = smem + a.nstages * a.gs_stage;
    float* const G1 = Wt + a.nstages * a.ws_stage;
    float* const Tot = G1 + a.g1_size + threadIdx.x;   // [RC*RW][blockDim.x] running totals, one column per thread

    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    uint32_t tn, th, tw, tnh;
    a.d_tiles_w.divmod(blockIdx.x, tnh, tw);
    a.d_tiles_h.divmod(tnh, tn, th);
    const int n0 = tn * a.TI;
    const int hi0 = th * a.TH;
    const int wq0 = tw * (a.SPRC * RW);           // first class-pixel column of the tile (wi = q*S + pw)
    const int ci0 = blockIdx.y * a.TCI;
    const int pad = a.g.pad;
    const int go_r0 = floor_div(hi0 + pad - (KS - 1), S);
    const int go_c0 = floor_div(wq0 * S + pad - (KS - 1), S);

    uint32_t cig, seg, t2, wsx, pw, ws, img, hr;
    a.d_segs.divmod(tid, cig, seg);
    if (S > 1 && a.class_major) {
        // stride > 1: order the segments by (row offset mod S, column parity) first, so that the lanes of a
        // warp share one set of valid taps instead of diverging over up to S*S different ones
        uint32_t t, hr2, cls;
        a.d_sprc.divmod(seg, t, ws);
        a.d_ths.divmod(t, t2, hr2);
        a.d_ti.divmod(t2, cls, img);       // class slowest: TI*(TH/S)*SPRC consecutive segments share it
        pw = cls % S;
        hr = hr2 * S + cls / S;
        wsx = 0;
    } else {
        a.d_spr.divmod(seg, t2, wsx);
        a.d_sprc.divmod(wsx, pw, ws);
        a.d_th.divmod(t2, img, hr);
    }
    const bool active = (int)cig < a.CGI;
    const int n = n0 + img, hi = hi0 + hr;
    const int q0 = wq0 + ws * RW;                  // class-pixel index of the thread's first pixel
    const int HW = a.g.H * a.g.W;

    constexpr bool PACKED = GX_PACKED && FAST && S == 1 && (RC % 2 == 0);
    float xv[RC][RW];
    float acc[RC][RW];
    uint64_t acc2[RC / 2][RW];
#pragma unroll
    for (int c = 0; c < RC / 2; ++c)
#pragma unroll
        for (int j = 0; j < RW; ++j) acc2[c][j] = 0ull;
#pragma unroll
    for (int c = 0; c < RC; ++c) {
        const int ci = ci0 + cig * RC + c;
        if (S == 1 && RW % 4 == 0 && a.vec_io) {
            // W and the segment start are multiples of 4 and the tensors 16-byte aligned: whole quads
            const bool okr = active && n < a.g.N && ci < a.g.Ci && hi < a.g.H;
            const float* xr = a.x + ((size_t)(n * a.g.Ci + ci) * HW + hi * a.g.W + q0);
#pragma unroll
            for (int j = 0; j < RW; j += 4) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (okr && q0 + j < a.g.W) v = __ldg(reinterpret_cast<const float4*>(xr + j));
                xv[c][j] = FAST ? -0.5f * v.x : v.x;
                xv[c][j + 1] = FAST ? -0.5f * v.y : v.y;
                xv[c][j + 2] = FAST ? -0.5f * v.z : v.z;
                xv[c][j + 3] = FAST ? -0.5f * v.w : v.w;
            }
#pragma unroll
            for (int j = 0; j < RW; ++j) acc[c][j] = 0.f;
            continue;
        }
#pragma unroll
        for (int j = 0; j < RW; ++j) {
            const int wi = (q0 + j) * S + pw;
            const bool ok = active && n < a.g.N && ci < a.g.Ci && hi < a.g.H && wi < a.g.W;
            const float v = ok ? __ldg(a.x + ((size_t)(n * a.g.Ci + ci) * a.x_plane + hi * a.x_row + wi * a.samp)) : 0.f;
            xv[c][j] = FAST ? -0.5f * v : v;
            acc[c][j] = 0.f;
        }
    }
    if (FAST) {
        for (int e = tid; e < a.g1_size; e += nthreads) G1[e] = 0.f;
    }

    const int nchunks = ceil_div(a.g.Co, a.CKO);
    uint32_t wgrp, wpr;                    // weight staging role of this thread (gx_stage_weights)
    a.d_wpp.divmod(tid, wgrp, wpr);

    auto fill = [&](int chunk, int stage) {
        const int coc0 = chunk * a.CKO;
        // (16-byte copies for the halo-free patches of 1x1 layers were measured here and lost 3 % - 256->64 56x56:
        // 480 -> 498 us - although the same change gains 5 % in the forward kernel)
        fill_patch(Gs + stage * a.gs_stage, a.gout, a.pd, n0, coc0, go_r0, go_c0, a.g.N, a.g.Co, a.g.Ho, a.g.Wo,
                   tid, nthreads);
        gx_stage_weights<KS>(a, Wt + stage * a.ws_stage, coc0, ci0, (int)wgrp, (int)wpr, tid, nthreads);
    };
    auto scale_weights = [&](int stage) {
        gx_scale_weights<KS>(a, Wt + stage * a.ws_stage, (int)wgrp, (int)wpr, tid, nthreads);
    };

    fill(0, 0);
    cp_async_commit();
    for (int c = 0; c < nchunks; ++c) {
        if (c + 1 < nchunks) {
            fill(c + 1, (c + 1) & 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        if (FAST) scale_weights(c & 1);
        __syncthreads();
        const float* gs = Gs + (c & 1) * a.gs_stage;
        if (FAST) {
            for (int e = tid; e < a.g1_size; e += nthreads) {
                float s = 0.f;
                for (int col = 0; col < a.CKO; ++col) s += gs[col * a.CH_STRIDE + e];
                G1[e] += s;
            }
        }
        if (active) {
            const int ncol = min(a.CKO, a.g.Co - c * a.CKO);
            const float* gimg = gs + img * a.pd.ROWS_PITCH;
            const float* wt = Wt + (c & 1) * a.ws_stage + cig * (KK * RC);
            const int goff_s1 = (int)ws * RW + ((int)hr + KS - 1) * a.pd.PITCH;
#pragma unroll 1
            for (int col = 0; col < ncol; ++col) {
                const float* gch = gimg + col * a.CH_STRIDE;
                const float* wch = wt + col * a.WCOL;
                if constexpr (S == 1) {
                    const float* gr = gch + goff_s1;     // row of tap kh = 0; later taps sit one row up each
#pragma unroll
                    for (int kh = 0; kh < KS; ++kh, gr -= a.pd.PITCH) {
                        float gv[RW + KS - 1];
                        load_run<RW + KS - 1, (RW % 4 == 0)>(gv, gr);
                        if constexpr (PACKED) {
                            // two channels per fused multiply-add: (s0, s1) * (g, g) + (acc0, acc1)
                            uint64_t g2[RW + KS - 1];
#pragma unroll
                            for (int i = 0; i < RW + KS - 1; ++i) g2[i] = pack2(gv[i], gv[i]);
#pragma unroll
                            for (int kw = 0; kw < KS; ++kw) {
                                const float4 t = *reinterpret_cast<const float4*>(wch + (kh * KS + kw) * RC);
                                const float wv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                                for (int cc = 0; cc < RC; cc += 2)
#pragma unroll
                                    for (int j = 0; j < RW; ++j)
                                        acc2[cc / 2][j] = fma2(pack2(gx_term<true>(wv[cc], xv[cc][j]), gx_term<true>(wv[cc + 1], xv[cc + 1][j])),
                                                               g2[j + KS - 1 - kw], acc2[cc / 2][j]);
                            }
                        } else {
#pragma unroll
                        for (int kw = 0; kw < KS; ++kw) {
                            const float4 t = *reinterpret_cast<const float4*>(wch + (kh * KS + kw) * RC);
                            const float wv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                            for (int cc = 0; cc < RC; ++cc)
#pragma unroll
                                for (int j = 0; j < RW; ++j)
                                    acc[cc][j] = fmaf(gx_term<FAST>(wv[cc], xv[cc][j]), gv[j + KS - 1 - kw], acc[cc][j]);
                        }
                        }
                    }
                } else if constexpr (S == 2 && RC == 4) {
                    // one pass over ALL output channels of the chunk per tap class: the class dispatch is outside
                    // the channel loop, whose body is then straight-line code (the enclosing loop ends after it)
                    const int ph = (hi + pad) & 1, pwp = ((int)pw + pad) & 1;
                    const int row0 = (hi + pad - ph) / 2 - go_r0;
                    const int col0 = q0 + ((int)pw + pad - pwp) / 2 - go_c0;
                    auto all_columns = [&](auto PH, auto PW) {
#pragma unroll 1
                        for (int cl = 0; cl < ncol; ++cl)
                            gx_taps_stride2<KS, RW, RC, FAST, decltype(PH)::value, decltype(PW)::value>(
                                acc, xv, gimg + cl * a.CH_STRIDE, wt + cl * a.WCOL, row0, col0, a.pd.PITCH);
                    };
                    using I0 = std::integral_constant<int, 0>;
                    using I1 = std::integral_constant<int, 1>;
                    switch (ph * 2 + pwp) {     // uniform across a warp when the segments are ordered by class
                        case 0: all_columns(I0{}, I0{}); break;
                        case 1: all_columns(I0{}, I1{}); break;
                        case 2: all_columns(I1{}, I0{}); break;
                        default: all_columns(I1{}, I1{}); break;
                    }
                    break;
                } else {
#pragma unroll
                    for (int kh = 0; kh < KS; ++kh) {
                        const int tr = hi + pad - kh;
                        if (tr % S != 0) continue;
                        const float* gr = gch + (tr / S - go_r0) * a.pd.PITCH;
#pragma unroll
                        for (int kw = 0; kw < KS; ++kw) {
                            const int tc = (int)pw + pad - kw;
                            if (tc % S != 0) continue;
                            const float* gp = gr + (q0 + tc / S - go_c0);
                            float gv[RW];
#pragma unroll
                            for (int j = 0; j < RW; ++j) gv[j] = gp[j];
                            const float4 t = *reinterpret_cast<const float4*>(wch + (kh * KS + kw) * RC);
                            const float wv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                            for (int cc = 0; cc < RC; ++cc)
#pragma unroll
                                for (int j = 0; j < RW; ++j)
                                    acc[cc][j] = fmaf(gx_term<FAST>(wv[cc], xv[cc][j]), gv[j], acc[cc][j]);
                        }
                    }
                }
            }
            // Two-level summation: the chunk's partial sums are folded into per-thread running totals
            // kept in shared memory, so a long sum over output channels loses far less precision than one
            // running fp32 accumulator would.
            if constexpr (PACKED) {
#pragma unroll
                for (int cc = 0; cc < RC; cc += 2)
#pragma unroll
                    for (int j = 0; j < RW; ++j) {
                        unpack2(acc2[cc / 2][j], acc[cc][j], acc[cc + 1][j]);
                        acc2[cc / 2][j] = 0ull;
                    }
            }
            if (KS == 1 || nchunks > 1) {      // a single chunk's sums stay in registers (3x3 kernels)
#pragma unroll
                for (int cc = 0; cc < RC; ++cc)
#pragma unroll
                    for (int j = 0; j < RW; ++j) {
                        float* t = Tot + (cc * RW + j) * nthreads;
                        *t = (c == 0 ? 0.f : *t) + acc[cc][j];
                        acc[cc][j] = 0.f;
                    }
            }
        }
        __syncthreads();
    }

    if (!active || n >= a.g.N || hi >= a.g.H) return;
    if (KS == 1 || nchunks > 1) {
#pragma unroll
        for (int cc = 0; cc < RC; ++cc)
#pragma unroll
            for (int j = 0; j < RW; ++j) acc[cc][j] = Tot[(cc * RW + j) * nthreads];
    }
    float box[RW];
    if (FAST) {
        // sum of g over the taps of each pixel = box sum of the channel-summed patch
#pragma unroll
        for (int j = 0; j < RW; ++j) box[j] = 0.f;
        const float* g1 = G1 + img * a.pd.ROWS_PITCH;
#pragma unroll
        for (int kh = 0; kh < KS; ++kh) {
            const int tr = hi + pad - kh;
            if (tr % S != 0) continue;
            const float* gr = g1 + (tr / S - go_r0) * a.pd.PITCH;
#pragma unroll
            for (int kw = 0; kw < KS; ++kw) {
                const int tc = (int)pw + pad - kw;
                if (tc % S != 0) continue;
                const float* gp = gr + (q0 + tc / S - go_c0);
#pragma unroll
                for (int j = 0; j < RW; ++j) box[j] += gp[j];
            }
        }
    }
#pragma unroll
    for (int c = 0; c < RC; ++c) {
        const int ci = ci0 + cig * RC + c;
        if (ci >= a.g.Ci) break;
        float* o = a.gx + ((size_t)(n * a.g.Ci + ci) * HW + hi * a.g.W);
        if (S == 1 && RW % 4 == 0 && a.vec_io) {
#pragma unroll
            for (int j = 0; j < RW; j += 4) {
                if (q0 + j >= a.g.W) break;
                float4 v;
                v.x = FAST ? 2.f * acc[c][j] - box[j] : acc[c][j];
                v.y = FAST ? 2.f * acc[c][j + 1] - box[j + 1] : acc[c][j + 1];
                v.z = FAST ? 2.f * acc[c][j + 2] - box[j + 2] : acc[c][j + 2];
                v.w = FAST ? 2.f * acc[c][j + 3] - box[j + 3] : acc[c][j + 3];
                float4* o4 = reinterpret_cast<float4*>(o + q0 + j);
                if (a.accumulate) {
                    const float4 old = *o4;
                    v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                }
                *o4 = v;
            }
            continue;
        }
        if (KS == 1 && S == 1 && a.samp > 1) {
            // sampled grid: pixel (hi, wi) of the grid is pixel (hi*samp, wi*samp) of the real tensor; the other
            // pixels of its samp x samp block are read by no output and get zero (left alone when accumulating)
            float* ob = a.gx + ((size_t)(n * a.g.Ci + ci) * a.x_plane + (size_t)hi * a.x_row);
#pragma unroll
            for (int j = 0; j < RW; ++j) {
                const int wi = q0 + j;
                if (wi >= a.g.W) break;
                const float v = FAST ? 2.f * acc[c][j] - box[j] : acc[c][j];
                float* px = ob + wi * a.samp;
                if (a.accumulate) { *px += v; continue; }
                if (a.samp_pairs) {
                    *reinterpret_cast<float2*>(px) = make_float2(v, 0.f);
                    if (hi * 2 + 1 < a.real_h) *reinterpret_cast<float2*>(px + a.real_w) = make_float2(0.f, 0.f);
                } else {
                    for (int dr = 0; dr < a.samp && hi * a.samp + dr < a.real_h; ++dr)
                        for (int dc = 0; dc < a.samp && wi * a.samp + dc < a.real_w; ++dc)
                            px[dr * a.real_w + dc] = (dr | dc) ? 0.f : v;
                }
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < RW; ++j) {
            const int wi = (q0 + j) * S + pw;
            if (wi < a.g.W) {
                const float v = FAST ? 2.f * acc[c][j] - box[j] : acc[c][j];
                o[wi] = a.accumulate ? o[wi] + v : v;
            }
        }
    }
}

// All output channels of one chunk for a thread's two segments whose tap classes are T0 and 3 - T0: the
// class dispatch happens once per chunk, outside this loop, so the loop body is straight-line code.
template <int KS, int RW, int RC, bool FAST, int T0>
__device__ __forceinline__ void gx_s2pair_columns(float (&acc)[2][RC][RW], const float (&xv)[2][RC][RW], const float* gimg,
                                                  const float* wt, int ncol, int ch_stride, int wcol, const int (&row0v)[2],
                                                  const int (&col0v)[2], int pitch) {
    constexpr int T1 = 3 - T0;
#pragma unroll 1
    for (int col = 0; col < ncol; ++col, gimg += ch_stride, wt += wcol) {
        gx_taps_stride2<KS, RW, RC, FAST, (T0 >> 1), (T0 & 1)>(acc[0], xv[0], gimg, wt, row0v[0], col0v[0], pitch);
        gx_taps_stride2<KS, RW, RC, FAST, (T1 >> 1), (T1 & 1)>(acc[1], xv[1], gimg, wt, row0v[1], col0v[1], pitch);
    }
}

// Stride-2 3x3 layers, balanced.  The four classes of input pixels (row offset mod 2, column parity)
// have 1, 2, 2 and 4 valid taps, so warps that each hold one class finish at very different times and
// wait for each other at every chunk barrier.  Here a thread owns TWO segments of the same row pair and
// column range: one of class c and one of the complementary class 3 - c (1 + 4 or 2 + 2 taps), so every
// warp carries 5 or 4 taps per pixel pair.  Everything else (staging, FAST form, two-level sums) is as in
// adder_gx_kernel; the thread-to-segment map is the class-major one with half as many classes.
template <int KS, int RW, int RC, bool FAST>
__global__ void __launch_bounds__(256, 2) adder_gx_s2pair_kernel(const GxArgs a) {
    constexpr int S = 2, KK = KS * KS, NSEG = 2;
    extern __shared__ __align__(16) float smem[];
    float* const Gs = smem;
    float* const Wt = smem + a.nstages * a.gs_stage;
    float* const G1 = Wt + a.nstages * a.ws_stage;
    float* const Tot = G1 + a.g1_size + threadIdx.x;   // [NSEG*RC*RW][blockDim.x]

    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    uint32_t tn, th, tw, tnh;
    a.d_tiles_w.divmod(blockIdx.x, tnh, tw);
    a.d_tiles_h.divmod(tnh, tn, th);
    const int n0 = tn * a.TI;
    const int hi0 = th * a.TH;
    const int wq0 = tw * (a.SPRC * RW);
    const int ci0 = blockIdx.y * a.TCI;
    const int pad = a.g.pad;
    const int go_r0 = floor_div(hi0 + pad - (KS - 1), S);
    const int go_c0 = floor_div(wq0 * S + pad - (KS - 1), S);

    uint32_t cig, seg, t, t2, ws, hr2, cls, img;
    a.d_segs.divmod(tid, cig, seg);            // d_segs divides by the segments per thread set (SEGS / 2)
    a.d_sprc.divmod(seg, t, ws);
    a.d_ths.divmod(t, t2, hr2);
    a.d_ti.divmod(t2, cls, img);               // cls in {0, 1}: TI*(TH/2)*SPRC consecutive threads share it
    const bool active = (int)cig < a.CGI;
    const int n = n0 + img;
    const int q0 = wq0 + ws * RW;
    const int HW = a.g.H * a.g.W;
    int pwv[NSEG], hiv[NSEG], tapcls[NSEG], row0v[NSEG], col0v[NSEG];
#pragma unroll
    for (int sg = 0; sg < NSEG; ++sg) {
        const int c = sg == 0 ? (int)cls : 3 - (int)cls;
        pwv[sg] = c & 1;
        hiv[sg] = hi0 + (int)hr2 * 2 + (c >> 1);
        const int ph = (hiv[sg] + pad) & 1, pwp = (pwv[sg] + pad) & 1;
        tapcls[sg] = ph * 2 + pwp;
        row0v[sg] = (hiv[sg] + pad - ph) / 2 - go_r0;
        col0v[sg] = q0 + (pwv[sg] + pad - pwp) / 2 - go_c0;
    }

    float xv[NSEG][RC][RW], acc[NSEG][RC][RW];
#pragma unroll
    for (int sg = 0; sg < NSEG; ++sg)
#pragma unroll
        for (int c = 0; c < RC; ++c) {
            const int ci = ci0 + cig * RC + c;
#pragma unroll
            for (int j = 0; j < RW; ++j) {
                const int wi = (q0 + j) * S + pwv[sg];
                const bool ok = active && n < a.g.N && ci < a.g.Ci && hiv[sg] < a.g.H && wi < a.g.W;
                const float v = ok ? __ldg(a.x + ((size_t)(n * a.g.Ci + ci) * HW + hiv[sg] * a.g.W + wi)) : 0.f;
                xv[sg][c][j] = FAST ? -0.5f * v : v;
                acc[sg][c][j] = 0.f;
            }
        }
    if (FAST) {
        for (int e = tid; e < a.g1_size; e += nthreads) G1[e] = 0.f;
    }

    const int nchunks = ceil_div(a.g.Co, a.CKO);
    uint32_t wgrp, wpr;                    // weight staging role of this thread (gx_stage_weights)
    a.d_wpp.divmod(tid, wgrp, wpr);

    auto fill = [&](int chunk, int stage) {
        const int coc0 = chunk * a.CKO;
        fill_patch(Gs + stage * a.gs_stage, a.gout, a.pd, n0, coc0, go_r0, go_c0, a.g.N, a.g.Co, a.g.Ho, a.g.Wo,
                   tid, nthreads);
        gx_stage_weights<KS>(a, Wt + stage * a.ws_stage, coc0, ci0, (int)wgrp, (int)wpr, tid, nthreads);
    };
    auto scale_weights = [&](int stage) {
        gx_scale_weights<KS>(a, Wt + stage * a.ws_stage, (int)wgrp, (int)wpr, tid, nthreads);
    };

    fill(0, 0);
    cp_async_commit();
    for (int c = 0; c < nchunks; ++c) {
        if (c + 1 < nchunks) {
            fill(c + 1, (c + 1) & 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        if (FAST) scale_weights(c & 1);
        __syncthreads();
        const float* gs = Gs + (c & 1) * a.gs_stage;
        if (FAST) {
            for (int e = tid; e < a.g1_size; e += nthreads) {
                float sum = 0.f;
                for (int col = 0; col < a.CKO; ++col) sum += gs[col * a.CH_STRIDE + e];
                G1[e] += sum;
            }
        }
        if (active) {
            const int ncol = min(a.CKO, a.g.Co - c * a.CKO);
            const float* gimg = gs + img * a.pd.ROWS_PITCH;
            const float* wt = Wt + (c & 1) * a.ws_stage + cig * (KK * RC);
            if (tapcls[1] == 3 - tapcls[0]) {       // always, for pad 1 and tiles that start on even rows
                switch (tapcls[0]) {                // uniform across a warp
                    case 0: gx_s2pair_columns<KS, RW, RC, FAST, 0>(acc, xv, gimg, wt, ncol, a.CH_STRIDE, a.WCOL, row0v, col0v, a.pd.PITCH); break;
                    case 1: gx_s2pair_columns<KS, RW, RC, FAST, 1>(acc, xv, gimg, wt, ncol, a.CH_STRIDE, a.WCOL, row0v, col0v, a.pd.PITCH); break;
                    case 2: gx_s2pair_columns<KS, RW, RC, FAST, 2>(acc, xv, gimg, wt, ncol, a.CH_STRIDE, a.WCOL, row0v, col0v, a.pd.PITCH); break;
                    default: gx_s2pair_columns<KS, RW, RC, FAST, 3>(acc, xv, gimg, wt, ncol, a.CH_STRIDE, a.WCOL, row0v, col0v, a.pd.PITCH); break;
                }
            } else
#pragma unroll 1
            for (int col = 0; col < ncol; ++col) {
                const float* gch = gimg + col * a.CH_STRIDE;
                const float* wch = wt + col * a.WCOL;
#pragma unroll
                for (int sg = 0; sg < NSEG; ++sg) {
                    switch (tapcls[sg]) {       // uniform across a warp
                        case 0: gx_taps_stride2<KS, RW, RC, FAST, 0, 0>(acc[sg], xv[sg], gch, wch, row0v[sg], col0v[sg], a.pd.PITCH); break;
                        case 1: gx_taps_stride2<KS, RW, RC, FAST, 0, 1>(acc[sg], xv[sg], gch, wch, row0v[sg], col0v[sg], a.pd.PITCH); break;
                        case 2: gx_taps_stride2<KS, RW, RC, FAST, 1, 0>(acc[sg], xv[sg], gch, wch, row0v[sg], col0v[sg], a.pd.PITCH); break;
                        default: gx_taps_stride2<KS, RW, RC, FAST, 1, 1>(acc[sg], xv[sg], gch, wch, row0v[sg], col0v[sg], a.pd.PITCH); break;
                    }
                }
            }
            if (nchunks > 1) {      // two-level summation, as in adder_gx_kernel
#pragma unroll
                for (int sg = 0; sg < NSEG; ++sg)
#pragma unroll
                    for (int cc = 0; cc < RC; ++cc)
#pragma unroll
                        for (int j = 0; j < RW; ++j) {
                            float* tp = Tot + ((sg * RC + cc) * RW + j) * nthreads;
                            *tp = (c == 0 ? 0.f : *tp) + acc[sg][cc][j];
                            acc[sg][cc][j] = 0.f;
                        }
            }
        }
        __syncthreads();
    }

    if (!active || n >= a.g.N) return;
#pragma unroll
    for (int sg = 0; sg < NSEG; ++sg) {
        const int hi = hiv[sg], pw = pwv[sg];
        if (hi >= a.g.H) continue;
        if (nchunks > 1) {
#pragma unroll
            for (int cc = 0; cc < RC; ++cc)
#pragma unroll
                for (int j = 0; j < RW; ++j) acc[sg][cc][j] = Tot[((sg * RC + cc) * RW + j) * nthreads];
        }
        float box[RW];
        if (FAST) {
#pragma unroll
            for (int j = 0; j < RW; ++j) box[j] = 0.f;
            const float* g1 = G1 + img * a.pd.ROWS_PITCH;
#pragma unroll
            for (int kh = 0; kh < KS; ++kh) {
                const int tr = hi + pad - kh;
                if (tr % S != 0) continue;
                const float* gr = g1 + (tr / S - go_r0) * a.pd.PITCH;
#pragma unroll
                for (int kw = 0; kw < KS; ++kw) {
                    const int tc = pw + pad - kw;
                    if (tc % S != 0) continue;
                    const float* gp = gr + (q0 + tc / S - go_c0);
#pragma unroll
                    for (int j = 0; j < RW; ++j) box[j] += gp[j];
                }
            }
        }
#pragma unroll
        for (int c = 0; c < RC; ++c) {
            const int ci = ci0 + cig * RC + c;
            if (ci >= a.g.Ci) break;
            float* o = a.gx + ((size_t)(n * a.g.Ci + ci) * HW + hi * a.g.W);
#pragma unroll
            for (int j = 0; j < RW; ++j) {
                const int wi = (q0 + j) * S + pw;
                if (wi < a.g.W) {
                    const float v = FAST ? 2.f * acc[sg][c][j] - box[j] : acc[sg][c][j];
                    o[wi] = a.accumulate ? o[wi] + v : v;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------

static int largest_divisor_le_mult(int n, int limit, int mult) {
    for (int d = limit < n ? limit : n; d >= 1; --d)
        if (n % d == 0 && (d % mult == 0 || d == n)) return d;
    return n <= limit ? n : mult;
}

static int pick_pitch_gx(int cols, int segs, int spr, int sprc, int th, int rows, int rw) {
    int best = cols, best_cost = 1 << 30;
    for (int pitch = cols; pitch < cols + 33; ++pitch) {
        int cost = 0;
        for (int w0 = 0; w0 < segs; w0 += 32) {
            int cnt[32] = {0};
            int worst = 0;
            for (int l = w0; l < w0 + 32 && l < segs; ++l) {
                const int wsx = l % spr, t2 = l / spr, hr = t2 % th, img = t2 / th;
                const int addr = (img * rows + hr) * pitch + (wsx % sprc) * rw;
                const int b = addr & 31;
                if (++cnt[b] > worst) worst = cnt[b];
            }
            cost += worst;
        }
        if (cost < best_cost) { best_cost = cost; best = pitch; }
    }
    return best;
}

struct GxPlan {
    GxArgs a;
    int threads, ks, s, rw, rc, fast;
    size_t smem;
    long long gx;
    int gy;
};

// nseg = 2: the paired stride-2 kernel (a thread owns two segments of complementary tap classes).
template <int KS, int S, int RW, int RC, bool FAST>
static int plan_gx_n(const Geom& g, const TileHint& hint, GxPlan& p, int nseg) {
    GxArgs& a = p.a;
    a.nseg = nseg;
    p.ks = KS; p.s = S; p.rw = RW; p.rc = RC; p.fast = FAST;
    a.g = g;
    const int threads_target = hint.threads > 0 ? hint.threads : 256;
    // stride > 1: more pixels per CTA, one tap class per warp.  1x1 layers tiled as one long row per image: 64
    // input channels per CTA, so that a staged value of g serves four times the threads (64->256 56x56: 683 -> 426 us)
    const int cg_max = hint.cg > 0 ? hint.cg : (S > 1 ? 2 : ((KS == 1 && g.H == 1) ? 16 : (g.Ci >= 128 ? 8 : 4)));
    a.CGI = ceil_div(g.Ci, RC) < cg_max ? ceil_div(g.Ci, RC) : cg_max;
    a.TCI = a.CGI * RC;
    a.TCIP = a.TCI;
    a.WCOL = a.TCI * KS * KS;
    int segs_target = threads_target / a.CGI * nseg;
    if (segs_target < 1) segs_target = 1;
    const int class_px = ceil_div(g.W, S);                 // pixels of one column parity in a row
    const int sprc_full = ceil_div(class_px, RW);
    a.SPRC = sprc_full * S <= segs_target ? sprc_full : (segs_target / S > 0 ? segs_target / S : 1);
    a.SPR = a.SPRC * S;
    int rows_target = segs_target / a.SPR;
    {   // short tiles won the sweeps (more CTAs, smaller patches), but keep at least a warp of segments
        int cap = 8 * S;
        if (cap * a.SPR < 32) cap = ceil_div(32, a.SPR);
        if (rows_target > cap) rows_target = cap;
    }
    if (rows_target < 1) rows_target = 1;
    if (hint.th > 0) {
        a.TH = hint.th < g.H ? hint.th : g.H;
    } else {
        a.TH = largest_divisor_le_mult(g.H, rows_target, S);
    }
    if (a.TH > g.H) a.TH = g.H;
    a.TI = 1;
    int ti_budget = 1;   // tile images before clamping to the batch: the chunk size must not depend on N
    if (a.TH == g.H) {
        a.TI = segs_target / (a.TH * a.SPR);
        ti_budget = a.TI > 1 ? a.TI : 1;
        if (a.TI < 1) a.TI = 1;
        if (a.TI > g.N) a.TI = g.N;
        if (a.TI < 1) a.TI = 1;
    }
    if (hint.ti > 0) a.TI = hint.ti;
    a.SEGS = a.TI * a.TH * a.SPR;
    if (nseg == 2 && (a.TH % S != 0 || a.SEGS % 2 != 0)) return ADDER_ERR_INTERNAL;   // needs whole row pairs
    const int threads = round_up(a.CGI * (a.SEGS / nseg), 32);
    p.threads = threads;
    if (threads > 256) return ADDER_ERR_INTERNAL;
    a.tiles_h = ceil_div(g.H, a.TH);
    a.tiles_w = ceil_div(sprc_full, a.SPRC);
    if (S > 1 && a.tiles_h > 1 && a.TH % S != 0) return ADDER_ERR_INTERNAL;
    PatchDims& pd = a.pd;
    pd.TI = a.TI;
    pd.ROWS = (S == 1) ? a.TH + KS - 1 : (a.TH + KS - 2) / S + 2;
    pd.COLS = a.SPRC * RW + (S - 1 + g.pad) / S - floor_div(g.pad - (KS - 1), S);
    if (S == 1 && RW % 4 == 0) {
        const int spr = a.SPR, th = a.TH, rows = pd.ROWS, segs = a.SEGS;
        pd.PITCH = pick_pitch_vec(pd.COLS, segs < 32 ? segs : 32, [=](int l, int& row, int& col) {
            const int ws = l % spr, t2 = l / spr;
            row = (t2 / th) * rows + (t2 % th); col = ws * RW; }, 8);
        // (at most 8 floats of padding per row: a conflict-free pitch of 24 for a 10-column patch halves the
        // output channels that fit a chunk, which costs more than two-way conflicts on the few loads of g -
        // 64->64 8x8: 80 -> 72 us, 32->32 16x16: 76 -> 69 us)
    } else {
        pd.PITCH = pick_pitch_gx(pd.COLS, a.SEGS, a.SPR, a.SPRC, a.TH, pd.ROWS, RW);
    }
    pd.ROWS_PITCH = pd.ROWS * pd.PITCH;
    a.CH_STRIDE = a.TI * pd.ROWS_PITCH;
    a.g1_size = FAST ? a.CH_STRIDE : 0;
    // shared memory per CTA in proportion to its threads, so that about 16 warps stay resident per SM.
    // The thread count used here is the one of a full tile (before TI is clamped to a small batch), so
    // that the chunk size, and with it the order of summation, does not depend on the batch size.
    const int threads_full = hint.ti > 0 ? threads : round_up(a.CGI * (ti_budget * a.TH * a.SPR / nseg), 32);
    const int budget_floats = (hint.smem_kb > 0 ? hint.smem_kb : (threads_full * nseg <= 64 ? 26 : threads_full * nseg <= 128 ? 52 : 104)) * 1024 / 4;
    int cko = hint.ck > 0 ? hint.ck : (KS == 1 ? 64 : 16);
    if (cko > g.Co) cko = g.Co;
    // All output channels in ONE chunk need no second stage: where that fits the budget it is taken, whatever the
    // default chunk size says - no chunk barrier, no running totals, and for 3x3 stride-1 layers the
    // three-CTAs-per-SM form of the kernel (32->32 16x16).
    bool whole = false;
    if (hint.ck <= 0 && KS == 3 && g.Co <= 64) {
        const int need1 = round_up(g.Co * ti_budget * pd.ROWS_PITCH, 4) + g.Co * a.WCOL +
                          (FAST ? ti_budget * pd.ROWS_PITCH : 0) + (nseg == 2 ? RC * RW * threads_full * nseg : 0);
        if (need1 <= budget_floats) { cko = g.Co; whole = true; }
    }
    while (cko > 1 && !whole) {
        const int need = 2 * (round_up(cko * ti_budget * pd.ROWS_PITCH, 4) + cko * a.WCOL) +
                         (FAST ? ti_budget * pd.ROWS_PITCH : 0) + RC * RW * threads_full * nseg;
        if (need <= budget_floats) break;
        --cko;
    }
    cko = ceil_div(g.Co, ceil_div(g.Co, cko));    // same number of chunks, evenly sized: no padded channels
    a.CKO = cko;
    pd.CH = cko;
    a.gs_stage = round_up(cko * a.CH_STRIDE, 4);
    a.ws_stage = cko * a.WCOL;
    const int nchunks = ceil_div(g.Co, cko);
    a.nstages = nchunks > 1 ? 2 : 1;
    // running totals in shared memory only where the kernels use them (several chunks, or the 1x1 kernels)
    const size_t tot = (nseg == 2 || KS == 1 || nchunks > 1) ? (size_t)RC * RW * threads * nseg : 0;
    const size_t smem = ((size_t)a.nstages * (a.gs_stage + a.ws_stage) + a.g1_size + tot) * sizeof(float);
    p.smem = smem;
    if (smem > 200 * 1024) return ADDER_ERR_UNSUPPORTED;
    pd.d_cols = FastDiv(pd.COLS);
    pd.d_rows = FastDiv(pd.ROWS);
    a.d_tiles_h = FastDiv(a.tiles_h);
    a.d_tiles_w = FastDiv(a.tiles_w);
    a.d_segs = FastDiv(a.SEGS / nseg);
    a.d_spr = FastDiv(a.SPR);
    a.d_sprc = FastDiv(a.SPRC);
    a.d_th = FastDiv(a.TH);
    a.class_major = (S > 1 && a.TH % S == 0) ? 1 : 0;
    a.d_ths = FastDiv(a.class_major ? a.TH / S : 1);
    a.d_ti = FastDiv(a.TI);
    a.WPP = a.TCI * KS * KS < threads ? a.TCI * KS * KS : threads;
    a.wgroups = threads / a.WPP;
    a.d_wpp = FastDiv(a.WPP);
    a.d_tci = FastDiv(a.TCI);
    a.d_kk = FastDiv(KS * KS);
    const long long gxd = (long long)ceil_div(g.N, a.TI) * a.tiles_h * a.tiles_w;
    const int gyd = ceil_div(g.Ci, a.TCI);
    p.gx = gxd; p.gy = gyd;
    if (gxd > 2147483647LL || gyd > 65535) return ADDER_ERR_UNSUPPORTED;
    return ADDER_OK;
}

template <int KS, int S, int RW, int RC, bool FAST>
static int plan_gx_t(const Geom& g, const TileHint& hint, GxPlan& p) {
    // 3x3 stride 2: the paired kernel (4-pixel segments only: wider ones spill with two segments per thread)
    // unless a tile hint asks for the one-class-per-thread kernel
    const bool tile_hint = (hint.threads | hint.cg | hint.th | hint.ti | hint.ck | hint.smem_kb) != 0;
    if (KS == 3 && S == 2 && RW <= 4 && !tile_hint && plan_gx_n<KS, S, RW, RC, FAST>(g, hint, p, 2) == ADDER_OK) return ADDER_OK;
    return plan_gx_n<KS, S, RW, RC, FAST>(g, hint, p, 1);
}

// The geometry the kernels tile: the layer itself, or - for a strided, unpadded 1x1 layer - the stride-1 layer on
// the grid of sampled pixels (every unsampled input pixel has a zero gradient and is not worth a thread).
static Geom gx_tiling_geom(const Geom& g) {
    Geom t = g;
    if (g.k == 1 && g.stride > 1 && g.pad == 0) { t.H = g.Ho; t.W = g.Wo; t.stride = 1; }
    return t;
}

template <int KS, int S, int RW, int RC, bool FAST>
static int launch_gx_t(const Geom& real, const float* gout, const float* x, const float* w, float* gx,
                       int accumulate, const TileHint& hint, cudaStream_t stream) {
    GxPlan p;
    const Geom g = gx_tiling_geom(real);
    const int st = plan_gx_t<KS, S, RW, RC, FAST>(g, hint, p);
    if (st != ADDER_OK) return st;
    p.a.gout = gout; p.a.x = x; p.a.w = w; p.a.gx = gx; p.a.accumulate = accumulate;
    p.a.samp = (KS == 1 && S == 1) ? real.stride : 1;
    p.a.x_plane = real.H * real.W; p.a.x_row = real.W * p.a.samp; p.a.real_h = real.H; p.a.real_w = real.W;
    p.a.samp_pairs = (p.a.samp == 2 && real.W % 2 == 0 && (reinterpret_cast<uintptr_t>(gx) & 7) == 0) ? 1 : 0;
    p.a.vec_io = (S == 1 && RW % 4 == 0 && g.W % 4 == 0 && p.a.samp == 1 &&
                  ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gx)) & 15) == 0) ? 1 : 0;
    if constexpr (KS == 3 && S == 2 && RW <= 4) {
        if (p.a.nseg == 2) {
            auto kern2 = adder_gx_s2pair_kernel<KS, RW, RC, FAST>;
            if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern2), p.smem) != ADDER_OK) return ADDER_ERR_CUDA;
            kern2<<<dim3((unsigned)p.gx, (unsigned)p.gy), p.threads, p.smem, stream>>>(p.a);
            return launched();
        }
    }
    if constexpr (S == 1 && RW == 4 && KS == 3) {
        if (p.a.nstages == 1 && 3 * (p.smem + 1024) <= 227 * 1024) {
            auto kern3 = adder_gx_kernel<KS, S, RW, RC, FAST, 3>;
            if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern3), p.smem) != ADDER_OK) return ADDER_ERR_CUDA;
            kern3<<<dim3((unsigned)p.gx, (unsigned)p.gy), p.threads, p.smem, stream>>>(p.a);
            return launched();
        }
    }
    auto kern = adder_gx_kernel<KS, S, RW, RC, FAST>;
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), p.smem) != ADDER_OK) return ADDER_ERR_CUDA;
    kern<<<dim3((unsigned)p.gx, (unsigned)p.gy), p.threads, p.smem, stream>>>(p.a);
    return launched();
}

// Register tile: 4 input channels x RW pixels.  8-pixel segments unless the layer is too small to fill
// the GPU with them (see choose_fwd_tile); 7-pixel segments for 7/14/28-wide planes.
static int choose_gx_rw(const Geom& g, const TileHint& hint) {
    if (hint.rw > 0) return hint.rw;
    const int class_px = ceil_div(g.W, g.stride);
    if (g.k == 1 && g.H == 1 && g.stride == 1) return 8;     // flattened 1x1 layer or column matrix
    if (g.k == 3 && g.stride == 2) return 4;     // the paired-class kernel, also with a ragged last segment (256->256 28x28: 2116 -> 1788 us)
    if ((class_px % 8 != 0) && (class_px % 7 == 0)) return 7;
    if (class_px % 4 != 0) return 8;
    if (g.k == 1 && class_px % 8 == 0) return 8;     // one tap per channel: the wider tile halves the loads per term
    return 4;      // 4-pixel segments won every sweep of the 3x3 ResNet-20 layer shapes
}

#define ADDER_GX_DISPATCH(CALL)                                                             \
    if (g.k == 3 && g.stride == 1) { ADDER_GX_TILES(3, 1, CALL) }                           \
    else if (g.k == 3 && g.stride == 2) { ADDER_GX_TILES(3, 2, CALL) }                      \
    else if (g.k == 1 && g.stride == 1) { ADDER_GX_TILES(1, 1, CALL) }                      \
    else if (g.k == 1 && g.stride == 2 && g.pad == 0) { ADDER_GX_TILES(1, 1, CALL) }          \
    else if (g.k == 1 && g.stride == 2) { ADDER_GX_TILES(1, 2, CALL) }
#define ADDER_GX_TILES(KS_, S_, CALL)                                                       \
    if (rw == 7) { if (fast) { CALL(KS_, S_, 7, 4, true) } else { CALL(KS_, S_, 7, 4, false) } }        \
    else if (rw == 4) { if (fast) { CALL(KS_, S_, 4, 4, true) } else { CALL(KS_, S_, 4, 4, false) } }   \
    else { if (fast) { CALL(KS_, S_, 8, 4, true) } else { CALL(KS_, S_, 8, 4, false) } }

int describe_gx(const Geom& layer, int fast, const TileHint& hint, char* buf, size_t n) {
    const Geom g = flatten_pointwise(layer, true);
    if (hint.is_default() && pointwise_applicable(g)) {
        snprintf(buf, n, "gx k=1 s=%d pointwise fast=%d: one thread per output position, 16 input channels per CTA, threads=256 "
                 "grid=(%d,%d) status=0", g.stride, fast, ceil_div(g.N * g.Ho * g.Wo, 256), ceil_div(g.Ci, 16));
        return ADDER_OK;
    }
    const Geom tg = gx_tiling_geom(g);
    const int rw = choose_gx_rw(tg, hint);
    GxPlan p;
    int st = ADDER_ERR_UNSUPPORTED;
#define ADDER_GX_PLAN(KS_, S_, RW_, RC_, FAST_) st = plan_gx_t<KS_, S_, RW_, RC_, FAST_>(tg, hint, p);
    ADDER_GX_DISPATCH(ADDER_GX_PLAN)
#undef ADDER_GX_PLAN
    if (st == ADDER_ERR_UNSUPPORTED && !((g.k == 1 || g.k == 3) && (g.stride == 1 || g.stride == 2))) return st;
    snprintf(buf, n,
             "gx k=%d s=%d RW=%d RC=%d fast=%d segs/thread=%d CGI=%d TCI=%d TI=%d TH=%d SPRC=%d SEGS=%d CKO=%d rows=%d cols=%d pitch=%d "
             "threads=%d smem=%zu grid=(%lld,%d) status=%d",
             p.ks, p.s, p.rw, p.rc, p.fast, p.a.nseg, p.a.CGI, p.a.TCI, p.a.TI, p.a.TH, p.a.SPRC, p.a.SEGS, p.a.CKO, p.a.pd.ROWS,
             p.a.pd.COLS, p.a.pd.PITCH, p.threads, p.smem, p.gx, p.gy, st);
    return ADDER_OK;
}

int launch_gx(const Geom& layer, const float* gout, const float* x, const float* w, float* gx, int fast,
              int accumulate, const TileHint& hint, cudaStream_t stream) {
    const Geom g = flatten_pointwise(layer, true);
    if (hint.is_default() && pointwise_applicable(g)) return launch_pointwise_gx(g, gout, x, w, gx, fast, accumulate, stream);
    const int rw = choose_gx_rw(gx_tiling_geom(g), hint);
#define ADDER_GX_LAUNCH(KS_, S_, RW_, RC_, FAST_) \
    return launch_gx_t<KS_, S_, RW_, RC_, FAST_>(g, gout, x, w, gx, accumulate, hint, stream);
    ADDER_GX_DISPATCH(ADDER_GX_LAUNCH)
#undef ADDER_GX_LAUNCH
    return ADDER_ERR_UNSUPPORTED;
}

}  // namespace adder
