// Input gradient of stride-1 adder layers, persistent multi-stage form:
//   gx[n,ci,y,x] = sum over (co,kh,kw) with 0 <= y+pad-kh < Ho, 0 <= x+pad-kw < Wo of
//                  clamp(w[co,ci,kh,kw] - x[n,ci,y,x], -1, 1) * g[n,co,y+pad-kh,x+pad-kw]
// (CONV_BACKWARD's grad_i, adder_cuda/adder.cu:245-246,:266, plus the col2im autograd runs for adder.py:32-33,
// as one gather per input pixel: no atomics, deterministic.)
//
// Differences from adder_gx_kernel (adder_bwd_input.cu), which keeps the stride-2 layers and odd widths:
//  * Persistent CTAs walking over (input-channel tile, pixel tile) units; a CTA's work is a flat sequence
//    of items (unit, output-channel chunk) streamed through a three-stage cp.async ring.  The unit's own
//    x tile travels with its first chunk (into a slot of its own), so nothing is fetched with exposed
//    latency at the start of a unit.  One block barrier per item (two at the end of a unit).
//  * Doubled rows of g.  The staged patch of g holds every value twice, so a 128-bit shared-memory load
//    yields two ready (g, g) operands for the packed multiply-add over two input channels
//        (s_a, s_b) * (g, g) + (acc_a, acc_b)        fma.rn.f32x2
//    with s = sat(w/2 + 1/2 - x/2) (one saturating add each; clamp(d,-1,1) = 2*sat(d/2+1/2) - 1) or, in the
//    exact form, s = min(max(w - x, -1), 1).  No register moves are spent on building (g, g) pairs.
//  * KG groups of threads share one tile and take every KG-th output channel of a chunk; the partial sums
//    are folded through shared memory at the end of a unit (more warps per SM on small planes).
//  * Lanes of a warp hold consecutive rows of the tile, row pitch an odd number of 16-byte words.
#include "common.cuh"
#include "kernels.h"
#include "patch_fill.cuh"
#include <cstdio>

namespace adder {

constexpr int GX_STAGES = 3;

struct GxPipeArgs {
    Geom g;
    const float* gout;
    const float* x;
    const float* w;
    float* gx;
    PatchDims pdg;       // patch of g of one chunk: [CKO][TI*G_ROWS][PITCH], rows doubled
    PatchDims pdx;       // the unit's x tile: [TCI][TI*TH][XP]
    int TI, TH, SPR, SEGS, CGI, KG, TCI, TCIP, CKO;
    int G_ROWS, PITCH, CH_STRIDE, XP, XCH;
    int gs_stage, ws_stage, xs_stage, stage_floats, g1_size, tot_floats, red_floats, x_slots, two_level;
    int tiles_h, tiles_w, n_px_tiles, n_units, nchunks, accumulate, vec_io, x_quads;
    FastDiv d_tiles_h, d_tiles_w, d_px_tiles, d_nchunks, d_group, d_segs, d_rows, d_th, d_xquads, d_tci9;
};

template <bool FAST>
__device__ __forceinline__ float gxp_term(float wv, float xv) {
    if (FAST) return __saturatef(wv + xv);                 // wv = w/2+1/2, xv = -x/2
    return fminf(fmaxf(wv - xv, -1.f), 1.f);
}

template <int KS, int RW, int RC, bool FAST>
__global__ void __launch_bounds__(256, 2) adder_gx_pipe_kernel(const GxPipeArgs a) {
    constexpr int KK = KS * KS;
    constexpr int GW = RW + KS - 1;          // values of g one segment touches per (co, kh)
    constexpr int NS = GX_STAGES;
    extern __shared__ __align__(16) float smem[];
    float* const Xt = smem + NS * a.stage_floats;          // x tiles of the units in flight: [x_slots][xs_stage]
    float* const G1 = Xt + a.x_slots * a.xs_stage;
    float* const Tot = G1 + a.g1_size;
    float* const Red = Tot + a.tot_floats;

    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    uint32_t kg, rem, cig, seg, ws, rowidx, img, hr;
    a.d_group.divmod(tid, kg, rem);
    a.d_segs.divmod(rem, cig, seg);
    a.d_rows.divmod(seg, ws, rowidx);
    a.d_th.divmod(rowidx, img, hr);
    const bool active = (int)kg < a.KG && (int)cig < a.CGI;
    const int pad = a.g.pad;
    const int HW = a.g.H * a.g.W;

    const int my_units = ((int)blockIdx.x < a.n_units) ? (a.n_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int n_items = my_units * a.nchunks;
    const int w_elems = a.CKO * a.TCI * KK;

    auto unit_origin = [&](int k, int& n0, int& hi0, int& wq0, int& ci0) {
        const uint32_t u = blockIdx.x + (uint32_t)k * gridDim.x;
        uint32_t ct, pt, tn, th, tw, tnh;
        a.d_px_tiles.divmod(u, ct, pt);
        a.d_tiles_w.divmod(pt, tnh, tw);
        a.d_tiles_h.divmod(tnh, tn, th);
        n0 = tn * a.TI; hi0 = th * a.TH; wq0 = tw * (a.SPR * RW); ci0 = ct * a.TCI;
    };

    // Weight slab of a chunk -> [col][tap][TCIP] (input channel innermost).  Element e = col*(TCI*KK) + r with
    // r = cil*KK + tap runs along contiguous global memory for each output channel.
    auto stage_weights = [&](float* wt, int coc0, int ci0) {
        const int nci = min(a.TCI, a.g.Ci - ci0);
        for (int e = tid; e < w_elems; e += nthreads) {
            uint32_t col, r;
            a.d_tci9.divmod(e, col, r);
            const int cil = r / KK, tap = r - cil * KK;
            const int co = coc0 + col;
            const bool ok = (co < a.g.Co) & (cil < nci);
            cp_async4(wt + (col * KK + tap) * a.TCIP + cil, ok ? a.w + ((size_t)co * a.g.Ci + ci0) * KK + r : a.w, ok);
        }
    };
    auto scale_weights = [&](float* wt) {      // FAST: w -> w/2 + 1/2, each thread the elements it copied itself
        for (int e = tid; e < w_elems; e += nthreads) {
            uint32_t col, r;
            a.d_tci9.divmod(e, col, r);
            const int cil = r / KK, tap = r - cil * KK;
            float* p = wt + (col * KK + tap) * a.TCIP + cil;
            *p = fmaf(*p, 0.5f, 0.5f);
        }
    };

    auto fill = [&](int item, int stage) {
        if (item >= n_items) return;
        uint32_t k, chunk;
        a.d_nchunks.divmod(item, k, chunk);
        int n0, hi0, wq0, ci0;
        unit_origin((int)k, n0, hi0, wq0, ci0);
        float* st = smem + stage * a.stage_floats;
        const int coc0 = chunk * a.CKO;
        fill_patch<true>(st, a.gout, a.pdg, n0, coc0, hi0 + pad - (KS - 1), wq0 + pad - (KS - 1), a.g.N, a.g.Co,
                         a.g.Ho, a.g.Wo, tid, nthreads);
        stage_weights(st + a.gs_stage, coc0, ci0);
        if (chunk == 0) {
            float* xt = Xt + ((int)k % a.x_slots) * a.xs_stage;
            if (a.x_quads)
                fill_patch_quads(xt, a.x, a.pdx, a.d_xquads, n0, ci0, hi0, wq0, a.g.N, a.g.Ci, a.g.H, a.g.W, tid, nthreads);
            else
                fill_patch<false>(xt, a.x, a.pdx, n0, ci0, hi0, wq0, a.g.N, a.g.Ci, a.g.H, a.g.W, tid, nthreads);
        }
    };

    float xv[RC][RW];
    uint64_t acc2[RC / 2][RW];
#pragma unroll
    for (int c = 0; c < RC / 2; ++c)
#pragma unroll
        for (int j = 0; j < RW; ++j) acc2[c][j] = 0ull;

#pragma unroll
    for (int s = 0; s < NS - 1; ++s) {
        fill(s, s);
        cp_async_commit();
    }
    int stage = 0, chunk = 0, unit_k = 0;
    for (int it = 0; it < n_items; ++it) {
        cp_async_wait<NS - 2>();
        float* const st = smem + stage * a.stage_floats;
        if (FAST) scale_weights(st + a.gs_stage);
        __syncthreads();      // item `it` is complete for everyone, and everyone is done with item it-1
        {
            const int fs = stage == 0 ? NS - 1 : stage - 1;
            fill(it + NS - 1, fs);
            cp_async_commit();
        }
        const float* gs = st;
        if (FAST) {
            // channel-summed patch of g (every second word of the doubled rows): the correction term's input
            for (int e = tid; e < a.g1_size; e += nthreads) {
                float s = 0.f;
                for (int col = 0; col < a.CKO; ++col) s += gs[col * a.CH_STRIDE + 2 * e];
                G1[e] = (chunk == 0 ? 0.f : G1[e]) + s;
            }
        }
        if (active) {
            if (chunk == 0) {
                const float* xt = Xt + (unit_k % a.x_slots) * a.xs_stage + (cig * RC) * a.XCH + (img * a.TH + hr) * a.XP + ws * RW;
#pragma unroll
                for (int c = 0; c < RC; ++c) {
                    float t[RW];
                    load_run<RW, (RW % 4 == 0)>(t, xt + c * a.XCH);
#pragma unroll
                    for (int j = 0; j < RW; ++j) xv[c][j] = FAST ? -0.5f * t[j] : t[j];
                }
            }
            const int ncol = min(a.CKO, a.g.Co - chunk * a.CKO);
            const float* gimg = gs + img * a.pdg.ROWS_PITCH + ws * (RW * 2);
            const float* wt = st + a.gs_stage + cig * RC;
#pragma unroll 1
            for (int col = kg; col < ncol; col += a.KG) {
                const float* gch = gimg + col * a.CH_STRIDE;
                const float* wch = wt + col * KK * a.TCIP;
#pragma unroll
                for (int kh = 0; kh < KS; ++kh) {
                    uint64_t g2[GW];
                    load_pairs<GW, true>(g2, gch + ((int)hr + KS - 1 - kh) * a.PITCH);
#pragma unroll
                    for (int kw = 0; kw < KS; ++kw) {
                        float wv[RC];
#pragma unroll
                        for (int c4 = 0; c4 < RC; c4 += 4) {
                            const float4 t = *reinterpret_cast<const float4*>(wch + (kh * KS + kw) * a.TCIP + c4);
                            wv[c4] = t.x; wv[c4 + 1] = t.y; wv[c4 + 2] = t.z; wv[c4 + 3] = t.w;
                        }
#pragma unroll
                        for (int cc = 0; cc < RC; cc += 2)
#pragma unroll
                            for (int j = 0; j < RW; ++j)
                                acc2[cc / 2][j] = fma2(pack2(gxp_term<FAST>(wv[cc], xv[cc][j]), gxp_term<FAST>(wv[cc + 1], xv[cc + 1][j])),
                                                       g2[j + KS - 1 - kw], acc2[cc / 2][j]);
                    }
                }
            }
            // Two-level summation for long sums (more than 1024 terms per pixel): a chunk's partial sums are
            // folded into running totals kept in shared memory, which loses far less precision than one
            // running fp32 accumulator would.  Shorter sums stay in registers across the chunks.
            if (a.two_level) {
                float* tp = Tot + rem + kg * a.d_group.div;
#pragma unroll
                for (int cc = 0; cc < RC; cc += 2)
#pragma unroll
                    for (int j = 0; j < RW; ++j) {
                        float s0, s1;
                        unpack2(acc2[cc / 2][j], s0, s1);
                        float* t0 = tp + (cc * RW + j) * nthreads;
                        float* t1 = tp + ((cc + 1) * RW + j) * nthreads;
                        *t0 = (chunk == 0 ? 0.f : *t0) + s0;
                        *t1 = (chunk == 0 ? 0.f : *t1) + s1;
                        acc2[cc / 2][j] = 0ull;
                    }
            }
        }
        if (++chunk == a.nchunks) {
            chunk = 0;
            // this thread's sums of channel pair cc: from the running totals (multi-chunk units) or registers
            auto pair_sums = [&](int cc, float (&s0)[RW], float (&s1)[RW]) {
                if (a.two_level) {
                    const float* tp = Tot + rem + kg * a.d_group.div;
#pragma unroll
                    for (int j = 0; j < RW; ++j) {
                        s0[j] = tp[(cc * RW + j) * nthreads];
                        s1[j] = tp[((cc + 1) * RW + j) * nthreads];
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < RW; ++j) unpack2(acc2[cc / 2][j], s0[j], s1[j]);
                }
            };
            if (a.KG > 1 && active && kg > 0) {
                float* r = Red + ((kg - 1) * (RC * RW)) * a.d_group.div + rem;
#pragma unroll
                for (int cc = 0; cc < RC; cc += 2) {
                    float s0[RW], s1[RW];
                    pair_sums(cc, s0, s1);
#pragma unroll
                    for (int j = 0; j < RW; ++j) {
                        r[(cc * RW + j) * a.d_group.div] = s0[j];
                        r[((cc + 1) * RW + j) * a.d_group.div] = s1[j];
                    }
                }
            }
            if (a.KG > 1 || FAST) __syncthreads();     // partial sums and the channel-summed patch are complete
            if (active && kg == 0) {
                int n0, hi0, wq0, ci0;
                unit_origin(unit_k, n0, hi0, wq0, ci0);
                const int n = n0 + img, hi = hi0 + hr, q0 = wq0 + ws * RW;
                if (n < a.g.N && hi < a.g.H && q0 < a.g.W) {
                    float box[RW];
#pragma unroll
                    for (int j = 0; j < RW; ++j) box[j] = 0.f;
                    if (FAST) {
                        // sum of g over the taps of each pixel = box sum of the channel-summed patch
                        const float* g1 = G1 + img * (a.G_ROWS * (a.PITCH / 2)) + ws * RW;
#pragma unroll
                        for (int kh = 0; kh < KS; ++kh) {
                            const float* gr = g1 + ((int)hr + KS - 1 - kh) * (a.PITCH / 2);
#pragma unroll
                            for (int kw = 0; kw < KS; ++kw)
#pragma unroll
                                for (int j = 0; j < RW; ++j) box[j] += gr[j + KS - 1 - kw];
                        }
                    }
#pragma unroll
                    for (int cc = 0; cc < RC; cc += 2) {
                        float sum[2][RW];
                        pair_sums(cc, sum[0], sum[1]);
                        for (int q = 1; q < a.KG; ++q) {
                            const float* r = Red + ((q - 1) * (RC * RW)) * a.d_group.div + rem;
#pragma unroll
                            for (int j = 0; j < RW; ++j) {
                                sum[0][j] += r[(cc * RW + j) * a.d_group.div];
                                sum[1][j] += r[((cc + 1) * RW + j) * a.d_group.div];
                            }
                        }
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int ci = ci0 + cig * RC + cc + h;
                            if (ci >= a.g.Ci) break;
                            float* o = a.gx + ((size_t)(n * a.g.Ci + ci) * HW + hi * a.g.W + q0);
                            if (RW % 4 == 0 && a.vec_io) {
#pragma unroll
                                for (int j = 0; j < RW; j += 4) {
                                    if (q0 + j >= a.g.W) break;
                                    float4 v;
                                    v.x = FAST ? 2.f * sum[h][j] - box[j] : sum[h][j];
                                    v.y = FAST ? 2.f * sum[h][j + 1] - box[j + 1] : sum[h][j + 1];
                                    v.z = FAST ? 2.f * sum[h][j + 2] - box[j + 2] : sum[h][j + 2];
                                    v.w = FAST ? 2.f * sum[h][j + 3] - box[j + 3] : sum[h][j + 3];
                                    float4* o4 = reinterpret_cast<float4*>(o + j);
                                    if (a.accumulate) {
                                        const float4 old = *o4;
                                        v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                                    }
                                    *o4 = v;
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < RW; ++j) {
                                    if (q0 + j < a.g.W) {
                                        const float v = FAST ? 2.f * sum[h][j] - box[j] : sum[h][j];
                                        o[j] = a.accumulate ? o[j] + v : v;
                                    }
                                }
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < RC / 2; ++c)
#pragma unroll
                for (int j = 0; j < RW; ++j) acc2[c][j] = 0ull;
            ++unit_k;
        }
        stage = stage + 1 == NS ? 0 : stage + 1;
    }
    cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------

struct GxPipePlan {
    GxPipeArgs a;
    int threads, grid, status, ks, rw, rc, fast;
    size_t smem;
};

static int gx_ctas_per_sm(size_t smem, int threads) {
    const int by_smem = (int)((227 * 1024) / (smem + 1024));
    const int by_regs = 65536 / (128 * threads);
    int c = by_smem < by_regs ? by_smem : by_regs;
    if (c > 2) c = 2;
    return c < 1 ? 1 : c;
}

template <int KS, int RW, int RC, bool FAST>
static GxPipePlan plan_gx_pipe_kg(const Geom& g, const TileHint& hint, int kg_forced);

// More reduction groups mean fewer pixels per CTA, i.e. smaller patches: when three stages of a decent
// chunk (4 output channels or more) do not fit next to the x tile, the group count is doubled.
template <int KS, int RW, int RC, bool FAST>
static GxPipePlan plan_gx_pipe_t(const Geom& g, const TileHint& hint) {
    GxPipePlan p = plan_gx_pipe_kg<KS, RW, RC, FAST>(g, hint, 0);
    if (hint.ck > 0) return p;
    for (int kg = p.a.KG * 2; kg <= 4 && g.Co >= 8 * kg; kg *= 2) {
        if (p.status == ADDER_OK && p.a.CKO >= 4 && p.a.CKO >= p.a.KG && 2 * (p.smem + 1024) <= 227 * 1024) break;
        p = plan_gx_pipe_kg<KS, RW, RC, FAST>(g, hint, kg);
    }
    return p;
}

template <int KS, int RW, int RC, bool FAST>
static GxPipePlan plan_gx_pipe_kg(const Geom& g, const TileHint& hint, int kg_forced) {
    GxPipePlan p;
    GxPipeArgs& a = p.a;
    p.status = ADDER_OK;
    p.ks = KS; p.rw = RW; p.rc = RC; p.fast = FAST;
    a.g = g;
    const int sms = sm_count();
    const int threads_target = hint.threads > 0 ? hint.threads : 256;
    const int cgi_want = hint.cg > 0 ? hint.cg : (16 / RC > 0 ? 16 / RC : 1);
    a.CGI = ceil_div(g.Ci, RC) < cgi_want ? ceil_div(g.Ci, RC) : cgi_want;
    a.TCI = a.CGI * RC;
    a.TCIP = a.TCI + 4;
    const int spr_full = ceil_div(g.W, RW);
    const long long all_threads = (long long)g.N * g.H * spr_full * ceil_div(g.Ci, RC);
    int kg = 1;
    if (hint.ck > 0) kg = hint.ck;      // tuning: the chunk hint carries the group count for this kernel
    else if (kg_forced > 0) kg = kg_forced;
    else {
        while (kg < 4 && all_threads * kg < (long long)sms * 512 && g.Co >= 8 * kg) kg *= 2;
    }
    a.KG = kg;
    int segs_target = threads_target / (a.CGI * a.KG);
    if (segs_target < 8) segs_target = 8;
    a.SPR = spr_full <= segs_target ? spr_full : segs_target;
    int rows_target = segs_target / a.SPR;
    if (rows_target < 1) rows_target = 1;
    if (hint.th > 0) a.TH = hint.th < g.H ? hint.th : g.H;
    else a.TH = largest_divisor_le(g.H, rows_target);
    a.TI = 1;
    if (a.TH == g.H) {
        a.TI = rows_target / a.TH;
        if (a.TI > g.N) a.TI = g.N;
        if (a.TI < 1) a.TI = 1;
    }
    if (hint.ti > 0) a.TI = hint.ti;
    a.SEGS = a.TI * a.TH * a.SPR;
    const int group = round_up(a.CGI * a.SEGS, 32);
    p.threads = group * a.KG;
    if (p.threads > 256) { p.status = ADDER_ERR_INTERNAL; return p; }
    a.G_ROWS = a.TH + KS - 1;
    const int g_cols = a.SPR * RW + KS - 1;
    {
        const int rows = a.TI * a.TH, th = a.TH, g_rows = a.G_ROWS;
        a.PITCH = pick_pitch_vec(2 * g_cols, 32, [=](int l, int& row, int& col) {
            const int wsl = l / rows, ri = l % rows;
            row = (ri / th) * g_rows + (ri % th); col = wsl * RW * 2; });
    }
    PatchDims& pg = a.pdg;
    pg.TI = a.TI; pg.ROWS = a.G_ROWS; pg.COLS = g_cols; pg.PITCH = a.PITCH; pg.ROWS_PITCH = a.G_ROWS * a.PITCH;
    pg.d_cols = FastDiv(g_cols); pg.d_rows = FastDiv(a.G_ROWS);
    a.CH_STRIDE = a.TI * pg.ROWS_PITCH;
    a.g1_size = FAST ? a.CH_STRIDE / 2 : 0;
    // the unit's own x tile (no halo)
    PatchDims& px = a.pdx;
    a.XP = a.SPR * RW;
    px.CH = a.TCI; px.TI = a.TI; px.ROWS = a.TH; px.COLS = a.XP; px.PITCH = a.XP; px.ROWS_PITCH = a.TH * a.XP;
    px.d_cols = FastDiv(a.XP); px.d_rows = FastDiv(a.TH);
    a.XCH = a.TI * px.ROWS_PITCH;
    a.xs_stage = round_up(a.TCI * a.XCH, 4);
    a.d_xquads = FastDiv(a.XP >= 4 ? a.XP / 4 : 1);
    a.red_floats = a.KG > 1 ? (a.KG - 1) * RC * RW * group : 0;
    // output channels per chunk: a multiple of the group count; three stages within the budget.  The sums
    // of a multi-chunk unit go through per-thread totals in shared memory.
    const int budget_floats = (hint.smem_kb > 0 ? hint.smem_kb : 108) * 1024 / 4 - a.red_floats - a.g1_size;
    int cko = 16 > a.KG ? 16 : a.KG;
    if (cko > g.Co) cko = g.Co;
    const bool long_sum = (long long)g.Co * KS * KS > 1024;
    auto slots_for = [&](int c) { return ceil_div(g.Co, c) > 1 ? 2 : GX_STAGES; };   // units in flight in the ring
    auto need = [&](int c) {
        const int tot = (long_sum && ceil_div(g.Co, c) > 1) ? RC * RW * p.threads : 0;
        return GX_STAGES * (round_up(c * a.CH_STRIDE, 4) + round_up(c * KS * KS * a.TCIP, 4)) + slots_for(c) * a.xs_stage + tot;
    };
    while (cko > a.KG && need(cko) > budget_floats) --cko;
    cko = ceil_div(g.Co, ceil_div(g.Co, cko));
    if (a.KG > 1) cko = round_up(cko, a.KG);
    a.CKO = cko;
    pg.CH = cko;
    a.nchunks = ceil_div(g.Co, cko);
    a.two_level = (long_sum && a.nchunks > 1) ? 1 : 0;
    a.tot_floats = a.two_level ? RC * RW * p.threads : 0;
    a.x_slots = slots_for(cko);
    a.gs_stage = round_up(cko * a.CH_STRIDE, 4);
    a.ws_stage = round_up(cko * KS * KS * a.TCIP, 4);
    a.stage_floats = a.gs_stage + a.ws_stage;
    p.smem = (size_t)(GX_STAGES * a.stage_floats + a.x_slots * a.xs_stage + a.g1_size + a.tot_floats + a.red_floats) * sizeof(float);
    if (p.smem > 200 * 1024) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.tiles_h = ceil_div(g.H, a.TH);
    a.tiles_w = ceil_div(spr_full, a.SPR);
    const long long px_tiles = (long long)ceil_div(g.N, a.TI) * a.tiles_h * a.tiles_w;
    const long long units = px_tiles * ceil_div(g.Ci, a.TCI);
    if (units > 2147483647LL || units < 1) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.n_px_tiles = (int)px_tiles;
    a.n_units = (int)units;
    const long long slots = (long long)sms * gx_ctas_per_sm(p.smem, p.threads);
    p.grid = (int)(units < slots ? units : slots);
    a.d_tiles_h = FastDiv(a.tiles_h);
    a.d_tiles_w = FastDiv(a.tiles_w);
    a.d_px_tiles = FastDiv(a.n_px_tiles);
    a.d_nchunks = FastDiv(a.nchunks);
    a.d_group = FastDiv(group);
    a.d_segs = FastDiv(a.SEGS);
    a.d_rows = FastDiv(a.TI * a.TH);
    a.d_th = FastDiv(a.TH);
    a.d_tci9 = FastDiv(a.TCI * KS * KS);
    return p;
}

template <int KS, int RW, int RC, bool FAST>
static int launch_gx_pipe_t(const Geom& g, const float* gout, const float* x, const float* w, float* gx,
                            int accumulate, const TileHint& hint, cudaStream_t stream) {
    GxPipePlan p = plan_gx_pipe_t<KS, RW, RC, FAST>(g, hint);
    if (p.status != ADDER_OK) return p.status;
    p.a.gout = gout; p.a.x = x; p.a.w = w; p.a.gx = gx; p.a.accumulate = accumulate;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gx)) & 15) == 0;
    p.a.vec_io = (RW % 4 == 0 && g.W % 4 == 0 && aligned) ? 1 : 0;
    p.a.x_quads = (g.W % 4 == 0 && p.a.XP % 4 == 0 && aligned) ? 1 : 0;
    auto kern = adder_gx_pipe_kernel<KS, RW, RC, FAST>;
    const int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), p.smem);
    if (st != ADDER_OK) return st;
    kern<<<p.grid, p.threads, p.smem, stream>>>(p.a);
    return launched();
}

// Stride-1 layers whose rows are cut into 8- or 4-pixel segments and whose input channels come in fours.
bool gx_pipe_applicable(const Geom& g, const TileHint& hint) {
    if (hint.variant == 1) return false;        // tuning: force the non-persistent kernels
    if (g.stride != 1 || !(g.k == 3 || g.k == 1)) return false;
    if (hint.rw == 7 || ((g.W % 8 != 0) && (g.W % 7 == 0))) return false;
    return g.Ci % 4 == 0;
}

static void choose_gx_pipe_tile(const Geom& g, const TileHint& hint, int& rw, int& rc) {
    if (hint.rw > 0 && hint.rm > 0) { rw = hint.rw; rc = hint.rm; return; }
    rc = (g.Ci % 8 == 0) ? 8 : 4;
    rw = 4;
}

#define ADDER_GXP_DISPATCH(CALL)                                                            \
    if (g.k == 3) { ADDER_GXP_TILES(3, CALL) } else if (g.k == 1) { ADDER_GXP_TILES(1, CALL) }
#define ADDER_GXP_TILES(KS_, CALL)                                                          \
    if (rw == 4 && rc == 8) { if (fast) { CALL(KS_, 4, 8, true) } else { CALL(KS_, 4, 8, false) } }       \
    else if (rw == 8 && rc == 4) { if (fast) { CALL(KS_, 8, 4, true) } else { CALL(KS_, 8, 4, false) } }  \
    else if (rw == 4 && rc == 4) { if (fast) { CALL(KS_, 4, 4, true) } else { CALL(KS_, 4, 4, false) } }

int describe_gx_pipe(const Geom& g, int fast, const TileHint& hint, char* buf, size_t n) {
    int rw = 4, rc = 8;
    choose_gx_pipe_tile(g, hint, rw, rc);
    GxPipePlan p;
    p.status = ADDER_ERR_UNSUPPORTED;
#define ADDER_GXP_PLAN(KS_, RW_, RC_, FAST_) p = plan_gx_pipe_t<KS_, RW_, RC_, FAST_>(g, hint);
    ADDER_GXP_DISPATCH(ADDER_GXP_PLAN)
#undef ADDER_GXP_PLAN
    snprintf(buf, n,
             "gx persistent k=%d s=1 RW=%d RC=%d fast=%d segs/thread=1 CGI=%d KG=%d TCI=%d TI=%d TH=%d SPR=%d SEGS=%d CKO=%d "
             "chunks=%d rows=%d cols=%d pitch=%d stages=%d threads=%d smem=%zu units=%d grid=(%d,1) status=%d",
             p.ks, p.rw, p.rc, p.fast, p.a.CGI, p.a.KG, p.a.TCI, p.a.TI, p.a.TH, p.a.SPR, p.a.SEGS, p.a.CKO, p.a.nchunks,
             p.a.G_ROWS, p.a.pdg.COLS, p.a.PITCH, GX_STAGES, p.threads, p.smem, p.a.n_units, p.grid, p.status);
    return ADDER_OK;
}

int launch_gx_pipe(const Geom& g, const float* gout, const float* x, const float* w, float* gx, int fast,
                   int accumulate, const TileHint& hint, cudaStream_t stream) {
    int rw = 4, rc = 8;
    choose_gx_pipe_tile(g, hint, rw, rc);
#define ADDER_GXP_LAUNCH(KS_, RW_, RC_, FAST_) \
    return launch_gx_pipe_t<KS_, RW_, RC_, FAST_>(g, gout, x, w, gx, accumulate, hint, stream);
    ADDER_GXP_DISPATCH(ADDER_GXP_LAUNCH)
#undef ADDER_GXP_LAUNCH
    return ADDER_ERR_UNSUPPORTED;
}

}  // namespace adder
