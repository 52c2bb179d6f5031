// Weight gradient of the adder convolution on NCHW tensors (implicit im2col), with the reference's
// adaptive rescale fused behind it:
//   gw[co,ci,kh,kw] = sum_{n,ho,wo} (xpad[n,ci,ho*S+kh,wo*S+kw] - w[co,ci,kh,kw]) * g[n,co,ho,wo]
//   gw_scaled       = eta * sqrt(Co*Ci*k*k) * gw / max(||gw||_2, 1e-12)
// (CONV_BACKWARD's grad_w, adder_cuda/adder.cu:247,:267, followed by adder.py:78.)
//
// The sum is evaluated as  sum x*g  -  w * sum g : one fused multiply-add per (co,ci,kh,kw,pixel)
// in the main kernel; the second term needs only a per-channel sum of g and is applied in the
// finishing kernel.  Padding pixels carry x = 0, so they still contribute -w*g, as in the
// reference where F.unfold feeds zeros to the kernel.
//
// Main kernel.  A CTA owns an output tile of TM = CGO*RM output channels x TCI = CGC*RC input
// channels x all k*k taps, and one of `splits` contiguous ranges of pixel tiles.  A thread owns
// RM x RC x k*k accumulators; the PL threads that share an output group split the row segments of
// each pixel tile between them and are folded together with warp shuffles at the end.  Each CTA
// writes its partial sums to its own slice of the workspace: no atomics, fixed summation order.
// Finishing kernels.  (1) sum the slices in double precision, subtract w * sum g, write the
// unscaled gradient and per-block partial sums of squares; (2) one block adds those partials
// in a fixed order and derives the scale; (3) the scale is applied to the gradient.
#include "common.cuh"
#include "kernels.h"
#include "patch_fill.cuh"
#include <cstdio>

#ifndef GW_MIN_BLOCKS
#define GW_MIN_BLOCKS 2
#endif
namespace adder {

template <int KS, int S, int RW, int RM, int RC>
__global__ void __launch_bounds__(256, GW_MIN_BLOCKS) adder_gw_kernel(const GwArgs a) {
    constexpr int KK = KS * KS;
    constexpr int XW = (RW - 1) * S + KS;
    constexpr bool VEC = (RW % 4 == 0);      // segment starts are 16-byte aligned in both patches
    extern __shared__ __align__(16) float smem[];
    float* const Xs = smem;
    float* const Gs = smem + 2 * a.xs_stage;
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *a.ticket = 0u;   // for the finishing kernel

    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    // Pixel tiles are dealt out as evenly as they go: the first `tiles_rem` ranges hold one tile more.
    // Which CTA of a row takes which range is rotated from one output tile (blockIdx.y) to the next, so
    // that the CTAs that share an SM (linear CTA ids one wave apart) do not all hold a long range.
    const int split = (int)((blockIdx.x + (unsigned)a.splits - (blockIdx.y * (unsigned)a.tiles_rem) % (unsigned)a.splits) % (unsigned)a.splits);
    uint32_t ct_o, ct_c;
    a.d_ci_tiles.divmod(blockIdx.y, ct_o, ct_c);
    const int co0 = ct_o * a.TM, ci0 = ct_c * a.TCI;

    uint32_t og, pl, cgc, cgo;
    a.d_pl.divmod(tid, og, pl);
    a.d_cgo.divmod(og, cgc, cgo);
    const bool active = (int)cgc < a.CGC;
    const bool do_gsum = active && cgc == 0 && ct_c == 0;

    float acc[RM][RC][KK];
    float gsum[RM];
#pragma unroll
    for (int m = 0; m < RM; ++m) {
        gsum[m] = 0.f;
#pragma unroll
        for (int c = 0; c < RC; ++c)
#pragma unroll
            for (int t = 0; t < KK; ++t) acc[m][c][t] = 0.f;
    }

    const int t_begin = split * a.tiles_per_split + min(split, a.tiles_rem);
    const int t_end = t_begin + a.tiles_per_split + (split < a.tiles_rem ? 1 : 0);

    auto fill = [&](int tile, int stage) {
        uint32_t tn, th, tw, tnh;
        a.d_tiles_w.divmod(tile, tnh, tw);
        a.d_tiles_h.divmod(tnh, tn, th);
        const int n0 = tn * a.TI, ho0 = th * a.TH, wo0 = tw * (a.SPR * RW);
        fill_patch(Xs + stage * a.xs_stage, a.x, a.pdx, n0, ci0, ho0 * S - a.g.pad, wo0 * S - a.g.pad, a.g.N,
                   a.g.Ci, a.g.H, a.g.W, tid, nthreads);
        if (a.g_quads)
            fill_patch_quads(Gs + stage * a.gs_stage, a.gout, a.pdg, a.d_gquads, n0, co0, ho0, wo0, a.g.N, a.g.Co, a.g.Ho,
                             a.g.Wo, tid, nthreads);
        else
            fill_patch(Gs + stage * a.gs_stage, a.gout, a.pdg, n0, co0, ho0, wo0, a.g.N, a.g.Co, a.g.Ho, a.g.Wo, tid,
                       nthreads);
    };

    if (t_begin < t_end) {
        fill(t_begin, 0);
        cp_async_commit();
    }
    for (int t = t_begin; t < t_end; ++t) {
        const int stage = (t - t_begin) & 1;
        if (t + 1 < t_end) {
            fill(t + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (active) {
            const float* xs = Xs + stage * a.xs_stage + (cgc * RC) * a.XCH_STRIDE;
            const float* gs = Gs + stage * a.gs_stage + (cgo * RM) * a.GCH_STRIDE;
#pragma unroll 1
            for (int seg = pl; seg < a.SEGS; seg += a.PL) {
                uint32_t t2, ws, img, hr;
                a.d_spr.divmod(seg, t2, ws);
                a.d_th.divmod(t2, img, hr);
                const float* gp = gs + (img * a.TH + hr) * a.pdg.PITCH + ws * RW;
                float gv[RM][RW];
#pragma unroll
                for (int m = 0; m < RM; ++m) {
                    if (RW % 4 == 0) {
#pragma unroll
                        for (int j = 0; j < RW; j += 4) {
                            const float4 v = *reinterpret_cast<const float4*>(gp + m * a.GCH_STRIDE + j);
                            gv[m][j] = v.x; gv[m][j + 1] = v.y; gv[m][j + 2] = v.z; gv[m][j + 3] = v.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < RW; ++j) gv[m][j] = gp[m * a.GCH_STRIDE + j];
                    }
                }
                if (do_gsum) {
#pragma unroll
                    for (int m = 0; m < RM; ++m) {
                        float s = 0.f;
#pragma unroll
                        for (int j = 0; j < RW; ++j) s += gv[m][j];
                        gsum[m] += s;
                    }
                }
                const float* xp = xs + (img * a.pdx.ROWS + hr * S) * a.pdx.PITCH + ws * (RW * S);
#pragma unroll
                for (int c = 0; c < RC; ++c) {
#pragma unroll
                    for (int kh = 0; kh < KS; ++kh) {
                        const float* xr = xp + c * a.XCH_STRIDE + kh * a.pdx.PITCH;
                        float xv[XW];
                        load_run<XW, VEC>(xv, xr);
#pragma unroll
                        for (int kw = 0; kw < KS; ++kw)
#pragma unroll
                            for (int m = 0; m < RM; ++m)
#pragma unroll
                                for (int j = 0; j < RW; ++j)
                                    acc[m][c][kh * KS + kw] = fmaf(xv[j * S + kw], gv[m][j], acc[m][c][kh * KS + kw]);
                    }
                }
            }
        }
        __syncthreads();
    }

    // fold the PL pixel lanes (PL is a power of two <= 32 and lanes of a group are adjacent)
    for (int off = a.PL >> 1; off > 0; off >>= 1) {
#pragma unroll
        for (int m = 0; m < RM; ++m) {
            gsum[m] += __shfl_xor_sync(0xffffffffu, gsum[m], off);
#pragma unroll
            for (int c = 0; c < RC; ++c)
#pragma unroll
                for (int t = 0; t < KK; ++t) acc[m][c][t] += __shfl_xor_sync(0xffffffffu, acc[m][c][t], off);
        }
    }
    if (!active || pl != 0) return;
    const int CoK = a.g.Co * a.g.Ci * KK;
    float* part = a.part + (size_t)split * CoK;
#pragma unroll
    for (int m = 0; m < RM; ++m) {
        const int co = co0 + cgo * RM + m;
        if (co >= a.g.Co) break;
        if (do_gsum) a.gsum_part[(size_t)split * a.g.Co + co] = gsum[m];
#pragma unroll
        for (int c = 0; c < RC; ++c) {
            const int ci = ci0 + cgc * RC + c;
            if (ci >= a.g.Ci) break;
#pragma unroll
            for (int t = 0; t < KK; ++t) part[(size_t)(co * a.g.Ci + ci) * KK + t] = acc[m][c][t];
        }
    }
}

constexpr int FIN_THREADS = 256;
constexpr int FIN_OUT = 8;                        // gradient elements per reduce block
constexpr int FIN_LANES = FIN_THREADS / FIN_OUT;  // threads that share one element and split the slices
constexpr int FUSED_FINISH_MAX = 1 << 17;         // gradients up to this many elements finish in one kernel

// gw[i] = sum_s part[s][i] - w[i] * sum_s gsum_part[s][co(i)], plus the block's partial of sum gw^2, in double
// precision and in slice order, so the result does not depend on scheduling.  This is the form for large
// gradients (more elements than FUSED_FINISH_MAX), whose slices are few and long: one thread per element, so a
// warp reads 128 consecutive bytes of every slice.  (Eight elements per block with the block's lanes spread
// over the slices, as the fused kernel below does for small gradients, took 57 us for the 14 slices of a
// 1024->256 1x1 layer: 32-byte pieces, most lanes idle.)  The block's 256 squares are added in a fixed order.
__global__ void __launch_bounds__(FIN_THREADS) adder_gw_reduce_flat_kernel(const GwFinishArgs a) {
    __shared__ double s_sq[FIN_THREADS];
    const int i = blockIdx.x * FIN_THREADS + threadIdx.x;
    double v2 = 0.0;
    if (i < a.CoK) {
        const int co = i / a.K;
        const float* p = a.part + i;
        const float* q = a.gsum_part + co;
        double s = 0.0, gs = 0.0;
#pragma unroll 8
        for (int sp = 0; sp < a.splits; ++sp) {
            s += (double)__ldcg(p + (size_t)sp * a.CoK);
            gs += (double)__ldg(q + (size_t)sp * a.Co);
        }
        const float vf = (float)(s - (double)a.w[i] * gs);
        if (a.accumulate) a.gw[i] += vf; else a.gw[i] = vf;
        v2 = (double)vf * (double)vf;
    }
    s_sq[threadIdx.x] = v2;
    __syncthreads();
    for (int off = FIN_THREADS / 2; off > 0; off >>= 1) {
        if ((int)threadIdx.x < off) s_sq[threadIdx.x] += s_sq[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) a.norm_part[blockIdx.x] = (float)s_sq[0];
}

// One block: adds the per-block partial sums of squares in a fixed order and writes
// scale = eta * sqrt(numel) / max(||gw||, 1e-12) (and the norm itself, if asked for).
__global__ void __launch_bounds__(1024) adder_gw_norm_kernel(const GwFinishArgs a, int nblocks, float* scale_out) {
    __shared__ double red[1024];
    double t = 0.0;
    for (int k = threadIdx.x; k < nblocks; k += 1024) t += (double)a.norm_part[k];
    red[threadIdx.x] = t;
    __syncthreads();
    for (int off = 512; off > 0; off >>= 1) {
        if ((int)threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const float nrm = (float)sqrt(red[0]);
        if (a.out_norm != nullptr) *a.out_norm = nrm;
        *scale_out = a.eta * sqrtf((float)a.CoK) / fmaxf(nrm, 1e-12f);
    }
}

// Small gradients: one kernel does all three finishing steps.  Every block reduces its 32 elements
// and publishes its partial sum of squares; the block that draws the last ticket adds the partials
// in index order (so the result does not depend on which block that is), derives the scale and
// applies it to the whole gradient.  The ticket counter is zeroed by the main kernel of the same call.
__global__ void __launch_bounds__(FIN_THREADS) adder_gw_finish_kernel(const GwFinishArgs a, int nblocks,
                                                                      unsigned int* ticket) {
    __shared__ double s_sum[FIN_LANES][FIN_OUT];
    __shared__ double s_gs[FIN_LANES][FIN_OUT];
    __shared__ double s_sq[FIN_THREADS];
    __shared__ bool s_last;
    const int o = threadIdx.x & (FIN_OUT - 1);
    const int lane = threadIdx.x / FIN_OUT;
    const int i = blockIdx.x * FIN_OUT + o;
    double s = 0.0, gs = 0.0;
    if (i < a.CoK) {
        const int co = i / a.K;
        const float* p = a.part + i;
        const float* q = a.gsum_part + co;
#pragma unroll 4
        for (int sp = lane; sp < a.splits; sp += FIN_LANES) {
            s += (double)p[(size_t)sp * a.CoK];
            gs += (double)q[(size_t)sp * a.Co];
        }
    }
    s_sum[lane][o] = s;
    s_gs[lane][o] = gs;
    __syncthreads();
    double v2 = 0.0;
    if (lane == 0 && i < a.CoK) {
        double t = 0.0, g = 0.0;
#pragma unroll
        for (int l = 0; l < FIN_LANES; ++l) { t += s_sum[l][o]; g += s_gs[l][o]; }
        const float vf = (float)(t - (double)a.w[i] * g);
        if (a.accumulate) a.gw[i] += vf; else a.gw[i] = vf;
        v2 = (double)vf * (double)vf;
    }
    s_sq[threadIdx.x] = (lane == 0) ? v2 : 0.0;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int k = 0; k < FIN_OUT; ++k) t += s_sq[k];
        a.norm_part[blockIdx.x] = (float)t;
        __threadfence();
        s_last = (atomicAdd(ticket, 1u) == (unsigned)(nblocks - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    double t = 0.0;
    for (int k = threadIdx.x; k < nblocks; k += FIN_THREADS) t += (double)__ldcg(a.norm_part + k);
    s_sq[threadIdx.x] = t;
    __syncthreads();
    for (int off = FIN_THREADS / 2; off > 0; off >>= 1) {
        if ((int)threadIdx.x < off) s_sq[threadIdx.x] += s_sq[threadIdx.x + off];
        __syncthreads();
    }
    const float nrm = (float)sqrt(s_sq[0]);
    if (threadIdx.x == 0 && a.out_norm != nullptr) *a.out_norm = nrm;
    if (a.eta > 0.f) {
        const float sc = a.eta * sqrtf((float)a.CoK) / fmaxf(nrm, 1e-12f);
        for (int k = threadIdx.x; k < a.CoK; k += FIN_THREADS) a.gw[k] = __ldcg(a.gw + k) * sc;
    }
}

__global__ void __launch_bounds__(FIN_THREADS) adder_gw_scale_kernel(float* gw, int n, const float* scale) {
    const float sc = *scale;
    const int i = blockIdx.x * FIN_THREADS + threadIdx.x;
    if (i < n) gw[i] *= sc;
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------

struct GwPlan {
    GwArgs a;
    int threads;
    size_t smem;
    int fin_blocks;
    int status;
    bool use_1x1 = false;   // 1x1 stride-1 layers with enough channels take the GEMM-style kernel
    bool use_pointwise = false;   // 1x1 stride-2 layers with few channels: adder_pointwise.cu
    bool use_pipe = false;        // 3x3 layers with channels in sixteens: adder_bwd_weight_pipe.cu
    bool use_tma = false;         // ... and stride 1, rows of 8-pixel segments: adder_bwd_weight_tma.cu
};

template <int KS, int S, int RW, int RM, int RC>
static GwPlan plan_gw_t(const Geom& g, const TileHint& hint) {
    GwPlan p;
    GwArgs& a = p.a;
    p.status = ADDER_OK;
    a.g = g;
    // output tile
    const int cgo_max = hint.cg > 0 ? hint.cg : (KS == 1 ? 8 : 8);
    a.CGO = ceil_div(g.Co, RM) < cgo_max ? ceil_div(g.Co, RM) : cgo_max;
    const int cgc_max = 16 / RC < 8 ? 8 : 16 / RC;
    a.CGC = ceil_div(g.Ci, RC) < cgc_max ? ceil_div(g.Ci, RC) : cgc_max;
    a.TM = a.CGO * RM;
    a.TCI = a.CGC * RC;
    const int threads_target = hint.threads > 0 ? hint.threads : 256;
    int pl = threads_target / (a.CGO * a.CGC);
    int pl2 = 1;
    while (pl2 * 2 <= pl && pl2 < 32) pl2 *= 2;
    a.PL = pl2;
    p.threads = round_up(a.CGO * a.CGC * a.PL, 32);
    if (p.threads > 256) { p.status = ADDER_ERR_INTERNAL; return p; }
    // pixel tile: aim at a few segments per pixel lane, shrinking until both stages fit in shared memory
    const int budget_bytes = (hint.smem_kb > 0 ? hint.smem_kb : 100) * 1024;
    const int spr_full = ceil_div(g.Wo, RW);
    int segs_target = a.PL * (KS == 1 ? 16 : 4);     // a 1x1 layer has 9x less work per pixel: larger pixel tiles
    if (segs_target < 16) segs_target = 16;
    PatchDims& px = a.pdx;
    PatchDims& pg = a.pdg;
    for (;; segs_target = segs_target / 2) {
        if (segs_target < 1) segs_target = 1;
        a.SPR = spr_full <= segs_target ? spr_full : segs_target;
        int rows_target = segs_target / a.SPR;
        if (rows_target < 1) rows_target = 1;
        if (hint.th > 0) {
            a.TH = hint.th < g.Ho ? hint.th : g.Ho;
        } else {
            const int d = largest_divisor_le(g.Ho, rows_target);
            a.TH = (2 * d > rows_target || d == g.Ho) ? d : (rows_target < g.Ho ? rows_target : g.Ho);
        }
        a.TI = 1;
        if (a.TH == g.Ho) {
            a.TI = rows_target / a.TH;
            if (a.TI > g.N) a.TI = g.N;
            if (a.TI < 1) a.TI = 1;
        }
        if (hint.ti > 0) a.TI = hint.ti;
        a.SEGS = a.TI * a.TH * a.SPR;
        px.CH = a.TCI; px.TI = a.TI;
        px.ROWS = (a.TH - 1) * S + KS;
        px.COLS = (a.SPR * RW - 1) * S + KS;
        {
            const int spr = a.SPR, th = a.TH, rows = px.ROWS, plv = a.PL;
            if (RW % 4 == 0)
                px.PITCH = pick_pitch_vec(px.COLS, 32, [=](int l, int& row, int& col) {
                    const int seg = l % plv, ws = seg % spr, t2 = seg / spr;
                    row = (t2 / th) * rows + (t2 % th) * S; col = ws * RW * S; });
            else
                px.PITCH = px.COLS | 1;
        }
        px.ROWS_PITCH = px.ROWS * px.PITCH;
        a.XCH_STRIDE = a.TI * px.ROWS_PITCH;
        pg.CH = a.TM; pg.TI = a.TI;
        pg.ROWS = a.TH;
        pg.COLS = a.SPR * RW;
        {
            const int spr = a.SPR, th = a.TH, plv = a.PL;
            if (RW % 4 == 0)
                pg.PITCH = pick_pitch_vec(pg.COLS, 32, [=](int l, int& row, int& col) {
                    const int seg = l % plv, ws = seg % spr, t2 = seg / spr;
                    row = (t2 / th) * th + (t2 % th); col = ws * RW; });
            else
                pg.PITCH = round_up(pg.COLS, 4) + 4;
        }
        pg.ROWS_PITCH = pg.ROWS * pg.PITCH;
        a.GCH_STRIDE = a.TI * pg.ROWS_PITCH;
        a.xs_stage = round_up(a.TCI * a.XCH_STRIDE, 4);
        a.gs_stage = round_up(a.TM * a.GCH_STRIDE, 4);
        p.smem = (size_t)2 * (a.xs_stage + a.gs_stage) * sizeof(float);
        if (p.smem <= (size_t)budget_bytes || segs_target == 1) break;
    }
    if (p.smem > 200 * 1024) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.tiles_h = ceil_div(g.Ho, a.TH);
    a.tiles_w = ceil_div(spr_full, a.SPR);
    const long long tiles_total = (long long)ceil_div(g.N, a.TI) * a.tiles_h * a.tiles_w;
    if (tiles_total > 2147483647LL) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.tiles_total = (int)tiles_total;
    a.n_ci_tiles = ceil_div(g.Ci, a.TCI);
    const int out_tiles = ceil_div(g.Co, a.TM) * a.n_ci_tiles;
    if (out_tiles > 65535) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    const int target_ctas = 2 * sm_count();
    int splits = ceil_div(target_ctas, out_tiles);
    if (splits > a.tiles_total) splits = a.tiles_total;
    if (splits < 1) splits = 1;
    a.splits = splits;
    a.tiles_per_split = a.tiles_total / splits;      // the first tiles_rem ranges hold one more
    a.tiles_rem = a.tiles_total % splits;
    px.d_cols = FastDiv(px.COLS); px.d_rows = FastDiv(px.ROWS);
    pg.d_cols = FastDiv(pg.COLS); pg.d_rows = FastDiv(pg.ROWS);
    // the g tile has no halo: 16-byte copies when its rows start on 16-byte boundaries in both memories
    // (the pointer's alignment is checked at launch)
    a.g_quads = (pg.COLS % 4 == 0 && pg.PITCH % 4 == 0 && g.Wo % 4 == 0 && (a.SPR * RW) % 4 == 0 &&
                 (a.TI * pg.ROWS_PITCH) % 4 == 0) ? 1 : 0;
    a.d_gquads = FastDiv(pg.COLS >= 4 ? pg.COLS / 4 : 1);
    a.d_tiles_h = FastDiv(a.tiles_h);
    a.d_tiles_w = FastDiv(a.tiles_w);
    a.d_spr = FastDiv(a.SPR);
    a.d_th = FastDiv(a.TH);
    a.d_pl = FastDiv(a.PL);
    a.d_cgo = FastDiv(a.CGO);
    a.d_ci_tiles = FastDiv(a.n_ci_tiles);
    p.fin_blocks = ceil_div(g.Co * g.Ci * KS * KS, FIN_OUT);
    return p;
}

static GwPlan plan_gw_generic(const Geom& g, const TileHint& hint);

static GwPlan plan_gw(const Geom& g, const TileHint& hint) {
    GwPlan p = plan_gw_generic(g, hint);
    if (p.status == ADDER_OK && gw_pipe_applicable(g, hint)) {
        const int sp = gw_pipe_splits(g, hint);
        if (sp > 0) {
            p.use_pipe = true;
            p.a.splits = sp;
        }
    }
    if (p.status == ADDER_OK && gw_tma_applicable(g, hint)) {
        const int sp = gw_tma_splits(g, hint);
        if (sp > 0) {
            p.use_tma = true;
            p.use_pipe = false;
            p.a.splits = sp;
        }
    }
    if (p.status == ADDER_OK && gw1x1_applicable(g) && hint.variant == 0) {     // variant 1 asks for the tiled kernel
        p.use_1x1 = true;
        p.a.splits = gw1x1_splits(g);
    }
    if (p.status == ADDER_OK && pointwise_applicable(g) && hint.is_default()) {
        p.use_pointwise = true;
        p.a.splits = pointwise_gw_splits(g);
    }
    return p;
}

static GwPlan plan_gw_generic(const Geom& g, const TileHint& hint) {
    const bool rw7 = (g.Wo % 8 != 0) && (g.Wo % 7 == 0);
    if (g.k == 3 && g.stride == 1) return rw7 ? plan_gw_t<3, 1, 7, 4, 2>(g, hint) : plan_gw_t<3, 1, 8, 4, 2>(g, hint);
    if (g.k == 3 && g.stride == 2) return rw7 ? plan_gw_t<3, 2, 7, 4, 2>(g, hint) : plan_gw_t<3, 2, 8, 4, 2>(g, hint);
    if (g.k == 1 && g.stride == 1) return rw7 ? plan_gw_t<1, 1, 7, 8, 4>(g, hint) : plan_gw_t<1, 1, 8, 8, 4>(g, hint);
    if (g.k == 1 && g.stride == 2) return rw7 ? plan_gw_t<1, 2, 7, 8, 4>(g, hint) : plan_gw_t<1, 2, 8, 8, 4>(g, hint);
    GwPlan p;
    p.status = ADDER_ERR_UNSUPPORTED;
    return p;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int describe_gw(const Geom& g, const TileHint& hint, char* buf, size_t n) {
    const GwPlan p = plan_gw(g, hint);
    if (p.status == ADDER_OK && p.use_tma) return describe_gw_tma(g, hint, buf, n);
    if (p.status == ADDER_OK && p.use_pipe) return describe_gw_pipe(g, hint, buf, n);
    if (p.status == ADDER_ERR_UNSUPPORTED && !((g.k == 1 || g.k == 3) && (g.stride == 1 || g.stride == 2))) return p.status;
    const GwArgs& a = p.a;
    snprintf(buf, n,
             "gw k=%d s=%d CGO=%d CGC=%d TM=%d TCI=%d PL=%d TI=%d TH=%d SPR=%d SEGS=%d xrows=%d xcols=%d xpitch=%d gpitch=%d "
             "threads=%d smem=%zu tiles=%d splits=%d tiles_per_split=%d+%d/%d out_tiles=%d fin_blocks=%d gemm1x1=%d pointwise=%d status=%d",
             g.k, g.stride, a.CGO, a.CGC, a.TM, a.TCI, a.PL, a.TI, a.TH, a.SPR, a.SEGS, a.pdx.ROWS, a.pdx.COLS, a.pdx.PITCH,
             a.pdg.PITCH, p.threads, p.smem, a.tiles_total, a.splits, a.tiles_per_split, a.tiles_rem, a.splits,
             ceil_div(g.Co, a.TM) * a.n_ci_tiles, p.fin_blocks, (int)p.use_1x1, (int)p.use_pointwise, p.status);
    return ADDER_OK;
}

size_t gw_workspace_bytes(const Geom& g, const TileHint& hint) {
    const GwPlan p = plan_gw(g, hint);
    if (p.status != ADDER_OK) return 0;
    const size_t CoK = (size_t)g.Co * g.Ci * g.k * g.k;
    size_t floats = align_up((size_t)p.a.splits * CoK, 64) + align_up((size_t)p.a.splits * g.Co, 64) +
                    align_up((size_t)p.fin_blocks + 2, 64);
    return floats * sizeof(float);
}

template <int KS, int S, int RW, int RM, int RC>
static int launch_main_t(const GwPlan& p, cudaStream_t stream) {
    auto kern = adder_gw_kernel<KS, S, RW, RM, RC>;
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), p.smem) != ADDER_OK) return ADDER_ERR_CUDA;
    const int out_tiles = ceil_div(p.a.g.Co, p.a.TM) * p.a.n_ci_tiles;
    kern<<<dim3((unsigned)p.a.splits, (unsigned)out_tiles), p.threads, p.smem, stream>>>(p.a);
    return launched();
}

int launch_gw(const Geom& g, const float* gout, const float* x, const float* w, float* gw, float eta,
              float* out_norm, int accumulate, void* workspace, size_t workspace_bytes, const TileHint& hint,
              cudaStream_t stream) {
    GwPlan p = plan_gw(g, hint);
    if (p.status != ADDER_OK) return p.status;
    const size_t need = gw_workspace_bytes(g, hint);
    if (workspace == nullptr || workspace_bytes < need) return ADDER_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return ADDER_ERR_ALIGNMENT;
    const size_t CoK = (size_t)g.Co * g.Ci * g.k * g.k;
    float* ws = static_cast<float*>(workspace);
    p.a.gout = gout; p.a.x = x;
    if ((reinterpret_cast<uintptr_t>(gout) & 15) != 0) p.a.g_quads = 0;
    p.a.part = ws;
    p.a.gsum_part = ws + align_up((size_t)p.a.splits * CoK, 64);
    float* norm_part = p.a.gsum_part + align_up((size_t)p.a.splits * g.Co, 64);
    unsigned int* ticket = reinterpret_cast<unsigned int*>(norm_part + p.fin_blocks + 1);
    p.a.ticket = ticket;

    const bool rw7 = (g.Wo % 8 != 0) && (g.Wo % 7 == 0);
    int st = ADDER_ERR_UNSUPPORTED;
    if (p.use_tma) {
        st = launch_gw_tma(g, gout, x, p.a.part, p.a.gsum_part, ticket, p.a.splits, hint, stream);
        if (st == ADDER_ERR_ALIGNMENT) {
            // no tensor map for these pointers (not 16-byte aligned): the cp.async kernel, same number of slices
            TileHint h2 = hint;
            h2.ti = p.a.splits;
            st = launch_gw_pipe(g, gout, x, p.a.part, p.a.gsum_part, ticket, p.a.splits, h2, stream);
        }
    }
    else if (p.use_pipe) st = launch_gw_pipe(g, gout, x, p.a.part, p.a.gsum_part, ticket, p.a.splits, hint, stream);
    else if (p.use_pointwise) st = launch_pointwise_gw(g, gout, x, p.a.part, p.a.gsum_part, ticket, p.a.splits, stream);
    else if (p.use_1x1) st = launch_gw1x1(g, gout, x, p.a.part, p.a.gsum_part, ticket, p.a.splits, stream);
    else if (g.k == 3 && g.stride == 1) st = rw7 ? launch_main_t<3, 1, 7, 4, 2>(p, stream) : launch_main_t<3, 1, 8, 4, 2>(p, stream);
    else if (g.k == 3 && g.stride == 2) st = rw7 ? launch_main_t<3, 2, 7, 4, 2>(p, stream) : launch_main_t<3, 2, 8, 4, 2>(p, stream);
    else if (g.k == 1 && g.stride == 1) st = rw7 ? launch_main_t<1, 1, 7, 8, 4>(p, stream) : launch_main_t<1, 1, 8, 8, 4>(p, stream);
    else if (g.k == 1 && g.stride == 2) st = rw7 ? launch_main_t<1, 2, 7, 8, 4>(p, stream) : launch_main_t<1, 2, 8, 8, 4>(p, stream);
    if (st != ADDER_OK) return st;

    GwFinishArgs f;
    f.part = p.a.part; f.gsum_part = p.a.gsum_part; f.w = w; f.gw = gw; f.norm_part = norm_part;
    f.out_norm = out_norm; f.CoK = (int)CoK; f.K = g.Ci * g.k * g.k; f.Co = g.Co; f.splits = p.a.splits;
    f.accumulate = accumulate; f.eta = eta;
    const bool need_norm = eta > 0.f || out_norm != nullptr;
    if (need_norm && CoK <= (size_t)FUSED_FINISH_MAX) {
        adder_gw_finish_kernel<<<p.fin_blocks, FIN_THREADS, 0, stream>>>(f, p.fin_blocks, ticket);
        return launched();
    }
    const int flat_blocks = ceil_div((int)CoK, FIN_THREADS);      // <= fin_blocks: the norm partials fit their array
    adder_gw_reduce_flat_kernel<<<flat_blocks, FIN_THREADS, 0, stream>>>(f);
    if (launched() != ADDER_OK) return ADDER_ERR_CUDA;
    if (need_norm) {
        float* scale = norm_part + p.fin_blocks;
        adder_gw_norm_kernel<<<1, 1024, 0, stream>>>(f, flat_blocks, scale);
        if (launched() != ADDER_OK) return ADDER_ERR_CUDA;
        if (eta > 0.f) {
            adder_gw_scale_kernel<<<ceil_div((int)CoK, FIN_THREADS), FIN_THREADS, 0, stream>>>(gw, (int)CoK, scale);
            if (launched() != ADDER_OK) return ADDER_ERR_CUDA;
        }
    }
    return ADDER_OK;
}

}  // namespace adder
