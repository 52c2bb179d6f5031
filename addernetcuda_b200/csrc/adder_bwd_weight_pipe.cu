// Weight gradient of the adder convolution, warp-tile form (main kernel only; the finishing kernels of
// adder_bwd_weight.cu follow it unchanged):
//   part[split][co,ci,kh,kw] = sum over the split's pixels of xpad[n,ci,ho*S+kh,wo*S+kw] * g[n,co,ho,wo]
//   gsum_part[split][co]     = sum over the split's pixels of g[n,co,ho,wo]
// so that gw = sum_split part - w * sum_split gsum_part (CONV_BACKWARD's grad_w, adder_cuda/adder.cu:247,:267).
//
// Differences from adder_gw_kernel (adder_bwd_weight.cu), which keeps the layers this one does not cover:
//  * A warp owns a 16 x 16 x k*k block of the gradient: lane (cgo, cgc) holds output channels cgo + 4m
//    (m < 4) and input channels cgc + 8c (c < 2), 72 accumulators for a 3x3 layer.  All lanes of a warp walk
//    the SAME pixels, so every shared-memory load is a broadcast (4 distinct addresses for g, 8 for x), the
//    lanes never have to be folded with shuffles, and the index arithmetic of a segment is warp-uniform.
//    Channel planes are padded to an odd number of 16-byte words, which puts the distinct addresses of one
//    load into distinct bank groups.
//  * A CTA is OT such warp blocks (a CO_T x CI_T block of the gradient) times PS pixel shares: the warps
//    of one block split the rows (PR ways) and the row segments (PW ways) of every item between them and
//    are folded through shared memory once, at the end of the kernel.
//  * Work is dealt out by ROWS, not by tiles: the N*Ho output rows are cut into `splits` contiguous ranges
//    that differ by at most one row quantum, and a CTA walks its range in items of up to TH rows of one
//    image through a double-buffered cp.async stage.  Every CTA therefore ends at (almost) the same time,
//    whatever the plane size.
//  * The per-channel sums of g are taken by all threads from the staged tile (a strip per thread), not by
//    one warp inside the multiply-add loop.
#include "common.cuh"
#include "kernels.h"
#include "patch_fill.cuh"
#include <cstdio>

namespace adder {

constexpr int GWP_WARPS = 8;
constexpr int GWP_LP = 33;       // lane pitch of the end-of-kernel exchange buffer (conflict-free transposed reads)

struct GwPipeArgs {
    Geom g;
    const float* gout;
    const float* x;
    float* part;
    float* gsum_part;
    unsigned int* ticket;
    PatchDims pdx;       // haloed input patch of one item: [CI_T][XROWS][XP], channel stride XCH
    PatchDims pdg;       // tile of g of one item:          [CO_T][TH][GP],    channel stride GCH
    int TH, SPR, PR, PW, OT, OTi, CO_T, CI_T, XCH, GCH, XP, GP;
    int xs_stage, stage_floats, splits, n_ci_blocks, g_quads, tpc, row_quantum;
    long long rows_total;
    FastDiv d_ho, d_pw, d_ot, d_oti, d_ci_blocks, d_gquads, d_tpc, d_kk_ci;
};

template <int KS, int S, int RW>
__global__ void __launch_bounds__(GWP_WARPS * 32, 2) adder_gw_pipe_kernel(const GwPipeArgs a) {
    constexpr int KK = KS * KS;
    constexpr int XW = (RW - 1) * S + KS;
    constexpr int RM = 4, RC = 2;
    constexpr int NE = RM * RC * KK;             // accumulators per lane
    extern __shared__ __align__(16) float smem[];
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *a.ticket = 0u;   // for the finishing kernel

    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int cgo = lane & 3, cgc = lane >> 2;
    uint32_t ps, ot, oto, oti, pr, pw, cob, cib;
    a.d_ot.divmod(warp, ps, ot);
    a.d_oti.divmod(ot, oto, oti);
    a.d_pw.divmod(ps, pr, pw);
    a.d_ci_blocks.divmod(blockIdx.y, cob, cib);
    const int co0 = cob * a.CO_T, ci0 = cib * a.CI_T;
    const int split = blockIdx.x;
    const bool do_gsum = cib == 0;

    // this CTA's range of output rows in the flattened (image, row) space, in whole row quanta
    const long long quanta = (a.rows_total + a.row_quantum - 1) / a.row_quantum;
    long long r_lo = quanta * split / a.splits * a.row_quantum;
    long long r_hi = quanta * (split + 1) / a.splits * a.row_quantum;
    if (r_hi > a.rows_total) r_hi = a.rows_total;
    if (r_lo > a.rows_total) r_lo = a.rows_total;
    const int R0 = (int)r_lo, R1 = (int)r_hi;
    const int Ho = a.g.Ho;

    auto item_rows = [&](int cur, int& n, int& r0) {
        uint32_t q, r;
        a.d_ho.divmod(cur, q, r);
        n = q; r0 = r;
        int nr = Ho - r0;
        if (nr > a.TH) nr = a.TH;
        if (nr > R1 - cur) nr = R1 - cur;
        return nr;
    };
    auto fill = [&](int cur, int stage) {
        int n, r0;
        (void)item_rows(cur, n, r0);
        float* xs = smem + stage * a.stage_floats;
        float* gs = xs + a.xs_stage;
        fill_patch<false>(xs, a.x, a.pdx, n, ci0, r0 * S - a.g.pad, -a.g.pad, a.g.N, a.g.Ci, a.g.H, a.g.W, tid, nthreads);
        if (a.g_quads)
            fill_patch_quads(gs, a.gout, a.pdg, a.d_gquads, n, co0, r0, 0, a.g.N, a.g.Co, a.g.Ho, a.g.Wo, tid, nthreads);
        else
            fill_patch<false>(gs, a.gout, a.pdg, n, co0, r0, 0, a.g.N, a.g.Co, a.g.Ho, a.g.Wo, tid, nthreads);
    };

    float acc[RM][RC][KK];
#pragma unroll
    for (int m = 0; m < RM; ++m)
#pragma unroll
        for (int c = 0; c < RC; ++c)
#pragma unroll
            for (int t = 0; t < KK; ++t) acc[m][c][t] = 0.f;
    float gstrip = 0.f;                              // this thread's strip of sum(g) of channel tid / tpc
    uint32_t gs_ch, gs_lane;
    a.d_tpc.divmod(tid, gs_ch, gs_lane);

    int cur_f = R0, cur_c = R0, stage = 0;
    if (cur_f < R1) {
        int n, r0;
        fill(cur_f, 0);
        cur_f += item_rows(cur_f, n, r0);
    }
    cp_async_commit();
    while (cur_c < R1) {
        cp_async_wait<0>();
        __syncthreads();          // this item has landed for everyone, and everyone is done with the previous one
        if (cur_f < R1) {
            int n, r0;
            fill(cur_f, stage ^ 1);
            cur_f += item_rows(cur_f, n, r0);
        }
        cp_async_commit();
        int n_img, r0_img;
        const int nr = item_rows(cur_c, n_img, r0_img);
        const float* Xs = smem + stage * a.stage_floats;
        const float* Gs = Xs + a.xs_stage;
        {
            const float* xs = Xs + (oti * 16 + cgc) * a.XCH + pw * (RW * S);
            const float* gs = Gs + (oto * 16 + cgo) * a.GCH + pw * RW;
#pragma unroll 1
            for (int r = pr; r < nr; r += a.PR) {
                const float* gr = gs + r * a.GP;
                const float* xr0 = xs + (r * S) * a.XP;
#pragma unroll 1
                for (int ws = pw; ws < a.SPR; ws += a.PW, gr += a.PW * RW, xr0 += a.PW * RW * S) {
                    float gv[RM][RW];
#pragma unroll
                    for (int m = 0; m < RM; ++m) load_run<RW, (RW % 4 == 0)>(gv[m], gr + (4 * m) * a.GCH);
#pragma unroll
                    for (int c = 0; c < RC; ++c) {
#pragma unroll
                        for (int kh = 0; kh < KS; ++kh) {
                            float xv[XW];
                            load_run<XW, ((RW * S) % 4 == 0)>(xv, xr0 + (8 * c) * a.XCH + kh * a.XP);
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
        }
        if (do_gsum && (int)gs_ch < a.CO_T) {
            // strip sums of g over the item's valid rows (fixed order: the result does not depend on scheduling)
            const float* gch = Gs + gs_ch * a.GCH;
            if (RW % 4 == 0) {
                const int qpr = a.g.Wo >> 2;
                for (int q = gs_lane; q < nr * qpr; q += a.tpc) {
                    const int r = q / qpr, c4 = q - r * qpr;
                    const float4 v = *reinterpret_cast<const float4*>(gch + r * a.GP + 4 * c4);
                    gstrip += (v.x + v.y) + (v.z + v.w);
                }
            } else {
                for (int e = gs_lane; e < nr * a.g.Wo; e += a.tpc) {
                    const int r = e / a.g.Wo, c = e - r * a.g.Wo;
                    gstrip += gch[r * a.GP + c];
                }
            }
        }
        cur_c += nr;
        stage ^= 1;
    }
    cp_async_wait<0>();
    __syncthreads();              // the stages are free: they become the exchange buffer

    // Every warp parks its accumulators as [warp][e][lane]; then all threads walk the CTA's block of the
    // gradient in global-memory order, add the PS pixel shares of each element and write it to the slice.
    {
        float* mine = smem + (size_t)warp * NE * GWP_LP + lane;
#pragma unroll
        for (int m = 0; m < RM; ++m)
#pragma unroll
            for (int c = 0; c < RC; ++c)
#pragma unroll
                for (int t = 0; t < KK; ++t) mine[((m * RC + c) * KK + t) * GWP_LP] = acc[m][c][t];
    }
    __syncthreads();
    const int Ci = a.g.Ci, Co = a.g.Co;
    const size_t CoK = (size_t)Co * Ci * KK;
    float* slice = a.part + (size_t)split * CoK;
    const int PS = GWP_WARPS / a.OT;
    const int block_elems = a.CO_T * a.CI_T * KK;
    for (int o = tid; o < block_elems; o += nthreads) {
        uint32_t col, r;
        a.d_kk_ci.divmod(o, col, r);                 // r = cil*KK + t
        const int cil = r / KK, t = r - cil * KK;
        const int otoe = col >> 4, rc = col & 15, otie = cil >> 4, ri = cil & 15;
        const int ln = (ri & 7) * 4 + (rc & 3);
        const int e = ((rc >> 2) * RC + (ri >> 3)) * KK + t;
        const int ote = otoe * a.OTi + otie;
        float s = 0.f;
        for (int p = 0; p < PS; ++p) s += smem[(size_t)(p * a.OT + ote) * NE * GWP_LP + e * GWP_LP + ln];
        const int co = co0 + col, ci = ci0 + cil;
        if (co < Co && ci < Ci) slice[((size_t)co * Ci + ci) * KK + t] = s;
    }
    if (do_gsum) {
        for (int off = a.tpc >> 1; off > 0; off >>= 1) gstrip += __shfl_xor_sync(0xffffffffu, gstrip, off);
        if (gs_lane == 0 && (int)gs_ch < a.CO_T && co0 + (int)gs_ch < Co)
            a.gsum_part[(size_t)split * Co + co0 + gs_ch] = gstrip;
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------

struct GwPipePlan {
    GwPipeArgs a;
    int threads, out_blocks, status, ks, s, rw;
    size_t smem;
};

static int odd_quads(int floats) {      // smallest size >= floats that is an odd number of 16-byte words
    int q = (floats + 3) / 4;
    if (q % 2 == 0) ++q;
    return 4 * q;
}

template <int KS, int S, int RW>
static GwPipePlan plan_gw_pipe_t(const Geom& g, const TileHint& hint) {
    GwPipePlan p;
    GwPipeArgs& a = p.a;
    p.status = ADDER_OK;
    p.ks = KS; p.s = S; p.rw = RW;
    a.g = g;
    const int sms = sm_count();
    const int tiles_o = g.Co / 16, tiles_i = g.Ci / 16;
    // warp blocks per CTA: as many as there are (up to 8), preferring wide input-channel extent (the
    // haloed x patch is the expensive operand to stage, and it is shared by the output-channel blocks)
    int oto = 1, oti = 1;
    if (hint.cg > 0) { oto = hint.cg; oti = hint.ck > 0 ? hint.ck : 1; }
    else {
        while (oto * oti * 2 <= GWP_WARPS) {
            if (oto <= oti && oto * 2 <= tiles_o) oto *= 2;
            else if (oti * 2 <= tiles_i) oti *= 2;
            else if (oto * 2 <= tiles_o) oto *= 2;
            else break;
        }
    }
    if (hint.cg <= 0) {
        // Every CTA writes its whole block of the gradient as a slice of partial sums, and the finishing
        // kernel reads them all back: keep that traffic small next to the layer's work (6 MB, or 4 bytes per
        // 500 multiply-adds for the big layers) by shrinking the block, which trades it for more staging.
        const double triples = (double)g.N * g.Ho * g.Wo * g.Co * g.Ci * KS * KS;
        double cap = triples / 500.0 * 4.0;
        if (cap < 6.0 * 1024 * 1024) cap = 6.0 * 1024 * 1024;
        while (oto * oti > 1 && 2.0 * sms * (256.0 * oto * oti * KS * KS) * 4.0 > cap) {
            if (oto >= oti) oto /= 2; else oti /= 2;
        }
    }
    if (oto > tiles_o || oti > tiles_i || tiles_o % oto || tiles_i % oti || GWP_WARPS % (oto * oti)) {
        p.status = ADDER_ERR_INTERNAL; return p;
    }
    a.OT = oto * oti; a.OTi = oti;
    a.CO_T = 16 * oto; a.CI_T = 16 * oti;
    const int PS = GWP_WARPS / a.OT;
    a.SPR = g.Wo / RW;
    // pixel shares: split the segments of a row first (up to what divides them), then the rows
    int pw = 1;
    while (pw * 2 <= PS && a.SPR % (pw * 2) == 0 && a.SPR / (pw * 2) >= 2) pw *= 2;
    a.PW = pw;
    a.PR = PS / pw;
    // rows per item: a multiple of PR, as many as the shared-memory budget allows (two stages, two CTAs per SM)
    const int budget_floats = (hint.smem_kb > 0 ? hint.smem_kb : 108) * 1024 / 4;
    a.XP = round_up((g.Wo - 1) * S + KS, 4);
    a.GP = round_up(g.Wo, 4);
    int th = hint.th > 0 ? hint.th : 8;
    if (th < a.PR) th = a.PR;
    th = th / a.PR * a.PR;
    if (th > round_up(g.Ho, a.PR)) th = round_up(g.Ho, a.PR);
    auto size_for = [&](int rows) {
        const int xr = (rows - 1) * S + KS;
        a.XCH = odd_quads(xr * a.XP);
        a.GCH = odd_quads(rows * a.GP);
        a.xs_stage = round_up(a.CI_T * a.XCH, 4);
        a.stage_floats = a.xs_stage + round_up(a.CO_T * a.GCH, 4);
        return 2 * a.stage_floats;
    };
    while (th > a.PR && size_for(th) > budget_floats) th -= a.PR;
    // items never cross an image: a row count that divides the plane height leaves no ragged last item
    if (hint.th <= 0)
        for (int d = th; d >= a.PR && 2 * d > th; d -= a.PR)
            if (g.Ho % d == 0) { th = d; break; }
    (void)size_for(th);
    a.TH = th;
    const int xrows = (th - 1) * S + KS;
    const size_t exch = (size_t)GWP_WARPS * 4 * 2 * KS * KS * GWP_LP;
    size_t floats = (size_t)2 * a.stage_floats;
    if (floats < exch) floats = exch;
    p.smem = floats * sizeof(float);
    if (p.smem > 200 * 1024) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    PatchDims& px = a.pdx;
    px.CH = a.CI_T; px.TI = 1; px.ROWS = xrows; px.COLS = (g.Wo - 1) * S + KS; px.PITCH = a.XP;
    px.ROWS_PITCH = xrows * a.XP; px.CHS = a.XCH;
    px.d_cols = FastDiv(px.COLS); px.d_rows = FastDiv(px.ROWS);
    PatchDims& pg = a.pdg;
    pg.CH = a.CO_T; pg.TI = 1; pg.ROWS = th; pg.COLS = g.Wo; pg.PITCH = a.GP; pg.ROWS_PITCH = th * a.GP; pg.CHS = a.GCH;
    pg.d_cols = FastDiv(pg.COLS); pg.d_rows = FastDiv(pg.ROWS);
    a.g_quads = (g.Wo % 4 == 0) ? 1 : 0;             // the pointer's alignment is checked at launch
    a.d_gquads = FastDiv(g.Wo >= 4 ? g.Wo / 4 : 1);
    a.n_ci_blocks = tiles_i / oti;
    p.out_blocks = (tiles_o / oto) * a.n_ci_blocks;
    if (p.out_blocks > 65535) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.rows_total = (long long)g.N * g.Ho;
    if (a.rows_total > 2147483647LL) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.row_quantum = a.PR;
    const int ctas_sm = (2 * (p.smem + 1024) <= 227 * 1024) ? 2 : 1;
    long long splits = hint.ti > 0 ? hint.ti : ((long long)sms * ctas_sm) / p.out_blocks;
    const long long quanta = (a.rows_total + a.row_quantum - 1) / a.row_quantum;
    if (splits > quanta) splits = quanta;
    if (splits < 1) splits = 1;
    a.splits = (int)splits;
    a.tpc = GWP_WARPS * 32 / a.CO_T;
    if (a.tpc > 32) a.tpc = 32;
    if (a.tpc < 1) a.tpc = 1;
    p.threads = GWP_WARPS * 32;
    a.d_ho = FastDiv(g.Ho);
    a.d_pw = FastDiv(a.PW);
    a.d_ot = FastDiv(a.OT);
    a.d_oti = FastDiv(a.OTi);
    a.d_ci_blocks = FastDiv(a.n_ci_blocks);
    a.d_tpc = FastDiv(a.tpc);
    a.d_kk_ci = FastDiv(a.CI_T * KS * KS);
    return p;
}

// Layers whose channels come in sixteens and whose output rows are whole 4-pixel segments, up to 64 wide.
// Pixels per row segment: 4 where the output rows are whole quads (also the 28- and 56-wide ImageNet planes:
// 128->128 on 28x28 went from 909 us with the pixel-lane kernel to 390 us), 7 for 14- and 7-wide planes.
static int gw_pipe_rw(const Geom& g) {
    if (g.Wo % 4 == 0) return 4;
    if (g.Wo % 7 == 0) return 7;
    return 0;
}

bool gw_pipe_applicable(const Geom& g, const TileHint& hint) {
    if (hint.variant == 1) return false;        // tuning: force the non-persistent kernels
    if (!(g.k == 3 && (g.stride == 1 || g.stride == 2))) return false;    // 1x1 layers: 8 sums per lane are too few
    if (g.Co % 16 != 0 || g.Ci % 16 != 0 || gw_pipe_rw(g) == 0 || g.Wo > 64) return false;
    return g.N >= 1;
}

#define ADDER_GWP_DISPATCH(CALL)                                                                  \
    if (g.k == 3 && g.stride == 1) { if (gw_pipe_rw(g) == 7) { CALL(3, 1, 7) } else { CALL(3, 1, 4) } }      \
    else if (g.k == 3 && g.stride == 2) { if (gw_pipe_rw(g) == 7) { CALL(3, 2, 7) } else { CALL(3, 2, 4) } }

int gw_pipe_splits(const Geom& g, const TileHint& hint) {
    GwPipePlan p;
    p.status = ADDER_ERR_UNSUPPORTED;
#define ADDER_GWP_PLAN(KS_, S_, RW_) p = plan_gw_pipe_t<KS_, S_, RW_>(g, hint);
    ADDER_GWP_DISPATCH(ADDER_GWP_PLAN)
    return p.status == ADDER_OK ? p.a.splits : 0;
}

int describe_gw_pipe(const Geom& g, const TileHint& hint, char* buf, size_t n) {
    GwPipePlan p;
    p.status = ADDER_ERR_UNSUPPORTED;
    ADDER_GWP_DISPATCH(ADDER_GWP_PLAN)
#undef ADDER_GWP_PLAN
    const GwPipeArgs& a = p.a;
    snprintf(buf, n,
             "gw warp-tile k=%d s=%d RW=%d block=%dx%d (warps %dx%d) shares=%d (rows %d x segs %d) TH=%d SPR=%d xpitch=%d "
             "gpitch=%d xch=%d gch=%d threads=%d smem=%zu rows=%lld splits=%d out_tiles=%d gemm1x1=0 pointwise=0 status=%d",
             p.ks, p.s, p.rw, a.CO_T, a.CI_T, a.OT / a.OTi, a.OTi, GWP_WARPS / a.OT, a.PR, a.PW, a.TH, a.SPR, a.XP, a.GP,
             a.XCH, a.GCH, p.threads, p.smem, a.rows_total, a.splits, p.out_blocks, p.status);
    return ADDER_OK;
}

template <int KS, int S, int RW>
static int launch_gw_pipe_t(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                            unsigned int* ticket, int splits, const TileHint& hint, cudaStream_t stream) {
    GwPipePlan p = plan_gw_pipe_t<KS, S, RW>(g, hint);
    if (p.status != ADDER_OK) return p.status;
    if (p.a.splits != splits) return ADDER_ERR_INTERNAL;
    p.a.gout = gout; p.a.x = x; p.a.part = part; p.a.gsum_part = gsum_part; p.a.ticket = ticket;
    if ((reinterpret_cast<uintptr_t>(gout) & 15) != 0) p.a.g_quads = 0;
    auto kern = adder_gw_pipe_kernel<KS, S, RW>;
    const int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), p.smem);
    if (st != ADDER_OK) return st;
    kern<<<dim3((unsigned)p.a.splits, (unsigned)p.out_blocks), p.threads, p.smem, stream>>>(p.a);
    return launched();
}

int launch_gw_pipe(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                   unsigned int* ticket, int splits, const TileHint& hint, cudaStream_t stream) {
#define ADDER_GWP_LAUNCH(KS_, S_, RW_) \
    return launch_gw_pipe_t<KS_, S_, RW_>(g, gout, x, part, gsum_part, ticket, splits, hint, stream);
    ADDER_GWP_DISPATCH(ADDER_GWP_LAUNCH)
#undef ADDER_GWP_LAUNCH
    return ADDER_ERR_UNSUPPORTED;
}

}  // namespace adder
