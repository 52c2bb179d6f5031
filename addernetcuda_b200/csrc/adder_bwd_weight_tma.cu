// Weight gradient of 3x3 stride-1 adder layers, warp-tile form fed by the tensor memory accelerator (main
// kernel only; the finishing kernels of adder_bwd_weight.cu follow it unchanged):
//   part[split][co,ci,kh,kw] = sum over the split's pixels of xpad[n,ci,ho+kh,wo+kw] * g[n,co,ho,wo]
//   gsum_part[split][co]     = sum over the split's pixels of g[n,co,ho,wo]
// (CONV_BACKWARD's grad_w, adder_cuda/adder.cu:247,:267, as sum x*g - w*sum g.)
//
// Same decomposition as adder_gw_pipe_kernel (adder_bwd_weight_pipe.cu): a warp owns a 16 x 16 x 9 block of the
// gradient with all lanes walking the same pixels, a CTA is OT warp blocks x PS pixel shares, the N*Ho output
// rows are dealt out in contiguous ranges, items of up to TH rows of one image are double-buffered.  What
// differs is how an item reaches shared memory: one elected thread issues two tiled bulk copies
// (cp.async.bulk.tensor, 4-d boxes of x and of g) that complete on an mbarrier.  No thread spends issue
// slots on address arithmetic, predicates or copy instructions; padding rows and columns, rows past the
// image and channels past the tensor arrive as zeros from the copy engine.
//
// Shared-memory layout = the boxes as the copy engine writes them: x [CI_T][XR][BX], g [CO_T][GR][BG], rows
// of BX = W+8.. floats starting 4 columns left of the image (box origins must be multiples of 16 bytes, the
// first tap column is -pad).  XR, GR and BX/4, BG/4 are made odd, so that the channel planes are an odd number
// of 16-byte words apart and the 8 (x) or 4 (g) distinct addresses of one warp-wide load fall into distinct
// bank groups.  A segment's 10 input values start 3 floats after a 16-byte boundary (pad 1): one scalar,
// two 128-bit and one scalar load.
#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"
#include <cstdio>

namespace adder {

constexpr int GWT_WARPS = 8;
constexpr int GWT_LP = 33;

struct GwTmaArgs {
    Geom g;
    float* part;
    float* gsum_part;
    unsigned int* ticket;
    int* error_flag;
    int TH, SPR, PR, PW, OT, OTi, CO_T, CI_T, XCH, GCH, BX, BG, XR, GR;
    int xs_stage, stage_floats, splits, n_ci_blocks, tpc, row_quantum;
    uint32_t item_bytes;
    long long rows_total;
    FastDiv d_ho, d_pw, d_ot, d_oti, d_ci_blocks, d_tpc, d_kk_ci, d_qpr;
};

template <int RW, int PAD>
__global__ void __launch_bounds__(GWT_WARPS * 32, 2)
adder_gw_tma_kernel(const GwTmaArgs a, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_g) {
    constexpr int KS = 3, KK = 9, XW = RW + KS - 1;
    constexpr int RM = 4, RC = 2, NE = RM * RC * KK;
    constexpr int XORG = PAD > 0 ? 4 : 0;            // shared-memory column of image column 0
    constexpr int OFF = (XORG - PAD) & 3;            // a segment's first tap column relative to a 16-byte boundary
    extern __shared__ __align__(128) float smem[];
    __shared__ __align__(8) uint64_t full[2];
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
    // elected thread: arm the stage's barrier with the bytes of both boxes, then start the two copies
    auto issue = [&](int cur, int stage) {
        int n, r0;
        (void)item_rows(cur, n, r0);
        float* xs = smem + stage * a.stage_floats;
        mbar_arrive_expect_tx(&full[stage], a.item_bytes);
        tma_load_box(xs, &map_x, &full[stage], -XORG, r0 - PAD, ci0, n);
        tma_load_box(xs + a.xs_stage, &map_g, &full[stage], 0, r0, co0, n);
    };

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_fence_init();
    }
    __syncthreads();

    float acc[RM][RC][KK];
#pragma unroll
    for (int m = 0; m < RM; ++m)
#pragma unroll
        for (int c = 0; c < RC; ++c)
#pragma unroll
            for (int t = 0; t < KK; ++t) acc[m][c][t] = 0.f;
    float gstrip = 0.f;
    uint32_t gs_ch, gs_lane;
    a.d_tpc.divmod(tid, gs_ch, gs_lane);

    int cur_f = R0, cur_c = R0, stage = 0, issued = 0, done = 0;
    uint32_t phases = 0u;                 // bit s: parity of the phase stage s completes next
    bool failed = false;
    if (tid == 0 && cur_f < R1) {
        int n, r0;
        issue(cur_f, 0);
        cur_f += item_rows(cur_f, n, r0);
        ++issued;
    }
    while (cur_c < R1) {
        const bool landed = mbar_wait(&full[stage], (phases >> stage) & 1u);
        // one block barrier per item: the item is in shared memory for everyone (or the wait gave up for
        // someone, and then everybody leaves), and everyone is done with the other stage
        if (!__syncthreads_and(landed ? 1 : 0)) { failed = true; break; }
        phases ^= 1u << stage;
        ++done;
        if (tid == 0 && cur_f < R1) {
            int n, r0;
            issue(cur_f, stage ^ 1);
            cur_f += item_rows(cur_f, n, r0);
            ++issued;
        }
        int n_img, r0_img;
        const int nr = item_rows(cur_c, n_img, r0_img);
        const float* Xs = smem + stage * a.stage_floats;
        const float* Gs = Xs + a.xs_stage;
        {
            const float* xs = Xs + (oti * 16 + cgc) * a.XCH + pw * RW;
            const float* gs = Gs + (oto * 16 + cgo) * a.GCH + pw * RW;
            const int gstep = a.PW * RW;
#pragma unroll 1
            for (int r = pr; r < nr; r += a.PR) {
                const float* gr = gs + r * a.BG;
                const float* xr0 = xs + r * a.BX;
#pragma unroll 1
                for (int ws = pw; ws < a.SPR; ws += a.PW, gr += gstep, xr0 += gstep) {
                    float gv[RM][RW];
#pragma unroll
                    for (int m = 0; m < RM; ++m) load_run<RW, true>(gv[m], gr + (4 * m) * a.GCH);
#pragma unroll
                    for (int c = 0; c < RC; ++c) {
#pragma unroll
                        for (int kh = 0; kh < KS; ++kh) {
                            float xv[XW];
                            load_run_off<XW, OFF>(xv, xr0 + (8 * c) * a.XCH + kh * a.BX + (XORG - PAD - OFF));
#pragma unroll
                            for (int kw = 0; kw < KS; ++kw)
#pragma unroll
                                for (int m = 0; m < RM; ++m)
#pragma unroll
                                    for (int j = 0; j < RW; ++j)
                                        acc[m][c][kh * KS + kw] = fmaf(xv[j + kw], gv[m][j], acc[m][c][kh * KS + kw]);
                        }
                    }
                }
            }
        }
        if (do_gsum && (int)gs_ch < a.CO_T) {
            // strip sums of g over the item's valid rows (fixed order: the result does not depend on scheduling)
            const float* gch = Gs + gs_ch * a.GCH;
            const int nq = nr * (int)a.d_qpr.div;
            for (int q = gs_lane; q < nq; q += a.tpc) {
                uint32_t r, c4;
                a.d_qpr.divmod(q, r, c4);
                const float4 v = *reinterpret_cast<const float4*>(gch + r * a.BG + 4 * c4);
                gstrip += (v.x + v.y) + (v.z + v.w);
            }
        }
        cur_c += nr;
        stage ^= 1;
    }
    if (failed) {
        // A copy never arrived.  Record it, give the copies this CTA started a last bounded chance to land
        // (shared memory must not be handed back while the copy engine may still write to it), and leave.
        if (tid == 0) {
            atomicExch(a.error_flag, 1);
            for (int s = stage; done < issued; s ^= 1, ++done)
                if (!mbar_wait(&full[s], (phases >> s) & 1u)) break;
        }
        return;
    }
    __syncthreads();              // the stages are free: they become the exchange buffer

    {
        float* mine = smem + (size_t)warp * NE * GWT_LP + lane;
#pragma unroll
        for (int m = 0; m < RM; ++m)
#pragma unroll
            for (int c = 0; c < RC; ++c)
#pragma unroll
                for (int t = 0; t < KK; ++t) mine[((m * RC + c) * KK + t) * GWT_LP] = acc[m][c][t];
    }
    __syncthreads();
    const int Ci = a.g.Ci, Co = a.g.Co;
    const size_t CoK = (size_t)Co * Ci * KK;
    float* slice = a.part + (size_t)split * CoK;
    const int PS = GWT_WARPS / a.OT;
    const int block_elems = a.CO_T * a.CI_T * KK;
    for (int o = tid; o < block_elems; o += nthreads) {
        uint32_t col, r;
        a.d_kk_ci.divmod(o, col, r);
        const int cil = r / KK, t = r - cil * KK;
        const int otoe = col >> 4, rc = col & 15, otie = cil >> 4, ri = cil & 15;
        const int ln = (ri & 7) * 4 + (rc & 3);
        const int e = ((rc >> 2) * RC + (ri >> 3)) * KK + t;
        const int ote = otoe * a.OTi + otie;
        float s = 0.f;
        for (int p = 0; p < PS; ++p) s += smem[(size_t)(p * a.OT + ote) * NE * GWT_LP + e * GWT_LP + ln];
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

struct GwTmaPlan {
    GwTmaArgs a;
    int threads, out_blocks, status;
    size_t smem;
};

static int odd_up(int v) { return v | 1; }
// smallest multiple of 4 >= v whose quarter is odd
static int odd_quads_width(int v) {
    int q = (v + 3) / 4;
    if (q % 2 == 0) ++q;
    return 4 * q;
}

template <int RW, int PAD>
static GwTmaPlan plan_gw_tma_t(const Geom& g, const TileHint& hint) {
    GwTmaPlan p;
    GwTmaArgs& a = p.a;
    p.status = ADDER_OK;
    a.g = g;
    const int sms = sm_count();
    const int tiles_o = g.Co / 16, tiles_i = g.Ci / 16;
    int oto = 1, oti = 1;
    if (hint.cg > 0) { oto = hint.cg; oti = hint.ck > 0 ? hint.ck : 1; }
    else {
        while (oto * oti * 2 <= GWT_WARPS) {
            if (oto <= oti && oto * 2 <= tiles_o) oto *= 2;
            else if (oti * 2 <= tiles_i) oti *= 2;
            else if (oto * 2 <= tiles_o) oto *= 2;
            else break;
        }
        // keep the slices of partial sums (written by every CTA, read back by the finishing kernel) small
        // next to the layer's work: 6 MB, or 4 bytes per 500 multiply-adds for the big layers
        const double triples = (double)g.N * g.Ho * g.Wo * g.Co * g.Ci * 9.0;
        double cap = triples / 500.0 * 4.0;
        if (cap < 6.0 * 1024 * 1024) cap = 6.0 * 1024 * 1024;
        while (oto * oti > 1 && 2.0 * sms * (256.0 * oto * oti * 9.0) * 4.0 > cap) {
            if (oto >= oti) oto /= 2; else oti /= 2;
        }
    }
    if (oto > tiles_o || oti > tiles_i || tiles_o % oto || tiles_i % oti || GWT_WARPS % (oto * oti)) {
        p.status = ADDER_ERR_INTERNAL; return p;
    }
    a.OT = oto * oti; a.OTi = oti;
    a.CO_T = 16 * oto; a.CI_T = 16 * oti;
    const int PS = GWT_WARPS / a.OT;
    a.SPR = g.Wo / RW;
    int pw = 1;
    while (pw * 2 <= PS && a.SPR % (pw * 2) == 0) pw *= 2;
    a.PW = pw;
    a.PR = PS / pw;
    const int xorg = PAD > 0 ? 4 : 0;
    a.BX = odd_quads_width(xorg + g.W + PAD);      // last tap column of the last segment: xorg + W + PAD - 1
    a.BG = odd_quads_width(g.Wo);
    const int budget_floats = (hint.smem_kb > 0 ? hint.smem_kb : 108) * 1024 / 4;
    int th = hint.th > 0 ? hint.th : 8;
    if (th < a.PR) th = a.PR;
    th = th / a.PR * a.PR;
    if (th > round_up(g.Ho, a.PR)) th = round_up(g.Ho, a.PR);
    auto size_for = [&](int rows) {
        a.XR = odd_up(rows + 2);
        a.GR = odd_up(rows);
        a.XCH = a.XR * a.BX;
        a.GCH = a.GR * a.BG;
        a.xs_stage = round_up(a.CI_T * a.XCH, 32);          // 128-byte aligned box destinations
        a.stage_floats = a.xs_stage + round_up(a.CO_T * a.GCH, 32);
        return 2 * a.stage_floats;
    };
    while (th > a.PR && size_for(th) > budget_floats) th -= a.PR;
    if (hint.th <= 0)
        for (int d = th; d >= a.PR && 2 * d > th; d -= a.PR)
            if (g.Ho % d == 0) { th = d; break; }
    (void)size_for(th);
    a.TH = th;
    if (a.XR > 256 || a.GR > 256 || a.BX > 256 || a.BG > 256 || a.CI_T > 256 || a.CO_T > 256) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.item_bytes = (uint32_t)((a.CI_T * a.XCH + a.CO_T * a.GCH) * sizeof(float));
    const size_t exch = (size_t)GWT_WARPS * 4 * 2 * 9 * GWT_LP;
    size_t floats = (size_t)2 * a.stage_floats;
    if (floats < exch) floats = exch;
    p.smem = floats * sizeof(float);
    if (p.smem > 200 * 1024) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.n_ci_blocks = tiles_i / oti;
    p.out_blocks = (tiles_o / oto) * a.n_ci_blocks;
    if (p.out_blocks > 65535) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.rows_total = (long long)g.N * g.Ho;
    if (a.rows_total > 2147483647LL) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.row_quantum = a.PR;
    const int ctas_sm = (2 * (p.smem + 2048) <= 227 * 1024) ? 2 : 1;
    long long splits = hint.ti > 0 ? hint.ti : ((long long)sms * ctas_sm) / p.out_blocks;
    const long long quanta = (a.rows_total + a.row_quantum - 1) / a.row_quantum;
    if (splits > quanta) splits = quanta;
    if (splits < 1) splits = 1;
    a.splits = (int)splits;
    a.tpc = GWT_WARPS * 32 / a.CO_T;
    if (a.tpc > 32) a.tpc = 32;
    if (a.tpc < 1) a.tpc = 1;
    p.threads = GWT_WARPS * 32;
    a.d_ho = FastDiv(g.Ho);
    a.d_pw = FastDiv(a.PW);
    a.d_ot = FastDiv(a.OT);
    a.d_oti = FastDiv(a.OTi);
    a.d_ci_blocks = FastDiv(a.n_ci_blocks);
    a.d_tpc = FastDiv(a.tpc);
    a.d_kk_ci = FastDiv(a.CI_T * 9);
    a.d_qpr = FastDiv(g.Wo / 4);
    return p;
}

// 3x3 stride-1 layers with channels in sixteens, rows of whole 8-pixel segments up to 64 wide, padding 0..2.
bool gw_tma_applicable(const Geom& g, const TileHint& hint) {
    if (hint.variant != 0) return false;          // tuning: 1 = non-persistent kernels, 2 = cp.async warp-tile kernel
    if (!(g.k == 3 && g.stride == 1 && g.pad <= 2)) return false;
    if (g.Co % 16 != 0 || g.Ci % 16 != 0 || g.Wo % 8 != 0 || g.Wo > 64 || g.W % 4 != 0) return false;
    return g.N >= 1;
}

#define ADDER_GWT_DISPATCH(CALL)                    \
    if (g.pad == 1) { CALL(8, 1) }                  \
    else if (g.pad == 0) { CALL(8, 0) }             \
    else if (g.pad == 2) { CALL(8, 2) }

int gw_tma_splits(const Geom& g, const TileHint& hint) {
    GwTmaPlan p;
    p.status = ADDER_ERR_UNSUPPORTED;
#define ADDER_GWT_PLAN(RW_, PAD_) p = plan_gw_tma_t<RW_, PAD_>(g, hint);
    ADDER_GWT_DISPATCH(ADDER_GWT_PLAN)
    return p.status == ADDER_OK ? p.a.splits : 0;
}

int describe_gw_tma(const Geom& g, const TileHint& hint, char* buf, size_t n) {
    GwTmaPlan p;
    p.status = ADDER_ERR_UNSUPPORTED;
    ADDER_GWT_DISPATCH(ADDER_GWT_PLAN)
#undef ADDER_GWT_PLAN
    const GwTmaArgs& a = p.a;
    snprintf(buf, n,
             "gw warp-tile tma k=3 s=1 RW=8 block=%dx%d (warps %dx%d) shares=%d (rows %d x segs %d) TH=%d SPR=%d xbox=%dx%d "
             "gbox=%dx%d threads=%d smem=%zu rows=%lld splits=%d out_tiles=%d gemm1x1=0 pointwise=0 status=%d",
             a.CO_T, a.CI_T, a.OT / a.OTi, a.OTi, GWT_WARPS / a.OT, a.PR, a.PW, a.TH, a.SPR, a.XR, a.BX, a.GR, a.BG,
             p.threads, p.smem, a.rows_total, a.splits, p.out_blocks, p.status);
    return ADDER_OK;
}

template <int RW, int PAD>
static int launch_gw_tma_t(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                           unsigned int* ticket, int splits, const TileHint& hint, cudaStream_t stream) {
    GwTmaPlan p = plan_gw_tma_t<RW, PAD>(g, hint);
    if (p.status != ADDER_OK) return p.status;
    if (p.a.splits != splits) return ADDER_ERR_INTERNAL;
    CUtensorMap map_x, map_g;
    if (!make_nchw_tensor_map(&map_x, x, g.N, g.Ci, g.H, g.W, p.a.BX, p.a.XR, p.a.CI_T, 1) ||
        !make_nchw_tensor_map(&map_g, gout, g.N, g.Co, g.Ho, g.Wo, p.a.BG, p.a.GR, p.a.CO_T, 1))
        return ADDER_ERR_ALIGNMENT;          // the caller falls back to the kernel without tensor maps
    p.a.part = part; p.a.gsum_part = gsum_part; p.a.ticket = ticket;
    const int fe = device_error_flag(&p.a.error_flag);
    if (fe != ADDER_OK) return fe;
    auto kern = adder_gw_tma_kernel<RW, PAD>;
    const int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), p.smem);
    if (st != ADDER_OK) return st;
    kern<<<dim3((unsigned)p.a.splits, (unsigned)p.out_blocks), p.threads, p.smem, stream>>>(p.a, map_x, map_g);
    return launched();
}

int launch_gw_tma(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                  unsigned int* ticket, int splits, const TileHint& hint, cudaStream_t stream) {
#define ADDER_GWT_LAUNCH(RW_, PAD_) \
    return launch_gw_tma_t<RW_, PAD_>(g, gout, x, part, gsum_part, ticket, splits, hint, stream);
    ADDER_GWT_DISPATCH(ADDER_GWT_LAUNCH)
#undef ADDER_GWT_LAUNCH
    return ADDER_ERR_UNSUPPORTED;
}

}  // namespace adder
