// Forward adder convolution, persistent multi-stage form:
//   out[n,co,ho,wo] = - sum_{ci,kh,kw} | xpad[n,ci,ho*S+kh,wo*S+kw] - w[co,ci,kh,kw] |
// (adder.py:32-39 feeding the CONV kernel of adder_cuda/adder.cu:19-70, on NCHW tensors with implicit im2col).
//
// Differences from adder_fwd_kernel (adder_fwd.cu), which stays as the general fallback:
//  * Persistent CTAs.  The grid is at most the number of CTAs the GPU holds at once; a CTA walks over its
//    share of the (output-channel tile, pixel tile) units.  The work of a CTA is a flat sequence of items
//    (unit, input-channel chunk) streamed through a three-stage cp.async ring, so the loads of the next
//    unit's first chunk are in flight while the last chunk of the current unit is computed: no CTA ever
//    sits in a load -> compute -> store sequence on its own.  One block barrier per item.
//  * Doubled input rows.  The staged input patch holds every value twice ([.., x, x, ..]), so one 128-bit
//    shared-memory load yields two ready (x, x) operands for the packed subtract
//        (w_a, w_b) - (x, x)      sub.rn.f32x2: one issue slot for two channels
//    and no register moves are spent on building pairs.  The two |d| accumulations stay scalar adds with
//    the absolute-value operand modifier: 1.5 issue slots and 2 FP32-pipe slots per |x-w| term.
//  * Reduction split inside the CTA.  KG groups of threads share one output tile and take every KG-th
//    input channel of a chunk; their partial sums are folded through shared memory at the end of a unit.
//    Layers with few pixels (64 channels on 8x8 planes) get 16 warps per SM that way without shrinking
//    the register tile.
//  * Lanes of a warp hold consecutive ROWS of the tile (not consecutive segments of a row): with a row
//    pitch that is an odd number of 16-byte words their 128-bit loads fall into distinct bank groups.
#include "common.cuh"
#include "kernels.h"
#include "patch_fill.cuh"
#include <cstdio>

namespace adder {

constexpr int FWD_STAGES = 3;

struct FwdPipeArgs {
    Geom g;
    const float* x;
    const float* w;
    float* out;
    PatchDims pd;                 // haloed input patch of one chunk: [CK][TI*IN_ROWS][PITCH], rows doubled
    int TI, TH, SPR, SEGS, CG, KG, TM, TMP, CK;
    int IN_ROWS, PITCH, CH_STRIDE;
    int xs_stage, ws_stage, wkk_pad, red_floats;
    int tiles_h, tiles_w, n_px_tiles, n_units, nchunks, vec_store;
    FastDiv d_tiles_h, d_tiles_w, d_px_tiles, d_nchunks, d_group, d_segs, d_rows, d_th, d_tm;
};

template <int KS, int S, int RW, int RM>
__global__ void __launch_bounds__(256, 2) adder_fwd_pipe_kernel(const FwdPipeArgs a) {
    constexpr int KK = KS * KS;
    constexpr int XW = (RW - 1) * S + KS;   // input values one segment touches per (ci, kh)
    constexpr int NS = FWD_STAGES;
    constexpr bool VEC = (RW * S) % 2 == 0;   // segment starts are multiples of 16 bytes in the doubled rows
    extern __shared__ __align__(16) float smem[];
    float* const Xs = smem;
    float* const Ws = smem + NS * a.xs_stage;
    float* const Red = Ws + NS * a.ws_stage;

    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    // thread role: reduction group, channel group, segment; segment -> (segment within row, image, tile row),
    // rows fastest
    uint32_t kg, rem, cg, seg, ws, rowidx, img, hr;
    a.d_group.divmod(tid, kg, rem);
    a.d_segs.divmod(rem, cg, seg);
    a.d_rows.divmod(seg, ws, rowidx);
    a.d_th.divmod(rowidx, img, hr);
    const bool active = (int)kg < a.KG && (int)cg < a.CG;
    const int xoff = (img * a.IN_ROWS + hr * S) * a.PITCH + ws * (RW * S) * 2;

    const int my_units = ((int)blockIdx.x < a.n_units) ? (a.n_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int n_items = my_units * a.nchunks;
    const int K = a.g.Ci * KK;
    const int w_elems = a.wkk_pad * a.TM;

    auto unit_origin = [&](int k, int& n0, int& ho0, int& wo_t0, int& co0) {
        const uint32_t u = blockIdx.x + (uint32_t)k * gridDim.x;
        uint32_t ct, pt, tn, th, tw, tnh;
        a.d_px_tiles.divmod(u, ct, pt);
        a.d_tiles_w.divmod(pt, tnh, tw);
        a.d_tiles_h.divmod(tnh, tn, th);
        n0 = tn * a.TI; ho0 = th * a.TH; wo_t0 = tw * (a.SPR * RW); co0 = ct * a.TM;
    };

    auto fill = [&](int item, int stage) {
        if (item >= n_items) return;
        uint32_t k, chunk;
        a.d_nchunks.divmod(item, k, chunk);
        int n0, ho0, wo_t0, co0;
        unit_origin((int)k, n0, ho0, wo_t0, co0);
        const int ci0 = chunk * a.CK;
        fill_patch<true>(Xs + stage * a.xs_stage, a.x, a.pd, n0, ci0, ho0 * S - a.g.pad, wo_t0 * S - a.g.pad, a.g.N,
                         a.g.Ci, a.g.H, a.g.W, tid, nthreads);
        float* wsm = Ws + stage * a.ws_stage;
        const int kbase = ci0 * KK;
        const int kk_lim = a.CK * KK;
        for (int e = tid; e < w_elems; e += nthreads) {
            uint32_t t, col, kkb;
            const int kk8 = e & 7;
            t = e >> 3;
            a.d_tm.divmod(t, kkb, col);
            const int kk = kkb * 8 + kk8;
            const int co = co0 + col;
            const bool ok = (co < a.g.Co) & (kk < kk_lim) & (kbase + kk < K);
            cp_async4(wsm + kk * a.TMP + col, ok ? a.w + ((size_t)co * K + kbase + kk) : a.w, ok);
        }
    };

    float acc[RM][RW];
#pragma unroll
    for (int m = 0; m < RM; ++m)
#pragma unroll
        for (int j = 0; j < RW; ++j) acc[m][j] = 0.f;

#pragma unroll
    for (int s = 0; s < NS - 1; ++s) {
        fill(s, s);
        cp_async_commit();
    }
    int stage = 0, chunk = 0, unit_k = 0;
    for (int it = 0; it < n_items; ++it) {
        cp_async_wait<NS - 2>();
        __syncthreads();      // item `it` has landed for everyone, and everyone is done with item it-1
        {
            const int fs = stage == 0 ? NS - 1 : stage - 1;      // the stage item it-1 used
            fill(it + NS - 1, fs);
            cp_async_commit();
        }
        if (active) {
            const float* xs = Xs + stage * a.xs_stage + xoff;
            const float* wsm = Ws + stage * a.ws_stage + cg * RM;
            const int nch = min(a.CK, a.g.Ci - chunk * a.CK);
#pragma unroll 1
            for (int cil = kg; cil < nch; cil += a.KG) {
#pragma unroll
                for (int kh = 0; kh < KS; ++kh) {
                    uint64_t x2[XW];
                    load_pairs<XW, VEC>(x2, xs + cil * a.CH_STRIDE + kh * a.PITCH);
#pragma unroll
                    for (int kw = 0; kw < KS; ++kw) {
                        const float* wr = wsm + (cil * KK + kh * KS + kw) * a.TMP;
                        float wv[RM];
#pragma unroll
                        for (int m4 = 0; m4 < RM; m4 += 4) {
                            const float4 t = *reinterpret_cast<const float4*>(wr + m4);
                            wv[m4] = t.x; wv[m4 + 1] = t.y; wv[m4 + 2] = t.z; wv[m4 + 3] = t.w;
                        }
#pragma unroll
                        for (int m = 0; m < RM; m += 2) {
                            const uint64_t w2 = pack2(wv[m], wv[m + 1]);
#pragma unroll
                            for (int j = 0; j < RW; ++j) {
                                float d0, d1;
                                unpack2(sub2(w2, x2[j * S + kw]), d0, d1);
                                acc[m][j] += fabsf(d0);
                                acc[m + 1][j] += fabsf(d1);
                            }
                        }
                    }
                }
            }
        }
        if (++chunk == a.nchunks) {
            // end of a unit: fold the reduction groups, store, start the next unit from zero
            chunk = 0;
            if (a.KG > 1) {
                if (active && kg > 0) {
                    float* r = Red + ((kg - 1) * (RM * RW)) * a.d_group.div + rem;
#pragma unroll
                    for (int m = 0; m < RM; ++m)
#pragma unroll
                        for (int j = 0; j < RW; ++j) r[(m * RW + j) * a.d_group.div] = acc[m][j];
                }
                __syncthreads();
                if (active && kg == 0) {
                    for (int q = 1; q < a.KG; ++q) {
                        const float* r = Red + ((q - 1) * (RM * RW)) * a.d_group.div + rem;
#pragma unroll
                        for (int m = 0; m < RM; ++m)
#pragma unroll
                            for (int j = 0; j < RW; ++j) acc[m][j] += r[(m * RW + j) * a.d_group.div];
                    }
                }
            }
            if (active && kg == 0) {
                int n0, ho0, wo_t0, co0;
                unit_origin(unit_k, n0, ho0, wo_t0, co0);
                const int n = n0 + img, ho = ho0 + hr, wo0 = wo_t0 + ws * RW;
                if (n < a.g.N && ho < a.g.Ho && wo0 < a.g.Wo) {
                    const int HoWo = a.g.Ho * a.g.Wo;
#pragma unroll
                    for (int m = 0; m < RM; ++m) {
                        const int co = co0 + cg * RM + m;
                        if (co >= a.g.Co) break;
                        float* o = a.out + ((size_t)(n * a.g.Co + co) * HoWo + ho * a.g.Wo + wo0);
                        if (RW % 4 == 0 && a.vec_store) {
#pragma unroll
                            for (int j = 0; j < RW; j += 4)
                                *reinterpret_cast<float4*>(o + j) =
                                    make_float4(-acc[m][j], -acc[m][j + 1], -acc[m][j + 2], -acc[m][j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < RW; ++j)
                                if (wo0 + j < a.g.Wo) o[j] = -acc[m][j];
                        }
                    }
                }
            }
            ++unit_k;
#pragma unroll
            for (int m = 0; m < RM; ++m)
#pragma unroll
                for (int j = 0; j < RW; ++j) acc[m][j] = 0.f;
        }
        stage = stage + 1 == NS ? 0 : stage + 1;
    }
    cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------

struct FwdPipePlan {
    FwdPipeArgs a;
    int threads, grid, status, ks, s, rw, rm;
    size_t smem;
};

// How many of these CTAs one SM holds (shared memory and 64 K registers at <= 128 per thread).
static int ctas_per_sm(size_t smem, int threads) {
    const int by_smem = (int)((227 * 1024) / (smem + 1024));
    const int by_regs = 65536 / (128 * threads);
    int c = by_smem < by_regs ? by_smem : by_regs;
    if (c > 2) c = 2;           // __launch_bounds__(256, 2)
    return c < 1 ? 1 : c;
}

template <int KS, int S, int RW, int RM>
static FwdPipePlan plan_fwd_pipe_kg(const Geom& g, const float* out, const TileHint& hint, int kg_forced);

// More reduction groups mean fewer pixels per CTA, i.e. smaller patches: when three stages of a decent
// chunk (4 input channels or more) do not fit, the group count is doubled.
template <int KS, int S, int RW, int RM>
static FwdPipePlan plan_fwd_pipe_t(const Geom& g, const float* out, const TileHint& hint) {
    FwdPipePlan p = plan_fwd_pipe_kg<KS, S, RW, RM>(g, out, hint, 0);
    if (hint.ck > 0) return p;
    for (int kg = p.a.KG * 2; kg <= 4 && g.Ci >= 8 * kg; kg *= 2) {
        if (p.status == ADDER_OK && p.a.CK >= 4 && p.a.CK >= p.a.KG && 2 * (p.smem + 1024) <= 227 * 1024) break;
        p = plan_fwd_pipe_kg<KS, S, RW, RM>(g, out, hint, kg);
    }
    return p;
}

template <int KS, int S, int RW, int RM>
static FwdPipePlan plan_fwd_pipe_kg(const Geom& g, const float* out, const TileHint& hint, int kg_forced) {
    FwdPipePlan p;
    FwdPipeArgs& a = p.a;
    p.status = ADDER_OK;
    p.ks = KS; p.s = S; p.rw = RW; p.rm = RM;
    a.g = g;
    const int sms = sm_count();
    const int threads_target = hint.threads > 0 ? hint.threads : 256;
    // channel groups: 16 output channels per CTA unless the layer has fewer
    const int cg_want = hint.cg > 0 ? hint.cg : (16 / RM > 0 ? 16 / RM : 1);
    a.CG = ceil_div(g.Co, RM) < cg_want ? ceil_div(g.Co, RM) : cg_want;
    a.TM = a.CG * RM;
    a.TMP = a.TM + 4;
    const int spr_full = ceil_div(g.Wo, RW);
    const long long px_threads = (long long)g.N * g.Ho * spr_full;            // one per segment
    const long long all_threads = px_threads * ceil_div(g.Co, RM);
    // reduction groups: split the input channels inside the CTA when the layer has too few register tiles
    // to give every SM 16 warps
    int kg = 1;
    if (hint.ck > 0) kg = hint.ck;      // tuning: the chunk hint carries the group count for this kernel
    else if (kg_forced > 0) kg = kg_forced;
    else {
        while (kg < 4 && all_threads * kg < (long long)sms * 512 && g.Ci >= 8 * kg) kg *= 2;
    }
    a.KG = kg;
    int segs_target = threads_target / (a.CG * a.KG);
    if (segs_target < 8) segs_target = 8;
    // pixel tile: whole rows first, then several rows, then several images
    a.SPR = spr_full <= segs_target ? spr_full : segs_target;
    int rows_target = segs_target / a.SPR;
    if (rows_target < 1) rows_target = 1;
    if (hint.th > 0) a.TH = hint.th < g.Ho ? hint.th : g.Ho;
    else a.TH = largest_divisor_le(g.Ho, rows_target);
    a.TI = 1;
    if (a.TH == g.Ho) {
        a.TI = rows_target / a.TH;
        if (a.TI > g.N) a.TI = g.N;
        if (a.TI < 1) a.TI = 1;
    }
    if (hint.ti > 0) a.TI = hint.ti;
    a.SEGS = a.TI * a.TH * a.SPR;
    const int group = round_up(a.CG * a.SEGS, 32);      // threads of one reduction group (whole warps)
    p.threads = group * a.KG;
    if (p.threads > 256) { p.status = ADDER_ERR_INTERNAL; return p; }
    a.IN_ROWS = (a.TH - 1) * S + KS;
    const int in_cols = (a.SPR * RW - 1) * S + KS;
    {
        const int rows = a.TI * a.TH, th = a.TH, in_rows = a.IN_ROWS;
        a.PITCH = pick_pitch_vec(2 * in_cols, 32, [=](int l, int& row, int& col) {
            const int wsl = l / rows, ri = l % rows;
            row = (ri / th) * in_rows + (ri % th) * S; col = wsl * RW * S * 2; });
    }
    PatchDims& pd = a.pd;
    pd.TI = a.TI; pd.ROWS = a.IN_ROWS; pd.COLS = in_cols; pd.PITCH = a.PITCH; pd.ROWS_PITCH = a.IN_ROWS * a.PITCH;
    pd.d_cols = FastDiv(in_cols); pd.d_rows = FastDiv(a.IN_ROWS);
    a.CH_STRIDE = a.TI * pd.ROWS_PITCH;
    a.red_floats = a.KG > 1 ? (a.KG - 1) * RM * RW * group : 0;
    // channels per chunk: a multiple of the group count, as many as three stages fit into the budget
    const int budget_floats = (hint.smem_kb > 0 ? hint.smem_kb : 100) * 1024 / 4 - a.red_floats;
    int ck = 8 > a.KG ? 8 : a.KG;
    if (ck > g.Ci) ck = g.Ci;
    while (ck > a.KG && FWD_STAGES * (round_up(ck * a.CH_STRIDE, 4) + round_up(ck * KS * KS, 8) * a.TMP) > budget_floats) --ck;
    ck = ceil_div(g.Ci, ceil_div(g.Ci, ck));         // same number of chunks, evenly sized
    if (a.KG > 1) ck = round_up(ck, a.KG);
    a.CK = ck;
    pd.CH = ck;
    a.nchunks = ceil_div(g.Ci, ck);
    a.wkk_pad = round_up(ck * KS * KS, 8);
    a.xs_stage = round_up(ck * a.CH_STRIDE, 4);
    a.ws_stage = a.wkk_pad * a.TMP;
    p.smem = (size_t)(FWD_STAGES * (a.xs_stage + a.ws_stage) + a.red_floats) * sizeof(float);
    if (p.smem > 200 * 1024) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.tiles_h = ceil_div(g.Ho, a.TH);
    a.tiles_w = ceil_div(spr_full, a.SPR);
    const long long px_tiles = (long long)ceil_div(g.N, a.TI) * a.tiles_h * a.tiles_w;
    const long long units = px_tiles * ceil_div(g.Co, a.TM);
    if (units > 2147483647LL || units < 1) { p.status = ADDER_ERR_UNSUPPORTED; return p; }
    a.n_px_tiles = (int)px_tiles;
    a.n_units = (int)units;
    const long long slots = (long long)sms * ctas_per_sm(p.smem, p.threads);
    p.grid = (int)(units < slots ? units : slots);
    a.d_tiles_h = FastDiv(a.tiles_h);
    a.d_tiles_w = FastDiv(a.tiles_w);
    a.d_px_tiles = FastDiv(a.n_px_tiles);
    a.d_nchunks = FastDiv(a.nchunks);
    a.d_group = FastDiv(group);
    a.d_segs = FastDiv(a.SEGS);
    a.d_rows = FastDiv(a.TI * a.TH);
    a.d_th = FastDiv(a.TH);
    a.d_tm = FastDiv(a.TM);
    a.vec_store = (RW % 4 == 0) && (g.Wo % RW == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    return p;
}

template <int KS, int S, int RW, int RM>
static int launch_fwd_pipe_t(const Geom& g, const float* x, const float* w, float* out, const TileHint& hint,
                             cudaStream_t stream) {
    FwdPipePlan p = plan_fwd_pipe_t<KS, S, RW, RM>(g, out, hint);
    if (p.status != ADDER_OK) return p.status;
    p.a.x = x; p.a.w = w; p.a.out = out;
    auto kern = adder_fwd_pipe_kernel<KS, S, RW, RM>;
    const int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), p.smem);
    if (st != ADDER_OK) return st;
    kern<<<p.grid, p.threads, p.smem, stream>>>(p.a);
    return launched();
}

// The persistent kernel covers 3x3 and 1x1 layers of either stride whose rows are cut into 8- or 4-pixel
// segments; planes 7, 14 or 28 wide keep the 7-pixel kernel of adder_fwd.cu.
bool fwd_pipe_applicable(const Geom& g, const TileHint& hint) {
    if (hint.rw == 7) return false;
    if ((g.Wo % 8 != 0) && (g.Wo % 7 == 0)) return false;
    if (g.Co % 4 != 0) return false;        // channel pairs, 128-bit weight loads
    if (hint.variant == 1) return false;    // tuning: force the non-persistent kernel
    return (g.k == 3 || g.k == 1) && (g.stride == 1 || g.stride == 2);
}

static void choose_fwd_pipe_tile(const Geom& g, const TileHint& hint, int& rw, int& rm) {
    if (hint.rw > 0 && hint.rm > 0) { rw = hint.rw; rm = hint.rm; return; }
    rm = 4;
    rw = (g.Wo % 8 == 0 || g.Wo > 16) ? 8 : 4;
}

#define ADDER_FWDP_DISPATCH(CALL)                                                           \
    if (g.k == 3 && g.stride == 1) { ADDER_FWDP_TILES(3, 1, CALL) }                         \
    else if (g.k == 3 && g.stride == 2) { ADDER_FWDP_TILES(3, 2, CALL) }                    \
    else if (g.k == 1 && g.stride == 1) { ADDER_FWDP_TILES(1, 1, CALL) }                    \
    else if (g.k == 1 && g.stride == 2) { ADDER_FWDP_TILES(1, 2, CALL) }
#define ADDER_FWDP_TILES(KS_, S_, CALL)                                                     \
    if (rw == 8 && rm == 8) { CALL(KS_, S_, 8, 8) }                                         \
    else if (rw == 8 && rm == 4) { CALL(KS_, S_, 8, 4) }                                    \
    else if (rw == 4 && rm == 4) { CALL(KS_, S_, 4, 4) }                                    \
    else if (rw == 4 && rm == 8) { CALL(KS_, S_, 4, 8) }

int describe_fwd_pipe(const Geom& g, const TileHint& hint, char* buf, size_t n) {
    int rw = 8, rm = 4;
    choose_fwd_pipe_tile(g, hint, rw, rm);
    FwdPipePlan p;
    p.status = ADDER_ERR_UNSUPPORTED;
#define ADDER_FWDP_PLAN(KS_, S_, RW_, RM_) p = plan_fwd_pipe_t<KS_, S_, RW_, RM_>(g, nullptr, hint);
    ADDER_FWDP_DISPATCH(ADDER_FWDP_PLAN)
#undef ADDER_FWDP_PLAN
    snprintf(buf, n,
             "fwd persistent k=%d s=%d RW=%d RM=%d CG=%d KG=%d TM=%d TI=%d TH=%d SPR=%d SEGS=%d CK=%d chunks=%d rows=%d "
             "cols=%d pitch=%d stages=%d threads=%d smem=%zu units=%d grid=(%d,1) status=%d",
             p.ks, p.s, p.rw, p.rm, p.a.CG, p.a.KG, p.a.TM, p.a.TI, p.a.TH, p.a.SPR, p.a.SEGS, p.a.CK, p.a.nchunks,
             p.a.IN_ROWS, p.a.pd.COLS, p.a.PITCH, FWD_STAGES, p.threads, p.smem, p.a.n_units, p.grid, p.status);
    return ADDER_OK;
}

int launch_fwd_pipe(const Geom& g, const float* x, const float* w, float* out, const TileHint& hint,
                    cudaStream_t stream) {
    int rw = 8, rm = 4;
    choose_fwd_pipe_tile(g, hint, rw, rm);
#define ADDER_FWDP_LAUNCH(KS_, S_, RW_, RM_) return launch_fwd_pipe_t<KS_, S_, RW_, RM_>(g, x, w, out, hint, stream);
    ADDER_FWDP_DISPATCH(ADDER_FWDP_LAUNCH)
#undef ADDER_FWDP_LAUNCH
    return ADDER_ERR_UNSUPPORTED;
}

}  // namespace adder
