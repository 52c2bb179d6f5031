// Forward adder convolution on NCHW tensors with implicit im2col:
//   out[n,co,ho,wo] = - sum_{ci,kh,kw} | xpad[n,ci,ho*S+kh,wo*S+kw] - w[co,ci,kh,kw] |
// (the reference computes the same sum on a materialised column matrix: adder.py:32-39 feeding
// the CONV kernel of adder_cuda/adder.cu:19-70).  Padding pixels are zero-valued inputs that
// still contribute |0 - w|, exactly as F.unfold presents them to the reference kernel.
//
// Work decomposition.  A CTA owns TM = CG*RM output channels and a pixel tile of TI images x TH
// output rows x SPR row segments of RW consecutive output pixels; a thread owns one segment and RM
// channels, i.e. an RM x RW register tile (8x8, 8x4, 4x4 or 7x8 pixels x channels, chosen by the
// launcher from the layer size).  Input channels are streamed in chunks of CK through a
// double-buffered shared-memory stage holding the haloed input patch [CK][TI*IN_ROWS][PITCH] and the
// weight slab [CK*KS*KS][TM+4] (channel innermost, so a thread's RM weights are 128-bit loads that
// the whole warp shares).  For each (ci, kh) a thread loads the (RW-1)*S+KS input values its segment
// touches once (128-/64-bit loads) and slides the KS taps over them in registers.  Per pair of
// channels one packed add.f32x2 forms both differences and two scalar adds accumulate |d|:
// 1.5 issue slots and 2 FP32-pipe slots per |x-w| term.
#ifndef ADDER_FWD_PACKED
#define ADDER_FWD_PACKED 1
#endif
#include "common.cuh"
#include "kernels.h"
#include "patch_fill.cuh"
#include <cstdio>

namespace adder {

template <int KS, int S, int RW, int RM>
__global__ void __launch_bounds__(256, 2) adder_fwd_kernel(const FwdArgs a) {
    constexpr int KK = KS * KS;
    constexpr int XW = (RW - 1) * S + KS;   // input values one segment touches per (ci, kh)
    extern __shared__ __align__(16) float smem[];
    float* const Xs = smem;
    float* const Ws = smem + a.nstages * a.xs_stage;

    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    uint32_t tn, th, tw, tnh;
    a.d_tiles_w.divmod(blockIdx.x, tnh, tw);
    a.d_tiles_h.divmod(tnh, tn, th);
    const int n0 = tn * a.TI;
    const int ho0 = th * a.TH;
    const int wo_t0 = tw * (a.SPR * RW);      // first output column of this tile
    const int wi0 = wo_t0 * S * a.pd.GS - a.g.pad;      // input column of patch column 0
    const int co0 = blockIdx.y * (a.CG * RM);
    const int hi0 = ho0 * S * a.pd.GS - a.g.pad;       // input row of patch row 0

    // thread role: (channel group, segment); segment -> (image, tile row, segment within row)
    uint32_t cg, seg, t2, ws, img, hr;
    a.d_segs.divmod(tid, cg, seg);
    a.d_spr.divmod(seg, t2, ws);
    a.d_th.divmod(t2, img, hr);
    const bool active = (int)cg < a.CG;
    const int xoff = (img * a.IN_ROWS + hr * S) * a.PITCH + ws * (RW * S);

    float acc[RM][RW];
#pragma unroll
    for (int m = 0; m < RM; ++m)
#pragma unroll
        for (int j = 0; j < RW; ++j) acc[m][j] = 0.f;

    const int K = a.g.Ci * KK;
    const int nchunks = ceil_div(a.g.Ci, a.CK);
    const int w_elems = a.wkk_pad * a.TM;      // wkk_pad = round_up(CK*KK, 8)

    auto fill = [&](int chunk, int stage) {
        const int ci0 = chunk * a.CK;
        if (KS == 1 && a.x_quads)
            fill_patch_quads(Xs + stage * a.xs_stage, a.x, a.pd, a.d_xquads, n0, ci0, hi0, wi0, a.g.N, a.g.Ci, a.g.H, a.g.W,
                             tid, nthreads);
        else
            fill_patch(Xs + stage * a.xs_stage, a.x, a.pd, n0, ci0, hi0, wi0, a.g.N, a.g.Ci, a.g.H, a.g.W, tid, nthreads);
        float* wsm = Ws + stage * a.ws_stage;
        const int kbase = ci0 * KK;
        const int kk_lim = a.CK * KK;
        // slab layout [ci][channel group][tap][RM]: a thread's RM channels of one tap are 128-bit loads, and the
        // taps of one input channel sit at compile-time offsets from each other
        for (int e = tid; e < w_elems; e += nthreads) {
            uint32_t t, col, kkb;
            const int kk8 = e & 7;
            t = e >> 3;
            a.d_tm.divmod(t, kkb, col);
            const int kk = kkb * 8 + kk8;
            if (kk >= kk_lim) continue;
            const int co = co0 + col;
            const bool ok = (co < a.g.Co) & (kbase + kk < K);
            const float* src = ok ? a.w + ((size_t)co * K + kbase + kk) : a.w;
            const int cil = kk / KK, tap = kk - cil * KK;
            cp_async4(wsm + cil * a.WCIL + ((col / RM) * KK + tap) * RM + (col % RM), src, ok);
        }
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
        __syncthreads();
        if (active) {
            const float* xc = Xs + (c & 1) * a.xs_stage + xoff;
            const float* wc = Ws + (c & 1) * a.ws_stage + cg * (KK * RM);
            const int nch = min(a.CK, a.g.Ci - c * a.CK);
#pragma unroll 1
            for (int cil = 0; cil < nch; ++cil, xc += a.CH_STRIDE, wc += a.WCIL) {
                const float* xr = xc;
#pragma unroll
                for (int kh = 0; kh < KS; ++kh, xr += a.PITCH) {
                    float xv[XW];
                    load_run<XW, (RW % 4 == 0)>(xv, xr);
#if ADDER_FWD_PACKED
                    uint64_t nx2[XW];
#pragma unroll
                    for (int i = 0; i < XW; ++i) nx2[i] = pack2(-xv[i], -xv[i]);
#endif
#pragma unroll
                    for (int kw = 0; kw < KS; ++kw) {
                        const float* wr = wc + (kh * KS + kw) * RM;
                        float wv[RM];
#pragma unroll
                        for (int m4 = 0; m4 < RM; m4 += 4) {
                            const float4 t = *reinterpret_cast<const float4*>(wr + m4);
                            wv[m4] = t.x; wv[m4 + 1] = t.y; wv[m4 + 2] = t.z; wv[m4 + 3] = t.w;
                        }
#if ADDER_FWD_PACKED
                        // |w - x| for two channels at once: one packed subtract, then two scalar add-abs
#pragma unroll
                        for (int m = 0; m < RM; m += 2) {
                            const uint64_t w2 = pack2(wv[m], wv[m + 1]);
#pragma unroll
                            for (int j = 0; j < RW; ++j) {
                                float d0, d1;
                                unpack2(add2(w2, nx2[j * S + kw]), d0, d1);
                                acc[m][j] += fabsf(d0);
                                acc[m + 1][j] += fabsf(d1);
                            }
                        }
#else
#pragma unroll
                        for (int m = 0; m < RM; ++m)
#pragma unroll
                            for (int j = 0; j < RW; ++j) acc[m][j] += fabsf(xv[j * S + kw] - wv[m]);
#endif
                    }
                }
            }
        }
        __syncthreads();
    }

    const int n = n0 + img, ho = ho0 + hr, wo0 = wo_t0 + ws * RW;
    const bool valid = active && n < a.g.N && ho < a.g.Ho && wo0 < a.g.Wo;
    if (valid) {
        const int HoWo = a.g.Ho * a.g.Wo;
#pragma unroll
        for (int m = 0; m < RM; ++m) {
            const int co = co0 + cg * RM + m;
            if (co >= a.g.Co) break;
            float* o = a.out + ((size_t)(n * a.g.Co + co) * HoWo + ho * a.g.Wo + wo0);
            if (RW % 4 == 0 && a.vec_store) {
#pragma unroll
                for (int j = 0; j < RW; j += 4)
                    *reinterpret_cast<float4*>(o + j) = make_float4(-acc[m][j], -acc[m][j + 1], -acc[m][j + 2], -acc[m][j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < RW; ++j)
                    if (wo0 + j < a.g.Wo) o[j] = -acc[m][j];
            }
        }
    }
    if (a.stats == nullptr) return;

    // Batch-norm statistics of this pixel tile: for each of the CTA's channels the sum of its outputs and of
    // their squares.  A thread adds its (at most RW) values in fp32; everything after that is double, in a
    // fixed order, so the slices can be combined without cancellation although no pivot is subtracted.
    float2* st = reinterpret_cast<float2*>(smem);           // [TM][SEGS]; the stages are free after the last barrier
    if (active) {
#pragma unroll
        for (int m = 0; m < RM; ++m) {
            float s = 0.f, q = 0.f;
            if (valid) {
#pragma unroll
                for (int j = 0; j < RW; ++j)
                    if (wo0 + j < a.g.Wo) { s -= acc[m][j]; q = fmaf(acc[m][j], acc[m][j], q); }
            }
            st[(cg * RM + m) * a.SEGS + seg] = make_float2(s, q);
        }
    }
    __syncthreads();
    const int tpc = a.stat_tpc;                             // power of two <= 32: the lanes of one channel sit in one warp
    if ((tid & ~31) >= a.TM * tpc) return;                  // whole warps only: the shuffles below need every lane
    const int ch = tid / tpc, l = tid - ch * tpc;
    double ds = 0.0, dq = 0.0;
    if (ch < a.TM) {
        const float2* row = st + ch * a.SEGS;
        for (int e = l; e < a.SEGS; e += tpc) { const float2 v = row[e]; ds += (double)v.x; dq += (double)v.y; }
    }
    for (int off = tpc >> 1; off > 0; off >>= 1) {
        ds += __shfl_xor_sync(0xffffffffu, ds, off);
        dq += __shfl_xor_sync(0xffffffffu, dq, off);
    }
    if (l == 0 && ch < a.TM && co0 + ch < a.g.Co) {
        double* o = a.stats + ((size_t)(co0 + ch) * a.stat_slices + blockIdx.x) * 2;
        o[0] = ds; o[1] = dq;
    }
}

// ------------------------------------------------------------------------------------------
// host side: tile plan + launch
// ------------------------------------------------------------------------------------------

// Smallest row pitch >= cols for which the 32 lanes of a warp (consecutive segments) read
// distinct shared-memory banks as often as possible; the cost is the worst bank multiplicity.
static int pick_pitch(int cols, int segs, int spr, int th, int in_rows, int seg_step, int row_step) {
    int best = cols, best_cost = 1 << 30;
    for (int pitch = cols; pitch < cols + 33; ++pitch) {
        int cost = 0;
        for (int w0 = 0; w0 < segs; w0 += 32) {
            int cnt[32] = {0};
            int worst = 0;
            for (int l = w0; l < w0 + 32 && l < segs; ++l) {
                const int ws = l % spr, t2 = l / spr, hr = t2 % th, img = t2 / th;
                const int addr = (img * in_rows + hr * row_step) * pitch + ws * seg_step;
                const int b = addr & 31;
                if (++cnt[b] > worst) worst = cnt[b];
            }
            cost += worst;
        }
        if (cost < best_cost) { best_cost = cost; best = pitch; }
    }
    return best;
}

struct FwdPlan {
    FwdArgs a;
    int threads, status, ks, s, rw, rm;
    size_t smem;
    long long gx;
    int gy;
};

template <int KS, int S, int RW, int RM>
static int plan_fwd_t(const Geom& g, const float* out, const TileHint& hint, FwdPlan& p) {
    if (hint.threads == 0) {
        // 128 threads per CTA unless that leaves the launch with fewer CTAs than two per SM (the deep, small
        // planes: 64->64 on 8x8 at batch 256 has 256 of them): then 256 threads, i.e. twice the channels per
        // CTA, so that every staged input patch is used twice as often (60 -> 56 us on that layer) - as long as
        // that still leaves about one CTA per SM.
        TileHint h2 = hint;
        if (KS == 1 && g.Co >= 64) {
            // 1x1 layers: one tap per staged input value, so twice the channels per CTA pays on every size
            // (1024->256 14x14: 429 -> 380 us)
            h2.threads = 256;
            if (plan_fwd_t<KS, S, RW, RM>(g, out, h2, p) == ADDER_OK) return ADDER_OK;
        }
        h2.threads = 128;
        const int st = plan_fwd_t<KS, S, RW, RM>(g, out, h2, p);
        if (st == ADDER_OK && p.gx * p.gy < 2LL * sm_count() && g.Co > p.a.TM) {
            FwdPlan q;
            h2.threads = 256;
            if (plan_fwd_t<KS, S, RW, RM>(g, out, h2, q) == ADDER_OK && 4 * q.gx * q.gy >= 3LL * sm_count()) p = q;
        }
        return st;
    }
    FwdArgs& a = p.a;
    p.ks = KS; p.s = S; p.rw = RW; p.rm = RM;
    a.g = g;
    const int threads_target = hint.threads;
    // few channel groups per CTA: the weight slab is re-staged by every CTA, the pixels are not
    const int cg_max = hint.cg > 0 ? hint.cg : (threads_target / 32 > 2 ? threads_target / 32 : 2);
    a.CG = ceil_div(g.Co, RM) < cg_max ? ceil_div(g.Co, RM) : cg_max;
    a.TM = a.CG * RM;
    a.TMP = a.TM + 4;
    int segs_target = threads_target / a.CG;
    if (segs_target < 1) segs_target = 1;
    const int spr_full = ceil_div(g.Wo, RW);   // segments in a full output row
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
    int ti_budget = 1;   // tile images before clamping to the batch: the chunk size must not depend on N
    if (a.TH == g.Ho) {
        a.TI = rows_target / a.TH;
        ti_budget = a.TI > 1 ? a.TI : 1;
        if (a.TI < 1) a.TI = 1;
        if (a.TI > g.N) a.TI = g.N;
        if (a.TI < 1) a.TI = 1;
    }
    if (hint.ti > 0) a.TI = hint.ti;
    a.SEGS = a.TI * a.TH * a.SPR;
    const int threads = round_up(a.CG * a.SEGS, 32);
    p.threads = threads;
    if (threads > 256) return ADDER_ERR_INTERNAL;
    a.IN_ROWS = (a.TH - 1) * S + KS;
    a.IN_COLS = (a.SPR * RW - 1) * S + KS;
    if (RW % 4 == 0) {
        const int spr = a.SPR, th = a.TH, rows = a.IN_ROWS, segs = a.SEGS;
        a.PITCH = pick_pitch_vec(a.IN_COLS, segs < 32 ? segs : 32, [=](int l, int& row, int& col) {
            const int ws = l % spr, t2 = l / spr;
            row = (t2 / th) * rows + (t2 % th) * S; col = ws * RW * S; });
    } else {
        a.PITCH = pick_pitch(a.IN_COLS, a.SEGS, a.SPR, a.TH, a.IN_ROWS, RW * S, S);
    }
    a.ROWS_PITCH = a.IN_ROWS * a.PITCH;
    a.pd.TI = a.TI; a.pd.ROWS = a.IN_ROWS; a.pd.COLS = a.IN_COLS; a.pd.PITCH = a.PITCH; a.pd.ROWS_PITCH = a.ROWS_PITCH;
    a.pd.d_cols = FastDiv(a.IN_COLS); a.pd.d_rows = FastDiv(a.IN_ROWS);
    // A strided 1x1 layer is a stride-1 layer on the sampled pixels: the kernel runs its stride-1 form (S = 1)
    // and the patch fill gathers every g.stride-th row and column, so nothing unsampled is staged.
    a.pd.GS = (KS == 1 && S == 1) ? g.stride : 1;
    // 1x1 stride-1 layers have no halo: where rows and tiles are whole quads the patch moves in 16-byte copies
    a.x_quads = (KS == 1 && S == 1 && g.stride == 1 && g.pad == 0 && a.IN_COLS % 4 == 0 && a.PITCH % 4 == 0 && g.W % 4 == 0 &&
                 (a.SPR * RW) % 4 == 0) ? 1 : 0;
    a.d_xquads = FastDiv(a.IN_COLS >= 4 ? a.IN_COLS / 4 : 1);
    a.CH_STRIDE = a.TI * a.ROWS_PITCH;
    // channel chunk: fill the shared-memory budget (two CTAs per SM) without exceeding Ci
    // shared memory per CTA in proportion to its threads, so that about 16 warps stay resident per SM
    const int budget_floats = (hint.smem_kb > 0 ? hint.smem_kb : 100) * 1024 / 4;
    int ck = hint.ck > 0 ? hint.ck : (KS == 1 ? 32 : 16);
    if (ck > g.Ci) ck = g.Ci;
    // All input channels in ONE chunk need no second stage; where that fits the budget it is taken (no chunk barrier).
    bool whole = false;
    if (hint.ck <= 0 && KS == 3 && g.Ci <= 64 &&
        round_up(g.Ci * ti_budget * a.ROWS_PITCH, 4) + g.Ci * KS * KS * a.TM <= budget_floats) {
        ck = g.Ci;
        whole = true;
    }
    while (ck > 1 && !whole) {
        const int need = 2 * (round_up(ck * ti_budget * a.ROWS_PITCH, 4) + ck * KS * KS * a.TM);
        if (need <= budget_floats) break;
        --ck;
    }
    ck = ceil_div(g.Ci, ceil_div(g.Ci, ck));      // same number of chunks, evenly sized: no padded channels
    a.CK = ck;
    a.pd.CH = ck;
    a.wkk_pad = round_up(a.CK * KS * KS, 8);
    a.xs_stage = round_up(a.CK * a.CH_STRIDE, 4);
    a.WCIL = a.TM * KS * KS;
    a.ws_stage = a.CK * a.WCIL;
    a.nstages = a.CK < g.Ci ? 2 : 1;
    size_t smem = (size_t)a.nstages * (a.xs_stage + a.ws_stage) * sizeof(float);
    const size_t stat_bytes = (size_t)a.TM * a.SEGS * sizeof(float2);   // the statistics epilogue reuses the stages
    if (smem < stat_bytes) smem = stat_bytes;
    p.smem = smem;
    a.stats = nullptr; a.stat_slices = 0;
    a.stat_tpc = 32;
    while (a.stat_tpc > 1 && a.TM * a.stat_tpc > threads) a.stat_tpc >>= 1;
    if (smem > 200 * 1024) return ADDER_ERR_UNSUPPORTED;
    a.tiles_h = ceil_div(g.Ho, a.TH);
    a.tiles_w = ceil_div(spr_full, a.SPR);
    const int tiles_n = ceil_div(g.N, a.TI);
    a.d_tiles_h = FastDiv(a.tiles_h);
    a.d_tiles_w = FastDiv(a.tiles_w);
    a.d_segs = FastDiv(a.SEGS);
    a.d_spr = FastDiv(a.SPR);
    a.d_th = FastDiv(a.TH);
    a.d_tm = FastDiv(a.TM);
    a.vec_store = (RW % 4 == 0) && (g.Wo % RW == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    const long long gx = (long long)tiles_n * a.tiles_h * a.tiles_w;
    const int gy = ceil_div(g.Co, a.TM);
    p.gx = gx; p.gy = gy;
    if (gx > 2147483647LL || gy > 65535) return ADDER_ERR_UNSUPPORTED;
    return ADDER_OK;
}

template <int KS, int S, int RW, int RM>
static int launch_fwd_t(const Geom& g, const float* x, const float* w, float* out, const TileHint& hint,
                        cudaStream_t stream, double* stats, int stat_slices) {
    FwdPlan p;
    const int st = plan_fwd_t<KS, S, RW, RM>(g, out, hint, p);
    if (st != ADDER_OK) return st;
    p.a.x = x; p.a.w = w; p.a.out = out;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) p.a.x_quads = 0;
    if (stats != nullptr) {
        if ((long long)stat_slices != p.gx || p.a.TM * p.a.stat_tpc > p.threads) return ADDER_ERR_WORKSPACE;
        p.a.stats = stats; p.a.stat_slices = stat_slices;
    }
    auto kern = adder_fwd_kernel<KS, S, RW, RM>;
    const int se = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), p.smem);
    if (se != ADDER_OK) return se;
    kern<<<dim3((unsigned)p.gx, (unsigned)p.gy), p.threads, p.smem, stream>>>(p.a);
    return launched();
}

// Register tile (pixels x channels per thread).  The widest tile has the fewest shared-memory loads
// per |x-w| term, but a layer with few pixels and channels then has too few threads to keep 148 SMs
// busy (64->64 on 8x8 at batch 256 would run on 512 warps), so narrower tiles are chosen until the
// launch has about 16 warps per SM.  Planes that are 7, 14 or 28 wide use 7-pixel segments.
static void choose_fwd_tile(const Geom& g, const TileHint& hint, int& rw, int& rm) {
    if (hint.rw > 0 && hint.rm > 0) { rw = hint.rw; rm = hint.rm; return; }
    const bool one_row = (g.k == 1 && g.H == 1);     // flattened 1x1 layer or column matrix: a ragged last segment costs little
    if (!one_row && (g.Wo % 8 != 0) && (g.Wo % 7 == 0)) { rw = 7; rm = 8; return; }
    if (g.Wo % 4 != 0) { rw = 8; rm = 8; return; }
    const int cand[3][2] = {{8, 8}, {8, 4}, {4, 4}};
    const long long want[3] = {100000, 30000, 0};     // thresholds found by sweeping the ResNet-20 layer shapes
    for (int c = 0; c < 3; ++c) {
        rw = cand[c][0]; rm = cand[c][1];
        if (g.Wo % rw != 0 && rw == 8 && !one_row) continue;
        const long long threads = (long long)g.N * g.Ho * ceil_div(g.Wo, rw) * ceil_div(g.Co, rm);
        if (threads >= want[c]) return;
    }
}

#define ADDER_FWD_DISPATCH(CALL)                                                            \
    if (g.k == 3 && g.stride == 1) { ADDER_FWD_TILES(3, 1, CALL) }                          \
    else if (g.k == 3 && g.stride == 2) { ADDER_FWD_TILES(3, 2, CALL) }                     \
    else if (g.k == 1 && g.stride == 1) { ADDER_FWD_TILES(1, 1, CALL) }                     \
    else if (g.k == 1 && g.stride == 2) { ADDER_FWD_TILES(1, 1, CALL) }
#define ADDER_FWD_TILES(KS_, S_, CALL)                                                      \
    if (rw == 7) { CALL(KS_, S_, 7, 8) }                                                    \
    else if (rw == 8 && rm == 8) { CALL(KS_, S_, 8, 8) }                                    \
    else if (rw == 8 && rm == 4) { CALL(KS_, S_, 8, 4) }                                    \
    else if (rw == 4 && rm == 4) { CALL(KS_, S_, 4, 4) }

int describe_fwd(const Geom& layer, const TileHint& hint, char* buf, size_t n) {
    const Geom g = flatten_pointwise(layer);
    if (hint.is_default() && pointwise_applicable(g)) {
        snprintf(buf, n, "fwd k=1 s=%d pointwise: one thread per output position, 16 output channels per CTA, threads=256 "
                 "grid=(%d,%d) status=0", g.stride, ceil_div(g.N * g.Ho * g.Wo, 256), ceil_div(g.Co, 16));
        return ADDER_OK;
    }
    int rw = 8, rm = 8;
    choose_fwd_tile(g, hint, rw, rm);
    FwdPlan p;
    int st = ADDER_ERR_UNSUPPORTED;
#define ADDER_FWD_PLAN(KS_, S_, RW_, RM_) st = plan_fwd_t<KS_, S_, RW_, RM_>(g, nullptr, hint, p);
    ADDER_FWD_DISPATCH(ADDER_FWD_PLAN)
#undef ADDER_FWD_PLAN
    if (st == ADDER_ERR_UNSUPPORTED && !((g.k == 1 || g.k == 3) && (g.stride == 1 || g.stride == 2))) return st;
    snprintf(buf, n,
             "fwd k=%d s=%d RW=%d RM=%d CG=%d TM=%d TI=%d TH=%d SPR=%d SEGS=%d CK=%d rows=%d cols=%d pitch=%d "
             "threads=%d smem=%zu grid=(%lld,%d) status=%d",
             p.ks, p.s, p.rw, p.rm, p.a.CG, p.a.TM, p.a.TI, p.a.TH, p.a.SPR, p.a.SEGS, p.a.CK, p.a.IN_ROWS, p.a.IN_COLS,
             p.a.PITCH, p.threads, p.smem, p.gx, p.gy, st);
    return ADDER_OK;
}

int fwd_stat_slices(const Geom& layer, const TileHint& hint) {
    const Geom g = flatten_pointwise(layer);
    if (hint.is_default() && pointwise_applicable(g)) return 0;
    int rw = 8, rm = 8;
    choose_fwd_tile(g, hint, rw, rm);
    FwdPlan p;
    int st = ADDER_ERR_UNSUPPORTED;
#define ADDER_FWD_PLAN(KS_, S_, RW_, RM_) st = plan_fwd_t<KS_, S_, RW_, RM_>(g, nullptr, hint, p);
    ADDER_FWD_DISPATCH(ADDER_FWD_PLAN)
#undef ADDER_FWD_PLAN
    if (st != ADDER_OK || p.a.TM * p.a.stat_tpc > p.threads || p.gx > (1 << 20)) return 0;
    return (int)p.gx;
}

int launch_fwd(const Geom& layer, const float* x, const float* w, float* out, const TileHint& hint,
               cudaStream_t stream, double* stats, int stat_slices) {
    const Geom g = flatten_pointwise(layer);
    if (hint.is_default() && pointwise_applicable(g)) {
        if (stats != nullptr) return ADDER_ERR_UNSUPPORTED;
        return launch_pointwise_fwd(g, x, w, out, stream);
    }
    int rw = 8, rm = 8;
    choose_fwd_tile(g, hint, rw, rm);
#define ADDER_FWD_LAUNCH(KS_, S_, RW_, RM_) \
    return launch_fwd_t<KS_, S_, RW_, RM_>(g, x, w, out, hint, stream, stats, stat_slices);
    ADDER_FWD_DISPATCH(ADDER_FWD_LAUNCH)
#undef ADDER_FWD_LAUNCH
    return ADDER_ERR_UNSUPPORTED;
}

}  // namespace adder
