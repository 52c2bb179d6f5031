// 1x1, stride-2, unpadded adder layers with few channels (the downsample branches of ResNet-20,
// resnet20.py:66-70: 16->32 and 32->64 channels).  With K = Ci = 16 or 32 these layers do about 6
// operations per byte and are bound by memory traffic, not by FP32 issue, and the tiled kernels spend
// most of their time staging patches they hardly use.  Here one thread owns one output position
// (n, ho, wo) <-> input pixel (n, 2ho, 2wo): it reads its 16 input channels (forward, input gradient)
// straight from global memory into registers, streams the other operand once, and the weights of the
// CTA's channel group sit in shared memory and are read as broadcast 128-bit loads.
//   forward         out[n,co,ho,wo]    = -sum_ci |x[n,ci,2ho,2wo] - w[co,ci]|            (adder.cu:19-70)
//   input gradient  gx[n,ci,2ho,2wo]   = sum_co clamp(w[co,ci] - x, -1, 1) * g[n,co,ho,wo], and 0 at the
//                   pixels no output reads (adder.cu:245-246 followed by col2im, adder.py:32-33)
// Lanes of a warp are consecutive wo, so the stride-2 reads of x use half of every sector and everything
// else is fully coalesced.
#include "common.cuh"
#include "kernels.h"

namespace adder {

constexpr int PW_THREADS = 256;
constexpr int PW_CT = 16;          // channels per thread (register tile) and per CTA channel group

struct PwArgs {
    const float* x;      // [N,Ci,H,W]
    const float* w;      // [Co,Ci]
    const float* g;      // [N,Co,Ho,Wo]   (input gradient only)
    float* out;          // forward: [N,Co,Ho,Wo]; input gradient: [N,Ci,H,W]
    int N, Ci, Co, H, W, Ho, Wo, S, P, accumulate, vec2;
    FastDiv d_wo, d_howo;
};

bool pointwise_applicable(const Geom& g) {
    // an empty batch goes to the tiled kernels, whose CTAs write all-zero slices for an empty tile range
    return g.N >= 1 && g.k == 1 && g.pad == 0 && g.stride == 2 && g.Ci <= 64 && g.Co <= 64 &&
           (long long)g.N * g.Ho * g.Wo < 2147483647LL;
}

static PwArgs make_pw_args(const Geom& g) {
    PwArgs a;
    a.x = nullptr; a.w = nullptr; a.g = nullptr; a.out = nullptr;
    a.N = g.N; a.Ci = g.Ci; a.Co = g.Co; a.H = g.H; a.W = g.W; a.Ho = g.Ho; a.Wo = g.Wo; a.S = g.stride;
    a.P = g.N * g.Ho * g.Wo;
    a.accumulate = 0; a.vec2 = 0;
    a.d_wo = FastDiv(g.Wo);
    a.d_howo = FastDiv(g.Ho * g.Wo);
    return a;
}

// grid (ceil(P/256), ceil(Co/16)); CIT = input channels held in registers (Ci rounded up to 16).
template <int CIT>
__global__ void __launch_bounds__(PW_THREADS) adder_pw_fwd_kernel(const PwArgs a) {
    __shared__ __align__(16) float ws[CIT * PW_CT];       // [ci][co of the group]
    const int co0 = blockIdx.y * PW_CT;
    for (int e = threadIdx.x; e < CIT * PW_CT; e += PW_THREADS) {
        const int ci = e / PW_CT, co = co0 + e % PW_CT;
        ws[e] = (ci < a.Ci && co < a.Co) ? __ldg(a.w + (size_t)co * a.Ci + ci) : 0.f;
    }
    __syncthreads();
    const int p = blockIdx.x * PW_THREADS + threadIdx.x;
    if (p >= a.P) return;
    uint32_t n, r, ho, wo;
    a.d_howo.divmod(p, n, r);
    a.d_wo.divmod(r, ho, wo);
    const int HW = a.H * a.W;
    const float* xp = a.x + (size_t)n * a.Ci * HW + (size_t)(ho * a.S) * a.W + wo * a.S;
    float xv[CIT];
#pragma unroll
    for (int ci = 0; ci < CIT; ++ci) xv[ci] = ci < a.Ci ? __ldg(xp + (size_t)ci * HW) : 0.f;   // padded pairs give |0-0|
    float acc[PW_CT];
#pragma unroll
    for (int m = 0; m < PW_CT; ++m) acc[m] = 0.f;
#pragma unroll
    for (int ci = 0; ci < CIT; ++ci) {
#pragma unroll
        for (int q = 0; q < PW_CT; q += 4) {
            const float4 t = *reinterpret_cast<const float4*>(ws + ci * PW_CT + q);
            acc[q] += fabsf(xv[ci] - t.x);
            acc[q + 1] += fabsf(xv[ci] - t.y);
            acc[q + 2] += fabsf(xv[ci] - t.z);
            acc[q + 3] += fabsf(xv[ci] - t.w);
        }
    }
    const int HoWo = a.Ho * a.Wo;
    float* o = a.out + ((size_t)n * a.Co + co0) * HoWo + r;
#pragma unroll
    for (int m = 0; m < PW_CT; ++m)
        if (co0 + m < a.Co) o[(size_t)m * HoWo] = -acc[m];
}

// grid (ceil(P/256), ceil(Ci/16)).  FAST: clamp(d,-1,1) = 2*sat(d/2 + 1/2) - 1 with w' = w/2 + 1/2 in
// shared memory and x' = -x/2 in registers; the correction is the sum of g over the output channels.
template <bool FAST>
__global__ void __launch_bounds__(PW_THREADS) adder_pw_gx_kernel(const PwArgs a) {
    extern __shared__ __align__(16) float wt[];            // [co][ci of the group]
    const int ci0 = blockIdx.y * PW_CT;
    for (int e = threadIdx.x; e < a.Co * PW_CT; e += PW_THREADS) {
        const int co = e / PW_CT, ci = ci0 + e % PW_CT;
        const float v = ci < a.Ci ? __ldg(a.w + (size_t)co * a.Ci + ci) : 0.f;
        wt[e] = FAST ? fmaf(v, 0.5f, 0.5f) : v;
    }
    __syncthreads();
    const int p = blockIdx.x * PW_THREADS + threadIdx.x;
    if (p >= a.P) return;
    uint32_t n, r, ho, wo;
    a.d_howo.divmod(p, n, r);
    a.d_wo.divmod(r, ho, wo);
    const int HW = a.H * a.W, HoWo = a.Ho * a.Wo;
    const int hi = ho * a.S, wi = wo * a.S;
    const size_t xoff = ((size_t)n * a.Ci + ci0) * HW + (size_t)hi * a.W + wi;
    float xv[PW_CT], acc[PW_CT];
#pragma unroll
    for (int c = 0; c < PW_CT; ++c) {
        const float v = ci0 + c < a.Ci ? __ldg(a.x + xoff + (size_t)c * HW) : 0.f;
        xv[c] = FAST ? -0.5f * v : v;
        acc[c] = 0.f;
    }
    const float* gp = a.g + (size_t)n * a.Co * HoWo + r;
    float gsum = 0.f;
#pragma unroll 4
    for (int co = 0; co < a.Co; ++co) {
        const float gv = __ldg(gp + (size_t)co * HoWo);
        gsum += gv;
        const float* wr = wt + co * PW_CT;
#pragma unroll
        for (int q = 0; q < PW_CT; q += 4) {
            const float4 t = *reinterpret_cast<const float4*>(wr + q);
            const float wv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float s = FAST ? __saturatef(wv[k] + xv[q + k]) : fminf(fmaxf(wv[k] - xv[q + k], -1.f), 1.f);
                acc[q + k] = fmaf(s, gv, acc[q + k]);
            }
        }
    }
    // the S x S block of input pixels that belongs to this output position: the sampled pixel gets the
    // gradient, the others are read by no output and get zero (left untouched when accumulating)
    float* o = a.out + xoff;
#pragma unroll
    for (int c = 0; c < PW_CT; ++c) {
        if (ci0 + c >= a.Ci) break;
        const float v = FAST ? 2.f * acc[c] - gsum : acc[c];
        float* oc = o + (size_t)c * HW;
        if (a.accumulate) {
            oc[0] += v;
            continue;
        }
        if (a.vec2) {          // S == 2, W even, 8-byte aligned rows: both pixels of a row in one store
            *reinterpret_cast<float2*>(oc) = make_float2(v, 0.f);
            if (hi + 1 < a.H) *reinterpret_cast<float2*>(oc + a.W) = make_float2(0.f, 0.f);
        } else {
            for (int dy = 0; dy < a.S && hi + dy < a.H; ++dy)
                for (int dx = 0; dx < a.S && wi + dx < a.W; ++dx) oc[dy * a.W + dx] = (dy == 0 && dx == 0) ? v : 0.f;
        }
    }
}

int launch_pointwise_fwd(const Geom& g, const float* x, const float* w, float* out, cudaStream_t stream) {
    PwArgs a = make_pw_args(g);
    a.x = x; a.w = w; a.out = out;
    const dim3 grid(ceil_div(a.P, PW_THREADS), ceil_div(g.Co, PW_CT));
    if (g.Ci <= 16) adder_pw_fwd_kernel<16><<<grid, PW_THREADS, 0, stream>>>(a);
    else if (g.Ci <= 32) adder_pw_fwd_kernel<32><<<grid, PW_THREADS, 0, stream>>>(a);
    else adder_pw_fwd_kernel<64><<<grid, PW_THREADS, 0, stream>>>(a);
    return launched();
}

int launch_pointwise_gx(const Geom& g, const float* gout, const float* x, const float* w, float* gx, int fast,
                        int accumulate, cudaStream_t stream) {
    PwArgs a = make_pw_args(g);
    a.x = x; a.w = w; a.g = gout; a.out = gx; a.accumulate = accumulate;
    a.vec2 = (g.stride == 2 && g.W % 2 == 0 && (reinterpret_cast<uintptr_t>(gx) & 7) == 0) ? 1 : 0;
    // The rows and columns past the last sampled pixel (H or W not reached by S*(Ho-1)+S-1) do not exist:
    // S*Ho >= H and S*Wo >= W for an unpadded 1x1 layer, so the S x S blocks tile the whole plane.
    const dim3 grid(ceil_div(a.P, PW_THREADS), ceil_div(g.Ci, PW_CT));
    const size_t smem = (size_t)g.Co * PW_CT * sizeof(float);
    if (fast) adder_pw_gx_kernel<true><<<grid, PW_THREADS, smem, stream>>>(a);
    else adder_pw_gx_kernel<false><<<grid, PW_THREADS, smem, stream>>>(a);
    return launched();
}

// ---------------------------------------------------------------------------------------------------
// Weight gradient of the same layers: sum_xg[co][ci] = sum over positions of g[n,co,ho,wo] * x[n,ci,2ho,2wo]
// and the per-channel sums of g; the common finishing kernels turn the slices into
// sum (x - w) g = sum_xg - w * sum_g, its norm and the rescaled gradient (adder.cu:247, adder.py:78).
// A CTA owns one of `splits` contiguous ranges of 64-position tiles.  Per tile it stages g [Co][64] and
// the sampled x [Ci][64] in shared memory (position innermost); thread (slice, tco, tci) multiplies a
// 4 x 4 block of channel pairs over its slice of the 64 positions with 128-bit shared-memory loads.
// The slices of a CTA are added in index order at the end, so the result does not depend on timing.
constexpr int PWG_PT = 64;
constexpr int PWG_PITCH = PWG_PT + 4;
constexpr int PWG_RED = 20;        // 16 products + 4 channel sums per thread

struct PwGwArgs {
    const float* g; const float* x;
    float* part; float* gsum_part; unsigned int* ticket;
    int N, Ci, Co, H, W, Ho, Wo, S, P, tiles, tiles_per_split, tiles_rem, OT, PS, nco4, nci4;
    FastDiv d_wo, d_howo, d_ot, d_nci4;
};

__global__ void __launch_bounds__(PW_THREADS) adder_pw_gw_kernel(const PwGwArgs a) {
    extern __shared__ __align__(16) float smem[];
    float* const Gs = smem;                                 // [nco4*4][PWG_PITCH]
    float* const Xs = smem + a.nco4 * 4 * PWG_PITCH;        // [nci4*4][PWG_PITCH]
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.ticket = 0u;     // for the finishing kernel
    const int tid = threadIdx.x;
    uint32_t slice, ot, tco, tci;
    a.d_ot.divmod(tid, slice, ot);
    a.d_nci4.divmod(ot, tco, tci);
    const bool active = (int)slice < a.PS;
    const int split = blockIdx.x;
    const int t_begin = split * a.tiles_per_split + min(split, a.tiles_rem);
    const int t_end = t_begin + a.tiles_per_split + (split < a.tiles_rem ? 1 : 0);
    const int q = tid & (PWG_PT - 1), lane4 = tid >> 6;
    const int HW = a.H * a.W, HoWo = a.Ho * a.Wo;
    const int per_slice = PWG_PT / a.PS;

    float acc[4][4], gs[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        gs[i] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    }
    for (int t = t_begin; t < t_end; ++t) {
        const int p = t * PWG_PT + q;
        const bool valid = p < a.P;
        uint32_t n = 0, r = 0, ho = 0, wo = 0;
        if (valid) {
            a.d_howo.divmod(p, n, r);
            a.d_wo.divmod(r, ho, wo);
        }
        const float* gb = a.g + (size_t)n * a.Co * HoWo + r;
        const float* xb = a.x + (size_t)n * a.Ci * HW + (size_t)(ho * a.S) * a.W + wo * a.S;
        // four loads in flight per thread and operand before the first store
        for (int c0 = lane4; c0 < a.nco4 * 4; c0 += 16) {
            float v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = (valid && c0 + 4 * k < a.Co) ? __ldg(gb + (size_t)(c0 + 4 * k) * HoWo) : 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (c0 + 4 * k < a.nco4 * 4) Gs[(c0 + 4 * k) * PWG_PITCH + q] = v[k];
        }
        for (int c0 = lane4; c0 < a.nci4 * 4; c0 += 16) {
            float v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = (valid && c0 + 4 * k < a.Ci) ? __ldg(xb + (size_t)(c0 + 4 * k) * HW) : 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (c0 + 4 * k < a.nci4 * 4) Xs[(c0 + 4 * k) * PWG_PITCH + q] = v[k];
        }
        __syncthreads();
        if (active) {
            const float* gp = Gs + tco * 4 * PWG_PITCH + slice * per_slice;
            const float* xp = Xs + tci * 4 * PWG_PITCH + slice * per_slice;
            for (int k4 = 0; k4 < per_slice; k4 += 4) {
                float4 gq[4], xq[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) gq[i] = *reinterpret_cast<const float4*>(gp + i * PWG_PITCH + k4);
#pragma unroll
                for (int j = 0; j < 4; ++j) xq[j] = *reinterpret_cast<const float4*>(xp + j * PWG_PITCH + k4);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    gs[i] += (gq[i].x + gq[i].y) + (gq[i].z + gq[i].w);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[i][j] = fmaf(gq[i].x, xq[j].x, acc[i][j]);
                        acc[i][j] = fmaf(gq[i].y, xq[j].y, acc[i][j]);
                        acc[i][j] = fmaf(gq[i].z, xq[j].z, acc[i][j]);
                        acc[i][j] = fmaf(gq[i].w, xq[j].w, acc[i][j]);
                    }
                }
            }
        }
        __syncthreads();
    }
    // add the slices of the CTA in index order
    float* red = smem;                                      // [PS][OT][PWG_RED]
    if (active) {
        float* o = red + ((size_t)slice * a.OT + ot) * PWG_RED;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[16 + i] = gs[i];
#pragma unroll
            for (int j = 0; j < 4; ++j) o[i * 4 + j] = acc[i][j];
        }
    }
    __syncthreads();
    if (tid >= a.OT) return;
    float tot[PWG_RED];
#pragma unroll
    for (int k = 0; k < PWG_RED; ++k) tot[k] = 0.f;
    for (int sl = 0; sl < a.PS; ++sl) {
        const float* o = red + ((size_t)sl * a.OT + tid) * PWG_RED;
#pragma unroll
        for (int k = 0; k < PWG_RED; ++k) tot[k] += o[k];
    }
    float* part = a.part + (size_t)split * a.Co * a.Ci;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int co = tco * 4 + i;
        if (co >= a.Co) break;
        if (tci == 0) a.gsum_part[(size_t)split * a.Co + co] = tot[16 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ci = tci * 4 + j;
            if (ci < a.Ci) part[(size_t)co * a.Ci + ci] = tot[i * 4 + j];
        }
    }
}

// Number of tile ranges (= CTAs): about four CTAs per SM, at most one per tile.
int pointwise_gw_splits(const Geom& g) {
    const int tiles = ceil_div(g.N * g.Ho * g.Wo, PWG_PT);
    const int target = 4 * sm_count();
    const int splits = tiles < target ? tiles : target;
    return splits < 1 ? 1 : splits;
}

int launch_pointwise_gw(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                        unsigned int* ticket, int splits, cudaStream_t stream) {
    PwGwArgs a;
    a.g = gout; a.x = x; a.part = part; a.gsum_part = gsum_part; a.ticket = ticket;
    a.N = g.N; a.Ci = g.Ci; a.Co = g.Co; a.H = g.H; a.W = g.W; a.Ho = g.Ho; a.Wo = g.Wo; a.S = g.stride;
    a.P = g.N * g.Ho * g.Wo;
    a.tiles = ceil_div(a.P, PWG_PT);
    a.tiles_per_split = a.tiles / splits;
    a.tiles_rem = a.tiles % splits;
    a.nco4 = ceil_div(g.Co, 4);
    a.nci4 = ceil_div(g.Ci, 4);
    a.OT = a.nco4 * a.nci4;                    // <= 256 for at most 64 x 64 channels
    int ps = 1;
    while (ps * 2 * a.OT <= PW_THREADS && ps * 2 <= PWG_PT / 4) ps *= 2;
    a.PS = ps;
    a.d_wo = FastDiv(g.Wo);
    a.d_howo = FastDiv(g.Ho * g.Wo);
    a.d_ot = FastDiv(a.OT);
    a.d_nci4 = FastDiv(a.nci4);
    const size_t stage = (size_t)(a.nco4 + a.nci4) * 4 * PWG_PITCH;
    const size_t red = (size_t)a.PS * a.OT * PWG_RED;
    const size_t smem = (stage > red ? stage : red) * sizeof(float);
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(adder_pw_gw_kernel), smem) != ADDER_OK)
        return ADDER_ERR_CUDA;
    adder_pw_gw_kernel<<<splits, PW_THREADS, smem, stream>>>(a);
    return launched();
}

}  // namespace adder
