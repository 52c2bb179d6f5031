// Weight gradient of a 1x1, unpadded adder layer as an fp32 SIMT "NT GEMM":
//   sum_xg[co][ci] = sum_{n,p} g[n][co][p] * x[n][ci][p]        (p runs over the Ho*Wo output pixels of an image)
// For a strided layer x[n][ci][p] is the sampled pixel (stride*(p / Wo), stride*(p % Wo)) of the input plane:
// the x tile is then gathered with 4-byte copies, everything else is unchanged (GATHER).
// Both operands are contiguous along p, so tiles [rows][32 pixels] are staged with 16-byte cp.async
// (4-byte when H*W is not a multiple of 4) and read back with 128-bit loads, four pixels at a time.
// The (image, pixel) pairs of the whole batch form ONE sequence that is cut into 32-pixel stages wherever
// they fall, also across image boundaries: a 7x7 plane (49 pixels) would otherwise fill its second stage
// to 17/32.
// CTA = 128 threads, output tile 128 co x 64 ci, thread tile 8 x 8 (rows interleaved by 16 / 8 so that
// the eight lanes of a quarter-warp read consecutive rows: conflict-free with a 36-float pitch).
// The batch is split over `splits` CTAs per output tile; each writes its slice of partial sums and
// the per-channel sums of g to the workspace, and the common finishing kernels do the rest
// (sum of slices, - w * sum g, norm, rescale).  No tensor cores: the result must stay fp32-exact.
#include "common.cuh"
#include "kernels.h"

namespace adder {

constexpr int G1_THREADS = 128;
constexpr int G1_TM = 128, G1_TN = 64, G1_KC = 32, G1_PITCH = 36;

struct Gw1x1Args {
    const float* g;      // [N, Co, HW]
    const float* x;      // [N, Ci, HW]
    float* part;         // [splits][Co*Ci]
    float* gsum_part;    // [splits][Co]
    unsigned int* ticket;
    int N, Co, Ci, HW, splits, stages_per_split, total_stages, chunks, n_ci_tiles;
    int x_plane, x_w, samp;   // GATHER: pixels of an input plane, its row length, sampling stride
    FastDiv d_wo;             // GATHER: divides a pixel index by Wo
    FastDiv d_hw;             // divides a position of the batch-wide pixel sequence by HW
    long long total_px;       // N * HW
};

template <bool VEC, bool GATHER, bool FLAT>
__global__ void __launch_bounds__(G1_THREADS, 3) adder_gw1x1_kernel(const Gw1x1Args a) {
    extern __shared__ __align__(16) float smem[];
    constexpr int G_STAGE = G1_TM * G1_PITCH, X_STAGE = G1_TN * G1_PITCH;
    float* const Gs = smem;                    // [2][128][36]
    float* const Xs = smem + 2 * G_STAGE;      // [2][64][36]
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *a.ticket = 0u;

    const int tid = threadIdx.x, tm = tid & 15, tn = tid >> 4;
    const int split = blockIdx.x;
    const int ct_o = blockIdx.y / a.n_ci_tiles, ct_c = blockIdx.y % a.n_ci_tiles;
    const int co0 = ct_o * G1_TM, ci0 = ct_c * G1_TN;
    // the (image, 32-pixel chunk) pairs of the whole batch form one sequence; this CTA owns a contiguous range
    const int s_begin = split * a.stages_per_split;
    const int s_end = min(s_begin + a.stages_per_split, a.total_stages);
    const int stages = s_end > s_begin ? s_end - s_begin : 0;
    const bool do_gsum = (ct_c == 0) && (tn == 0);

    float acc[8][8];
    float gs[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        gs[i] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    }

    // Pixel q of stage `st` -> offset of that pixel inside tensor t[N][C][plane] at channel 0.  FLAT: the stages cut
    // the batch-wide pixel sequence; otherwise every image starts a new stage and (n, k0) are the stage's.
    int st_n = 0, st_k0 = 0;
    long long st_kf = 0;
    auto inside = [&](int q) { return FLAT ? (st_kf + q < a.total_px) : (st_k0 + q < a.HW); };
    auto locate = [&](int q, int C, int plane, bool gather, size_t& off) {
        uint32_t n = (uint32_t)st_n, px = (uint32_t)(st_k0 + q);
        if (FLAT) a.d_hw.divmod((uint32_t)(st_kf + q), n, px);
        if (gather) {
            uint32_t ho, wo;
            a.d_wo.divmod(px, ho, wo);
            off = (size_t)n * C * plane + (size_t)ho * a.samp * a.x_w + wo * a.samp;
        } else {
            off = (size_t)n * C * plane + px;
        }
    };
    auto fill = [&](int st, int buf) {
        st_kf = (long long)(s_begin + st) * G1_KC;
        st_n = (s_begin + st) / a.chunks;
        st_k0 = ((s_begin + st) % a.chunks) * G1_KC;
        float* gd = Gs + buf * G_STAGE;
        float* xd = Xs + buf * X_STAGE;
        if (VEC) {
            for (int e = tid; e < G1_TM * (G1_KC / 4); e += G1_THREADS) {
                const int r = e >> 3, q = (e & 7) * 4;
                const bool ok = (co0 + r < a.Co) && inside(q);
                size_t off = 0;
                if (ok) locate(q, a.Co, a.HW, false, off);
                cp_async16(gd + r * G1_PITCH + q, ok ? a.g + off + (size_t)(co0 + r) * a.HW : a.g, ok);
            }
            if (GATHER) {
                for (int e = tid; e < G1_TN * G1_KC; e += G1_THREADS) {
                    const int r = e >> 5, q = e & 31;
                    const bool ok = (ci0 + r < a.Ci) && inside(q);
                    size_t off = 0;
                    if (ok) locate(q, a.Ci, a.x_plane, true, off);
                    cp_async4(xd + r * G1_PITCH + q, ok ? a.x + off + (size_t)(ci0 + r) * a.x_plane : a.x, ok);
                }
            } else {
                for (int e = tid; e < G1_TN * (G1_KC / 4); e += G1_THREADS) {
                    const int r = e >> 3, q = (e & 7) * 4;
                    const bool ok = (ci0 + r < a.Ci) && inside(q);
                    size_t off = 0;
                    if (ok) locate(q, a.Ci, a.HW, false, off);
                    cp_async16(xd + r * G1_PITCH + q, ok ? a.x + off + (size_t)(ci0 + r) * a.HW : a.x, ok);
                }
            }
        } else {
            for (int e = tid; e < G1_TM * G1_KC; e += G1_THREADS) {
                const int r = e >> 5, q = e & 31;
                const bool ok = (co0 + r < a.Co) && inside(q);
                size_t off = 0;
                if (ok) locate(q, a.Co, a.HW, false, off);
                cp_async4(gd + r * G1_PITCH + q, ok ? a.g + off + (size_t)(co0 + r) * a.HW : a.g, ok);
            }
            for (int e = tid; e < G1_TN * G1_KC; e += G1_THREADS) {
                const int r = e >> 5, q = e & 31;
                const bool ok = (ci0 + r < a.Ci) && inside(q);
                size_t off = 0;
                if (ok) locate(q, a.Ci, a.x_plane, GATHER, off);
                cp_async4(xd + r * G1_PITCH + q, ok ? a.x + off + (size_t)(ci0 + r) * a.x_plane : a.x, ok);
            }
        }
    };

    if (stages > 0) {
        fill(0, 0);
        cp_async_commit();
    }
    for (int st = 0; st < stages; ++st) {
        const int buf = st & 1;
        if (st + 1 < stages) {
            fill(st + 1, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const float* gp = Gs + buf * G_STAGE + tm * G1_PITCH;
        const float* xp = Xs + buf * X_STAGE + tn * G1_PITCH;
#pragma unroll 2
        for (int k4 = 0; k4 < G1_KC; k4 += 4) {
            float4 gq[8], xq[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) gq[i] = *reinterpret_cast<const float4*>(gp + i * 16 * G1_PITCH + k4);
#pragma unroll
            for (int j = 0; j < 8; ++j) xq[j] = *reinterpret_cast<const float4*>(xp + j * 8 * G1_PITCH + k4);
            if (do_gsum) {
#pragma unroll
                for (int i = 0; i < 8; ++i) gs[i] += (gq[i].x + gq[i].y) + (gq[i].z + gq[i].w);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[i][j] = fmaf(gq[i].x, xq[j].x, acc[i][j]);
                    acc[i][j] = fmaf(gq[i].y, xq[j].y, acc[i][j]);
                    acc[i][j] = fmaf(gq[i].z, xq[j].z, acc[i][j]);
                    acc[i][j] = fmaf(gq[i].w, xq[j].w, acc[i][j]);
                }
        }
        __syncthreads();
    }

    float* part = a.part + (size_t)split * a.Co * a.Ci;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int co = co0 + i * 16 + tm;
        if (co >= a.Co) continue;
        if (do_gsum) a.gsum_part[(size_t)split * a.Co + co] = gs[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int ci = ci0 + j * 8 + tn;
            if (ci < a.Ci) part[(size_t)co * a.Ci + ci] = acc[i][j];
        }
    }
}

bool gw1x1_applicable(const Geom& g) {
    return g.k == 1 && g.pad == 0 && g.Co >= 64 && g.Ci >= 32 && g.N >= 1;     // any stride: strided layers gather x
}

// Stages cut the batch-wide pixel sequence (one division more per staged element) where stages that restart with
// every image would stay more than 8 % empty: 7x7 planes (49 pixels: 23 %) and 14x14 (196: 12.5 %), not 28x28.
static bool gw1x1_flat(const Geom& g) {
    const int hw = g.Ho * g.Wo;
    const int padded = ceil_div(hw, G1_KC) * G1_KC;
    return (padded - hw) * 100 > 8 * padded;
}

// Number of batch slices (CTAs per output tile): about three CTAs per SM in total.
int gw1x1_splits(const Geom& g) {
    const int out_tiles = ceil_div(g.Co, G1_TM) * ceil_div(g.Ci, G1_TN);
    const int total = gw1x1_flat(g) ? (int)(((long long)g.N * g.Ho * g.Wo + G1_KC - 1) / G1_KC)
                                    : g.N * ceil_div(g.Ho * g.Wo, G1_KC);
    // all CTAs in ONE wave of three per SM: rounding up (14 slices x 32 tiles = 448 CTAs for 444 places) sends a
    // handful of CTAs into a second wave that takes as long as the first
    int splits = (3 * sm_count()) / out_tiles;
    if (splits > total) splits = total;
    if (splits < 1) splits = 1;
    const int per = ceil_div(total, splits);
    return ceil_div(total, per);
}

int launch_gw1x1(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                 unsigned int* ticket, int splits, cudaStream_t stream) {
    Gw1x1Args a;
    a.g = gout; a.x = x; a.part = part; a.gsum_part = gsum_part; a.ticket = ticket;
    a.N = g.N; a.Co = g.Co; a.Ci = g.Ci; a.HW = g.Ho * g.Wo;
    a.x_plane = g.H * g.W; a.x_w = g.W; a.samp = g.stride; a.d_wo = FastDiv((uint32_t)g.Wo);
    const bool gather = g.stride != 1;
    a.splits = splits;
    a.total_px = (long long)g.N * a.HW;
    if (a.total_px > 2147483647LL) return ADDER_ERR_UNSUPPORTED;
    a.d_hw = FastDiv((uint32_t)a.HW);
    a.chunks = ceil_div(a.HW, G1_KC);
    const bool flat = gw1x1_flat(g);
    a.total_stages = flat ? (int)((a.total_px + G1_KC - 1) / G1_KC) : g.N * a.chunks;
    a.stages_per_split = ceil_div(a.total_stages, splits);
    a.n_ci_tiles = ceil_div(g.Ci, G1_TN);
    const int out_tiles = ceil_div(g.Co, G1_TM) * a.n_ci_tiles;
    if (out_tiles > 65535) return ADDER_ERR_UNSUPPORTED;
    const size_t smem = (size_t)2 * (G1_TM + G1_TN) * G1_PITCH * sizeof(float);
    const bool vec_g = (a.HW % 4 == 0) && ((reinterpret_cast<uintptr_t>(gout) & 15) == 0);
    const bool vec = vec_g && (gather || (reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const dim3 grid(splits, out_tiles);
    auto run = [&](auto kern) -> int {
        if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem) != ADDER_OK) return ADDER_ERR_CUDA;
        kern<<<grid, G1_THREADS, smem, stream>>>(a);
        return ADDER_OK;
    };
    int st;
    if (flat) {
        if (gather) st = vec ? run(adder_gw1x1_kernel<true, true, true>) : run(adder_gw1x1_kernel<false, true, true>);
        else st = vec ? run(adder_gw1x1_kernel<true, false, true>) : run(adder_gw1x1_kernel<false, false, true>);
    } else {
        if (gather) st = vec ? run(adder_gw1x1_kernel<true, true, false>) : run(adder_gw1x1_kernel<false, true, false>);
        else st = vec ? run(adder_gw1x1_kernel<true, false, false>) : run(adder_gw1x1_kernel<false, false, false>);
    }
    if (st != ADDER_OK) return st;
    return launched();
}

}  // namespace adder
