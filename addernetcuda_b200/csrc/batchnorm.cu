// Training-mode BatchNorm2d (+ optional residual add and ReLU) around the adder layers, NCHW fp32.
//
// The reference networks follow every adder layer with nn.BatchNorm2d and usually a ReLU
// (resnet20.py:28-40, resnet50.py:38-53).  For the 16-64 channel CIFAR layers the library batch-norm
// kernels launch one CTA per channel and leave most of the GPU idle; these kernels split every
// channel's reduction over many CTAs instead.  Per channel c with M = N*H*W elements:
//   forward   mean = sum(y)/M, var = sum((y-mean)^2)/M, invstd = rsqrt(var + eps)
//             z = gamma*(y-mean)*invstd + beta [+ residual] [ReLU]
//   backward  dz' = dz * (z > 0) when ReLU was applied
//             dgamma = sum(dz' * yhat), dbeta = sum(dz'), yhat = (y-mean)*invstd
//             dy = gamma*invstd * (dz' - dbeta/M - yhat*dgamma/M);  dresidual = dz'
// Reductions: each CTA sums its slice in fp32 per thread (shifted by a per-channel pivot, so that the
// variance does not cancel), slices are combined in double precision in index order: deterministic.
#include "common.cuh"
#include "kernels.h"

namespace adder {

constexpr int BN_THREADS = 256;

// Block-wide sum of two doubles; result valid in thread 0.
__device__ __forceinline__ void block_sum2(double& a, double& b) {
    __shared__ double sa[BN_THREADS / 32], sb[BN_THREADS / 32];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, off);
        b += __shfl_xor_sync(0xffffffffu, b, off);
    }
    if ((threadIdx.x & 31) == 0) { sa[threadIdx.x >> 5] = a; sb[threadIdx.x >> 5] = b; }
    __syncthreads();
    if (threadIdx.x == 0) {
        a = 0.0; b = 0.0;
        for (int k = 0; k < BN_THREADS / 32; ++k) { a += sa[k]; b += sb[k]; }
    }
    __syncthreads();
}

// Element e of channel c's M = N*HW values lives at ((e / HW) * C + c) * HW + e % HW.
struct BnGeom {
    int N, C, HW, M, splits, per_split;   // per_split: elements of one channel handled by one CTA (multiple of 4)
    FastDiv d_hw;
};

// grid (splits, C): partial sums of (y - pivot) and (y - pivot)^2 with pivot = y[0, c, 0].
__global__ void __launch_bounds__(BN_THREADS) bn_stats_kernel(const float* __restrict__ y, BnGeom g, double* __restrict__ part) {
    const int c = blockIdx.y, sp = blockIdx.x;
    const float pivot = __ldg(y + (size_t)c * g.HW);
    const int e0 = sp * g.per_split;
    const int e1 = min(e0 + g.per_split, g.M);
    float s = 0.f, q = 0.f;
    const bool vec = (g.HW % 4 == 0);
    if (vec) {
        for (int e = e0 + threadIdx.x * 4; e < e1; e += BN_THREADS * 4) {
            uint32_t n, r;
            g.d_hw.divmod(e, n, r);
            const float4 v = __ldg(reinterpret_cast<const float4*>(y + ((size_t)n * g.C + c) * g.HW + r));
            const float a0 = v.x - pivot, a1 = v.y - pivot, a2 = v.z - pivot, a3 = v.w - pivot;
            s += (a0 + a1) + (a2 + a3);
            q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
    } else {
        for (int e = e0 + threadIdx.x; e < e1; e += BN_THREADS) {
            uint32_t n, r;
            g.d_hw.divmod(e, n, r);
            const float a0 = __ldg(y + ((size_t)n * g.C + c) * g.HW + r) - pivot;
            s += a0;
            q += a0 * a0;
        }
    }
    double ds = s, dq = q;
    block_sum2(ds, dq);
    if (threadIdx.x == 0) {
        part[((size_t)c * g.splits + sp) * 2] = ds;
        part[((size_t)c * g.splits + sp) * 2 + 1] = dq;
    }
}

struct BnFwdArgs {
    const float* y; const float* gamma; const float* beta; const float* residual;
    float* z; float* save_mean; float* save_invstd; float* running_mean; float* running_var;
    long long* num_batches;   // optional counter (nn.BatchNorm2d.num_batches_tracked), incremented once per call
    const double* part;       // [C][nparts][2]
    int nparts;               // slices per channel in `part`
    int pivoted;              // 1: sums of (y - y[0,c,0]) from bn_stats_kernel; 0: plain sums from the forward adder kernel
    float eps, momentum;
    int relu;
};

// grid (splits, C): finish the statistics (every CTA of a channel adds the same slices in the same
// order), CTA 0 of the channel stores them and updates the running estimates, then normalise.
__global__ void __launch_bounds__(BN_THREADS) bn_apply_kernel(BnFwdArgs a, BnGeom g) {
    const int c = blockIdx.y, sp = blockIdx.x;
    __shared__ float s_mean, s_invstd;
    double s = 0.0, q = 0.0;
    for (int k = threadIdx.x; k < a.nparts; k += BN_THREADS) {
        const double2 v = *reinterpret_cast<const double2*>(a.part + ((size_t)c * a.nparts + k) * 2);
        s += v.x;
        q += v.y;
    }
    block_sum2(s, q);
    if (threadIdx.x == 0) {
        const double pivot = a.pivoted ? (double)__ldg(a.y + (size_t)c * g.HW) : 0.0;
        const double m1 = s / g.M;
        double var = q / g.M - m1 * m1;
        if (var < 0.0) var = 0.0;
        const double mean = pivot + m1;
        const float invstd = (float)(1.0 / sqrt(var + (double)a.eps));
        s_mean = (float)mean;
        s_invstd = invstd;
        if (sp == 0 && c == 0 && a.num_batches != nullptr) *a.num_batches += 1;
        if (sp == 0) {
            a.save_mean[c] = (float)mean;
            a.save_invstd[c] = invstd;
            if (a.running_mean != nullptr) {
                const double unbiased = g.M > 1 ? var * g.M / (g.M - 1) : var;
                a.running_mean[c] = (float)((1.0 - a.momentum) * a.running_mean[c] + a.momentum * mean);
                a.running_var[c] = (float)((1.0 - a.momentum) * a.running_var[c] + a.momentum * unbiased);
            }
        }
    }
    __syncthreads();
    const float mean = s_mean;
    const float sc = s_invstd * a.gamma[c];
    const float sh = a.beta[c];
    const int e0 = sp * g.per_split;
    const int e1 = min(e0 + g.per_split, g.M);
    if (g.HW % 4 == 0) {
        for (int e = e0 + threadIdx.x * 4; e < e1; e += BN_THREADS * 4) {
            uint32_t n, r;
            g.d_hw.divmod(e, n, r);
            const size_t off = ((size_t)n * g.C + c) * g.HW + r;
            const float4 v = __ldg(reinterpret_cast<const float4*>(a.y + off));
            float4 o = make_float4(fmaf(v.x - mean, sc, sh), fmaf(v.y - mean, sc, sh), fmaf(v.z - mean, sc, sh),
                                   fmaf(v.w - mean, sc, sh));
            if (a.residual != nullptr) {
                const float4 rr = __ldg(reinterpret_cast<const float4*>(a.residual + off));
                o.x += rr.x; o.y += rr.y; o.z += rr.z; o.w += rr.w;
            }
            if (a.relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
            *reinterpret_cast<float4*>(a.z + off) = o;
        }
    } else {
        for (int e = e0 + threadIdx.x; e < e1; e += BN_THREADS) {
            uint32_t n, r;
            g.d_hw.divmod(e, n, r);
            const size_t off = ((size_t)n * g.C + c) * g.HW + r;
            float o = fmaf(__ldg(a.y + off) - mean, sc, sh);
            if (a.residual != nullptr) o += __ldg(a.residual + off);
            if (a.relu) o = fmaxf(o, 0.f);
            a.z[off] = o;
        }
    }
}

struct BnBwdArgs {
    const float* dz; const float* y; const float* z; const float* gamma; const float* save_mean; const float* save_invstd;
    float* dy; float* dresidual; float* dgamma; float* dbeta;
    double* part;
    int relu;
};

// grid (splits, C): partial sums of dz' and dz' * yhat.
__global__ void __launch_bounds__(BN_THREADS) bn_bwd_reduce_kernel(BnBwdArgs a, BnGeom g) {
    const int c = blockIdx.y, sp = blockIdx.x;
    const float mean = a.save_mean[c], invstd = a.save_invstd[c];
    const int e0 = sp * g.per_split;
    const int e1 = min(e0 + g.per_split, g.M);
    float s = 0.f, q = 0.f;
    if (g.HW % 4 == 0) {
        for (int e = e0 + threadIdx.x * 4; e < e1; e += BN_THREADS * 4) {
            uint32_t n, r;
            g.d_hw.divmod(e, n, r);
            const size_t off = ((size_t)n * g.C + c) * g.HW + r;
            float4 d = __ldg(reinterpret_cast<const float4*>(a.dz + off));
            const float4 v = __ldg(reinterpret_cast<const float4*>(a.y + off));
            if (a.relu) {
                const float4 zz = __ldg(reinterpret_cast<const float4*>(a.z + off));
                d.x = zz.x > 0.f ? d.x : 0.f; d.y = zz.y > 0.f ? d.y : 0.f;
                d.z = zz.z > 0.f ? d.z : 0.f; d.w = zz.w > 0.f ? d.w : 0.f;
            }
            s += (d.x + d.y) + (d.z + d.w);
            q += (d.x * (v.x - mean) + d.y * (v.y - mean)) + (d.z * (v.z - mean) + d.w * (v.w - mean));
        }
    } else {
        for (int e = e0 + threadIdx.x; e < e1; e += BN_THREADS) {
            uint32_t n, r;
            g.d_hw.divmod(e, n, r);
            const size_t off = ((size_t)n * g.C + c) * g.HW + r;
            float d = __ldg(a.dz + off);
            if (a.relu && !(__ldg(a.z + off) > 0.f)) d = 0.f;
            s += d;
            q += d * (__ldg(a.y + off) - mean);
        }
    }
    double ds = s, dq = (double)q * (double)invstd;
    block_sum2(ds, dq);
    if (threadIdx.x == 0) {
        a.part[((size_t)c * g.splits + sp) * 2] = ds;
        a.part[((size_t)c * g.splits + sp) * 2 + 1] = dq;
    }
}

// grid (splits, C): dy (and the residual branch's gradient); CTA 0 of a channel stores dgamma, dbeta.
__global__ void __launch_bounds__(BN_THREADS) bn_bwd_apply_kernel(BnBwdArgs a, BnGeom g) {
    const int c = blockIdx.y, sp = blockIdx.x;
    __shared__ float s_db, s_dg;
    if (threadIdx.x == 0) {
        double s = 0.0, q = 0.0;
        for (int k = 0; k < g.splits; ++k) {
            s += a.part[((size_t)c * g.splits + k) * 2];
            q += a.part[((size_t)c * g.splits + k) * 2 + 1];
        }
        s_db = (float)s;
        s_dg = (float)q;
        if (sp == 0) { a.dbeta[c] = (float)s; a.dgamma[c] = (float)q; }
    }
    __syncthreads();
    const float mean = a.save_mean[c], invstd = a.save_invstd[c];
    const float k0 = a.gamma[c] * invstd;
    const float mb = s_db / g.M, mg = s_dg / g.M * invstd;      // yhat * dgamma / M = (y-mean) * invstd * dgamma / M
    const int e0 = sp * g.per_split;
    const int e1 = min(e0 + g.per_split, g.M);
    if (g.HW % 4 == 0) {
        for (int e = e0 + threadIdx.x * 4; e < e1; e += BN_THREADS * 4) {
            uint32_t n, r;
            g.d_hw.divmod(e, n, r);
            const size_t off = ((size_t)n * g.C + c) * g.HW + r;
            float4 d = __ldg(reinterpret_cast<const float4*>(a.dz + off));
            const float4 v = __ldg(reinterpret_cast<const float4*>(a.y + off));
            if (a.relu) {
                const float4 zz = __ldg(reinterpret_cast<const float4*>(a.z + off));
                d.x = zz.x > 0.f ? d.x : 0.f; d.y = zz.y > 0.f ? d.y : 0.f;
                d.z = zz.z > 0.f ? d.z : 0.f; d.w = zz.w > 0.f ? d.w : 0.f;
            }
            if (a.dresidual != nullptr) *reinterpret_cast<float4*>(a.dresidual + off) = d;
            const float4 o = make_float4(k0 * (d.x - mb - (v.x - mean) * mg), k0 * (d.y - mb - (v.y - mean) * mg),
                                         k0 * (d.z - mb - (v.z - mean) * mg), k0 * (d.w - mb - (v.w - mean) * mg));
            *reinterpret_cast<float4*>(a.dy + off) = o;
        }
    } else {
        for (int e = e0 + threadIdx.x; e < e1; e += BN_THREADS) {
            uint32_t n, r;
            g.d_hw.divmod(e, n, r);
            const size_t off = ((size_t)n * g.C + c) * g.HW + r;
            float d = __ldg(a.dz + off);
            if (a.relu && !(__ldg(a.z + off) > 0.f)) d = 0.f;
            if (a.dresidual != nullptr) a.dresidual[off] = d;
            a.dy[off] = k0 * (d - mb - (__ldg(a.y + off) - mean) * mg);
        }
    }
}

// ------------------------------------------------------------------------------------------ host

static int bn_geom(int n, int c, int hw, BnGeom* g) {
    if (n <= 0 || c <= 0 || hw <= 0) return ADDER_ERR_BAD_SHAPE;
    if ((long long)n * c * hw > 2147483647LL || c > 65535) return ADDER_ERR_UNSUPPORTED;
    g->N = n; g->C = c; g->HW = hw; g->M = n * hw;
    const int sms = sm_count();
    // about 4 CTAs per SM in total, at least 4096 elements per CTA, at most 64 slices per channel
    int splits = ceil_div(4 * sms, c);
    const int max_by_work = g->M / 4096 > 0 ? g->M / 4096 : 1;
    if (splits > max_by_work) splits = max_by_work;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    g->per_split = round_up(ceil_div(g->M, splits), 4);
    g->splits = ceil_div(g->M, g->per_split);
    g->d_hw = FastDiv((uint32_t)hw);
    return ADDER_OK;
}

// Evaluation mode: batch norm with running statistics is a fixed per-channel affine map, so the layer after
// an adder convolution collapses to z = y*scale[c] + shift[c] [+ residual] [ReLU] in one pass.
__global__ void __launch_bounds__(BN_THREADS) affine_act_kernel(const float* __restrict__ y, const float* __restrict__ scale,
                                                                const float* __restrict__ shift,
                                                                const float* __restrict__ residual, float* __restrict__ z,
                                                                int relu, int C, int HW, long long total, int vec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (vec) {
        const int hw4 = HW >> 2;
        for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < (total >> 2); q += stride) {
            const int c = (int)((q / hw4) % C);
            const float sc = __ldg(scale + c), sh = __ldg(shift + c);
            float4 v = reinterpret_cast<const float4*>(y)[q];
            v.x = fmaf(v.x, sc, sh); v.y = fmaf(v.y, sc, sh); v.z = fmaf(v.z, sc, sh); v.w = fmaf(v.w, sc, sh);
            if (residual != nullptr) {
                const float4 r = reinterpret_cast<const float4*>(residual)[q];
                v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
            }
            if (relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
            reinterpret_cast<float4*>(z)[q] = v;
        }
    } else {
        for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
            const int c = (int)((e / HW) % C);
            float v = fmaf(y[e], __ldg(scale + c), __ldg(shift + c));
            if (residual != nullptr) v += residual[e];
            z[e] = relu ? fmaxf(v, 0.f) : v;
        }
    }
}

}  // namespace adder

using namespace adder;

extern "C" {

int adder_b200_affine_forward(const float* y, const float* scale, const float* shift, const float* residual, float* z,
                              int relu, int n, int c, int hw, void* stream) {
    if (n < 0 || c <= 0 || hw <= 0) return ADDER_ERR_BAD_SHAPE;
    if (n == 0) return ADDER_OK;
    if (y == nullptr || scale == nullptr || shift == nullptr || z == nullptr) return ADDER_ERR_NULL_POINTER;
    const long long total = (long long)n * c * hw;
    uintptr_t bits = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(z);
    if (residual != nullptr) bits |= reinterpret_cast<uintptr_t>(residual);
    const int vec = (hw % 4 == 0 && (bits & 15) == 0) ? 1 : 0;
    const long long work = vec ? total / 4 : total;
    long long blocks = (work + BN_THREADS - 1) / BN_THREADS;
    const long long cap = 8LL * sm_count();
    if (blocks > cap) blocks = cap;
    affine_act_kernel<<<(unsigned)blocks, BN_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(y, scale, shift, residual, z,
                                                                                             relu, c, hw, total, vec);
    return launched();
}

size_t adder_b200_batchnorm_workspace_bytes(int n, int c, int hw) {
    BnGeom g;
    if (bn_geom(n, c, hw, &g) != ADDER_OK) return 0;
    return (size_t)c * g.splits * 2 * sizeof(double);
}

static int bn_forward(const float* y, const double* stats, int stat_slices, const float* gamma, const float* beta,
                      const float* residual, float* z, float* save_mean, float* save_invstd, float* running_mean,
                      float* running_var, long long* num_batches_tracked, float eps, float momentum, int relu,
                      void* workspace, size_t workspace_bytes, int n, int c, int hw, void* stream) {
    BnGeom g;
    const int st = bn_geom(n, c, hw, &g);
    if (st != ADDER_OK) return st;
    if (!y || !gamma || !beta || !z || !save_mean || !save_invstd) return ADDER_ERR_NULL_POINTER;
    if ((running_mean == nullptr) != (running_var == nullptr)) return ADDER_ERR_NULL_POINTER;
    if (hw % 4 == 0 && (((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(z) |
                          reinterpret_cast<uintptr_t>(residual)) & 15) != 0)) return ADDER_ERR_ALIGNMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid(g.splits, c);
    BnFwdArgs a{y, gamma, beta, residual, z, save_mean, save_invstd, running_mean, running_var, num_batches_tracked,
                nullptr, 0, 0, eps, momentum, relu};
    if (stats != nullptr) {
        if (stat_slices <= 0) return ADDER_ERR_BAD_SHAPE;
        if ((reinterpret_cast<uintptr_t>(stats) & 15) != 0) return ADDER_ERR_ALIGNMENT;
        a.part = stats; a.nparts = stat_slices; a.pivoted = 0;
        bn_apply_kernel<<<grid, BN_THREADS, 0, s>>>(a, g);
        return launched();
    }
    if (workspace == nullptr || workspace_bytes < (size_t)c * g.splits * 2 * sizeof(double)) return ADDER_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return ADDER_ERR_ALIGNMENT;
    double* part = static_cast<double*>(workspace);
    bn_stats_kernel<<<grid, BN_THREADS, 0, s>>>(y, g, part);
    a.part = part; a.nparts = g.splits; a.pivoted = 1;
    bn_apply_kernel<<<grid, BN_THREADS, 0, s>>>(a, g);
    return launched(2);
}

int adder_b200_batchnorm_forward(const float* y, const float* gamma, const float* beta, const float* residual,
                                 float* z, float* save_mean, float* save_invstd, float* running_mean,
                                 float* running_var, long long* num_batches_tracked, float eps, float momentum,
                                 int relu, void* workspace, size_t workspace_bytes, int n, int c, int hw,
                                 void* stream) {
    return bn_forward(y, nullptr, 0, gamma, beta, residual, z, save_mean, save_invstd, running_mean, running_var,
                      num_batches_tracked, eps, momentum, relu, workspace, workspace_bytes, n, c, hw, stream);
}

int adder_b200_batchnorm_forward_from_stats(const float* y, const double* stats, int stat_slices, const float* gamma,
                                            const float* beta, const float* residual, float* z, float* save_mean,
                                            float* save_invstd, float* running_mean, float* running_var,
                                            long long* num_batches_tracked, float eps, float momentum, int relu, int n,
                                            int c, int hw, void* stream) {
    if (stats == nullptr) return ADDER_ERR_NULL_POINTER;
    return bn_forward(y, stats, stat_slices, gamma, beta, residual, z, save_mean, save_invstd, running_mean,
                      running_var, num_batches_tracked, eps, momentum, relu, nullptr, 0, n, c, hw, stream);
}

int adder_b200_batchnorm_backward(const float* dz, const float* y, const float* z, const float* gamma,
                                  const float* save_mean, const float* save_invstd, float* dy, float* dresidual,
                                  float* dgamma, float* dbeta, int relu, void* workspace, size_t workspace_bytes,
                                  int n, int c, int hw, void* stream) {
    BnGeom g;
    const int st = bn_geom(n, c, hw, &g);
    if (st != ADDER_OK) return st;
    if (!dz || !y || !gamma || !save_mean || !save_invstd || !dy || !dgamma || !dbeta) return ADDER_ERR_NULL_POINTER;
    if (relu && z == nullptr) return ADDER_ERR_NULL_POINTER;
    if (workspace == nullptr || workspace_bytes < (size_t)c * g.splits * 2 * sizeof(double)) return ADDER_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return ADDER_ERR_ALIGNMENT;
    if (hw % 4 == 0 && (((reinterpret_cast<uintptr_t>(dz) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(z) |
                          reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dresidual)) & 15) != 0))
        return ADDER_ERR_ALIGNMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    BnBwdArgs a{dz, y, z, gamma, save_mean, save_invstd, dy, dresidual, dgamma, dbeta, static_cast<double*>(workspace), relu};
    const dim3 grid(g.splits, c);
    bn_bwd_reduce_kernel<<<grid, BN_THREADS, 0, s>>>(a, g);
    bn_bwd_apply_kernel<<<grid, BN_THREADS, 0, s>>>(a, g);
    return launched(2);
}

}  // extern "C"
