// Shared device/host helpers for the adder-convolution kernels (sm_100a, fp32 SIMT).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace adder {

// Geometry of one adder2d layer on NCHW fp32 tensors (square kernel, symmetric padding):
// the quantities adder.py:22-31 of the reference derives from X.size() and W.size().
struct Geom {
    int N, Ci, H, W, Co, Ho, Wo, k, stride, pad;
};

// A 1x1, stride-1, unpadded layer has no notion of rows: every pixel is computed from the same pixel of the
// input.  Tiling it as one row of H*W pixels per image gives long runs of aligned 8-pixel segments (56x56
// planes: input gradient 702 -> 567 us on 256->64 at batch 64).  Planes that are 7, 14 or 28 wide keep
// their rows: 7-pixel segments, 28 to a warp, measured faster there than 8-pixel segments with a ragged end.
// (The input gradient also flattens such a plane when H*W is a multiple of 8 - 28x28 - because it then shares a
// staged value of g between 64 input channels: 512->128 28x28 561 -> 496 us; the forward measured slower that way.)
inline Geom flatten_pointwise(const Geom& g, bool whole_octets_too = false) {
    Geom f = g;
    const bool sevens = (g.W % 8 != 0) && (g.W % 7 == 0) && !(whole_octets_too && (g.H * g.W) % 8 == 0);
    if (g.k == 1 && g.stride == 1 && g.pad == 0 && g.H > 1 && !sevens && (long long)g.H * g.W <= 2147483647LL) {
        f.W = g.H * g.W; f.H = 1; f.Wo = f.W; f.Ho = 1;
    }
    return f;
}

// Unsigned division by a runtime constant with one multiply-high and one shift.
// Exact for every numerator n < 2^31 and divisor 1 <= d < 2^31 (round-up method:
// m = ceil(2^(32+s) / d) - 2^32 with s = ceil(log2 d); n / d = (umulhi(n, m) + n) >> s).
struct FastDiv {
    uint32_t mul, shift, div;
    FastDiv() : mul(0), shift(0), div(1) {}
    explicit FastDiv(uint32_t d) : div(d) {
        uint32_t s = 0;
        while ((1ull << s) < d) ++s;
        shift = s;
        mul = (uint32_t)((((1ull << s) - d) << 32) / d + 1);
    }
    __host__ __device__ __forceinline__ uint32_t quot(uint32_t n) const {
#ifdef __CUDA_ARCH__
        return (__umulhi(n, mul) + n) >> shift;   // n < 2^31 so the add cannot wrap
#else
        return (uint32_t)((((uint64_t)n * mul) >> 32) + n) >> shift;
#endif
    }
    __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
        q = quot(n);
        r = n - q * div;
    }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// 4-byte asynchronous global->shared copy; when !valid nothing is read and the word is zeroed.
__device__ __forceinline__ void cp_async4(float* dst_smem, const float* src, bool valid) {
    const int sz = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(sz));
}
// 16-byte variant (both addresses 16-byte aligned).
__device__ __forceinline__ void cp_async16(float* dst_smem, const float* src, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Packed FP32 pairs (sm_100 add/fma .f32x2): one issue slot does the work of two scalar instructions.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// Loads N consecutive floats from shared memory into registers.  When ALIGNED the address is a
// multiple of 16 bytes and the run is fetched with 128-/64-bit loads (10 values = 2 x LDS.128 + 1 x
// LDS.64 instead of 10 scalar loads); otherwise one scalar load per value.
template <int N, bool ALIGNED>
__device__ __forceinline__ void load_run(float (&dst)[N], const float* __restrict__ src) {
    if (ALIGNED) {
        int i = 0;
#pragma unroll
        for (; i + 4 <= N; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            dst[i] = v.x; dst[i + 1] = v.y; dst[i + 2] = v.z; dst[i + 3] = v.w;
        }
        if (N % 4 >= 2) {
            const float2 v = *reinterpret_cast<const float2*>(src + (N / 4) * 4);
            dst[(N / 4) * 4] = v.x; dst[(N / 4) * 4 + 1] = v.y;
        }
        if (N % 2 == 1) dst[N - 1] = src[N - 1];
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) dst[i] = src[i];
    }
}

// Loads N consecutive (v, v) pairs (2N floats of a row stored with every value doubled) into 64-bit
// registers.  When ALIGNED the address is a multiple of 16 bytes: 128-bit loads, two pairs each;
// otherwise the address is still a multiple of 8 bytes (doubled rows start pairs on even words).
template <int N, bool ALIGNED>
__device__ __forceinline__ void load_pairs(uint64_t (&dst)[N], const float* __restrict__ src) {
    if (ALIGNED) {
#pragma unroll
        for (int i = 0; i + 2 <= N; i += 2) {
            const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(src + 2 * i);
            dst[i] = v.x; dst[i + 1] = v.y;
        }
        if (N % 2 == 1) dst[N - 1] = *reinterpret_cast<const unsigned long long*>(src + 2 * (N - 1));
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) dst[i] = *reinterpret_cast<const unsigned long long*>(src + 2 * i);
    }
}

// Row pitch (in floats) for a shared-memory patch read with 128-bit loads by lanes whose start
// addresses are a0[l] + row[l] * pitch: the smallest multiple of 4 >= cols (up to +32) minimising,
// over the four quarter-warps, the worst number of lanes that fall into one 16-byte bank group.
template <typename F>
inline int pick_pitch_vec(int cols, int nlanes, F lane_row_and_col, int slack = 32) {
    int best = (cols + 3) / 4 * 4, best_cost = 1 << 30;
    for (int pitch = (cols + 3) / 4 * 4; pitch <= (cols + 3) / 4 * 4 + slack; pitch += 4) {
        int cost = 0;
        for (int q0 = 0; q0 < nlanes; q0 += 8) {
            int cnt[8] = {0}, worst = 0;
            for (int l = q0; l < q0 + 8 && l < nlanes; ++l) {
                int row, col;
                lane_row_and_col(l, row, col);
                const int grp = ((row * pitch + col) >> 2) & 7;
                if (++cnt[grp] > worst) worst = cnt[grp];
            }
            cost += worst;
        }
        if (cost < best_cost) { best_cost = cost; best = pitch; }
    }
    return best;
}

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int round_up(int a, int b) { return ceil_div(a, b) * b; }
// floor(a / b) for b > 0 and any sign of a.
__host__ __device__ __forceinline__ int floor_div(int a, int b) {
    int q = a / b;
    return (a % b != 0 && (a < 0)) ? q - 1 : q;
}

// ---- host-side helpers shared by the tile planners -------------------------------------------------
inline int largest_divisor_le(int n, int limit) {
    for (int d = limit < n ? limit : n; d >= 1; --d)
        if (n % d == 0) return d;
    return 1;
}

// SM count of the current device (148 when no device is visible, e.g. when only planning on a CPU box).
inline int sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 148;
    return sms;
}

}  // namespace adder
