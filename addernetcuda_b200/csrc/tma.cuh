// Tensor-memory-accelerator helpers: tiled bulk loads (cp.async.bulk.tensor) of boxes of an NCHW tensor
// into shared memory, completion on an mbarrier, bounded waits.
//
// Only the plain form is used: one CTA loads into its own shared memory from this GPU's own global memory.
// Coordinates may be negative or run past the tensor: those elements arrive as zeros, which is how padding,
// halos and ragged edges are produced without a single predicated instruction.  The innermost coordinate
// of every load is a multiple of 4 floats (16 bytes), as the hardware requires.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "common.cuh"

namespace adder {

// ---- host: tensor maps --------------------------------------------------------------------------
// Encodes a 4-d fp32 tensor map over a contiguous NCHW tensor: dims (innermost first) W, H, C, N and the
// box to copy per load.  Returns false when the driver entry point is missing or rejects the geometry
// (base not 16-byte aligned, a stride not a multiple of 16 bytes, a box extent over 256): callers then
// take a kernel that does not need tensor maps.
bool make_nchw_tensor_map(CUtensorMap* map, const float* base, int N, int C, int H, int W, int box_w, int box_h,
                          int box_c, int box_n);

// Address (on the current device) of the int that kernels set when a bounded wait gives up.
int device_error_flag(int** flag);

// ---- device ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
// Makes freshly initialised barriers visible to the asynchronous proxy (the copy engine) before first use.
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// One arrival that also announces `bytes` of copies to come: the phase completes when they have landed.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Waits for the phase with the given parity, at most MBAR_WAIT_LIMIT polls (each poll already blocks for a
// while inside the hardware).  Returns false when it gave up: the caller reports that and leaves.
constexpr int MBAR_WAIT_LIMIT = 1 << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < MBAR_WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}

// Box load: dst (128-byte aligned shared memory) <- tensor box at coordinates (x, y, c, n), x a multiple of 4.
__device__ __forceinline__ void tma_load_box(float* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int c, int n) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(c), "r"(n) : "memory");
}

// Loads N consecutive floats that start OFF floats (0..3) after a 16-byte aligned shared-memory address:
// scalar / 64-bit loads up to the next 16-byte boundary, 128-bit loads in the middle, the rest as a tail.
template <int N, int OFF>
__device__ __forceinline__ void load_run_off(float (&dst)[N], const float* __restrict__ base) {
    constexpr int LEAD = (4 - OFF) % 4 < N ? (4 - OFF) % 4 : N;
    const float* src = base + OFF;
    int i = 0;
    if (LEAD == 1 || LEAD == 3) { dst[0] = src[0]; i = 1; }
    if (LEAD >= 2) {
        const float2 v = *reinterpret_cast<const float2*>(src + i);
        dst[i] = v.x; dst[i + 1] = v.y; i += 2;
    }
#pragma unroll
    for (; i + 4 <= N; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);
        dst[i] = v.x; dst[i + 1] = v.y; dst[i + 2] = v.z; dst[i + 3] = v.w;
    }
    if (N - i >= 2) {
        const float2 v = *reinterpret_cast<const float2*>(src + i);
        dst[i] = v.x; dst[i + 1] = v.y; i += 2;
    }
    if (N - i == 1) dst[i] = src[i];
}

}  // namespace adder
