// Cooperative asynchronous copy of a zero-filled rectangular patch of an NCHW tensor into shared
// memory: dst[(c*TI + i)*ROWS_PITCH + r*PITCH + q] = src[n0+i, c0+c, row0+r, col0+q], or 0 where
// any index falls outside the tensor (that is how padding and ragged tile edges are produced).
#pragma once
#include "common.cuh"

namespace adder {

struct PatchDims {
    int CH, TI, ROWS, COLS, PITCH, ROWS_PITCH;   // patch extents and shared-memory pitches
    FastDiv d_cols, d_rows, d_ti;
};

__device__ __forceinline__ void fill_patch(float* dst, const float* __restrict__ src, const PatchDims& p,
                                           int n0, int c0, int row0, int col0, int N, int C, int Hs, int Ws,
                                           int tid, int nthreads) {
    const int elems = p.CH * p.TI * p.ROWS * p.COLS;
    const int plane = Hs * Ws;
    for (int e = tid; e < elems; e += nthreads) {
        uint32_t rho, q, rho2, r, c, i;
        p.d_cols.divmod(e, rho, q);
        p.d_rows.divmod(rho, rho2, r);
        p.d_ti.divmod(rho2, c, i);
        const int n = n0 + (int)i, ch = c0 + (int)c, row = row0 + (int)r, col = col0 + (int)q;
        const bool ok = (n < N) & (ch < C) & (row >= 0) & (row < Hs) & (col >= 0) & (col < Ws);
        const float* s = ok ? src + ((size_t)(n * C + ch) * plane + row * Ws + col) : src;
        cp_async4(dst + (c * p.TI + i) * p.ROWS_PITCH + r * p.PITCH + q, s, ok);
    }
}

}  // namespace adder
