// Cooperative asynchronous copy of a zero-filled rectangular patch of an NCHW tensor into shared
// memory: dst[(c*TI + i)*ROWS_PITCH + r*PITCH + q] = src[n0+i, c0+c, row0+r*GS, col0+q*GS], or 0 where
// any index falls outside the tensor (that is how padding and ragged tile edges are produced).
#pragma once
#include "common.cuh"

namespace adder {

struct PatchDims {
    int CH, TI, ROWS, COLS, PITCH, ROWS_PITCH;   // patch extents and shared-memory pitches
    int CHS = 0;                                 // channel stride if it is not TI*ROWS_PITCH (padded planes)
    int GS = 1;                                  // gather stride: patch position (r, q) reads src[row0 + r*GS, col0 + q*GS]
    FastDiv d_cols, d_rows;
};

// With DUP every value is stored twice in a row (dst[... + r*PITCH + 2*q] and the word after it; PITCH then
// counts the doubled row), so that a 64-bit shared-memory load yields the pair (v, v) a packed f32x2
// instruction wants as its broadcast operand, without any register moves.
template <bool DUP = false>
__device__ __forceinline__ void fill_patch(float* dst, const float* __restrict__ src, const PatchDims& p,
                                           int n0, int c0, int row0, int col0, int N, int C, int Hs, int Ws,
                                           int tid, int nthreads) {
    // The (image, row, column) decoding and the bounds test are done once per patch position and
    // reused for every channel of the chunk; per channel only two adds and the copy remain.
    const int plane_elems = p.TI * p.ROWS * p.COLS;
    const int plane = Hs * Ws;
    const int ch_stride = p.CHS ? p.CHS : p.TI * p.ROWS_PITCH;
    const int nch = C - c0 < p.CH ? C - c0 : p.CH;      // channels past the tensor's end are zero-filled
    for (int e = tid; e < plane_elems; e += nthreads) {
        uint32_t rho, q, i, r;
        p.d_cols.divmod(e, rho, q);
        p.d_rows.divmod(rho, i, r);
        const int n = n0 + (int)i, row = row0 + (int)r * p.GS, col = col0 + (int)q * p.GS;
        const bool ok = (n < N) & (row >= 0) & (row < Hs) & (col >= 0) & (col < Ws);
        const float* s = ok ? src + ((size_t)(n * C + c0) * plane + row * Ws + col) : src;
        float* d = dst + i * p.ROWS_PITCH + r * p.PITCH + (DUP ? 2 * q : q);
#pragma unroll 4
        for (int c = 0; c < p.CH; ++c) {
            const bool okc = ok & (c < nch);
            const float* sc = okc ? s + (size_t)c * plane : src;
            cp_async4(d + c * ch_stride, sc, okc);
            if (DUP) cp_async4(d + c * ch_stride + 1, sc, okc);
        }
    }
}

// The same copy in 16-byte pieces, for patches without a halo whose rows start on a 16-byte boundary in
// both memories: COLS, PITCH, col0 and Ws multiples of 4, src 16-byte aligned, row0/col0 >= 0 not
// required (a quad is either wholly inside the row or wholly outside it, because Ws % 4 == 0).
// `d_quads` divides by COLS / 4.
__device__ __forceinline__ void fill_patch_quads(float* dst, const float* __restrict__ src, const PatchDims& p,
                                                 const FastDiv& d_quads, int n0, int c0, int row0, int col0, int N,
                                                 int C, int Hs, int Ws, int tid, int nthreads) {
    const int qcols = p.COLS >> 2;
    const int plane_quads = p.TI * p.ROWS * qcols;
    const int plane = Hs * Ws;
    const int ch_stride = p.CHS ? p.CHS : p.TI * p.ROWS_PITCH;
    const int nch = C - c0 < p.CH ? C - c0 : p.CH;
    for (int e = tid; e < plane_quads; e += nthreads) {
        uint32_t rho, q, i, r;
        d_quads.divmod(e, rho, q);
        p.d_rows.divmod(rho, i, r);
        const int n = n0 + (int)i, row = row0 + (int)r, col = col0 + 4 * (int)q;
        const bool ok = (n < N) & (row >= 0) & (row < Hs) & (col >= 0) & (col < Ws);
        const float* s = ok ? src + ((size_t)(n * C + c0) * plane + row * Ws + col) : src;
        float* d = dst + i * p.ROWS_PITCH + r * p.PITCH + 4 * q;
#pragma unroll 4
        for (int c = 0; c < p.CH; ++c) {
            const bool okc = ok & (c < nch);
            cp_async16(d + c * ch_stride, okc ? s + (size_t)c * plane : src, okc);
        }
    }
}

}  // namespace adder
