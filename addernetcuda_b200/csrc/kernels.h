// Internal interface between the C-ABI layer (api.cu) and the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include "common.cuh"
#include "patch_fill.cuh"
#include "../../include/adder_b200.h"

namespace adder {

// Optional overrides of the tile heuristics (0 = choose automatically).  Used for tuning sweeps.
struct TileHint {
    int threads = 0;   // CTA size target
    int cg = 0;        // channel groups per CTA
    int th = 0;        // tile rows
    int ti = 0;        // tile images
    int ck = 0;        // channels per shared-memory stage
    int smem_kb = 0;   // shared-memory budget per CTA
    int rw = 0;        // pixels per thread segment (register tile width)
    int rm = 0;        // channels per thread (register tile height)
    int variant = 0;   // weight gradient: 0 = automatic, 1 = the tiled kernel with pixel lanes, 2 = the warp-tile
                       // kernel that stages with cp.async where the default would use tiled bulk copies
    bool is_default() const { return !(threads | cg | th | ti | ck | smem_kb | rw | rm | variant); }
};

struct FwdArgs {
    Geom g;
    const float* x;
    const float* w;
    float* out;
    int TI, TH, SPR, SEGS, CG, TM, TMP, CK;
    int IN_ROWS, IN_COLS, PITCH, ROWS_PITCH, CH_STRIDE;
    int xs_stage, ws_stage, wkk_pad, WCIL, tiles_h, tiles_w, vec_store;
    int nstages;         // shared-memory stages: 2 when the input channels take several chunks, else 1
    int x_quads;         // 1x1 layers: the halo-free input patch is staged with 16-byte copies
    FastDiv d_xquads;    // divides by the patch's quads per row
    double* stats;       // optional [Co][stat_slices][2]: per pixel tile, the sum of its outputs and of their squares
    int stat_slices, stat_tpc;   // slices = pixel tiles of the launch; tpc = threads that share one channel's reduction
    PatchDims pd;        // haloed input patch staged per input-channel chunk
    FastDiv d_tiles_h, d_tiles_w, d_segs, d_spr, d_th, d_tm;
};

struct GxArgs {
    Geom g;
    const float* gout;   // [N,Co,Ho,Wo]
    const float* x;      // [N,Ci,H,W]
    const float* w;      // [Co,Ci,k,k]
    float* gx;           // [N,Ci,H,W]
    PatchDims pd;        // patch of g staged per output-channel chunk
    int TI, TH, SPRC, SPR, SEGS, CGI, TCI, TCIP, WCOL, CKO, CH_STRIDE;
    int gs_stage, ws_stage, g1_size, tiles_h, tiles_w, accumulate, class_major;
    FastDiv d_tiles_h, d_tiles_w, d_segs, d_spr, d_sprc, d_th, d_ths, d_ti, d_wpp, d_kk, d_tci;
    int vec_io;          // x is read and grad_x written as aligned quads
    // A strided 1x1 layer (pad 0) runs as a stride-1 layer on the grid of sampled pixels: `g` then describes that
    // grid (H = Ho, W = Wo), and x / grad_x are addressed through these strides of the REAL tensor.  samp = 1
    // (x_plane = H*W, x_row = W) for every other layer.
    int samp, x_plane, x_row, real_h, real_w, samp_pairs;   // samp_pairs: (value, 0) pairs can be stored as aligned 64-bit words
    int nseg;            // segments per thread: 2 in the paired stride-2 kernel, else 1
    int WPP, wgroups;    // weight staging: pairs per pass and output-channel groups (adder_bwd_input.cu)
    int nstages;         // shared-memory stages: 2 when the output channels take several chunks, else 1
};

struct GwArgs {
    Geom g;
    const float* gout;
    const float* x;
    float* part;         // [splits][Co*K] partial sums of x*g
    float* gsum_part;    // [splits][Co]   partial sums of g
    unsigned int* ticket; // zeroed by the main kernel, counted up by the finishing kernel's blocks
    PatchDims pdx;       // haloed input patch [TCI][TI*IN_ROWS][PITCH]
    PatchDims pdg;       // tile of g          [TM][TI*TH][GP]
    int TI, TH, SPR, SEGS;        // pixel tile (as in the forward kernel)
    int CGO, CGC, TM, TCI;        // output tile: TM = CGO*RM channels out, TCI = CGC*RC channels in
    int PL;                       // pixel lanes: threads that share one output tile and split the segments
    int XCH_STRIDE, GCH_STRIDE;
    int xs_stage, gs_stage, tiles_h, tiles_w, tiles_total, splits, tiles_per_split, tiles_rem, n_ci_tiles;
    FastDiv d_tiles_h, d_tiles_w, d_spr, d_th, d_pl, d_cgo, d_ci_tiles, d_gquads;
    int g_quads;         // the g tile is staged with 16-byte copies
};

struct GwFinishArgs {
    const float* part;
    const float* gsum_part;
    const float* w;
    float* gw;           // [Co*K] result (scaled when eta > 0)
    float* norm_part;    // [finish blocks] partial sums of squares
    float* out_norm;     // optional: ||gw||_2 before scaling
    int CoK, K, Co, splits, accumulate;
    float eta;
};

// Every kernel launch of the library is counted (adder_b200_launch_count): callers use it to state how
// many of these kernels a step launched.  A relaxed atomic increment on the host; nothing on the device.
void count_launch(int n = 1);
// After a launch: the status of the launch, counting it when it went through.
inline int launched(int n = 1) {
    if (cudaGetLastError() != cudaSuccess) return ADDER_ERR_CUDA;
    count_launch(n);
    return ADDER_OK;
}

// Opt a kernel in to `bytes` of dynamic shared memory.  The attribute is set once per (kernel, device), to
// the device's opt-in maximum, and remembered; later calls cost a lock and a table lookup.
int ensure_dynamic_smem(const void* kernel, size_t bytes);

int launch_fwd(const Geom& g, const float* x, const float* w, float* out, const TileHint& hint, cudaStream_t s,
               double* stats = nullptr, int stat_slices = 0);
// Number of per-channel statistic slices the forward kernel of this geometry writes (one per pixel tile);
// 0 when that kernel has no fused statistics.
int fwd_stat_slices(const Geom& g, const TileHint& hint);
int launch_gx(const Geom& g, const float* gout, const float* x, const float* w, float* gx, int fast,
              int accumulate, const TileHint& hint, cudaStream_t s);
size_t gw_workspace_bytes(const Geom& g, const TileHint& hint);
int launch_gw(const Geom& g, const float* gout, const float* x, const float* w, float* gw, float eta,
              float* out_norm, int accumulate, void* workspace, size_t workspace_bytes, const TileHint& hint,
              cudaStream_t s);

// 1x1 stride-2 layers with at most 64 channels: one thread per output position (adder_pointwise.cu).
// Chosen automatically unless a tile hint asks for the tiled kernels.
bool pointwise_applicable(const Geom& g);
int launch_pointwise_fwd(const Geom& g, const float* x, const float* w, float* out, cudaStream_t stream);
int launch_pointwise_gx(const Geom& g, const float* gout, const float* x, const float* w, float* gx, int fast,
                        int accumulate, cudaStream_t stream);
int pointwise_gw_splits(const Geom& g);
int launch_pointwise_gw(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                        unsigned int* ticket, int splits, cudaStream_t stream);

// Warp-tile weight gradient with row-range scheduling (adder_bwd_weight_pipe.cu)
bool gw_pipe_applicable(const Geom& g, const TileHint& hint);
int gw_pipe_splits(const Geom& g, const TileHint& hint);
int launch_gw_pipe(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                   unsigned int* ticket, int splits, const TileHint& hint, cudaStream_t stream);
int describe_gw_pipe(const Geom& g, const TileHint& hint, char* buf, size_t n);

// The same fed by tiled bulk copies (adder_bwd_weight_tma.cu): 3x3 stride-1 layers
bool gw_tma_applicable(const Geom& g, const TileHint& hint);
int gw_tma_splits(const Geom& g, const TileHint& hint);
int launch_gw_tma(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                  unsigned int* ticket, int splits, const TileHint& hint, cudaStream_t stream);
int describe_gw_tma(const Geom& g, const TileHint& hint, char* buf, size_t n);

bool gw1x1_applicable(const Geom& g);
int gw1x1_splits(const Geom& g);
int launch_gw1x1(const Geom& g, const float* gout, const float* x, float* part, float* gsum_part,
                 unsigned int* ticket, int splits, cudaStream_t stream);

int describe_fwd(const Geom& g, const TileHint& hint, char* buf, size_t n);
int describe_gx(const Geom& g, int fast, const TileHint& hint, char* buf, size_t n);
int describe_gw(const Geom& g, const TileHint& hint, char* buf, size_t n);

}  // namespace adder
