/*
 * adder_b200.h — C ABI of libadder_b200.so: the adder-convolution hot path of AdderNet
 * (forward, input gradient, weight gradient with the adaptive rescale) as sm_100a CUDA kernels.
 *
 * This is the boundary a host framework binds instead of the pybind11 module `adder_cuda` of
 * LingYeAI/AdderNetCUDA (adder_cuda/adder_cuda.cpp:88-93).  Plain pointers and sizes only.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer to contiguous fp32 data on the current CUDA device, unless
 *     stated otherwise; the caller owns every buffer (inputs, outputs, workspace); the library
 *     neither allocates nor frees device memory;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  All work is
 *     enqueued asynchronously on it; no call synchronises the device;
 *   - every function that can fail returns an int status: ADDER_OK (0) or one of the ADDER_ERR_*
 *     codes below; nothing is printed and the process is never aborted (the reference prints and
 *     calls abort() on shapes it cannot tile, adder_cuda/adder.cu:294-297,:436-439);
 *   - kernels are atomic-free and deterministic: the same inputs give bit-identical outputs;
 *   - NCHW entry points take the layer geometry as (n, ci, h, w, co, k, stride, pad): batch, input
 *     channels, input height/width, output channels, square kernel size, stride, symmetric zero
 *     padding.  Output size is ho = (h - k + 2*pad) / stride + 1 (integer division), wo likewise,
 *     as in adder.py:26-31.  Supported: k in {1, 3}, stride in {1, 2}, any other extent.
 */
#ifndef ADDER_B200_H_
#define ADDER_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ADDER_B200_VERSION 100

#if defined(__GNUC__)
#define ADDER_API __attribute__((visibility("default")))
#else
#define ADDER_API
#endif

enum {
    ADDER_OK = 0,
    ADDER_ERR_NULL_POINTER = 1,  /* a required pointer is NULL */
    ADDER_ERR_BAD_SHAPE = 2,     /* non-positive extent, kernel larger than the padded input, ... */
    ADDER_ERR_UNSUPPORTED = 3,   /* kernel size / stride / extent outside what the kernels cover */
    ADDER_ERR_ALIGNMENT = 4,     /* a pointer is not aligned as documented */
    ADDER_ERR_WORKSPACE = 5,     /* workspace missing or smaller than the *_workspace_bytes() answer */
    ADDER_ERR_CUDA = 6,          /* the CUDA runtime rejected a launch or an attribute */
    ADDER_ERR_INTERNAL = 7,      /* tile planner produced an impossible plan (a bug) */
    ADDER_ERR_TOO_LARGE = 8,     /* the layer needs more scratch than a fixed-capacity entry point owns */
    ADDER_ERR_TIMEOUT = 9        /* a bounded device-side wait ran out (a peer rank never arrived) */
};

/* flags for the backward entry points */
#define ADDER_FLAG_FAST_CLAMP 1  /* input gradient: saturating-add form of clamp(); differs from the
                                    exact form by about 1e-7 per term */
#define ADDER_FLAG_ACCUMULATE 2  /* add into the output buffer(s) instead of overwriting them */

/* Human-readable name of a status code (static storage, never NULL). */
ADDER_API const char* adder_b200_status_string(int status);

/* ADDER_B200_VERSION of the loaded library. */
ADDER_API int adder_b200_version(void);

/* Number of kernels this library has launched in this process so far (a host-side counter; launches
 * replayed from a captured CUDA graph are not seen).  No reference counterpart: a benchmark uses the
 * difference across one eager step to state how many of these kernels a step runs. */
ADDER_API unsigned long long adder_b200_launch_count(void);

/* Output extent of a layer; ADDER_ERR_BAD_SHAPE if the geometry is invalid.
 * Replaces the size arithmetic of adder2d_function (adder.py:26-31). */
ADDER_API int adder_b200_output_size(int h, int w, int k, int stride, int pad, int* ho, int* wo);

/* ---- fused NCHW path: what adder2d_function + adder.forward/backward compute ------------- */

/* out[n,co,ho,wo] = -sum_{ci,kh,kw} |xpad[n,ci,ho*s+kh,wo*s+kw] - w[co,ci,kh,kw]|.
 * x[n,ci,h,w], w[co,ci,k,k] -> out[n,co,ho,wo] (overwritten).
 * Replaces adder2d_function's unfold/permute glue (adder.py:32-34,38-39), adder.forward
 * (adder.py:45-60) and ADDER_CONV (adder_cuda/adder_cuda.cpp:37-46, adder.cu:19-70,:274-320). */
ADDER_API int adder_b200_forward(const float* x, const float* w, float* out, int n, int ci, int h, int wd, int co, int k,
                       int stride, int pad, void* stream);

/* grad_x[n,ci,y,x] = sum over the taps (co,kh,kw) that read that pixel of
 *                    clamp(w[co,ci,kh,kw] - x[n,ci,y,x], -1, 1) * grad_out[n,co,ho,wo].
 * Replaces the grad_i half of ADDER_BACKWARD (adder_cuda.cpp:74-86, adder.cu:245-246,:266) plus
 * the col2im that autograd runs for adder.py:32-33.  flags: ADDER_FLAG_FAST_CLAMP, _ACCUMULATE. */
ADDER_API int adder_b200_backward_input(const float* grad_out, const float* x, const float* w, float* grad_x, int n, int ci,
                              int h, int wd, int co, int k, int stride, int pad, int flags, void* stream);

/* Bytes of scratch the weight-gradient entry points need for this geometry on the current device. */
ADDER_API size_t adder_b200_backward_weight_workspace_bytes(int n, int ci, int h, int wd, int co, int k, int stride, int pad);

/* grad_w[co,ci,kh,kw] = sum_{n,ho,wo} (xpad - w) * grad_out, then, when eta > 0, the adaptive
 * rescale grad_w <- eta * sqrt(numel(grad_w)) * grad_w / max(||grad_w||_2, 1e-12) (adder.py:78 with
 * eta = 0.2).  eta <= 0 leaves the gradient unscaled.  out_norm (optional, may be NULL): receives
 * ||grad_w||_2 before scaling.  workspace: 256-byte aligned device scratch of at least
 * adder_b200_backward_weight_workspace_bytes(); contents need not be initialised and are
 * clobbered.  flags: ADDER_FLAG_ACCUMULATE (only meaningful with eta <= 0).
 * Replaces the grad_w half of ADDER_BACKWARD / ADDER_CONV_WEIGHT (adder_cuda.cpp:48-59,:74-86,
 * adder.cu:247,:267) and the rescale line adder.py:78. */
ADDER_API int adder_b200_backward_weight(const float* grad_out, const float* x, const float* w, float* grad_w, float eta,
                               float* out_norm, void* workspace, size_t workspace_bytes, int n, int ci, int h,
                               int wd, int co, int k, int stride, int pad, int flags, void* stream);

/* The same weight gradient for callers that may not allocate: plugin hosts whose memory manager owns
 * the whole GPU and forbids cudaMalloc in plugins (it stalls every stream and escapes their
 * accounting), and bindings that are only handed input and output pointers and have no allocator to
 * ask for a workspace.  The scratch is a fixed array of ADDER_B200_STATIC_SCRATCH_BYTES inside the
 * library (one per GPU that loads it, held until exit); the call allocates and frees nothing.
 * A layer whose partial sums need more returns ADDER_ERR_TOO_LARGE: use the workspace-taking entry
 * point for it.  All calls on a device share that array, so calls that can overlap on the GPU
 * (different streams without a dependency) race: serialise them.  Nothing in the array needs
 * clearing between calls.  The first call on each device looks up the array's device address, and with
 * CUDA's lazy module loading that look-up is also the moment the driver loads this part of the library and
 * reserves the array's 8 MiB: make one warm-up call per device (n = 0 is enough) at plug-in initialisation,
 * before the host's memory manager claims the GPU and outside any stream capture; later calls then truly
 * allocate nothing.  Results are identical to adder_b200_backward_weight().
 * This entry point has no counterpart in the reference. */
#define ADDER_B200_STATIC_SCRATCH_BYTES (8u << 20)
ADDER_API size_t adder_b200_static_scratch_bytes(void);
ADDER_API int adder_b200_backward_weight_static(const float* grad_out, const float* x, const float* w, float* grad_w,
                                                float eta, float* out_norm, int n, int ci, int h, int wd, int co,
                                                int k, int stride, int pad, void* stream);

/* Both gradients of one layer: adder.backward (adder.py:62-80) in one call. */
ADDER_API int adder_b200_backward(const float* grad_out, const float* x, const float* w, float* grad_x, float* grad_w,
                        float eta, void* workspace, size_t workspace_bytes, int n, int ci, int h, int wd, int co,
                        int k, int stride, int pad, int flags, void* stream);

/* ---- column-matrix path: the reference extension's own entry points ------------------------
 * Layouts as in adder_cuda/adder.cu:26-30: w[Co,K], x[K,P], y / grad_y[Co,P], grad_w[Co,K],
 * grad_i[K,P].  Any K, P, Co >= 1 (the reference requires Co and P divisible by 16, 12 or 8). */

/* y = -sum_k |w[co,k] - x[k,p]| (y is overwritten).  ADDER_CONV, adder_cuda.cpp:37-46. */
ADDER_API int adder_b200_conv_col(const float* x, const float* w, float* y, int K, int P, int Co, void* stream);

/* Scratch bytes for the two column entry points that produce grad_w. */
ADDER_API size_t adder_b200_col_workspace_bytes(int K, int P, int Co);

/* grad_w += sum_p (x - w) * grad_y (accumulates, as the reference's atomicAdd does).
 * ADDER_CONV_WEIGHT, adder_cuda.cpp:48-59. */
ADDER_API int adder_b200_conv_weight_col(const float* grad_y, const float* x, const float* w, float* grad_w, int K, int P,
                               int Co, void* workspace, size_t workspace_bytes, void* stream);

/* grad_i += sum_co clamp(w - x, -1, 1) * grad_y (accumulates).  ADDER_CONV_INPUT,
 * adder_cuda.cpp:61-72; computes the formula the reference intends (its own kernel drops the
 * multiplication by grad_y for w - x < -1, adder.cu:17,:170). */
ADDER_API int adder_b200_conv_input_col(const float* grad_y, const float* x, const float* w, float* grad_i, int K, int P,
                              int Co, void* stream);

/* Both of the above in one call.  ADDER_BACKWARD, adder_cuda.cpp:74-86. */
ADDER_API int adder_b200_backward_col(const float* grad_y, const float* x, const float* w, float* grad_w, float* grad_i,
                            int K, int P, int Co, void* workspace, size_t workspace_bytes, void* stream);

/* ---- the batch normalisation that follows every adder layer (training mode) ------------------
 * The reference networks wrap each adder2d in nn.BatchNorm2d (+ReLU, + the residual add at the end
 * of a block): resnet20.py:28-40, resnet50.py:38-53.  These entry points compute exactly that on
 * NCHW fp32 tensors [n, c, hw]: batch statistics per channel (biased variance for normalising,
 * unbiased for running_var, as torch.nn.BatchNorm2d), z = gamma*(y-mean)*invstd + beta
 * [+ residual] [then ReLU].  save_mean / save_invstd [c] are outputs kept for the backward pass;
 * running_mean / running_var [c] may both be NULL; num_batches_tracked (one int64, may be NULL) is
 * incremented by one.  Workspace: 16-byte aligned scratch of
 * adder_b200_batchnorm_workspace_bytes(); tensors must be 16-byte aligned when hw % 4 == 0. */
ADDER_API size_t adder_b200_batchnorm_workspace_bytes(int n, int c, int hw);
ADDER_API int adder_b200_batchnorm_forward(const float* y, const float* gamma, const float* beta,
                                           const float* residual, float* z, float* save_mean, float* save_invstd,
                                           float* running_mean, float* running_var, long long* num_batches_tracked,
                                           float eps, float momentum, int relu, void* workspace,
                                           size_t workspace_bytes, int n, int c, int hw, void* stream);
/* The same layer pair with the statistics pass folded into the adder layer that produces y
 * (resnet20.py:28-29: conv1 then bn1).  adder_b200_forward_with_stats is adder_b200_forward that also
 * writes, for every output channel and every pixel tile of the launch, the sum of the tile's outputs and
 * of their squares in double precision: stats[co][stat_slices][2] (16-byte aligned), stat_slices =
 * adder_b200_forward_stat_slices(same geometry), which is 0 for the geometries whose forward kernel has
 * no such epilogue (use the two calls above for those).  adder_b200_batchnorm_forward_from_stats then
 * normalises y from those slices without reading y a first time; slices are added in index order, so
 * the result is deterministic. */
ADDER_API int adder_b200_forward_stat_slices(int n, int ci, int h, int wd, int co, int k, int stride, int pad);
ADDER_API int adder_b200_forward_with_stats(const float* x, const float* w, float* out, double* stats, int stat_slices,
                                            int n, int ci, int h, int wd, int co, int k, int stride, int pad,
                                            void* stream);
ADDER_API int adder_b200_batchnorm_forward_from_stats(const float* y, const double* stats, int stat_slices,
                                                      const float* gamma, const float* beta, const float* residual,
                                                      float* z, float* save_mean, float* save_invstd,
                                                      float* running_mean, float* running_var,
                                                      long long* num_batches_tracked, float eps, float momentum,
                                                      int relu, int n, int c, int hw, void* stream);
/* Backward of batch normalisation: dz is the gradient of z; with relu != 0 it is first masked by z > 0 (z: the
 * forward output).  Outputs: dy, dgamma[c], dbeta[c] and, when dresidual != NULL, the gradient of the
 * residual input (= the masked dz). */
ADDER_API int adder_b200_batchnorm_backward(const float* dz, const float* y, const float* z, const float* gamma,
                                            const float* save_mean, const float* save_invstd, float* dy,
                                            float* dresidual, float* dgamma, float* dbeta, int relu, void* workspace,
                                            size_t workspace_bytes, int n, int c, int hw, void* stream);

/* Evaluation mode of the same layer: with running statistics batch norm is the per-channel affine map
 * scale = gamma / sqrt(running_var + eps), shift = beta - running_mean * scale, so the layer after an adder
 * convolution is z = y*scale[c] + shift[c] [+ residual] [then ReLU] in one pass over [n, c, hw] (what
 * test.py:68-90 of the reference evaluates through nn.BatchNorm2d.eval()).  residual may be NULL. */
ADDER_API int adder_b200_affine_forward(const float* y, const float* scale, const float* shift, const float* residual,
                                        float* z, int relu, int n, int c, int hw, void* stream);

/* Kernels that wait for the copy engine do so with a bounded number of polls; a wait that runs out sets a
 * flag on the device and the kernel returns early (its output is then garbage).  This reads the flag of the
 * current device into *status (0 = never happened) and, with reset != 0, clears it.  Synchronises with
 * the device.  No reference counterpart. */
ADDER_API int adder_b200_device_status(int* status, int reset);

/* ---- gradient exchange between the GPUs of one node (batch-sharded training) ---------------------
 * The reference trains on one GPU (nn.DataParallel appears only in its evaluation script, test.py:37); with
 * one process per GPU the per-rank gradients (adder weight gradients already rescaled, adder.py:78) have to
 * be averaged once per step.  adder_b200_peer_allreduce does that for one flat fp32 bucket in ONE kernel
 * over peer memory: every rank stores its bucket into a receive area of every rank, signals per chunk, waits
 * (bounded) for the other ranks' chunks and adds them in rank order - bit-identical results on all ranks.
 *
 * Set-up, once per bucket: each rank allocates a zeroed, 16-byte aligned receive area of
 * adder_b200_peer_area_bytes(n, world) bytes in ordinary device memory, exports it with
 * adder_b200_ipc_export (handle + offset of the pointer inside its allocation), the ranks exchange those 72
 * bytes by any means, map each other's areas with adder_b200_ipc_open (once per distinct handle per process)
 * and synchronise once; then adder_b200_peer_comm_create(areas = the world area pointers as seen from this
 * process, own area included; n % 4 == 0; chunks = 0 lets the library choose; max_polls bounds the wait, a
 * poll being 32-256 ns).  first_rank / ranks_here / data[ranks_here] describe the ranks this process drives:
 * one in production; several only to emulate a multi-rank exchange on one GPU (a single cooperative launch).
 * The call is stream-ordered and can be captured in a CUDA graph (the epoch counter lives in device memory).
 * A wait that ran out leaves ADDER_ERR_TIMEOUT in the communicator's status word: read it with
 * adder_b200_peer_comm_status (a device-to-host copy; reset != 0 clears it). */
ADDER_API size_t adder_b200_peer_area_bytes(long long n, int world);
ADDER_API int adder_b200_ipc_export(const void* ptr, unsigned char* handle64, unsigned long long* offset);
ADDER_API int adder_b200_ipc_open(const unsigned char* handle64, unsigned long long offset, void** ptr);
ADDER_API int adder_b200_ipc_close(void* ptr, unsigned long long offset);
ADDER_API int adder_b200_peer_comm_create(void** comm, int world, int first_rank, int ranks_here, float* const* data,
                                          void* const* areas, long long n, int chunks, int max_polls);
ADDER_API int adder_b200_peer_allreduce(void* comm, void* stream);
ADDER_API int adder_b200_peer_comm_status(void* comm, int* status, unsigned* epoch, int reset);
ADDER_API int adder_b200_peer_comm_destroy(void* comm);

#ifdef ADDER_B200_TUNING
/* ---- tuning build only (libadder_b200_tuning.so, compiled with -DADDER_B200_TUNING) ---------------
 * The product library exports none of these and keeps no tile state: any thread calling a setter would
 * change every other thread's kernels.  Parameter sweeps and the tests that must reach a particular
 * kernel variant load the tuning library instead.  No reference counterpart. */

/* Overrides the tile heuristics of one kernel family for subsequent calls from any thread
 * (op: 0 forward, 1 input gradient, 2 weight gradient; a value of 0 restores the automatic choice). */
ADDER_API int adder_b200_set_tile_hint(int op, int threads, int channel_groups, int tile_rows, int tile_images,
                             int chunk_channels, int smem_kb);

/* Overrides the per-thread register tile of one kernel family (pixels per thread segment: 4, 7 or 8;
 * channels per thread: 4 or 8; 0,0 restores the automatic choice). */
ADDER_API int adder_b200_set_micro_tile(int op, int pixels_per_thread, int channels_per_thread);

/* Kernel family of the weight gradient (op 2; ignored for the other ops): 0 = automatic, 1 = the tiled
 * kernel with pixel lanes everywhere (also instead of the 1x1 GEMM kernel), 2 = the warp-tile kernel that
 * stages with cp.async where the default would use tiled bulk copies. */
ADDER_API int adder_b200_set_variant(int op, int variant);
#endif /* ADDER_B200_TUNING */

/* Writes a one-line description of the tile plan the library would use for this layer on the
 * current device (op: 0 forward, 1 input gradient, 2 weight gradient) into buf (NUL-terminated,
 * truncated to buf_bytes).  Launches nothing; works without a GPU.  No reference counterpart. */
ADDER_API int adder_b200_describe_plan(int op, int n, int ci, int h, int wd, int co, int k, int stride, int pad,
                                       int flags, char* buf, size_t buf_bytes);

#ifdef __cplusplus
}
#endif
#endif /* ADDER_B200_H_ */
