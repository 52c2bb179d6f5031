// Weight gradient for callers that cannot hand over a workspace: the scratch lives inside the
// library, in a fixed-size __device__ array, so this entry point never allocates.
//
// Who needs it.  Some hosts are not allowed to allocate device memory at the point where they call a
// plugin: a serving process whose memory manager has claimed the whole GPU up front and treats any
// cudaMalloc from a plugin as a bug (it stalls every stream of the device and escapes the manager's
// accounting), or a foreign-language binding that is only ever handed input and output pointers by
// its framework and has no allocator it could ask for the workspace that
// adder_b200_backward_weight() wants.  Those callers pass inputs and outputs only.
//
// Limits and sharing.  The array is ADDER_B200_STATIC_SCRATCH_BYTES (8 MiB) per GPU that loads the
// library, held until the process exits.  A geometry whose partial sums do not fit is refused with
// ADDER_ERR_TOO_LARGE (all 20 adder layers of ResNet-20 at batch 256 fit; the wide ResNet-50 layers
// do not).  Every call on a device uses the same array and finds the previous call's contents in
// it; that is harmless, because the kernels write every scratch word they later read (each CTA
// stores its whole slice of partial sums, including CTAs that had no pixels to process), so nothing
// has to be cleared.  For the same reason two calls that run on the GPU at the same time (different
// streams, no dependency) would overwrite each other's partial sums: serialise them.
//
// Set-up.  Host code cannot use the array's name as a device address.  The first call on each device
// resolves the real address with cudaGetSymbolAddress() while that device is current and caches it;
// make that first call outside any stream capture.
#include <atomic>
#include "kernels.h"

namespace {

constexpr size_t kScratchBytes = ADDER_B200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_addr[kMaxDevices];   // zero-initialised: address not resolved yet

// Device address of g_static_scratch on the current device (resolved once per device).
int scratch_address(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ADDER_ERR_CUDA;
    void* p = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return ADDER_ERR_CUDA;
        }
        g_scratch_addr[dev].store(p, std::memory_order_release);   // racing threads resolve the same address
    }
    *out = p;
    return ADDER_OK;
}

}  // namespace

extern "C" {

size_t adder_b200_static_scratch_bytes(void) { return kScratchBytes; }

int adder_b200_backward_weight_static(const float* grad_out, const float* x, const float* w, float* grad_w, float eta,
                                      float* out_norm, int n, int ci, int h, int wd, int co, int k, int stride,
                                      int pad, void* stream) {
    if (w == nullptr || grad_w == nullptr) return ADDER_ERR_NULL_POINTER;
    if (n > 0 && (grad_out == nullptr || x == nullptr)) return ADDER_ERR_NULL_POINTER;
    // Same geometry rules and the same scratch requirement as the workspace-taking entry point.
    const size_t need = adder_b200_backward_weight_workspace_bytes(n, ci, h, wd, co, k, stride, pad);
    if (need == 0)   // invalid geometry or no plan: the workspace-taking entry point reports which (it cannot launch without scratch)
        return adder_b200_backward_weight(grad_out, x, w, grad_w, eta, out_norm, nullptr, 0, n, ci, h, wd, co, k, stride,
                                          pad, 0, stream);
    if (need > kScratchBytes) return ADDER_ERR_TOO_LARGE;
    void* scratch = nullptr;
    const int st = scratch_address(&scratch);
    if (st != ADDER_OK) return st;
    return adder_b200_backward_weight(grad_out, x, w, grad_w, eta, out_norm, scratch, kScratchBytes, n, ci, h, wd, co,
                                      k, stride, pad, 0, stream);
}

}  // extern "C"
