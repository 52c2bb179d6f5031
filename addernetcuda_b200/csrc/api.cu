// extern "C" layer of libadder_b200.so: argument validation, geometry, dispatch to the kernels.
#include <atomic>
#include <map>
#include <mutex>
#include <utility>
#include "kernels.h"

using namespace adder;

namespace {

#ifdef ADDER_B200_TUNING
// Tuning build only (libadder_b200_tuning.so): process-wide overrides of the tile heuristics, set through
// adder_b200_set_tile_hint / _set_micro_tile / _set_variant.  The product library has none of this: its
// kernels are always chosen by the planners, and it keeps no mutable state besides the launch counter
// and the documented static scratch array.
struct HintSlot {
    std::atomic<int> threads{0}, cg{0}, th{0}, ti{0}, ck{0}, smem_kb{0}, rw{0}, rm{0}, variant{0};
    TileHint load() const {
        TileHint h;
        h.threads = threads.load(std::memory_order_relaxed);
        h.cg = cg.load(std::memory_order_relaxed);
        h.th = th.load(std::memory_order_relaxed);
        h.ti = ti.load(std::memory_order_relaxed);
        h.ck = ck.load(std::memory_order_relaxed);
        h.smem_kb = smem_kb.load(std::memory_order_relaxed);
        h.rw = rw.load(std::memory_order_relaxed);
        h.rm = rm.load(std::memory_order_relaxed);
        h.variant = variant.load(std::memory_order_relaxed);
        return h;
    }
};
HintSlot g_hints[3];
TileHint current_hint(int op) { return g_hints[op].load(); }
#else
TileHint current_hint(int) { return TileHint(); }
#endif
std::atomic<unsigned long long> g_launches{0};


// Validates a layer geometry and fills Geom.  Every tensor must have fewer than 2^31 elements
// (the kernels index tiles with 32-bit integers and element offsets with 64-bit ones).
int make_geom(int n, int ci, int h, int wd, int co, int k, int stride, int pad, Geom* g) {
    if (n < 0 || ci <= 0 || h <= 0 || wd <= 0 || co <= 0 || k <= 0 || stride <= 0 || pad < 0) return ADDER_ERR_BAD_SHAPE;
    if (h + 2 * pad < k || wd + 2 * pad < k) return ADDER_ERR_BAD_SHAPE;
    if (!((k == 1 || k == 3) && (stride == 1 || stride == 2))) return ADDER_ERR_UNSUPPORTED;
    if (pad >= k) return ADDER_ERR_UNSUPPORTED;   // a tap row made only of padding never occurs in the callers
    g->N = n; g->Ci = ci; g->H = h; g->W = wd; g->Co = co; g->k = k; g->stride = stride; g->pad = pad;
    g->Ho = (h - k + 2 * pad) / stride + 1;
    g->Wo = (wd - k + 2 * pad) / stride + 1;
    const long long lim = 2147483647LL;
    if ((long long)n * ci * h * wd > lim || (long long)n * co * g->Ho * g->Wo > lim || (long long)co * ci * k * k > lim)
        return ADDER_ERR_UNSUPPORTED;
    return ADDER_OK;
}

int make_col_geom(int K, int P, int Co, Geom* g) {
    if (K <= 0 || P < 0 || Co <= 0) return ADDER_ERR_BAD_SHAPE;
    // X[K,P] is an NCHW tensor [1,K,1,P]; W[Co,K] is [Co,K,1,1]; Y[Co,P] is [1,Co,1,P].
    return make_geom(1, K, 1, P > 0 ? P : 1, Co, 1, 1, 0, g);
}

}  // namespace

namespace adder {
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

int ensure_dynamic_smem(const void* kernel, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, size_t> granted;     // (kernel, device) -> bytes opted in
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return ADDER_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    auto it = granted.find({kernel, dev});
    if (it == granted.end()) {
        int optin = 0;
        if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess || optin <= 0)
            return ADDER_ERR_CUDA;
        // the opt-in limit covers static and dynamic shared memory together
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess) {
            (void)cudaGetLastError();
            return ADDER_ERR_CUDA;
        }
        const int dyn = optin - (int)fa.sharedSizeBytes;
        if (dyn <= 0 || cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) != cudaSuccess) {
            (void)cudaGetLastError();
            return ADDER_ERR_CUDA;
        }
        it = granted.emplace(std::make_pair(kernel, dev), (size_t)dyn).first;
    }
    return bytes <= it->second ? ADDER_OK : ADDER_ERR_UNSUPPORTED;
}
}  // namespace adder

extern "C" {

const char* adder_b200_status_string(int status) {
    switch (status) {
        case ADDER_OK: return "ok";
        case ADDER_ERR_NULL_POINTER: return "null pointer";
        case ADDER_ERR_BAD_SHAPE: return "bad shape";
        case ADDER_ERR_UNSUPPORTED: return "unsupported kernel size, stride or extent";
        case ADDER_ERR_ALIGNMENT: return "misaligned pointer";
        case ADDER_ERR_WORKSPACE: return "workspace missing or too small";
        case ADDER_ERR_CUDA: return "CUDA runtime error";
        case ADDER_ERR_INTERNAL: return "internal tile-planning error";
        case ADDER_ERR_TOO_LARGE: return "layer needs more scratch than the fixed in-library array holds";
        case ADDER_ERR_TIMEOUT: return "a bounded device-side wait ran out (a peer rank never arrived)";
        default: return "unknown status";
    }
}

int adder_b200_version(void) { return ADDER_B200_VERSION; }

unsigned long long adder_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int adder_b200_output_size(int h, int w, int k, int stride, int pad, int* ho, int* wo) {
    if (ho == nullptr || wo == nullptr) return ADDER_ERR_NULL_POINTER;
    if (h <= 0 || w <= 0 || k <= 0 || stride <= 0 || pad < 0 || h + 2 * pad < k || w + 2 * pad < k)
        return ADDER_ERR_BAD_SHAPE;
    *ho = (h - k + 2 * pad) / stride + 1;
    *wo = (w - k + 2 * pad) / stride + 1;
    return ADDER_OK;
}

int adder_b200_forward(const float* x, const float* w, float* out, int n, int ci, int h, int wd, int co, int k,
                       int stride, int pad, void* stream) {
    Geom g;
    const int st = make_geom(n, ci, h, wd, co, k, stride, pad, &g);
    if (st != ADDER_OK) return st;
    if (n == 0) return ADDER_OK;
    if (x == nullptr || w == nullptr || out == nullptr) return ADDER_ERR_NULL_POINTER;
    return launch_fwd(g, x, w, out, current_hint(0), static_cast<cudaStream_t>(stream));
}

int adder_b200_forward_stat_slices(int n, int ci, int h, int wd, int co, int k, int stride, int pad) {
    Geom g;
    if (make_geom(n, ci, h, wd, co, k, stride, pad, &g) != ADDER_OK || n == 0) return 0;
    return fwd_stat_slices(g, current_hint(0));
}

int adder_b200_forward_with_stats(const float* x, const float* w, float* out, double* stats, int stat_slices, int n,
                                  int ci, int h, int wd, int co, int k, int stride, int pad, void* stream) {
    Geom g;
    const int st = make_geom(n, ci, h, wd, co, k, stride, pad, &g);
    if (st != ADDER_OK) return st;
    if (n == 0) return ADDER_ERR_BAD_SHAPE;      // an empty batch has no statistics
    if (x == nullptr || w == nullptr || out == nullptr || stats == nullptr) return ADDER_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(stats) & 15) != 0) return ADDER_ERR_ALIGNMENT;
    if (stat_slices <= 0 || stat_slices != fwd_stat_slices(g, current_hint(0))) return ADDER_ERR_WORKSPACE;
    return launch_fwd(g, x, w, out, current_hint(0), static_cast<cudaStream_t>(stream), stats, stat_slices);
}

int adder_b200_backward_input(const float* grad_out, const float* x, const float* w, float* grad_x, int n, int ci,
                              int h, int wd, int co, int k, int stride, int pad, int flags, void* stream) {
    Geom g;
    const int st = make_geom(n, ci, h, wd, co, k, stride, pad, &g);
    if (st != ADDER_OK) return st;
    if (n == 0) return ADDER_OK;
    if (grad_out == nullptr || x == nullptr || w == nullptr || grad_x == nullptr) return ADDER_ERR_NULL_POINTER;
    return launch_gx(g, grad_out, x, w, grad_x, (flags & ADDER_FLAG_FAST_CLAMP) != 0,
                     (flags & ADDER_FLAG_ACCUMULATE) != 0, current_hint(1), static_cast<cudaStream_t>(stream));
}

size_t adder_b200_backward_weight_workspace_bytes(int n, int ci, int h, int wd, int co, int k, int stride, int pad) {
    Geom g;
    if (make_geom(n, ci, h, wd, co, k, stride, pad, &g) != ADDER_OK) return 0;
    if (n == 0) g.N = 1;
    return gw_workspace_bytes(g, current_hint(2));
}

int adder_b200_backward_weight(const float* grad_out, const float* x, const float* w, float* grad_w, float eta,
                               float* out_norm, void* workspace, size_t workspace_bytes, int n, int ci, int h,
                               int wd, int co, int k, int stride, int pad, int flags, void* stream) {
    Geom g;
    const int st = make_geom(n, ci, h, wd, co, k, stride, pad, &g);
    if (st != ADDER_OK) return st;
    if (w == nullptr || grad_w == nullptr) return ADDER_ERR_NULL_POINTER;
    if (n > 0 && (grad_out == nullptr || x == nullptr)) return ADDER_ERR_NULL_POINTER;
    // An empty batch still defines the gradient (all zeros); the kernels handle N = 0 tiles.
    return launch_gw(g, grad_out, x, w, grad_w, eta, out_norm, (flags & ADDER_FLAG_ACCUMULATE) != 0, workspace,
                     workspace_bytes, current_hint(2), static_cast<cudaStream_t>(stream));
}

int adder_b200_backward(const float* grad_out, const float* x, const float* w, float* grad_x, float* grad_w,
                        float eta, void* workspace, size_t workspace_bytes, int n, int ci, int h, int wd, int co,
                        int k, int stride, int pad, int flags, void* stream) {
    int st = adder_b200_backward_input(grad_out, x, w, grad_x, n, ci, h, wd, co, k, stride, pad, flags, stream);
    if (st != ADDER_OK) return st;
    return adder_b200_backward_weight(grad_out, x, w, grad_w, eta, nullptr, workspace, workspace_bytes, n, ci, h, wd,
                                      co, k, stride, pad, flags & ADDER_FLAG_ACCUMULATE, stream);
}

int adder_b200_conv_col(const float* x, const float* w, float* y, int K, int P, int Co, void* stream) {
    Geom g;
    const int st = make_col_geom(K, P, Co, &g);
    if (st != ADDER_OK) return st;
    if (P == 0) return ADDER_OK;
    if (x == nullptr || w == nullptr || y == nullptr) return ADDER_ERR_NULL_POINTER;
    return launch_fwd(g, x, w, y, current_hint(0), static_cast<cudaStream_t>(stream));
}

size_t adder_b200_col_workspace_bytes(int K, int P, int Co) {
    Geom g;
    if (make_col_geom(K, P, Co, &g) != ADDER_OK) return 0;
    return gw_workspace_bytes(g, current_hint(2));
}

int adder_b200_conv_weight_col(const float* grad_y, const float* x, const float* w, float* grad_w, int K, int P,
                               int Co, void* workspace, size_t workspace_bytes, void* stream) {
    Geom g;
    const int st = make_col_geom(K, P, Co, &g);
    if (st != ADDER_OK) return st;
    if (P == 0) return ADDER_OK;   // accumulating nothing
    if (grad_y == nullptr || x == nullptr || w == nullptr || grad_w == nullptr) return ADDER_ERR_NULL_POINTER;
    return launch_gw(g, grad_y, x, w, grad_w, 0.f, nullptr, 1, workspace, workspace_bytes, current_hint(2),
                     static_cast<cudaStream_t>(stream));
}

int adder_b200_conv_input_col(const float* grad_y, const float* x, const float* w, float* grad_i, int K, int P,
                              int Co, void* stream) {
    Geom g;
    const int st = make_col_geom(K, P, Co, &g);
    if (st != ADDER_OK) return st;
    if (P == 0) return ADDER_OK;
    if (grad_y == nullptr || x == nullptr || w == nullptr || grad_i == nullptr) return ADDER_ERR_NULL_POINTER;
    return launch_gx(g, grad_y, x, w, grad_i, 0, 1, current_hint(1), static_cast<cudaStream_t>(stream));
}

int adder_b200_backward_col(const float* grad_y, const float* x, const float* w, float* grad_w, float* grad_i,
                            int K, int P, int Co, void* workspace, size_t workspace_bytes, void* stream) {
    int st = adder_b200_conv_input_col(grad_y, x, w, grad_i, K, P, Co, stream);
    if (st != ADDER_OK) return st;
    return adder_b200_conv_weight_col(grad_y, x, w, grad_w, K, P, Co, workspace, workspace_bytes, stream);
}

int adder_b200_describe_plan(int op, int n, int ci, int h, int wd, int co, int k, int stride, int pad, int flags,
                             char* buf, size_t buf_bytes) {
    if (buf == nullptr || buf_bytes == 0) return ADDER_ERR_NULL_POINTER;
    Geom g;
    const int st = make_geom(n, ci, h, wd, co, k, stride, pad, &g);
    if (st != ADDER_OK) return st;
    buf[0] = 0;
    if (op == 0) return describe_fwd(g, current_hint(0), buf, buf_bytes);
    if (op == 1) return describe_gx(g, (flags & ADDER_FLAG_FAST_CLAMP) != 0, current_hint(1), buf, buf_bytes);
    if (op == 2) return describe_gw(g, current_hint(2), buf, buf_bytes);
    return ADDER_ERR_BAD_SHAPE;
}

#ifdef ADDER_B200_TUNING
int adder_b200_set_tile_hint(int op, int threads, int channel_groups, int tile_rows, int tile_images,
                             int chunk_channels, int smem_kb) {
    if (op < 0 || op > 2) return ADDER_ERR_BAD_SHAPE;
    HintSlot& s = g_hints[op];
    s.threads.store(threads); s.cg.store(channel_groups); s.th.store(tile_rows); s.ti.store(tile_images);
    s.ck.store(chunk_channels); s.smem_kb.store(smem_kb);
    return ADDER_OK;
}

int adder_b200_set_variant(int op, int variant) {
    if (op < 0 || op > 2 || variant < 0 || variant > 2) return ADDER_ERR_BAD_SHAPE;
    g_hints[op].variant.store(variant);
    return ADDER_OK;
}

int adder_b200_set_micro_tile(int op, int pixels_per_thread, int channels_per_thread) {
    if (op < 0 || op > 2) return ADDER_ERR_BAD_SHAPE;
    g_hints[op].rw.store(pixels_per_thread);
    g_hints[op].rm.store(channels_per_thread);
    return ADDER_OK;
}
#endif  // ADDER_B200_TUNING

}  // extern "C"
