// Host side of the tensor-map helpers and the device error flag that bounded waits report to.
#include <atomic>
#include <mutex>
#include "kernels.h"
#include "tma.cuh"

namespace adder {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's encoder, fetched through the runtime (the library does not link libcuda).
EncodeTiledFn encoder() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            (void)cudaGetLastError();
    });
    return fn;
}

// Set by kernels whose bounded wait ran out (tma.cuh); one int per GPU that loads the library.
__device__ int g_device_error = 0;
constexpr int kMaxDevices = 64;
std::atomic<int*> g_flag_addr[kMaxDevices];

}  // namespace

bool make_nchw_tensor_map(CUtensorMap* map, const float* base, int N, int C, int H, int W, int box_w, int box_h,
                          int box_c, int box_n) {
    EncodeTiledFn enc = encoder();
    if (enc == nullptr) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || W % 4 != 0 || box_w % 4 != 0) return false;
    if (box_w > 256 || box_h > 256 || box_c > 256 || box_n > 256 || box_w < 1 || box_h < 1 || box_c < 1 || box_n < 1) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)W * 4, (cuuint64_t)W * H * 4, (cuuint64_t)W * H * C * 4};
    const cuuint32_t box[4] = {(cuuint32_t)box_w, (cuuint32_t)box_h, (cuuint32_t)box_c, (cuuint32_t)box_n};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

int device_error_flag(int** flag) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ADDER_ERR_CUDA;
    int* p = g_flag_addr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        void* q = nullptr;
        if (cudaGetSymbolAddress(&q, g_device_error) != cudaSuccess || q == nullptr) {
            (void)cudaGetLastError();
            return ADDER_ERR_CUDA;
        }
        p = static_cast<int*>(q);
        g_flag_addr[dev].store(p, std::memory_order_release);
    }
    *flag = p;
    return ADDER_OK;
}

}  // namespace adder

extern "C" int adder_b200_device_status(int* status, int reset) {
    if (status == nullptr) return ADDER_ERR_NULL_POINTER;
    int* flag = nullptr;
    const int st = adder::device_error_flag(&flag);
    if (st != ADDER_OK) return st;
    if (cudaMemcpy(status, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return ADDER_ERR_CUDA;
    if (reset && *status != 0 && cudaMemset(flag, 0, sizeof(int)) != cudaSuccess) return ADDER_ERR_CUDA;
    return ADDER_OK;
}
