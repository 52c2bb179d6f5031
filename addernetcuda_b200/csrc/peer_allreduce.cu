// One-shot average of a flat fp32 gradient bucket over the GPUs of one node, through peer memory.
//
// The reference trains on one GPU (its only multi-GPU construct is nn.DataParallel for evaluation,
// test.py:37); batch-sharded training needs one exchange per step: the average of the ranks' gradients,
// adder weight gradients already rescaled per rank (adder.py:78).  For the bucket sizes of the CIFAR
// networks (ResNet-20: 1.09 MB in all) a ring all-reduce is all latency, so this kernel does the exchange
// in one step:
//
//   every rank owns a RECEIVE AREA that its peers can address (CUDA IPC mapping over NVLink):
//       slots  [parity 2][source rank][slot floats]      flags  [parity 2][source rank][MAX_CHUNKS]
//   CTA c of rank r   1. stores chunk c of r's bucket into slot [parity][r] of EVERY rank's area (its own too),
//                     2. fences and writes the call's epoch into flag [parity][r][c] of every rank,
//                     3. waits until flags [parity][0..world)[c] of its OWN area carry the epoch (bounded),
//                     4. adds the world copies of chunk c in rank order, scales by 1/world and writes the
//                        result back into r's bucket.
// One wait per call, on chunk granularity: CTA c depends only on CTA c of the other ranks, and it pushes
// before it waits, so no rank waits for data that itself is waiting.  The sum runs in rank order on every
// rank: replicas receive bit-identical averages.  Slots and flags alternate between two parities by epoch:
// a rank can start call e+1 while a slower peer still reads call e's slots, and cannot reach call e+2 before
// that peer has finished e (its own flags for e+1 are still missing).  The epoch lives in device memory and
// is advanced by the last CTA of each call, so a captured CUDA graph can replay the launch unchanged.
//
// A wait that runs out (a peer that never launched) does not hang: the CTA records ADDER_ERR_TIMEOUT in the
// communicator's status word, skips the reduction and returns; the host reads the word with
// adder_b200_peer_comm_status.  No multicast, no TMA: plain 128-bit peer stores and local loads.
#include <cuda.h>
#include "common.cuh"
#include "kernels.h"
#include <cstring>
#include <vector>

namespace adder {

constexpr int PEER_MAX_CHUNKS = 256;
constexpr int PEER_THREADS = 256;
constexpr int PEER_MAX_WORLD = 16;

struct PeerArgs {
    float* data;                 // this rank's bucket [n]: input and (averaged) output
    float* area[PEER_MAX_WORLD]; // receive area of every rank, as addressed from this rank
    unsigned* state;             // local: [0] completed epochs, [1] CTAs done in the current call, [2] status
    long long n4;                // bucket length in 128-bit words
    long long slot4;             // 128-bit words per slot
    long long flags_off4;        // offset of the flag block inside an area, in 128-bit words
    int rank, world, chunks, max_polls;
    float scale;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// grid (chunks, ranks in this launch): ranks > 1 only when several ranks are emulated on one GPU (cooperative
// launch: their CTAs wait on each other).
__global__ void __launch_bounds__(PEER_THREADS) peer_allreduce_kernel(const PeerArgs* __restrict__ all) {
    const PeerArgs& a = all[blockIdx.y];
    __shared__ unsigned s_epoch;
    __shared__ int s_fail;
    const int tid = threadIdx.x;
    if (tid == 0) {
        s_epoch = *reinterpret_cast<volatile unsigned*>(a.state) + 1u;
        s_fail = 0;
    }
    __syncthreads();
    const unsigned epoch = s_epoch;
    const int parity = (int)(epoch & 1u);
    const int c = blockIdx.x;
    const long long per = (a.n4 + a.chunks - 1) / a.chunks;
    const long long q0 = (long long)c * per;
    const long long q1 = q0 + per < a.n4 ? q0 + per : a.n4;
    const float4* src = reinterpret_cast<const float4*>(a.data);

    // 1. push
    const long long my_slot = ((long long)parity * a.world + a.rank) * a.slot4;
    for (long long q = q0 + tid; q < q1; q += PEER_THREADS) {
        const float4 v = src[q];
        for (int p = 0; p < a.world; ++p) reinterpret_cast<float4*>(a.area[p])[my_slot + q] = v;
    }
    __syncthreads();
    // 2. signal, 3. wait
    if (tid < a.world) {
        __threadfence_system();
        unsigned* theirs = reinterpret_cast<unsigned*>(reinterpret_cast<float4*>(a.area[tid]) + a.flags_off4);
        st_release_sys(theirs + ((size_t)parity * a.world + a.rank) * PEER_MAX_CHUNKS + c, epoch);
        const unsigned* mine = reinterpret_cast<const unsigned*>(reinterpret_cast<const float4*>(a.area[a.rank]) + a.flags_off4) +
                               ((size_t)parity * a.world + tid) * PEER_MAX_CHUNKS + c;
        int polls = 0;
        while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
            if (++polls > a.max_polls) { atomicExch(&s_fail, 1); break; }
            __nanosleep(polls < 64 ? 32 : 256);
        }
    }
    __syncthreads();
    if (s_fail) {
        if (tid == 0) atomicExch(a.state + 2, (unsigned)ADDER_ERR_TIMEOUT);
    } else {
        // 4. reduce in rank order
        const float4* in = reinterpret_cast<const float4*>(a.area[a.rank]) + (long long)parity * a.world * a.slot4;
        float4* dst = reinterpret_cast<float4*>(a.data);
        for (long long q = q0 + tid; q < q1; q += PEER_THREADS) {
            float4 s = __ldcg(in + q);
            for (int p = 1; p < a.world; ++p) {
                const float4 v = __ldcg(in + (long long)p * a.slot4 + q);
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            dst[q] = make_float4(s.x * a.scale, s.y * a.scale, s.z * a.scale, s.w * a.scale);
        }
    }
    // 5. the last CTA of the call advances the epoch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(a.state + 1, 1u) == gridDim.x - 1) {
            a.state[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(a.state) = epoch;
        }
    }
}

struct PeerComm {
    PeerArgs* d_args = nullptr;
    unsigned* d_state = nullptr;
    int ranks_here = 0, chunks = 0, device = -1;
};

typedef CUresult (*AddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

static AddressRangeFn address_range_fn() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return reinterpret_cast<AddressRangeFn>(p);
}

}  // namespace adder

using namespace adder;

extern "C" {

size_t adder_b200_peer_area_bytes(long long n, int world) {
    if (n <= 0 || world < 1 || world > PEER_MAX_WORLD) return 0;
    const long long slot4 = (n + 3) / 4;
    return (size_t)(2LL * world * slot4 * 16 + 2LL * world * PEER_MAX_CHUNKS * 4);
}

int adder_b200_ipc_export(const void* ptr, unsigned char* handle64, unsigned long long* offset) {
    if (ptr == nullptr || handle64 == nullptr || offset == nullptr) return ADDER_ERR_NULL_POINTER;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    AddressRangeFn range = address_range_fn();
    if (range == nullptr) return ADDER_ERR_CUDA;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return ADDER_ERR_CUDA;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
        (void)cudaGetLastError();
        return ADDER_ERR_CUDA;
    }
    std::memcpy(handle64, &h, 64);
    *offset = (unsigned long long)(reinterpret_cast<CUdeviceptr>(ptr) - base);
    return ADDER_OK;
}

int adder_b200_ipc_open(const unsigned char* handle64, unsigned long long offset, void** ptr) {
    if (handle64 == nullptr || ptr == nullptr) return ADDER_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    void* base = nullptr;
    if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        (void)cudaGetLastError();
        return ADDER_ERR_CUDA;
    }
    *ptr = static_cast<char*>(base) + offset;
    return ADDER_OK;
}

int adder_b200_ipc_close(void* ptr, unsigned long long offset) {
    if (ptr == nullptr) return ADDER_ERR_NULL_POINTER;
    if (cudaIpcCloseMemHandle(static_cast<char*>(ptr) - offset) != cudaSuccess) {
        (void)cudaGetLastError();
        return ADDER_ERR_CUDA;
    }
    return ADDER_OK;
}

int adder_b200_peer_comm_create(void** comm, int world, int first_rank, int ranks_here, float* const* data,
                                void* const* areas, long long n, int chunks, int max_polls) {
    if (comm == nullptr || data == nullptr || areas == nullptr) return ADDER_ERR_NULL_POINTER;
    if (world < 1 || world > PEER_MAX_WORLD || ranks_here < 1 || first_rank < 0 || first_rank + ranks_here > world ||
        n <= 0 || n % 4 != 0 || max_polls < 1)
        return ADDER_ERR_BAD_SHAPE;
    const long long n4 = n / 4;
    if (chunks <= 0) {
        // enough CTAs to have ~16 KB in flight each, never more than one per SM: all CTAs of a call are resident
        // together, so a CTA never waits for a chunk whose pusher has no SM to run on
        long long want = (n4 * 16 + 16383) / 16384;
        const int cap = sm_count() / ranks_here;
        chunks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    }
    if (chunks > PEER_MAX_CHUNKS || (long long)chunks * ranks_here > sm_count()) return ADDER_ERR_UNSUPPORTED;
    for (int p = 0; p < world; ++p)
        if (areas[p] == nullptr || (reinterpret_cast<uintptr_t>(areas[p]) & 15) != 0) return ADDER_ERR_ALIGNMENT;
    std::vector<PeerArgs> host(ranks_here);
    PeerComm* pc = new PeerComm();
    pc->ranks_here = ranks_here;
    pc->chunks = chunks;
    if (cudaGetDevice(&pc->device) != cudaSuccess || cudaMalloc(&pc->d_args, sizeof(PeerArgs) * ranks_here) != cudaSuccess ||
        cudaMalloc(&pc->d_state, sizeof(unsigned) * 4 * ranks_here) != cudaSuccess ||
        cudaMemset(pc->d_state, 0, sizeof(unsigned) * 4 * ranks_here) != cudaSuccess) {
        (void)cudaGetLastError();
        if (pc->d_args) cudaFree(pc->d_args);
        if (pc->d_state) cudaFree(pc->d_state);
        delete pc;
        return ADDER_ERR_CUDA;
    }
    for (int r = 0; r < ranks_here; ++r) {
        PeerArgs& a = host[r];
        if (data[r] == nullptr || (reinterpret_cast<uintptr_t>(data[r]) & 15) != 0) {
            cudaFree(pc->d_args); cudaFree(pc->d_state); delete pc;
            return data[r] == nullptr ? ADDER_ERR_NULL_POINTER : ADDER_ERR_ALIGNMENT;
        }
        a.data = data[r];
        for (int p = 0; p < PEER_MAX_WORLD; ++p) a.area[p] = p < world ? static_cast<float*>(areas[p]) : nullptr;
        a.state = pc->d_state + 4 * r;
        a.n4 = n4;
        a.slot4 = n4;
        a.flags_off4 = 2LL * world * n4;
        a.rank = first_rank + r;
        a.world = world;
        a.chunks = chunks;
        a.max_polls = max_polls;
        a.scale = 1.0f / (float)world;
    }
    if (cudaMemcpy(pc->d_args, host.data(), sizeof(PeerArgs) * ranks_here, cudaMemcpyHostToDevice) != cudaSuccess) {
        (void)cudaGetLastError();
        cudaFree(pc->d_args); cudaFree(pc->d_state); delete pc;
        return ADDER_ERR_CUDA;
    }
    *comm = pc;
    return ADDER_OK;
}

int adder_b200_peer_allreduce(void* comm, void* stream) {
    if (comm == nullptr) return ADDER_ERR_NULL_POINTER;
    PeerComm* pc = static_cast<PeerComm*>(comm);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid(pc->chunks, pc->ranks_here);
    if (pc->ranks_here > 1) {
        const PeerArgs* arg = pc->d_args;
        void* params[] = {&arg};
        if (cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(peer_allreduce_kernel), grid, dim3(PEER_THREADS), params,
                                        0, s) != cudaSuccess) {
            (void)cudaGetLastError();
            return ADDER_ERR_CUDA;
        }
        return launched();
    }
    peer_allreduce_kernel<<<grid, PEER_THREADS, 0, s>>>(pc->d_args);
    return launched();
}

int adder_b200_peer_comm_status(void* comm, int* status, unsigned* epoch, int reset) {
    if (comm == nullptr || status == nullptr) return ADDER_ERR_NULL_POINTER;
    PeerComm* pc = static_cast<PeerComm*>(comm);
    std::vector<unsigned> st(4 * pc->ranks_here);
    if (cudaMemcpy(st.data(), pc->d_state, st.size() * sizeof(unsigned), cudaMemcpyDeviceToHost) != cudaSuccess) {
        (void)cudaGetLastError();
        return ADDER_ERR_CUDA;
    }
    *status = 0;
    for (int r = 0; r < pc->ranks_here; ++r)
        if (st[4 * r + 2] != 0) *status = (int)st[4 * r + 2];
    if (epoch != nullptr) *epoch = st[0];
    if (reset && *status != 0)
        for (int r = 0; r < pc->ranks_here; ++r)
            if (cudaMemset(pc->d_state + 4 * r + 2, 0, sizeof(unsigned)) != cudaSuccess) return ADDER_ERR_CUDA;
    return ADDER_OK;
}

int adder_b200_peer_comm_destroy(void* comm) {
    if (comm == nullptr) return ADDER_ERR_NULL_POINTER;
    PeerComm* pc = static_cast<PeerComm*>(comm);
    cudaFree(pc->d_args);
    cudaFree(pc->d_state);
    delete pc;
    return ADDER_OK;
}

}  // extern "C"
