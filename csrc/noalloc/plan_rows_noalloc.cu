// Allocation-free variant of the dispatch plan kernel; see plan_rows_noalloc.h for the contract.
#include "plan_rows_noalloc.h"

#include <cuda_runtime.h>

#include <climits>
#include <mutex>

namespace {

// Cursor storage shared by every call on a device: [0] row cursor, [1] count of slots that fell outside
// their expert's range, [64 + l] slot cursor of local expert l.  File-scope device memory: part of the library image, never allocated at run time.
static __device__ __align__(256) int g_plan_scratch[NEP_NOALLOC_MAX_LOCAL_EXPERTS + 64];

constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;
constexpr unsigned kFull = 0xffffffffu;

thread_local const char* t_last_error = "";

// The symbol's name is a host-side stand-in; kernels need the address the device uses, looked up
// once per device with that device current.
void* g_scratch_address[kMaxDevices] = {};
std::mutex g_setup_mutex;

int scratch_for_current_device(int** out) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
        t_last_error = e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range";
        return NEP_NOALLOC_CUDA_ERROR;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* address = nullptr;
        e = cudaGetSymbolAddress(&address, g_plan_scratch);
        if (e != cudaSuccess || address == nullptr) {
            t_last_error = e != cudaSuccess ? cudaGetErrorString(e) : "null symbol address";
            return NEP_NOALLOC_CUDA_ERROR;
        }
        g_scratch_address[device] = address;
    }
    *out = static_cast<int*>(g_scratch_address[device]);
    return NEP_NOALLOC_OK;
}

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// One warp per chunk of 32 tokens: find the tokens with a local choice, reserve their rows with one
// atomic per chunk, reserve expert-major slots with one atomic per local choice.
__global__ void __launch_bounds__(kThreads) plan_rows_kernel(const int* __restrict__ topk, int tokens, int K, int source_rank, int lo,
                                                             int Le, const int* __restrict__ eoff, int expand, int* __restrict__ meta,
                                                             int* scratch) {
    const int lane = threadIdx.x & 31;
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int GW = (gridDim.x * blockDim.x) >> 5;
    int* row_cursor = scratch;
    int* expert_cursor = scratch + 64;
    const int chunks = (tokens + 31) / 32;
    for (int c = gw; c < chunks; c += GW) {
        const int tok = c * 32 + lane;
        const int* mine = topk + (long long)tok * K;
        bool has = false;
        if (tok < tokens)
            for (int k = 0; k < K; ++k) {
                const int e = mine[k];
                has |= (e >= lo && e < lo + Le);
            }
        const unsigned hm = __ballot_sync(kFull, has);
        if (hm == 0) continue;
        int base = 0;
        if (lane == 0) base = atomicAdd(row_cursor, __popc(hm));
        base = __shfl_sync(kFull, base, 0);
        if (!has) continue;
        const int row = base + __popc(hm & lanemask_lt());
        int* m = meta + (long long)row * (K + 2);
        m[0] = source_rank;
        m[1] = tok;
        for (int k = 0; k < K; ++k) {
            const int e = mine[k];
            int v = -1;
            if (e >= lo && e < lo + Le) {
                const int le = e - lo;
                v = le;
                if (expand) {
                    v = eoff[le] + atomicAdd(&expert_cursor[le], 1);
                    if (v < 0 || v >= eoff[le + 1]) {  // offsets that do not fit the routing: never hand out a foreign slot
                        atomicAdd(scratch + 1, 1);
                        v = -1;
                    }
                }
            }
            m[2 + k] = v;
        }
    }
}

// Row count of the call, or -1 when a slot fell outside its expert's range.
__global__ void publish_count_kernel(const int* scratch, int* row_count_out) { *row_count_out = scratch[1] != 0 ? -1 : scratch[0]; }

}  // namespace

extern "C" const char* nep_noalloc_last_error(void) { return t_last_error; }

extern "C" int nep_plan_rows_noalloc(const int* topk_i32, int tokens, int topk, int source_rank, int expert_lo, int local_experts,
                                     const int* expert_offsets, int expand, int* meta_out, int* row_count_out, void* stream) {
    t_last_error = "";
    if ((topk_i32 == nullptr && tokens > 0) || (meta_out == nullptr && tokens > 0) || row_count_out == nullptr || tokens < 0 || topk <= 0 || local_experts <= 0 ||
        expert_lo < 0 || source_rank < 0 || (expand && expert_offsets == nullptr))
        return NEP_NOALLOC_BAD_ARGUMENT;
    if (local_experts > NEP_NOALLOC_MAX_LOCAL_EXPERTS || topk > 32 || tokens > (1 << 24)) return NEP_NOALLOC_TOO_LARGE;
    if (expert_lo > INT_MAX - local_experts) return NEP_NOALLOC_BAD_ARGUMENT;  // expert_lo + local_experts must fit an int
    int* scratch = nullptr;
    const int setup = scratch_for_current_device(&scratch);
    if (setup != NEP_NOALLOC_OK) return setup;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps the previous call's cursors: clear the part this call uses.
    cudaError_t e = cudaMemsetAsync(scratch, 0, size_t(64 + local_experts) * sizeof(int), s);
    if (e == cudaSuccess && tokens > 0) {
        const int chunks = (tokens + 31) / 32;
        int blocks = (chunks + (kThreads / 32) - 1) / (kThreads / 32);
        if (blocks > 1184) blocks = 1184;  // 148 SMs x 8 resident blocks
        // cudaLaunchKernel returns this launch's own error; an older sticky error is not picked up and blamed on it
        void* args[] = {(void*)&topk_i32, (void*)&tokens, (void*)&topk, (void*)&source_rank, (void*)&expert_lo, (void*)&local_experts,
                        (void*)&expert_offsets, (void*)&expand, (void*)&meta_out, (void*)&scratch};
        e = cudaLaunchKernel((const void*)plan_rows_kernel, dim3(blocks), dim3(kThreads), args, 0, s);
    }
    if (e == cudaSuccess) {
        const int* scratch_in = scratch;
        void* args[] = {(void*)&scratch_in, (void*)&row_count_out};
        e = cudaLaunchKernel((const void*)publish_count_kernel, dim3(1), dim3(1), args, 0, s);
    }
    if (e != cudaSuccess) {
        t_last_error = cudaGetErrorString(e);
        return NEP_NOALLOC_CUDA_ERROR;
    }
    return NEP_NOALLOC_OK;
}
