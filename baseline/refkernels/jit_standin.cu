// Ahead-of-time stand-in for the reference's kernel JIT.
//
// The reference compiles its four kernels at run time through a third-party JIT (csrc/jit.cpp) whose headers
// are not part of the mounted checkout, so its stock build cannot be produced offline.  This file implements
// the same interface (csrc/include/nano_ep/jit.hpp:13-63) without a JIT: the reference's own kernel templates
// (dispatch_main.cuh, dispatch_epilogue.cuh, combine_main.cuh, combine_epilogue.cuh, included unmodified, one
// translation unit each: standin_*.cu) are instantiated for the benchmark geometries, block shapes and shared-memory sizes come from the reference's
// own plan functions in layout.hpp, and launches go through cudaLaunchKernelExC with the cooperative and
// programmatic-stream-serialization attributes the reference asks for.  Everything else of the comparison build
// (peer.cu, pipeline.cu, the epilogue wrappers, bindings.cpp and the Python package) is the reference's code as is.
//
// It is a measuring aid, not part of the product: numbers obtained with it are labelled "reference kernels, AOT
// stand-in, not the stock build".
#include <ATen/cuda/CUDAContextLight.h>
#include <c10/cuda/CUDAException.h>
#include <c10/util/Exception.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <nano_ep/jit.hpp>
#include <string_view>
#include <tuple>

#include "standin_table.hpp"

namespace nano_ep {

namespace {

using Key = StandinKey;

std::mutex table_mutex;
std::map<Key, JitKernel>& table() {
    static std::map<Key, JitKernel> entries;
    return entries;
}
std::map<std::pair<const void*, int>, bool>& prepared() {
    static std::map<std::pair<const void*, int>, bool> done;
    return done;
}

void fill_table() {
    standin_add_dispatch_main();
    standin_add_dispatch_epilogue(int(at::cuda::getCurrentDeviceProperties()->sharedMemPerBlockOptin));
    standin_add_combine_main();
    standin_add_combine_epilogue();
}

const JitKernel& lookup(const Key& key, const char* what) {
    std::lock_guard<std::mutex> lock(table_mutex);
    if (table().empty()) fill_table();
    const auto entry = table().find(key);
    TORCH_CHECK(entry != table().end(), "reference-kernel stand-in: ", what,
                " was not instantiated for this geometry (hidden ", std::get<1>(key), ", topk ", std::get<2>(key), ", ranks ",
                std::get<3>(key), ", experts per rank ", std::get<4>(key), ", max tokens ", std::get<5>(key), ", alignment ",
                std::get<6>(key), ")");
    const JitKernel& kernel = entry->second;
    const int device = c10::cuda::current_device();
    bool& ready = prepared()[{kernel.function, device}];
    if (!ready) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(kernel.function, cudaFuncAttributeMaxDynamicSharedMemorySize, kernel.smem_bytes));
        if (kernel.cooperative) {
            int blocks = 0;
            C10_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel.function, kernel.threads, kernel.smem_bytes));
            TORCH_CHECK(blocks > 0, what, " cannot fit one staged block per SM");
        }
        ready = true;
    }
    return kernel;
}

}  // namespace

void standin_put(const StandinKey& key, const JitKernel& kernel) { table()[key] = kernel; }

void init_jit(const std::string&) {}

bool use_pdl() {
    const auto* disable_pdl = std::getenv("NANO_EP_DISABLE_PDL");
    return at::cuda::getCurrentDeviceProperties()->major >= 9 && !(disable_pdl && std::string_view(disable_pdl) == "1");
}

void launch_kernel(const JitKernel& kernel, cudaStream_t stream, int sms, bool pdl, std::span<void*> args) {
    TORCH_INTERNAL_ASSERT(int(args.size()) == kernel.parameters);
    cudaLaunchAttribute attributes[2];
    unsigned count = 0;
    if (kernel.cooperative) {
        attributes[count].id = cudaLaunchAttributeCooperative;
        attributes[count].val.cooperative = 1;
        ++count;
    }
    if (pdl) {
        attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(sms);
    config.blockDim = dim3(kernel.threads);
    config.dynamicSmemBytes = size_t(kernel.smem_bytes);
    config.stream = stream;
    config.attrs = attributes;
    config.numAttrs = count;
    C10_CUDA_CHECK(cudaLaunchKernelExC(&config, kernel.function, args.data()));
}

const JitKernel& dispatch_main_kernel(
    int64_t hidden, int64_t topk, int64_t ranks, int64_t experts, int64_t tokens, int64_t alignment, bool cached) {
    return lookup(Key{int(StandinKind::DispatchMain), hidden, topk, ranks, experts, tokens, cached ? 1 : alignment, cached, false, false,
                      false, false},
                  "dispatch_main");
}

const JitKernel& dispatch_epilogue_kernel(
    int64_t hidden, int64_t topk, int64_t experts, bool cached, bool expand, bool weights, bool zero_padding) {
    return lookup(Key{int(StandinKind::DispatchEpilogue), hidden, topk, 0, experts, 0, 1, cached, expand, false, weights,
                      expand && zero_padding},
                  "dispatch_epilogue");
}

const JitKernel& combine_main_kernel(
    int64_t hidden, int64_t topk, int64_t ranks, int64_t, int64_t tokens, bool expand, bool multiple, bool weights) {
    return lookup(Key{int(StandinKind::CombineMain), hidden, topk, ranks, 0, tokens, 1, false, expand, multiple, weights, false},
                  "combine_main");
}

const JitKernel& combine_epilogue_kernel(
    int64_t hidden, int64_t topk, int64_t ranks, int64_t experts, int64_t tokens, bool expand, bool multiple, bool weights) {
    return lookup(Key{int(StandinKind::CombineEpilogue), hidden, topk, ranks, experts, tokens, 1, false, expand, multiple, weights, false},
                  "combine_epilogue");
}

void prepare_dispatch(int64_t hidden, int64_t topk, int64_t ranks, int64_t experts, int64_t tokens, int64_t alignment, bool cached,
                      bool expand, bool weights, bool zero_padding) {
    dispatch_main_kernel(hidden, topk, ranks, experts, tokens, alignment, cached);
    dispatch_epilogue_kernel(hidden, topk, experts, cached, expand, weights, zero_padding);
}

void prepare_combine(int64_t hidden, int64_t topk, int64_t ranks, int64_t experts, int64_t tokens, bool expand, bool multiple,
                     bool weights) {
    combine_main_kernel(hidden, topk, ranks, experts, tokens, expand, multiple, weights);
    combine_epilogue_kernel(hidden, topk, ranks, experts, tokens, expand, multiple, weights);
}

}  // namespace nano_ep
