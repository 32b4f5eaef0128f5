// Shared declarations of the reference-kernel stand-in (see jit_standin.cu).
#pragma once
#include <cstdint>
#include <tuple>

namespace nano_ep {

enum class StandinKind : int { DispatchMain, DispatchEpilogue, CombineMain, CombineEpilogue };

struct JitKernel {
    const void* function;
    StandinKind kind;
    int threads, smem_bytes;
    bool cooperative;
    int parameters;
};

// kind, hidden, topk, ranks, experts per rank, max tokens, alignment, then five mode bits
using StandinKey = std::tuple<int, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, bool, bool, bool, bool, bool>;
void standin_put(const StandinKey& key, const JitKernel& kernel);

// Each of the reference's kernel headers is its own translation unit (as under its JIT): they cannot share one.
void standin_add_dispatch_main();
void standin_add_dispatch_epilogue(int shared_memory_optin);
void standin_add_combine_main();
void standin_add_combine_epilogue();

// The benchmark geometries: (hidden, topk, experts, ranks, max tokens, alignment)
#define NANO_EP_STANDIN_GEOMETRIES(X) \
    X(7168, 8, 256, 1, 4096, 128)     \
    X(7168, 8, 256, 2, 4096, 128)     \
    X(7168, 8, 256, 4, 4096, 128)     \
    X(7168, 8, 256, 8, 4096, 128)     \
    X(4096, 8, 256, 2, 256, 128)      \
    X(4096, 8, 256, 4, 256, 128)      \
    X(4096, 8, 256, 8, 256, 128)

}  // namespace nano_ep
