// Instantiations of the reference's combine epilogue kernel (csrc/combine_epilogue.cuh, included unmodified).
#include "combine_epilogue.cuh"
#include "layout.hpp"
#include "standin_table.hpp"

namespace nano_ep {
namespace {
template <int H, int K, int R, int64_t L, int64_t T>
void add() {
    const auto plan = HiddenRowPlan::make(H);
    const int warps = plan.max_warps();
    standin_put(StandinKey{int(StandinKind::CombineEpilogue), H, K, R, L, T, 1, false, true, false, false, false},
                JitKernel{reinterpret_cast<const void*>(&combine_epilogue_kernel<H, K, R, L, T, true, false, false>),
                          StandinKind::CombineEpilogue, warps * 32, int(warps * plan.stage_bytes), false, 7});
}
}  // namespace

void standin_add_combine_epilogue() {
#define X(H, K, E, R, T, A) add<H, K, R, (E) / (R), T>();
    NANO_EP_STANDIN_GEOMETRIES(X)
#undef X
}
}  // namespace nano_ep
