// Instantiations of the reference's combine main kernel (csrc/combine_main.cuh, included unmodified):
// expert-major layout, one row per assignment, no gate weights.
#include "combine_main.cuh"
#include "layout.hpp"
#include "standin_table.hpp"

namespace nano_ep {
namespace {
template <int H, int K, int R, int64_t T>
void add() {
    const auto plan = HiddenRowPlan::make(H, true);
    const int warps = plan.max_warps();
    standin_put(StandinKey{int(StandinKind::CombineMain), H, K, R, 0, T, 1, false, true, false, false, false},
                JitKernel{reinterpret_cast<const void*>(&combine_main_kernel<H, K, R, T, nv_bfloat16, true, false, false>),
                          StandinKind::CombineMain, warps * 32, int(warps * plan.stage_bytes), true, 9});
}
}  // namespace

void standin_add_combine_main() {
#define X(H, K, E, R, T, A) add<H, K, R, T>();
    NANO_EP_STANDIN_GEOMETRIES(X)
#undef X
}
}  // namespace nano_ep
