// Instantiations of the reference's dispatch epilogue kernel (csrc/dispatch_epilogue.cuh, included unmodified):
// expert-major layout with gate weights and zero padding, fresh and cached.
#include <algorithm>

#include "dispatch_epilogue.cuh"
#include "layout.hpp"
#include "standin_table.hpp"

namespace nano_ep {
namespace {
template <int H, int K, int L, bool kCached>
void add(int optin) {
    const auto plan = PayloadRowPlan::make(H, K);
    const int warps = int(std::min<int64_t>(plan.total_warps, optin / plan.stage_bytes));
    standin_put(StandinKey{int(StandinKind::DispatchEpilogue), H, K, 0, L, 0, 1, kCached, true, false, true, true},
                JitKernel{reinterpret_cast<const void*>(&dispatch_epilogue_kernel<H, K, L, kCached, true, true, true>),
                          StandinKind::DispatchEpilogue, warps * 32, int(warps * plan.stage_bytes), false, 14});
}
}  // namespace

void standin_add_dispatch_epilogue(int optin) {
#define X(H, K, E, R, T, A)              \
    add<H, K, (E) / (R), false>(optin);   \
    add<H, K, (E) / (R), true>(optin);
    NANO_EP_STANDIN_GEOMETRIES(X)
#undef X
}
}  // namespace nano_ep
