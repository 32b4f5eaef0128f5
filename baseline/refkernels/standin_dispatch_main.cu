// Instantiations of the reference's dispatch main kernel (csrc/dispatch_main.cuh, included unmodified).
#include "dispatch_main.cuh"
#include "layout.hpp"
#include "standin_table.hpp"

namespace nano_ep {
namespace {
template <int H, int K, int R, int L, int64_t T, int64_t A, bool kCached>
void add() {
    const auto plan = make_dispatch_payload_plan(H, K, R, L, dispatch_notify_warps(kCached));
    standin_put(StandinKey{int(StandinKind::DispatchMain), H, K, R, L, T, kCached ? 1 : A, kCached, false, false, false, false},
                JitKernel{reinterpret_cast<const void*>(&dispatch_main_kernel<H, K, R, L, T, (kCached ? int64_t(1) : A), kCached>),
                          StandinKind::DispatchMain, plan.total_warps * 32, int(plan.num_bytes), true, 16});
}
}  // namespace

void standin_add_dispatch_main() {
#define X(H, K, E, R, T, A)                \
    add<H, K, R, (E) / (R), T, A, false>(); \
    add<H, K, R, (E) / (R), T, A, true>();
    NANO_EP_STANDIN_GEOMETRIES(X)
#undef X
}
}  // namespace nano_ep
