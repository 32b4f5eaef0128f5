// Grouped GEMM for expert FFNs on sm_100a: tcgen05.mma with TMEM accumulators, TMA-fed operand
// tiles, mbarrier pipelines, warp-specialised persistent CTAs.
//
//   out[m, :] = epilogue( A[m, :] @ W[e(m)]^T )     for every 128-row block m of the expert-major
//                                                   activation matrix; e(m) from expert_offsets.
//
// The reference library has no GEMM at all (its kernels only move data); this kernel is what lets
// dispatch feed the expert up-projection and the down-projection feed combine on the same GPU.
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 =
// epilogue (each reads its own quarter of the 128 TMEM lanes).  Tile = 128 x 256 x 64 (bf16, fp32
// accumulate), 4 shared-memory stages of 48 KB, two 256-column accumulators in TMEM so the epilogue
// of tile i overlaps the mainloop of tile i+1.
//
// Epilogues:
//   kPlain   : out[128 x 256] = bf16(acc)
//   kSwiGLU  : the B tile holds 128 gate rows and the 128 matching up rows of the fused [2I, H]
//              weight; out[128 x 128] = bf16(silu(gate) * up)
//   kScatter : (fused down-projection + combine) acc * gate weight of the slot -> bf16 -> stored
//              straight into the source rank's return partition over NVLink (peer pointer).
// Optional tile gating (fused dispatch + up-projection): the producer waits until the row block's
// ready counter reaches its expected value before loading A.
//
// All waits are bounded; on expiry the CTA records a code in `status`, stops issuing work, still
// joins the final barrier and frees its TMEM.
#include "grouped_gemm_sm100.hpp"

#include <cuda_bf16.h>

#include "tc_prim.cuh"

namespace nep {
namespace gemm {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kABytes = BM * BK * 2;  // 16 KB
constexpr int kBBytes = BN * BK * 2;  // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kMaxExperts = 1024;
// kScatter stages its 128 x 256 bf16 output tile in shared memory (one 512-byte row per thread,
// padded to 528 bytes against bank conflicts) and sends each row with one bulk store.
constexpr int kOutRowBytes = BN * 2;
constexpr int kOutPitch = kOutRowBytes + 16;
constexpr int kOutStageBytes = 4 * 32 * kOutPitch;

// 2-D tiled TMA load into this CTA's shared memory (unicast).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
constexpr uint32_t kInstrDesc = instr_desc_bf16(BM, BN);

constexpr int kMaxStages = 4;
struct SharedStorage {
    uint64_t full[kMaxStages], empty[kMaxStages], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort;
    int offsets[kMaxExperts + 1];
};

__device__ __forceinline__ int find_expert(const int* offsets, int experts, int row) {
    int lo = 0, hi = experts;  // offsets[lo] <= row < offsets[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (offsets[mid] <= row) lo = mid; else hi = mid;
    }
    return lo;
}

template <int kMode, int kStages>
__global__ void __launch_bounds__(kThreads, 1) grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                   const __grid_constant__ CUtensorMap map_b, const Args args) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* tiles = smem;  // kStages x (A 16 KB | B 32 KB), 1024-byte aligned
    SharedStorage& sh = *reinterpret_cast<SharedStorage*>(smem + kStages * kStageBytes);
    uint8_t* out_stage = smem + kStages * kStageBytes + ((sizeof(SharedStorage) + 127) / 128) * 128;  // kScatter only
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint64_t limit_ns = args.timeout_ns;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sh.full[s], 1);
            mbar_init(&sh.empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sh.tmem_full[a], 1);
            mbar_init(&sh.tmem_empty[a], 4);  // one arrival per epilogue warp
        }
        sh.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (int i = threadIdx.x; i <= args.num_experts; i += kThreads) {
        const int64_t off = args.expert_offsets[i];
        sh.offsets[i] = int(off);
        // one expert per 128-row block: offsets must be multiples of 128, start at 0 and end at the row count
        if ((off & 127) != 0 || (i == 0 && off != 0) || (i == args.num_experts && off != int64_t(args.m_blocks) * BM)) {
            sh.abort = 1;
            if (atomicCAS(args.status, 0u, uint32_t(kGemmBadOffsets)) == 0u) args.status[1] = uint32_t(i);
        }
    }
    if (warp == 1) tmem_alloc(&sh.tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh.tmem_base;

    const int m_blocks = args.m_blocks, n_tiles = args.n_tiles, k_blocks = args.k_blocks;
    const int total_tiles = m_blocks * n_tiles;
    volatile int* abort_flag = &sh.abort;

    auto fail = [&](uint32_t code) {
        *abort_flag = 1;
        if (atomicCAS(args.status, 0u, code) == 0u) args.status[1] = blockIdx.x;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                const int mb = tile / n_tiles, nt = tile % n_tiles;
                const int row0 = mb * BM;
                const int expert = find_expert(sh.offsets, args.num_experts, row0);
                if (args.tile_ready != nullptr) {
                    // Rows of this block are written by the dispatch pull of the same GPU; wait for all of them.
                    const int want = args.tile_expected[mb];
                    const uint64_t start = timer_ns();
                    while (ld_acquire_gpu(args.tile_ready + mb) < want) {
                        __nanosleep(64);
                        if (timer_ns() - start > limit_ns) {
                            fail(kGemmTileTimeout);
                            break;
                        }
                    }
                    if (*abort_flag) break;
                    asm volatile("fence.proxy.async;" ::: "memory");
                }
                const int b_row0 = expert * args.b_rows_per_expert + (kMode == kSwiGLU ? nt * (BN / 2) : nt * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&sh.empty[stage], phase ^ 1u, limit_ns)) {
                        fail(kGemmPipeTimeout);
                        break;
                    }
                    uint8_t* a_dst = tiles + stage * kStageBytes;
                    uint8_t* b_dst = a_dst + kABytes;
                    mbar_expect_tx(&sh.full[stage], kStageBytes);
                    tma_load_2d(a_dst, &map_a, kb * BK, row0, &sh.full[stage]);
                    if (kMode == kSwiGLU) {
                        tma_load_2d(b_dst, &map_b, kb * BK, b_row0, &sh.full[stage]);
                        tma_load_2d(b_dst + kBBytes / 2, &map_b, kb * BK, b_row0 + args.swiglu_up_row_offset, &sh.full[stage]);
                    } else {
                        tma_load_2d(b_dst, &map_b, kb * BK, b_row0, &sh.full[stage]);
                        tma_load_2d(b_dst + kBBytes / 2, &map_b, kb * BK, b_row0 + BN / 2, &sh.full[stage]);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++local) {
                const int acc = local & 1;
                const uint32_t acc_phase = uint32_t(local >> 1) & 1u;
                if (!mbar_wait(&sh.tmem_empty[acc], acc_phase ^ 1u, limit_ns)) {
                    fail(kGemmPipeTimeout);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&sh.full[stage], phase, limit_ns)) {
                        fail(kGemmPipeTimeout);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint8_t* a_tile = tiles + stage * kStageBytes;
                    const uint64_t a_desc = smem_desc_sw128(a_tile);
                    const uint64_t b_desc = smem_desc_sw128(a_tile + kABytes);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // 16 bf16 = 32 bytes along K inside the 128-byte swizzle row: +2 in 16-byte units
                        tc_mma(d_tmem, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), kInstrDesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(&sh.empty[stage]);  // frees the stage once these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit(&sh.tmem_full[acc]);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++local) {
            const int acc = local & 1;
            const uint32_t acc_phase = uint32_t(local >> 1) & 1u;
            const int mb = tile / n_tiles, nt = tile % n_tiles;
            const int row = mb * BM + quarter * 32 + lane;
            bool ok = mbar_wait(&sh.tmem_full[acc], acc_phase, limit_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) fail(kGemmPipeTimeout);
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(acc * BN);
            if (kMode == kSwiGLU) {
                __nv_bfloat16* out_row = args.out + int64_t(row) * args.ldo + nt * (BN / 2);
                // 32 gate + 32 up columns per step, the next step's TMEM loads in flight while this one is
                // converted and stored
                uint32_t g[2][32], u[2][32];
                tmem_ld32(taddr, g[0]);
                tmem_ld32(taddr + BN / 2, u[0]);
#pragma unroll
                for (int step = 0; step < BN / 2 / 32; ++step) {
                    const int cur = step & 1, c = step * 32;
                    tmem_ld_wait();
                    if (step + 1 < BN / 2 / 32) {
                        tmem_ld32(taddr + c + 32, g[cur ^ 1]);
                        tmem_ld32(taddr + BN / 2 + c + 32, u[cur ^ 1]);
                    }
                    uint32_t o[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float a = silu(__uint_as_float(g[cur][2 * j])) * __uint_as_float(u[cur][2 * j]);
                        const float b = silu(__uint_as_float(g[cur][2 * j + 1])) * __uint_as_float(u[cur][2 * j + 1]);
                        o[j] = pack_bf16(a, b);
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) st_v4(out_row + c + q * 8, o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                }
            } else if (kMode == kPlain) {
                __nv_bfloat16* out_row = args.out + int64_t(row) * args.ldo + nt * BN;
                const float scale = args.row_scale != nullptr ? args.row_scale[row] : 1.f;
                uint32_t v[2][32];
                tmem_ld32(taddr, v[0]);
#pragma unroll
                for (int step = 0; step < BN / 32; ++step) {
                    const int cur = step & 1, c = step * 32;
                    tmem_ld_wait();
                    if (step + 1 < BN / 32) tmem_ld32(taddr + c + 32, v[cur ^ 1]);
                    uint32_t o[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) o[j] = pack_bf16(__uint_as_float(v[cur][2 * j]) * scale, __uint_as_float(v[cur][2 * j + 1]) * scale);
#pragma unroll
                    for (int q = 0; q < 4; ++q) st_v4(out_row + c + q * 8, o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                }
            } else {
                // kScatter: acc * gate weight -> bf16 row in shared memory -> one 512-byte bulk store into
                // the source rank's return partition (peer memory over NVLink, or local).  Padding rows
                // are skipped.
                __nv_bfloat16* out_row = nullptr;
                float scale = 1.f;
                const int a = args.slot_map[row];
                if (a >= 0) {
                    const int recv_row = a / args.topk, k = a % args.topk;
                    const int* meta = args.recv_metadata + int64_t(recv_row) * (args.topk + 2);
                    const int src = meta[0], tok = meta[1];
                    scale = args.slot_weights != nullptr ? args.slot_weights[row] : 1.f;
                    if (recv_row >= args.recv_rows || src < 0 || src >= args.ranks || tok < 0 || tok >= args.max_tokens) {
                        // impossible provenance: skip the row and report it, as the push kernel does
                        if (atomicCAS(args.status, 0u, uint32_t(kGemmBadMetadata)) == 0u) args.status[1] = uint32_t(row);
                    } else
                    out_row = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(args.peers[src]) + args.ret_offset +
                                                               (int64_t(k) * args.max_tokens + tok) * int64_t(args.ldo) * 2) +
                              nt * BN;
                }
                uint8_t* my_row = out_stage + (quarter * 32 + lane) * kOutPitch;
                // the previous tile's bulk store must have finished reading this row buffer
                // The row is sent as two 256-byte halves, each its own bulk group: before a half of the
                // staging row is overwritten only the store that last read THAT half has to be done
                // (wait_group.read 1 = everything but the newest group), so a store is always in flight.
                uint32_t v[2][32];
                tmem_ld32(taddr, v[0]);
#pragma unroll
                for (int step = 0; step < BN / 32; ++step) {
                    const int cur = step & 1, c = step * 32;
                    if (step == 0 || step == BN / 64) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    tmem_ld_wait();
                    if (step + 1 < BN / 32) tmem_ld32(taddr + c + 32, v[cur ^ 1]);
                    uint32_t o[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        o[j] = pack_bf16(__uint_as_float(v[cur][2 * j]) * scale, __uint_as_float(v[cur][2 * j + 1]) * scale);
#pragma unroll
                    for (int q = 0; q < 4; ++q) st_shared_v4(my_row + c * 2 + q * 16, o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                    if (step == BN / 64 - 1 || step == BN / 32 - 1) {
                        const int half = step == BN / 64 - 1 ? 0 : 1;
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        if (out_row != nullptr) bulk_store_row(out_row + half * (BN / 2), my_row + half * (kOutRowBytes / 2), kOutRowBytes / 2);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.tmem_empty[acc]);
        }
        if (kMode == kScatter) {
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            __threadfence_system();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

size_t shared_bytes(int mode, int stages) {
    return size_t(stages) * kStageBytes + ((sizeof(SharedStorage) + 127) / 128) * 128 + (mode == kScatter ? kOutStageBytes : 0) + 128;
}

template <int kMode, int kStages>
cudaError_t launch_mode(const CUtensorMap& a, const CUtensorMap& b, const Args& args, int grid, cudaStream_t stream) {
    auto* fn = grouped_gemm_kernel<kMode, kStages>;
    const size_t smem = shared_bytes(kMode, kStages);
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    fn<<<grid, kThreads, smem, stream>>>(a, b, args);
    return cudaGetLastError();
}

// `stages` = 4 by default; 3 leaves ~75 KB of shared memory per SM for a co-resident transfer kernel.
cudaError_t launch(const CUtensorMap& a, const CUtensorMap& b, const Args& args, int mode, int stages, int grid, cudaStream_t stream) {
    if (args.num_experts > kMaxExperts) return cudaErrorInvalidValue;
    if (mode == kPlain && stages == 4) return launch_mode<kPlain, 4>(a, b, args, grid, stream);
    if (mode == kPlain && stages == 3) return launch_mode<kPlain, 3>(a, b, args, grid, stream);
    if (mode == kSwiGLU && stages == 4) return launch_mode<kSwiGLU, 4>(a, b, args, grid, stream);
    if (mode == kSwiGLU && stages == 3) return launch_mode<kSwiGLU, 3>(a, b, args, grid, stream);
    if (mode == kScatter) return launch_mode<kScatter, 3>(a, b, args, grid, stream);
    return cudaErrorInvalidValue;
}

int kernel_registers(int mode) {
    cudaFuncAttributes attr{};
    const void* fn = mode == kPlain ? (const void*)grouped_gemm_kernel<kPlain, 4>
                   : mode == kSwiGLU ? (const void*)grouped_gemm_kernel<kSwiGLU, 4>
                                     : (const void*)grouped_gemm_kernel<kScatter, 3>;
    if (cudaFuncGetAttributes(&attr, fn) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return attr.numRegs;
}

}  // namespace gemm
}  // namespace nep
