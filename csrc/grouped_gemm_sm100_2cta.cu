// Grouped GEMM with CTA pairs: tcgen05.mma.cta_group::2 computes a 256 x 256 tile on two SMs.
//
// Same math and epilogues (plain with optional row scale, SwiGLU) as grouped_gemm_sm100.cu, but a
// cluster of two CTAs shares every B tile: each CTA loads its own 128 activation rows and HALF of
// the 256 weight rows, the leader CTA issues one MMA for the pair, and each CTA keeps the
// accumulator of its own 128 rows in its own TMEM.  Per CTA and k-block that is 32 KB of operand
// traffic instead of 48 KB, which is what limits the single-CTA kernel (L2 -> SM bandwidth), and it
// leaves room for six pipeline stages.
//
// Work unit = (expert, pair of consecutive 128-row blocks of that expert, output column tile).
// An expert with an odd number of row blocks leaves the second CTA of its last pair without rows:
// that CTA still feeds the pair's MMA (its loads read rows that are simply not used) and skips its
// stores.
//
// Pair protocol
//   * TMA loads of both CTAs complete on the LEADER's full barrier (the leader expects the bytes of
//     both); all bulk loads are plain unicast loads into the issuing CTA's own shared memory.
//   * The leader's MMA thread commits to the empty barrier and the accumulator-full barrier of BOTH
//     CTAs (one commit per CTA).
//   * Epilogue warps of both CTAs arrive on the leader's accumulator-empty barrier.
// All waits are bounded; a CTA that gives up records a status code, and both CTAs still meet at the
// final cluster barrier and free their TMEM.
#include "grouped_gemm_sm100.hpp"

#include <cuda_bf16.h>

#include "tc_prim.cuh"

namespace nep {
namespace gemm {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kABytes = BM * BK * 2;        // 16 KB: this CTA's activation rows
constexpr int kBHalfBytes = BN / 2 * BK * 2;  // 16 KB: this CTA's half of the weight rows
constexpr int kStageBytes = kABytes + kBHalfBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kMaxExperts = 1024;
constexpr int kMaxStages = 6;
// kScatter stages each 512-byte output row in shared memory (padded rows) before one bulk store.
constexpr int kOutRowBytes = BN * 2;
constexpr int kOutPitch = kOutRowBytes + 16;
constexpr int kOutStageBytes = 4 * 32 * kOutPitch;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on a barrier given by its shared::cluster address (own or peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled TMA load into this CTA's shared memory; completion bytes go to the barrier at
// `bar_cluster_addr`, which may live in the peer CTA of the pair (unicast data path).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// completion of all earlier MMAs of the pair -> one arrival on the barrier at `bar_cluster_addr`
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// pair tile: M = 256 (128 rows per CTA), N = 256
constexpr uint32_t kInstrDescPair = instr_desc_bf16(2 * BM, BN);

struct PairShared {
    uint64_t full[kMaxStages], empty[kMaxStages], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort;
    int offsets[kMaxExperts + 1];     // row offsets
    int pair_start[kMaxExperts + 1];  // exclusive prefix of ceil(blocks / 2)
};

struct PairTile {
    int row0;    // first row of this CTA's block
    int valid;   // this CTA's block exists
    int expert;
};

__device__ __forceinline__ PairTile locate_pair(const PairShared& sh, int experts, int pair_index, int cta) {
    int lo = 0, hi = experts;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (sh.pair_start[mid] <= pair_index) lo = mid; else hi = mid;
    }
    const int block = 2 * (pair_index - sh.pair_start[lo]) + cta;
    PairTile t;
    t.expert = lo;
    t.row0 = sh.offsets[lo] + block * BM;
    t.valid = t.row0 < sh.offsets[lo + 1];
    return t;
}

template <int kMode, int kStages>
__global__ void __launch_bounds__(kThreads, 1) grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                        const __grid_constant__ CUtensorMap map_b, const Args args) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* tiles = smem;
    PairShared& sh = *reinterpret_cast<PairShared*>(smem + kStages * kStageBytes);
    uint8_t* out_stage = smem + kStages * kStageBytes + ((sizeof(PairShared) + 127) / 128) * 128;  // kScatter only
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();
    const bool leader = cta == 0;
    const uint64_t limit_ns = args.timeout_ns;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sh.full[s], 1);   // leader: one expect_tx arrival covering both CTAs' bytes
            mbar_init(&sh.empty[s], 1);  // one commit from the leader's MMA thread
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sh.tmem_full[a], 1);
            mbar_init(&sh.tmem_empty[a], 8);  // leader: four epilogue warps of each CTA
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
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < args.num_experts; ++e) {
            sh.pair_start[e] = acc;
            const int blocks = (sh.offsets[e + 1] - sh.offsets[e]) / BM;
            acc += (blocks + 1) / 2;
        }
        sh.pair_start[args.num_experts] = acc;
    }
    if (warp == 1) tmem_alloc_pair(&sh.tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // both CTAs have initialised their barriers before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = sh.tmem_base;

    const int n_tiles = args.n_tiles, k_blocks = args.k_blocks;
    const int total_pairs = sh.pair_start[args.num_experts];
    const int total_tiles = total_pairs * n_tiles;
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    volatile int* abort_flag = &sh.abort;
    auto fail = [&](uint32_t code) {
        *abort_flag = 1;
        if (atomicCAS(args.status, 0u, code) == 0u) args.status[1] = blockIdx.x;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = cluster_id; tile < total_tiles && !*abort_flag; tile += num_clusters) {
                const int pair_index = tile / n_tiles, nt = tile % n_tiles;
                const PairTile t = locate_pair(sh, args.num_experts, pair_index, int(cta));
                // this CTA's half of the weight rows: CTA 0 -> first 128 rows of the tile (gate rows for
                // SwiGLU), CTA 1 -> second 128 rows (up rows for SwiGLU)
                int b_row;
                if (kMode == kSwiGLU)
                    b_row = t.expert * args.b_rows_per_expert + nt * (BN / 2) + (cta ? args.swiglu_up_row_offset : 0);
                else
                    b_row = t.expert * args.b_rows_per_expert + nt * BN + int(cta) * (BN / 2);
                if (args.tile_ready != nullptr && t.valid) {
                    // this CTA's rows are written by the dispatch pull of the same GPU; wait for all of them
                    const int mb = t.row0 / BM;
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
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&sh.empty[stage], phase ^ 1u, limit_ns)) {
                        fail(kGemmPipeTimeout);
                        break;
                    }
                    uint8_t* a_dst = tiles + stage * kStageBytes;
                    uint8_t* b_dst = a_dst + kABytes;
                    const uint32_t full_on_leader = map_to_cta(smem_u32(&sh.full[stage]), 0);
                    if (leader) mbar_expect_tx(&sh.full[stage], 2 * kStageBytes);
                    tma_load_2d_pair(a_dst, &map_a, kb * BK, t.row0, full_on_leader);
                    tma_load_2d_pair(b_dst, &map_b, kb * BK, b_row, full_on_leader);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader && elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            for (int tile = cluster_id; tile < total_tiles && !*abort_flag; tile += num_clusters, ++local) {
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
                    for (int k = 0; k < BK / 16; ++k)
                        tc_mma_pair(d_tmem, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), kInstrDescPair, (kb | k) != 0 ? 1u : 0u);
                    // free the stage in both CTAs once these MMAs have read it
                    tc_commit_pair(map_to_cta(smem_u32(&sh.empty[stage]), 0));
                    tc_commit_pair(map_to_cta(smem_u32(&sh.empty[stage]), 1));
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit_pair(map_to_cta(smem_u32(&sh.tmem_full[acc]), 0));
                tc_commit_pair(map_to_cta(smem_u32(&sh.tmem_full[acc]), 1));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = cluster_id; tile < total_tiles && !*abort_flag; tile += num_clusters, ++local) {
            const int acc = local & 1;
            const uint32_t acc_phase = uint32_t(local >> 1) & 1u;
            const int pair_index = tile / n_tiles, nt = tile % n_tiles;
            const PairTile t = locate_pair(sh, args.num_experts, pair_index, int(cta));
            const int row = t.row0 + quarter * 32 + lane;
            bool ok = mbar_wait(&sh.tmem_full[acc], acc_phase, limit_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) fail(kGemmPipeTimeout);
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(acc * BN);
            if (t.valid) {
                if (kMode == kSwiGLU) {
                    __nv_bfloat16* out_row = args.out + int64_t(row) * args.ldo + nt * (BN / 2);
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
                } else if (kMode == kScatter) {
                    // acc * gate weight -> bf16 row in shared memory -> one 512-byte bulk store into the
                    // source rank's return partition (peer memory over NVLink, or local); padding rows skipped
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
                } else {
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
                        for (int j = 0; j < 16; ++j)
                            o[j] = pack_bf16(__uint_as_float(v[cur][2 * j]) * scale, __uint_as_float(v[cur][2 * j + 1]) * scale);
#pragma unroll
                        for (int q = 0; q < 4; ++q) st_v4(out_row + c + q * 8, o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh.tmem_empty[acc]), 0));
        }
        if (kMode == kScatter) {
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            __threadfence_system();
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer may still be reading this CTA's operands / signalling its barriers
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

template <int kMode, int kStages>
cudaError_t launch_pair_mode(const CUtensorMap& a, const CUtensorMap& b, const Args& args, int grid, cudaStream_t stream) {
    auto* fn = grouped_gemm_pair_kernel<kMode, kStages>;
    const size_t smem = size_t(kStages) * kStageBytes + ((sizeof(PairShared) + 127) / 128) * 128 + (kMode == kScatter ? kOutStageBytes : 0) + 256;
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(unsigned(grid));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, fn, a, b, args);
}

}  // namespace

// `grid` is rounded down to an even number of CTAs (one cluster = two CTAs on two SMs).  Plain and
// SwiGLU run six operand stages; the scatter epilogue needs shared memory for its row staging and runs four.
cudaError_t launch_pair(const CUtensorMap& a, const CUtensorMap& b, const Args& args, int mode, int grid, cudaStream_t stream, int stages) {
    if (args.num_experts > kMaxExperts) return cudaErrorInvalidValue;
    grid &= ~1;
    if (grid < 2) return cudaErrorInvalidValue;
    if (mode == kPlain) return launch_pair_mode<kPlain, 6>(a, b, args, grid, stream);
    // four stages leave ~95 KB of shared memory per SM for a co-resident transfer kernel
    if (mode == kSwiGLU && stages == 4) return launch_pair_mode<kSwiGLU, 4>(a, b, args, grid, stream);
    if (mode == kSwiGLU) return launch_pair_mode<kSwiGLU, 6>(a, b, args, grid, stream);
    if (mode == kScatter) return launch_pair_mode<kScatter, 4>(a, b, args, grid, stream);
    return cudaErrorInvalidValue;
}

}  // namespace gemm
}  // namespace nep
