// Launch interface of the tcgen05 grouped GEMM (see grouped_gemm_sm100.cu).
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace nep {
namespace gemm {

enum Mode : int { kPlain = 0, kSwiGLU = 1, kScatter = 2 };
enum GemmStatus : uint32_t { kGemmOk = 0, kGemmPipeTimeout = 101, kGemmTileTimeout = 102, kGemmBadOffsets = 103, kGemmBadMetadata = 104 };

struct Args {
    const int64_t* expert_offsets;  // [E+1] padded exclusive row offsets, multiples of 128
    int num_experts;
    int m_blocks;            // total rows / 128
    int n_tiles;             // output column tiles per row block (256 wide; 128 wide for SwiGLU)
    int k_blocks;            // K / 64
    int b_rows_per_expert;   // rows of the flattened weight per expert (N, or 2*I for SwiGLU)
    int swiglu_up_row_offset;  // I: distance from a gate row to its up row
    __nv_bfloat16* out;      // [rows, ldo] (kPlain / kSwiGLU)
    int ldo;                 // output row length in elements (also the hidden size for kScatter)
    const float* row_scale;  // kPlain: optional per-row factor applied in FP32 before the bf16 round
    uint32_t* status;        // 2 words: [0] first error code, [1] CTA
    uint64_t timeout_ns;
    // tile gating (optional): row block mb may be loaded once tile_ready[mb] >= tile_expected[mb]
    const int* tile_ready;
    const int* tile_expected;
    // kScatter: rows go to the source ranks' return partitions
    const int* slot_map;        // [rows] -> recv_row * topk + k, -1 padding
    const int* recv_metadata;   // [N, topk + 2]
    const float* slot_weights;  // [rows] gate weight per slot or null
    void* peers[32];
    int64_t ret_offset;         // byte offset of the return partitions (parity applied) in a window
    int64_t max_tokens;
    int topk;
    int ranks;      // kScatter: valid source ranks are [0, ranks)
    int recv_rows;  // kScatter: rows of recv_metadata
};

size_t shared_bytes(int mode, int stages);
cudaError_t launch(const CUtensorMap& a, const CUtensorMap& b, const Args& args, int mode, int stages, int grid, cudaStream_t stream);
int kernel_registers(int mode);
// CTA-pair variant (tcgen05 cta_group::2, 256 x 256 tiles on two SMs); modes kPlain and kSwiGLU.
cudaError_t launch_pair(const CUtensorMap& a, const CUtensorMap& b, const Args& args, int mode, int grid, cudaStream_t stream, int stages = 6);

}  // namespace gemm
}  // namespace nep
