"""tcgen05 grouped GEMM against a plain PyTorch fp32 reference of the same op."""

import pytest
import torch

from nanoep_b200.ops import grouped_gemm as gg

pytestmark = pytest.mark.gpu


def _offsets(blocks_per_expert):
    rows = [0]
    for b in blocks_per_expert:
        rows.append(rows[-1] + 128 * b)
    return torch.tensor(rows, dtype=torch.int64, device="cuda")


def _check(a, w, offsets, swiglu):
    out = gg.grouped_gemm(a, w, offsets, swiglu=swiglu)
    torch.cuda.synchronize()
    gg.check_status()
    ref = gg.grouped_gemm_reference(a, w, offsets, swiglu=swiglu)
    # bf16 output of an fp32-accumulated product: relative error of one bf16 ulp plus accumulation noise
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item() / 8 + 1e-3)
    return out


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("blocks,K,N", [([1], 64, 256), ([1, 2, 0, 1], 256, 512), ([3, 1, 2], 1024, 768)])
def test_small_shapes(blocks, K, N, swiglu):
    torch.manual_seed(1)
    offsets = _offsets(blocks)
    rows = int(offsets[-1])
    a = (torch.randn(rows, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(len(blocks), N, K, device="cuda") * 0.1).to(torch.bfloat16)
    _check(a, w, offsets, swiglu)


def test_identity_weights_expose_layout_errors():
    """W = stacked identity blocks: the output must reproduce the input columns exactly."""
    K = N = 256
    offsets = _offsets([2, 1])
    a = torch.randn(384, K, device="cuda").to(torch.bfloat16)
    w = torch.eye(N, K, device="cuda").to(torch.bfloat16).repeat(2, 1, 1).contiguous()
    w[1] *= 2
    out = gg.grouped_gemm(a, w, offsets)
    torch.cuda.synchronize()
    gg.check_status()
    assert torch.equal(out[:256], a[:256])
    assert torch.equal(out[256:], (a[256:].float() * 2).to(torch.bfloat16))


def test_many_tiles_persistent_schedule():
    """More tiles than CTAs and both accumulators in flight (wraps every pipeline several times)."""
    torch.manual_seed(2)
    blocks = [5, 0, 7, 3, 9, 1, 4, 6]
    offsets = _offsets(blocks)
    rows = int(offsets[-1])
    K, I = 2048, 1024
    a = (torch.randn(rows, K, device="cuda") * 0.3).to(torch.bfloat16)
    w13 = (torch.randn(len(blocks), 2 * I, K, device="cuda") * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(len(blocks), K, I, device="cuda") * 0.05).to(torch.bfloat16)
    h = _check(a, w13, offsets, True)
    _check(h, w2, offsets, False)
    # a small grid forces many tiles per CTA
    out_small = gg.grouped_gemm(a, w13, offsets, swiglu=True, max_ctas=3)
    torch.cuda.synchronize()
    gg.check_status()
    assert torch.equal(out_small, h)


def test_tile_gating_waits_for_ready_counters():
    """Producer-side gating: tiles only start when their counter reached the expected value."""
    torch.manual_seed(3)
    offsets = _offsets([2, 2])
    a = (torch.randn(512, 128, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(2, 256, 128, device="cuda") * 0.1).to(torch.bfloat16)
    ready = torch.tensor([128, 128, 128, 128], dtype=torch.int32, device="cuda")
    expected = torch.tensor([128, 100, 128, 1], dtype=torch.int32, device="cuda")
    out = gg.grouped_gemm(a, w, offsets, tile_ready=ready, tile_expected=expected)
    torch.cuda.synchronize()
    gg.check_status()
    torch.testing.assert_close(out.float(), gg.grouped_gemm_reference(a, w, offsets), rtol=2e-2, atol=2e-2)
    # a counter that never reaches its value: the bounded wait gives up and reports, nothing hangs
    never = torch.zeros(4, dtype=torch.int32, device="cuda")
    gg.grouped_gemm(a, w, offsets, tile_ready=never, tile_expected=expected, timeout_s=0.2)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="timed out"):
        gg.check_status()
    assert torch.ones(2, device="cuda").sum().item() == 2


@pytest.mark.parametrize("swiglu", [False, True])
def test_cta_pair_kernel_matches_reference_and_single_cta(swiglu):
    """tcgen05 cta_group::2 variant: experts with odd and even block counts, an empty expert, many tiles."""
    torch.manual_seed(5)
    blocks = [3, 2, 0, 1, 4, 5]
    offsets = _offsets(blocks)
    rows = int(offsets[-1])
    K, N = 512, 512
    a = (torch.randn(rows, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(len(blocks), N, K, device="cuda") * 0.1).to(torch.bfloat16)
    single = gg.grouped_gemm(a, w, offsets, swiglu=swiglu)
    n_out = N // 2 if swiglu else N
    out = torch.full((rows, n_out), float("nan"), dtype=torch.bfloat16, device="cuda")
    gg.grouped_gemm(a, w, offsets, swiglu=swiglu, pair=True, out=out)
    torch.cuda.synchronize()
    gg.check_status()
    ref = gg.grouped_gemm_reference(a, w, offsets, swiglu=swiglu)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    assert torch.equal(out, single), "pair and single-CTA kernels accumulate in the same order"
    small = gg.grouped_gemm(a, w, offsets, swiglu=swiglu, pair=True, max_ctas=4)
    torch.cuda.synchronize()
    gg.check_status()
    assert torch.equal(small, single)


def test_offsets_off_the_block_grid_are_reported():
    """One expert per 128-row block: offsets that are not multiples of 128, or that do not end at the row count, are refused."""
    a = torch.zeros(256, 128, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(2, 256, 128, dtype=torch.bfloat16, device="cuda")
    for bad in ([0, 100, 256], [0, 128, 128]):
        out = gg.grouped_gemm(a, w, torch.tensor(bad, dtype=torch.int64, device="cuda"))
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="expert_offsets"):
            gg.check_status()
        del out
    assert torch.ones(2, device="cuda").sum().item() == 2
