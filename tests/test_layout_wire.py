"""The native window layout must agree with the independent Python wire spec (CPU; needs the built
extension but no GPU)."""

import pytest

from nanoep_b200.testing import wire


@pytest.fixture(scope="module")
def native():
    from nanoep_b200.utils.build import load_extension

    return load_extension()


@pytest.mark.parametrize(
    "geom",
    [(1, 5, 256, 3, 3), (2, 8, 256, 2, 4), (8, 4096, 7168, 8, 256), (8, 8192, 4096, 6, 64), (4, 2153, 512, 32, 260 * 4), (32, 7, 768, 1, 32)],
)
@pytest.mark.parametrize("per_rank", [False, True])
def test_layout_matches_wire_spec(native, geom, per_rank):
    ranks, tmax, hidden, topk, experts = geom
    got = native.window_layout(ranks, tmax, hidden, topk, experts, per_rank)
    want = wire.window_regions(ranks, tmax, hidden, topk, experts, per_rank)
    for key, value in want.items():
        assert got[key] == value, key
    assert got["row_bytes"] % 16 == 0
    for key, value in got.items():
        if key.endswith("_offset") or key.endswith("_stride"):
            assert value % 256 == 0, key


def test_layout_rejects_bad_geometry(native):
    for bad in [(3, 8, 256, 2, 6), (2, 0, 256, 2, 4), (2, 8, 256, 33, 64), (2, 8, 256, 2, 5), (64, 8, 256, 2, 64), (2, 8, 252, 2, 4)]:
        with pytest.raises(Exception):
            native.window_layout(*bad)


def test_dsv3_window_size(native):
    # 8 ranks x 4096 tokens x 7168 bf16, top-8 of 256: two staging copies (2 x 59 MB) + one return area (8 x 59 MB)
    got = native.window_layout(8, 4096, 7168, 8, 256)
    assert got["row_bytes"] == 14368
    assert 0.58e9 < got["num_bytes"] < 0.62e9


def test_return_partitions_follow_the_reduction_mode(native):
    # per-rank pre-reduction returns one row per (token, rank): min(R, K) partitions, indexed by rank when R <= K
    assert native.window_layout(2, 64, 256, 8, 16, True)["ret_parts"] == 2
    assert native.window_layout(2, 64, 256, 8, 16, True)["rank_indexed"] == 1
    assert native.window_layout(8, 64, 256, 2, 16, True)["ret_parts"] == 2
    assert native.window_layout(8, 64, 256, 2, 16, True)["rank_indexed"] == 0
    assert native.window_layout(2, 64, 256, 8, 16, False)["ret_parts"] == 8
    small = native.window_layout(2, 4096, 7168, 8, 64, True)["num_bytes"]
    full = native.window_layout(2, 4096, 7168, 8, 64, False)["num_bytes"]
    assert full - small > 5 * 4096 * 7168 * 2
