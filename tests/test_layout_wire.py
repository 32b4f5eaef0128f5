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
def test_layout_matches_wire_spec(native, geom):
    ranks, tmax, hidden, topk, experts = geom
    got = native.window_layout(ranks, tmax, hidden, topk, experts)
    want = wire.window_regions(ranks, tmax, hidden, topk, experts)
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
    # 8 ranks x 4096 tokens x 7168 bf16, top-8 of 256: about 1.06 GB per rank with both parities
    got = native.window_layout(8, 4096, 7168, 8, 256)
    assert got["row_bytes"] == 14368
    assert 1.0e9 < got["num_bytes"] < 1.2e9
