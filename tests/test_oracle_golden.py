"""The numpy oracle against vectors produced by the DIMQ reference itself."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import dimq_oracle as o

PACK_CASES = ["arange17", "arange257x7", "n1", "n2", "allmax9", "rand4099", "rand2d"]


@pytest.mark.parametrize("name", PACK_CASES)
def test_pack_unpack_u4_matches_reference(golden, name):
    idx = golden[f"pack_{name}_idx"]
    packed = golden[f"pack_{name}_packed"]
    assert np.array_equal(o.pack_u4(idx), packed)
    assert np.array_equal(o.pack_bits(idx, 4), packed)
    assert np.array_equal(o.unpack_u4(packed, idx.size), idx.reshape(-1))


def test_pack_u4_odd_length_is_nine_bytes(golden):
    # dimq_cuda_backend/tests/test_reference_and_export.py:19-27
    assert golden["pack_arange17_packed"].size == 9
    assert o.pack_u4(golden["pack_arange17_idx"]).size == 9


def test_pack_u4_rejects_out_of_range():
    with pytest.raises(ValueError):
        o.pack_u4(np.array([16], dtype=np.uint8))


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("n", [0, 1, 2, 7, 8, 9, 17, 257, 4099])
def test_pack_bits_round_trip_and_size(bits, n):
    rng = np.random.default_rng(bits * 1000 + n)
    idx = rng.integers(0, 1 << bits, size=n, dtype=np.uint8)
    packed = o.pack_bits(idx, bits)
    assert packed.size == (n * bits + 7) // 8
    assert np.array_equal(o.unpack_bits(packed, n, bits), idx)
    if n and (n * bits) % 8:
        assert packed[-1] >> ((n * bits) % 8) == 0  # tail bits are zero


def test_pack_bits_layouts_by_hand():
    # 2-bit: four per byte, lowest bits first
    assert o.pack_bits(np.array([1, 2, 3, 0, 3]), 2).tolist() == [1 | 2 << 2 | 3 << 4 | 0 << 6, 3]
    # 3-bit: eight indices in three bytes
    idx = np.array([1, 2, 3, 4, 5, 6, 7, 0])
    stream = sum(int(v) << (3 * j) for j, v in enumerate(idx))
    assert o.pack_bits(idx, 3).tolist() == [stream & 255, (stream >> 8) & 255, (stream >> 16) & 255]
    # 8-bit: identity
    assert o.pack_bits(np.array([7, 200, 255]), 8).tolist() == [7, 200, 255]


@pytest.mark.parametrize("k", [4, 8, 16, 256])
def test_hard_quantize_matches_reference(golden, k):
    idx = o.hard_quantize(golden[f"hq_k{k}_w"], golden[f"hq_k{k}_centers"])
    assert np.array_equal(idx, golden[f"hq_k{k}_idx"])
    vals = o.dequantize(idx, golden[f"hq_k{k}_centers"])
    assert np.array_equal(vals, golden[f"hq_k{k}_vals"])


def test_hard_quantize_reference_unit_case(golden):
    idx = o.hard_quantize(golden["hq_lin_w"], golden["hq_lin_centers"])
    assert np.array_equal(idx, golden["hq_lin_idx"])


@pytest.mark.parametrize("book", ["sorted", "dups", "unsorted", "withnan", "withinf", "tiny"])
def test_hard_quantize_adversarial(golden, book):
    idx = o.hard_quantize(golden["hq_adv_w"], golden[f"hq_adv_{book}_centers"])
    assert np.array_equal(idx, golden[f"hq_adv_{book}_idx"])


def test_hard_quantize_ties_go_to_lowest_index():
    idx = o.hard_quantize(np.array([0.5, 1.5], dtype=np.float32), np.array([0.0, 1.0, 2.0], dtype=np.float32))
    assert idx.tolist() == [0, 1]


def test_grouped_codebooks_are_slicewise_reference(golden):
    idx = o.hard_quantize_grouped(golden["grp_w"], golden["grp_codebooks"], 8)
    assert np.array_equal(idx, golden["grp_idx"])
    for g in range(3):
        cb = o.quantile_codebook(golden["grp_w"][8 * g : 8 * g + 8], 8)
        np.testing.assert_allclose(cb, golden["grp_codebooks"][g], rtol=1e-6, atol=1e-9)


@pytest.mark.parametrize("k", [4, 8, 16, 256])
def test_quantile_codebook_matches_reference_init(golden, k):
    cb = o.quantile_codebook(golden[f"hq_k{k}_w"], k)
    np.testing.assert_allclose(cb, golden[f"hq_k{k}_centers"], rtol=2e-6, atol=1e-9)


def test_quantize_activation_u4_matches_reference(golden):
    for i, (s, z) in enumerate(golden["aq_grid"]):
        q = o.quantize_activation_u4(golden["aq_x"], float(s), int(z))
        assert np.array_equal(q, golden[f"aq_q{i}"]), (s, z)


def test_product_table_matches_reference_bitwise(golden):
    t = o.build_product_table(golden["pt_cb_f16_as_f32"], 0.125, 8)
    assert np.array_equal(t, golden["pt_table_f16"])
    t = o.build_product_table(golden["pt_cb_f32"], 0.2, 7)
    assert np.array_equal(t, golden["pt_table_f32"])


def test_linear_lut_a4_matches_reference(golden):
    y = o.linear_lut_a4(golden["lin_x"], golden["lin_packed"], golden["lin_cb"], 0.2, 7, 6, 11, golden["lin_bias"])
    np.testing.assert_allclose(y, golden["lin_y_lut"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(y, golden["lin_y_deq"], rtol=1e-5, atol=1e-5)
    y = o.linear_lut_a4(golden["lin_x"], golden["lin_packed"], golden["lin_cb"], 0.2, 7, 6, 11, None)
    np.testing.assert_allclose(y, golden["lin_y_nobias"], rtol=1e-5, atol=1e-5)
    y = o.linear_lut_a4(golden["linb_x"], golden["linb_packed"], golden["linb_cb"], 0.3, 8, 24, 64, None)
    assert y.shape == (2, 5, 24)
    np.testing.assert_allclose(y, golden["linb_y_lut"], rtol=1e-5, atol=1e-5)


def test_conv2d_lut_a4_matches_reference(golden):
    y = o.conv2d_lut_a4(golden["conv_x"], golden["conv_packed"], golden["conv_cb"], 0.25, 7, (5, 3, 3, 3),
                        golden["conv_bias"], stride=(2, 1), padding=(1, 1))
    np.testing.assert_allclose(y, golden["conv_y_deq"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(y, golden["conv_y_lut"], rtol=1e-5, atol=1e-5)
    y = o.conv2d_lut_a4(golden["convg_x"], golden["convg_packed"], golden["conv_cb"], 0.25, 7, (6, 2, 3, 2), None,
                        stride=(1, 2), padding=(2, 1), dilation=(2, 1), groups=2)
    np.testing.assert_allclose(y, golden["convg_y_deq"], rtol=1e-5, atol=1e-5)


def test_weight_only_paths_match_reference(golden):
    y = o.linear_wq(golden["wq_lin_x"], golden["wq_lin_packed"], golden["wq_lin_cb"], 4, 48, 96, golden["wq_lin_bias"])
    np.testing.assert_allclose(y, golden["wq_lin_y"], rtol=1e-5, atol=1e-6)
    idx = o.hard_quantize(golden["wq_lin_w"], golden["wq_lin_cb"])
    assert np.array_equal(o.pack_u4(idx), golden["wq_lin_packed"])
    assert np.array_equal(o.dequantize(idx, golden["wq_lin_cb"]), golden["wq_lin_what"])
    y = o.conv2d_wq(golden["wq_conv_x"], golden["wq_conv_packed"], golden["wq_conv_cb"], 4, (8, 4, 3, 3),
                    stride=(1, 1), padding=(1, 1))
    np.testing.assert_allclose(y, golden["wq_conv_y"], rtol=1e-5, atol=1e-5)
    y = o.conv2d_wq(golden["wq_conv_x"], golden["wq_conv_packed"], golden["wq_conv_cb"], 4, (8, 4, 3, 3),
                    stride=(2, 2), padding=(1, 1))
    np.testing.assert_allclose(y, golden["wq_conv_y_s2"], rtol=1e-5, atol=1e-5)


# ---- the C restatement (oracle/dimq_oracle.c) against the same vectors -------

def test_c_oracle_matches_reference_vectors(golden):
    from oracle import c_oracle as c

    for name in PACK_CASES:
        idx, packed = golden[f"pack_{name}_idx"], golden[f"pack_{name}_packed"]
        assert np.array_equal(c.pack_bits(idx, 4), packed)
        assert np.array_equal(c.unpack_bits(packed, idx.size, 4), idx.reshape(-1))
    for bits in (2, 3, 8):
        idx = np.random.default_rng(bits).integers(0, 1 << bits, size=1237, dtype=np.uint8)
        assert np.array_equal(c.pack_bits(idx, bits), o.pack_bits(idx, bits))
        assert np.array_equal(c.unpack_bits(o.pack_bits(idx, bits), idx.size, bits), idx)
    for k in (4, 8, 16, 256):
        assert np.array_equal(c.hard_quantize(golden[f"hq_k{k}_w"], golden[f"hq_k{k}_centers"]), golden[f"hq_k{k}_idx"])
    for book in ("sorted", "dups", "unsorted", "withnan", "withinf", "tiny"):
        assert np.array_equal(c.hard_quantize(golden["hq_adv_w"], golden[f"hq_adv_{book}_centers"]),
                              golden[f"hq_adv_{book}_idx"]), book
    assert np.array_equal(c.hard_quantize(golden["grp_w"], golden["grp_codebooks"], 8), golden["grp_idx"])
    for i, (s, z) in enumerate(golden["aq_grid"]):
        assert np.array_equal(c.quantize_activation_u4(golden["aq_x"], float(s), int(z)), golden[f"aq_q{i}"])
    assert np.array_equal(c.product_table(golden["pt_cb_f32"], 0.2, 7), golden["pt_table_f32"])
    y = c.linear_lut_a4(golden["lin_x"], golden["lin_packed"], golden["lin_cb"], 0.2, 7, 6, 11, golden["lin_bias"])
    np.testing.assert_allclose(y, golden["lin_y_lut"], rtol=1e-5, atol=1e-5)
    y = c.conv2d_lut_a4(golden["conv_x"], golden["conv_packed"], golden["conv_cb"], 0.25, 7, (5, 3, 3, 3),
                        golden["conv_bias"], stride=(2, 1), padding=(1, 1))
    np.testing.assert_allclose(y, golden["conv_y_lut"], rtol=1e-5, atol=1e-5)
    y = c.conv2d_lut_a4(golden["convg_x"], golden["convg_packed"], golden["conv_cb"], 0.25, 7, (6, 2, 3, 2), None,
                        stride=(1, 2), padding=(2, 1), dilation=(2, 1), groups=2)
    np.testing.assert_allclose(y, golden["convg_y_deq"], rtol=1e-5, atol=1e-5)
    y = c.linear_wq(golden["wq_lin_x"], golden["wq_lin_packed"], 4, golden["wq_lin_cb"], 48, 96, golden["wq_lin_bias"])
    np.testing.assert_allclose(y, golden["wq_lin_y"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_linear_prepack_order_by_hand(bits):
    """The tiled index order: unit (row block rb, 128-k range kr) is contiguous, its rows in order, and the
    dequantised weight read back through the tiles is the one read from the canonical stream."""
    n, k = 48, 384
    rng = np.random.default_rng(bits)
    idx = rng.integers(0, 1 << bits, size=(n, k)).astype(np.uint8)
    packed = o.pack_bits(idx.reshape(-1), bits)
    tiled = o.linear_prepack(packed, n, k, bits)
    assert tiled.shape == packed.shape and sorted(tiled.tolist()) == sorted(packed.tolist())
    piece = 16 * bits
    for rb, kr, r in ((0, 0, 0), (1, 2, 5), (2, 1, 15)):
        at = ((rb * (k // 128) + kr) * 16 + r) * piece
        want = o.pack_bits(idx[rb * 16 + r, kr * 128:(kr + 1) * 128], bits)
        assert np.array_equal(tiled[at:at + piece], want)

