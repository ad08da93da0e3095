"""GPU parity of the byte/integer kernels (bit-exact class), through the C ABI."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import dimq_oracle as o

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(cuda_device):
    from dimq_b200 import ops as _ops

    _ops.require_extension()
    return _ops


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_pack_unpack_u4_reference_case(ops, golden):
    # dimq_cuda_backend/tests/test_cuda_ops.py:31-39
    indices = (torch.arange(257, dtype=torch.uint8, device="cuda") * 7) % 16
    packed = ops.pack_u4(indices)
    restored = ops.unpack_u4(packed, indices.numel())
    assert np.array_equal(packed.cpu().numpy(), golden["pack_arange257x7_packed"])
    assert torch.equal(restored, indices)
    assert torch.equal(torch.ops.dimq.pack_u4(indices), packed)


@pytest.mark.parametrize("name", ["arange17", "n1", "n2", "allmax9", "rand4099", "rand2d"])
def test_pack_u4_golden(ops, golden, name):
    idx = golden[f"pack_{name}_idx"]
    packed = ops.pack_u4(_cuda(idx))
    assert np.array_equal(packed.cpu().numpy(), golden[f"pack_{name}_packed"])
    assert np.array_equal(ops.unpack_u4(packed, idx.size).cpu().numpy(), idx.reshape(-1))


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("n", [0, 1, 2, 7, 8, 9, 15, 16, 17, 257, 4099, (1 << 20) + 3])
def test_pack_bits_matches_oracle(ops, bits, n):
    rng = np.random.default_rng(bits * 7919 + n)
    idx = rng.integers(0, 1 << bits, size=n, dtype=np.uint8)
    want = o.pack_bits(idx, bits) if n < 100000 else c_oracle.pack_bits(idx, bits)
    got = ops.pack_bits(_cuda(idx), bits)
    assert got.numel() == (n * bits + 7) // 8
    assert np.array_equal(got.cpu().numpy(), want)
    back = ops.unpack_bits(got, n, bits)
    assert np.array_equal(back.cpu().numpy(), idx)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_pack_bits_unaligned_views_and_patterns(ops, bits):
    n = 1000
    base = (torch.arange(n + 3, dtype=torch.int64, device="cuda") * 7 % (1 << bits)).to(torch.uint8)
    view = base[3:]  # data pointer no longer 16-byte aligned
    want = o.pack_bits(view.cpu().numpy(), bits)
    assert np.array_equal(ops.pack_bits(view, bits).cpu().numpy(), want)
    allmax = torch.full((n,), (1 << bits) - 1, dtype=torch.uint8, device="cuda")
    assert np.array_equal(ops.pack_bits(allmax, bits).cpu().numpy(), o.pack_bits(allmax.cpu().numpy(), bits))
    packed = _cuda(np.concatenate([[0], want]).astype(np.uint8))[1:]
    assert np.array_equal(ops.unpack_bits(packed, n, bits).cpu().numpy(), view.cpu().numpy())


def test_pack_masks_high_bits_like_the_reference_kernel(ops):
    # csrc/dimq_pack.cu:19,22 masks with 0x0F instead of validating
    idx = torch.tensor([0x1F, 0xF3, 0x07], dtype=torch.uint8, device="cuda")
    assert ops.pack_u4(idx).cpu().tolist() == [0x3F, 0x07]


def test_unpack_checks(ops):
    with pytest.raises(RuntimeError):
        ops.unpack_u4(torch.zeros(3, dtype=torch.uint8, device="cuda"), 8)
    with pytest.raises(RuntimeError):
        ops.pack_u4(torch.zeros(3, dtype=torch.int32, device="cuda"))
    assert ops.unpack_u4(torch.zeros(0, dtype=torch.uint8, device="cuda"), 0).numel() == 0
    assert ops.pack_u4(torch.zeros(0, dtype=torch.uint8, device="cuda")).numel() == 0


def test_quantize_activation_u4_golden(ops, golden):
    x = _cuda(golden["aq_x"])
    for i, (s, z) in enumerate(golden["aq_grid"]):
        q = ops.quantize_activation_u4(x, float(s), int(z))
        assert np.array_equal(q.cpu().numpy(), golden[f"aq_q{i}"]), (s, z)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_quantize_activation_u4_dtypes_and_boundaries(ops, dtype):
    torch.manual_seed(11)
    x = torch.cat([torch.randn(5003) * 3, (torch.arange(-40, 41) * 0.1)]).to(dtype).cuda()
    for s, z in [(0.2, 7), (0.125, 8), (1.0, 0), (0.37, 15)]:
        want = o.quantize_activation_u4(x.float().cpu().numpy(), s, z)
        got = ops.quantize_activation_u4(x, s, z)
        assert np.array_equal(got.cpu().numpy(), want)
        assert got.shape == x.shape
    with pytest.raises(RuntimeError):
        ops.quantize_activation_u4(x, 0.0, 3)
    with pytest.raises(RuntimeError):
        ops.quantize_activation_u4(x, 1.0, 16)


def test_product_table_bitwise(ops, golden):
    # dimq_cuda_backend/tests/test_cuda_ops.py:42-48 (there with rtol 1e-3; here bit-exact)
    cb = torch.linspace(-1.0, 1.0, 16, device="cuda", dtype=torch.float16)
    t = ops.build_product_table(cb, 0.125, 8)
    assert t.shape == (16, 16) and t.dtype == torch.float32
    assert np.array_equal(t.cpu().numpy(), golden["pt_table_f16"])
    t = ops.build_product_table(_cuda(golden["pt_cb_f32"]), 0.2, 7)
    assert np.array_equal(t.cpu().numpy(), golden["pt_table_f32"])
    grouped = ops.build_product_table_grouped(_cuda(np.stack([golden["pt_cb_f32"], golden["pt_cb_f32"] * 2])), 0.2, 7)
    assert np.array_equal(grouped[0].cpu().numpy(), golden["pt_table_f32"])
    assert np.array_equal(grouped[1].cpu().numpy(), o.build_product_table(golden["pt_cb_f32"] * 2, 0.2, 7))
    with pytest.raises(RuntimeError):
        ops.build_product_table(torch.zeros(8, device="cuda"), 0.2, 7)


@pytest.mark.parametrize("k", [4, 8, 16, 256])
def test_hard_quantize_golden(ops, golden, k):
    w = _cuda(golden[f"hq_k{k}_w"])
    cb = _cuda(golden[f"hq_k{k}_centers"])
    bits = {4: 2, 8: 3, 16: 4, 256: 8}[k]
    idx, packed = ops.hard_quantize(w, cb, bits=bits)
    assert np.array_equal(idx.cpu().numpy(), golden[f"hq_k{k}_idx"])
    assert np.array_equal(packed.cpu().numpy(), o.pack_bits(golden[f"hq_k{k}_idx"], bits))


@pytest.mark.parametrize("book", ["sorted", "dups", "unsorted", "withnan", "withinf", "tiny"])
def test_hard_quantize_adversarial(ops, golden, book):
    idx, _ = ops.hard_quantize(_cuda(golden["hq_adv_w"]), _cuda(golden[f"hq_adv_{book}_centers"]))
    assert np.array_equal(idx.cpu().numpy(), golden[f"hq_adv_{book}_idx"])


@pytest.mark.parametrize("entries", [1, 2, 3, 5, 8, 12, 16, 37, 200, 256])
@pytest.mark.parametrize("kind", ["normal", "dups", "tiny", "huge", "zeros", "grid"])
def test_hard_quantize_sorted_codebook_search(ops, entries, kind):
    """Sorted finite codebooks take the bisection path; it must give the scan's answer bit for bit:
    duplicates, exact midpoints, weights equal to codewords, denormal and overflowing distances,
    signed zeros, non-finite weights, codeword counts that are not powers of two."""
    from oracle import c_oracle

    rng = np.random.default_rng(entries * 7 + len(kind))
    np.seterr(over="ignore", invalid="ignore")  # the "huge" case overflows on purpose
    if kind == "normal":
        cb = np.sort(rng.standard_normal(entries).astype(np.float32) * 0.05)
    elif kind == "dups":
        cb = np.sort(rng.choice(np.array([-0.5, -0.25, 0.0, 0.25, 0.5], np.float32), entries))
    elif kind == "tiny":
        cb = np.sort((rng.integers(-20, 20, entries) * np.float32(1e-44)).astype(np.float32))  # denormals
    elif kind == "huge":
        cb = np.sort((rng.standard_normal(entries) * 1e38).astype(np.float32))
        cb = np.clip(cb, -3.0e38, 3.0e38)
    elif kind == "zeros":
        cb = np.sort(np.concatenate([np.full(entries // 2, -0.0, np.float32), np.zeros(entries - entries // 2, np.float32)]))
    else:
        cb = (np.arange(entries, dtype=np.float32) - entries // 2) * np.float32(0.125)
    cb = cb.astype(np.float32)
    mids = (cb[:-1] + cb[1:]) / 2 if entries > 1 else cb
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 3.4e38, -3.4e38, 1e-45, -1e-45], np.float32)
    scale = np.float32(max(float(np.abs(cb).max()), 1e-3) * 1.5)
    w = np.concatenate([cb, mids, np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf)),
                        special, (rng.standard_normal(4096) * scale).astype(np.float32)]).astype(np.float32)
    w = np.resize(w, (w.size + 7) // 8 * 8).reshape(-1, 8)
    want = c_oracle.hard_quantize(w, cb[None, :], w.shape[0])
    idx, _ = ops.hard_quantize(_cuda(w), _cuda(cb))
    got = idx.cpu().numpy()
    bad = np.argwhere(got != want)
    assert bad.size == 0, (kind, entries, w[tuple(bad[0])], got[tuple(bad[0])], want[tuple(bad[0])], cb)


def test_hard_quantize_reference_unit_case_and_wrapper(ops, golden):
    from dimq_b200.export import hard_quantize_weight

    w = torch.from_numpy(golden["hq_lin_w"])
    centers = torch.from_numpy(golden["hq_lin_centers"])
    w_q, idx = hard_quantize_weight(w, centers, chunk_size=17)  # tests/test_dimq_math.py:35-43
    assert w_q.shape == w.shape and idx.shape == w.shape and idx.dtype == torch.int64
    assert torch.unique(w_q).numel() <= centers.numel()
    assert np.array_equal(idx.numpy().astype(np.uint8), golden["hq_lin_idx"])


def test_hard_quantize_grouped(ops, golden):
    idx, packed = ops.hard_quantize(_cuda(golden["grp_w"]), _cuda(golden["grp_codebooks"]), group_rows=8, bits=3)
    assert np.array_equal(idx.cpu().numpy(), golden["grp_idx"])
    assert np.array_equal(packed.cpu().numpy(), o.pack_bits(golden["grp_idx"], 3))
    # groups whose row length is not a multiple of 8: threads straddle codebooks
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((7, 13)) * 0.02).astype(np.float32)
    cbs = np.stack([o.quantile_codebook(w[r : r + 1], 4) for r in range(7)])
    idx, packed = ops.hard_quantize(_cuda(w), _cuda(cbs), group_rows=1, bits=2)
    want = o.hard_quantize_grouped(w, cbs, 1)
    assert np.array_equal(idx.cpu().numpy(), want)
    assert np.array_equal(packed.cpu().numpy(), o.pack_bits(want, 2))


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_hard_quantize_pack_full_size_export(ops, bits):
    """The ViT-L sized export (4 194 304 weights): indices and packed bytes equal the CPU oracle's."""
    rng = np.random.default_rng(100 + bits)
    w = (rng.standard_normal((4096, 1024)) * 0.02).astype(np.float32)
    cb = o.quantile_codebook(w[:256], 1 << bits)
    want_idx = c_oracle.hard_quantize(w, cb)
    want_packed = c_oracle.pack_bits(want_idx, bits)
    idx, packed = ops.hard_quantize(_cuda(w), _cuda(cb), bits=bits)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert np.array_equal(packed.cpu().numpy(), want_packed)
    # size-independent property: unpack(pack(idx)) == idx and the fused packing equals pack(idx)
    assert torch.equal(ops.unpack_bits(packed, idx.numel(), bits).view_as(idx), idx)
    assert torch.equal(ops.pack_bits(idx, bits), packed)
    _, packed_only = ops.hard_quantize(_cuda(w), _cuda(cb), bits=bits, return_indices=False)
    assert torch.equal(packed_only, packed)


def test_export_helpers_round_trip(ops, golden):
    from dimq_b200 import export

    idx = torch.from_numpy(golden["pack_arange17_idx"])
    packed = export.pack_u4_indices(idx)  # dimq_cuda_backend/tests/test_reference_and_export.py:19-27
    assert packed.dtype == torch.uint8 and packed.numel() == 9 and not packed.is_cuda
    assert torch.equal(export.unpack_u4_indices(packed, idx.numel()), idx)
    with pytest.raises(ValueError):
        export.pack_u4_indices(torch.tensor([16], dtype=torch.uint8))
    w = torch.from_numpy(golden["hq_k16_w"])
    cb = torch.from_numpy(golden["hq_k16_centers"])
    assert np.array_equal(export.assign_weight_indices(w, cb).numpy(), golden["hq_k16_idx"])


# ---- QAT side: straight-through fake quantisation (quant/dimq_wrapper.py:72-75) ----------------------

@pytest.mark.parametrize("key", ["hq_k4", "hq_k8", "hq_k16", "hq_k256"])
def test_fake_quant_weight_matches_reference_expression(ops, golden, key):
    """Forward value bit-equal to  w + (centers[idx] - w)  built from the reference's own outputs
    (hard_quantize_weight's values), gradient = identity on the weight, none on the centres."""
    from dimq_b200.qat import fake_quant_weight

    w = torch.from_numpy(golden[key + "_w"]).cuda().requires_grad_(True)
    centers = torch.from_numpy(golden[key + "_centers"]).cuda().requires_grad_(True)
    out = fake_quant_weight(w, centers, 262144)
    want = golden[key + "_w"] + (golden[key + "_vals"] - golden[key + "_w"])      # fp32, operation by operation
    assert np.array_equal(out.detach().cpu().numpy(), want)
    g = torch.randn_like(out)
    out.backward(g)
    assert torch.equal(w.grad, g) and centers.grad is None
    fq, idx = ops.fake_quantize_ste(w.detach(), centers.detach(), return_indices=True)
    assert np.array_equal(idx.cpu().numpy(), golden[key + "_idx"].astype(np.uint8))
    assert torch.equal(fq, out.detach())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fake_quant_weight_half_types_and_groups(ops, dtype):
    """16-bit weights: every operation rounds to the weight's type, as PyTorch evaluates the expression;
    grouped codebooks apply slice by slice."""
    from dimq_b200.qat import fake_quant_weight

    torch.manual_seed(0)
    w = (torch.randn(300, 77) * 0.05).to(dtype).cuda()
    books = torch.sort(torch.randn(3, 8) * 0.05, dim=1).values.cuda()
    out = fake_quant_weight(w, books, group_rows=128)
    idx, _ = ops.hard_quantize(w, books, group_rows=128)
    rows = torch.arange(300, device="cuda") // 128
    hard = books[rows[:, None], idx.long()].to(dtype)
    assert torch.equal(out, w + (hard - w))
    with pytest.raises(ValueError):
        fake_quant_weight(w, books[:, :0])
