"""The CPU oracle against the golden vectors generated from the reference's reference.py and
against the known-answer tables of the reference's own tests (tests/test_reference.py:20-49,
tests/test_ops.py:192, tests/test_swiglu_epilogue.py:96-101)."""
import os

import numpy as np
import pytest

from oracle import paired_nvfp4_oracle as orc

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_weight_vectors.npz"))


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_weight_path_matches_reference_outputs(name):
    w = G[f"{name}_w"]
    pruned = orc.prune_paired_4of8(w)
    assert np.array_equal(pruned, G[f"{name}_pruned"])
    packed, sf, dq = orc.quantize_weight(pruned)
    assert np.array_equal(packed, G[f"{name}_packed"])
    assert np.array_equal(sf, G[f"{name}_sf"])
    assert np.array_equal(dq, G[f"{name}_dq"], equal_nan=True)
    assert np.array_equal(orc.dequantize_weight(packed, sf), G[f"{name}_dq2"], equal_nan=True)
    assert orc.is_paired_4of8(pruned) and orc.is_paired_4of8(dq)


def test_round_to_e2m1_weight_table_and_midpoints():
    assert np.array_equal(orc.round_to_e2m1_weight(G["round_x"]), G["round_y"])
    # tests/test_reference.py:27-30
    x = np.array([0.2, 0.3, 0.8, 1.3, 1.8, 2.6, 3.6, 5.1, 100.0, -0.3, -7.0], np.float32)
    want = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, 6.0, -0.5, -6.0], np.float32)
    assert np.array_equal(orc.round_to_e2m1_weight(x), want)


def test_pack_unpack_tables():
    assert np.array_equal(orc.pack_e2m1(G["pack_vals"][None]), G["pack_bytes"])
    assert np.array_equal(orc.unpack_e2m1(np.arange(256, dtype=np.uint8)[None]), G["unpack_vals"])
    assert np.array_equal(orc.unpack_e2m1(G["pack_bytes"])[0], G["pack_vals"])


def test_e4m3_codec_matches_torch_cast_table():
    assert np.array_equal(orc.f32_to_e4m3_bits(G["e4m3_in"]), G["e4m3_bits"])
    allb = np.arange(256, dtype=np.uint8)
    vals = orc.e4m3_bits_to_f32(allb)
    ok = ~np.isnan(vals)
    back = orc.f32_to_e4m3_bits(vals[ok])
    # -0 keeps its sign bit
    assert np.array_equal(back, allb[ok])
    assert orc.f32_to_e4m3_bits(np.float32(1.0)) == orc.BENIGN_SF_BYTE == 0x38
    assert orc.f32_to_e4m3_bits(np.float32(1e9)) == 0x7E and orc.f32_to_e4m3_bits(np.float32(np.inf)) == 0x7E


def test_prune_density_is_half():
    rng = np.random.default_rng(0)
    w = orc.prune_paired_4of8(rng.standard_normal((2, 16, 64)).astype(np.float32))
    assert orc.is_paired_4of8(w)
    assert (w == 0).mean() == 0.5
    assert not orc.is_paired_4of8(rng.standard_normal((2, 16, 64)).astype(np.float32))


def test_e2m1_rne_ties_go_to_even():
    x = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.75, -0.1, -0.0, 0.26, 5.01], np.float32)
    want = np.array([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -1.0, -0.0, -0.0, 0.5, 6.0], np.float32)
    codes = orc.f32_to_e2m1_code_rne(x)
    got = orc.e2m1_code_to_f32(codes)
    assert np.array_equal(got, want)
    assert codes[9] == 8 and codes[10] == 8  # the sign survives on zero


def test_interleave_permutation_known_answer():
    # tests/test_swiglu_epilogue.py:96-101
    perm = orc.interleave_gate_up_rows(128)
    assert perm.shape == (256,)
    assert list(perm[:32]) == list(range(32)) and list(perm[32:64]) == list(range(128, 160))
    assert list(perm[64:96]) == list(range(32, 64)) and sorted(perm) == list(range(256))
    with pytest.raises(ValueError):
        orc.interleave_gate_up_rows(96)


def test_sf_layout_closed_form():
    rows, k, g = 200, 32 * 6, 3
    assert orc.sf_numel(rows, k, g) == 3 * 256 * 8
    nat = (np.arange(g * rows * 6) % 251).astype(np.uint8).reshape(g, rows, 6)
    sw = orc.swizzle_sf(nat, 0)
    assert np.array_equal(orc.unswizzle_sf(sw, g, rows, k), nat)
    # row 33, kb 5, group 1: atom (1*2+0)*2+1 = 5 -> 2560 + 1*16 + 1*4 + 1
    assert orc.sf_offset(33, 5, 1, rows, k) == 5 * 512 + 16 + 4 + 1
    offs = orc.sf_offset(*np.meshgrid(np.arange(rows), np.arange(6), np.arange(g), indexing="ij"), rows, k)
    assert len(np.unique(offs)) == offs.size


def test_quant_act_fill_count_and_scale_path():
    # exact count of benign bytes: numel - sum(counts) * KB (tests/test_ops.py:192-225)
    rng = np.random.default_rng(1)
    E, max_n, K = 3, 70, 160
    x = orc.f32_to_bf16_bits(rng.standard_normal((E, max_n, K)).astype(np.float32))
    counts = np.array([70, 0, 13], np.int32)
    b_act, valid, sfb = orc.quant_act(x, np.ones(1, np.float32), counts)
    n_quant = int(counts.sum()) * (K // 32)
    written = orc.unswizzle_sf(sfb, E, max_n, K)[valid]
    assert sfb.size == orc.sf_numel(max_n, K, E)
    assert (sfb == 0x38).sum() >= sfb.size - n_quant
    assert (sfb != 0).all()
    assert written.size == n_quant
    # dequantised activations stay within the 4-bit noise floor
    dq = orc.dequant_act(b_act, sfb, max_n, K)
    xr = orc.bf16_bits_to_f32(x)
    rel = np.linalg.norm((dq - xr)[valid]) / np.linalg.norm(xr[valid])
    assert 0.02 < rel < 0.3
    # an all-zero block quantizes to scale ue4m3(g) and zero codes; zero gscale gives scale 0 and zero codes
    z = np.zeros((1, 1, 32), np.uint16)
    b, _, s = orc.quant_act(z, np.array([2.0], np.float32), np.array([1], np.int32))
    assert s[0] == orc.f32_to_e4m3_bits(np.float32(2.0)) and not b.any()
    b, _, s = orc.quant_act(x[:1, :1, :32], np.array([1e-6], np.float32), np.array([1], np.int32))
    assert s[0] == 0 and not (b & 0x77).any()


def test_compress_roundtrip_and_shapes():
    rng = np.random.default_rng(2)
    E, M, K = 2, 130, 320
    w = orc.prune_paired_4of8(rng.standard_normal((E, M, K)).astype(np.float32))
    w[0, 3, 8:16] = 0  # all-zero chunk
    w[0, 4, 16:24] = 0
    w[0, 4, 22] = 1.0  # single pair at index 3
    w[0, 5, 24:32] = 0
    w[0, 5, 26] = -2.0  # single pair at index 1
    packed, sf, dq = orc.quantize_weight(w)
    a_comp, e_meta, sfa = orc.compress(packed, sf, K)
    MA, KA, ME, KE = orc.physical_dims(M, K)
    assert a_comp.shape == (E, M, 80) and (MA, KA) == (130, 160)
    assert e_meta.shape == (E, 256, 32) and (ME, KE) == (256, 32)
    assert sfa.size == orc.sf_numel(M, K, E)
    dense = orc.decompress(a_comp, e_meta, M, K)
    assert np.array_equal(orc.unpack_e2m1(dense), orc.unpack_e2m1(packed))
    assert np.array_equal(orc.unswizzle_sf(sfa, E, M, K), sf)
    # aligned shapes: exactly half the dense bytes (tests/test_ops.py:82-90)
    p2 = np.zeros((1, 128, 128), np.uint8)
    a2, e2, _ = orc.compress(p2, np.zeros((1, 128, 8), np.uint8), 256)
    assert a2.size * 2 == p2.size and e2.shape == (1, 128, 16)


def test_scatter_matches_gather_then_quant():
    rng = np.random.default_rng(3)
    T, K, E, cap, topk = 40, 64, 4, 8, 2
    a1 = orc.f32_to_bf16_bits(rng.standard_normal((T, K)).astype(np.float32))
    ids = np.stack([rng.permutation(6)[:topk] for _ in range(T)])  # experts 0..5, local = 1..4
    flat_tok, dest, counts = orc.make_dispatch(ids, 1, E, cap)
    assert counts.max() == cap and (dest == E * cap).any()
    b_act, written, sfb = orc.scatter_quant_act(a1, flat_tok, dest, None, np.ones(E, np.float32), E, cap)
    assert np.array_equal(written.sum(1), counts)
    x = np.zeros((E, cap, K), np.uint16)
    keep = dest != E * cap
    x.reshape(E * cap, K)[dest[keep]] = a1[flat_tok[keep]]
    b2, valid2, sfb2 = orc.quant_act(x, np.ones(E, np.float32), counts)
    assert np.array_equal(written, valid2) and np.array_equal(b_act, b2) and np.array_equal(sfb, sfb2)
    assert (sfb != 0).all()


def test_group_mm_reference_on_plumbing_config():
    rng = np.random.default_rng(4)
    E, M, K, max_n = 2, 64, 128, 12
    w = orc.prune_paired_4of8(rng.standard_normal((E, M, K)).astype(np.float32))
    packed, sf, dq = orc.quantize_weight(w)
    x = orc.f32_to_bf16_bits(rng.standard_normal((E, max_n, K)).astype(np.float32))
    counts = np.array([12, 5], np.int32)
    b_act, valid, sfb = orc.quant_act(x, np.ones(1, np.float32), counts)
    out = orc.group_mm(dq, b_act, sfb, np.ones(E, np.float32), counts, sentinel=-12345.0)
    assert (out[1, 5:] == -12345.0).all()
    want = np.einsum("etk,emk->etm", orc.bf16_bits_to_f32(x), w)
    rel = orc.rel_frobenius(out[valid], want[valid])
    assert 0.02 < rel < 0.3
