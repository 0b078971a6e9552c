"""GPU parity: the three activation quantizers and compress against the CPU oracle, bit for bit.
All calls go through torch.ops.paired_nvfp4.* -> ctypes -> the C ABI of libpaired_nvfp4_b200.so."""
import numpy as np
import pytest
import torch

from oracle import paired_nvfp4_oracle as orc
from helpers import bf16_tensor, bf16_bits, u8, dev, make_acts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import paired_nvfp4_kernels  # noqa: F401  registers torch.ops.paired_nvfp4
    return torch.ops.paired_nvfp4


def check_quant(ops_out, oracle_out):
    b_act, sfb = ops_out
    ob, valid, osfb = oracle_out
    got_b = u8(b_act)
    assert got_b.shape == ob.shape
    assert np.array_equal(got_b[valid], ob[valid]), "e2m1 codes differ"
    assert np.array_equal(u8(sfb), osfb), "scale buffer differs"


QUANT_CASES = [
    # E, max_n, K, counts, per-expert gscale
    (8, 256, 1024, "rand", True),      # the reference's CPU-plumbing config
    (3, 70, 160, [70, 0, 13], False),  # ragged: K/32 = 5 (K-slop in the scale atoms), empty expert
    (2, 1, 32, [1, 1], True),          # minimum sizes
    (4, 130, 96, [130, 129, 1, 0], True),   # two row atoms, KB = 3
    (8, 16, 4096, "rand", True),       # decode-shaped
    (2, 300, 7168, [300, 77], False),
]


@pytest.mark.parametrize("E,max_n,K,counts,gpe", QUANT_CASES)
def test_quant_act_bit_exact(ops, E, max_n, K, counts, gpe):
    rng = np.random.default_rng(E * 1000 + K)
    x = make_acts(E, max_n, K, seed=K + max_n, scale=1.0)
    cnt = rng.integers(1, max_n + 1, E).astype(np.int32) if counts == "rand" else np.array(counts, np.int32)
    g = (rng.uniform(0.5, 300.0, E) if gpe else np.array([2.5])).astype(np.float32)
    out = ops.quant_act(bf16_tensor(x), dev(g), dev(cnt), 128)
    torch.cuda.synchronize()
    check_quant(out, orc.quant_act(x, g, cnt))
    # exact number of benign bytes: numel - sum(counts) * KB, unless a quantized scale is 0x38 itself
    sfb = u8(out[1])
    assert sfb.size == orc.sf_numel(max_n, K, E)
    assert (sfb == 0x38).sum() >= sfb.size - int(cnt.sum()) * (K // 32)
    assert (sfb != 0).all() or g.min() < 1e-3


def test_quant_act_ties_zero_blocks_saturation_and_zero_scale(ops):
    E, max_n, K = 2, 8, 256
    x = np.zeros((E, max_n, K), np.float32)
    # block amax 6 -> scale 1.0 -> values sit exactly on e2m1 midpoints
    mid = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0,
                    -6.0, 0.0, -0.0, 0.1, -0.1, 0.24, 0.26, 5.9, 7.0, 3.0, 4.0, 2.0, 1.5, 1.0, 0.5, 6.0, -6.0],
                   np.float32)
    x[0, 0, :32] = mid
    x[0, 1, 32:64] = mid * 2.0         # scale 2.0
    x[0, 2, :32] = 3.0e38              # huge -> scale saturates at 448
    x[0, 3, :32] = 1e-30               # tiny -> scale rounds to 0 -> all-zero codes
    x[0, 4] = np.linspace(-8, 8, K)
    x[1] = np.random.default_rng(7).standard_normal((max_n, K)) * 100
    xb = orc.f32_to_bf16_bits(x)
    cnt = np.array([8, 5], np.int32)
    for g in (np.array([1.0], np.float32), np.array([1.0, 1e-6], np.float32), np.array([448.0 * 6 / 7.0, 0.001], np.float32)):
        out = ops.quant_act(bf16_tensor(xb), dev(g), dev(cnt), 64)
        torch.cuda.synchronize()
        check_quant(out, orc.quant_act(xb, g, cnt))


GATED_CASES = [
    # E, max_n, N, counts, interleaved, activation, beta, linear_beta
    (4, 64, 256, [64, 1, 0, 33], False, "silu", 1.0, -1.0),
    (4, 64, 256, [64, 1, 0, 33], True, "silu", 1.702, 1.0),      # beta / linear_beta ignored for silu
    (2, 40, 768, [40, 7], False, "situ", 1.702, 1.0),
    (2, 40, 768, [40, 7], True, "situ", 1.702, -1.0),
    (3, 130, 96, [130, 2, 64], True, "silu", 1.0, -1.0),
    (8, 16, 14336, "rand", False, "silu", 1.0, -1.0),            # Mixtral decode shape
]


@pytest.mark.parametrize("E,max_n,N,counts,inter,act,beta,lbeta", GATED_CASES)
def test_silu_mul_quant_act(ops, E, max_n, N, counts, inter, act, beta, lbeta):
    rng = np.random.default_rng(N + max_n)
    x2 = orc.f32_to_bf16_bits((rng.standard_normal((E, max_n, 2 * N)) * 2.0).astype(np.float32))
    cnt = rng.integers(1, max_n + 1, E).astype(np.int32) if counts == "rand" else np.array(counts, np.int32)
    g = rng.uniform(1.0, 50.0, E).astype(np.float32)
    x2_t = bf16_tensor(x2)
    fused = ops.silu_mul_quant_act(x2_t, dev(g), dev(cnt), 128, inter, act, beta, lbeta)
    # (1) byte identity of the fused op with the unfused chain on the device
    y = ops.gated_act(x2_t, inter, act, beta, lbeta)
    chain = ops.quant_act(y, dev(g), dev(cnt), 128)
    torch.cuda.synchronize()
    valid = np.arange(max_n)[None, :] < cnt[:, None]
    assert np.array_equal(u8(fused[0])[valid], u8(chain[0])[valid])
    assert np.array_equal(u8(fused[1]), u8(chain[1]))
    # (2) the quantization tail against the oracle, given the device's activation values
    y_bits = bf16_bits(y)
    kind = orc.ACT_SITU if act == "situ" else orc.ACT_SILU
    ob, ovalid, osfb, _ = orc.silu_mul_quant_act(x2, g, cnt, inter, kind, beta, lbeta, act_bits=y_bits)
    assert np.array_equal(u8(fused[0])[ovalid], ob[ovalid]) and np.array_equal(u8(fused[1]), osfb)
    # (3) the activation itself against the float32 numpy restatement: CUDA's expf / tanhf may differ
    #     from numpy's in the last place, which can move a bf16 rounding by one ulp on a few elements
    gate, up = orc.split_gate_up(orc.bf16_bits_to_f32(x2), inter)
    want = orc.f32_to_bf16_bits(orc.gated_act(gate, up, kind, beta, lbeta))
    dist = orc.bf16_ulp_distance(y_bits, want)
    assert dist.max() <= 1, f"activation differs by {dist.max()} bf16 ulp"
    assert (dist == 0).mean() > 0.995


def test_gated_activation_argument_checks(ops):
    x2 = torch.zeros(1, 4, 128, dtype=torch.bfloat16, device="cuda")
    g = torch.ones(1, device="cuda")
    c = torch.ones(1, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="activation must be"):
        ops.silu_mul_quant_act(x2, g, c, 64, False, "gelu", 1.0, -1.0)
    with pytest.raises(RuntimeError, match="beta must be positive"):
        ops.silu_mul_quant_act(x2, g, c, 64, False, "situ", 0.0, -1.0)


SCATTER_CASES = [
    # T, K, E_total, first, E_local, cap, topk, with_weights
    (64, 256, 8, 0, 8, 16, 2, False),
    (200, 1024, 16, 4, 8, 32, 4, True),      # one EP rank: most routings are non-local
    (33, 96, 4, 0, 4, 4, 2, True),           # over capacity, KB = 3
    (4096, 2048, 128, 0, 128, 64, 8, True),  # Qwen3-shaped routing, small cap -> many drops
]


@pytest.mark.parametrize("T,K,Etot,first,E,cap,topk,with_w", SCATTER_CASES)
def test_scatter_quant_act(ops, T, K, Etot, first, E, cap, topk, with_w):
    rng = np.random.default_rng(T + K)
    a1 = orc.f32_to_bf16_bits(rng.standard_normal((T, K)).astype(np.float32))
    logits = rng.standard_normal((T, Etot))
    ids = np.argsort(-logits, axis=1)[:, :topk]
    flat_tok, dest, counts = orc.make_dispatch(ids, first, E, cap)
    w = rng.uniform(0.05, 1.0, T * topk).astype(np.float32) if with_w else None
    g = rng.uniform(1.0, 20.0, E).astype(np.float32)
    b_act, sfb = ops.scatter_quant_act(bf16_tensor(a1), dev(flat_tok), dev(dest), dev(w) if with_w else None,
                                       dev(g), dev(counts), cap)
    torch.cuda.synchronize()
    assert tuple(b_act.shape) == (E, cap, K // 2)
    ob, written, osfb = orc.scatter_quant_act(a1, flat_tok, dest, w, g, E, cap)
    assert np.array_equal(u8(b_act)[written], ob[written])
    assert np.array_equal(u8(sfb), osfb)
    assert (u8(sfb) != 0).all()


COMPRESS_CASES = [(2, 256, 512, 1), (3, 130, 320, 2), (1, 128, 256, 3), (8, 2048, 1024, 4), (2, 64, 96, 5)]


@pytest.mark.parametrize("E,M,K,seed", COMPRESS_CASES)
def test_compress_bytes(ops, E, M, K, seed):
    rng = np.random.default_rng(seed)
    w = orc.prune_paired_4of8(rng.standard_normal((E, M, K)).astype(np.float32))
    # sprinkle the single-pair and empty-chunk corner cases
    w[0, 0, :8] = 0
    w[0, 1, :8] = 0
    w[0, 1, 6] = 1.0
    w[0, 2, :8] = 0
    w[0, 2, 3] = -1.0
    packed, sf, _ = orc.quantize_weight(w)
    packed[0, 3, 0] = 0x88   # negative zeros count as zero
    a_comp, e_meta, sfa = ops.compress(dev(packed), dev(sf), K)
    torch.cuda.synchronize()
    oa, oe, os_ = orc.compress(packed, sf, K)
    assert tuple(a_comp.shape) == oa.shape and tuple(e_meta.shape) == oe.shape and sfa.numel() == os_.size
    assert np.array_equal(u8(a_comp), oa)
    assert np.array_equal(u8(e_meta), oe)
    assert np.array_equal(u8(sfa), os_)
    if K % 64 == 0:
        assert a_comp.numel() * 2 == packed.size


def test_compress_rejects_per16_scales(ops):
    E, M, K = 1, 256, 256
    w_packed = torch.zeros(E, M, K // 2, dtype=torch.uint8, device="cuda")
    w_sf16 = torch.zeros(E, M, K // 16, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="ceil"):
        ops.compress(w_packed, w_sf16, K)


def test_silu_table_matches_direct_evaluation(ops):
    """SiLU goes through a 65536-entry table filled on the device; every possible gate value (all bf16 bit
    patterns, NaNs and infinities included) must give the same bits as evaluating the expression."""
    from paired_nvfp4_kernels import ops as pyops
    bits = np.arange(65536, dtype=np.uint16).reshape(2048, 32)
    rng = np.random.default_rng(7)
    for up_scale in (1.0, 37.5):
        up = orc.f32_to_bf16_bits((rng.standard_normal((2048, 32)) * up_scale).astype(np.float32))
        if up_scale == 1.0:
            up[:] = 0x3F80          # up = 1: the output is the table entry itself
        x2 = bf16_tensor(np.concatenate([bits, up], axis=1)[None])
        try:
            y_table = bf16_bits(ops.gated_act(x2))
            pyops.set_silu_table(False)
            y_direct = bf16_bits(ops.gated_act(x2))
        finally:
            pyops.set_silu_table(True)
        assert np.array_equal(y_table, y_direct)
