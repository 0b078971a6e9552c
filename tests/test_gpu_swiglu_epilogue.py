"""GPU parity of the fused GEMM1 + gated activation + requantise op: byte-identical to the unfused chain
(group_mm on the interleaved W13, then silu_mul_quant_act(interleaved=True)), for every fused tactic, both
activations, ragged counts and partial tiles (the reference's tests/test_swiglu_epilogue.py:28-153)."""
import numpy as np
import pytest
import torch

from oracle import paired_nvfp4_oracle as orc
from helpers import bf16_tensor, bf16_bits, u8, dev, make_acts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pnk():
    import paired_nvfp4_kernels
    return paired_nvfp4_kernels


def build(N, K, E, max_n, counts, seed):
    ops = torch.ops.paired_nvfp4
    rng = np.random.default_rng(seed)
    w13 = orc.prune_paired_4of8(rng.standard_normal((E, 2 * N, K)).astype(np.float32))
    perm = orc.interleave_gate_up_rows(N)
    packed, sf, w_dq = orc.quantize_weight(w13[:, perm])
    a_comp, e_meta, sfa = ops.compress(dev(packed), dev(sf), K)
    x = make_acts(E, max_n, K, seed + 1)
    cnt = np.asarray(counts, np.int32)
    b_act, sfb = ops.quant_act(bf16_tensor(x), dev(np.ones(1, np.float32)), dev(cnt), 2 * N)
    alphas = np.linspace(0.5, 1.5, E).astype(np.float32)
    return dict(a_comp=a_comp, e_meta=e_meta, sfa=sfa, b_act=b_act, sfb=sfb, al=dev(alphas), cnt=dev(cnt),
                counts=cnt, w_dq=w_dq)


CASES = [
    # N, K, E, max_n, counts
    (128, 256, 2, 40, [40, 7]),
    (768, 512, 3, 300, [300, 0, 129]),      # several token tiles, an empty expert
    (64, 128, 1, 16, [16]),                 # one 128-row tile, small-batch path
    (2048, 1024, 2, 16, [9, 16]),           # decode-like
    (192, 768, 2, 130, [130, 64]),
    (384, 1536, 9, 520, [520, 0, 300, 1, 257, 128, 519, 33, 256]),   # many ragged experts, several token tiles each
    (128, 1280, 6, 330, [257, 320, 330, 64, 321, 289]),   # narrow tail tiles (two M units per item) over one M unit
    (512, 256, 4, 580, [576, 300, 577, 290]),             # ... over four M units, a one-stage K loop
    (128, 3072, 3, 330, [257, 320, 64]),                  # ... with 512-K stages
]


@pytest.mark.parametrize("N,K,E,max_n,counts", CASES)
@pytest.mark.parametrize("act,beta,lbeta", [("silu", 1.0, -1.0), ("situ", 1.702, 1.0), ("situ", 2.0, -1.0)])
def test_fused_equals_unfused_bytes(pnk, N, K, E, max_n, counts, act, beta, lbeta):
    ops = torch.ops.paired_nvfp4
    o = build(N, K, E, max_n, counts, seed=N + K)
    g2 = dev(np.linspace(3.0, 40.0, E).astype(np.float32))
    valid = np.arange(max_n)[None, :] < o["counts"][:, None]
    names = ops.group_mm_swiglu_configs()
    # the reference's four names and ids, then this build's addition
    assert names[:4] == ["fused_2sm_256x64_k512", "fused_2sm_256x64", "fused_1sm_128x64", "fused_2sm_256x128"]
    assert names[4:] == ["fused_1sm_128x128", "fused_2sm_256x256"]
    # unfused chain on the same interleaved weight; the GEMM tile choice does not change a single bit of its
    # accumulation order per output element, but compare like with like anyway
    base_cfg = {0: 6, 1: 4, 2: 5, 3: 0, 4: 2, 5: 1}
    for cid, cm, cn in pnk.fused_swiglu_tactics():
        out1 = torch.zeros(E, max_n, 2 * N, dtype=torch.bfloat16, device="cuda")
        ops.group_mm(out1, o["a_comp"], o["e_meta"], o["sfa"], o["b_act"], o["sfb"], o["al"], o["cnt"], 2 * N, K,
                     base_cfg[cid], cm, cn)
        want_b, want_sf = ops.silu_mul_quant_act(out1, g2, o["cnt"], N, True, act, beta, lbeta)
        got_b, got_sf = ops.group_mm_swiglu_quant(o["a_comp"], o["e_meta"], o["sfa"], o["b_act"], o["sfb"], o["al"],
                                                  o["cnt"], g2, 2 * N, K, cid, cm, cn, act, beta, lbeta)
        torch.cuda.synchronize()
        assert tuple(got_b.shape) == (E, max_n, N // 2)
        assert np.array_equal(u8(got_b)[valid], u8(want_b)[valid]), f"codes differ for tactic {(cid, cm, cn)}"
        assert np.array_equal(u8(got_sf), u8(want_sf)), f"scales differ for tactic {(cid, cm, cn)}"
        assert (u8(got_sf) != 0).all()


def test_fused_argument_checks(pnk):
    ops = torch.ops.paired_nvfp4
    o = build(64, 128, 1, 16, [16], seed=1)
    g2 = dev(np.ones(1, np.float32))
    args = (o["a_comp"], o["e_meta"], o["sfa"], o["b_act"], o["sfb"], o["al"], o["cnt"], g2, 128, 128)
    with pytest.raises(RuntimeError, match="activation must be"):
        ops.group_mm_swiglu_quant(*args, 0, 2, 1, "gelu", 1.0, -1.0)
    with pytest.raises(RuntimeError, match="beta must be positive"):
        ops.group_mm_swiglu_quant(*args, 0, 2, 1, "situ", -1.0, -1.0)
    with pytest.raises(RuntimeError, match="even cluster_m"):
        ops.group_mm_swiglu_quant(*args, 0, 1, 1, "silu", 1.0, -1.0)
