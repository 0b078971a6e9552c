"""Seeded random sweep over shapes, counts and tile variants: group_mm against the oracle (relative Frobenius
error, untouched padding, device status word) and the fused gate_up op against the unfused chain (bytes).  The
shapes deliberately mix M and K tails, empty and full experts, one-tile and many-tile problems."""
import numpy as np
import pytest
import torch

from oracle import paired_nvfp4_oracle as orc
from helpers import bf16_tensor, dev, make_acts, make_weights

pytestmark = pytest.mark.gpu

SENTINEL = -12352.0


@pytest.mark.parametrize("seed", [101, 102, 103])
def test_group_mm_random_shapes(seed):
    import paired_nvfp4_kernels as pnk
    from paired_nvfp4_kernels import ops as pyops
    ops = torch.ops.paired_nvfp4
    rng = np.random.default_rng(seed)
    for it in range(20):
        E = int(rng.integers(1, 9))
        M = int(rng.choice([128, 200, 256, 384, 640, 1024]))
        K = int(rng.choice([32, 96, 256, 320, 512, 768, 1024, 2048, 2560]))
        max_n = int(rng.choice([8, 16, 24, 33, 64, 100, 128, 200, 257, 512, 700]))
        counts = rng.integers(0, max_n + 1, E).astype(np.int32)
        if rng.random() < 0.3:
            counts[rng.integers(0, E)] = max_n
        cfg = int(rng.integers(0, 9))
        packed, sf, w_dq = make_weights(E, M, K, 1000 * seed + it, 1.0)
        x = make_acts(E, max_n, K, 2000 * seed + it)
        g = np.ones(1, np.float32)
        al = np.linspace(0.5, 2.0, E).astype(np.float32)
        a_comp, e_meta, sfa = ops.compress(dev(packed), dev(sf), K)
        b_act, sfb = ops.quant_act(bf16_tensor(x), dev(g), dev(counts), M)
        out = torch.full((E, max_n, M), SENTINEL, dtype=torch.bfloat16, device="cuda")
        name = pnk.group_mm_configs()[cfg]
        cm, cn = pnk.valid_clusters(name)[0]
        ops.group_mm(out, a_comp, e_meta, sfa, b_act, sfb, dev(al), dev(counts), M, K, cfg, cm, cn)
        torch.cuda.synchronize()
        case = dict(E=E, M=M, K=K, max_n=max_n, counts=counts.tolist(), cfg=cfg)
        assert pyops.group_mm_device_status() == 0, case
        got = out.float().cpu().numpy()
        ob, valid, osfb = orc.quant_act(x, g, counts)
        want = orc.group_mm(w_dq, ob, osfb, al, counts, sentinel=SENTINEL)
        assert (got[~valid] == SENTINEL).all(), case
        if valid.any():
            assert orc.rel_frobenius(got[valid], want[valid]) <= 5e-3, case


@pytest.mark.parametrize("seed", [201, 202])
def test_fused_gate_up_random_shapes(seed):
    import paired_nvfp4_kernels as pnk
    from paired_nvfp4_kernels import ops as pyops
    ops = torch.ops.paired_nvfp4
    rng = np.random.default_rng(seed)
    for it in range(15):
        big = it % 5 == 0
        E = int(rng.integers(1, 9))
        N = 1024 if big else int(rng.choice([64, 128, 192, 512]))
        M = 2 * N
        K = int(rng.choice([32, 256, 320, 768, 1024, 2048]))
        max_n = 1024 if big else int(rng.choice([8, 16, 24, 33, 64, 100, 200, 257]))
        counts = rng.integers(0, max_n + 1, E).astype(np.int32)
        fcfg = int(rng.integers(0, 6))
        act = ["silu", "situ"][int(rng.integers(0, 2))]
        beta, lb = (1.702, 1.0) if act == "situ" else (1.0, -1.0)
        packed, sf, _ = make_weights(E, M, K, 3000 * seed + it, 1.0)
        perm = pnk.interleave_gate_up_rows(N).numpy()
        packed, sf = np.ascontiguousarray(packed[:, perm]), np.ascontiguousarray(sf[:, perm])
        x = make_acts(E, max_n, K, 4000 * seed + it)
        g = np.ones(1, np.float32)
        al = np.linspace(0.5, 2.0, E).astype(np.float32)
        g2 = rng.uniform(0.5, 4.0, E).astype(np.float32)
        a_comp, e_meta, sfa = ops.compress(dev(packed), dev(sf), K)
        b_act, sfb = ops.quant_act(bf16_tensor(x), dev(g), dev(counts), M)
        name = ops.group_mm_swiglu_configs()[fcfg]
        cm = 2 if "2sm" in name else 1
        fb, fsf = ops.group_mm_swiglu_quant(a_comp, e_meta, sfa, b_act, sfb, dev(al), dev(counts), dev(g2), M, K, fcfg,
                                            cm, 1, act, beta, lb)
        base = {0: 6, 1: 4, 2: 5, 3: 0, 4: 2, 5: 1}[fcfg]
        out = torch.zeros((E, max_n, M), dtype=torch.bfloat16, device="cuda")
        ops.group_mm(out, a_comp, e_meta, sfa, b_act, sfb, dev(al), dev(counts), M, K, base, cm, 1)
        y = ops.gated_act(out, True, act, beta, lb)
        rb, rsf = ops.quant_act(y, dev(g2), dev(counts), K)
        torch.cuda.synchronize()
        case = dict(E=E, N=N, K=K, max_n=max_n, counts=counts.tolist(), fcfg=fcfg, act=act)
        assert pyops.group_mm_device_status() == 0, case
        valid = torch.arange(max_n, device="cuda")[None, :] < dev(counts)[:, None]
        assert torch.equal(fsf, rsf), case
        assert torch.equal(fb[valid], rb[valid]), case
