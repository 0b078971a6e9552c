"""GPU parity of the routing-side ops against the oracle: dispatch_plan (int32 / int64 ids, EP ranks,
undersized cap, many local experts, single- and multi-chunk plans), planned scatter == flat scatter bytes,
FP4-on-the-wire pair == scatter-quant with a shared scale, finalize with NaN-poisoned dropped rows
(the cases of the reference's tests/test_moe_routing.py:26-198)."""
import numpy as np
import pytest
import torch

from oracle import paired_nvfp4_oracle as orc
from helpers import bf16_tensor, bf16_bits, u8, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import paired_nvfp4_kernels  # noqa: F401
    return torch.ops.paired_nvfp4


PLAN_CASES = [
    # T, topk, E_total, rank, world, cap, dtype
    (1, 8, 128, 0, 1, 4, torch.int64),
    (16, 2, 8, 0, 1, 16, torch.int32),
    (300, 4, 64, 1, 4, 64, torch.int64),        # one EP rank of four
    (1024, 8, 128, 0, 1, 32, torch.int32),      # 8192 routings: 8 chunks, cap too small -> drops
    (4096, 8, 256, 3, 8, 256, torch.int64),     # EP rank 3 of 8
    (2000, 6, 512, 0, 1, 40, torch.int32),      # 512 local experts
    (128, 8, 8, 0, 1, 2000, torch.int64),       # few experts, large cap
    (0, 2, 8, 0, 1, 4, torch.int32),            # no tokens
]


def route(T, topk, Etot, seed):
    rng = np.random.default_rng(seed)
    if T == 0:
        return np.zeros((0, topk), np.int64)
    return np.argsort(-rng.standard_normal((T, Etot)), axis=1)[:, :topk].astype(np.int64)


@pytest.mark.parametrize("T,topk,Etot,rank,world,cap,dtype", PLAN_CASES)
def test_dispatch_plan(ops, T, topk, Etot, rank, world, cap, dtype):
    E = Etot // world
    ids = route(T, topk, Etot, T + Etot)
    counts, rd, st, sr = ops.dispatch_plan(torch.from_numpy(ids).to(dtype).cuda(), E * rank, E, cap)
    torch.cuda.synchronize()
    oc, ord_, ost, osr = orc.dispatch_plan(ids, E * rank, E, cap)
    assert np.array_equal(counts.cpu().numpy(), oc)
    assert np.array_equal(rd.cpu().numpy(), ord_)
    assigned = ost >= 0
    assert np.array_equal(st.cpu().numpy()[assigned], ost[assigned])
    assert np.array_equal(sr.cpu().numpy()[assigned], osr[assigned])


def test_plan_replays_in_a_cuda_graph(ops):
    T, topk, Etot, cap = 512, 4, 32, 96
    ids_a, ids_b = route(T, topk, Etot, 1), route(T, topk, Etot, 2)
    ids = torch.from_numpy(ids_a).cuda()
    ops.dispatch_plan(ids, 0, Etot, cap)   # warm up outside capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        outs = ops.dispatch_plan(ids, 0, Etot, cap)
    for src in (ids_b, ids_a):
        ids.copy_(torch.from_numpy(src))
        g.replay()
        torch.cuda.synchronize()
        oc, ord_, _, _ = orc.dispatch_plan(src, 0, Etot, cap)
        assert np.array_equal(outs[0].cpu().numpy(), oc) and np.array_equal(outs[1].cpu().numpy(), ord_)


@pytest.mark.parametrize("T,K,Etot,rank,world,cap,topk,with_w", [
    (64, 256, 8, 0, 1, 16, 2, False), (300, 1024, 16, 1, 2, 64, 4, True), (33, 96, 4, 0, 1, 4, 2, True),
    (2048, 2048, 128, 0, 1, 64, 8, True)])
def test_planned_scatter_equals_flat_scatter_and_oracle(ops, T, K, Etot, rank, world, cap, topk, with_w):
    E = Etot // world
    rng = np.random.default_rng(T + K)
    ids = route(T, topk, Etot, K)
    a1 = orc.f32_to_bf16_bits(rng.standard_normal((T, K)).astype(np.float32))
    w = rng.uniform(0.05, 1.0, T * topk).astype(np.float32) if with_w else None
    g = rng.uniform(1.0, 20.0, E).astype(np.float32)
    a1_t, g_t, w_t = bf16_tensor(a1), dev(g), (dev(w) if with_w else None)
    counts, rd, st, sr = ops.dispatch_plan(torch.from_numpy(ids).cuda(), E * rank, E, cap)
    b_p, sf_p = ops.scatter_quant_act_planned(a1_t, st, sr, w_t, g_t, counts, cap)
    flat_tok, dest, _ = orc.make_dispatch(ids, E * rank, E, cap)
    b_f, sf_f = ops.scatter_quant_act(a1_t, dev(flat_tok), dev(dest), w_t, g_t, counts, cap)
    torch.cuda.synchronize()
    oc, _, ost, osr = orc.dispatch_plan(ids, E * rank, E, cap)
    ob, valid, osfb = orc.scatter_quant_act_planned(a1, ost, osr, w, g, oc, cap)
    assert np.array_equal(u8(b_p)[valid], ob[valid]) and np.array_equal(u8(sf_p), osfb)
    assert np.array_equal(u8(b_p)[valid], u8(b_f)[valid]) and np.array_equal(u8(sf_p), u8(sf_f))


@pytest.mark.parametrize("T,K,E,cap,topk", [(500, 512, 16, 48, 4), (70, 96, 4, 20, 2), (120, 7168, 8, 40, 3),
                                            (64, 1056, 2, 130, 2)])
def test_fp4_wire_pair_equals_scatter_quant(ops, T, K, E, cap, topk):
    rng = np.random.default_rng(9)
    ids = route(T, topk, E, 9)
    a1 = orc.f32_to_bf16_bits(rng.standard_normal((T, K)).astype(np.float32))
    g = np.array([7.5], np.float32)
    a1_t, g_t = bf16_tensor(a1), dev(g)
    counts, rd, st, sr = ops.dispatch_plan(torch.from_numpy(ids).cuda(), 0, E, cap)
    q, qsf = ops.quant_rows(a1_t, g_t)
    b_w, sf_w = ops.scatter_fp4_planned(q, qsf, st, counts, cap)
    b_s, sf_s = ops.scatter_quant_act_planned(a1_t, st, sr, None, g_t, counts, cap)
    torch.cuda.synchronize()
    oq, oqsf = orc.quant_rows(a1, g)
    assert np.array_equal(u8(q), oq) and np.array_equal(u8(qsf), oqsf)
    valid = np.arange(cap)[None, :] < counts.cpu().numpy()[:, None]
    assert np.array_equal(u8(b_w)[valid], u8(b_s)[valid]) and np.array_equal(u8(sf_w), u8(sf_s))
    assert (u8(sf_w) != 0).all()


@pytest.mark.parametrize("with_w", [False, True])
def test_finalize_bit_identical_with_poisoned_padding(ops, with_w):
    T, K, E, cap, topk = 200, 1032, 8, 40, 3
    rng = np.random.default_rng(4)
    ids = route(T, topk, 12, 4)   # experts 8..11 are not local -> dropped routings
    counts, rd, st, sr = ops.dispatch_plan(torch.from_numpy(ids).cuda(), 0, E, cap)
    fused = rng.standard_normal((E * cap, K)).astype(np.float32)
    fb = orc.f32_to_bf16_bits(fused)
    used = np.zeros(E * cap, bool)
    rdn = rd.cpu().numpy()
    used[rdn[rdn >= 0]] = True
    fb[~used] = 0x7FC0            # NaN in every row no routing points at
    w = rng.uniform(0.0, 1.0, (T, topk)).astype(np.float32) if with_w else None
    out = torch.zeros(T, K, dtype=torch.bfloat16, device="cuda")
    ops.moe_finalize(out, bf16_tensor(fb).view(E, cap, K), rd, dev(w) if with_w else None)
    torch.cuda.synchronize()
    want = orc.moe_finalize(fb, rdn, w)
    assert np.array_equal(bf16_bits(out), want)
    assert not np.isnan(orc.bf16_bits_to_f32(want)).any()


@pytest.mark.parametrize("rows,width,dtype", [(37, 16, torch.uint8), (200, 224, torch.uint8), (65, 512, torch.bfloat16)])
def test_gather_rows(rows, width, dtype):
    import paired_nvfp4_kernels  # noqa: F401
    ops = torch.ops.paired_nvfp4
    g = torch.Generator(device="cpu").manual_seed(rows + width)
    src = torch.randint(0, 255, (rows, width), generator=g, dtype=torch.uint8)
    src = (src.to(torch.float32) - 128).to(dtype).cuda() if dtype != torch.uint8 else src.cuda()
    idx = torch.randint(-1, rows, (3 * rows + 5,), generator=g, dtype=torch.int32).cuda()
    got = ops.gather_rows(src, idx)
    want = src[idx.clamp(min=0).long()]
    want[idx < 0] = 0
    assert torch.equal(got, want)
    assert ops.gather_rows(src, idx[:0]).shape == (0, width)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ops.gather_rows(src[:, :4].contiguous(), idx)


@pytest.mark.parametrize("rows,width,dtype", [(37, 16, torch.uint8), (203, 7168, torch.bfloat16), (8, 264, torch.bfloat16)])
def test_zero_rows(rows, width, dtype):
    import paired_nvfp4_kernels  # noqa: F401
    ops = torch.ops.paired_nvfp4
    g = torch.Generator(device="cpu").manual_seed(rows + width)
    dst = torch.randint(1, 255, (rows, width), generator=g, dtype=torch.uint8).to(dtype).cuda()
    flags = torch.randint(-1, 3, (rows,), generator=g, dtype=torch.int32).cuda()
    want = dst.clone()
    want[flags < 0] = 0
    ops.zero_rows(dst, flags)
    assert torch.equal(dst, want)
    ops.zero_rows(dst[:0], flags[:0])
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ops.zero_rows(dst[:, :4].contiguous(), flags)


def test_zero_rows_parts():
    import paired_nvfp4_kernels  # noqa: F401
    ops = torch.ops.paired_nvfp4
    g = torch.Generator(device="cpu").manual_seed(5)
    parts = [torch.randint(1, 255, (21, 64), generator=g, dtype=torch.uint8).cuda() for _ in range(3)]
    flags = torch.randint(-1, 3, (63,), generator=g, dtype=torch.int32).cuda()
    want = torch.cat(parts).clone()
    want[flags < 0] = 0
    ops.zero_rows_parts(parts, flags)
    assert torch.equal(torch.cat(parts), want)
