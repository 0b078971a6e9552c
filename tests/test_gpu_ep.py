"""Expert parallelism on two GPUs: the exchanged forward pass must give every rank, bit for bit, what one GPU
holding all experts computes for the same tokens (row placement inside an expert does not change a row's
result, and moe_finalize sums in top-k order).  Skipped on a single-GPU box."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for _p in (ROOT, os.path.join(ROOT, "grouped-sparse-gemm_b200"), os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

E, H, I, T, TOPK, CAP = 8, 512, 256, 96, 2, 64


def _weights(device):
    """Compressed W13 (gate/up rows interleaved) and W2 of all E experts, from a fixed seed."""
    import paired_nvfp4_kernels as pnk
    from paired_nvfp4_kernels import reference as wref
    ops = torch.ops.paired_nvfp4
    g = torch.Generator(device=device).manual_seed(2024)
    w13 = torch.randn((E, 2 * I, H), generator=g, device=device) * 0.05
    w2 = torch.randn((E, H, I), generator=g, device=device) * 0.05
    p13, s13, _ = wref.quantize_weight(wref.prune_paired_4of8(w13))
    perm = pnk.interleave_gate_up_rows(I, device=device)
    p13, s13 = p13[:, perm].contiguous(), s13[:, perm].contiguous()
    p2, s2, _ = wref.quantize_weight(wref.prune_paired_4of8(w2))
    return (p13, s13), (p2, s2)


def _tokens(rank, device):
    g = torch.Generator(device="cpu").manual_seed(77 + rank)
    x = torch.randn((T, H), generator=g).to(torch.bfloat16).to(device)
    ids = torch.stack([torch.randperm(E, generator=g)[:TOPK] for _ in range(T)]).to(device)
    w = torch.rand((T, TOPK), generator=g).to(device)
    return x, ids, w


def _ffn(ops, ep, w13, w2, lo, hi, device, group_world):
    a13 = ops.compress(w13[0][lo:hi].contiguous(), w13[1][lo:hi].contiguous(), H)
    a2 = ops.compress(w2[0][lo:hi].contiguous(), w2[1][lo:hi].contiguous(), I)
    n = hi - lo
    one = torch.ones(1, device=device)
    ones = torch.ones(n, device=device)
    return ep.ExpertParallelFFN(a13, a2, H, I, CAP, ones, ones, one, ones, fused_config=3, config_id=0, cluster_m=2)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import paired_nvfp4_kernels  # noqa: F401
        from paired_nvfp4_kernels import ep
        ops = torch.ops.paired_nvfp4
        w13, w2 = _weights(device)
        epr = E // world
        ffn = _ffn(ops, ep, w13, w2, rank * epr, (rank + 1) * epr, device, world)
        x, ids, w = _tokens(rank, device)
        plan = ep.build_plan(ids, epr)
        out, counts = ffn.forward(x, plan, w)
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"ep{rank}.npy"), out.view(torch.int16).cpu().numpy())
        np.save(os.path.join(out_dir, f"cnt{rank}.npy"), counts.cpu().numpy())
        # the same pass in three token slices, exchanges on a second stream
        plans = ep.build_chunk_plans(ids, epr, 3)
        out3 = torch.zeros_like(out)
        slice_counts = ep.forward_chunked(ffn, x, plans, w, out3, torch.cuda.Stream())
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"ep3_{rank}.npy"), out3.view(torch.int16).cpu().numpy())
        np.save(os.path.join(out_dir, f"cnt3_{rank}.npy"), torch.stack(slice_counts).sum(0).cpu().numpy())
    finally:
        dist.destroy_process_group()


def _single(out_dir, world):
    """All experts on one GPU, both ranks' tokens as one batch in rank order (the arrival order of the exchange)."""
    import paired_nvfp4_kernels  # noqa: F401
    ops = torch.ops.paired_nvfp4
    device = torch.device("cuda", 0)
    w13, w2 = _weights(device)
    a13 = ops.compress(w13[0], w13[1], H)
    a2 = ops.compress(w2[0], w2[1], I)
    xs, idss, ws = zip(*[_tokens(r, device) for r in range(world)])
    x, ids, w = torch.cat(xs), torch.cat(idss), torch.cat(ws)
    one, ones = torch.ones(1, device=device), torch.ones(E, device=device)
    counts, route_dest, src_tok, _ = ops.dispatch_plan(ids, 0, E, CAP)
    q, q_sf = ops.quant_rows(x, one)
    b1, sfb1 = ops.scatter_fp4_planned(q, q_sf, src_tok, counts, CAP)
    b2, sfb2 = ops.group_mm_swiglu_quant(a13[0], a13[1], a13[2], b1, sfb1, ones, counts, ones, 2 * I, H, 3, 2, 1)
    y = torch.empty((E, CAP, H), dtype=torch.bfloat16, device=device)
    ops.group_mm(y, a2[0], a2[1], a2[2], b2, sfb2, ones, counts, H, I, 0, 2, 1)
    out = torch.empty((x.size(0), H), dtype=torch.bfloat16, device=device)
    ops.moe_finalize(out, y, route_dest, w)
    torch.cuda.synchronize()
    return out.view(torch.int16).cpu().numpy(), counts.cpu().numpy()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_forward_matches_single_gpu(tmp_path):
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    want, want_counts = _single(str(tmp_path), world)
    got = np.concatenate([np.load(tmp_path / f"ep{r}.npy") for r in range(world)])
    got_counts = np.concatenate([np.load(tmp_path / f"cnt{r}.npy") for r in range(world)])
    assert np.array_equal(got_counts, want_counts)
    assert np.array_equal(got, want)
    got3 = np.concatenate([np.load(tmp_path / f"ep3_{r}.npy") for r in range(world)])
    cnt3 = np.concatenate([np.load(tmp_path / f"cnt3_{r}.npy") for r in range(world)])
    assert np.array_equal(cnt3, want_counts) and (want_counts <= CAP).all()
    assert np.array_equal(got3, want)
