"""Expert-parallel forward (paired_nvfp4_kernels.ep) on CPU: world_size-2 and -3 gloo process groups.

The kernels need a GPU, so the module is driven with a stand-in for torch.ops.paired_nvfp4 built on the numpy
oracle (tests/ep_cpu_ops.py).  Everything around the kernels is the product code: the fixed-capacity slab plan,
the wire rows, both equal-split all-to-alls, the return order and the final weighted sum.  The result of every
rank must equal, bit for bit, what one process holding all experts computes for that rank's tokens - including
routings dropped by an expert's capacity (decided in arrival order: source rank major, then routing order)
and by the slab capacity.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for _p in (ROOT, os.path.join(ROOT, "grouped-sparse-gemm_b200"), os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

H, I = 64, 32


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _weights(experts):
    from oracle import paired_nvfp4_oracle as orc
    rng = np.random.default_rng(7)
    w13 = orc.quantize_weight(orc.prune_paired_4of8(rng.standard_normal((experts, 2 * I, H)).astype(np.float32)))[2]
    w2 = orc.quantize_weight(orc.prune_paired_4of8(rng.standard_normal((experts, H, I)).astype(np.float32)))[2]
    return torch.from_numpy(w13), torch.from_numpy(w2)


def _tokens(rank, tokens, topk, experts, seed):
    rng = np.random.default_rng(seed + 17 * rank)
    ids = np.stack([rng.permutation(experts)[:topk] for _ in range(tokens)]).astype(np.int64)
    w = rng.random((tokens, topk)).astype(np.float32)
    x = torch.from_numpy(rng.standard_normal((tokens, H)).astype(np.float32)).to(torch.bfloat16)
    return x, torch.from_numpy(ids), torch.from_numpy(w)


def _ffn(ep, ops, w13, w2, lo, hi, cap, slab, world, rank, exchange=None):
    n = hi - lo
    one, ones = torch.ones(1), torch.ones(n)
    return ep.ExpertParallelFFN((w13[lo:hi], None, None), (w2[lo:hi], None, None), H, I, cap, ones, ones, one, ones,
                                slab, ops=ops, world=world, rank=rank, exchange=exchange)


def _worker(rank, world, port, tokens, topk, epr, cap, slab, seed, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ep_cpu_ops import CpuOps
        from paired_nvfp4_kernels import ep
        w13, w2 = _weights(world * epr)
        ffn = _ffn(ep, CpuOps(), w13, w2, rank * epr, (rank + 1) * epr, cap, slab, world, rank)
        x, ids, w = _tokens(rank, tokens, topk, world * epr, seed)
        out, counts, route_slot = ffn.forward(x, ids, w)
        np.save(os.path.join(result_dir, f"out{rank}.npy"), out.view(torch.int16).numpy())
        np.save(os.path.join(result_dir, f"cnt{rank}.npy"), counts.numpy())
        np.save(os.path.join(result_dir, f"slot{rank}.npy"), route_slot.numpy())
    finally:
        dist.destroy_process_group()


def _single_process(world, tokens, topk, epr, cap, slab, seed):
    """One process, all experts, every rank's tokens in rank order.  Routings that a rank's slab would not have
    carried are masked out first (expert id -1), then the expert capacity acts in arrival order."""
    from ep_cpu_ops import CpuOps
    from oracle import paired_nvfp4_oracle as orc
    ops = CpuOps()
    experts = world * epr
    w13, w2 = _weights(experts)
    xs, idss, ws = zip(*[_tokens(r, tokens, topk, experts, seed) for r in range(world)])
    masked = []
    for ids in idss:
        _, slot, _, _ = orc.dispatch_plan(ids.numpy() // epr, 0, world, slab)
        masked.append(torch.where(torch.from_numpy(slot) < 0, torch.full_like(ids, -1), ids))
    x, ids, w = torch.cat(xs), torch.cat(masked), torch.cat(ws)
    one, ones = torch.ones(1), torch.ones(experts)
    counts, route_dest, src_tok, _ = ops.dispatch_plan(ids, 0, experts, cap)
    q, q_sf = ops.quant_rows(x, one)
    b1, _, sfb1 = orc.scatter_fp4_planned(q.numpy(), q_sf.numpy(), src_tok.numpy(), counts.numpy(), cap)
    b2, sfb2 = ops.group_mm_swiglu_quant(w13, None, None, torch.from_numpy(b1), torch.from_numpy(sfb1), ones, counts, ones,
                                         2 * I, H, 0, 2, 1, "silu", 1.0, -1.0)
    y = torch.zeros((experts, cap, H), dtype=torch.bfloat16)
    ops.group_mm(y, w2, None, None, b2, sfb2, ones, counts, H, I, 0, 2, 1)
    out = torch.zeros((x.size(0), H), dtype=torch.bfloat16)
    ops.moe_finalize(out, y.view(experts * cap, H), route_dest, w)
    return out.view(torch.int16).numpy(), counts.numpy(), int((route_dest < 0).sum())


@pytest.mark.parametrize("world,tokens,topk,epr,cap,slab", [
    (2, 37, 3, 4, 1000, 128),       # nothing dropped
    (2, 64, 2, 3, 9, 128),          # expert capacity drops
    (3, 20, 4, 2, 11, 24),          # three ranks; the slab (24 rows) drops routings as well
])
def test_forward_matches_single_process(tmp_path, world, tokens, topk, epr, cap, slab):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, tokens, topk, epr, cap, slab, 4242, str(tmp_path)), nprocs=world, join=True)
    want, want_counts, want_drops = _single_process(world, tokens, topk, epr, cap, slab, 4242)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    got_counts = np.concatenate([np.load(tmp_path / f"cnt{r}.npy") for r in range(world)])
    assert np.array_equal(got_counts, want_counts)
    assert np.array_equal(got, want)
    slot_drops = sum(int((np.load(tmp_path / f"slot{r}.npy") < 0).sum()) for r in range(world))
    if slab < 128:
        assert slot_drops > 0, "the small-slab case is meant to drop routings"
    if cap < 1000:
        assert want_drops > slot_drops, "the small-capacity cases are meant to drop routings at the experts"
