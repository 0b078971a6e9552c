"""Expert parallelism on the GPU.  The exchanged forward pass must give every rank, bit for bit, what one GPU
holding all experts computes for the same tokens (row placement inside an expert does not change a row's
result, and moe_finalize sums in top-k order).  Three forms: one rank (the exchange is the identity, everything
else - slab plan, wire rows, plan on the strided ids, placement, return order - is the real path), two ranks
emulated on one GPU (both ranks' halves run one after the other, the all-to-all is a slab swap in Python), and two
real ranks over NCCL (skipped on a single-GPU box).  The last two also with the direct exchange, where the producing
kernels store wire rows and expert outputs straight into the other rank's buffers (on one GPU: into the other
emulated rank's buffers; on two: into peer memory opened through CUDA IPC)."""
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

E, H, I, T, TOPK, CAP, SLAB = 8, 512, 256, 96, 2, 64, 256


def _weights(device):
    """Compressed W13 (gate/up rows interleaved) and W2 of all E experts, from a fixed seed."""
    import paired_nvfp4_kernels as pnk
    from paired_nvfp4_kernels import reference as wref
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


def _ffn(ops, ep, w13, w2, lo, hi, device, world, rank, exchange=None, slab=SLAB, peers=None):
    a13 = ops.compress(w13[0][lo:hi].contiguous(), w13[1][lo:hi].contiguous(), H)
    a2 = ops.compress(w2[0][lo:hi].contiguous(), w2[1][lo:hi].contiguous(), I)
    n = hi - lo
    one = torch.ones(1, device=device)
    ones = torch.ones(n, device=device)
    return ep.ExpertParallelFFN(a13, a2, H, I, CAP, ones, ones, one, ones, slab, fused_config=3, config_id=0, cluster_m=2,
                                world=world, rank=rank, exchange=exchange, peers=peers)


def _single(world, device=None):
    """All experts on one GPU, the ranks' tokens as one batch in rank order (the arrival order of the exchange)."""
    import paired_nvfp4_kernels  # noqa: F401
    ops = torch.ops.paired_nvfp4
    device = device or torch.device("cuda", 0)
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


def test_wire_rows_match_oracle():
    """pack_wire_rows against the numpy restatement on every defined byte, and the receiver's view of it:
    dispatch_plan on the ids inside the rows, scatter_fp4_wire == scatter_fp4_planned on the unpacked rows."""
    import paired_nvfp4_kernels  # noqa: F401
    from oracle import paired_nvfp4_oracle as orc
    from paired_nvfp4_kernels import ops as pyops
    ops = torch.ops.paired_nvfp4
    dev = torch.device("cuda", 0)
    for K, tokens, topk, world, epr, slab in [(512, 50, 3, 4, 2, 64), (96, 33, 2, 2, 3, 16), (7168, 20, 4, 2, 4, 48)]:
        rng = np.random.default_rng(K + tokens)
        x = torch.from_numpy(rng.standard_normal((tokens, K)).astype(np.float32)).to(torch.bfloat16).to(dev)
        ids = torch.from_numpy(np.stack([rng.permutation(world * epr)[:topk] for _ in range(tokens)]).astype(np.int64)).to(dev)
        g = torch.full((1,), 3.5, device=dev)
        q, q_sf = ops.quant_rows(x, g)
        slab_counts, route_slot, slot_tok, slot_route = ops.dispatch_plan(torch.div(ids, epr, rounding_mode="floor"), 0, world, slab)
        wire = ops.pack_wire_rows(q, q_sf, ids, slot_tok, slot_route, slab_counts, slab, epr)
        torch.cuda.synchronize()
        assert wire.shape == (world * slab, orc.wire_row_bytes(K)) == (world * slab, pyops.wire_row_bytes(K))
        want, defined = orc.pack_wire_rows(q.cpu().numpy(), q_sf.cpu().numpy(), ids.cpu().numpy(), slot_tok.cpu().numpy(),
                                           slot_route.cpu().numpy(), slab_counts.cpu().numpy(), slab, epr)
        assert np.array_equal(wire.cpu().numpy()[defined], want[defined])
        # receiver side, as rank 1 would see slab 1 of every sender (here: this one sender's slab, repeated)
        recv = wire[slab:2 * slab].repeat(2, 1).contiguous()
        rid = pyops.wire_expert_ids(recv)
        assert rid.shape == (2 * slab, 1) and not rid.is_contiguous()
        counts, route_dest, src_tok, _ = ops.dispatch_plan(rid, 0, epr, 40)
        oc, ord_, ost, _ = orc.dispatch_plan(rid.cpu().numpy().astype(np.int64), 0, epr, 40)
        assert np.array_equal(counts.cpu().numpy(), oc) and np.array_equal(route_dest.cpu().numpy(), ord_)
        b, sfb = ops.scatter_fp4_wire(recv, K, src_tok, counts, 40)
        rq, rsf, _ = orc.unpack_wire_rows(recv.cpu().numpy(), K)
        ob, valid, osfb = orc.scatter_fp4_planned(rq, rsf, ost, oc, 40)
        torch.cuda.synchronize()
        assert np.array_equal(b.cpu().numpy()[valid], ob[valid]) and np.array_equal(sfb.cpu().numpy(), osfb)


def test_one_rank_forward_matches_direct_path():
    import paired_nvfp4_kernels  # noqa: F401
    from paired_nvfp4_kernels import ep
    ops = torch.ops.paired_nvfp4
    device = torch.device("cuda", 0)
    w13, w2 = _weights(device)
    ffn = _ffn(ops, ep, w13, w2, 0, E, device, 1, 0)
    x, ids, w = _tokens(0, device)
    out, counts, route_slot = ffn.forward(x, ids, w)
    torch.cuda.synchronize()
    want, want_counts = _single(1, device)
    assert int((route_slot < 0).sum()) == 0
    assert np.array_equal(counts.cpu().numpy(), want_counts)
    assert np.array_equal(out.view(torch.int16).cpu().numpy(), want)


@pytest.mark.parametrize("slab", [SLAB, 80])
def test_two_ranks_emulated_on_one_gpu(slab):
    """Both ranks' halves on one GPU, one after the other; the all-to-all is a swap of slabs.  With slab = 80
    some routings do not fit their slab and must drop exactly as the single-GPU path drops them when the
    same routings are masked out."""
    import paired_nvfp4_kernels  # noqa: F401
    from paired_nvfp4_kernels import ep
    ops = torch.ops.paired_nvfp4
    device = torch.device("cuda", 0)
    world, epr = 2, E // 2
    w13, w2 = _weights(device)
    ffns = [_ffn(ops, ep, w13, w2, r * epr, (r + 1) * epr, device, world, r, slab=slab) for r in range(world)]
    toks = [_tokens(r, device) for r in range(world)]

    def swap(per_rank):      # rank r receives slab r of every sender, in sender order
        return [torch.cat([per_rank[s][r * slab:(r + 1) * slab] for s in range(world)]).contiguous() for r in range(world)]

    sent = [ffns[r].plan_and_pack(toks[r][0], toks[r][1]) for r in range(world)]
    recv = swap([s[0] for s in sent])
    backs = [ffns[r].local_ffn(recv[r]) for r in range(world)]
    ret = swap([b[0] for b in backs])
    outs = []
    for r in range(world):
        out = torch.empty((T, H), dtype=torch.bfloat16, device=device)
        ops.moe_finalize(out, ret[r], sent[r][1], toks[r][2])
        outs.append(out)
    torch.cuda.synchronize()
    dropped = sum(int((s[1] < 0).sum()) for s in sent)
    if slab == SLAB:
        assert dropped == 0
        want, want_counts = _single(world, device)
    else:
        assert dropped > 0
        # the single-GPU path with the same routings masked out (expert id -1 is nobody's expert)
        a13 = ops.compress(w13[0], w13[1], H)
        a2 = ops.compress(w2[0], w2[1], I)
        ids = torch.cat([torch.where(sent[r][1] < 0, torch.full_like(toks[r][1], -1), toks[r][1]) for r in range(world)])
        x, w = torch.cat([t[0] for t in toks]), torch.cat([t[2] for t in toks])
        one, ones = torch.ones(1, device=device), torch.ones(E, device=device)
        counts, route_dest, src_tok, _ = ops.dispatch_plan(ids, 0, E, CAP)
        q, q_sf = ops.quant_rows(x, one)
        b1, sfb1 = ops.scatter_fp4_planned(q, q_sf, src_tok, counts, CAP)
        b2, sfb2 = ops.group_mm_swiglu_quant(a13[0], a13[1], a13[2], b1, sfb1, ones, counts, ones, 2 * I, H, 3, 2, 1)
        y = torch.empty((E, CAP, H), dtype=torch.bfloat16, device=device)
        ops.group_mm(y, a2[0], a2[1], a2[2], b2, sfb2, ones, counts, H, I, 0, 2, 1)
        o = torch.empty((x.size(0), H), dtype=torch.bfloat16, device=device)
        ops.moe_finalize(o, y, route_dest, w)
        torch.cuda.synchronize()
        want, want_counts = o.view(torch.int16).cpu().numpy(), counts.cpu().numpy()
    got = torch.cat(outs).view(torch.int16).cpu().numpy()
    got_counts = torch.cat([b[1] for b in backs]).cpu().numpy()
    assert np.array_equal(got_counts, want_counts)
    assert np.array_equal(got, want)


def test_pack_wire_rows_parts_equals_pack_wire_rows():
    import paired_nvfp4_kernels  # noqa: F401
    from paired_nvfp4_kernels import ops as pyops
    ops = torch.ops.paired_nvfp4
    dev = torch.device("cuda", 0)
    K, tokens, topk, world, epr, slab = 512, 50, 3, 4, 2, 64
    rng = np.random.default_rng(3)
    x = torch.from_numpy(rng.standard_normal((tokens, K)).astype(np.float32)).to(torch.bfloat16).to(dev)
    ids = torch.from_numpy(np.stack([rng.permutation(world * epr)[:topk] for _ in range(tokens)]).astype(np.int64)).to(dev)
    q, q_sf = ops.quant_rows(x, torch.full((1,), 3.5, device=dev))
    slab_counts, _, slot_tok, slot_route = ops.dispatch_plan(torch.div(ids, epr, rounding_mode="floor"), 0, world, slab)
    wire = ops.pack_wire_rows(q, q_sf, ids, slot_tok, slot_route, slab_counts, slab, epr)
    parts = [torch.zeros((slab, pyops.wire_row_bytes(K)), dtype=torch.uint8, device=dev) for _ in range(world)]
    ops.pack_wire_rows_parts(q, q_sf, ids, slot_tok, slot_route, slab_counts, slab, epr, parts)
    torch.cuda.synchronize()
    live = (torch.arange(slab, device=dev)[None, :] < slab_counts[:, None]).reshape(-1)
    got = torch.cat(parts)
    used = K // 2 + K // 32                               # the bytes after the scales are padding, but for the id
    assert torch.equal(got[live][:, :used], wire[live][:, :used])
    assert torch.equal(pyops.wire_expert_ids(got), pyops.wire_expert_ids(wire))     # dead slots carry -1 in both


@pytest.mark.parametrize("slab", [SLAB, 80])
def test_two_ranks_emulated_direct_exchange(slab):
    """The direct exchange with both ranks in one process: each rank's kernels store into the other's buffers."""
    import paired_nvfp4_kernels  # noqa: F401
    from paired_nvfp4_kernels import ep
    from paired_nvfp4_kernels import ops as pyops
    ops = torch.ops.paired_nvfp4
    device = torch.device("cuda", 0)
    world, epr = 2, E // 2
    w13, w2 = _weights(device)
    pbs = [ep.PeerBuffers(world, r, slab, H, pyops.wire_row_bytes(H), device, local_only=True) for r in range(world)]
    for pb in pbs:
        pb.recv, pb.ret = [p.recv_own for p in pbs], [p.ret_own for p in pbs]
        pb.ret_own.fill_(float("nan"))       # every row a sender reads must have been written by somebody
    ffns = [_ffn(ops, ep, w13, w2, r * epr, (r + 1) * epr, device, world, r, slab=slab, peers=pbs[r]) for r in range(world)]
    toks = [_tokens(r, device) for r in range(world)]
    slots = [ffns[r].send_direct(toks[r][0], toks[r][1]) for r in range(world)]
    counts = [ffns[r].local_ffn_direct() for r in range(world)]
    outs = []
    for r in range(world):
        out = torch.empty((T, H), dtype=torch.bfloat16, device=device)
        ops.moe_finalize(out, pbs[r].ret_own, slots[r], toks[r][2])
        outs.append(out)
    torch.cuda.synchronize()
    # the all-to-all form of the same pass is the yardstick (itself checked against the single-GPU path above)
    ref = [_ffn(ops, ep, w13, w2, r * epr, (r + 1) * epr, device, world, r, slab=slab) for r in range(world)]
    sent = [ref[r].plan_and_pack(toks[r][0], toks[r][1]) for r in range(world)]

    def swap(per_rank):
        return [torch.cat([per_rank[s][r * slab:(r + 1) * slab] for s in range(world)]).contiguous() for r in range(world)]

    backs = [ref[r].local_ffn(rv) for r, rv in enumerate(swap([s[0] for s in sent]))]
    ret = swap([b[0] for b in backs])
    for r in range(world):
        want = torch.empty((T, H), dtype=torch.bfloat16, device=device)
        ops.moe_finalize(want, ret[r], sent[r][1], toks[r][2])
        torch.cuda.synchronize()
        assert torch.equal(slots[r], sent[r][1]) and torch.equal(counts[r], backs[r][1])
        assert torch.equal(outs[r].view(torch.int16), want.view(torch.int16))
        assert not torch.isnan(outs[r].float()).any()
    for pb in pbs:
        pb.close()


def _worker(rank, world, port, out_dir, direct=False, one_gpu=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    if one_gpu:          # both ranks on GPU 0, the fences over gloo (NCCL wants a GPU per rank)
        torch.cuda.set_device(0)
        device = torch.device("cuda", 0)
        dist.init_process_group("gloo", rank=rank, world_size=world)
    else:
        torch.cuda.set_device(rank)
        device = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import paired_nvfp4_kernels  # noqa: F401
        from paired_nvfp4_kernels import ep
        ops = torch.ops.paired_nvfp4
        w13, w2 = _weights(device)
        epr = E // world
        peers = None
        if direct:
            from paired_nvfp4_kernels import ops as pyops
            peers = ep.PeerBuffers(world, rank, SLAB, H, pyops.wire_row_bytes(H), device)
        ffn = _ffn(ops, ep, w13, w2, rank * epr, (rank + 1) * epr, device, world, rank, peers=peers)
        x, ids, w = _tokens(rank, device)
        for _ in range(3 if direct else 1):      # direct: the buffers are reused pass after pass
            out, counts, _ = ffn.forward(x, ids, w)
        torch.cuda.synchronize()
        if peers is not None:
            peers.close()
        np.save(os.path.join(out_dir, f"ep{rank}.npy"), out.view(torch.int16).cpu().numpy())
        np.save(os.path.join(out_dir, f"cnt{rank}.npy"), counts.cpu().numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("direct", [False, True])
def test_two_rank_forward_matches_single_gpu(tmp_path, direct):
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path), direct), nprocs=world, join=True)
    want, want_counts = _single(world)
    got = np.concatenate([np.load(tmp_path / f"ep{r}.npy") for r in range(world)])
    got_counts = np.concatenate([np.load(tmp_path / f"cnt{r}.npy") for r in range(world)])
    assert np.array_equal(got_counts, want_counts)
    assert np.array_equal(got, want)


def test_two_processes_one_gpu_direct_exchange(tmp_path):
    """The direct exchange between two real processes that share GPU 0: buffers allocated by the library, their
    interprocess handles exchanged and opened in the other process, rows stored straight into the other rank's
    buffers, three passes over the same buffers.  (No kernel of one process waits for the other: the fences are
    host-side collectives.)"""
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path), True, True), nprocs=world, join=True)
    want, want_counts = _single(world)
    got = np.concatenate([np.load(tmp_path / f"ep{r}.npy") for r in range(world)])
    got_counts = np.concatenate([np.load(tmp_path / f"cnt{r}.npy") for r in range(world)])
    assert np.array_equal(got_counts, want_counts)
    assert np.array_equal(got, want)
