"""Expert-parallel exchange (paired_nvfp4_kernels.ep) on CPU: world_size-2 and -3 gloo process groups.

The kernels either side of the exchange need a GPU; here the local expert FFN is a stand-in
(row * (global expert + 1) + 0.25, with per-expert capacity drops from the numpy oracle's dispatch_plan),
so the test pins the host logic: who sends what where, arrival order, the inverse exchange and the final
weighted sum per token.
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
for _p in (ROOT, os.path.join(ROOT, "grouped-sparse-gemm_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _routing(rank, tokens, topk, experts, seed):
    rng = np.random.default_rng(seed + 17 * rank)
    ids = np.stack([rng.permutation(experts)[:topk] for _ in range(tokens)]).astype(np.int64)
    w = rng.random((tokens, topk)).astype(np.float32)
    x = rng.standard_normal((tokens, 8)).astype(np.float32)
    return ids, w, x


def _worker(rank, world, port, tokens, topk, epr, cap, seed, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import paired_nvfp4_oracle as orc
        from paired_nvfp4_kernels import ep
        experts = world * epr
        ids, w, x = _routing(rank, tokens, topk, experts, seed)
        plan = ep.build_plan(torch.from_numpy(ids), epr)
        assert plan.n_send == tokens * topk
        assert sorted(plan.order.tolist()) == list(range(tokens * topk))
        # rows leave grouped by destination rank, in routing order inside a group
        dest = (ids.reshape(-1) // epr)[plan.order.numpy()]
        assert np.all(np.diff(dest) >= 0)
        for r in range(world):
            grp = plan.order.numpy()[dest == r]
            assert np.all(np.diff(grp) > 0)
        assert np.array_equal(plan.inv_pos.numpy().reshape(-1)[plan.order.numpy()], np.arange(tokens * topk))

        rows = torch.from_numpy(x)[plan.send_tok.long()].contiguous()
        recv_rows = ep.dispatch(plan, rows)
        recv_e = ep.dispatch(plan, plan.send_expert)
        assert recv_rows.shape[0] == plan.n_recv == recv_e.numel()
        assert int(recv_e.min()) >= 0 and int(recv_e.max()) < epr
        # local stand-in FFN with capacity drops decided exactly like the device plan
        counts, route_dest, src_tok, _ = orc.dispatch_plan(recv_e.numpy().reshape(-1, 1).astype(np.int64), 0, epr, cap)
        glob = recv_e.numpy().astype(np.int64) + rank * epr
        y = recv_rows.numpy() * (glob[:, None] + 1) + 0.25
        y[route_dest.reshape(-1) < 0] = 0.0          # dropped routings come back as zero rows
        back = ep.combine(plan, torch.from_numpy(y.astype(np.float32)).contiguous())
        out = (back.numpy()[plan.inv_pos.numpy().astype(np.int64)] * w[:, :, None]).sum(1)
        np.save(os.path.join(result_dir, f"out{rank}.npy"), out)
        np.save(os.path.join(result_dir, f"drop{rank}.npy"), np.array([int((route_dest < 0).sum())]))
    finally:
        dist.destroy_process_group()


def _expected(world, tokens, topk, epr, cap, seed):
    """Single-process restatement: arrival order at rank r is source rank major, then routing order."""
    experts = world * epr
    data = [_routing(r, tokens, topk, experts, seed) for r in range(world)]
    kept = {}
    for r in range(world):
        seen = np.zeros(epr, dtype=np.int64)
        for src in range(world):
            ids = data[src][0].reshape(-1)
            for i in np.nonzero(ids // epr == r)[0]:
                e = ids[i] - r * epr
                kept[(src, int(i))] = seen[e] < cap
                seen[e] += 1
    outs = []
    for r in range(world):
        ids, w, x = data[r]
        out = np.zeros((tokens, x.shape[1]), dtype=np.float32)
        for t in range(tokens):
            for j in range(topk):
                if kept[(r, t * topk + j)]:
                    out[t] += w[t, j] * (x[t] * (ids[t, j] + 1) + 0.25)
        outs.append(out)
    return outs, sum(1 for v in kept.values() if not v)


@pytest.mark.parametrize("world,tokens,topk,epr,cap", [(2, 37, 3, 4, 1000), (2, 64, 2, 3, 9), (3, 20, 4, 2, 11)])
def test_exchange_round_trip(tmp_path, world, tokens, topk, epr, cap):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, tokens, topk, epr, cap, 4242, str(tmp_path)), nprocs=world, join=True)
    want, want_drops = _expected(world, tokens, topk, epr, cap, 4242)
    drops = 0
    for r in range(world):
        got = np.load(tmp_path / f"out{r}.npy")
        np.testing.assert_allclose(got, want[r], rtol=1e-5, atol=1e-5)
        drops += int(np.load(tmp_path / f"drop{r}.npy")[0])
    assert drops == want_drops
    if cap < 1000:
        assert drops > 0, "the small-capacity case is meant to drop routings"
