"""Expert-parallel token exchange around the local expert FFN.

One process per GPU.  The E experts are sharded contiguously: rank r owns experts
[r * experts_per_rank, (r + 1) * experts_per_rank).  Every rank holds its own tokens and their top-k
routing.  A forward pass is

    dispatch   each routing (token t, slot j) travels to the rank that owns topk_ids[t, j], as the
               token's activation row (NVFP4 codes + scales on the wire) plus the local expert id
    local FFN  dispatch_plan -> scatter_fp4_planned -> group_mm (gate_up, fused SwiGLU + quantize)
               -> group_mm (down), all on the receiving rank's experts
    combine    the expert output row of every routing travels back to where the routing came from
    finalize   out[t] = sum_j w[t, j] * returned_row(t, j)

dispatch and combine are one all_to_all_single per tensor over the process group (NCCL over NVLink
on GPUs, gloo in the CPU tests).  This module holds the host-side plan and the two exchanges; it is
device agnostic, the kernels either side of it are torch.ops.paired_nvfp4.*.  The reference leaves
this step to its caller (the serving framework's fused-MoE layer: vllm_integration/); the plan
tensors match what its dispatch_plan / moe_finalize ops consume (csrc/ops.cu:548-575).
"""
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class ExchangePlan:
    """The exchange of one rank for one routing.  Rows travel in `order`: routings sorted by
    destination rank, ties in routing order (token major, then top-k slot)."""
    world: int
    rank: int
    experts_per_rank: int
    tokens: int
    topk: int
    order: torch.Tensor        # int64 [n]  routing index t * topk + j of every sent row
    send_tok: torch.Tensor     # int32 [n]  token of every sent row
    send_expert: torch.Tensor  # int32 [n]  expert id local to the destination rank
    inv_pos: torch.Tensor      # int32 [tokens, topk]  position of routing (t, j) in the send order
    send_counts: List[int]     # rows to each rank
    recv_counts: List[int]     # rows from each rank

    @property
    def n_send(self) -> int:
        return int(sum(self.send_counts))

    @property
    def n_recv(self) -> int:
        return int(sum(self.recv_counts))


def build_plan(topk_ids: torch.Tensor, experts_per_rank: int, group: Optional[dist.ProcessGroup] = None) -> ExchangePlan:
    """Plan for topk_ids [tokens, topk] (global expert ids, on the compute device).  Exchanges the
    per-rank row counts (one small all-to-all and one host read): the only host synchronisation of
    a forward pass, and only once per routing."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    assert topk_ids.dim() == 2
    tokens, topk = topk_ids.shape
    flat = topk_ids.reshape(-1).to(torch.int64)
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    assert int(dest.max()) < world and int(dest.min()) >= 0, "expert id outside [0, world * experts_per_rank)"
    order = torch.sort(dest, stable=True).indices
    send_counts_t = torch.bincount(dest, minlength=world).to(torch.int64)
    recv_counts_t = torch.empty_like(send_counts_t)
    dist.all_to_all_single(recv_counts_t, send_counts_t, group=group)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    return ExchangePlan(
        world=world, rank=rank, experts_per_rank=experts_per_rank, tokens=tokens, topk=topk, order=order,
        send_tok=torch.div(order, topk, rounding_mode="floor").to(torch.int32).contiguous(),
        send_expert=(flat[order] - dest[order] * experts_per_rank).to(torch.int32).contiguous(),
        inv_pos=inv.to(torch.int32).reshape(tokens, topk).contiguous(),
        send_counts=[int(v) for v in send_counts_t.tolist()], recv_counts=[int(v) for v in recv_counts_t.tolist()])


def dispatch(plan: ExchangePlan, rows: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """rows [n_send, ...] in send order -> [n_recv, ...] grouped by source rank."""
    assert rows.size(0) == plan.n_send and rows.is_contiguous()
    out = rows.new_empty((plan.n_recv,) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows, plan.recv_counts, plan.send_counts, group=group)
    return out


def combine(plan: ExchangePlan, rows: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """The inverse exchange: rows [n_recv, ...] in arrival order -> [n_send, ...] in send order."""
    assert rows.size(0) == plan.n_recv and rows.is_contiguous()
    out = rows.new_empty((plan.n_send,) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows, plan.send_counts, plan.recv_counts, group=group)
    return out


class ExpertParallelFFN:
    """The expert FFN of one rank (its shard of the experts) behind dispatch / combine.

    Weights are the outputs of torch.ops.paired_nvfp4.compress for the local experts (w13 with gate/up
    rows interleaved for the fused epilogue).  forward() runs the whole pass for this rank's tokens."""

    def __init__(self, w13, w2, hidden, inter, cap, alphas1, alphas2, gscale1, gscale2, fused_config=3, config_id=0,
                 cluster_m=2, group=None):
        self.w13, self.w2 = w13, w2            # (a_comp, e_meta, sfa) each
        self.hidden, self.inter, self.cap = hidden, inter, cap
        self.al1, self.al2, self.g1, self.g2 = alphas1, alphas2, gscale1, gscale2
        self.fused_config, self.config_id, self.cluster_m = fused_config, config_id, cluster_m
        self.group = group
        self.num_local = w13[0].size(0)

    def forward(self, x, plan: ExchangePlan, topk_weights, out=None):
        ops = torch.ops.paired_nvfp4
        E, H, I, cap = self.num_local, self.hidden, self.inter, self.cap
        # NVFP4 on the wire: quantize each token once, send codes + scales
        q, q_sf = ops.quant_rows(x, self.g1)
        send_q = ops.gather_rows(q, plan.send_tok)
        send_sf = ops.gather_rows(q_sf, plan.send_tok)
        recv_q = dispatch(plan, send_q, self.group)
        recv_sf = dispatch(plan, send_sf, self.group)
        recv_e = dispatch(plan, plan.send_expert, self.group)
        counts, route_dest, src_tok, _ = ops.dispatch_plan(recv_e.view(-1, 1), 0, E, cap)
        b1, sfb1 = ops.scatter_fp4_planned(recv_q, recv_sf, src_tok, counts, cap)
        b2, sfb2 = ops.group_mm_swiglu_quant(self.w13[0], self.w13[1], self.w13[2], b1, sfb1, self.al1, counts, self.g2,
                                             2 * I, H, self.fused_config, self.cluster_m, 1, "silu", 1.0, -1.0)
        y = torch.empty((E, cap, H), dtype=torch.bfloat16, device=x.device)
        ops.group_mm(y, self.w2[0], self.w2[1], self.w2[2], b2, sfb2, self.al2, counts, H, I, self.config_id,
                     self.cluster_m, 1)
        back = ops.gather_rows(y.view(E * cap, H), route_dest.view(-1))   # dropped routings return zero rows
        ret = combine(plan, back, self.group)
        if out is None:
            out = torch.empty((plan.tokens, H), dtype=torch.bfloat16, device=x.device)
        ops.moe_finalize(out, ret, plan.inv_pos, topk_weights)
        return out, counts


def build_chunk_plans(topk_ids: torch.Tensor, experts_per_rank: int, chunks: int,
                      group: Optional[dist.ProcessGroup] = None) -> List[ExchangePlan]:
    """One exchange plan per contiguous slice of the tokens (every rank must use the same `chunks`)."""
    tokens = topk_ids.size(0)
    bounds = [tokens * c // chunks for c in range(chunks + 1)]
    return [build_plan(topk_ids[bounds[c]:bounds[c + 1]].contiguous(), experts_per_rank, group) for c in range(chunks)]


def forward_chunked(ffn: "ExpertParallelFFN", x: torch.Tensor, plans: List[ExchangePlan], topk_weights: torch.Tensor,
                    out: torch.Tensor, comm_stream: torch.cuda.Stream):
    """The same pass as ExpertParallelFFN.forward with the tokens cut into len(plans) slices: the
    all-to-all of one slice runs on `comm_stream` while the GEMMs of another run on the current
    stream.  Returns the per-slice expert counts."""
    ops = torch.ops.paired_nvfp4
    E, H, I, cap = ffn.num_local, ffn.hidden, ffn.inter, ffn.cap
    main = torch.cuda.current_stream()
    bounds = [0]
    for pl in plans:
        bounds.append(bounds[-1] + pl.tokens)
    keep = []          # every tensor that crosses streams stays referenced until both streams have met again

    def on_comm(after: torch.cuda.Event, fn):
        with torch.cuda.stream(comm_stream):
            comm_stream.wait_event(after)
            res = fn()
            done = torch.cuda.Event()
            done.record(comm_stream)
        return res, done

    def prep(c):
        pl = plans[c]
        q, q_sf = ops.quant_rows(x[bounds[c]:bounds[c + 1]], ffn.g1)
        send = (ops.gather_rows(q, pl.send_tok), ops.gather_rows(q_sf, pl.send_tok), pl.send_expert)
        ev = torch.cuda.Event()
        ev.record(main)
        keep.extend(send)
        return send, ev

    def exchange_out(c, send, ev):
        return on_comm(ev, lambda: tuple(dispatch(plans[c], t, ffn.group) for t in send))

    def compute(c, recv, ev):
        main.wait_event(ev)
        recv_q, recv_sf, recv_e = recv
        counts, route_dest, src_tok, _ = ops.dispatch_plan(recv_e.view(-1, 1), 0, E, cap)
        b1, sfb1 = ops.scatter_fp4_planned(recv_q, recv_sf, src_tok, counts, cap)
        b2, sfb2 = ops.group_mm_swiglu_quant(ffn.w13[0], ffn.w13[1], ffn.w13[2], b1, sfb1, ffn.al1, counts, ffn.g2,
                                             2 * I, H, ffn.fused_config, ffn.cluster_m, 1, "silu", 1.0, -1.0)
        y = torch.empty((E, cap, H), dtype=torch.bfloat16, device=x.device)
        ops.group_mm(y, ffn.w2[0], ffn.w2[1], ffn.w2[2], b2, sfb2, ffn.al2, counts, H, I, ffn.config_id,
                     ffn.cluster_m, 1)
        back = ops.gather_rows(y.view(E * cap, H), route_dest.view(-1))
        done = torch.cuda.Event()
        done.record(main)
        keep.extend((recv_q, recv_sf, recv_e, back))
        return back, done, counts

    n = len(plans)
    sends = [prep(c) for c in range(n)]
    recvs = [None] * n
    recvs[0] = exchange_out(0, *sends[0])
    rets, all_counts = [None] * n, []
    for c in range(n):
        if c + 1 < n:
            recvs[c + 1] = exchange_out(c + 1, *sends[c + 1])      # travels while slice c is multiplied
        back, done, counts = compute(c, *recvs[c])
        all_counts.append(counts)
        rets[c] = on_comm(done, lambda b=back, c=c: combine(plans[c], b, ffn.group))
    for c in range(n):
        ret, ev = rets[c]
        main.wait_event(ev)
        keep.append(ret)
        ops.moe_finalize(out[bounds[c]:bounds[c + 1]], ret, plans[c].inv_pos, topk_weights[bounds[c]:bounds[c + 1]])
    # the communication stream may not run ahead into memory this pass is still using
    comm_stream.wait_stream(main)
    for t in keep:
        t.record_stream(comm_stream)
        t.record_stream(main)
    return all_counts
