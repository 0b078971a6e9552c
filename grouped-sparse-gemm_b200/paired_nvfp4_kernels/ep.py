"""Expert-parallel token exchange around the local expert FFN.

One process per GPU.  The E experts are sharded contiguously: rank r owns experts
[r * experts_per_rank, (r + 1) * experts_per_rank).  Every rank holds its own tokens and their top-k
routing.  A forward pass is

    plan       the rank's routings are sorted by destination rank into fixed-capacity slabs of `slab`
               rows per destination (dispatch_plan with "experts" = ranks)
    pack       each token is quantized once (quant_rows) and every live slot becomes one wire row:
               NVFP4 codes + scales + the expert id local to the receiver; dead slots carry id -1
    dispatch   ONE equal-split all-to-all of the slabs
    local FFN  dispatch_plan on the ids inside the received rows -> scatter_fp4_wire -> group_mm
               (gate_up, fused SwiGLU + quantize) -> group_mm_rows (down; every expert output row is written
               straight into the slot it came from) + zero_rows for the slots no expert kept
    combine    ONE equal-split all-to-all back (bf16 rows)
    finalize   out[t] = sum_j w[t, j] * returned_row(t, j)

Every shape is fixed by (tokens, topk, world, slab): nothing is read back to the host, no split sizes
are exchanged, so a whole forward pass with fresh routing can be captured in a CUDA graph like the
single-GPU path.  The price is the padding of the slabs: `slab` must cover the busiest destination
(a routing that does not fit is dropped like one past an expert's capacity; the caller sees it as a
-1 in the returned slot map).

Two exchanges.  The plain one: torch.distributed's all-to-all (NCCL over NVLink on GPUs, gloo in the
CPU tests) either side of the local FFN.  The direct one (PeerBuffers, one node, GPUs with peer
access): every rank's receive and return buffers are opened in every other rank's process, and the
kernels that produce the rows store them where they are wanted - pack_wire_rows_parts writes slab w
into rank w's receive buffer, group_mm_rows_parts writes every expert output row into the return
buffer of the rank that sent the token, while the tensor cores work on the next tiles.  Nothing is
copied a second time and no all-to-all runs; two small all-reduces per pass order the stores against
their readers (rows landed before the receiver plans; outputs landed before the sender combines).

This module holds the order of operations and the exchange, the kernels are
torch.ops.paired_nvfp4.* (or, in the CPU tests, a stand-in object with the same methods).  The reference leaves this step to its
caller (the serving framework's fused-MoE layer); dispatch_plan / moe_finalize are the ops it
provides either side of it (csrc/ops.cu:374-411, 548-575).
"""
from typing import Callable, Optional

import torch
import torch.distributed as dist


def slab_rows(tokens: int, topk: int, world: int, headroom: float = 1.125) -> int:
    """Rows per destination slab: the mean load of a destination rank times `headroom`, rounded up to 128."""
    mean = tokens * topk / world
    return min(tokens * topk, (int(mean * headroom) + 127) // 128 * 128)


class _TorchOps:
    """torch.ops.paired_nvfp4 plus the one helper that is a view, not an operator."""

    def __init__(self):
        from . import ops as pyops
        self._ns = torch.ops.paired_nvfp4
        self.wire_expert_ids = pyops.wire_expert_ids

    def __getattr__(self, name):
        return getattr(self._ns, name)


class _RawCuda:
    """A device pointer as an object torch.as_tensor understands (the CUDA array interface)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerBuffers:
    """The receive and return buffers of every rank, visible to all of them.

    recv[r] uint8 [world * slab, wire row bytes]: slab s holds the wire rows rank s sent to rank r.
    ret[r]  bf16  [world * slab, hidden]:         slab w holds the expert outputs of the rows rank r sent to rank w.
    Index r is the owner.  Each rank allocates its own pair through the library (plain cudaMalloc, so that the
    interprocess handle names exactly that allocation), the 64-byte handles are all-gathered, and every rank maps
    the others' buffers into its own device's address space (pnv_peer_buffer_open: cudaIpcOpenMemHandle with lazy
    peer access).  One node, GPUs with peer access.

    close() is a collective (it ends with a barrier): every rank unmaps the others' buffers, then frees its own."""

    def __init__(self, world, rank, slab, hidden, row_bytes, device, group=None, local_only=False):
        import ctypes
        from . import _cabi
        self._cabi, self._lib = _cabi, _cabi.lib
        self.world, self.rank, self.slab, self.group = world, rank, slab, group
        self.device = torch.device(device)
        rows = world * slab
        self._sizes = (rows * row_bytes, rows * hidden * 2)
        self._own_ptrs, self._opened, handles = [], [], []
        self._collective = world > 1 and not local_only
        self.recv, self.ret = [None] * world, [None] * world
        self.recv_own = self.ret_own = None
        # A failure on one rank (no memory, no peer path, interprocess handles not permitted) must not leave the
        # others inside a collective: every rank goes through the same collectives whatever happened to it, the
        # outcome is agreed on at the end, and then every rank raises or none does.
        error = None
        try:
            with torch.cuda.device(self.device):
                for nbytes in self._sizes:
                    ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
                    _cabi.check(self._lib.pnv_peer_buffer_alloc(nbytes, ctypes.byref(ptr), handle))
                    self._own_ptrs.append(ptr.value)
                    handles.append(handle.raw)
            self.recv_own = self._view(self._own_ptrs[0], 0).view(rows, row_bytes)
            self.ret_own = self._view(self._own_ptrs[1], 1).view(torch.bfloat16).view(rows, hidden)
            # dead slots are recognised by the id inside the row: start with all of them dead
            self.recv_own.view(torch.int32)[:, row_bytes // 4 - 4].fill_(-1)
            self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.recv[rank], self.ret[rank] = self.recv_own, self.ret_own
            torch.cuda.synchronize(self.device)
        except Exception as ex:          # noqa: BLE001  (reported below, on every rank)
            error = f"rank {rank}: {ex}"
        if local_only:                      # tests: all ranks in one process link their buffers themselves
            if error:
                raise RuntimeError(error)
            return
        everyone = [None] * world
        dist.all_gather_object(everyone, (handles, error), group=group)
        if not any(err for _, err in everyone):
            try:
                with torch.cuda.device(self.device):
                    for r in range(world):
                        if r == rank:
                            continue
                        views = []
                        for which, handle in enumerate(everyone[r][0]):
                            ptr = ctypes.c_void_p()
                            _cabi.check(self._lib.pnv_peer_buffer_open(handle, ctypes.byref(ptr)))
                            self._opened.append(ptr.value)
                            views.append(self._view(ptr.value, which))
                        self.recv[r] = views[0].view(rows, row_bytes)
                        self.ret[r] = views[1].view(torch.bfloat16).view(rows, hidden)
            except Exception as ex:      # noqa: BLE001
                error = f"rank {rank}: {ex}"
        outcome = [None] * world
        dist.all_gather_object(outcome, error, group=group)
        errors = [err for _, err in everyone if err] + [err for err in outcome if err]
        if errors:
            self.close()
            raise RuntimeError("direct exchange unavailable: " + "; ".join(sorted(set(errors))))

    def _view(self, ptr, which):
        # no device argument: torch takes the device from the pointer itself and never copies
        return torch.as_tensor(_RawCuda(ptr, self._sizes[which]))

    def recv_parts(self):
        """Where this rank's slab for rank w goes: slab `rank` of rank w's receive buffer."""
        s, r = self.slab, self.rank
        return [self.recv[w][r * s:(r + 1) * s] for w in range(self.world)]

    def ret_parts(self):
        """Where the outputs of the rows rank w sent here go: slab `rank` of rank w's return buffer."""
        s, r = self.slab, self.rank
        return [self.ret[w][r * s:(r + 1) * s] for w in range(self.world)]

    def fence(self):
        """Every rank's stores issued so far have landed before anything enqueued after this runs, on every
        rank: a one-element all-reduce on the current stream (kernels complete, and with them their stores to
        peer memory, before the collective that follows them in the stream starts)."""
        if self.world > 1 and dist.is_initialized():
            dist.all_reduce(self._token, group=self.group)

    def close(self):
        """Unmap the other ranks' buffers, then free this rank's.  A collective (two barriers) unless the buffers
        were linked inside one process."""
        if self._lib is None:
            return
        collective = self._collective and dist.is_initialized()
        torch.cuda.synchronize(self.device)
        if collective:
            dist.barrier(group=self.group)          # nobody stores into anybody's buffers any more
        self.recv, self.ret, self.recv_own, self.ret_own = [], [], None, None
        with torch.cuda.device(self.device):
            for ptr in self._opened:
                self._lib.pnv_peer_buffer_close(ptr)
            self._opened = []
            if collective:
                dist.barrier(group=self.group)      # every mapping of this rank's buffers is gone
            for ptr in self._own_ptrs:
                self._lib.pnv_peer_buffer_free(ptr)
            self._own_ptrs = []
        self._lib = None


class ExpertParallelFFN:
    """The expert FFN of one rank (its shard of the experts) behind dispatch / combine.

    Weights are the outputs of torch.ops.paired_nvfp4.compress for the local experts (w13 with gate/up
    rows interleaved for the fused epilogue).  forward() runs the whole pass for this rank's tokens."""

    def __init__(self, w13, w2, hidden, inter, cap, alphas1, alphas2, gscale1, gscale2, slab, fused_config=3,
                 config_id=0, cluster_m=2, fused_cluster_m=None, group=None, ops=None, world=None, rank=None,
                 exchange=None, peers=None):
        self.w13, self.w2 = w13, w2            # (a_comp, e_meta, sfa) each
        self.hidden, self.inter, self.cap, self.slab = hidden, inter, cap, slab
        self.al1, self.al2, self.g1, self.g2 = alphas1, alphas2, gscale1, gscale2
        self.fused_config, self.config_id, self.cluster_m = fused_config, config_id, cluster_m
        self.fused_cluster_m = cluster_m if fused_cluster_m is None else fused_cluster_m
        self.group = group
        self.ops = ops if ops is not None else _TorchOps()
        self.world = world if world is not None else dist.get_world_size(group)
        self.rank = rank if rank is not None else dist.get_rank(group)
        self.num_local = w13[0].size(0)
        self._exchange = exchange              # tests: a stand-in for the all-to-all
        self.peers = peers                     # PeerBuffers: the direct exchange instead of the all-to-alls

    # ---- the two halves either side of the exchanges -----------------------------------------------

    def plan_and_pack(self, x, topk_ids, mark=None):
        """-> (wire rows [world * slab, row bytes], slot of every routing int32 [tokens, topk] or -1)."""
        ops, mark = self.ops, mark or (lambda name: None)
        dest_rank = torch.div(topk_ids, self.num_local, rounding_mode="floor")
        slab_counts, route_slot, slot_tok, slot_route = ops.dispatch_plan(dest_rank, 0, self.world, self.slab)
        mark("send_plan")
        q, q_sf = ops.quant_rows(x, self.g1)
        mark("quant_rows")
        wire = ops.pack_wire_rows(q, q_sf, topk_ids, slot_tok, slot_route, slab_counts, self.slab, self.num_local)
        mark("pack_wire_rows")
        return wire, route_slot

    def exchange(self, rows):
        """Slab w of `rows` goes to rank w; slab w of the result came from rank w."""
        if self._exchange is not None:
            return self._exchange(rows)
        if self.world == 1:
            return rows
        out = torch.empty_like(rows)
        dist.all_to_all_single(out, rows, group=self.group)
        return out

    def local_ffn(self, wire, mark=None):
        """Received wire rows -> (expert output rows in slot order [world * slab, hidden], counts)."""
        ops, mark = self.ops, mark or (lambda name: None)
        E, H, I, cap = self.num_local, self.hidden, self.inter, self.cap
        counts, route_dest, src_tok, _ = ops.dispatch_plan(ops.wire_expert_ids(wire), 0, E, cap)
        mark("dispatch_plan")
        b1, sfb1 = ops.scatter_fp4_wire(wire, H, src_tok, counts, cap)
        mark("scatter_fp4_wire")
        b2, sfb2 = ops.group_mm_swiglu_quant(self.w13[0], self.w13[1], self.w13[2], b1, sfb1, self.al1, counts, self.g2,
                                             2 * I, H, self.fused_config, self.fused_cluster_m, 1, "silu", 1.0, -1.0)
        mark("group_mm_gate_up")
        # the receiver's plan has one routing per wire row, so its src_tok is the slot every expert row came from
        back = torch.empty((wire.size(0), H), dtype=torch.bfloat16, device=wire.device)
        ops.zero_rows(back, route_dest.view(-1))             # dead and dropped slots return zero rows
        mark("zero_rows")
        ops.group_mm_rows(back, src_tok, self.w2[0], self.w2[1], self.w2[2], b2, sfb2, self.al2, counts, H, I,
                          self.config_id, self.cluster_m, 1)
        mark("group_mm_down")
        return back, counts

    # ---- the direct exchange: the same pass with the rows stored where they are wanted ----------------

    def send_direct(self, x, topk_ids, mark=None):
        """plan + quantize + pack, the wire rows going straight into the receivers' buffers.  -> slot map."""
        ops, mark = self.ops, mark or (lambda name: None)
        dest_rank = torch.div(topk_ids, self.num_local, rounding_mode="floor")
        slab_counts, route_slot, slot_tok, slot_route = ops.dispatch_plan(dest_rank, 0, self.world, self.slab)
        mark("send_plan")
        q, q_sf = ops.quant_rows(x, self.g1)
        mark("quant_rows")
        ops.pack_wire_rows_parts(q, q_sf, topk_ids, slot_tok, slot_route, slab_counts, self.slab, self.num_local,
                                 self.peers.recv_parts())
        mark("pack_wire_rows")
        return route_slot

    def local_ffn_direct(self, mark=None):
        """The local FFN on this rank's receive buffer, expert outputs stored into the senders' return buffers."""
        ops, mark = self.ops, mark or (lambda name: None)
        E, H, I, cap = self.num_local, self.hidden, self.inter, self.cap
        wire = self.peers.recv_own
        ids = ops.wire_expert_ids(wire)
        counts, route_dest, src_tok, _ = ops.dispatch_plan(ids, 0, E, cap)
        mark("dispatch_plan")
        b1, sfb1 = ops.scatter_fp4_wire(wire, H, src_tok, counts, cap)
        mark("scatter_fp4_wire")
        b2, sfb2 = ops.group_mm_swiglu_quant(self.w13[0], self.w13[1], self.w13[2], b1, sfb1, self.al1, counts, self.g2,
                                             2 * I, H, self.fused_config, self.fused_cluster_m, 1, "silu", 1.0, -1.0)
        mark("group_mm_gate_up")
        parts = self.peers.ret_parts()
        # live rows this rank had no room for come back as zeros; dead slots are never read by their sender
        dropped = torch.where(ids.reshape(-1) >= 0, route_dest.view(-1), torch.zeros_like(route_dest.view(-1)))
        ops.zero_rows_parts(parts, dropped)
        mark("zero_rows")
        ops.group_mm_rows_parts(parts, src_tok, self.w2[0], self.w2[1], self.w2[2], b2, sfb2, self.al2, counts, H, I,
                                self.config_id, self.cluster_m, 1)
        mark("group_mm_down")
        return counts

    def forward_direct(self, x, topk_ids, topk_weights, out=None, mark=None):
        mark = mark or (lambda name: None)
        route_slot = self.send_direct(x, topk_ids, mark)
        self.peers.fence()                     # every rank's wire rows are in place
        mark("all_to_all_dispatch")
        counts = self.local_ffn_direct(mark)
        self.peers.fence()                     # every rank's expert outputs are in place
        mark("all_to_all_combine")
        if out is None:
            out = torch.empty((x.size(0), self.hidden), dtype=torch.bfloat16, device=x.device)
        self.ops.moe_finalize(out, self.peers.ret_own, route_slot, topk_weights)
        mark("moe_finalize")
        return out, counts, route_slot

    def forward(self, x, topk_ids, topk_weights, out=None, mark: Optional[Callable[[str], None]] = None):
        """x bf16 [tokens, hidden], topk_ids int32/int64 [tokens, topk] (global expert ids), topk_weights
        float32 [tokens, topk] or None.  Returns (out, local expert counts, slot map of this rank's routings)."""
        if self.peers is not None:
            return self.forward_direct(x, topk_ids, topk_weights, out, mark)
        mark = mark or (lambda name: None)
        wire, route_slot = self.plan_and_pack(x, topk_ids, mark)
        recv = self.exchange(wire)
        mark("all_to_all_dispatch")
        back, counts = self.local_ffn(recv, mark)
        ret = self.exchange(back)
        mark("all_to_all_combine")
        if out is None:
            out = torch.empty((x.size(0), self.hidden), dtype=torch.bfloat16, device=x.device)
        self.ops.moe_finalize(out, ret, route_slot, topk_weights)
        mark("moe_finalize")
        return out, counts, route_slot
