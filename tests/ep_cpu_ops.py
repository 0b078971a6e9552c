"""A CPU stand-in for torch.ops.paired_nvfp4 built on the numpy oracle, with the method names and tensor
shapes paired_nvfp4_kernels.ep uses.  It lets the expert-parallel forward (plan, pack, the two exchanges, local
FFN, finalize) run over gloo process groups without a GPU.  Test infrastructure only: the product path takes
its kernels from the CUDA library and has no such branch.

"Weights" are dequantised float32 tensors [E_local, M, K] in the first slot of the (a_comp, e_meta, sfa)
triples; w13 is [gate | up] halves, not interleaved."""
import numpy as np
import torch

from oracle import paired_nvfp4_oracle as orc


def _np(t):
    return t.detach().cpu().numpy()


def _bits(t):
    return _np(t.contiguous().view(torch.int16)).view(np.uint16)


def _from_bits(b):
    return torch.from_numpy(np.ascontiguousarray(b).view(np.int16)).view(torch.bfloat16)


class CpuOps:
    def dispatch_plan(self, ids, first, num_local, cap):
        c, rd, st, sr = orc.dispatch_plan(_np(ids).astype(np.int64), first, num_local, cap)
        return tuple(torch.from_numpy(a) for a in (c, rd, st, sr))

    def quant_rows(self, x, gscale):
        q, sf = orc.quant_rows(_bits(x), _np(gscale))
        return torch.from_numpy(q), torch.from_numpy(sf)

    def pack_wire_rows(self, q, q_sf, ids, slot_tok, slot_route, slab_counts, slab, epr):
        wire, _ = orc.pack_wire_rows(_np(q), _np(q_sf), _np(ids), _np(slot_tok), _np(slot_route), _np(slab_counts),
                                     slab, epr)
        return torch.from_numpy(wire)

    def wire_expert_ids(self, wire):
        rb = wire.size(1)
        return wire.view(torch.int32)[:, rb // 4 - 4: rb // 4 - 3]

    def scatter_fp4_wire(self, wire, k, src_tok, counts, cap):
        q, q_sf, _ = orc.unpack_wire_rows(_np(wire), k)
        b, _, sfb = orc.scatter_fp4_planned(q, q_sf, _np(src_tok), _np(counts), cap)
        return torch.from_numpy(b), torch.from_numpy(sfb)

    def group_mm_swiglu_quant(self, w, _e, _s, b1, sfb1, alphas, counts, gscale, features, k, cfg, cm, cn, act, beta, lb):
        o = orc.group_mm(_np(w), _np(b1), _np(sfb1), _np(alphas), _np(counts))
        b2, _, sfb2, _ = orc.silu_mul_quant_act(orc.f32_to_bf16_bits(o), _np(gscale), _np(counts))
        return torch.from_numpy(b2), torch.from_numpy(sfb2)

    def group_mm(self, out, w, _e, _s, b2, sfb2, alphas, counts, features, k, cfg, cm, cn):
        o = orc.group_mm(_np(w), _np(b2), _np(sfb2), _np(alphas), _np(counts))
        cnt = _np(counts)
        for e in range(o.shape[0]):
            out[e, :int(cnt[e])] = _from_bits(orc.f32_to_bf16_bits(o[e, :int(cnt[e])]))

    def group_mm_rows(self, out, row_map, w, _e, _s, b2, sfb2, alphas, counts, features, k, cfg, cm, cn):
        o = orc.group_mm(_np(w), _np(b2), _np(sfb2), _np(alphas), _np(counts))
        cnt, to = _np(counts), _np(row_map).reshape(o.shape[0], -1)
        for e in range(o.shape[0]):
            for r in range(int(cnt[e])):
                if to[e, r] >= 0:
                    out[int(to[e, r])] = _from_bits(orc.f32_to_bf16_bits(o[e, r]))

    def zero_rows(self, dst, flags):
        dst[flags < 0] = 0

    def gather_rows(self, src, idx):
        i = idx.long()
        out = src[i.clamp(min=0)].clone()
        out[i < 0] = 0
        return out

    def moe_finalize(self, out, fused, route_dest, w):
        bits = orc.moe_finalize(_bits(fused), _np(route_dest), None if w is None else _np(w))
        out.copy_(_from_bits(bits))
