"""torch.ops.paired_nvfp4.* : argument validation, output allocation, stream lookup, then one call
into the C ABI.  Mirrors the reference's op layer (csrc/ops.cu) schema for schema: same names,
argument meaning, output shapes and error substrings.  Every forward op only enqueues work on the
current CUDA stream of the tensors' device; nothing synchronises or reads device memory.
"""
import ctypes

import torch

from . import _cabi

_lib = _cabi.lib
SF_BLOCK = 32
_ARCH_SM = 100
_dev_info = {}


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg() if callable(msg) else msg)


_sm_margin = 0


def set_sm_margin(n):
    """Leave `n` SMs out of every persistent launch (the kernels size their grids from the SM count passed
    in), so that a collective running on another stream finds SMs to run on.  0 restores full-width launches."""
    global _sm_margin
    _sm_margin = max(0, int(n))


def _device_info(device):
    """(sm_version, sm_count) of a CUDA device, queried once (reference: csrc/ops.cu:86-103)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    info = _dev_info.get(idx)
    if info is None:
        props = torch.cuda.get_device_properties(idx)
        info = (props.major * 10 + props.minor, props.multi_processor_count)
        _dev_info[idx] = info
    if _sm_margin:
        return info[0], max(1, info[1] - _sm_margin)
    return info


def _check_arch(t):
    v = _device_info(t.device)[0]
    _check(v == _ARCH_SM, lambda: f"paired_nvfp4 ops in this module are built for SM{_ARCH_SM} but the tensor "
                                  f"is on a compute capability {v // 10}.{v % 10} device")


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _check_gscale_counts(gscale, counts, E):
    _check(gscale.dtype == torch.float32, "gscale must be float32")
    _check(gscale.numel() == E or gscale.numel() == 1, "gscale must be [E] (per expert) or [1] (shared)")
    _check(counts.dtype == torch.int32 and counts.numel() == E, "expert_num_tokens must be [E] int32")
    _check(gscale.is_contiguous() and counts.is_contiguous(), "gscale and expert_num_tokens must be contiguous")


def _act_kind(activation, beta):
    if activation == "silu":
        return 0
    if activation == "situ":
        _check(beta > 0, lambda: f"situ: beta must be positive, got {beta}")
        return 1
    raise RuntimeError(f"activation must be 'silu' or 'situ', got '{activation}'")


def compress(w_packed, w_blockscale, k):
    """csrc/ops.cu:156-223."""
    _check(w_packed.is_cuda and w_blockscale.is_cuda, "inputs must be CUDA tensors")
    _check_arch(w_packed)
    _check(w_packed.dim() == 3, "w_packed must be [E, out_features, K/2]")
    _check(w_blockscale.dim() == 3, "w_blockscale must be [E, out_features, ceil(K/SFVecSize)]")
    _check(w_packed.is_contiguous() and w_blockscale.is_contiguous(), "inputs must be contiguous")
    _check(w_packed.dtype == torch.uint8, "w_packed must be uint8 (2 e2m1 per byte)")
    E, M, K = w_packed.size(0), w_packed.size(1), int(k)
    _check(K % 2 == 0 and w_packed.size(2) == K // 2, "w_packed last dim must equal K/2")
    _check(w_blockscale.size(0) == E and w_blockscale.size(1) == M,
           "w_blockscale must match w_packed in [E, out_features]")
    kb = (K + SF_BLOCK - 1) // SF_BLOCK
    _check(w_blockscale.size(2) == kb,
           lambda: f"w_blockscale last dim must be ceil(K/{SF_BLOCK}) = {kb}, got {w_blockscale.size(2)}. The "
                   f"sparse NVFP4 MMA uses one scale per {SF_BLOCK} dense K elements; checkpoints quantized "
                   "with 16-element groups are incompatible")
    _check(w_blockscale.element_size() == 1, "w_blockscale must be a 1-byte (e4m3) dtype")
    m_ac, k_ac, m_e, k_e = _cabi.physical_dims(M, K)
    dev = w_packed.device
    a_comp = torch.empty((E, m_ac, k_ac // 2), dtype=torch.uint8, device=dev)
    e_meta = torch.empty((E, m_e, k_e), dtype=torch.uint8, device=dev)
    sfa = torch.empty((_cabi.sf_numel(M, K, E),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(_lib.pnv_compress(w_packed.data_ptr(), w_blockscale.data_ptr(), E, M, K, a_comp.data_ptr(),
                                      e_meta.data_ptr(), sfa.data_ptr(), _stream(w_packed)))
    return a_comp, e_meta, sfa


def quant_act(x, gscale, expert_num_tokens, features):
    """csrc/ops.cu:230-262.  `features` is accepted for API symmetry; the layouts do not use it."""
    _check(x.is_cuda and gscale.is_cuda and expert_num_tokens.is_cuda, "inputs must be CUDA")
    _check_arch(x)
    _check(x.dim() == 3, "x must be [E, max_n, K]")
    _check(x.dtype == torch.bfloat16 and x.is_contiguous(), "x must be contiguous bf16")
    E, max_n, K = x.shape
    _check(K % SF_BLOCK == 0, lambda: f"K must be a multiple of {SF_BLOCK}, got {K}")
    _check_gscale_counts(gscale, expert_num_tokens, E)
    gpe = 1 if gscale.numel() == E else 0
    b_act = torch.empty((E, max_n, K // 2), dtype=torch.uint8, device=x.device)
    sfb = torch.empty((_cabi.sf_numel(max_n, K, E),), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _cabi.check(_lib.pnv_quant_act(x.data_ptr(), gscale.data_ptr(), gpe, expert_num_tokens.data_ptr(), E, max_n,
                                       K, b_act.data_ptr(), sfb.data_ptr(), _device_info(x.device)[1], _stream(x)))
    return b_act, sfb


def silu_mul_quant_act(x2, gscale, expert_num_tokens, features, interleaved=False, activation="silu",
                       beta=1.0, linear_beta=-1.0):
    """csrc/ops.cu:269-306."""
    _check(x2.is_cuda and gscale.is_cuda and expert_num_tokens.is_cuda, "inputs must be CUDA")
    _check_arch(x2)
    _check(x2.dim() == 3, "x2 must be [E, max_n, 2N] ([gate | up] halves)")
    _check(x2.dtype == torch.bfloat16 and x2.is_contiguous(), "x2 must be contiguous bf16")
    E, max_n = x2.size(0), x2.size(1)
    _check(x2.size(2) % 2 == 0, lambda: f"x2 last dim must be even ([gate | up]), got {x2.size(2)}")
    N = x2.size(2) // 2
    _check(N % SF_BLOCK == 0, lambda: f"intermediate width N must be a multiple of {SF_BLOCK}, got {N}")
    _check_gscale_counts(gscale, expert_num_tokens, E)
    gpe = 1 if gscale.numel() == E else 0
    kind = _act_kind(activation, beta)
    b_act = torch.empty((E, max_n, N // 2), dtype=torch.uint8, device=x2.device)
    sfb = torch.empty((_cabi.sf_numel(max_n, N, E),), dtype=torch.uint8, device=x2.device)
    with torch.cuda.device(x2.device):
        _cabi.check(_lib.pnv_silu_mul_quant_act(
            x2.data_ptr(), gscale.data_ptr(), gpe, expert_num_tokens.data_ptr(), E, max_n, N, 1 if interleaved else 0,
            kind, float(beta), float(linear_beta), b_act.data_ptr(), sfb.data_ptr(), _device_info(x2.device)[1],
            _stream(x2)))
    return b_act, sfb


def scatter_quant_act(a1, flat_tok, dest_global, topk_weights, gscale, expert_num_tokens, cap):
    """csrc/ops.cu:314-367.  expert_num_tokens only supplies E."""
    _check(a1.is_cuda and flat_tok.is_cuda and dest_global.is_cuda and gscale.is_cuda and expert_num_tokens.is_cuda,
           "inputs must be CUDA")
    _check_arch(a1)
    _check(a1.dim() == 2, "a1 must be [T, K] (token-order hidden states)")
    _check(a1.dtype == torch.bfloat16 and a1.is_contiguous(), "a1 must be contiguous bf16")
    K = a1.size(1)
    _check(K % SF_BLOCK == 0, lambda: f"K must be a multiple of {SF_BLOCK}, got {K}")
    _check(flat_tok.dtype == torch.int64 and dest_global.dtype == torch.int64, "flat_tok and dest_global must be int64")
    _check(flat_tok.dim() == 1 and dest_global.dim() == 1 and flat_tok.numel() == dest_global.numel(),
           "flat_tok and dest_global must be same-length 1D")
    _check(flat_tok.is_contiguous() and dest_global.is_contiguous(), "plan tensors must be contiguous")
    _check(cap > 0, "cap must be positive")
    n = flat_tok.numel()
    E = expert_num_tokens.numel()
    _check_gscale_counts(gscale, expert_num_tokens, E)
    gpe = 1 if gscale.numel() == E else 0
    w_ptr = None
    if topk_weights is not None:
        _check(topk_weights.is_cuda and topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
               and topk_weights.numel() == n, "topk_weights must be contiguous float32 [N]")
        w_ptr = topk_weights.data_ptr()
    # one extra trailing row, as in the reference: b_act is a view of an (E*cap + 1)-row buffer
    b_ext = torch.empty((E * cap + 1, K // 2), dtype=torch.uint8, device=a1.device)
    b_act = b_ext.narrow(0, 0, E * cap).view(E, cap, K // 2)
    sfb = torch.empty((_cabi.sf_numel(cap, K, E),), dtype=torch.uint8, device=a1.device)
    with torch.cuda.device(a1.device):
        _cabi.check(_lib.pnv_scatter_quant_act(
            a1.data_ptr(), flat_tok.data_ptr(), dest_global.data_ptr(), w_ptr, gscale.data_ptr(), gpe, n, K, E,
            int(cap), b_ext.data_ptr(), sfb.data_ptr(), _device_info(a1.device)[1], _stream(a1)))
    return b_act, sfb


def dispatch_plan(topk_ids, first_expert, num_local_experts, cap):
    """csrc/ops.cu:374-411.  Returns (expert_num_tokens, route_dest, src_tok, src_route).

    Beyond the reference's contiguous [T, topk] ids, a [T, 1] view with a row stride is accepted (one id per
    row of a wider buffer: the expert ids inside the wire rows of an expert-parallel dispatch)."""
    _check(topk_ids.is_cuda, "topk_ids must be CUDA")
    _check(topk_ids.dim() == 2, "topk_ids must be [T, topk]")
    strided = (not topk_ids.is_contiguous()) and topk_ids.size(1) == 1 and topk_ids.stride(0) >= 1
    _check(topk_ids.is_contiguous() or strided, "topk_ids must be contiguous [T, topk] (or a strided [T, 1] view)")
    _check(topk_ids.dtype in (torch.int32, torch.int64), "topk_ids must be int32 or int64")
    E = int(num_local_experts)
    _check(1 <= E <= 4096, lambda: f"num_local_experts must be in [1, 4096], got {E}")
    _check(cap >= 1, "cap must be positive")
    _check(E * cap < (1 << 31), "E * cap must fit int32")
    T, topk = topk_ids.shape
    _check(T * topk < (1 << 31), "T * topk must fit int32")
    i32 = dict(dtype=torch.int32, device=topk_ids.device)
    counts = torch.empty((E,), **i32)
    route_dest = torch.empty((T, topk), **i32)
    src_tok = torch.empty((E * cap,), **i32)
    src_route = torch.empty((E * cap,), **i32)
    n_scratch = int(_lib.pnv_dispatch_plan_scratch_ints(T * topk, E))
    scratch = torch.empty((max(n_scratch, 1),), **i32)
    with torch.cuda.device(topk_ids.device):
        _cabi.check(_lib.pnv_dispatch_plan_strided(
            topk_ids.data_ptr(), 1 if topk_ids.dtype == torch.int64 else 0, topk_ids.stride(0) if strided else 1, T, topk,
            int(first_expert), E, int(cap), counts.data_ptr(), route_dest.data_ptr(), src_tok.data_ptr(),
            src_route.data_ptr(), scratch.data_ptr(), _stream(topk_ids)))
    return counts, route_dest, src_tok, src_route


def scatter_quant_act_planned(a1, src_tok, src_route, topk_weights, gscale, expert_num_tokens, cap):
    """csrc/ops.cu:418-468."""
    _check(a1.is_cuda and src_tok.is_cuda and src_route.is_cuda and gscale.is_cuda and expert_num_tokens.is_cuda,
           "inputs must be CUDA")
    _check_arch(a1)
    _check(a1.dim() == 2, "a1 must be [T, K] (token-order hidden states)")
    _check(a1.dtype == torch.bfloat16 and a1.is_contiguous(), "a1 must be contiguous bf16")
    K = a1.size(1)
    _check(K % SF_BLOCK == 0, lambda: f"K must be a multiple of {SF_BLOCK}, got {K}")
    E = expert_num_tokens.numel()
    _check_gscale_counts(gscale, expert_num_tokens, E)
    _check(cap > 0, "cap must be positive")
    _check(src_tok.dtype == torch.int32 and src_route.dtype == torch.int32 and src_tok.is_contiguous()
           and src_route.is_contiguous() and src_tok.numel() == E * cap and src_route.numel() == E * cap,
           "src_tok and src_route must be contiguous int32 [E * cap] (dispatch_plan output)")
    w_ptr = None
    if topk_weights is not None:
        _check(topk_weights.is_cuda and topk_weights.dtype == torch.float32 and topk_weights.is_contiguous(),
               "topk_weights must be contiguous float32 [T * topk]")
        w_ptr = topk_weights.data_ptr()
    b_act = torch.empty((E, cap, K // 2), dtype=torch.uint8, device=a1.device)
    sfb = torch.empty((_cabi.sf_numel(cap, K, E),), dtype=torch.uint8, device=a1.device)
    with torch.cuda.device(a1.device):
        _cabi.check(_lib.pnv_scatter_quant_act_planned(
            a1.data_ptr(), src_tok.data_ptr(), src_route.data_ptr(), w_ptr, gscale.data_ptr(),
            1 if gscale.numel() == E else 0, expert_num_tokens.data_ptr(), K, E, int(cap), b_act.data_ptr(),
            sfb.data_ptr(), _device_info(a1.device)[1], _stream(a1)))
    return b_act, sfb


def quant_rows(x, gscale):
    """csrc/ops.cu:476-500."""
    _check(x.is_cuda and gscale.is_cuda, "inputs must be CUDA")
    _check_arch(x)
    _check(x.dim() == 2 and x.dtype == torch.bfloat16 and x.is_contiguous(), "x must be contiguous bf16 [T, K]")
    T, K = x.shape
    _check(K % SF_BLOCK == 0, lambda: f"K must be a multiple of {SF_BLOCK}, got {K}")
    _check(gscale.dtype == torch.float32 and gscale.numel() >= 1,
           "gscale must be float32 with the shared global scale first")
    q = torch.empty((T, K // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty((T, K // SF_BLOCK), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _cabi.check(_lib.pnv_quant_rows(x.data_ptr(), gscale.data_ptr(), T, K, q.data_ptr(), sf.data_ptr(),
                                        _device_info(x.device)[1], _stream(x)))
    return q, sf


def scatter_fp4_planned(q, q_sf, src_tok, expert_num_tokens, cap):
    """csrc/ops.cu:502-541."""
    _check(q.is_cuda and q_sf.is_cuda and src_tok.is_cuda and expert_num_tokens.is_cuda, "inputs must be CUDA")
    _check_arch(q)
    _check(q.dim() == 2 and q.dtype == torch.uint8 and q.is_contiguous(),
           "q must be contiguous uint8 [T, K/2] (quant_rows output)")
    K = q.size(1) * 2
    _check(K % SF_BLOCK == 0, lambda: f"K must be a multiple of {SF_BLOCK}, got {K}")
    _check(q_sf.dim() == 2 and q_sf.size(0) == q.size(0) and q_sf.size(1) == K // SF_BLOCK and q_sf.element_size() == 1
           and q_sf.is_contiguous(), lambda: f"q_sf must be contiguous 1-byte [T, K/{SF_BLOCK}] (quant_rows output)")
    E = expert_num_tokens.numel()
    _check(expert_num_tokens.dtype == torch.int32 and expert_num_tokens.is_contiguous(),
           "expert_num_tokens must be contiguous int32 [E]")
    _check(cap > 0, "cap must be positive")
    _check(src_tok.dtype == torch.int32 and src_tok.is_contiguous() and src_tok.numel() == E * cap,
           "src_tok must be contiguous int32 [E * cap] (dispatch_plan output)")
    b_act = torch.empty((E, cap, K // 2), dtype=torch.uint8, device=q.device)
    sfb = torch.empty((_cabi.sf_numel(cap, K, E),), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        _cabi.check(_lib.pnv_scatter_fp4_planned(q.data_ptr(), q_sf.data_ptr(), src_tok.data_ptr(),
                                                 expert_num_tokens.data_ptr(), K, E, int(cap), b_act.data_ptr(),
                                                 sfb.data_ptr(), _device_info(q.device)[1], _stream(q)))
    return b_act, sfb


def wire_row_bytes(k):
    """Bytes of one wire row of the expert-parallel dispatch for hidden size k."""
    return int(_lib.pnv_wire_row_bytes(int(k)))


def _check_pack_args(q, q_sf, topk_ids, slot_tok, slot_route, slab_counts, slab, experts_per_rank):
    _check(q.is_cuda and q_sf.is_cuda and topk_ids.is_cuda and slot_tok.is_cuda and slot_route.is_cuda
           and slab_counts.is_cuda, "inputs must be CUDA")
    _check_arch(q)
    _check(q.dim() == 2 and q.dtype == torch.uint8 and q.is_contiguous(), "q must be contiguous uint8 [T, K/2]")
    K = q.size(1) * 2
    _check(K % SF_BLOCK == 0, lambda: f"K must be a multiple of {SF_BLOCK}, got {K}")
    _check(q_sf.dim() == 2 and q_sf.size(0) == q.size(0) and q_sf.size(1) == K // SF_BLOCK and q_sf.element_size() == 1
           and q_sf.is_contiguous(), lambda: f"q_sf must be contiguous 1-byte [T, K/{SF_BLOCK}]")
    _check(topk_ids.dtype in (torch.int32, torch.int64) and topk_ids.is_contiguous(), "topk_ids must be contiguous int32/int64")
    ranks = slab_counts.numel()
    _check(slab_counts.dtype == torch.int32 and slab_counts.is_contiguous(), "slab_counts must be contiguous int32 [ranks]")
    _check(slab >= 1 and experts_per_rank >= 1, "slab and experts_per_rank must be positive")
    _check(slot_tok.dtype == torch.int32 and slot_route.dtype == torch.int32 and slot_tok.is_contiguous()
           and slot_route.is_contiguous() and slot_tok.numel() == ranks * slab and slot_route.numel() == ranks * slab,
           "slot_tok and slot_route must be contiguous int32 [ranks * slab] (dispatch_plan output)")
    return K, ranks


def _parts_array(parts, rows, width, dtype, what):
    """A host array of the parts' device pointers, after shape checks (each part [rows, width] of dtype)."""
    _check(1 <= len(parts) <= 16, lambda: f"{what}: between 1 and 16 parts, got {len(parts)}")
    for t in parts:
        _check(t.is_cuda and t.dtype == dtype and t.dim() == 2 and t.is_contiguous() and t.size(0) == rows
               and t.size(1) == width, lambda: f"{what}: every part must be contiguous CUDA {dtype} [{rows}, {width}]")
    return (ctypes.c_void_p * len(parts))(*[t.data_ptr() for t in parts])


def pack_wire_rows(q, q_sf, topk_ids, slot_tok, slot_route, slab_counts, slab, experts_per_rank):
    """quant_rows output -> wire rows in fixed-capacity slabs, one slab of `slab` rows per destination rank
    (see pnv_pack_wire_rows).  slot_tok / slot_route / slab_counts are dispatch_plan's outputs for the routings
    keyed by destination rank.  Returns uint8 [ranks * slab, wire_row_bytes(K)]."""
    K, ranks = _check_pack_args(q, q_sf, topk_ids, slot_tok, slot_route, slab_counts, slab, experts_per_rank)
    wire = torch.empty((ranks * slab, wire_row_bytes(K)), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        _cabi.check(_lib.pnv_pack_wire_rows(q.data_ptr(), q_sf.data_ptr(), topk_ids.data_ptr(),
                                            1 if topk_ids.dtype == torch.int64 else 0, slot_tok.data_ptr(),
                                            slot_route.data_ptr(), slab_counts.data_ptr(), ranks, int(slab),
                                            int(experts_per_rank), K, wire.data_ptr(), _stream(q)))
    return wire


def pack_wire_rows_parts(q, q_sf, topk_ids, slot_tok, slot_route, slab_counts, slab, experts_per_rank, wire_parts):
    """pack_wire_rows with slab w written into wire_parts[w] (uint8 [slab, wire_row_bytes(K)] each, possibly another
    GPU's memory opened in this process): the pack is then the dispatch.  Mutates the parts."""
    K, ranks = _check_pack_args(q, q_sf, topk_ids, slot_tok, slot_route, slab_counts, slab, experts_per_rank)
    _check(len(wire_parts) == ranks, lambda: f"one wire part per destination rank: {ranks}, got {len(wire_parts)}")
    arr = _parts_array(wire_parts, int(slab), wire_row_bytes(K), torch.uint8, "pack_wire_rows_parts")
    with torch.cuda.device(q.device):
        _cabi.check(_lib.pnv_pack_wire_rows_parts(q.data_ptr(), q_sf.data_ptr(), topk_ids.data_ptr(),
                                                  1 if topk_ids.dtype == torch.int64 else 0, slot_tok.data_ptr(),
                                                  slot_route.data_ptr(), slab_counts.data_ptr(), ranks, int(slab),
                                                  int(experts_per_rank), K, arr, _stream(q)))


def wire_expert_ids(wire):
    """The [rows, 1] int32 view of the expert ids inside wire rows (input of dispatch_plan on the receiver)."""
    _check(wire.dim() == 2 and wire.dtype == torch.uint8 and wire.is_contiguous() and wire.size(1) % 16 == 0,
           "wire must be contiguous uint8 [rows, wire_row_bytes(K)]")
    rb = wire.size(1)
    return wire.view(torch.int32)[:, rb // 4 - 4: rb // 4 - 3]


def scatter_fp4_wire(wire, k, src_tok, expert_num_tokens, cap):
    """Received wire rows -> group_mm's activation operands, as scatter_fp4_planned does for separate code and
    scale tensors (csrc/ops.cu:502-541)."""
    _check(wire.is_cuda and src_tok.is_cuda and expert_num_tokens.is_cuda, "inputs must be CUDA")
    _check_arch(wire)
    K = int(k)
    _check(K % SF_BLOCK == 0, lambda: f"K must be a multiple of {SF_BLOCK}, got {K}")
    _check(wire.dim() == 2 and wire.dtype == torch.uint8 and wire.is_contiguous() and wire.size(1) == wire_row_bytes(K),
           "wire must be contiguous uint8 [rows, wire_row_bytes(K)]")
    E = expert_num_tokens.numel()
    _check(expert_num_tokens.dtype == torch.int32 and expert_num_tokens.is_contiguous(),
           "expert_num_tokens must be contiguous int32 [E]")
    _check(cap > 0, "cap must be positive")
    _check(src_tok.dtype == torch.int32 and src_tok.is_contiguous() and src_tok.numel() == E * cap,
           "src_tok must be contiguous int32 [E * cap] (dispatch_plan output)")
    b_act = torch.empty((E, cap, K // 2), dtype=torch.uint8, device=wire.device)
    sfb = torch.empty((_cabi.sf_numel(cap, K, E),), dtype=torch.uint8, device=wire.device)
    with torch.cuda.device(wire.device):
        _cabi.check(_lib.pnv_scatter_fp4_wire(wire.data_ptr(), src_tok.data_ptr(), expert_num_tokens.data_ptr(), K, E,
                                              int(cap), b_act.data_ptr(), sfb.data_ptr(), _device_info(wire.device)[1],
                                              _stream(wire)))
    return b_act, sfb


def moe_finalize(out, fused, route_dest, topk_weights):
    """csrc/ops.cu:548-575.  Mutates `out` in place."""
    _check(out.is_cuda and fused.is_cuda and route_dest.is_cuda, "inputs must be CUDA")
    _check(out.dim() == 2 and out.dtype == torch.bfloat16 and out.is_contiguous(), "out must be contiguous bf16 [T, K]")
    _check(fused.dtype == torch.bfloat16 and fused.is_contiguous() and fused.dim() >= 2,
           "fused must be contiguous bf16 [E, cap, K] (or [E * cap, K])")
    T, K = out.shape
    _check(fused.size(-1) == K, "fused and out must share K")
    _check(K % 8 == 0, "K must be a multiple of 8")
    _check(route_dest.dtype == torch.int32 and route_dest.is_contiguous() and route_dest.dim() == 2
           and route_dest.size(0) == T, "route_dest must be contiguous int32 [T, topk] (dispatch_plan output)")
    topk = route_dest.size(1)
    w_ptr = None
    if topk_weights is not None:
        _check(topk_weights.is_cuda and topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
               and topk_weights.numel() == T * topk, "topk_weights must be contiguous float32 [T, topk]")
        w_ptr = topk_weights.data_ptr()
    with torch.cuda.device(out.device):
        _cabi.check(_lib.pnv_moe_finalize(out.data_ptr(), fused.data_ptr(), route_dest.data_ptr(), w_ptr, T, topk, K,
                                          _stream(out)))


def set_silu_table(enabled):
    """Testing aid: evaluate SiLU through the library's lookup table (default) or directly."""
    _cabi.check(_lib.pnv_set_silu_table(1 if enabled else 0))


def gather_rows(src, idx):
    """dst[i] = src[idx[i]] for idx[i] >= 0, a zero row otherwise: the permutation step either side of
    the expert-parallel exchange (token rows into send order, expert outputs into return order)."""
    _check(src.is_cuda and idx.is_cuda, "inputs must be CUDA")
    _check(src.dim() == 2 and src.is_contiguous(), "src must be contiguous [rows, width]")
    _check(idx.dtype == torch.int32 and idx.is_contiguous() and idx.dim() == 1, "idx must be contiguous int32 [n]")
    row_bytes = src.size(1) * src.element_size()
    _check(row_bytes % 16 == 0, lambda: f"rows must be a multiple of 16 bytes, got {row_bytes}")
    dst = torch.empty((idx.numel(), src.size(1)), dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device):
        _cabi.check(_lib.pnv_gather_rows(src.data_ptr(), idx.data_ptr(), idx.numel(), row_bytes, dst.data_ptr(),
                                         _stream(src)))
    return dst


def gated_act(x2, interleaved=False, activation="silu", beta=1.0, linear_beta=-1.0):
    """The unfused gated activation (gated_act, csrc/layout.cuh:204-216): bf16 [..., 2N] -> [..., N]."""
    _check(x2.is_cuda and x2.dtype == torch.bfloat16 and x2.is_contiguous(), "x2 must be contiguous CUDA bf16")
    N = x2.size(-1) // 2
    _check(N % SF_BLOCK == 0, lambda: f"intermediate width N must be a multiple of {SF_BLOCK}, got {N}")
    kind = _act_kind(activation, beta)
    y = torch.empty(x2.shape[:-1] + (N,), dtype=torch.bfloat16, device=x2.device)
    rows = x2.numel() // (2 * N) if N else 0
    with torch.cuda.device(x2.device):
        _cabi.check(_lib.pnv_gated_act(x2.data_ptr(), rows, N, 1 if interleaved else 0, kind, float(beta),
                                       float(linear_beta), y.data_ptr(), _stream(x2)))
    return y


_workspaces = {}


def _split_workspace(t, experts, features, max_n):
    """(pointer, bytes) of the split-K workspace for a group_mm launch on t's device and current stream, or
    (None, 0) when the launch does not split.  The reference allocates its workspace inside the op as well
    (csrc/group_mm.cuh:163-165); here it is kept per (device, stream), zeroed once, because every launch
    leaves its counters zero.  Under stream capture a fresh zeroed buffer is made instead, so a graph never
    shares the buffer with work outside it."""
    sm = _device_info(t.device)[1]
    need = int(_lib.pnv_group_mm_workspace_bytes(int(experts), int(features), int(max_n), sm))
    if need == 0:
        return None, 0
    if torch.cuda.is_current_stream_capturing():
        ws = torch.zeros((need,), dtype=torch.uint8, device=t.device)
        return ws, need
    key = (t.device.index, torch.cuda.current_stream(t.device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros((need,), dtype=torch.uint8, device=t.device)
        _workspaces[key] = ws
    return ws, need


def group_mm_configs():
    """csrc/ops.cu:665-670."""
    return _cabi.group_mm_config_names()


def _group_mm(out, row_map, a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens, features, k, config_id,
              cluster_m, cluster_n, out_parts=None):
    ts = (a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens) + (() if out_parts is not None else (out,))
    _check(all(t.is_cuda for t in ts), "all tensors must be CUDA")
    _check_arch(b_act)
    _check(b_act.dim() == 3 and a_comp.dim() == 3 and e_meta.dim() == 3, "b_act, a_comp and e_meta must be 3D")
    E, M, K, max_n = a_comp.size(0), int(features), int(k), b_act.size(1)
    _check(b_act.size(0) == E and e_meta.size(0) == E, "expert dim mismatch")
    parts_arr = None
    if row_map is None:
        _check(out.dim() == 3, "out must be 3D")
        _check(out.size(0) == E, "expert dim mismatch")
        _check(out.size(1) == max_n and out.size(2) == M, "out must be [E, max_n, features]")
    else:
        _check(row_map.is_cuda and row_map.dtype == torch.int32 and row_map.is_contiguous()
               and row_map.numel() == E * max_n, "row_map must be contiguous int32 [E * max_n]")
        if out_parts is None:
            _check(out.dim() == 2 and out.size(1) == M, "out must be [rows, features]")
        else:
            _check(len(out_parts) >= 1, "at least one output part")
            parts_arr = _parts_array(out_parts, out_parts[0].size(0), M, torch.bfloat16, "group_mm_rows_parts")
    _check(b_act.size(2) == K // 2, "b_act must be [E, max_n, K/2]")
    _check(out_parts is not None or out.dtype == torch.bfloat16, "out must be bf16")
    _check(a_comp.dtype == torch.uint8 and e_meta.dtype == torch.uint8 and b_act.dtype == torch.uint8
           and sfa.element_size() == 1 and sfb.element_size() == 1,
           "a_comp, e_meta and b_act must be uint8; sfa, sfb 1-byte")
    _check(all(t.is_contiguous() for t in ts), "all group_mm tensors must be contiguous")
    _check(alphas.dtype == torch.float32 and alphas.numel() == E, "alphas must be [E] float32")
    _check(expert_num_tokens.dtype == torch.int32 and expert_num_tokens.numel() == E,
           "expert_num_tokens must be [E] int32 (real per-expert token counts, <= max_n)")
    m_ac, k_ac, m_e, k_e = _cabi.physical_dims(M, K)
    _check(a_comp.size(1) == m_ac and a_comp.size(2) == k_ac // 2 and e_meta.size(1) == m_e and e_meta.size(2) == k_e,
           lambda: f"a_comp / e_meta shapes do not match compress() output for features={M}, k={K} "
                   "(check the features / k arguments)")
    _check(sfa.numel() >= _cabi.sf_numel(M, K, E), "sfa is smaller than the SFA layout")
    _check(sfb.numel() >= _cabi.sf_numel(max_n, K, E), "sfb is smaller than the SFB layout")
    with torch.cuda.device(b_act.device):
        ws, ws_bytes = _split_workspace(b_act, E, M, max_n)
        tail = (a_comp.data_ptr(), e_meta.data_ptr(), sfa.data_ptr(), b_act.data_ptr(), sfb.data_ptr(),
                alphas.data_ptr(), expert_num_tokens.data_ptr(), E, M, K, max_n, int(config_id), int(cluster_m),
                int(cluster_n), _device_info(b_act.device)[1], 1, ws.data_ptr() if ws is not None else None, ws_bytes,
                _stream(b_act))
        if row_map is None:
            _cabi.check(_lib.pnv_group_mm(out.data_ptr(), *tail))
        elif parts_arr is None:
            _cabi.check(_lib.pnv_group_mm_rows(out.data_ptr(), row_map.data_ptr(), *tail))
        else:
            _cabi.check(_lib.pnv_group_mm_rows_parts(parts_arr, len(out_parts), out_parts[0].size(0), row_map.data_ptr(),
                                                     *tail))


def group_mm(out, a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens, features, k, config_id=0,
             cluster_m=2, cluster_n=1):
    """csrc/ops.cu:672-735.  Mutates `out` in place."""
    _group_mm(out, None, a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens, features, k, config_id,
              cluster_m, cluster_n)


def group_mm_rows(out, row_map, a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens, features, k, config_id=0,
                  cluster_m=2, cluster_n=1):
    """group_mm whose token row (e, t) lands in row row_map[e * max_n + t] of out [rows, features] (skipped where
    negative).  Mutates `out` in place; rows no kept token maps to are left alone."""
    _group_mm(out, row_map, a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens, features, k, config_id,
              cluster_m, cluster_n)


def group_mm_rows_parts(out_parts, row_map, a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens, features, k,
                        config_id=0, cluster_m=2, cluster_n=1):
    """group_mm_rows whose logical output [len(out_parts) * rows, features] is spread over out_parts (bf16
    [rows, features] each, possibly other GPUs' memory opened in this process).  Mutates the parts."""
    _group_mm(None, row_map, a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens, features, k, config_id,
              cluster_m, cluster_n, out_parts=list(out_parts))


def zero_rows_parts(parts, flags):
    """zero_rows over a parts table: flags [len(parts) * rows]; row q is row q % rows of parts[q // rows]."""
    _check(len(parts) >= 1 and flags.is_cuda, "inputs must be CUDA")
    rows, width = parts[0].size(0), parts[0].size(1)
    arr = _parts_array(parts, rows, width, parts[0].dtype, "zero_rows_parts")
    _check(flags.dtype == torch.int32 and flags.is_contiguous() and flags.numel() == len(parts) * rows,
           "flags must be contiguous int32 [parts * rows]")
    row_bytes = width * parts[0].element_size()
    _check(row_bytes % 16 == 0, lambda: f"rows must be a multiple of 16 bytes, got {row_bytes}")
    with torch.cuda.device(flags.device):
        _cabi.check(_lib.pnv_zero_rows_parts(arr, len(parts), rows, flags.data_ptr(), row_bytes, _stream(flags)))


def zero_rows(dst, flags):
    """dst[i] = 0 where flags[i] < 0; the other rows are left alone.  Mutates `dst` in place."""
    _check(dst.is_cuda and flags.is_cuda, "inputs must be CUDA")
    _check(dst.dim() == 2 and dst.is_contiguous(), "dst must be contiguous [rows, width]")
    _check(flags.dtype == torch.int32 and flags.is_contiguous() and flags.numel() == dst.size(0),
           "flags must be contiguous int32 [rows]")
    row_bytes = dst.size(1) * dst.element_size()
    _check(row_bytes % 16 == 0, lambda: f"rows must be a multiple of 16 bytes, got {row_bytes}")
    with torch.cuda.device(dst.device):
        _cabi.check(_lib.pnv_zero_rows(dst.data_ptr(), flags.data_ptr(), dst.size(0), row_bytes, _stream(dst)))


def group_mm_swiglu_configs():
    """csrc/ops.cu:585-589."""
    return _cabi.group_mm_swiglu_config_names()


def group_mm_swiglu_quant(a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens, gscale, features, k,
                          config_id=0, cluster_m=2, cluster_n=1, activation="silu", beta=1.0, linear_beta=-1.0):
    """csrc/ops.cu:591-658.  GEMM1 + gated activation + GEMM2's input quantization in one kernel;
    returns GEMM2's operands (b_act [E, max_n, N/2], sfb)."""
    ts = (a_comp, e_meta, sfa, b_act, sfb, alphas, expert_num_tokens, gscale)
    _check(all(t.is_cuda for t in ts), "all tensors must be CUDA")
    _check_arch(b_act)
    E, M, K, max_n = a_comp.size(0), int(features), int(k), b_act.size(1)
    N = M // 2
    _check(M % 128 == 0, lambda: "features (2N) must be a multiple of 128 (whole 64-row gate/up blocks per CTA), "
                                 f"got {M}")
    _check(b_act.dim() == 3 and b_act.size(0) == E and b_act.size(2) == K // 2, "b_act must be [E, max_n, K/2]")
    _check(all(t.is_contiguous() for t in (a_comp, e_meta, sfa, b_act, sfb, alphas)), "inputs must be contiguous")
    _check(alphas.dtype == torch.float32 and alphas.numel() == E, "alphas must be [E] float32")
    _check_gscale_counts(gscale, expert_num_tokens, E)
    m_ac, k_ac, m_e, k_e = _cabi.physical_dims(M, K)
    _check(a_comp.size(1) == m_ac and a_comp.size(2) == k_ac // 2 and e_meta.size(1) == m_e and e_meta.size(2) == k_e,
           lambda: f"a_comp / e_meta shapes do not match compress() output for features={M}, k={K}")
    _check(sfa.numel() >= _cabi.sf_numel(M, K, E), "sfa is smaller than the SFA layout")
    _check(sfb.numel() >= _cabi.sf_numel(max_n, K, E), "sfb is smaller than the SFB layout")
    kind = _act_kind(activation, beta)
    b_out = torch.empty((E, max_n, N // 2), dtype=torch.uint8, device=b_act.device)
    sfb_out = torch.empty((_cabi.sf_numel(max_n, N, E),), dtype=torch.uint8, device=b_act.device)
    with torch.cuda.device(b_act.device):
        ws, ws_bytes = _split_workspace(b_act, E, M, max_n)
        _cabi.check(_lib.pnv_group_mm_swiglu_quant(
            b_out.data_ptr(), sfb_out.data_ptr(), a_comp.data_ptr(), e_meta.data_ptr(), sfa.data_ptr(),
            b_act.data_ptr(), sfb.data_ptr(), alphas.data_ptr(), expert_num_tokens.data_ptr(), gscale.data_ptr(),
            1 if gscale.numel() == E else 0, E, M, K, max_n, int(config_id), int(cluster_m), int(cluster_n), kind,
            float(beta), float(linear_beta), _device_info(b_act.device)[1], 1,
            ws.data_ptr() if ws is not None else None, ws_bytes, _stream(b_act)))
    return b_out, sfb_out


def group_mm_device_status():
    """Status word of the bounded waits inside group_mm (0 = all completed); synchronises."""
    import ctypes
    v = ctypes.c_int()
    _cabi.check(_lib.pnv_group_mm_device_status(ctypes.byref(v)))
    return v.value
