"""paired_nvfp4_kernels for B200 (sm_100a): paired-4:8 sparse NVFP4 grouped MoE GEMM ops.

Importing this package loads ``libpaired_nvfp4_b200.so`` (hand-written sm_100a CUDA behind a C ABI)
and registers ``torch.ops.paired_nvfp4.*`` with the reference project's operator schemas
(csrc/ops.cu:739-773), so code written against the reference's package runs unchanged.  The helper
surface of the reference's ``paired_nvfp4_kernels/__init__.py`` (tactic enumeration, the gate/up
interleave permutation, availability probes) is provided under the same names.

There is no CPU or eager-PyTorch fallback: without the compiled library the import fails.
"""
import torch

from . import _cabi, ops

__version__ = "0.1.0"

__all__ = [
    "DEFAULT_TACTIC",
    "all_tactics",
    "fused_swiglu_tactics",
    "interleave_gate_up_rows",
    "built_archs",
    "group_mm_configs",
    "is_available",
    "loaded_arch",
    "suggest_tactic",
    "valid_clusters",
]

_LOADED_SM = 100

# (config_id, cluster_m, cluster_n): also the schema defaults of torch.ops.paired_nvfp4.group_mm
DEFAULT_TACTIC = (0, 2, 1)
_CLUSTER_DIMS = (1, 2, 4)


def _register():
    lib = torch.library.Library("paired_nvfp4", "DEF")
    lib.define("compress(Tensor w_packed, Tensor w_blockscale, int k) -> (Tensor, Tensor, Tensor)")
    lib.define("quant_act(Tensor x, Tensor gscale, Tensor expert_num_tokens, int features) -> (Tensor, Tensor)")
    lib.define("silu_mul_quant_act(Tensor x2, Tensor gscale, Tensor expert_num_tokens, int features, "
               "bool interleaved=False, str activation=\"silu\", float beta=1.0, float linear_beta=-1.0) "
               "-> (Tensor, Tensor)")
    lib.define("scatter_quant_act(Tensor a1, Tensor flat_tok, Tensor dest_global, Tensor? topk_weights, "
               "Tensor gscale, Tensor expert_num_tokens, int cap) -> (Tensor, Tensor)")
    lib.define("dispatch_plan(Tensor topk_ids, int first_expert, int num_local_experts, int cap) "
               "-> (Tensor, Tensor, Tensor, Tensor)")
    lib.define("scatter_quant_act_planned(Tensor a1, Tensor src_tok, Tensor src_route, Tensor? topk_weights, "
               "Tensor gscale, Tensor expert_num_tokens, int cap) -> (Tensor, Tensor)")
    lib.define("quant_rows(Tensor x, Tensor gscale) -> (Tensor, Tensor)")
    lib.define("scatter_fp4_planned(Tensor q, Tensor q_sf, Tensor src_tok, Tensor expert_num_tokens, int cap) "
               "-> (Tensor, Tensor)")
    lib.define("moe_finalize(Tensor(a!) out, Tensor fused, Tensor route_dest, Tensor? topk_weights) -> ()")
    lib.define("gather_rows(Tensor src, Tensor idx) -> Tensor")
    lib.define("pack_wire_rows(Tensor q, Tensor q_sf, Tensor topk_ids, Tensor slot_tok, Tensor slot_route, "
               "Tensor slab_counts, int slab, int experts_per_rank) -> Tensor")
    lib.define("scatter_fp4_wire(Tensor wire, int k, Tensor src_tok, Tensor expert_num_tokens, int cap) "
               "-> (Tensor, Tensor)")
    lib.define("group_mm(Tensor(a!) out, Tensor a_comp, Tensor e_meta, Tensor sfa, Tensor b_act, Tensor sfb, "
               "Tensor alphas, Tensor expert_num_tokens, int features, int k, "
               f"int config_id={DEFAULT_TACTIC[0]}, int cluster_m={DEFAULT_TACTIC[1]}, "
               f"int cluster_n={DEFAULT_TACTIC[2]}) -> ()")
    lib.define("group_mm_rows(Tensor(a!) out, Tensor row_map, Tensor a_comp, Tensor e_meta, Tensor sfa, Tensor b_act, "
               "Tensor sfb, Tensor alphas, Tensor expert_num_tokens, int features, int k, "
               f"int config_id={DEFAULT_TACTIC[0]}, int cluster_m={DEFAULT_TACTIC[1]}, "
               f"int cluster_n={DEFAULT_TACTIC[2]}) -> ()")
    lib.define("zero_rows(Tensor(a!) dst, Tensor flags) -> ()")
    lib.define("group_mm_rows_parts(Tensor(a!)[] out_parts, Tensor row_map, Tensor a_comp, Tensor e_meta, Tensor sfa, "
               "Tensor b_act, Tensor sfb, Tensor alphas, Tensor expert_num_tokens, int features, int k, "
               f"int config_id={DEFAULT_TACTIC[0]}, int cluster_m={DEFAULT_TACTIC[1]}, "
               f"int cluster_n={DEFAULT_TACTIC[2]}) -> ()")
    lib.define("zero_rows_parts(Tensor(a!)[] parts, Tensor flags) -> ()")
    lib.define("pack_wire_rows_parts(Tensor q, Tensor q_sf, Tensor topk_ids, Tensor slot_tok, Tensor slot_route, "
               "Tensor slab_counts, int slab, int experts_per_rank, Tensor(a!)[] wire_parts) -> ()")
    lib.define("group_mm_configs() -> str[]")
    lib.define("group_mm_swiglu_quant(Tensor a_comp, Tensor e_meta, Tensor sfa, Tensor b_act, Tensor sfb, "
               "Tensor alphas, Tensor expert_num_tokens, Tensor gscale, int features, int k, int config_id=0, "
               f"int cluster_m={DEFAULT_TACTIC[1]}, int cluster_n={DEFAULT_TACTIC[2]}, "
               "str activation=\"silu\", float beta=1.0, float linear_beta=-1.0) -> (Tensor, Tensor)")
    lib.define("group_mm_swiglu_configs() -> str[]")
    lib.define("gated_act(Tensor x2, bool interleaved=False, str activation=\"silu\", float beta=1.0, "
               "float linear_beta=-1.0) -> Tensor")
    lib.impl("compress", ops.compress, "CUDA")
    lib.impl("quant_act", ops.quant_act, "CUDA")
    lib.impl("silu_mul_quant_act", ops.silu_mul_quant_act, "CUDA")
    lib.impl("scatter_quant_act", ops.scatter_quant_act, "CUDA")
    lib.impl("dispatch_plan", ops.dispatch_plan, "CUDA")
    lib.impl("scatter_quant_act_planned", ops.scatter_quant_act_planned, "CUDA")
    lib.impl("quant_rows", ops.quant_rows, "CUDA")
    lib.impl("scatter_fp4_planned", ops.scatter_fp4_planned, "CUDA")
    lib.impl("moe_finalize", ops.moe_finalize, "CUDA")
    lib.impl("gather_rows", ops.gather_rows, "CUDA")
    lib.impl("pack_wire_rows", ops.pack_wire_rows, "CUDA")
    lib.impl("scatter_fp4_wire", ops.scatter_fp4_wire, "CUDA")
    lib.impl("group_mm", ops.group_mm, "CUDA")
    lib.impl("group_mm_rows", ops.group_mm_rows, "CUDA")
    lib.impl("zero_rows", ops.zero_rows, "CUDA")
    lib.impl("group_mm_rows_parts", ops.group_mm_rows_parts, "CUDA")
    lib.impl("zero_rows_parts", ops.zero_rows_parts, "CUDA")
    lib.impl("pack_wire_rows_parts", ops.pack_wire_rows_parts, "CUDA")
    lib.impl("gated_act", ops.gated_act, "CUDA")
    lib.impl("group_mm_swiglu_quant", ops.group_mm_swiglu_quant, "CUDA")
    lib.impl("group_mm_configs", ops.group_mm_configs, "CompositeExplicitAutograd")
    lib.impl("group_mm_swiglu_configs", ops.group_mm_swiglu_configs, "CompositeExplicitAutograd")
    return lib


_LIB = _register()   # kept alive for the life of the process


def _current_sm():
    if not torch.cuda.is_available():
        return None
    major, minor = torch.cuda.get_device_capability()
    return major * 10 + minor


def loaded_arch():
    """SM number the loaded library was built for (100)."""
    return _LOADED_SM


def built_archs():
    """SM numbers with compiled kernels in this installation."""
    return [_LOADED_SM]


def is_available():
    """Can the ops run here?  Needs a CUDA device of the architecture the library was built for (the
    operators themselves are registered at import, or the import would have failed)."""
    return _current_sm() == _LOADED_SM and all(
        hasattr(torch.ops.paired_nvfp4, op) for op in ("compress", "quant_act", "group_mm"))


def group_mm_configs():
    """Names of the tile variants, indexed by config_id."""
    return list(torch.ops.paired_nvfp4.group_mm_configs())


def _needs_cta_pair(config_name):
    """Variant names read <kind>_<1sm|2sm>_<rows>x<tokens>[_k512]; "2sm" variants run on pairs of CTAs."""
    fields = config_name.split("_")
    return len(fields) > 1 and fields[1] == "2sm"


def valid_clusters(config_name, max_product=16):
    """(cluster_m, cluster_n) pairs the op accepts for one tile variant: both from {1, 2, 4}, product at most
    max_product, and an even cluster_m where the variant runs on CTA pairs."""
    pair = _needs_cta_pair(config_name)
    return [(cm, cn) for cm in _CLUSTER_DIMS for cn in _CLUSTER_DIMS
            if cm * cn <= max_product and not (pair and cm % 2 == 1)]


def all_tactics(max_cluster_product=16):
    """Every candidate (config_id, cluster_m, cluster_n); the op re-validates each one."""
    return [(cid, cm, cn) for cid, name in enumerate(group_mm_configs())
            for cm, cn in valid_clusters(name, max_cluster_product)]


def interleave_gate_up_rows(n, device=None):
    """Row order of W13 ([gate; up], 2n rows) for a GEMM whose epilogue pairs gate and up values:
    64-row blocks holding gate rows 32b..32b+31 followed by up rows n+32b..n+32b+31.  Apply to the
    dense packed weight and its block scales before compress().  n must be a multiple of 64."""
    if n % 64:
        raise ValueError(f"intermediate size must be a multiple of 64, got {n}")
    gate = torch.arange(n, device=device).view(n // 32, 1, 32)
    return torch.cat([gate, gate + n], dim=1).reshape(-1)


def fused_swiglu_tactics(max_cluster_product=16):
    """Candidate (config_id, cluster_m, cluster_n) for group_mm_swiglu_quant; empty if the fused op is absent."""
    configs = getattr(torch.ops.paired_nvfp4, "group_mm_swiglu_configs", None)
    if configs is None:
        return []
    tactics = []
    for cid, name in enumerate(configs()):
        tactics.extend((cid, cm, cn) for cm, cn in valid_clusters(name, max_cluster_product))
    return tactics


def suggest_tactic(max_n):
    """A reasonable group_mm tactic for a per-expert token capacity of max_n, without autotuning:
    64-column tiles when max_n fits one, the 128-column default otherwise."""
    names = group_mm_configs()
    if max_n <= 64:
        return (names.index("sparse_1sm_128x64"), 1, 1)
    return DEFAULT_TACTIC
