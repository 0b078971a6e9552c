"""No-GPU checks of the boundary: the shared library loads, exports every symbol the header
declares, answers its size queries like the oracle, and the operator surface is registered with the
reference's schemas (tests/test_registration.py:19-54 of the reference)."""
import ctypes
import os
import re

import pytest
import torch

from oracle import paired_nvfp4_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pnk():
    import paired_nvfp4_kernels
    return paired_nvfp4_kernels


def test_library_exports_every_declared_symbol(pnk):
    from paired_nvfp4_kernels import _cabi
    header = open(os.path.join(ROOT, "include", "paired_nvfp4_b200.h")).read()
    declared = set(re.findall(r"\b(pnv_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(_cabi.SIGNATURES), "ctypes binding and header disagree"
    assert lib.pnv_abi_version() == 2


def test_size_queries_match_oracle(pnk):
    from paired_nvfp4_kernels import _cabi
    for M, K in [(2048, 1024), (130, 320), (1, 32), (28672, 4096), (4096, 14336), (127, 96)]:
        assert _cabi.physical_dims(M, K) == orc.physical_dims(M, K)
        for groups in (1, 8):
            assert _cabi.sf_numel(M, K, groups) == orc.sf_numel(M, K, groups)


def test_ops_registered_with_reference_schemas(pnk):
    ns = torch.ops.paired_nvfp4
    for op in ("compress", "quant_act", "silu_mul_quant_act", "scatter_quant_act", "group_mm", "group_mm_configs",
               "dispatch_plan", "scatter_quant_act_planned", "quant_rows", "scatter_fp4_planned", "moe_finalize",
               "group_mm_swiglu_quant", "group_mm_swiglu_configs"):
        assert hasattr(ns, op), op
    schema = str(ns.group_mm.default._schema)
    cid, cm, cn = pnk.DEFAULT_TACTIC
    assert f"int config_id={cid}" in schema and f"int cluster_m={cm}" in schema and f"int cluster_n={cn}" in schema
    s = str(ns.silu_mul_quant_act.default._schema)
    assert 'bool interleaved=False' in s and 'str activation="silu"' in s and "float linear_beta=-1." in s
    assert "Tensor? topk_weights" in str(ns.scatter_quant_act.default._schema)


def test_tactic_helpers(pnk):
    names = pnk.group_mm_configs()
    assert names[:8] == ["sparse_2sm_256x128", "sparse_2sm_256x256", "sparse_1sm_128x128", "sparse_1sm_128x256",
                         "sparse_2sm_256x64", "sparse_1sm_128x64", "sparse_2sm_256x64_k512", "sparse_1sm_128x64_k512"]
    tactics = pnk.all_tactics()
    assert pnk.DEFAULT_TACTIC in tactics
    for cid, cm, cn in tactics:
        assert cm * cn <= 16 and cm in (1, 2, 4) and cn in (1, 2, 4)
        if names[cid].split("_")[1] == "2sm":
            assert cm % 2 == 0
    assert pnk.loaded_arch() == 100 and pnk.built_archs() == [100]
    assert pnk.suggest_tactic(4096) == pnk.DEFAULT_TACTIC


def test_interleave_matches_oracle(pnk):
    for n in (64, 128, 768):
        assert pnk.interleave_gate_up_rows(n).tolist() == orc.interleave_gate_up_rows(n).tolist()
    with pytest.raises(ValueError):
        pnk.interleave_gate_up_rows(96)


def test_cpu_tensors_are_rejected_not_computed(pnk):
    x = torch.zeros(1, 4, 64, dtype=torch.bfloat16)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.paired_nvfp4.quant_act(x, torch.ones(1), torch.ones(1, dtype=torch.int32), 64)
