"""The package's torch weight spec (paired_nvfp4_kernels.reference) against the golden vectors
generated from the reference project's own reference.py, and against the numpy oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import paired_nvfp4_oracle as orc

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_weight_vectors.npz"))


@pytest.fixture(scope="module")
def ref():
    from paired_nvfp4_kernels import reference
    return reference


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_matches_reference_outputs(ref, name):
    w = torch.from_numpy(G[f"{name}_w"])
    pruned = ref.prune_paired_4of8(w)
    assert torch.equal(pruned, torch.from_numpy(G[f"{name}_pruned"]))
    packed, sf, dq = ref.quantize_weight(pruned)
    assert np.array_equal(packed.numpy(), G[f"{name}_packed"])
    assert np.array_equal(sf.numpy(), G[f"{name}_sf"])
    assert np.array_equal(dq.numpy(), G[f"{name}_dq"], equal_nan=True)
    assert np.array_equal(ref.dequantize_weight(packed, sf).numpy(), G[f"{name}_dq2"], equal_nan=True)
    assert ref.is_paired_4of8(pruned)


def test_known_answer_tables(ref):
    assert np.array_equal(ref.round_to_e2m1(torch.from_numpy(G["round_x"])).numpy(), G["round_y"])
    assert np.array_equal(ref.pack_e2m1(torch.from_numpy(G["pack_vals"])[None]).numpy(), G["pack_bytes"])
    assert np.array_equal(ref.unpack_e2m1(torch.arange(256, dtype=torch.uint8)[None]).numpy(), G["unpack_vals"])
    vals = torch.tensor(ref.E2M1_VALUES + tuple(-v for v in ref.E2M1_VALUES[1:]) + (0.0,))
    assert torch.equal(ref.unpack_e2m1(ref.pack_e2m1(vals[None]))[0], vals)


def test_agrees_with_numpy_oracle_on_random_weights(ref):
    g = torch.Generator().manual_seed(5)
    w = torch.randn(2, 24, 256, generator=g) * 0.02
    pruned = ref.prune_paired_4of8(w)
    assert np.array_equal(pruned.numpy(), orc.prune_paired_4of8(w.numpy()))
    packed, sf, dq = ref.quantize_weight(pruned)
    op, os_, od = orc.quantize_weight(pruned.numpy())
    assert np.array_equal(packed.numpy(), op) and np.array_equal(sf.numpy(), os_) and np.array_equal(dq.numpy(), od)
    assert (pruned == 0).float().mean().item() == 0.5
    assert not ref.is_paired_4of8(torch.randn(2, 16, 64, generator=g))
