"""Generate the golden vectors under tests/golden/ from the reference's own executable weight spec.

Run once in a checkout that has the reference project available:

    python tests/golden/make_golden.py /path/to/reference

It loads ``paired_nvfp4_kernels/reference.py`` by file path (importing the package itself needs a
compiled extension) and records, for a few small seeded weights, the outputs of
``prune_paired_4of8``, ``quantize_weight``, ``dequantize_weight``, ``round_to_e2m1`` and
``pack_e2m1``/``unpack_e2m1``.  The vectors are committed; the tests never read the reference.
"""
import importlib.util
import os
import sys

import numpy as np
import torch


def load_reference(root):
    path = os.path.join(root, "paired_nvfp4_kernels", "reference.py")
    spec = importlib.util.spec_from_file_location("paired_nvfp4_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    root = sys.argv[1]
    ref = load_reference(root)
    here = os.path.dirname(os.path.abspath(__file__))
    out = {}
    cases = [("a", 1000, (2, 16, 128), 1.0), ("b", 1001, (3, 40, 256), 0.02), ("c", 1002, (1, 130, 96), 4.0)]
    for name, seed, shape, scale in cases:
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(shape, generator=g) * scale
        if name == "c":
            # exercise scale saturation, an all-zero block and exact e2m1 midpoints
            w[0, 0, :32] = 0.0
            w[0, 1, :32] = 5000.0
            w[0, 2, :8] = torch.tensor([0.75, 6.0, 1.75, 0.0, 3.5, 0.0, 0.25, 5.0]) * 2.0
        wp = ref.prune_paired_4of8(w)
        packed, sf, dq = ref.quantize_weight(wp)
        out[f"{name}_w"] = w.numpy()
        out[f"{name}_pruned"] = wp.numpy()
        out[f"{name}_packed"] = packed.numpy()
        out[f"{name}_sf"] = sf.numpy()
        out[f"{name}_dq"] = dq.numpy()
        out[f"{name}_dq2"] = ref.dequantize_weight(packed, sf).numpy()
    x = torch.linspace(-7.0, 7.0, 1121)  # step 0.0125: hits every midpoint exactly
    out["round_x"] = x.numpy()
    out["round_y"] = ref.round_to_e2m1(x).numpy()
    vals = torch.tensor(ref.E2M1_VALUES + tuple(-v for v in ref.E2M1_VALUES[1:]) + (0.0,))
    out["pack_vals"] = vals.numpy()
    out["pack_bytes"] = ref.pack_e2m1(vals[None]).numpy()
    out["unpack_vals"] = ref.unpack_e2m1(torch.arange(256, dtype=torch.uint8)[None]).numpy()
    # e4m3 cast table over a fine positive grid (what quantize_weight's scale cast does)
    s = torch.cat([torch.logspace(-13, 2.65, 4000), torch.tensor([448.0, 0.0, 2.0 ** -9, 2.0 ** -10])])
    s = s.clamp(max=448.0)
    out["e4m3_in"] = s.numpy()
    out["e4m3_bits"] = s.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.savez_compressed(os.path.join(here, "reference_weight_vectors.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
