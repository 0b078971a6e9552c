"""Seeded input builders shared by the GPU parity tests (numpy on the host, torch for device I/O)."""
import numpy as np
import torch

from oracle import paired_nvfp4_oracle as orc


def bf16_tensor(bits, device="cuda"):
    """uint16 bf16 bit patterns -> torch.bfloat16 tensor on `device`."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).to(device)


def bf16_bits(t):
    """torch.bfloat16 tensor -> uint16 bit patterns (numpy, host)."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def u8(t):
    return t.detach().contiguous().cpu().numpy()


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def make_weights(E, M, K, seed, scale=1.0):
    """Seeded N(0, scale) weights -> pruned paired-4:8 -> NVFP4.  Returns (packed, sf, dequant)."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((E, M, K)) * scale).astype(np.float32)
    return orc.quantize_weight(orc.prune_paired_4of8(w))


def make_acts(E, max_n, K, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    return orc.f32_to_bf16_bits((rng.standard_normal((E, max_n, K)) * scale).astype(np.float32))
