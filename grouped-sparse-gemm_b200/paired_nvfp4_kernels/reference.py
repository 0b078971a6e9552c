"""Executable description of the checkpoint format ``compress`` consumes, in plain torch (runs on
CPU or GPU).  Same public names and results as the reference project's
``paired_nvfp4_kernels/reference.py``; checkpoint producers and tests call these.

A weight ``W[E, M, K]`` is stored as

  * paired 4:8 sparse along K -- of the four adjacent value pairs in every run of eight, the two
    with the smaller |a| + |b| are zero;
  * NVFP4 -- one UE4M3 scale per 32 consecutive K values, ``s = e4m3(clamp(amax / 6, 1e-12, 448))``,
    and 4-bit e2m1 codes of ``w / s`` (nearest value, exact midpoints to the smaller magnitude,
    saturating at 6, never a negative zero);
  * two codes per byte, the lower K index in the low nibble.

A per-expert fp32 ``alpha`` applied by the GEMM epilogue carries any per-tensor scales.
"""
import torch

SF_BLOCK = 32
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# strict upper edges of the buckets that map to codes 0..6 (code 7 takes the rest)
_E2M1_EDGES = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def _pairs(w):
    E, M, K = w.shape
    if K % 8:
        raise AssertionError(K)
    return w.reshape(E, M, K // 8, 4, 2)


def prune_paired_4of8(w):
    """Zero the two weakest of every four adjacent K-pairs (strength = |a| + |b|)."""
    wp = _pairs(w)
    strength = wp.abs().sum(-1)
    # stable descending order, so equal strengths keep the pair with the lower index
    strongest = strength.sort(dim=-1, descending=True, stable=True).indices[..., :2]
    keep = torch.zeros_like(strength, dtype=torch.bool).scatter_(-1, strongest, True)
    return torch.where(keep.unsqueeze(-1), wp, torch.zeros((), dtype=w.dtype, device=w.device)).reshape(w.shape)


def is_paired_4of8(w):
    """True iff no run of eight K values has more than two non-zero pairs."""
    live_pairs = (_pairs(w) != 0).any(-1).sum(-1)
    return bool((live_pairs <= 2).all())


def _e2m1_code(a):
    """Magnitude -> code 0..7: count the bucket edges strictly below the magnitude."""
    edges = torch.tensor(_E2M1_EDGES, dtype=a.dtype, device=a.device)
    return torch.bucketize(a, edges, right=False)   # a > edge  <=>  edge counted


def round_to_e2m1(x):
    """Nearest e2m1 value with the sign kept; midpoints go down in magnitude; saturates at +-6."""
    lut = torch.tensor(E2M1_VALUES, dtype=x.dtype, device=x.device)
    mag = lut[_e2m1_code(x.abs())]
    return torch.where(x < 0, -mag, torch.where(x > 0, mag, torch.zeros_like(mag)))


def pack_e2m1(vals):
    """e2m1-valued floats [..., K] -> uint8 [..., K/2]; even K index in the low nibble."""
    code = _e2m1_code(vals.abs()).to(torch.uint8)
    nib = torch.where((vals < 0) & (code != 0), code | 8, code)
    pair = nib.reshape(*nib.shape[:-1], -1, 2)
    return (pair[..., 0] | (pair[..., 1] << 4)).contiguous()


def unpack_e2m1(packed):
    """uint8 [..., K/2] -> float32 [..., K]."""
    lut = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32, device=packed.device)
    nib = torch.stack((packed & 0xF, packed >> 4), dim=-1).reshape(*packed.shape[:-1], -1)
    return lut[nib.long()]


def quantize_weight(w):
    """Paired-4:8-sparse w[E, M, K] -> (w_packed u8[E, M, K/2], w_blockscale u8[E, M, K/32] raw UE4M3
    in natural order, w_dequant f32[E, M, K] = code value x scale)."""
    E, M, K = w.shape
    if K % SF_BLOCK:
        raise AssertionError(K)
    blocks = w.float().reshape(E, M, K // SF_BLOCK, SF_BLOCK)
    target = blocks.abs().amax(-1, keepdim=True) / 6.0
    scale8 = target.clamp(min=1e-12, max=448.0).to(torch.float8_e4m3fn)
    scale = scale8.float()
    q = round_to_e2m1(blocks / scale)
    w_dequant = (q * scale).reshape(E, M, K)
    return pack_e2m1(q.reshape(E, M, K)), scale8.squeeze(-1).contiguous().view(torch.uint8), w_dequant


def dequantize_weight(w_packed, w_blockscale):
    """(u8[E, M, K/2], u8[E, M, K/32]) -> f32[E, M, K]."""
    q = unpack_e2m1(w_packed)
    E, M, K = q.shape
    scale = w_blockscale.view(torch.float8_e4m3fn).float().unsqueeze(-1)
    return (q.reshape(E, M, K // SF_BLOCK, SF_BLOCK) * scale).reshape(E, M, K)
