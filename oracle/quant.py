"""FP8 KV-cache codec oracle (test infrastructure only).

Restates tests/quant.py:3-66.  Token record = 656 bytes (README.md:162-170):
  bytes   0..511  512 x float8_e4m3fn  "nope" part, quantised per 128-wide tile
  bytes 512..527  4 x float32          per-tile scale (= amax/448)
  bytes 528..655  64 x bfloat16        "rope" part, stored unquantised
"""
from __future__ import annotations

import torch

BYTES_PER_TOKEN = 656


def quantize_k_cache(k: torch.Tensor, dv: int = 512, tile: int = 128) -> torch.Tensor:
    """k: [num_blocks, block_size, 1, d] bf16 -> [num_blocks, block_size, 1, 656] e4m3 bytes.

    tests/quant.py:3-35: scale = max|x| over the tile / 448 (computed in the
    input dtype, stored as fp32); q = (fp32(x) / fp32(scale)) cast to e4m3.
    """
    nb, bs, hk, d = k.shape
    assert hk == 1 and dv % tile == 0
    nt = dv // tile
    x = k.reshape(nb, bs, d)
    esz = x.element_size()
    out = torch.empty((nb, bs, dv + 4 * nt + esz * (d - dv)), dtype=torch.float8_e4m3fn)
    nope = out[..., :dv]
    scales = out[..., dv:dv + 4 * nt].view(torch.float32)
    rope = out[..., dv + 4 * nt:].view(x.dtype)
    rope[:] = x[..., dv:]
    for t in range(nt):
        seg = x[..., t * tile:(t + 1) * tile]
        s = seg.abs().max(dim=-1).values / 448.0          # input dtype, as the reference
        scales[..., t] = s
        nope[..., t * tile:(t + 1) * tile] = (seg.float() / s.unsqueeze(-1).float()).to(torch.float8_e4m3fn)
    return out.view(nb, bs, 1, -1)


def dequantize_k_cache(qk: torch.Tensor, dv: int = 512, tile: int = 128, d: int = 576) -> torch.Tensor:
    """Inverse (tests/quant.py:38-66): bf16( fp32(e4m3) * fp32 scale ), rope copied."""
    nb, bs, hk, _ = qk.shape
    assert hk == 1
    nt = dv // tile
    raw = qk.reshape(nb, bs, -1)
    if raw.dtype != torch.float8_e4m3fn:
        raw = raw.view(torch.float8_e4m3fn)
    nope = raw[..., :dv]
    scales = raw[..., dv:dv + 4 * nt].view(torch.float32)
    rope = raw[..., dv + 4 * nt:].view(torch.bfloat16)
    out = torch.empty((nb, bs, d), dtype=torch.bfloat16)
    out[..., dv:] = rope
    for t in range(nt):
        out[..., t * tile:(t + 1) * tile] = nope[..., t * tile:(t + 1) * tile].float() * scales[..., t].unsqueeze(-1)
    return out.view(nb, bs, 1, d)
