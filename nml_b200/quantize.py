"""NVFP4 recipe-v2 quantizer in torch tensor operations (CPU or CUDA).

Produces the three physical components of a logical weight from bf16/f16/f32 values,
following the recipe the reference fixes (crates/nml-parameter/src/lib.rs:483-538,
tools/nvfp4/convert.py:357-410):

    g      = amax(W) / (448 * 6)                      (1.0 for an all-zero tensor)
    scale  = e4m3fn_nearest_even(block_amax / 6 / g)  per 16 consecutive values of the last axis
    code   = e2m1_nearest_even(w / (scale * g))       0 where the block scale rounds to 0
    packed = even column in the low nibble

It exists to make synthetic weights at benchmark sizes (a 201088 x 2880 table takes a
fraction of a second on the GPU); it is checked byte-for-byte against the parity oracle in
the CPU tests.  It is host-side input preparation, not part of the timed path.
"""
from __future__ import annotations

import torch

_E2M1_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def _e4m3_table(device) -> torch.Tensor:
    """The 127 valid unsigned E4M3FN values in code order (ascending)."""
    bits = torch.arange(0x7F, device=device, dtype=torch.int32)
    exponent = (bits >> 3).float()
    fraction = (bits & 7).float()
    normal = (1.0 + fraction / 8.0) * torch.exp2(exponent - 7.0)
    subnormal = fraction * 2.0 ** -9
    return torch.where((bits >> 3) == 0, subnormal, normal)


def encode_e4m3fn(values: torch.Tensor) -> torch.Tensor:
    """Nearest valid code, ties to the even code, saturating at 448 (code 0x7e)."""
    table = _e4m3_table(values.device)
    v = values.float().clamp(min=0.0)
    upper = torch.bucketize(v, table).clamp(max=table.numel() - 1)  # first code with value >= v
    lower = (upper - 1).clamp(min=0)
    d_upper = (table[upper] - v).abs()
    d_lower = (v - table[lower]).abs()
    take_lower = (d_lower < d_upper) | ((d_lower == d_upper) & ((lower & 1) == 0))
    return torch.where(take_lower, lower, upper).to(torch.uint8)


def decode_e4m3fn(bits: torch.Tensor) -> torch.Tensor:
    return _e4m3_table(bits.device)[bits.long()]


def quantize(weight: torch.Tensor, chunk_rows: int = 16384):
    """weight [..., K] -> (payload u8 [..., ceil(K/2)], block_scales u8 [..., ceil(K/16)],
    global_scale f32 scalar), all on weight's device."""
    if weight.dim() == 0 or weight.shape[-1] == 0:
        raise ValueError("invalid NVFP4 source tensor shape")
    width = weight.shape[-1]
    rows = weight.reshape(-1, width)
    if not torch.isfinite(rows.float()).all():
        raise ValueError("NVFP4 source tensor contains a non-finite value")
    amax = rows.float().abs().amax()
    g = amax / (448.0 * 6.0)
    g = torch.where(g == 0, torch.ones_like(g), g).to(torch.float32)
    thresholds = torch.tensor(_E2M1_THRESHOLDS, dtype=torch.float32, device=weight.device)
    pad = (-width) % 16
    payloads, scales = [], []
    for start in range(0, rows.shape[0], chunk_rows):
        values = rows[start:start + chunk_rows].float()
        if pad:
            values = torch.nn.functional.pad(values, (0, pad))
        blocks = values.reshape(values.shape[0], -1, 16)
        raw = (blocks.abs().amax(dim=-1) / 6.0) / g
        scale_bits = encode_e4m3fn(raw)
        effective = (decode_e4m3fn(scale_bits) * g).unsqueeze(-1)
        normalized = torch.where(effective == 0, torch.zeros_like(blocks), blocks / effective)
        magnitude = normalized.abs()
        codes = (magnitude.unsqueeze(-1) > thresholds).sum(dim=-1)
        # a value exactly on a boundary whose lower code is odd rounds up to the even code
        for index in (1, 3, 5):
            codes = codes + (magnitude == thresholds[index]).long()
        codes = codes.to(torch.uint8) | (torch.signbit(normalized).to(torch.uint8) << 3)
        codes = codes.reshape(codes.shape[0], -1)[:, :width]
        if width & 1:
            codes = torch.nn.functional.pad(codes, (0, 1))
        payloads.append(codes[:, 0::2] | (codes[:, 1::2] << 4))
        scales.append(scale_bits)
    payload = torch.cat(payloads).reshape(*weight.shape[:-1], (width + 1) // 2)
    block_scales = torch.cat(scales).reshape(*weight.shape[:-1], (width + 15) // 16)
    return payload.contiguous(), block_scales.contiguous(), g.reshape(())


def quantize_parameter(name: str, weight: torch.Tensor):
    """Convenience: quantize and wrap as an ``ops.NvFp4Parameter`` of weight's dtype."""
    from .ops import NvFp4Parameter
    payload, block_scales, g = quantize(weight)
    dtype = weight.dtype if weight.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16
    return NvFp4Parameter.nvfp4(name, tuple(weight.shape), dtype, payload, block_scales, g)
