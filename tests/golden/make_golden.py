"""Generates the golden fixtures in this directory from the reference's own Python tools.

Run where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

It imports ``tools/nvfp4/convert.py`` (``quantize_tensor``, the recipe-v2
quantizer, convert.py:357-410) and ``tools/nvfp4/extract_fixture.py``
(``decode_row``, the spec-level decoder, extract_fixture.py:169-190) and
freezes their outputs on small seeded tensors into ``nvfp4_golden.npz``.
The tests load the .npz only; the reference checkout is not needed to run them.

Inputs are produced with numpy's PCG64 so that they do not depend on the torch
version; bf16 rounding is done with integer arithmetic for the same reason.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def bf16_round(values: np.ndarray) -> np.ndarray:
    """f32 -> nearest-even bf16 bit patterns (uint16)."""
    bits = np.ascontiguousarray(values, np.float32).view(np.uint32)
    bias = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    return ((bits + bias) >> np.uint32(16)).astype(np.uint16)


def bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


CASES = {
    # name: (shape, std, tweak)
    "normal_8x64": ((8, 64), 0.02, None),
    "odd_width_5x17": ((5, 17), 0.02, None),
    "width_33": ((3, 33), 1.0, None),
    "experts_3x10x48": ((3, 10, 48), 0.02, None),
    "zero_blocks_4x32": ((4, 32), 0.02, "zero_blocks"),
    "all_zero_2x16": ((2, 16), 0.0, None),
    "wide_range_6x80": ((6, 80), 0.02, "wide_range"),
    "gpt_oss_row_2x2880": ((2, 2880), 0.02, None),
}


def main() -> int:
    if len(sys.argv) < 2:
        print("usage: make_golden.py <path of a checkout of the reference project>")
        return 2
    reference = Path(sys.argv[1])
    convert = load(reference / "tools/nvfp4/convert.py", "nml_ref_convert")
    extract = load(reference / "tools/nvfp4/extract_fixture.py", "nml_ref_extract")
    rng = np.random.Generator(np.random.PCG64(20250101))
    out = {}
    for name, (shape, std, tweak) in CASES.items():
        values = (rng.standard_normal(shape) * std).astype(np.float32)
        if tweak == "zero_blocks":
            values[1, :16] = 0.0
            values[2, 16:] = 0.0
            values[3, :] = 0.0
        if tweak == "wide_range":
            # tiny rows next to a large outlier: exercises subnormal and zero block scales
            values[0] *= 1e-4
            values[1] *= 1e-6
            values[2, 5] = 3.0
        bits = bf16_round(values)
        tensor = bf16_tensor(bits).reshape(shape)
        payload, scales, g = convert.quantize_tensor(tensor, 2048, torch.device("cpu"), torch)
        payload = payload.numpy().copy()
        scales = scales.numpy().copy()
        g32 = np.float32(g.item())
        width = shape[-1]
        rows = int(np.prod(shape[:-1]))
        decoded = np.zeros((rows, width), np.float32)
        flat_payload = payload.reshape(rows, -1)
        flat_scales = scales.reshape(rows, -1)
        for row in range(rows):
            decoded[row] = np.array(
                extract.decode_row(bytes(flat_payload[row]), bytes(flat_scales[row]), float(g32),
                                   width), np.float32)
        out[f"{name}.source_bf16"] = bits
        out[f"{name}.payload"] = payload
        out[f"{name}.scales"] = scales
        out[f"{name}.global"] = np.array(g32, np.float32)
        out[f"{name}.decoded"] = decoded.reshape(shape)

    # The fixture input vector of extract_fixture.py:22-26,95-98 and its projection
    # of the two GPT-OSS-width rows above, accumulated exactly (math.fsum) as the
    # reference tool does.
    import math
    inputs = 2880
    x = np.array([np.float32(((i * 17) % 251 - 125) / 64.0) for i in range(inputs)], np.float32)
    decoded = out["gpt_oss_row_2x2880.decoded"]
    out["fixture_input_2880"] = x
    out["fixture_projection_2x2880"] = np.array(
        [math.fsum(float(a) * float(b) for a, b in zip(x, decoded[r])) for r in range(2)],
        np.float64)
    np.savez_compressed(HERE / "nvfp4_golden.npz", **out)
    print(f"wrote {HERE / 'nvfp4_golden.npz'} with {len(out)} arrays")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
