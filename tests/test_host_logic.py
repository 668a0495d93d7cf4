"""Host-side choices that need no GPU: the split count of the attention decode launch, the
decode-step shape constants and its HBM bound, the YaRN frequencies."""
import math

import torch


def test_attention_split_count():
    from nml_b200.ops import _attention_splits
    sms = 148
    # enough (sequence, kv head) pairs to fill the GPU: no split
    assert _attention_splits(512, 257, sms) == 1
    assert _attention_splits(4096, 257, sms) == 1
    # few pairs: split until about two CTAs per SM, never more than one split per 8 pages
    assert _attention_splits(64, 257, sms) == 5
    assert _attention_splits(8, 257, sms) == 32
    assert _attention_splits(8, 9, sms) == 1          # a sliding window of 128 tokens
    assert _attention_splits(1, 10_000, sms) == 64    # the kernel's limit
    for pairs in (1, 3, 17, 100, 1000):
        previous = None
        for pages in (1, 8, 64, 257, 4096):
            splits = _attention_splits(pairs, pages, sms)
            assert 1 <= splits <= 64 and splits <= max(1, pages // 8)
            assert previous is None or splits >= previous
            previous = splits


def test_decode_step_shape_and_bound():
    from nml_b200.decode_step import GptOssShape, yarn_inverse_frequencies
    shape = GptOssShape()
    # products/serve/src/gpt_oss/config.rs:101-142
    assert (shape.layers, shape.hidden, shape.experts, shape.experts_per_token) == (24, 2880, 32, 4)
    assert shape.query_width == 4096 and shape.key_value_width == 512
    # the bound the step is compared with: ~18.1 GB per step at batch 64 over 4096 prior tokens
    nbytes = shape.weight_bytes_per_step(64, 4096)
    assert 17.9e9 < nbytes < 18.3e9
    frequencies, factor = yarn_inverse_frequencies(shape, torch.device("cpu"))
    assert frequencies.shape == (32,) and torch.all(frequencies[:-1] >= frequencies[1:])
    assert frequencies[0].item() == 1.0                       # fastest rotation is kept
    slowest = 1.0 / (shape.rope_factor * shape.rope_theta ** (31 / 32))
    assert math.isclose(frequencies[-1].item(), slowest, rel_tol=1e-5)  # slowest is interpolated
    assert math.isclose(factor, 0.1 * math.log(32.0) + 1.0)


def test_f16_narrowing_bound_of_the_wide_linear():
    # The dense linear narrows BF16 activations to F16, a 256-row tile times one power of two
    # that puts the tile's largest magnitude into [2^14, 2^15).  The arithmetic of that pass,
    # restated with torch on the CPU: elements down to 2^-28 of the tile's largest survive
    # exactly, smaller ones are off by at most 2^-39 of it, and nothing overflows.
    generator = torch.Generator().manual_seed(5)
    tile = torch.randn((256, 512), generator=generator)
    tile *= torch.exp2(torch.randint(-8, 1, (256, 1), generator=generator).float())  # rows within 2^8
    tile[:, ::7] *= 2.0 ** -30   # elements far below their row
    tile[3] = 0.0
    tile = tile.to(torch.bfloat16)
    largest = tile.float().abs().max()
    exponent = math.floor(math.log2(float(largest)))
    down = 2.0 ** (14 - exponent)
    narrowed = (tile.float() * down).to(torch.float16)
    assert torch.isfinite(narrowed).all()
    assert 2.0 ** 14 <= float(narrowed.float().abs().max()) < 2.0 ** 15
    restored = narrowed.float() / down
    exact = tile.float().abs() >= float(largest) * 2.0 ** -28
    assert torch.equal(restored[exact], tile.float()[exact])
    assert float((restored - tile.float()).abs().max()) <= float(largest) * 2.0 ** -39
    assert (restored[3] == 0).all()
