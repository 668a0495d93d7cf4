"""Paged-attention decode through the C ABI against a plain PyTorch fp32 evaluation of the
same operator (softmax over the visible tokens plus the sink column, f32 throughout).

Tolerance: the kernel multiplies 16-bit keys and queries exactly and accumulates in f32; the
probabilities are narrowed to the cache's 16-bit type for the second product (numerator and
denominator use the same narrowed values); what else differs from the f32 evaluation is the
order of the sums and the final narrowing to the 16-bit output, so
|a - e| <= 2^-7 |e| + 2e-3 (one output ulp of bf16 plus accumulation noise on values of
order one)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def reference(query, key_cache, value_cache, page_table, lengths, sinks, window, scale):
    batch, heads, dim = query.shape
    pages, page, kv_heads, _ = key_cache.shape
    group = heads // kv_heads
    out = torch.zeros((batch, heads, dim), dtype=torch.float32, device=query.device)
    for b in range(batch):
        n = int(lengths[b])
        if n == 0:
            continue
        table = page_table[b, : -(-n // page)].long()
        keys = key_cache[table].reshape(-1, kv_heads, dim)[:n].float()
        values = value_cache[table].reshape(-1, kv_heads, dim)[:n].float()
        start = max(0, n - window) if window else 0
        keys, values = keys[start:], values[start:]
        q = query[b].float().view(kv_heads, group, dim)
        scores = torch.einsum("hgd,thd->hgt", q, keys) * scale
        if sinks is not None:
            column = sinks.view(kv_heads, group, 1)
            weights = torch.softmax(torch.cat((scores, column), dim=-1), dim=-1)[..., :-1]
        else:
            weights = torch.softmax(scores, dim=-1)
        out[b] = torch.einsum("hgt,thd->hgd", weights, values).reshape(heads, dim)
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("batch,kv_heads,lengths,window,with_sinks,splits", [
    (3, 2, [1, 17, 100], 0, True, 1),
    (4, 8, [4097, 333, 16, 2049], 0, True, 4),
    (4, 8, [4097, 333, 16, 127], 128, True, 3),
    (2, 1, [64, 0], 0, False, 2),
    (5, 3, [700, 701, 702, 703, 15], 128, False, None),
])
def test_decode_attention_matches_fp32_reference(dtype, batch, kv_heads, lengths, window,
                                                with_sinks, splits):
    from nml_b200 import ops, _abi
    g = torch.Generator(device="cuda").manual_seed(batch * 100 + kv_heads)
    heads, dim, page = kv_heads * 8, 64, 16
    table_width = -(-max(lengths) // page) + 1
    pages = batch * table_width + 3
    key_cache = torch.randn((pages, page, kv_heads, dim), device="cuda", generator=g).to(dtype)
    value_cache = torch.randn((pages, page, kv_heads, dim), device="cuda", generator=g).to(dtype)
    # every sequence owns a random set of physical pages
    order = torch.randperm(pages, device="cuda", generator=g)[: batch * table_width]
    page_table = order.view(batch, table_width).to(torch.int32).contiguous()
    query = torch.randn((batch, heads, dim), device="cuda", generator=g).to(dtype)
    sinks = torch.randn(heads, device="cuda", generator=g) if with_sinks else None
    d_lengths = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    scale = dim ** -0.5
    out = ops.paged_attention_decode(query, key_cache, value_cache, page_table, d_lengths, sinks,
                                     sliding_window=window or None, scale=scale, splits=splits)
    torch.cuda.synchronize()
    assert _abi.device_status(0x1) == 0
    expected = reference(query, key_cache, value_cache, page_table, lengths, sinks, window, scale)
    a, e = out.float(), expected
    assert torch.isfinite(a).all()
    assert ((a - e).abs() <= 2.0 ** -7 * e.abs() + 2e-3).all(), (a - e).abs().max().item()
    for b, n in enumerate(lengths):
        if n == 0:
            assert (a[b] == 0).all()


def test_decode_attention_rejects_unsupported_geometry():
    from nml_b200 import ops, _abi
    cache = torch.zeros((4, 16, 2, 32), dtype=torch.bfloat16, device="cuda")  # head_dim 32
    query = torch.zeros((1, 16, 32), dtype=torch.bfloat16, device="cuda")
    table = torch.zeros((1, 4), dtype=torch.int32, device="cuda")
    lengths = torch.ones(1, dtype=torch.int32, device="cuda")
    with pytest.raises(_abi.NvFp4Error) as error:
        ops.paged_attention_decode(query, cache, cache, table, lengths)
    assert error.value.code == _abi.INVALID_ARGUMENT
