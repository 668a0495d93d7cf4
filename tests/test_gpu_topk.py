"""Row-wise top-k of 16-bit logits through the C ABI: values and indices must equal a stable
descending sort (equal values to the lower index) exactly; it is compare-and-select work."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,columns,k", [(1, 201088, 8), (64, 25136, 1), (7, 8192, 16),
                                            (3, 8193, 4), (5, 100, 16), (1024, 25136, 8),
                                            (2, 50272, 8)])
def test_topk_rows_matches_stable_sort(rows, columns, k, dtype):
    from nml_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(rows + columns)
    logits = (torch.randn((rows, columns), device="cuda", generator=g) * 3).to(dtype)
    logits[:, ::7] = logits[:, 3:4]  # many exact ties
    if columns > 200:
        logits[0, 10:14] = float("nan")  # never selected
        logits[-1, :50] = float("inf")
    values, indices = ops.topk_rows(logits, k, index_offset=1000)
    clean = torch.nan_to_num(logits.float(), nan=float("-inf"), posinf=float("inf"))
    e_values, order = torch.sort(clean, dim=1, descending=True, stable=True)
    assert torch.equal(values, e_values[:, :k])
    assert torch.equal(indices.long(), order[:, :k] + 1000)


def test_topk_rows_on_a_strided_view():
    from nml_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(5)
    wide = torch.randn((6, 9000), device="cuda", generator=g).to(torch.bfloat16)
    view = wide[:, 8:8008]  # rows 9000 apart, first column not 16-byte aligned for odd rows
    values, indices = ops.topk_rows(view, 5)
    e_values, order = torch.sort(view.float(), dim=1, descending=True, stable=True)
    assert torch.equal(values, e_values[:, :5]) and torch.equal(indices.long(), order[:, :5])


@pytest.mark.parametrize("parts,rows,k", [(2, 5, 1), (8, 64, 8), (4, 1, 16), (16, 33, 16)])
def test_topk_merge_equals_topk_of_the_unsharded_row(parts, rows, k):
    # per-shard candidates merged with the per-shard order (larger value, then lower index):
    # the result must be the top-k of the whole row, also with many equal values across shards
    from nml_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(parts * 100 + rows + k)
    columns = 512  # per shard
    # few distinct values, so that ties within and across shards are certain
    logits = (torch.randint(-6, 6, (rows, parts * columns), device="cuda", generator=g)
              .float() / 4).to(torch.bfloat16)
    gathered = torch.empty((parts, rows, 2 * k), dtype=torch.int32, device="cuda")
    for p in range(parts):
        values, indices = ops.topk_rows(logits[:, p * columns:(p + 1) * columns], k,
                                        index_offset=p * columns)
        gathered[p, :, :k] = values.view(torch.int32)
        gathered[p, :, k:] = indices
    merged_values, merged_indices = ops.topk_merge(gathered.view(torch.float32)[:, :, :k],
                                                   gathered[:, :, k:], k)
    order = torch.sort(logits.float(), dim=1, descending=True, stable=True)
    assert torch.equal(merged_values, order.values[:, :k])
    assert torch.equal(merged_indices.long(), order.indices[:, :k])
    # empty candidates (negative index) are skipped
    gathered[0, :, k:] = -1
    rest_values, rest_indices = ops.topk_merge(gathered.view(torch.float32)[:, :, :k],
                                               gathered[:, :, k:], k)
    rest = torch.sort(logits[:, columns:].float(), dim=1, descending=True, stable=True)
    assert torch.equal(rest_values, rest.values[:, :k])
    assert torch.equal(rest_indices.long(), rest.indices[:, :k] + columns)
