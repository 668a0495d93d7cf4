"""Embedding gather/decode through the C ABI against the oracle: bit-exact."""
import numpy as np
import pytest
import torch

import oracle
from helpers import make_weight, rng

pytestmark = pytest.mark.gpu


def run_case(vocabulary, width, indices, dtype, index_dtype, seed=3):
    from nml_b200 import ops, _abi
    import gpu_util as gu
    triple = make_weight(seed, (vocabulary, width))
    weight = gu.parameter("embedding", triple, width, dtype)
    idx = torch.tensor(indices, dtype=index_dtype).cuda()
    out = ops.token_embedding(weight, idx)
    torch.cuda.synchronize()
    expected = oracle.from_f32(oracle.embedding(np.asarray(indices).ravel(), *triple, width),
                               dtype)
    assert np.array_equal(gu.from_device_bits(out).reshape(-1, width), expected)
    assert tuple(out.shape) == tuple(idx.shape) + (width,)
    assert _abi.device_status(0x1) == 0


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
def test_odd_width_17(dtype, index_dtype):
    # crates/nml/tests/nvfp4_contract.rs:119-178: V=7, W=17, ids [[6,0],[3,3]]
    run_case(7, 17, [[6, 0], [3, 3]], dtype, index_dtype)


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
def test_gpt_oss_width_edges_and_repeats(dtype):
    vocabulary = 1000
    ids = [0, vocabulary - 1, 5, 5, 5, 999, 0, 17]
    run_case(vocabulary, 2880, ids, dtype, torch.int32)


def test_batch_8192_random_ids_bit_exact():
    vocabulary = 4096
    ids = rng(11).integers(0, vocabulary, 8192)
    run_case(vocabulary, 2880, ids.tolist(), oracle.BF16, torch.int32)


def test_widths_not_multiple_of_16_and_tiny():
    for width in (1, 2, 15, 16, 31, 33, 48):
        run_case(9, width, [8, 0, 4], oracle.BF16, torch.int64, seed=width)


def test_golden_rows_decode_bit_exact(golden):
    from nml_b200 import ops
    import gpu_util as gu
    name = "gpt_oss_row_2x2880"
    triple = (golden[f"{name}.payload"], golden[f"{name}.scales"], golden[f"{name}.global"])
    weight = gu.parameter("golden", triple, 2880, oracle.BF16)
    out = ops.token_embedding(weight, torch.tensor([1, 0], dtype=torch.int32).cuda())
    torch.cuda.synchronize()
    expected = oracle.from_f32(golden[f"{name}.decoded"][[1, 0]], oracle.BF16)
    assert np.array_equal(gu.from_device_bits(out), expected)


def test_out_of_range_index_reads_zero_and_sets_status():
    from nml_b200 import ops, _abi
    import gpu_util as gu
    triple = make_weight(5, (6, 32))
    weight = gu.parameter("embedding", triple, 32, oracle.BF16)
    _abi.device_status(0x1)  # clear
    out = ops.token_embedding(weight, torch.tensor([2, 6, -1, 1], dtype=torch.int64).cuda())
    torch.cuda.synchronize()
    bits = gu.from_device_bits(out)
    expected = oracle.from_f32(oracle.embedding([2, 1], *triple, 32), oracle.BF16)
    assert np.array_equal(bits[[0, 3]], expected)
    assert (bits[[1, 2]] == 0).all()
    assert _abi.device_status(0x1) & _abi.STATUS_INDEX_RANGE
    assert _abi.device_status(0x1) == 0  # cleared by the previous read
