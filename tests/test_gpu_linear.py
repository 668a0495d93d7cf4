"""NVFP4 linear through the C ABI against the oracle's f32-accumulated output.

Bar for every case: max relative error <= 2e-2 and mean relative error <= 2e-3 (see
gpu_util.assert_gemm_close for the exact definition)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import make_activation, make_weight, rng

pytestmark = pytest.mark.gpu


def run_linear(M, K, N, dtype, policy, with_bias=False, seed=0, sample_rows=None,
               expect_kernel=None):
    from nml_b200 import ops, _abi
    import gpu_util as gu
    triple = make_weight(100 + seed, (N, K))
    weight = gu.parameter("w", triple, K, dtype)
    x_bits, x32 = make_activation(200 + seed, (M, K), dtype=dtype)
    bias_bits = bias32 = None
    if with_bias:
        bias_bits, bias32 = make_activation(300 + seed, (N,), std=0.5, dtype=dtype)
    x = gu.to_device_bits(x_bits, dtype)
    bias = None if bias_bits is None else gu.to_device_bits(bias_bits, dtype)
    previous = _abi.set_kernel_policy(policy)
    try:
        y = ops.linear(x, weight, bias)
        torch.cuda.synchronize()
        kernel = _abi.last_linear_kernel()
    finally:
        _abi.set_kernel_policy(previous)
    assert _abi.device_status(0x1) == 0
    if expect_kernel is not None:
        assert kernel.startswith(expect_kernel), kernel
    rows = np.arange(M) if sample_rows is None or sample_rows >= M else np.sort(
        rng(seed).choice(M, sample_rows, replace=False))
    expected = oracle.linear(x32[rows], *triple, bias32)
    actual = gu.device_f32(y)[rows]
    return gu.assert_gemm_close(actual, expected, f"M={M} K={K} N={N} policy={policy}")


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
@pytest.mark.parametrize("M,K,N,bias", [(1, 16, 5, True), (3, 16, 5, False), (3, 16, 5, True),
                                        (2, 17, 4, True), (17, 80, 33, False), (1, 17, 5, False),
                                        (3, 33, 4, True), (1, 2880, 64, False)])
def test_portable_kernel_odd_shapes(dtype, M, K, N, bias):
    # shapes of crates/nml-kernel-nvfp4/tests/cpu_contract.rs:106-129 and
    # crates/nml/tests/nvfp4_contract.rs:48-117, plus odd extents
    from nml_b200 import _abi
    run_linear(M, K, N, dtype, _abi.POLICY_SIMT, bias, seed=M + K + N, expect_kernel="simt")


def test_contract_linear_closed_form_inputs():
    # crates/nml/tests/nvfp4_contract.rs:48-117, tolerance of :528-531
    from nml_b200 import ops
    import gpu_util as gu
    K, N = 16, 5
    source = ((np.float32(27.0) - np.arange(N * K, dtype=np.float32)) / np.float32(17.0)).reshape(
        N, K)
    triple = oracle.quantize_tensor(source)
    decoded = oracle.dequantize_tensor(*triple, K)
    bias = np.array([-0.5, -0.125, 0.0, 0.25, 0.75], np.float32)
    for dtype, t in ((oracle.F16, 1e-2), (oracle.BF16, 6e-2)):
        for rows, with_bias in ((3, False), (3, True), (1, True)):
            x = ((np.arange(rows * K, dtype=np.float32) - np.float32(19.0)) /
                 np.float32(13.0)).reshape(rows, K)
            weight = gu.parameter("w", triple, K, dtype)
            y = ops.linear(gu.to_device_bits(oracle.from_f32(x, dtype), dtype), weight,
                           gu.to_device_bits(oracle.from_f32(bias, dtype), dtype)
                           if with_bias else None)
            expected = x @ decoded.T + (bias if with_bias else 0.0)
            assert (np.abs(gu.device_f32(y) - expected) <= t + t * np.abs(expected)).all()


UMMA_CASES = [(1, 64, 128), (16, 128, 128), (17, 256, 200), (64, 2880, 2880), (100, 2880, 640),
              (130, 512, 384), (300, 1024, 256), (1, 2880, 5760)]


# POLICY_UMMA picks the variant with decoded weights in tensor memory where the shape allows
# it (outputs a multiple of 4, K <= 3072, tiles of at most 128 activation rows, which all of
# these cases get); POLICY_UMMA_SMEM forces the shared-memory ring.
@pytest.mark.parametrize("M,K,N", UMMA_CASES)
def test_tensor_core_kernel_f16_activations(M, K, N):
    from nml_b200 import _abi
    run_linear(M, K, N, oracle.F16, _abi.POLICY_UMMA, with_bias=(M % 2 == 0), seed=M + N,
               expect_kernel="umma_tmem_weights_af16")


@pytest.mark.parametrize("M,K,N", UMMA_CASES)
def test_tensor_core_kernel_bf16_activations(M, K, N):
    from nml_b200 import _abi
    run_linear(M, K, N, oracle.BF16, _abi.POLICY_UMMA, with_bias=(M % 2 == 1), seed=M + N,
               expect_kernel="umma_tmem_weights_abf16")


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
@pytest.mark.parametrize("M,K,N", UMMA_CASES + [(16, 4096, 2880), (64, 128, 130)])
def test_tensor_core_kernel_shared_memory_weight_ring(M, K, N, dtype):
    from nml_b200 import _abi
    run_linear(M, K, N, dtype, _abi.POLICY_UMMA_SMEM, with_bias=(M % 2 == 1), seed=M + N + 1,
               expect_kernel="umma_swapab_a")


@pytest.mark.parametrize("M,K,N", [(64, 128, 130), (33, 16384, 512)])
def test_tensor_core_kernel_falls_back_to_shared_memory_ring(M, K, N):
    # a scale buffer (128 rows x K/16 bytes, rows padded apart) that does not fit beside the
    # rings even alone, or an output count that breaks the bulk scale copy
    from nml_b200 import _abi
    run_linear(M, K, N, oracle.BF16, _abi.POLICY_UMMA, seed=M + N + 2,
               expect_kernel="umma_swapab_abf16")


@pytest.mark.parametrize("M,K,N", [(200, 8192, 256), (512, 4096, 2880), (40, 4096, 384),
                                   (4096, 4096, 2880)])
def test_tensor_core_kernel_with_one_scale_buffer(M, K, N):
    # K >= 4096: 256- and 512-byte scale rows are copied row by row with a padded pitch, and
    # where two such buffers do not fit the kernel runs with one (units take turns on it)
    from nml_b200 import _abi
    run_linear(M, K, N, oracle.BF16, _abi.POLICY_UMMA, seed=M + N + 3, with_bias=True,
               sample_rows=48)


CONFIG_SHAPES = [(2880, 5120), (4096, 2880), (2880, 5760), (2880, 2880)]


@pytest.mark.parametrize("K,N", CONFIG_SHAPES)
@pytest.mark.parametrize("M", [1, 16, 64])
def test_config_shapes_small_m_full_oracle(K, N, M):
    # decode shapes: the weight-streaming kernel (these weights stay in L2, so it also takes
    # M = 64 as four groups of 16 rows)
    from nml_b200 import _abi
    run_linear(M, K, N, oracle.BF16, _abi.POLICY_AUTO, seed=K + N + M, expect_kernel="stream")


@pytest.mark.parametrize("K,N", CONFIG_SHAPES)
@pytest.mark.parametrize("M", [1, 16, 64])
def test_config_shapes_small_m_tensor_core_kernel(K, N, M):
    # the tcgen05 kernel on the same shapes (it serves them when streaming is not possible)
    from nml_b200 import _abi
    run_linear(M, K, N, oracle.BF16, _abi.POLICY_UMMA, seed=K + N + M, expect_kernel="umma")


@pytest.mark.parametrize("K,N", CONFIG_SHAPES)
@pytest.mark.parametrize("M", [512, 4096, 16384])
def test_config_shapes_large_m_sampled_rows(K, N, M):
    from nml_b200 import _abi
    run_linear(M, K, N, oracle.BF16, _abi.POLICY_AUTO, seed=K + N + M, sample_rows=24,
               expect_kernel="umma")


_UNEMBEDDING = {}


def unembedding_weight():
    """The 201088 x 2880 table, quantized once for all row counts (the CPU side of these
    cases is dominated by generating it)."""
    if "triple" not in _UNEMBEDDING:
        _UNEMBEDDING["triple"] = make_weight(4242, (201088, 2880))
    return _UNEMBEDDING["triple"]


@pytest.mark.parametrize("M", [1, 16, 64, 512, 1024, 4096, 16384])
def test_unembedding_shape(M):
    # every row count of the shape sweep (and 1024 of the logits configuration) on the
    # vocabulary projection; the oracle evaluates a seeded sample of rows over all columns
    from nml_b200 import ops, _abi
    import gpu_util as gu
    triple = unembedding_weight()
    if "weight" not in _UNEMBEDDING:
        _UNEMBEDDING["weight"] = gu.parameter("head", triple, 2880, oracle.BF16)
    weight = _UNEMBEDDING["weight"]
    x_bits, x32 = make_activation(200 + M, (M, 2880))
    y = ops.linear(gu.to_device_bits(x_bits, oracle.BF16), weight)
    torch.cuda.synchronize()
    assert _abi.device_status(0x1) == 0
    assert _abi.last_linear_kernel().startswith("stream" if M <= 16 else "umma")
    rows = np.arange(M) if M <= 4 else np.sort(rng(M).choice(M, 4, replace=False))
    expected = oracle.linear(x32[rows], *triple, None)
    actual = y[torch.from_numpy(rows).cuda()].float().cpu().numpy()
    del y
    gu.assert_gemm_close(actual, expected, f"unembedding M={M}")


def _plain_linear(x, weight, outputs):
    """The same call without scratch: BF16 operands."""
    from nml_b200 import ops, _abi
    plain = torch.empty((x.shape[0], outputs), dtype=x.dtype, device=x.device)
    request = _abi.Linear(activation=x.data_ptr(), payload=weight.payload.data_ptr(),
                          block_scales=weight.block_scales.data_ptr(),
                          global_scale=weight.global_scale.data_ptr(), bias=None,
                          output=plain.data_ptr(), stream=ops._stream(x), rows=x.shape[0],
                          outputs=outputs, inputs=x.shape[1], dtype=_abi.BF16)
    _abi.call("nml_nvfp4_sm100_linear", request)
    torch.cuda.synchronize()
    assert _abi.last_linear_kernel().startswith("umma_swapab_abf16")
    return plain


def _verdict(M):
    from nml_b200 import ops, _abi
    lib = _abi.load()
    assert lib.nml_nvfp4_sm100_linear_workspace_bytes(M, 201088, 2880, _abi.BF16) > 0
    offset = lib.nml_nvfp4_sm100_linear_workspace_verdict_offset(M, 201088, 2880, _abi.BF16)
    device = torch.device("cuda", torch.cuda.current_device())
    scratch = ops._LINEAR_SCRATCH[(device, torch.cuda.current_stream(device).cuda_stream)]
    return int(scratch[offset:offset + 4].view(torch.int32).item())


@pytest.mark.parametrize("M", [512, 700])
def test_wide_weight_runs_on_narrowed_f16_operands(M):
    # BF16 rows of a wide weight run as F16 operands, one power of two per 256-row tile, when
    # the request carries scratch and every row lies within 2^8 of its tile's largest; tiles
    # may differ by any factor, rows of zeros pass, the last tile is partial at M = 700
    from nml_b200 import ops, _abi
    import gpu_util as gu
    triple = unembedding_weight()
    if "weight" not in _UNEMBEDDING:
        _UNEMBEDDING["weight"] = gu.parameter("head", triple, 2880, oracle.BF16)
    weight = _UNEMBEDDING["weight"]
    _, x32 = make_activation(777 + M, (M, 2880))
    exponents = rng(778).integers(-3, 4, size=M)
    exponents[256:512] += 50
    exponents[512:] -= 60
    x32 = x32 * np.exp2(exponents)[:, None].astype(np.float32)
    x32[5] = 0.0
    x = torch.from_numpy(x32).to(torch.bfloat16).cuda()
    x32 = x.float().cpu().numpy()
    y = ops.linear(x, weight)
    torch.cuda.synchronize()
    assert _abi.device_status(0x1) == 0
    assert _abi.last_linear_kernel().startswith("umma_swapab_narrowed_af16")
    assert _verdict(M) == 0
    plain = _plain_linear(x, weight, 201088)
    assert torch.isfinite(y).all()
    assert (y[5] == 0).all()
    # the same operands in another 16-bit format: a rounding step apart, up to cancellation
    difference = (y.float() - plain.float()).abs()
    slack = 1e-3 * plain.float().abs().amax(dim=1, keepdim=True)
    assert (difference <= 2.0 ** -7 * plain.float().abs() + slack).all()
    rows = np.array([0, 5, 300, M - 1])
    expected = oracle.linear(x32[rows], *triple, None)
    gu.assert_gemm_close(y[torch.from_numpy(rows).cuda()].float().cpu().numpy(), expected,
                         "narrowed rows")


@pytest.mark.parametrize("case", ["row_far_below_its_tile", "infinity", "tiny_tile"])
def test_wide_weight_keeps_bf16_operands_where_narrowing_would_lose_bits(case):
    # the device decides: the verdict word is raised and the BF16-operand kernel writes the
    # output, bit for bit what the call gives without scratch
    from nml_b200 import ops, _abi
    import gpu_util as gu
    triple = unembedding_weight()
    if "weight" not in _UNEMBEDDING:
        _UNEMBEDDING["weight"] = gu.parameter("head", triple, 2880, oracle.BF16)
    weight = _UNEMBEDDING["weight"]
    M = 512
    _, x32 = make_activation(779, (M, 2880))
    if case == "row_far_below_its_tile":
        x32[300] *= 2.0 ** -20
    elif case == "infinity":
        x32[17, 100] = np.inf
    else:
        x32[256:] *= 2.0 ** -120
    x = torch.from_numpy(x32).to(torch.bfloat16).cuda()
    y = ops.linear(x, weight)
    torch.cuda.synchronize()
    assert _abi.device_status(0x1) == 0
    assert _verdict(M) == 1
    plain = _plain_linear(x, weight, 201088)
    assert torch.equal(y.view(torch.int16), plain.view(torch.int16))


@pytest.mark.parametrize("M", [4500, 16384])
def test_unembedding_visits_every_tile_once_when_rows_are_walked_in_blocks(M):
    # more than 24 MB of activations: the row tiles are walked in blocks of 8 (18 tiles at
    # M = 4500: two full blocks and a block of two, the last tile partial).  Equal input rows must give equal output
    # rows, and no element of a poisoned output may survive.
    from nml_b200 import ops
    import gpu_util as gu
    triple = unembedding_weight()
    if "weight" not in _UNEMBEDDING:
        _UNEMBEDDING["weight"] = gu.parameter("head", triple, 2880, oracle.BF16)
    weight = _UNEMBEDDING["weight"]
    x_bits, x32 = make_activation(31, (1, 2880))
    x = gu.to_device_bits(x_bits, oracle.BF16).expand(M, 2880).contiguous()
    out = torch.full((M, 201088), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear(x, weight, out=out)
    torch.cuda.synchronize()
    first = out[0].clone()
    assert torch.isfinite(first).all()
    for start in range(0, M, 1024):  # chunks bound the temporaries
        block = out[start:start + 1024]
        assert torch.equal(block.view(torch.int16), first.view(torch.int16).expand_as(block))
    expected = oracle.linear(x32, *triple, None)
    gu.assert_gemm_close(first.float().cpu().numpy()[None], expected, "blocked walk")


def test_single_linear_of_the_cpu_runnable_configuration():
    # X bf16 [16, 2880], W [5760, 2880]
    from nml_b200 import _abi
    run_linear(16, 2880, 5760, oracle.BF16, _abi.POLICY_AUTO, seed=7)


QKV_CASES = [(1, 2880, (4096, 512, 512), True), (8, 2880, (4096, 512, 512), False),
             (64, 2880, (4096, 512, 512), True), (300, 2880, (4096, 512, 512), True),
             (16, 256, (130, 64, 200), True),     # odd output counts: shared-memory weight ring
             (5, 80, (33, 16, 7), True)]          # K not a multiple of 64: three SIMT launches


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
@pytest.mark.parametrize("M,K,outputs,with_bias", QKV_CASES)
def test_fused_qkv_matches_three_linears_and_oracle(M, K, outputs, with_bias, dtype):
    # crates/nml-ir/src/nvfp4_backend.rs:221-380: Q, K and V share the activation; every
    # projection has its own weight triple, global scale and bias
    from nml_b200 import ops, _abi
    import gpu_util as gu
    x_bits, x32 = make_activation(900 + M, (M, K), dtype=dtype)
    x = gu.to_device_bits(x_bits, dtype)
    weights, biases, triples, biases32 = [], [], [], []
    for i, n in enumerate(outputs):
        triple = make_weight(910 + i + n, (n, K))
        triples.append(triple)
        weights.append(gu.parameter(f"w{i}", triple, K, dtype))
        if with_bias and i != 1:  # the key projection goes without a bias
            bits, b32 = make_activation(920 + i, (n,), std=0.5, dtype=dtype)
            biases.append(gu.to_device_bits(bits, dtype))
            biases32.append(b32)
        else:
            biases.append(None)
            biases32.append(None)
    fused = ops.linear_qkv(x, weights[0], biases[0], weights[1], biases[1], weights[2], biases[2])
    torch.cuda.synchronize()
    assert _abi.device_status(0x1) == 0
    for i in range(3):
        expected = oracle.linear(x32, *triples[i], biases32[i])
        gu.assert_gemm_close(gu.device_f32(fused[i]), expected, f"qkv projection {i} M={M}")
    if M <= 64:
        # Same tile height either way, so the same instruction stream per row -- once the
        # K split over a cluster (whose width follows the tile count of the launch) is off.
        previous = _abi.set_kernel_policy(_abi.POLICY_NO_SPLIT_K)
        try:
            fused = ops.linear_qkv(x, weights[0], biases[0], weights[1], biases[1], weights[2],
                                   biases[2])
            for i in range(3):
                single = ops.linear(x, weights[i], biases[i])
                torch.cuda.synchronize()
                assert torch.equal(fused[i].view(torch.int16), single.view(torch.int16)), i
        finally:
            _abi.set_kernel_policy(previous)
    assert _abi.device_status(0x1) == 0


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
@pytest.mark.parametrize("M,K,N", [(1, 2880, 5760), (16, 2880, 2880), (32, 4096, 2880),
                                   (16, 1024, 640), (8, 2880, 128)])
def test_split_k_over_a_cluster_matches_oracle_and_unsplit_kernel(M, K, N, dtype):
    # few weight tiles and few rows: the K range is cut over the CTAs of a cluster and the
    # partial tiles meet in rank 0's shared memory
    from nml_b200 import ops, _abi
    import gpu_util as gu
    triple = make_weight(1000 + N, (N, K))
    weight = gu.parameter("w", triple, K, dtype)
    x_bits, x32 = make_activation(1001 + M, (M, K), dtype=dtype)
    x = gu.to_device_bits(x_bits, dtype)
    previous = _abi.set_kernel_policy(_abi.POLICY_UMMA)
    try:
        split = ops.linear(x, weight)
        again = ops.linear(x, weight)
        _abi.set_kernel_policy(_abi.POLICY_NO_SPLIT_K)
        unsplit = ops.linear(x, weight)
        assert _abi.last_linear_kernel().startswith("umma")
    finally:
        _abi.set_kernel_policy(previous)
    torch.cuda.synchronize()
    assert _abi.device_status(0x1) == 0
    assert torch.equal(split.view(torch.int16), again.view(torch.int16))  # deterministic
    expected = oracle.linear(x32, *triple, None)
    gu.assert_gemm_close(gu.device_f32(split), expected, f"split M={M} K={K} N={N}")
    gu.assert_gemm_close(gu.device_f32(unsplit), expected, f"unsplit M={M} K={K} N={N}")


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
@pytest.mark.parametrize("M,K,N,policy_name", [
    (1, 4096, 2880, "POLICY_AUTO"), (16, 4096, 2880, "POLICY_AUTO"),   # weight-streaming kernel
    (64, 4096, 2880, "POLICY_UMMA"), (300, 4096, 2880, "POLICY_AUTO"),  # tcgen05, both homes
    (520, 2880, 2880, "POLICY_UMMA_SMEM"), (5, 48, 20, "POLICY_SIMT")])
def test_residual_operand_equals_a_separate_add(M, K, N, policy_name, dtype):
    # products/serve/src/gpt_oss/graph.rs:534-543: hidden + o_proj(attention).  The epilogue
    # narrows the projection, adds the residual and narrows again, so the fused call equals the
    # two-step evaluation bit for bit, also when the residual is the output buffer itself.
    from nml_b200 import ops, _abi
    import gpu_util as gu
    triple = make_weight(1300, (N, K))
    weight = gu.parameter("w", triple, K, dtype)
    x_bits, _ = make_activation(1301, (M, K), dtype=dtype)
    bias_bits, _ = make_activation(1302, (N,), std=0.5, dtype=dtype)
    res_bits, _ = make_activation(1303, (M, N), std=2.0, dtype=dtype)
    x, bias = gu.to_device_bits(x_bits, dtype), gu.to_device_bits(bias_bits, dtype)
    residual = gu.to_device_bits(res_bits, dtype)
    previous = _abi.set_kernel_policy(getattr(_abi, policy_name))
    try:
        plain = ops.linear(x, weight, bias)
        fused = ops.linear(x, weight, bias, residual=residual)
        in_place = residual.clone()
        ops.linear(x, weight, bias, out=in_place, residual=in_place)
        torch.cuda.synchronize()
    finally:
        _abi.set_kernel_policy(previous)
    two_step = (plain.float() + residual.float()).to(plain.dtype)
    assert torch.equal(fused.view(torch.int16), two_step.view(torch.int16))
    assert torch.equal(in_place.view(torch.int16), two_step.view(torch.int16))
    with pytest.raises(ValueError):
        ops.linear(x, weight, bias, residual=residual[:, :-1])
    assert _abi.device_status(0x1) == 0
