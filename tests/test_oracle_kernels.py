"""Pins the CPU oracle's kernels to the closed-form cases of the reference's own tests:
crates/nml-kernel-nvfp4/tests/cpu_contract.rs and crates/nml/tests/nvfp4_contract.rs.
Each case is checked against an independent float64 evaluation written here, with the
tolerance the reference test states."""
import numpy as np
import pytest

import oracle
from helpers import Lcg

MAG = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def dense64(payload, scales, g, width):
    """float64 decode: value * scale * global, no intermediate rounding
    (cpu_contract.rs:44-67)."""
    payload = np.asarray(payload, np.uint8)
    scales = np.asarray(scales, np.uint8)
    lead = payload.shape[:-1]
    p = payload.reshape(-1, payload.shape[-1])
    s = scales.reshape(-1, scales.shape[-1])
    rows = p.shape[0]
    out = np.zeros((rows, width))
    for col in range(width):
        byte = p[:, col // 2]
        code = np.where(col % 2 == 0, byte & 0x0F, byte >> 4)
        val = np.where(code & 8, -MAG[code & 7], MAG[code & 7])
        sb = s[:, col // 16].astype(np.int64)
        e, f = (sb >> 3) & 0xF, sb & 7
        sc = np.where(e == 0, f * 2.0 ** -9, (1 + f / 8.0) * 2.0 ** (e - 7.0))
        out[:, col] = val * sc * float(g)
    return out.reshape(lead + (width,))


def test_embedding_odd_width_selected_rows():
    # cpu_contract.rs:87-104
    values = (np.arange(51, dtype=np.float32) / np.float32(8.0) - np.float32(3.0)).reshape(3, 17)
    payload, scales, g = oracle.quantize_tensor(values)
    out = oracle.embedding([2, 0], payload, scales, g, 17)
    expected = dense64(payload, scales, g, 17)[[2, 0]]
    assert np.abs(out - expected).max() < 1e-6
    with pytest.raises(IndexError):
        oracle.embedding([3], payload, scales, g, 17)
    with pytest.raises(IndexError):
        oracle.embedding([-1], payload, scales, g, 17)


def test_linear_with_bias_odd_width():
    # cpu_contract.rs:106-129
    values = (np.arange(68, dtype=np.float32) / np.float32(11.0) - np.float32(2.5)).reshape(4, 17)
    payload, scales, g = oracle.quantize_tensor(values)
    x = (np.arange(34, dtype=np.float32) / np.float32(13.0) - np.float32(1.0)).reshape(2, 17)
    bias = np.array([0.5, -0.25, 1.0, -2.0], np.float32)
    out = oracle.linear(x, payload, scales, g, bias)
    expected = x.astype(np.float64) @ dense64(payload, scales, g, 17).T + bias
    assert np.abs(out - expected).max() < 2e-5
    out64 = oracle.linear(x, payload, scales, g, bias, mode=1)
    assert np.allclose(out64, expected, rtol=1e-7, atol=1e-7)  # f64 sum, narrowed to f32 once


def test_grouped_projection_uneven_and_empty_experts():
    # cpu_contract.rs:131-160
    values = (np.arange(120, dtype=np.float32) / np.float32(17.0) - np.float32(3.0)).reshape(
        4, 10, 3)
    payload, scales, g = oracle.quantize_tensor(values)
    x = np.array([1.0, 2.0, -1.0, -0.5, 1.5, 3.0, 2.0, 0.0, 0.25], np.float32).reshape(3, 3)
    experts = [2, 2, 0]
    bias = (np.arange(40, dtype=np.float32) / np.float32(100.0)).reshape(4, 10)
    out = oracle.grouped_projection(x, experts, payload, scales, g, bias)
    dense = dense64(payload, scales, g, 3)
    for a, e in enumerate(experts):
        expected = dense[e] @ x[a].astype(np.float64) + bias[e]
        assert np.abs(out[a] - expected).max() < 2e-5
    with pytest.raises(IndexError):
        oracle.grouped_projection(x, [0, 4, 0], payload, scales, g, bias)


def swiglu64(gate_up):
    gate = np.minimum(gate_up[0::2], 7.0)
    up = np.clip(gate_up[1::2], -7.0, 7.0)
    return (up + 1.0) * gate * (1.0 / (1.0 + np.exp(-1.702 * gate)))


def moe64(hidden, idx, w, gate, gate_bias, down, down_bias, H, I):
    tokens, k = idx.shape
    gd = dense64(gate[0], gate[1], gate[2], H)
    dd = dense64(down[0], down[1], down[2], I)
    out = np.zeros((tokens, H))
    for t in range(tokens):
        for r in range(k):
            e = idx[t, r]
            gu = gd[e] @ hidden[t].astype(np.float64) + gate_bias[e]
            act = swiglu64(gu)
            out[t] += float(w[t, r]) * (dd[e] @ act + down_bias[e])
    return out


def test_routed_swiglu_interleaved_clamped_semantics():
    # cpu_contract.rs:162-231
    gate_values = (np.arange(48, dtype=np.float32) / np.float32(5.0) - np.float32(4.0)).reshape(
        3, 8, 2)
    down_values = (np.arange(24, dtype=np.float32) / np.float32(7.0) - np.float32(1.5)).reshape(
        3, 2, 4)
    gate = oracle.quantize_tensor(gate_values)
    down = oracle.quantize_tensor(down_values)
    hidden = np.array([1.0, -0.5, 0.25, 2.0], np.float32).reshape(2, 2)
    idx = np.array([[0, 2], [2, 0]])
    w = np.array([[0.75, 0.25], [0.4, 0.6]], np.float32)
    gb = np.zeros((3, 8), np.float32)
    db = np.zeros((3, 2), np.float32)
    out = oracle.routed_clamped_swiglu(hidden, idx, w, gate, gb, down, db)
    expected = moe64(hidden, idx, w, gate, gb, down, db, 2, 4)
    assert np.abs(out - expected).max() < 3e-5


def test_routed_swiglu_generated_shapes():
    # cpu_contract.rs:233-344 with the generator of :346-357
    lcg = Lcg()
    for tokens, H, E, I, k in [(1, 3, 4, 5, 2), (3, 5, 6, 7, 2), (4, 3, 7, 3, 3)]:
        gate_values = lcg.values(E * H * I * 2, 2.5).reshape(E, 2 * I, H)
        down_values = lcg.values(E * I * H, 2.0).reshape(E, H, I)
        gate = oracle.quantize_tensor(gate_values)
        down = oracle.quantize_tensor(down_values)
        hidden = lcg.values(tokens * H, 1.25).reshape(tokens, H)
        gb = lcg.values(E * I * 2, 0.2).reshape(E, 2 * I)
        db = lcg.values(E * H, 0.2).reshape(E, H)
        idx = np.zeros((tokens, k), np.int64)
        w = np.zeros((tokens, k), np.float32)
        for t in range(tokens):
            raw = [np.float32(0.25) + lcg.unit() + np.float32(r) * np.float32(0.1)
                   for r in range(k)]
            norm = np.float32(0.0)
            for v in raw:
                norm = np.float32(norm + v)
            for r, v in enumerate(raw):
                idx[t, r] = (t * (r + 1) + r * 2) % (E - 1)
                w[t, r] = np.float32(v / norm)
        out = oracle.routed_clamped_swiglu(hidden, idx, w, gate, gb, down, db)
        expected = moe64(hidden, idx, w, gate, gb, down, db, H, I)
        tol = 3e-4 * np.maximum(np.abs(expected), 1.0)
        assert (np.abs(out - expected) <= tol).all(), (tokens, H, E, I, k)
        # the two-stage restatement agrees with the single-pass one
        ids = idx.astype(np.int32).ravel()
        act = oracle.expert_gate_up(hidden, ids, k, gate, gb)
        weighted = oracle.expert_down(act, ids, w.ravel(), down, db)
        staged = weighted.reshape(tokens, k, H).astype(np.float64).sum(axis=1)
        assert (np.abs(staged - expected) <= tol).all()


def contract_close(actual, expected, t):
    # nvfp4_contract.rs:528-531
    return (np.abs(actual - expected) <= t + t * np.abs(expected)).all()


@pytest.mark.parametrize("dtype,t", [(oracle.F16, 1e-2), (oracle.BF16, 6e-2)])
@pytest.mark.parametrize("rows,with_bias", [(3, False), (3, True), (1, True)])
def test_contract_linear_through_16bit_handler(dtype, t, rows, with_bias):
    # nvfp4_contract.rs:48-117
    K, N = 16, 5
    x = ((np.arange(rows * K, dtype=np.float32) - np.float32(19.0)) / np.float32(13.0)).reshape(
        rows, K)
    source = ((np.float32(27.0) - np.arange(N * K, dtype=np.float32)) / np.float32(17.0)).reshape(
        N, K)
    bias = np.array([-0.5, -0.125, 0.0, 0.25, 0.75], np.float32)
    payload, scales, g = oracle.quantize_tensor(source)
    decoded = oracle.dequantize_tensor(payload, scales, g, K)
    expected = x @ decoded.T + (bias if with_bias else 0.0)
    out16, out32 = oracle.linear_16(oracle.from_f32(x, dtype), payload, scales, g, dtype,
                                    oracle.from_f32(bias, dtype) if with_bias else None)
    assert contract_close(oracle.to_f32(out16, dtype), expected, t)
    assert np.array_equal(out16, oracle.from_f32(out32, dtype))


@pytest.mark.parametrize("dtype,t", [(oracle.F16, 1e-2), (oracle.BF16, 6e-2)])
def test_contract_embedding(dtype, t):
    # nvfp4_contract.rs:119-178
    V, W = 7, 17
    source = ((np.arange(V * W, dtype=np.float32) - np.float32(41.0)) / np.float32(19.0)).reshape(
        V, W)
    payload, scales, g = oracle.quantize_tensor(source)
    decoded = oracle.dequantize_tensor(payload, scales, g, W)
    idx = [6, 0, 3, 3]
    out = oracle.embedding(idx, payload, scales, g, W)
    assert np.array_equal(out.view(np.uint32), decoded[idx].view(np.uint32))
    assert contract_close(oracle.to_f32(oracle.from_f32(out, dtype), dtype), decoded[idx], t)


def contract_route_reference(router, k, dtype):
    # nvfp4_contract.rs:450-470: sort logits descending, ties to the lower index,
    # softmax over the selected logits, weight rounded to the activation dtype.
    tokens, E = router.shape
    ids = np.zeros((tokens, k), np.int32)
    w = np.zeros((tokens, k), np.float32)
    for t in range(tokens):
        order = sorted(range(E), key=lambda e: (-float(router[t, e]), e))[:k]
        m = max(router[t, e] for e in order)
        ex = np.array([np.exp(np.float32(router[t, e] - m)) for e in order], np.float32)
        ids[t] = order
        w[t] = oracle.to_f32(oracle.from_f32(ex / ex.sum(dtype=np.float32), dtype), dtype)
    return ids, w


@pytest.mark.parametrize("dtype,t", [(oracle.F16, 1e-2), (oracle.BF16, 6e-2)])
@pytest.mark.parametrize("tokens", [2, 1])
def test_contract_experts_with_routing(dtype, t, tokens):
    # nvfp4_contract.rs:180-312,406-500
    E, H, I, k = 3, 4, 5, 2
    hidden = np.array([((i * 7 % 19) - 9.0) / 4.0 for i in range(tokens * H)],
                      np.float32).reshape(tokens, H)
    router = np.array([((i * 5 % 13) - 6.0) / 3.0 for i in range(tokens * E)],
                      np.float32).reshape(tokens, E)
    gate_source = ((np.arange(E * H * 2 * I, dtype=np.float32) - np.float32(41.0)) /
                   np.float32(23.0)).reshape(E, 2 * I, H)
    down_source = ((np.float32(17.0) - np.arange(E * I * H, dtype=np.float32)) /
                   np.float32(29.0)).reshape(E, H, I)
    gb = ((np.arange(E * 2 * I, dtype=np.float32) - np.float32(9.0)) / np.float32(31.0)).reshape(
        E, 2 * I)
    db = ((np.float32(5.0) - np.arange(E * H, dtype=np.float32)) / np.float32(37.0)).reshape(E, H)
    gate = oracle.quantize_tensor(gate_source)
    down = oracle.quantize_tensor(down_source)
    r = lambda v: oracle.to_f32(oracle.from_f32(v, dtype), dtype)
    ids, w32, w16 = oracle.route(router, k, dtype)
    ref_ids, ref_w = contract_route_reference(router, k, dtype)
    assert np.array_equal(ids, ref_ids)
    assert np.abs(oracle.to_f32(w16, dtype) - ref_w).max() <= 2 ** -8
    out = oracle.routed_clamped_swiglu(r(hidden), ids, oracle.to_f32(w16, dtype), gate, r(gb),
                                       down, r(db))
    expected = moe64(r(hidden), ref_ids, ref_w, gate, r(gb), down, r(db), H, I)
    assert contract_close(r(out), expected, t)


def test_exp_det_accuracy_and_edges():
    xs = np.concatenate([np.linspace(-87.0, 0.0, 20001), -np.logspace(-8, 1.9, 500)])
    got = np.array([oracle.exp_det(x) for x in xs])
    want = np.exp(xs.astype(np.float32).astype(np.float64))
    assert np.abs(got / want - 1.0).max() < 2.5e-7
    assert oracle.exp_det(0.0) == 1.0
    assert oracle.exp_det(-100.0) == 0.0
    assert oracle.exp_det(float("-inf")) == 0.0


def test_route_ties_masks_and_degenerate_rows():
    # ties go to the lower expert index (crates/nml-ir/src/lib.rs:3534-3605)
    logits = np.zeros((3, 8), np.float32)
    logits[1, [5, 2]] = 1.0
    logits[2, :] = -np.inf
    ids, w32, w16 = oracle.route(logits, 4, oracle.BF16, active=[1, 1, 1])
    assert ids[0].tolist() == [0, 1, 2, 3]
    assert ids[1].tolist() == [2, 5, 0, 1]
    assert np.allclose(w32[0], 0.25)
    assert np.isclose(w32.sum(axis=1)[:2], 1.0, atol=1e-6).all()
    # all -inf row: probabilities 0, normaliser clamps to epsilon, weights 0
    assert ids[2].tolist() == [0, 1, 2, 3] and (w32[2] == 0).all()
    # masked tokens: expert -1 and weight 0 (crates/nml-ir/src/lib.rs:1426-1436)
    ids, w32, w16 = oracle.route(logits, 2, oracle.BF16, active=[0, 1, 0])
    assert (ids[0] == -1).all() and (w32[0] == 0).all() and (w16[0] == 0).all()
    assert ids[1].tolist() == [2, 5]


def plan_reference(ids, experts, block):
    """Independent numpy statement of crates/nml-ir/src/lib.rs:5644-5779."""
    ids = np.asarray(ids, np.int32)
    A = ids.size
    max_blocks = (A + min(A, experts) * (block - 1) + block - 1) // block
    sorted_assignments = np.full(max_blocks * block, A, np.int32)
    block_experts = np.full(max_blocks, -1, np.int32)
    if A <= experts:
        sorted_assignments[np.arange(A) * block] = np.arange(A)
        block_experts[:A] = ids
        return sorted_assignments, block_experts, A
    prefix = 0
    for e in range(experts):
        assigned = ids == e
        positions = np.cumsum(assigned) - 1
        count = int(assigned.sum())
        padded = (count + block - 1) // block * block
        sorted_assignments[prefix + positions[assigned]] = np.nonzero(assigned)[0]
        block_experts[prefix // block:(prefix + padded) // block] = e
        prefix += padded
    return sorted_assignments, block_experts, prefix // block


@pytest.mark.parametrize("A,E,seed", [(8, 32, 1), (32, 32, 2), (33, 32, 3), (256, 32, 4),
                                      (1000, 7, 5), (16384, 32, 6), (40, 4, 7)])
def test_assignment_plan_matches_reference_construction(A, E, seed):
    r = np.random.default_rng(seed)
    ids = r.integers(0, E, A).astype(np.int32)
    if seed % 2 == 0:
        ids[r.integers(0, A, max(1, A // 7))] = -1  # masked routes
    if E > 3:
        ids[ids == 1] = 0  # force an empty expert
    s, b, active = oracle.assignment_plan(ids, E, 16)
    rs, rb, ractive = plan_reference(ids, E, 16)
    assert np.array_equal(s, rs) and np.array_equal(b, rb) and active == ractive
    assert s.size == oracle.plan_capacity(A, E)[1]


def test_plan_capacity_figures():
    # T=4096,k=4 -> 1054 blocks / 16864 slots; T=64 -> 46 blocks
    assert oracle.plan_capacity(16384, 32) == (1054, 16864)
    assert oracle.plan_capacity(256, 32)[0] == 46


def test_avx2_and_scalar_evaluations_return_identical_bits():
    from helpers import make_activation, make_weight
    w = make_weight(1, (96, 2880))
    _, x = make_activation(2, (5, 2880))
    bias = np.linspace(-1, 1, 96, dtype=np.float32)
    try:
        oracle.set_avx2(False)
        scalar = oracle.linear(x, *w, bias)
    finally:
        oracle.set_avx2(True)
    vector = oracle.linear(x, *w, bias)
    assert np.array_equal(scalar.view(np.uint32), vector.view(np.uint32))
    odd = make_weight(3, (7, 49))
    _, xo = make_activation(4, (3, 49))
    try:
        oracle.set_avx2(False)
        scalar = oracle.linear(xo, *odd)
    finally:
        oracle.set_avx2(True)
    assert np.array_equal(scalar.view(np.uint32), oracle.linear(xo, *odd).view(np.uint32))
