"""Routing, assignment plan and routed experts through the C ABI against the oracle.

Routing ids, routing weights and the plan are integer/selection work: bit-exact.  The two
expert projections are GEMM outputs: the 2e-2 / 2e-3 relative-error bar against the oracle's
f32-accumulated result computed from the same inputs."""
import numpy as np
import pytest
import torch

import oracle
from helpers import Lcg, make_activation, make_weight, rng

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,k,dtype", [(4096, 32, 4, oracle.BF16),
                                                   (64, 32, 4, oracle.BF16),
                                                   (7, 3, 2, oracle.F16), (33, 128, 8, oracle.BF16),
                                                   (5, 200, 16, oracle.F16), (1, 32, 4, oracle.BF16)])
def test_route_ids_and_weights_bit_exact(tokens, experts, k, dtype):
    from nml_b200 import ops
    import gpu_util as gu
    logits = (rng(tokens + experts).standard_normal((tokens, experts)) * 0.6).astype(np.float32)
    ids, w = ops.route(torch.from_numpy(logits).cuda(), k, gu.TORCH_DTYPE[dtype])
    e_ids, _, e_w16 = oracle.route(logits, k, dtype)
    assert np.array_equal(ids.cpu().numpy(), e_ids)
    assert np.array_equal(gu.from_device_bits(w), e_w16)


def test_route_ties_masks_and_degenerate_rows():
    from nml_b200 import ops
    import gpu_util as gu
    logits = np.zeros((6, 32), np.float32)
    logits[1, [5, 2]] = 1.0
    logits[2, :] = -np.inf
    logits[3] = np.round(rng(1).standard_normal(32) * 2) / 2  # many exact ties
    logits[4, :] = 80.0
    logits[4, 7] = -80.0
    logits[5] = rng(2).standard_normal(32).astype(np.float32) * 1e-7  # ties after exp rounding
    active = np.array([1, 1, 1, 1, 0, 1], np.uint8)
    for mask in (None, active):
        ids, w = ops.route(torch.from_numpy(logits).cuda(), 4, torch.bfloat16,
                           None if mask is None else torch.from_numpy(mask).bool().cuda())
        e_ids, _, e_w16 = oracle.route(logits, 4, oracle.BF16, active=mask)
        assert np.array_equal(ids.cpu().numpy(), e_ids)
        assert np.array_equal(gu.from_device_bits(w), e_w16)
    assert ids.cpu().numpy()[0].tolist() == [0, 1, 2, 3]
    assert (ids.cpu().numpy()[4] == -1).all()


@pytest.mark.parametrize("A,E,seed", [(8, 32, 1), (32, 32, 2), (33, 32, 3), (256, 32, 4),
                                      (1000, 7, 5), (16384, 32, 6), (40, 4, 7), (5000, 256, 8),
                                      (70000, 32, 9)])
def test_assignment_plan_bit_exact(A, E, seed):
    from nml_b200 import ops
    r = rng(seed)
    ids = r.integers(0, E, A).astype(np.int32)
    if seed % 2 == 0:
        ids[r.integers(0, A, max(1, A // 7))] = -1
    if E > 3:
        ids[ids == 1] = 0
    plan = ops.moe_assignment_plan(torch.from_numpy(ids).cuda(), E)
    s, b, active = oracle.assignment_plan(ids, E, 16)
    assert int(plan.active_blocks.item()) == active
    assert np.array_equal(plan.sorted_assignments.cpu().numpy(), s)
    assert np.array_equal(plan.block_experts.cpu().numpy(), b)


def test_assignment_plan_expert_parallel_slice():
    # ids outside [offset, offset + local) are left out like masked routes
    from nml_b200 import ops
    ids = rng(3).integers(0, 32, 2000).astype(np.int32)
    offset, local = 8, 8
    plan = ops.moe_assignment_plan(torch.from_numpy(ids).cuda(), local, expert_offset=offset)
    shifted = np.where((ids >= offset) & (ids < offset + local), ids - offset, -1).astype(np.int32)
    s, b, active = oracle.assignment_plan(shifted, local, 16)
    assert int(plan.active_blocks.item()) == active
    assert np.array_equal(plan.sorted_assignments.cpu().numpy(), s)
    assert np.array_equal(plan.block_experts.cpu().numpy(), b)


def make_experts(seed, E, H, I, dtype, std=0.02, bias_std=0.02):
    gate = make_weight(seed, (E, 2 * I, H), std)
    down = make_weight(seed + 1, (E, H, I), std)
    gb_bits, gb = make_activation(seed + 2, (E, 2 * I), bias_std, dtype)
    db_bits, db = make_activation(seed + 3, (E, H), bias_std, dtype)
    return gate, down, (gb_bits, gb), (db_bits, db)


def run_routed(tokens, H, E, I, k, dtype, policy, seed=0, std=0.02, mask=None):
    from nml_b200 import ops, _abi
    import gpu_util as gu
    gate, down, (gb_bits, gb), (db_bits, db) = make_experts(seed, E, H, I, dtype, std)
    x_bits, x = make_activation(seed + 9, (tokens, H), 1.0, dtype)
    logits = (rng(seed + 10).standard_normal((tokens, E)) * 0.6).astype(np.float32)
    ids, w32, w16 = oracle.route(logits, k, dtype, active=mask)
    w = oracle.to_f32(w16, dtype)
    gate_p = gu.parameter("gate_up", gate, H, dtype)
    down_p = gu.parameter("down", down, I, dtype)
    d_x = gu.to_device_bits(x_bits, dtype)
    d_gb = gu.to_device_bits(gb_bits, dtype)
    d_db = gu.to_device_bits(db_bits, dtype)
    d_ids = torch.from_numpy(ids).cuda()
    d_w = gu.to_device_bits(w16, dtype)
    previous = _abi.set_kernel_policy(policy)
    try:
        plan = ops.moe_assignment_plan(d_ids.reshape(-1), E)
        activated = ops.expert_gate_up(d_x, plan, gate_p, d_gb, k)
        weighted = ops.expert_down(activated, plan, down_p, d_db, d_w.reshape(-1), k)
        combined = ops.combine(weighted, tokens, k, d_ids.reshape(-1), E, 0)
        fused = ops.routed_experts(d_x, d_ids, d_w, gate_p, d_gb, down_p, d_db)
        end_to_end = ops.routed_clamped_swiglu_masked(
            d_x, torch.from_numpy(logits).cuda(), gate_p, d_gb, down_p, d_db, k,
            None if mask is None else torch.from_numpy(np.asarray(mask, np.uint8)).bool().cuda())
        torch.cuda.synchronize()
    finally:
        _abi.set_kernel_policy(previous)
    assert _abi.device_status(0x1) == 0
    valid = ids.ravel() >= 0
    # stage 1: gate/up + SwiGLU from the same hidden rows
    e_act = oracle.expert_gate_up(x, ids.ravel(), k, gate, gb)
    gu.assert_gemm_close(gu.device_f32(activated)[valid], e_act[valid], "gate_up")
    # stage 2: down from the device's own (narrowed) activations
    act_in = gu.device_f32(activated)
    e_weighted = oracle.expert_down(act_in, ids.ravel(), w.ravel(), down, db)
    gu.assert_gemm_close(gu.device_f32(weighted)[valid], e_weighted[valid], "down")
    # stage 3: the k-way sum is f32 with one narrowing: bit-exact against the oracle
    w_bits = gu.from_device_bits(weighted).copy()
    w_bits[~valid] = 0
    assert np.array_equal(gu.from_device_bits(combined),
                          oracle.combine(w_bits, tokens, k, dtype, mode=0))
    assert np.array_equal(gu.from_device_bits(fused), gu.from_device_bits(combined))
    assert np.array_equal(gu.from_device_bits(end_to_end), gu.from_device_bits(combined))
    # whole layer against the reference CPU semantics (f32 activations between the two
    # projections, crates/nml-kernel-nvfp4/src/lib.rs:333-448).  The device path narrows the
    # activations and the weighted rows to the activation dtype like the reference's device
    # path does, so the layer-level bar is the norm-wise error ||a - e|| / ||e|| <= 1e-2
    # (elementwise bars do not survive the cancellation in tiny random layers).
    safe_ids = np.where(ids < 0, 0, ids)
    e_layer = oracle.routed_clamped_swiglu(x, safe_ids, np.where(ids < 0, 0, w), gate, gb, down,
                                           db)
    m = oracle.error_metrics(gu.device_f32(fused), e_layer)
    assert m["norm_rel"] <= 1e-2, m
    return m


@pytest.mark.parametrize("tokens,H,E,I,k", [(1, 3, 4, 5, 2), (3, 5, 6, 7, 2), (4, 3, 7, 3, 3),
                                            (2, 4, 3, 5, 2), (1, 4, 3, 5, 2), (40, 48, 4, 24, 2)])
@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.F16])
def test_routed_experts_small_shapes_portable_kernel(tokens, H, E, I, k, dtype):
    # shapes of crates/nml-kernel-nvfp4/tests/cpu_contract.rs:236-238 and
    # crates/nml/tests/nvfp4_contract.rs:180-184
    from nml_b200 import _abi
    run_routed(tokens, H, E, I, k, dtype, _abi.POLICY_SIMT, seed=tokens + H + E, std=1.0)


def test_routed_experts_masked_tokens_and_empty_experts():
    from nml_b200 import _abi
    mask = np.ones(40, np.uint8)
    mask[[0, 7, 39]] = 0
    run_routed(40, 64, 6, 32, 2, oracle.BF16, _abi.POLICY_SIMT, seed=5, mask=mask)


@pytest.mark.parametrize("tokens", [1, 2, 16, 64, 300])
def test_routed_experts_gpt_oss_width(tokens):
    # hidden 2880, intermediate 2880, top-4; 8 experts keep the CPU oracle fast
    from nml_b200 import _abi
    run_routed(tokens, 2880, 8, 2880, 4, oracle.BF16, _abi.POLICY_AUTO, seed=tokens)


@pytest.mark.parametrize("dtype,t", [(oracle.F16, 1e-2), (oracle.BF16, 6e-2)])
@pytest.mark.parametrize("tokens", [2, 1])
def test_contract_experts_closed_form_inputs(dtype, t, tokens):
    # crates/nml/tests/nvfp4_contract.rs:180-312 with its own tolerance (:510-534):
    # |a - e| <= t + t |e| against the f32 reference evaluation
    from nml_b200 import ops
    import gpu_util as gu
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
    bits = lambda v: oracle.from_f32(v, dtype)
    r = lambda v: oracle.to_f32(bits(v), dtype)
    out = ops.routed_clamped_swiglu(
        gu.to_device_bits(bits(hidden), dtype), torch.from_numpy(router).cuda(),
        gu.parameter("gate", gate, H, dtype), gu.to_device_bits(bits(gb), dtype),
        gu.parameter("down", down, I, dtype), gu.to_device_bits(bits(db), dtype), k)
    torch.cuda.synchronize()
    ids, _, w16 = oracle.route(router, k, dtype)
    expected = oracle.routed_clamped_swiglu(r(hidden), ids, oracle.to_f32(w16, dtype), gate,
                                            r(gb), down, r(db))
    assert (np.abs(gu.device_f32(out) - expected) <= t + t * np.abs(expected)).all()


@pytest.mark.parametrize("tokens,E,k,H,I,dtype", [
    (1, 8, 4, 512, 384, oracle.BF16),      # sparse schedule form (A <= E), 16-slot tiles
    (3, 8, 4, 512, 384, oracle.F16),
    (40, 8, 4, 512, 384, oracle.BF16),     # ~20 slots per expert: 32-slot tiles
    (100, 8, 4, 512, 384, oracle.BF16),    # ~50: 64-slot tiles
    (250, 8, 4, 512, 384, oracle.F16),     # ~125: 128-slot tiles
    (700, 8, 4, 512, 384, oracle.BF16),    # ~350: 256-slot tiles, several slot tiles per expert
    (96, 32, 4, 2880, 2880, oracle.BF16),  # GPT-OSS widths, 128-row tail tile on the down side
])
@pytest.mark.parametrize("weights_in_smem", [False, True])
def test_routed_experts_tensor_core_kernel(tokens, E, k, H, I, dtype, weights_in_smem):
    # both homes of the decoded weight tiles: tensor memory (default) and the shared-memory ring
    from nml_b200 import _abi
    mask = None
    if tokens >= 40:
        mask = np.ones(tokens, np.uint8)
        mask[rng(tokens).integers(0, tokens, tokens // 9)] = 0
    policy = _abi.POLICY_UMMA_SMEM if weights_in_smem else _abi.POLICY_UMMA
    run_routed(tokens, H, E, I, k, dtype, policy, seed=tokens + E, mask=mask)


def test_tensor_core_experts_match_portable_kernel_with_expert_offset():
    # Expert-parallel form of the kernel ABI: global expert ids in block_experts, a device
    # scalar expert_offset, weights of the local experts only; other blocks are skipped.
    from nml_b200 import ops, _abi
    import gpu_util as gu
    dtype = oracle.BF16
    E, local, offset, H, I, k, tokens = 8, 4, 4, 256, 128, 2, 64
    gate, down, (gb_bits, gb), (db_bits, db) = make_experts(77, E, H, I, dtype)
    x_bits, x = make_activation(78, (tokens, H), 1.0, dtype)
    logits = (rng(79).standard_normal((tokens, E)) * 0.6).astype(np.float32)
    ids, _, w16 = oracle.route(logits, k, dtype)
    sl = slice(offset, offset + local)
    gate_l = gu.parameter("gate", (gate[0][sl], gate[1][sl], gate[2]), H, dtype)
    down_l = gu.parameter("down", (down[0][sl], down[1][sl], down[2]), I, dtype)
    d_x = gu.to_device_bits(x_bits, dtype)
    d_gb = gu.to_device_bits(gb_bits[sl], dtype)
    d_db = gu.to_device_bits(db_bits[sl], dtype)
    d_ids = torch.from_numpy(ids).cuda()
    d_w = gu.to_device_bits(w16, dtype)
    d_offset = torch.tensor(offset, dtype=torch.int32).cuda()
    plan = ops.moe_assignment_plan(d_ids.reshape(-1), E)  # global plan, as the reference builds
    results = {}
    for policy in (_abi.POLICY_SIMT, _abi.POLICY_UMMA):
        previous = _abi.set_kernel_policy(policy)
        try:
            act = ops.expert_gate_up(d_x, plan, gate_l, d_gb, k, expert_offset=d_offset)
            out = ops.expert_down(act, plan, down_l, d_db, d_w.reshape(-1), k,
                                  expert_offset=d_offset, use_active_blocks=False)
            torch.cuda.synchronize()
        finally:
            _abi.set_kernel_policy(previous)
        results[policy] = (gu.device_f32(act), gu.device_f32(out))
    assert _abi.device_status(0x1) == 0
    is_local = (ids.ravel() >= offset) & (ids.ravel() < offset + local)
    e_act = oracle.expert_gate_up(x, ids.ravel(), k, gate, gb)
    for policy, (act, out) in results.items():
        gu.assert_gemm_close(act[is_local], e_act[is_local], f"gate_up policy {policy}")
        assert (act[~is_local] == 0).all() and (out[~is_local] == 0).all()
        e_out = oracle.expert_down(act, ids.ravel(), oracle.to_f32(w16, dtype).ravel(), down, db)
        gu.assert_gemm_close(out[is_local], e_out[is_local], f"down policy {policy}")


def test_routed_layer_at_the_benchmark_size_against_sampled_oracle():
    # T = 4096, 32 experts, top-4, hidden = intermediate = 2880: the large-batch path (rows
    # permuted into schedule-slot order, 256- and 128-slot tiles, un-permute in the down
    # epilogue).  The schedule is compared in full, bit for bit; each projection on a seeded
    # sample of tokens against the oracle evaluated on the same inputs; the k-way sum bit for
    # bit from the device's own weighted rows.
    import ctypes
    from nml_b200 import ops, _abi
    import gpu_util as gu
    dtype = oracle.BF16
    T, E, k, H, I = 4096, 32, 4, 2880, 2880
    gate, down, (gb_bits, gb), (db_bits, db) = make_experts(4000, E, H, I, dtype)
    x_bits, x = make_activation(4009, (T, H), 1.0, dtype)
    router = make_activation(4010, (E, H), 0.02, dtype)[1]
    logits = (x @ router.T).astype(np.float32)
    active = np.ones(T, np.uint8)
    active[rng(4011).integers(0, T, 37)] = 0
    ids, _, w16 = oracle.route(logits, k, dtype, active=active)
    w = oracle.to_f32(w16, dtype)
    lib = _abi.load()
    layout = _abi.RoutedWorkspaceLayout()
    assert lib.nml_nvfp4_sm100_routed_swiglu_workspace_layout(T, H, I, E, k,
                                                              ctypes.byref(layout)) == 0
    assert layout.slot_ordered == 1
    size = lib.nml_nvfp4_sm100_routed_swiglu_workspace_bytes(T, H, I, E, k)
    workspace = torch.zeros(size, dtype=torch.uint8, device="cuda")
    d_ids, d_w = torch.from_numpy(ids).cuda(), gu.to_device_bits(w16, dtype)
    out = ops.routed_experts(gu.to_device_bits(x_bits, dtype), d_ids, d_w,
                             gu.parameter("gate_up", gate, H, dtype),
                             gu.to_device_bits(gb_bits, dtype), gu.parameter("down", down, I, dtype),
                             gu.to_device_bits(db_bits, dtype), workspace=workspace)
    # the operator API routes on the device: same ids, same weights, same result
    routed = ops.routed_clamped_swiglu_masked(
        gu.to_device_bits(x_bits, dtype), torch.from_numpy(logits).cuda(),
        gu.parameter("gate_up", gate, H, dtype), gu.to_device_bits(gb_bits, dtype),
        gu.parameter("down", down, I, dtype), gu.to_device_bits(db_bits, dtype), k,
        torch.from_numpy(active).bool().cuda())
    torch.cuda.synchronize()
    assert _abi.device_status(0x1) == 0
    assert torch.equal(out.view(torch.int16), routed.view(torch.int16))

    def region(offset, count, torch_dtype):
        width = torch.empty((), dtype=torch_dtype).element_size()
        return workspace[offset:offset + count * width].view(torch_dtype)

    positions, blocks = int(layout.schedule_positions), int(layout.schedule_blocks)
    sorted_dev = region(layout.sorted_assignments, positions, torch.int32).cpu().numpy()
    blocks_dev = region(layout.block_experts, blocks, torch.int32).cpu().numpy()
    e_sorted, e_blocks, e_active = oracle.assignment_plan(ids.ravel(), E, 16)
    assert int(region(layout.active_blocks, 1, torch.int32).item()) == e_active
    assert np.array_equal(sorted_dev, e_sorted) and np.array_equal(blocks_dev, e_blocks)

    sample = np.sort(rng(4012).choice(T, 64, replace=False))
    sample_ids = ids[sample]
    assignments = (sample[:, None] * k + np.arange(k)[None, :]).ravel()
    valid = sample_ids.ravel() >= 0
    slot_of = np.full(T * k, -1, np.int64)
    live = sorted_dev < T * k
    slot_of[sorted_dev[live]] = np.nonzero(live)[0]
    slots = torch.from_numpy(slot_of[assignments[valid]]).cuda()
    # stage 1: gate/up + SwiGLU, device rows in slot order
    slot_activated = region(layout.slot_activated, positions * I, torch.bfloat16).view(positions, I)
    act_dev = slot_activated[slots].float().cpu().numpy()
    e_act = oracle.expert_gate_up(x[sample], sample_ids.ravel(), k, gate, gb)
    gu.assert_gemm_close(act_dev, e_act[valid], "gate_up at T=4096")
    # stage 2: down x routing weight from the device's own narrowed activations
    weighted = region(layout.weighted, T * k * H, torch.bfloat16).view(T * k, H)
    weighted_dev = weighted[torch.from_numpy(assignments).cuda()]
    act_in = np.zeros((assignments.size, I), np.float32)
    act_in[valid] = act_dev
    e_weighted = oracle.expert_down(act_in, sample_ids.ravel(), w[sample].ravel(), down, db)
    gu.assert_gemm_close(weighted_dev.float().cpu().numpy()[valid], e_weighted[valid],
                         "down at T=4096")
    # stage 3: k-way sum, bit for bit
    w_bits = gu.from_device_bits(weighted_dev).copy()
    w_bits[~valid] = 0
    assert np.array_equal(gu.from_device_bits(out[torch.from_numpy(sample).cuda()]),
                          oracle.combine(w_bits, sample.size, k, dtype, mode=0))
    assert (gu.device_f32(out)[active == 0] == 0).all()
