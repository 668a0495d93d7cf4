"""Expert-parallel layer and column-sharded unembedding on real devices.

One GPU: the layer with a single rank still walks the whole exchange path (dispatch plan, row
gather, indexed combine kernels) and must equal the plain routed layer bit for bit.  Two or
more GPUs: NCCL ranks, each compared with a single-device evaluation of its own tokens."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_single_rank_exchange_path_equals_routed_layer():
    from ep_common import build_problem, tensor_to_bits
    from nml_b200 import expert_parallel as ep, ops, _abi
    gate, gb, down, db, x, logits, active = build_problem(200, 8, 512, 384, seed=11,
                                                          device="cuda")
    k = 4
    expected = ops.routed_clamped_swiglu_masked(x, logits, gate, gb, down, db, k, active)
    layer = ep.LocalExperts(gate, gb, down, db, 8, 0)
    for schedule in ("alltoall", "allreduce"):
        out = ep.ExpertParallelMoE(layer, k, schedule=schedule)(x, logits, active)
        torch.cuda.synchronize()
        assert np.array_equal(tensor_to_bits(out), tensor_to_bits(expected)), schedule
    # the peer-push exchange with a single rank stores into its own buffers and raises its own
    # flags; the local layer then runs with one route per row, which may select another tile
    # variant (another f32 summation order), so this one is compared to GEMM tolerance
    import oracle
    moe = ep.ExpertParallelMoE(layer, k, schedule="push")
    for _ in range(2):  # the second call reuses the buffers with the next epoch
        out = moe(x, logits, active)
    torch.cuda.synchronize()
    a = oracle.to_f32(tensor_to_bits(out), oracle.BF16)
    e = oracle.to_f32(tensor_to_bits(expected), oracle.BF16)
    assert np.isfinite(a).all()
    assert np.linalg.norm(a - e) <= 1e-2 * np.linalg.norm(e)
    assert ((e == 0).all(axis=1) <= (a == 0).all(axis=1)).all()  # masked tokens stay zero
    head = ep.ShardedUnembedding(ops.NvFp4Parameter("t", (8 * 768, 512), gate.dtype,
                                                    gate.payload.reshape(8 * 768, 256),
                                                    gate.block_scales.reshape(8 * 768, 32),
                                                    gate.global_scale))
    assert np.array_equal(tensor_to_bits(head(x)), tensor_to_bits(ops.linear(x, head.weight)))
    assert _abi.device_status(0x1) == 0


def test_dispatch_plan_gather_and_combine_kernels_against_numpy():
    from ep_common import OracleBackend, bits_to_tensor, tensor_to_bits
    from nml_b200.expert_parallel import CudaBackend
    from helpers import make_activation, rng
    device, reference = CudaBackend(), OracleBackend()
    r = rng(5)
    for assignments, ranks, per_rank in ((64, 8, 4), (4096 * 4, 8, 4), (1000, 2, 16), (7, 4, 1)):
        ids = r.integers(0, ranks * per_rank, assignments).astype(np.int32)
        ids[r.integers(0, assignments, assignments // 5)] = -1
        got = device.dispatch_plan(torch.from_numpy(ids).cuda(), ranks, per_rank)
        want = reference.dispatch_plan(torch.from_numpy(ids), ranks, per_rank)
        for g, w in zip(got, want):
            assert np.array_equal(g.cpu().numpy(), w.numpy())
    k, tokens, width = 4, 50, 64
    source = bits_to_tensor(make_activation(1, (tokens, width))[0])
    index = torch.from_numpy(r.integers(-1, tokens * k, 300).astype(np.int32))
    assert np.array_equal(tensor_to_bits(device.gather_rows(source.cuda(), index.cuda(), k)),
                          tensor_to_bits(reference.gather_rows(source, index, k)))
    rows = bits_to_tensor(make_activation(2, (300, width))[0])
    slot = torch.from_numpy(r.integers(-1, 300, tokens * k).astype(np.int32))
    assert np.array_equal(
        tensor_to_bits(device.combine_rows(rows.cuda(), slot.cuda(), tokens, k)),
        tensor_to_bits(reference.combine_rows(rows, slot, tokens, k)))


@pytest.mark.parametrize("fused_return", [True, False])
@pytest.mark.parametrize("ranks,experts,tokens,skewed", [
    (2, 8, 96, False), (4, 8, 40, False), (8, 32, 64, False), (8, 8, 512, False),
    (8, 32, 64, True), (4, 8, 40, True)])
def test_push_schedule_with_several_ranks_emulated_on_one_device(ranks, experts, tokens, skewed,
                                                                 fused_return):
    # No kernel of the peer-push schedule waits for a flag that an earlier launch has not
    # raised when the stages are replayed stage by stage over all ranks, so G ranks can run on
    # one device with every "peer" buffer local.  This exercises the whole protocol (regions,
    # counts, arrival and return flags, epochs over two consecutive layers) and compares every
    # rank's output with the oracle's evaluation of the layer.  With `fused_return` the down
    # projection stores its rows into the senders' return buffers itself (through the row
    # targets that receive_meta fills) and return_rows only raises the flags.  `skewed`: a
    # router that sends every route of every rank to the first four experts, i.e. to one or two
    # owners, which then receive each sender's whole region (regions hold a sender's full
    # assignment count, so no routing can overflow them).
    from ep_common import OracleBackend, build_problem, tensor_to_bits
    from nml_b200 import _abi, expert_parallel as ep
    import gpu_util as gu
    import oracle
    k, hidden, inter = 4, 512, 384
    per_rank = tokens
    gate, gb, down, db, x, logits, active = build_problem(per_rank * ranks, experts, hidden,
                                                          inter, seed=31 + ranks, device="cuda")
    if skewed:
        logits = logits.clone()
        logits[:, :k] += 50.0
    backend = ep.CudaBackend()
    exchanges = ep.PeerExchange.emulated(ranks, per_rank * k, hidden, torch.bfloat16, "cuda")
    layers = [ep.LocalExperts.shard(gate, gb, down, db, r, ranks) for r in range(ranks)]
    shard = lambda t, r: t[r * per_rank:(r + 1) * per_rank].contiguous()
    for repeat in range(2):  # two layers in a row on the same buffers
        plans, outputs = [], []
        for r in range(ranks):
            ids, weights = backend.route(shard(logits, r), k, torch.bfloat16, shard(active, r))
            order, local_expert, slot_of, counts = backend.dispatch_plan(
                ids.reshape(-1), ranks, experts // ranks)
            backend.push_rows(shard(x, r), order, local_expert, weights.reshape(-1), counts,
                              exchanges[r], k)
            plans.append((ids, weights, slot_of))
        computed = []
        for r in range(ranks):
            if fused_return:
                recv_ids, recv_weights, received, targets = backend.receive_meta(
                    exchanges[r], torch.bfloat16, with_targets=True)
                assert int((targets != 0).sum().item()) == int(received.item())
                backend.routed_experts(exchanges[r].rows, recv_ids, recv_weights, layers[r],
                                       live_routes=per_rank * k, leave_masked_rows=True,
                                       row_targets=targets)
                computed.append(None)
            else:
                recv_ids, recv_weights, received = backend.receive_meta(exchanges[r],
                                                                        torch.bfloat16)
                computed.append(backend.routed_experts(exchanges[r].rows, recv_ids, recv_weights,
                                                       layers[r], live_routes=per_rank * k,
                                                       leave_masked_rows=True))
            assert int(received.item()) == int((recv_ids >= 0).sum().item())
        for r in range(ranks):
            backend.return_rows(computed[r], exchanges[r])
        for r in range(ranks):
            if fused_return:  # the wait folded into the combine launch
                outputs.append(backend.combine_returns(exchanges[r], plans[r][2], per_rank, k))
            else:
                backend.wait_returns(exchanges[r])
                outputs.append(backend.combine_rows(exchanges[r].back, plans[r][2], per_rank, k))
        torch.cuda.synchronize()
        assert _abi.device_status(0x1) == 0
        total = sum(int((p[0] >= 0).sum().item()) for p in plans)
        assert total == sum(int((exchanges[r].sync[:ranks]).sum().item()) for r in range(ranks))
    reference = OracleBackend()
    full = ep.LocalExperts(gate.__class__(gate.name, gate.shape, gate.dtype, gate.payload.cpu(),
                                          gate.block_scales.cpu(), gate.global_scale.cpu()),
                           gb.cpu(),
                           down.__class__(down.name, down.shape, down.dtype, down.payload.cpu(),
                                          down.block_scales.cpu(), down.global_scale.cpu()),
                           db.cpu(), experts, 0)
    for r in range(ranks):
        ids, weights, _ = plans[r]
        expected = reference.layer_f32(shard(x, r).cpu(), ids.cpu(), weights.cpu(), full)
        gu.assert_layer_close(gu.device_f32(outputs[r]), expected, f"rank {r} of {ranks}")
        masked = ~shard(active, r).cpu().numpy()
        assert (gu.device_f32(outputs[r])[masked] == 0).all()


def test_push_schedule_wait_runs_out_and_reports_instead_of_hanging():
    # A sender that never pushes: the owner's wait gives up after `wait_limit` polls, sets the
    # timeout bits of the status word, treats the sender as having sent nothing and returns.
    from nml_b200 import _abi, expert_parallel as ep
    backend = ep.CudaBackend()
    exchanges = ep.PeerExchange.emulated(2, 64, 64, torch.bfloat16, "cuda")
    exchanges[0].state[0] = 1  # rank 0 believes exchange 1 is under way; nobody has pushed
    ids, weights, received = backend.receive_meta(exchanges[0], torch.bfloat16, wait_limit=2000)
    backend.wait_returns(exchanges[0], wait_limit=2000)
    torch.cuda.synchronize()
    status = _abi.device_status(0x1)
    assert status & _abi.STATUS_PEER_TIMEOUT and status & _abi.STATUS_BARRIER_TIMEOUT
    assert int(received.item()) == 0 and (ids == -1).all()
    assert _abi.device_status(0x1) == 0  # reading cleared it; the context is still usable
    assert torch.ones(4, device="cuda").sum().item() == 4


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def nccl_worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        from ep_common import build_problem, tensor_to_bits
        from nml_b200 import expert_parallel as ep, ops
        tokens_total, experts, hidden, inter, k = 64 * world, 8, 512, 384, 4
        gate, gb, down, db, x, logits, active = build_problem(tokens_total, experts, hidden,
                                                              inter, seed=23, device="cuda")
        lo, hi = ep.shard_range(tokens_total, rank, world)
        mine = (x[lo:hi].contiguous(), logits[lo:hi].contiguous(), active[lo:hi].contiguous())
        from ep_common import OracleBackend
        reference = OracleBackend()
        cpu = lambda p: p.__class__(p.name, p.shape, p.dtype, p.payload.cpu(),
                                    p.block_scales.cpu(), p.global_scale.cpu())
        full = ep.LocalExperts(cpu(gate), gb.cpu(), cpu(down), db.cpu(), experts, 0)
        r_ids, r_weights = reference.route(mine[1].cpu(), k, torch.bfloat16, mine[2].cpu())
        expected = reference.layer_f32(mine[0].cpu(), r_ids, r_weights, full)
        layer = ep.LocalExperts.shard(gate, gb, down, db, rank, world)
        outcome = {}
        for schedule in ("alltoall", "allreduce", "push"):
            moe = ep.ExpertParallelMoE(layer, k, schedule=schedule)
            out = moe(*mine)
            if schedule == "push":
                out = moe(*mine)  # a second call reuses the mapped buffers
            torch.cuda.synchronize()
            outcome[schedule] = (tensor_to_bits(out), expected)
        table = ops.NvFp4Parameter("t", (experts * 2 * inter, hidden), gate.dtype,
                                   gate.payload.reshape(-1, hidden // 2),
                                   gate.block_scales.reshape(-1, hidden // 16), gate.global_scale)
        head = ep.ShardedUnembedding(table)
        logits_out = head(mine[0])
        # the sampler's view: per-shard candidates merged across ranks must be the top-k of
        # the gathered logits (stable order: larger value, then lower vocabulary index)
        merged_values, merged_indices = head.topk(mine[0], 8)
        order = torch.sort(logits_out.float(), dim=1, descending=True, stable=True)
        outcome["topk"] = (bool(torch.equal(merged_values, order.values[:, :8])),
                           bool(torch.equal(merged_indices, order.indices[:, :8])),
                           bool(torch.equal(head.argmax(mine[0]), order.indices[lo:hi, 0])))
        import oracle
        unembed_expected = oracle.linear(  # the sharded head gathers the rows of every rank
            oracle.to_f32(tensor_to_bits(x), oracle.BF16), table.payload.cpu().numpy(),
            table.block_scales.cpu().numpy(), np.float32(table.global_scale.item()), None)
        outcome["unembed"] = (tensor_to_bits(logits_out), unembed_expected)
        results[rank] = outcome
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_nccl_ranks_match_single_device_evaluation():
    import torch.multiprocessing as mp
    import oracle
    world = min(torch.cuda.device_count(), 4)
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(nccl_worker, args=(world, free_port(), results), nprocs=world, join=True)
    # every rank's output against the oracle's evaluation of its own tokens (layers: the
    # layer bar of gpu_util.assert_layer_close; the sharded linear: the GEMM bar)
    import gpu_util as gu
    for rank in range(world):
        outcome = results[rank]
        assert outcome["topk"] == (True, True, True), f"rank {rank}: {outcome['topk']}"
        for schedule in ("alltoall", "allreduce", "push", "unembed"):
            out, expected = outcome[schedule]
            what = f"{schedule} rank {rank} of {world}"
            if schedule == "unembed":
                gu.assert_gemm_close(oracle.to_f32(out, oracle.BF16), expected, what)
            else:
                # the all-reduce schedule (the reference's scheme) narrows every rank's partial
                # sum and reduces in the activation dtype: roundings the token exchange does
                # not have, hence three times the mean bar
                gu.assert_layer_close(oracle.to_f32(out, oracle.BF16), expected, what,
                                      mean_bar=6e-3 if schedule == "allreduce" else 2e-3)
