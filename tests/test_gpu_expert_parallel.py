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
    # the peer-push exchange with a single rank stores into its own buffers; the local layer
    # then runs over `capacity` rows with the tail masked, which may select another tile
    # variant (another f32 summation order), so this one is compared to GEMM tolerance
    import oracle
    for factor in (1.0, 2.0):
        out = ep.ExpertParallelMoE(layer, k, schedule="push", capacity_factor=factor)(
            x, logits, active)
        torch.cuda.synchronize()
        a = oracle.to_f32(tensor_to_bits(out), oracle.BF16)
        e = oracle.to_f32(tensor_to_bits(expected), oracle.BF16)
        assert np.isfinite(a).all()
        assert np.linalg.norm(a - e) <= 1e-2 * np.linalg.norm(e), factor
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


def test_push_exchange_layout_with_several_ranks_emulated_on_one_device():
    # The push, receive-meta and return kernels never wait for another rank, so the exchange
    # of G ranks can be replayed rank after rank on one device with every "peer" buffer local:
    # this pins the placement rule (rank r's rows for rank d follow those of ranks < r, in r's
    # send order) and the way home without any peer mapping.
    from ep_common import bits_to_tensor, tensor_to_bits
    from nml_b200 import _abi
    from nml_b200.expert_parallel import CudaBackend, PeerBuffers
    from helpers import make_activation, rng
    backend = CudaBackend()
    r = rng(77)
    for ranks, per_rank, tokens, k, width in ((2, 4, 64, 4, 64), (4, 2, 37, 2, 128),
                                              (8, 4, 512, 4, 64)):
        assignments = tokens * k
        capacity = ranks * assignments
        hidden, plans, weights = [], [], []
        for rank in range(ranks):
            hidden.append(bits_to_tensor(make_activation(100 + rank, (tokens, width))[0]).cuda())
            ids = r.integers(0, ranks * per_rank, assignments).astype(np.int32)
            ids[r.integers(0, assignments, assignments // 7)] = -1
            plans.append(backend.dispatch_plan(torch.from_numpy(ids).cuda(), ranks, per_rank))
            weights.append(bits_to_tensor(make_activation(200 + rank, (assignments,))[0]).cuda())
        count_matrix = torch.stack([p[3] for p in plans]).contiguous()
        peers = []
        for rank in range(ranks):
            rows = torch.full((capacity, width), float("nan"), dtype=torch.bfloat16,
                              device="cuda")
            meta = torch.full((capacity, 4), -7, dtype=torch.int32, device="cuda")
            back = torch.full((assignments, width), float("nan"), dtype=torch.bfloat16,
                              device="cuda")
            peers.append(PeerBuffers(rows.data_ptr(), meta.data_ptr(), back.data_ptr(), rows,
                                     meta, back))
        for rank in range(ranks):
            order, local_expert, _, counts = plans[rank]
            backend.push_rows(hidden[rank], order, local_expert, weights[rank], counts,
                              count_matrix, peers, rank, k, capacity)
        torch.cuda.synchronize()
        matrix = count_matrix.cpu().numpy()
        for destination in range(ranks):
            position = 0
            for rank in range(ranks):
                order = plans[rank][0].cpu().numpy()
                local_expert = plans[rank][1].cpu().numpy()
                first = int(matrix[rank, :destination].sum())
                for i in range(int(matrix[rank, destination])):
                    slot = first + i
                    got = peers[destination].rows[position]
                    want = hidden[rank][order[slot] // k]
                    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
                    meta = peers[destination].meta[position].cpu().numpy()
                    assert meta[0] == local_expert[slot] and meta[2] == rank and meta[3] == slot
                    assert meta[1] == int(weights[rank].view(torch.int16)[order[slot]]) & 0xffff
                    position += 1
            ids, w, received = backend.receive_meta(peers[destination].meta, count_matrix,
                                                    torch.bfloat16, ranks, destination, capacity)
            assert int(received.item()) == position == int(matrix[:, destination].sum())
            assert (ids[position:] == -1).all() and (ids[:position] >= 0).all()
            # identity "computation": the rows go home unchanged
            backend.return_rows(peers[destination].rows, peers[destination].meta, count_matrix,
                                peers, destination, capacity, assignments)
        torch.cuda.synchronize()
        for rank in range(ranks):
            order = plans[rank][0].cpu().numpy()
            sent = int(matrix[rank].sum())
            for slot in range(sent):
                want = hidden[rank][order[slot] // k]
                assert torch.equal(peers[rank].back[slot].view(torch.int16),
                                   want.view(torch.int16))
            assert torch.isnan(peers[rank].back[sent:].float()).all()  # nothing else was written
    assert _abi.device_status(0x1) == 0


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
        expected = ops.routed_clamped_swiglu_masked(mine[0], mine[1], gate, gb, down, db, k,
                                                    mine[2])
        layer = ep.LocalExperts.shard(gate, gb, down, db, rank, world)
        outcome = {}
        for schedule in ("alltoall", "allreduce", "push"):
            moe = ep.ExpertParallelMoE(layer, k, schedule=schedule)
            out = moe(*mine)
            if schedule == "push":
                out = moe(*mine)  # a second call reuses the mapped buffers
            torch.cuda.synchronize()
            outcome[schedule] = (tensor_to_bits(out), tensor_to_bits(expected))
        table = ops.NvFp4Parameter("t", (experts * 2 * inter, hidden), gate.dtype,
                                   gate.payload.reshape(-1, hidden // 2),
                                   gate.block_scales.reshape(-1, hidden // 16), gate.global_scale)
        logits_out = ep.ShardedUnembedding(table)(mine[0])
        outcome["unembed"] = (tensor_to_bits(logits_out), tensor_to_bits(ops.linear(x, table)))
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
    # A shard sees other batch sizes than the single device (rows per expert, output columns),
    # so the tile variant and with it the f32 accumulation order may differ: the results agree
    # to GEMM tolerance, bit for bit only when both sides select the same variant.
    for rank in range(world):
        outcome = results[rank]
        for schedule in ("alltoall", "allreduce", "push", "unembed"):
            out, expected = outcome[schedule]
            a, e = oracle.to_f32(out, oracle.BF16), oracle.to_f32(expected, oracle.BF16)
            assert np.isfinite(a).all(), f"{schedule} rank {rank}"
            assert np.linalg.norm(a - e) <= 1e-2 * np.linalg.norm(e), f"{schedule} rank {rank}"
