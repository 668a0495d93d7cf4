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
        for schedule in ("alltoall", "allreduce"):
            out = ep.ExpertParallelMoE(layer, k, schedule=schedule)(*mine)
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
        for schedule in ("alltoall", "allreduce", "unembed"):
            out, expected = outcome[schedule]
            a, e = oracle.to_f32(out, oracle.BF16), oracle.to_f32(expected, oracle.BF16)
            assert np.isfinite(a).all(), f"{schedule} rank {rank}"
            assert np.linalg.norm(a - e) <= 1e-2 * np.linalg.norm(e), f"{schedule} rank {rank}"
