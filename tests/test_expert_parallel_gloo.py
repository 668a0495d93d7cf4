"""The distributed logic of the expert-parallel layer and of the column-sharded unembedding,
run as two CPU ranks over gloo.  Device calls are replaced by the oracle-backed stand-in of
ep_common.OracleBackend (the product has no CPU path); what is under test is the exchange:
count all-to-all, split sizes, row and metadata all-to-all-v, the return trip, the indexed
combine, the all-gather/all-reduce schedule and the column all-gather."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, schedule, results):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ep_common import OracleBackend, build_problem, tensor_to_bits
        from nml_b200 import expert_parallel as ep
        tokens_total, experts, hidden, inter, k = 12, 4, 32, 16, 2
        gate, gb, down, db, x, logits, active = build_problem(tokens_total, experts, hidden,
                                                              inter, seed=40)
        backend = OracleBackend()
        layer = ep.LocalExperts.shard(gate, gb, down, db, rank, world)
        moe = ep.ExpertParallelMoE(layer, k, schedule=schedule, backend=backend)
        lo, hi = ep.shard_range(tokens_total, rank, world)
        out = moe(x[lo:hi].contiguous(), logits[lo:hi].contiguous(), active[lo:hi].contiguous())
        # single-device evaluation of the same tokens with all experts local
        full = ep.LocalExperts(gate, gb, down, db, experts, 0)
        ids, weights = backend.route(logits[lo:hi], k, torch.bfloat16, active[lo:hi])
        expected = backend.routed_experts(x[lo:hi], ids, weights, full)
        results[(schedule, rank)] = (tensor_to_bits(out), tensor_to_bits(expected),
                                     moe.last_counts)
        if schedule == "alltoall":
            # column-sharded unembedding on the same ranks
            from helpers import make_weight
            from ep_common import bits_to_tensor
            from nml_b200 import ops
            payload, scales, g = make_weight(77, (24, hidden))
            table = ops.NvFp4Parameter.nvfp4("table", (24, hidden), torch.bfloat16,
                                             torch.from_numpy(payload), torch.from_numpy(scales),
                                             torch.tensor(float(g)))
            head = ep.ShardedUnembedding(table, backend=backend)
            logits_out = head(x[lo:hi].contiguous())
            reference = backend.linear(x, table)
            results[("unembed", rank)] = (tensor_to_bits(logits_out), tensor_to_bits(reference))
            # the sampler's view: per-shard candidates merged across ranks
            values, indices = head.topk(x[lo:hi].contiguous(), 3)
            picked = head.argmax(x[lo:hi].contiguous())
            results[("topk", rank)] = (values.numpy(), indices.numpy(), picked.numpy(),
                                       reference.float().numpy(), lo, hi)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("schedule", ["alltoall", "allreduce"])
def test_two_cpu_ranks(schedule):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, free_port(), schedule, results), nprocs=world, join=True)
    import oracle
    for rank in range(world):
        out, expected, counts = results[(schedule, rank)]
        if schedule == "alltoall":
            assert np.array_equal(out, expected), f"rank {rank}"
            send, recv = counts
            assert len(send) == world and len(recv) == world
        else:
            a = oracle.to_f32(out, oracle.BF16)
            e = oracle.to_f32(expected, oracle.BF16)
            assert np.abs(a - e).max() <= 2e-2 * max(1.0, np.abs(e).max())
    if schedule == "alltoall":
        total_sent = sum(sum(results[(schedule, r)][2][0]) for r in range(world))
        total_received = sum(sum(results[(schedule, r)][2][1]) for r in range(world))
        assert total_sent == total_received > 0
        for rank in range(world):
            got, reference = results[("unembed", rank)]
            assert np.array_equal(got, reference)
            values, indices, picked, logits, lo, hi = results[("topk", rank)]
            order = np.argsort(-logits, axis=1, kind="stable")[:, :3]  # ties: lower index first
            assert np.array_equal(values, np.take_along_axis(logits, order, axis=1))
            assert np.array_equal(np.take_along_axis(logits, indices, axis=1), values)
            assert np.array_equal(picked, order[lo:hi, 0])


def test_shard_range_follows_the_contiguous_rule():
    from nml_b200.expert_parallel import shard_range
    assert [shard_range(32, r, 8) for r in (0, 3, 7)] == [(0, 4), (12, 16), (28, 32)]
    assert shard_range(201088, 7, 8) == (175952, 201088)
    with pytest.raises(ValueError):
        shard_range(10, 0, 4)
