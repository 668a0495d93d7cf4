"""Shared pieces of the expert-parallel tests: a numpy stand-in for the device calls (used by
the CPU/gloo ranks only, built on the parity oracle) and deterministic problem builders."""
from __future__ import annotations

import numpy as np
import torch

import oracle
from helpers import make_activation, make_weight, rng


def bits_to_tensor(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16)


def tensor_to_bits(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def triple(parameter):
    return (parameter.payload.cpu().numpy(), parameter.block_scales.cpu().numpy(),
            np.float32(parameter.global_scale.item()))


class OracleBackend:
    """CPU stand-in for nml_b200.expert_parallel.CudaBackend (tests only): the same operations
    with the semantics of the device kernels, evaluated by the parity oracle."""

    dtype = oracle.BF16

    def route(self, logits, top_k, dtype, active):
        ids, _, w16 = oracle.route(logits.numpy(), top_k, self.dtype,
                                   None if active is None else active.numpy().astype(np.uint8))
        return torch.from_numpy(ids), bits_to_tensor(w16)

    def dispatch_plan(self, expert_ids, ranks, experts_per_rank):
        ids = expert_ids.numpy()
        assignments = ids.size
        destination = np.where(ids >= 0, ids // experts_per_rank, ranks)
        order = np.argsort(destination, kind="stable")
        valid = int((destination < ranks).sum())
        send_order = np.full(assignments, -1, np.int32)
        send_order[:valid] = order[:valid]
        local = np.full(assignments, -1, np.int32)
        local[:valid] = ids[order[:valid]] - destination[order[:valid]] * experts_per_rank
        slot_of = np.full(assignments, -1, np.int32)
        slot_of[order[:valid]] = np.arange(valid, dtype=np.int32)
        counts = np.bincount(destination[destination < ranks], minlength=ranks).astype(np.int32)
        return (torch.from_numpy(send_order), torch.from_numpy(local), torch.from_numpy(slot_of),
                torch.from_numpy(counts))

    def topk_merge(self, values, indices, k):
        v, i = values.numpy(), indices.numpy()
        parts, rows, _ = v.shape
        out_v = np.full((rows, k), -np.inf, np.float32)
        out_i = np.full((rows, k), -1, np.int32)
        for r in range(rows):
            cv, ci = v[:, r, :k].reshape(-1), i[:, r, :k].reshape(-1)
            keep = ci >= 0
            order = np.lexsort((ci[keep], -cv[keep]))[:k]  # larger value, then lower index
            out_v[r, :order.size] = cv[keep][order]
            out_i[r, :order.size] = ci[keep][order]
        return torch.from_numpy(out_v), torch.from_numpy(out_i)

    def gather_rows(self, source, row_index, divisor):
        index = row_index.numpy()
        bits = tensor_to_bits(source)
        out = np.zeros((index.size, bits.shape[1]), np.uint16)
        ok = index >= 0
        out[ok] = bits[index[ok] // divisor]
        return bits_to_tensor(out)

    def combine_rows(self, rows, row_index, tokens, top_k):
        values = oracle.to_f32(tensor_to_bits(rows), self.dtype)
        index = row_index.numpy().reshape(tokens, top_k)
        out = np.zeros((tokens, rows.shape[1]), np.float32)
        for route in range(top_k):  # route order, f32 accumulation, one narrowing
            ok = index[:, route] >= 0
            out[ok] += values[index[ok, route]]
        return bits_to_tensor(oracle.from_f32(out, self.dtype))

    def routed_experts(self, hidden, expert_ids, routing_weights, layer, expert_offset=0,
                       live_routes=0, leave_masked_rows=False):
        tokens, top_k = expert_ids.shape
        ids = expert_ids.numpy().astype(np.int32) - expert_offset
        ids = np.where((expert_ids.numpy() >= 0) & (ids >= 0) & (ids < layer.experts_local), ids,
                       -1).astype(np.int32)
        x = oracle.to_f32(tensor_to_bits(hidden), self.dtype)
        w = oracle.to_f32(tensor_to_bits(routing_weights), self.dtype)
        gate, down = triple(layer.gate_up), triple(layer.down)
        gate_bias = oracle.to_f32(tensor_to_bits(layer.gate_up_bias), self.dtype)
        down_bias = oracle.to_f32(tensor_to_bits(layer.down_bias), self.dtype)
        narrow = lambda v: oracle.to_f32(oracle.from_f32(v, self.dtype), self.dtype)
        activated = narrow(oracle.expert_gate_up(x, ids.ravel(), top_k, gate, gate_bias))
        weighted = oracle.from_f32(
            oracle.expert_down(activated, ids.ravel(), w.ravel(), down, down_bias), self.dtype)
        weighted[ids.ravel() < 0] = 0
        return bits_to_tensor(oracle.combine(weighted, tokens, top_k, self.dtype, mode=0))

    def topk(self, logits, k, index_offset):
        # descending, equal values to the lower index (a stable sort keeps index order)
        values, order = torch.sort(logits.float(), dim=1, descending=True, stable=True)
        return values[:, :k].contiguous(), (order[:, :k] + index_offset).to(torch.int32).contiguous()

    def layer_f32(self, hidden, expert_ids, routing_weights, layer):
        """The routed layer with the device path's narrowing of the two intermediates, as f32
        BEFORE the final narrowing: the reference point of the GEMM bar for layer outputs."""
        tokens, top_k = expert_ids.shape
        ids = expert_ids.numpy().astype(np.int32)
        x = oracle.to_f32(tensor_to_bits(hidden), self.dtype)
        w = oracle.to_f32(tensor_to_bits(routing_weights), self.dtype)
        gate, down = triple(layer.gate_up), triple(layer.down)
        gate_bias = oracle.to_f32(tensor_to_bits(layer.gate_up_bias), self.dtype)
        down_bias = oracle.to_f32(tensor_to_bits(layer.down_bias), self.dtype)
        narrow = lambda v: oracle.to_f32(oracle.from_f32(v, self.dtype), self.dtype)
        activated = narrow(oracle.expert_gate_up(x, ids.ravel(), top_k, gate, gate_bias))
        weighted = narrow(oracle.expert_down(activated, ids.ravel(), w.ravel(), down, down_bias))
        weighted[ids.ravel() < 0] = 0
        return weighted.reshape(tokens, top_k, -1).sum(axis=1, dtype=np.float32)

    def linear(self, hidden, weight, bias=None):
        out16, _ = oracle.linear_16(tensor_to_bits(hidden), *triple(weight), self.dtype)
        return bits_to_tensor(out16)


def build_problem(tokens_total, experts, hidden, intermediate, seed, device="cpu"):
    """Global (unsharded) parameters and inputs, identical on every rank."""
    from nml_b200 import ops
    dtype = oracle.BF16

    def parameter(name, t, width):
        payload, scales, g = t
        return ops.NvFp4Parameter.nvfp4(
            name, tuple(payload.shape[:-1]) + (width,), torch.bfloat16,
            torch.from_numpy(payload).to(device), torch.from_numpy(scales).to(device),
            torch.tensor(float(g), dtype=torch.float32, device=device))

    gate = parameter("gate_up", make_weight(seed, (experts, 2 * intermediate, hidden)), hidden)
    down = parameter("down", make_weight(seed + 1, (experts, hidden, intermediate)), intermediate)
    gate_bias = bits_to_tensor(make_activation(seed + 2, (experts, 2 * intermediate), 0.02)[0])
    down_bias = bits_to_tensor(make_activation(seed + 3, (experts, hidden), 0.02)[0])
    x = bits_to_tensor(make_activation(seed + 4, (tokens_total, hidden))[0])
    logits = torch.from_numpy(
        (rng(seed + 5).standard_normal((tokens_total, experts)) * 0.7).astype(np.float32))
    active = torch.from_numpy(rng(seed + 6).random(tokens_total) > 0.1)
    return (gate, gate_bias.to(device), down, down_bias.to(device), x.to(device),
            logits.to(device), active.to(device))
