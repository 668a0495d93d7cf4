"""Expert-parallel routed layer and column-sharded unembedding over one process per GPU.

Placement follows the reference's contiguous rule for sharded axes
(crates/nml-sharding/src/lib.rs:180-213): rank r of G owns experts [r*E/G, (r+1)*E/G) and
output columns [r*N/G, (r+1)*N/G).  The reference executes sharded experts by replicating all
tokens on every device and all-reducing the partial outputs
(crates/nml-ir/src/lib.rs:9596-9728).  Two schedules are provided:

``alltoall``  tokens stay sharded by batch; each routed assignment travels to the rank that
              owns its expert and back (two NCCL all-to-all-v), the owner computes only rows
              routed to it, and the token's home rank sums its k returned rows in route order.
              Every per-assignment row is produced by the same kernels as on one GPU, so the
              result equals the single-GPU result bit for bit.
``push``      the same exchange in this library's own kernels, with no collective and no host
              synchronisation inside the layer: every rank maps the others' buffers (torch
              symmetric memory), the dispatch kernel stores each routed row straight into its
              owner's buffer over NVLink and raises an arrival flag there, the owner's next
              kernel waits (bounded) for the flags of all senders; results come back the same
              way.  Every sender has its own region in every receive buffer, so placement is
              deterministic and cannot overflow whatever the routing.  CUDA only.
``allreduce`` the reference's scheme: hidden states are all-gathered, every rank runs its local
              experts over all tokens and partial outputs are summed with an all-reduce.  No
              host synchronisation; meant for decode-size batches.

The device work (routing, dispatch plan, row gather, expert projections, indexed combine) goes
through the C ABI.  ``backend`` exists so that the distributed logic can be exercised by CPU
ranks over gloo with a stand-in for those device calls; the product backend is
``CudaBackend`` and there is no CPU implementation in this package.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _abi, ops


def shard_range(extent: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous shard [start, stop) of an axis; the extent must divide evenly
    (crates/nml-sharding/src/lib.rs:152-158)."""
    if extent % world != 0:
        raise ValueError(f"axis extent {extent} does not divide evenly over {world} devices")
    length = extent // world
    return rank * length, (rank + 1) * length


class CudaBackend:
    """Device operations of the expert-parallel layer, all through the C ABI."""

    def route(self, logits, top_k, dtype, active):
        return ops.route(logits, top_k, dtype, active)

    def dispatch_plan(self, expert_ids: torch.Tensor, ranks: int, experts_per_rank: int):
        assignments = expert_ids.numel()
        device = expert_ids.device
        send_order = torch.empty(assignments, dtype=torch.int32, device=device)
        local_expert = torch.empty(assignments, dtype=torch.int32, device=device)
        slot_of = torch.empty(assignments, dtype=torch.int32, device=device)
        counts = torch.empty(ranks, dtype=torch.int32, device=device)
        request = _abi.EpDispatchPlan(
            expert_ids=expert_ids.data_ptr(), send_order=send_order.data_ptr(),
            local_expert=local_expert.data_ptr(), slot_of_assignment=slot_of.data_ptr(),
            send_counts=counts.data_ptr(), stream=ops._stream(expert_ids),
            assignments=assignments, ranks=ranks, experts_per_rank=experts_per_rank)
        _abi.call("nml_nvfp4_sm100_ep_dispatch_plan", request)
        return send_order, local_expert, slot_of, counts

    def gather_rows(self, source: torch.Tensor, row_index: torch.Tensor, divisor: int):
        rows, width = row_index.numel(), source.shape[1]
        out = torch.empty((rows, width), dtype=source.dtype, device=source.device)
        if rows == 0:
            return out
        request = _abi.GatherRows(source=source.data_ptr(), row_index=row_index.data_ptr(),
                                  output=out.data_ptr(), stream=ops._stream(source), rows=rows,
                                  source_rows=source.shape[0], width=width,
                                  index_divisor=divisor, dtype=ops._code(source.dtype))
        _abi.call("nml_nvfp4_sm100_gather_rows", request)
        return out

    def combine_rows(self, rows: torch.Tensor, row_index: torch.Tensor, tokens: int, top_k: int):
        out = torch.empty((tokens, rows.shape[1]), dtype=rows.dtype, device=rows.device)
        source = rows if rows.shape[0] > 0 else torch.zeros((1, rows.shape[1]), dtype=rows.dtype,
                                                            device=rows.device)
        request = _abi.CombineRows(rows=source.data_ptr(), row_index=row_index.data_ptr(),
                                   output=out.data_ptr(), stream=ops._stream(rows),
                                   tokens=tokens, experts_per_token=top_k,
                                   hidden_size=rows.shape[1], row_count=rows.shape[0],
                                   dtype=ops._code(rows.dtype))
        _abi.call("nml_nvfp4_sm100_combine_rows", request)
        return out

    def push_rows(self, hidden, order, local_expert, weights, counts, exchange, top_k):
        request = _abi.EpPushRows(
            source=hidden.data_ptr(), send_order=order.data_ptr(),
            local_expert=local_expert.data_ptr(), routing_weights=weights.data_ptr(),
            send_counts=counts.data_ptr(), exchange=exchange.descriptor(),
            stream=ops._stream(hidden), assignments=order.numel(), source_rows=hidden.shape[0],
            experts_per_token=top_k, dtype=ops._code(hidden.dtype))
        _abi.call("nml_nvfp4_sm100_ep_push_rows", request)

    def receive_meta(self, exchange, dtype, wait_limit=0, with_targets=False):
        """Expert ids, routing weights and count of the rows that arrived; with
        ``with_targets`` also the address of every row's place in its sender's return buffer
        (the table the down projection stores through)."""
        rows = exchange.ranks * exchange.region_rows
        device = exchange.rows.device
        ids = torch.empty((rows, 1), dtype=torch.int32, device=device)
        weights = torch.empty((rows, 1), dtype=dtype, device=device)
        received = torch.empty(1, dtype=torch.int32, device=device)
        targets = torch.empty(rows, dtype=torch.int64, device=device) if with_targets else None
        request = _abi.EpReceiveMeta(
            exchange=exchange.descriptor(), expert_ids=ids.data_ptr(),
            routing_weights=weights.data_ptr(), received=received.data_ptr(),
            stream=ops._stream(ids), wait_limit=wait_limit, dtype=ops._code(dtype),
            row_targets=None if targets is None else targets.data_ptr())
        _abi.call("nml_nvfp4_sm100_ep_receive_meta", request)
        if with_targets:
            return ids, weights, received, targets
        return ids, weights, received

    def return_rows(self, computed, exchange):
        """Copies the computed rows to their senders and raises the return flags; with
        ``computed`` None (rows already stored through row targets) only the flags."""
        request = _abi.EpReturnRows(
            computed=None if computed is None else computed.data_ptr(),
            exchange=exchange.descriptor(), stream=ops._stream(exchange.rows),
            dtype=ops._code(exchange.rows.dtype))
        _abi.call("nml_nvfp4_sm100_ep_return_rows", request)

    def wait_returns(self, exchange, wait_limit=0):
        request = _abi.EpWaitReturns(exchange=exchange.descriptor(),
                                     stream=ops._stream(exchange.rows), wait_limit=wait_limit)
        _abi.call("nml_nvfp4_sm100_ep_wait_returns", request)

    def combine_returns(self, exchange, row_index, tokens, top_k, wait_limit=0):
        """Waits for the owners' return flags and sums every token's returned rows, in one
        launch (each block waits for itself)."""
        out = torch.empty((tokens, exchange.width), dtype=exchange.rows.dtype,
                          device=exchange.rows.device)
        request = _abi.EpWaitReturns(
            exchange=exchange.descriptor(), stream=ops._stream(exchange.rows),
            wait_limit=wait_limit, row_index=row_index.data_ptr(), output=out.data_ptr(),
            tokens=tokens, experts_per_token=top_k, dtype=ops._code(out.dtype))
        _abi.call("nml_nvfp4_sm100_ep_wait_returns", request)
        return out

    def routed_experts(self, hidden, expert_ids, routing_weights, layer, expert_offset=0,
                       live_routes=0, leave_masked_rows=False, row_targets=None):
        return ops.routed_experts(hidden, expert_ids, routing_weights, layer.gate_up,
                                  layer.gate_up_bias, layer.down, layer.down_bias,
                                  expert_offset=expert_offset, live_routes=live_routes,
                                  leave_masked_rows=leave_masked_rows, row_targets=row_targets)

    def linear(self, hidden, weight, bias=None):
        return ops.linear(hidden, weight, bias)

    def topk(self, logits, k, index_offset):
        return ops.topk_rows(logits, k, index_offset)

    def topk_merge(self, values, indices, k):
        return ops.topk_merge(values, indices, k)


@dataclass
class LocalExperts:
    """The expert parameters one rank holds (slices on axis 0 of the global tensors)."""

    gate_up: object       # NvFp4Parameter [L, 2I, H]
    gate_up_bias: object  # [L, 2I]
    down: object          # NvFp4Parameter [L, H, I]
    down_bias: object     # [L, H]
    experts_total: int
    expert_offset: int

    @property
    def experts_local(self) -> int:
        return self.gate_up_bias.shape[0]

    @staticmethod
    def shard(gate_up, gate_up_bias, down, down_bias, rank: int, world: int) -> "LocalExperts":
        """Slices global (replicated) expert parameters for ``rank``."""
        experts = gate_up_bias.shape[0]
        start, stop = shard_range(experts, rank, world)
        return LocalExperts(gate_up.slice_rows(start, stop), gate_up_bias[start:stop].contiguous(),
                            down.slice_rows(start, stop), down_bias[start:stop].contiguous(),
                            experts, start)


class PeerExchange:
    """The buffers of the peer-push schedule: one allocation per rank in symmetric memory
    (receive rows and meta with one region per sender, return rows, sync words), mapped into
    every rank's address space, plus this rank's local state words.  Collective over `group`
    at construction; sized once for `region_rows` assignments per rank and reused by every
    call (and every layer) that fits."""

    def __init__(self, region_rows: int, width: int, dtype, device, group=None,
                 emulate: tuple | None = None):
        """``emulate=(rank, ranks)`` builds one of several exchanges that live on ONE device
        (see ``emulated``): no process group is involved and `bases` is filled in later."""
        self.world = dist.get_world_size(group) if dist.is_initialized() and not emulate else 1
        self.ranks = emulate[1] if emulate else self.world
        self.rank = emulate[0] if emulate else (
            dist.get_rank(group) if dist.is_initialized() else 0)
        if self.ranks > _abi.EP_MAX_RANKS:
            raise ValueError(f"at most {_abi.EP_MAX_RANKS} ranks")
        self.region_rows, self.width, self.dtype = region_rows, width, dtype
        element = torch.empty((), dtype=dtype).element_size()
        align = lambda n: -(-n // 256) * 256
        rows = self.ranks * region_rows
        self._rows_bytes = align(rows * width * element)
        self._meta_bytes = align(rows * 16)
        self._back_bytes = align(region_rows * width * element)
        self._sync_bytes = align(_abi.EP_SYNC_WORDS * 4)
        total = self._rows_bytes + self._meta_bytes + self._back_bytes + self._sync_bytes
        if self.world == 1:
            self.block = torch.zeros(total, dtype=torch.uint8, device=device)
            bases = [self.block.data_ptr()]
        else:
            import os
            # plain peer mappings only: this path never uses multicast (multimem) accesses
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symmetric
            self.block = symmetric.empty(total, dtype=torch.uint8, device=device)
            self.block.zero_()
            handle = symmetric.rendezvous(self.block,
                                          group if group is not None else dist.group.WORLD)
            bases = [int(p) for p in handle.buffer_ptrs]
            if bases[self.rank] != self.block.data_ptr():
                raise RuntimeError("symmetric memory handle does not describe the local buffer")
            # every rank has zeroed its flags before any rank may push
            torch.cuda.synchronize(device)
            dist.barrier(group)
        self.bases = bases
        offset = 0
        self.rows = self.block[offset:offset + rows * width * element].view(dtype).view(rows, width)
        offset += self._rows_bytes
        self.meta = self.block[offset:offset + rows * 16].view(torch.int32).view(rows, 4)
        offset += self._meta_bytes
        self.back = self.block[offset:offset + region_rows * width * element].view(dtype).view(
            region_rows, width)
        offset += self._back_bytes
        self.sync = self.block[offset:offset + _abi.EP_SYNC_WORDS * 4].view(torch.int32)
        self.state = torch.zeros(_abi.EP_STATE_WORDS, dtype=torch.int32, device=device)
        self._descriptor = None

    @staticmethod
    def emulated(ranks: int, region_rows: int, width: int, dtype, device) -> list:
        """`ranks` exchanges on one device whose "peers" are each other's buffers.  No kernel
        of the exchange waits for a flag that an earlier launch has not already raised when
        the stages are replayed stage by stage over all ranks, so the whole protocol can be
        exercised on one GPU."""
        group = [PeerExchange(region_rows, width, dtype, device, emulate=(r, ranks))
                 for r in range(ranks)]
        bases = [x.block.data_ptr() for x in group]
        for x in group:
            x.bases = bases
        return group

    def descriptor(self) -> "_abi.EpExchange":
        if self._descriptor is None:
            pad = [None] * (_abi.EP_MAX_RANKS - self.ranks)
            table = lambda offset: (_abi._vp * _abi.EP_MAX_RANKS)(
                *([b + offset for b in self.bases] + pad))
            self._descriptor = _abi.EpExchange(
                peer_rows=table(0), peer_meta=table(self._rows_bytes),
                peer_back=table(self._rows_bytes + self._meta_bytes),
                peer_sync=table(self._rows_bytes + self._meta_bytes + self._back_bytes),
                local_state=self.state.data_ptr(), ranks=self.ranks, rank=self.rank,
                region_rows=self.region_rows, width=self.width)
        return self._descriptor


class ExpertParallelMoE:
    """Routed clamped-SwiGLU layer with experts sharded over the ranks of ``group``.

    ``forward(hidden, router_logits)`` takes this rank's tokens ``[T_local, H]`` and their
    f32 router logits ``[T_local, E]`` (the router is a replicated dense linear) and returns
    this rank's output rows ``[T_local, H]``.
    """

    def __init__(self, layer: LocalExperts, experts_per_token: int, group=None,
                 schedule: str = "alltoall", backend=None, exchange: PeerExchange | None = None,
                 wait_limit: int = 0, fused_return: bool | None = None):
        if schedule not in ("alltoall", "allreduce", "push"):
            raise ValueError("schedule must be 'alltoall', 'push' or 'allreduce'")
        # push schedule: mapped buffers, shared between layers when passed in, else allocated
        # on first use for that call's token count (a later, larger batch reallocates: a
        # collective, done only after every rank has drained its stream)
        self.exchange = exchange
        self.wait_limit = wait_limit
        # push schedule: the down projection stores its rows into the senders' return buffers
        # itself (False: a separate copy kernel after the layer).  None: fused for decode-size
        # batches only -- the projection's epilogue stores 64-byte pieces, which NVLink carries
        # at a fraction of the rate of the copy kernel's whole rows (at 4096 tokens on 2 GPUs
        # the fused layer took 1.04 ms against 0.77 ms; at 64 tokens 150 us against 168 us).
        self.fused_return = fused_return
        self.layer = layer
        self.top_k = experts_per_token
        self.group = group
        self.schedule = schedule
        self.backend = backend or CudaBackend()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if layer.experts_total != layer.experts_local * self.world:
            raise ValueError("expert count must divide evenly over the devices of the group")
        if layer.expert_offset != self.rank * layer.experts_local:
            raise ValueError("local experts must be the contiguous shard of this rank")
        self.last_counts = None  # (rows sent per rank, rows received per rank) of the last call

    # ------------------------------------------------------------------ all-to-all
    def _forward_alltoall(self, hidden, router_logits, active_tokens):
        backend, group, k = self.backend, self.group, self.top_k
        tokens, width = hidden.shape
        ids, weights = backend.route(router_logits, k, hidden.dtype, active_tokens)
        order, local_expert, slot_of, counts = backend.dispatch_plan(
            ids.reshape(-1), self.world, self.layer.experts_local)
        recv_counts = torch.empty_like(counts)
        if self.world > 1:
            dist.all_to_all_single(recv_counts, counts, group=group)
        else:
            recv_counts.copy_(counts)
        # NCCL needs the split sizes on the host: the one synchronisation of this schedule.
        send_c = [int(c) for c in counts.cpu().tolist()]
        recv_c = [int(c) for c in recv_counts.cpu().tolist()]
        self.last_counts = (send_c, recv_c)
        n_send, n_recv = sum(send_c), sum(recv_c)

        send_rows = backend.gather_rows(hidden, order[:n_send], k)  # token permute
        flat_weights = weights.reshape(-1).view(torch.int16)
        send_meta = torch.stack(
            [local_expert[:n_send],
             flat_weights.index_select(0, order[:n_send].long()).to(torch.int32)], dim=1
        ).contiguous()
        recv_rows = torch.empty((n_recv, width), dtype=hidden.dtype, device=hidden.device)
        recv_meta = torch.empty((n_recv, 2), dtype=torch.int32, device=hidden.device)
        if self.world > 1:
            dist.all_to_all_single(recv_rows, send_rows, recv_c, send_c, group=group)
            dist.all_to_all_single(recv_meta, send_meta, recv_c, send_c, group=group)
        else:
            recv_rows, recv_meta = send_rows, send_meta

        if n_recv > 0:
            recv_ids = recv_meta[:, 0].contiguous().reshape(n_recv, 1)
            recv_weights = recv_meta[:, 1].to(torch.int16).view(hidden.dtype).reshape(n_recv, 1)
            computed = backend.routed_experts(recv_rows, recv_ids, recv_weights.contiguous(),
                                              self.layer)
        else:
            computed = recv_rows
        returned = torch.empty((n_send, width), dtype=hidden.dtype, device=hidden.device)
        if self.world > 1:
            dist.all_to_all_single(returned, computed, send_c, recv_c, group=group)
        else:
            returned = computed
        return backend.combine_rows(returned, slot_of, tokens, k)  # unpermute + k-way sum

    # ------------------------------------------------------------------ peer push
    def _exchange_for(self, assignments, width, dtype, device):
        x = self.exchange
        if x is None or x.region_rows < assignments or x.width != width or x.dtype != dtype:
            if x is not None:
                # no rank may still be storing into the old mapping
                torch.cuda.synchronize(device)
                if self.world > 1:
                    dist.barrier(self.group)
            self.exchange = x = PeerExchange(-(-assignments // 16) * 16, width, dtype, device,
                                             self.group)
        return x

    def _forward_push(self, hidden, router_logits, active_tokens):
        backend, k = self.backend, self.top_k
        tokens, width = hidden.shape
        assignments = tokens * k
        exchange = self._exchange_for(assignments, width, hidden.dtype, hidden.device)
        ids, weights = backend.route(router_logits, k, hidden.dtype, active_tokens)
        order, local_expert, slot_of, counts = backend.dispatch_plan(
            ids.reshape(-1), self.world, self.layer.experts_local)
        backend.push_rows(hidden, order, local_expert, weights.reshape(-1), counts, exchange, k)
        # of the world * region_rows rows an owner's buffer holds, about `assignments` are live
        fused = self.fused_return if self.fused_return is not None else assignments <= 1024
        if fused:
            # the down projection's epilogue stores every result row straight into its
            # sender's return buffer; what is left of the return trip is raising the flags
            recv_ids, recv_weights, _, targets = backend.receive_meta(
                exchange, hidden.dtype, self.wait_limit, with_targets=True)
            backend.routed_experts(exchange.rows, recv_ids, recv_weights, self.layer,
                                   live_routes=assignments, leave_masked_rows=True,
                                   row_targets=targets)
            backend.return_rows(None, exchange)
        else:
            recv_ids, recv_weights, _ = backend.receive_meta(exchange, hidden.dtype,
                                                             self.wait_limit)
            computed = backend.routed_experts(exchange.rows, recv_ids, recv_weights, self.layer,
                                              live_routes=assignments, leave_masked_rows=True)
            backend.return_rows(computed, exchange)
        return backend.combine_returns(exchange, slot_of, tokens, k, self.wait_limit)

    # ------------------------------------------------------------------ all-reduce
    def _forward_allreduce(self, hidden, router_logits, active_tokens):
        backend, group, k = self.backend, self.group, self.top_k
        tokens, width = hidden.shape
        ids, weights = backend.route(router_logits, k, hidden.dtype, active_tokens)
        if self.world > 1:
            all_hidden = torch.empty((self.world * tokens, width), dtype=hidden.dtype,
                                     device=hidden.device)
            all_ids = torch.empty((self.world * tokens, k), dtype=ids.dtype, device=ids.device)
            all_weights = torch.empty((self.world * tokens, k), dtype=weights.dtype,
                                      device=weights.device)
            dist.all_gather_into_tensor(all_hidden, hidden.contiguous(), group=group)
            dist.all_gather_into_tensor(all_ids, ids, group=group)
            dist.all_gather_into_tensor(all_weights, weights, group=group)
        else:
            all_hidden, all_ids, all_weights = hidden, ids, weights
        partial = backend.routed_experts(all_hidden, all_ids, all_weights, self.layer,
                                         expert_offset=self.layer.expert_offset)
        if self.world > 1:
            dist.all_reduce(partial, group=group)
            return partial[self.rank * tokens:(self.rank + 1) * tokens].contiguous()
        return partial

    def forward(self, hidden: torch.Tensor, router_logits: torch.Tensor,
                active_tokens: torch.Tensor | None = None) -> torch.Tensor:
        if hidden.dim() != 2 or router_logits.dim() != 2 or \
                router_logits.shape[0] != hidden.shape[0] or \
                router_logits.shape[1] != self.layer.experts_total:
            raise ValueError("routing tensors do not match the token and hidden extents")
        if self.schedule == "alltoall":
            return self._forward_alltoall(hidden, router_logits, active_tokens)
        if self.schedule == "push":
            return self._forward_push(hidden, router_logits, active_tokens)
        return self._forward_allreduce(hidden, router_logits, active_tokens)

    __call__ = forward


class ShardedUnembedding:
    """The vocabulary projection with output columns sharded over the ranks of ``group``.

    Rank r holds rows [r*N/G, (r+1)*N/G) of the packed table (payload and block scales sliced
    on axis 0, global scale replicated).  Every logit is produced by the same kernels as on
    one GPU.  What leaves a rank is chosen by the caller:

    ``forward``  all logits on every rank (an all-gather of the logit columns: rows x N values
                 land on every rank, which is what bounds it);
    ``topk`` / ``argmax``  each rank reduces its own columns to k candidates per row and only
                 those k * G (value, index) pairs are exchanged and merged, which is all a
                 sampler needs (the reference plans the same for its column-sharded head,
                 PRODUCT.md:673-674).  Ties go to the lower vocabulary index.
    """

    def __init__(self, weight, group=None, backend=None, already_sharded: bool = False):
        self.group = group
        self.backend = backend or CudaBackend()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if already_sharded:
            self.weight = weight
            self.columns_total = weight.shape[0] * self.world
        else:
            start, stop = shard_range(weight.shape[0], self.rank, self.world)
            self.weight = weight.slice_rows(start, stop)
            self.columns_total = weight.shape[0]
        self.column_offset = self.rank * (self.columns_total // self.world)

    def _all_rows(self, hidden: torch.Tensor, gather_rows: bool) -> torch.Tensor:
        if self.world > 1 and gather_rows:
            all_hidden = torch.empty((self.world * hidden.shape[0], hidden.shape[1]),
                                     dtype=hidden.dtype, device=hidden.device)
            dist.all_gather_into_tensor(all_hidden, hidden.contiguous(), group=self.group)
            return all_hidden
        return hidden

    def forward(self, hidden: torch.Tensor, gather_rows: bool = True,
                gather_columns: bool = True) -> torch.Tensor:
        local = self.backend.linear(self._all_rows(hidden, gather_rows), self.weight)
        if self.world == 1 or not gather_columns:
            return local
        gathered = torch.empty((self.world * local.shape[0], local.shape[1]), dtype=local.dtype,
                               device=local.device)
        dist.all_gather_into_tensor(gathered, local.contiguous(), group=self.group)
        return gathered.view(self.world, local.shape[0], local.shape[1]).permute(
            1, 0, 2).reshape(local.shape[0], self.columns_total)

    __call__ = forward

    def topk(self, hidden: torch.Tensor, k: int, gather_rows: bool = True):
        """(values f32 [rows, k], vocabulary indices i64 [rows, k]) of the k largest logits of
        every row, rows of all ranks when ``gather_rows`` (else of ``hidden`` as given, which
        must then be the same on every rank)."""
        local = self.backend.linear(self._all_rows(hidden, gather_rows), self.weight)
        values, indices = self.backend.topk(local, k, self.column_offset)
        if self.world == 1:
            return values, indices.long()
        rows = local.shape[0]
        # one collective: every rank's [rows, 2 k] block of value bits and indices; the merge
        # keeps the order of the per-shard selection (larger value, then lower index), so the
        # result is the top-k of the unsharded row whatever the ties
        packed = torch.cat((values.contiguous().view(torch.int32), indices), dim=1)
        gathered = torch.empty((self.world, rows, 2 * k), dtype=torch.int32,
                               device=local.device)
        dist.all_gather_into_tensor(gathered.view(self.world * rows, 2 * k), packed,
                                    group=self.group)
        best, position = self.backend.topk_merge(gathered.view(torch.float32)[:, :, :k],
                                                 gathered[:, :, k:], k)
        return best, position.long()

    def argmax(self, hidden: torch.Tensor, gather_rows: bool = True) -> torch.Tensor:
        """Greedy pick for this rank's rows of ``hidden`` (i64 [rows])."""
        rows = hidden.shape[0]
        _, indices = self.topk(hidden, 1, gather_rows)
        if self.world > 1 and gather_rows:
            return indices[self.rank * rows:(self.rank + 1) * rows, 0]
        return indices[:, 0]
