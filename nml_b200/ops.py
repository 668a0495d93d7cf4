"""Operator API of the NVFP4 path, mirroring the reference's graph operators.

The names and argument meaning follow the reference's ``nml::Graph`` operators
(crates/nml-ir/src/lib.rs): ``linear`` (:4841), ``linear_qkv`` (:4884),
``token_embedding`` (:2816), ``routed_clamped_swiglu`` / ``routed_clamped_swiglu_masked``
(:1257, :1286) over a logical ``Parameter::nvfp4`` (crates/nml-parameter/src/lib.rs:168).
The shape and dtype checks are those of the reference's operator builders and of its
custom-call handlers (crates/nml-kernel-nvfp4/src/cuda.rs:216-308 and following); a
violation raises ``ValueError`` before anything is launched.

Every operator ends in a call through the C ABI declared in
``include/nml_nvfp4_sm100.h``.  torch supplies device memory and the current stream; no
operator has a PyTorch or CPU implementation behind it.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _abi

_DTYPE_CODE = {torch.float16: _abi.F16, torch.bfloat16: _abi.BF16}


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError("NVFP4 operations support F16 and BF16 only") from None


def _stream(tensor: torch.Tensor) -> int:
    # The C ABI rejects a null stream like the reference adapter does.  torch's default
    # stream has handle 0; its explicit, non-null spelling is cudaStreamLegacy (0x1).
    handle = torch.cuda.current_stream(tensor.device).cuda_stream
    return handle if handle != 0 else 0x1


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def _require_cuda(*tensors: torch.Tensor | None) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise RuntimeError("NVFP4 operators run on a CUDA device only (no CPU fallback)")
        if tensor is not None and not tensor.is_contiguous():
            raise ValueError("NVFP4 operators require row-major contiguous tensors")


@dataclass
class NvFp4Parameter:
    """One logical NVFP4 weight: the three physical components of recipe v2.

    ``shape`` is the logical shape ``[..., K]``; ``payload`` is u8 ``[..., ceil(K/2)]``,
    ``block_scales`` u8 ``[..., ceil(K/16)]`` and ``global_scale`` an f32 scalar tensor
    (crates/nml-parameter/src/lib.rs:163-206).
    """

    name: str
    shape: tuple
    dtype: torch.dtype
    payload: torch.Tensor
    block_scales: torch.Tensor
    global_scale: torch.Tensor

    @staticmethod
    def nvfp4(name: str, shape, dtype: torch.dtype, payload: torch.Tensor,
              block_scales: torch.Tensor, global_scale: torch.Tensor) -> "NvFp4Parameter":
        shape = tuple(int(d) for d in shape)
        if not shape or shape[-1] <= 0 or any(d <= 0 for d in shape):
            raise ValueError("invalid NVFP4 logical weight shape")
        _code(dtype)
        width = shape[-1]
        if payload.dtype != torch.uint8 or block_scales.dtype != torch.uint8:
            raise ValueError("NVFP4 payloads and block scales must use U8 buffers")
        if tuple(payload.shape) != shape[:-1] + ((width + 1) // 2,):
            raise ValueError(
                f"NVFP4 payload extent mismatch: expected {shape[:-1] + ((width + 1) // 2,)}, "
                f"received {tuple(payload.shape)}")
        if tuple(block_scales.shape) != shape[:-1] + ((width + 15) // 16,):
            raise ValueError(
                f"NVFP4 block-scale extent mismatch: expected "
                f"{shape[:-1] + ((width + 15) // 16,)}, received {tuple(block_scales.shape)}")
        if global_scale.dtype != torch.float32 or global_scale.numel() != 1:
            raise ValueError("NVFP4 global scales must be F32 scalars")
        return NvFp4Parameter(name, shape, dtype, payload.contiguous(),
                              block_scales.contiguous(), global_scale.reshape(()).contiguous())

    def slice_rows(self, start: int, stop: int, name: str | None = None) -> "NvFp4Parameter":
        """Rows [start, stop) of axis 0 (expert or output-column shards); the global scale is
        shared, block boundaries are untouched (crates/nml-parameter/src/lib.rs:285-312)."""
        return NvFp4Parameter(name or f"{self.name}[{start}:{stop}]",
                              (stop - start,) + self.shape[1:], self.dtype,
                              self.payload[start:stop].contiguous(),
                              self.block_scales[start:stop].contiguous(), self.global_scale)


_LINEAR_SCRATCH: dict = {}


def linear(input: torch.Tensor, weight: NvFp4Parameter, bias: torch.Tensor | None = None,
           out: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
    """``[..., K] x [N, K]^T (+ bias[N])`` with f32 accumulation; result in the input dtype.
    ``residual`` (shape and dtype of the result; may be ``out`` itself) is added to the narrowed
    result in the kernel's epilogue: bit for bit ``linear(...) + residual`` of the reference
    graph's output projection (products/serve/src/gpt_oss/graph.rs:534-543) in one launch.
    Calls the library can run faster with scratch (BF16 rows >= 512 on weights with >= 16384
    outputs) get a buffer cached per device and stream; the library decides on the device
    whether the faster kernel may write the output."""
    if input.dim() == 0:
        raise ValueError("linear input requires at least one dimension")
    if len(weight.shape) != 2:
        raise ValueError("linear requires a rank-2 NVFP4 weight")
    outputs, inputs = weight.shape
    dtype = _code(input.dtype)
    if input.dtype != weight.dtype:
        raise ValueError("NVFP4 linear dtypes are inconsistent")
    if input.shape[-1] != inputs:
        raise ValueError(
            f"linear input extent {input.shape[-1]} does not match rows of {inputs} values")
    if bias is not None and (tuple(bias.shape) != (outputs,) or bias.dtype != input.dtype):
        raise ValueError("NVFP4 linear bias must be a length-N activation vector")
    rows = input.numel() // inputs
    if rows <= 0:
        raise ValueError("NVFP4 linear row extent must be positive")
    _require_cuda(input, weight.payload, weight.block_scales, weight.global_scale, bias)
    result_shape = tuple(input.shape[:-1]) + (outputs,)
    if out is None:
        out = torch.empty(result_shape, dtype=input.dtype, device=input.device)
    elif tuple(out.shape) != result_shape or out.dtype != input.dtype:
        raise ValueError("NVFP4 linear component and output shapes are inconsistent")
    if residual is not None:
        if tuple(residual.shape) != result_shape or residual.dtype != input.dtype or \
                not residual.is_contiguous():
            raise ValueError("NVFP4 linear residual must match the result's shape and dtype")
        _require_cuda(residual)
    # scratch for the F16 copy of the activations that wide weights decode fastest against
    scratch = None
    size = _abi.load().nml_nvfp4_sm100_linear_workspace_bytes(rows, outputs, inputs, dtype)
    if size:
        key = (input.device, torch.cuda.current_stream(input.device).cuda_stream)
        scratch = _LINEAR_SCRATCH.get(key)
        if scratch is None or scratch.numel() < size:
            scratch = torch.empty(size, dtype=torch.uint8, device=input.device)
            _LINEAR_SCRATCH[key] = scratch
    request = _abi.Linear(activation=_ptr(input), payload=_ptr(weight.payload),
                          block_scales=_ptr(weight.block_scales),
                          global_scale=_ptr(weight.global_scale), bias=_ptr(bias),
                          output=_ptr(out), stream=_stream(input), rows=rows, outputs=outputs,
                          inputs=inputs, dtype=dtype, residual=_ptr(residual),
                          workspace=_ptr(scratch),
                          workspace_bytes=0 if scratch is None else scratch.numel())
    _abi.call("nml_nvfp4_sm100_linear", request)
    return out


def linear_qkv(input: torch.Tensor, query_weight: NvFp4Parameter, query_bias,
               key_weight: NvFp4Parameter, key_bias, value_weight: NvFp4Parameter, value_bias):
    """Three projections over one activation (crates/nml-ir/src/lib.rs:4884-4928), one launch
    (``nml_nvfp4_sm100_linear_qkv``).  Projections of different dtype or width cannot share a
    launch and are evaluated one by one, as the reference does (nvfp4_backend.rs:243-268)."""
    weights = (query_weight, key_weight, value_weight)
    biases = (query_bias, key_bias, value_bias)
    if input.dim() == 0:
        raise ValueError("linear input requires at least one dimension")
    same = all(len(w.shape) == 2 and w.shape[1] == query_weight.shape[1] and
               w.dtype == input.dtype for w in weights)
    if not same:
        return tuple(linear(input, w, b) for w, b in zip(weights, biases))
    inputs = query_weight.shape[1]
    if input.shape[-1] != inputs:
        raise ValueError(
            f"linear input extent {input.shape[-1]} does not match rows of {inputs} values")
    for w, b in zip(weights, biases):
        if b is not None and (tuple(b.shape) != (w.shape[0],) or b.dtype != input.dtype):
            raise ValueError("NVFP4 linear bias must be a length-N activation vector")
        _require_cuda(w.payload, w.block_scales, w.global_scale, b)
    _require_cuda(input)
    rows = input.numel() // inputs
    if rows <= 0:
        raise ValueError("NVFP4 linear row extent must be positive")
    outs = tuple(torch.empty(tuple(input.shape[:-1]) + (w.shape[0],), dtype=input.dtype,
                             device=input.device) for w in weights)
    three = _abi._vp * 3
    request = _abi.LinearQkv(
        activation=_ptr(input), payload=three(*[_ptr(w.payload) for w in weights]),
        block_scales=three(*[_ptr(w.block_scales) for w in weights]),
        global_scale=three(*[_ptr(w.global_scale) for w in weights]),
        bias=three(*[_ptr(b) for b in biases]), output=three(*[_ptr(o) for o in outs]),
        stream=_stream(input), rows=rows,
        outputs=(_abi._i64 * 3)(*[w.shape[0] for w in weights]), inputs=inputs,
        dtype=_code(input.dtype))
    _abi.call("nml_nvfp4_sm100_linear_qkv", request)
    return outs


def token_embedding(weight: NvFp4Parameter, indices: torch.Tensor,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """Decodes rows ``indices`` of a ``[vocabulary, width]`` table; result ``indices.shape +
    [width]`` in the table's logical dtype."""
    if len(weight.shape) != 2:
        raise ValueError("embedding requires a rank-2 NVFP4 weight")
    if indices.dtype not in (torch.int32, torch.int64):
        raise ValueError("NVFP4 embedding supports I32 and I64 indices")
    vocabulary, width = weight.shape
    rows = indices.numel()
    if rows <= 0:
        raise ValueError("NVFP4 embedding row extent must be positive")
    _require_cuda(indices, weight.payload, weight.block_scales, weight.global_scale)
    result_shape = tuple(indices.shape) + (width,)
    if out is None:
        out = torch.empty(result_shape, dtype=weight.dtype, device=indices.device)
    elif tuple(out.shape) != result_shape or out.dtype != weight.dtype:
        raise ValueError("NVFP4 embedding output shape is inconsistent")
    request = _abi.Embedding(indices=_ptr(indices), payload=_ptr(weight.payload),
                             block_scales=_ptr(weight.block_scales),
                             global_scale=_ptr(weight.global_scale), output=_ptr(out),
                             stream=_stream(indices), rows=rows, vocabulary=vocabulary,
                             width=width, dtype=_code(weight.dtype),
                             indices_are_i64=1 if indices.dtype == torch.int64 else 0)
    _abi.call("nml_nvfp4_sm100_embedding", request)
    return out


# ------------------------------------------------------------------ routed experts

def route(router_logits: torch.Tensor, experts_per_token: int, dtype: torch.dtype,
          active_tokens: torch.Tensor | None = None):
    """Top-k routing: returns ``(expert_ids i32 [T, k], routing_weights dtype [T, k])``.

    Softmax over all experts in f32, top-k by descending probability with ties to the lower
    expert index, renormalised; masked tokens get expert -1 and weight 0
    (crates/nml-ir/src/lib.rs:1411-1437)."""
    if router_logits.dim() != 2 or router_logits.dtype != torch.float32:
        raise ValueError("router logits must be F32 [tokens, experts]")
    tokens, experts = router_logits.shape
    if experts_per_token <= 0 or experts_per_token > experts:
        raise ValueError("experts per token must be positive and not exceed the expert count")
    if active_tokens is not None and (active_tokens.dtype != torch.bool or
                                      tuple(active_tokens.shape) != (tokens,)):
        raise ValueError("active MoE token mask must be Bool [tokens]")
    _require_cuda(router_logits, active_tokens)
    ids = torch.empty((tokens, experts_per_token), dtype=torch.int32, device=router_logits.device)
    weights = torch.empty((tokens, experts_per_token), dtype=dtype, device=router_logits.device)
    request = _abi.Route(logits=_ptr(router_logits), active_tokens=_ptr(active_tokens),
                         expert_ids=_ptr(ids), routing_weights=_ptr(weights),
                         stream=_stream(router_logits), tokens=tokens, experts=experts,
                         experts_per_token=experts_per_token, dtype=_code(dtype))
    _abi.call("nml_nvfp4_sm100_route", request)
    return ids, weights


@dataclass
class AssignmentPlan:
    """The schedule of crates/nml-ir/src/lib.rs:5644-5779 (device tensors)."""

    sorted_assignments: torch.Tensor  # i32 [positions]
    block_experts: torch.Tensor       # i32 [blocks]
    active_blocks: torch.Tensor       # i32 scalar
    block_size: int = 16


def moe_assignment_plan(expert_ids: torch.Tensor, experts: int,
                        expert_offset: int = 0) -> AssignmentPlan:
    if expert_ids.dtype != torch.int32:
        raise ValueError("expert ids must be I32")
    assignments = expert_ids.numel()
    try:
        blocks, positions = _abi.plan_capacity(assignments, experts)
    except _abi.NvFp4Error as error:
        raise ValueError(error.message) from None
    _require_cuda(expert_ids)
    device = expert_ids.device
    plan = AssignmentPlan(torch.empty(positions, dtype=torch.int32, device=device),
                          torch.empty(blocks, dtype=torch.int32, device=device),
                          torch.empty((), dtype=torch.int32, device=device))
    request = _abi.AssignmentPlan(expert_ids=_ptr(expert_ids),
                                  sorted_assignments=_ptr(plan.sorted_assignments),
                                  block_experts=_ptr(plan.block_experts),
                                  active_blocks=_ptr(plan.active_blocks),
                                  stream=_stream(expert_ids), assignments=assignments,
                                  experts=experts, schedule_positions=positions,
                                  schedule_blocks=blocks, block_size=16,
                                  expert_offset=expert_offset)
    _abi.call("nml_nvfp4_sm100_assignment_plan", request)
    return plan


def _check_experts(hidden_size, gate_up: NvFp4Parameter, gate_up_bias, down: NvFp4Parameter,
                   down_bias, dtype):
    if len(gate_up.shape) != 3 or len(down.shape) != 3 or gate_up_bias.dim() != 2 or \
            down_bias.dim() != 2:
        raise ValueError(
            "clamped SwiGLU expects hidden [tokens, hidden], router [tokens, experts], gate/up "
            "[experts, 2*intermediate, hidden], gate/up bias [experts, 2*intermediate], down "
            "[experts, hidden, intermediate], and down bias [experts, hidden]")
    experts, doubled, gate_inputs = gate_up.shape
    if doubled <= 0 or doubled % 2 != 0 or gate_inputs != hidden_size or \
            down.shape != (experts, hidden_size, doubled // 2) or \
            tuple(gate_up_bias.shape) != (experts, doubled) or \
            tuple(down_bias.shape) != (experts, hidden_size):
        raise ValueError("clamped SwiGLU expert parameter dimensions are inconsistent")
    for tensor_dtype in (gate_up.dtype, down.dtype, gate_up_bias.dtype, down_bias.dtype):
        if tensor_dtype != dtype:
            raise ValueError(
                "clamped SwiGLU weights, biases, and hidden states must use one dtype")
    return experts, doubled // 2


def expert_gate_up(hidden: torch.Tensor, plan: AssignmentPlan, gate_up: NvFp4Parameter,
                   gate_up_bias: torch.Tensor, experts_per_token: int,
                   expert_offset: torch.Tensor | None = None,
                   use_active_blocks: bool = True) -> torch.Tensor:
    """activated ``[tokens * k, intermediate]``; rows of unscheduled routes are not written."""
    tokens, hidden_size = hidden.shape
    experts, doubled, _ = gate_up.shape
    intermediate = doubled // 2
    assignments = tokens * experts_per_token
    _require_cuda(hidden, gate_up.payload, gate_up_bias)
    activated = torch.zeros((assignments, intermediate), dtype=hidden.dtype, device=hidden.device)
    request = _abi.ExpertGateUp(
        hidden=_ptr(hidden), sorted_assignments=_ptr(plan.sorted_assignments),
        block_experts=_ptr(plan.block_experts), payload=_ptr(gate_up.payload),
        block_scales=_ptr(gate_up.block_scales), global_scale=_ptr(gate_up.global_scale),
        bias=_ptr(gate_up_bias), activated=_ptr(activated), stream=_stream(hidden),
        tokens=tokens, assignments=assignments,
        schedule_positions=plan.sorted_assignments.numel(),
        schedule_blocks=plan.block_experts.numel(), hidden_size=hidden_size,
        intermediate_size=intermediate, experts=experts, experts_per_token=experts_per_token,
        block_size=16, dtype=_code(hidden.dtype),
        active_blocks=_ptr(plan.active_blocks) if use_active_blocks else None,
        expert_offset=_ptr(expert_offset))
    _abi.call("nml_nvfp4_sm100_expert_gate_up", request)
    return activated


def expert_down(activated: torch.Tensor, plan: AssignmentPlan, down: NvFp4Parameter,
                down_bias: torch.Tensor, routing_weights: torch.Tensor, experts_per_token: int,
                expert_offset: torch.Tensor | None = None,
                use_active_blocks: bool = True) -> torch.Tensor:
    """weighted ``[tokens * k, hidden]`` = (activated . W_down^T + bias) * routing weight."""
    assignments, intermediate = activated.shape
    experts, hidden_size, _ = down.shape
    _require_cuda(activated, down.payload, down_bias, routing_weights)
    weighted = torch.zeros((assignments, hidden_size), dtype=activated.dtype,
                           device=activated.device)
    request = _abi.ExpertDown(
        activated=_ptr(activated), sorted_assignments=_ptr(plan.sorted_assignments),
        block_experts=_ptr(plan.block_experts), payload=_ptr(down.payload),
        block_scales=_ptr(down.block_scales), global_scale=_ptr(down.global_scale),
        bias=_ptr(down_bias), routing_weights=_ptr(routing_weights),
        weighted_output=_ptr(weighted), stream=_stream(activated), assignments=assignments,
        schedule_positions=plan.sorted_assignments.numel(),
        schedule_blocks=plan.block_experts.numel(), intermediate_size=intermediate,
        hidden_size=hidden_size, experts=experts, experts_per_token=experts_per_token,
        block_size=16, dtype=_code(activated.dtype),
        active_blocks=_ptr(plan.active_blocks) if use_active_blocks else None,
        expert_offset=_ptr(expert_offset))
    _abi.call("nml_nvfp4_sm100_expert_down", request)
    return weighted


def combine(weighted: torch.Tensor, tokens: int, experts_per_token: int,
            expert_ids: torch.Tensor | None = None, experts: int = 0,
            expert_offset: int = 0) -> torch.Tensor:
    """Sums the k weighted rows of every token in f32 and narrows once."""
    hidden_size = weighted.shape[-1]
    _require_cuda(weighted, expert_ids)
    out = torch.empty((tokens, hidden_size), dtype=weighted.dtype, device=weighted.device)
    request = _abi.Combine(weighted=_ptr(weighted), expert_ids=_ptr(expert_ids),
                           output=_ptr(out), stream=_stream(weighted), tokens=tokens,
                           experts_per_token=experts_per_token, hidden_size=hidden_size,
                           experts=experts, expert_offset=expert_offset,
                           dtype=_code(weighted.dtype))
    _abi.call("nml_nvfp4_sm100_combine", request)
    return out


_WORKSPACES: dict = {}


def routed_experts(hidden: torch.Tensor, expert_ids: torch.Tensor,
                   routing_weights: torch.Tensor, gate_up: NvFp4Parameter,
                   gate_up_bias: torch.Tensor, down: NvFp4Parameter, down_bias: torch.Tensor,
                   expert_offset: int = 0, out: torch.Tensor | None = None,
                   workspace: torch.Tensor | None = None, live_routes: int = 0,
                   leave_masked_rows: bool = False,
                   row_targets: torch.Tensor | None = None) -> torch.Tensor:
    """The routed layer from given routes, one C-ABI call (plan, gate/up + SwiGLU, down,
    k-way sum); the unit of the reference's CPU target ``nml.nvfp4.routed_swiglu``
    (crates/nml-kernel-nvfp4/src/ffi.rs:228-428).  ``workspace`` (u8, 256-byte aligned, at
    least ``nml_nvfp4_sm100_routed_swiglu_workspace_bytes``) replaces the cached scratch
    buffer, e.g. to inspect the intermediates afterwards.  ``live_routes`` (optional) tells
    the kernel selection how many routes are expected not to be masked.  ``leave_masked_rows``
    (one route per token only) skips the k-way sum pass: rows of masked tokens stay untouched;
    with it, ``row_targets`` (I64 ``[tokens]`` device addresses, 0 to skip a row) sends every
    token's result row to its address instead of ``out`` (an expert-parallel owner: into the
    senders' return buffers)."""
    if hidden.dim() != 2 or expert_ids.dim() != 2 or \
            tuple(routing_weights.shape) != tuple(expert_ids.shape) or \
            expert_ids.shape[0] != hidden.shape[0]:
        raise ValueError("routing tensors do not match the token and hidden extents")
    tokens, hidden_size = hidden.shape
    top_k = expert_ids.shape[1]
    experts, intermediate = _check_experts(hidden_size, gate_up, gate_up_bias, down, down_bias,
                                           hidden.dtype)
    if expert_ids.dtype != torch.int32 or routing_weights.dtype != hidden.dtype:
        raise ValueError("NVFP4 routed SwiGLU activations and biases must share F16 or BF16")
    _require_cuda(hidden, expert_ids, routing_weights, gate_up.payload, gate_up_bias,
                  down.payload, down_bias)
    size = _abi.load().nml_nvfp4_sm100_routed_swiglu_workspace_bytes(
        tokens, hidden_size, intermediate, experts, top_k)
    if size == 0:
        raise ValueError("MoE routing schedule must be addressable by i32 indices")
    if workspace is None:
        key = (hidden.device, torch.cuda.current_stream(hidden.device).cuda_stream)
        workspace = _WORKSPACES.get(key)
        if workspace is None or workspace.numel() < size:
            workspace = torch.empty(size, dtype=torch.uint8, device=hidden.device)
            _WORKSPACES[key] = workspace
    elif workspace.dtype != torch.uint8 or workspace.numel() < size or not workspace.is_cuda:
        raise ValueError("the routed-layer workspace must be a device U8 buffer of at least "
                         f"{size} bytes")
    if row_targets is not None:
        if not (leave_masked_rows and top_k == 1):
            raise ValueError("row targets need one route per token and leave_masked_rows")
        if row_targets.dtype != torch.int64 or tuple(row_targets.shape) != (tokens,) or \
                not row_targets.is_contiguous():
            raise ValueError("row targets must be I64 [tokens] device addresses")
        _require_cuda(row_targets)
    if out is None:
        out = torch.empty_like(hidden) if row_targets is None else hidden  # not written
    request = _abi.RoutedSwiglu(
        hidden=_ptr(hidden), expert_ids=_ptr(expert_ids), routing_weights=_ptr(routing_weights),
        gate_payload=_ptr(gate_up.payload), gate_scales=_ptr(gate_up.block_scales),
        gate_global=_ptr(gate_up.global_scale), gate_bias=_ptr(gate_up_bias),
        down_payload=_ptr(down.payload), down_scales=_ptr(down.block_scales),
        down_global=_ptr(down.global_scale), down_bias=_ptr(down_bias), output=_ptr(out),
        workspace=_ptr(workspace), workspace_bytes=workspace.numel(), stream=_stream(hidden),
        tokens=tokens, hidden_size=hidden_size, intermediate_size=intermediate, experts=experts,
        experts_per_token=top_k, expert_offset=expert_offset, dtype=_code(hidden.dtype),
        live_routes_hint=live_routes,
        flags=_abi.ROUTED_LEAVE_MASKED_ROWS if leave_masked_rows and top_k == 1 else 0,
        row_targets=_ptr(row_targets))
    _abi.call("nml_nvfp4_sm100_routed_swiglu", request)
    return out


def routed_clamped_swiglu(hidden: torch.Tensor, router_logits: torch.Tensor,
                          gate_up_weights: NvFp4Parameter, gate_up_bias: torch.Tensor,
                          down_weights: NvFp4Parameter, down_bias: torch.Tensor,
                          experts_per_token: int) -> torch.Tensor:
    """Routed clamped residual SwiGLU (crates/nml-ir/src/lib.rs:1257-1277)."""
    return routed_clamped_swiglu_masked(hidden, router_logits, gate_up_weights, gate_up_bias,
                                        down_weights, down_bias, experts_per_token, None)


def routed_clamped_swiglu_masked(hidden: torch.Tensor, router_logits: torch.Tensor,
                                 gate_up_weights: NvFp4Parameter, gate_up_bias: torch.Tensor,
                                 down_weights: NvFp4Parameter, down_bias: torch.Tensor,
                                 experts_per_token: int,
                                 active_tokens: torch.Tensor | None) -> torch.Tensor:
    """As ``routed_clamped_swiglu`` with a runtime active-token mask: masked tokens create no
    expert work and return an exact zero row (crates/nml-ir/src/lib.rs:1279-1308,1490-1498)."""
    if hidden.dim() != 2 or router_logits.dim() != 2:
        raise ValueError(
            "clamped SwiGLU expects hidden [tokens, hidden], router [tokens, experts], gate/up "
            "[experts, 2*intermediate, hidden], gate/up bias [experts, 2*intermediate], down "
            "[experts, hidden, intermediate], and down bias [experts, hidden]")
    experts, _ = _check_experts(hidden.shape[1], gate_up_weights, gate_up_bias, down_weights,
                                down_bias, hidden.dtype)
    if router_logits.shape[0] != hidden.shape[0] or router_logits.shape[1] != experts:
        raise ValueError("clamped SwiGLU expert parameter dimensions are inconsistent")
    ids, weights = route(router_logits, experts_per_token, hidden.dtype, active_tokens)
    return routed_experts(hidden, ids, weights, gate_up_weights, gate_up_bias, down_weights,
                          down_bias)


# ------------------------------------------------------------------ attention (decode)

_ATTENTION_SCRATCH: dict = {}


def _attention_splits(pairs: int, visible_pages: int, sms: int) -> int:
    """Splits of the visible pages per (sequence, kv head).  The decode kernel runs at the HBM
    rate once about two CTAs per SM are busy, and every further split only adds partial
    results for the second pass: split until there are 2 * sms CTAs, at most one split per 8
    pages (measured on B200 at 4096 tokens: batch 64, 512 pairs, is fastest unsplit; batch 8
    gains 1.5x from 2 to 8 splits and nothing beyond)."""
    wanted = -(-2 * sms // max(1, pairs))
    return max(1, min(wanted, max(1, visible_pages // 8), 64))


def paged_attention_decode(query: torch.Tensor, key_cache: torch.Tensor,
                           value_cache: torch.Tensor, page_table: torch.Tensor,
                           sequence_lengths: torch.Tensor, sinks: torch.Tensor | None = None,
                           sliding_window: int | None = None, scale: float | None = None,
                           splits: int | None = None) -> torch.Tensor:
    """One query token per sequence over a paged K/V cache
    (``Graph::paged_attention``, crates/nml-ir/src/lib.rs:4717-4730, for a query length of one).

    ``query`` [batch, query_heads, head_dim]; caches [physical_pages, page_size, kv_heads,
    head_dim]; ``page_table`` i32 [batch, logical_pages]; ``sequence_lengths`` i32 [batch]
    (visible tokens, the query token included); ``sinks`` f32 [query_heads] or None."""
    if query.dim() != 3 or key_cache.dim() != 4 or key_cache.shape != value_cache.shape:
        raise ValueError("paged attention expects query [batch, heads, dim] and K/V caches "
                         "[pages, page_size, kv_heads, dim] of one shape")
    batch, query_heads, head_dim = query.shape
    pages, page_size, kv_heads, cache_dim = key_cache.shape
    if cache_dim != head_dim or query_heads % kv_heads != 0:
        raise ValueError("paged query/KV head geometry is incompatible")
    if query.dtype != key_cache.dtype or query.dtype != value_cache.dtype:
        raise ValueError("query and paged K/V cache dtypes must match")
    if page_table.dtype != torch.int32 or sequence_lengths.dtype != torch.int32 or \
            page_table.dim() != 2 or page_table.shape[0] != batch or \
            tuple(sequence_lengths.shape) != (batch,):
        raise ValueError("page table must be I32 [batch, pages], sequence lengths I32 [batch]")
    if sinks is not None and (sinks.dtype != torch.float32 or tuple(sinks.shape) != (query_heads,)):
        raise ValueError("attention sinks must be F32 [query_heads]")
    _require_cuda(query, key_cache, value_cache, page_table, sequence_lengths, sinks)
    if splits is None:
        sms = torch.cuda.get_device_properties(query.device).multi_processor_count
        visible = page_table.shape[1] if not sliding_window else -(-sliding_window // page_size) + 1
        splits = _attention_splits(batch * kv_heads, visible, sms)
    lib = _abi.load()
    size = lib.nml_sm100_paged_attention_decode_workspace_bytes(batch, query_heads, splits)
    key = (query.device, torch.cuda.current_stream(query.device).cuda_stream)
    scratch = _ATTENTION_SCRATCH.get(key)
    if scratch is None or scratch.numel() < size:
        scratch = torch.empty(size, dtype=torch.uint8, device=query.device)
        _ATTENTION_SCRATCH[key] = scratch
    out = torch.empty_like(query)
    request = _abi.PagedAttentionDecode(
        query=_ptr(query), key_cache=_ptr(key_cache), value_cache=_ptr(value_cache),
        page_table=_ptr(page_table), sequence_lengths=_ptr(sequence_lengths), sinks=_ptr(sinks),
        output=_ptr(out), workspace=_ptr(scratch), workspace_bytes=scratch.numel(),
        stream=_stream(query), batch=batch, query_heads=query_heads, kv_heads=kv_heads,
        head_dim=head_dim, page_size=page_size, physical_pages=pages,
        table_width=page_table.shape[1], sliding_window=sliding_window or 0, splits=splits,
        scale=float(scale if scale is not None else head_dim ** -0.5), dtype=_code(query.dtype))
    _abi.call("nml_sm100_paged_attention_decode", request)
    return out


def topk_rows(logits: torch.Tensor, k: int, index_offset: int = 0):
    """(values f32 [rows, k], indices i32 [rows, k]) of the k largest entries of every row of a
    16-bit matrix, descending, equal values to the lower index (``nml_nvfp4_sm100_topk_rows``)."""
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("top-k expects a matrix with contiguous rows")
    rows, columns = logits.shape
    if not 0 < k <= min(16, columns):
        raise ValueError("top-k supports 1 <= k <= 16")
    if not logits.is_cuda:
        raise RuntimeError("NVFP4 operators run on a CUDA device only (no CPU fallback)")
    lib = _abi.load()
    size = lib.nml_nvfp4_sm100_topk_rows_workspace_bytes(rows, columns, k)
    scratch = torch.empty(size, dtype=torch.uint8, device=logits.device)
    values = torch.empty((rows, k), dtype=torch.float32, device=logits.device)
    indices = torch.empty((rows, k), dtype=torch.int32, device=logits.device)
    request = _abi.TopkRows(logits=_ptr(logits), values=_ptr(values), indices=_ptr(indices),
                            workspace=_ptr(scratch), workspace_bytes=size,
                            stream=_stream(logits), rows=rows, columns=columns,
                            row_stride=logits.stride(0), k=k, index_offset=index_offset,
                            dtype=_code(logits.dtype))
    _abi.call("nml_nvfp4_sm100_topk_rows", request)
    return values, indices


def topk_merge(values: torch.Tensor, indices: torch.Tensor, k: int):
    """(values f32 [rows, k], indices i32 [rows, k]): the k best of every row among the
    candidates of several parts (shards or ranks), ``values`` f32 and ``indices`` i32 of shape
    ``[parts, rows, >= k]`` with the same strides (views into one gathered block are fine);
    larger value first, equal values to the lower index, negative indices are empty
    (``nml_nvfp4_sm100_topk_merge``)."""
    if values.dim() != 3 or values.shape != indices.shape or values.stride() != indices.stride():
        raise ValueError("top-k merge expects values and indices of one shape and layout")
    if values.dtype != torch.float32 or indices.dtype != torch.int32:
        raise ValueError("top-k merge takes F32 values and I32 indices")
    parts, rows, width = values.shape
    pitch = values.stride(1)
    if values.stride(2) != 1 or values.stride(0) != rows * pitch or not 0 < k <= min(16, width) \
            or parts * k > 512:
        raise ValueError("top-k merge: candidates must be row-contiguous, k <= 16, parts * k <= 512")
    if not values.is_cuda or not indices.is_cuda:
        raise RuntimeError("NVFP4 operators run on a CUDA device only (no CPU fallback)")
    out_values = torch.empty((rows, k), dtype=torch.float32, device=values.device)
    out_indices = torch.empty((rows, k), dtype=torch.int32, device=values.device)
    request = _abi.TopkMerge(values=values.data_ptr(), indices=indices.data_ptr(),
                             out_values=_ptr(out_values), out_indices=_ptr(out_indices),
                             stream=_stream(values), parts=parts, rows=rows, pitch=pitch, k=k)
    _abi.call("nml_nvfp4_sm100_topk_merge", request)
    return out_values, out_indices
