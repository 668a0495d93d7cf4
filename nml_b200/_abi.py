"""ctypes binding of ``include/nml_nvfp4_sm100.h`` (the C ABI of the sm_100a NVFP4 library).

The structures mirror the header field for field.  ``load()`` fails loudly when the shared
object is missing: there is no CPU or PyTorch fallback for any operation.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libnml_nvfp4_sm100.so"
_LIB = None

F16 = 1
BF16 = 2

OK = 0
INVALID_ARGUMENT = 1
LAUNCH_FAILURE = 2

STATUS_BARRIER_TIMEOUT = 1
STATUS_TMEM_ALLOC = 2
STATUS_INDEX_RANGE = 4
STATUS_PEER_TIMEOUT = 8

ROUTED_LEAVE_MASKED_ROWS = 1

STATIC_SCRATCH_BYTES = 8 << 20

POLICY_AUTO = 0
POLICY_SIMT = 1
POLICY_UMMA = 2
POLICY_UMMA_SMEM = 3  # tcgen05 with the decoded-weight ring in shared memory
POLICY_NO_SPLIT_K = 5  # tcgen05, never cut K over a cluster
POLICY_STREAM = 6  # the weight-streaming kernels for few rows

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int32
_sz = ctypes.c_size_t


class Linear(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("activation", _vp), ("payload", _vp),
                ("block_scales", _vp), ("global_scale", _vp), ("bias", _vp), ("output", _vp),
                ("stream", _vp), ("rows", _i64), ("outputs", _i64), ("inputs", _i64),
                ("dtype", _i32), ("residual", _vp), ("workspace", _vp),
                ("workspace_bytes", _sz)]


class LinearQkv(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("activation", _vp), ("payload", _vp * 3),
                ("block_scales", _vp * 3), ("global_scale", _vp * 3), ("bias", _vp * 3),
                ("output", _vp * 3), ("stream", _vp), ("rows", _i64), ("outputs", _i64 * 3),
                ("inputs", _i64), ("dtype", _i32)]


class Embedding(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("indices", _vp), ("payload", _vp), ("block_scales", _vp),
                ("global_scale", _vp), ("output", _vp), ("stream", _vp), ("rows", _i64),
                ("vocabulary", _i64), ("width", _i64), ("dtype", _i32),
                ("indices_are_i64", ctypes.c_uint8)]


class ExpertGateUp(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("hidden", _vp), ("sorted_assignments", _vp),
                ("block_experts", _vp), ("payload", _vp), ("block_scales", _vp),
                ("global_scale", _vp), ("bias", _vp), ("activated", _vp), ("stream", _vp),
                ("tokens", _i64), ("assignments", _i64), ("schedule_positions", _i64),
                ("schedule_blocks", _i64), ("hidden_size", _i64), ("intermediate_size", _i64),
                ("experts", _i64), ("experts_per_token", _i64), ("block_size", _i32),
                ("dtype", _i32), ("active_blocks", _vp), ("expert_offset", _vp)]


class ExpertDown(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("activated", _vp), ("sorted_assignments", _vp),
                ("block_experts", _vp), ("payload", _vp), ("block_scales", _vp),
                ("global_scale", _vp), ("bias", _vp), ("routing_weights", _vp),
                ("weighted_output", _vp), ("stream", _vp), ("assignments", _i64),
                ("schedule_positions", _i64), ("schedule_blocks", _i64),
                ("intermediate_size", _i64), ("hidden_size", _i64), ("experts", _i64),
                ("experts_per_token", _i64), ("block_size", _i32), ("dtype", _i32),
                ("active_blocks", _vp), ("expert_offset", _vp), ("row_targets", _vp)]


class Route(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("logits", _vp), ("active_tokens", _vp),
                ("expert_ids", _vp), ("routing_weights", _vp), ("stream", _vp),
                ("tokens", _i64), ("experts", _i64), ("experts_per_token", _i64),
                ("dtype", _i32)]


class AssignmentPlan(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("expert_ids", _vp), ("sorted_assignments", _vp),
                ("block_experts", _vp), ("active_blocks", _vp), ("stream", _vp),
                ("assignments", _i64), ("experts", _i64), ("schedule_positions", _i64),
                ("schedule_blocks", _i64), ("block_size", _i32), ("expert_offset", _i32)]


class Combine(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("weighted", _vp), ("expert_ids", _vp), ("output", _vp),
                ("stream", _vp), ("tokens", _i64), ("experts_per_token", _i64),
                ("hidden_size", _i64), ("experts", _i64), ("expert_offset", _i32),
                ("dtype", _i32)]


class RoutedSwiglu(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("hidden", _vp), ("expert_ids", _vp),
                ("routing_weights", _vp), ("gate_payload", _vp), ("gate_scales", _vp),
                ("gate_global", _vp), ("gate_bias", _vp), ("down_payload", _vp),
                ("down_scales", _vp), ("down_global", _vp), ("down_bias", _vp), ("output", _vp),
                ("workspace", _vp), ("workspace_bytes", _sz), ("stream", _vp), ("tokens", _i64),
                ("hidden_size", _i64), ("intermediate_size", _i64), ("experts", _i64),
                ("experts_per_token", _i64), ("expert_offset", _i32), ("dtype", _i32),
                ("live_routes_hint", _i64), ("flags", _i32), ("row_targets", _vp)]


class EpDispatchPlan(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("expert_ids", _vp), ("send_order", _vp),
                ("local_expert", _vp), ("slot_of_assignment", _vp), ("send_counts", _vp),
                ("stream", _vp), ("assignments", _i64), ("ranks", _i64),
                ("experts_per_rank", _i64)]


class GatherRows(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("source", _vp), ("row_index", _vp), ("output", _vp),
                ("stream", _vp), ("rows", _i64), ("source_rows", _i64), ("width", _i64),
                ("index_divisor", _i32), ("dtype", _i32)]


class CombineRows(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("rows", _vp), ("row_index", _vp), ("output", _vp),
                ("stream", _vp), ("tokens", _i64), ("experts_per_token", _i64),
                ("hidden_size", _i64), ("row_count", _i64), ("dtype", _i32)]


class TopkRows(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("logits", _vp), ("values", _vp), ("indices", _vp),
                ("workspace", _vp), ("workspace_bytes", _sz), ("stream", _vp), ("rows", _i64),
                ("columns", _i64), ("row_stride", _i64), ("k", _i64), ("index_offset", _i32),
                ("dtype", _i32)]


class PagedAttentionDecode(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("query", _vp), ("key_cache", _vp), ("value_cache", _vp),
                ("page_table", _vp), ("sequence_lengths", _vp), ("sinks", _vp), ("output", _vp),
                ("workspace", _vp), ("workspace_bytes", _sz), ("stream", _vp), ("batch", _i64),
                ("query_heads", _i64), ("kv_heads", _i64), ("head_dim", _i64),
                ("page_size", _i64), ("physical_pages", _i64), ("table_width", _i64),
                ("sliding_window", _i64), ("splits", _i64), ("scale", ctypes.c_float),
                ("dtype", _i32)]


class RoutedWorkspaceLayout(ctypes.Structure):
    _fields_ = [("sorted_assignments", _sz), ("block_experts", _sz), ("active_blocks", _sz),
                ("activated", _sz), ("weighted", _sz), ("permuted_hidden", _sz),
                ("slot_activated", _sz), ("schedule_blocks", _i64), ("schedule_positions", _i64),
                ("slot_ordered", _i32)]


EP_MAX_RANKS = 16


EP_SYNC_WORDS = 3 * EP_MAX_RANKS
EP_STATE_WORDS = 4


class EpExchange(ctypes.Structure):
    _fields_ = [("peer_rows", _vp * EP_MAX_RANKS), ("peer_meta", _vp * EP_MAX_RANKS),
                ("peer_back", _vp * EP_MAX_RANKS), ("peer_sync", _vp * EP_MAX_RANKS),
                ("local_state", _vp), ("ranks", _i64), ("rank", _i64), ("region_rows", _i64),
                ("width", _i64)]


class EpPushRows(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("source", _vp), ("send_order", _vp),
                ("local_expert", _vp), ("routing_weights", _vp), ("send_counts", _vp),
                ("exchange", EpExchange), ("stream", _vp), ("assignments", _i64),
                ("source_rows", _i64), ("experts_per_token", _i64), ("dtype", _i32)]


class EpReceiveMeta(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("exchange", EpExchange), ("expert_ids", _vp),
                ("routing_weights", _vp), ("received", _vp), ("stream", _vp),
                ("wait_limit", _i64), ("dtype", _i32), ("row_targets", _vp)]


class EpReturnRows(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("computed", _vp), ("exchange", EpExchange),
                ("stream", _vp), ("dtype", _i32)]


class EpWaitReturns(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("exchange", EpExchange), ("stream", _vp),
                ("wait_limit", _i64), ("row_index", _vp), ("output", _vp), ("tokens", _i64),
                ("experts_per_token", _i64), ("dtype", _i32)]


class TopkMerge(ctypes.Structure):
    _fields_ = [("struct_size", _sz), ("values", _vp), ("indices", _vp), ("out_values", _vp),
                ("out_indices", _vp), ("stream", _vp), ("parts", _i64), ("rows", _i64),
                ("pitch", _i64), ("k", _i64)]


# name -> request structure, for the entry points of the form fn(const Request*, char*, size_t)
REQUEST_ENTRY_POINTS = {
    "nml_nvfp4_sm100_topk_merge": TopkMerge,
    "nml_nvfp4_sm100_ep_push_rows": EpPushRows,
    "nml_nvfp4_sm100_ep_receive_meta": EpReceiveMeta,
    "nml_nvfp4_sm100_ep_return_rows": EpReturnRows,
    "nml_nvfp4_sm100_ep_wait_returns": EpWaitReturns,
    "nml_nvfp4_sm100_linear": Linear,
    "nml_nvfp4_sm100_linear_qkv": LinearQkv,
    "nml_nvfp4_sm100_embedding": Embedding,
    "nml_nvfp4_sm100_expert_gate_up": ExpertGateUp,
    "nml_nvfp4_sm100_expert_down": ExpertDown,
    "nml_nvfp4_sm100_route": Route,
    "nml_nvfp4_sm100_assignment_plan": AssignmentPlan,
    "nml_nvfp4_sm100_combine": Combine,
    "nml_nvfp4_sm100_routed_swiglu": RoutedSwiglu,
    "nml_nvfp4_sm100_routed_swiglu_static": RoutedSwiglu,
    "nml_nvfp4_sm100_ep_dispatch_plan": EpDispatchPlan,
    "nml_nvfp4_sm100_gather_rows": GatherRows,
    "nml_nvfp4_sm100_combine_rows": CombineRows,
    "nml_sm100_paged_attention_decode": PagedAttentionDecode,
    "nml_nvfp4_sm100_topk_rows": TopkRows,
}

OTHER_ENTRY_POINTS = [
    "nml_nvfp4_sm100_linear_workspace_bytes",
    "nml_nvfp4_sm100_linear_workspace_verdict_offset",
    "nml_nvfp4_sm100_routed_swiglu_workspace_bytes",
    "nml_nvfp4_sm100_routed_swiglu_workspace_layout",
    "nml_nvfp4_sm100_plan_capacity",
    "nml_nvfp4_sm100_device_status",
    "nml_nvfp4_sm100_set_kernel_policy",
    "nml_nvfp4_sm100_last_linear_kernel",
    "nml_nvfp4_sm100_last_linear_tile_rows",
    "nml_nvfp4_sm100_abi_version",
    "nml_sm100_paged_attention_decode_workspace_bytes",
    "nml_nvfp4_sm100_topk_rows_workspace_bytes",
]


class NvFp4Error(RuntimeError):
    """A C-ABI call returned a nonzero status; ``code`` is 1 (invalid argument) or 2 (launch)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


def library_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m nml_b200.build` "
            "(there is no fallback path)")
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, struct in REQUEST_ENTRY_POINTS.items():
        fn = getattr(lib, name)
        fn.restype = _i32
        fn.argtypes = [ctypes.POINTER(struct), ctypes.c_char_p, _sz]
    lib.nml_nvfp4_sm100_linear_workspace_bytes.restype = _sz
    lib.nml_nvfp4_sm100_linear_workspace_bytes.argtypes = [_i64, _i64, _i64, _i32]
    lib.nml_nvfp4_sm100_linear_workspace_verdict_offset.restype = _sz
    lib.nml_nvfp4_sm100_linear_workspace_verdict_offset.argtypes = [_i64, _i64, _i64, _i32]
    lib.nml_nvfp4_sm100_routed_swiglu_workspace_bytes.restype = _sz
    lib.nml_nvfp4_sm100_routed_swiglu_workspace_bytes.argtypes = [_i64] * 5
    lib.nml_nvfp4_sm100_routed_swiglu_workspace_layout.restype = _i32
    lib.nml_nvfp4_sm100_routed_swiglu_workspace_layout.argtypes = [_i64] * 5 + [
        ctypes.POINTER(RoutedWorkspaceLayout)]
    lib.nml_nvfp4_sm100_topk_rows_workspace_bytes.restype = _sz
    lib.nml_nvfp4_sm100_topk_rows_workspace_bytes.argtypes = [_i64] * 3
    lib.nml_sm100_paged_attention_decode_workspace_bytes.restype = _sz
    lib.nml_sm100_paged_attention_decode_workspace_bytes.argtypes = [_i64] * 3
    lib.nml_nvfp4_sm100_plan_capacity.restype = _i32
    lib.nml_nvfp4_sm100_plan_capacity.argtypes = [_i64, _i64, ctypes.POINTER(_i64),
                                                  ctypes.POINTER(_i64)]
    lib.nml_nvfp4_sm100_device_status.restype = _i32
    lib.nml_nvfp4_sm100_device_status.argtypes = [_vp, _i32, ctypes.POINTER(_i32)]
    lib.nml_nvfp4_sm100_set_kernel_policy.restype = _i32
    lib.nml_nvfp4_sm100_set_kernel_policy.argtypes = [_i32]
    lib.nml_nvfp4_sm100_last_linear_kernel.restype = ctypes.c_char_p
    lib.nml_nvfp4_sm100_last_linear_kernel.argtypes = []
    lib.nml_nvfp4_sm100_last_linear_tile_rows.restype = _i32
    lib.nml_nvfp4_sm100_last_linear_tile_rows.argtypes = []
    lib.nml_nvfp4_sm100_abi_version.restype = _i32
    lib.nml_nvfp4_sm100_abi_version.argtypes = []
    _LIB = lib
    return lib


def call(name: str, request: ctypes.Structure, struct_size: int | None = None) -> None:
    """Invokes a request entry point; raises NvFp4Error on a nonzero return."""
    lib = load()
    request.struct_size = ctypes.sizeof(request) if struct_size is None else struct_size
    message = ctypes.create_string_buffer(256)
    code = getattr(lib, name)(ctypes.byref(request), message, len(message))
    if code != OK:
        raise NvFp4Error(code, message.value.decode("utf-8", "replace"))


def call_raw(name: str, request_pointer, message_capacity: int = 256):
    """Returns (code, message) without raising; accepts a NULL request pointer."""
    lib = load()
    message = ctypes.create_string_buffer(max(message_capacity, 1))
    code = getattr(lib, name)(request_pointer, message if message_capacity else None,
                              message_capacity)
    return code, message.value.decode("utf-8", "replace")


def plan_capacity(assignments: int, experts: int):
    blocks, positions = _i64(), _i64()
    if load().nml_nvfp4_sm100_plan_capacity(assignments, experts, ctypes.byref(blocks),
                                            ctypes.byref(positions)) != OK:
        raise NvFp4Error(INVALID_ARGUMENT, "MoE routing schedule must be addressable by i32")
    return blocks.value, positions.value


def set_kernel_policy(policy: int) -> int:
    return load().nml_nvfp4_sm100_set_kernel_policy(policy)


def last_linear_tile_rows() -> int:
    return int(load().nml_nvfp4_sm100_last_linear_tile_rows())


def last_linear_kernel() -> str:
    return load().nml_nvfp4_sm100_last_linear_kernel().decode()


def device_status(stream: int, clear: bool = True) -> int:
    status = _i32()
    code = load().nml_nvfp4_sm100_device_status(_vp(stream), 1 if clear else 0,
                                                ctypes.byref(status))
    if code != OK:
        raise NvFp4Error(code, "cannot read the device status word")
    return status.value
