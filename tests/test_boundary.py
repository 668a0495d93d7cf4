"""The C-ABI boundary without a GPU: the library loads, exports every symbol the header
declares, and rejects malformed requests with the reference adapter's return convention
(crates/nml-kernel-nvfp4/src/turing_adapter.cu:13-22,672-682,738-753,788-808) before any
device call is made."""
import ctypes
import re
from pathlib import Path

import pytest

from nml_b200 import _abi

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "nml_nvfp4_sm100.h").read_text()


def test_library_exports_every_declared_symbol():
    declared = set(re.findall(r"\b(nml_(?:nvfp4_)?sm100_[a-z0-9_]+)\s*\(", HEADER))
    assert declared == set(_abi.REQUEST_ENTRY_POINTS) | set(_abi.OTHER_ENTRY_POINTS)
    lib = ctypes.CDLL(str(_abi.library_path()))
    for name in declared:
        assert getattr(lib, name) is not None
    assert _abi.load().nml_nvfp4_sm100_abi_version() == 2


def test_reference_binding_patch_names_exported_entry_points():
    # the Rust glue a maintainer applies binds four of the header's entry points by name and
    # registers one custom-call target per entry point
    patch = (ROOT / "include" / "reference_sm100_binding.patch").read_text()
    added = "\n".join(line[1:] for line in patch.splitlines()
                      if line.startswith("+") and not line.startswith("+++"))
    bound = set(re.findall(r"fn (nml_nvfp4_sm100_[a-z0-9_]+)\(", added))
    assert bound == {"nml_nvfp4_sm100_linear", "nml_nvfp4_sm100_embedding",
                     "nml_nvfp4_sm100_expert_gate_up", "nml_nvfp4_sm100_expert_down"}
    assert bound <= set(_abi.REQUEST_ENTRY_POINTS)
    targets = set(re.findall(r'"(nml\.nvfp4\.sm100\.[a-z_]+)"', added))
    assert {"nml.nvfp4.sm100." + name[len("nml_nvfp4_sm100_"):] for name in bound} <= targets


def test_struct_sizes_match_reference_prefix():
    # The reference structs (nml_nvfp4.h:18-92) on LP64: Linear 96, Embedding 88,
    # ExpertGateUp 152, ExpertDown 152 bytes; the two trailing pointers add 16.
    assert _abi.Linear.residual.offset == 96  # the reference struct ends here
    assert _abi.Linear.workspace.offset == 104
    assert _abi.Linear.workspace_bytes.offset == 112
    assert ctypes.sizeof(_abi.Linear) == 120
    assert ctypes.sizeof(_abi.Embedding) == 88
    assert _abi.ExpertGateUp.active_blocks.offset == 152
    assert _abi.ExpertDown.active_blocks.offset == 152
    assert ctypes.sizeof(_abi.ExpertGateUp) == 168


FAKE = 0x1000  # never dereferenced: validation fails before any launch


def linear_request(**overrides):
    fields = dict(activation=FAKE, payload=FAKE, block_scales=FAKE, global_scale=FAKE, bias=None,
                  output=FAKE, stream=FAKE, rows=1, outputs=16, inputs=16, dtype=_abi.BF16)
    fields.update(overrides)
    return _abi.Linear(**fields)


@pytest.mark.parametrize("name", sorted(_abi.REQUEST_ENTRY_POINTS))
def test_null_and_truncated_requests_are_invalid_arguments(name):
    struct = _abi.REQUEST_ENTRY_POINTS[name]
    code, message = _abi.call_raw(name, None)
    assert code == _abi.INVALID_ARGUMENT and message
    request = struct()
    request.struct_size = 8
    code, message = _abi.call_raw(name, ctypes.byref(request))
    assert code == _abi.INVALID_ARGUMENT and ("truncated" in message or "invalid" in message)
    # a zeroed request of full size has null pointers and non-positive extents
    request.struct_size = ctypes.sizeof(struct)
    code, message = _abi.call_raw(name, ctypes.byref(request))
    assert code == _abi.INVALID_ARGUMENT and "invalid" in message
    # no message buffer is fine too
    assert _abi.call_raw(name, ctypes.byref(request), 0)[0] == _abi.INVALID_ARGUMENT


@pytest.mark.parametrize("override", [dict(activation=None), dict(payload=None),
                                      dict(block_scales=None), dict(global_scale=None),
                                      dict(output=None), dict(stream=None), dict(rows=0),
                                      dict(outputs=-1), dict(inputs=2 ** 31)])
def test_linear_rejects_bad_fields(override):
    with pytest.raises(_abi.NvFp4Error) as error:
        _abi.call("nml_nvfp4_sm100_linear", linear_request(**override))
    assert error.value.code == _abi.INVALID_ARGUMENT
    assert error.value.message == "invalid NVFP4 linear request"


def test_linear_rejects_unknown_dtype_and_truncated_struct():
    with pytest.raises(_abi.NvFp4Error) as error:
        _abi.call("nml_nvfp4_sm100_linear", linear_request(dtype=3))
    assert error.value.message == "NVFP4 linear supports F16 and BF16 only"
    with pytest.raises(_abi.NvFp4Error) as error:
        _abi.call("nml_nvfp4_sm100_linear", linear_request(), struct_size=40)
    assert error.value.message == "truncated NVFP4 linear request"


def test_message_is_truncated_to_capacity():
    request = linear_request(rows=0)
    request.struct_size = ctypes.sizeof(request)
    code, message = _abi.call_raw("nml_nvfp4_sm100_linear", ctypes.byref(request), 8)
    assert code == _abi.INVALID_ARGUMENT and message == "invalid"


def test_expert_requests_check_schedule_geometry():
    fields = dict(hidden=FAKE, sorted_assignments=FAKE, block_experts=FAKE, payload=FAKE,
                  block_scales=FAKE, global_scale=FAKE, bias=FAKE, activated=FAKE, stream=FAKE,
                  tokens=2, assignments=4, schedule_positions=64, schedule_blocks=4,
                  hidden_size=16, intermediate_size=16, experts=4, experts_per_token=2,
                  block_size=16, dtype=_abi.BF16)
    for override in (dict(block_size=32), dict(assignments=5), dict(schedule_positions=63),
                     dict(schedule_blocks=0), dict(experts=0), dict(bias=None)):
        with pytest.raises(_abi.NvFp4Error) as error:
            _abi.call("nml_nvfp4_sm100_expert_gate_up", _abi.ExpertGateUp(**{**fields,
                                                                              **override}))
        assert error.value.message == "invalid NVFP4 expert gate/up request"
    # the reference-sized struct (without the trailing pointers) is accepted as a struct:
    # it gets past the size check and fails on dtype instead
    request = _abi.ExpertGateUp(**{**fields, "dtype": 9})
    with pytest.raises(_abi.NvFp4Error) as error:
        _abi.call("nml_nvfp4_sm100_expert_gate_up", request, struct_size=152)
    assert error.value.message == "NVFP4 experts support F16 and BF16 only"


def test_plan_capacity_rule():
    # crates/nml-ir/src/lib.rs:5662-5688
    assert _abi.plan_capacity(16384, 32) == (1054, 16864)
    assert _abi.plan_capacity(256, 32) == (46, 736)
    assert _abi.plan_capacity(8, 32) == (8, 128)
    with pytest.raises(_abi.NvFp4Error):
        _abi.plan_capacity(2 ** 31 - 1, 32)


def test_workspace_size_is_monotone_and_aligned():
    size = _abi.load().nml_nvfp4_sm100_routed_swiglu_workspace_bytes
    small = size(64, 2880, 2880, 32, 4)
    large = size(4096, 2880, 2880, 32, 4)
    assert 0 < small < large and small % 256 == 0 and large % 256 == 0
    assert size(0, 2880, 2880, 32, 4) == 0


def test_linear_scratch_is_offered_only_where_the_narrowed_operands_pay():
    lib = _abi.load()
    size = lib.nml_nvfp4_sm100_linear_workspace_bytes
    verdict = lib.nml_nvfp4_sm100_linear_workspace_verdict_offset
    wide = size(512, 201088, 2880, _abi.BF16)
    # the narrowed rows, a magnitude per row, a factor per 256-row tile, the verdict word
    assert wide >= 512 * 2880 * 2 + 512 * 4 + 2 * 4 + 4 and wide % 256 == 0
    assert size(16384, 201088, 2880, _abi.BF16) > wide
    assert 512 * 2880 * 2 <= verdict(512, 201088, 2880, _abi.BF16) <= wide - 4
    assert verdict(512, 201088, 2880, _abi.BF16) % 4 == 0
    for rows, outputs, inputs, dtype in ((511, 201088, 2880, _abi.BF16),   # few rows
                                         (512, 5760, 2880, _abi.BF16),     # narrow weight
                                         (512, 201088, 2880, _abi.F16),    # already F16
                                         (512, 201088, 2872, _abi.BF16),   # K not in 64s
                                         (0, 201088, 2880, _abi.BF16),
                                         (512, 201088, 2880, 77)):
        assert size(rows, outputs, inputs, dtype) == 0
        assert verdict(rows, outputs, inputs, dtype) == 0


def test_operators_refuse_cpu_tensors():
    import torch
    from nml_b200 import ops
    weight = ops.NvFp4Parameter.nvfp4("w", (4, 16), torch.bfloat16,
                                      torch.zeros((4, 8), dtype=torch.uint8),
                                      torch.zeros((4, 1), dtype=torch.uint8),
                                      torch.ones((), dtype=torch.float32))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.linear(torch.zeros((1, 16), dtype=torch.bfloat16), weight)
    with pytest.raises(ValueError):
        ops.linear(torch.zeros((1, 15), dtype=torch.bfloat16), weight)
    with pytest.raises(ValueError):
        ops.linear(torch.zeros((1, 16), dtype=torch.float32), weight)
    with pytest.raises(ValueError):
        ops.NvFp4Parameter.nvfp4("w", (4, 16), torch.bfloat16,
                                 torch.zeros((4, 7), dtype=torch.uint8),
                                 torch.zeros((4, 1), dtype=torch.uint8),
                                 torch.ones((), dtype=torch.float32))
