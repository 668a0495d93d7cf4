"""ctypes/numpy front end of the C parity oracle in ``nvfp4_oracle.c``.

TEST INFRASTRUCTURE: a CPU restatement of the reference's NVFP4 CPU path.  It
is the checker for the CUDA kernels, never the thing shipped or measured as
the product.  Parity status: pinned (see the header of ``nvfp4_oracle.c``).

Array conventions: 16-bit floating tensors travel as ``numpy.uint16`` bit
patterns together with a dtype code (1 = f16, 2 = bf16), the same codes the
kernel ABI uses.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libnvfp4_oracle.so"
_LIB = None

F16 = 1
BF16 = 2

__all__ = [
    "F16", "BF16", "build", "lib", "decode_e2m1", "decode_e4m3fn_scale", "encode_e4m3fn_scale",
    "encode_e2m1", "global_scale", "quantize_row", "quantize_tensor", "dequantize_row", "dequantize_tensor",
    "validate_weight", "to_f32", "from_f32", "embedding", "linear", "linear_16",
    "grouped_projection", "routed_clamped_swiglu", "expert_gate_up", "expert_down", "route",
    "assignment_plan", "plan_capacity", "combine", "exp_det", "threads", "set_threads",
    "error_metrics", "set_avx2",
]


def build(force: bool = False) -> Path:
    """Compile the C oracle next to its source (gcc, a second or two)."""
    source = _HERE / "nvfp4_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libnvfp4_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        build()
        _LIB = ctypes.CDLL(str(_LIB_PATH))
        _declare(_LIB)
    return _LIB


_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_f32p = ctypes.POINTER(ctypes.c_float)
_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)
_sz = ctypes.c_size_t


def _declare(l: ctypes.CDLL) -> None:
    l.nml_oracle_decode_e2m1.restype = ctypes.c_float
    l.nml_oracle_decode_e2m1.argtypes = [ctypes.c_uint8]
    l.nml_oracle_decode_e4m3fn_scale.restype = ctypes.c_int
    l.nml_oracle_decode_e4m3fn_scale.argtypes = [ctypes.c_uint8, _f32p]
    l.nml_oracle_encode_e4m3fn_scale.restype = ctypes.c_uint8
    l.nml_oracle_encode_e4m3fn_scale.argtypes = [ctypes.c_float]
    l.nml_oracle_encode_e2m1.restype = ctypes.c_uint8
    l.nml_oracle_encode_e2m1.argtypes = [ctypes.c_float]
    l.nml_oracle_global_scale.restype = ctypes.c_float
    l.nml_oracle_global_scale.argtypes = [_f32p, _sz]
    l.nml_oracle_quantize_row.restype = None
    l.nml_oracle_quantize_row.argtypes = [_f32p, _sz, ctypes.c_float, _u8p, _u8p]
    l.nml_oracle_quantize_tensor.restype = ctypes.c_float
    l.nml_oracle_quantize_tensor.argtypes = [_f32p, _sz, _sz, _u8p, _u8p]
    l.nml_oracle_validate_weight.restype = ctypes.c_int
    l.nml_oracle_validate_weight.argtypes = [_u8p, _u8p, ctypes.c_float, _sz, _sz]
    l.nml_oracle_dequantize_row.restype = ctypes.c_int
    l.nml_oracle_dequantize_row.argtypes = [_u8p, _u8p, ctypes.c_float, _sz, _f32p]
    l.nml_oracle_to_f32.restype = None
    l.nml_oracle_to_f32.argtypes = [_u16p, _sz, ctypes.c_int, _f32p]
    l.nml_oracle_from_f32.restype = None
    l.nml_oracle_from_f32.argtypes = [_f32p, _sz, ctypes.c_int, _u16p]
    l.nml_oracle_embedding.restype = ctypes.c_longlong
    l.nml_oracle_embedding.argtypes = [_i64p, _sz, _u8p, _u8p, ctypes.c_float, _sz, _sz, _f32p]
    l.nml_oracle_linear.restype = None
    l.nml_oracle_linear.argtypes = [_f32p, _sz, _u8p, _u8p, ctypes.c_float, _sz, _sz, _f32p,
                                    _f32p, ctypes.c_int]
    l.nml_oracle_linear_16.restype = None
    l.nml_oracle_linear_16.argtypes = [_u16p, _sz, _u8p, _u8p, ctypes.c_float, _sz, _sz, _u16p,
                                       ctypes.c_int, _u16p, _f32p, ctypes.c_int]
    l.nml_oracle_grouped_projection.restype = ctypes.c_longlong
    l.nml_oracle_grouped_projection.argtypes = [_f32p, _i64p, _sz, _u8p, _u8p, ctypes.c_float,
                                                _sz, _sz, _sz, _f32p, _f32p, ctypes.c_int]
    l.nml_oracle_routed_clamped_swiglu.restype = ctypes.c_longlong
    l.nml_oracle_routed_clamped_swiglu.argtypes = [
        _f32p, _sz, _i64p, _f32p, _sz, _u8p, _u8p, ctypes.c_float, _f32p, _u8p, _u8p,
        ctypes.c_float, _f32p, _sz, _sz, _sz, _f32p, ctypes.c_int]
    l.nml_oracle_expert_gate_up.restype = None
    l.nml_oracle_expert_gate_up.argtypes = [_f32p, _i32p, _sz, _sz, _u8p, _u8p, ctypes.c_float,
                                            _f32p, _sz, _sz, _f32p, ctypes.c_int]
    l.nml_oracle_expert_down.restype = None
    l.nml_oracle_expert_down.argtypes = [_f32p, _i32p, _f32p, _sz, _u8p, _u8p, ctypes.c_float,
                                         _f32p, _sz, _sz, _f32p, ctypes.c_int]
    l.nml_oracle_exp_det.restype = ctypes.c_float
    l.nml_oracle_exp_det.argtypes = [ctypes.c_float]
    l.nml_oracle_route.restype = None
    l.nml_oracle_route.argtypes = [_f32p, _u8p, _sz, _sz, _sz, ctypes.c_int, _i32p, _f32p, _u16p]
    l.nml_oracle_assignment_plan.restype = ctypes.c_int32
    l.nml_oracle_assignment_plan.argtypes = [_i32p, _sz, _sz, _sz, _i32p, _i32p]
    l.nml_oracle_combine.restype = None
    l.nml_oracle_combine.argtypes = [_u16p, _sz, _sz, _sz, ctypes.c_int, ctypes.c_int, _u16p]
    l.nml_oracle_threads.restype = ctypes.c_int
    l.nml_oracle_set_avx2.argtypes = [ctypes.c_int]
    l.nml_oracle_set_threads.argtypes = [ctypes.c_int]


def _c(array: np.ndarray, dtype) -> np.ndarray:
    return np.ascontiguousarray(array, dtype=dtype)


def _p(array: np.ndarray | None, ptype):
    if array is None:
        return ctypes.cast(None, ptype)
    return array.ctypes.data_as(ptype)


# ----------------------------------------------------------------- codec

def decode_e2m1(code: int) -> float:
    return float(lib().nml_oracle_decode_e2m1(code & 0xFF))


def decode_e4m3fn_scale(bits: int) -> float:
    """Raises ValueError for the byte patterns the reference rejects."""
    value = ctypes.c_float()
    if not lib().nml_oracle_decode_e4m3fn_scale(bits & 0xFF, ctypes.byref(value)):
        raise ValueError(f"invalid NVFP4 E4M3FN scale bits 0x{bits:02x}")
    return float(value.value)


def encode_e4m3fn_scale(value: float) -> int:
    return int(lib().nml_oracle_encode_e4m3fn_scale(value))


def encode_e2m1(value: float) -> int:
    return int(lib().nml_oracle_encode_e2m1(value))


def global_scale(values: np.ndarray) -> np.float32:
    v = _c(values, np.float32).ravel()
    return np.float32(lib().nml_oracle_global_scale(_p(v, _f32p), v.size))


def quantize_row(values: np.ndarray, g: float):
    v = _c(values, np.float32).ravel()
    payload = np.zeros((v.size + 1) // 2, np.uint8)
    scales = np.zeros((v.size + 15) // 16, np.uint8)
    lib().nml_oracle_quantize_row(_p(v, _f32p), v.size, np.float32(g), _p(payload, _u8p),
                                  _p(scales, _u8p))
    return payload, scales


def quantize_tensor(values: np.ndarray):
    """values [..., width] f32 -> (payload [..., ceil(w/2)], scales [..., ceil(w/16)], g)."""
    v = _c(values, np.float32)
    width = v.shape[-1]
    rows = v.size // width
    payload = np.zeros(v.shape[:-1] + ((width + 1) // 2,), np.uint8)
    scales = np.zeros(v.shape[:-1] + ((width + 15) // 16,), np.uint8)
    g = lib().nml_oracle_quantize_tensor(_p(v, _f32p), rows, width, _p(payload, _u8p),
                                         _p(scales, _u8p))
    return payload, scales, np.float32(g)


def dequantize_row(payload, scales, g, width) -> np.ndarray:
    payload = _c(payload, np.uint8).ravel()
    scales = _c(scales, np.uint8).ravel()
    if payload.size != (width + 1) // 2 or scales.size != (width + 15) // 16:
        raise ValueError("invalid encoded extent")
    out = np.zeros(width, np.float32)
    code = lib().nml_oracle_dequantize_row(_p(payload, _u8p), _p(scales, _u8p), np.float32(g),
                                           width, _p(out, _f32p))
    if code:
        raise ValueError({1: "invalid global scale", 2: "nonzero padding",
                          3: "invalid scale byte", 4: "zero scale with nonzero value"}[code])
    return out


def validate_weight(payload, scales, g, rows, width) -> int:
    payload = _c(payload, np.uint8)
    scales = _c(scales, np.uint8)
    return int(lib().nml_oracle_validate_weight(_p(payload, _u8p), _p(scales, _u8p),
                                                np.float32(g), rows, width))


def dequantize_tensor(payload, scales, g, width) -> np.ndarray:
    """Full dense f32 decode of a [..., width] tensor (used for secondary checks only)."""
    payload = _c(payload, np.uint8)
    scales = _c(scales, np.uint8)
    lead = payload.shape[:-1]
    rows = int(np.prod(lead)) if lead else 1
    idx = np.arange(rows, dtype=np.int64)
    return embedding(idx, payload.reshape(rows, -1), scales.reshape(rows, -1), g, width).reshape(
        lead + (width,))


# ------------------------------------------------------- 16-bit floating

def to_f32(bits: np.ndarray, dtype: int) -> np.ndarray:
    b = _c(bits, np.uint16)
    out = np.zeros(b.shape, np.float32)
    lib().nml_oracle_to_f32(_p(b, _u16p), b.size, dtype, _p(out, _f32p))
    return out


def from_f32(values: np.ndarray, dtype: int) -> np.ndarray:
    v = _c(values, np.float32)
    out = np.zeros(v.shape, np.uint16)
    lib().nml_oracle_from_f32(_p(v, _f32p), v.size, dtype, _p(out, _u16p))
    return out


# --------------------------------------------------------------- kernels

def embedding(indices, payload, scales, g, width) -> np.ndarray:
    """f32 rows before narrowing.  Raises IndexError like the reference CPU path."""
    idx = _c(indices, np.int64).ravel()
    payload = _c(payload, np.uint8)
    scales = _c(scales, np.uint8)
    vocabulary = payload.shape[0]
    out = np.zeros((idx.size, width), np.float32)
    bad = lib().nml_oracle_embedding(_p(idx, _i64p), idx.size, _p(payload, _u8p),
                                     _p(scales, _u8p), np.float32(g), vocabulary, width,
                                     _p(out, _f32p))
    if bad:
        raise IndexError(f"embedding index {idx[bad - 1]} is outside vocabulary extent {vocabulary}")
    return out


def linear(x, payload, scales, g, bias=None, mode: int = 0) -> np.ndarray:
    """x [rows, K] f32 -> [rows, N] f32 (mode 0: reference f32 order, 1: f64 accumulate)."""
    x = _c(x, np.float32)
    payload = _c(payload, np.uint8)
    scales = _c(scales, np.uint8)
    rows, inputs = x.shape
    outputs = payload.shape[0]
    b = None if bias is None else _c(bias, np.float32)
    out = np.zeros((rows, outputs), np.float32)
    lib().nml_oracle_linear(_p(x, _f32p), rows, _p(payload, _u8p), _p(scales, _u8p),
                            np.float32(g), outputs, inputs, _p(b, _f32p), _p(out, _f32p), mode)
    return out


def linear_16(x_bits, payload, scales, g, dtype, bias_bits=None, mode: int = 0):
    """The CPU handler path: returns (narrowed bits [rows, N], f32 before narrowing)."""
    x = _c(x_bits, np.uint16)
    payload = _c(payload, np.uint8)
    scales = _c(scales, np.uint8)
    rows, inputs = x.shape
    outputs = payload.shape[0]
    b = None if bias_bits is None else _c(bias_bits, np.uint16)
    out16 = np.zeros((rows, outputs), np.uint16)
    out32 = np.zeros((rows, outputs), np.float32)
    lib().nml_oracle_linear_16(_p(x, _u16p), rows, _p(payload, _u8p), _p(scales, _u8p),
                               np.float32(g), outputs, inputs, _p(b, _u16p), dtype,
                               _p(out16, _u16p), _p(out32, _f32p), mode)
    return out16, out32


def grouped_projection(x, expert_indices, payload, scales, g, bias=None, mode: int = 0):
    x = _c(x, np.float32)
    e = _c(expert_indices, np.int64).ravel()
    payload = _c(payload, np.uint8)
    scales = _c(scales, np.uint8)
    experts, outputs = payload.shape[0], payload.shape[1]
    inputs = x.shape[1]
    b = None if bias is None else _c(bias, np.float32)
    out = np.zeros((e.size, outputs), np.float32)
    bad = lib().nml_oracle_grouped_projection(_p(x, _f32p), _p(e, _i64p), e.size,
                                              _p(payload, _u8p), _p(scales, _u8p), np.float32(g),
                                              experts, outputs, inputs, _p(b, _f32p),
                                              _p(out, _f32p), mode)
    if bad:
        raise IndexError(f"expert index {e[bad - 1]} is outside expert count {experts}")
    return out


def routed_clamped_swiglu(hidden, router_indices, routing_weights, gate, gate_bias, down,
                          down_bias, mode: int = 0) -> np.ndarray:
    """gate/down are (payload, scales, g) triples; returns [tokens, H] f32."""
    hidden = _c(hidden, np.float32)
    tokens, hidden_size = hidden.shape
    idx = _c(router_indices, np.int64).reshape(tokens, -1)
    top_k = idx.shape[1]
    w = _c(routing_weights, np.float32).reshape(tokens, top_k)
    gp, gs, gg = _c(gate[0], np.uint8), _c(gate[1], np.uint8), np.float32(gate[2])
    dp, ds, dg = _c(down[0], np.uint8), _c(down[1], np.uint8), np.float32(down[2])
    experts, doubled = gp.shape[0], gp.shape[1]
    intermediate = doubled // 2
    gb = _c(gate_bias, np.float32)
    db = _c(down_bias, np.float32)
    out = np.zeros((tokens, hidden_size), np.float32)
    bad = lib().nml_oracle_routed_clamped_swiglu(
        _p(hidden, _f32p), tokens, _p(idx, _i64p), _p(w, _f32p), top_k, _p(gp, _u8p),
        _p(gs, _u8p), gg, _p(gb, _f32p), _p(dp, _u8p), _p(ds, _u8p), dg, _p(db, _f32p), experts,
        hidden_size, intermediate, _p(out, _f32p), mode)
    if bad:
        raise IndexError(f"expert index {idx.ravel()[bad - 1]} is outside expert count {experts}")
    return out


def expert_gate_up(hidden, expert_ids, top_k, gate, gate_bias, mode: int = 0) -> np.ndarray:
    """activated [A, I] f32 before narrowing; rows of masked (-1) routes stay zero."""
    hidden = _c(hidden, np.float32)
    ids = _c(expert_ids, np.int32).ravel()
    gp, gs, gg = _c(gate[0], np.uint8), _c(gate[1], np.uint8), np.float32(gate[2])
    intermediate = gp.shape[1] // 2
    gb = _c(gate_bias, np.float32)
    out = np.zeros((ids.size, intermediate), np.float32)
    lib().nml_oracle_expert_gate_up(_p(hidden, _f32p), _p(ids, _i32p), ids.size, top_k,
                                    _p(gp, _u8p), _p(gs, _u8p), gg, _p(gb, _f32p),
                                    hidden.shape[1], intermediate, _p(out, _f32p), mode)
    return out


def expert_down(activated, expert_ids, routing_weights, down, down_bias, mode: int = 0):
    """weighted [A, H] f32 before narrowing; rows of masked (-1) routes stay zero."""
    act = _c(activated, np.float32)
    ids = _c(expert_ids, np.int32).ravel()
    w = _c(routing_weights, np.float32).ravel()
    dp, ds, dg = _c(down[0], np.uint8), _c(down[1], np.uint8), np.float32(down[2])
    hidden_size = dp.shape[1]
    db = _c(down_bias, np.float32)
    out = np.zeros((ids.size, hidden_size), np.float32)
    lib().nml_oracle_expert_down(_p(act, _f32p), _p(ids, _i32p), _p(w, _f32p), ids.size,
                                 _p(dp, _u8p), _p(ds, _u8p), dg, _p(db, _f32p), hidden_size,
                                 act.shape[1], _p(out, _f32p), mode)
    return out


# --------------------------------------------------------------- routing

def exp_det(x: float) -> float:
    return float(lib().nml_oracle_exp_det(np.float32(x)))


def route(logits, top_k: int, dtype: int = BF16, active=None):
    """Returns (ids [T,k] i32, weights f32 [T,k], weights narrowed to dtype as bits [T,k])."""
    logits = _c(logits, np.float32)
    tokens, experts = logits.shape
    if top_k > 64:
        raise ValueError("oracle supports at most 64 routes per token")
    a = None if active is None else _c(active, np.uint8)
    ids = np.zeros((tokens, top_k), np.int32)
    w32 = np.zeros((tokens, top_k), np.float32)
    w16 = np.zeros((tokens, top_k), np.uint16)
    lib().nml_oracle_route(_p(logits, _f32p), _p(a, _u8p), tokens, experts, top_k, dtype,
                           _p(ids, _i32p), _p(w32, _f32p), _p(w16, _u16p))
    return ids, w32, w16


def plan_capacity(assignments: int, experts: int, block: int = 16):
    """(max_blocks, positions) of the assignment schedule."""
    nonempty = min(assignments, experts)
    max_blocks = (assignments + nonempty * (block - 1) + block - 1) // block
    return max_blocks, max_blocks * block


def assignment_plan(expert_ids, experts: int, block: int = 16):
    """Returns (sorted_assignments [positions], block_experts [max_blocks], active_blocks)."""
    ids = _c(expert_ids, np.int32).ravel()
    max_blocks, positions = plan_capacity(ids.size, experts, block)
    sorted_assignments = np.zeros(positions, np.int32)
    block_experts = np.zeros(max_blocks, np.int32)
    active = lib().nml_oracle_assignment_plan(_p(ids, _i32p), ids.size, experts, block,
                                              _p(sorted_assignments, _i32p),
                                              _p(block_experts, _i32p))
    return sorted_assignments, block_experts, int(active)


def combine(weighted_bits, tokens, top_k, dtype, mode: int = 0) -> np.ndarray:
    w = _c(weighted_bits, np.uint16).reshape(tokens * top_k, -1)
    hidden_size = w.shape[1]
    out = np.zeros((tokens, hidden_size), np.uint16)
    lib().nml_oracle_combine(_p(w, _u16p), tokens, top_k, hidden_size, dtype, mode,
                             _p(out, _u16p))
    return out


def set_avx2(enabled: bool) -> None:
    """Chooses between the AVX2 and the scalar evaluation of the dot product; both perform
    the same operations in the same order and return the same bits."""
    lib().nml_oracle_set_avx2(1 if enabled else 0)


def threads() -> int:
    return int(lib().nml_oracle_threads())


def set_threads(count: int) -> None:
    lib().nml_oracle_set_threads(int(count))


# ---------------------------------------------------------------- metrics

def error_metrics(actual: np.ndarray, expected: np.ndarray) -> dict:
    """Relative-error figures for a GEMM output against the f32 oracle output.

    Elementwise relative error is unbounded where the expected value is near
    zero, so the denominator is floored at 1% of the RMS of the expected
    tensor: err_i = |a_i - e_i| / max(|e_i|, 0.01 * rms(e)).  ``max_rel`` and
    ``mean_rel`` are the figures the parity tests bound (2e-2 and 2e-3).  Also
    reported: the reference's own mixed form |a-e| / (1 + |e|)
    (crates/nml/tests/nvfp4_contract.rs:528-531) and the norm-wise error.
    """
    a = np.asarray(actual, np.float64).ravel()
    e = np.asarray(expected, np.float64).ravel()
    rms = float(np.sqrt(np.mean(e * e))) if e.size else 0.0
    floor = max(0.01 * rms, 1e-30)
    rel = np.abs(a - e) / np.maximum(np.abs(e), floor)
    mixed = np.abs(a - e) / (1.0 + np.abs(e))
    norm = float(np.linalg.norm(a - e) / max(np.linalg.norm(e), 1e-30))
    return {"max_rel": float(rel.max()) if rel.size else 0.0,
            "mean_rel": float(rel.mean()) if rel.size else 0.0,
            "max_mixed": float(mixed.max()) if mixed.size else 0.0,
            "norm_rel": norm}
