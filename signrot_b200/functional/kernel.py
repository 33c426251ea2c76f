"""Kernel-level operators with the names, argument meaning and error behaviour of
`signrot.functional.kernel` (signrot/functional/kernel.py:15-227), implemented on the
C ABI of libsignrot_b200.so.

Outputs are allocated here (the reference allocates them in its pybind layer,
signrot/kernels/bindings.cpp:24,123-124,255) and handed to the library as raw device
pointers.  Every operator launches on PyTorch's current stream, performs no host
synchronisation and is therefore CUDA-graph capturable.

Additional fused operators that have no single counterpart in the reference are at the
bottom: `w4a4_linear`, `rotate_quant`, `hadamard`.
"""
from __future__ import annotations

import math

import torch

from .. import _lib
from .._lib import ptr, require_cuda, run

__all__ = [
    "ShapeHandler", "PackedQuantizedTensor",
    "matmul_si4_si4", "matmul_ui4_si4", "matmul_grouped",
    "sym_quant", "sym_quant_dynamic", "asym_quant_dynamic",
    "sym_quant_dynamic_moe", "asym_quant_dynamic_moe", "sym_dequant_moe",
    "kv_quant_pack", "rope_qk", "swiglu", "rmsnorm", "sym_dequant",
    "asym_quant_f16_si4", "asym_quant_f16_ui4", "sum_i4", "matmul_colrow_i8_i32",
    "w4a4_linear", "grouped_linear", "rotate_quant", "hadamard", "hadamard_heads",
    "add_rmsnorm_quant", "w4a4_swiglu", "rtn_pack", "moe_route", "moe_gather", "moe_combine",
]


class ShapeHandler:
    """Flattens every dimension but the last and restores it (kernel.py:15-29)."""

    def __init__(self, x: torch.Tensor):
        self.size_excl_last = x.numel() // x.shape[-1]
        self.shape_excl_last = tuple(x.shape[:-1])

    def flatten(self, x: torch.Tensor):
        return x.view(self.size_excl_last, -1)

    def unflatten(self, x: torch.Tensor):
        return x.view(self.shape_excl_last + (-1,))

    def unflatten_scale(self, x: torch.Tensor):
        return x.view(self.shape_excl_last)


class PackedQuantizedTensor:
    """Carrier of packed codes, per-token scales and optional zeros (kernel.py:32-52)."""

    def __init__(self, quantized_x: torch.Tensor, scales_x: torch.Tensor, zeros_x: torch.Tensor | None = None):
        self.quantized_x = quantized_x
        self.scales_x = scales_x
        self.zeros_x = zeros_x

    def size(self):
        return self.quantized_x.size()

    @property
    def device(self):
        return self.quantized_x.device

    @property
    def dtype(self):
        return self.quantized_x.dtype


def _rows(x: torch.Tensor):
    """(2-D view, leading shape)."""
    lead = x.shape[:-1]
    return x.view(-1, x.shape[-1]), lead


def _check_dtype(name, t, dtype):
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected {dtype}, got {t.dtype}")


# ---------------------------------------------------------------------------- GEMM

def _matmul(name, A, B, a_unsigned):
    assert A.shape[-1] % 32 == 0, "A.shape[-1]: {} must be multiplication of 32".format(A.shape[-1])
    A2, a_lead = _rows(A)
    B2, b_lead = _rows(B)
    dev = require_cuda(name, A2, B2)
    _check_dtype(name, A2, torch.uint8)
    _check_dtype(name, B2, torch.uint8)
    if A2.shape[1] != B2.shape[1]:
        raise RuntimeError(f"{name}: inner dimensions differ ({A2.shape[1]} vs {B2.shape[1]} packed bytes)")
    M, N, K = A2.shape[0], B2.shape[0], A2.shape[1] * 2
    C = torch.empty((M, N), dtype=torch.int32, device=dev)
    run(dev, "sr_matmul_i4", ptr(A2), ptr(B2), M, N, K, int(a_unsigned), ptr(C))
    return C.view(*a_lead, *b_lead)


def matmul_si4_cols(A, begin, end, B):
    """`matmul_si4_si4(A[:, begin:end], B)` on packed columns [begin, end) of a 2-D code matrix without copying the
    slice out (the K-slice product of a row-parallel linear).  begin and the row width must be multiples of 16 bytes."""
    dev = require_cuda("matmul", A, B)
    _check_dtype("matmul", A, torch.uint8)
    _check_dtype("matmul", B, torch.uint8)
    if A.dim() != 2 or B.dim() != 2 or B.shape[1] != end - begin or begin % 16 or A.shape[1] % 16 or (end - begin) % 32:
        raise RuntimeError(f"matmul: bad column range [{begin}, {end}) of a {tuple(A.shape)} code matrix")
    M, N = A.shape[0], B.shape[0]
    C = torch.empty((M, N), dtype=torch.int32, device=dev)
    run(dev, "sr_matmul_i4_ld", A.data_ptr() + begin, A.shape[1], ptr(B), M, N, 2 * (end - begin), 0, ptr(C))
    return C


def matmul_si4_si4(A, B):
    """int32 `unpack_i4(A) @ unpack_i4(B).T` (kernel.py:67-73)."""
    return _matmul("matmul", A, B, False)


def matmul_ui4_si4(A, B):
    """Same with unsigned activation codes (kernel.py:75-81)."""
    return _matmul("matmul_ui4_si4", A, B, True)


def matmul_grouped(problem_sizes, ptr_a, ptr_b, ptr_c, lda, ldb, ldc, signed_a=True, max_k=0):
    """Grouped 4-bit GEMM, C_i = A_i @ B_i^T for every problem in one launch; all metadata
    stays on the device (kernel.py:83-92).  `max_k` (optional) is an upper bound on k known
    to the caller; it only affects occupancy."""
    dev = require_cuda("matmul_grouped", problem_sizes, ptr_a, ptr_b, ptr_c, lda, ldb, ldc)
    if problem_sizes.dtype != torch.int32 or problem_sizes.dim() != 2 or problem_sizes.shape[1] != 3:
        raise RuntimeError("problem_sizes must be int32 [problem_count, 3] (m, n, k) rows")
    P = problem_sizes.shape[0]
    for t in (ptr_a, ptr_b, ptr_c, lda, ldb, ldc):
        if t.dtype != torch.int64 or t.numel() != P:
            raise RuntimeError("pointer/ld arrays must be int64 with one entry per problem")
    run(dev, "sr_matmul_grouped", ptr(problem_sizes), P, ptr(ptr_a), ptr(ptr_b), ptr(ptr_c), ptr(lda), ptr(ldb),
        ptr(ldc), int(bool(signed_a)), int(max_k))


# ---------------------------------------------------------------------------- quantizers

def sym_quant(x, scale):
    """Codes for a given per-row scale (kernel.py:94-98)."""
    assert x.dtype == scale.dtype == torch.float16
    x2, lead = _rows(x)
    scale = scale.view(-1)
    dev = require_cuda("sym_quant", x2, scale)
    if scale.numel() != x2.shape[0]:
        raise RuntimeError("sym_quant: scale must have one entry per row")
    q = torch.empty((x2.shape[0], (x2.shape[1] + 1) // 2), dtype=torch.uint8, device=dev)
    run(dev, "sr_sym_quant", ptr(x2), ptr(scale), x2.shape[0], x2.shape[1], ptr(q))
    return q.view(*lead, -1)


def sym_quant_dynamic(x, clip_ratio=1.0):
    """Per-row amax, scale and symmetric int4 codes in one launch (kernel.py:101-110).
    Returns (packed_q, scale) with scale shaped (*x.shape[:-1], 1)."""
    assert x.dtype == torch.float16
    x2, lead = _rows(x.contiguous())
    dev = require_cuda("sym_quant_dynamic", x2)
    rows, cols = x2.shape
    q = torch.empty((rows, (cols + 1) // 2), dtype=torch.uint8, device=dev)
    scale = torch.empty((rows, 1), dtype=torch.float16, device=dev)
    run(dev, "sr_sym_quant_dynamic", ptr(x2), rows, cols, float(clip_ratio), ptr(q), ptr(scale))
    return q.view(*lead, -1), scale.view(*lead, 1)


def asym_quant_dynamic(x, clip_ratio=1.0):
    """Per-row min/max, scale, zero and unsigned codes in one launch (kernel.py:113-120)."""
    assert x.dtype == torch.float16
    x2, lead = _rows(x.contiguous())
    dev = require_cuda("asym_quant_dynamic", x2)
    rows, cols = x2.shape
    q = torch.empty((rows, (cols + 1) // 2), dtype=torch.uint8, device=dev)
    scale = torch.empty((rows, 1), dtype=torch.float16, device=dev)
    zero = torch.empty((rows, 1), dtype=torch.float16, device=dev)
    run(dev, "sr_asym_quant_dynamic", ptr(x2), rows, cols, float(clip_ratio), ptr(q), ptr(scale), ptr(zero))
    return q.view(*lead, -1), scale.view(*lead, 1), zero.view(*lead, 1)


def _moe_args(name, x, sign, expert_ids):
    if x.dim() != 2 or x.dtype != torch.float16:
        raise RuntimeError(f"{name} expects a 2D fp16 [rows, cols] tensor")
    dev = require_cuda(name, x, sign, expert_ids)
    if expert_ids.dtype != torch.int32 or expert_ids.numel() != x.shape[0]:
        raise RuntimeError("expert_ids must be int32 with one entry per row")
    if sign is not None and (sign.dtype != torch.int8 or sign.dim() != 2 or sign.shape[1] != x.shape[1]):
        raise RuntimeError(f"{name}: sign must be int8 [num_experts, cols]")
    return dev


def sym_quant_dynamic_moe(x, sign, expert_ids, clip_ratio=1.0):
    """`sym_quant_dynamic` on rows multiplied by sign[expert_ids[r]] (kernel.py:123-128)."""
    assert x.dtype == torch.float16
    x = x.contiguous()
    dev = _moe_args("sym_quant_dynamic_moe", x, sign, expert_ids)
    rows, cols = x.shape
    q = torch.empty((rows, (cols + 1) // 2), dtype=torch.uint8, device=dev)
    scale = torch.empty((rows, 1), dtype=torch.float16, device=dev)
    run(dev, "sr_sym_quant_dynamic_moe", ptr(x), ptr(sign), ptr(expert_ids), rows, cols, float(clip_ratio), ptr(q),
        ptr(scale))
    return q, scale


def asym_quant_dynamic_moe(x, sign, expert_ids, clip_ratio=1.0):
    """Asymmetric variant of `sym_quant_dynamic_moe` -> (q, scale, zero) (kernel.py:131-134)."""
    assert x.dtype == torch.float16
    x = x.contiguous()
    dev = _moe_args("asym_quant_dynamic_moe", x, sign, expert_ids)
    rows, cols = x.shape
    q = torch.empty((rows, (cols + 1) // 2), dtype=torch.uint8, device=dev)
    scale = torch.empty((rows, 1), dtype=torch.float16, device=dev)
    zero = torch.empty((rows, 1), dtype=torch.float16, device=dev)
    run(dev, "sr_asym_quant_dynamic_moe", ptr(x), ptr(sign), ptr(expert_ids), rows, cols, float(clip_ratio), ptr(q),
        ptr(scale), ptr(zero))
    return q, scale, zero


def sym_dequant_moe(q, scale_row, w_scales, expert_ids, zero_row=None, w_sum=None):
    """out[r, c] = (q[r, c] - zero_row[r] * w_sum[e, c]) * scale_row[r] * w_scales[e, c],
    e = expert_ids[r] (kernel.py:137-145)."""
    assert q.dtype == torch.int32
    scale_row = scale_row.contiguous()
    dev = require_cuda("sym_dequant_moe", q, scale_row, w_scales, expert_ids, zero_row, w_sum)
    if q.dim() != 2:
        raise RuntimeError("q must be int32 [rows, cols]")
    rows, cols = q.shape
    if scale_row.dtype != torch.float16 or scale_row.numel() != rows:
        raise RuntimeError("scale_row must be fp16 with one entry per row")
    if w_scales.dtype != torch.float16 or w_scales.dim() != 2 or w_scales.shape[1] != cols:
        raise RuntimeError("w_scales must be fp16 [num_experts, cols]")
    if expert_ids.dtype != torch.int32 or expert_ids.numel() != rows:
        raise RuntimeError("expert_ids must be int32 with one entry per row")
    if (zero_row is None) != (w_sum is None):
        raise RuntimeError("zero_row and w_sum must be given together")
    if zero_row is not None:
        if zero_row.dtype != torch.int8 or zero_row.numel() != rows:
            raise RuntimeError("zero_row must be int8 with one entry per row")
        if w_sum.dtype != torch.int32 or w_sum.dim() != 2 or w_sum.shape != w_scales.shape:
            raise RuntimeError("w_sum must be int32 [num_experts, cols]")
    out = torch.empty((rows, cols), dtype=torch.float16, device=dev)
    run(dev, "sr_sym_dequant_moe", ptr(q), ptr(scale_row), ptr(w_scales), ptr(expert_ids), ptr(zero_row), ptr(w_sum),
        rows, cols, ptr(out))
    return out


def kv_quant_pack(x):
    """KV-cache asymmetric uint4 quantize + pack; returns (packed_q, param) with
    param[..., 0] the scale and param[..., 1] the zero point (kernel.py:148-155)."""
    assert x.dtype == torch.float16
    x = x.contiguous()
    dev = require_cuda("kv_quant_pack", x)
    cols = x.shape[-1]
    if cols % 2:
        raise RuntimeError("kv_quant_pack expects an even last dimension")
    rows = x.numel() // cols if cols else 0
    q = torch.empty((*x.shape[:-1], cols // 2), dtype=torch.uint8, device=dev)
    param = torch.empty((*x.shape[:-1], 2), dtype=torch.float16, device=dev)
    run(dev, "sr_kv_quant_pack", ptr(x), rows, cols, ptr(q), ptr(param))
    return q, param


def rope_qk(q, k, cos, sin):
    """In-place rotary embedding for q [B,T,Hq,D] and k [B,T,Hk,D] (kernel.py:158-166)."""
    cos, sin = cos.contiguous(), sin.contiguous()
    dev = require_cuda("rope_qk", q, k, cos, sin)
    if q.dim() != 4 or k.dim() != 4:
        raise RuntimeError("rope_qk expects [B, T, H, D] q/k")
    if cos.dim() != 3:
        raise RuntimeError("rope_qk expects [B or 1, T, D] cos/sin")
    if cos.shape != sin.shape:
        raise RuntimeError("cos and sin must have the same shape")
    if q.dtype != torch.float16 or k.dtype != torch.float16:
        raise RuntimeError("rope_qk expects fp16 q/k")
    if cos.dtype != torch.float16:
        raise RuntimeError("rope_qk expects fp16 cos/sin")
    if k.shape[0] != q.shape[0] or k.shape[1] != q.shape[1] or k.shape[3] != q.shape[3]:
        raise RuntimeError("q and k must agree on batch, sequence and head_dim")
    if cos.shape[1] != q.shape[1] or cos.shape[2] != q.shape[3]:
        raise RuntimeError("cos/sin must be [B or 1, T, head_dim]")
    run(dev, "sr_rope_qk", ptr(q), ptr(k), ptr(cos), ptr(sin), q.shape[0], q.shape[1], cos.shape[0], q.shape[2],
        k.shape[2], q.shape[3])
    return q, k


def swiglu(gate, up):
    """silu(gate) * up with the reference's two fp16 roundings (kernel.py:169-171)."""
    gate, up = gate.contiguous(), up.contiguous()
    dev = require_cuda("swiglu", gate, up)
    if gate.shape != up.shape:
        raise RuntimeError("gate and up must have the same shape")
    if gate.dtype != torch.float16:
        raise RuntimeError("swiglu expects fp16 input")
    out = torch.empty_like(gate)
    run(dev, "sr_swiglu", ptr(gate), ptr(up), gate.numel(), ptr(out))
    return out


def rmsnorm(x, eps, mean_dim):
    """RMSNorm over the last dimension, fp32 accumulation, fp16 in/out (kernel.py:174-176)."""
    assert x.dtype == torch.float16
    x = x.contiguous()
    dev = require_cuda("rmsnorm", x)
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    out = torch.empty_like(x)
    run(dev, "sr_rmsnorm", ptr(x), rows, cols, float(eps), int(mean_dim), ptr(out))
    return out


def add_rmsnorm_quant(x, delta, eps, mean_dim, clip_ratio=1.0, asym=False, return_normed=False):
    """Residual add -> RMSNorm -> per-token int4 quantizer in one launch: what a decoder layer does
    between a branch's output projection and the next quantized projections (`hidden + branch`,
    signrot.nn.RMSNorm, signrot.nn.Quantizer / AsymQuantizer), with the same rounding points.
    `delta` may be None.  Returns (x + delta or x itself, PackedQuantizedTensor[, normalised row])."""
    if x.dtype != torch.float16 or (delta is not None and delta.dtype != torch.float16):
        raise RuntimeError("add_rmsnorm_quant expects fp16 input")
    x = x.contiguous()
    if delta is not None:
        delta = delta.contiguous()
        if delta.shape != x.shape:
            raise RuntimeError("x and delta must have the same shape")
    dev = require_cuda("add_rmsnorm_quant", x, delta)
    x2, lead = _rows(x)
    rows, cols = x2.shape
    q = torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev)
    scale = torch.empty((rows, 1), dtype=torch.float16, device=dev)
    zero = torch.empty((rows, 1), dtype=torch.float16, device=dev) if asym else None
    total = torch.empty_like(x) if delta is not None else None
    normed = torch.empty_like(x) if return_normed else None
    run(dev, "sr_add_rmsnorm_quant", ptr(x), ptr(delta), rows, cols, float(eps), int(mean_dim), float(clip_ratio),
        int(bool(asym)), ptr(total), ptr(normed), ptr(q), ptr(scale), ptr(zero))
    packed = PackedQuantizedTensor(q.view(*lead, -1), scale.view(*lead, 1),
                                   zero.view(*lead, 1).to(torch.int8) if asym else None)
    out = (total if delta is not None else x, packed)
    return out + (normed,) if return_normed else out


def sym_dequant(q, scale_row, scale_col, bits=32):
    """fp16 `q * scale_row * scale_col` from int32 accumulators (kernel.py:179-185)."""
    assert q.dtype == torch.int32
    assert scale_row.dtype == scale_col.dtype == torch.float16
    if bits != 32:
        raise RuntimeError("Unsupported data type")
    q2, lead = _rows(q)
    scale_row = scale_row.view(-1)
    dev = require_cuda("sym_dequant", q2, scale_row, scale_col)
    rows, cols = q2.shape
    if scale_row.numel() != rows or scale_col.numel() != cols:
        raise RuntimeError("sym_dequant: scale_row / scale_col do not match q")
    out = torch.empty((rows, cols), dtype=torch.float16, device=dev)
    run(dev, "sr_sym_dequant", ptr(q2), ptr(scale_row), ptr(scale_col), rows, cols, ptr(out))
    return out.view(*lead, -1)


def _asym_given(name, entry, q, scale, zero):
    assert q.dtype == torch.float16
    assert scale.dtype == zero.dtype == torch.float16
    x2, lead = _rows(q)
    scale, zero = scale.view(-1), zero.view(-1)
    dev = require_cuda(name, x2, scale, zero)
    rows, cols = x2.shape
    if scale.numel() != rows or zero.numel() != rows:
        raise RuntimeError(f"{name}: scale / zero must have one entry per row")
    out = torch.empty((rows, (cols + 1) // 2), dtype=torch.uint8, device=dev)
    run(dev, entry, ptr(x2), ptr(scale), ptr(zero), rows, cols, ptr(out))
    return out.view(*lead, -1)


def asym_quant_f16_si4(q, scale, zero):
    """clamp(rint(x/scale) + zero, -8, 7), packed (kernel.py:188-194)."""
    return _asym_given("asym_quant_f16_si4", "sr_asym_quant_f16_si4", q, scale, zero)


def asym_quant_f16_ui4(q, scale, zero):
    """clamp(rint(x/scale) + zero, 0, 15), packed (kernel.py:197-203)."""
    return _asym_given("asym_quant_f16_ui4", "sr_asym_quant_f16_ui4", q, scale, zero)


def sum_i4(x, is_signed=True, dtype=torch.int32) -> torch.Tensor:
    """Row sums of packed 4-bit values (kernel.py:206-212)."""
    assert x.dtype == torch.uint8, "packed int4 tensor must be torch.uint8"
    x2, lead = _rows(x)
    dev = require_cuda("sum_i4", x2)
    out = torch.empty((x2.shape[0], 1), dtype=torch.int32, device=dev)
    run(dev, "sr_sum_i4", ptr(x2), x2.shape[0], x2.shape[1], int(bool(is_signed)), ptr(out))
    out = out.view(*lead, 1)
    if dtype is not None and out.dtype != dtype:
        out = out.to(dtype=dtype)
    return out


def matmul_colrow_i8_i32(a_col, b_row) -> torch.Tensor:
    """Rank-1 int32 product a_col [.., 1] (int8) times b_row [1, C] (int32) (kernel.py:215-227)."""
    assert a_col.dtype == torch.int8, "a_col must be torch.int8"
    assert b_row.dtype == torch.int32, "b_row must be torch.int32"
    a2, lead = _rows(a_col)
    assert a2.shape[1] == 1, "a_col must have last dimension == 1"
    if b_row.dim() == 1:
        b_row = b_row.view(1, -1)
    assert b_row.dim() == 2 and b_row.shape[0] == 1, "b_row must have shape [1, C]"
    dev = require_cuda("matmul_colrow_i8_i32", a2, b_row)
    out = torch.empty((a2.shape[0], b_row.shape[1]), dtype=torch.int32, device=dev)
    run(dev, "sr_matmul_colrow_i8_i32", ptr(a2), ptr(b_row), a2.shape[0], b_row.shape[1], ptr(out))
    return out.view(*lead, b_row.shape[1])


# ---------------------------------------------------------------------------- fused operators

def grouped_linear(packed: PackedQuantizedTensor, expert_ids, row_offsets, weight, weight_scales, weight_sum=None,
                   expected_rows=0):
    """fp16 `dequant(packed[r] @ weight[e_r].T)` for expert-sorted rows in ONE launch: the grouped
    GEMM plus expert-indexed dequant of the sparse MoE block (signrot/nn/moe.py:114-162,
    functional/kernel.py:83-110 + 146-159).  `packed` rows sorted by expert, `expert_ids` int32
    [rows], `row_offsets` int32 [E + 1] (first row of every expert, last entry = rows), `weight`
    uint8 [E, N, K/2], `weight_scales` fp16 [E, N], `weight_sum` int32 [E, N] when `packed.zeros_x` is set."""
    qx, sx, zx = packed.quantized_x, packed.scales_x, packed.zeros_x
    assert qx.dim() == 2 and weight.dim() == 3
    assert qx.shape[-1] % 16 == 0, "A.shape[-1]: {} must be multiplication of 32".format(qx.shape[-1] * 2)
    sx = sx.reshape(-1)
    E, N = weight.shape[0], weight.shape[1]
    rows, K = qx.shape[0], qx.shape[1] * 2
    if zx is not None:
        zx = zx.reshape(-1)
        if weight_sum is None:
            raise RuntimeError("grouped_linear: asymmetric activations need weight_sum")
    dev = require_cuda("grouped_linear", qx, sx, zx, expert_ids, row_offsets, weight, weight_scales,
                       weight_sum if zx is not None else None)
    _check_dtype("grouped_linear", qx, torch.uint8)
    _check_dtype("grouped_linear", weight, torch.uint8)
    _check_dtype("grouped_linear", sx, torch.float16)
    _check_dtype("grouped_linear", weight_scales, torch.float16)
    _check_dtype("grouped_linear", expert_ids, torch.int32)
    _check_dtype("grouped_linear", row_offsets, torch.int32)
    if weight.shape[2] != qx.shape[1] or weight_scales.numel() != E * N or sx.numel() != rows \
            or expert_ids.numel() != rows or row_offsets.numel() != E + 1:
        raise RuntimeError("grouped_linear: shapes of activations, weights, scales and offsets do not match")
    if not (qx.is_contiguous() and weight.is_contiguous() and weight_scales.is_contiguous()):
        raise RuntimeError("grouped_linear: operands must be contiguous")
    if zx is not None:
        _check_dtype("grouped_linear", zx, torch.int8)
        _check_dtype("grouped_linear", weight_sum, torch.int32)
    out = torch.empty((rows, N), dtype=torch.float16, device=dev)
    run(dev, "sr_grouped_linear", ptr(qx), ptr(sx), ptr(zx), ptr(expert_ids), ptr(row_offsets), ptr(weight),
        ptr(weight_scales), ptr(weight_sum) if zx is not None else None, rows, E, N, K, int(expected_rows), ptr(out))
    return out


_WS_BYTES = {}          # (M, N, K) -> bytes of split-K scratch the tensor-core GEMM wants for this shape (0: none)
_SPLIT_COUNTERS = {}    # (device index, stream) -> the zeroed, self-resetting counters of that stream's split-K launches


def _splitk_scratch(dev, M, N, K):
    """(workspace, bytes, counters) for `sr_w4a4_linear_ws`, or (None, 0, None) when the shape does not split K.
    The workspace comes from the caching allocator per call; the counters are one small buffer per stream."""
    import ctypes
    key = (M, N, K)
    need = _WS_BYTES.get(key)
    if need is None:
        out = ctypes.c_int64(0)
        from .._lib import call_nostream
        call_nostream("sr_w4a4_linear_ws_bytes", M, N, K, ctypes.byref(out))
        need = _WS_BYTES[key] = int(out.value)
    if need == 0:
        return None, 0, None
    ckey = (dev.index if dev.index is not None else torch.cuda.current_device(), torch.cuda.current_stream(dev).cuda_stream)
    cnt = _SPLIT_COUNTERS.get(ckey)
    if cnt is None:
        if torch.cuda.is_current_stream_capturing():
            return None, 0, None        # first use inside a capture: no zero-fill there; this call runs unsplit
        cnt = _SPLIT_COUNTERS[ckey] = torch.zeros(1024, dtype=torch.int32, device=dev)
    return torch.empty(need, dtype=torch.uint8, device=dev), need, cnt


def w4a4_linear(packed: PackedQuantizedTensor, weight, weight_scales, weight_sum=None, bias=None):
    """fp16 `dequant(packed @ weight.T) (+ bias)`: the GEMM, the asymmetric zero correction
    and the dequant of `Linear4bit.forward` (signrot/nn/linear.py:36-50) in one kernel.
    `weight` uint8 [N, K/2], `weight_scales` fp16 [N] or [N, 1], `weight_sum` int32 [N] or
    [N, 1] (needed when `packed.zeros_x` is set)."""
    qx, sx, zx = packed.quantized_x, packed.scales_x, packed.zeros_x
    assert qx.shape[-1] % 16 == 0, "A.shape[-1]: {} must be multiplication of 32".format(qx.shape[-1] * 2)
    q2, lead = _rows(qx)
    sx = sx.reshape(-1)
    ws = weight_scales.reshape(-1)
    if zx is not None:
        zx = zx.reshape(-1)
        if weight_sum is None:
            raise RuntimeError("w4a4_linear: asymmetric activations need weight_sum")
        weight_sum = weight_sum.reshape(-1)
    dev = require_cuda("w4a4_linear", q2, sx, zx, weight, ws, weight_sum if zx is not None else None, bias)
    _check_dtype("w4a4_linear", q2, torch.uint8)
    _check_dtype("w4a4_linear", weight, torch.uint8)
    _check_dtype("w4a4_linear", sx, torch.float16)
    _check_dtype("w4a4_linear", ws, torch.float16)
    M, N, K = q2.shape[0], weight.shape[0], q2.shape[1] * 2
    if weight.shape[1] != q2.shape[1] or ws.numel() != N or sx.numel() != M:
        raise RuntimeError("w4a4_linear: shapes of activations, weight and scales do not match")
    if zx is not None:
        _check_dtype("w4a4_linear", zx, torch.int8)
        _check_dtype("w4a4_linear", weight_sum, torch.int32)
    if bias is not None:
        _check_dtype("w4a4_linear", bias, torch.float16)
    out = torch.empty((M, N), dtype=torch.float16, device=dev)
    scratch, scratch_bytes, counters = _splitk_scratch(dev, M, N, K)
    if scratch is not None:
        # few output tiles for the GPU (e.g. 256 rows against a 4096-wide weight): K split over CTA pairs, same bits
        run(dev, "sr_w4a4_linear_ws", ptr(q2), ptr(sx), ptr(zx), ptr(weight), ptr(ws),
            ptr(weight_sum) if zx is not None else None, ptr(bias), M, N, K, ptr(out), ptr(scratch), scratch_bytes,
            ptr(counters))
        return out.view(*lead, N)
    run(dev, "sr_w4a4_linear", ptr(q2), ptr(sx), ptr(zx), ptr(weight), ptr(ws),
        ptr(weight_sum) if zx is not None else None, ptr(bias), M, N, K, ptr(out))
    return out.view(*lead, N)


def w4a4_swiglu(packed: PackedQuantizedTensor, weight, weight_scales, weight_sum=None, bias=None):
    """gate_proj, up_proj and SwiGLU of an MLP in one launch for up to 32 rows.  `weight` is
    [2N, K/2]: the gate rows followed by the up rows (scales, sums and bias likewise).  Same bits
    as `swiglu(w4a4_linear(gate half), w4a4_linear(up half))`; larger batches take exactly that
    route here."""
    qx, sx, zx = packed.quantized_x, packed.scales_x, packed.zeros_x
    qx = qx.contiguous()
    q2, lead = _rows(qx)
    M, N2, K = q2.shape[0], weight.shape[0], q2.shape[1] * 2
    N = N2 // 2
    if N2 % 2 or weight.shape[1] != q2.shape[1] or weight_scales.numel() != N2 or sx.numel() != M:
        raise RuntimeError("w4a4_swiglu: shapes of activations, weight and scales do not match")
    if M > 32:
        ws = weight_scales.reshape(-1)
        wsum = weight_sum.reshape(-1) if weight_sum is not None else None
        half = lambda t, a: None if t is None else t[a * N:(a + 1) * N]
        gate = w4a4_linear(packed, weight[:N], ws[:N], half(wsum, 0), half(bias, 0))
        up = w4a4_linear(packed, weight[N:], ws[N:], half(wsum, 1), half(bias, 1))
        return swiglu(gate, up)
    sx = sx.reshape(-1)
    ws = weight_scales.reshape(-1)
    if zx is not None:
        zx = zx.reshape(-1)
        if weight_sum is None:
            raise RuntimeError("w4a4_swiglu: asymmetric activations need weight_sum")
        weight_sum = weight_sum.reshape(-1)
    dev = require_cuda("w4a4_swiglu", q2, sx, zx, weight, ws, weight_sum if zx is not None else None, bias)
    for name, t, dt in (("codes", q2, torch.uint8), ("weight", weight, torch.uint8), ("scales", sx, torch.float16),
                        ("weight scales", ws, torch.float16)):
        _check_dtype("w4a4_swiglu", t, dt)
    if not weight.is_contiguous():
        raise RuntimeError("w4a4_swiglu: weight must be contiguous")
    out = torch.empty((M, N), dtype=torch.float16, device=dev)
    run(dev, "sr_w4a4_swiglu", ptr(q2), ptr(sx), ptr(zx), ptr(weight), ptr(ws),
        ptr(weight_sum) if zx is not None else None, ptr(bias), M, N, K, ptr(out))
    return out.view(*lead, N)


def moe_route(router_logits, top_k, renormalize=True):
    """Softmax (fp32), top-k, renormalisation and the sort of the routed rows by expert in one launch
    (signrot/nn/moe.py:159-190).  router_logits fp16 [T, E].  Returns (weights fp16 [T, k],
    chosen int32 [T, k], tok int32 [R], eid int32 [R], inv int32 [R], row_offsets int32 [E + 1])."""
    if router_logits.dtype != torch.float16 or router_logits.dim() != 2:
        raise RuntimeError("moe_route expects fp16 [tokens, experts] logits")
    logits = router_logits.contiguous()
    dev = require_cuda("moe_route", logits)
    T, E = logits.shape
    R = T * top_k
    weights = torch.empty((T, top_k), dtype=torch.float16, device=dev)
    chosen = torch.empty((T, top_k), dtype=torch.int32, device=dev)
    tok = torch.empty((R,), dtype=torch.int32, device=dev)
    eid = torch.empty((R,), dtype=torch.int32, device=dev)
    inv = torch.empty((R,), dtype=torch.int32, device=dev)
    row_off = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    run(dev, "sr_moe_route", ptr(logits), T, E, int(top_k), int(bool(renormalize)), ptr(weights), ptr(chosen),
        ptr(tok), ptr(eid), ptr(inv), ptr(row_off))
    return weights, chosen, tok, eid, inv, row_off


def moe_gather(packed: PackedQuantizedTensor, tok):
    """Per routed row a copy of its token's codes, scale and zero (moe.py:192-194)."""
    q, s, z = packed.quantized_x.contiguous(), packed.scales_x.contiguous(), packed.zeros_x
    if z is not None:
        z = z.contiguous()
    dev = require_cuda("moe_gather", q, s, z, tok)
    R = tok.numel()
    q_out = torch.empty((R, q.shape[-1]), dtype=torch.uint8, device=dev)
    s_out = torch.empty((R, 1), dtype=torch.float16, device=dev)
    z_out = torch.empty((R, 1), dtype=torch.int8, device=dev) if z is not None else None
    run(dev, "sr_moe_gather", ptr(q), ptr(s), ptr(z), ptr(tok), R, q.shape[-1], ptr(q_out), ptr(s_out), ptr(z_out))
    return PackedQuantizedTensor(q_out, s_out, z_out)


def moe_combine(y, weights, inv, row_range=None, out_fp32=False):
    """Un-permute and weighted sum of the expert outputs (moe.py:231-235): y fp16 [R, hidden] in
    sorted row order, weights fp16 [T, k], inv int32 [T * k] -> fp16 [T, hidden].  `row_range`
    (int32 [2] on the device): only sorted rows lo <= r < hi count; `out_fp32`: the unrounded fp32
    sum (for a sum across expert-parallel ranks)."""
    y = y.contiguous()
    dev = require_cuda("moe_combine", y, weights, inv, row_range)
    T, k = weights.shape
    out = torch.empty((T, y.shape[-1]), dtype=torch.float32 if out_fp32 else torch.float16, device=dev)
    run(dev, "sr_moe_combine", ptr(y), ptr(weights), ptr(inv), ptr(row_range), T, k, y.shape[-1], int(bool(out_fp32)),
        ptr(out))
    return out


def rtn_pack(weight, sign=None, mse=False):
    """Offline weight preparation on the GPU: per-channel symmetric int4 round-to-nearest of a
    float weight [N, K] with the SignRot sign unfolded before and refolded after (rtn_fwrd,
    fake_quant/gptq_utils.py:411-465), written as the packed codes and fp16 scales that
    `Linear4bit.from_float` (signrot/nn/linear.py:52-73) would store.  Returns
    (uint8 [N, K/2], fp16 [N, 1])."""
    if weight.dim() != 2 or weight.dtype not in _lib.DTYPE_TAG:
        raise RuntimeError("rtn_pack expects a 2-D fp16, bf16 or fp32 weight")
    weight = weight.contiguous()
    if sign is not None:
        sign = sign.to(device=weight.device, dtype=torch.int8).contiguous()
        if sign.numel() != weight.shape[1]:
            raise RuntimeError("rtn_pack: one sign per input channel")
    dev = require_cuda("rtn_pack", weight, sign)
    n, k = weight.shape
    packed = torch.empty((n, k // 2), dtype=torch.uint8, device=dev)
    scale = torch.empty((n, 1), dtype=torch.float16, device=dev)
    run(dev, "sr_rtn_pack", ptr(weight), _lib.DTYPE_TAG[weight.dtype], n, k, ptr(sign), int(bool(mse)), ptr(packed),
        ptr(scale))
    return packed, scale


def had_scale(n: int) -> float:
    """The scale the reference passes to the transform: 1/sqrt(n) evaluated in fp32
    (signrot/functional/hadamard.py:81)."""
    return float(1.0 / torch.tensor(n).sqrt())


_HADK_CACHE = {}


def _hadk_as(hadK, device, dtype):
    """`hadK` on `device` in `dtype`.  A table that already is there is passed through; any other is converted once
    and the copy kept: the rotation kernels are launched with programmatic dependent launch and read the table
    before they wait for the kernel in front of them, so it must not be the output of a cast enqueued just before."""
    if hadK.device == device and hadK.dtype == dtype and hadK.is_contiguous():
        return hadK
    key = (hadK.data_ptr(), hadK._version, tuple(hadK.shape), hadK.dtype, str(device), dtype)
    hit = _HADK_CACHE.get(key)
    if hit is None:
        if len(_HADK_CACHE) > 64:
            _HADK_CACHE.clear()
        hit = hadK.to(device=device, dtype=dtype).contiguous()
        if hit.is_cuda and not torch.cuda.is_current_stream_capturing():
            torch.cuda.current_stream(hit.device).synchronize()     # once per table: the copy is complete before any use
        _HADK_CACHE[key] = hit
    return hit


def hadamard(x, hadK=None, K=1, sign=None, fp32_mode=False, out_dtype=None, scale=None):
    """`matmul_hadU_cuda(x, hadK, K)` (signrot/functional/hadamard.py:78-87), optionally
    followed by the +-1 `sign` multiply and the cast of `OnlineHadamard.forward`
    (signrot/nn/hadamard.py:26-42), in one launch.  Output dtype defaults to x.dtype."""
    x = x.contiguous()
    n = x.shape[-1]
    x2, lead = _rows(x)
    if x.dtype not in _lib.DTYPE_TAG:
        raise RuntimeError(f"hadamard: unsupported dtype {x.dtype}")
    out_dtype = out_dtype or x.dtype
    if K > 1:
        want = torch.float32 if (fp32_mode or x.dtype == torch.float32) else torch.float16
        hadK = _hadk_as(hadK, x.device, want)
    else:
        hadK = None
    dev = require_cuda("hadamard", x2, hadK, sign)
    out = torch.empty(x2.shape, dtype=out_dtype, device=dev)
    run(dev, "sr_hadamard", ptr(x2), _lib.DTYPE_TAG[x.dtype], x2.shape[0], n, ptr(hadK), int(K),
        had_scale(n) if scale is None else float(scale), ptr(sign),
        int(bool(fp32_mode) or x.dtype == torch.float32), ptr(out), _lib.DTYPE_TAG[out_dtype])
    return out.view(*lead, n)


def hadamard_heads(x, heads: int, fp32_mode=False):
    """(H_heads (x) I) / sqrt(heads) over the last dimension viewed as [heads, head_dim]: the
    o_proj input rotation (fake_quant/quant_utils.py:287-291) without transposes."""
    x = x.contiguous()
    n = x.shape[-1]
    x2, lead = _rows(x)
    dev = require_cuda("hadamard_heads", x2)
    out = torch.empty_like(x2)
    run(dev, "sr_hadamard_heads", ptr(x2), _lib.DTYPE_TAG[x.dtype], x2.shape[0], int(heads), n // heads,
        had_scale(heads), int(bool(fp32_mode)), ptr(out), _lib.DTYPE_TAG[x.dtype])
    return out.view(*lead, n)


def rotate_quant(x, hadK=None, K=1, sign=None, expert_ids=None, heads=0, clip_ratio=1.0, asym=False,
                 return_rotated=False):
    """Online rotation + sign + per-token int4 quantization in one pass over each row:
    `ActQuantWrapper.kernel_quantize` (fake_quant/quant_utils.py:278-292).  x is fp16 or
    bf16 (bf16 is rounded to fp16 first, as the reference's `x.to(torch.float16)`).
    Returns a PackedQuantizedTensor (zeros as int8 when asym), and the rotated fp16 rows
    when `return_rotated`."""
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("rotate_quant: activations must be fp16 or bf16")
    x = x.contiguous()
    n = x.shape[-1]
    x2, lead = _rows(x)
    if K > 1:
        hadK = _hadk_as(hadK, x.device, torch.float16)
    else:
        hadK = None
    dev = require_cuda("rotate_quant", x2, hadK, sign, expert_ids)
    rows = x2.shape[0]
    q = torch.empty((rows, n // 2), dtype=torch.uint8, device=dev)
    scale = torch.empty((rows, 1), dtype=torch.float16, device=dev)
    zero = torch.empty((rows, 1), dtype=torch.float16, device=dev) if asym else None
    rot = torch.empty((rows, n), dtype=torch.float16, device=dev) if return_rotated else None
    s = had_scale(heads) if heads else had_scale(n)
    run(dev, "sr_rotate_quant", ptr(x2), _lib.DTYPE_TAG[x.dtype], rows, n, ptr(hadK), int(K), s, ptr(sign),
        ptr(expert_ids), int(heads), float(clip_ratio), int(bool(asym)), ptr(q), ptr(scale), ptr(zero), ptr(rot))
    packed = PackedQuantizedTensor(q.view(*lead, -1), scale.view(*lead, 1),
                                   zero.view(*lead, 1).to(torch.int8) if asym else None)
    if return_rotated:
        return packed, rot.view(*lead, n)
    return packed
