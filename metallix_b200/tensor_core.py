"""The tcgen05 / TMEM / TMA matrix product (sm_100a), or the reason it is not
used for a given call."""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

STORE_BF16, STORE_F32, SWIGLU, RELU_SQUARED, GEGLU = 0, 1, 2, 3, 4


def why_not(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> str:
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return "operands must be bfloat16"
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        return "operands must be [m, k] and [n, k]"
    if a.stride(1) != 1 or w.stride(1) != 1:
        return "rows must be contiguous"
    if a.data_ptr() % 16 or w.data_ptr() % 16:
        return "operands must start on 16-byte boundaries"
    if not ops._fn("mxb_gemm_tcgen05_supported")(a.shape[0], w.shape[0], a.shape[1], a.stride(0), w.stride(0)):
        return "k and the row strides must be multiples of 8"
    if out_dtype not in (torch.bfloat16, torch.float32):
        return "the result must be bfloat16 or float32"
    return ""


def supports(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> bool:
    return why_not(a, w, out_dtype) == ""


def _launch(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, n: int, epilogue: int) -> torch.Tensor:
    ops._call("mxb_gemm_tcgen05", out.data_ptr(), a.data_ptr(), w.data_ptr(), a.shape[0], n, a.shape[1],
              a.stride(0), w.stride(0), out.stride(0), epilogue, ops.status_word(a.device).data_ptr(),
              ops._stream())
    return out


def gemm(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [m, k] times w [n, k] transposed on tcgen05 tensor cores."""
    reason = why_not(a, w, out_dtype)
    if reason:
        raise ops.KernelError("the tcgen05 kernel does not take this call: " + reason)
    m, n = a.shape[0], w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    ops._need(out.shape == (m, n) and out.dtype == out_dtype and out.stride(1) == 1, "out does not fit")
    return _launch(out, a, w, n, STORE_BF16 if out_dtype == torch.bfloat16 else STORE_F32)


def gemm_swiglu(a: torch.Tensor, gate_up: torch.Tensor, out: Optional[torch.Tensor] = None,
                activation: str = "silu") -> torch.Tensor:
    """act(a gate^T) * (a up^T) for gate_up = [gate rows; up rows], without
    gate and up ever reaching memory; act is silu or ("gelu_tanh") the tanh
    form of gelu. Returns bfloat16 [m, inter]."""
    reason = why_not(a, gate_up, torch.bfloat16)
    if reason:
        raise ops.KernelError("the tcgen05 kernel does not take this call: " + reason)
    ops._need(gate_up.shape[0] % 2 == 0, "gate and up rows must pair up")
    m, inter = a.shape[0], gate_up.shape[0] // 2
    if out is None:
        out = torch.empty((m, inter), dtype=torch.bfloat16, device=a.device)
    ops._need(out.shape == (m, inter) and out.dtype == torch.bfloat16 and out.stride(1) == 1, "out does not fit")
    return _launch(out, a, gate_up, inter, {"silu": SWIGLU, "gelu_tanh": GEGLU}[activation])


def gemm_grouped(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, groups: int, epilogue: int) -> torch.Tensor:
    """Row tile i of a ``[m, k]`` (128 rows a tile, m a whole number of them)
    times matrix tile_group[i] of w ``[groups * n, k]`` transposed; tiles with a
    negative entry are left out, and their rows of the result are not written.
    ``epilogue``: STORE_BF16, STORE_F32, RELU_SQUARED (bfloat16 max(c, 0)^2) or
    SWIGLU (every matrix of w holds its gate rows and then as many up rows;
    the result is bfloat16 silu(gate) * up, half as wide as a matrix has rows)."""
    reason = why_not(a, w, torch.bfloat16)
    if reason:
        raise ops.KernelError("the tcgen05 kernel does not take this call: " + reason)
    ops._need(w.shape[0] % groups == 0 and a.shape[0] % 128 == 0 and tile_group.dtype == torch.int32
              and tile_group.numel() >= a.shape[0] // 128, "the groups do not fit")
    m, group_rows = a.shape[0], w.shape[0] // groups
    ops._need(epilogue != SWIGLU or group_rows % 2 == 0, "gate and up rows must pair up")
    n = group_rows // 2 if epilogue == SWIGLU else group_rows
    out = torch.empty((m, n), dtype=torch.float32 if epilogue == STORE_F32 else torch.bfloat16, device=a.device)
    ops._call("mxb_gemm_tcgen05_grouped", out.data_ptr(), a.data_ptr(), w.data_ptr(), tile_group.data_ptr(), m, n,
              a.shape[1], groups, group_rows, a.stride(0), w.stride(0), out.stride(0), epilogue,
              ops.status_word(a.device).data_ptr(), ops._stream())
    return out
