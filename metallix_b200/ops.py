"""Python face of the hand-written CUDA kernels.

Every function checks its tensors (device, dtype, layout, sizes) and raises
``KernelError`` for what the kernels do not take; it never falls back to
another implementation. Kernels run on torch's current CUDA stream.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a cache slot or position outside its table",
               4: "a block-table entry outside the page pool", 8: "non-finite logits",
               16: "a bounded wait inside a kernel ran out"}


class KernelError(RuntimeError):
    pass


_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_SIGNATURES = {
    "mxb_embed": [_P, _P, _I, _P, _I, _I, _I, _F, _P, _P],
    "mxb_rmsnorm": [_P, _I, _P, _I, _P, _P, _I, _I, _F, _P],
    "mxb_add_rmsnorm": [_P, _P, _I, _P, _I, _P, _I, _I, _F, _P],
    "mxb_add_summands_rmsnorm": [_P, _P, _I, _P, _I, _P, _I, _I, _F, _P],
    "mxb_add": [_P, _P, _I, _L, _P],
    "mxb_copy_units": [_P, _I, _I, _L, _P, _I, _P, _P],
    "mxb_qk_norm_rope_cache": [_P, _P, _P, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P,
                               _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "mxb_paged_attention_tile": [_P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I,
                                 _F, _I, _P, _L, _I, _I, _F, _I, _I, _F, _P, _P, _P],
    "mxb_short_conv": [_P, _L, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "mxb_selective_scan": [_P, _L, _P, _L, _P, _P, _P, _P, _L, _P, _P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                           _I, _P, _P],
    "mxb_route_experts": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _L, _P],
    "mxb_expert_rows": [_P, _P, _P, _I, _I, _I, _P],
    "mxb_expert_rows_tile": [],
    "mxb_expert_rows_experts": [],
    "mxb_expert_gather_rows": [_P, _P, _P, _I, _I, _I, _I, _P],
    "mxb_expert_combine_rows": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "mxb_experts_add_identity": [_P, _P, _P, _I, _I, _I, _P],
    "mxb_experts_routed": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "mxb_add_gated_rows": [_P, _P, _P, _L, _I, _I, _I, _P],
    "mxb_pair_add_rmsnorm": [_P, _P, _I, _P, _I, _F, _P, _P, _P, _P, _I, _P, _I, _I, _F, _P],
    "mxb_add_bias": [_P, _L, _I, _P, _P, _L, _I, _I, _I, _P],
    "mxb_delta_rule_max_dim": [],
    "mxb_delta_rule": [_P, _L, _I, _I, _I, _P, _L, _I, _P, _L, _P, _P, _P, _L, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                       _I, _I, _P, _P],
    "mxb_add_cast": [_P, _P, _I, _P, _I, _L, _P],
    "mxb_gelu_gate_rows": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "mxb_stream_mix": [_P, _P, _P, _L, _L, _F, _F, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P],
    "mxb_weighted_sum": [_P, _P, _P, _L, _L, _F, _F, _I, _I, _I, _P],
    "mxb_mlstm_state_values": [_I, _I, _I],
    "mxb_mlstm_scan": [_P, _L, _I, _I, _I, _I, _I, _P, _P, _F, _F, _P, _L, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                       _I, _P, _P],
    "mxb_head_norm_gate": [_P, _P, _P, _L, _I, _P, _I, _I, _I, _I, _F, _P],
    "mxb_latent_cache": [_P, _L, _P, _F, _I, _I, _I, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "mxb_latent_heads": [_P, _L, _P, _L, _P, _L, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I,
                         _I, _P, _P],
    "mxb_rotate_into": [_P, _L, _I, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _I, _I, _P, _P],
    "mxb_relu_squared": [_P, _P, _L, _I, _P],
    "mxb_paged_attention_decode": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I,
                                   _F, _I, _P, _L, _F, _I, _F, _P, _P, _P],
    "mxb_postnorm_add_rmsnorm": [_P, _P, _I, _I, _P, _F, _P, _I, _P, _F, _I, _I, _P],
    "mxb_sigmoid_gate": [_P, _P, _P, _L, _L, _L, _I, _I, _I, _P],
    "mxb_softcap": [_P, _F, _L, _P],
    "mxb_paged_attention_decode_supported": [_I, _I, _I, _I],
    "mxb_paged_attention_decode_project_supported": [_I, _I, _I, _I, _I, _P, _L],
    "mxb_paged_attention_decode_project": [_P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I,
                                           _F, _P, _L, _I, _P, _P, _L, _F, _I, _F, _P, _P, _P],
    "mxb_paged_attention_split_keys": [],
    "mxb_set_decode_resident_blocks": [_I, _I],
    "mxb_flash_prefill": [_P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _L, _F, _I, _F,
                          _P, _P, _P],
    "mxb_flash_prefill_supported": [_I, _I, _I, _I],
    "mxb_flash_prefill_tile": [],
    "mxb_flash_prefill_tcgen05": [_P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P,
                                  _P, _L, _F, _I, _F, _P, _P, _P],
    "mxb_flash_prefill_tcgen05_supported": [_I, _I, _I, _I, _I],
    "mxb_flash_prefill_tcgen05_tile": [],
    "mxb_gemm_simple": [_P, _I, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P],
    "mxb_gemm_skinny": [_P, _I, _P, _P, _I, _I, _I, _L, _L, _L, _I, _I, _P],
    "mxb_gemm_skinny_supported": [_I, _I, _I, _L, _L],
    "mxb_gemm_stream": [_P, _I, _P, _P, _I, _I, _I, _L, _L, _L, _I, _I, _P, _P],
    "mxb_gemm_stream_supported": [_I, _I, _I, _L, _L, _I],
    "mxb_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _P, _P],
    "mxb_gemm_tcgen05_supported": [_I, _I, _I, _L, _L],
    "mxb_gemm_tcgen05_grouped": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _L, _L, _I, _P, _P],
    "mxb_silu_mul": [_P, _P, _I, _L, _I, _I, _P],
    "mxb_argmax": [_P, _L, _I, _I, _P, _P, _P, _P],
    "mxb_argmax_pieces": [_I, _I],
    "mxb_sample_icdf": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P],
    "mxb_icdf_pieces": [_I],
    "mxb_sample_race": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P],
    "mxb_set_chained_launches": [_I],
    "mxb_nucleus_mask": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P],
}
_functions = {}
_status = {}


def _fn(name: str):
    fn = _functions.get(name)
    if fn is None:
        library = build.kernels()
        try:
            fn = getattr(library, name)
        except AttributeError:
            raise KernelError(f"the kernel library has no entry point {name}") from None
        fn.argtypes = _SIGNATURES[name]
        fn.restype = ctypes.c_int
        _functions[name] = fn
    return fn


_launches = 0


def launch_count() -> int:
    """How many of this library's kernel entry points have been called
    (a replayed CUDA graph counts the calls it captured)."""
    return _launches


def count_launches(count: int) -> None:
    global _launches
    _launches += count


def _call(name: str, *args) -> None:
    global _launches
    _launches += 1
    code = _fn(name)(*args)
    if code != 0:
        raise KernelError(f"{name} failed to launch: CUDA error {code}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle; this runs once per launch, so it takes the short way."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _need(condition: bool, message: str) -> None:
    if not condition:
        raise KernelError(message)


def _check(tensor: torch.Tensor, name: str, dtypes, dims: Optional[int] = None) -> None:
    if (isinstance(tensor, torch.Tensor) and tensor.is_cuda and tensor.dtype in dtypes and tensor.is_contiguous()
            and (dims is None or tensor.dim() == dims)):
        return   # the messages below are built only for what fails
    _need(isinstance(tensor, torch.Tensor), f"{name} must be a tensor")
    _need(tensor.is_cuda, f"{name} must be on a CUDA device; there is no CPU path")
    _need(tensor.dtype in dtypes, f"{name} has dtype {tensor.dtype}, expected one of {dtypes}")
    _need(tensor.is_contiguous(), f"{name} must be contiguous")
    if dims is not None:
        _need(tensor.dim() == dims, f"{name} must have {dims} dimensions, has {tensor.dim()}")


def require_cuda() -> None:
    """Fails loudly where the kernels cannot run."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: metallix_b200 runs on a B200 only and has no CPU path")
    build.kernels()


_chained: Optional[bool] = None


def set_chained_launches(enabled: bool) -> None:
    """Lets consecutive kernels of this library overlap (programmatic dependent
    launch): a kernel may start, and fetch weights, while its predecessor is
    still running, and waits for the predecessor before it reads its output.
    The switch belongs to the library; an engine sets it to its own choice
    before it launches."""
    global _chained
    if _chained is not enabled:
        _fn("mxb_set_chained_launches")(1 if enabled else 0)
        _chained = bool(enabled)


TIMELINE_SOURCES = ("norms", "sandwich_norms", "gemm_load", "gemm_stream", "qk_rope", "attention")


def timeline(reset: bool = True):
    """[(nanoseconds, source)] in time order: when each chained kernel
    launched since the last reset got past the wait for the kernel ahead of
    it. Needs the library built with METALLIX_B200_TIMELINE=1 in the
    environment (a build of its own, next to the usual one)."""
    library = build.kernels()
    events = []
    for source in TIMELINE_SOURCES:
        function = getattr(library, f"mxb_timeline_{source}", None)
        if function is None:
            raise KernelError("this build records no timeline: set METALLIX_B200_TIMELINE=1 before the first use")
        function.argtypes = [ctypes.c_void_p, ctypes.c_int]
        function.restype = ctypes.c_int
        buffer = (ctypes.c_ulonglong * 8192)()
        count = function(buffer, 1 if reset else 0)
        events.extend((int(buffer[i]), source) for i in range(count))
    return sorted(events)


def status_word(device) -> torch.Tensor:
    """The int32 word kernels set bits in instead of trapping."""
    word = _status.get(device)
    if word is None:
        key = torch.device(device).index or 0
        if key not in _status:
            _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
        word = _status[device] = _status[key]   # torch.device objects and strings find it directly next time
    return word


_status_host = {}


def fetch_status(device) -> None:
    """Queues a copy of the status word to pinned host memory on the current
    stream; ``raise_status`` reads it once the stream has been synchronised
    (by reading the step's results, say), which saves a synchronisation of
    its own."""
    word = status_word(device)
    host = _status_host.get(device)
    if host is None:
        host = _status_host[device] = torch.zeros(1, dtype=torch.int32, pin_memory=True)
    host.copy_(word, non_blocking=True)


def raise_status(device) -> None:
    """Raises on what the last ``fetch_status`` copy brought (the caller has
    synchronised since); clears the device word then."""
    host = _status_host.get(device)
    value = int(host[0]) if host is not None else 0
    if value:
        status_word(device).zero_()
        reasons = [text for bit, text in STATUS_BITS.items() if value & bit]
        raise KernelError("a kernel refused its input: " + "; ".join(reasons))


def check_status(device) -> None:
    """Reads the status word (synchronises) and raises on any bit; clears it."""
    word = status_word(device)
    value = int(word.item())
    if value:
        word.zero_()
        reasons = [text for bit, text in STATUS_BITS.items() if value & bit]
        raise KernelError("a kernel refused its input: " + "; ".join(reasons))


# ------------------------------------------------------------------ embedding
def embed(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None,
          scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[ids[t]] * scale as float32."""
    _check(ids, "ids", (torch.int32,), 1)
    _check(table, "table", tuple(_CODES), 2)
    tokens, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=ids.device)
    _check(out, "out", (torch.float32,), 2)
    _need(out.shape == (tokens, hidden), "out has the wrong shape")
    _call("mxb_embed", out.data_ptr(), table.data_ptr(), _CODES[table.dtype], ids.data_ptr(),
          tokens, hidden, vocab, float(scale), status_word(ids.device).data_ptr(), _stream())
    return out


# ----------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows_index: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis, float32 inside.
    ``rows_index`` picks the rows of ``x`` to normalise."""
    _check(x, "x", tuple(_CODES))
    _check(weight, "weight", (torch.float32,), 1)
    size = x.shape[-1]
    _need(weight.numel() == size, f"weight has {weight.numel()} values for rows of {size}")
    rows = x.numel() // size if rows_index is None else rows_index.numel()
    if rows_index is not None:
        _check(rows_index, "rows_index", (torch.int32,), 1)
        _need(x.dim() == 2, "rows_index needs a 2-d input")
        shape = (rows, size)
    else:
        shape = tuple(x.shape)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=x.device)
    _check(out, "out", (out_dtype,))
    _need(out.numel() == rows * size, "out has the wrong size")
    _call("mxb_rmsnorm", out.data_ptr(), _CODES[out_dtype], x.data_ptr(), _CODES[x.dtype],
          weight.data_ptr(), _ptr(rows_index), rows, size, float(eps), _stream())
    return out


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += delta in float32 (in place), then returns RMSNorm(x) * w. A delta
    of three dimensions, float32 ``[parts, rows, size]``, is a sum its producer
    left in parts: they are added up in their order first."""
    _check(x, "x", (torch.float32,), 2)
    _check(weight, "weight", (torch.float32,), 1)
    rows, size = x.shape
    _need(weight.numel() == size, "weight has the wrong size")
    if out is None:
        out = torch.empty((rows, size), dtype=out_dtype, device=x.device)
    _check(out, "out", (out_dtype,), 2)
    _need(out.shape == x.shape, "out has the wrong shape")
    if delta.dim() == 3:
        _check(delta, "delta", (torch.float32,), 3)
        _need(delta.shape[1:] == x.shape and delta.shape[0] >= 1, "the summands and x differ in shape")
        _call("mxb_add_summands_rmsnorm", x.data_ptr(), delta.data_ptr(), delta.shape[0], out.data_ptr(),
              _CODES[out_dtype], weight.data_ptr(), rows, size, float(eps), _stream())
        return out
    _check(delta, "delta", tuple(_CODES), 2)
    _need(delta.shape == x.shape, "delta and x differ in shape")
    _call("mxb_add_rmsnorm", x.data_ptr(), delta.data_ptr(), _CODES[delta.dtype], out.data_ptr(),
          _CODES[out_dtype], weight.data_ptr(), rows, size, float(eps), _stream())
    return out


def add_(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta, the sum in float32."""
    _check(x, "x", (torch.float32,))
    _check(delta, "delta", tuple(_CODES))
    _need(delta.shape == x.shape, "delta and x differ in shape")
    _call("mxb_add", x.data_ptr(), delta.data_ptr(), _CODES[delta.dtype], x.numel(), _stream())
    return x


def pair_add_rmsnorm(x: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor], scale: float,
                     weight: Optional[torch.Tensor], second_weight: Optional[torch.Tensor], eps: float,
                     out_dtype: torch.dtype, rows_index: Optional[torch.Tensor] = None):
    """x += scale * (a + b) in float32 (in place; ``a`` and ``b`` are optional,
    each float32 or bfloat16), then RMSNorm(x) * weight and, with
    ``second_weight``, RMSNorm(x) * second_weight from the same pass over the
    row: what a layer needs whose two sublayers read the same input. Returns
    the one result, or the two as a pair; None without ``weight`` (the sum
    alone). ``rows_index`` picks rows of x (then nothing is added)."""
    _check(x, "x", (torch.float32,), 2)
    size = x.shape[1]
    for name, delta in (("a", a), ("b", b)):
        if delta is not None:
            _check(delta, name, tuple(_CODES), 2)
            _need(delta.shape == x.shape, f"{name} and x differ in shape")
    rows = x.shape[0]
    if rows_index is not None:
        _check(rows_index, "rows_index", (torch.int32,), 1)
        _need(a is None and b is None, "rows are picked only where nothing is added")
        rows = rows_index.numel()
    first = second = None
    if weight is not None:
        _check(weight, "weight", (torch.float32,), 1)
        _need(weight.numel() == size, "weight has the wrong size")
        first = torch.empty((rows, size), dtype=out_dtype, device=x.device)
        if second_weight is not None:
            _check(second_weight, "second_weight", (torch.float32,), 1)
            _need(second_weight.numel() == size, "second_weight has the wrong size")
            second = torch.empty((rows, size), dtype=out_dtype, device=x.device)
    else:
        _need(second_weight is None, "a second weight without a first")
    _need(out_dtype in _CODES, "out_dtype must be float32 or bfloat16")
    _call("mxb_pair_add_rmsnorm", x.data_ptr(), _ptr(a), _CODES[a.dtype] if a is not None else F32, _ptr(b),
          _CODES[b.dtype] if b is not None else F32, float(scale), _ptr(weight), _ptr(second_weight), _ptr(first),
          _ptr(second), _CODES[out_dtype], _ptr(rows_index), rows, size, float(eps), _stream())
    if weight is None:
        return None
    return (first, second) if second_weight is not None else first


def add_bias(x: torch.Tensor, bias: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x + bias over the last axis, for x ``[tokens, width]`` float32 (a product's
    unrounded result) or already of ``out_dtype``; the sum is float32 and is
    rounded once. Rows of x may be strided."""
    _need(x.is_cuda and x.dim() == 2 and x.stride(1) == 1 and x.dtype in _CODES, "x must be [tokens, width]")
    _check(bias, "bias", (torch.float32,), 1)
    _need(bias.numel() == x.shape[1], "one bias value per column")
    _need(out_dtype in _CODES and (x.dtype == torch.float32 or x.dtype == out_dtype), "x must be float32 or of out_dtype")
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _call("mxb_add_bias", x.data_ptr(), x.stride(0), _CODES[x.dtype], bias.data_ptr(), out.data_ptr(), out.stride(0),
          _CODES[out_dtype], x.shape[0], x.shape[1], _stream())
    return out


def postnorm_add_rmsnorm(x: torch.Tensor, delta: torch.Tensor, post_weight: torch.Tensor, post_eps: float,
                         next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                         out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """x += RMSNorm(delta) * post_weight in float32 (in place); with
    ``next_weight`` returns RMSNorm(x) * next_weight in ``out_dtype``, else
    None. ``delta`` is ``[rows, size]``, or float32 ``[parts, rows, size]``
    whose parts are added up first."""
    _check(x, "x", (torch.float32,), 2)
    _check(post_weight, "post_weight", (torch.float32,), 1)
    rows, size = x.shape
    _need(post_weight.numel() == size, "post_weight has the wrong size")
    if delta.dim() == 3:
        _check(delta, "delta", (torch.float32,), 3)
        _need(delta.shape[1:] == x.shape and delta.shape[0] >= 1, "the summands and x differ in shape")
        parts = delta.shape[0]
    else:
        _check(delta, "delta", tuple(_CODES), 2)
        _need(delta.shape == x.shape, "delta and x differ in shape")
        parts = 1
    out = None
    if next_weight is not None:
        _check(next_weight, "next_weight", (torch.float32,), 1)
        _need(next_weight.numel() == size and out_dtype in _CODES, "next_weight or out_dtype does not fit")
        out = torch.empty((rows, size), dtype=out_dtype, device=x.device)
    _call("mxb_postnorm_add_rmsnorm", x.data_ptr(), delta.data_ptr(), _CODES[delta.dtype], parts,
          post_weight.data_ptr(), float(post_eps), _ptr(out), _CODES[out_dtype] if out is not None else 0,
          _ptr(next_weight), float(next_eps), rows, size, _stream())
    return out


def sigmoid_gate(a: torch.Tensor, gate: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = a * sigmoid(gate), float32 inside; ``a`` and ``gate`` are
    [rows, width] with unit column stride (rows may be strided: a column range
    of a wider product)."""
    for name, tensor in (("a", a), ("gate", gate)):
        _need(tensor.is_cuda and tensor.dtype in _CODES and tensor.dim() == 2 and tensor.stride(1) == 1,
              f"{name} must be a CUDA [rows, width] tensor with unit column stride")
    _need(a.shape == gate.shape and a.dtype == gate.dtype, "a and gate differ in shape or dtype")
    if out is None:
        out = torch.empty(a.shape, dtype=a.dtype, device=a.device)
    _need(out.shape == a.shape and out.dtype == a.dtype and out.stride(1) == 1, "out does not fit")
    _call("mxb_sigmoid_gate", out.data_ptr(), a.data_ptr(), gate.data_ptr(), out.stride(0), a.stride(0),
          gate.stride(0), a.shape[0], a.shape[1], _CODES[a.dtype], _stream())
    return out


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap), in place (float32)."""
    _check(x, "x", (torch.float32,))
    _need(cap > 0.0, "the cap must be positive")
    _call("mxb_softcap", x.data_ptr(), float(cap), x.numel(), _stream())
    return x


# ------------------------------------- several residual streams, Dynamic Tanh
MAX_STREAMS = 8


def stream_mix(streams: torch.Tensor, result: Optional[torch.Tensor] = None,
               channel_scale: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
               out_weights: Optional[torch.Tensor] = None, in_weights: Optional[torch.Tensor] = None,
               alpha: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
               norm_bias: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
               rows_index: Optional[torch.Tensor] = None, read: bool = True, keep_streams: bool = True,
               second: Optional[torch.Tensor] = None, weights=(1.0, 1.0)) -> Optional[torch.Tensor]:
    """One pass over ``streams`` (float32 ``[tokens, s, width]``, in place).

    With ``result`` ``[tokens, width]`` (rows may be strided): every stream t
    becomes sum_s mix[s, t] x_s + out_weights[t] * (channel_scale * y), where
    y = weights[0] * result (+ weights[1] * second). Then, with ``read``:
    u = sum_s in_weights[s] x_s (the plain sum without ``in_weights``) and, with
    ``alpha`` (a scalar tensor), Dynamic Tanh tanh(alpha u) * norm_weight +
    norm_bias; returns that as ``[rows, width]`` in ``out_dtype``.
    ``rows_index`` (int32): only those tokens are worked on.
    ``keep_streams=False``: the new streams are not stored (a step's last read)."""
    _check(streams, "streams", (torch.float32,), 3)
    tokens, count, width = streams.shape
    _need(1 <= count <= MAX_STREAMS, f"{count} residual streams; the kernel takes 1..{MAX_STREAMS}")
    rows = tokens
    if rows_index is not None:
        _check(rows_index, "rows_index", (torch.int32,), 1)
        rows = rows_index.numel()
    result_code, lda, ldb = F32, 0, 0
    if result is not None:
        for name, tensor in (("result", result), ("second", second)):
            if tensor is None:
                continue
            _need(tensor.is_cuda and tensor.dtype in _CODES and tensor.dim() == 2 and tensor.stride(1) == 1
                  and tensor.shape == (tokens, width) and tensor.dtype == result.dtype,
                  f"{name} must be a CUDA [tokens, width] tensor with unit column stride")
        result_code, lda = _CODES[result.dtype], result.stride(0)
        ldb = second.stride(0) if second is not None else 0
        for name, tensor, size in (("mix", mix, count * count), ("out_weights", out_weights, count)):
            _need(tensor is not None, f"{name} is needed to write a result back")
            _check(tensor, name, (torch.float32,))
            _need(tensor.numel() == size, f"{name} must have {size} values")
    else:
        _need(second is None, "a second result needs a first")
    for name, tensor, size in (("channel_scale", channel_scale, width), ("in_weights", in_weights, count),
                               ("alpha", alpha, 1), ("norm_weight", norm_weight, width), ("norm_bias", norm_bias, width)):
        if tensor is not None:
            _check(tensor, name, (torch.float32,))
            _need(tensor.numel() == size, f"{name} must have {size} values")
    out = None
    if read:
        _need(out_dtype in _CODES, "out_dtype must be float32 or bfloat16")
        _need(alpha is None or norm_weight is not None, "Dynamic Tanh needs its weight")
        out = torch.empty((rows, width), dtype=out_dtype, device=streams.device)
    _call("mxb_stream_mix", streams.data_ptr(), _ptr(result), _ptr(second), lda, ldb, float(weights[0]),
          float(weights[1]), result_code, _ptr(channel_scale), _ptr(mix), _ptr(out_weights), _ptr(in_weights),
          _ptr(alpha), _ptr(norm_weight), _ptr(norm_bias), _ptr(out), _CODES[out_dtype] if out is not None else F32,
          _ptr(rows_index), rows, width, count, 1 if keep_streams else 0, _stream())
    return out


def weighted_sum(x: torch.Tensor, y: torch.Tensor, a: float, b: float) -> torch.Tensor:
    """a * x + b * y as float32 ``[rows, width]`` (rows of x and y may be strided)."""
    for name, tensor in (("x", x), ("y", y)):
        _need(tensor.is_cuda and tensor.dtype in _CODES and tensor.dim() == 2 and tensor.stride(1) == 1,
              f"{name} must be a CUDA [rows, width] tensor with unit column stride")
    _need(x.shape == y.shape and x.dtype == y.dtype, "x and y differ in shape or dtype")
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    _call("mxb_weighted_sum", out.data_ptr(), x.data_ptr(), y.data_ptr(), x.stride(0), y.stride(0), float(a), float(b),
          x.shape[0], x.shape[1], _CODES[x.dtype], _stream())
    return out


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    """max(x, 0)^2, float32 inside."""
    _check(x, "x", tuple(_CODES))
    out = torch.empty_like(x)
    _call("mxb_relu_squared", out.data_ptr(), x.data_ptr(), x.numel(), _CODES[x.dtype], _stream())
    return out


# ------------------------------------------------ short convolution over time
def short_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
               token_request: torch.Tensor, row_start: torch.Tensor, row_length: torch.Tensor,
               request_slots: torch.Tensor, residual: bool = False, activation: Optional[str] = None,
               longest: int = 0) -> torch.Tensor:
    """A causal convolution over time on each channel of the packed tokens
    x ``[tokens, channels]`` (rows may be strided): y_t = bias + sum_j
    w[:, j] x_(t - taps + 1 + j), zeros before a sequence's start; the result is
    y, or x + y with ``residual``, passed through ``activation`` ("silu").
    ``weight`` is float32 and tap-major, ``[taps, channels]`` (row j is
    w[:, j]), its last row the current token's. ``state`` (float32 ``[slots, taps - 1, channels]``) holds each
    request's last inputs of earlier steps and is moved on by this step's;
    request row r owns tokens ``row_start[r] .. + row_length[r]`` and the slot
    ``request_slots[r]`` (a row of length 0 touches nothing). ``longest``: the
    most tokens of a row if known; a step of single tokens (1) moves the state
    on in the same launch."""
    _need(x.is_cuda and x.dtype in _CODES and x.dim() == 2 and x.stride(1) == 1, "x must be [tokens, channels]")
    tokens, channels = x.shape
    _check(weight, "weight", (torch.float32,), 2)
    taps = weight.shape[0]
    _need(weight.shape[1] == channels and 1 <= taps <= 64, "weight must be [taps, channels]")
    if bias is not None:
        _check(bias, "bias", (torch.float32,), 1)
        _need(bias.numel() == channels, "bias must have one value per channel")
    _check(state, "state", (torch.float32,), 3)
    _need(state.shape[1:] == (taps - 1, channels), f"state must be [slots, {taps - 1}, {channels}]")
    for name, tensor in (("token_request", token_request), ("row_start", row_start), ("row_length", row_length),
                         ("request_slots", request_slots)):
        _check(tensor, name, (torch.int32,), 1)
    rows = row_start.numel()
    _need(token_request.numel() == tokens and row_length.numel() == rows and request_slots.numel() >= rows,
          "the step's integer lists do not fit its tokens and rows")
    _need(activation in (None, "silu"), f"unknown activation {activation!r}")
    out = torch.empty((tokens, channels), dtype=x.dtype, device=x.device)
    _call("mxb_short_conv", x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(bias), state.data_ptr(),
          token_request.data_ptr(), row_start.data_ptr(), row_length.data_ptr(), request_slots.data_ptr(),
          out.data_ptr(), tokens, rows, channels, taps, state.shape[0], 1 if residual else 0,
          1 if activation == "silu" else 0, int(longest), _CODES[x.dtype], status_word(x.device).data_ptr(), _stream())
    return out


# ------------------------------------------------ selective state-space scan
SCAN_STATES = 256   # the most states per channel the scan keeps in registers


def selective_scan(x: torch.Tensor, step: torch.Tensor, step_bias: torch.Tensor, a: torch.Tensor, b: torch.Tensor,
                   c: torch.Tensor, d: torch.Tensor, z: torch.Tensor, state: torch.Tensor, row_start: torch.Tensor,
                   row_length: torch.Tensor, request_slots: torch.Tensor, longest: int = 0) -> torch.Tensor:
    """S <- exp(dt A) S + dt x B, y = S C + D x, out = y silu(z) per channel,
    token by token along each request row, dt = softplus(step + step_bias).
    x, z ``[tokens, channels]`` and b, c ``[tokens, states]`` in the compute
    type (rows may be strided; b and c share a row stride); ``step`` float32
    ``[tokens, channels]``; ``a`` float32 ``[channels, states]``; ``state``
    float32 ``[slots, channels, states]``, read and moved on. ``longest``: the
    most tokens of a row if known (1 picks the kernel for single tokens)."""
    dtype = x.dtype
    for name, tensor in (("x", x), ("z", z), ("b", b), ("c", c)):
        _need(tensor.is_cuda and tensor.dtype == dtype and dtype in _CODES and tensor.dim() == 2
              and tensor.stride(1) == 1, f"{name} must be a CUDA [tokens, width] tensor with unit column stride")
    tokens, channels = x.shape
    states = b.shape[1]
    _need(z.shape == x.shape and c.shape == b.shape and b.shape[0] == tokens and b.stride(0) == c.stride(0),
          "x, z, b and c do not fit one another")
    _need(0 < states <= SCAN_STATES, f"{states} states per channel; up to {SCAN_STATES} are taken")
    _need(step.is_cuda and step.dtype == torch.float32 and step.shape == x.shape and step.stride(1) == 1,
          "step must be float32 [tokens, channels]")
    _check(step_bias, "step_bias", (torch.float32,), 1)
    _check(d, "d", (torch.float32,), 1)
    _check(a, "a", (torch.float32,), 2)
    _check(state, "state", (torch.float32,), 3)
    _need(step_bias.numel() == channels and d.numel() == channels and a.shape == (channels, states)
          and state.shape[1:] == (channels, states), "the scan's parameters or state do not fit its channels and states")
    for name, tensor in (("row_start", row_start), ("row_length", row_length), ("request_slots", request_slots)):
        _check(tensor, name, (torch.int32,), 1)
    rows = row_start.numel()
    _need(row_length.numel() == rows and request_slots.numel() >= rows, "the step's row lists differ in length")
    out = torch.empty((tokens, channels), dtype=dtype, device=x.device)
    _call("mxb_selective_scan", x.data_ptr(), x.stride(0), step.data_ptr(), step.stride(0), step_bias.data_ptr(),
          a.data_ptr(), b.data_ptr(), c.data_ptr(), b.stride(0), d.data_ptr(), z.data_ptr(), z.stride(0),
          state.data_ptr(), row_start.data_ptr(), row_length.data_ptr(), request_slots.data_ptr(), out.data_ptr(),
          rows, channels, states, state.shape[0], int(longest), _CODES[dtype], status_word(x.device).data_ptr(),
          _stream())
    return out


# ------------------------------------------------------------ routed experts
ROUTER_OUTPUTS = 1024   # the most router outputs the routing kernel keeps in shared memory


def route_experts(logits: torch.Tensor, correction: torch.Tensor, experts: int, top: int, scores: str = "softmax",
                  groups: Optional[tuple] = None, scale: float = 1.0):
    """Scores over all router outputs (``scores``: "softmax" over the row, or
    "sigmoid" of each logit on its own), the ``top`` largest score + correction
    chosen, weights = the chosen scores over their sum, times ``scale``.
    ``groups`` = (count, keep): the outputs form ``count`` equal groups of
    neighbours and only outputs of the ``keep`` groups with the largest sum of
    their two largest score + correction can be chosen. ``logits`` is float32
    ``[tokens, outputs]`` whose rows may be strided. Returns (chosen int32
    ``[tokens, top]``, weights float32 ``[tokens, top]``, dense float32
    ``[tokens, experts]`` with each real expert's weight or zero, float32
    ``[tokens]`` weight that fell on the outputs from ``experts`` on, which
    stand for experts that return their input)."""
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1,
          "logits must be float32 [tokens, outputs] with unit column stride")
    _check(correction, "correction", (torch.float32,), 1)
    tokens, outputs = logits.shape
    _need(correction.numel() == outputs and 0 <= experts <= outputs and 0 < top <= outputs
          and outputs <= ROUTER_OUTPUTS, "the router's sizes do not fit")
    _need(scores in ("softmax", "sigmoid"), f"unknown scores {scores!r}")
    count, keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
    if count > 1:
        _need(outputs % count == 0 and 1 <= keep <= count and keep * (outputs // count) >= top
              and outputs <= ROUTER_OUTPUTS // 2, "the router's groups do not fit")
    device = logits.device
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=device)
    dense = torch.empty((tokens, experts), dtype=torch.float32, device=device)
    on_identity = torch.empty((tokens,), dtype=torch.float32, device=device)
    _call("mxb_route_experts", logits.data_ptr(), correction.data_ptr(), chosen.data_ptr(), weights.data_ptr(),
          dense.data_ptr(), on_identity.data_ptr(), tokens, outputs, experts, top, 1 if scores == "sigmoid" else 0,
          count, keep, float(scale), logits.stride(0), _stream())
    return chosen, weights, dense, on_identity


def expert_rows(chosen: torch.Tensor, experts: int):
    """Sorts the (token, choice) pairs by expert. Returns (position int32
    ``[tokens, top]``: each pair's row in the sorted array, -1 where the choice
    is not a real expert; tile_group int32 ``[tiles]``: the expert of each tile
    of ``expert_rows_tile()`` rows, -1 for tiles left empty; the sorted array's
    rows, every expert's share rounded up to whole tiles)."""
    _check(chosen, "chosen", (torch.int32,), 2)
    tile = expert_rows_tile()
    pairs = chosen.numel()
    _need(1 <= experts <= int(_fn("mxb_expert_rows_experts")()), "too many experts to sort by")
    tiles = (pairs + experts * (tile - 1) + tile - 1) // tile
    position = torch.empty(chosen.shape, dtype=torch.int32, device=chosen.device)
    tile_group = torch.empty((tiles,), dtype=torch.int32, device=chosen.device)
    _call("mxb_expert_rows", chosen.data_ptr(), position.data_ptr(), tile_group.data_ptr(), pairs, experts, tiles,
          _stream())
    return position, tile_group, tiles * tile


def expert_rows_tile() -> int:
    return int(_fn("mxb_expert_rows_tile")())


def expert_gather_rows(h: torch.Tensor, position: torch.Tensor, rows: int) -> torch.Tensor:
    """``[rows, hidden]`` with h[t] at position[t, k] for every pair that has
    a position; the other rows are left as they are found."""
    _check(h, "h", tuple(_CODES), 2)
    _check(position, "position", (torch.int32,), 2)
    _need(position.shape[0] == h.shape[0], "a row of positions per token")
    out = torch.empty((rows, h.shape[1]), dtype=h.dtype, device=h.device)
    _call("mxb_expert_gather_rows", h.data_ptr(), position.data_ptr(), out.data_ptr(), position.numel(), h.shape[1],
          position.shape[1], _CODES[h.dtype], _stream())
    return out


def expert_combine_rows(rows: torch.Tensor, position: torch.Tensor, weights: torch.Tensor, on_identity: torch.Tensor,
                        h: torch.Tensor) -> torch.Tensor:
    """y[t] = sum_k weights[t, k] rows[position[t, k]] + on_identity[t] h[t], float32."""
    _check(rows, "rows", (torch.float32,), 2)
    _check(position, "position", (torch.int32,), 2)
    _check(weights, "weights", (torch.float32,), 2)
    _check(on_identity, "on_identity", (torch.float32,), 1)
    _check(h, "h", tuple(_CODES), 2)
    tokens, hidden = h.shape
    _need(rows.shape[1] == hidden and position.shape == weights.shape and position.shape[0] == tokens
          and on_identity.numel() == tokens, "rows, positions, weights and h do not fit")
    y = torch.empty((tokens, hidden), dtype=torch.float32, device=h.device)
    _call("mxb_expert_combine_rows", rows.data_ptr(), position.data_ptr(), weights.data_ptr(), on_identity.data_ptr(),
          h.data_ptr(), y.data_ptr(), tokens, hidden, position.shape[1], _CODES[h.dtype], _stream())
    return y


def experts_add_identity(y: torch.Tensor, h: torch.Tensor, on_identity: torch.Tensor) -> torch.Tensor:
    """y[t] += on_identity[t] * h[t] (y float32, in place)."""
    _check(y, "y", (torch.float32,), 2)
    _check(h, "h", tuple(_CODES), 2)
    _check(on_identity, "on_identity", (torch.float32,), 1)
    _need(h.shape == y.shape and on_identity.numel() == y.shape[0], "y, h and the weights do not fit")
    _call("mxb_experts_add_identity", y.data_ptr(), h.data_ptr(), on_identity.data_ptr(), y.shape[0], y.shape[1],
          _CODES[h.dtype], _stream())
    return y


def experts_routed(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, chosen: torch.Tensor,
                   weights: torch.Tensor, experts: int, ff: int, gated: bool = False) -> torch.Tensor:
    """sum_k weight[t, k] W_down[e] relu(W_up[e] h_t)^2 over a token's chosen
    experts e = chosen[t, k] < experts, plus h_t times the weights of chosen
    indices from ``experts`` on; float32 ``[tokens, hidden]``. Only the chosen
    experts' weights are read. w_up ``[experts * ff, hidden]``, w_down
    ``[experts * hidden, ff]``. ``gated``: an expert is W_down (silu(W_gate h) *
    (W_up h)) and w_up holds, expert by expert, its gate rows and then its up
    rows, ``[experts * 2 * ff, hidden]``."""
    dtype = h.dtype
    _check(h, "h", tuple(_CODES), 2)
    _check(w_up, "w_up", (dtype,), 2)
    _check(w_down, "w_down", (dtype,), 2)
    _check(chosen, "chosen", (torch.int32,), 2)
    _check(weights, "weights", (torch.float32,), 2)
    tokens, hidden = h.shape
    top = chosen.shape[1]
    _need(chosen.shape == (tokens, top) and weights.shape == (tokens, top), "chosen and weights must be [tokens, top]")
    _need(w_up.shape == (experts * ff * (2 if gated else 1), hidden) and w_down.shape == (experts * hidden, ff),
          "the experts' stacked weights do not fit")
    act = torch.empty((tokens * top, ff), dtype=torch.float32, device=h.device)
    y = torch.empty((tokens, hidden), dtype=torch.float32, device=h.device)
    _call("mxb_experts_routed", h.data_ptr(), w_up.data_ptr(), w_down.data_ptr(), chosen.data_ptr(),
          weights.data_ptr(), act.data_ptr(), y.data_ptr(), tokens, hidden, experts, ff, top, _CODES[dtype],
          1 if gated else 0, _stream())
    return y


def add_gated_rows(y: torch.Tensor, x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """y[t] += sigmoid(gate[t]) * x[t] (y float32, in place): ``gate`` is float32, one
    number per token (a column of a wider tensor will do)."""
    _check(y, "y", (torch.float32,), 2)
    _check(x, "x", tuple(_CODES), 2)
    _need(x.shape == y.shape, "x and y differ in shape")
    _need(gate.is_cuda and gate.dtype == torch.float32 and gate.dim() in (1, 2) and gate.shape[0] == y.shape[0]
          and (gate.dim() == 1 or gate.shape[1] == 1), "gate must be float32 [tokens] or [tokens, 1]")
    _call("mxb_add_gated_rows", y.data_ptr(), x.data_ptr(), gate.data_ptr(), gate.stride(0), y.shape[0], y.shape[1],
          _CODES[x.dtype], _stream())
    return y


# ------------------------------------------------------ input from the token
def add_cast(x: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """x += delta in float32 (in place; nothing is added without a delta);
    returns x in ``out_dtype``."""
    _check(x, "x", (torch.float32,))
    if delta is not None:
        _check(delta, "delta", tuple(_CODES))
        _need(delta.shape == x.shape, "delta and x differ in shape")
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _need(out_dtype in _CODES, "out_dtype must be float32 or bfloat16")
    _call("mxb_add_cast", x.data_ptr(), _ptr(delta), _CODES[delta.dtype] if delta is not None else F32,
          out.data_ptr(), _CODES[out_dtype], x.numel(), _stream())
    return out


def gelu_gate_rows(gate: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, offset: int) -> torch.Tensor:
    """gelu_tanh(gate[t]) * table[ids[t], offset : offset + dim] for gate ``[tokens, dim]``."""
    _check(gate, "gate", tuple(_CODES), 2)
    _check(table, "table", (gate.dtype,), 2)
    _check(ids, "ids", (torch.int32,), 1)
    tokens, dim = gate.shape
    _need(ids.numel() == tokens and 0 <= offset and offset + dim <= table.shape[1], "the table's columns do not fit")
    out = torch.empty_like(gate)
    _call("mxb_gelu_gate_rows", gate.data_ptr(), table.data_ptr(), ids.data_ptr(), out.data_ptr(), tokens, dim,
          table.shape[1], offset, table.shape[0], _CODES[gate.dtype], status_word(gate.device).data_ptr(), _stream())
    return out


# ------------------------------------------------------- matrix-memory recurrence
def mlstm_state_values(heads: int, dim: int, vdim: int) -> int:
    """float32 values one request's state of the recurrence takes."""
    return int(_fn("mxb_mlstm_state_values")(heads, dim, vdim))


def mlstm_scan(proj: torch.Tensor, offsets, i_bias: torch.Tensor, f_bias: torch.Tensor, cap: float,
               state: torch.Tensor, row_start: torch.Tensor, row_length: torch.Tensor,
               request_slots: torch.Tensor, heads: int, dim: int, vdim: int, longest: int = 1) -> torch.Tensor:
    """The matrix-memory recurrence over a step's tokens. ``proj``
    ``[tokens, columns]`` holds, from the column ``offsets`` (q, k, v, i, f)
    on, heads * dim queries and keys, heads * vdim values and one input- and
    one forget-gate pre-activation per head. Request row r brings
    ``row_length[r]`` consecutive tokens from packed token ``row_start[r]`` on
    (0: a padding row) and owns slot ``request_slots[r]`` of ``state``
    (float32 ``[slots, mlstm_state_values]``, advanced in place). Returns
    float32 ``[tokens, heads * vdim]``: each head's C^T q over its bounded
    normaliser, before the head norm. ``longest`` (the most tokens any row
    brings, as the host knows it) chooses the form: from 8 tokens on the
    rows are worked on in chunks of 16 tokens side by side, below that token
    by token; the two agree to rounding."""
    _need(proj.is_cuda and proj.dtype in _CODES and proj.dim() == 2 and proj.stride(1) == 1,
          "proj must be a CUDA [tokens, columns] tensor with unit column stride")
    _check(state, "state", (torch.float32,), 2)
    _need(state.shape[1] == mlstm_state_values(heads, dim, vdim), "state slots have the wrong size")
    for name, tensor in (("row_start", row_start), ("row_length", row_length), ("request_slots", request_slots)):
        _check(tensor, name, (torch.int32,), 1)
    rows = row_start.numel()
    _need(row_length.numel() == rows and request_slots.numel() >= rows, "row lists differ in length")
    for name, tensor in (("i_bias", i_bias), ("f_bias", f_bias)):
        _check(tensor, name, (torch.float32,), 1)
        _need(tensor.numel() == heads, f"{name} must have one value per head")
    q_off, k_off, v_off, i_off, f_off = (int(o) for o in offsets)
    _need(max(q_off + heads * dim, k_off + heads * dim, v_off + heads * vdim, i_off + heads, f_off + heads)
          <= proj.shape[1], "the column offsets reach beyond proj")
    _need(cap > 0.0, "the cap on the gates must be positive")
    tokens = proj.shape[0]
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=proj.device)
    _call("mxb_mlstm_scan", proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, i_off, f_off, i_bias.data_ptr(),
          f_bias.data_ptr(), float(cap), float(dim) ** -0.5, state.data_ptr(), state.stride(0), state.shape[0],
          row_start.data_ptr(), row_length.data_ptr(), request_slots.data_ptr(), out.data_ptr(), rows, heads, dim,
          vdim, _CODES[proj.dtype], int(longest), status_word(proj.device).data_ptr(), _stream())
    return out


def head_norm_gate(x: torch.Tensor, weight: torch.Tensor, gate: Optional[torch.Tensor], heads: int, eps: float,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """Each head of x (float32 ``[tokens, heads * vdim]``) over its root mean
    square, times ``weight`` (all heads' size), times sigmoid(gate) (same shape,
    rows may be strided)."""
    _check(x, "x", (torch.float32,), 2)
    _check(weight, "weight", (torch.float32,), 1)
    tokens, width = x.shape
    _need(width % heads == 0 and weight.numel() == width, "x, weight and the heads do not fit")
    gate_code, ldg = F32, 0
    if gate is not None:
        _need(gate.is_cuda and gate.dtype in _CODES and gate.dim() == 2 and gate.stride(1) == 1
              and gate.shape == x.shape, "gate must be [tokens, heads * vdim] with unit column stride")
        gate_code, ldg = _CODES[gate.dtype], gate.stride(0)
    _need(out_dtype in _CODES, "out_dtype must be float32 or bfloat16")
    out = torch.empty((tokens, width), dtype=out_dtype, device=x.device)
    _call("mxb_head_norm_gate", x.data_ptr(), weight.data_ptr(), _ptr(gate), ldg, gate_code, out.data_ptr(),
          _CODES[out_dtype], tokens, heads, width // heads, float(eps), _stream())
    return out


# ------------------------------------------------------------ the delta rule
def delta_rule_max_dim() -> int:
    return int(_fn("mxb_delta_rule_max_dim")())


def delta_rule(qkv: torch.Tensor, offsets, beta: torch.Tensor, step: torch.Tensor, step_bias: torch.Tensor,
               rate: torch.Tensor, state: torch.Tensor, row_start: torch.Tensor, row_length: torch.Tensor,
               request_slots: torch.Tensor, heads: int, groups: int, dim: int, vdim: int,
               longest: int = 0) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel over a step's
    tokens. ``qkv`` ``[tokens, columns]`` holds, from the column ``offsets``
    (q, k, v) on, groups * dim queries and keys and heads * vdim values (after
    their convolution and activation); head h reads group h // (heads / groups).
    ``beta`` ``[tokens, heads]`` of qkv's type (a view of a wider tensor will do)
    are the pre-activations of the write strength, ``step`` float32
    ``[tokens, heads * dim]`` those of the step size, to which ``step_bias``
    ``[heads * dim]`` is added; ``rate`` ``[heads]`` is positive. Per head:
    q and k become unit vectors (q times dim^-1/2), g = exp(-rate softplus(step
    + bias)), S <- g S (by rows); u = sigmoid(beta) (v - S^T k); S <- S + k u^T;
    o = S^T q. ``state`` float32 ``[slots, heads, vdim, dim]`` (S transposed: a
    value column's key channels side by side) is advanced in place; request row r brings ``row_length[r]`` tokens from packed token
    ``row_start[r]`` on (0: a padding row) and owns slot ``request_slots[r]``.
    Returns float32 ``[tokens, heads * vdim]``. ``longest``: the most tokens of
    a row if known (a step of single tokens gets smaller blocks)."""
    _need(qkv.is_cuda and qkv.dtype in _CODES and qkv.dim() == 2 and qkv.stride(1) == 1,
          "qkv must be a CUDA [tokens, columns] tensor with unit column stride")
    tokens = qkv.shape[0]
    _need(beta.is_cuda and beta.dtype == qkv.dtype and beta.dim() == 2 and beta.stride(1) == 1
          and beta.shape == (tokens, heads), "beta must be [tokens, heads] of qkv's type")
    _need(step.is_cuda and step.dtype == torch.float32 and step.dim() == 2 and step.stride(1) == 1
          and step.shape == (tokens, heads * dim), "step must be float32 [tokens, heads * dim]")
    _check(step_bias, "step_bias", (torch.float32,), 1)
    _check(rate, "rate", (torch.float32,), 1)
    _need(step_bias.numel() == heads * dim and rate.numel() == heads, "step_bias or rate has the wrong size")
    _check(state, "state", (torch.float32,), 4)
    _need(state.shape[1:] == (heads, vdim, dim), f"state must be [slots, {heads}, {vdim}, {dim}]")
    _need(heads % groups == 0 and 0 < dim <= delta_rule_max_dim(), "the head layout does not fit")
    for name, tensor in (("row_start", row_start), ("row_length", row_length), ("request_slots", request_slots)):
        _check(tensor, name, (torch.int32,), 1)
    rows = row_start.numel()
    _need(row_length.numel() == rows and request_slots.numel() >= rows, "row lists differ in length")
    q_off, k_off, v_off = (int(o) for o in offsets)
    _need(max(q_off + groups * dim, k_off + groups * dim, v_off + heads * vdim) <= qkv.shape[1],
          "the column offsets reach beyond qkv")
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=qkv.device)
    _call("mxb_delta_rule", qkv.data_ptr(), qkv.stride(0), q_off, k_off, v_off, beta.data_ptr(), beta.stride(0), 0,
          step.data_ptr(), step.stride(0), step_bias.data_ptr(), rate.data_ptr(), state.data_ptr(), state.stride(0),
          state.shape[0], row_start.data_ptr(), row_length.data_ptr(), request_slots.data_ptr(), out.data_ptr(), rows,
          heads, groups, dim, vdim, _CODES[qkv.dtype], int(longest), status_word(qkv.device).data_ptr(), _stream())
    return out


# ------------------------------------------------- attention through a latent
def latent_cache(x: torch.Tensor, weight: torch.Tensor, eps: float, rank: int, cache: Optional[torch.Tensor],
                 slots: Optional[torch.Tensor], positions: torch.Tensor, cos: Optional[torch.Tensor],
                 sin: Optional[torch.Tensor], interleaved: bool) -> Optional[torch.Tensor]:
    """x ``[tokens, rank + rot]`` (rows may be strided): the first ``rank``
    values are RMS-normed with ``weight``, the rest rotated by the positions,
    and both stored at ``slots`` of the one-plane pool
    ``[pages, 1, 1, page_tokens, rank + rot]``. Without a cache the rows are
    returned instead, ``[tokens, rank + rot]``."""
    _need(x.is_cuda and x.dtype in _CODES and x.dim() == 2 and x.stride(1) == 1, "x must be [tokens, rank + rot]")
    tokens = x.shape[0]
    rows = None
    if cache is None:
        _need(slots is None, "slots need a cache")
        rows = torch.empty((tokens, x.shape[1]), dtype=x.dtype, device=x.device)
        cache = rows.view(tokens, 1, 1, 1, x.shape[1])
    _check(cache, "cache", (x.dtype,), 5)
    num_pages, planes, kv_heads, page_tokens, width = cache.shape
    _need(planes == 1 and kv_heads == 1 and width == x.shape[1] and 0 < rank <= width,
          "cache must be [pages, 1, 1, page_tokens, rank + rot]")
    _check(weight, "weight", (torch.float32,), 1)
    _need(weight.numel() == rank, "the latent's norm weight has the wrong size")
    if rows is None:
        _check(slots, "slots", (torch.int32,), 1)
        _need(slots.numel() == tokens, "one slot per token")
    _check(positions, "positions", (torch.int32,), 1)
    _need(positions.numel() == tokens, "one position per token")
    rotary_dim, table_positions = _tables(cos, sin, width - rank)
    _call("mxb_latent_cache", x.data_ptr(), x.stride(0), weight.data_ptr(), float(eps), rank, width - rank, rotary_dim,
          1 if interleaved else 0, _ptr(cos), _ptr(sin), table_positions, positions.data_ptr(), _ptr(slots),
          cache.data_ptr(), page_tokens, num_pages, tokens, _CODES[x.dtype], status_word(x.device).data_ptr(),
          _stream())
    return rows


def latent_heads(q: torch.Tensor, up: torch.Tensor, shared: torch.Tensor, shared_off: int, q_heads: torch.Tensor,
                 cache: Optional[torch.Tensor], slots: Optional[torch.Tensor], positions: torch.Tensor,
                 cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], interleaved: bool, dim: int, rot: int,
                 vdim: int) -> None:
    """Whole key and value rows per head from what a latent was widened to.
    ``q`` ``[tokens, heads * (dim + rot)]`` (its rotated parts not yet rotated),
    ``up`` ``[tokens, heads * dim + heads * vdim]`` (every head's unrotated key
    part, then every head's values), ``shared[:, shared_off:shared_off + rot]``
    the already rotated key part all heads share. Writes ``q_heads``
    ``[tokens, heads, hd]`` = [q_u | rot(q_r) | 0] and, at ``slots`` of
    ``cache`` ``[pages, 2, heads, page_tokens, hd]``, K = [k_h | shared | 0]
    and V = [v_h | 0]."""
    dtype = q.dtype
    for name, tensor in (("q", q), ("up", up), ("shared", shared)):
        _need(tensor.is_cuda and tensor.dtype == dtype and tensor.dtype in _CODES and tensor.dim() == 2
              and tensor.stride(1) == 1, f"{name} must be a CUDA [tokens, columns] tensor with unit column stride")
    _check(q_heads, "q_heads", (dtype,), 3)
    tokens, heads, hd = q_heads.shape
    _need(q.shape == (tokens, heads * (dim + rot)) and up.shape == (tokens, heads * (dim + vdim))
          and shared.shape[0] == tokens and shared_off + rot <= shared.shape[1] and dim + rot <= hd and vdim <= hd,
          "q, up, shared and q_heads do not fit the head layout")
    num_pages, page_tokens = 0, 1
    if cache is not None:
        _check(cache, "cache", (dtype,), 5)
        _need(cache.shape[1] == 2 and cache.shape[2] == heads and cache.shape[4] == hd,
              "cache must be [pages, 2, heads, page_tokens, hd]")
        num_pages, page_tokens = cache.shape[0], cache.shape[3]
        _check(slots, "slots", (torch.int32,), 1)
        _need(slots.numel() == tokens, "one slot per token")
    _check(positions, "positions", (torch.int32,), 1)
    rotary_dim, table_positions = _tables(cos, sin, rot)
    _call("mxb_latent_heads", q.data_ptr(), q.stride(0), up.data_ptr(), up.stride(0), shared.data_ptr(), shared.stride(0),
          shared_off, q_heads.data_ptr(), _ptr(cache), _ptr(slots) if cache is not None else None, positions.data_ptr(),
          _ptr(cos), _ptr(sin), table_positions, rotary_dim, 1 if interleaved else 0, heads, dim, rot, vdim, hd,
          page_tokens, num_pages, tokens, _CODES[dtype], status_word(q.device).data_ptr(), _stream())


def _tables(cos, sin, width: int):
    if cos is None:
        return 0, 0
    _check(cos, "cos", (torch.float32,), 2)
    _check(sin, "sin", (torch.float32,), 2)
    _need(cos.shape == sin.shape and cos.shape[1] * 2 <= width, "cos and sin do not fit the rotated width")
    return cos.shape[1] * 2, cos.shape[0]


def rotate_into(src: torch.Tensor, src_off: int, src_step: int, dst: torch.Tensor, dst_off: int, rot: int,
                positions: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                interleaved: bool) -> None:
    """For every token and head: the ``rot`` values at
    ``src[token, src_off + head * src_step ...]`` rotated by the token's
    position into ``dst[token, head, dst_off ...]`` (dst ``[tokens, heads, step]``)."""
    _need(src.is_cuda and src.dtype in _CODES and src.dim() == 2 and src.stride(1) == 1, "src must be [tokens, columns]")
    _check(dst, "dst", (src.dtype,), 3)
    tokens, heads, step = dst.shape
    _need(src.shape[0] == tokens and src_off + (heads - 1) * src_step + rot <= src.shape[1] and dst_off + rot <= step,
          "the rotated values do not fit src or dst")
    _check(positions, "positions", (torch.int32,), 1)
    rotary_dim, table_positions = _tables(cos, sin, rot)
    _call("mxb_rotate_into", src.data_ptr(), src.stride(0), src_off, src_step, dst.data_ptr(), dst_off, step, heads, rot,
          rotary_dim, 1 if interleaved else 0, _ptr(cos), _ptr(sin), table_positions, positions.data_ptr(), tokens,
          _CODES[src.dtype], status_word(src.device).data_ptr(), _stream())


# ------------------------------------------------------- copies in the cache
def copy_units(pool: torch.Tensor, pairs: torch.Tensor) -> None:
    """pool[:, target] = pool[:, source] for every (source, target) row of
    ``pairs`` (int32 ``[count, 2]`` on the device); ``pool`` is contiguous
    ``[entries, units, ...]``: the pages of a group's layers, or (with a leading
    dimension of one) the slots of a state tensor. No target may be another
    pair's source."""
    _need(pool.is_cuda and pool.is_contiguous() and pool.dim() >= 2, "pool must be a contiguous device tensor")
    _need(pairs.is_cuda and pairs.dtype == torch.int32 and pairs.dim() == 2 and pairs.shape[1] == 2
          and pairs.is_contiguous(), "pairs must be int32 [count, 2] on the device")
    entries, units = pool.shape[0], pool.shape[1]
    unit_bytes = pool[0, 0].numel() * pool.element_size()
    _call("mxb_copy_units", pool.data_ptr(), entries, units, unit_bytes, pairs.data_ptr(), pairs.shape[0],
          status_word(pool.device).data_ptr(), _stream())


# ------------------------------------------------- q/k norm, rotation, cache
def qk_norm_rope_cache(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_out: Optional[torch.Tensor],
                       cache: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                       positions: torch.Tensor, q_weight: Optional[torch.Tensor],
                       k_weight: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                       sin: Optional[torch.Tensor], eps: float, interleaved: bool = False,
                       norm_scope: str = "head") -> None:
    """RMSNorm of q and k (if weights are given; ``norm_scope`` "head": each
    head by itself, weights of head_dim values; "projection": all of a token's
    query heads together and all of its key heads together, weights as wide as
    the projections), rotation by ``positions`` (if tables are given; pairs
    (i, i + rotary_dim / 2), or (2i, 2i + 1) when ``interleaved``), q written to ``q_out``
    [tokens, heads, head_dim], k and v written into ``cache``
    [pages, 2, kv_heads, page_tokens, head_dim] at ``slots`` (a negative slot
    skips the token; ``cache=None`` writes nothing). q, k and v are
    [tokens, heads * head_dim] views whose rows may be strided."""
    dtype = q.dtype
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        _need(tensor.is_cuda and tensor.dtype == dtype and tensor.dtype in _CODES and tensor.dim() == 2
              and tensor.stride(1) == 1, f"{name} must be a CUDA [tokens, width] tensor with unit column stride")
    tokens = q.shape[0]
    _check(positions, "positions", (torch.int32,), 1)
    _need(positions.numel() == tokens and k.shape[0] == tokens and v.shape[0] == tokens, "token counts differ")
    if cache is not None:
        _check(cache, "cache", (dtype,), 5)
        num_pages, two, kv_heads, page_tokens, head_dim = cache.shape
        _need(two == 2, "cache must be [pages, 2, kv_heads, page_tokens, head_dim]")
        _check(slots, "slots", (torch.int32,), 1)
        _need(slots.numel() == tokens, "one slot per token")
    else:
        _need(q_out is not None, "nothing to write")
        head_dim = q_out.shape[-1]
        kv_heads = k.shape[1] // head_dim
        num_pages, page_tokens = 0, 1
    _need(q.shape[1] % head_dim == 0 and k.shape[1] == kv_heads * head_dim and v.shape[1] == kv_heads * head_dim,
          "q, k, v widths do not match the head layout")
    heads = q.shape[1] // head_dim
    if q_out is not None:
        _check(q_out, "q_out", (dtype,), 3)
        _need(q_out.shape == (tokens, heads, head_dim), "q_out must be [tokens, heads, head_dim]")
    _need(norm_scope in ("head", "projection"), f"unknown norm scope {norm_scope!r}")
    for name, weight, width in (("q_weight", q_weight, heads * head_dim), ("k_weight", k_weight, kv_heads * head_dim)):
        if weight is not None:
            _check(weight, name, (torch.float32,), 1)
            if norm_scope == "head":
                _need(weight.numel() == head_dim, f"{name} must have head_dim values")
            else:
                _need(weight.numel() == width, f"{name} must have {width} values, one per value of the projection")
    rotary_dim, table_positions = 0, 0
    if cos is not None:
        _check(cos, "cos", (torch.float32,), 2)
        _check(sin, "sin", (torch.float32,), 2)
        _need(cos.shape == sin.shape, "cos and sin differ in shape")
        table_positions, rotary_dim = cos.shape[0], cos.shape[1] * 2
        _need(rotary_dim <= head_dim, "rotary_dim exceeds head_dim")
    _call("mxb_qk_norm_rope_cache", q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0),
          v.stride(0), _ptr(q_out), _ptr(cache), _ptr(slots), positions.data_ptr(), _ptr(q_weight),
          _ptr(k_weight), _ptr(cos), _ptr(sin), table_positions, rotary_dim, 1 if interleaved else 0,
          1 if norm_scope == "projection" else 0, tokens, heads, kv_heads,
          head_dim, page_tokens, num_pages, float(eps), _CODES[dtype],
          status_word(q.device).data_ptr(), _stream())


def norm_rotate_heads(x: torch.Tensor, head_dim: int, positions: torch.Tensor,
                      weight: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                      sin: Optional[torch.Tensor] = None, eps: float = 0.0, interleaved: bool = False,
                      norm_scope: str = "head") -> torch.Tensor:
    """RMSNorm (if ``weight``) and rotation (if tables) of x
    [tokens, n * head_dim]; returns [tokens, n, head_dim]. Writes no cache."""
    _need(x.dim() == 2 and x.shape[1] % head_dim == 0, "x must be [tokens, n * head_dim]")
    out = torch.empty((x.shape[0], x.shape[1] // head_dim, head_dim), dtype=x.dtype, device=x.device)
    empty = x[:, :0]
    qk_norm_rope_cache(x, empty, empty, out, None, None, positions, weight, None, cos, sin, eps,
                       interleaved=interleaved, norm_scope=norm_scope)
    return out


def write_cache(k: torch.Tensor, v: torch.Tensor, cache: torch.Tensor, slots: torch.Tensor,
                positions: torch.Tensor) -> None:
    """Stores k and v [tokens, kv_heads * head_dim] as they are at ``slots``."""
    qk_norm_rope_cache(k[:, :0], k, v, None, cache, slots, positions, None, None, None, None, 0.0)


# ------------------------------------------------------------------ attention
def _sink(sink, heads: int):
    """(has_sink, score, pointer) as the attention kernels take a sink: None for
    none, a number for one score that all heads share, or a float32 tensor
    ``[heads]`` with a score per query head."""
    if sink is None:
        return 0, 0.0, None
    if isinstance(sink, torch.Tensor):
        _need(sink.is_cuda and sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == heads,
              f"a sink per head must be {heads} contiguous float32 values on the device")
        return 1, 0.0, sink.data_ptr()
    return 1, float(sink), None


def paged_attention_tile(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor,
                         block_tables: torch.Tensor, tile_request: torch.Tensor,
                         tile_start: torch.Tensor, tile_length: torch.Tensor,
                         positions: torch.Tensor, scale: float, window: int = 0, chunk: int = 0,
                         gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                         gate_per_head: bool = False, sink=None) -> torch.Tensor:
    """Attention of every query token over its request's cached keys (itself
    included) in float32; q is [tokens, heads, head_dim], out
    [tokens, heads, value_dim] with value_dim at most head_dim (the first
    that many values of a value row). ``cache`` is
    [pages, planes, kv_heads, page_tokens, head_dim]: two planes hold keys and
    values, one plane holds rows that are keys and values at once. ``window``:
    only the last that many positions are seen; ``chunk``: only the keys of the
    query's own chunk of that many positions, counted from position 0;
    ``softcap`` c: scores pass c tanh(s / c) ahead of the softmax;
    ``gate`` ([tokens, heads * value_dim], or [tokens, heads] with
    ``gate_per_head``; rows may be strided): the output is multiplied by
    sigmoid(gate) as it is written; ``sink``: the score of one more key that
    has no value and that every query sees (0.0: one more in the softmax's
    denominator)."""
    dtype = q.dtype
    _check(q, "q", tuple(_CODES), 3)
    _check(out, "out", (dtype,), 3)
    _check(cache, "cache", (dtype,), 5)
    tokens, heads, head_dim = q.shape
    num_pages, planes, kv_heads, page_tokens, cache_dim = cache.shape
    _need(planes in (1, 2) and cache_dim == head_dim, "cache must be [pages, 1 or 2, kv_heads, page_tokens, head_dim]")
    value_dim = out.shape[2]
    _need(out.shape[:2] == q.shape[:2] and 0 < value_dim <= head_dim, "out must be [tokens, heads, value_dim <= head_dim]")
    _need(heads % kv_heads == 0, f"{heads} query heads cannot share {kv_heads} key/value heads")
    _need(0 < head_dim <= 576, f"head_dim {head_dim} is outside 1..576")
    _need(softcap >= 0.0, "the cap on the scores cannot be negative")
    _check(block_tables, "block_tables", (torch.int32,), 2)
    for name, tensor in (("tile_request", tile_request), ("tile_start", tile_start),
                         ("tile_length", tile_length), ("positions", positions)):
        _check(tensor, name, (torch.int32,), 1)
    tiles = tile_request.numel()
    _need(tile_start.numel() == tiles and tile_length.numel() == tiles, "tile lists differ in length")
    _need(positions.numel() == tokens, "one position per token")
    if gate is not None and gate_per_head:
        _need(gate.is_cuda and gate.dtype == dtype and gate.dim() == 2 and gate.stride(1) == 1
              and gate.shape == (tokens, heads), "a per-head gate must be [tokens, heads] in q's type")
        gate_stride = gate.stride(0)
    else:
        gate_stride = _gate_stride(gate, out)
    _call("mxb_paged_attention_tile", q.data_ptr(), cache.data_ptr(), out.data_ptr(),
          block_tables.data_ptr(), block_tables.shape[1], tile_request.data_ptr(),
          tile_start.data_ptr(), tile_length.data_ptr(), positions.data_ptr(), tiles, heads,
          kv_heads, head_dim, page_tokens, num_pages, int(window or 0), int(chunk or 0), float(scale), _CODES[dtype],
          _ptr(gate), gate_stride, planes, value_dim, float(softcap), 1 if gate_per_head else 0,
          *_sink(sink, heads), status_word(q.device).data_ptr(), _stream())
    return out


def flash_prefill_supported(head_dim: int, heads: int, kv_heads: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core prompt kernel takes this head layout."""
    if dtype not in _CODES:
        return False
    return bool(_fn("mxb_flash_prefill_supported")(head_dim, heads, kv_heads, _CODES[dtype]))


def flash_prefill_tile() -> int:
    """Query tokens per tile of the tensor-core prompt kernel."""
    return _fn("mxb_flash_prefill_tile")()


PROMPT_KERNEL = "auto"   # what flash_prefill's "auto" means: "auto", "tcgen05" or "mma" (for comparisons)


def flash_prefill_tcgen05_supported(head_dim: int, heads: int, kv_heads: int, page_tokens: int,
                                    dtype: torch.dtype) -> bool:
    """Whether the tcgen05 prompt kernel takes this head layout and page size."""
    if dtype not in _CODES:
        return False
    return bool(_fn("mxb_flash_prefill_tcgen05_supported")(head_dim, heads, kv_heads, page_tokens, _CODES[dtype]))


KEY_SHARES = None   # an int forces the number of blocks that share a query tile's keys (tests, comparisons)


def flash_key_shares(blocks: int, longest_context: int, window: int = 0, chunk: int = 0) -> int:
    """How many blocks share the keys of a query tile of the tcgen05 prompt
    kernel: one, unless the step has so few (tile, head) blocks and so many
    keys that most SMs would stand idle (a portion of a prompt behind a long
    context). Each share keeps at least 1,024 keys."""
    if KEY_SHARES is not None:
        return max(1, int(KEY_SHARES))
    keys = min(longest_context, window) if window else longest_context
    if chunk:
        keys = min(keys, chunk)
    if blocks >= 100 or keys < 2048:
        return 1
    return max(1, min(8, 148 // blocks, keys // 1024))


def flash_prefill(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_tables: torch.Tensor,
                  tile_request: torch.Tensor, tile_start: torch.Tensor, tile_length: torch.Tensor,
                  positions: torch.Tensor, scale: float, window: int = 0, kernel: str = "auto",
                  longest_context: int = 0, chunk: int = 0, gate: Optional[torch.Tensor] = None,
                  softcap: float = 0.0, sink=None) -> torch.Tensor:
    """Causal attention of prompt portions on the tensor cores (bfloat16,
    float32 softmax and accumulation); tiles hold up to 128 consecutive tokens
    of one request. ``kernel``: "tcgen05" (TMA, tensor memory), "mma" (the
    warp-level kernel) or "auto" (tcgen05 where it takes the page size).
    ``longest_context`` (the most keys any of the tiles sees, 0: unknown)
    lets the tcgen05 kernel share a tile's keys out among several blocks when
    the tiles alone would leave most of the GPU idle. ``softcap`` c: scores
    pass c tanh(s / c) ahead of the softmax. ``sink``: the score of one more
    key that has no value and that every query sees."""
    _need(softcap >= 0.0, "the cap on the scores cannot be negative")
    _check(q, "q", (torch.bfloat16,), 3)
    _check(out, "out", (torch.bfloat16,), 3)
    _check(cache, "cache", (torch.bfloat16,), 5)
    _need(out.shape == q.shape, "out and q differ in shape")
    tokens, heads, head_dim = q.shape
    num_pages, two, kv_heads, page_tokens, cache_dim = cache.shape
    _need(two == 2 and cache_dim == head_dim, "cache must be [pages, 2, kv_heads, page_tokens, head_dim]")
    _need(flash_prefill_supported(head_dim, heads, kv_heads, q.dtype),
          f"the tensor-core prompt kernel does not take head_dim {head_dim} with {heads}/{kv_heads} heads")
    _check(block_tables, "block_tables", (torch.int32,), 2)
    for name, tensor in (("tile_request", tile_request), ("tile_start", tile_start),
                         ("tile_length", tile_length), ("positions", positions)):
        _check(tensor, name, (torch.int32,), 1)
    tiles = tile_request.numel()
    _need(tile_start.numel() == tiles and tile_length.numel() == tiles, "tile lists differ in length")
    _need(positions.numel() == tokens, "one position per token")
    if kernel == "auto":
        kernel = PROMPT_KERNEL
    _need(kernel in ("auto", "tcgen05", "mma"), f"unknown prompt-attention kernel {kernel!r}")
    gate_stride = _gate_stride(gate, q)
    tcgen05 = flash_prefill_tcgen05_supported(head_dim, heads, kv_heads, page_tokens, q.dtype)
    if gate is not None and (gate.data_ptr() % 16 or (gate_stride * 2) % 16):
        tcgen05 = False   # its epilogue reads the gate 16 bytes at a time
    _need(tcgen05 or kernel != "tcgen05",
          f"the tcgen05 prompt kernel does not take head_dim {head_dim} with pages of {page_tokens} tokens")
    if tcgen05 and kernel != "mma":
        _need(q.is_contiguous() and cache.is_contiguous(), "q and cache must be contiguous")
        shares = flash_key_shares(tiles * heads, int(longest_context), int(window or 0), int(chunk or 0))
        partial = None
        if shares > 1:
            partial = torch.empty(tokens * heads * shares * (head_dim + 2), dtype=torch.float32, device=q.device)
        _call("mxb_flash_prefill_tcgen05", q.data_ptr(), cache.data_ptr(), out.data_ptr(),
              block_tables.data_ptr(), block_tables.shape[1], tile_request.data_ptr(), tile_start.data_ptr(),
              tile_length.data_ptr(), positions.data_ptr(), tokens, tiles, heads, kv_heads, head_dim,
              page_tokens, num_pages, int(window or 0), int(chunk or 0), float(scale), _CODES[q.dtype], shares, _ptr(partial),
              _ptr(gate), gate_stride, float(softcap), *_sink(sink, heads),
              status_word(q.device).data_ptr(), _stream())
        if shares > 1:
            global _launches
            _launches += 1   # the kernel that puts the shares together
        return out
    _call("mxb_flash_prefill", q.data_ptr(), cache.data_ptr(), out.data_ptr(), block_tables.data_ptr(),
          block_tables.shape[1], tile_request.data_ptr(), tile_start.data_ptr(), tile_length.data_ptr(),
          positions.data_ptr(), tiles, heads, kv_heads, head_dim, page_tokens, num_pages,
          int(window or 0), int(chunk or 0), float(scale), _CODES[q.dtype], _ptr(gate), gate_stride, float(softcap),
          *_sink(sink, heads), status_word(q.device).data_ptr(), _stream())
    return out


def decode_attention_supported(head_dim: int, heads: int, kv_heads: int, dtype: torch.dtype) -> bool:
    """Whether the split-key decode kernel takes this head layout."""
    if dtype not in _CODES:
        return False
    return bool(_fn("mxb_paged_attention_decode_supported")(head_dim, heads, kv_heads, _CODES[dtype]))


def decode_split_keys() -> int:
    return _fn("mxb_paged_attention_split_keys")()


def set_decode_resident_blocks(blocks: int, many: int = 2048) -> None:
    """How many blocks of the bfloat16 decode attention the GPU holds at once
    (444: three on each of 148 SMs), and into how many blocks a step with more
    (token, key/value head) pairs than that is cut (2,048). A pair gets that
    many blocks divided by the number of pairs, each walking over its 128-key
    tiles; where a block would be left fewer than two tiles, and with
    ``blocks`` 0, every tile has a block of its own. For comparisons and tests."""
    _need(_fn("mxb_set_decode_resident_blocks")(int(blocks), int(many)) == 0,
          "the number of resident blocks cannot be negative nor exceed that of a step with many pairs")


def paged_attention_decode(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor,
                           block_tables: torch.Tensor, row_token: torch.Tensor,
                           row_request: torch.Tensor, positions: torch.Tensor, scale: float,
                           longest_context: int, window: int = 0,
                           partial: Optional[torch.Tensor] = None, chunk: int = 0,
                           gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                           sink=None) -> torch.Tensor:
    """Attention of single tokens over their requests' cached keys, split
    along the keys. ``row_token[i]`` is the token (row of q and out) of the
    i-th decoded request, negative for a padding row; ``row_request[i]`` its
    row of ``block_tables``. ``longest_context`` bounds positions + 1 and
    fixes the number of splits. ``partial`` is float32 scratch of
    rows * heads * splits * (head_dim + 2) values, allocated here if absent.
    ``gate`` ([tokens, heads * head_dim] in q's type, rows may be strided):
    the output is multiplied by sigmoid(gate) as it is written. ``softcap`` c:
    scores pass c tanh(s / c) ahead of the softmax. ``sink``: the score of one
    more key that has no value and that every query sees (it joins the
    denominator where the splits are put together)."""
    dtype = q.dtype
    _need(softcap >= 0.0, "the cap on the scores cannot be negative")
    _check(q, "q", tuple(_CODES), 3)
    _check(out, "out", (dtype,), 3)
    _check(cache, "cache", (dtype,), 5)
    _need(out.shape == q.shape, "out and q differ in shape")
    tokens, heads, head_dim = q.shape
    num_pages, two, kv_heads, page_tokens, cache_dim = cache.shape
    _need(two == 2 and cache_dim == head_dim, "cache must be [pages, 2, kv_heads, page_tokens, head_dim]")
    _need(decode_attention_supported(head_dim, heads, kv_heads, dtype),
          f"the split-key decode kernel does not take head_dim {head_dim} with {heads}/{kv_heads} heads in {dtype}")
    _check(block_tables, "block_tables", (torch.int32,), 2)
    for name, tensor in (("row_token", row_token), ("row_request", row_request), ("positions", positions)):
        _check(tensor, name, (torch.int32,), 1)
    rows = row_token.numel()
    _need(row_request.numel() == rows and positions.numel() == tokens, "row lists do not fit")
    splits = max(1, -(-int(longest_context) // decode_split_keys()))
    need = rows * heads * splits * (head_dim + 2)
    if partial is None:
        partial = torch.empty(need, dtype=torch.float32, device=q.device)
    _check(partial, "partial", (torch.float32,))
    _need(partial.numel() >= need, f"partial holds {partial.numel()} values, {need} are needed")
    gate_stride = _gate_stride(gate, q)
    _call("mxb_paged_attention_decode", q.data_ptr(), cache.data_ptr(), out.data_ptr(), partial.data_ptr(),
          block_tables.data_ptr(), block_tables.shape[1], row_token.data_ptr(), row_request.data_ptr(),
          positions.data_ptr(), rows, heads, kv_heads, head_dim, page_tokens, num_pages, splits,
          int(window or 0), int(chunk or 0), float(scale), _CODES[dtype], _ptr(gate), gate_stride, float(softcap),
          *_sink(sink, heads), status_word(q.device).data_ptr(), _stream())
    return out


def _gate_stride(gate: Optional[torch.Tensor], q: torch.Tensor) -> int:
    """Checks an output gate against q [tokens, heads, head_dim]; its row stride."""
    if gate is None:
        return 0
    tokens, heads, head_dim = q.shape
    _need(gate.is_cuda and gate.dtype == q.dtype and gate.dim() == 2 and gate.stride(1) == 1
          and gate.shape == (tokens, heads * head_dim), "gate must be [tokens, heads * head_dim] in q's type")
    _need(gate.data_ptr() % 4 == 0 and gate.stride(0) % 2 == 0, "gate rows must start on 4-byte boundaries")
    return gate.stride(0)


def decode_project_supported(head_dim: int, heads: int, kv_heads: int, dtype: torch.dtype, tokens: int,
                             weight: torch.Tensor) -> bool:
    """Whether ``paged_attention_decode_project`` takes this shape."""
    if dtype not in _CODES or weight.dtype != torch.bfloat16 or weight.dim() != 2 or weight.stride(1) != 1:
        return False
    return bool(_fn("mxb_paged_attention_decode_project_supported")(
        head_dim, heads, kv_heads, _CODES[dtype], tokens, weight.data_ptr(), weight.stride(0)))


def paged_attention_decode_project(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                                   row_token: torch.Tensor, row_request: torch.Tensor, positions: torch.Tensor,
                                   scale: float, longest_context: int, weight: torch.Tensor,
                                   window: int = 0, chunk: int = 0,
                                   gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                                   sink=None) -> torch.Tensor:
    """``paged_attention_decode`` followed at once by the output projection
    ``weight`` ``[hidden, heads * head_dim]``, for steps of up to 64 tokens in
    bfloat16. Returns float32 ``[heads, tokens, hidden]``: the projection's sum
    over k left in one summand per head, for ``add_rmsnorm`` to add up. With
    ``gate`` the heads' output is multiplied by sigmoid(gate) ahead of the projection."""
    _check(q, "q", (torch.bfloat16,), 3)
    _check(cache, "cache", (torch.bfloat16,), 5)
    tokens, heads, head_dim = q.shape
    num_pages, two, kv_heads, page_tokens, cache_dim = cache.shape
    _need(two == 2 and cache_dim == head_dim, "cache must be [pages, 2, kv_heads, page_tokens, head_dim]")
    _need(weight.is_cuda and weight.dim() == 2 and weight.shape[1] == heads * head_dim, "weight does not fit the heads")
    _need(decode_project_supported(head_dim, heads, kv_heads, q.dtype, tokens, weight),
          f"the decode kernel with the projection does not take {tokens} tokens of {heads}/{kv_heads} heads of {head_dim}")
    _check(block_tables, "block_tables", (torch.int32,), 2)
    for name, tensor in (("row_token", row_token), ("row_request", row_request), ("positions", positions)):
        _check(tensor, name, (torch.int32,), 1)
    rows = row_token.numel()
    _need(row_request.numel() == rows and positions.numel() == tokens, "row lists do not fit")
    splits = max(1, -(-int(longest_context) // decode_split_keys()))
    partial = torch.empty(rows * heads * splits * (head_dim + 2), dtype=torch.float32, device=q.device)
    hidden = weight.shape[0]
    summands = torch.empty((heads, tokens, hidden), dtype=torch.float32, device=q.device)
    gate_stride = _gate_stride(gate, q)
    _call("mxb_paged_attention_decode_project", q.data_ptr(), cache.data_ptr(), partial.data_ptr(),
          block_tables.data_ptr(), block_tables.shape[1], row_token.data_ptr(), row_request.data_ptr(),
          positions.data_ptr(), rows, tokens, heads, kv_heads, head_dim, page_tokens, num_pages, splits,
          int(window or 0), int(chunk or 0), float(scale), weight.data_ptr(), weight.stride(0), hidden, summands.data_ptr(),
          _ptr(gate), gate_stride, float(softcap), *_sink(sink, heads),
          status_word(q.device).data_ptr(), _stream())
    return summands


# ------------------------------------------------------------ matrix products
def gemm_simple(a: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [m, k] times w [n, k] transposed on CUDA cores, float32 accumulation
    in a fixed order."""
    _need(a.is_cuda and w.is_cuda, "operands must be on a CUDA device")
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "shapes do not match a @ w.T")
    _need(a.dtype == w.dtype and a.dtype in _CODES, "operands must share float32 or bfloat16")
    _need(a.stride(1) == 1 and w.stride(1) == 1, "rows must be contiguous")
    out_dtype = out_dtype or a.dtype
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    _need(out.shape == (m, n) and out.dtype == out_dtype and out.stride(1) == 1, "out does not fit")
    _call("mxb_gemm_simple", out.data_ptr(), _CODES[out_dtype], a.data_ptr(), w.data_ptr(),
          _CODES[a.dtype], m, n, k, a.stride(0), w.stride(0), out.stride(0), _stream())
    return out


# Up to this many rows "auto" takes the weight-streaming kernel; beyond it every
# block would re-read too much of x and the library product is faster.
SKINNY_ROWS = 16


def gemm_skinny_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes a [m, k] times w [n, k]
    transposed: bfloat16, at most 64 rows, k a multiple of 32, rows on 16-byte
    boundaries."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        return False
    if a.stride(1) != 1 or w.stride(1) != 1 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    return bool(_fn("mxb_gemm_skinny_supported")(a.shape[0], w.shape[0], a.shape[1], a.stride(0), w.stride(0)))


STREAM_COLUMNS = 16384   # wider outputs (the vocabulary) keep the load-based kernel: enough blocks hide its latency


def gemm_stream_supported(a: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> bool:
    """Whether the bulk-copy weight-streaming kernel takes a [m, k] times w
    [n, k] transposed: bfloat16, at most 16 rows, k a multiple of 16, rows on
    16-byte boundaries, a block's rows of w and a fitting shared memory."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        return False
    if a.stride(1) != 1 or w.stride(1) != 1 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    n = w.shape[0]
    if swiglu and n % 2:
        return False
    return bool(_fn("mxb_gemm_stream_supported")(a.shape[0], n, a.shape[1], a.stride(0), w.stride(0),
                                                 n // 2 if swiglu else 0))


# With rows of W longer than STREAM_K the load-based kernel is ahead of the
# library up to this many columns (at 1 / 8 rows 3.2 / 3.1 against 2.5 / 2.7 TB/s
# on 4,096 x 4,096, 4.1 / 3.9 against 3.1 / 3.3 on 4,096 x 12,288) and behind it
# from 5,120 columns on (4.4 / 4.1 against 4.8 / 4.8 TB/s on 5,120 x 8,192, 5.2 /
# 5.0 against 5.7 / 5.8 on 5,120 x 25,600, 4.3 / 4.1 against 4.8 / 5.1 on 10,240 x
# 5,120), until the width of a vocabulary gives it thousands of blocks.
LOAD_COLUMNS = 4096
STREAM_K = 3072   # beyond this k the load-based kernel reads W faster than whole rows by bulk copy


def gemm_skinny_takes(a: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> bool:
    """Whether one of the two weight-streaming kernels takes the call."""
    return gemm_stream_supported(a, w, swiglu) or gemm_skinny_supported(a, w)


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}   # act of a gated feed-forward, act(gate) * up


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                swiglu: bool = False, out: Optional[torch.Tensor] = None, kernel: str = "auto",
                activation: str = "silu") -> torch.Tensor:
    """a [m <= 64, k] times w [n, k] transposed, reading w once. With
    ``swiglu`` w holds gate rows then up rows and the result is
    act(gate) * up, [m, n / 2], act being ``activation`` ("silu", "gelu_tanh"). ``kernel``: "stream" (rows of w by bulk copy
    into shared memory, m <= 16), "load" (16-byte loads into registers) or
    "auto": stream where it takes the shape, the output is not wider than
    STREAM_COLUMNS and k is at most STREAM_K (the layers of a small model,
    where fetching W ahead of the wait for x is what counts; with the long
    rows of a large model the loads read faster: 4.8 against 3.2 TB/s on
    [8, 25600] x [5120, 25600])."""
    _need(a.is_cuda and w.is_cuda and a.shape[1] == w.shape[1], "operands do not fit a @ w.T on a CUDA device")
    _need(kernel in ("auto", "stream", "load"), f"unknown weight-streaming kernel {kernel!r}")
    streams = kernel != "load" and gemm_stream_supported(a, w, swiglu)
    _need(streams or kernel != "stream", "the bulk-copy kernel does not take this shape")
    _need(streams or gemm_skinny_supported(a, w), "the weight-streaming kernels take bfloat16, at most 64 rows, "
          "k a multiple of 32 (16 up to 16 rows) and rows on 16-byte boundaries")
    _need(out_dtype in (torch.bfloat16, torch.float32), "out_dtype must be bfloat16 or float32")
    m, k = a.shape
    n = w.shape[0]
    _need(not swiglu or n % 2 == 0, "gate and up rows must pair up")
    columns = n // 2 if swiglu else n
    if out is None:
        out = torch.empty((m, columns), dtype=out_dtype, device=a.device)
    _need(out.shape == (m, columns) and out.dtype == out_dtype and out.stride(1) == 1, "out does not fit")
    loads = gemm_skinny_supported(a, w)
    if streams and (kernel == "stream" or not loads or (columns <= STREAM_COLUMNS and k <= STREAM_K)):
        _call("mxb_gemm_stream", out.data_ptr(), _CODES[out_dtype], a.data_ptr(), w.data_ptr(), m, n, k,
              a.stride(0), w.stride(0), out.stride(0), columns if swiglu else 0, GATE_ACTIVATIONS[activation],
              status_word(a.device).data_ptr(), _stream())
        return out
    _call("mxb_gemm_skinny", out.data_ptr(), _CODES[out_dtype], a.data_ptr(), w.data_ptr(), m, n, k,
          a.stride(0), w.stride(0), out.stride(0), columns if swiglu else 0, GATE_ACTIVATIONS[activation], _stream())
    return out


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
              backend: str = "auto", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bfloat16 a [m, k] times w [n, k] transposed with float32 accumulation.

    ``backend``: "skinny" is the weight-streaming kernel for at most 64 rows,
    "tcgen05" the hand-written tensor-core kernel, "cublas" the library product
    (where the reference calls a library matmul too), "simple" the plain
    CUDA-core kernel. "auto": the weight-streaming kernel up to 16 rows, else
    the library for a plain product (fused products pick the tcgen05 kernel
    themselves, see ``parts/feed_forward.py``)."""
    _need(a.is_cuda and w.is_cuda, "operands must be on a CUDA device")
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "operands must be bfloat16")
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "shapes do not match a @ w.T")
    _need(out_dtype in (torch.bfloat16, torch.float32), "out_dtype must be bfloat16 or float32")
    if backend == "simple":
        return gemm_simple(a, w, out_dtype=out_dtype, out=out)
    # "auto": up to 16 rows; with the long rows of a large model up to 8 (beyond
    # that the library reads them faster: 8B-shaped decode steps of 9 to 16
    # requests took 5.6 ms, of 18 to 24 requests through the library 5.0)
    few = SKINNY_ROWS if a.shape[1] <= STREAM_K else SKINNY_ROWS // 2
    if a.shape[1] > STREAM_K and LOAD_COLUMNS < w.shape[0] <= STREAM_COLUMNS:
        few = 0   # long rows and a middling width: the library reads these faster at any row count
    if (backend == "skinny" or (backend == "auto" and a.shape[0] <= few)) and gemm_skinny_takes(a, w):
        return gemm_skinny(a, w, out_dtype=out_dtype, out=out)
    _need(backend != "skinny", "the weight-streaming kernel does not take this shape")
    if backend == "tcgen05":
        from . import tensor_core
        _need(tensor_core.supports(a, w, out_dtype), "the tcgen05 kernel does not take this call: "
              + tensor_core.why_not(a, w, out_dtype))
        return tensor_core.gemm(a, w, out_dtype=out_dtype, out=out)
    if backend not in ("auto", "cublas"):
        raise KernelError(f"unknown gemm backend {backend!r}")
    # "auto" beyond the few rows of a decode step: a plain product goes to the
    # library, as in the reference (its 2-SM tiles beat the one-SM tcgen05
    # kernel here by 1.2x to 2x on this model's shapes); the tcgen05 kernel runs
    # where the product is fused with what follows it (SwiGLU).
    if out_dtype == torch.float32:
        result = torch.mm(a, w.t(), out_dtype=torch.float32)
    else:
        result = torch.mm(a, w.t())
    if out is not None:
        out.copy_(result)
        return out
    return result


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, activation: str = "silu") -> torch.Tensor:
    """out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i], float32 inside; act is
    silu, or with ``activation="gelu_tanh"`` the tanh form of gelu."""
    _check(gate_up, "gate_up", tuple(_CODES), 2)
    tokens, width = gate_up.shape
    _need(width % 2 == 0, "gate_up must hold gate and up side by side")
    inter = width // 2
    if out is None:
        out = torch.empty((tokens, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(out, "out", (gate_up.dtype,), 2)
    _need(out.shape == (tokens, inter), "out has the wrong shape")
    _call("mxb_silu_mul", out.data_ptr(), gate_up.data_ptr(), _CODES[gate_up.dtype], tokens, inter,
          GATE_ACTIVATIONS[activation], _stream())
    return out


# -------------------------------------------------------------------- picking
def _logit_rows(logits: torch.Tensor):
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1,
          "logits must be CUDA float32 [rows, vocab] with contiguous rows")
    _need(logits.shape[0] <= 65535, f"the pick kernels take up to 65535 rows at a time, not {logits.shape[0]}")
    return logits.shape[0], logits.shape[1], logits.stride(0)


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Lowest index of each row's maximum; -1 and a status bit for a row with
    a non-finite value."""
    rows, vocab, stride = _logit_rows(logits)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(out, "out", (torch.int32,), 1)
    # the first pass leaves one (value, index) pair per piece of a row here
    scratch = torch.empty(rows * _fn("mxb_argmax_pieces")(rows, vocab), dtype=torch.int64, device=logits.device)
    _call("mxb_argmax", logits.data_ptr(), stride, rows, vocab, out.data_ptr(), scratch.data_ptr(),
          status_word(logits.device).data_ptr(), _stream())
    global _launches
    _launches += 1   # two kernels
    return out


def sample_icdf(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor,
                stream_id: torch.Tensor, position: torch.Tensor, legal: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inverse-CDF temperature sampling in token-id order, float64 weights;
    the uniform of row r is a function of (seed[r], stream_id[r], position[r])."""
    rows, vocab, stride = _logit_rows(logits)
    _check(temperature, "temperature", (torch.float64,), 1)
    _check(seed, "seed", (torch.int64, torch.uint64), 1)
    _check(stream_id, "stream_id", (torch.int64, torch.uint64), 1)
    _check(position, "position", (torch.int32,), 1)
    _need(temperature.numel() == rows and seed.numel() == rows and stream_id.numel() == rows
          and position.numel() == rows, "one temperature, seed, stream and position per row")
    if legal is not None:
        _check(legal, "legal", (torch.uint8, torch.bool), 2)
        _need(legal.shape == (rows, vocab), "legal must be [rows, vocab]")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    # per piece of a row: its maximum, its weight, its last id of positive weight
    scratch = torch.empty(3 * rows * _fn("mxb_icdf_pieces")(vocab), dtype=torch.int64, device=logits.device)
    _call("mxb_sample_icdf", logits.data_ptr(), stride, rows, vocab, temperature.data_ptr(),
          seed.data_ptr(), stream_id.data_ptr(), position.data_ptr(), _ptr(legal), out.data_ptr(),
          scratch.data_ptr(), status_word(logits.device).data_ptr(), _stream())
    global _launches
    _launches += 2   # three kernels
    return out


def sample_race(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor,
                position: torch.Tensor, legal: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gumbel-max sampling with Philox noise keyed by (seed, position, id)."""
    rows, vocab, stride = _logit_rows(logits)
    _check(temperature, "temperature", (torch.float64,), 1)
    _check(seed, "seed", (torch.int64, torch.uint64), 1)
    _check(position, "position", (torch.int32,), 1)
    _need(temperature.numel() == rows and seed.numel() == rows and position.numel() == rows,
          "one temperature, seed and position per row")
    if legal is not None:
        _check(legal, "legal", (torch.uint8, torch.bool), 2)
        _need(legal.shape == (rows, vocab), "legal must be [rows, vocab]")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    scratch = torch.empty(2 * rows * _fn("mxb_argmax_pieces")(rows, vocab), dtype=torch.int64, device=logits.device)
    _call("mxb_sample_race", logits.data_ptr(), stride, rows, vocab, temperature.data_ptr(),
          seed.data_ptr(), position.data_ptr(), _ptr(legal), out.data_ptr(), scratch.data_ptr(),
          status_word(logits.device).data_ptr(), _stream())
    global _launches
    _launches += 1   # two kernels
    return out


def nucleus_mask(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor,
                 top_k: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """uint8 [rows, vocab]: 1 where a token is inside the row's top-k then
    top-p nucleus (descending logit, lower id first on ties)."""
    rows, vocab, stride = _logit_rows(logits)
    _check(temperature, "temperature", (torch.float64,), 1)
    _check(top_p, "top_p", (torch.float64,), 1)
    _check(top_k, "top_k", (torch.int32,), 1)
    _need(temperature.numel() == rows and top_p.numel() == rows and top_k.numel() == rows,
          "one temperature, top_p and top_k per row")
    _need(vocab <= 1 << 22, f"the top-k/top-p kernel takes vocabularies up to {1 << 22} ids, not {vocab}")
    if out is None:
        out = torch.empty((rows, vocab), dtype=torch.uint8, device=logits.device)
    _check(out, "out", (torch.uint8,), 2)
    _call("mxb_nucleus_mask", logits.data_ptr(), stride, rows, vocab, temperature.data_ptr(),
          top_p.data_ptr(), top_k.data_ptr(), out.data_ptr(), status_word(logits.device).data_ptr(),
          _stream())
    return out
