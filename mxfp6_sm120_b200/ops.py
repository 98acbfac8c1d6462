"""Python operator surface of the B200 W6A8 library.

Names, argument meaning and error behaviour follow the reference's
``python/mxfp6/ops.py`` so that callers can switch libraries; every function
forwards raw device pointers to the C ABI in ``libmxfp6_b200.so``.  There is no
fallback: a missing library raises ``ImportError`` and a non-sm_100 GPU raises
``RuntimeError``.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from ._loader import check, library, load_library

SCALE_VECTOR_SIZE = 32
# (N, K) pairs the static tile/split-K table was measured on: the dense
# projections of a 27B-class decoder (hidden 5120, intermediate 17408).
TUNED_NK = frozenset(
    {
        (7168, 5120),
        (5120, 6144),
        (34816, 5120),
        (5120, 17408),
        (2048, 5120),
    }
)
TUNED_M = frozenset((1, 2, 4, 8, 16, 24, 32, 64, 96, 512, 1024, 2048, 4096, 8192))

_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1}


# MXFP6_AUTOTUNE=on / cache_only makes gemm() tune (or look up) a shape on its first use; read
# once at import so that the hot path pays one global load.
_AUTOTUNE_ON_FIRST_USE = os.environ.get("MXFP6_AUTOTUNE", "off").strip().lower() not in (
    "", "0", "false", "no", "off")


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def _require_cuda_uint8_contiguous(tensor: torch.Tensor, name: str) -> None:
    if tensor.device.type != "cuda":
        raise ValueError(f"{name} must be a CUDA tensor; got {tensor.device}")
    if tensor.dtype != torch.uint8:
        raise TypeError(f"{name} must have dtype torch.uint8; got {tensor.dtype}")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _require_sm100(device: torch.device) -> None:
    index = device.index if device.index is not None else torch.cuda.current_device()
    capability = torch.cuda.get_device_capability(index)
    if capability != (10, 0):
        raise RuntimeError(
            f"MXFP6 native GEMM requires SM100 (B200); device {index} is "
            f"SM{capability[0]}{capability[1]}"
        )


def _resolve_device(device: torch.device | str | int | None) -> torch.device:
    if device is None:
        resolved = torch.device("cuda", torch.cuda.current_device())
    elif isinstance(device, int) and not isinstance(device, bool):
        resolved = torch.device("cuda", device)
    else:
        resolved = torch.device(device)
    if resolved.type != "cuda":
        raise ValueError(f"workspace device must be CUDA; got {resolved}")
    if resolved.index is None:
        resolved = torch.device("cuda", torch.cuda.current_device())
    _require_sm100(resolved)
    load_library()
    return resolved


_STAT_KEYS = (
    "layouts",
    "max_reduction_bytes",
    "max_barrier_bytes",
    "arena_bytes",
    "lanes",
    "total_arena_bytes",
    "planning",
    "frozen",
    "persistent_launches",
    "fallback_launches",
)


def begin_workspace_planning(device: torch.device | str | int | None = None) -> None:
    """Collect split-K workspace layouts selected during subsequent warm-up."""
    resolved = _resolve_device(device)
    with torch.cuda.device(resolved):
        check(library().mxfp6_workspace_begin_planning())


def finalize_workspace_planning(
    device: torch.device | str | int | None = None,
) -> dict[str, int]:
    """Freeze the arena capacity and allocate its current-stream lane."""
    resolved = _resolve_device(device)
    stats = (ctypes.c_int64 * 10)()
    with torch.cuda.device(resolved):
        check(library().mxfp6_workspace_finalize_planning(_stream(resolved), stats))
    return dict(zip(_STAT_KEYS, (int(v) for v in stats)))


def workspace_stats(device: torch.device | str | int | None = None) -> dict[str, int]:
    """Return planner capacity and launch counters for ``device``."""
    resolved = _resolve_device(device)
    stats = (ctypes.c_int64 * 10)()
    with torch.cuda.device(resolved):
        check(library().mxfp6_workspace_stats(stats))
    return dict(zip(_STAT_KEYS, (int(v) for v in stats)))


def workspace_barriers_zero(device: torch.device | str | int | None = None) -> bool:
    """Synchronize and verify every frozen lane's counter tail is zero."""
    resolved = _resolve_device(device)
    flag = ctypes.c_int(0)
    with torch.cuda.device(resolved):
        check(library().mxfp6_workspace_barriers_zero(ctypes.byref(flag)))
    return bool(flag.value)


def device_status(device: torch.device | str | int | None = None, reset: bool = True) -> int:
    """Synchronize and return the bounded-wait status word (0 = no wait expired)."""
    resolved = _resolve_device(device)
    value = ctypes.c_int(0)
    with torch.cuda.device(resolved):
        check(library().mxfp6_b200_device_status(ctypes.byref(value), int(reset)))
    return int(value.value)


_SPLIT_MODES = {"cluster": 1, "workspace": 2, "off": 3}


def set_split_k_mode(mode: str) -> None:
    """Choose how launches with too few tiles split K.

    ``"cluster"`` (default): thread-block clusters reduce through distributed shared
    memory, no scratch.  ``"workspace"``: FP32 partial tiles in the split-K arena
    (the reference's Stream-K workspace model).  ``"off"``: never split.
    """
    if mode not in _SPLIT_MODES:
        raise ValueError(f"mode must be one of {sorted(_SPLIT_MODES)}")
    check(library().mxfp6_set_split_k_mode(_SPLIT_MODES[mode]))


def set_cta_pair_mode(enabled: bool) -> None:
    """Run dense launches with m > 128, n % 128 == 0 and n >= 256 on CTA pairs (default) or not."""
    check(library().mxfp6_set_cta_pair_mode(1 if enabled else 0))


def is_cta_pair_enabled() -> bool:
    return library().mxfp6_get_cta_pair_mode() == 1


def set_stream_kernel_mode(enabled: bool) -> None:
    """Run dense launches of at most 64 rows on the weight-streaming kernel (default) or not."""
    check(library().mxfp6_set_stream_kernel_mode(1 if enabled else 0))


def is_stream_kernel_enabled() -> bool:
    return library().mxfp6_get_stream_kernel_mode() == 1


_KERNEL_NAMES = ("persistent", "cta_pair", "stream")


def w6a8_config_abi(anchor: torch.Tensor | None = None) -> str:
    """Name of the set of explicit GEMM configurations (ids mean nothing under another name).

    ``anchor`` is accepted for the reference's signature (it only selects the device there).
    """
    return library().mxfp6_w6a8_config_abi().decode()


def w6a8_configs() -> list[dict[str, int | str]]:
    """Every explicit configuration: id, kernel family, token tile, cluster and scratch split."""
    lib = library()
    rows = []
    for config_id in range(lib.mxfp6_w6a8_config_count()):
        out = (ctypes.c_int * 4)()
        check(lib.mxfp6_w6a8_config_describe(config_id, out))
        rows.append({"config_id": config_id, "kernel": _KERNEL_NAMES[out[0]],
                     "tile_tokens": int(out[1]), "cluster_k": int(out[2]), "splits": int(out[3])})
    return rows


def set_w6a8_config(
    anchor: torch.Tensor | torch.device | str | int | None,
    m: int,
    n: int,
    k: int,
    config_id: int,
    swizzle: int = 1,
    raster_order: int = 0,
    output_dtype: torch.dtype | None = None,
) -> bool:
    """Pin one exact ``(m, n, k, output dtype)`` problem on ``anchor``'s device to a configuration.

    Later :func:`gemm_w6a8` / :func:`gemm_from_float` calls with that shape run
    ``config_id`` (see :func:`w6a8_configs`); a negative id removes the entry.
    ``swizzle`` and ``raster_order`` are scheduler knobs of the reference's kernels
    and are validated, then ignored: the kernels here have one tile order.
    """
    if swizzle not in (1, 2, 4, 8):
        raise ValueError(f"swizzle must be 1, 2, 4 or 8; got {swizzle}")
    if raster_order not in (0, 1, 2):
        raise ValueError(f"raster_order must be 0, 1 or 2; got {raster_order}")
    _validate_problem(m, n, k)
    dtype = _validate_output_dtype(torch.float16 if output_dtype is None else output_dtype)
    device = anchor.device if isinstance(anchor, torch.Tensor) else anchor
    resolved = _resolve_device(device)
    with torch.cuda.device(resolved):
        check(library().mxfp6_set_w6a8_config(m, n, k, _DTYPE_CODE[dtype], int(config_id)))
    return True


def is_stream_k_enabled() -> bool:
    """Whether split-K uses the workspace arena (the reference's MXFP6_STREAM_K switch)."""
    return library().mxfp6_get_split_k_mode() == 2


def _refuse(failed: bool, message: str, kind: type[Exception] = ValueError) -> None:
    """One line per argument rule: raise ``kind(message)`` when the rule is broken."""
    if failed:
        raise kind(message)


def _validate_problem(m: int, n: int, k: int) -> None:
    _refuse(m <= 0, f"m must be positive; got {m}")
    _refuse(n <= 0 or n % 8 != 0, f"n must be a positive multiple of 8; got {n}")
    _refuse(k <= 0 or k % 128 != 0, f"k must be a positive multiple of 128; got {k}")


def _validate_output_dtype(out_dtype: torch.dtype) -> torch.dtype:
    _refuse(out_dtype not in _DTYPE_CODE,
            f"out_dtype must be torch.float16 or torch.bfloat16; got {out_dtype}", TypeError)
    return out_dtype


class _Operand:
    """What both operand containers share: where the bytes live and the logical extent."""

    values: torch.Tensor
    rows: int
    k: int

    @property
    def device(self) -> torch.device:
        return self.values.device

    @property
    def shape(self) -> tuple[int, int]:
        return (self.rows, self.k)


@dataclass(frozen=True)
class PackedMXFP6Tensor(_Operand):
    """MXFP6 operand as the kernels read it: ``values`` = E3M2 codes, four per three bytes,
    row-major ``[rows, 3k/4]`` flattened; ``scales`` = UE8M0 bytes in 128 x 4 atoms;
    ``logical_scales`` = the same scales as ``[rows, k/32]`` when the producer kept them."""

    values: torch.Tensor
    scales: torch.Tensor
    rows: int
    k: int
    logical_scales: torch.Tensor | None = None


@dataclass(frozen=True)
class MXFP8Tensor(_Operand):
    """MXFP8 activation: ``values`` = one E4M3 byte per element, ``[rows, k]`` flattened;
    ``scales`` = UE8M0 bytes in 128 x 4 atoms."""

    values: torch.Tensor
    scales: torch.Tensor
    rows: int
    k: int

    def dequantized_values(self) -> torch.Tensor:
        """The codes as a ``[rows, k]`` ``float8_e4m3fn`` matrix (scales not applied)."""
        return self.values.view(self.rows, self.k).view(torch.float8_e4m3fn)


def _validate_float_activation(input: torch.Tensor) -> tuple[int, int]:
    _refuse(input.device.type != "cuda", f"input must be a CUDA tensor; got {input.device}")
    _refuse(input.dtype not in _DTYPE_CODE,
            f"input must have dtype torch.float16 or torch.bfloat16; got {input.dtype}", TypeError)
    _refuse(input.ndim != 2, f"input must have shape [M,K]; got {tuple(input.shape)}")
    _refuse(not input.is_contiguous(), "input must be contiguous")
    rows, k = map(int, input.shape)
    _refuse(min(rows, k) <= 0 or k % SCALE_VECTOR_SIZE != 0,
            "M must be positive and K a positive multiple of 32")
    return rows, k


def packed_scale_numel(rows: int, k: int) -> int:
    """Bytes of a packed scale buffer: ceil128(rows) * ceil4(k / 32)."""
    groups = (k // SCALE_VECTOR_SIZE + 3) // 4 * 4
    return (rows + 127) // 128 * 128 * groups


# --------------------------------------------------------------------------- layout


def pack_fp6(codes: torch.Tensor) -> torch.Tensor:
    """Pack CUDA uint8 E3M2 codes, four 6-bit values into three bytes.

    ``codes`` may have any shape, must be contiguous, and must contain a number
    of elements divisible by four.  Only each byte's low six bits are used.  The
    returned packed representation is one-dimensional.
    """
    _require_cuda_uint8_contiguous(codes, "codes")
    if codes.numel() % 4:
        raise ValueError("codes.numel() must be divisible by four")
    n = codes.numel()
    out = torch.empty(n // 4 * 3, dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        check(library().mxfp6_pack_fp6(codes.data_ptr(), n, out.data_ptr(), _stream(codes.device)))
    return out


def unpack_fp6(packed: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Unpack a physical E3M2 bitstream to CUDA uint8 codes ``[rows, k]``."""
    _require_cuda_uint8_contiguous(packed, "packed")
    if rows <= 0 or k <= 0 or k % 4:
        raise ValueError("rows must be positive and k must be divisible by four")
    if packed.numel() < rows * k // 4 * 3:
        raise ValueError("packed is too small for rows * k codes")
    out = torch.empty((rows, k), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        check(
            library().mxfp6_unpack_fp6(
                packed.data_ptr(), rows, k, out.data_ptr(), _stream(packed.device)
            )
        )
    return out


def pad_fp6(packed: torch.Tensor) -> torch.Tensor:
    """Pad packed FP6 12-byte segments to aligned 16-byte MMA segments."""
    _require_cuda_uint8_contiguous(packed, "packed")
    if packed.ndim < 1 or packed.shape[-1] <= 0 or packed.shape[-1] % 12:
        raise ValueError("packed last dimension must be a positive multiple of 12")
    shape = (*packed.shape[:-1], packed.shape[-1] // 12 * 16)
    out = torch.empty(shape, dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        check(
            library().mxfp6_pad_fp6(
                packed.data_ptr(), packed.numel(), out.data_ptr(), _stream(packed.device)
            )
        )
    return out


def to_mma_k64_weight(weight: torch.Tensor) -> torch.Tensor:
    """Per expert, the ``[N, 64]`` code matrix transposed and packed again (the layout one of
    the reference's SM120 kernels reads; no kernel here needs it, the op is kept for callers)."""
    _require_cuda_uint8_contiguous(weight, "weight")
    _refuse(weight.ndim != 3 or weight.shape[2] != 48, "weight must contain packed [E,N,64] FP6 values")
    experts, rows = int(weight.shape[0]), int(weight.shape[1])
    per_expert = unpack_fp6(weight, experts * rows, 64).view(experts, rows, 64)
    swapped = per_expert.permute(0, 2, 1).contiguous().view(experts * 64, rows)
    return pack_fp6(swapped).view_as(weight)


def expand_fp6_to_fp8(packed: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Losslessly expand packed E3M2 to a ``torch.float8_e4m3fn`` matrix."""
    _require_cuda_uint8_contiguous(packed, "packed")
    if rows <= 0 or k <= 0 or k % 16:
        raise ValueError("rows must be positive and k must be divisible by 16")
    if packed.numel() < rows * k // 4 * 3:
        raise ValueError("packed is too small for rows * k codes")
    out = torch.empty((rows, k), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        check(
            library().mxfp6_expand_fp6_to_fp8(
                packed.data_ptr(), rows, k, out.data_ptr(), _stream(packed.device)
            )
        )
    return out.view(torch.float8_e4m3fn)


def pack_scales(logical: torch.Tensor) -> torch.Tensor:
    """Reorder logical UE8M0 scales to the packed 128x4-atom physical layout.

    ``logical`` is a contiguous CUDA uint8 tensor of shape ``[rows, k / 32]``.
    Byte values are encoded UE8M0 exponents (``0x7f`` represents 1.0).
    """
    _require_cuda_uint8_contiguous(logical, "logical scales")
    if logical.ndim != 2 or logical.shape[0] <= 0 or logical.shape[1] <= 0:
        raise ValueError("logical scales must have shape [rows, k / 32]")
    rows, k_blocks = (int(v) for v in logical.shape)
    k = k_blocks * SCALE_VECTOR_SIZE
    out = torch.empty(packed_scale_numel(rows, k), dtype=torch.uint8, device=logical.device)
    with torch.cuda.device(logical.device):
        check(
            library().mxfp6_pack_scales(
                logical.data_ptr(), rows, k, out.data_ptr(), _stream(logical.device)
            )
        )
    return out


def unpack_scales(packed: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Convert packed scales back to logical ``[rows, k / 32]``."""
    _require_cuda_uint8_contiguous(packed, "packed scales")
    if rows <= 0 or k <= 0 or k % SCALE_VECTOR_SIZE:
        raise ValueError("rows must be positive and k must be divisible by 32")
    if packed.numel() < packed_scale_numel(rows, k):
        raise ValueError("packed scales are too small for rows x k")
    out = torch.empty((rows, k // SCALE_VECTOR_SIZE), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        check(
            library().mxfp6_unpack_scales(
                packed.data_ptr(), rows, k, out.data_ptr(), _stream(packed.device)
            )
        )
    return out


def pack_grouped_scales(
    logical: torch.Tensor,
    expert_offsets: torch.Tensor,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Pack logical scales independently for each contiguous expert group.

    ``logical`` has shape ``[M, K / 32]`` after MoE routing and
    ``expert_offsets`` contains ``E + 1`` int64 row offsets.  The returned
    scale offsets keep every expert on a 128-row scale-atom boundary.
    """
    _require_cuda_uint8_contiguous(logical, "logical scales")
    _refuse(logical.ndim != 2 or 0 in logical.shape, "logical scales must have shape [M, K / 32]")
    offsets_ok = (expert_offsets.device == logical.device and expert_offsets.dtype == torch.int64
                  and expert_offsets.ndim == 1 and expert_offsets.numel() >= 2
                  and expert_offsets.is_contiguous())
    _refuse(not offsets_ok, "expert_offsets must be a contiguous CUDA int64 tensor with E+1 entries")
    rows, groups = map(int, logical.shape)
    experts = expert_offsets.numel() - 1
    # Upper bound of padded rows: every expert may add up to 127 rows of padding.
    padded_rows = (rows + 127) // 128 * 128 + 128 * min(experts, rows)
    k = groups * SCALE_VECTOR_SIZE
    scale_offsets = torch.empty(experts + 1, dtype=torch.int64, device=logical.device)
    packed = torch.empty(
        padded_rows * ((groups + 3) // 4 * 4), dtype=torch.uint8, device=logical.device
    )
    stream = _stream(logical.device)
    with torch.cuda.device(logical.device):
        check(
            library().mxfp6_grouped_scale_offsets(
                expert_offsets.data_ptr(), experts, scale_offsets.data_ptr(), stream
            )
        )
        check(
            library().mxfp6_pack_grouped_scales(
                logical.data_ptr(),
                expert_offsets.data_ptr(),
                scale_offsets.data_ptr(),
                experts,
                padded_rows,
                k,
                packed.data_ptr(),
                stream,
            )
        )
    return packed, scale_offsets


def pack_operand(codes: torch.Tensor, logical_scales: torch.Tensor) -> PackedMXFP6Tensor:
    """``[rows, k]`` E3M2 codes + ``[rows, k/32]`` UE8M0 scales -> the packed operand (the
    logical scales stay attached, so ``unpack_operand`` gives them back without a kernel)."""
    for tensor, name in ((codes, "codes"), (logical_scales, "logical_scales")):
        _require_cuda_uint8_contiguous(tensor, name)
    _refuse(codes.ndim != 2, "codes must have shape [rows, k]")
    rows, k = map(int, codes.shape)
    want = (rows, k // SCALE_VECTOR_SIZE)
    _refuse(k % SCALE_VECTOR_SIZE != 0 or tuple(logical_scales.shape) != want,
            f"logical_scales must have shape {want}; got {tuple(logical_scales.shape)}")
    _refuse(codes.device != logical_scales.device, "codes and logical_scales must be on the same device")
    return PackedMXFP6Tensor(pack_fp6(codes), pack_scales(logical_scales), rows, k, logical_scales)


def unpack_operand(operand: PackedMXFP6Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The inverse of :func:`pack_operand`: ``(codes [rows, k], logical scales [rows, k/32])``."""
    scales = operand.logical_scales
    if scales is None:
        scales = unpack_scales(operand.scales, operand.rows, operand.k)
    return unpack_fp6(operand.values, operand.rows, operand.k), scales


# ----------------------------------------------------------------------- quantizers


def _quantize_mxfp8_raw(
    input: torch.Tensor,
    values: torch.Tensor,
    packed: torch.Tensor | None,
    logical: torch.Tensor | None,
) -> None:
    rows, k = (int(v) for v in input.shape)
    with torch.cuda.device(input.device):
        check(
            library().mxfp6_quantize_mxfp8(
                input.data_ptr(),
                _DTYPE_CODE[input.dtype],
                rows,
                k,
                values.data_ptr(),
                _ptr(packed),
                _ptr(logical),
                _stream(input.device),
            )
        )


def quantize_mxfp8(input: torch.Tensor) -> MXFP8Tensor:
    """Dynamically map a contiguous FP16/BF16 ``[M,K]`` activation to MXFP8.

    Quantization uses one power-of-two UE8M0 scale per 32 consecutive K
    values.  The returned value bytes and scales are already in the layouts
    consumed by the native W6A8 kernels.
    """
    rows, k = _validate_float_activation(input)
    _require_sm100(input.device)
    load_library()
    values = torch.empty(rows * k, dtype=torch.uint8, device=input.device)
    scales = torch.empty(packed_scale_numel(rows, k), dtype=torch.uint8, device=input.device)
    _quantize_mxfp8_raw(input, values, scales, None)
    return MXFP8Tensor(values, scales, rows, k)


def quantize_mxfp8_logical(input: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantize to MXFP8 with row-major ``[M,K/32]`` UE8M0 scales."""
    rows, k = _validate_float_activation(input)
    _require_sm100(input.device)
    load_library()
    values = torch.empty((rows, k), dtype=torch.uint8, device=input.device)
    scales = torch.empty((rows, k // SCALE_VECTOR_SIZE), dtype=torch.uint8, device=input.device)
    _quantize_mxfp8_raw(input, values, None, scales)
    return values.view(torch.float8_e4m3fn), scales


def quantize_mxfp8_dual(
    input: torch.Tensor,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Quantize once and emit both the logical and the packed scale layouts."""
    rows, k = _validate_float_activation(input)
    _require_sm100(input.device)
    load_library()
    values = torch.empty((rows, k), dtype=torch.uint8, device=input.device)
    logical = torch.empty((rows, k // SCALE_VECTOR_SIZE), dtype=torch.uint8, device=input.device)
    packed = torch.empty(packed_scale_numel(rows, k), dtype=torch.uint8, device=input.device)
    _quantize_mxfp8_raw(input, values, packed, logical)
    return values.view(torch.float8_e4m3fn), logical, packed


def quantize_mxfp8_dual_out(
    output: torch.Tensor,
    logical_scales: torch.Tensor,
    packed_scales: torch.Tensor,
    input: torch.Tensor,
) -> None:
    """Write one MXFP8 value tensor and both scale layouts in one kernel."""
    rows, k = _validate_float_activation(input)
    _require_sm100(input.device)
    expected = (
        (output, torch.uint8, (rows, k), "output"),
        (logical_scales, torch.uint8, (rows, k // SCALE_VECTOR_SIZE), "logical_scales"),
    )
    for tensor, dtype, shape, name in expected:
        if (
            tensor.device != input.device
            or tensor.dtype != dtype
            or tensor.shape != shape
            or not tensor.is_contiguous()
        ):
            raise ValueError(f"{name} must be contiguous CUDA {dtype} {shape}")
    packed_size = packed_scale_numel(rows, k)
    if (
        packed_scales.device != input.device
        or packed_scales.dtype != torch.uint8
        or packed_scales.numel() < packed_size
        or not packed_scales.is_contiguous()
    ):
        raise ValueError(
            "packed_scales must be contiguous CUDA uint8 with at least "
            f"{packed_size} values"
        )
    load_library()
    _quantize_mxfp8_raw(input, output, packed_scales, logical_scales)


def rmsnorm_quantize_mxfp8(
    input: torch.Tensor,
    weight: torch.Tensor,
    eps: float = 1e-6,
    *,
    residual: torch.Tensor | None = None,
    values: torch.Tensor | None = None,
    scales: torch.Tensor | None = None,
) -> MXFP8Tensor:
    """(Residual add,) RMSNorm and MXFP8 quantization of a ``[M,K]`` activation in one pass.

    With ``residual`` the input is first updated IN PLACE to ``round(input + residual)``
    (the residual stream of a decoder layer).  Then ``y = ((x * rsqrt(mean(x^2) + eps)) *
    weight)`` rounded once to the input dtype (the rule of
    ``torch.nn.functional.rms_norm``) is quantized like :func:`quantize_mxfp8`.
    ``values`` / ``scales`` let a caller reuse buffers (CUDA-graph capture).
    """
    rows, k = _validate_float_activation(input)
    if residual is not None and (
        residual.shape != input.shape or residual.dtype != input.dtype
        or residual.device != input.device or not residual.is_contiguous()
    ):
        raise ValueError("residual must match the input's shape, dtype and device")
    if weight.dtype != input.dtype or weight.shape != (k,) or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous [K] tensor of the input dtype")
    if weight.device != input.device:
        raise ValueError("weight must be on the input's device")
    _require_sm100(input.device)
    load_library()
    if values is None:
        values = torch.empty(rows * k, dtype=torch.uint8, device=input.device)
    if scales is None:
        scales = torch.empty(packed_scale_numel(rows, k), dtype=torch.uint8, device=input.device)
    if values.numel() < rows * k or scales.numel() < packed_scale_numel(rows, k):
        raise ValueError("values / scales are too small for the activation")
    with torch.cuda.device(input.device):
        check(
            library().mxfp6_rmsnorm_quantize_mxfp8(
                input.data_ptr(), _ptr(residual), None if residual is None else input.data_ptr(),
                _DTYPE_CODE[input.dtype], weight.data_ptr(), float(eps), rows, k,
                values.data_ptr(), scales.data_ptr(), None, _stream(input.device),
            )
        )
    return MXFP8Tensor(values, scales, rows, k)


def quantize_activation(input: torch.Tensor) -> MXFP8Tensor:
    """Alias of :func:`quantize_mxfp8` (the 16-to-8 activation mapping)."""
    return quantize_mxfp8(input)


def quantize_mxfp6(input: torch.Tensor) -> PackedMXFP6Tensor:
    """Dynamically map a contiguous FP16/BF16 ``[rows,K]`` matrix to packed MXFP6."""
    rows, k = _validate_float_activation(input)
    _require_sm100(input.device)
    load_library()
    values = torch.empty(rows * k // 4 * 3, dtype=torch.uint8, device=input.device)
    scales = torch.empty(packed_scale_numel(rows, k), dtype=torch.uint8, device=input.device)
    with torch.cuda.device(input.device):
        check(
            library().mxfp6_quantize_mxfp6(
                input.data_ptr(),
                _DTYPE_CODE[input.dtype],
                rows,
                k,
                values.data_ptr(),
                scales.data_ptr(),
                None,
                _stream(input.device),
            )
        )
    return PackedMXFP6Tensor(values, scales, rows, k)


# --------------------------------------------------------------------------- dense GEMM


def gemm_w6a8_plan(m: int, n: int, k: int, tile_tokens: int = 0, splits: int = 0) -> dict[str, int]:
    """Tile/split-K choice the library makes for a dense problem (host arithmetic)."""
    _validate_problem(m, n, k)
    plan = (ctypes.c_int64 * 10)()
    check(library().mxfp6_gemm_w6a8_plan(m, n, k, tile_tokens, splits, plan))
    keys = ("tile_tokens", "splits", "stages", "grid", "partial_bytes", "counter_bytes",
            "cluster_k", "cta_pair", "kernel", "smem_bytes")
    out = dict(zip(keys, (int(v) for v in plan)))
    out["kernel"] = _KERNEL_NAMES[out["kernel"]]
    return out


def gemm_w6a8(
    a: MXFP8Tensor,
    b: PackedMXFP6Tensor,
    alpha: float = 1.0,
    *,
    out_dtype: torch.dtype = torch.float16,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Compute native ``MXFP8(A) @ MXFP6(B).T`` on SM100."""
    out_dtype = _validate_output_dtype(out_dtype)
    _refuse(not isinstance(a, MXFP8Tensor), "a must be an MXFP8Tensor instance", TypeError)
    _refuse(not isinstance(b, PackedMXFP6Tensor), "b must be a PackedMXFP6Tensor instance", TypeError)
    _refuse(a.k != b.k, f"a.k and b.k must match; got {a.k} and {b.k}")
    _refuse(a.device != b.device, "a and b must be on the same CUDA device")
    _validate_problem(a.rows, b.rows, a.k)
    for operand, label in ((a, "a"), (b, "b")):
        _require_cuda_uint8_contiguous(operand.values, f"{label}.values")
        _require_cuda_uint8_contiguous(operand.scales, f"{label}.scales")
    _require_sm100(a.device)
    load_library()
    if out is None:
        out = torch.empty((a.rows, b.rows), dtype=out_dtype, device=a.device)
    elif out.shape != (a.rows, b.rows) or out.dtype != out_dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous [M,N] tensor of out_dtype")
    with torch.cuda.device(a.device):
        check(
            library().mxfp6_gemm_w6a8(
                a.values.data_ptr(),
                a.scales.data_ptr(),
                b.values.data_ptr(),
                b.scales.data_ptr(),
                a.rows,
                b.rows,
                a.k,
                float(alpha),
                out.data_ptr(),
                _DTYPE_CODE[out_dtype],
                _stream(a.device),
            )
        )
    return out


def gemm_w6a8_config(
    a: MXFP8Tensor,
    b: PackedMXFP6Tensor,
    alpha: float = 1.0,
    *,
    out_dtype: torch.dtype = torch.float16,
    tile_tokens: int = 0,
    splits: int = 0,
    scratch: torch.Tensor | None = None,
    config_id: int | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Run one explicit configuration: ``config_id`` (see :func:`w6a8_configs`), or a
    tile/split-K pair of the persistent kernel with caller-owned scratch."""
    out_dtype = _validate_output_dtype(out_dtype)
    _validate_problem(a.rows, b.rows, a.k)
    _require_sm100(a.device)
    load_library()
    if config_id is not None:
        if out is None:
            out = torch.empty((a.rows, b.rows), dtype=out_dtype, device=a.device)
        with torch.cuda.device(a.device):
            check(
                library().mxfp6_gemm_w6a8_config(
                    a.values.data_ptr(), a.scales.data_ptr(), b.values.data_ptr(),
                    b.scales.data_ptr(), a.rows, b.rows, a.k, float(alpha), out.data_ptr(),
                    _DTYPE_CODE[out_dtype], int(config_id), _stream(a.device),
                )
            )
        return out
    plan = gemm_w6a8_plan(a.rows, b.rows, a.k, tile_tokens, splits)
    need = plan["partial_bytes"] + plan["counter_bytes"]
    if need and (scratch is None or scratch.numel() * scratch.element_size() < need):
        scratch = torch.zeros(need, dtype=torch.uint8, device=a.device)
    out = torch.empty((a.rows, b.rows), dtype=out_dtype, device=a.device)
    with torch.cuda.device(a.device):
        check(
            library().mxfp6_gemm_w6a8_ex(
                a.values.data_ptr(),
                a.scales.data_ptr(),
                b.values.data_ptr(),
                b.scales.data_ptr(),
                a.rows,
                b.rows,
                a.k,
                float(alpha),
                out.data_ptr(),
                _DTYPE_CODE[out_dtype],
                tile_tokens,
                splits,
                _ptr(scratch),
                0 if scratch is None else scratch.numel() * scratch.element_size(),
                _stream(a.device),
            )
        )
    return out


def gemm_from_float(
    a: torch.Tensor,
    b: PackedMXFP6Tensor,
    alpha: float = 1.0,
    *,
    out_dtype: torch.dtype = torch.float16,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Quantize FP16/BF16 A to MXFP8 and run the native W6A8 GEMM.

    Weight B remains packed at six bits.  Quantization and GEMM are launched
    back to back on the current CUDA stream.
    """
    out_dtype = _validate_output_dtype(out_dtype)
    rows, k = _validate_float_activation(a)
    if not isinstance(b, PackedMXFP6Tensor):
        raise TypeError("b must be a PackedMXFP6Tensor instance")
    if k != b.k:
        raise ValueError(f"a.shape[1] and b.k must match; got {k} and {b.k}")
    if a.device != b.device:
        raise ValueError("a and b must be on the same CUDA device")
    _validate_problem(rows, b.rows, k)
    _require_sm100(a.device)
    load_library()
    stage_values = torch.empty(rows * k, dtype=torch.uint8, device=a.device)
    stage_scales = torch.empty(packed_scale_numel(rows, k), dtype=torch.uint8, device=a.device)
    if out is None:
        out = torch.empty((rows, b.rows), dtype=out_dtype, device=a.device)
    elif out.shape != (rows, b.rows) or out.dtype != out_dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous [M,N] tensor of out_dtype")
    with torch.cuda.device(a.device):
        check(
            library().mxfp6_gemm_from_float(
                a.data_ptr(),
                _DTYPE_CODE[a.dtype],
                b.values.data_ptr(),
                b.scales.data_ptr(),
                rows,
                b.rows,
                k,
                float(alpha),
                out.data_ptr(),
                _DTYPE_CODE[out_dtype],
                stage_values.data_ptr(),
                stage_scales.data_ptr(),
                _stream(a.device),
            )
        )
    return out


def gemm_packed(
    a: torch.Tensor,
    b: torch.Tensor,
    sfa: torch.Tensor,
    sfb: torch.Tensor,
    m: int,
    n: int,
    k: int,
    alpha: float = 1.0,
    *,
    out_dtype: torch.dtype = torch.float16,
) -> torch.Tensor:
    """Low-level ``A @ B.T`` for already packed MXFP6 values and scales (W6A6).

    The activation operand is expanded losslessly from E3M2 to E4M3
    (:func:`expand_fp6_to_fp8`) and then takes the W6A8 kernel, which computes
    the same products exactly.
    """
    out_dtype = _validate_output_dtype(out_dtype)
    _validate_problem(m, n, k)
    for tensor, name in ((a, "a"), (b, "b"), (sfa, "sfa"), (sfb, "sfb")):
        _require_cuda_uint8_contiguous(tensor, name)
    devices = {a.device, b.device, sfa.device, sfb.device}
    if len(devices) != 1:
        raise ValueError("a, b, sfa, and sfb must be on the same CUDA device")
    _require_sm100(a.device)
    load_library()
    expanded = expand_fp6_to_fp8(a, m, k).view(torch.uint8).reshape(-1)
    return gemm_w6a8(
        MXFP8Tensor(expanded, sfa, m, k),
        PackedMXFP6Tensor(b, sfb, n, k),
        alpha,
        out_dtype=out_dtype,
    )


def warmup_w6a8(
    b: PackedMXFP6Tensor,
    m_values: tuple[int, ...] | list[int],
    *,
    out_dtype: torch.dtype = torch.float16,
) -> None:
    """Run every listed batch size once (tensor maps, lanes and kernels get set up)."""
    for m in m_values:
        a = torch.zeros((int(m), b.k), dtype=torch.bfloat16, device=b.device)
        gemm_from_float(a, b, out_dtype=out_dtype)
    torch.cuda.synchronize(b.device)


def autotune_w6a8(
    a: torch.Tensor | MXFP8Tensor,
    b: PackedMXFP6Tensor,
    *,
    out_dtype: torch.dtype = torch.float16,
    force: bool = False,
):
    """Pick, install and cache the fastest explicit configuration for this problem before
    graph capture (see :mod:`.autotune`).  Shapes of the measured table keep the default
    plan unless ``force=True`` or ``MXFP6_AUTOTUNE_EXACT`` is set; returns the installed
    ``W6A8Config`` or ``None``."""
    from . import autotune

    out_dtype = _validate_output_dtype(out_dtype)
    if not isinstance(b, PackedMXFP6Tensor):
        raise TypeError("b must be a PackedMXFP6Tensor instance")
    if isinstance(a, torch.Tensor):
        _validate_float_activation(a)
        a = quantize_mxfp8(a)
    elif not isinstance(a, MXFP8Tensor):
        raise TypeError("a must be an FP16/BF16 Tensor or MXFP8Tensor")
    if a.k != b.k or a.device != b.device:
        raise ValueError("a and b must have matching K and CUDA device")
    _validate_problem(a.rows, b.rows, a.k)
    _require_sm100(a.device)
    load_library()
    if (not force and is_tuned_shape(a.rows, b.rows, a.k) and not autotune.should_tune_exact_shapes()
            and not autotune.is_autotune_cache_only()):
        return None
    return autotune.ensure_w6a8_tuned(a, b, out_dtype=out_dtype, force=force)


def gemm(
    a: torch.Tensor | MXFP8Tensor | PackedMXFP6Tensor,
    b: PackedMXFP6Tensor,
    alpha: float = 1.0,
    *,
    out_dtype: torch.dtype = torch.float16,
) -> torch.Tensor:
    """Compute ``A @ B.T`` using the native kernels.

    FP16/BF16 activation tensors are dynamically mapped 16-to-8 and use W6A8
    for every batch size.  :class:`MXFP8Tensor` skips that conversion.  Packed
    MXFP6 activation inputs keep the W6A6-compatible API.
    """
    out_dtype = _validate_output_dtype(out_dtype)
    if isinstance(a, torch.Tensor):
        if not isinstance(b, PackedMXFP6Tensor):
            raise TypeError("FP16/BF16 activation input requires a PackedMXFP6Tensor weight")
        if _AUTOTUNE_ON_FIRST_USE:
            autotune_w6a8(a, b, out_dtype=out_dtype)  # no-op once the shape has a decision
        return gemm_from_float(a, b, alpha, out_dtype=out_dtype)
    if isinstance(a, MXFP8Tensor):
        if not isinstance(b, PackedMXFP6Tensor):
            raise TypeError("MXFP8 activation requires a PackedMXFP6Tensor weight")
        return gemm_w6a8(a, b, alpha, out_dtype=out_dtype)
    if not isinstance(a, PackedMXFP6Tensor):
        raise TypeError("a must be an FP16/BF16 Tensor, MXFP8Tensor, or PackedMXFP6Tensor")
    if not isinstance(b, PackedMXFP6Tensor):
        raise TypeError("b must be a PackedMXFP6Tensor instance")
    if a.k != b.k:
        raise ValueError(f"a.k and b.k must match; got {a.k} and {b.k}")
    if a.device != b.device:
        raise ValueError("a and b must be on the same CUDA device")
    return gemm_packed(
        a.values, b.values, a.scales, b.scales, a.rows, b.rows, a.k, alpha, out_dtype=out_dtype
    )


def gemm_from_codes(
    a_codes: torch.Tensor,
    b_codes: torch.Tensor,
    sfa_logical: torch.Tensor,
    sfb_logical: torch.Tensor,
    alpha: float = 1.0,
    *,
    out_dtype: torch.dtype = torch.float16,
) -> torch.Tensor:
    """Convenience path that packs both operands before ``A @ B.T``."""
    return gemm(
        pack_operand(a_codes, sfa_logical),
        pack_operand(b_codes, sfb_logical),
        alpha,
        out_dtype=out_dtype,
    )


def is_tuned_shape(m: int, n: int, k: int) -> bool:
    """Return whether a problem is one the static table was measured on."""
    return m in TUNED_M and (n, k) in TUNED_NK


def is_available() -> bool:
    """Return whether the library can load and the current GPU is SM100."""
    if not torch.cuda.is_available():
        return False
    try:
        load_library()
        return torch.cuda.get_device_capability() == (10, 0)
    except (ImportError, OSError, RuntimeError):
        return False
