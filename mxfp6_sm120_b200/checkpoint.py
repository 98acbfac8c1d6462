"""Reading MXFP6 checkpoints into the operand layout the kernels take.

An MXFP6 checkpoint stores, per linear layer, ``<name>.weight`` (E3M2 codes, four to three
bytes, ``[N, 3K/4]`` uint8) and ``<name>.weight_scale`` (logical OCP-MX UE8M0 scales,
``[N, K/32]`` uint8).  The kernels want the scales in 128 x 4 atoms
(``PackedMXFP6Tensor.scales``) and, for a routed-MoE layer, the experts stacked:
``[E, 2I, 3H/4]`` gate rows then up rows, ``[E, H, 3I/4]`` down rows, the shared expert as
one more matrix behind them, the router and shared-expert gate rows as one BF16 matrix.
This is what the reference's layer benchmark builds from the Qwen3.5 checkpoint
(benchmarks/benchmark_qwen35_moe_layer.py:351-542: names :146-151, tensor-parallel slices
:363-376, scale packing :351-354); here it is a library function with the layer prefix,
the expert count and the tensor-parallel slice as arguments.

Sources: a ``.safetensors`` file, a directory of them (with or without
``model.safetensors.index.json``), a ``.pt`` file holding a ``dict`` of tensors, or a
mapping already in memory.  Everything here is host-side preparation: tensors are sliced
and packed with torch on the source's device and moved once.
"""

from __future__ import annotations

import json
from collections.abc import Mapping
from dataclasses import dataclass
from pathlib import Path

import torch

from .ops import SCALE_VECTOR_SIZE, PackedMXFP6Tensor, packed_scale_numel

_ATOM_ROWS = 128
_ATOM_BYTES = 512


class TensorSource:
    """Named tensors of a checkpoint, opened lazily file by file."""

    def __init__(self, source):
        self._memory: Mapping[str, torch.Tensor] | None = None
        self._files: dict[str, Path] = {}      # tensor name -> file
        self._open: dict[Path, object] = {}
        if isinstance(source, Mapping):
            self._memory = source
            return
        path = Path(source)
        if path.is_dir():
            index = path / "model.safetensors.index.json"
            if index.exists():
                weight_map = json.loads(index.read_text())["weight_map"]
                self._files = {name: path / file for name, file in weight_map.items()}
            else:
                for file in sorted(path.glob("*.safetensors")):
                    for name in self._handle(file).keys():
                        self._files[name] = file
            if not self._files:
                raise FileNotFoundError(f"no safetensors files under {path}")
        elif path.suffix == ".safetensors":
            self._files = {name: path for name in self._handle(path).keys()}
        elif path.suffix in (".pt", ".pth", ".bin"):
            loaded = torch.load(path, map_location="cpu", weights_only=True)
            if not isinstance(loaded, Mapping):
                raise ValueError(f"{path} does not hold a dict of tensors")
            self._memory = loaded
        else:
            raise ValueError(f"unsupported checkpoint source: {path}")

    def _handle(self, file: Path):
        if file not in self._open:
            from safetensors import safe_open

            self._open[file] = safe_open(file, framework="pt", device="cpu")
        return self._open[file]

    def close(self) -> None:
        """Drop the open file handles (tensors already returned stay valid)."""
        self._open.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __contains__(self, name: str) -> bool:
        return name in (self._memory if self._memory is not None else self._files)

    def get(self, name: str, rows: slice | None = None, columns: slice | None = None) -> torch.Tensor:
        if self._memory is not None:
            if name not in self._memory:
                raise KeyError(name)
            value = self._memory[name]
        else:
            if name not in self._files:
                raise KeyError(name)
            value = self._handle(self._files[name]).get_tensor(name)
        if rows is not None:
            value = value[rows]
        if columns is not None:
            value = value[:, columns]
        return value.contiguous()


def pack_scales_host(logical: torch.Tensor) -> torch.Tensor:
    """Logical UE8M0 scales ``[rows, K/32]`` -> the 128 x 4 atom layout, with torch on the
    tensor's own device (the layout and the 0x7f padding of ``pack_scales``)."""
    if logical.dtype != torch.uint8 or logical.ndim != 2:
        raise ValueError("logical scales must be a uint8 matrix [rows, K/32]")
    rows, groups = (int(v) for v in logical.shape)
    atoms_per_row_block = (groups + 3) // 4
    out = torch.full((packed_scale_numel(rows, groups * SCALE_VECTOR_SIZE),), 0x7F, dtype=torch.uint8,
                     device=logical.device)
    row = torch.arange(rows, device=logical.device).view(-1, 1)
    group = torch.arange(groups, device=logical.device).view(1, -1)
    inner = row % _ATOM_ROWS
    offset = (((row // _ATOM_ROWS) * atoms_per_row_block + group // 4) * _ATOM_BYTES
              + (inner % 32) * 16 + (inner // 32) * 4 + group % 4)
    out[offset.reshape(-1)] = logical.reshape(-1)
    return out


def _check_linear(values: torch.Tensor, scales: torch.Tensor, name: str) -> tuple[int, int]:
    if values.dtype != torch.uint8 or values.ndim != 2 or scales.dtype != torch.uint8 or scales.ndim != 2:
        raise ValueError(f"{name}: weight and weight_scale must be uint8 matrices")
    rows, packed = (int(v) for v in values.shape)
    if packed % 3 or (packed // 3 * 4) % SCALE_VECTOR_SIZE:
        raise ValueError(f"{name}: packed row length {packed} is not 3K/4 with K a multiple of 32")
    k = packed // 3 * 4
    if tuple(scales.shape) != (rows, k // SCALE_VECTOR_SIZE):
        raise ValueError(f"{name}: weight_scale must have shape [{rows}, {k // SCALE_VECTOR_SIZE}]")
    return rows, k


def load_linear(source, name: str, device=None, rows: slice | None = None,
                input_columns: slice | None = None) -> PackedMXFP6Tensor:
    """One linear layer: ``<name>.weight`` + ``<name>.weight_scale`` -> ``PackedMXFP6Tensor``.

    ``rows`` keeps a slice of the output features (column-parallel sharding);
    ``input_columns`` a slice of the INPUT features in elements (row-parallel sharding), a
    multiple of 128 at both ends so that codes, scale groups and atoms split cleanly.
    """
    tensors = source if isinstance(source, TensorSource) else TensorSource(source)
    code_columns = scale_columns = None
    if input_columns is not None:
        lo, hi = input_columns.start or 0, input_columns.stop
        if hi is None or lo % 128 or hi % 128:
            raise ValueError("input_columns must be given in elements, multiples of 128")
        code_columns = slice(lo * 3 // 4, hi * 3 // 4)
        scale_columns = slice(lo // SCALE_VECTOR_SIZE, hi // SCALE_VECTOR_SIZE)
    values = tensors.get(f"{name}.weight", rows, code_columns)
    scales = tensors.get(f"{name}.weight_scale", rows, scale_columns)
    n, k = _check_linear(values, scales, name)
    if device is not None:
        values, scales = values.to(device), scales.to(device)
    return PackedMXFP6Tensor(values.reshape(-1), pack_scales_host(scales), n, k, logical_scales=scales)


@dataclass
class MoeLayerCheckpoint:
    """A routed-MoE layer as read from a checkpoint: the routed experts followed by the
    shared expert in both stacks (the reference's ``MxLayerWeights``,
    benchmarks/benchmark_qwen35_moe_layer.py:64-73,528-542)."""

    hidden: int
    intermediate: int          # this rank's share
    experts: int               # routed experts
    w1: PackedMXFP6Tensor      # [(E + 1) * 2I, H]
    w2: PackedMXFP6Tensor      # [(E + 1) * H, I]
    combined_gate: torch.Tensor  # [E + 1, H] BF16: router rows, then the shared expert's gate row

    def stacks(self):
        """``(w1 [E+1, 2I, 3H/4], w1_scales, w2 [E+1, H, 3I/4], w2_scales)`` as
        ``qwen35_moe_b1_out`` takes them."""
        e1, i, h = self.experts + 1, self.intermediate, self.hidden
        return (self.w1.values.view(e1, 2 * i, h * 3 // 4), self.w1.scales,
                self.w2.values.view(e1, h, i * 3 // 4), self.w2.scales)

    def _split(self, stacked: PackedMXFP6Tensor, rows_per_expert: int):
        e = self.experts
        codes = rows_per_expert * stacked.k * 3 // 4
        atoms = packed_scale_numel(rows_per_expert, stacked.k)
        routed = PackedMXFP6Tensor(stacked.values[: e * codes], stacked.scales[: e * atoms],
                                   e * rows_per_expert, stacked.k)
        shared = PackedMXFP6Tensor(stacked.values[e * codes:], stacked.scales[e * atoms:],
                                   rows_per_expert, stacked.k)
        return routed, shared

    def moe_layer(self, topk: int = 8):
        """The layer object of this package (routed stacks and the shared expert apart);
        views, no copies."""
        from .moe_layer import MoeLayer
        from .qwen35 import MoeShape

        w1, shared_w1 = self._split(self.w1, 2 * self.intermediate)
        w2, shared_w2 = self._split(self.w2, self.hidden)
        return MoeLayer(MoeShape(self.hidden, self.intermediate, self.experts, topk), w1, w2,
                        shared_w1, shared_w2)


def load_moe_layer(source, prefix: str, experts: int, device=None, tp_rank: int = 0,
                   tp_size: int = 1) -> MoeLayerCheckpoint:
    """Read ``<prefix>.experts.<e>.{gate,up,down}_proj``, ``<prefix>.shared_expert.*``,
    ``<prefix>.gate.weight`` and ``<prefix>.shared_expert_gate.weight``.

    Tensor parallelism slices the intermediate dimension as the reference does: rows of
    gate / up, input columns of down (benchmarks/benchmark_qwen35_moe_layer.py:363-376).
    """
    tensors = source if isinstance(source, TensorSource) else TensorSource(source)
    if tp_size < 1 or not 0 <= tp_rank < tp_size:
        raise ValueError("tp_rank must lie in [0, tp_size)")
    probe = tensors.get(f"{prefix}.experts.0.gate_proj.weight")
    full_inter, hidden = int(probe.shape[0]), int(probe.shape[1]) // 3 * 4
    if full_inter % tp_size or (full_inter // tp_size) % _ATOM_ROWS:
        raise ValueError("the intermediate size must split into multiples of 128 per rank")
    inter = full_inter // tp_size
    rows = slice(tp_rank * inter, (tp_rank + 1) * inter)
    code_cols = slice(rows.start * 3 // 4, rows.stop * 3 // 4)
    scale_cols = slice(rows.start // SCALE_VECTOR_SIZE, rows.stop // SCALE_VECTOR_SIZE)

    names = [f"{prefix}.experts.{e}" for e in range(experts)] + [f"{prefix}.shared_expert"]
    w1_codes, w1_scales, w2_codes, w2_scales = [], [], [], []
    for name in names:
        for proj in ("gate_proj", "up_proj"):
            codes = tensors.get(f"{name}.{proj}.weight", rows)
            scales = tensors.get(f"{name}.{proj}.weight_scale", rows)
            if _check_linear(codes, scales, f"{name}.{proj}") != (inter, hidden):
                raise ValueError(f"{name}.{proj}: expected [{inter}, {hidden}] after slicing")
            w1_codes.append(codes)
            w1_scales.append(scales)
        codes = tensors.get(f"{name}.down_proj.weight", None, code_cols)
        scales = tensors.get(f"{name}.down_proj.weight_scale", None, scale_cols)
        if _check_linear(codes, scales, f"{name}.down_proj") != (hidden, inter):
            raise ValueError(f"{name}.down_proj: expected [{hidden}, {inter}] after slicing")
        w2_codes.append(codes)
        w2_scales.append(scales)

    def stack(codes, scales, k):
        values = torch.cat(codes, dim=0)
        logical = torch.cat(scales, dim=0)
        if device is not None:
            values, logical = values.to(device), logical.to(device)
        return PackedMXFP6Tensor(values.reshape(-1), pack_scales_host(logical), int(values.shape[0]), k)

    gate = torch.cat([tensors.get(f"{prefix}.gate.weight"),
                      tensors.get(f"{prefix}.shared_expert_gate.weight")], dim=0).to(torch.bfloat16)
    if tuple(gate.shape) != (experts + 1, hidden):
        raise ValueError(f"router and shared-expert gate rows must stack to [{experts + 1}, {hidden}]")
    if device is not None:
        gate = gate.to(device)
    return MoeLayerCheckpoint(hidden, inter, experts, stack(w1_codes, w1_scales, hidden),
                              stack(w2_codes, w2_scales, inter), gate.contiguous())


def moe_layer_tensors(prefix: str, hidden: int, intermediate: int, w1_codes: torch.Tensor,
                      w1_scales: torch.Tensor, w2_codes: torch.Tensor, w2_scales: torch.Tensor,
                      combined_gate: torch.Tensor) -> dict[str, torch.Tensor]:
    """The checkpoint names of a layer given as stacks: ``w1_codes`` ``[E+1, 2I, 3H/4]``,
    ``w1_scales`` logical ``[E+1, 2I, H/32]``, ``w2_codes`` ``[E+1, H, 3I/4]``, ``w2_scales``
    ``[E+1, H, I/32]`` (the last matrix is the shared expert), ``combined_gate`` ``[E+1, H]``.
    The inverse of :func:`load_moe_layer`; with ``save_tensors`` it writes test fixtures and
    exports of layers quantized in memory."""
    experts = int(w1_codes.shape[0]) - 1
    out: dict[str, torch.Tensor] = {}
    for e in range(experts + 1):
        name = f"{prefix}.experts.{e}" if e < experts else f"{prefix}.shared_expert"
        out[f"{name}.gate_proj.weight"] = w1_codes[e, :intermediate].contiguous()
        out[f"{name}.up_proj.weight"] = w1_codes[e, intermediate:].contiguous()
        out[f"{name}.gate_proj.weight_scale"] = w1_scales[e, :intermediate].contiguous()
        out[f"{name}.up_proj.weight_scale"] = w1_scales[e, intermediate:].contiguous()
        out[f"{name}.down_proj.weight"] = w2_codes[e].contiguous()
        out[f"{name}.down_proj.weight_scale"] = w2_scales[e].contiguous()
    out[f"{prefix}.gate.weight"] = combined_gate[:experts].contiguous()
    out[f"{prefix}.shared_expert_gate.weight"] = combined_gate[experts:].contiguous()
    return {name: value.cpu() for name, value in out.items()}


def save_tensors(tensors: Mapping[str, torch.Tensor], path) -> None:
    """Write a dict of tensors as ``.safetensors`` or ``.pt`` (by the suffix)."""
    path = Path(path)
    if path.suffix == ".safetensors":
        from safetensors.torch import save_file

        save_file({k: v.contiguous() for k, v in tensors.items()}, str(path))
    elif path.suffix in (".pt", ".pth"):
        torch.save(dict(tensors), path)
    else:
        raise ValueError("path must end in .safetensors or .pt")
