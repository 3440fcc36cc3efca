"""Weight-plane files of the reference's FasterTransformer fork, and quantise-on-load.

The fork's LLaMA loader (models/llama/LlamaDecoderLayerWeight.cc:377-403, ``int8_mode == 5``) reads, per decoder layer
and tensor-parallel rank, five raw files without header

    <dir>/model.layers.<l>.attention.query_key_value.weight.<rank>.bin      planes [w_bits][3*hidden/tp][hidden/32]
    <dir>/model.layers.<l>.attention.dense.weight.<rank>.bin                planes [w_bits][hidden][hidden/tp/32]
    <dir>/model.layers.<l>.mlp.gate_proj.weight.<rank>.bin                  planes [w_bits][ffn/tp][hidden/32]
    <dir>/model.layers.<l>.mlp.up_proj.weight.<rank>.bin                    planes [w_bits][ffn/tp][hidden/32]
    <dir>/model.layers.<l>.mlp.down_proj.weight.<rank>.bin                  planes [w_bits][hidden][ffn/tp/32]

each holding the bit-planes of that rank's shard as 32-bit little-endian words in the engine's layout (bit 31 - j of
word kw of plane b = bit b of the code of input feature 32 kw + j; engine/common/pack.cu:54-62).  The loader declares the
buffers as 16-bit elements (``w_bits*hidden x 3*hidden/16/tp`` halves, ...): the same bytes.  It never loads scales
(":404 TODO: Load scales") and ships no packer, so two things here have no counterpart in the reference and are this
library's own convention: the scale / zero-point files written next to each weight file

    ....weight.<rank>.scale.bin     fp16 [rows][groups]      ....weight.<rank>.zero.bin     uint8 [rows][groups]

and the packer itself (:func:`quantize_and_shard`), which quantises fp16 weights on the GPU with the library's
quantise-on-load kernel (min/max calibration of algorithm/quantize/quantizer.py) and shards rows / input features the
way :mod:`tp_linear` does.  Reading and writing files is plain numpy and needs no GPU.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Tuple

import numpy as np

# reference file stem -> (fused parts along the output rows, parallel direction)
FT_LINEARS: Dict[str, Tuple[int, str]] = {
    "attention.query_key_value": (3, "column"),
    "attention.dense": (1, "row"),
    "mlp.gate_proj": (1, "column"),
    "mlp.up_proj": (1, "column"),
    "mlp.down_proj": (1, "row"),
}


def shard_path(directory, layer: int, name: str, rank: int, what: str = "weight") -> Path:
    """File of one linear layer's shard; ``what`` is "weight" (the reference's file), "scale" or "zero" (ours)."""
    if name not in FT_LINEARS:
        raise KeyError(f"{name!r} is not one of {sorted(FT_LINEARS)}")
    stem = f"model.layers.{layer}.{name}.weight.{rank}"
    return Path(directory) / (stem + (".bin" if what == "weight" else f".{what}.bin"))


def shard_shape(name: str, hidden: int, ffn: int, tp: int, w_bits: int) -> Tuple[int, int, int]:
    """(planes, rows, words per row) of a rank's weight file when the split is even (what the reference's loader assumes)."""
    parts, direction = FT_LINEARS[name]
    out_f = {"attention.query_key_value": 3 * hidden, "attention.dense": hidden, "mlp.gate_proj": ffn, "mlp.up_proj": ffn, "mlp.down_proj": hidden}[name]
    in_f = ffn if name == "mlp.down_proj" else hidden
    if direction == "column":
        return w_bits, out_f // tp, in_f // 32
    return w_bits, out_f, in_f // tp // 32


def write_shard(directory, layer: int, name: str, rank: int, planes: np.ndarray, scale: np.ndarray | None = None, zero: np.ndarray | None = None) -> None:
    """planes: uint32 [w_bits][rows][K/32]; scale fp16 / zero uint8 [rows] or [rows][groups] (optional)."""
    p = np.ascontiguousarray(planes)
    if p.dtype not in (np.uint32, np.int32) or p.ndim != 3:
        raise ValueError("planes must be 32-bit words [w_bits][rows][K/32]")
    Path(directory).mkdir(parents=True, exist_ok=True)
    p.astype("<u4", copy=False).tofile(shard_path(directory, layer, name, rank))
    if scale is not None:
        np.ascontiguousarray(scale, dtype="<f2").tofile(shard_path(directory, layer, name, rank, "scale"))
    if zero is not None:
        np.ascontiguousarray(zero, dtype=np.uint8).tofile(shard_path(directory, layer, name, rank, "zero"))


def read_shard(directory, layer: int, name: str, rank: int, w_bits: int, rows: int, K: int, groups: int | None = None):
    """Returns (planes uint32 [w_bits][rows][K/32], scale or None, zero or None).  A missing weight file raises (the
    reference only warns and keeps random data, utils/memory_utils.cu:319-320); a file of the wrong size raises too."""
    path = shard_path(directory, layer, name, rank)
    want = w_bits * rows * (K // 32)
    data = np.fromfile(path, dtype="<u4")
    if data.size != want:
        raise ValueError(f"{path}: {data.size * 4} bytes, {want * 4} expected for [{w_bits}][{rows}][{K // 32}] words")
    planes = data.reshape(w_bits, rows, K // 32)
    scale = zero = None
    sp, zp = shard_path(directory, layer, name, rank, "scale"), shard_path(directory, layer, name, rank, "zero")
    if sp.exists():
        scale = np.fromfile(sp, dtype="<f2")
        if groups is not None and scale.size != rows * groups:
            raise ValueError(f"{sp}: {scale.size} scales, {rows * groups} expected")
        scale = scale.reshape(rows, -1) if scale.size != rows else scale
    if zp.exists():
        zero = np.fromfile(zp, dtype=np.uint8)
        zero = zero.reshape(rows, -1) if zero.size != rows else zero
    return planes, scale, zero


def split_ranges(total: int, tp: int, unit: int):
    """Shard boundaries in whole ``unit``s, the first ranks one unit larger when it does not divide (11008 over 4 ranks in
    units of 128: 2816, 2816, 2688, 2688).  The reference only supports even splits; this is what they become then."""
    units = total // unit
    base, extra = divmod(units, tp)
    out, at = [], 0
    for r in range(tp):
        n = (base + (1 if r < extra else 0)) * unit
        out.append((at, at + n))
        at += n
    return out


def quantize_and_shard(abq, torch, w_half, name: str, tp: int, w_bits: int, group_size: int = 0, symmetric: bool = False):
    """Quantise one full fp16 weight [out][in] on the GPU and cut it into the ranks' shards.

    Returns a list over ranks of (planes uint32 [w_bits][rows][K_local/32], scale, zero) numpy arrays ready for
    :func:`write_shard`.  Column-parallel layers split the output rows of every fused part, row-parallel layers split the
    input features in whole 128-feature units (and their scale groups with them); calibration happens before the split,
    so every rank quantises against the same ranges as the unsharded model."""
    parts, direction = FT_LINEARS[name]
    N, K = w_half.shape
    G = K // group_size if group_size else 1
    planes = torch.empty((w_bits, N, K // 32), dtype=torch.int32, device="cuda")
    scale = torch.empty((N, G) if group_size else (N,), dtype=torch.float16, device="cuda")
    zero = torch.empty((N, G) if group_size else (N,), dtype=torch.uint8, device="cuda")
    abq.quantize_weights_half(w_half.contiguous(), planes, scale, zero, N, K, w_bits, group_size, symmetric)
    torch.cuda.synchronize()
    planes, scale, zero = planes.cpu().numpy().view(np.uint32), scale.cpu().numpy(), zero.cpu().numpy()
    shards = []
    if direction == "column":
        per = N // parts
        for (b, e) in split_ranges(per, tp, 128 if per % 128 == 0 else 1):
            rows = np.concatenate([np.arange(p * per + b, p * per + e) for p in range(parts)])
            shards.append((planes[:, rows, :], scale[rows], zero[rows]))
    else:
        for (b, e) in split_ranges(K, tp, 128):
            if group_size and (b % group_size or e % group_size):
                raise ValueError(f"input-feature shard [{b}, {e}) cuts a scale group of {group_size}")
            s, z = (scale[:, b // group_size:e // group_size], zero[:, b // group_size:e // group_size]) if group_size else (scale, zero)
            shards.append((np.ascontiguousarray(planes[:, :, b // 32:e // 32]), np.ascontiguousarray(s), np.ascontiguousarray(z)))
    return shards
