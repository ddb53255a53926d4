"""Block-FP8 expert weights straight from a Hugging Face safetensors checkpoint.

DeepSeek-style checkpoints store every expert projection as E4M3 bytes `[out, in]` plus an
fp32 `weight_scale_inv` per 128x128 block -- exactly the two tensors the expert GEMMs of this
library read. This module copies them from disk into `[E, 2F, D]` / `[E, D, F]` device tensors
(gate rows then up rows, `nn.Linear` order) without ever forming a bf16 copy: ranged reads of
one tensor at a time through a pinned staging buffer, the host-to-device copies queued on the
current stream. Nothing of the rest of the model is read.

Behavioural model: the reference's importer (`src/mlops/sequential_moe/precision/
checkpoint.py:18-267`, ranged reader `precision/safetensors.py:37-209`): encodings are taken
from `config.json`'s `quantization_config` and anything but `quant_method = "fp8"`, `fmt =
"e4m3"`, `weight_block_size = [128, 128]` is refused rather than guessed; gate and up join
losslessly only when their boundary falls on a scale block (`join_gate_up`, `:238-257`).
"""

from __future__ import annotations

import json
import os
import struct
from pathlib import Path

import torch

from .weights import BLOCK, BlockFP8Weight

_DTYPES = {
    "F8_E4M3": torch.float8_e4m3fn, "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
    "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8,
}


class SafeTensorsDirectory:
    """Name -> (file, dtype, shape, byte range) of every tensor in a folder of `.safetensors`
    shards (through `model.safetensors.index.json` when there is one), and ranged reads."""

    def __init__(self, directory):
        self.directory = Path(directory)
        self.files: dict[str, tuple[Path, torch.dtype, tuple[int, ...], int, int]] = {}
        self._handles: dict[Path, int] = {}
        index = self.directory / "model.safetensors.index.json"
        if index.exists():
            shards = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        else:
            shards = sorted(p.name for p in self.directory.glob("*.safetensors"))
        if not shards:
            raise FileNotFoundError(f"no .safetensors shard in {self.directory}")
        for shard in shards:
            path = self.directory / shard
            with open(path, "rb") as handle:
                (header_bytes,) = struct.unpack("<Q", handle.read(8))
                header = json.loads(handle.read(header_bytes))
            base = 8 + header_bytes
            for name, entry in header.items():
                if name == "__metadata__":
                    continue
                dtype = _DTYPES.get(entry["dtype"])
                if dtype is None:
                    raise ValueError(f"{name}: safetensors dtype {entry['dtype']!r} is not supported here")
                begin, end = entry["data_offsets"]
                self.files[name] = (path, dtype, tuple(entry["shape"]), base + begin, end - begin)

    def _fd(self, path: Path) -> int:
        fd = self._handles.get(path)
        if fd is None:
            fd = self._handles[path] = os.open(path, os.O_RDONLY)
        return fd

    def meta(self, name):
        _path, dtype, shape, _offset, _nbytes = self.files[name]
        return dtype, shape

    def copy_into(self, name, destination: torch.Tensor) -> torch.Tensor:
        """Reads tensor `name` into the CPU tensor `destination` (same dtype, same number of
        elements, contiguous; a pinned staging buffer typically) with `pread`, a chunk at a time."""
        path, dtype, shape, offset, nbytes = self.files[name]
        if destination.device.type != "cpu" or not destination.is_contiguous():
            raise ValueError("copy_into reads into a contiguous CPU tensor")
        if destination.dtype != dtype or destination.numel() * destination.element_size() != nbytes:
            raise ValueError(f"{name}: destination does not match {dtype} {shape}")
        view = memoryview(destination.view(torch.uint8).reshape(-1).numpy())
        fd, done = self._fd(path), 0
        while done < nbytes:
            got = os.preadv(fd, [view[done:min(done + (8 << 20), nbytes)]], offset + done)
            if got <= 0:
                raise IOError(f"{name}: short read from {path}")
            done += got
        return destination

    def tensor(self, name) -> torch.Tensor:
        dtype, shape = self.meta(name)
        return self.copy_into(name, torch.empty(shape, dtype=dtype))

    def close(self):
        for fd in self._handles.values():
            os.close(fd)
        self._handles.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class BlockFP8Checkpoint:
    """A checkpoint whose `config.json` declares E4M3 weights with 128x128 block scales."""

    def __init__(self, directory):
        self.directory = Path(directory)
        config_path = self.directory / "config.json"
        config = json.loads(config_path.read_text()) if config_path.exists() else {}
        quant = config.get("quantization_config") or config.get("text_config", {}).get("quantization_config") or {}
        method = quant.get("quant_method")
        if method != "fp8":
            raise ValueError(f"block-FP8 ingest needs quant_method='fp8' in config.json, found {method!r}; other "
                             "encodings are not inferred from tensor names or dtypes")
        if quant.get("fmt", "e4m3") != "e4m3" or quant.get("weight_block_size") != [BLOCK, BLOCK]:
            raise ValueError("block-FP8 ingest needs fmt='e4m3' and weight_block_size=[128, 128]")
        self.source = SafeTensorsDirectory(directory)

    def close(self):
        self.source.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def projection_meta(self, prefix, shape):
        """Checks that `<prefix>.weight` / `<prefix>.weight_scale_inv` exist with the shapes of a
        block-FP8 `[out, in]` matrix; returns their names."""
        out, inner = shape
        weight, scale = prefix + ".weight", prefix + ".weight_scale_inv"
        for name in (weight, scale):
            if name not in self.source.files:
                raise KeyError(f"{name} is not in the checkpoint")
        dtype, found = self.source.meta(weight)
        if dtype != torch.float8_e4m3fn or found != (out, inner):
            raise ValueError(f"{weight}: expected E4M3 {(out, inner)}, found {dtype} {found}")
        expected = (-(-out // BLOCK), -(-inner // BLOCK))
        dtype, found = self.source.meta(scale)
        if dtype != torch.float32 or found != expected:
            raise ValueError(f"{scale}: expected fp32 {expected}, found {dtype} {found}")
        return weight, scale

    def projection(self, prefix, shape):
        """`(data E4M3 [out, in], scale fp32 [out/128, in/128])` of one matrix, on the CPU."""
        weight, scale = self.projection_meta(prefix, shape)
        data, scales = self.source.tensor(weight), self.source.tensor(scale)
        if not bool(torch.isfinite(scales).all()) or bool((scales < 0).any()):
            raise ValueError(f"{scale}: weight scales must be finite and nonnegative")
        return data, scales


def join_gate_up(gate, up):
    """`[gate; up]` as one `[2F, D]` matrix with its scales, losslessly: possible only when the
    boundary falls on a scale block (F a multiple of 128)."""
    (gate_data, gate_scale), (up_data, up_scale) = gate, up
    if gate_data.shape != up_data.shape or gate_scale.shape != up_scale.shape:
        raise ValueError("gate and up need matching shapes and scale layouts")
    if gate_data.shape[0] % BLOCK:
        raise ValueError("the gate/up boundary must fall on a 128-row scale block")
    return torch.cat((gate_data, up_data), 0), torch.cat((gate_scale, up_scale), 0)


def load_experts(checkpoint, prefix, experts, hidden, intermediate, *, device, dtype=torch.bfloat16,
                 names=("gate_proj", "up_proj", "down_proj")):
    """The experts `experts` (an iterable of indices: all of them, or one rank's shard) under
    `<prefix>.<index>.<gate|up|down>.weight[_scale_inv]` as `(w13, w2)` containers on `device`:
    `w13 [E, 2F, D]` gate rows then up rows, `w2 [E, D, F]`, logical dtype `dtype` (the dtype
    their gradients get). One matrix at a time goes through a pinned buffer; the device copies
    are asynchronous on the current stream (two staging buffers alternate)."""
    source = checkpoint if isinstance(checkpoint, BlockFP8Checkpoint) else BlockFP8Checkpoint(checkpoint)
    experts = list(experts)
    D, F = int(hidden), int(intermediate)
    if F % BLOCK:
        raise ValueError("the gate/up boundary must fall on a 128-row scale block")
    device = torch.device(device)
    cuda = device.type == "cuda"
    w13_q = torch.empty((len(experts), 2 * F, D), dtype=torch.float8_e4m3fn, device=device)
    w13_s = torch.empty((len(experts), 2 * F // BLOCK, -(-D // BLOCK)), dtype=torch.float32, device=device)
    w2_q = torch.empty((len(experts), D, F), dtype=torch.float8_e4m3fn, device=device)
    w2_s = torch.empty((len(experts), -(-D // BLOCK), F // BLOCK), dtype=torch.float32, device=device)
    gate_name, up_name, down_name = names
    largest = max(F * D, D * F)
    staging = [(torch.empty(largest, dtype=torch.uint8, pin_memory=cuda),
                torch.empty(largest // (BLOCK * BLOCK) + D + F, dtype=torch.float32, pin_memory=cuda),
                torch.cuda.Event() if cuda else None) for _ in range(2)]
    turn = 0

    def ship(matrix_prefix, shape, data_out, scale_out):
        nonlocal turn
        weight, scale = source.projection_meta(matrix_prefix, shape)
        data_buffer, scale_buffer, event = staging[turn % 2]
        turn += 1
        if event is not None:
            event.synchronize()  # the copy that last used this buffer has been read by the device
        out, inner = shape
        data = data_buffer[: out * inner].view(torch.float8_e4m3fn).view(out, inner)
        scales = scale_buffer[: scale_out.numel()].view(scale_out.shape)
        source.source.copy_into(weight, data)
        source.source.copy_into(scale, scales)
        if not bool(torch.isfinite(scales).all()) or bool((scales < 0).any()):
            raise ValueError(f"{scale}: weight scales must be finite and nonnegative")
        data_out.view(torch.uint8).copy_(data.view(torch.uint8), non_blocking=True)
        scale_out.copy_(scales, non_blocking=True)
        if event is not None:
            event.record()

    rows = F // BLOCK
    for slot, expert in enumerate(experts):
        base = f"{prefix}.{expert}"
        ship(f"{base}.{gate_name}", (F, D), w13_q[slot, :F], w13_s[slot, :rows])
        ship(f"{base}.{up_name}", (F, D), w13_q[slot, F:], w13_s[slot, rows:])
        ship(f"{base}.{down_name}", (D, F), w2_q[slot], w2_s[slot])
    if cuda:
        for _data, _scale, event in staging:
            event.synchronize()
    return BlockFP8Weight(w13_q, w13_s, dtype=dtype), BlockFP8Weight(w2_q, w2_s, dtype=dtype)
