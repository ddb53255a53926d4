"""Block-FP8 checkpoint ingest on the CPU: a small DeepSeek-style safetensors folder is written
by hand (two shards with an index, E4M3 weights and fp32 `weight_scale_inv`), then read back
expert by expert into the `[E, 2F, D]` / `[E, D, F]` containers; bytes and scales must survive
untouched, and everything the importer does not understand must be refused, as the reference's
importer refuses it (src/mlops/sequential_moe/precision/checkpoint.py:41-66, 238-257)."""

import json
import struct

import pytest
import torch

from oracle import moe_oracle as O

_NAMES = {torch.float8_e4m3fn: "F8_E4M3", torch.float32: "F32", torch.bfloat16: "BF16"}


def _write_shard(path, tensors):
    header, blobs, offset = {}, [], 0
    for name, tensor in tensors.items():
        raw = tensor.contiguous().view(torch.uint8).reshape(-1).numpy().tobytes()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    encoded = json.dumps(header).encode()
    encoded += b" " * (-len(encoded) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for raw in blobs:
            handle.write(raw)


def _checkpoint(folder, experts=4, hidden=256, inner=128, quant=None):
    g = torch.Generator().manual_seed(8)
    shards, weight_map, truth = [{}, {}], {}, {}
    for e in range(experts):
        for which, shape in (("gate_proj", (inner, hidden)), ("up_proj", (inner, hidden)),
                             ("down_proj", (hidden, inner))):
            data, scale = O.quantize_blocks(torch.randn(1, *shape, generator=g))
            prefix = f"model.layers.3.mlp.experts.{e}.{which}"
            shards[e % 2][prefix + ".weight"] = data[0]
            shards[e % 2][prefix + ".weight_scale_inv"] = scale[0]
            truth[(e, which)] = (data[0], scale[0])
    shards[0]["model.layers.3.mlp.gate.weight"] = torch.randn(experts, hidden, generator=g).bfloat16()
    for i, shard in enumerate(shards):
        name = f"model-{i + 1:05d}-of-00002.safetensors"
        _write_shard(folder / name, shard)
        weight_map.update({key: name for key in shard})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    quant = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128]} if quant is None else quant
    (folder / "config.json").write_text(json.dumps({"quantization_config": quant}))
    return truth


def test_experts_come_back_byte_for_byte(tmp_path):
    from mlops_b200 import checkpoint

    truth = _checkpoint(tmp_path)
    with checkpoint.BlockFP8Checkpoint(tmp_path) as source:
        w13, w2 = checkpoint.load_experts(source, "model.layers.3.mlp.experts", [1, 3], 256, 128, device="cpu")
        gate = source.projection("model.layers.3.mlp.experts.0.gate_proj", (128, 256))
        assert torch.equal(gate[0].view(torch.uint8), truth[(0, "gate_proj")][0].view(torch.uint8))
    assert w13.shape == (2, 256, 256) and w2.shape == (2, 256, 128) and w13.dtype == torch.bfloat16
    for slot, e in enumerate((1, 3)):
        expected = torch.cat((truth[(e, "gate_proj")][0], truth[(e, "up_proj")][0]), 0)
        assert torch.equal(w13._data[slot].view(torch.uint8), expected.view(torch.uint8))
        assert torch.equal(w13._scale[slot], torch.cat((truth[(e, "gate_proj")][1], truth[(e, "up_proj")][1]), 0))
        assert torch.equal(w2._data[slot].view(torch.uint8), truth[(e, "down_proj")][0].view(torch.uint8))
        assert torch.equal(w2._scale[slot], truth[(e, "down_proj")][1])
    # the container dequantises to what the checkpoint's own bytes and scales mean
    dense = O.dequantize_blocks(w2._data, w2._scale, torch.bfloat16)
    assert torch.equal(w2.dequantize(), dense)


def test_unknown_encodings_and_bad_layouts_are_refused(tmp_path):
    from mlops_b200 import checkpoint

    folder = tmp_path / "awq"
    folder.mkdir()
    _checkpoint(folder, quant={"quant_method": "awq"})
    with pytest.raises(ValueError, match="quant_method"):
        checkpoint.BlockFP8Checkpoint(folder)
    folder = tmp_path / "blocks"
    folder.mkdir()
    _checkpoint(folder, quant={"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [64, 64]})
    with pytest.raises(ValueError, match="weight_block_size"):
        checkpoint.BlockFP8Checkpoint(folder)
    folder = tmp_path / "ok"
    folder.mkdir()
    _checkpoint(folder)
    with checkpoint.BlockFP8Checkpoint(folder) as source:
        with pytest.raises(KeyError):
            source.projection("model.layers.3.mlp.experts.9.gate_proj", (128, 256))
        with pytest.raises(ValueError, match="expected E4M3"):
            source.projection("model.layers.3.mlp.experts.0.gate_proj", (256, 128))
        with pytest.raises(ValueError, match="boundary"):
            checkpoint.load_experts(source, "model.layers.3.mlp.experts", [0], 256, 64, device="cpu")
    gate = (torch.zeros(64, 256, dtype=torch.float8_e4m3fn), torch.zeros(1, 2))
    with pytest.raises(ValueError, match="boundary"):
        checkpoint.join_gate_up(gate, gate)
