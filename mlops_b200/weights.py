"""A block-FP8 expert-weight container for hosts that do not have the reference installed.

`BlockFP8Weight` here has the reference container's shape (`src/mlops/block_fp8.py:49-154`
of als244/mlops): `_data` E4M3 `[E, out, in]`, `_scale` fp32 `[E, ceil(out/128),
ceil(in/128)]`, a logical dtype that is the dtype of the gradients it receives, rows in
`nn.Linear` order. The provider accepts either class (anything that carries `_data` and
`_scale`). Quantisation runs on this library's CUDA kernel; publication from a master weight
(`container.copy_(master)`) re-quantises as at construction.
"""

from __future__ import annotations

import torch
from torch.utils._python_dispatch import return_and_correct_aliasing

from . import ops

FP8 = torch.float8_e4m3fn


def components(weight):
    """`(data, scale)` of a block-FP8 container (this class or the reference's)."""
    data = getattr(weight, "_data", None)
    scale = getattr(weight, "_scale", None)
    if data is None or scale is None:
        raise TypeError("expected a BlockFP8Weight container (E4M3 data with 128x128 block scales)")
    return data, scale


def is_block_fp8(weight) -> bool:
    data = getattr(weight, "_data", None)
    scale = getattr(weight, "_scale", None)
    return (
        isinstance(data, torch.Tensor) and isinstance(scale, torch.Tensor) and data.dtype == FP8
        and data.dim() == 3 and scale.dtype == torch.float32
        and tuple(scale.shape) == (data.shape[0], -(-data.shape[1] // 128), -(-data.shape[2] // 128))
    )


class _Quantize(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight, dtype):
        data, scale = ops.quantize_blocks(weight.detach())
        return BlockFP8Weight(data, scale, dtype=weight.dtype if dtype is None else dtype)

    @staticmethod
    def backward(ctx, grad):
        return grad, None  # straight through: the container's gradient is the weight's


class BlockFP8Weight(torch.Tensor):
    @staticmethod
    def __new__(cls, data, scale, *, dtype=torch.bfloat16):
        if data.dim() != 3 or data.dtype != FP8:
            raise ValueError("Expected E4M3 data [experts, out, in]")
        experts, out, inner = data.shape
        expected = (experts, -(-out // 128), -(-inner // 128))
        if tuple(scale.shape) != expected or scale.dtype != torch.float32:
            raise ValueError(f"Expected FP32 block scales {expected}")
        value = torch.Tensor._make_wrapper_subclass(cls, tuple(data.shape), device=data.device, dtype=dtype)
        value._data, value._scale = data, scale
        return value

    def __repr__(self):
        return f"BlockFP8Weight(shape={tuple(self.shape)}, logical_dtype={self.dtype}, device={self.device})"

    @classmethod
    def quantize(cls, weight, *, dtype=None):
        """A container of `weight [E, out, in]` (bf16 or fp32, on a CUDA device)."""
        if weight.dim() != 3:
            raise ValueError("Expected an [experts, out, in] weight")
        return _Quantize.apply(weight, dtype)

    def components(self):
        return self._data, self._scale

    def dequantize(self, *, dtype=None):
        scale = self._scale.repeat_interleave(128, 1).repeat_interleave(128, 2)
        scale = scale[:, : self.shape[1], : self.shape[2]]
        return (self._data.float() * scale).to(self.dtype if dtype is None else dtype)

    def __tensor_flatten__(self):
        return ["_data", "_scale"], (self.dtype,)

    @staticmethod
    def __tensor_unflatten__(inner, metadata, outer_size, outer_stride):
        return BlockFP8Weight(inner["_data"], inner["_scale"], dtype=metadata[0])

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        aten, first = torch.ops.aten, args[0]
        if func is aten.detach.default:
            out = cls(first._data.detach(), first._scale.detach(), dtype=first.dtype)
            return return_and_correct_aliasing(func, args, kwargs, out)
        if func is aten.clone.default:
            return cls(first._data.clone(), first._scale.clone(), dtype=first.dtype)
        if func is aten.copy_.default:
            destination, source = args[:2]
            if isinstance(destination, cls):
                data, scale = source.components() if isinstance(source, cls) else ops.quantize_blocks(source)
                destination._data.copy_(data)
                destination._scale.copy_(scale)
                return destination
            return destination.copy_(source.dequantize(dtype=destination.dtype))
        if func in (aten.empty_like.default, aten.zeros_like.default, aten.ones_like.default):
            return func(first._data, **dict(kwargs, dtype=kwargs.get("dtype", first.dtype)))
        if func is aten.new_empty_strided.default:
            return func(first._data, *args[1:], **dict(kwargs, dtype=kwargs.get("dtype", first.dtype)))
        raise NotImplementedError(f"{func}: use the container's components or dequantize()")
