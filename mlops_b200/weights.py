"""Block-FP8 expert weights as this library sees them.

The expert GEMMs read two plain tensors per weight: E4M3 bytes `[E, out, in]` and one fp32
scale per 128x128 block, `[E, ceil(out/128), ceil(in/128)]` -- the storage of the
reference's `mlops.block_fp8.BlockFP8Weight` (als244/mlops `src/mlops/block_fp8.py:49-68`).
Any object that carries them as `_data` and `_scale` is accepted (`split`, `holds_blocks`),
so the reference's own container goes straight through.

For callers that do not have the reference installed, `BlockFP8Weight` below is a tensor
subclass with the same two attributes: it looks like a `[E, out, in]` tensor of the dtype its
gradient should have (so an optimizer or autograd can treat it as a parameter), is built by
this library's CUDA quantiser, and re-quantises when a master weight is copied into it.
"""

from __future__ import annotations

import torch
from torch.utils._python_dispatch import return_and_correct_aliasing

from . import ops

FP8 = torch.float8_e4m3fn
BLOCK = 128


def _scale_shape(shape):
    experts, out, inner = shape
    return (experts, (out + BLOCK - 1) // BLOCK, (inner + BLOCK - 1) // BLOCK)


def holds_blocks(weight) -> bool:
    """Whether `weight` carries E4M3 data with matching 128x128 block scales."""
    data, scale = getattr(weight, "_data", None), getattr(weight, "_scale", None)
    if not (isinstance(data, torch.Tensor) and isinstance(scale, torch.Tensor)):
        return False
    return (data.dtype == FP8 and data.dim() == 3 and scale.dtype == torch.float32
            and tuple(scale.shape) == _scale_shape(data.shape))


def split(weight):
    """`(data, scale)` of a block-FP8 container; TypeError for anything else."""
    if not holds_blocks(weight):
        raise TypeError("expected block-FP8 expert weights: E4M3 `_data` [E, out, in] with fp32 `_scale` "
                        "per 128x128 block")
    return weight._data, weight._scale




class _StraightThrough(torch.autograd.Function):
    """quantize(): the container's gradient is handed to the master weight unchanged."""

    @staticmethod
    def forward(ctx, master, logical):
        data, scale = ops.quantize_blocks(master.detach())
        return BlockFP8Weight(data, scale, dtype=logical or master.dtype)

    @staticmethod
    def backward(ctx, grad):
        return grad, None


def _like(func, args, kwargs):
    # factory ops autograd and optimizers call on a parameter: answer with an ordinary tensor
    # of the logical dtype, shaped like the data
    source = args[0]
    kwargs = dict(kwargs)
    kwargs.setdefault("dtype", source.dtype)
    return func(source._data, *args[1:], **kwargs)


def _detach(func, args, kwargs):
    source = args[0]
    alias = BlockFP8Weight(source._data.detach(), source._scale.detach(), dtype=source.dtype)
    return return_and_correct_aliasing(func, args, kwargs, alias)  # detach is a view: keep it one


def _clone(func, args, kwargs):
    source = args[0]
    return BlockFP8Weight(source._data.clone(), source._scale.clone(), dtype=source.dtype)


def _copy(func, args, kwargs):
    target, source = args[0], args[1]
    if not isinstance(target, BlockFP8Weight):  # container -> ordinary tensor: its values
        return target.copy_(source.dequantize(dtype=target.dtype))
    if isinstance(source, BlockFP8Weight):
        data, scale = source._data, source._scale
    else:  # publication of a master weight: quantise it as at construction
        data, scale = ops.quantize_blocks(source.to(target.device))
    target._data.copy_(data)
    target._scale.copy_(scale)
    return target


_ATEN = torch.ops.aten
_HANDLERS = {
    _ATEN.detach.default: _detach,
    _ATEN.clone.default: _clone,
    _ATEN.copy_.default: _copy,
    _ATEN.empty_like.default: _like,
    _ATEN.zeros_like.default: _like,
    _ATEN.ones_like.default: _like,
    _ATEN.new_empty_strided.default: _like,
}


class BlockFP8Weight(torch.Tensor):
    """`[E, out, in]` expert weights stored as E4M3 with 128x128 block scales."""

    @staticmethod
    def __new__(cls, data, scale, *, dtype=torch.bfloat16):
        if not (isinstance(data, torch.Tensor) and data.dtype == FP8 and data.dim() == 3):
            raise ValueError("data: E4M3 tensor [experts, out, in] wanted")
        if scale.dtype != torch.float32 or tuple(scale.shape) != _scale_shape(data.shape):
            raise ValueError(f"scale: fp32 tensor {_scale_shape(data.shape)} wanted for data {tuple(data.shape)}")
        self = torch.Tensor._make_wrapper_subclass(cls, data.shape, dtype=dtype, device=data.device)
        self._data = data
        self._scale = scale
        return self

    @classmethod
    def quantize(cls, master, *, dtype=None):
        """Container of the CUDA tensor `master [E, out, in]` (bf16 or fp32). Differentiable:
        the gradient of the container is the gradient of `master`."""
        if master.dim() != 3:
            raise ValueError("master weight: [experts, out, in] wanted")
        return _StraightThrough.apply(master, dtype)

    def components(self):
        return self._data, self._scale

    def dequantize(self, *, dtype=None):
        _e, out, inner = self.shape
        per_element = self._scale.repeat_interleave(BLOCK, 1).repeat_interleave(BLOCK, 2)[:, :out, :inner]
        return (self._data.float() * per_element).to(dtype or self.dtype)

    def __repr__(self):
        return f"{type(self).__name__}({tuple(self.shape)}, grads in {self.dtype}, on {self.device})"

    # ---- what torch.compile / AOTAutograd need to take the container apart and rebuild it
    def __tensor_flatten__(self):
        return ["_data", "_scale"], self.dtype

    @staticmethod
    def __tensor_unflatten__(inner, logical, outer_size, outer_stride):
        return BlockFP8Weight(inner["_data"], inner["_scale"], dtype=logical)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        handler = _HANDLERS.get(func)
        if handler is None:
            raise NotImplementedError(
                f"{func} on a BlockFP8Weight: take `.components()` or `.dequantize()` first")
        return handler(func, args, kwargs or {})
