"""Stride arithmetic for the view-like ATen ops.

The reference turns reshape/unsqueeze/... into aliases and transpose/slice/expand
into CuPy views at run time (cuda_compiler/subgraph_analyzer.py:463-603,
cuda_runtime/cuda_executor.py:596-658).  Here every such op is resolved at compile
time to (offset, shape, strides) over the producing buffer, using PyTorch's own
view rules on meta tensors, so no kernel runs unless the result really cannot be
expressed as strides.
"""

from __future__ import annotations

import torch

from cuda_compiler.cuda_program import TensorView

INT64_MAX = 2**63 - 1


def _meta(view: TensorView) -> torch.Tensor:
    return torch.empty_strided(tuple(view.shape), tuple(view.strides), dtype=torch.uint8, device="meta")


def _from_meta(base: TensorView, m: torch.Tensor, dtype: str | None = None) -> TensorView:
    return TensorView(base.buffer, base.offset + int(m.storage_offset()), tuple(int(s) for s in m.shape),
                      tuple(int(s) for s in m.stride()), dtype or base.dtype)


def contiguous_strides(shape) -> tuple[int, ...]:
    strides, acc = [], 1
    for extent in reversed(list(shape)):
        strides.append(acc)
        acc *= max(int(extent), 1)
    return tuple(reversed(strides))


def like_strides(shape, like: TensorView) -> tuple[int, ...]:
    """Dense strides for ``shape`` that keep the dimension order of ``like`` (so an
    elementwise result of a channels-last tensor stays channels-last)."""
    if len(shape) != len(like.shape) or tuple(shape) != tuple(like.shape):
        return contiguous_strides(shape)
    order = sorted(range(len(shape)), key=lambda d: (like.strides[d], -d), reverse=True)
    if any(like.strides[d] == 0 and shape[d] != 1 for d in range(len(shape))):
        return contiguous_strides(shape)
    strides = [0] * len(shape)
    acc = 1
    for d in reversed(order):
        strides[d] = acc
        acc *= max(int(shape[d]), 1)
    return tuple(strides)


def try_reshape(view: TensorView, shape) -> TensorView | None:
    """``view.view(shape)`` if PyTorch can express it without copying, else None."""
    try:
        return _from_meta(view, _meta(view).view(tuple(int(s) for s in shape)))
    except RuntimeError:
        return None


def transpose(view: TensorView, d0: int, d1: int) -> TensorView:
    return _from_meta(view, _meta(view).transpose(d0, d1))


def permute(view: TensorView, dims) -> TensorView:
    return _from_meta(view, _meta(view).permute(*dims))


def unsqueeze(view: TensorView, dim: int) -> TensorView:
    return _from_meta(view, _meta(view).unsqueeze(dim))


def squeeze(view: TensorView, dim: int) -> TensorView:
    return _from_meta(view, _meta(view).squeeze(dim))


def expand(view: TensorView, size) -> TensorView:
    return _from_meta(view, _meta(view).expand(*[int(s) for s in size]))


def slice_(view: TensorView, dim: int, start, end, step) -> TensorView:
    start = 0 if start is None else int(start)
    end = INT64_MAX if end is None else int(end)
    step = 1 if step is None else int(step)
    return _from_meta(view, torch.ops.aten.slice.Tensor(_meta(view), dim, start, end, step))


def broadcast_to(view: TensorView, shape) -> TensorView:
    """Express ``view`` in the index space of ``shape`` (stride 0 where broadcast)."""
    shape = tuple(int(s) for s in shape)
    if tuple(view.shape) == shape:
        return view
    return _from_meta(view, _meta(view).expand(shape) if len(view.shape) == len(shape) else _meta(view).broadcast_to(shape))
