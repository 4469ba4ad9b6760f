"""Grouped softmax / log-softmax over an unsorted index.

Same signatures and arithmetic as ``torch_scatter/composite/softmax.py:9-51`` upstream: subtract
the per-group maximum, exponentiate, normalise by the per-group sum.  The grouped max and sum are
this package's scatter kernels; the element-wise steps and the read-back are ATen.
"""
from typing import Optional

import torch

from ..scatter import scatter_max, scatter_sum
from ..utils import broadcast


def _read_back(per_group: torch.Tensor, index: torch.Tensor, full_index: torch.Tensor, dim: int) -> torch.Tensor:
    """``per_group`` read back at every element's group, i.e. ``per_group.gather(dim, full_index)``, done by
    this package's row-gather kernel (the index is read once per entry, rows move in 16-byte packs)."""
    return torch.ops.torch_scatter.gather_rows(per_group, full_index, dim)


def _fused_ok(src: torch.Tensor, index: torch.Tensor) -> bool:
    """The two-pass fused kernels apply: a 1-D ascending index over fp32 / fp16 / bf16 CUDA data.  Checking the
    order costs one small kernel and a host sync (the same kind upstream pays to infer ``dim_size``)."""
    if index.dim() != 1 or index.numel() == 0 or not src.is_cuda:
        return False
    if not torch.jit.is_scripting():
        if torch.compiler.is_compiling():   # whether the index is sorted is a property of the data: not traceable
            return False
    if not (src.dtype == torch.float32 or src.dtype == torch.float16 or src.dtype == torch.bfloat16):
        return False
    return torch.ops.torch_scatter.index_is_sorted(index)


def _require_float(src: torch.Tensor, name: str) -> None:
    if not torch.is_floating_point(src):
        raise ValueError(f'`{name}` can only be computed over tensors '
                         'with floating point data types.')


def scatter_softmax(src: torch.Tensor, index: torch.Tensor,
                    dim: int = -1,
                    dim_size: Optional[int] = None) -> torch.Tensor:
    _require_float(src, 'scatter_softmax')
    if _fused_ok(src, index):
        return torch.ops.torch_scatter.softmax_sorted(src, index, dim, dim_size, False)
    full_index = broadcast(index, src, dim)
    group_max = scatter_max(src, full_index, dim=dim, dim_size=dim_size)[0]
    shifted_exp = (src - _read_back(group_max, index, full_index, dim)).exp_()
    group_sum = scatter_sum(shifted_exp, full_index, dim, dim_size=dim_size)
    return shifted_exp.div(_read_back(group_sum, index, full_index, dim))


def scatter_log_softmax(src: torch.Tensor, index: torch.Tensor, dim: int = -1,
                        eps: float = 1e-12,
                        dim_size: Optional[int] = None) -> torch.Tensor:
    _require_float(src, 'scatter_log_softmax')
    if _fused_ok(src, index):  # eps (1e-12 under a sum that is at least 1) is below fp32 resolution
        return torch.ops.torch_scatter.softmax_sorted(src, index, dim, dim_size, True)
    full_index = broadcast(index, src, dim)
    group_max = scatter_max(src, full_index, dim=dim, dim_size=dim_size)[0]
    shifted = src - _read_back(group_max, index, full_index, dim)
    group_sum = scatter_sum(shifted.exp(), full_index, dim, dim_size=dim_size)
    log_norm = _read_back(group_sum.add_(eps).log_(), index, full_index, dim)
    return shifted.sub_(log_norm)
