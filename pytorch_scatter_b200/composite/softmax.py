"""Grouped softmax / log-softmax over an unsorted index.

Same signatures and arithmetic as ``torch_scatter/composite/softmax.py:9-51`` upstream: subtract
the per-group maximum, exponentiate, normalise by the per-group sum.  The grouped max and sum are
this package's scatter kernels; the element-wise steps and the read-back are ATen.
"""
from typing import Optional

import torch

from ..scatter import scatter_max, scatter_sum
from ..utils import broadcast


def _require_float(src: torch.Tensor, name: str) -> None:
    if not torch.is_floating_point(src):
        raise ValueError(f'`{name}` can only be computed over tensors '
                         'with floating point data types.')


def scatter_softmax(src: torch.Tensor, index: torch.Tensor,
                    dim: int = -1,
                    dim_size: Optional[int] = None) -> torch.Tensor:
    _require_float(src, 'scatter_softmax')
    index = broadcast(index, src, dim)
    group_max = scatter_max(src, index, dim=dim, dim_size=dim_size)[0]
    shifted_exp = (src - group_max.gather(dim, index)).exp_()
    group_sum = scatter_sum(shifted_exp, index, dim, dim_size=dim_size)
    return shifted_exp.div(group_sum.gather(dim, index))


def scatter_log_softmax(src: torch.Tensor, index: torch.Tensor, dim: int = -1,
                        eps: float = 1e-12,
                        dim_size: Optional[int] = None) -> torch.Tensor:
    _require_float(src, 'scatter_log_softmax')
    index = broadcast(index, src, dim)
    group_max = scatter_max(src, index, dim=dim, dim_size=dim_size)[0]
    shifted = src - group_max.gather(dim, index)
    group_sum = scatter_sum(shifted.exp(), index, dim, dim_size=dim_size)
    log_norm = group_sum.add_(eps).log_().gather(dim, index)
    return shifted.sub_(log_norm)
