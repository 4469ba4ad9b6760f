"""Grouped standard deviation over an unsorted index.

Same signature and two-pass arithmetic as ``torch_scatter/composite/std.py:8-39`` upstream: group
means first, then the sum of squared deviations, divided by ``max(count - 1, 1) + 1e-6`` when
``unbiased``.  fp32 data over an ascending 1-D index takes a fused three-pass form of the same arithmetic.
"""
from typing import Optional

import torch

from ..scatter import scatter_sum
from ..utils import broadcast
from .softmax import _fused_ok, _read_back


def scatter_std(src: torch.Tensor, index: torch.Tensor, dim: int = -1,
                out: Optional[torch.Tensor] = None,
                dim_size: Optional[int] = None,
                unbiased: bool = True) -> torch.Tensor:
    if out is not None:
        dim_size = out.size(dim)
    if dim < 0:
        dim = src.dim() + dim
    if out is None and src.dtype == torch.float32 and _fused_ok(src, index):
        # ascending 1-D index: three passes (means, squared deviations fused into the read-back, their sums)
        return torch.ops.torch_scatter.std_sorted(src, index, dim, dim_size, unbiased)

    # group sizes, counted over the index as given (before broadcasting)
    index_dim = dim if index.dim() > dim else index.dim() - 1
    ones = torch.ones(index.size(), dtype=src.dtype, device=src.device)
    count = scatter_sum(ones, index, index_dim, dim_size=dim_size)

    full_index = broadcast(index, src, dim)
    total = scatter_sum(src, full_index, dim, dim_size=dim_size)
    count = broadcast(count, total, dim).clamp(1)
    mean = total.div(count)

    deviation = src - _read_back(mean, index, full_index, dim)
    out = scatter_sum(deviation * deviation, full_index, dim, out, dim_size)

    if unbiased:
        count = count.sub(1).clamp_(1)
    return out.div(count + 1e-6).sqrt()
