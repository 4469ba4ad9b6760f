"""Parameter lists for tests, mirroring ``torch_scatter/testing.py:5-19`` upstream.

``devices`` holds CUDA devices only: this build has no CPU kernels.
"""
from typing import Any

import torch

reductions = ['sum', 'add', 'mean', 'min', 'max']

dtypes = [
    torch.half, torch.bfloat16, torch.float, torch.double, torch.int,
    torch.long
]
grad_dtypes = [torch.float, torch.double]

devices = []
if torch.cuda.is_available():
    devices += [torch.device('cuda:0')]


def tensor(x: Any, dtype: torch.dtype, device: torch.device):
    return None if x is None else torch.tensor(x, device=device).to(dtype)
