import torch


def broadcast(src: torch.Tensor, other: torch.Tensor, dim: int):
    """Expand ``src`` (an index) to the shape of ``other`` around ``dim``.

    A 1-D ``src`` is placed on ``dim``; otherwise trailing singleton dims are appended.  The result
    is a stride-0 view, never a copy (same contract as ``torch_scatter/utils.py:4-13`` upstream).
    """
    if dim < 0:
        dim = other.dim() + dim
    if src.dim() == 1:
        for _ in range(0, dim):
            src = src.unsqueeze(0)
    for _ in range(src.dim(), other.dim()):
        src = src.unsqueeze(-1)
    src = src.expand(other.size())
    return src
