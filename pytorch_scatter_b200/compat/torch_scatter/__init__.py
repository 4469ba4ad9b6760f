"""Name shim: makes ``import torch_scatter`` resolve to the B200 build.

Put the directory that holds this package (``pytorch_scatter_b200/compat``) and the repository root
on ``sys.path``; code written against upstream's ``torch_scatter`` (its own test-suite included) then
imports the sm_100a operators unchanged.  Sub-modules ``torch_scatter.utils``, ``.testing``,
``.composite``, ``.scatter``, ``.segment_coo`` and ``.segment_csr`` are aliased as well.
"""
import sys

import pytorch_scatter_b200 as _impl
from pytorch_scatter_b200 import *  # noqa: F401,F403
from pytorch_scatter_b200 import __version__, composite, scatter as _scatter_fn, testing, utils  # noqa: F401
import pytorch_scatter_b200.scatter as _scatter_mod
import pytorch_scatter_b200.segment_coo as _segment_coo_mod
import pytorch_scatter_b200.segment_csr as _segment_csr_mod

__all__ = list(_impl.__all__)

for _name, _mod in (('utils', utils), ('testing', testing), ('composite', composite), ('scatter', _scatter_mod),
                    ('segment_coo', _segment_coo_mod), ('segment_csr', _segment_csr_mod)):
    sys.modules[__name__ + '.' + _name] = _mod
for _sub in ('softmax', 'logsumexp', 'std'):
    sys.modules[__name__ + '.composite.' + _sub] = sys.modules['pytorch_scatter_b200.composite.' + _sub]
# `from torch_scatter import scatter` must give the function, as upstream does
scatter = _scatter_fn
