"""B200 (sm_100a) implementation of Arcaine's scaled-dot-product-attention path.

The arithmetic lives in ``libarc_sdpa.so`` (hand-written CUDA behind a C ABI,
``include/arc_sdpa.h``); this package is the Python host side: tensor plumbing
(:mod:`arcaine_b200.ops`), multi-GPU sharding (:mod:`arcaine_b200.sharded`) and
the in-tree build (:mod:`arcaine_b200.build`).  There is no CPU or PyTorch
fallback: without the library the operators raise.
"""
from . import ops  # noqa: F401
from .ops import *  # noqa: F401,F403

__version__ = "0.1.0"
