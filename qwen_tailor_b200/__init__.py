"""B200-native (sm_100a) implementation of the GatedDeltaNet / GQA-decode attention hot path.

The operators keep the call signatures of the reference's Python modules of the same names (``gated_delta``, ``gdn_nax``,
``kernels``, ``batch``, ``batch_spec``, ``prefix_cache``) over CUDA ``torch.Tensor``s; all arithmetic runs in the hand-written
CUDA kernels of libgdn_b200.so (C ABI: include/gdn_b200.h).  There is no CPU fallback.
"""
from .config import Cfg  # noqa: F401

__version__ = "0.1.0"
