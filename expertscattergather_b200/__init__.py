"""B200 (sm_100a) fused expert gather / scatter with the reference's ``egs`` interface.

    from expertscattergather_b200 import ExpertGather, ExpertScatter

or, to serve code written against the reference package name::

    import expertscattergather_b200; expertscattergather_b200.install_as_egs()
    from egs import ExpertGather, ExpertScatter
"""
from __future__ import annotations

import sys

from .torch_interface import ExpertGather, ExpertGatherScatter, ExpertScatter
from .kernels import ExpertGatherFunction, ExpertScatterFunction, create_kernels
from . import ops

__all__ = ["ExpertGather", "ExpertScatter", "ExpertGatherScatter", "ExpertGatherFunction", "ExpertScatterFunction", "create_kernels",
           "ops", "install_as_egs"]
__version__ = "0.1.0"


def install_as_egs() -> None:
    """Registers this package under the reference's import names (``egs``, ``egs.torch_interface``,
    ``egs.triton_kernels``) so that ``from egs import ExpertGather`` resolves to the B200 kernels."""
    from . import kernels, torch_interface
    me = sys.modules[__name__]
    sys.modules.setdefault("egs", me)
    sys.modules.setdefault("egs.torch_interface", torch_interface)
    sys.modules.setdefault("egs.triton_kernels", kernels)
