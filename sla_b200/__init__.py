"""sla_b200: B200 (sm_100a) implementation of Sparse-Linear Attention behind the reference's API.

    from sla_b200 import SparseLinearAttention, SageSparseLinearAttention
    from sla_b200 import get_block_map, _attention          # operator-level names

``install_aliases()`` registers the reference's import names (``sparse_linear_attention`` and
``SageSLA``) so that existing ``from sparse_linear_attention import SparseLinearAttention`` code
runs unchanged.
"""
import sys
import types

from .core import SageSparseLinearAttention, SparseLinearAttention
from .graphs import graphed
from .ops import _attention, block_map, get_block_map, sage_sla_attention, sla_attention

__all__ = ["SparseLinearAttention", "SageSparseLinearAttention", "get_block_map", "_attention", "block_map",
           "sla_attention", "sage_sla_attention", "install_aliases", "graphed"]


def install_aliases() -> None:
    """Make `import sparse_linear_attention` / `import SageSLA` resolve to this package."""
    pkg = types.ModuleType("sparse_linear_attention")
    pkg.SparseLinearAttention = SparseLinearAttention
    utils = types.ModuleType("sparse_linear_attention.utils")
    utils.get_block_map = get_block_map
    kernel = types.ModuleType("sparse_linear_attention.kernel")
    kernel._attention = _attention
    core = types.ModuleType("sparse_linear_attention.core")
    core.SparseLinearAttention = SparseLinearAttention
    pkg.utils, pkg.kernel, pkg.core = utils, kernel, core
    sage = types.ModuleType("SageSLA")
    sage.SageSparseLinearAttention = SageSparseLinearAttention
    for m in (pkg, utils, kernel, core, sage):
        sys.modules[m.__name__] = m
