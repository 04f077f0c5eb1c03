"""B200-native block-sparse attention with the Python API of linxihui/dkernel."""
__version__ = "0.1.0"

from .interface import SparseAttention, LocalStrideSparseAttention, combine_attn_partitions
from .utils import get_sparse_attn_mask

__all__ = [
    "SparseAttention",
    "LocalStrideSparseAttention",
    "get_sparse_attn_mask",
    "combine_attn_partitions",
]
