"""Key-padding ("sparse KV") attention under the reference's module path
(src/para_attn/sparse_attn.py:14-69, 607-640): ``sparse_kv_attn_func`` and
``SparseKVAttnMode``. The structured-sparsity and focus-attention modes of that file are
outside the context-parallel attention path and are not built."""
from .para_attn_interface import SparseKVAttnMode, sparse_kv_attn_func

__all__ = ["SparseKVAttnMode", "sparse_kv_attn_func"]
