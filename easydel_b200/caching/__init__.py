from .paged import PagedBatchMeta, PagedKVCache, PagedLayerView
from .transformer import TransformerCache, TransformerCacheView

__all__ = ["PagedBatchMeta", "PagedKVCache", "PagedLayerView", "TransformerCache", "TransformerCacheView"]
