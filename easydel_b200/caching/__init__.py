from .paged import PagedBatchMeta, PagedKVCache, PagedLayerView
from .transformer import TransformerCache, TransformerCacheView

__all__ = ["PagedBatchMeta", "PagedKVCache", "PagedLayerView", "TransformerCache", "TransformerCacheView"]

from .turboquant_paged import TurboQuantLayerView, TurboQuantPagedKVCache  # noqa: E402,F401
__all__ = [*__all__, "TurboQuantLayerView", "TurboQuantPagedKVCache"]
