"""Mixins of ``EasyDeLBaseModule``: checkpoint bridge, generation, cache-requirement discovery."""

from .bridge import EasyBridgeMixin
from .generation import EasyGenerationMixin
from .operation_cache import (CacheType, ExecutionMode, LayerOperationInfo, OperationCacheMixin, OperationsCacheInfo)

__all__ = ["CacheType", "EasyBridgeMixin", "EasyGenerationMixin", "ExecutionMode", "LayerOperationInfo",
           "OperationCacheMixin", "OperationsCacheInfo"]
