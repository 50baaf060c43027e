from .dp_router import DataParallelEngine
from .engine import CompletionOutput, RequestOutput, eSurge
from .kv_manager import GroupManager, KVCacheCoordinator
from .metrics import MetricsCollector
from .page_pool import PagePool, hash_page_tokens, hash_request_pages
from .runner import ModelRunner
from .scheduler import EngineRequest, RequestStatus, Scheduler, SchedulerConfig, SchedulerOutput

__all__ = ["eSurge", "RequestOutput", "CompletionOutput", "MetricsCollector", "PagePool", "ModelRunner", "Scheduler",
           "SchedulerConfig", "SchedulerOutput", "EngineRequest", "RequestStatus", "hash_page_tokens",
           "hash_request_pages", "DataParallelEngine", "KVCacheCoordinator", "GroupManager"]
