from .manager import (KEEP_ALL, KEEP_CHUNK, KEEP_WINDOW, CacheError, CacheManager, OutOfPages, OutOfSlots, Retention)

__all__ = ["KEEP_ALL", "KEEP_CHUNK", "KEEP_WINDOW", "CacheError", "CacheManager", "OutOfPages", "OutOfSlots",
           "Retention"]
