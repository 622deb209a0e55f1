from .os_cache import MemoryManager, OSCacheManager

__all__ = ['MemoryManager', 'OSCacheManager']
