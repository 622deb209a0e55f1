from .os_cache import MemoryManager, OSCacheManager
from .read_ahead import ReadAheadManager

__all__ = ['MemoryManager', 'OSCacheManager', 'ReadAheadManager']
