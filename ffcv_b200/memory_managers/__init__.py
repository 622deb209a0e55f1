from .direct_read import DirectReadManager, FileDescriptors
from .os_cache import MemoryManager, OSCacheManager

__all__ = ['DirectReadManager', 'FileDescriptors', 'MemoryManager', 'OSCacheManager']
