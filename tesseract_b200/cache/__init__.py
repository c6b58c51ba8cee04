from .manager import CacheManager
from .pages import OutOfPages, PagePool, StateSlots
