from .manager import (CacheError, CacheManager, GroupSpec, OutOfPages, PageAllocator,
                      Reservation, SlotAllocator, chain_hash)

__all__ = ["CacheError", "CacheManager", "GroupSpec", "OutOfPages", "PageAllocator",
           "Reservation", "SlotAllocator", "chain_hash"]
