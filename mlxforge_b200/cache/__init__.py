from .manager import CacheLayout, CacheManager, GroupLayout, KVLane, StateLane
from .pages import OutOfPages, OutOfSlots, PagePool, SequenceCache, SlotPool
