from .manager import (CacheError, CacheFull, KVRequirement, StateRequirement, PagePool, KVGroup,
                      CacheManager)
