from .manager import (CacheError, CacheLayout, CacheManager, OutOfPages, OutOfSlots, PageGroup,  # noqa: F401
                      layout_of)
