from .allocator import IdAllocator, OutOfPages  # noqa: F401
from .manager import CacheManager, PagedKVView, PageGroup, StateView  # noqa: F401


def num_pages_for_budget(cache_specs, page_size: int, element_size: int, budget_bytes: int) -> int:
    """How many pages each group gets when ``budget_bytes`` is shared by all of them
    (src/llmserve/kvcache/paged.py:221-227: bytes of one page = 2 * layers * kv_heads * page_size *
    head_dim * element size)."""
    from ..parts.base import PagedKVSpec

    per_page = sum(
        2 * s.kv_heads * page_size * s.head_dim * element_size for s in cache_specs if isinstance(s, PagedKVSpec)
    )
    return max(1, budget_bytes // per_page) if per_page else 1
