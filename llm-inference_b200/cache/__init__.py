from .paged_cache import CacheGroup, PagedCache, plan_groups, split_budget, window_pages

__all__ = ["CacheGroup", "PagedCache", "plan_groups", "split_budget", "window_pages"]
