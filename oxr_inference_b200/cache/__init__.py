from oxr_inference_b200.cache.manager import RELEASED, CacheManager, RequestCache, pages_for
from oxr_inference_b200.cache.pages import PagePool
from oxr_inference_b200.cache.plan import CachePlan, EntryPlan, GroupPlan, make_cache_plan

__all__ = ["RELEASED", "CacheManager", "CachePlan", "EntryPlan", "GroupPlan", "PagePool", "RequestCache",
           "make_cache_plan", "pages_for"]
