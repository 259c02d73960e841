"""Paged key/value cache manager with layer groups and per-request state slots."""

from .manager import AppendPlan, CacheError, CacheManager, GroupSpec, OutOfPages, PagePool, group_needs  # noqa: F401
