"""Content-addressed cache of preparation results (task profiles, link calibrations)."""
from .cache import ContentStore, StoreMode, kernel_library_digest

__all__ = ["ContentStore", "StoreMode", "kernel_library_digest"]
