"""Registry of cache-clearing callables (``olmax/caches.py:1-8``)."""

from typing import Callable, List

cache_clears: List[Callable[[], None]] = []


def clear_caches() -> None:
    for fn in cache_clears:
        fn()
