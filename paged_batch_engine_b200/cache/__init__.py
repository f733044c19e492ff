from .manager import NO_PAGE, CacheError, CacheManager, KVGroupSpec, PagePoolView

__all__ = ["NO_PAGE", "CacheError", "CacheManager", "KVGroupSpec", "PagePoolView", "CacheStorage",
           "LayerCache"]


def __getattr__(name):   # storage needs torch and the parts; the manager alone does not
    if name in ("CacheStorage", "LayerCache"):
        from . import storage
        return getattr(storage, name)
    raise AttributeError(name)
