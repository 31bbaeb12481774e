from .storage import CacheBinding, DeviceCache, KVStream

__all__ = ["CacheBinding", "DeviceCache", "KVStream"]
