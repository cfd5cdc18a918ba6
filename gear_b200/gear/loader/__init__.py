from .offline_loader import OfflineLoader

__all__ = ["OfflineLoader"]
