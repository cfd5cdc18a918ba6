from .shared_dataset import SharedDataset

__all__ = ["SharedDataset"]
