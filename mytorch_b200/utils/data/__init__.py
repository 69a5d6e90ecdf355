from .data_loader import DataLoader, DevicePrefetcher
from .dataset import Dataset
