"""Utilities: SFT preprocessing, checkpoint I/O, logging/metrics, failure detection."""
from tah_b200.utils.data_prepare import preprocess_dataset

__all__ = ["preprocess_dataset"]
