"""rannc_b200: automatic model partitioning middleware for PyTorch on B200."""
__version__ = "0.1.0"
