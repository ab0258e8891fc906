"""dynamiq_sigcomm_artifact_b200: compressed-gradient all-reduce for PyTorch DDP on B200 GPUs."""
__version__ = "0.1.0"
