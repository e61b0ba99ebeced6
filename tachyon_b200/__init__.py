"""B200-native CUDA backend for Tachyon's Granite mixture-of-experts block."""
from .weights import Matrix  # noqa: F401
