"""gruboros-b200: byte-level minGRU language-model training for NVIDIA B200 (sm_100a)."""
__version__ = "0.1.0"
