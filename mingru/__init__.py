"""Public model API (same import paths as the reference: ``from mingru.minLM import minLM``)."""
from gruboros_b200.models.mingru import minGRU
from gruboros_b200.models.minlm import minLM

__all__ = ["minGRU", "minLM"]
