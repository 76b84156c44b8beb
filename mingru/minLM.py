"""``from mingru.minLM import minLM`` - see gruboros_b200.models.minlm for the implementation."""
from gruboros_b200.models.minlm import CausalDepthWiseConv1d, FeedForward, minLM

__all__ = ["minLM", "FeedForward", "CausalDepthWiseConv1d"]
