"""``from mingru.minGRU import minGRU`` - see gruboros_b200.models.mingru for the implementation."""
from gruboros_b200.models.mingru import g, heinsen_associative_scan_log, log_g, minGRU

__all__ = ["minGRU", "g", "log_g", "heinsen_associative_scan_log"]
