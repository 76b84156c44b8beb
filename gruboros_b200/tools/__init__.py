"""Offline tools: corpus extraction, metrics aggregation, loss-curve fitting."""
