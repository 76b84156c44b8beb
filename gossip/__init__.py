"""Public gossip API (same import path as the reference: ``from gossip import EvolutionaryTrainingNode``)."""
from gruboros_b200.parallel.gossip import EvolutionaryTrainingNode, FitnessTracker, NetworkUtils

__all__ = ["EvolutionaryTrainingNode", "FitnessTracker", "NetworkUtils"]
