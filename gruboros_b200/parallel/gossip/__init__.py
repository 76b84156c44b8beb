"""Evolutionary gossip protocol (population-based training over NVLink peer memory or TCP)."""
from .coordinator import FilesystemCoordinator
from .fitness import FitnessTracker
from .logger import GossipLogger
from .network import NetworkUtils
from .node import EvolutionaryTrainingNode, WeightUpdate, blend_alpha, pair_ranks

__all__ = ["EvolutionaryTrainingNode", "FitnessTracker", "NetworkUtils", "FilesystemCoordinator", "GossipLogger",
           "WeightUpdate", "pair_ranks", "blend_alpha"]
