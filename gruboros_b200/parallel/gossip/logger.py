"""Structured per-rank event log of the gossip protocol.

Same file name and 12-column TSV schema as the reference (gossip/structured_logger.py:10-78):
`<output>/gossip/<ip>_<port>_rank_<r>.tsv` with unix_timestamp, node_identity, global_rank, dp_rank, event_type,
step, ema_loss, correlation_id, peer_addr, data_size_mb, transfer_time_ms, message.  The directory is created
here (the reference leaves that to its launch scripts).
"""
from __future__ import annotations

import threading
import time
import uuid
from pathlib import Path

from .network import NetworkUtils

COLUMNS = ["unix_timestamp", "node_identity", "global_rank", "dp_rank", "event_type", "step", "ema_loss",
           "correlation_id", "peer_addr", "data_size_mb", "transfer_time_ms", "message"]


class GossipLogger:
    def __init__(self, node_id, global_rank, local_rank, data_parallel_rank, output_dir=None):
        self.node_id, self.global_rank = node_id, global_rank
        self.local_rank, self.data_parallel_rank = local_rank, data_parallel_rank
        self.local_ip, self.gossip_port = NetworkUtils.get_node_identity(local_rank)
        self.node_identity = f"{self.local_ip}:{self.gossip_port}"
        log_dir = Path(output_dir) / "gossip" if output_dir else Path("gossip")
        log_dir.mkdir(parents=True, exist_ok=True)
        safe = self.node_identity.replace(":", "_").replace(".", "_")
        self.log_file = log_dir / f"{safe}_rank_{global_rank}.tsv"
        self.lock = threading.Lock()
        if not self.log_file.exists():
            self.log_file.write_text("\t".join(COLUMNS) + "\n")

    def log_event(self, event_type, step=None, fitness=None, correlation_id=None, peer_addr=None,
                  data_size_bytes=None, transfer_time_ms=None, message=""):
        row = [f"{time.time():.6f}", self.node_identity, str(self.global_rank), str(self.data_parallel_rank),
               event_type, "" if step is None else str(step), "" if fitness is None else f"{fitness:.6f}",
               correlation_id or "", peer_addr or "",
               "" if not data_size_bytes else f"{data_size_bytes / 1e6:.3f}",
               "" if transfer_time_ms is None else f"{transfer_time_ms:.2f}", str(message).replace("\t", " ").replace("\n", " ")]
        with self.lock:
            with open(self.log_file, "a") as f:
                f.write("\t".join(row) + "\n")

    @staticmethod
    def generate_correlation_id() -> str:
        return uuid.uuid4().hex[:8]
