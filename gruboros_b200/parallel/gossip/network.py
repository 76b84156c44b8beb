"""Peer discovery and socket helpers for the TCP transport of the gossip protocol.

Conventions are the reference's (gossip/network_utils.py:12-149): every rank listens on 29501 + local_rank; the
peer list is every (node, local rank) pair of the job except oneself, with node names taken from
`scontrol show hostnames $SLURM_JOB_NODELIST` or the first column of `hostfile-job*.txt`, and RANKS_PER_NODE
ranks per node (8 when unset).  In addition, with neither SLURM nor a hostfile but a multi-rank single-node job
(RANK/WORLD_SIZE from torchrun) the peers are the other local ranks on localhost, so a bare 8-GPU box mixes too.
"""
from __future__ import annotations

import glob
import os
import socket
import subprocess

BASE_PORT = 29501


class NetworkUtils:
    @staticmethod
    def optimize_socket(sock) -> None:
        sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        for opt in (socket.SO_SNDBUF, socket.SO_RCVBUF):
            sock.setsockopt(socket.SOL_SOCKET, opt, 16 * 1024 * 1024)
        if hasattr(socket, "TCP_QUICKACK"):
            sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_QUICKACK, 1)

    @staticmethod
    def get_gossip_port(local_rank: int) -> int:
        return int(os.environ.get("GOSSIP_BASE_PORT", BASE_PORT)) + local_rank

    @staticmethod
    def _discover_peer_nodes(logger=None) -> list[str]:
        nodelist = os.environ.get("SLURM_JOB_NODELIST")
        if nodelist:
            try:
                out = subprocess.run(["scontrol", "show", "hostnames", nodelist], capture_output=True, text=True,
                                     check=True).stdout
                return sorted({h for h in out.split() if h})
            except Exception as exc:
                if logger:
                    logger.warning(f"scontrol failed: {exc}")
        files = glob.glob(f"hostfile-job{os.environ.get('SLURM_JOB_ID', '*')}.txt")
        if files:
            try:
                with open(files[0]) as f:
                    return sorted({line.split()[0] for line in f if line.strip()})
            except OSError as exc:
                if logger:
                    logger.warning(f"could not read {files[0]}: {exc}")
        return []

    @staticmethod
    def get_bootstrap_nodes(global_rank: int, local_rank: int, logger=None) -> list[str]:
        nodes = NetworkUtils._discover_peer_nodes(logger)
        try:
            ranks_per_node = int(os.environ["RANKS_PER_NODE"])
        except (KeyError, ValueError):
            ranks_per_node = 8
        if not nodes:
            world = int(os.environ.get("WORLD_SIZE", "1"))
            local_world = int(os.environ.get("LOCAL_WORLD_SIZE", world))
            if world > 1 and local_world == world:
                return [f"localhost:{NetworkUtils.get_gossip_port(r)}" for r in range(world) if r != local_rank]
            if logger:
                logger.error(f"rank {global_rank}: no peer nodes found; gossip will not mix")
            return []
        me = socket.getfqdn().split(".")[0]
        peers = []
        for node in nodes:
            for lr in range(ranks_per_node):
                if node.startswith(me) and lr == local_rank:
                    continue
                peers.append(f"{node}:{NetworkUtils.get_gossip_port(lr)}")
        return peers

    @staticmethod
    def get_local_node_address() -> str:
        master = os.environ.get("MASTER_ADDR", "localhost")
        if master in ("localhost", "127.0.0.1"):
            return "localhost"
        try:
            with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as s:
                s.connect((master, 80))
                return s.getsockname()[0]
        except OSError:
            try:
                return socket.gethostbyname(socket.gethostname())
            except OSError:
                return "localhost"

    @staticmethod
    def get_node_identity(local_rank: int) -> tuple[str, int]:
        return NetworkUtils.get_local_node_address(), NetworkUtils.get_gossip_port(local_rank)
