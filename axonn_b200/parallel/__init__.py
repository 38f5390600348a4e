"""Peer-memory communication: symmetric heap, fused compute+collective kernels,
expert parallelism and the liveness watchdog."""
