"""Multi-GPU plumbing: symmetric buffers over NVLink peer memory, the sharded DP step engine, expert parallelism."""
