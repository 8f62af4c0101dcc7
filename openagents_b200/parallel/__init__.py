"""Multi-GPU plumbing: the symmetric heap over NVLink peer memory / NVSwitch multicast, the
tensor-parallel communicator used by the serving engine, and the data-parallel sharded optimizer."""
