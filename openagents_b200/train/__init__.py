"""Data-parallel trainer: GPT-2-shape model on the sm_100a kernels, sharded AdamW fused with its
collectives, checkpoint layout with content digests, and the run/window state machine."""
