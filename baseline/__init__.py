"""Plain PyTorch baselines (cuBLAS ``torch.matmul``, fused SDPA, NCCL collectives, stock optimizers).

These are the comparison arm, never the product: nothing here calls this repository's kernels or engine.  The
reference repository contains no inference or training engine to run, so the "NCCL + cuBLAS build" it is compared
against is restated here in the most direct PyTorch form of the same benchmark configurations.
"""
