"""Stock-PyTorch baselines (cuBLAS GEMMs, SDPA attention, torch optimizers, NCCL collectives) of the
benchmark configs, measured on the same box as the hand-written kernels."""
