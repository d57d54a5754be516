"""b200-train: a Blackwell-native (sm_100a) training framework.

Sub-packages: ``ops`` (hand-written CUDA kernels + their eager oracles), ``models`` (GPT dense /
MoE, LoRA, MMDiT, HSTU), ``parallel`` (mesh, FSDP/ZeRO engine, TP/SP, EP, pipeline, sharded
embeddings, symmetric memory), ``optim``, ``data``, ``checkpoint``, ``trainer``, ``config``,
``logging``, ``utils``.
"""
__version__ = "0.1.0"
