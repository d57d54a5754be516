"""Worker (gloo, 4 ranks): tensor-parallel pipeline stages (tensor 2 x pipeline 2) write one ``torch_dist`` checkpoint -
every rank its own slices of its own stage, placed by global rank inside its tensor-parallel sub-group - that loads into
the unsplit model and back into the same layout.  argv: checkpoint directory"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.checkpoint import megatron as M
from mlperf_training_b200.models.gpt import GPT, GPTConfig
from mlperf_training_b200.parallel.mesh import Mesh, MeshSpec
from mlperf_training_b200.parallel.pipeline import GPTStage
from mlperf_training_b200.parallel.tensor import TPContext
root = sys.argv[1]
dist.init_process_group("gloo")
rank = dist.get_rank()
cfg = GPTConfig(n_layers=4, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_hidden=96, vocab_size=128, seq_len=32, dtype="fp32")
full = GPT(cfg, device="cpu", seed=11)
mesh = Mesh(MeshSpec(tp=2, pp=2))
tp = TPContext(mesh.group("tp"), comm="nccl", device="cpu")
stage = GPTStage(cfg, mesh.index("pp"), 2, device="cpu", tp=tp)
stage.load_from_full(full)
M.save_torch_dist(stage, root, iteration=1)
back = GPT(cfg, device="cpu", seed=99)
M.load_torch_dist(back, root)
ok = all(torch.equal(a, b) for (_, a), (_, b) in zip(full.named_parameters(), back.named_parameters()))
again = GPTStage(cfg, mesh.index("pp"), 2, device="cpu", tp=tp)
M.load_torch_dist(again, root)
ok &= all(torch.equal(a, b) for (_, a), (_, b) in zip(stage.named_parameters(), again.named_parameters()))
print(f"RESULT rank {rank} ok={ok}", flush=True)
dist.barrier(); dist.destroy_process_group()
