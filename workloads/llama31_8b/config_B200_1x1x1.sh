# Llama-3.1-8B pre-training, 1 node x 1 B200 (same per-GPU work).  Values are defaults: a variable already exported wins.
export DGXNNODES=1
export DGXNGPU=1
export NGPU=1
export TRAIN_MODE=pretrain
export EXP=conf/llama3.1_8B-pretrain-mxfp8.yaml
# batch / schedule (reference: small_llm_pretraining/primus/config_MI355X_1x8x1.sh:17-22)
export GBS=4
export MBS=1
export SEQ_LEN=8192
export LR=8e-4
export MIN_LR_RATIO=0.1
export LR_WARMUP_ITERS=64
export LR_DECAY_ITERS=1199936
export TRAIN_ITERS=1200000
export EVAL_INTERVAL=384
export EVAL_ITERS=32
export TARGET_EVAL_LOSS=3.3
# precision / kernels
export PRECISION=mxfp8
export WARMUP_TRAIN_STEPS=2
export WARMUP_EVAL_STEPS=1
# data
export DATA_KIND=synthetic
# communication (NVLink 5 / NVSwitch; NVLS left to NCCL's default)
export NCCL_MIN_CTAS=32
export TORCH_NCCL_HIGH_PRIORITY=1
export CUDA_DEVICE_MAX_CONNECTIONS=1
# MLLOG submission metadata
export MLLOG_SUBMISSION_PLATFORM=1xB200x1
