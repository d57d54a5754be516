# DLRMv4 / HSTU generative recommender, 1 node x 8 B200.
# Reference counterpart: recommendation_v4/hstu/config_MI355X_1x8x1.sh.
export DGXNNODES=1
export DGXNGPU=8
export NGPU=8
export TRAIN_MODE=hstu
export EXP=conf/hstu_yambda.yaml
export MASTER_ADDR=127.0.0.1
export NCCL_SOCKET_IFNAME=lo
export BATCH_PER_GPU=128
export HSTU_LAYERS=8
export HSTU_DIM=512
export HSTU_HEADS=4
export MAX_SEQ_LEN=4096
export TABLE_ROWS=400000000
export TABLE_DIM=256
export DENSE_LR=1e-6
export SPARSE_LR=1e-6
export LR_WARMUP_STEPS=24000
export CLIP_GRAD=1.0
export AUC_THRESHOLD=0.75
export EVAL_INTERVAL_STEPS=280
export HSTU_ATTN_PRECISION=fp8
export EMB_A2A=fused
export TRAIN_PIPELINE=1
export DATA_KIND=synthetic
export MLLOG_SUBMISSION_PLATFORM=1xB200x8
