# FLUX.1-schnell MMDiT flow-matching training: settings shared by every system file.
# Reference counterpart: flux1/primus/config_common.sh.
export TRAIN_MODE=flux
export EXP=conf/flux.1_schnell_t2i-pretrain.yaml
export LOCAL_BATCH=32
export IMG_SIZE=256
export TXT_TOKENS=256
export LR=2.5e-4
export WEIGHT_DECAY=0.1
export ADAM_BETA2=0.95
export PROMPT_DROPOUT=0.1
export TARGET_EVAL_LOSS=0.586
export EVAL_EVERY_SAMPLES=262144
export PRECISION=mxfp8
export FSDP_RESHARD_AFTER_FORWARD=0
export FSDP_COMM=fused
export GRAD_CHECKPOINT_RATIO=0.0
export SEED=10007
export DATA_KIND=synthetic
