# FLUX.1-schnell, 1 node x 8 B200, local batch 32 (global 256).
source "$(dirname "${BASH_SOURCE[0]}")/config_common.sh"
export DGXNNODES=1
export DGXNGPU=8
export NGPU=8
export GBS=256
export LR_WARMUP_ITERS=800
export MLLOG_SUBMISSION_PLATFORM=1xB200x8
