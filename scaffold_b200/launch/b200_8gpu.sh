#!/bin/bash
# One 8 x B200 node: generate the fractal library, then train to the target Dice.
#
#   scaffold_b200/launch/b200_8gpu.sh [problem_scale] [dc_num_shards "D H W"] [extra `scaffold benchmark` flags...]
#
#   scaffold_b200/launch/b200_8gpu.sh 7                 # 8 data-parallel replicas
#   scaffold_b200/launch/b200_8gpu.sh 8 "1 1 2"         # 4 replicas x 2 shards along W (fused halo)
#   scaffold_b200/launch/b200_8gpu.sh 9 "2 2 2"         # one replica over all 8 GPUs
#
# One rank per GPU over NCCL; the halo exchange, the cross-shard GroupNorm statistics and the gradient
# all-reduce run over NVLink peer memory from inside the kernels (fused is the default of all three).
# Role of the reference's job script: scripts/scaffold-matrix.job:15-28.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REPO="$(cd "$HERE/../.." && pwd)"
SCALE="${1:-7}"
SHARDS="${2:-1 1 1}"
shift $(( $# > 2 ? 2 : $# ))
GPUS="${GPUS:-8}"
CONFIG="${CONFIG:-$REPO/scaffold_b200/configs/benchmark_default.yml}"
export MASTER_ADDR="${MASTER_ADDR:-127.0.0.1}"
export MASTER_PORT="${MASTER_PORT:-29500}"
# export PROFILE_TORCH=ON        # bounded torch.profiler trace of a few steps per rank
# export SCAFFOLD_NVTX=1         # NVTX ranges around the regions of a step

cd "$REPO"
python -m scaffold_b200.build    # nvcc -> scaffold_b200/_native/libscaffold_b200.so (a no-op when up to date)

# the fractal library (IFS categories + instances) is generated once and reused by every scale
python -m torch.distributed.run --nnodes=1 --nproc-per-node="$GPUS" --master-addr "$MASTER_ADDR" \
    --master-port "$MASTER_PORT" -m scaffold_b200.cli generate_fractals -c "$CONFIG" --problem-scale "$SCALE"

# shellcheck disable=SC2086
python -m torch.distributed.run --nnodes=1 --nproc-per-node="$GPUS" --master-addr "$MASTER_ADDR" \
    --master-port "$MASTER_PORT" -m scaffold_b200.cli benchmark -c "$CONFIG" --problem-scale "$SCALE" \
    --dc-num-shards $SHARDS "$@"
