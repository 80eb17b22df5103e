#!/bin/bash
# Time to validation Dice: this framework and the reference's pieces on the SAME generated dataset.
#
#   baseline/time_to_dice.sh <gpus> <problem_scale> <n_instances_per_class> <local_batch> <out_dir> [max_epochs]
#
# 1. `scaffold generate_fractals` + `scaffold benchmark` (this framework) until target_dice 0.95;
# 2. `baseline/reference_train.py` (reference U-Net, losses, optimizer, scheduler, dataset class) on the dataset
#    that step 1 generated, same batch size, seeds and schedule.
# Both write train_stats.csv; the summary lines land in <out_dir>/summary.txt.
set -euo pipefail
GPUS="${1:-1}"; SCALE="${2:-7}"; NINST="${3:-32}"; BATCH="${4:-1}"; OUT="${5:-out/ttd}"; MAXEP="${6:-120}"
REPO="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
cd "$REPO"
WORK="${WORK:-/tmp/scaffold_ttd}"
mkdir -p "$OUT" "$WORK"
cat > "$WORK/override.yml" <<YML
base_run_dir: $WORK/runs
dataset_dir: $WORK/datasets
fract_base_dir: $WORK/fractals
problem_scale: $SCALE
n_instances_used_per_fractal: $NINST
local_batch_size: $BATCH
warmup_batches: 4
epochs: $MAXEP
dataloader_num_workers: 4
job_name: ttd
YML
CFG="$REPO/scaffold_b200/configs/benchmark_default.yml"
LAUNCH="python"
if [ "$GPUS" -gt 1 ]; then
  LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node=$GPUS --master-addr 127.0.0.1 --master-port 29533"
fi
t0=$(date +%s)
$LAUNCH -m scaffold_b200.cli generate_fractals -c "$CFG" -c "$WORK/override.yml" > "$OUT/generate.log" 2>&1
$LAUNCH -m scaffold_b200.cli benchmark -c "$CFG" -c "$WORK/override.yml" > "$OUT/ours.log" 2>&1
t1=$(date +%s)
RUN_DIR="$(ls -d "$WORK"/runs/*ttd* | tail -n 1)"
cp "$RUN_DIR/train_stats.csv" "$OUT/ours_train_stats.csv"
DATASET="$(python -c "import yaml,sys; print(yaml.safe_load(open('$RUN_DIR/run_metadata.yaml'))['result']['dataset_path'])")"
{
  echo "ours: gpus=$GPUS scale=$SCALE instances/class=$NINST batch/replica=$BATCH  (datagen + training wall: $((t1 - t0)) s)"
  grep -E "FOM|Median of epoch" "$OUT/ours.log" | tail -3
} > "$OUT/summary.txt"
REFL="python"
if [ "$GPUS" -gt 1 ]; then
  REFL="python -m torch.distributed.run --nnodes=1 --nproc-per-node=$GPUS --master-addr 127.0.0.1 --master-port 29534"
fi
$REFL baseline/reference_train.py --dataset-dir "$DATASET" --n-categories 5 --scale "$SCALE" --batch "$BATCH" \
    --max-epochs "$MAXEP" --workers 4 --out "$OUT/reference" > "$OUT/reference.log" 2>&1 || true
cp "$OUT/reference/train_stats.csv" "$OUT/reference_train_stats.csv" 2>/dev/null || true
{ echo "reference:"; tail -n 1 "$OUT/reference.log"; } >> "$OUT/summary.txt"
cat "$OUT/summary.txt"
