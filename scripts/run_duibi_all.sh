#!/usr/bin/env bash
# Runs the comparison matrix (full / LoRA x single / DP / TP) one configuration after another, as the
# reference's scripts/run_duibi_all.sh does; every run writes its own output directory.
set -euo pipefail
cd "$(dirname "$0")/.."
ITER=${ITER:-20}
for cfg in configs/experiments/duibi/*.yaml; do
  name=$(basename "$cfg" .yaml)
  gpus=$(python - "$cfg" <<'PY'
import sys, yaml
y = yaml.safe_load(open(sys.argv[1]))
r, d = y.get("runtime", {}), y.get("distributed", {})
print(r.get("tp_size", 1) * r.get("dp_size", 1) * d.get("pp_size", 1))
PY
)
  echo "== $name on $gpus GPU(s)"
  if [ "$gpus" -gt 1 ]; then
    python -m torch.distributed.run --nnodes=1 --nproc-per-node="$gpus" --master-addr 127.0.0.1 \
      scripts/run_colocate.py --config "$cfg" --iterations "$ITER" --output-dir "outputs/duibi/$name" --synthetic
  else
    python scripts/run_colocate.py --config "$cfg" --iterations "$ITER" --output-dir "outputs/duibi/$name" --synthetic
  fi
done
