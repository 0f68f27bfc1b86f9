#!/usr/bin/env bash
# Pipeline bubble test: the same SFT job with pp=1 and pp=2 (1F1B), printing iteration time so that the
# bubble fraction (pp-1)/num_micro_batches can be compared with the measured slowdown.
set -euo pipefail
cd "$(dirname "$0")/.."
for cfg in configs/training/pp_equiv_pp1.yaml configs/training/pp_equiv_pp2.yaml; do
  gpus=$(python -c "import yaml,sys; y=yaml.safe_load(open('$cfg')); print(y.get('distributed',{}).get('pp_size',1)*y.get('runtime',{}).get('tp_size',1)*y.get('runtime',{}).get('dp_size',1))")
  echo "== $cfg ($gpus GPUs)"
  python -m torch.distributed.run --nnodes=1 --nproc-per-node="$gpus" --master-addr 127.0.0.1 \
    scripts/run_colocate.py --config "$cfg" --synthetic --output-dir "outputs/bubble/$(basename "$cfg" .yaml)"
done
