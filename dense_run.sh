#!/bin/bash
# Dense S-SGD baseline (NCCL all-reduce), one process per GPU.
#   dnn=resnet50 nworkers=8 ./dense_run.sh [extra trainer flags]
cd "$(dirname "$0")"
dnn="${dnn:-resnet20}"
source exp_configs/$dnn.conf
nworkers="${nworkers:-4}"
nwpernode="${nwpernode:-$nworkers}"
PY="${PY:-python}"
NCCL_DEBUG="${NCCL_DEBUG:-WARN}" $PY -m torch.distributed.run --nnodes=1 --nproc-per-node "$nworkers" \
    --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29534}" dense_trainer.py --dnn $dnn --dataset $dataset \
    --max-epochs $max_epochs --batch-size $batch_size --nworkers $nworkers --data-dir $data_dir --lr $lr \
    --nsteps-update $nstepsupdate --nwpernode $nwpernode "$@"
