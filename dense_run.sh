#!/bin/bash
# Dense S-SGD baseline (NCCL all-reduce), one process per GPU.
#   dnn=resnet50 nworkers=8 ./dense_run.sh [extra trainer flags]
cd "$(dirname "$0")"
dnn="${dnn:-resnet20}"
source exp_configs/$dnn.conf
nworkers="${nworkers:-4}"
nwpernode="${nwpernode:-$nworkers}"
PY="${PY:-python}"
# several machines: run this script on every node with nnodes=<N> node_rank=<i> master_addr=<host of node 0>;
# nworkers is then the number of GPUs used on each node
nnodes="${nnodes:-1}"
node_rank="${node_rank:-0}"
master_addr="${master_addr:-127.0.0.1}"
NCCL_DEBUG="${NCCL_DEBUG:-WARN}" $PY -m torch.distributed.run --nnodes="$nnodes" --node-rank "$node_rank" --nproc-per-node "$nworkers" \
    --master-addr "$master_addr" --master-port "${MASTER_PORT:-29534}" dense_trainer.py --dnn $dnn --dataset $dataset \
    --max-epochs $max_epochs --batch-size $batch_size --nworkers $nworkers --data-dir $data_dir --lr $lr \
    --nsteps-update $nstepsupdate --nwpernode $nwpernode "$@"
