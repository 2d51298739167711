#!/bin/bash
# gTop-k S-SGD on one NVSwitch box, one process per GPU.
#   dnn=resnet20 nworkers=8 density=0.001 compressor=gtopk ./gtopk_run.sh [extra trainer flags]
# Honours the same variables as the reference's gtopk_mpi.sh (dnn, density, compressor, nworkers)
# plus everything exp_configs/$dnn.conf reads (lr, batch_size, max_epochs, data_dir).
cd "$(dirname "$0")"
dnn="${dnn:-resnet20}"
density="${density:-0.001}"
source exp_configs/$dnn.conf
compressor="${compressor:-gtopk}"
nworkers="${nworkers:-4}"
nwpernode="${nwpernode:-$nworkers}"
sigmascale=2.5
PY="${PY:-python}"
# several machines: run this script on every node with nnodes=<N> node_rank=<i> master_addr=<host of node 0>;
# nworkers is then the number of GPUs used on each node
nnodes="${nnodes:-1}"
node_rank="${node_rank:-0}"
master_addr="${master_addr:-127.0.0.1}"
$PY -m torch.distributed.run --nnodes="$nnodes" --node-rank "$node_rank" --nproc-per-node "$nworkers" --master-addr "$master_addr" \
    --master-port "${MASTER_PORT:-29533}" gtopk_trainer.py --dnn $dnn --dataset $dataset \
    --max-epochs $max_epochs --batch-size $batch_size --nworkers $nworkers --data-dir $data_dir --lr $lr \
    --nwpernode $nwpernode --nsteps-update $nstepsupdate --compression --sigma-scale $sigmascale \
    --density $density --compressor $compressor "$@"
