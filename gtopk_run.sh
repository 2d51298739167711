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
$PY -m torch.distributed.run --nnodes=1 --nproc-per-node "$nworkers" --master-addr 127.0.0.1 \
    --master-port "${MASTER_PORT:-29533}" gtopk_trainer.py --dnn $dnn --dataset $dataset \
    --max-epochs $max_epochs --batch-size $batch_size --nworkers $nworkers --data-dir $data_dir --lr $lr \
    --nwpernode $nwpernode --nsteps-update $nstepsupdate --compression --sigma-scale $sigmascale \
    --density $density --compressor $compressor "$@"
