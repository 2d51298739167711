#!/bin/bash
# Single-GPU training:  dnn=resnet20 ./single.sh [extra trainer flags]
cd "$(dirname "$0")"
dnn="${dnn:-resnet20}"
source exp_configs/$dnn.conf
PY="${PY:-python}"
$PY dl_trainer.py --dnn $dnn --dataset $dataset --max-epochs $max_epochs --batch-size $batch_size \
    --data-dir $data_dir --lr $lr --nsteps-update $nstepsupdate "$@"
