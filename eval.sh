#!/bin/bash
# Evaluate the checkpoints of one run epoch by epoch:
#   model_path=weights/<prefix>/resnet20-n4-bs32-lr0.1000 dnn=resnet20 dataset=cifar10 nepochs=141 ./eval.sh
cd "$(dirname "$0")"
dnn="${dnn:-resnet20}"
dataset="${dataset:-cifar10}"
data_dir="${data_dir:-./data}"
nepochs="${nepochs:-90}"
PY="${PY:-python}"
$PY evaluate.py --model-path "$model_path" --dnn $dnn --dataset $dataset --data-dir $data_dir --nepochs $nepochs
