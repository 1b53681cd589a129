#!/bin/bash
# Multi-node data-parallel / ZeRO-1 run, one process per GPU.  Start this on every node with the same MASTER_ADDR:
#   NNODES=2 NODE_RANK=0 MASTER_ADDR=10.0.0.1 ./run_gpt2_124M_torchrun.sh
# (the in-kernel NVLink path covers one NVSwitch domain; across nodes the NCCL backend is used: -cb nccl)
NNODES=${NNODES:-2}; NODE_RANK=${NODE_RANK:-0}; MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}; MASTER_PORT=${MASTER_PORT:-29500}
python -m torch.distributed.run --nnodes=$NNODES --node-rank=$NODE_RANK --nproc-per-node 8 --master-addr $MASTER_ADDR --master-port $MASTER_PORT \
    train_gpt2.py -i "dev/data/fineweb10B/fineweb_train_*.bin" -j "dev/data/fineweb10B/fineweb_val_*.bin" -o log_gpt2_124M_multi \
    -v 250 -s 20000 -g 144 -h 1 -b 64 -t 1024 -d 2097152 -r 0 -z 1 -c 0.1 -l 0.0006 -q 0.1 -u 700 -n 1000 -y 1 -e d12 -cb nccl
