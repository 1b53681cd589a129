#!/bin/bash
#SBATCH --job-name=llmc-b200-multinode
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=8
#SBATCH --gres=gpu:8
# One task per GPU; ranks rendezvous through a file on a shared file system (the reference's -pi fs scheme).
sync_dir=$HOME/llmc_b200_sync_$SLURM_JOB_ID
mkdir -p $sync_dir
srun bash -c 'python train_gpt2.py -i "dev/data/fineweb10B/fineweb_train_*.bin" -j "dev/data/fineweb10B/fineweb_val_*.bin" \
    -o log_gpt2_124M_multi -v 250 -s 20000 -g 144 -h 1 -b 64 -t 1024 -d 2097152 -r 0 -z 1 -c 0.1 -l 0.0006 -q 0.1 -u 700 -n 1000 -y 1 -e d12 \
    -pn $SLURM_NTASKS -pr $SLURM_PROCID -pg 8 -pi fs -pf '"$sync_dir"' -cb nccl'
