#!/bin/bash
# GPT-3 (125M) on FineWeb, 300B tokens, context 2048
# 8 x B200
# The run restarts itself from the latest checkpoint until the DONE file of the last step exists
# (same crash-resume scheme as the reference's scripts/run_*.sh).
NPROC=${NPROC:-8}
out_dir="log_gpt3_125M"
done_file="$out_dir/DONE_00572204"
train_data="${TRAIN_DATA:-dev/data/fineweb10B/fineweb_train_*.bin}"
val_data="${VAL_DATA:-dev/data/fineweb10B/fineweb_val_*.bin}"
while true; do
    if [ -f "$done_file" ]; then
        echo "File $done_file exists. Exiting the loop."
        break
    fi
    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node $NPROC train_gpt2.py \
        -i "$train_data" -j "$val_data" -o $out_dir \
        -v 250 -s 20000 -g 144 -h 1 \
        -b 32 -t 2048 -d 524288 -r 0 -z 1 -c 0.1 -l 0.0006 -q 0.1 -u 700 \
        -n 10000 -nk 5 -nm 100000 -sl 7.0 -sg 7.0 \
        -y 1 -wd 1800 -e "gpt3:c768"
    sleep 1
done
