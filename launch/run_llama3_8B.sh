#!/bin/bash
# LLaMA-3.1 8B architecture on one node of 8 B200 (ZeRO-1 over this library's in-kernel NVLink path), with the restart loop of the
# GPT-2 scripts.  Token shards are the 32-bit files of the reference (dev/data/*.py --model_desc llama-3); pass pretrained weights
# as a model file made by `python -m llmc_b200.utils.llama_convert --hf-dir <dir> --out llama3_8B.bin`, or keep the descriptor for
# random initialisation.
#   micro-batch 1 x 8192 tokens per GPU, 524288 tokens per step (8 accumulation steps), SwiGLU recomputed in backward (-r 1)
#   memory per GPU: 16 GB parameters + 16 GB gradients + 12 GB optimizer shards + about 36 GB activations
NPROC=${NPROC:-8}
MODEL=${MODEL:-llama3:8B}
OUT=${OUT:-log_llama3_8B}
TRAIN=${TRAIN:-"data/llama3_train_*.bin"}
VAL=${VAL:-"data/llama3_val_*.bin"}
STEPS=${STEPS:-10000}
DONE="$OUT/DONE_$(printf '%08d' $STEPS)"
while true; do
    [ -f "$DONE" ] && echo "$DONE exists, training is complete" && break
    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node $NPROC train_llama3.py \
        --model "$MODEL" --input_bin "$TRAIN" --input_val_bin "$VAL" --output_dir "$OUT" \
        --batch_size 1 --sequence_length 8192 --total_batch_size 524288 --zero_stage 1 --recompute 1 \
        --learning_rate 3e-4 --warmup_iters 700 --learning_rate_decay_frac 0.1 --weight_decay 0.1 \
        --num_iterations $STEPS --val_loss_every 250 --val_max_steps 20 --sample_every 0 --overfit_single_batch 0 \
        --checkpoint_every 1000 --resume 1 --watchdog_s 1800
    sleep 1
done
