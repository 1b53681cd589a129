"""GPT-2 / GPT-3 pretraining on B200 with the flags of the reference trainer, e.g.

    python train_gpt2.py -e d12 -b 64 -t 1024 -d 524288 -z 1 -l 6e-4 -u 700 -q 0.0 -c 0.1 -i 'data/train_*.bin' -j 'data/val_*.bin'
    torchrun --standalone --nproc-per-node 8 train_gpt2.py -e d12 -b 64 -t 1024 -d 524288 -z 1 ...

See ``llm.c_b200/train.py`` for the flag list."""
import sys

from llmc_b200.train import main

if __name__ == "__main__":
    sys.exit(main())
