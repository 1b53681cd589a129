"""This framework against the unmodified reference binary on one GPU (baseline/_ref/train_gpt2cu, built as baseline/README.md
says; the tests skip when it is absent): loss curves from the same initialisation and data, and checkpoints written by one
trainer resumed by the other (reference: train_gpt2.cu write_checkpoint / load_state, test_gpt2.cu:326-367)."""
import io
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))

pytestmark = pytest.mark.gpu


def _module():
    import loss_parity
    if not os.path.exists(loss_parity.EXE):
        pytest.skip("baseline/_ref/train_gpt2cu is not built")
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return loss_parity


SMALL = ["--model", "d6", "--batch", "8", "--seq", "256", "--total-batch", "4096", "--tol", "0.03"]


def test_loss_curve_matches_the_reference_trainer():
    lp = _module()
    out = io.StringIO()
    worst = lp.loss_parity(lp.parse(SMALL + ["--steps", "10"]), out)
    assert worst < 0.03, out.getvalue()


def test_checkpoints_cross_load_with_the_reference_trainer():
    lp = _module()
    out = io.StringIO()
    worst = lp.cross_load(lp.parse(SMALL + ["--cross-load", "--checkpoint-step", "5"]), out)
    assert worst < 0.03, out.getvalue()
