"""The ncu post-processor (llmc_b200/profile_step.py report): both CSV layouts that ncu writes, phase classification, scaling of
the per-layer phases, DRAM / tensor-pipe columns and the efficiency score."""
import io

from llmc_b200 import profile_step

KERNELS = [("encoder_fwd_kernel(a)", 10, 1e6, 2e6, 0.0), ("void <unnamed>::layernorm_fwd_kernel(a)", 5, 1e6, 1e6, 0.0),
           ("void <unnamed>::gemm2_kernel<0,0,0>(a)", 100, 5e6, 5e6, 70.0), ("void <unnamed>::gemm2_kernel<0,0,0>(a)", 300, 9e6, 9e6, 80.0),
           ("classifier_kernel(a)", 200, 4e8, 4e8, 0.0), ("void <unnamed>::gemm2_kernel<0,1,0>(a)", 300, 9e6, 9e6, 75.0),
           ("ln_bwd_kernel(a)", 50, 1e8, 1e8, 0.0), ("norm_sq_kernel(a)", 20, 1e8, 0.0, 0.0), ("adamw_pack_kernel<true>(a)", 80, 4e8, 4e8, 0.0)]
TC = "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active"


def long_csv(steps=2):
    head = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'
    out, k = ["==PROF== Connected\n", head], 0
    for _ in range(steps):
        for name, us, rd, wr, tc in KERNELS:
            for metric, unit, val in (("gpu__time_duration.sum", "us", us), ("dram__bytes_read.sum", "Mbyte", rd / 1e6),
                                      ("dram__bytes_write.sum", "byte", wr), (TC, "%", tc)):
                out.append('"%d","1","python","h","%s","1","7","(256, 1, 1)","(1, 1, 1)","0","10.0","x","%s","%s","%s"\n' % (k, name, metric, unit, val))
            k += 1
    return "".join(out)


def raw_csv():
    head = ["ID", "Kernel Name", "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum", TC]
    units = ["", "", "us", "byte", "byte", "%"]
    lines = [",".join('"%s"' % h for h in head), ",".join('"%s"' % u for u in units)]
    for k, (name, us, rd, wr, tc) in enumerate(KERNELS):
        lines.append(",".join('"%s"' % x for x in (k, name, us, rd, wr, tc)))
    return "\n".join(lines) + "\n"


def test_report_phases_and_scaling(tmp_path):
    for text in (long_csv(), raw_csv()):
        path = tmp_path / "launches.csv"
        path.write_text(text)
        buf = io.StringIO()
        res = profile_step.report(str(path), out=buf, layers_profiled=1, layers_model=12)
        ph = res["phases"]
        assert abs(ph["enc"]["t"] - 10e3) < 1 and abs(ph["fwd"]["t"] - 12 * 105e3) < 1          # per-layer work x 12
        assert abs(ph["cls"]["t"] - 800e3) < 1                                                  # LM head fwd + loss + LM head bwd GEMM, once
        assert abs(ph["bwd"]["t"] - 12 * 50e3) < 1 and abs(ph["opt"]["t"] - 100e3) < 1
        text_out = buf.getvalue()
        assert "efficiency" in text_out and "summary for 12 layers" in text_out
        # the classifier moves 800 MB in 200 us = 4000 GB/s
        row = [l for l in text_out.splitlines() if l.startswith("cls") and "classifier" in l][0]
        assert row.split()[-1] == "4000"


def test_report_takes_the_last_step(tmp_path):
    path = tmp_path / "launches.csv"
    path.write_text(long_csv(steps=3))
    res = profile_step.report(str(path), out=io.StringIO())
    assert sum(a["n"] for a in res["kernels"].values()) == len(KERNELS)


def test_dataset_entry_points_and_eval_summary(tmp_path, capsys):
    import json
    import numpy as np
    from llmc_b200.eval import summarize_eval
    from llmc_b200.utils import data_prep, vislog
    txt = tmp_path / "input.txt"
    txt.write_text("First Citizen:\nBefore we proceed.\n\nAll:\nSpeak, speak.\n\n" * 40)
    assert data_prep.main(["tinyshakespeare", str(txt), "-o", str(tmp_path / "ts"), "--encoder", "bytes"]) == 0
    head = np.fromfile(str(tmp_path / "ts_val.bin"), dtype=np.int32, count=3)
    assert head[0] == 20240520 and head[1] == 1
    jl = tmp_path / "fw.jsonl"
    jl.write_text("\n".join(json.dumps({"text": "document %d " % i * 20}) for i in range(30)))
    assert data_prep.main(["fineweb", str(jl), "-o", str(tmp_path / "fw"), "--encoder", "bytes", "--shard-size", "2000"]) == 0
    assert (tmp_path / "fw_val_000000.bin").exists() and (tmp_path / "fw_train_000001.bin").exists()
    hs = tmp_path / "hs.jsonl"
    hs.write_text(json.dumps({"ctx": "A man is", "endings": ["running", "a", "b", "c"], "label": 0}) + "\n")
    assert data_prep.main(["hellaswag", str(hs), "-o", str(tmp_path / "hs.bin"), "--encoder", "bytes"]) == 0
    assert np.fromfile(str(tmp_path / "hs.bin"), dtype=np.int32, count=3)[0] == 20240522
    # evaluation summary: mean over sub-tasks, missing files reported, average over what is there
    res = tmp_path / "results"
    res.mkdir()
    (res / "mmlu_5shot.json").write_text(json.dumps({"results": {"a": {"acc": 0.25}, "b": {"acc": 0.35}}}))
    (res / "hellaswag_10shot.json").write_text(json.dumps({"results": {"hellaswag": {"acc": 0.3, "acc_norm": 0.5}}}))
    scores = summarize_eval.summarize(str(res))
    assert abs(scores["mmlu_5shot.json"] - 30.0) < 1e-9 and abs(scores["hellaswag_10shot.json"] - 50.0) < 1e-9
    assert "missing" in capsys.readouterr().out
    # log visualiser: streams and the command line (the figure itself needs matplotlib)
    log = tmp_path / "main.log"
    log.write_text("s:0 tel:10.9\ns:0 trl:10.8 lr:0.0001 norm:1.5\ns:1 trl:10.1 lr:0.0002 norm:1.2\ns:1 eval:0.25\n")
    assert vislog.main([str(log), "--out", str(tmp_path / "c.png")]) == 0
    out = capsys.readouterr().out
    assert "trl" in out and "eval" in out


def test_loss_parity_helpers(tmp_path):
    """The comparison tool's parsing and bookkeeping (the runs themselves need a GPU and the reference binary)."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
    import loss_parity as lp
    text = "step    1/10 | loss 10.978783 (+nanz)| norm 1.2 (+nanz)| lr 8.57e-07 | 944.66 ms | 19.2% bf16 MFU | 555001 tok/s\n" \
           "val loss 10.9\nstep    2/10 | loss 10.500000 (+0.10z)| norm 1.1\n"
    assert lp.losses_from(text) == {1: 10.978783, 2: 10.5}
    for name in ("DONE_00000005", "DONE_00000010", "model_00000010.bin", "state_00000010_00000.bin"):
        (tmp_path / name).write_bytes(b"x")
    lp.forget_later_checkpoints(str(tmp_path), 5)
    assert sorted(os.listdir(tmp_path)) == ["DONE_00000005", "model_00000010.bin", "state_00000010_00000.bin"]
    out = io.StringIO()
    worst = lp.compare("t", {6: 1.0, 7: 2.0}, {6: 1.01, 7: 1.98}, range(6, 8), 0.05, out)
    assert abs(worst - 0.02) < 1e-9 and "largest difference" in out.getvalue()
    assert lp.compare("t", {6: 1.0}, {}, range(6, 7), 0.05, io.StringIO()) == float("inf")
    a = lp.parse(["--cross-load", "--checkpoint-step", "3", "--model", "d6"])
    assert a.cross_load and a.checkpoint_step == 3 and a.model == "d6"


def test_both_kernel_libraries_build_and_identify_themselves():
    """The normal and the debug build of the kernel library compile for sm_100a without a GPU, and each says which one it is."""
    import ctypes
    from llmc_b200 import build
    normal, dbg = build.build_cuda(), build.build_cuda_debug()
    assert ctypes.CDLL(normal).llmc_debug_checks_enabled() == 0
    assert ctypes.CDLL(dbg).llmc_debug_checks_enabled() == 1
