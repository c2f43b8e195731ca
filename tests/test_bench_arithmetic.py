"""The roofline arithmetic of bench.py without a GPU: the bytes a decode step has to read and the
work of a prompt, at the Qwen3-8B layer sizes the default run uses; the peaks file's reading; the
answers that need no GPU (more than one GPU, the reference arm)."""
import json
import os
import subprocess
import sys


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402
import ultima_b200 as u  # noqa: E402


def test_bytes_of_a_decode_step_and_work_of_a_prompt():
    cfg = u.config_from_dict(dict(bench.QWEN3_8B))
    # 36 layers of (6144 + 4096 + 3 * 12288) x 4096 weights and the head, two bytes each
    layer = 4096 * (4096 + 2 * 1024) + 4096 * 4096 + 3 * 4096 * 12288
    mats = 36 * layer + 151936 * 4096
    assert bench.weight_bytes(cfg) == 2 * mats + 4 * (36 * (2 * 4096 + 2 * 128) + 4096)
    assert abs(bench.weight_bytes(cfg) / 1e9 - 15.14) < 0.01
    # keys and values of one position: 36 layers x 8 heads x 128 x 2 tensors x 2 bytes = 144 KiB
    assert bench.kv_bytes_per_token(cfg, 2) == 147456
    # one prompt of 2,048 tokens: 28.45 TFLOP in the products, 1.24 in causal attention, the head once
    f = bench.prefill_flops(cfg, 2048)
    assert abs(f / 1e12 - 29.7) < 0.05
    assert f == 2 * 2048 * 36 * layer + 36 * 4 * 32 * 128 * (2048 * 2049 // 2) + 2 * 151936 * 4096


def test_peaks_come_from_the_file_when_it_is_there(tmp_path, monkeypatch):
    assert bench.peaks()["source"] in ("fallback", "measured")
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.peaks() == {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                             "source": "fallback"}
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6900, "bf16_tflops": 1650.5,
                                                              "bf16_tflops_sustained": 1410}))
    assert bench.peaks() == {"hbm_gbs": 6900.0, "bf16_tflops": 1650.5, "bf16_tflops_sustained": 1410.0,
                             "source": "measured"}
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6900, "bf16_tflops": 1650.5}))
    assert bench.peaks()["bf16_tflops_sustained"] == 1650.5
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert bench.peaks()["source"] == "fallback"


def test_more_than_one_gpu_is_answered_with_one_line_and_code_2():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True,
                       timeout=300)
    lines = [x for x in p.stdout.splitlines() if x.strip()]
    assert p.returncode == 2 and len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_unavailable_where_it_cannot_be_built(tmp_path, monkeypatch, capsys):
    """Neither a program built before nor the reference's sources: one JSON line with the reason, code 0."""
    import argparse
    os.makedirs(tmp_path / "baseline")
    (tmp_path / "baseline" / "ref_bench.cpp").write_text("// stand-in\n")
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    monkeypatch.setenv("ULTIMA_REFERENCE_DIR", str(tmp_path / "nowhere"))
    assert bench.run_reference(argparse.Namespace(steps=None, warmup=3)) == 0
    lines = [x for x in capsys.readouterr().out.splitlines() if x.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and "sources are not on this machine" in d["unavailable"] and "\n" not in d["unavailable"]
