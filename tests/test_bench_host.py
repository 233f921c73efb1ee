"""What `bench.py` decides on the host (CPU): where its peaks come from, its flop and byte counts, and what it
answers when asked for more than one GPU or for the reference arm."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path):
    assert bench.peaks(str(tmp_path)) == (6650.0, 1590.0, "fallback")
    f = tmp_path / "MEASURED_PEAKS.json"
    f.write_text(json.dumps({"hbm_gbs": 7012.5, "bf16_tflops": 1633.0, "bf16_tflops_sustained": 1420.0}))
    assert bench.peaks(str(tmp_path)) == (7012.5, 1633.0, "measured")
    f.write_text(json.dumps({"hbm_gbs": {"value": 7000, "unit": "GB/s"}, "bf16_tflops": None}))
    assert bench.peaks(str(tmp_path)) == (7000.0, 1590.0, "measured")
    for junk in ("not json", "[1, 2]", json.dumps({"hbm_gbs": "fast", "bf16_tflops": -1})):
        f.write_text(junk)
        assert bench.peaks(str(tmp_path)) == (6650.0, 1590.0, "fallback")


def test_prompt_step_flops_are_those_of_the_products_attention_and_head():
    cfg = type("C", (), dict(n_embd=768, inner_dim=3072, n_layer=12, n_head=12, vocab_size=50257))
    flops = bench.prefill_flops(cfg, [1024, 1024], 2)
    gemm = 2.0 * 2048 * (4 * 768 * 768 + 2 * 768 * 3072) * 12
    attn = 2 * 4.0 * 64 * (1024 * 1025 / 2) * 12 * 12
    head = 2.0 * 2 * 768 * 50257
    assert flops == gemm + attn + head
    assert 0.38e12 < flops < 0.40e12          # 0.348 + 0.039 TFLOP of GPT-2 small at 2 x 1,024 tokens


def test_more_than_one_gpu_is_one_line_and_status_2():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "4"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_the_reference_arm_prints_one_line_a_measurement_or_why_there_is_none():
    """One layer, one sequence, a few tokens: seconds on the host cores where the reference's sources and a
    compiler are at hand; elsewhere the line says what is missing."""
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "4",
                        "--warmup", "3", "--layers", "1", "--batch", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and len(r.stdout.strip().splitlines()) == 1
    line = json.loads(r.stdout)
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert line["unavailable"] and "\n" not in line["unavailable"]
    else:
        assert line["value"] > 0 and line["e2e"]["value"] > 0 and line["prefill"]["value"] > 0
        assert line["config"]["same_config"] is False and line["config"]["n_layer"] == 1
        assert line["steps"] == 4 and line["warmup"] == 3 and "contexts 515 to 519" in line["metric"]
