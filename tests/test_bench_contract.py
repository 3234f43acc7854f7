"""What bench.py promises without a GPU: more than one GPU is refused with one line and exit code 2, the
reference arm says in one JSON line why it cannot run, and the byte and flop counts behind the roofline
figures follow from the configuration."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line():
    r = run_bench("--gpus", "2")
    assert r.returncode == 2
    lines = [l for l in (r.stdout + r.stderr).splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    r = run_bench("--impl", "reference")
    assert r.returncode == 0
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_roofline_counts_follow_from_the_configuration():
    sys.path.insert(0, ROOT)
    import bench

    cfg = dict(bench.SIZES["medium"])
    D, I, V, L = cfg["n_embd"], cfg["n_inner"] or 4 * cfg["n_embd"], cfg["vocab_size"], cfg["n_layer"]
    weight_bytes, kv_per_token, lin_flops = bench.model_bytes_and_flops(cfg, L)
    matrices = L * (3 * D * D + D * D + 2 * D * I)
    assert kv_per_token == L * 2 * D * 2                      # keys and values of every layer, bfloat16
    assert lin_flops == 2 * matrices                          # one multiply-add per matrix element and token
    # every matrix and the tied table once in bfloat16, biases and norm vectors in float32
    vectors = L * (3 * D + D + I + D + 4 * D) + 2 * D
    assert weight_bytes == 2 * (matrices + V * D) + 4 * vectors
    assert set(bench.SIZES) == {"medium", "large", "xl"}
    for name, heads in (("medium", 16), ("large", 20), ("xl", 25)):
        assert bench.SIZES[name]["n_embd"] // bench.SIZES[name]["n_head"] == 64 and bench.SIZES[name]["n_head"] == heads
