"""What bench.py promises without a GPU: more than one GPU is refused with one
line and exit code 2; the reference arm prints its ``unavailable`` record and
exits 0; the byte and flop counts behind the roofline fractions are what a hand
count of the Qwen3-8B shapes gives."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          cwd=ROOT, timeout=120)


def test_more_than_one_gpu_is_refused():
    p = _run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_is_unavailable():
    p = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    record = json.loads(p.stdout.strip().splitlines()[-1])
    assert record["impl"] == "reference" and isinstance(record["unavailable"], str) and "\n" not in record["unavailable"]


def test_bytes_and_flops_of_the_qwen3_8b_shape():
    import bench
    c = dict(bench.QWEN3_8B)
    assert (c["num_hidden_layers"], c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"],
            c["head_dim"], c["intermediate_size"], c["vocab_size"]) == (36, 4096, 32, 8, 128, 12288, 151936)
    per_layer = 4096 * 6144 + 4096 * 4096 + 3 * 4096 * 12288            # q|k|v, o, gate, up, down
    assert bench.layer_weight_elements(c) == per_layer
    # a decode step of 8 requests holding 2,049 tokens each: all weights once, the cache of the requests
    ctx = [2049] * 8
    weights = 36 * (per_layer + 2 * 4096 + 2 * 128) + 4096 + 151936 * 4096 + 8 * 4096
    cache = 36 * 2 * 8 * 128 * sum(ctx)
    assert bench.decode_step_bytes(c, 36, ctx) == 2.0 * (weights + cache)
    assert abs(bench.decode_step_bytes(c, 36, ctx) / 1e9 - 17.55) < 0.05
    # a prompt of 2,048 tokens, one wanted row: products, causal attention (half of T x T), the output row
    flops = 2.0 * 2048 * 36 * per_layer + 36 * 2.0 * 32 * 128 * 2048.0 * 2048 + 2.0 * 4096 * 151936
    assert bench.prefill_flops(c, 36, 2048) == flops
    assert abs(flops / 1e12 - 29.7) < 0.1
