"""The command line as a user runs it, ``python -m chibillm_b200``, on the GPU:
several prompts submitted together so that the scheduler mixes prompt portions
and decoded tokens, against the plain implementation; random weights from a
configuration file; the profiling mode."""
import json
import os
import subprocess
import sys

import pytest

import helpers
import plain_qwen3
import tiny_configs

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_module(args, cwd=ROOT):
    return subprocess.run([sys.executable, "-m", "chibillm_b200", *args], cwd=cwd, capture_output=True, text=True,
                          timeout=600)


def test_four_prompts_through_the_scheduler(tmp_path):
    folder = helpers.make_model_dir(tmp_path, "B", seed=1)
    config, weights = plain_qwen3.read_model_folder(folder)
    prompts = list(helpers.random_requests(384, [1, 7, 23, 40], seed=1).values())
    expected = [plain_qwen3.generate_greedy(config, weights, p, 12) for p in prompts]
    prompt_file = tmp_path / "prompts.txt"
    prompt_file.write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n")
    metrics = tmp_path / "m.jsonl"
    args = ["--context-length", "64", "--max-tokens", "12", "--max-seqs", "3", "--max-batch-tokens", "16",
            "--prefill-chunk", "8", "--dtype", "float32", "--ignore-eos", "--prompt-file", str(prompt_file),
            "--metrics-jsonl", str(metrics)]
    done = run_module(args + [folder])
    assert done.returncode == 0, done.stderr
    assert [[int(t) for t in line.split()] for line in done.stdout.splitlines()] == expected
    assert "sequences 3 | batch 16 tok | prompt portion 8 tok" in done.stderr
    records = [json.loads(line) for line in metrics.read_text().splitlines()]
    assert [r["prompt_tokens"] for r in records] == [1, 7, 23, 40]
    for r in records:
        assert r["output_tokens"] == 12 and r["stop_reason"] == "len_limit"
        assert r["processed_prompt_tokens"] == r["prompt_tokens"]
        assert r["decode_step"]["samples"] == 11 and r["inter_token"]["samples"] == 11
        assert 0 < r["decode_step"]["p50_seconds"] <= r["decode_step"]["p95_seconds"]
    assert records[3]["prefill_batches"] >= 3        # 40 tokens under a budget of 16 a step

    # the same model from its configuration and seed, bfloat16, one after the other
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny_configs.get("B")))
    again = run_module(args[:-4] + ["--prompt-file", str(prompt_file), "--random", str(cfg_path),
                                    "--weights-seed", "1"])
    assert again.returncode == 0, again.stderr
    assert again.stdout == done.stdout


def test_profile_mode_prints_a_table(tmp_path):
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny_configs.get("D128")))
    done = run_module(["--random", str(cfg_path), "--context-length", "256", "--max-tokens", "5", "--ignore-eos",
                       "--prompt-ids", ",".join(str(i) for i in range(1, 151)), "--profile-passes"])
    assert done.returncode == 0, done.stderr
    assert len(done.stdout.split()) == 5
    table = [l for l in done.stderr.splitlines() if l.startswith("[cuda-profile]")]
    passes = [l for l in done.stderr.splitlines() if l.startswith("[cuda-pass]")]
    assert len(passes) == 5 and "tokens=150" in passes[0] and "tokens=1 " in passes[1]
    assert table[-1].split()[1:4] == ["all", "instrumented", "work"]
    names = " ".join(table)
    for expected in ("gemm_bf16", "few rows", "many rows", "embed", "sample", "attention"):
        assert expected in names, f"{expected} is missing from the profile"
    shares = [float(l.split("share=")[1].rstrip("%")) for l in table[:-1]]
    assert abs(sum(shares) - 100.0) < 1.0 and shares == sorted(shares, reverse=True)

    # the same tokens without the profiling mode
    plain = run_module(["--random", str(cfg_path), "--context-length", "256", "--max-tokens", "5", "--ignore-eos",
                        "--prompt-ids", ",".join(str(i) for i in range(1, 151))])
    assert plain.returncode == 0 and plain.stdout.split() == done.stdout.split()
