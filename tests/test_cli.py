"""The command line's options (the reference's rules, src/cli_options.cc:28-101)
and the read-eval-print loop on a CPU stand-in for the kernels."""
import io
import json

import pytest

import helpers
import plain_qwen3
from chibillm_b200 import cli
from reference_ops import ReferenceKernels


def test_defaults_and_values():
    o = cli.parse_cli_options([])
    assert (o.context_length, o.max_tokens, o.stream, o.progress) == (32768, 8192, True, True)
    o = cli.parse_cli_options(["--context-length", "4096", "--max-tokens", "7", "--no-stream",
                               "--progress=off", "--metrics-jsonl", "m.jsonl", "models/x",
                               "--temperature", "0.7", "--seed", "3", "--dtype", "float32",
                               "--prompt-ids", "1,2,3", "--prompt-ids", "4 5", "--quantize", "none",
                               "--prompt-cache-mib", "0", "--ignore-eos"])
    assert (o.context_length, o.max_tokens, o.stream, o.progress) == (4096, 7, False, False)
    assert (o.metrics_jsonl, o.model_directory, o.temperature, o.seed, o.dtype) == \
           ("m.jsonl", "models/x", 0.7, 3, "float32")
    assert o.prompts == [[1, 2, 3], [4, 5]] and o.ignore_eos
    assert cli.parse_cli_options(["-h"]).help


@pytest.mark.parametrize("argv,message", [
    (["--context-length"], "missing value for --context-length"),
    (["--context-length", "100"], "invalid token limit for --context-length: 100"),   # no multiple of 16
    (["--context-length", "0"], "invalid token limit"),
    (["--max-tokens", "x"], "invalid token limit for --max-tokens: x"),
    (["--metrics-jsonl", "--no-stream"], "missing path for --metrics-jsonl"),
    (["--quantize", "q8"], "invalid quantization: q8"),
    (["--quantize", "q4"], "not built"),
    (["--serve"], "not built"),
    (["--kv-cache-tokens", "64"], "requires --serve"),
    (["--prompt-cache-mib", "128"], "not built"),
    (["--bogus"], "unexpected argument: --bogus"),
    (["a", "b"], "unexpected argument: b"),
    (["--temperature", "-1"], "invalid temperature"),
    (["--prompt-ids", "1,x"], "token ids must be integers"),
])
def test_errors(argv, message):
    with pytest.raises(cli.CliError) as e:
        cli.parse_cli_options(argv)
    assert message in str(e.value)


def test_main_prints_usage_on_error(capsys):
    assert cli.main(["--bogus"]) == 1
    err = capsys.readouterr().err
    assert "unexpected argument: --bogus" in err and "Usage:" in err
    assert cli.main(["--help"]) == 0
    assert "Usage:" in capsys.readouterr().out


def test_repl_on_cpu(tmp_path, monkeypatch):
    """Two turns with history, /reset, a bad line, /quit; replies equal the plain
    implementation's greedy tokens."""
    folder = helpers.make_model_dir(tmp_path, "A", seed=2)
    config, weights = plain_qwen3.read_model_folder(folder)
    import chibillm_b200.api as api
    real = api.LLM

    def cpu_llm(model_dir, **kw):
        kw.update(device="cpu", kernels=ReferenceKernels(), dtype="float32")
        return real(model_dir, **kw)

    monkeypatch.setattr(api, "LLM", cpu_llm)
    metrics = tmp_path / "m.jsonl"
    options = cli.parse_cli_options([folder, "--context-length", "128", "--max-tokens", "4", "--ignore-eos",
                                     "--no-stream", "--metrics-jsonl", str(metrics)])
    stdin = io.StringIO("5 6 7\n\nnot ids\n8,9\n/reset\n5 6 7\n/quit\n")
    out, err = io.StringIO(), io.StringIO()
    assert cli.run(options, stdin, out, err) == 0
    first = plain_qwen3.generate_greedy(config, weights, [5, 6, 7], 4)
    second = plain_qwen3.generate_greedy(config, weights, [5, 6, 7] + first + [8, 9], 4)
    replies = [l.replace("ids> ", "").strip() for l in out.getvalue().splitlines()]
    replies = [l for l in replies if l and l[0].isdigit()]
    assert replies == [" ".join(map(str, first)), " ".join(map(str, second)), " ".join(map(str, first))]
    assert "history cleared" in out.getvalue()
    assert "[limits] context 128 tok | max output 4 tok" in err.getvalue()
    assert "token ids must be integers" in err.getvalue()
    records = [json.loads(l) for l in metrics.read_text().splitlines()]
    assert [r["prompt_tokens"] for r in records] == [3, 9, 3]
    assert all(r["output_tokens"] == 4 and r["finish_reason"] == "len_limit" for r in records)


def test_missing_model_is_reported(tmp_path):
    err = io.StringIO()
    options = cli.parse_cli_options([str(tmp_path / "nowhere")])
    assert cli.run(options, io.StringIO(""), io.StringIO(), err) == 1
    assert "failed to load model from" in err.getvalue()


def test_scheduler_options_and_their_derivation(tmp_path):
    o = cli.parse_cli_options(["--max-seqs", "3", "--max-batch-tokens", "16", "--prefill-chunk", "8",
                               "--kv-block-size", "8", "--kv-blocks", "40", "--context-length", "264",
                               "--random", "cfg.json", "--weights-seed", "7", "--device", "cuda:1", "--profile"])
    assert (o.max_seqs, o.max_batch_tokens, o.prefill_chunk, o.kv_block_size, o.kv_blocks) == (3, 16, 8, 8, 40)
    assert (o.random_config, o.weights_seed, o.device, o.profile, o.profile_passes) == \
           ("cfg.json", 7, "cuda:1", True, False)
    # what is left open follows the number of sequences (one: the reference's conversation values)
    d = cli.parse_cli_options([]).derived()
    assert (d.max_seqs, d.max_batch_tokens, d.prefill_chunk) == (1, 512, 64)
    d = cli.parse_cli_options(["--max-seqs", "8"]).derived()
    assert (d.max_batch_tokens, d.prefill_chunk) == (4096, 1024)
    prompts = tmp_path / "p.txt"
    prompts.write_text("1 2 3\n\n# a comment\n4,5\n")
    assert cli.parse_cli_options(["--prompt-file", str(prompts), "--prompt-ids", "6"]).prompts == \
           [[1, 2, 3], [4, 5], [6]]
    for argv, message in ((["--max-seqs", "0"], "invalid count for --max-seqs"),
                          (["--kv-block-size", "12", "--context-length", "64"], "invalid token limit"),
                          (["--device", "cpu"], "invalid device"),
                          (["--random", "c.json", "folder"], "not both"),
                          (["--prompt-file", str(tmp_path / "none")], "failed to read prompt file")):
        with pytest.raises(cli.CliError) as e:
            cli.parse_cli_options(argv)
        assert message in str(e.value)


def test_several_prompts_run_together_on_cpu(tmp_path):
    """Four prompts submitted at once with room for three: portions of 8 beside
    decoded tokens, the fourth waits for a finish.  Greedy tokens equal the plain
    implementation's; with --random the folder is replaced by a configuration."""
    import tiny_configs
    folder = helpers.make_model_dir(tmp_path, "B", seed=1)
    config, weights = plain_qwen3.read_model_folder(folder)
    prompts = list(helpers.random_requests(384, [1, 7, 23, 40], seed=1).values())
    expected = [plain_qwen3.generate_greedy(config, weights, p, 6) for p in prompts]
    argv = ["--context-length", "64", "--max-tokens", "6", "--max-seqs", "3", "--max-batch-tokens", "16",
            "--prefill-chunk", "8", "--dtype", "float32", "--ignore-eos", "--no-stream"]
    for p in prompts:
        argv += ["--prompt-ids", ",".join(map(str, p))]
    out, err = io.StringIO(), io.StringIO()
    assert cli.run(cli.parse_cli_options(argv + [folder]), io.StringIO(""), out, err,
                   kernels=ReferenceKernels(), device="cpu") == 0, err.getvalue()
    assert [[int(t) for t in line.split()] for line in out.getvalue().splitlines()] == expected
    assert "sequences 3 | batch 16 tok | prompt portion 8 tok | pages 12 x 16 tok" in err.getvalue()
    assert err.getvalue().count("[stop] len_limit") == 4

    # the same weights from a configuration file and a seed
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny_configs.get("B")))
    out2 = io.StringIO()
    assert cli.run(cli.parse_cli_options(argv + ["--random", str(cfg_path), "--weights-seed", "1"]),
                   io.StringIO(""), out2, io.StringIO(), kernels=ReferenceKernels(), device="cpu") == 0
    assert out2.getvalue() == out.getvalue()
