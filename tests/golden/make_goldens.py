#!/usr/bin/env python3
"""Makes the golden files of tests/golden/ from nireo/chibillm's own code.

    CHIBILLM_REFERENCE_DIR=/path/to/chibillm python tests/golden/make_goldens.py

Builds ``anchor_driver`` from the reference's unmodified .cc files (taken from
that directory, never copied here), ``metal_cpu_shim.cc`` and
``anchor_driver.cc`` with g++ (C++23), writes the tiny model folders A and B
from their seeds, and runs the driver on them:

1. generation: the reference's scheduler, engine, batch builder, block
   manager, KV cache and layer code produce greedy tokens for every request
   under two scheduler settings (one generous, one so tight that prompts are
   cut into portions, requests wait for pages and pages are used again);
2. logits: each request's prompt plus what was generated runs alone as one
   batch, and again one token at a time; the logits of every position are kept.

What is kept under tests/golden/tiny_<name>/: ``golden.json`` (the requests,
the tokens, the step log, the sha256 of the weights file the goldens belong
to, and how far the reference's own ways of running agree with one another)
and one ``whole_<id>.f32`` per request ([positions, vocab] little-endian
float32).  Needs nlohmann/json.hpp (searched under the Python prefix, or
NLOHMANN_JSON_INCLUDE).  Which part of the chain is the reference's code and
which is restated is said at the top of metal_cpu_shim.cc.
"""
from __future__ import annotations

import glob
import hashlib
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import tiny_configs  # noqa: E402

REFERENCE_SOURCES = [
    "qwen/qwen_layer.cc", "qwen/qwen_weights.cc", "qwen/qwen_configs.cc", "qwen/qwen3_5_model_state.cc",
    "model_format/safetensors.cc", "model_format/weight_reader.cc", "tensor/functions.cc",
    "tensor/tensor_ops.cc", "tensor/attention.cc", "tensor/matrix.cc", "tensor/deltanet.cc",
    "metal/metal_kv_cache.cc", "block_manager.cc", "seq.cc", "scheduler.cc", "model_batch.cc",
    "model_runner.cc", "inference_engine.cc", "prefix_cache.cc",
]

# the workloads of the two tiny configurations: prompt lengths, new tokens, page size
WORKLOADS = {
    "A": {"seed": 0, "prompts": [5, 11, 17], "new_tokens": 8, "block_size": 4, "prompt_seed": 100,
          "generate": [
              {"name": "roomy", "max_sequences": 4, "max_batch_tokens": 128, "prefill_chunk_tokens": 64,
               "kv_block_count": 64},
              {"name": "tight", "max_sequences": 2, "max_batch_tokens": 7, "prefill_chunk_tokens": 3,
               "kv_block_count": 11}]},
    "B": {"seed": 1, "prompts": [1, 7, 23, 40], "new_tokens": 12, "block_size": 16, "prompt_seed": 101,
          "generate": [
              {"name": "roomy", "max_sequences": 4, "max_batch_tokens": 128, "prefill_chunk_tokens": 64,
               "kv_block_count": 32},
              {"name": "chunk8", "max_sequences": 3, "max_batch_tokens": 16, "prefill_chunk_tokens": 8,
               "kv_block_count": 7}]},
}


def find_json_include() -> str:
    env = os.environ.get("NLOHMANN_JSON_INCLUDE")
    if env:
        return env
    hits = glob.glob(os.path.join(sys.prefix, "**", "nlohmann", "json.hpp"), recursive=True)
    if not hits:
        raise SystemExit("nlohmann/json.hpp not found; set NLOHMANN_JSON_INCLUDE")
    return os.path.dirname(os.path.dirname(hits[0]))


def build_driver(reference_dir: str, build_dir: str) -> str:
    src = os.path.join(reference_dir, "src")
    flags = ["-std=c++23", "-O1", "-w", "-I", src, "-I", find_json_include()]
    jobs = []
    objects = []
    for path in [os.path.join(src, s) for s in REFERENCE_SOURCES] + [
            os.path.join(HERE, "metal_cpu_shim.cc"), os.path.join(HERE, "anchor_driver.cc")]:
        obj = os.path.join(build_dir, os.path.relpath(path, "/").replace("/", "_") + ".o")
        objects.append(obj)
        jobs.append(subprocess.Popen(["g++", *flags, "-c", path, "-o", obj]))
    for job in jobs:
        if job.wait() != 0:
            raise SystemExit("compiling the driver failed")
    exe = os.path.join(build_dir, "anchor_driver")
    subprocess.run(["g++", *objects, "-o", exe], check=True)
    return exe


def sha256_of(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def read_rows(path: str, vocab: int) -> np.ndarray:
    return np.fromfile(path, dtype="<f4").reshape(-1, vocab)


def make_one(name: str, exe: str, work: str) -> None:
    from chibillm_b200.weights import write_random_model

    w = WORKLOADS[name]
    cfg = tiny_configs.get(name)
    vocab = cfg["vocab_size"]
    model_dir = write_random_model(cfg, os.path.join(work, f"model_{name}"), seed=w["seed"],
                                   dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(w["prompt_seed"])
    prompts = {i + 1: torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(w["prompts"])}

    def run(job: dict, tag: str) -> str:
        out = os.path.join(work, f"out_{name}_{tag}")
        job_path = os.path.join(work, f"job_{name}_{tag}.json")
        with open(job_path, "w") as f:
            json.dump(job, f)
        subprocess.run([exe, model_dir, job_path, out], check=True)
        return out

    gens = [dict(g_, max_new_tokens=w["new_tokens"], ignore_eos=False) for g_ in w["generate"]]
    out1 = run({"block_size": w["block_size"],
                "requests": [{"id": i, "tokens": t} for i, t in prompts.items()], "generate": gens}, "gen")
    generated = json.load(open(os.path.join(out1, "generated.json")))
    first = generated[gens[0]["name"]]
    for g_ in gens[1:]:
        if generated[g_["name"]]["tokens"] != first["tokens"]:
            raise SystemExit(f"{name}: the reference's tokens differ between scheduler settings")

    # every position of prompt + generated (the last generated token is never fed)
    full = {i: prompts[i] + first["tokens"][str(i)][:-1] for i in prompts}
    out2 = run({"block_size": w["block_size"],
                "requests": [{"id": i, "tokens": t} for i, t in full.items()]}, "whole")

    dest = os.path.join(HERE, f"tiny_{name}")
    os.makedirs(dest, exist_ok=True)
    agreement = {"steps_vs_whole": 0.0, "sampled_rows_vs_whole": 0.0}
    for i, tokens in full.items():
        whole = read_rows(os.path.join(out2, f"whole_{i}.f32"), vocab)
        steps = read_rows(os.path.join(out2, f"steps_{i}.f32"), vocab)
        assert whole.shape == (len(tokens), vocab) == steps.shape
        scale = float(np.abs(whole).max())
        agreement["steps_vs_whole"] = max(agreement["steps_vs_whole"],
                                          float(np.abs(whole - steps).max()) / scale)
        n_prompt = len(prompts[i])
        for g_ in gens:
            rows = read_rows(os.path.join(out1, f"gen_{g_['name']}_{i}.f32"), vocab)
            want = whole[n_prompt - 1:n_prompt - 1 + rows.shape[0]]
            agreement["sampled_rows_vs_whole"] = max(agreement["sampled_rows_vs_whole"],
                                                     float(np.abs(rows - want).max()) / scale)
            greedy = [int(np.argmax(r)) for r in rows]
            assert greedy == first["tokens"][str(i)], "argmax of the logits is not the sampled token"
        whole.astype("<f4").tofile(os.path.join(dest, f"whole_{i}.f32"))
    if max(agreement.values()) > 2e-5:
        raise SystemExit(f"{name}: the reference's own ways of running disagree: {agreement}")
    golden = {
        "config": name, "weights_seed": w["seed"], "weights_dtype": "bfloat16",
        "weights_sha256": sha256_of(os.path.join(model_dir, "model.safetensors")),
        "block_size": w["block_size"], "new_tokens": w["new_tokens"],
        "prompts": {str(i): t for i, t in prompts.items()},
        "generate": {g_["name"]: dict(g_, tokens=generated[g_["name"]]["tokens"],
                                      reasons=generated[g_["name"]]["reasons"],
                                      steps=" ".join(f"{p}:{t}:{n}" for p, t, n in generated[g_["name"]]["steps"]))
                     for g_ in gens},
        "relative_disagreement_within_the_reference": agreement,
    }
    with open(os.path.join(dest, "golden.json"), "w") as f:
        f.write(json.dumps(golden, sort_keys=True).replace('}, "', '},\n "').replace('], "', '],\n "') + "\n")
    print(f"tiny {name}: {sum(len(t) for t in full.values())} positions, agreement {agreement}")


def main() -> None:
    reference_dir = os.environ.get("CHIBILLM_REFERENCE_DIR")
    if not reference_dir or not os.path.isdir(os.path.join(reference_dir, "src")):
        raise SystemExit("set CHIBILLM_REFERENCE_DIR to a checkout of nireo/chibillm")
    with tempfile.TemporaryDirectory() as work:
        exe = build_driver(reference_dir, work)
        for name in WORKLOADS:
            make_one(name, exe, work)


if __name__ == "__main__":
    main()
