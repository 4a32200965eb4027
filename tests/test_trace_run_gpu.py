"""``bin/trace_run`` as a user runs it: a subprocess fed JSON steps on standard input, logits read
back from ``<out>/<step>.f32``.  Same requests whole, tail decoded one by one, in changing
portions, and mixed with so few pages that they are used again; float32 and bfloat16."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import engine_cases as ec
from helpers import (TINY, collect, first_mismatch, make_model_dir, peak_tokens, trace_mixed, trace_portions,
                     trace_tail_decode, trace_whole)

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def replay(folder, dtype, steps, out_dir, vocab, max_tokens, extra=()):
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out",
           str(out_dir), "--max-tokens", str(max_tokens), *extra]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = out_dir / f"{s['step']}.f32"
        if wanted:
            arr = np.fromfile(path, dtype="<f4")
            assert arr.size == wanted * vocab
            outputs[s["step"]] = torch.from_numpy(arr.reshape(wanted, vocab).copy())
        else:
            assert not path.exists()
    return collect(steps, outputs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_four_ways(tmp_path, name, dtype):
    folder = make_model_dir(tmp_path, name)
    vocab = TINY[name]["config"].vocab_size
    requests = ec.requests_for(name, (100, 37, 61, 150, 45), seed=7)
    want = ec.plain_logits(folder, requests, dtype)
    for kind, steps in (("whole", trace_whole(requests)), ("tail", trace_tail_decode(requests)),
                        ("portions", trace_portions(requests, seed=3)), ("mixed", trace_mixed(requests, seed=4))):
        got = replay(folder, dtype, steps, tmp_path / f"out_{kind}", vocab, peak_tokens(steps, 64),
                     extra=("--page-size", str(TINY[name]["page_size"])))
        ec.check_against(got, want, dtype, f"trace_run {name} {dtype} {kind}")


def test_trace_run_steps_without_wanted_logits_and_default_page_size(tmp_path):
    folder = make_model_dir(tmp_path, "A")
    vocab = TINY["A"]["config"].vocab_size
    requests = ec.requests_for("A", (50, 20), seed=8)
    a, b = requests["r0"], requests["r1"]
    steps = [
        {"step": 0, "entries": [{"id": "r0", "tokens": a[:30], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "r1", "tokens": b[:2], "want": [1]}], "end": []},  # r0 sits out
        {"step": 2, "entries": [{"id": "r0", "tokens": a[30:], "want": [19]}, {"id": "r1", "tokens": b[2:], "want": [0, 17]}],
         "end": ["r0", "r1"]},
    ]
    got = replay(folder, "float32", steps, tmp_path / "out", vocab, 128)
    want = ec.plain_logits(folder, requests, "float32")
    assert sorted(got["r0"]) == [49] and sorted(got["r1"]) == [1, 2, 19]
    assert first_mismatch(got, want, ec.TOL_F32) is None
