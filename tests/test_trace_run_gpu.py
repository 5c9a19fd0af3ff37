"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read back from files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import replay_modes
from helpers import assert_close, random_tokens
from plain_qwen2 import logits_of, read_folder
from tiny_configs import PAGE_SIZE, make_model_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL = {"float32": 1e-4, "bfloat16": 3e-2}


PORTION_SIZES = [2, 17, 3, 31, 2, 16, 8, 22]


def _trace_lines(seqs, alone):
    """One trace with all four ways of cutting: `alone["w"]` whole in one step, `alone["o"]` with its last 32 tokens one
    by one, `alone["p"]` in portions of changing size - each alone and ended before the next - and then `seqs` mixed
    as MIXED_PLAN says, up to four live, with pages of ended requests taken again."""
    lines = []

    def add(entries, end=()):
        lines.append({"step": len(lines), "entries": entries, "end": list(end)})
    w, o, p = alone["w"], alone["o"], alone["p"]
    add([{"id": "w", "tokens": w, "want": list(range(len(w)))}], ["w"])
    head = len(o) - 32
    add([{"id": "o", "tokens": o[:head], "want": [head - 1]}])
    for i in range(head, len(o)):
        add([{"id": "o", "tokens": o[i:i + 1], "want": [0]}], ["o"] if i == len(o) - 1 else [])
    at = 0
    for size in PORTION_SIZES:
        piece = p[at:at + size]
        at += len(piece)
        add([{"id": "p", "tokens": piece, "want": list(range(len(piece)))}], ["p"] if at == len(p) else [])
    assert at == len(p)
    done = {k: 0 for k in seqs}
    for item in replay_modes.MIXED_PLAN:
        if isinstance(item, str):
            lines[-1]["end"].append(item.split()[1])
            continue
        entries = []
        for k, n in item:
            if n > 0:
                entries.append({"id": k, "tokens": seqs[k][done[k]:done[k] + n], "want": list(range(n))})
                done[k] += n
        add(entries)
    lines[-1]["end"] = [k for k in seqs if k not in ("a", "b", "c")]
    return lines


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_trace_run_all_ways_of_cutting(tmp_path, name, dtype):
    folder = make_model_folder(tmp_path, name, dtype=torch.bfloat16)
    config, weights = read_folder(folder)
    V = config["vocab_size"]
    seqs = {k: random_tokens(V, n, 30 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    alone = {"w": random_tokens(V, 75, 40), "o": random_tokens(V, 90, 41), "p": random_tokens(V, sum(PORTION_SIZES), 42)}
    lines = _trace_lines(seqs, alone)
    out_dir = os.path.join(str(tmp_path), "out")
    # The page size of the configuration (B: 8 tokens) and no more live requests than the plan needs.
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
         "--out", out_dir, "--max-tokens", str(replay_modes.mixed_pool_tokens()), "--page-size", str(PAGE_SIZE[name]),
         "--max-live", "4"],
        input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {l['step']}" for l in lines]
    got = {k: [] for k in list(seqs) + list(alone)}
    for l in lines:
        data = np.fromfile(os.path.join(out_dir, f"{l['step']}.f32"), dtype="<f4").reshape(-1, V)
        at = 0
        for e in l["entries"]:
            got[e["id"]].append(torch.from_numpy(data[at:at + len(e["want"])].copy()))
            at += len(e["want"])
        assert at == data.shape[0]
    for k, tokens in seqs.items():
        assert_close(torch.cat(got[k]), logits_of(config, weights, tokens), REL[dtype], k)
    assert_close(torch.cat(got["w"]), logits_of(config, weights, alone["w"]), REL[dtype], "whole")
    assert_close(torch.cat(got["o"]), logits_of(config, weights, alone["o"])[-33:], REL[dtype], "last 32 one by one")
    assert_close(torch.cat(got["p"]), logits_of(config, weights, alone["p"]), REL[dtype], "portions")
