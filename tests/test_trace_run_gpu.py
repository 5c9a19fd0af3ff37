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
from tiny_configs import make_model_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL = {"float32": 1e-4, "bfloat16": 3e-2}


def _trace_lines(seqs):
    lines, done, step = [], {k: 0 for k in seqs}, 0
    pending_end = []
    for item in replay_modes.MIXED_PLAN:
        if isinstance(item, str):
            lines[-1]["end"].append(item.split()[1])
            continue
        entries = []
        for k, n in item:
            if n > 0:
                entries.append({"id": k, "tokens": seqs[k][done[k]:done[k] + n], "want": list(range(n))})
                done[k] += n
        lines.append({"step": step, "entries": entries, "end": []})
        step += 1
    lines[-1]["end"] = [k for k in seqs if k not in ("a", "b", "c")]
    return lines


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_trace_run_mixed(tmp_path, name, dtype):
    folder = make_model_folder(tmp_path, name, dtype=torch.bfloat16)
    config, weights = read_folder(folder)
    V = config["vocab_size"]
    seqs = {k: random_tokens(V, n, 30 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    lines = _trace_lines(seqs)
    out_dir = os.path.join(str(tmp_path), "out")
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
         "--out", out_dir, "--max-tokens", str(replay_modes.mixed_pool_tokens())],
        input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {l['step']}" for l in lines]
    got = {k: [] for k in seqs}
    for l in lines:
        data = np.fromfile(os.path.join(out_dir, f"{l['step']}.f32"), dtype="<f4").reshape(-1, V)
        at = 0
        for e in l["entries"]:
            got[e["id"]].append(torch.from_numpy(data[at:at + len(e["want"])].copy()))
            at += len(e["want"])
        assert at == data.shape[0]
    for k, tokens in seqs.items():
        assert_close(torch.cat(got[k]), logits_of(config, weights, tokens), REL[dtype], k)
