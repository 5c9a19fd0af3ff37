"""The reference arm: kimxinw/kvcache itself, unmodified, built and driven as its own README drives it.

The reference is no Python package (no setup.py or pyproject.toml): it is a CMake project of
CUDA executables.  What CMakeLists.txt:58-78 builds for generation are three programs out of
three translation units plus cuBLAS:

    qwen_infer        apps/qwen_infer.cu + src/qwen_kernels.cu, -DCUDAG   (CUDA-graph decode)
    qwen_infer_eager  the same two files without the definition
    qwen_serve        apps/qwen_serve.cu + src/qwen_kernels.cu            (continuous batching)

`build()` copies the reference's tree, byte for byte, into `baseline/_ref/src` and compiles these
three with nvcc for sm_100a (the one change against its CMake default of sm_86, which is a
command-line option there too: -DCMAKE_CUDA_ARCHITECTURES, CMakeLists.txt:8-11).  Nothing of
kvcache_b200 is on the path of a run: the programs read `weights.bin` and `manifest.tsv`
(tools/dump_weights.py:31-66, src/include/qwen_loader.h:27-59), token ids on standard input,
and print token ids (apps/qwen_infer.cu:60-71,234; apps/qwen_serve.cu:57-67,206-212).

`export_weights()` is tools/dump_weights.py for a model folder on disk instead of a checkpoint
from the hub: every tensor in float16, in one blob, `lm_head.weight` written even when the
head is tied (tools/dump_weights.py:24-26), one manifest line per tensor.

The model's sizes are compiled into the reference (apps/qwen_serve.cu:20-23): it runs the
Qwen2.5-0.5B shape and nothing else, 8 running requests and a pool of 512 pages of 16 tokens.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import shutil
import subprocess
import sys
import threading
import time
from typing import Dict, List, Optional, Sequence, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
HOME = os.path.join(HERE, "_ref")
SRC = os.path.join(HOME, "src")
BIN = os.path.join(HOME, "bin")
PROGRAMS = {
    "qwen_infer": (["apps/qwen_infer.cu", "src/qwen_kernels.cu"], ["-DCUDAG"]),
    "qwen_infer_eager": (["apps/qwen_infer.cu", "src/qwen_kernels.cu"], []),
    "qwen_serve": (["apps/qwen_serve.cu", "src/qwen_kernels.cu"], []),
}
COPIED = ("apps", "src", "tools", "ref", "tests", "CMakeLists.txt", "README.md")

# Sizes the reference has compiled in (apps/qwen_serve.cu:20-23).
REFERENCE_SHAPE = {"hidden_size": 896, "num_hidden_layers": 24, "num_attention_heads": 14, "num_key_value_heads": 2,
                   "intermediate_size": 4864, "vocab_size": 151936, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0}
SERVE_MAX_BATCH, SERVE_POOL_PAGES, SERVE_PAGE = 8, 512, 16
SERVE_EOS = (151645, 151643)


class ReferenceUnavailable(RuntimeError):
    """The reference cannot be built or run here; the message is one line."""


def reference_source() -> Optional[str]:
    """The reference's own tree: $KVCACHE_B200_REFERENCE, or a folder `reference` beside this repository."""
    for candidate in (os.environ.get("KVCACHE_B200_REFERENCE"), os.path.join(REPO, "..", "reference")):
        if candidate and os.path.isfile(os.path.join(candidate, "apps", "qwen_serve.cu")):
            return os.path.abspath(candidate)
    return None


def _nvcc() -> str:
    for candidate in (os.environ.get("KVCACHE_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise ReferenceUnavailable("nvcc not found: the reference's programs cannot be compiled")


def _tree_digest(root: str) -> str:
    h = hashlib.sha256()
    for folder, _, files in sorted(os.walk(root)):
        for name in sorted(files):
            if name.endswith((".cu", ".h", ".py", ".txt")):
                path = os.path.join(folder, name)
                h.update(os.path.relpath(path, root).encode())
                with open(path, "rb") as fh:
                    h.update(fh.read())
    return h.hexdigest()[:16]


def build(force: bool = False, log=None) -> Dict[str, str]:
    """Copies the reference (if its tree is at hand) and compiles its three generation programs.
    Returns {program: path}.  Raises ReferenceUnavailable with the reason otherwise."""
    log = log or (lambda m: print(f"[reference] {m}", file=sys.stderr, flush=True))
    source = reference_source()
    if source is not None and (force or not os.path.isdir(SRC) or _tree_digest(source) != _tree_digest(SRC)):
        if os.path.isdir(SRC):
            shutil.rmtree(SRC)
        os.makedirs(SRC)
        for name in COPIED:
            path = os.path.join(source, name)
            if os.path.isdir(path):
                shutil.copytree(path, os.path.join(SRC, name))
            elif os.path.isfile(path):
                shutil.copy2(path, os.path.join(SRC, name))
        for folder, _, files in os.walk(SRC):                     # the copy keeps the source's modes: make it removable
            os.chmod(folder, 0o755)
            for name in files:
                os.chmod(os.path.join(folder, name), 0o644)
        log(f"copied the reference's tree ({_tree_digest(SRC)}) into {os.path.relpath(SRC, REPO)}")
    if not os.path.isfile(os.path.join(SRC, "apps", "qwen_serve.cu")):
        raise ReferenceUnavailable("the reference's sources are neither under baseline/_ref/src nor beside the repository")
    os.makedirs(BIN, exist_ok=True)
    digest = _tree_digest(SRC)
    stamp_path = os.path.join(BIN, "BUILD.json")
    stamp = {}
    if os.path.isfile(stamp_path):
        with open(stamp_path) as fh:
            stamp = json.load(fh)
    out = {}
    commands = {}
    for program, (sources, defines) in PROGRAMS.items():
        target = os.path.join(BIN, program)
        out[program] = target
        cmd = [_nvcc(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", *defines,
               "-I", os.path.join(SRC, "src", "include"), "-o", target, *[os.path.join(SRC, s) for s in sources], "-lcublas"]
        commands[program] = " ".join(os.path.relpath(c, REPO) if os.path.isabs(c) and c.startswith(REPO) else c for c in cmd)
        if not force and os.path.isfile(target) and stamp.get("sources") == digest:
            continue
        log(f"compiling {program} for sm_100a ...")
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise ReferenceUnavailable(f"nvcc failed on the reference's {program}: {proc.stderr.strip().splitlines()[-1] if proc.stderr.strip() else proc.returncode}")
    with open(stamp_path, "w") as fh:
        json.dump({"sources": digest, "commands": commands}, fh, indent=1)
    return out


def programs() -> Dict[str, str]:
    """Paths of the built programs; builds them if they are missing."""
    found = {p: os.path.join(BIN, p) for p in PROGRAMS}
    if all(os.path.isfile(path) and os.access(path, os.X_OK) for path in found.values()):
        return found
    return build()


# ---- weights in the reference's format -----------------------------------------------------------

def export_weights(model_folder: str, out_dir: str) -> str:
    """Writes `weights.bin` and `manifest.tsv` for the tensors of `model_folder/model.safetensors`:
    float16, row-major, one after the other; manifest lines `name<TAB>offset<TAB>nbytes<TAB>shape_csv`
    (tools/dump_weights.py:31-66).  A tied head is stored a second time as `lm_head.weight`
    (tools/dump_weights.py:24-26).  The folder's config.json must have the sizes the reference has compiled in."""
    import torch
    from safetensors import safe_open
    with open(os.path.join(model_folder, "config.json")) as fh:
        config = json.load(fh)
    for key, value in REFERENCE_SHAPE.items():
        if config.get(key) != value:
            raise ReferenceUnavailable(f"the reference has {key} = {value} compiled in; the model folder has {config.get(key)}")
    os.makedirs(out_dir, exist_ok=True)
    offset = 0
    lines = []
    with safe_open(os.path.join(model_folder, "model.safetensors"), framework="pt", device="cpu") as f, \
            open(os.path.join(out_dir, "weights.bin"), "wb") as blob:
        names = list(f.keys())

        def put(name: str, tensor) -> None:
            nonlocal offset
            data = tensor.contiguous().to(torch.float16).numpy().tobytes()
            blob.write(data)
            lines.append(f"{name}\t{offset}\t{len(data)}\t{','.join(str(d) for d in tensor.shape)}\n")
            offset += len(data)

        for name in names:
            put(name, f.get_tensor(name))
        if "lm_head.weight" not in names:
            put("lm_head.weight", f.get_tensor("model.embed_tokens.weight"))
    with open(os.path.join(out_dir, "manifest.tsv"), "w") as fh:
        fh.writelines(lines)
    return out_dir


# ---- running the programs --------------------------------------------------------------------------

def _id_lines(text: str) -> List[List[int]]:
    out = []
    for line in text.splitlines():
        parts = line.split()
        if parts and all(p.lstrip("-").isdigit() for p in parts):
            out.append([int(p) for p in parts])
    return out


_BENCH = re.compile(r"\[bench\] (\w+) steps=(\d+) median=([\d.]+) us/tok mean=([\d.]+) us/tok ([\d.]+) tok/s")


def run_infer(weights_dir: str, prompt: Sequence[int], max_new: int, graph: bool = True, timeout: float = 900.0):
    """One sequence through `qwen_infer` (CUDA-graph decode) or `qwen_infer_eager`.  Returns (generated ids,
    {"steps", "median_us", "mean_us"} from its own `[bench]` line: wall clock per decoded token, copies and
    synchronisation included, the first min(16, max_new / 4) steps left out - apps/qwen_infer.cu:30-38,194-209)."""
    program = programs()["qwen_infer" if graph else "qwen_infer_eager"]
    proc = subprocess.run([program, weights_dir, str(max_new)], input=" ".join(str(t) for t in prompt) + "\n",
                          capture_output=True, text=True, timeout=timeout)
    if proc.returncode != 0:
        raise ReferenceUnavailable(f"{os.path.basename(program)} exited with {proc.returncode}: {proc.stderr.strip()[-200:]}")
    ids = _id_lines(proc.stdout)
    if len(ids) != 1:
        raise ReferenceUnavailable(f"{os.path.basename(program)} printed {len(ids)} lines of ids: {proc.stderr.strip()[-200:]}")
    match = _BENCH.search(proc.stderr)
    bench = None if match is None else {"steps": int(match.group(2)), "median_us": float(match.group(3)),
                                         "mean_us": float(match.group(4))}
    return ids[0], bench


def run_serve(weights_dir: str, requests: Sequence[Tuple[int, Sequence[int]]], timeout: float = 1800.0):
    """Requests `(max_new, prompt ids)` through `qwen_serve` in its stdin protocol (apps/qwen_serve.cu:57-67).
    Returns (generated ids per request, seconds between its two lines on standard error - "[serve] N requests"
    after the weights are loaded and "[serve] done." after the last step - and its decode step count)."""
    program = programs()["qwen_serve"]
    text = f"{len(requests)}\n" + "".join(f"{n} " + " ".join(str(t) for t in p) + "\n" for n, p in requests)
    proc = subprocess.Popen([program, weights_dir], stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    stamps: Dict[str, float] = {}
    err_lines: List[str] = []

    def read_err() -> None:
        for line in proc.stderr:
            now = time.perf_counter()
            err_lines.append(line)
            if "requests, max_batch" in line:
                stamps["start"] = now
            elif "[serve] done." in line:
                stamps["done"] = now

    out_chunks: List[str] = []
    readers = [threading.Thread(target=read_err, daemon=True),
               threading.Thread(target=lambda: out_chunks.append(proc.stdout.read()), daemon=True)]
    for r in readers:
        r.start()
    proc.stdin.write(text)
    proc.stdin.close()
    try:
        code = proc.wait(timeout=timeout)
    except subprocess.TimeoutExpired:
        proc.kill()
        raise ReferenceUnavailable(f"qwen_serve did not finish within {timeout:.0f} s") from None
    for r in readers:
        r.join()
    if code != 0 or "start" not in stamps or "done" not in stamps:
        raise ReferenceUnavailable(f"qwen_serve exited with {code}: {''.join(err_lines).strip()[-200:]}")
    ids = _id_lines("".join(out_chunks))
    if len(ids) != len(requests):
        raise ReferenceUnavailable(f"qwen_serve printed {len(ids)} lines of ids for {len(requests)} requests")
    match = re.search(r"decode_steps=(\d+)", "".join(err_lines))
    return ids, stamps["done"] - stamps["start"], int(match.group(1)) if match else None


if __name__ == "__main__":
    for name, path in build(force="--force" in sys.argv).items():
        print(f"built {os.path.relpath(path, REPO)}")
