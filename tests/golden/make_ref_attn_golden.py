"""Makes tests/golden/ref_attn.json and ref_attn_out.f32 by running the reference's own numpy attention,
ref/ref_attn.py of kimxinw/kvcache - the one piece of the reference's arithmetic that runs without a GPU (its model
code is CUDA with one checkpoint's sizes compiled in).  The script draws q [8, 64], K and V [8, 128, 64] from
numpy's default_rng(0) and writes softmax(q K^T / sqrt(64)) V per head; tests/test_plain.py draws the same inputs
again, checks them against the digests recorded here, and compares the plain implementation's attention (and, on
the GPU, the kernels) with the reference's output.

    python tests/golden/make_ref_attn_golden.py --reference <checkout of kimxinw/kvcache>
"""
import argparse
import hashlib
import json
import os
import runpy
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of kimxinw/kvcache (read only)")
    args = parser.parse_args()
    script = os.path.join(os.path.abspath(args.reference), "ref", "ref_attn.py")
    before = os.getcwd()
    with tempfile.TemporaryDirectory() as tmp:
        os.chdir(tmp)                                   # the script writes data/*.bin under the current folder
        try:
            runpy.run_path(script, run_name="__main__")
        finally:
            os.chdir(before)
        digests = {}
        for name in ("q", "K", "V"):
            with open(os.path.join(tmp, "data", f"{name}.bin"), "rb") as fh:
                digests[name] = hashlib.sha256(fh.read()).hexdigest()
        out = np.fromfile(os.path.join(tmp, "data", "out_ref.bin"), dtype=np.float32)
    assert out.size == 8 * 64
    out.astype("<f4").tofile(os.path.join(HERE, "ref_attn_out.f32"))
    with open(os.path.join(HERE, "ref_attn.json"), "w", encoding="utf-8") as fh:
        json.dump({"source": "ref/ref_attn.py", "heads": 8, "keys": 128, "head_dim": 64, "seed": 0,
                   "inputs_sha256": digests, "output": "ref_attn_out.f32 (float32 little-endian, [heads, head_dim])"},
                  fh, indent=1)
        fh.write("\n")
    print("wrote", os.path.join(HERE, "ref_attn_out.f32"), "and ref_attn.json")


if __name__ == "__main__":
    main()
