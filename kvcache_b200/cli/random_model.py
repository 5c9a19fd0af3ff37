"""Writes a model folder with seeded random weights from a config.json:
    python -m kvcache_b200.cli.random_model --config config.json --out DIR --seed 0 [--dtype bfloat16|float32]
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="random_model")
    parser.add_argument("--config", required=True, help="a config.json of a registered architecture")
    parser.add_argument("--out", required=True)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    args = parser.parse_args(argv)
    import torch
    from .. import models  # noqa: F401
    from ..config.registry import config_from_dict
    from ..weights.random_init import write_random_model
    with open(args.config, "r", encoding="utf-8") as fh:
        config = config_from_dict(json.load(fh), args.config)
    write_random_model(args.out, config, args.seed, torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    print(args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
