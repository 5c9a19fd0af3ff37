"""qwen_serve: several sequences through continuous batching, ids in, ids out.

In the manner of the reference's program (apps/qwen_serve.cu:7, :49-67, :205-212):
    qwen_serve [dir]      stdin: "NSEQ" then one line "max_new id0 id1 ..." per sequence
                          stdout: one line of generated ids per sequence, in input order
    stderr: "[serve] N requests, max_batch=.., pool=.. blocks" and "[serve] done. decode_steps=.. peak_batch=.."
What the reference fixes in code is an option here: --max-batch (MAXB = 8), --num-blocks
(NUM_BLOCKS = 512), --block-size (BLOCK = 16); end tokens come from config.json instead of the two
hard-coded ids (apps/qwen_serve.cu:21-23).  Requests decode greedily unless --temperature is given.
"""
from __future__ import annotations

import argparse
import sys


def parse_requests(text: str):
    lines = text.splitlines()
    if not lines:
        raise ValueError("expected 'NSEQ' on the first line")
    count = int(lines[0].split()[0])
    requests = []
    for line in lines[1:1 + count]:
        fields = [int(t) for t in line.split()]
        if len(fields) < 2:
            raise ValueError(f"a request line is 'max_new id0 id1 ...', got '{line}'")
        requests.append((fields[0], fields[1:]))
    if len(requests) != count:
        raise ValueError(f"{count} requests announced, {len(requests)} given")
    return requests


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="qwen_serve", description="continuous batching over token ids")
    parser.add_argument("dir", nargs="?", default="data/qwen05b")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--max-batch", type=int, default=8)
    parser.add_argument("--num-blocks", type=int, default=512)
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--max-tokens-per-step", type=int, default=2048)
    parser.add_argument("--chunk-size", type=int, default=2048)
    parser.add_argument("--admission", default="reserve", choices=["reserve", "optimistic"])
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--no-graph", dest="graph", action="store_false", default=True)
    parser.add_argument("--time-kernels", action="store_true",
                        help="CUDA events around every kernel; a table per class of kernel on stderr (implies --no-graph)")
    args = parser.parse_args(argv)

    if args.time_kernels:
        args.graph = False
    try:
        requests = parse_requests(sys.stdin.read())
    except ValueError as exc:
        print(f"[serve] bad input: {exc}", file=sys.stderr)
        return 1
    print(f"[serve] {len(requests)} requests, max_batch={args.max_batch}, pool={args.num_blocks} blocks", file=sys.stderr)

    from ..config.options import EngineOptions
    from ..engine.llm import LLM
    from ..engine.scheduler import RequestRejected
    from ..sampling.params import SamplingParams
    llm = LLM(args.dir, EngineOptions(dtype=args.dtype, page_size=args.block_size, num_pages=args.num_blocks,
                                      max_running=args.max_batch, max_tokens_per_step=args.max_tokens_per_step,
                                      chunk_size=args.chunk_size, admission=args.admission, use_graphs=args.graph,
                                      seed=args.seed))
    params = [SamplingParams(max_new_tokens=max_new, temperature=args.temperature, seed=args.seed + i,
                             ignore_eos=args.ignore_eos) for i, (max_new, _) in enumerate(requests)]
    if args.time_kernels:
        llm.core.kernels.start_timing()
    try:
        outputs = llm.generate([ids for _, ids in requests], params)
    except RequestRejected as exc:
        print(f"[serve] request refused: {exc}", file=sys.stderr)
        return 1
    if args.time_kernels:
        from ..kernels.timing import format_report
        print(format_report(llm.core.kernels.stop_timing(), max(llm.last_stats.steps, 1)), file=sys.stderr)
    stats = llm.last_stats
    print(f"[serve] done. decode_steps={stats.steps} peak_batch={stats.peak_running} "
          f"prefill_tokens={stats.prefill_tokens} generated={stats.generated} preemptions={stats.preemptions} "
          f"peak_blocks={stats.peak_pages} seconds={llm.last_seconds:.3f}", file=sys.stderr)
    # The fields of the reference's EngineStats (src/include/engine.h:33-45), as its demo prints them.
    print(f"[serve] stats iters={stats.steps} tokens={stats.generated} gpu_ms={stats.gpu_us / 1e3:.2f} "
          f"wall_ms={stats.wall_us / 1e3:.2f} slot_steps={stats.slot_steps} useful_steps={stats.useful_steps} "
          f"slot_util={stats.slot_utilisation:.3f} finished={stats.finished} avg_latency_ms={stats.avg_latency_us / 1e3:.2f} "
          f"p99_latency_ms={stats.p99_latency_us / 1e3:.2f}", file=sys.stderr)
    for out in outputs:
        print(" ".join(str(t) for t in out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
