"""qwen_infer: one sequence, prompt ids on standard input, generated ids on standard output.

In the manner of the reference's program (apps/qwen_infer.cu:59-71, :233-236):
    qwen_infer [dir] [max_new=32]      stdin: prompt ids      stdout: one line of generated ids
    stderr: "[infer] prompt_len=.. max_new=.." and "[bench] <tag> steps=.. median=.. us/tok mean=.. us/tok .. tok/s"
Like the reference it always generates `max_new` tokens (no end-token check) and times each
decoded token by wall clock, dropping the first min(16, max_new / 4) steps and reporting the
median (apps/qwen_infer.cu:30-38, :194-209).  The reference's compile-time switch between
eager and CUDA-graph decoding (-DCUDAG) is the option --graph / --no-graph here.
"""
from __future__ import annotations

import argparse
import sys
import time


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="qwen_infer", description="single-sequence greedy generation")
    parser.add_argument("dir", nargs="?", default="data/qwen05b", help="model folder (config.json, model.safetensors)")
    parser.add_argument("max_new", nargs="?", type=int, default=32)
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--block-size", type=int, default=16, help="tokens per cache page (reference: BLOCK = 16)")
    parser.add_argument("--graph", dest="graph", action="store_true", default=True)
    parser.add_argument("--no-graph", dest="graph", action="store_false")
    parser.add_argument("--time-kernels", action="store_true",
                        help="CUDA events around every kernel of the decode steps; a table per class of kernel on stderr (implies --no-graph)")
    args = parser.parse_args(argv)

    if args.time_kernels:
        args.graph = False
    prompt = [int(t) for t in sys.stdin.read().split()]
    if not prompt:
        print("no prompt ids on stdin", file=sys.stderr)
        return 1
    print(f"[infer] prompt_len={len(prompt)} max_new={args.max_new}", file=sys.stderr)

    from ..config.options import EngineOptions
    from ..engine.llm import LLM
    from ..sampling.params import SamplingParams
    total = len(prompt) + args.max_new + 4          # the reference's private pool: P + max_new + 4 (qwen_infer.cu:73-76)
    llm = LLM(args.dir, EngineOptions(dtype=args.dtype, page_size=args.block_size, max_cached_tokens=total + args.block_size,
                                      max_running=1, max_tokens_per_step=max(len(prompt), 1), chunk_size=max(len(prompt), 1),
                                      use_graphs=args.graph, seed=args.seed))
    params = SamplingParams(max_new_tokens=args.max_new, temperature=args.temperature, seed=args.seed, ignore_eos=True)
    request = llm.scheduler.add_request(prompt, params)
    times = []
    llm.pipelined = False                            # each step is timed with its tokens read, as the reference does
    while llm.has_work():
        start = time.perf_counter()
        llm.step()
        times.append((time.perf_counter() - start) * 1e6)
        if args.time_kernels and len(times) == 1:
            llm.core.kernels.start_timing()          # from the first decoded token on
    if args.time_kernels:
        from ..kernels.timing import format_report
        print(format_report(llm.core.kernels.stop_timing(), max(len(times) - 1, 1)), file=sys.stderr)
    llm.core.kernels.check_errors()
    print(" ".join(str(t) for t in request.output))
    decode = times[1:]                               # the first step is the prompt
    drop = min(16, args.max_new // 4)
    timed = sorted(decode[drop:])
    tag = "graph" if args.graph else "eager"
    if not timed:
        print(f"[bench] {tag}: no timed steps", file=sys.stderr)
    else:
        median, mean = timed[len(timed) // 2], sum(timed) / len(timed)
        print(f"[bench] {tag} steps={len(timed)} median={median:.1f} us/tok mean={mean:.1f} us/tok {1e6 / median:.1f} tok/s",
              file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
