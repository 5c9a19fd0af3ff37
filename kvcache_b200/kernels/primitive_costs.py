"""python -m kvcache_b200.kernels.primitive_costs

Prints what the building blocks of the warp-specialised kernels cost on this GPU, in clocks on an
otherwise idle SM: waits on mbarriers, shuffles and votes, the issue of tensor-core MMAs and
commits, a TMA page copy, a load from tensor memory.  The layout of the helper warps of
csrc/attention_tc.cu and csrc/attention_flash.cu follows from these numbers.
"""
from __future__ import annotations


def main() -> None:
    from .api import CudaKernels
    costs = CudaKernels("cuda:0").primitive_costs()
    for name, clocks in costs.items():
        print(f"{clocks:8.1f} clocks  {name}")


if __name__ == "__main__":
    main()
