"""What one of an SM's four schedulers can issue of the instructions of a softmax tile: ex2 with and
without independent fma beside it, the whole loop of a 64-score row, the packing into bfloat16 pairs,
three-input maxima; one and two warps per scheduler. Prints cycles per round.

    python -m research_2_b200.profiling.sfu_probe
"""

from __future__ import annotations

import ctypes as C

from ..csrc.build import kernel_library

ROWS = [
    "16 ex2, one warp per scheduler",
    "16 ex2 + 48 fma, one warp",
    "16 ex2 + 96 fma, one warp",
    "16 ex2 + 128 fma, one warp",
    "16 ex2, two warps per scheduler",
    "16 ex2 + 96 fma, two warps",
    "a 64-score row (scale, 64 ex2, sums, 32 packs), one warp",
    "a 64-score row, two warps",
    "32 packs (+ 32 adds), one warp",
    "32 packs (+ 32 adds), two warps",
    "32 three-input maxima, one warp",
    "32 three-input maxima, two warps",
]


def main() -> int:
    lib = kernel_library("sfu_probe")
    out = (C.c_double * 16)()
    n = lib.r2_sfu_probe(out, 16)
    if n < 0:
        print("the probe failed")
        return 1
    for name, value in zip(ROWS, list(out)[:n]):
        print(f"{value:8.1f} cycles a round  {name}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
