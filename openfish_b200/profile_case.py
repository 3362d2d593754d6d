"""Runs a few decodes of one synthetic batch, printing the per-kernel device times: the small,
self-contained workload that profiler captures are taken on.

    python -m openfish_b200.profile_case <state_len> <T> <N> <repeats>
"""
import sys

import torch

import openfish_b200 as of
from openfish_b200 import synth


def main(state_len, T, N, repeats):
    scores = synth.make_scores_device(T, N, state_len, 0x0F16, "cuda")
    gb = of.gpubuf_init(T, N, state_len)
    res = [torch.empty((N, T), dtype=torch.uint8).pin_memory() for _ in range(3)]
    for _ in range(repeats):
        of.decode_into(scores, state_len, gb, *res)
        print(gb.last_decode_ms(), flush=True)
    gb.free()


if __name__ == "__main__":
    main(*[int(x) for x in sys.argv[1:5]])
