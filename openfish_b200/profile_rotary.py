"""Runs the rotary embedding a few times on the encoder's packed QKV shape, printing the device
time of each call: the small, self-contained workload that profiler captures are taken on.

    python -m openfish_b200.profile_rotary <batch> <repeats>
"""
import sys

import numpy as np
import torch

import openfish_b200 as of


def main(batch, repeats):
    S, H, D = 1666, 8, 64
    half = D // 2
    pos = np.arange(S)[:, None] * (10000.0 ** (-np.arange(half) / half))[None, :]
    sin = torch.from_numpy(np.sin(pos).astype(np.float32)).cuda()
    cos = torch.from_numpy(np.cos(pos).astype(np.float32)).cuda()
    xs = [torch.randn((batch, S, 3, H, D), device="cuda", dtype=torch.float16) for _ in range(4)]
    for i in range(repeats):
        of.rotary_emb_gpu(xs[i % 4], sin, cos, batch, S, 2 * H, D, half, S * 3 * H * D, 3 * H * D, D)
        print("rotary %.4f ms" % of.last_rotary_ms(), flush=True)


if __name__ == "__main__":
    main(int(sys.argv[1]), int(sys.argv[2]))
