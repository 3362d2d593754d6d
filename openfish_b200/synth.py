"""Seeded synthetic CRF scores that stand in for a basecaller's output.

score[t][n][c] = 5*tanh(1.5*z), z ~ N(0,1), plus +4 on one planted transition per timestep
and chunk, rounded once to fp16.  The planted transition follows the score layout the
reference documents (src/beam_search.c:211-231): stepping from k-mer p to
q = ((p << 2) & (ns-1)) | b uses column 4*q + (p >> 2*(state_len-1)).

`make_scores` is the host (numpy) generator used for small parity cases and fixtures;
`make_scores_device` builds benchmark-sized tensors directly in GPU memory with torch.
"""
import numpy as np


def planted_columns(T, N, state_len, seed, p_step=1.0):
    """Column index [T][N] of the planted transition, or -1 where the path stays."""
    rng = np.random.default_rng(seed + 1)
    ns = 4 ** state_len
    state = rng.integers(0, ns, size=N)
    cols = np.full((T, N), -1, dtype=np.int64)
    for t in range(T):
        b = rng.integers(0, 4, size=N)
        step = rng.random(N) < p_step
        new = ((state << 2) & (ns - 1)) | b
        col = new * 4 + (state >> (2 * (state_len - 1)))
        cols[t] = np.where(step, col, -1)
        state = np.where(step, new, state)
    return cols


def make_scores(T, N, state_len, seed, C=None, p_step=1.0, bump=4.0):
    """float16 scores [T][N][C] (C defaults to the reference-valid 4*4^state_len)."""
    ns = 4 ** state_len
    C = C or 4 * ns
    rng = np.random.default_rng(seed)
    x = 5.0 * np.tanh(1.5 * rng.standard_normal((T, N, C), dtype=np.float32))
    cols = planted_columns(T, N, state_len, seed, p_step)
    tt, nn = np.nonzero(cols >= 0)
    x[tt, nn, cols[tt, nn]] += bump
    return x.astype(np.float16)


def make_scores_device(T, N, state_len, seed, device, C=None, p_step=1.0, bump=4.0, t_block=64):
    """Same distribution, generated in GPU memory block by block; returns a torch fp16 tensor."""
    import torch
    ns = 4 ** state_len
    C = C or 4 * ns
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = torch.empty((T, N, C), dtype=torch.float16, device=device)
    cols = torch.from_numpy(planted_columns(T, N, state_len, seed, p_step)).to(device)
    n_idx = torch.arange(N, device=device)
    for t0 in range(0, T, t_block):
        t1 = min(T, t0 + t_block)
        z = torch.randn((t1 - t0, N, C), generator=gen, device=device, dtype=torch.float32)
        z = 5.0 * torch.tanh(1.5 * z)
        c = cols[t0:t1]
        keep = c >= 0
        tt = torch.arange(t1 - t0, device=device)[:, None].expand_as(c)[keep]
        z[tt, n_idx[None, :].expand_as(c)[keep], c[keep]] += bump
        out[t0:t1] = z.to(torch.float16)
    return out
