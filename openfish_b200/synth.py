"""Seeded synthetic CRF scores that stand in for a basecaller's output.

score[t][n][c] = 5*tanh(1.5*z), z ~ N(0,1), plus +4 on one planted transition per timestep
and chunk, rounded once to fp16.  The planted transition follows the score layout the
reference documents (src/beam_search.c:211-231): stepping from k-mer p to
q = ((p << 2) & (ns-1)) | b uses column 4*q + (p >> 2*(state_len-1)).

Every element comes from a counter-based generator keyed on (seed, GLOBAL chunk index, t, c):
a 64-bit mix of the key gives two 32-bit uniforms, Box-Muller turns them into z.  A chunk's
scores therefore do not depend on the batch it sits in, on its position in that batch or on
the GPU that generates it: the shard [first_chunk, first_chunk + N) of a larger job is exactly
that slice of the job's tensor.  The planted path of a chunk is keyed on (seed + 1, global
chunk index) in the same way.

`make_scores` is the host (numpy) generator used for small parity cases; `make_scores_device`
builds benchmark-sized tensors directly in GPU memory with torch.  The two use the same keys
and the same formulas; their values agree except where the host's and the device's
transcendental functions differ in the last bit before the rounding to fp16.
"""
import numpy as np

_M64 = (1 << 64) - 1
_C1, _C2, _GOLD = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB, 0x9E3779B97F4A7C15
_T_SPAN, _C_SPAN = 1 << 20, 1 << 16  # key = (chunk * _T_SPAN + t) * _C_SPAN + c: T < 2^20, C < 2^16


def _planted_path(T, state_len, seed, chunk, p_step):
    """Columns [T] of the planted transitions of one chunk (by global index), -1 where it stays."""
    rng = np.random.default_rng([seed + 1, chunk])
    ns = 4 ** state_len
    state = int(rng.integers(0, ns))
    bases = rng.integers(0, 4, size=T)
    steps = rng.random(T) < p_step
    cols = np.full(T, -1, dtype=np.int64)
    for t in range(T):
        if steps[t]:
            new = ((state << 2) & (ns - 1)) | int(bases[t])
            cols[t] = new * 4 + (state >> (2 * (state_len - 1)))
            state = new
    return cols


def planted_columns(T, N, state_len, seed, p_step=1.0, first_chunk=0):
    """Column index [T][N] of the planted transition, or -1 where the path stays."""
    return np.stack([_planted_path(T, state_len, seed, first_chunk + n, p_step) for n in range(N)], axis=1)


def _seed_word(seed):
    return ((seed & _M64) * _GOLD + 0x632BE59BD9B4E019) & _M64


def make_scores(T, N, state_len, seed, C=None, p_step=1.0, bump=4.0, first_chunk=0):
    """float16 scores [T][N][C] (C defaults to the reference-valid 4*4^state_len) of the chunks
    first_chunk .. first_chunk + N - 1."""
    ns = 4 ** state_len
    C = C or 4 * ns
    assert T < _T_SPAN and C < _C_SPAN
    u64 = np.uint64
    t = np.arange(T, dtype=u64)[:, None, None]
    n = (np.arange(N, dtype=u64) + u64(first_chunk))[None, :, None]
    c = np.arange(C, dtype=u64)[None, None, :]
    with np.errstate(over="ignore"):
        x = (n * u64(_T_SPAN) + t) * u64(_C_SPAN) + c + u64(_seed_word(seed))
        x = (x ^ (x >> u64(30))) * u64(_C1)
        x = (x ^ (x >> u64(27))) * u64(_C2)
        x = x ^ (x >> u64(31))
    u1 = ((x >> u64(32)).astype(np.float32) + np.float32(0.5)) * np.float32(2.0 ** -32)
    u2 = ((x & u64(0xFFFFFFFF)).astype(np.float32) + np.float32(0.5)) * np.float32(2.0 ** -32)
    z = np.sqrt(np.float32(-2.0) * np.log(u1)) * np.cos(np.float32(2.0 * np.pi) * u2)
    s = np.float32(5.0) * np.tanh(np.float32(1.5) * z.astype(np.float32))
    cols = planted_columns(T, N, state_len, seed, p_step, first_chunk)
    tt, nn = np.nonzero(cols >= 0)
    s[tt, nn, cols[tt, nn]] += np.float32(bump)
    return s.astype(np.float16)


def make_scores_device(T, N, state_len, seed, device, C=None, p_step=1.0, bump=4.0, t_block=32, first_chunk=0):
    """Same generator in GPU memory, block of timesteps by block; returns a torch fp16 tensor
    [T][N][C] holding the chunks first_chunk .. first_chunk + N - 1."""
    import torch
    ns = 4 ** state_len
    C = C or 4 * ns
    assert T < _T_SPAN and C < _C_SPAN

    def signed(v):  # a 64-bit pattern as the int64 torch computes with (multiplication wraps)
        return v - (1 << 64) if v >= (1 << 63) else v

    def lsr(v, k):  # logical shift right of an int64 tensor
        return (v >> k) & ((1 << (64 - k)) - 1)

    out = torch.empty((T, N, C), dtype=torch.float16, device=device)
    cols = torch.from_numpy(planted_columns(T, N, state_len, seed, p_step, first_chunk)).to(device)
    n_key = (torch.arange(N, device=device, dtype=torch.int64) + first_chunk)[None, :, None] * _T_SPAN
    c_key = torch.arange(C, device=device, dtype=torch.int64)[None, None, :]
    n_idx = torch.arange(N, device=device)
    for t0 in range(0, T, t_block):
        t1 = min(T, t0 + t_block)
        t_key = torch.arange(t0, t1, device=device, dtype=torch.int64)[:, None, None]
        x = (n_key + t_key) * _C_SPAN + c_key + signed(_seed_word(seed))
        x = (x ^ lsr(x, 30)) * signed(_C1)
        x = (x ^ lsr(x, 27)) * signed(_C2)
        x = x ^ lsr(x, 31)
        u1 = (lsr(x, 32).to(torch.float32) + 0.5) * (2.0 ** -32)
        u2 = ((x & 0xFFFFFFFF).to(torch.float32) + 0.5) * (2.0 ** -32)
        del x
        z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos((2.0 * np.pi) * u2)
        del u1, u2
        z = 5.0 * torch.tanh(1.5 * z)
        cb = cols[t0:t1]
        keep = cb >= 0
        tt = torch.arange(t1 - t0, device=device)[:, None].expand_as(cb)[keep]
        z[tt, n_idx[None, :].expand_as(cb)[keep], cb[keep]] += bump
        out[t0:t1] = z.to(torch.float16)
    return out
