"""Generates the committed golden fixtures from the UNMODIFIED reference.

Run where the reference checkout is present (its location is taken from the environment variable
OPENFISH_REF, else the oracle Makefile's default) and the reference library has been built
(make -C oracle ref):

    python tests/golden/make_golden.py

Outputs (all under tests/golden/):
  ref_fast_chunk.npz   the reference's own golden vector test/data/{scores,moves,sequence,
                       qstring}.blob (the case test/test.sh:26-40 checks; decoded with the
                       fast-model options q_scale=0.97, q_shift=-1.8 of src/main.c:256-258).
                       The fp32 scores are exactly fp16 representable and stored as fp16.
  synth_<name>.npz     seeded synthetic fp16 scores with the reference CPU decoder's moves,
                       sequence, qstring (openfish_decode_cpu), its bwd / fwd+bwd / post
                       tensors (src/decode_cpu.c:13-147) and the per-timestep outputs of its
                       beam_search_cpu / generate_sequence_cpu (states, qual, base_probs,
                       total_probs; src/beam_search.c:441-496, 49-99).  Cases whose options
                       carry a temperature other than 1 were decoded with that value as
                       beam_search_cpu's score_scale argument (src/beam_search.c:129,233), the
                       one place the reference has for it (its own decoder passes 1.0f).
  rotary_small.npz     fp16 activations, sin/cos tables and openfish_rotary_emb_cpu's fp32 result.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from openfish_b200 import synth  # noqa: E402

REF = os.environ.get("OPENFISH_REF", "/root/reference")
OUT = os.path.dirname(os.path.abspath(__file__))

# name, state_len, T, N, seed, C, p_step, options
CASES = [
    ("fast", 3, 200, 4, 101, None, 1.0, {}),
    ("hac", 4, 96, 2, 102, None, 1.0, {}),
    ("sup", 5, 48, 1, 103, None, 1.0, {}),
    ("fast_c320", 3, 64, 3, 104, 320, 1.0, {}),
    ("fast_stays", 3, 200, 2, 105, None, 0.3, dict(q_scale=0.97, q_shift=-1.8)),
    ("hac_cut10", 4, 64, 2, 106, None, 0.6, dict(beam_cut=10.0)),
    ("fast_temp07", 3, 200, 3, 107, None, 0.8, dict(temperature=0.7)),
    ("hac_temp16", 4, 96, 2, 108, None, 1.0, dict(temperature=1.6, q_scale=0.95, q_shift=-0.2)),
]


def main():
    d = os.path.join(REF, "test", "data")
    sc32 = np.fromfile(os.path.join(d, "scores.blob"), np.float32).reshape(1666, 1, 256)
    sc16 = sc32.astype(np.float16)
    assert (sc16.astype(np.float32) == sc32).all(), "golden scores are not fp16-exact"
    np.savez_compressed(os.path.join(OUT, "ref_fast_chunk.npz"), scores=sc16,
                        **{k: np.fromfile(os.path.join(d, k + ".blob"), np.uint8).reshape(1, 1666)
                           for k in ("moves", "sequence", "qstring")})
    for name, sl, T, N, seed, C, p_step, okw in CASES:
        sc = synth.make_scores(T, N, sl, seed, C=C, p_step=p_step)
        f = sc.astype(np.float32)
        scale = float(okw.get("temperature", 1.0))
        t = oracle.ref_decode_tensors(f, sl, oracle.decoder_init(**okw), score_scale=scale)
        r = {k: t.pop(k) for k in ("moves", "sequence", "qstring")}
        if scale == 1.0:  # the decoder's own entry point must say the same
            whole = oracle.ref_decode(f, sl, oracle.decoder_init(**okw))
            assert all(np.array_equal(whole[k], r[k]) for k in r)
        np.savez_compressed(os.path.join(OUT, "synth_%s.npz" % name), scores=sc,
                            state_len=sl, opt_keys=np.array(list(okw.keys()), dtype="U16"),
                            opt_values=np.array(list(okw.values()), dtype=np.float64),
                            **r, **t)
        print(name, sc.shape, "seq lens", r["moves"].sum(1))
    rng = np.random.default_rng(7)
    B, S, H, D = 2, 9, 3, 16  # packed [B][S][3][H][D]; rotate Q and K heads (2H), leave V
    x = rng.standard_normal((B, S, 3, H, D)).astype(np.float16)
    half = D // 2
    pos = np.arange(S)[:, None] * (10000.0 ** (-np.arange(half) / half))[None, :]
    sin, cos = np.sin(pos).astype(np.float32), np.cos(pos).astype(np.float32)
    y = x.astype(np.float32).copy()
    oracle.ref_rotary(y.reshape(-1), sin, cos, half, S * 3 * H * D, 3 * H * D, D, B, S, 2 * H)
    np.savez_compressed(os.path.join(OUT, "rotary_small.npz"), x=x, sin=sin, cos=cos, out=y)
    print("rotary", x.shape)


if __name__ == "__main__":
    main()
