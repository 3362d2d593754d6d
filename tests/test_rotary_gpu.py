"""Rotary embedding through the C ABI against the CPU oracle (tolerance 1e-3 absolute plus
1e-3 relative: results are fp16, the oracle works in fp32 on the same fp16 inputs)."""
import numpy as np
import pytest

from conftest import load_golden

pytestmark = pytest.mark.gpu


def tables(S, half, theta=10000.0):
    pos = np.arange(S)[:, None] * (theta ** (-np.arange(half) / half))[None, :]
    return np.sin(pos).astype(np.float32), np.cos(pos).astype(np.float32)


def run(of, x16, sin, cos, B, S, nheads, half, sb, ss, sh):
    import torch
    x = torch.from_numpy(x16.copy()).cuda()
    of.rotary_emb_gpu(x, torch.from_numpy(sin).cuda(), torch.from_numpy(cos).cuda(), B, S, nheads,
                      2 * half, half, sb, ss, sh)
    return x.cpu().numpy()


def close(a16, ref32):
    d = np.abs(a16.astype(np.float32) - ref32)
    return bool((d <= 1e-3 + 1e-3 * np.abs(ref32)).all())


def test_fixture_from_reference(native_lib):
    g = load_golden("rotary_small")
    B, S, _, H, D = g["x"].shape
    out = run(native_lib, g["x"], g["sin"], g["cos"], B, S, 2 * H, D // 2, S * 3 * H * D, 3 * H * D, D)
    assert close(out, g["out"])
    assert np.array_equal(out[:, :, 2], g["x"][:, :, 2])  # V is not touched


def test_packed_qkv_shape_of_the_encoder(native_lib, oracle_mod):
    # [N][T][3][H=8][D=64], Q and K heads rotated in one call (nheads = 16), V left alone
    B, S, H, D = 4, 1666, 8, 64
    rng = np.random.default_rng(3)
    x = rng.standard_normal((B, S, 3, H, D)).astype(np.float16)
    sin, cos = tables(S, D // 2)
    out = run(native_lib, x, sin, cos, B, S, 2 * H, D // 2, S * 3 * H * D, 3 * H * D, D)
    ref = x.astype(np.float32).copy()
    oracle_mod.rotary(ref.reshape(-1), sin, cos, D // 2, S * 3 * H * D, 3 * H * D, D, B, S, 2 * H)
    assert close(out, ref)
    assert np.array_equal(out[:, :, 2], x[:, :, 2])


@pytest.mark.parametrize("B,S,H,D,half", [(1, 1, 1, 2, 1), (2, 5, 3, 6, 3), (3, 33, 2, 24, 4), (2, 7, 2, 16, 8)])
def test_odd_shapes_take_the_scalar_path(native_lib, oracle_mod, B, S, H, D, half):
    rng = np.random.default_rng(B * 100 + S)
    x = rng.standard_normal((B, S, H, D)).astype(np.float16)
    sin, cos = tables(S, half)
    out = run(native_lib, x, sin, cos, B, S, H, half, S * H * D, H * D, D)
    ref = x.astype(np.float32).copy()
    oracle_mod.rotary(ref.reshape(-1), sin, cos, half, S * H * D, H * D, D, B, S, H)
    assert close(out, ref)


def test_full_size_against_the_oracle(native_lib, oracle_mod):
    # the encoder's whole packed QKV tensor [32][1666][3][8][64] (BASELINE configuration 4) against
    # the CPU routine on the same fp16 values, every element
    import torch
    B, S, H, D = 32, 1666, 8, 64
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((B, S, 3, H, D), generator=g, device="cuda", dtype=torch.float32).half()
    ref = x.float().cpu().numpy()
    sin, cos = tables(S, D // 2)
    oracle_mod.rotary(ref.reshape(-1), sin, cos, D // 2, S * 3 * H * D, 3 * H * D, D, B, S, 2 * H)
    native_lib.rotary_emb_gpu(x, torch.from_numpy(sin).cuda(), torch.from_numpy(cos).cuda(), B, S, 2 * H, D,
                              D // 2, S * 3 * H * D, 3 * H * D, D)
    assert close(x.cpu().numpy(), ref)


def test_full_size_round_trip(native_lib):
    # config-sized tensor: rotating by +theta then by -theta gives the input back up to two
    # fp16 roundings
    import torch
    B, S, H, D = 32, 1666, 8, 64
    g = torch.Generator(device="cuda").manual_seed(1)
    x0 = torch.randn((B, S, 3, H, D), generator=g, device="cuda", dtype=torch.float32).half()
    sin, cos = tables(S, D // 2)
    x = x0.clone()
    s, c = torch.from_numpy(sin).cuda(), torch.from_numpy(cos).cuda()
    args = (B, S, 2 * H, D, D // 2, S * 3 * H * D, 3 * H * D, D)
    native_lib.rotary_emb_gpu(x, s, c, *args)
    assert not torch.equal(x, x0)
    native_lib.rotary_emb_gpu(x, (-s).contiguous(), c, *args)
    assert float((x.float() - x0.float()).abs().max()) <= 6e-3
    assert torch.equal(x[:, :, 2], x0[:, :, 2])
