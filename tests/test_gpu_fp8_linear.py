"""The FP8 linear layers' activation quantiser (magi_div_clamp_to_e4m3) byte for byte against the fixture the reference's
div_clamp_to produced and against the oracle on a large case, and the two linear mirrors against the oracle's fp32
statement of what the reference's quantised linears compute."""
import numpy as np
import pytest
import torch

from oracle import chunk_attn_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mb():
    import magi_b200
    return magi_b200


def test_quantiser_is_byte_identical_to_the_reference_fixture(mb, golden_dir):
    z = np.load(f"{golden_dir}/div_clamp.npz")
    x = torch.from_numpy(z["x"].copy()).view(torch.bfloat16).cuda()
    got_c = mb.div_clamp_to(x, torch.from_numpy(z["scale_c"]))
    got_s = mb.inference.div_clamp_to(x.reshape(4, 12, -1), torch.from_numpy(z["scale_s"]))
    torch.cuda.synchronize()
    assert got_c.dtype == torch.float8_e4m3fn and got_s.shape == (4, 12, x.shape[1])
    assert np.array_equal(got_c.cpu().view(torch.uint8).numpy(), z["out_c"])
    assert np.array_equal(got_s.cpu().view(torch.uint8).numpy(), z["out_s"])


def test_quantiser_large_strided_input_against_the_oracle(mb):
    g = torch.Generator().manual_seed(61)
    rows, cols = 3001, 6144
    base = (torch.randn(rows, cols + 64, generator=g) * 40).to(torch.bfloat16)
    x = base[:, 32:32 + cols]                                  # row stride != cols, 16-byte aligned start
    scale = torch.rand(cols, generator=g) * 0.5 + 0.01
    got = mb.div_clamp_to(x.cuda(), scale)
    torch.cuda.synchronize()
    want = O.div_clamp_to(x, scale)
    assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8))
    with pytest.raises(mb.MagiError) as e:
        mb.div_clamp_to(torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda"), torch.ones(1))
    assert e.value.code == mb._lib.E_BADARG


@pytest.mark.parametrize("kind", ["per_tensor", "per_channel"])
def test_linear_mirrors_against_the_oracle(mb, kind):
    from magi_b200 import inference as inf
    g = torch.Generator().manual_seed(67)
    S, K, N = 300, 1024, 768
    x = (torch.randn(S, 1, K, generator=g) * 2).to(torch.bfloat16)
    w8 = (torch.randn(N, K, generator=g) * 20).to(torch.float8_e4m3fn)
    w_scale = torch.tensor([0.003])
    if kind == "per_tensor":
        in_scale = torch.full((K,), 0.02)
        lin = inf.PerTensorQuantizedFp8Linear(w8.cuda().unsqueeze(0), w_scale, in_scale)
        ref = O.fp8_linear(x, in_scale, w8, 0.02, 0.003)
    else:
        smooth = torch.rand(1, K, generator=g) * 0.05 + 0.01
        in_scale = torch.tensor([0.7])
        lin = inf.PerChannelQuantizedFp8Linear(w8.cuda().unsqueeze(0), w_scale, in_scale, smooth)
        ref = O.fp8_linear(x, smooth, w8, 0.7, 0.003)
    y = lin(x.cuda())
    torch.cuda.synchronize()
    assert y.shape == (S, 1, N) and y.dtype == torch.bfloat16
    err = (y.float().cpu() - ref).abs().max().item()
    assert err <= ref.abs().max().item() * 2 ** -7 and O.cosine(y.cpu(), ref) >= 0.99999, (err, O.cosine(y.cpu(), ref))
