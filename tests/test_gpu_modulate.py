"""The gated post-norm residual kernel (magi_bias_modulate_add) through the C ABI: against the fixture the reference's own
bias_modulate_add produced (<= 1 bf16 ulp), against the CPU oracle on the 24B hidden size with strided gates and both
map widths, the plain gating mode, and the planner-style error report for a bad map entry."""
import types

import numpy as np
import pytest
import torch

from oracle import chunk_attn_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mb():
    import magi_b200
    return magi_b200


def _norm(gamma, beta, eps=1e-6):
    return types.SimpleNamespace(weight=gamma, bias=beta, eps=eps, zero_centered_gamma=True)


def _assert_one_ulp(got, want, what):
    got, want = got.float().cpu(), want.float().cpu()
    diff = (got - want).abs()
    assert (diff <= want.abs() * 2 ** -7 + 1e-6).all(), f"{what}: more than one bf16 ulp off (max diff {diff.max().item()})"


def test_matches_the_reference_fixture(mb, golden_dir):
    from magi_b200 import inference
    z = np.load(f"{golden_dir}/modulate.npz")
    bf = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16)
    for tag in ("f32", "bf16"):
        x = torch.from_numpy(z[f"{tag}_x"]) if tag == "f32" else bf(z[f"{tag}_x"])
        res, gate, want = bf(z[f"{tag}_res"]), bf(z[f"{tag}_gate"]), bf(z[f"{tag}_out"])
        h = x.shape[-1]
        gate_mlp = gate.cuda().chunk(2, dim=-1)[1]          # a strided half of the fused gates, as the layer passes it
        got = inference.bias_modulate_add(x.cuda(), res.cuda(), torch.from_numpy(z[f"{tag}_cmap"]).cuda(), gate_mlp,
                                          _norm(torch.from_numpy(z[f"{tag}_gamma"]), torch.from_numpy(z[f"{tag}_beta"])))
        torch.cuda.synchronize()
        assert got.shape == x.shape and got.dtype == torch.bfloat16
        _assert_one_ulp(got, want, tag)
        assert (got.cpu().view(torch.int16) == want.view(torch.int16)).float().mean().item() > 0.99
    assert mb.Context.get().status() == 0


@pytest.mark.parametrize("h,xdt,mapdt", [(6144, torch.float32, torch.int64), (3072, torch.bfloat16, torch.int32), (8192, torch.float32, torch.int32), (136, torch.bfloat16, torch.int64)])
def test_hidden_sizes_dtypes_and_maps_against_the_oracle(mb, h, xdt, mapdt):
    S, n = 777, 4
    g = torch.Generator().manual_seed(h)
    x = (torch.randn(S, 1, h, generator=g) * 2 - 0.3).to(xdt)
    res = torch.randn(S, 1, h, generator=g).to(torch.bfloat16)
    gate = torch.tanh(torch.randn(1, n, h, generator=g)).to(torch.bfloat16)
    cmap = torch.randint(0, n, (S, 1), generator=g).to(mapdt)
    gamma, beta = 0.1 * torch.randn(h, generator=g), 0.05 * torch.randn(h, generator=g)
    got = mb.bias_modulate_add(x.cuda(), res.cuda(), cmap.cuda(), gate.cuda(), _norm(gamma, beta))
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    _assert_one_ulp(got, O.bias_modulate_add(x, res, cmap, gate, gamma, beta).to(torch.bfloat16), f"h={h}")


def test_gating_alone_and_bad_map_entry(mb):
    S, n, h = 300, 3, 1024
    g = torch.Generator().manual_seed(5)
    x = torch.randn(S, h, generator=g)
    gate = torch.randn(n, h, generator=g)
    cmap = torch.randint(0, n, (S,), generator=g).to(torch.int32)
    got = mb.bias_modulate_add(x.cuda(), None, cmap.cuda(), gate.cuda(), None)     # range_mod only: y = x * gate[map]
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), (x * gate[cmap.long()]).to(torch.bfloat16))
    bad = cmap.clone()
    bad[17] = n
    out = torch.full((S, h), 9.0, dtype=torch.bfloat16, device="cuda")
    mb.bias_modulate_add(x.cuda(), None, bad.cuda(), gate.cuda(), None, out=out)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == mb._lib.E_RANGE                  # reported through the device status word
    assert (out[17].float() == 9).all() and torch.equal(out[16].cpu(), got[16].cpu())
    assert mb.Context.get().status() == 0                                # reading clears it
    with pytest.raises(mb.MagiError) as e:
        mb.bias_modulate_add(torch.zeros(4, 100, device="cuda"), None, None, torch.zeros(1, 100, device="cuda"), None)
    assert e.value.code == mb._lib.E_BADARG                              # hidden must be a multiple of 8
