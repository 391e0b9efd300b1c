"""Cross-checks of the kernel and the oracle against two independent implementations on the GPU box:

* torch.nn.functional.scaled_dot_product_attention in fp32 with an explicit boolean block mask, and
* the third-party kernel the reference itself dispatches to when MagiAttention is absent: a loop of
  flash_attn_func over the ranges, shaped as in core_attention (inference/model/dit/dit_module.py:1049-1065).
  The reference pins flash-attn 2.4.2; the image carries a later 2.x, so this check is skipped when that build has no
  kernel for the device.

Neither is a dispatch target of the library; they are only compared with, and flash-attn is only ever loaded in a
child process."""
import numpy as np
import pytest
import torch

from gpu_util import as_segments, assert_close
from oracle import chunk_attn_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(C, n, Hq, Hkv, seed):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(n * C, Hq, 128, generator=g)).to(torch.bfloat16)
    k = (torch.randn(n * C, Hkv, 128, generator=g)).to(torch.bfloat16)
    v = (torch.randn(n * C, Hkv, 128, generator=g)).to(torch.bfloat16)
    return q, k, v


def test_against_sdpa_with_boolean_block_mask():
    import magi_b200 as mb
    from magi_b200 import host
    C, n, Hq, Hkv = 200, 3, 8, 2
    q, k, v = _inputs(C, n, Hq, Hkv, 91)
    qr, kr = host.q_ranges_for_chunks(n, C), np.array([[0, C], [0, 2 * C], [2 * C, 3 * C]], dtype=np.int32)   # k-start > 0 for chunk 2
    out, _ = mb.chunk_attn(q.cuda(), k.cuda(), v.cuda(), qr, kr, C, n * C)
    mask = O.block_mask(qr, as_segments(kr), n * C, n * C).cuda()
    qf = q.cuda().float().permute(1, 0, 2)[None]                                    # [1, Hq, S, 128]
    kf = k.cuda().float().repeat_interleave(Hq // Hkv, dim=1).permute(1, 0, 2)[None]
    vf = v.cuda().float().repeat_interleave(Hq // Hkv, dim=1).permute(1, 0, 2)[None]
    with torch.nn.attention.sdpa_kernel(torch.nn.attention.SDPBackend.MATH):
        ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, attn_mask=mask[None, None])
    ref = ref[0].permute(1, 0, 2)
    torch.cuda.synchronize()
    assert_close(out, ref.cpu(), what="kernel vs SDPA (fp32, boolean block mask)")
    # and the oracle agrees with SDPA to fp32 rounding
    want, _ = O.range_attention(q.float(), k.float(), v.float(), qr, as_segments(kr))
    assert (want - ref.cpu()).abs().max().item() < 2e-5


_FLASH_CHILD = r"""
import sys, numpy as np, torch
inp, outp = sys.argv[1], sys.argv[2]
z = torch.load(inp)
try:
    import flash_attn
    q, k, v, qr, kr = z["q"].cuda(), z["k"].cuda(), z["v"].cuda(), z["qr"], z["kr"]
    outs = []
    for i in range(qr.shape[0]):          # the loop of core_attention, inference/model/dit/dit_module.py:1052-1065, bs == 1
        o = flash_attn.flash_attn_func(q=q[None, qr[i, 0]:qr[i, 1]], k=k[None, kr[i, 0]:kr[i, 1]],
                                       v=v[None, kr[i, 0]:kr[i, 1]], deterministic=False)
        outs.append(o[0])
    torch.cuda.synchronize()
    torch.save({"out": torch.cat(outs, dim=0).cpu(), "version": flash_attn.__version__}, outp)
except Exception as e:                     # no flash-attn, or no kernel image for this device in the installed build
    torch.save({"skip": f"{type(e).__name__}: {str(e)[:160]}"}, outp)
"""


def test_against_the_reference_fallback_loop_of_flash_attn_func(tmp_path):
    """flash-attn runs in a child process, so this process only ever loads the library under test."""
    import subprocess
    import sys
    import magi_b200 as mb
    from magi_b200 import host
    C, n, Hq, Hkv = 1560, 4, 24, 8                       # one latent frame of 30x52 patches per chunk, 4.5B heads
    q, k, v = _inputs(C, n, Hq, Hkv, 92)
    qr, kr = host.q_ranges_for_chunks(n, C), host.default_k_ranges(n, C)
    inp, outp = str(tmp_path / "in.pt"), str(tmp_path / "out.pt")
    torch.save({"q": q, "k": k, "v": v, "qr": torch.as_tensor(qr), "kr": torch.as_tensor(kr)}, inp)
    subprocess.run([sys.executable, "-c", _FLASH_CHILD, inp, outp], check=True, timeout=300)
    z = torch.load(outp)
    if "skip" in z:
        pytest.skip(f"flash-attn reference loop unavailable: {z['skip']}")
    ref = z["out"]
    out, _ = mb.chunk_attn(q.cuda(), k.cuda(), v.cuda(), qr, kr, C, n * C)
    torch.cuda.synchronize()
    # two bf16 kernels with different summation orders: compare both with the fp32 oracle and with each other
    want, _ = O.range_attention(q.float(), k.float(), v.float(), qr, as_segments(kr))
    assert_close(out, want, what="kernel vs oracle")
    assert_close(ref, want, what=f"flash_attn_func loop ({z['version']}) vs oracle")
    assert (out.float().cpu() - ref.float()).abs().max().item() <= 2e-2
