"""Generate the golden fixtures in this directory from the reference's own CPU-runnable code.

Run in a container where the reference checkout is mounted (pass its root with --ref) and where
flash-attn is importable:

    python tests/golden/make_golden.py --ref <reference root>

What is produced (all seeded, small enough to commit):
  prologue.npz   x (bf16 bits), gamma, beta, sin, cos -> reference FusedLayerNorm (gamma+1) in fp32,
                 then flash-attn's pure-torch rotary (apply_rotary_emb_torch), cast to bf16; plus the
                 fp32 intermediate.  Call order as in FullyParallelAttention.get_q.
  rope.npz       build_rotary_pos_embed(...) outputs for a few (T_total,H,W) with the caller's
                 ref_feat_shape rule, incl. keeping only the last T*H*W rows.
  attn_cfg0.npz  the CPU fp32 benchmark case (3 chunks x 128 tokens, 8/2 heads; q,k,v come from seed 0): the output
                 of torch's scaled_dot_product_attention under the explicit boolean block mask.
  ulysses.npz    head/sequence ownership of the reference's all_to_all_input_split /
                 all_to_all_output_split, obtained by running them on gloo CPU ranks
                 (cp = 2 with an uneven split, cp = 4 with KV-head replication).

The reference holds no attention fixture of its own; see the oracle's header.
"""
import argparse
import math
import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().copy()


def gen_prologue(ref_mod, out_dir):
    from flash_attn.layers.rotary import apply_rotary_emb_torch
    g = torch.Generator().manual_seed(11)
    T, H, D = 96, 6, 128
    x = (torch.randn(T, H, D, generator=g) * 1.7 + 0.3).to(torch.bfloat16)
    gamma = 0.1 * torch.randn(D, generator=g)
    beta = 0.02 * torch.randn(D, generator=g)
    cfg = types.SimpleNamespace(apply_layernorm_1p=True, layernorm_epsilon=1e-6, params_dtype=torch.float32)
    ln = ref_mod.FusedLayerNorm(cfg, D)
    with torch.no_grad():
        ln.weight.copy_(gamma)
        ln.bias.copy_(beta)
    sin, cos = ref_mod.build_rotary_pos_embed(
        [4, 4, 6], bands=ref_mod.freq_bands(16, step=1), dim=128, in_pixels=False,
        ref_feat_shape=[4, 4 / math.sqrt(24 / 256), 6 / math.sqrt(24 / 256)])
    with torch.no_grad():
        y = ln(x.float())                         # [T,H,D] fp32
        y_b = y.unsqueeze(0)                      # b s h d
        r = apply_rotary_emb_torch(y_b, cos, sin)[0]
    np.savez_compressed(os.path.join(out_dir, "prologue.npz"), x=bf16_bits(x), gamma=gamma.numpy(),
                        beta=beta.numpy(), sin=sin.numpy(), cos=cos.numpy(), ln_fp32=y.numpy(),
                        out_fp32=r.numpy(), out_bf16=bf16_bits(r))


def gen_rope(ref_mod, out_dir):
    out = {}
    for name, (T_total, T_keep, H, W) in {"a": (3, 3, 5, 7), "b": (6, 2, 8, 8), "c": (5, 4, 30, 52)}.items():
        r = math.sqrt((H * W) / 256)
        sin, cos = ref_mod.build_rotary_pos_embed([T_total, H, W], bands=ref_mod.freq_bands(16, step=1), dim=128,
                                                  in_pixels=False, ref_feat_shape=[T_total, H / r, W / r])
        emb = torch.cat([sin, cos], -1)[-(T_keep * H * W):]
        if name == "c":  # large grid: keep a strided sample of rows
            idx = torch.arange(0, emb.shape[0], 37)
            out[f"{name}_idx"] = idx.numpy()
            emb = emb[idx]
        out[f"{name}_shape"] = np.array([T_total, T_keep, H, W])
        out[f"{name}_emb"] = emb.numpy()
    np.savez_compressed(os.path.join(out_dir, "rope.npz"), **out)


def gen_attn_cfg0(out_dir):
    g = torch.Generator(device="cpu").manual_seed(0)
    S, Hq, Hkv, D, C = 384, 8, 2, 128, 128
    q = torch.randn(S, Hq, D, generator=g) * (1 / math.sqrt(D))
    k = torch.randn(S, Hkv, D, generator=g) * (1 / math.sqrt(D))
    v = torch.randn(S, Hkv, D, generator=g) * (1 / math.sqrt(D))
    mask = torch.zeros(S, S, dtype=torch.bool)
    for i in range(3):
        mask[i * C:(i + 1) * C, :(i + 1) * C] = True
    kk = torch.repeat_interleave(k, Hq // Hkv, dim=1)
    vv = torch.repeat_interleave(v, Hq // Hkv, dim=1)
    o = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1)[None], kk.transpose(0, 1)[None], vv.transpose(0, 1)[None], attn_mask=mask)[0].transpose(0, 1)
    # q, k, v are regenerated from seed 0 by the test; their float64 sums guard against generator drift
    np.savez_compressed(os.path.join(out_dir, "attn_cfg0.npz"), out=o.contiguous().numpy(),
                        sums=np.array([q.double().sum().item(), k.double().sum().item(), v.double().sum().item()]))


def _ulysses_worker(rank, world, ref_root, port, case, ret_dir):
    sys.path.insert(0, ref_root)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from inference.infra.distributed import parallel_state as mpu
    from inference.infra.parallelism import context_parallel as cp
    mpu.initialize_model_parallel(cp_size=world)
    S, Hq, Hkv, D = case
    splits = [S // world + (1 if i < S % world else 0) for i in range(world)]
    off = sum(splits[:rank])
    g = torch.Generator().manual_seed(5)
    qfull = torch.randn(S, Hq, D, generator=g)
    kvfull = torch.randn(S, Hkv, 2 * D, generator=g)
    q_loc = qfull[off:off + splits[rank]].contiguous()
    kv_loc = kvfull[off:off + splits[rank]].contiguous()
    q_x, h = cp.all_to_all_input_split(q_loc, splits)
    h.wait()
    kv_x, h = cp.all_to_all_input_split(kv_loc, splits)
    h.wait()
    o_x, h = cp.all_to_all_output_split(q_x.contiguous(), splits)
    h.wait()
    # the reference's final rearrange "(cp sq b) hn hd -> sq b (cp hn hd)" with b = 1
    from einops import rearrange
    o_fin = rearrange(o_x, "(cp sq b) hn hd -> (sq) b (cp hn hd)", cp=world, b=1)
    np.savez(os.path.join(ret_dir, f"r{rank}.npz"), q_x=q_x.numpy(), kv_x=kv_x.numpy(), o_fin=o_fin.numpy())
    dist.barrier()
    dist.destroy_process_group()


def gen_ulysses(ref_root, out_dir):
    import torch.multiprocessing as mp
    out = {}
    for tag, world, case, port in (("cp2", 2, (11, 4, 2, 8), 29611), ("cp4", 4, (10, 8, 2, 8), 29612)):
        with tempfile.TemporaryDirectory() as td:
            mp.spawn(_ulysses_worker, args=(world, ref_root, port, case, td), nprocs=world, join=True)
            out[f"{tag}_case"] = np.array(case)
            for r in range(world):
                z = np.load(os.path.join(td, f"r{r}.npz"))
                for key in ("q_x", "kv_x", "o_fin"):
                    out[f"{tag}_r{r}_{key}"] = z[key]
    np.savez_compressed(os.path.join(out_dir, "ulysses.npz"), **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="root of the MAGI-1 checkout")
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    sys.path.insert(0, a.ref)
    only = set(a.only.split(",")) if a.only else None
    if only is None or "prologue" in only or "rope" in only:
        import inference.model.dit.dit_module as ref_mod
        if only is None or "prologue" in only:
            gen_prologue(ref_mod, a.out)
        if only is None or "rope" in only:
            gen_rope(ref_mod, a.out)
    if only is None or "attn" in only:
        gen_attn_cfg0(a.out)
    if only is None or "ulysses" in only:
        gen_ulysses(a.ref, a.out)
    print("wrote fixtures to", a.out)


if __name__ == "__main__":
    main()
