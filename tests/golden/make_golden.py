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

  kranges.npz    the reference's k-range generators run as they are (SampleTransport.generate_default_kvrange,
                 generate_noise2clean_kvrange, generate_kvrange_for_prefix_video, generate_kvrange_for_denoising_video,
                 get_denoise_step_of_each_chunk, generate_sequences and VideoDiTModel.generate_kv_range_for_uncondition,
                 executed from the reference's source files, with a SimpleNamespace standing in for `self`) over every
                 forward step of the shipped 24B schedule and a few variations.
  cp_xattn.npz   cp_ulysses_process (scatter_to_context_parallel_region of x / condition_map / rope +
                 cp_update_cross_attn_qkv_range), and the scatter with cp_shuffle_num 2, run unmodified on gloo CPU ranks.

  modulate.npz   the reference's bias_modulate_add (dit_module.py:288-307) with its own FusedLayerNorm, the Triton gating
                 kernel inside it replaced by the one-line torch statement of what it computes (y[row] = x[row] *
                 gate[map[row]]: Triton needs a GPU), for an fp32 and a bf16 projection output.

  div_clamp.npz  the reference's div_clamp_to (dit_module.py:364-384) on bf16 activations with a per-channel and a
                 scalar scale: values around and beyond the e4m3 range, subnormal results, exact ties of both roundings.

  linear_prologue.npz  get_q / get_k / get_v from their first line: the reference's CustomLayerNormLinear
                 (dit_module.py:390-425, bf16 torch.nn.Linear members) forward_q / forward_k / forward_v on CPU, then
                 the reference's FusedLayerNorm and flash-attn's pure-torch rotary, in get_q's order (:953-963).

  xqkv.npz       FullyParallelAttention.get_xqkv (dit_module.py:1005-1021) called unbound on a namespace that carries the
                 reference's own CustomLayerNormLinear (forward_qx), torch.nn.Linear linear_kv_xattn and two FusedLayerNorm
                 modules: the cross-attention query, key and value from hidden states and caption states.

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


# ------------------------------------------------------------------------------------------------ k-range generators
def _reference_functions(path, names):
    """Compile the named functions / methods straight from a reference source file, without importing the module around
    them (inference.pipeline.video_generate pulls in T5, the VAE and packages this container does not have).  The code
    that runs is the reference's own text; nothing of it is stored here."""
    import ast
    from typing import Dict, List, Tuple, Union  # noqa: F401 - names the reference's annotations use
    with open(path) as f:
        tree = ast.parse(f.read())
    found = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in names and node.name not in found:
            node.decorator_list = []
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"torch": torch, "List": List, "Tuple": Tuple, "Dict": Dict, "Union": Union, "np": np}
            exec(compile(mod, path, "exec"), ns)
            found[node.name] = ns[node.name]
    missing = set(names) - set(found)
    if missing:
        raise RuntimeError(f"{path}: not found: {sorted(missing)}")
    return found


def gen_kranges(ref_root, out_dir):
    vg = os.path.join(ref_root, "inference", "pipeline", "video_generate.py")
    names = ["generate_sequences", "get_denoise_step_of_each_chunk", "get_batch_size_and_chunk_token_nums",
             "generate_kvrange_for_prefix_video", "generate_default_kvrange", "generate_noise2clean_kvrange",
             "generate_kvrange_for_denoising_video", "generate_denoise_status_and_sequences", "total_forward_step"]
    fn = _reference_functions(vg, names)
    out = {}

    def make_self(num_steps, window_size, chunk_num, n2c, clean, prefix_chunks, batch=1, lat_h=90, lat_w=160):
        prefix = torch.zeros(1, 1, prefix_chunks * 6, 1, 1) if prefix_chunks else None
        ti = types.SimpleNamespace(latent_size=[1, 16, chunk_num * 6, lat_h, lat_w], num_steps=num_steps, chunk_num=chunk_num,
                                   prefix_video=prefix)
        me = types.SimpleNamespace(chunk_width=6, window_size=window_size, transport_inputs=[ti], device="cpu",
                                   model_config=types.SimpleNamespace(patch_size=2),
                                   runtime_config=types.SimpleNamespace(noise2clean_kvrange=list(n2c), clean_chunk_kvrange=clean))
        for n in names[1:]:
            setattr(me, n, types.MethodType(fn[n], me))
        if batch != 1:   # the reference hard-codes batch 1; its range code nevertheless carries batch offsets
            tok = me.get_batch_size_and_chunk_token_nums(0)[1]
            me.get_batch_size_and_chunk_token_nums = lambda infer_idx: (batch, tok)
        return me

    # generate_denoise_status_and_sequences calls the module-level generate_sequences
    fn["generate_denoise_status_and_sequences"].__globals__["generate_sequences"] = fn["generate_sequences"]

    cases = {
        # the shipped 24B base schedule (example/24B/24B_base_config.json): 32 steps, window 4, 96 frames -> 4 chunks
        "base24b": dict(num_steps=32, window_size=4, chunk_num=4, n2c=[5, 4, 3, 2], clean=1, prefix_chunks=0),
        # a longer clip so the steady state (4 chunks in flight, prefix behind them) is reached; distill schedule
        "long16": dict(num_steps=16, window_size=4, chunk_num=9, n2c=[5, 4, 3, 2], clean=1, prefix_chunks=0),
        # image/video-to-video: two prefix chunks; clean_chunk_kvrange -1 falls back to the last window
        "prefix": dict(num_steps=8, window_size=4, chunk_num=7, n2c=[5, 4, 3, 2], clean=-1, prefix_chunks=2),
        # no windows configured: every chunk sees everything before it
        "default": dict(num_steps=8, window_size=4, chunk_num=5, n2c=[], clean=-1, prefix_chunks=0),
        # batch offsets (k_batch_start = i * range_num)
        "batch2": dict(num_steps=8, window_size=4, chunk_num=5, n2c=[3, 2], clean=1, prefix_chunks=0, batch=2),
    }
    for tag, c in cases.items():
        me = make_self(**c)
        rows = []
        kr_all = []
        for step in range(me.total_forward_step(0)):
            (per_stage, stage, idx), (chunk_offset, chunk_start, chunk_end, t_start, t_end) = \
                me.generate_denoise_status_and_sequences(0, step)
            # slice_point / denoising_range_num / fwd_extra_1st_chunk as forward_velocity derives them (video_generate.py:606-628)
            extra = chunk_start > chunk_offset and idx == 0
            slice_point = chunk_start - 1 if extra else chunk_start
            n_den = chunk_end - chunk_start + (1 if extra else 0)
            steps_of = me.get_denoise_step_of_each_chunk(0, per_stage, t_start, t_end, idx, has_clean_t=extra)
            kr = me.generate_kvrange_for_denoising_video(infer_idx=0, slice_point=slice_point, denoising_range_num=n_den,
                                                         denoise_step_of_each_chunk=steps_of)
            rows.append([step, chunk_offset, chunk_start, chunk_end, t_start, t_end, idx, int(extra), slice_point, n_den,
                         len(kr_all)] + steps_of + [-1] * (8 - len(steps_of)))
            kr_all.append(kr.numpy().astype(np.int32))
        out[f"{tag}_cfg"] = np.array([c["num_steps"], c["window_size"], c["chunk_num"], c["clean"], c["prefix_chunks"],
                                      c.get("batch", 1), me.get_batch_size_and_chunk_token_nums(0)[1]] + list(c["n2c"]))
        out[f"{tag}_steps"] = np.array(rows, dtype=np.int32)
        out[f"{tag}_kr_len"] = np.array([len(k) for k in kr_all], dtype=np.int32)
        out[f"{tag}_kr"] = np.concatenate(kr_all)
        for range_num in (1, 2, 7):
            out[f"{tag}_prefix{range_num}"] = me.generate_kvrange_for_prefix_video(0, range_num).numpy().astype(np.int32)
    # neither kind of window configured: generate_kvrange_for_prefix_video falls back to 8 chunks
    me = make_self(num_steps=8, window_size=4, chunk_num=12, n2c=[], clean=-1, prefix_chunks=0)
    out["fallback8_prefix12"] = me.generate_kvrange_for_prefix_video(0, 12).numpy().astype(np.int32)

    # the unconditional pass: every chunk sees only itself, chunks laid out as batch (dit_model.py:92-101); the method asks
    # for the current CUDA device, which this container does not have
    from unittest import mock
    un = _reference_functions(os.path.join(ref_root, "inference", "model", "dit", "dit_model.py"),
                              ["generate_kv_range_for_uncondition"])["generate_kv_range_for_uncondition"]
    real_to = torch.Tensor.to

    def cpu_to(self, *a, **k):
        a = tuple("cpu" if isinstance(x, str) and x.startswith("cuda") else x for x in a)
        return real_to(self, *a, **k)
    with mock.patch.object(torch.cuda, "current_device", lambda: 0), mock.patch.object(torch.Tensor, "to", cpu_to):
        me = types.SimpleNamespace(model_config=types.SimpleNamespace(t_patch_size=1, patch_size=2))
        out["uncond"] = un(me, torch.zeros(5, 16, 6, 90, 160)).numpy().astype(np.int32)
    np.savez_compressed(os.path.join(out_dir, "kranges.npz"), **out)


def _cp_xattn_worker(rank, world, ref_root, port, ret_dir):
    sys.path.insert(0, ref_root)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from inference.common import PackedCrossAttnParams
    from inference.infra.distributed import parallel_state as mpu
    from inference.infra.parallelism import context_parallel as cp
    mpu.initialize_model_parallel(cp_size=world)
    out = {}

    def params(chunk_tokens, n_ranges, caps):
        cq = torch.arange(n_ranges + 1, dtype=torch.int32) * chunk_tokens
        ck = torch.tensor([0] + list(np.cumsum(caps)), dtype=torch.int32)
        return PackedCrossAttnParams(q_ranges=torch.stack([cq[:-1], cq[1:]], 1), kv_ranges=torch.stack([ck[:-1], ck[1:]], 1),
                                     cu_seqlens_q=cq, cu_seqlens_kv=ck, max_seqlen_q=chunk_tokens, max_seqlen_kv=800)

    # (a) cp_ulysses_process as the model calls it: x [S, N, D], condition_map [S], rope [S, 96]; batch 1 and batch 2
    for tag, (C, n, N, caps) in {"a": (37, 3, 1, [5, 3, 9]), "b": (10, 5, 1, [4, 7, 3, 6, 2])}.items():
        S = C * n
        g = torch.Generator().manual_seed(21)
        x = torch.randn(S, N, 8, generator=g)
        cmap = torch.arange(S, dtype=torch.int32) // C
        rope = torch.randn(S, 96, generator=g)
        xs, cm, rp, splits, xp = cp.cp_ulysses_process(world, x, cmap, rope, None, params(C, n * N, caps))
        out.update({f"{tag}_in": np.array([C, n, N] + caps), f"{tag}_x": xs.numpy(), f"{tag}_cmap": cm.numpy(), f"{tag}_rope": rp.numpy(),
                    f"{tag}_splits": np.array(splits), f"{tag}_q": xp.q_ranges.numpy(), f"{tag}_k": xp.kv_ranges.numpy(),
                    f"{tag}_maxq": np.array([xp.max_seqlen_q, xp.max_seqlen_kv])})
    # (b) the scatter alone with a shuffled split (cp_shuffle_num 2, used by the reference's other CP strategy).  The range
    # update is not run that way: with more than one batch element or shuffle piece its own closing assertion
    # (unique q boundaries vs unique k boundaries) fails unless the surviving captions happen to be adjacent.
    C, n, shuffle = 24, 4, 2
    S = C * n
    splits = [S // world] * world
    out.update({"s_in": np.array([C, n, shuffle]), "s_splits": np.array(splits)})
    g = torch.Generator().manual_seed(22)
    x = torch.randn(S, 1, 4, generator=g)
    out["s_x"] = cp.scatter_to_context_parallel_region(x, splits, cp_shuffle_num=shuffle).numpy()
    np.savez(os.path.join(ret_dir, f"r{rank}.npz"), **out)
    dist.barrier()
    dist.destroy_process_group()


def gen_cp_xattn(ref_root, out_dir):
    import torch.multiprocessing as mp
    out = {}
    for world, port in ((2, 29621), (4, 29622)):
        with tempfile.TemporaryDirectory() as td:
            mp.spawn(_cp_xattn_worker, args=(world, ref_root, port, td), nprocs=world, join=True)
            for r in range(world):
                z = np.load(os.path.join(td, f"r{r}.npz"))
                for key in z.files:
                    out[f"cp{world}_r{r}_{key}"] = z[key]
    np.savez_compressed(os.path.join(out_dir, "cp_xattn.npz"), **out)


def gen_modulate(ref_mod, out_dir):
    def range_mod_torch(x, c_mapping, gatings):   # what range_mod_triton returns, on the CPU
        s, b, h = x.shape
        xf = x.transpose(0, 1).flatten(0, 1)
        y = xf * gatings.flatten(0, 1)[c_mapping.transpose(0, 1).flatten(0, 1).long()]
        return y.reshape(b, s, h).transpose(0, 1)
    ref_mod.range_mod_triton = range_mod_torch
    out = {}
    for tag, (S, n, h, xdt) in {"f32": (24, 3, 512, torch.float32), "bf16": (16, 2, 1536, torch.bfloat16)}.items():
        g = torch.Generator().manual_seed(31 + h)
        cfg = types.SimpleNamespace(apply_layernorm_1p=True, layernorm_epsilon=1e-6, params_dtype=torch.float32)
        ln = ref_mod.FusedLayerNorm(cfg, h)
        with torch.no_grad():
            ln.weight.copy_(0.1 * torch.randn(h, generator=g))
            ln.bias.copy_(0.05 * torch.randn(h, generator=g))
        x = (torch.randn(S, 1, h, generator=g) * 3 + 0.5).to(xdt)
        res = torch.randn(S, 1, h, generator=g).to(torch.bfloat16)
        gate = torch.tanh(torch.randn(1, n, 2 * h, generator=g)).to(torch.bfloat16)   # soft-capped adaLN gates, msa | mlp
        cmap = (torch.arange(S) * n // S).reshape(S, 1)                               # int64, as torch.arange gives
        with torch.no_grad():
            y = ref_mod.bias_modulate_add(x, res, cmap, gate.chunk(2, dim=-1)[1], ln).to(torch.bfloat16)
        out.update({f"{tag}_x": x.float().numpy() if xdt == torch.float32 else bf16_bits(x), f"{tag}_res": bf16_bits(res),
                    f"{tag}_gate": bf16_bits(gate), f"{tag}_cmap": cmap.numpy(), f"{tag}_gamma": ln.weight.detach().numpy(),
                    f"{tag}_beta": ln.bias.detach().numpy(), f"{tag}_out": bf16_bits(y)})
    np.savez_compressed(os.path.join(out_dir, "modulate.npz"), **out)


def gen_div_clamp(ref_mod, out_dir):
    g = torch.Generator().manual_seed(53)
    rows, cols = 48, 256
    x = (torch.randn(rows, cols, generator=g) * torch.logspace(-3, 3, cols)).to(torch.bfloat16)
    x[0, :16] = torch.tensor([0.0, -0.0, 448.0, -448.0, 464.0, 480.0, 1e30, -1e30, 2 ** -9, 2 ** -10, 3 * 2 ** -10, 2 ** -7,
                              0.0625, 17.0, 18.0, 19.0]).to(torch.bfloat16)           # edges of e4m3, ties, saturation
    scale_c = (torch.rand(cols, generator=g) * 3 + 0.05).float()
    scale_c[:16] = 1.0
    scale_s = torch.tensor([0.37])
    out = {"x": bf16_bits(x), "scale_c": scale_c.numpy(), "scale_s": scale_s.numpy()}
    with torch.no_grad():
        out["out_c"] = ref_mod.div_clamp_to(x, scale_c).view(torch.uint8).numpy()
        out["out_s"] = ref_mod.div_clamp_to(x.reshape(4, 12, cols), scale_s).view(torch.uint8).numpy()
    np.savez_compressed(os.path.join(out_dir, "div_clamp.npz"), **out)


def gen_linear_prologue(ref_mod, out_dir):
    from flash_attn.layers.rotary import apply_rotary_emb_torch
    g = torch.Generator().manual_seed(23)
    T, K, Hq, Hkv, D = 136, 128, 3, 1, 128
    mcfg = types.SimpleNamespace(apply_layernorm_1p=True, layernorm_epsilon=1e-6, params_dtype=torch.bfloat16, num_layers=4)
    ecfg = types.SimpleNamespace(fp8_quant=False)
    lin = ref_mod.CustomLayerNormLinear(K, Hq * D, Hkv * D, 1, mcfg, ecfg)
    with torch.no_grad():
        for name in ("q", "k", "v"):
            getattr(lin, name).weight.copy_((torch.randn(getattr(lin, name).weight.shape, generator=g) * K ** -0.5).to(torch.bfloat16))
    x = (torch.randn(T, 1, K, generator=g) * 1.3).to(torch.bfloat16)          # [sq, b, hidden]: the output of forward_ln
    ncfg = types.SimpleNamespace(apply_layernorm_1p=True, layernorm_epsilon=1e-6, params_dtype=torch.float32)
    out = {"x": bf16_bits(x[:, 0])}
    sin, cos = ref_mod.build_rotary_pos_embed(
        [2, 4, 17], bands=ref_mod.freq_bands(16, step=1), dim=128, in_pixels=False,
        ref_feat_shape=[2, 4 / math.sqrt(68 / 256), 17 / math.sqrt(68 / 256)])
    out["sin"], out["cos"] = sin.numpy(), cos.numpy()
    with torch.no_grad():
        for name, fwd in (("q", lin.forward_q), ("k", lin.forward_k)):
            gamma = 0.1 * torch.randn(D, generator=g)
            beta = 0.02 * torch.randn(D, generator=g)
            ln = ref_mod.FusedLayerNorm(ncfg, D)
            ln.weight.copy_(gamma)
            ln.bias.copy_(beta)
            y = fwd(x)                                                          # bf16 [sq, b, hn * hd]
            y = y.reshape(y.size(0), y.size(1), -1, D).float()
            y = ln(y).transpose(0, 1).contiguous()                              # b sq hn hd
            r = apply_rotary_emb_torch(y, cos, sin).to(torch.bfloat16)[0]       # (sq b) hn hd with b = 1
            out["w" + name], out["gamma_" + name], out["beta_" + name] = bf16_bits(getattr(lin, name).weight), gamma.numpy(), beta.numpy()
            out[name] = bf16_bits(r)
        out["wv"] = bf16_bits(lin.v.weight)
        out["v"] = bf16_bits(lin.forward_v(x)[:, 0].reshape(T, Hkv, D))
    np.savez_compressed(os.path.join(out_dir, "linear_prologue.npz"), **out)


def gen_xqkv(ref_mod, out_dir):
    g = torch.Generator().manual_seed(29)
    T, K, Hq, Hkv, D, cap_dim, Y = 72, 128, 2, 1, 128, 128, 40
    mcfg = types.SimpleNamespace(apply_layernorm_1p=True, layernorm_epsilon=1e-6, params_dtype=torch.bfloat16, num_layers=4)
    lin = ref_mod.CustomLayerNormLinear(K, Hq * D, Hkv * D, 1, mcfg, types.SimpleNamespace(fp8_quant=False))
    kv_lin = torch.nn.Linear(cap_dim, 2 * Hkv * D, bias=False, dtype=torch.bfloat16)
    ncfg = types.SimpleNamespace(apply_layernorm_1p=True, layernorm_epsilon=1e-6, params_dtype=torch.float32)
    qn, kn = ref_mod.FusedLayerNorm(ncfg, D), ref_mod.FusedLayerNorm(ncfg, D)
    with torch.no_grad():
        lin.qx.weight.copy_((torch.randn(Hq * D, K, generator=g) * K ** -0.5).to(torch.bfloat16))
        kv_lin.weight.copy_((torch.randn(2 * Hkv * D, cap_dim, generator=g) * cap_dim ** -0.5).to(torch.bfloat16))
        for ln in (qn, kn):
            ln.weight.copy_(0.1 * torch.randn(D, generator=g))
            ln.bias.copy_(0.02 * torch.randn(D, generator=g))
    x = (torch.randn(T, 1, K, generator=g) * 1.3).to(torch.bfloat16)
    y = torch.randn(Y, cap_dim, generator=g).to(torch.bfloat16)
    me = types.SimpleNamespace(linear_qkv=lin, q_layernorm_xattn=qn, k_layernorm_xattn=kn, linear_kv_xattn=kv_lin,
                               hidden_size_per_attention_head=D)
    with torch.no_grad():
        q, k, v = ref_mod.FullyParallelAttention.get_xqkv(me, x, y)
    np.savez_compressed(os.path.join(out_dir, "xqkv.npz"), x=bf16_bits(x[:, 0]), y=bf16_bits(y), wqx=bf16_bits(lin.qx.weight),
                        wkv=bf16_bits(kv_lin.weight), gq=qn.weight.detach().numpy(), bq=qn.bias.detach().numpy(),
                        gk=kn.weight.detach().numpy(), bk=kn.bias.detach().numpy(), q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="root of the MAGI-1 checkout")
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    sys.path.insert(0, a.ref)
    only = set(a.only.split(",")) if a.only else None
    if only is None or only & {"prologue", "rope", "modulate", "div_clamp", "linear_prologue", "xqkv"}:
        import inference.model.dit.dit_module as ref_mod
        if only is None or "prologue" in only:
            gen_prologue(ref_mod, a.out)
        if only is None or "rope" in only:
            gen_rope(ref_mod, a.out)
        if only is None or "modulate" in only:
            gen_modulate(ref_mod, a.out)
        if only is None or "div_clamp" in only:
            gen_div_clamp(ref_mod, a.out)
        if only is None or "linear_prologue" in only:
            gen_linear_prologue(ref_mod, a.out)
        if only is None or "xqkv" in only:
            gen_xqkv(ref_mod, a.out)
    if only is None or "attn" in only:
        gen_attn_cfg0(a.out)
    if only is None or "ulysses" in only:
        gen_ulysses(a.ref, a.out)
    if only is None or "kranges" in only:
        gen_kranges(a.ref, a.out)
    if only is None or "cp_xattn" in only:
        gen_cp_xattn(a.ref, a.out)
    print("wrote fixtures to", a.out)


if __name__ == "__main__":
    main()
