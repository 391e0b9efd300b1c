"""The C-ABI library loads on a CPU-only box and exports exactly what include/magi_attn.h declares."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "magi_attn.h")


def _declared():
    src = open(HEADER).read()
    return sorted(set(re.findall(r"MAGI_API\s+[\w\s\*]+?\b(magi_\w+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    import magi_b200
    lib = C.CDLL(magi_b200.LIB_PATH)
    names = _declared()
    assert len(names) >= 17
    for n in names:
        assert hasattr(lib, n), f"{n} declared in magi_attn.h but not exported"
    assert sorted(magi_b200._lib.EXPORTS) == [n for n in names if n in magi_b200._lib.EXPORTS]
    missing_in_shim = [n for n in names if n not in magi_b200._lib.EXPORTS]
    assert not missing_in_shim, f"shim does not bind {missing_in_shim}"


def test_version_and_error_strings():
    import magi_b200
    lib = magi_b200._lib.lib
    assert lib.magi_version() >= 100
    assert lib.magi_strerror(0) == b"ok"
    for code in range(-8, 0):
        assert lib.magi_strerror(code) not in (b"ok", b"unknown error")
    assert lib.magi_strerror(-99) == b"unknown error"


def test_struct_layouts_match_the_header(tmp_path):
    """ctypes mirrors vs sizeof/offsetof computed by the C compiler from the real header."""
    import magi_b200
    L = magi_b200._lib
    probe = tmp_path / "probe.c"
    fields = {
        "magi_attn_params": ["q", "k", "v", "out", "lse", "total_q", "q_ranges", "n_ranges", "softmax_scale", "cache",
                             "prefix_chunk_ids", "q_scale", "scale_chunk_tokens", "q_lo", "o_peer_ptrs", "o_peer_offsets",
                             "n_o_peers", "o_head_offset"],
        "magi_prologue_params": ["x", "T", "gamma", "eps", "cos", "out", "out_stride_block", "heads_per_block",
                                 "out_block_ptrs", "x_heads_per_block", "x_stride_block"],
        "magi_kv_cache_desc": ["dtype", "chunk_tokens", "n_kv_heads"],
        "magi_modulate_params": ["x", "residual", "residual_dtype", "gate", "gate_stride", "condition_map", "n_gates", "gamma",
                                 "eps", "gamma_plus_one", "out", "out_stride", "rows", "hidden"],
        "magi_linear_prologue_params": ["x", "x_stride", "w", "w_stride", "T", "H", "in_features", "eps", "gamma", "beta",
                                        "rot_pairs", "heads_per_block", "cos", "sin", "out", "out_stride_t", "out_stride_h",
                                        "out_stride_block", "out_block_ptrs", "dtype", "plain_odd_heads", "x_scale", "w_scale"],
    }
    body = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){"]
    for s, fs in fields.items():
        body.append(f'printf("{s} %zu\\n", sizeof({s}));')
        for f in fs:
            body.append(f'printf("{s}.{f} %zu\\n", offsetof({s}, {f}));')
    body.append("return 0;}")
    probe.write_text("\n".join(body))
    exe = tmp_path / "probe"
    subprocess.check_call(["gcc", str(probe), "-o", str(exe)])
    out = subprocess.check_output([str(exe)], text=True).split("\n")
    mirror = {"magi_attn_params": L.AttnParams, "magi_prologue_params": L.PrologueParams, "magi_kv_cache_desc": L.KVCacheDesc,
              "magi_modulate_params": L.ModulateParams, "magi_linear_prologue_params": L.LinearPrologueParams}
    for line in out:
        if not line:
            continue
        key, val = line.split()
        if "." in key:
            s, f = key.split(".")
            assert getattr(mirror[s], f).offset == int(val), key
        else:
            assert C.sizeof(mirror[key]) == int(val), key


def test_no_gpu_means_loud_failure_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    import magi_b200
    h = C.c_void_p()
    rc = magi_b200._lib.lib.magi_ctx_create(0, C.byref(h))
    assert rc < 0 and not h.value
    with pytest.raises((magi_b200.MagiError, RuntimeError, AssertionError)):
        magi_b200.Context(0)
