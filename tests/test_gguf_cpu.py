"""The checkpoint loader's header walk and tensor checks, without a GPU (small extents).

Mirrors what the reference's engine refuses when it binds the same tensors
(clef.c:194-205 `bind_experts`, clef.c:55-57 the epsilon key)."""
import ctypes as C

import pytest
import torch

from cleffa_b200.omni import load_library
from tests.gguf_writer import BF16, F32, omni_kv, omni_layers, write_gguf

H, FFN, E = 64, 32, 4
EPS_KEY = "clef.attention.layer_norm_rms_epsilon"


def layer(seed):
    g = torch.Generator().manual_seed(seed)
    w = tuple(torch.randn(s, generator=g).to(torch.bfloat16) for s in ((E, H), (E, 2 * FFN, H), (E, H, FFN)))
    return w, torch.randn(H, generator=g)


def check(path, n_layer=2, dims=(H, FFN, E)):
    lib = load_library()
    err = C.create_string_buffer(512)
    eps = C.c_float(0)
    ok = lib.clef_omni_gguf_check(str(path).encode(), n_layer, *dims, C.byref(eps), err, 512)
    return ok, eps.value, err.value.decode()


@pytest.fixture()
def good(tmp_path):
    layers = [layer(1), layer(2)]
    tensors = omni_layers([w for w, _ in layers], [n for _, n in layers], H, FFN, E)
    kv = omni_kv(H, FFN, E, used=2, n_layer=2)
    return tmp_path, kv, tensors


def test_well_formed_file_passes(good):
    tmp, kv, tensors = good
    write_gguf(tmp / "ok.gguf", kv, tensors)
    ok, eps, err = check(tmp / "ok.gguf")
    assert ok, err
    assert eps == pytest.approx(1e-6)
    write_gguf(tmp / "ok64.gguf", kv, tensors, alignment=64)
    assert check(tmp / "ok64.gguf")[0]


@pytest.mark.parametrize("case, message", [
    ("missing", "missing or invalid rank-3 expert tensor blk.1.ffn_down_exps.weight"),
    ("f32_experts", "missing or invalid rank-3 expert tensor blk.0.ffn_gate_up_exps.weight"),
    ("extent", "missing or invalid tensor blk.1.ffn_router.weight"),
    ("norm_type", "missing or invalid tensor blk.0.ffn_norm.weight"),
    ("no_eps", "missing rms eps"),
    ("eps_value", "unsupported Omni decoder/head geometry or routing configuration"),
    ("not_clef", "not a clef GGUF"),
    ("no_expert_count", "missing or invalid clef.moe.expert_count"),
    ("no_width", "missing or invalid clef.embedding_length"),
    ("used_gt_experts", "unsupported Omni decoder/head geometry or routing configuration"),
    ("no_renorm", "unsupported Omni decoder/head geometry or routing configuration"),
    ("renorm_off", "unsupported Omni decoder/head geometry or routing configuration"),
    ("layers", "the checkpoint has 2 layers"),
    ("missing_layer", "blk.2.ffn_norm.weight"),
    ("magic", "bad magic"),
    ("version", "unsupported version"),
    ("truncated", "past the end of the file"),
    ("misaligned", "not aligned"),
    ("dims", "unsupported Omni decoder/head geometry or routing configuration"),
])
def test_malformed_files_are_refused(good, case, message):
    tmp, kv, tensors = good
    args, n_layer, dims = {}, 2, (H, FFN, E)
    if case == "missing":
        del tensors["blk.1.ffn_down_exps.weight"]
    elif case == "f32_experts":
        tensors["blk.0.ffn_gate_up_exps.weight"] = (F32, tensors["blk.0.ffn_gate_up_exps.weight"][1].float())
    elif case == "extent":
        tensors["blk.1.ffn_router.weight"] = (BF16, tensors["blk.1.ffn_router.weight"][1][:, : H - 8].contiguous())
    elif case == "norm_type":
        tensors["blk.0.ffn_norm.weight"] = (BF16, tensors["blk.0.ffn_norm.weight"][1].to(torch.bfloat16))
    elif case == "no_eps":
        del kv[EPS_KEY]
    elif case == "eps_value":
        kv[EPS_KEY] = 1e-5
    elif case == "not_clef":
        kv["general.architecture"] = "llama"
    elif case == "no_expert_count":
        del kv["clef.moe.expert_count"]
    elif case == "no_width":
        del kv["clef.embedding_length"]
    elif case == "used_gt_experts":
        kv["clef.moe.expert_used_count"] = E + 1
    elif case == "no_renorm":
        del kv["clef.moe.normalize_topk"]
    elif case == "renorm_off":
        kv["clef.moe.normalize_topk"] = False
    elif case == "layers":
        n_layer = 3
    elif case == "missing_layer":
        n_layer, kv["clef.block_count"] = 3, 3
    elif case == "magic":
        args["magic"] = b"GGML"
    elif case == "version":
        args["version"] = 2
    elif case == "truncated":
        args["truncate"] = 100
    elif case == "misaligned":
        args["misalign"] = "blk.1.ffn_router.weight"
    elif case == "dims":
        dims = (2048, 768, 128)
    write_gguf(tmp / "bad.gguf", kv, tensors, **args)
    ok, _, err = check(tmp / "bad.gguf", n_layer, dims)
    assert not ok and message in err, err


def test_garbage_and_missing_files(tmp_path):
    assert "cannot open" in check(tmp_path / "nope.gguf")[2]
    (tmp_path / "short.gguf").write_bytes(b"GGUF")
    assert "too short" in check(tmp_path / "short.gguf")[2]
    # counts that promise more than the file holds
    (tmp_path / "lie.gguf").write_bytes(b"GGUF" + (3).to_bytes(4, "little") + (1 << 40).to_bytes(8, "little") + (0).to_bytes(8, "little") + b"\0" * 64)
    assert not check(tmp_path / "lie.gguf")[0]
    # a string length that runs past the end
    (tmp_path / "str.gguf").write_bytes(b"GGUF" + (3).to_bytes(4, "little") + (0).to_bytes(8, "little") + (1).to_bytes(8, "little") + (1 << 50).to_bytes(8, "little") + b"\0" * 32)
    assert "truncated" in check(tmp_path / "str.gguf")[2]


def test_loader_is_callable_from_a_c_host(good, tmp_path):
    """The reference's host is C: a C program built against the header and the shared library
    checks a file (no GPU needed for this entry point)."""
    import subprocess
    from pathlib import Path

    from cleffa_b200.omni import _LIB_PATH

    tmp, kv, tensors = good
    write_gguf(tmp / "ok.gguf", kv, tensors)
    src = tmp_path / "host.c"
    src.write_text(r'''
#include <stdio.h>
#include "clef_cuda_omni.h"
int main(int argc, char **argv) {
    char err[256] = "";
    float eps = 0.f;
    if (argc < 2) return 2;
    if (!clef_omni_gguf_check(argv[1], 2, 64, 32, 4, &eps, err, sizeof err)) { printf("refused: %s\n", err); return 1; }
    printf("ok eps=%g\n", eps);
    return 0;
}
''')
    root = Path(__file__).resolve().parents[1]
    exe = tmp_path / "host"
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", str(root / "include"), str(src), "-o", str(exe),
                    "-L", str(_LIB_PATH.parent), "-lclef_cuda_omni", f"-Wl,-rpath,{_LIB_PATH.parent}"], check=True)
    out = subprocess.run([str(exe), str(tmp / "ok.gguf")], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.startswith("ok eps=1e-06"), out.stdout + out.stderr
    out = subprocess.run([str(exe), str(tmp / "absent.gguf")], capture_output=True, text=True)
    assert out.returncode == 1 and "cannot open" in out.stdout
