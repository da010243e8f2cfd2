"""The C-ABI library loads without a GPU and exports every function the header declares."""
import ctypes
import re
from pathlib import Path

import pytest

from cleffa_b200 import build as omni_build
from cleffa_b200 import omni

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "clef_cuda_omni.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#ifdef CLEF_ENGINE_H.*?#endif", "", text, flags=re.S)    # inline adapter for the reference's clef_config
    return sorted(set(re.findall(r"\b(clef_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    return ctypes.CDLL(str(omni_build.build()))


def test_header_declares_the_reference_entry_points():
    names = declared_functions()
    for ref_name in ("clef_omni_reserve", "clef_omni_free", "clef_omni_begin", "clef_omni_trace_reserve",
                     "clef_omni_complete", "clef_omni_keepalive", "clef_gpu_dump_routes"):
        assert ref_name in names            # clef_metal_internal.h:65-70, clef_engine.h:178
    assert "clef_omni_encode_moe" in names  # MoE half of clef_omni_encode_layer (clef_metal_internal.h:79)


def test_library_exports_every_declared_symbol(lib):
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_python_mirror_binds_every_declared_symbol():
    assert sorted(omni.EXPORTS) == declared_functions()
    omni.load_library()


def test_missing_library_is_an_error_not_a_fallback(tmp_path):
    with pytest.raises(omni.OmniError):
        omni.load_library(tmp_path / "libclef_cuda_omni.so")


def test_header_compiles_as_c_and_cxx(tmp_path):
    import subprocess
    for comp, std, ext in (("gcc", "-std=c11", "c"), ("g++", "-std=c++17", "cc")):
        src = tmp_path / f"t.{ext}"
        src.write_text('#include "clef_cuda_omni.h"\nint main(void) { return sizeof(clef_omni_config) == 20 ? 0 : 1; }\n')
        subprocess.run([comp, std, "-Wall", "-Werror", "-I", str(ROOT / "include"), str(src), "-o", str(tmp_path / "t")], check=True)
        subprocess.run([str(tmp_path / "t")], check=True)


def test_open_without_a_gpu_fails_loudly():
    """No CPU path exists behind the boundary: without a usable CUDA device the context cannot
    be opened, and the message says why."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("this box has a GPU")
    with pytest.raises(omni.OmniError, match="cuda: "):
        omni.OmniBackend(0)


def reference_dir():
    import os
    for cand in (os.environ.get("CLEF_REFERENCE_DIR"), ROOT.parent / "reference"):     # or a checkout beside this repository
        if cand and (Path(cand) / "clef_engine.h").exists():
            return Path(cand)
    return None


@pytest.mark.skipif(reference_dir() is None, reason="no checkout of the reference engine (set CLEF_REFERENCE_DIR)")
def test_integration_stub_builds_against_the_reference_headers(tmp_path, lib):
    """tests/integration_stub.c is the binding the integration guide shows.  It is compiled with the
    reference's own clef_engine.h in front of this repository's header, so clef_config,
    clef_layer_w and gguf_tensor (clef_engine.h:18-40, clef_gguf.h:31-39) are the real types,
    and linked against the library so every call resolves."""
    import subprocess
    stub = ROOT / "tests" / "integration_stub.c"
    md = (ROOT / "INTEGRATION.md").read_text()
    body = stub.read_text().split("*/", 1)[1].strip()
    assert body in md, "the integration guide must show the stub that is compiled here"
    main = tmp_path / "main.c"
    main.write_text('#include <stdbool.h>\n#include <stddef.h>\nvoid cuda_backend_close(void);\n'
                    'int main(int argc, char **argv) { (void)argv; if (argc > 99) cuda_backend_close(); return 0; }\n')
    exe = tmp_path / "stub"
    libdir = omni_build.LIB.parent
    subprocess.run(["gcc", "-std=c11", "-D_GNU_SOURCE", "-Wall", "-Wextra", "-Werror", "-I", str(reference_dir()), "-I", str(ROOT / "include"),
                    str(stub), str(main), "-L", str(libdir), "-lclef_cuda_omni", f"-Wl,-rpath,{libdir}", "-o", str(exe)], check=True)
    subprocess.run([str(exe)], check=True)
