"""CPU tests of the boundary: the shared library builds, loads and exports every symbol that
include/ek_b200.h declares; without a GPU it refuses to create a backend instead of falling
back to anything."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import importlib.util
    spec = importlib.util.spec_from_file_location("ek_build", os.path.join(ROOT, "expert-kit_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    path = mod.build()
    return ctypes.CDLL(path)


def declared_functions():
    src = open(os.path.join(ROOT, "include", "ek_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ek_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in ek_b200.h but not exported"


def test_layout_version_matches_the_header():
    import ek_b200._lib as L
    src = open(os.path.join(ROOT, "include", "ek_b200.h")).read()
    assert int(re.search(r"#define EK_TILE_LAYOUT_VERSION (\d+)", src).group(1)) == L.EK_TILE_LAYOUT_VERSION


def test_binding_covers_the_header():
    import ek_b200._lib as L
    assert sorted(L.SIGNATURES) == declared_functions()


def test_status_names(lib):
    lib.ek_status_name.restype = ctypes.c_char_p
    assert lib.ek_status_name(0) == b"EK_OK"
    assert lib.ek_status_name(1) == b"EK_EXPERT_NOT_FOUND"
    assert lib.ek_status_name(17) == b"EK_TIMEOUT"


def test_create_validates_config_and_never_falls_back():
    import torch
    import ek_b200
    with pytest.raises(ek_b200.EKError) as e:
        ek_b200.Backend(ek_b200.BackendConfig(hidden=100, intermediate=64, n_experts=8, top_k=2))
    assert e.value.status_name == "EK_INVALID_INPUT"
    if not torch.cuda.is_available():
        with pytest.raises(ek_b200.EKError) as e:
            ek_b200.Backend(ek_b200.BackendConfig(hidden=128, intermediate=64, n_experts=8, top_k=2))
        assert e.value.status_name == "EK_CUDA"
        assert "no CPU path" in str(e.value)


def test_expert_id_parsing_matches_expert_key():
    from ek_b200.client import parse_expert_id
    assert parse_expert_id("qwen3/l0-e6") == ("qwen3", 0, 6)
    assert parse_expert_id("ds-tiny/l12-e255") == ("ds-tiny", 12, 255)
    import ek_b200
    for bad in ("qwen3-l0-e6", "qwen3/l0", "qwen3/lx-e1"):
        with pytest.raises(ek_b200.EKError):
            parse_expert_id(bad)


def test_cpp_host_mirror_compiles_and_refuses_without_a_gpu(lib, tmp_path):
    """include/ek_b200.hpp (ExpertDB / ExpertBackend / EKInstanceGate over the C ABI) compiles
    warning-free and links; with no CUDA device the create error surfaces as EKError, exit code 3."""
    import subprocess
    import torch
    import helpers as Hh
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the GPU test runs the driver")
    exe = Hh.build_host_shim(tmp_path)
    r = subprocess.run([exe, "256", "128", "4", "4", "2", "1"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 3, (r.returncode, r.stderr)
    assert "no CUDA device" in r.stderr and "EK_CUDA" in r.stderr
