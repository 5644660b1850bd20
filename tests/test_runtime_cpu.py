"""The torch-free runtime on the CPU: argument surface, variant rules, registry, loader (with a fake nvcc), pool.
Modelled on the reference's runtime tests (reference: tests/cake/_runtime/test_config.py, test_registry.py,
test_loader.py, test_workspace.py, test_torch_free.py)."""

from __future__ import annotations

import argparse
import ctypes
import os
import stat
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

import miles_ext_kernels_b200 as package
from miles_ext_kernels_b200 import cake
from miles_ext_kernels_b200.cake._runtime import config, loader, registry, spec, workspace

ROOT = Path(__file__).resolve().parents[1]


def _parse(*argv):
    parser = argparse.ArgumentParser()
    package.add_arguments(parser)
    return parser.parse_args(list(argv))


# ---- spec ----------------------------------------------------------------------------------------------------------
def test_flag_and_opspec_validation():
    with pytest.raises(ValueError, match="is not a --cake-<op>-<what> flag"):
        spec.Flag("--gdn-x", dict(default=0, help=""))
    with pytest.raises(ValueError, match="are missing"):
        spec.Flag("--cake-gdn-x", dict(default=0))
    with pytest.raises(ValueError, match="dest follows"):
        spec.Flag("--cake-gdn-x", dict(default=0, help="", dest="y"))
    assert spec.Flag("--cake-gdn-recompute-state", dict(default=False, help="")).dest == "cake_gdn_recompute_state"
    with pytest.raises(ValueError, match="variants"):
        spec.OpSpec("x", "", variants=("fast", "det"))
    with pytest.raises(ValueError, match="must start with"):
        spec.OpSpec("x", "", variants=("det",), flags=(spec.Flag("--cake-y-z", dict(default=0, help="")),))
    op = cake.op_spec("kda")
    assert op.has_variant_flag and not op.shows_variant_flag and op.cli_choices == ("det",)
    assert cake.op_spec("gdn").selector == "--linear-attention-backend cake"
    with pytest.raises(KeyError):
        cake.op_spec("rmsnorm")


# ---- config --------------------------------------------------------------------------------------------------------
def test_cli_defaults_to_fast_and_det_under_deterministic_mode():
    args = _parse()
    args.linear_attention_backend = "cake"
    package.validate_args(args)
    assert args.cake_gdn_variant == "fast"
    args = _parse()
    args.linear_attention_backend, args.deterministic_mode = "cake", True
    package.validate_args(args)
    assert args.cake_gdn_variant == "det"
    args = _parse("--cake-gdn-variant", "fast")
    args.linear_attention_backend, args.deterministic_mode = "cake", True
    with pytest.raises(ValueError, match="not bit-reproducible"):
        package.validate_args(args)
    args = _parse("--cake-deterministic")
    args.linear_attention_backend = "cake"
    package.validate_args(args)
    assert args.cake_gdn_variant == "det"


def test_options_of_an_unselected_op_are_rejected():
    args = _parse("--cake-gdn-recompute-state")
    with pytest.raises(ValueError, match="requires --linear-attention-backend cake"):
        package.validate_args(args)
    args = _parse("--cake-workspace-pool-bytes", "-1")
    with pytest.raises(ValueError, match=">= 0"):
        package.validate_args(args)


def test_kda_validation_rejects_context_parallelism_and_other_layouts():
    args = _parse()
    args.kda_backend, args.context_parallel_size = "cake", 2
    with pytest.raises(ValueError, match="context parallelism"):
        package.validate_args(args)
    args = _parse()
    args.kda_backend, args.qkv_format = "cake", "bshd"
    with pytest.raises(ValueError, match="--qkv-format thd"):
        package.validate_args(args)


def test_configure_replaces_the_state_and_checks_keys():
    assert cake.variant("gdn") == "det"  # never configured: det
    package.configure(cake_gdn_variant="fast", cake_gdn_recompute_state=True, not_ours=1)
    assert cake.variant("gdn") == "fast" and cake.option("gdn", "cake_gdn_recompute_state") is True
    package.configure({"cake_workspace_pool_bytes": 16})
    assert cake.variant("gdn") == "det" and cake.option(None, "cake_workspace_pool_bytes") == 16
    with pytest.raises(ValueError, match="unknown cake option"):
        package.configure(cake_gdn_typo=1)
    with pytest.raises(ValueError, match="must be one of"):
        package.configure(cake_gdn_variant="slow")
    with pytest.raises(ValueError, match="not bit-reproducible"):
        package.configure(cake_gdn_variant="fast", deterministic_mode=True)
    with pytest.raises(KeyError):
        cake.option("gdn", "nope")
    package.configure(argparse.Namespace(cake_gdn_variant=None, other=3))
    assert cake.variant("gdn") == "det"


# ---- torch-free imports ----------------------------------------------------------------------------------------------
def test_importing_the_package_and_op_modules_imports_neither_torch_nor_the_implementation():
    code = textwrap.dedent(
        """
        import sys
        sys.modules["torch"] = None
        import miles_ext_kernels_b200, miles_ext_kernels_b200.cake
        from miles_ext_kernels_b200.cake import gdn, kda
        import argparse
        p = argparse.ArgumentParser(); miles_ext_kernels_b200.add_arguments(p)
        miles_ext_kernels_b200.configure(cake_gdn_variant="det")
        assert not any(m.startswith("miles_ext_kernels_b200.cake._impl.gdn") for m in sys.modules)
        assert "ctypes" not in sys.modules or True
        print(sorted(gdn.__all__))
        """
    )
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert "chunk_gated_delta_rule" in out.stdout


def test_the_package_works_under_the_reference_name():
    code = textwrap.dedent(
        """
        import importlib, sys
        sys.modules["miles_ext_kernels"] = importlib.import_module("miles_ext_kernels_b200")
        import miles_ext_kernels
        from miles_ext_kernels_b200.cake.gdn import OP
        assert miles_ext_kernels.SOURCES == ("cake",) and OP.name == "gdn"
        """
    )
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr


# ---- loader --------------------------------------------------------------------------------------------------------
def _fake_nvcc(tmp_path: Path, fail: bool = False) -> Path:
    log = tmp_path / "nvcc.log"
    script = tmp_path / "bin" / "nvcc"
    script.parent.mkdir()
    body = f"""#!{sys.executable}
import sys
if "--version" in sys.argv:
    print("nvcc: NVIDIA (R) Cuda compiler driver\\nCuda compilation tools, release 12.9, V12.9.86")
    raise SystemExit(0)
open({str(log)!r}, "a").write(" ".join(sys.argv[1:]) + "\\n")
if {fail!r}:
    sys.stderr.write("fake: compile error\\n"); raise SystemExit(1)
open(sys.argv[sys.argv.index("-o") + 1], "wb").write(b"not a real library")
"""
    script.write_text(body)
    script.chmod(script.stat().st_mode | stat.S_IEXEC)
    return script


def test_build_goes_to_the_cache_once_and_no_build_raises(tmp_path, monkeypatch):
    nvcc = _fake_nvcc(tmp_path)
    monkeypatch.setenv("CUDA_HOME", str(nvcc.parent.parent))
    monkeypatch.setenv("MILES_EXT_KERNELS_CACHE_DIR", str(tmp_path / "cache"))
    monkeypatch.setattr(loader, "_IN_TREE", tmp_path / "nothing_prebuilt")
    found = loader.find_nvcc()
    assert found == str(nvcc) and loader.get_cuda_version() == loader.CudaVersion(12, 9, "12.9.86")
    assert loader.get_cuda_version().cudart == 12090
    library = loader.library_spec()
    with loader.no_build():
        with pytest.raises(RuntimeError, match="would compile inside a call: prebuild"):
            library.build()
    path = library.build()
    assert path.parent == tmp_path / "cache" and path.read_bytes() == b"not a real library"
    assert library.build() == path
    command = (tmp_path / "nvcc.log").read_text().splitlines()
    assert len(command) == 1 and "-gencode=arch=compute_100a,code=sm_100a" in command[0] and "-lineinfo" in command[0]
    with loader.no_build():
        assert library.build() == path  # cached: no compile
    assert not list(path.parent.glob("*.tmp.so"))


def test_a_failed_compile_reports_the_command_and_leaves_nothing(tmp_path, monkeypatch):
    nvcc = _fake_nvcc(tmp_path, fail=True)
    monkeypatch.setenv("CUDA_HOME", str(nvcc.parent.parent))
    monkeypatch.setenv("MILES_EXT_KERNELS_CACHE_DIR", str(tmp_path / "cache"))
    monkeypatch.setattr(loader, "_IN_TREE", tmp_path / "nothing_prebuilt")
    with pytest.raises(RuntimeError, match="(?s)nvcc failed to build libmek_b200 .*fake: compile error"):
        loader.library_spec().build()
    assert not list((tmp_path / "cache").glob("*.so"))


def test_toolkit_too_old_and_unknown_arch(tmp_path, monkeypatch):
    nvcc = _fake_nvcc(tmp_path)
    monkeypatch.setenv("CUDA_HOME", str(nvcc.parent.parent))
    monkeypatch.setitem(loader.MIN_CUDA, "sm_100a", (13, 4))
    with pytest.raises(RuntimeError, match="needs CUDA 13.4 or newer"):
        loader.check_toolkit("sm_100a", "the kernels")
    with pytest.raises(NotImplementedError):
        loader.LibrarySpec("libmek_b200", "sm_90a")
    with pytest.raises(KeyError):
        loader.LibrarySpec("libnope", "sm_100a")


def test_the_built_library_exports_every_declared_symbol():
    """The C-ABI library loads without a GPU and exports everything include/mek_gdn.h declares."""
    names = loader.declared_symbols()
    assert {"mek_gdn_wy_fwd", "mek_gdn_fwd_h", "mek_gdn_fwd_o", "mek_gdn_bwd_dh", "mek_gdn_bwd_tail",
            "mek_build_cuda_version", "mek_last_error"} <= set(names)
    library = loader.load_library()  # built in the tree by build(); compiled here if it is missing
    dll = ctypes.CDLL(str(library.path))
    for name in names:
        assert hasattr(dll, name), name
    assert library.build_cuda_version == loader.get_cuda_version().cudart
    with pytest.raises(ValueError):
        library.check(1)
    with pytest.raises(NotImplementedError):
        library.check(2)
    with pytest.raises(RuntimeError):
        library.check(3)


def test_native_argument_checks_run_without_a_gpu():
    """Extent checks happen before any CUDA call: a bad call reports MEK_ERR_* and its text on a CPU-only box."""
    library = loader.load_library()
    code = library.mek_gdn_l2norm(None, None, None, ctypes.c_int64(0), 1, ctypes.c_int64(0), None)
    assert code == 1 and "l2norm" in library.last_error()


# ---- registry --------------------------------------------------------------------------------------------------------
def test_prebuild_is_keyword_only_and_release_reaches_imported_implementations(monkeypatch):
    import inspect

    from miles_ext_kernels_b200.cake._impl import gdn as implementation

    signature = inspect.signature(implementation.prebuild)
    assert all(p.kind is inspect.Parameter.KEYWORD_ONLY for p in signature.parameters.values())
    assert list(signature.parameters) == ["device", "max_workers"]
    called = []
    monkeypatch.setattr(implementation, "release", lambda: called.append("gdn"))
    assert package.release() == 0 and called == ["gdn"]
    with pytest.raises(KeyError):
        registry.prebuild("nope")


# ---- workspace -------------------------------------------------------------------------------------------------------
def test_the_pool_reuses_evicts_and_releases():
    import torch

    package.configure(cake_workspace_pool_bytes=1024)
    a = workspace.take("gdn", "x", (64,), torch.float32, "cpu")
    b = workspace.take("gdn", "x", (32,), torch.float32, "cpu")
    assert a.data_ptr() == b.data_ptr() and b.shape == (32,)
    c = workspace.take("gdn", "y", (200,), torch.float32, "cpu")  # 800 B: evicts x (256 B + 800 B > 1024 B)
    assert workspace.stats()["cpu"]["evictions"] >= 1 and workspace.stats()["cpu"]["bytes"] == 800
    big = workspace.take("gdn", "z", (1024,), torch.float32, "cpu")  # above the bound: a plain allocation
    assert big.numel() == 1024 and workspace.stats()["cpu"]["bytes"] == 800
    assert c.numel() == 200 and package.release() == 800
    package.configure()
    fresh = workspace.take("gdn", "x", (8,), torch.float32, "cpu")
    assert fresh.numel() == 8 and workspace.stats()["cpu"]["bytes"] == 0
