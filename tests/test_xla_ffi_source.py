"""The XLA FFI layer is shipped as source (jaxlib is not available where these tests run): check
that it is complete and self-consistent -- every kernel entry point of the C header has a handler,
the handler names in the C++ file, the JAX shim and INTEGRATION.md agree, the handlers type-check
against a stand-in of the FFI header surface they use, and the build gate says plainly when jax is
missing."""
import ast
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FFI = os.path.join(ROOT, "train_gpt_b200", "xla_ffi")

# entry points that are queries or self-tests, not kernels an XLA program would call
NOT_BOUND = {"tg_version", "tg_last_cuda_error", "tg_set_gemm_reserved_sms", "tg_selftest_quantise_division", "tg_selftest_bounded_wait",
             "tg_rmsnorm_bwd_static_max_scratch_bytes"}


def _cc():
    return open(os.path.join(FFI, "xla_ffi.cc")).read()


def _handler_names():
    return sorted(re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\(\s*(Tg\w+)", _cc()))


def _shim_targets():
    tree = ast.parse(open(os.path.join(FFI, "jax_shim.py")).read())
    for node in ast.walk(tree):
        if isinstance(node, ast.Assign) and any(getattr(t, "id", None) == "FFI_TARGETS" for t in node.targets):
            return sorted(ast.literal_eval(node.value))
    raise AssertionError("FFI_TARGETS not found in jax_shim.py")


def test_every_kernel_entry_point_has_a_handler():
    header = open(os.path.join(ROOT, "include", "train_gpt_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(tg_[a-z0-9_]+)\s*\(", header))
    called = set(re.findall(r"\b(tg_[a-z0-9_]+)\s*\(", _cc()))
    missing = declared - NOT_BOUND - called
    assert not missing, f"no XLA handler calls {sorted(missing)}"
    assert called <= declared, f"handlers call undeclared symbols {sorted(called - declared)}"


def test_handler_names_agree_between_cc_shim_and_integration_doc():
    names = _handler_names()
    assert len(names) >= 15 and len(set(names)) == len(names)
    assert names == _shim_targets()
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    for n in names:
        assert n in doc, f"{n} is not mentioned in INTEGRATION.md"
    # every target the shim calls through ffi_call is a registered one
    shim = open(os.path.join(FFI, "jax_shim.py")).read()
    used = set(re.findall(r'ffi_call\(\s*"(Tg\w+)"', shim)) | set(re.findall(r'_gemm\(\s*"(Tg\w+)"', shim))
    assert used and used <= set(names)


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_handlers_type_check_against_the_stand_in_header():
    r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", f"-I{os.path.join(ROOT, 'tests', 'ffi_stub')}",
                        f"-I{os.path.join(ROOT, 'include')}", os.path.join(FFI, "xla_ffi.cc")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]


def test_build_gate_reports_missing_jax():
    from train_gpt_b200.xla_ffi import build
    if build.ffi_include_dir() is None:
        with pytest.raises(RuntimeError, match="jax is not installed"):
            build.build()
        with pytest.raises(ImportError):
            import train_gpt_b200.xla_ffi.jax_shim  # noqa: F401
    else:                                                    # a JAX host: the command at least names the right files
        cmd = build.command(build.ffi_include_dir())
        assert any(c.endswith("xla_ffi.cc") for c in cmd) and "-ltrain_gpt_b200" in cmd
