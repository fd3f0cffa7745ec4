"""The Rust side of the boundary is shipped as source (crates/katsu-cuda: Cargo.toml, build.rs,
src/ffi.rs, src/lib.rs); no Rust toolchain exists in the build image, so what can be checked
without compiling is checked here as text: the generated extern block matches the header function
for function and argument for argument, the safe layer calls only declared functions, and the
build script takes every kernel source with the flags of katsu_b200/build.py."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CRATE = os.path.join(ROOT, "crates", "katsu-cuda")
sys.path.insert(0, CRATE)
import gen_ffi  # noqa: E402


def extern_block():
    text = open(os.path.join(CRATE, "src", "ffi.rs")).read()
    body = text[text.index('extern "C" {'):]
    return {m.group(1): [a for a in m.group(2).split(",") if a.strip()]
            for m in re.finditer(r"pub fn (katsu_cuda_\w+)\(([^)]*)\)", body)}


def test_generated_ffi_is_up_to_date():
    assert subprocess.run([sys.executable, os.path.join(CRATE, "gen_ffi.py"), "--check"]).returncode == 0


def test_extern_block_matches_the_header_name_by_name_and_arity_by_arity():
    declared = {name: args for name, _, args in gen_ffi.declarations()}
    rust = extern_block()
    assert set(rust) == set(declared)
    for name, args in declared.items():
        assert len(rust[name]) == len(args), name
    assert len(declared) >= 40


def test_safe_layer_calls_only_declared_functions():
    lib = open(os.path.join(CRATE, "src", "lib.rs")).read()
    used = set(re.findall(r"ffi::(katsu_cuda_\w+)", lib))
    assert used and used <= set(extern_block())
    for must in ("katsu_cuda_conv2d_fwd_bias_relu", "katsu_cuda_conv2d_bwd_scaled", "katsu_cuda_matmul_fwd",
                 "katsu_cuda_matmul_bwd", "katsu_cuda_allreduce_sum", "katsu_cuda_alloc", "katsu_cuda_free"):
        assert must in used, must


def test_build_script_takes_every_kernel_source_with_the_library_flags():
    build = open(os.path.join(CRATE, "build.rs")).read()
    # the source set is the directory listing, not a hand-kept list
    assert "read_dir" in build and 'ext == "cu"' in build
    assert not re.findall(r'"\w+\.cu"', build)
    from katsu_b200 import build as native

    for flag in native.NVCC_FLAGS:
        if flag in ("-Xptxas", "-v", "-I") or os.path.isabs(flag):
            continue  # register report and include paths are the Python build's own
        assert f'"{flag}"' in build, flag
    assert "rustc-link-lib=dylib=katsu_cuda" in build


def test_manifest_names_the_crate_and_its_build_script():
    manifest = open(os.path.join(CRATE, "Cargo.toml")).read()
    assert 'name = "katsu-cuda"' in manifest and 'build = "build.rs"' in manifest
