"""The Rust side of the boundary (bindings/rust) cannot be compiled in this image; what can be checked without a
Rust toolchain is that its `extern "C"` block IS the header: src/backend/cuda/ffi.rs is generated from
include/sage_cuda.h, must be up to date, must declare every function the library exports from that header with the
same number of arguments, and the safe wrappers may only call functions that exist."""
import os
import re
import subprocess
import sys

import sage_b200 as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUST = os.path.join(ROOT, "bindings", "rust")


def header_functions():
    text = open(os.path.join(ROOT, "include", "sage_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(sage_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.S):
        args = " ".join(m.group(2).split())
        out[m.group(1)] = 0 if args in ("", "void") else len(args.split(","))
    return out


def test_ffi_block_is_generated_from_the_header_and_up_to_date():
    assert subprocess.call([sys.executable, os.path.join(RUST, "gen_ffi.py"), "--check"]) == 0, \
        "bindings/rust/src/backend/cuda/ffi.rs is stale: run python bindings/rust/gen_ffi.py"


def test_ffi_declares_every_exported_function_with_the_same_arity():
    hdr = header_functions()
    ffi = open(os.path.join(RUST, "src", "backend", "cuda", "ffi.rs")).read()
    decl = {m.group(1): (0 if not m.group(2).strip() else len(m.group(2).split(","))) for m in re.finditer(r"pub fn (sage_\w+)\(([^)]*)\)", ffi)}
    assert len(hdr) >= 50 and set(decl) == set(hdr), sorted(set(hdr) ^ set(decl))
    assert all(decl[k] == hdr[k] for k in hdr), [k for k in hdr if decl[k] != hdr[k]]
    assert all(hasattr(S.lib, k) for k in decl)          # ... and the library really exports them


def test_safe_wrappers_only_call_declared_functions_and_cover_the_trait():
    mod = open(os.path.join(RUST, "src", "backend", "cuda", "mod.rs")).read()
    trait = open(os.path.join(RUST, "src", "backend.rs")).read()
    called = set(re.findall(r"\b(sage_[a-z0-9_]+)\(", mod))
    assert called and called <= set(header_functions()), sorted(called - set(header_functions()))
    # every method the trait requires is implemented by CudaBackend
    required = set(re.findall(r"^\s*fn (\w+)\(", trait[trait.index("pub trait Backend"):], flags=re.M))
    implemented = set(re.findall(r"^\s*fn (\w+)\(", mod[mod.index("impl Backend for CudaBackend"):], flags=re.M))
    assert required and required <= implemented, sorted(required - implemented)
    # the op-level entry points a compute() needs are all reachable from the wrappers
    for name in ("sage_map", "sage_reduce", "sage_reduce_arg", "sage_gather", "sage_scatter", "sage_unslice", "sage_concat",
                 "sage_gemm_strided_batched", "sage_im2col", "sage_col2im", "sage_softmax", "sage_log_sum_exp", "sage_layer_norm",
                 "sage_pool2d", "sage_conv2d_nhwc", "sage_alloc", "sage_free", "sage_upload", "sage_download", "sage_memset",
                 "sage_module_get", "sage_launch", "sage_last_oom"):
        assert name in called, name
