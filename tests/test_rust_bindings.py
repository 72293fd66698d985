"""The Rust side of the boundary is shipped as source (rust/vfkv-sys, rust/backend_cuda) and is
not compiled here: no Rust toolchain in this image.  What can be checked without one: every
function include/*.h declares is declared in rust/vfkv-sys/src/lib.rs with the same number of
arguments, the file is what its generator writes today, and the backend module only calls
functions that exist."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_RS = os.path.join(ROOT, "rust", "vfkv-sys", "src", "lib.rs")


def header_functions():
    fns = {}
    for header in ("vfkv.h", "vfkv_next.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"#[^\n]*", "", text)
        for m in re.finditer(r"\b(vfkv_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*;", text):
            args = m.group(2).strip()
            fns[m.group(1)] = 0 if args in ("", "void") else len(args.split(","))
    return fns


def rust_functions():
    text = open(LIB_RS).read()
    fns = {}
    for m in re.finditer(r"pub fn (vfkv_[a-z0-9_]+)\(([^)]*)\)", text):
        args = m.group(2).strip()
        fns[m.group(1)] = 0 if not args else len(args.split(","))
    return fns


def test_every_header_function_is_declared_in_rust_with_the_same_arity():
    c, r = header_functions(), rust_functions()
    assert len(c) >= 100
    assert sorted(c) == sorted(r), set(c) ^ set(r)
    assert {n: c[n] for n in c if c[n] != r[n]} == {}


def test_lib_rs_is_what_the_generator_writes(tmp_path):
    before = open(LIB_RS).read()
    subprocess.run([sys.executable, os.path.join(ROOT, "rust", "vfkv-sys", "gen_bindings.py")], check=True,
                   capture_output=True)
    assert open(LIB_RS).read() == before


def test_backend_module_calls_only_declared_functions():
    declared = rust_functions()
    for name in ("mod.rs", "kv_cache.rs"):
        text = open(os.path.join(ROOT, "rust", "backend_cuda", name)).read()
        used = set(re.findall(r"sys::(vfkv_[a-z0-9_]+)\(", text))
        assert used and used <= set(declared), used - set(declared)
        for fn in used:                     # argument counts of the calls, one argument per top-level comma
            for m in re.finditer(r"sys::" + fn + r"\(", text):
                depth, i, n, seen = 1, m.end(), 0, False
                while depth:
                    ch = text[i]
                    if ch in "([{":
                        depth += 1
                    elif ch in ")]}":
                        depth -= 1
                    elif ch == "," and depth == 1:
                        n += 1
                        seen = False
                        i += 1
                        continue
                    if depth and not ch.isspace():
                        seen = True
                    i += 1
                n_args = n + (1 if seen else 0)
                assert n_args == declared[fn], (name, fn, n_args, declared[fn])
