"""CPU tests of the boundary: the library loads, exports every symbol the header declares, and
refuses contract violations with the reference's messages — no compute, no GPU."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "mummu_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mummu_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(cuda_lib):
    names = header_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(cuda_lib.lib, name), f"{name} declared in mummu_cuda.h but not exported"
    assert set(names) == set(cuda_lib.SYMBOLS), "ctypes table and header disagree"
    assert b"sm_100a" in cuda_lib.lib.mummu_cuda_version()


def test_config_contract_messages(cuda_lib):
    """nn/moe.rs:62-76 and the should_panic tests at :2354-2374."""
    from mummu_b200 import moe
    with pytest.raises(moe.MoeContractError, match="num_experts_per_tok"):
        moe.SparseMoeConfig(4, 3, 4, 0).init()
    with pytest.raises(moe.MoeContractError, match="num_experts_per_tok"):
        moe.SparseMoeConfig(4, 3, 4, 5).init()
    with pytest.raises(moe.MoeContractError, match="num_experts must be >= 2"):
        moe.SparseMoeConfig(4, 3, 1, 1).init()
    with pytest.raises(moe.MoeContractError, match="hidden_size and expert_intermediate_size"):
        moe.SparseMoeConfig(0, 3, 4, 2).init()
    with pytest.raises(moe.MoeContractError, match="256-value super-blocks"):
        moe.SparseMoeConfig(100, 256, 4, 2).init(weight_dtype=cuda_lib.Q4_K, act_dtype=cuda_lib.F16)


def test_null_handle_is_refused_not_crashed(cuda_lib):
    rc = cuda_lib.lib.mummu_moe_forward(None, None, None, 1, 1, 0, 0, None)
    assert rc == cuda_lib.ERR_CONTRACT
    assert "null" in cuda_lib.last_error()
    assert cuda_lib.lib.mummu_moe_destroy(None) == cuda_lib.OK


def test_rust_crate_binds_every_declared_symbol_and_builds_every_source():
    """crates/mummu-cuda is not compiled on this image (no Rust toolchain), so it is kept in step
    by text: its `extern "C"` block names exactly the header's functions, and its build script
    compiles exactly the sources the Python build compiles."""
    from mummu_b200 import build
    lib_rs = open(os.path.join(ROOT, "crates", "mummu-cuda", "src", "lib.rs")).read()
    block = lib_rs[lib_rs.index('extern "C" {'):]
    block = block[:block.index("\n    }\n")]
    bound = sorted(set(re.findall(r"pub fn (mummu_[a-z0-9_]+)\s*\(", block)))
    assert bound == header_symbols()
    build_rs = open(os.path.join(ROOT, "crates", "mummu-cuda", "build.rs")).read()
    listed = re.findall(r'"([a-z0-9_]+\.cu)"', build_rs[build_rs.index("const SOURCES"):build_rs.index("];")])
    assert sorted(listed) == sorted(build.SOURCES)


def _top_level_args(arglist: str) -> int:
    arglist = arglist.strip()
    if arglist in ("", "void"):
        return 0
    depth, n = 0, 1
    for ch in arglist:
        depth += ch in "([<"
        depth -= ch in ")]>"
        n += ch == "," and depth == 0
    return n


def test_argument_counts_agree_between_header_ctypes_and_rust(cuda_lib):
    """Names alone do not catch a parameter added on one side only: the number of parameters of
    every export must be the same in the header, in the ctypes table and in the Rust `extern "C"`
    block, and every call of a `sys::` function in the crate must pass that many arguments."""
    header = open(os.path.join(ROOT, "include", "mummu_cuda.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    h_counts = {m.group(1): _top_level_args(m.group(2))
                for m in re.finditer(r"\b(mummu_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", header, flags=re.S)}
    assert set(h_counts) == set(cuda_lib.SYMBOLS)
    for name, (_, argtypes) in cuda_lib.SYMBOLS.items():
        assert len(argtypes) == h_counts[name], f"{name}: ctypes has {len(argtypes)} parameters, the header {h_counts[name]}"
    lib_rs = open(os.path.join(ROOT, "crates", "mummu-cuda", "src", "lib.rs")).read()
    block = lib_rs[lib_rs.index('extern "C" {'):]
    block = block[:block.index("\n    }\n")]
    r_counts = {m.group(1): _top_level_args(m.group(2))
                for m in re.finditer(r"pub fn (mummu_[a-z0-9_]+)\s*\((.*?)\)\s*(?:->[^;]*)?;", block, flags=re.S)}
    assert r_counts == h_counts
    rest = lib_rs[lib_rs.index('extern "C" {') + len(block):]
    rest = "\n".join(line for line in rest.splitlines() if not line.lstrip().startswith("//"))
    calls = 0
    for m in re.finditer(r"sys::(mummu_[a-z0-9_]+)\s*\(", rest):
        depth, i = 1, m.end()
        while depth:
            depth += rest[i] in "([{"
            depth -= rest[i] in ")]}"
            i += 1
        got = _top_level_args(rest[m.end():i - 1])
        assert got == h_counts[m.group(1)], f"a call of {m.group(1)} in lib.rs passes {got} arguments, it takes {h_counts[m.group(1)]}"
        calls += 1
    assert calls >= 20
