"""The `qlora-cuda` Rust crate (the drop-in sibling of the reference's `qlora-wgpu`) cannot be compiled here
(no Rust toolchain), so its contract with the C ABI is checked as text: every function in the crate's
`extern "C"` block must be declared in include/qlora_cuda.h with the same number of arguments, every status
and mode constant must have the header's value, and the crate must export the items `qlora-wgpu` exports
(qlora-wgpu/src/lib.rs:25-32)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _strip_c_comments(text):
    return re.sub(r"/\*.*?\*/", "", text, flags=re.S)


def _header_functions():
    text = _strip_c_comments(open(os.path.join(ROOT, "include", "qlora_cuda.h")).read())
    out = {}
    for m in re.finditer(r"\b(qlc_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if args in ("", "void") else args.count(",") + 1
    return out


def _rust_extern_functions():
    text = open(os.path.join(ROOT, "qlora-cuda", "src", "ffi.rs")).read()
    text = re.sub(r"//.*", "", text)
    block = re.search(r'extern "C" \{(.*)\n\}', text, flags=re.S).group(1)
    out = {}
    for m in re.finditer(r"pub fn (\w+)\s*\((.*?)\)\s*(?:->\s*[^;]+)?;", block, flags=re.S):
        args = [a for a in m.group(2).split(",") if a.strip()]
        out[m.group(1)] = len(args)
    return out


def test_every_extern_is_a_header_symbol_with_the_same_arity():
    hdr, rs = _header_functions(), _rust_extern_functions()
    assert len(rs) >= 25
    for name, n in rs.items():
        assert name in hdr, f"{name} is bound in qlora-cuda/src/ffi.rs but not declared in include/qlora_cuda.h"
        assert hdr[name] == n, f"{name}: header takes {hdr[name]} arguments, ffi.rs passes {n}"


def test_constants_match_the_header():
    hdr = open(os.path.join(ROOT, "include", "qlora_cuda.h")).read()
    rs = open(os.path.join(ROOT, "qlora-cuda", "src", "ffi.rs")).read()
    consts = dict(re.findall(r"pub const (QLC_\w+): c_int = (\d+);", rs))
    assert len(consts) >= 10
    for name, val in consts.items():
        m = re.search(rf"#define {name} (\d+)", hdr)
        assert m and m.group(1) == val, name


def test_crate_exports_what_qlora_wgpu_exports():
    lib = open(os.path.join(ROOT, "qlora-cuda", "src", "lib.rs")).read()
    for item in ("GpuContext", "gpu_dequantize", "gpu_matmul", "gpu_matmul_trans_a", "gpu_matmul_trans_b",
                 "gpu_qlora_backward", "gpu_qlora_forward"):
        assert re.search(rf"pub use [^;]*\b{item}\b", lib, flags=re.S), item
    ctx = open(os.path.join(ROOT, "qlora-cuda", "src", "context.rs")).read()
    assert "pub fn try_new_blocking() -> Result<Option<Self>, QloraError>" in ctx
    assert "impl Drop for GpuContext" in ctx
    kern = open(os.path.join(ROOT, "qlora-cuda", "src", "kernels.rs")).read()
    assert "ctx: Option<&GpuContext>" in kern and "Result<QloraGrads, QloraError>" in kern
