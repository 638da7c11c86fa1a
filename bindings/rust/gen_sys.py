"""Writes frink-b200-sys/src/lib.rs from include/frink_b200.h: one `extern "C"` declaration per entry point, in the
header's order and with its argument names.  Run from the repository root after the header changes:

    python bindings/rust/gen_sys.py
"""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
TYPES = {"int": "c_int", "float": "f32", "size_t": "usize", "uint64_t": "u64", "int32_t": "i32", "uint8_t": "u8", "char": "c_char", "void": "c_void",
         "fk_ctx": "FkCtx", "fk_comm": "FkComm", "fk_matvec_launch": "FkMatvecLaunch"}

HEAD = '''//! Raw declarations of `libfrink_b200.so`'s C ABI, one per entry point of `include/frink_b200.h`, in the
//! header's order and with the header's argument names (written by `bindings/rust/gen_sys.py`).  Semantics,
//! units and the frink interface each call replaces are documented in the header; nothing here adds behaviour.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_int, c_void};

/// Opaque context (`fk_ctx`): one per device, created by `fk_init`.
#[repr(C)]
pub struct FkCtx {
    _private: [u8; 0],
}
/// Opaque resident weights (`struct fk_weight_s`).
#[repr(C)]
pub struct FkWeightS {
    _private: [u8; 0],
}
pub type FkWeight = *mut FkWeightS;
/// Opaque peer-memory communicator (`fk_comm`).
#[repr(C)]
pub struct FkComm {
    _private: [u8; 0],
}
/// `fk_matvec_launch`: one matvec of a multi-matvec call.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct FkMatvecLaunch {
    pub kind: c_int,
    pub weights_host: *const u8,
    pub len: usize,
    pub rows: c_int,
    pub row_bytes: c_int,
    pub n_blocks_per_row: c_int,
}

/// `fk_status`.
pub const FK_OK: c_int = 0;
pub const FK_DRIVER_INIT: c_int = 1;
pub const FK_KERNEL: c_int = 2;
pub const FK_LAUNCH: c_int = 3;
pub const FK_UNSUPPORTED: c_int = 4;
pub const FK_COMM: c_int = 5;
pub const FK_INVALID: c_int = 6;

/// GGML type tags the library has kernels for.
pub const FK_Q8_0: c_int = 8;
pub const FK_Q4_K: c_int = 12;
pub const FK_Q5_K: c_int = 13;
pub const FK_Q6_K: c_int = 14;
pub const FK_MXFP4: c_int = 39;

extern "C" {
'''


def rust_type(t):
    t = t.strip()
    if re.fullmatch(r"\w+\s*\*\s*const\s*\*", t):              # T* const* : an array of pointers
        return "*const *mut " + TYPES[t.split("*")[0].strip()]
    ptr, const = t.count("*"), t.startswith("const ")
    base = t.replace("const", "").replace("*", "").strip()
    r = "FkWeight" if base == "fk_weight" else TYPES[base]
    for lvl in range(ptr):
        r = ("*const " if (const and lvl == 0) else "*mut ") + r
    return r


def main():
    h = open(os.path.join(ROOT, "include", "frink_b200.h")).read()
    h = re.sub(r"/\*.*?\*/", "", h, flags=re.S)
    h = re.sub(r"typedef struct fk_matvec_launch \{.*?\} fk_matvec_launch;", "", h, flags=re.S)
    decls = re.findall(r"\n((?:int|void|size_t|const char\*)\s+fk_\w+\s*\([^;]*\));", h)
    out = []
    for d in decls:
        ret, name, args = re.match(r"(.*?)\s*(fk_\w+)\s*\((.*)\)$", " ".join(d.split())).groups()
        al = []
        if args.strip() != "void":
            for a in args.split(","):
                ty, nm = re.match(r"(.*?)(\w+)$", a.strip()).groups()
                al.append(f"{nm}: {rust_type(ty)}")
        r = "" if ret.strip() == "void" else " -> " + rust_type(ret)
        line = f"    pub fn {name}({', '.join(al)}){r};"
        if len(line) > 118:
            line = f"    pub fn {name}(\n" + "".join(f"        {p},\n" for p in al) + f"    ){r};"
        out.append(line)
    path = os.path.join(ROOT, "bindings", "rust", "frink-b200-sys", "src", "lib.rs")
    open(path, "w").write(HEAD + "\n".join(out) + "\n}\n")
    print(len(out), "functions ->", path)


if __name__ == "__main__":
    main()
