"""Prints the Rust `extern "C"` block for every prototype of mx230_attn.h.

    python include/gen_rust_extern.py > mx230_sys.rs

Pointer arguments keep their C element type (`*const f32`, `*mut i8`, ...); a cudarc `CUdeviceptr` (u64) is
passed with `as *const f32` / `as *mut f32`.  Opaque structs become zero-sized `#[repr(C)]` types.
"""
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SCALAR = {"int": "c_int", "float": "f32", "size_t": "usize", "long long": "c_longlong", "uint64_t": "u64",
          "uint32_t": "u32", "unsigned char": "u8", "int8_t": "i8", "char": "c_char", "void": "c_void",
          "unsigned int": "c_uint", "double": "f64", "uint16_t": "u16", "int32_t": "i32", "int64_t": "i64"}
OPAQUE = {"mx230_handle": "Mx230Handle", "mx230_kv_pool": "Mx230KvPool", "mx230_sched": "Mx230Sched",
          "mx230_splitkv_comm": "Mx230SplitKvComm"}


def rust_type(c: str) -> str:
    c = " ".join(c.split())
    stars = c.count("*")
    base = c.replace("*", " ")
    const = bool(re.search(r"\bconst\b", base))
    base = " ".join(w for w in base.split() if w != "const")
    t = OPAQUE.get(base) or SCALAR.get(base)
    if t is None:
        raise SystemExit(f"unmapped C type {c!r}")
    for i in range(stars):
        t = ("*const " if const and i == 0 else "*mut ") + t
    return t


def main(header: str) -> None:
    text = re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)
    for m in re.finditer(r"typedef struct (\w+) \1;", text):
        OPAQUE.setdefault(m.group(1), "".join(p.capitalize() for p in m.group(1).split("_")))
    print("// Generated from mx230_attn.h by gen_rust_extern.py; link with `-l dylib=mx230_attn`.")
    print("#![allow(non_camel_case_types, dead_code)]")
    print("use std::ffi::{c_char, c_int, c_longlong, c_uint, c_void};")
    for name in sorted(set(OPAQUE.values())):
        print(f"#[repr(C)] pub struct {name} {{ _p: [u8; 0] }}")
    print('extern "C" {')
    for m in re.finditer(r"\n((?:const\s+)?[\w ]+?[\s\*]+)(mx230_\w+)\s*\(([^;{]*?)\)\s*;", text):
        ret, name, args = " ".join(m.group(1).split()), m.group(2), m.group(3)
        parts = []
        for a in args.split(","):
            a = " ".join(a.split())
            if a in ("void", ""):
                continue
            mm = re.match(r"(.*?)(\w+)$", a)
            arg = mm.group(2)
            parts.append(f"{'r#' if arg in ('type', 'ref', 'in', 'loop', 'move') else ''}{arg}: {rust_type(mm.group(1))}")
        r = "" if ret == "void" else f" -> {rust_type(ret)}"
        line = f"    pub fn {name}({', '.join(parts)}){r};"
        if len(line) > 118:   # wrap long prototypes, several arguments per line
            rows, cur = [], "       "
            for p_ in parts:
                if len(cur) + len(p_) + 2 > 116:
                    rows.append(cur.rstrip())
                    cur = "       "
                cur += " " + p_ + ","
            rows.append(cur.rstrip())
            line = f"    pub fn {name}(\n" + "\n".join(rows) + f"\n    ){r};"
        print(line)
    print("}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "mx230_attn.h"))
