#!/usr/bin/env python
"""Regenerates the `extern "C"` block of src/lib.rs (and its copy in INTEGRATION.md) from include/b200tile.h.

    python rust/b200tile-sys/gen_ffi.py            # rewrites src/lib.rs in place
    python rust/b200tile-sys/gen_ffi.py --check    # exit 1 when src/lib.rs is out of date (used by the tests)
"""
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "..", "include", "b200tile.h")
LIB_RS = os.path.join(HERE, "src", "lib.rs")
INTEGRATION = os.path.join(HERE, "..", "..", "INTEGRATION.md")   # carries a copy of the block for readers
BEGIN, END = "// --- generated: begin ---\n", "// --- generated: end ---\n"

TYPES = {"int": "c_int", "unsigned": "c_uint", "float": "f32", "double": "f64", "uint64_t": "u64", "int64_t": "i64",
         "uint32_t": "u32", "int32_t": "i32", "void": "c_void", "char": "c_char", "b200tile_config": "B200Config",
         "b200tile_status_t": "B200Status", "b200tile_compile_options": "B200CompileOptions"}


def rust_type(c: str) -> str:
    toks = c.replace("*", " * ").split()
    const = "const" in toks
    toks = [t for t in toks if t != "const"]
    stars = toks.count("*")
    base = TYPES[" ".join(t for t in toks if t != "*")]
    for _ in range(stars):
        base = ("*const " if const else "*mut ") + base
    return base


def declarations():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#define\s+B200TILE_API[^\n]*", "", text)
    for d in re.findall(r"B200TILE_API\s+([^;]+?);", text, flags=re.S):
        d = " ".join(d.split())
        m = re.match(r"(.+?)\s*\b(b200tile_\w+)\s*\((.*)\)$", d)
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        out = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                arr = re.match(r"(.+?)\s+(\w+)\[(\d*)\]$", a)
                if arr:
                    out.append(f"{arr.group(2)}: {rust_type(arr.group(1) + ' *')}")
                    continue
                mm = re.match(r"(.*?)(\w+)$", a)
                ty, nm = mm.group(1), mm.group(2)
                squeezed = ty.replace(" ", "")
                if squeezed == "constchar*const*":
                    out.append(f"{nm}: *const *const c_char")
                elif squeezed == "constvoid*const*":
                    out.append(f"{nm}: *const *const c_void")
                else:
                    out.append(f"{nm}: {rust_type(ty)}")
        yield name, out, "" if ret == "void" else " -> " + rust_type(ret)


def render() -> str:
    lines = []
    for name, args, ret in declarations():
        cur, parts = f"    pub fn {name}(", []
        for i, a in enumerate(args):
            piece = a + (", " if i < len(args) - 1 else "")
            if len(cur) + len(piece) > 108:
                parts.append(cur.rstrip())
                cur = " " * 8 + piece
            else:
                cur += piece
        parts.append(cur + f"){ret};")
        lines.append("\n".join(parts))
    return "\n".join(lines) + "\n"


def main() -> int:
    stale = 0
    for path in (LIB_RS, INTEGRATION):
        src = open(path).read()
        a, b = src.index(BEGIN) + len(BEGIN), src.index(END)
        new = src[:a] + render() + src[b:]
        if "--check" in sys.argv:
            stale |= int(new != src)
        else:
            open(path, "w").write(new)
    return stale


if __name__ == "__main__":
    sys.exit(main())
