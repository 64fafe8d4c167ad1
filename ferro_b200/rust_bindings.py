"""Writes the Rust `extern "C"` declarations for the whole C ABI from include/ferro_b200.h.

    python -m ferro_b200.rust_bindings > include/ferro_b200_sys.rs

ferro's host is Rust; the file this prints is what a maintainer drops into
crates/ferro-cuda/src/ (module `b200_sys`) to bind the library: `#[repr(C)]`
structs for the header's structs, opaque types for its handles, constants for
its enums and `#define`s of integers, and one `pub fn` per `FB_API` entry,
argument names kept.  The committed include/ferro_b200_sys.rs is checked
against this generator by tests/test_abi.py, so it cannot drift from the header.
"""
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADERS = [os.path.join(ROOT, "include", "ferro_b200_kinds.h"), os.path.join(ROOT, "include", "ferro_b200.h")]

SCALARS = {
    "int": "c_int", "float": "f32", "double": "f64", "char": "c_char", "void": "c_void",
    "uint64_t": "u64", "int64_t": "i64", "uint32_t": "u32", "int32_t": "i32", "uint16_t": "u16", "uint8_t": "u8",
    "size_t": "usize",
}


def strip_comments(text):
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def camel(name):
    name = name[3:] if name.startswith("fb_") else name
    return "".join(p.capitalize() for p in name.split("_"))


class Types:
    def __init__(self):
        self.structs = {}      # C name -> [(field, ctype, array_len or None)]
        self.opaque = []       # C names of handles
        self.fn_types = {}     # C name -> rust type text
        self.consts = []       # (name, value text)
        self.defines = {}      # integer #defines, for array lengths

    def rust_type(self, ctype):
        """'const float*' -> '*const f32' and so on."""
        t = " ".join(ctype.replace("*", " * ").split())
        if t in self.fn_types:
            return self.fn_types[t]
        if t == "fb_stream_t":
            return "Stream"
        toks = t.split()
        # read right to left: base [const] (* [const])*
        base_const = False
        while toks and toks[0] in ("const", "struct", "enum", "unsigned"):
            if toks[0] == "const":
                base_const = True
            toks = toks[1:]
        base, rest = toks[0], toks[1:]
        if rest and rest[0] == "const":
            base_const, rest = True, rest[1:]
        if base in SCALARS:
            r = SCALARS[base]
        elif base in self.structs or base in self.opaque:
            r = camel(base)
        elif base == "fb_stream_t":
            r = "Stream"
        else:
            raise ValueError(f"unknown C type {ctype!r}")
        const = base_const
        for tok in rest:
            if tok == "*":
                r = ("*const " if const else "*mut ") + r
                const = False
            elif tok == "const":
                const = True
            else:
                raise ValueError(f"cannot read {ctype!r}")
        return r


def parse(headers=HEADERS):
    ty = Types()
    fns = []
    for path in headers:
        text = strip_comments(open(path).read())
        for name, m in re.findall(r"^#define[ \t]+(FB_[A-Z0-9_]+)[ \t]+(\(?[ \t]*\d+u?[ \t]*(?:<<[ \t]*\d+)?[ \t]*\)?)[ \t]*$", text, flags=re.M):
            v = eval(m.replace("u", ""), {"__builtins__": {}})  # integer expressions such as (16u << 20)
            ty.defines[name] = int(v)
            ty.consts.append((name, str(int(v)), "u64" if int(v) > 0x7FFFFFFF else "c_int"))
        for body in re.findall(r"enum\s+\w+\s*\{(.*?)\}", text, flags=re.S):
            nxt = 0
            for item in body.split(","):
                item = item.strip()
                if not item:
                    continue
                if "=" in item:
                    n, v = [x.strip() for x in item.split("=")]
                    nxt = int(v, 0)
                else:
                    n = item
                ty.consts.append((n, str(nxt), "c_int"))
                nxt += 1
        for cname in re.findall(r"typedef\s+struct\s+(\w+)\s+\1\s*;", text):
            ty.opaque.append(cname)
        for ret, cname, args in re.findall(r"typedef\s+(\w[\w\s\*]*?)\(\s*\*\s*(\w+)\s*\)\s*\((.*?)\)\s*;", text, flags=re.S):
            ty.fn_types[cname] = (ret.strip(), args.strip())
        for cname, body in re.findall(r"typedef\s+struct\s+(\w+)\s*\{(.*?)\}\s*\1\s*;", text, flags=re.S):
            fields = []
            for decl in body.split(";"):
                decl = " ".join(decl.split())
                if not decl:
                    continue
                m = re.match(r"(.+?)\s*((?:\w+(?:\[\w+\])?\s*,\s*)*\w+(?:\[\w+\])?)$", decl)
                ctype, names = m.group(1), m.group(2)
                for nm in names.split(","):
                    nm = nm.strip()
                    arr = None
                    am = re.match(r"(\w+)\[(\w+)\]", nm)
                    if am:
                        nm, arr = am.group(1), am.group(2)
                        arr = ty.defines.get(arr, arr)
                    fields.append((nm, ctype, arr))
            ty.structs[cname] = fields
        for ret, name, args in re.findall(r"FB_API\s+([\w\s\*]+?)\b(fb_\w+)\s*\((.*?)\)\s*;", text, flags=re.S):
            params = []
            args = " ".join(args.split())
            if args and args != "void":
                for a in args.split(","):
                    a = a.strip()
                    m = re.match(r"(.+?)(\w+)$", a)
                    params.append((m.group(2), m.group(1).strip()))
            if all(name != f[0] for f in fns):
                fns.append((name, ret.strip(), params))
    # function pointer typedefs -> rust text (needs the other types first)
    for cname, (ret, args) in list(ty.fn_types.items()):
        ps = []
        for a in [x.strip() for x in args.split(",") if x.strip() and x.strip() != "void"]:
            m = re.match(r"(.+?)(\w+)$", a)
            ps.append(f"{m.group(2)}: {Types.rust_type(ty, m.group(1).strip())}")
        r = "" if ret == "void" else f" -> {Types.rust_type(ty, ret)}"
        ty.fn_types[cname] = f"Option<unsafe extern \"C\" fn({', '.join(ps)}){r}>"
    return ty, fns


RUST_KEYWORDS = {"type", "ref", "fn", "in", "move", "box", "loop", "match", "impl", "mod", "use", "as", "dyn", "where"}


def generate():
    ty, fns = parse()
    out = []
    w = out.append
    w("// Raw bindings to libferro_b200.so: one declaration per entry of include/ferro_b200.h.")
    w("// Generated by `python -m ferro_b200.rust_bindings`; do not edit by hand.")
    w("#![allow(non_camel_case_types, dead_code)]")
    w("use std::os::raw::{c_char, c_int, c_void};")
    w("")
    w("/// cudaStream_t (cudarc: `stream.cu_stream()` cast to this).")
    w("pub type Stream = *mut c_void;")
    w("")
    for name, val, t in ty.consts:
        w(f"pub const {name}: {t} = {val};")
    w("")
    for cname in ty.opaque:
        w(f"/// Opaque handle (`{cname}`).")
        w(f"#[repr(C)] pub struct {camel(cname)} {{ _private: [u8; 0] }}")
    w("")
    for cname, rust in ty.fn_types.items():
        w(f"pub type {camel(cname)} = {rust};")
    ty.fn_types = {k: camel(k) for k in ty.fn_types}
    w("")
    for cname, fields in ty.structs.items():
        w("#[repr(C)] #[derive(Clone, Copy)]")
        w(f"pub struct {camel(cname)} {{")
        for nm, ctype, arr in fields:
            rt = ty.rust_type(ctype)
            if arr is not None:
                rt = f"[{rt}; {arr}]"
            nm = f"r#{nm}" if nm in RUST_KEYWORDS else nm
            w(f"    pub {nm}: {rt},")
        w("}")
    w("")
    w('#[link(name = "ferro_b200")]')
    w('extern "C" {')
    for name, ret, params in fns:
        ps = ", ".join(f"{('r#' + n) if n in RUST_KEYWORDS else n}: {ty.rust_type(t)}" for n, t in params)
        r = "" if ret == "void" else f" -> {ty.rust_type(ret)}"
        w(f"    pub fn {name}({ps}){r};")
    w("}")
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    sys.stdout.write(generate())
