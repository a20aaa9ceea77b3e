"""The Rust crate's FFI declarations against ``include/dash_attn.h``.

The crate (``crates/dash-attn-b200``) cannot be compiled where this repository is built - there is no
Rust toolchain - so what can be held mechanically is held here: ``src/ffi.rs`` declares every function
the header declares and no other, with as many parameters; every ``#[repr(C)]`` struct lists the
header's fields in the header's order with types of the same size; the enum values agree; ``build.rs``
compiles every ``.cu`` file of the library; and ``src/lib.rs`` writes out all three methods of
``AttentionBackend`` (crates/dash-ops/src/attention.rs:289-352)."""
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "dash_attn.h").read_text()
CRATE = ROOT / "crates" / "dash-attn-b200"
FFI = (CRATE / "src" / "ffi.rs").read_text()

C_NO_COMMENTS = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
RUST_NO_COMMENTS = re.sub(r"//[^\n]*", "", FFI)

#: C type -> the Rust types of the same size and meaning
SAME = {
    "int32_t": {"i32"}, "int64_t": {"i64"}, "uint64_t": {"u64"}, "float": {"f32"}, "int": {"c_int", "i32"},
    "size_t": {"usize"}, "const void *": {"*const c_void"}, "void *": {"*mut c_void"},
    "const uint32_t *": {"*const u32"},
}


def c_functions():
    out = {}
    for ret, name, args in re.findall(r"([\w \*]+?)\b(dash_(?:attn|rope|sample)\w*)\s*\(([^;{]*?)\)\s*;", C_NO_COMMENTS):
        args = args.strip()
        out[name] = 0 if args in ("", "void") else len(args.split(","))
    return out


def rust_functions():
    block = RUST_NO_COMMENTS[RUST_NO_COMMENTS.index('extern "C"'):]
    out = {}
    for name, args in re.findall(r"pub fn (\w+)\s*\((.*?)\)\s*(?:->[^;]+)?;", block, flags=re.S):
        args = [a for a in args.split(",") if a.strip()]
        out[name] = len(args)
    return out


def c_struct(name):
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), C_NO_COMMENTS, flags=re.S).group(1)
    fields = []
    for decl in body.split(";"):
        decl = " ".join(decl.split())
        if not decl:
            continue
        m = re.match(r"((?:const )?\w+(?: \*)?)\s*(.*)", decl)
        ctype, names = m.group(1).strip(), m.group(2)
        for item in names.split(","):
            item = item.strip()
            pointer = item.startswith("*")
            item = item.lstrip("* ")
            arr = re.match(r"(\w+)\[(\d+)\]", item)
            t = ctype + (" *" if pointer and not ctype.endswith("*") else "")
            fields.append((arr.group(1), t, int(arr.group(2))) if arr else (item, t, 0))
    return fields


def rust_struct(name):
    body = re.search(r"#\[repr\(C\)\]\s*(?:#\[derive\([^\)]*\)\]\s*)?pub struct %s \{(.*?)\n\}" % name, RUST_NO_COMMENTS, flags=re.S).group(1)
    fields = []
    for fname, ftype in re.findall(r"pub (\w+):\s*([^,\n]+),", body):
        arr = re.match(r"\[(\w+); (\d+)\]", ftype.strip())
        fields.append((fname, arr.group(1), int(arr.group(2))) if arr else (fname, ftype.strip(), 0))
    return fields


def test_every_function_of_the_header_is_declared_with_as_many_parameters():
    c, rust = c_functions(), rust_functions()
    assert len(c) >= 19
    assert set(c) == set(rust), f"only in the header: {sorted(set(c) - set(rust))}; only in ffi.rs: {sorted(set(rust) - set(c))}"
    for name, n in c.items():
        assert rust[name] == n, f"{name}: {n} parameters in the header, {rust[name]} in ffi.rs"


def test_structs_are_repr_c_field_for_field():
    for name in ("dash_attn_params", "dash_attn_decode_params", "dash_rope_tables", "dash_rope_params", "dash_sample_params"):
        c, rust = c_struct(name), rust_struct(name)
        assert [f[0] for f in c] == [f[0] for f in rust], f"{name}: the fields or their order differ"
        for (fname, ctype, clen), (_, rtype, rlen) in zip(c, rust):
            assert clen == rlen, f"{name}.{fname}: array of {clen} in the header, {rlen} in ffi.rs"
            assert rtype in SAME[ctype], f"{name}.{fname}: {ctype} in the header, {rtype} in ffi.rs"


def test_constants_agree():
    for names in re.findall(r"enum \{(.*?)\};", C_NO_COMMENTS, flags=re.S):
        for name, value in re.findall(r"(DASH_ATTN_\w+) = (\d+)", names):
            if name == "DASH_ATTN_PROBE_COUNT":
                continue
            m = re.search(r"pub const %s: \w+ = (-?\d+);" % name, FFI)
            assert m and int(m.group(1)) == int(value), f"{name} = {value} in the header"


def test_build_rs_compiles_every_source_of_the_library():
    sources = sorted(p.name for p in (ROOT / "dashmag_b200" / "csrc").glob("*.cu"))
    listed = sorted(re.findall(r'"(\w+\.cu)"', (CRATE / "build.rs").read_text()))
    assert listed == sources
    assert "compute_100a" in (CRATE / "build.rs").read_text()


def test_lib_rs_writes_out_the_three_methods():
    lib = (CRATE / "src" / "lib.rs").read_text()
    assert "impl AttentionBackend for CubeBackend" in lib
    for method, call in (("attention_forward", "dash_attn_forward("), ("attention_backward", "dash_attn_backward("),
                         ("attention_decode", "dash_attn_decode(")):
        assert re.search(r"fn %s\(" % method, lib) and call in lib
    assert "reference::" not in lib, "no fallback to the reference on this path"
