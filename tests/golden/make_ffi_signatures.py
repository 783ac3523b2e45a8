"""Extracts the argument lists of the reference's FFI declarations into ``ffi_signatures.json``.

    python tests/golden/make_ffi_signatures.py [path-to-the-reference-checkout]

Sources read (text only, nothing is compiled or run):
  * ``src/ffi.rs``      every ``pub fn name(arg: type, ...) [-> ret];`` inside the ``extern "C"`` blocks;
  * ``src/eccllib.rs``  the argument order of every ``lib().ecclXxx(...)`` call (the vendor binding itself is an
                        external crate; the call sites fix the order).
Output: {"ffi": {name: {"args": [[arg_name, kind], ...], "ret": kind}}, "eccl": {name: [arg_name, ...]}} with kind one
of ptr / int / uint / float / size.  ``tests/test_ffi_signatures.py`` checks ``include/ubridge_b200.h`` against it.
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

# the declarations on the quantized-linear / fused-MoE path (the rest of ffi.rs is out of scope)
ON_PATH = re.compile(r"^(moe_(f16|bf16)|indexed_moe_(f16|bf16)|dequant_(f16|bf16)|moe_align_block_size|"
                     r"invoke_fused_moe_(f16|bf16)|topk_softmax_(f32|f16|bf16)|topsaten_topk_softmax_f32|"
                     r"topsaten_moe_align_block_size|topsaten_fused_moe_gemm|topsaten_release_graph_workspace_pool|"
                     r"topsaten_rms_norm)$")


def rust_kind(t: str) -> str:
    t = t.strip()
    if t.startswith("*"):
        return "ptr"
    if t in ("c_int", "i32", "::core::ffi::c_int", "c_long", "i64"):
        return "int"
    if t in ("u32", "c_uint", "u64"):
        return "uint"
    if t in ("f32", "f64", "c_float"):
        return "float"
    if t in ("usize", "size_t"):
        return "size"
    if t.endswith("Stream_t"):
        return "ptr"
    return t


def parse_ffi(text: str) -> dict:
    out = {}
    for m in re.finditer(r"pub fn (\w+)\s*\((.*?)\)\s*(?:->\s*([\w:]+))?\s*;", text, flags=re.S):
        name, args, ret = m.group(1), m.group(2), m.group(3)
        items = []
        args = re.sub(r"//[^\n]*", "", args)
        for a in args.split(","):
            a = a.strip()
            if not a or ":" not in a:
                continue
            an, at = a.split(":", 1)
            items.append([an.strip(), rust_kind(at)])
        out[name] = {"args": items, "ret": rust_kind(ret) if ret else "void"}
    return out


def parse_eccl(text: str) -> dict:
    out = {}
    for m in re.finditer(r"\.\s*(eccl\w+)\s*\((.*?)\)", text, flags=re.S):
        names = [re.sub(r"[&\s]|mut\b|\.as_mut_ptr\(\)?", "", a).strip() for a in m.group(2).split(",") if a.strip()]
        out[m.group(1)] = names
    return out


def extract(ref_root: str) -> dict:
    ffi = {k: v for k, v in parse_ffi(open(os.path.join(ref_root, "src", "ffi.rs")).read()).items() if ON_PATH.match(k)}
    eccl = parse_eccl(open(os.path.join(ref_root, "src", "eccllib.rs")).read())
    return {"ffi": ffi, "eccl": eccl}


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_ffi_signatures.py <path of an Ubridge checkout>")
    root = sys.argv[1]
    data = extract(root)
    with open(os.path.join(HERE, "ffi_signatures.json"), "w") as f:
        json.dump(data, f, indent=1, sort_keys=True)
    print("%d ffi declarations, %d eccl call sites" % (len(data["ffi"]), len(data["eccl"])))
