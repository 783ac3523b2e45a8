"""CPU: every reference-named export in include/ubridge_b200.h has the argument list the reference's Rust side
declares for it (src/ffi.rs, src/eccllib.rs): same count, same order, same names, same kind of type.  All-int32
argument runs link whatever their order, so the NAMES are what catches a permutation."""
import importlib.util
import json
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "ffi_signatures.json")
REFERENCE = os.environ.get("UB_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))  # a checkout of Ubridge, if any


def _c_kind(t: str) -> str:
    t = t.strip()
    if "*" in t or t.endswith("_t") and t.startswith("ecclComm"):
        return "ptr"
    if t in ("size_t",):
        return "size"
    if t in ("float", "double"):
        return "float"
    if t in ("uint32_t", "unsigned", "unsigned int"):
        return "uint"
    if t in ("int", "int32_t", "int64_t", "long"):
        return "int"
    return t


def _header_decls():
    hdr = open(os.path.join(ROOT, "include", "ubridge_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    out = {}
    for m in re.finditer(r"^\s*([A-Za-z_][\w\s\*]*?)\b(\w+)\s*\(([^;{}]*)\)\s*;", hdr, flags=re.M):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        items = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                mm = re.match(r"^(.*?)(\w+)$", a)
                items.append((mm.group(2), mm.group(1).strip()))
        out[name] = (ret, items)
    return out


def _load():
    return json.load(open(GOLDEN))


def test_fixture_is_current_when_the_reference_is_present():
    if not os.path.isdir(REFERENCE):
        pytest.skip("reference checkout not on this machine; the committed fixture stands")
    spec = importlib.util.spec_from_file_location("mk", os.path.join(ROOT, "tests", "golden", "make_ffi_signatures.py"))
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    assert mk.extract(REFERENCE) == _load()


def test_every_reference_named_export_matches_ffi_rs():
    ref = _load()["ffi"]
    decls = _header_decls()
    assert len(ref) == 17
    for name, sig in sorted(ref.items()):
        assert name in decls, "reference FFI function missing from the header: " + name
        ret, items = decls[name]
        want = sig["args"]
        assert len(items) == len(want), "%s: %d arguments, the reference declares %d" % (name, len(items), len(want))
        for i, ((hname, htype), (rname, rkind)) in enumerate(zip(items, want)):
            assert hname.lower() == rname.lower(), "%s: argument %d is `%s`, the reference has `%s`" % (name, i, hname, rname)
            assert _c_kind(htype) == rkind, "%s: argument %d (%s) is %s, the reference has %s" % (name, i, hname, htype, rkind)
        assert ("void" if ret == "void" else _c_kind(ret)) == sig["ret"], name


def test_eccl_exports_keep_the_call_sites_argument_order():
    ref = _load()["eccl"]
    decls = _header_decls()
    assert len(ref) == 18
    alias = {"uniqueid": "id", "comm_id": "id"}
    for name, want in sorted(ref.items()):
        assert name in decls, name
        got = [n for n, _ in decls[name][1]]
        want = [alias.get(w, w) for w in want]
        assert [g.lower() for g in got] == want, "%s: %s vs the reference's call site %s" % (name, got, want)
