"""CPU: the C-ABI library loads without a GPU and exports what include/sdq.h declares."""
import ctypes as C
import os
import re
import subprocess


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "sdq.h")).read()
    return sorted(set(re.findall(r"SDQ_API[^;(]*?\b(sdq_\w+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared()
    for must in ("sdq_qgemm", "sdq_quantize_activations", "sdq_qgemm_prequantized",
                 "sdq_quantize_rows", "sdq_pack_sdcpp", "sdq_pack_open", "sdq_weight_upload"):
        assert must in names
    assert len(names) >= 30


def test_library_exports_every_declared_symbol(pkg):
    lib = C.CDLL(pkg.lib_path())
    for name in declared():
        assert hasattr(lib, name), name
    out = subprocess.run(["nm", "-D", "--defined-only", pkg.lib_path()], capture_output=True, text=True).stdout
    exported = set(re.findall(r" T (sdq_\w+)", out))
    assert set(declared()) <= exported
    # nothing but the C ABI leaks out of the kernel library
    assert not re.findall(r" T (?!sdq_)\w+", out)


def test_binding_covers_every_symbol(pkg):
    assert sorted(pkg.sdq._SIGS) == declared()


def test_no_fallback_without_init(pkg):
    """Before sdq_init every compute entry point refuses: there is no CPU path behind the ABI."""
    code = (
        "import ctypes as C, sys\n"
        "lib = C.CDLL(sys.argv[1])\n"
        "lib.sdq_last_error.restype = C.c_char_p\n"
        "rc = lib.sdq_qgemm(C.c_uint64(1), None, C.c_int64(1), None, None, C.c_uint32(0), None)\n"
        "assert rc == 3, rc\n"
        "assert b'sdq_init' in lib.sdq_last_error()\n"
        "p = C.c_void_p()\n"
        "assert lib.sdq_pack_open(b'/nonexistent/x.sdcpp', 0, C.byref(p)) == 4\n"
        "assert lib.sdq_last_error() == b'sdcpp: cannot open /nonexistent/x.sdcpp'\n"
        "assert lib.sdq_device() == -1\n"
    )
    r = subprocess.run([os.sys.executable, "-c", code, pkg.lib_path()], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_pack_reader_runs_on_cpu(pkg, golden_dir):
    """The .sdcpp reader is host code: listing and error messages need no device."""
    import json
    gold = json.load(open(os.path.join(golden_dir, "golden.json")))
    lib = pkg.sdq.load_library()
    h = C.c_void_p()
    path = os.path.join(golden_dir, "tiny_model.sdcpp")
    assert lib.sdq_pack_open(path.encode(), 0, C.byref(h)) == 0
    n = lib.sdq_pack_count(h)
    assert n == gold["sdcpp_listing"]["count"]
    lines = []
    for i in range(n):
        e = pkg.sdq.Entry()
        assert lib.sdq_pack_entry(h, i, C.byref(e)) == 0
        dims = [str(e.dims[k]) for k in range(e.ndim)]
        lines.append("%s %d %d %s %d %d" % (C.string_at(e.name, e.name_len).decode(), e.dtype, e.ndim, ",".join(dims) or "-",
                                            e.file_offset, e.nbytes))
    assert "\n".join(sorted(lines)) + "\n" == gold["sdcpp_listing"]["listing"]
    assert lib.sdq_pack_close(h) == 0


def test_pack_reader_errors_match_reference(pkg, golden_dir, tmp_path):
    import json
    gold = json.load(open(os.path.join(golden_dir, "golden.json")))
    lib = pkg.sdq.load_library()
    good = open(os.path.join(golden_dir, "tiny_model.sdcpp"), "rb").read()
    cases = {"truncated_half": good[: len(good) // 2], "truncated_header": good[:40],
             "short": good[:10], "bad_magic": b"XDCP" + good[4:],
             "bad_version": good[:4] + (2).to_bytes(4, "little") + good[8:]}
    for tag, data in cases.items():
        p = tmp_path / tag
        p.write_bytes(data)
        h = C.c_void_p()
        assert lib.sdq_pack_open(str(p).encode(), 0, C.byref(h)) != 0, tag
        assert lib.sdq_last_error().decode() == gold["loader_errors"][tag].replace("<path>", str(p)), tag
    h = C.c_void_p()
    missing = str(tmp_path / "missing.sdcpp")
    assert lib.sdq_pack_open(missing.encode(), 0, C.byref(h)) != 0
    assert lib.sdq_last_error().decode() == "sdcpp: cannot open " + missing
