"""CPU: differential fuzzing of the .sdcpp reader.

Random damage to a valid pack (byte flips in the header, truncations, spliced garbage): the
C reader (sdq_pack_open), the numpy restatement (oracle.pack_oracle.parse) and -- where
oracle/_ref is present -- the reference's own loader must agree on accept/reject, on the
error text, and on the listing of an accepted file.  The reader is host code: no GPU needed."""
import ctypes as C
import os

import numpy as np

from oracle import pack_oracle


def _ours(lib, Entry, path):
    h = C.c_void_p()
    rc = lib.sdq_pack_open(path.encode(), 0, C.byref(h))
    if rc != 0:
        return None, lib.sdq_last_error().decode(errors="replace")
    lines = []
    for i in range(lib.sdq_pack_count(h)):
        e = Entry()
        assert lib.sdq_pack_entry(h, i, C.byref(e)) == 0
        dims = ",".join(str(e.dims[k]) for k in range(e.ndim)) or "-"
        lines.append((C.string_at(e.name, e.name_len), e.dtype, e.ndim, dims, e.file_offset, e.nbytes))
    lib.sdq_pack_close(h)
    return sorted(lines), None


def _oracle(buf):
    try:
        ents = pack_oracle.parse(buf)
    except ValueError as e:
        return None, str(e)
    dt = {"F32": 0, "I8": 2}
    return sorted((n.encode("utf-8", "surrogateescape"), dt[d], len(s), ",".join(map(str, s)) or "-", o, nb)
                  for n, (d, s, o, nb) in ents.items()), None


def test_reader_agrees_with_restatement_and_reference_on_damaged_files(pkg, golden_dir, tmp_path):
    lib = pkg.sdq.load_library()
    Entry = pkg.sdq.Entry
    good = open(os.path.join(golden_dir, "tiny_model.sdcpp"), "rb").read()
    header_len = 360                                   # the blob of this fixture starts here
    try:
        from oracle.binding import Reference
        ref = Reference() if Reference.available() else None
    except Exception:
        ref = None
    rng = np.random.default_rng(7)
    path = str(tmp_path / "fuzz.sdcpp")
    accepted = rejected = 0
    for it in range(400):
        b = bytearray(good)
        kind = it % 4
        if kind == 0:                                  # flip 1-3 header bytes
            for _ in range(int(rng.integers(1, 4))):
                b[int(rng.integers(0, header_len))] = int(rng.integers(0, 256))
        elif kind == 1:                                # truncate anywhere
            b = b[: int(rng.integers(0, len(b)))]
        elif kind == 2:                                # overwrite a header field with an extreme value
            pos = int(rng.integers(4, header_len - 8))
            b[pos:pos + 8] = [0, 1, 2**31 - 1, 2**32 - 1, 2**63 - 1, 2**64 - 1][int(rng.integers(0, 6))].to_bytes(8, "little")
        else:                                          # truncate inside the header and append noise
            cut = int(rng.integers(8, header_len))
            b = b[:cut] + bytes(rng.integers(0, 256, int(rng.integers(0, 64)), dtype=np.uint8))
        data = bytes(b)
        with open(path, "wb") as f:
            f.write(data)
        ours, ours_err = _ours(lib, Entry, path)
        want, want_err = _oracle(data)
        assert (ours is None) == (want is None), (it, ours_err, want_err)
        if ours is None:
            rejected += 1
            assert ours_err.replace(" " + path, "") == want_err, (it, ours_err, want_err)
        else:
            accepted += 1
            assert ours == want, it
        if ref is not None:
            try:
                n, _ = ref.load_sdcpp_listing(path)
                ref_ok, ref_err = True, None
            except RuntimeError as e:
                ref_ok, ref_err = False, str(e)
            assert ref_ok == (ours is not None), (it, ref_err, ours_err)
            if not ref_ok and not ref_err.startswith("std::"):
                # (a huge entry count makes the reference's vector::reserve throw std::bad_alloc
                #  before it reads on; the reader here reports the truncation instead)
                assert ref_err == ours_err, (it, ref_err, ours_err)
            elif ref_ok:
                assert n == len(ours)
    assert accepted > 10 and rejected > 100
