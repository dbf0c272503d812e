"""numpy restatement of the .sdcpp v1 file format and packer -- TEST INFRASTRUCTURE ONLY.

Follows tools/quantize/pack_sdcpp.py (packer, lines 54-124) and
src/serde/sdcpp.cpp (loader, lines 47-133) of JasonHonKL/Self-evolve-diffusion-cpp.
The per-row arithmetic is the C oracle's `orc_quant_rows_packer`; this module
adds the file logic: which tensors are quantized, entry order, header bytes,
blob offsets.  Parity status: pinned against files written by the reference's
own packer (fixtures under tests/golden/).

Layout, little-endian, no padding:  b'SDCP' | u32 version=1 | u32 count |
per tensor { u32 name_len | name | u8 dtype (0 int8 rowwise, 1 f32 raw) |
u32 ndim | i64 dims[ndim] | u64 offset into blob } | blob.  dtype 0 blob =
numel int8 then rows=numel/dims[-1] f32 scales; dtype 1 blob = numel f32.
"""
import json
import struct

import numpy as np

MAGIC, VERSION = b"SDCP", 1
MIN_QUANT_NUMEL = 65536                      # pack_sdcpp.py:23
FLOAT_DTYPES = {"BF16": 2, "F16": 2, "F32": 4}
INT_DTYPES = {"I8": (np.int8, 1), "U8": (np.uint8, 1), "I32": (np.int32, 4), "I64": (np.int64, 8)}


def write_safetensors(path, tensors):
    """tensors: list of (name, dtype_str, shape, raw_bytes) in file order."""
    hdr, off = {}, 0
    for name, dt, shape, raw in tensors:
        hdr[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
    js = json.dumps(hdr, separators=(",", ":")).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)) + js)
        for _, _, _, raw in tensors:
            f.write(raw)


def read_safetensors_header(path):
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        hdr = json.loads(f.read(n))
    return hdr, 8 + n


def to_f32(raw, dt, oracle):
    """pack_sdcpp.py:38-42."""
    if dt == "BF16":
        return oracle.bf16_to_f32(np.frombuffer(raw, np.uint16))
    if dt == "F16":
        return oracle.f16_to_f32(np.frombuffer(raw, np.uint16))
    if dt == "F32":
        return np.frombuffer(raw, np.float32)
    return np.frombuffer(raw, INT_DTYPES[dt][0]).astype(np.float32)


def pack(in_path, out_path, oracle, only="", dtype_preserve=""):
    """pack_sdcpp.py:54-124 restated; returns the plan [(name, code, dims, off, numel, rows)]."""
    only_l = [p for p in only.split(",") if p]
    preserve = set(p for p in dtype_preserve.split(":") if p)
    hdr, base = read_safetensors_header(in_path)
    tens = [(n, e) for n, e in hdr.items()
            if n != "__metadata__" and (not only_l or any(n.startswith(p) for p in only_l))]
    tens.sort(key=lambda t: t[1]["data_offsets"][0])
    plan, off = [], 0
    for name, e in tens:
        dims, dt = e["shape"], e["dtype"]
        numel = int(np.prod(dims, dtype=np.int64)) if dims else 1
        if dt not in FLOAT_DTYPES and dt not in INT_DTYPES:
            raise ValueError("unsupported dtype %s for %s" % (dt, name))
        quant = dt in FLOAT_DTYPES and dt not in preserve and numel >= MIN_QUANT_NUMEL
        rows = numel // dims[-1] if (quant and dims and dims[-1]) else 0
        plan.append((name, 0 if quant else 1, dims, off, numel, rows))
        off += numel + rows * 4 if quant else numel * 4
    data = open(in_path, "rb").read()
    with open(out_path, "wb") as out:
        out.write(MAGIC + struct.pack("<II", VERSION, len(plan)))
        for name, code, dims, o, numel, rows in plan:
            nb = name.encode()
            out.write(struct.pack("<I", len(nb)) + nb + struct.pack("<B", code))
            out.write(struct.pack("<I", len(dims)) + struct.pack("<%dq" % len(dims), *dims))
            out.write(struct.pack("<Q", o))
        for (name, code, dims, o, numel, rows), (_, e) in zip(plan, tens):
            beg, end = e["data_offsets"]
            x = to_f32(data[base + beg: base + end], e["dtype"], oracle)
            if code == 0:
                q, s = oracle.quant_rows_packer(x.reshape(rows, dims[-1]))
                out.write(q.tobytes())
                out.write(s.tobytes())
            else:
                out.write(np.ascontiguousarray(x, np.float32).tobytes())
    return plan


def parse(buf):
    """src/serde/sdcpp.cpp:47-133 restated: returns {name: (dtype_str, shape, offset, nbytes)}
    with offsets from the start of the file; raises ValueError('sdcpp: ...') like the loader."""
    def fail(m):
        raise ValueError("sdcpp: " + m)
    if len(buf) < 16:
        fail("truncated file")
    if buf[:4] != MAGIC:
        fail("bad magic")
    pos = 4

    def take(n):
        nonlocal pos
        if len(buf) - pos < n:
            fail("truncated file")
        b = buf[pos:pos + n]
        pos += n
        return b
    if struct.unpack("<I", take(4))[0] != 1:
        fail("unsupported version")
    count = struct.unpack("<I", take(4))[0]
    es = []
    for _ in range(count):
        nl = struct.unpack("<I", take(4))[0]
        name = take(nl).decode("utf-8", "surrogateescape")
        code = take(1)[0]
        if code > 1:
            fail("bad dtype code")
        nd = struct.unpack("<I", take(4))[0]
        if nd > 8:
            fail("ndim too large")
        dims, numel = [], 1
        for _ in range(nd):
            d = struct.unpack("<q", take(8))[0]
            if d < 0:
                fail("negative dim")
            if d and numel > (1 << 40) // d:
                fail("tensor too large")
            numel *= d
            dims.append(d)
        off = struct.unpack("<Q", take(8))[0]
        if code == 0:
            if nd == 0 or dims[-1] < 1:
                fail("quantized tensor needs a last dim")
            rows = numel // dims[-1]
            blob = numel + rows * 4
        else:
            rows, blob = 0, numel * 4
        es.append((name, code, dims, off, numel, rows, blob))
    data_size = len(buf) - pos
    for name, code, dims, off, numel, rows, blob in es:
        if off > data_size or blob > data_size - off:
            fail("data out of bounds")
    out = {}
    for name, code, dims, off, numel, rows, blob in es:
        if code == 0:
            out.setdefault(name, ("I8", dims, pos + off, numel))
            out.setdefault(name + ".scale", ("F32", [rows], pos + off + numel, rows * 4))
        else:
            out.setdefault(name, ("F32", dims, pos + off, blob))
    return out
