"""ctypes binding of the sdq C ABI (include/sdq.h).

There is no CPU fallback here: every compute call goes to libsdq.so, and a
missing library or device raises.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# flags / codes of include/sdq.h
A_HOST, OUT_HOST, GELU_TANH, FORCE_SIMT, SYNC, LN_TREE_SUMS, LN_AFFINE = 0x1, 0x2, 0x4, 0x8, 0x10, 0x20, 0x40
SDPA_V_FP16 = 0x80
SDPA_K_FP16 = 0x100
F32, BF16, F16 = 0, 1, 2
MODE_PACKER, MODE_ROWWISE = 0, 1
SRC_HOST, DST_HOST = 0x1, 0x2
PACK_UPLOAD = 0x1
DT_F32, DT_I8 = 0, 2
ERR_DEVICE_TIMEOUT = 6
SELFTEST_WAIT_CODE = 0x7e01
STATIC_MAX_ROWS, STATIC_MAX_AQ_BYTES = 32768, 33554432


def lib_path():
    return os.path.join(HERE, "libsdq.so")


def build(verbose=False):
    """Compile libsdq.so (and libsd_b200.so) for sm_100a with nvcc, in-tree."""
    r = subprocess.run(["make", "-C", HERE, "-j8"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building libsdq.so failed:\n" + r.stdout[-4000:] + r.stderr[-4000:])
    if verbose:
        print(r.stdout)


class SdqError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("sdq error %d: %s" % (code, msg))
        self.code = code
        self.msg = msg


class Entry(C.Structure):
    _fields_ = [("name", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("dims", C.c_int64 * 8), ("data", C.c_void_p), ("nbytes", C.c_uint64),
                ("file_offset", C.c_uint64), ("weight", C.c_uint64), ("name_len", C.c_uint64)]


_SIGS = {
    "sdq_init": (C.c_int, [C.c_int]),
    "sdq_shutdown": (C.c_int, []),
    "sdq_device": (C.c_int, []),
    "sdq_version": (C.c_int, []),
    "sdq_last_error": (C.c_char_p, []),
    "sdq_launch_count": (C.c_int64, []),
    "sdq_int8_mma_probe": (C.c_int, [C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "sdq_selftest_wait_expiry": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p]),
    "sdq_malloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "sdq_free": (C.c_int, [C.c_void_p]),
    "sdq_malloc_host": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "sdq_free_host": (C.c_int, [C.c_void_p]),
    "sdq_memcpy_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "sdq_memcpy_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "sdq_memset": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "sdq_stream_sync": (C.c_int, [C.c_void_p]),
    "sdq_stream_create": (C.c_int, [C.POINTER(C.c_void_p)]),
    "sdq_stream_destroy": (C.c_int, [C.c_void_p]),
    "sdq_weight_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.POINTER(C.c_uint64)]),
    "sdq_weight_wrap_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.POINTER(C.c_uint64)]),
    "sdq_weight_lookup": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "sdq_weight_info": (C.c_int, [C.c_uint64, C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                  C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "sdq_weight_release": (C.c_int, [C.c_uint64]),
    "sdq_qgemm": (C.c_int, [C.c_uint64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_quantize_activations": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "sdq_layernorm_mod_quantize": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_float,
                                             C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_qgemm_prequantized": (C.c_int, [C.c_uint64, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_qgemm_colsplit": (C.c_int, [C.c_uint64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.POINTER(C.c_void_p),
                                     C.c_int, C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_ipc_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "sdq_ipc_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "sdq_ipc_close": (C.c_int, [C.c_void_p]),
    "sdq_ffn_pair": (C.c_int, [C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_int64,
                               C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_fweight_upload": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_uint32, C.POINTER(C.c_uint64)]),
    "sdq_fmatmul": (C.c_int, [C.c_uint64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_sdpa": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int,
                           C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_qgemm_residual": (C.c_int, [C.c_uint64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_ffn_block": (C.c_int, [C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_int64,
                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_uint32, C.c_void_p]),
    "sdq_qgemm_static_scratch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64,
                                           C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_quantize_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int, C.c_void_p,
                                    C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_dequant_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_uint32, C.c_void_p]),
    "sdq_pack_sdcpp": (C.c_int, [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p]),
    "sdq_pack_open": (C.c_int, [C.c_char_p, C.c_uint32, C.POINTER(C.c_void_p)]),
    "sdq_pack_count": (C.c_int64, [C.c_void_p]),
    "sdq_pack_pinned": (C.c_int, [C.c_void_p]),
    "sdq_pack_entry": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(Entry)]),
    "sdq_pack_find": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(Entry)]),
    "sdq_pack_close": (C.c_int, [C.c_void_p]),
}


def load_library():
    p = lib_path()
    if not os.path.exists(p):
        raise FileNotFoundError(
            "%s is missing: build it with __graft_entry__.build() (there is no fallback path)" % p)
    lib = C.CDLL(p)
    for name, (res, args) in _SIGS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


def _np_ptr(a):
    return a.ctypes.data_as(C.c_void_p)


class DeviceBuffer:
    """A device allocation made through sdq_malloc."""

    def __init__(self, sdq, nbytes):
        self.sdq = sdq
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        sdq._ck(sdq.lib.sdq_malloc(C.byref(p), max(1, self.nbytes)))
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, sdq, arr, stream=None):
        arr = np.ascontiguousarray(arr)
        b = cls(sdq, arr.nbytes)
        if arr.nbytes:
            sdq._ck(sdq.lib.sdq_memcpy_h2d(b.ptr, _np_ptr(arr), arr.nbytes, stream))
            sdq.sync(stream)
        return b

    def to_numpy(self, dtype, shape, stream=None):
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        if out.nbytes:
            self.sdq._ck(self.sdq.lib.sdq_memcpy_d2h(_np_ptr(out), self.ptr, out.nbytes, stream))
            self.sdq.sync(stream)
        return out

    def free(self):
        if self.ptr:
            self.sdq.lib.sdq_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Pack:
    """An open .sdcpp file (sdq_pack_open)."""

    def __init__(self, sdq, path, upload=False):
        self.sdq = sdq
        h = C.c_void_p()
        sdq._ck(sdq.lib.sdq_pack_open(os.fsencode(path), PACK_UPLOAD if upload else 0, C.byref(h)))
        self.h = h

    def pinned(self):
        return bool(self.sdq.lib.sdq_pack_pinned(self.h))

    def entries(self):
        out = []
        for i in range(self.sdq.lib.sdq_pack_count(self.h)):
            e = Entry()
            self.sdq._ck(self.sdq.lib.sdq_pack_entry(self.h, i, C.byref(e)))
            out.append(self._conv(e))
        return out

    def find(self, name):
        e = Entry()
        self.sdq._ck(self.sdq.lib.sdq_pack_find(self.h, name.encode(), C.byref(e)))
        return self._conv(e)

    @staticmethod
    def _conv(e):
        dims = [int(e.dims[i]) for i in range(e.ndim)]
        return {"name": C.string_at(e.name, e.name_len).decode(errors="replace"), "dtype": int(e.dtype), "dims": dims, "data": e.data,
                "nbytes": int(e.nbytes), "file_offset": int(e.file_offset), "weight": int(e.weight)}

    def array(self, entry):
        """Copy of an entry's bytes as a numpy array (host view of the mapping)."""
        dt = np.int8 if entry["dtype"] == DT_I8 else np.float32
        raw = C.string_at(entry["data"], entry["nbytes"])
        return np.frombuffer(raw, dtype=dt).reshape(entry["dims"]).copy()

    def close(self):
        if self.h:
            self.sdq.lib.sdq_pack_close(self.h)
            self.h = None


class Sdq:
    """One process, one GPU."""

    def __init__(self, device=0):
        self.lib = load_library()
        self._ck(self.lib.sdq_init(device))
        self.device = device

    def _ck(self, rc):
        if rc != 0:
            raise SdqError(rc, (self.lib.sdq_last_error() or b"").decode())

    def sync(self, stream=None):
        self._ck(self.lib.sdq_stream_sync(stream))

    def stream_create(self):
        p = C.c_void_p()
        self._ck(self.lib.sdq_stream_create(C.byref(p)))
        return p.value

    def stream_destroy(self, stream):
        self._ck(self.lib.sdq_stream_destroy(stream))

    def launches(self):
        return int(self.lib.sdq_launch_count())

    def int8_mma_probe(self, iters):
        """(seconds, TOPS) of the MMA-issue-bound int8 probe."""
        sec, tops = C.c_double(), C.c_double()
        self._ck(self.lib.sdq_int8_mma_probe(iters, C.byref(sec), C.byref(tops)))
        return sec.value, tops.value

    def selftest_wait_expiry(self, limit_ms, stream=None):
        """Launches the warp that waits on a barrier nothing arrives on; returns the device word
        that receives its outcome.  The next sync raises SdqError(ERR_DEVICE_TIMEOUT)."""
        out = self.to_device(np.full(1, -1, np.int32))
        self._ck(self.lib.sdq_selftest_wait_expiry(limit_ms, out.ptr, stream))
        return out

    # ---- memory ----
    def alloc(self, nbytes):
        return DeviceBuffer(self, nbytes)

    def to_device(self, arr):
        return DeviceBuffer.from_numpy(self, arr)

    def alloc_pinned(self, shape, dtype):
        """numpy array over pinned host memory (freed with free_pinned)."""
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        self._ck(self.lib.sdq_malloc_host(C.byref(p), max(1, n)))
        buf = (C.c_char * max(1, n)).from_address(p.value)
        arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
        return arr, p.value

    def free_pinned(self, ptr):
        self._ck(self.lib.sdq_free_host(ptr))

    # ---- weights ----
    def weight_upload(self, q, scale):
        q = np.ascontiguousarray(q, np.int8)
        scale = np.ascontiguousarray(scale, np.float32)
        N, K = q.shape
        assert scale.shape == (N,)
        h = C.c_uint64()
        self._ck(self.lib.sdq_weight_upload(_np_ptr(q), _np_ptr(scale), N, K, C.byref(h)))
        return int(h.value)

    def weight_wrap_device(self, q_ptr, scale_ptr, N, K):
        h = C.c_uint64()
        self._ck(self.lib.sdq_weight_wrap_device(q_ptr, scale_ptr, N, K, C.byref(h)))
        return int(h.value)

    def weight_lookup(self, host_ptr):
        h = C.c_uint64()
        self._ck(self.lib.sdq_weight_lookup(host_ptr, C.byref(h)))
        return int(h.value)

    def weight_info(self, w):
        n, k, q, s = C.c_int64(), C.c_int64(), C.c_void_p(), C.c_void_p()
        self._ck(self.lib.sdq_weight_info(w, C.byref(n), C.byref(k), C.byref(q), C.byref(s)))
        return int(n.value), int(k.value), q.value, s.value

    def weight_release(self, w):
        self._ck(self.lib.sdq_weight_release(w))

    # ---- hot path ----
    def qgemm(self, w, A_ptr, M, out_ptr, bias_ptr=None, flags=0, stream=None):
        """Raw call: pointers are device (or host with A_HOST / OUT_HOST)."""
        self._ck(self.lib.sdq_qgemm(w, A_ptr, M, out_ptr, bias_ptr, flags, stream))

    def qgemm_host(self, w, A, bias=None, gelu=False, force_simt=False):
        """numpy in, numpy out through the host-pointer path of sdq_qgemm."""
        A = np.ascontiguousarray(A, np.float32)
        N, K, _, _ = self.weight_info(w)
        M = A.shape[0]
        assert A.shape[1] == K
        out = np.empty((M, N), np.float32)
        flags = A_HOST | OUT_HOST | (GELU_TANH if gelu else 0) | (FORCE_SIMT if force_simt else 0)
        db = self.to_device(np.ascontiguousarray(bias, np.float32)) if bias is not None else None
        self._ck(self.lib.sdq_qgemm(w, _np_ptr(A), M, _np_ptr(out), db.ptr if db else None, flags, None))
        return out

    def quantize_activations(self, A):
        """numpy [M,K] -> (aq int8 [M,K], a_scale f32 [M]) through the device kernel."""
        A = np.ascontiguousarray(A, np.float32)
        M, K = A.shape
        dA = self.to_device(A)
        dq, ds = self.alloc(M * K), self.alloc(M * 4)
        self._ck(self.lib.sdq_quantize_activations(dA.ptr, M, K, dq.ptr, ds.ptr, None))
        self.sync()
        return dq.to_numpy(np.int8, (M, K)), ds.to_numpy(np.float32, (M,))

    def layernorm_mod_quantize(self, X, shift, scale, eps=1e-6, want_h=False, tree_sums=False,
                               affine=False):
        """numpy [M,K] -> (aq, a_scale[, h]) through the fused LayerNorm+modulation+quantize kernel."""
        X = np.ascontiguousarray(X, np.float32)
        M, K = X.shape
        dX, dsh, dsc = self.to_device(X), self.to_device(np.ascontiguousarray(shift, np.float32)), \
            self.to_device(np.ascontiguousarray(scale, np.float32))
        dq, ds = self.alloc(M * K), self.alloc(M * 4)
        dh = self.alloc(M * K * 4) if want_h else None
        self._ck(self.lib.sdq_layernorm_mod_quantize(dX.ptr, M, K, dsh.ptr, dsc.ptr, eps, dq.ptr, ds.ptr,
                                                     dh.ptr if dh else None,
                                                     (LN_TREE_SUMS if tree_sums else 0) |
                                                     (LN_AFFINE if affine else 0), None))
        self.sync()
        out = (dq.to_numpy(np.int8, (M, K)), ds.to_numpy(np.float32, (M,)))
        return out + (dh.to_numpy(np.float32, (M, K)),) if want_h else out

    def qgemm_debug(self, w, A, bias=None, gelu=False, force_simt=False):
        """Both halves with every intermediate returned: (aq, a_scale, acc, out)."""
        A = np.ascontiguousarray(A, np.float32)
        N, K, _, _ = self.weight_info(w)
        M = A.shape[0]
        dA = self.to_device(A)
        dq, ds = self.alloc(M * K), self.alloc(M * 4)
        dacc, dout = self.alloc(M * N * 4), self.alloc(M * N * 4)
        db = self.to_device(np.ascontiguousarray(bias, np.float32)) if bias is not None else None
        self._ck(self.lib.sdq_quantize_activations(dA.ptr, M, K, dq.ptr, ds.ptr, None))
        flags = (GELU_TANH if gelu else 0) | (FORCE_SIMT if force_simt else 0) | SYNC
        self._ck(self.lib.sdq_qgemm_prequantized(w, dq.ptr, ds.ptr, M, dout.ptr, db.ptr if db else None,
                                                 dacc.ptr, flags, None))
        return (dq.to_numpy(np.int8, (M, K)), ds.to_numpy(np.float32, (M,)),
                dacc.to_numpy(np.int32, (M, N)), dout.to_numpy(np.float32, (M, N)))

    def qgemm_colsplit(self, w, A_ptr, M, col0, N_total, out_ptrs, bias_ptr=None, flags=0, stream=None):
        """One column block of a linear, written into every buffer of `out_ptrs` ([M, N_total] each)."""
        arr = (C.c_void_p * len(out_ptrs))(*out_ptrs)
        self._ck(self.lib.sdq_qgemm_colsplit(w, A_ptr, M, col0, N_total, arr, len(out_ptrs), bias_ptr, flags, stream))

    def ipc_export(self, dptr):
        buf = C.create_string_buffer(64)
        self._ck(self.lib.sdq_ipc_export(dptr, buf))
        return buf.raw

    def ipc_open(self, handle):
        p = C.c_void_p()
        self._ck(self.lib.sdq_ipc_open(C.create_string_buffer(handle, 64), C.byref(p)))
        return p.value

    def ipc_close(self, dptr):
        self._ck(self.lib.sdq_ipc_close(dptr))

    def ffn_pair_host(self, w1, b1, w2, b2, x):
        """numpy in, numpy out through the chunked host-pointer pipeline of sdq_ffn_pair."""
        x = np.ascontiguousarray(x, np.float32)
        M = x.shape[0]
        N2 = self.weight_info(w2)[0]
        y = np.empty((M, N2), np.float32)
        d1 = self.to_device(np.ascontiguousarray(b1, np.float32)) if b1 is not None else None
        d2 = self.to_device(np.ascontiguousarray(b2, np.float32)) if b2 is not None else None
        self._ck(self.lib.sdq_ffn_pair(w1, d1.ptr if d1 else None, w2, d2.ptr if d2 else None, _np_ptr(x), M,
                                       None, _np_ptr(y), A_HOST | OUT_HOST, None))
        return y

    def fweight_upload(self, w_kn):
        """fp32 weight [K,N] (numpy) -> handle for fmatmul."""
        w_kn = np.ascontiguousarray(w_kn, np.float32)
        h = C.c_uint64(0)
        self._ck(self.lib.sdq_fweight_upload(_np_ptr(w_kn), w_kn.shape[0], w_kn.shape[1], A_HOST, C.byref(h)))
        return h.value

    def fmatmul_host(self, w, A, N, bias=None, force_simt=False):
        """numpy in, numpy out through the host-pointer path of sdq_fmatmul."""
        A = np.ascontiguousarray(A, np.float32)
        M = A.shape[0]
        out = np.empty((M, N), np.float32)
        db = self.to_device(np.ascontiguousarray(bias, np.float32)) if bias is not None else None
        self._ck(self.lib.sdq_fmatmul(w, _np_ptr(A), M, _np_ptr(out), db.ptr if db else None,
                                      A_HOST | OUT_HOST | (FORCE_SIMT if force_simt else 0), None))
        return out

    def sdpa_np(self, q, k, v, heads, force_simt=False, v_fp16=False, k_fp16=False):
        """numpy in, numpy out through sdq_sdpa."""
        q, k, v = [np.ascontiguousarray(a, np.float32) for a in (q, k, v)]
        Lq, Cc = q.shape
        dq, dk, dv = self.to_device(q), self.to_device(k), self.to_device(v)
        dout = self.alloc(max(Lq * Cc * 4, 4))
        self._ck(self.lib.sdq_sdpa(dq.ptr, dk.ptr, dv.ptr, Lq, k.shape[0], Cc, heads, dout.ptr,
                                   SYNC | (FORCE_SIMT if force_simt else 0) | (SDPA_V_FP16 if v_fp16 else 0) |
                                   (SDPA_K_FP16 if k_fp16 else 0),
                                   None))
        return dout.to_numpy(np.float32, (Lq, Cc))

    def qgemm_residual_np(self, w, A, x, gate=None, bias=None, inplace=True, force_simt=False):
        """numpy in, numpy out: x + (qgemm(A, W) + bias) * gate through sdq_qgemm_residual, with
        the residual either updated in place (out == residual) or read from a second buffer."""
        A, x = np.ascontiguousarray(A, np.float32), np.ascontiguousarray(x, np.float32)
        M, N = x.shape
        dA, dx = self.to_device(A), self.to_device(x)
        dg = self.to_device(np.ascontiguousarray(gate, np.float32)) if gate is not None else None
        db = self.to_device(np.ascontiguousarray(bias, np.float32)) if bias is not None else None
        dout = dx if inplace else self.alloc(M * N * 4)
        self._ck(self.lib.sdq_qgemm_residual(w, dA.ptr, M, dx.ptr, dg.ptr if dg else None, dout.ptr,
                                             db.ptr if db else None,
                                             SYNC | (FORCE_SIMT if force_simt else 0), None))
        return dout.to_numpy(np.float32, (M, N))

    def ffn_block_np(self, w1, b1, w2, b2, x, shift, scale, gate, eps=1e-6, tree_sums=False):
        """numpy in, numpy out through sdq_ffn_block (the reference's ffn_fwd, in place on x)."""
        x = np.ascontiguousarray(x, np.float32)
        M, D = x.shape
        dx = self.to_device(x)
        dev = [self.to_device(np.ascontiguousarray(a, np.float32)) if a is not None else None
               for a in (b1, b2, shift, scale, gate)]
        p = [d.ptr if d else None for d in dev]
        self._ck(self.lib.sdq_ffn_block(w1, p[0], w2, p[1], dx.ptr, M, p[2], p[3], p[4], eps,
                                        SYNC | (LN_TREE_SUMS if tree_sums else 0), None))
        return dx.to_numpy(np.float32, (M, D))

    def qgemm_static_scratch(self, wq_ptr, ws_ptr, N, K, A_ptr, M, out_ptr, bias_ptr=None, flags=0,
                             stream=None):
        """The no-allocation variant: raw device pointers, scratch inside the library image."""
        self._ck(self.lib.sdq_qgemm_static_scratch(wq_ptr, ws_ptr, N, K, A_ptr, M, out_ptr, bias_ptr,
                                                   flags, stream))

    # ---- quantizers ----
    def quantize_rows(self, src, src_dtype, mode):
        """src: numpy [rows,last] of float32 (F32) or uint16 bit patterns (BF16/F16)."""
        src = np.ascontiguousarray(src)
        rows, last = src.shape
        q = np.empty((rows, last), np.int8)
        s = np.empty((rows,), np.float32)
        self._ck(self.lib.sdq_quantize_rows(_np_ptr(src), src_dtype, rows, last, mode, _np_ptr(q),
                                            _np_ptr(s), SRC_HOST | DST_HOST, None))
        return q, s

    def dequant_rows(self, q, scale):
        q = np.ascontiguousarray(q, np.int8)
        scale = np.ascontiguousarray(scale, np.float32)
        rows, last = q.shape
        w = np.empty((rows, last), np.float32)
        self._ck(self.lib.sdq_dequant_rows(_np_ptr(q), _np_ptr(scale), rows, last, _np_ptr(w),
                                           SRC_HOST | DST_HOST, None))
        return w

    # ---- packs ----
    def pack_sdcpp(self, src, dst, only="", dtype_preserve=""):
        self._ck(self.lib.sdq_pack_sdcpp(os.fsencode(src), os.fsencode(dst), only.encode(),
                                         dtype_preserve.encode()))

    def open_pack(self, path, upload=False):
        return Pack(self, path, upload)
