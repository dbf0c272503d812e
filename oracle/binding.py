"""ctypes/numpy bindings for the CPU oracle -- TEST INFRASTRUCTURE ONLY.

`oracle` is the plain-C restatement (liboracle.so, built from qgemm_oracle.c);
`ref` is the reference's own code compiled from its sources (_ref/libsdref.so),
present wherever it was built or carried along.  Nothing under the product
package imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(HERE, "liboracle.so")
_REF_SO = os.path.join(HERE, "_ref", "libsdref.so")

i64, f32p, i8p, i32p, u16p = C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p


def build(quiet=True):
    """Compile liboracle.so (and _ref/libsdref.so where the reference tree is mounted)."""
    out = subprocess.run(["make", "-C", HERE], capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if not quiet:
        print(out.stdout)


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


class Oracle:
    def __init__(self):
        if not os.path.exists(_ORACLE_SO):
            build()
        L = self.lib = C.CDLL(_ORACLE_SO)
        L.orc_threads.restype = C.c_int
        for name in ("orc_act_quant_rows", "orc_dot_s32", "orc_rescale", "orc_qgemm",
                     "orc_bias_add", "orc_gelu_tanh", "orc_quantize_rowwise",
                     "orc_quant_rows_packer", "orc_dequant_rows", "orc_f32_to_bf16",
                     "orc_bf16_to_f32", "orc_f16_to_f32", "orc_set_threads", "orc_layernorm_mod",
                     "orc_residual_add", "orc_layernorm_affine", "orc_matmul_f32", "orc_sdpa"):
            getattr(L, name).restype = None

    def threads(self):
        return int(self.lib.orc_threads())

    def set_threads(self, n):
        self.lib.orc_set_threads(C.c_int(n))

    def act_quant_rows(self, A):
        A = _c(A, np.float32)
        M, K = A.shape
        aq = np.empty((M, K), np.int8)
        sc = np.empty((M,), np.float32)
        self.lib.orc_act_quant_rows(_ptr(A), i64(M), i64(K), _ptr(aq), _ptr(sc))
        return aq, sc

    def dot_s32(self, aq, bq):
        aq, bq = _c(aq, np.int8), _c(bq, np.int8)
        M, K = aq.shape
        N = bq.shape[0]
        acc = np.empty((M, N), np.int32)
        self.lib.orc_dot_s32(_ptr(aq), _ptr(bq), i64(M), i64(N), i64(K), _ptr(acc))
        return acc

    def rescale(self, acc, a_scale, b_scale):
        acc, a_scale, b_scale = _c(acc, np.int32), _c(a_scale, np.float32), _c(b_scale, np.float32)
        M, N = acc.shape
        out = np.empty((M, N), np.float32)
        self.lib.orc_rescale(_ptr(acc), _ptr(a_scale), _ptr(b_scale), i64(M), i64(N), _ptr(out))
        return out

    def qgemm(self, A, Bq, bs):
        A, Bq, bs = _c(A, np.float32), _c(Bq, np.int8), _c(bs, np.float32)
        M, K = A.shape
        N = Bq.shape[0]
        out = np.zeros((M, N), np.float32)
        self.lib.orc_qgemm(_ptr(A), _ptr(Bq), _ptr(bs), i64(M), i64(N), i64(K), _ptr(out))
        return out

    def bias_add(self, y, b, inplace=False):
        y = y if inplace else np.array(y, dtype=np.float32, order="C", copy=True)
        b = _c(b, np.float32)
        self.lib.orc_bias_add(_ptr(y), _ptr(b), i64(y.shape[0]), i64(y.shape[1]))
        return y

    def residual_add(self, x, y, gate=None):
        """x + y * gate (one fused multiply-add per element) or x + y; returns a new array."""
        x = np.array(x, dtype=np.float32, order="C", copy=True)
        y = _c(y, np.float32)
        gate = None if gate is None else _c(gate, np.float32)
        self.lib.orc_residual_add(_ptr(x), _ptr(y), None if gate is None else _ptr(gate),
                                  i64(x.shape[0]), i64(x.shape[1]))
        return x

    def gelu_tanh(self, x, inplace=False):
        x = x if inplace else np.array(x, dtype=np.float32, order="C", copy=True)
        self.lib.orc_gelu_tanh(_ptr(x), i64(x.size))
        return x

    def quantize_rowwise(self, W):
        W = _c(W, np.float32)
        N, K = W.shape
        q = np.empty((N, K), np.int8)
        s = np.empty((N,), np.float32)
        self.lib.orc_quantize_rowwise(_ptr(W), i64(N), i64(K), _ptr(q), _ptr(s))
        return q, s

    def quant_rows_packer(self, x):
        x = _c(x, np.float32)
        rows, last = x.shape
        q = np.empty((rows, last), np.int8)
        s = np.empty((rows,), np.float32)
        self.lib.orc_quant_rows_packer(_ptr(x), i64(rows), i64(last), _ptr(q), _ptr(s))
        return q, s

    def dequant_rows(self, q, scale):
        q, scale = _c(q, np.int8), _c(scale, np.float32)
        rows, last = q.shape
        w = np.empty((rows, last), np.float32)
        self.lib.orc_dequant_rows(_ptr(q), _ptr(scale), i64(rows), i64(last), _ptr(w))
        return w

    def layernorm_mod(self, x, shift, scale, eps=1e-6):
        x, shift, scale = _c(x, np.float32), _c(shift, np.float32), _c(scale, np.float32)
        M, K = x.shape
        y = np.empty((M, K), np.float32)
        self.lib.orc_layernorm_mod(_ptr(x), i64(M), i64(K), _ptr(shift), _ptr(scale), C.c_float(eps), _ptr(y))
        return y

    def layernorm_affine(self, x, weight, bias, eps=1e-6):
        x, weight, bias = _c(x, np.float32), _c(weight, np.float32), _c(bias, np.float32)
        M, K = x.shape
        y = np.empty((M, K), np.float32)
        self.lib.orc_layernorm_affine(_ptr(x), i64(M), i64(K), _ptr(weight), _ptr(bias), C.c_float(eps), _ptr(y))
        return y

    def matmul_f32(self, a, w, bias=None):
        a, w = _c(a, np.float32), _c(w, np.float32)
        bias = None if bias is None else _c(bias, np.float32)
        M, K = a.shape
        N = w.shape[1]
        out = np.empty((M, N), np.float32)
        self.lib.orc_matmul_f32(_ptr(a), i64(M), i64(K), _ptr(w), i64(N),
                                None if bias is None else _ptr(bias), _ptr(out))
        return out

    def sdpa(self, q, k, v, heads):
        q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
        Lq, Cc = q.shape
        out = np.empty((Lq, Cc), np.float32)
        self.lib.orc_sdpa(_ptr(q), _ptr(k), _ptr(v), i64(Lq), i64(k.shape[0]), i64(Cc), C.c_int(heads), _ptr(out))
        return out

    def f32_to_bf16(self, x):
        x = _c(x, np.float32)
        o = np.empty(x.shape, np.uint16)
        self.lib.orc_f32_to_bf16(_ptr(x), _ptr(o), i64(x.size))
        return o

    def bf16_to_f32(self, b):
        b = _c(b, np.uint16)
        o = np.empty(b.shape, np.float32)
        self.lib.orc_bf16_to_f32(_ptr(b), _ptr(o), i64(b.size))
        return o

    def f16_to_f32(self, h):
        h = _c(h, np.uint16)
        o = np.empty(h.shape, np.float32)
        self.lib.orc_f16_to_f32(_ptr(h), _ptr(o), i64(h.size))
        return o


class Reference:
    """The reference's own compiled code (sd::qgemm etc.) behind C wrappers."""

    @staticmethod
    def available():
        return os.path.exists(_REF_SO)

    def __init__(self):
        if not os.path.exists(_REF_SO):
            raise FileNotFoundError(_REF_SO)
        L = self.lib = C.CDLL(_REF_SO)
        L.sdref_nthreads.restype = C.c_int
        L.sdref_set_nthreads.restype = None
        L.sdref_qgemm.restype = C.c_int64
        L.sdref_qgemm_time.restype = C.c_double
        L.sdref_quantize_rowwise.restype = None
        L.sdref_to_bf16.restype = None
        L.sdref_load_sdcpp_listing.restype = C.c_int64

    def nthreads(self):
        return int(self.lib.sdref_nthreads())

    def set_nthreads(self, n):
        self.lib.sdref_set_nthreads(C.c_int(n))

    def qgemm(self, A, Bq, bs):
        A, Bq, bs = _c(A, np.float32), _c(Bq, np.int8), _c(bs, np.float32)
        M, K = A.shape
        N = Bq.shape[0]
        out = np.zeros((M, N), np.float32)
        self.lib.sdref_qgemm(_ptr(A), i64(M), i64(K), _ptr(Bq), i64(N), _ptr(bs), _ptr(out))
        return out

    def qgemm_time(self, A, Bq, bs, reps=1):
        A, Bq, bs = _c(A, np.float32), _c(Bq, np.int8), _c(bs, np.float32)
        M, K = A.shape
        N = Bq.shape[0]
        return float(self.lib.sdref_qgemm_time(_ptr(A), i64(M), i64(K), _ptr(Bq), i64(N),
                                               _ptr(bs), C.c_int(reps)))

    def quantize_rowwise(self, W):
        W = _c(W, np.float32)
        N, K = W.shape
        q = np.empty((N, K), np.int8)
        s = np.empty((N,), np.float32)
        self.lib.sdref_quantize_rowwise(_ptr(W), i64(N), i64(K), _ptr(q), _ptr(s))
        return q, s

    def to_bf16(self, x):
        x = _c(x, np.float32)
        o = np.empty(x.shape, np.uint16)
        self.lib.sdref_to_bf16(_ptr(x), _ptr(o), i64(x.size))
        return o

    def layernorm(self, x, eps=1e-6):
        x = _c(x, np.float32)
        M, K = x.shape
        y = np.empty((M, K), np.float32)
        self.lib.sdref_layernorm.restype = None
        self.lib.sdref_layernorm(_ptr(x), i64(M), i64(K), C.c_float(eps), _ptr(y))
        return y

    # ---- caller-side helpers of src/model/ovi_dit.cpp (ref_shim_dit.cpp) ----
    def gated_add(self, x, y, gate):
        x = np.array(x, dtype=np.float32, order="C", copy=True)
        y, gate = _c(y, np.float32), _c(gate, np.float32)
        self.lib.sdref_gated_add.restype = None
        self.lib.sdref_gated_add(_ptr(x), _ptr(y), _ptr(gate), i64(x.shape[0]), i64(x.shape[1]))
        return x

    def add(self, x, y):
        x = np.array(x, dtype=np.float32, order="C", copy=True)
        y = _c(y, np.float32)
        self.lib.sdref_add.restype = None
        self.lib.sdref_add(_ptr(x), _ptr(y), i64(x.size))
        return x

    def mod_rows(self, x, shift, scale):
        x, shift, scale = _c(x, np.float32), _c(shift, np.float32), _c(scale, np.float32)
        y = np.empty(x.shape, np.float32)
        self.lib.sdref_mod_rows.restype = None
        self.lib.sdref_mod_rows(_ptr(x), _ptr(shift), _ptr(scale), i64(x.shape[0]), i64(x.shape[1]), _ptr(y))
        return y

    def gelu_tanh(self, x):
        x = np.array(x, dtype=np.float32, order="C", copy=True)
        self.lib.sdref_gelu_tanh.restype = None
        self.lib.sdref_gelu_tanh(_ptr(x), i64(x.size))
        return x

    def mlin_i8(self, x, Bq, bs, bias=None):
        x, Bq, bs = _c(x, np.float32), _c(Bq, np.int8), _c(bs, np.float32)
        bias = None if bias is None else _c(bias, np.float32)
        M, K = x.shape
        N = Bq.shape[0]
        y = np.zeros((M, N), np.float32)
        self.lib.sdref_mlin_i8.restype = None
        self.lib.sdref_mlin_i8(_ptr(x), i64(M), i64(K), _ptr(Bq), _ptr(bs),
                               None if bias is None else _ptr(bias), i64(N), _ptr(y))
        return y

    def ffn_fwd(self, x, e, q1, s1, b1, q2, s2, b2):
        """The reference's ffn_fwd on x[M,D] with the [6,D] modulation table e; returns new x."""
        x = np.array(x, dtype=np.float32, order="C", copy=True)
        e, q1, s1, q2, s2 = _c(e, np.float32), _c(q1, np.int8), _c(s1, np.float32), _c(q2, np.int8), _c(s2, np.float32)
        b1 = None if b1 is None else _c(b1, np.float32)
        b2 = None if b2 is None else _c(b2, np.float32)
        M, D = x.shape
        F = q1.shape[0]
        self.lib.sdref_ffn_fwd.restype = None
        self.lib.sdref_ffn_fwd(_ptr(x), i64(M), i64(D), i64(F), _ptr(e), _ptr(q1), _ptr(s1),
                               None if b1 is None else _ptr(b1), _ptr(q2), _ptr(s2),
                               None if b2 is None else _ptr(b2))
        return x

    def layernorm_affine(self, x, w, b, eps=1e-6):
        x, w, b = _c(x, np.float32), _c(w, np.float32), _c(b, np.float32)
        M, K = x.shape
        y = np.empty((M, K), np.float32)
        self.lib.sdref_layernorm_affine.restype = None
        self.lib.sdref_layernorm_affine(_ptr(x), i64(M), i64(K), _ptr(w), _ptr(b), C.c_float(eps), _ptr(y))
        return y

    def matmul(self, a, w, bias=None):
        """sd::matmul: a[M,K] @ w[K,N] + bias, fp32."""
        a, w = _c(a, np.float32), _c(w, np.float32)
        bias = None if bias is None else _c(bias, np.float32)
        M, K = a.shape
        N = w.shape[1]
        out = np.zeros((M, N), np.float32)
        self.lib.sdref_matmul.restype = None
        self.lib.sdref_matmul(_ptr(a), i64(M), i64(K), _ptr(w), i64(N),
                              None if bias is None else _ptr(bias), _ptr(out))
        return out

    def sdpa(self, q, k, v, heads):
        """blk::sdpa, exact fp32 attention."""
        q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
        Lq, Cc = q.shape
        out = np.zeros((Lq, Cc), np.float32)
        self.lib.sdref_sdpa.restype = None
        self.lib.sdref_sdpa(_ptr(q), _ptr(k), _ptr(v), i64(Lq), i64(k.shape[0]), i64(Cc), C.c_int(heads), _ptr(out))
        return out

    def load_sdcpp_listing(self, path):
        """(count, listing) or raises RuntimeError with the loader's message."""
        buf = C.create_string_buffer(1 << 20)
        n = self.lib.sdref_load_sdcpp_listing(path.encode(), buf, i64(len(buf)))
        text = buf.value.decode(errors="replace")
        if n < 0:
            raise RuntimeError(text)
        return int(n), text
