"""numpy-level access to the two CPU checkers.

TEST INFRASTRUCTURE ONLY (tests, smoke check, benchmark CPU-baseline legs).

* ``Oracle``    -- oracle/liboracle.so, the plain-C restatement (tbn_oracle.c).
* ``Reference`` -- oracle/_ref/libtbn_ref.so, the reference's own sources compiled
                   with the wrappers of ref_shim.cpp (present only where it was built).

Both expose the same method names where the functionality overlaps, so a test can
run the same case through either.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libtbn_ref.so")

#: Tiling with which every shape of the benchmark configurations passes the
#: reference's divisibility checks (GeMM.hpp:24-37); its default 32x32 micro-tile does not.
REF_TILING = (64, 64, 128, 16, 8)

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_i32p = C.POINTER(C.c_int32)
_u32p = C.POINTER(C.c_uint32)
_i64p = C.POINTER(C.c_int64)


def reference_tree():
    """Where the reference's sources lie: $TBN_REFERENCE, else a checkout named "reference" beside this repository."""
    return os.environ.get("TBN_REFERENCE") or os.path.abspath(os.path.join(_HERE, "..", "..", "reference"))


def build(force=False):
    """Compiles liboracle.so (and _ref when the reference tree is present)."""
    if force or not os.path.exists(ORACLE_SO) or \
            os.path.getmtime(ORACLE_SO) < os.path.getmtime(os.path.join(_HERE, "tbn_oracle.c")):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    ref_root = reference_tree()
    if os.path.isdir(os.path.join(ref_root, "GeMM", "05-final")):
        if force or not os.path.exists(REF_SO) or \
                os.path.getmtime(REF_SO) < os.path.getmtime(os.path.join(_HERE, "ref_shim.cpp")):
            subprocess.run(["make", "-C", _HERE, "REF=" + ref_root, "_ref/libtbn_ref.so"], check=True,
                           capture_output=True)


def reference_available():
    return os.path.exists(REF_SO)


def _p(a, t):
    return a.ctypes.data_as(t)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i64arr(v):
    return np.asarray(v, dtype=np.int64)


class _Base:
    prefix = ""

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{self.prefix}{what} failed with status {rc}: {self.last_error()}")

    def last_error(self):
        return ""

    def _fn(self, name):
        return getattr(self.lib, self.prefix + name)

    # ---- shared surface ---------------------------------------------------
    def quantize_to_binary(self, w, thr=0.0):
        w = _f32(w)
        out = np.empty(w.shape, dtype=np.uint8)
        self._check(self._fn("quantize_to_binary")(_p(w, _f32p), C.c_int64(w.size), C.c_float(thr),
                                                   _p(out, _u8p)), "quantize_to_binary")
        return out

    def quantize_to_ternary(self, w, lo=-0.1, hi=0.1):
        w = _f32(w)
        out = np.empty(w.shape, dtype=np.int8)
        self._check(self._fn("quantize_to_ternary")(_p(w, _f32p), C.c_int64(w.size), C.c_float(lo),
                                                    C.c_float(hi), _p(out, _i8p)), "quantize_to_ternary")
        return out

    def binary_pack(self, data):
        """int8 +-1 [K,N] -> bytes [N*K/8] (column-major plane, bit set <=> -1)."""
        data = np.ascontiguousarray(data, dtype=np.int8)
        rows, cols = data.shape
        bits = np.zeros(rows * cols // 8 if rows % 8 == 0 else 1, dtype=np.uint8)
        self._check(self._fn("binary_pack")(_p(data, _i8p), C.c_uint32(rows), C.c_uint32(cols),
                                            _p(bits, _u8p)), "binary_pack")
        return bits

    def ternary_pack(self, data):
        data = np.ascontiguousarray(data, dtype=np.int8)
        rows, cols = data.shape
        pos = np.zeros(max(rows * cols // 8, 1), dtype=np.uint8)
        neg = np.zeros_like(pos)
        self._check(self._fn("ternary_pack")(_p(data, _i8p), C.c_uint32(rows), C.c_uint32(cols),
                                             _p(pos, _u8p), _p(neg, _u8p)), "ternary_pack")
        return pos, neg

    def ternary_pack_from_float(self, data, lo=-0.1, hi=0.1):
        data = _f32(data)
        rows, cols = data.shape
        pos = np.zeros(max(rows * cols // 8, 1), dtype=np.uint8)
        neg = np.zeros_like(pos)
        self._check(self._fn("ternary_pack_from_float")(_p(data, _f32p), C.c_uint32(rows), C.c_uint32(cols),
                                                        C.c_float(lo), C.c_float(hi), _p(pos, _u8p),
                                                        _p(neg, _u8p)), "ternary_pack_from_float")
        return pos, neg

    def ternary_codes(self, t):
        t = np.ascontiguousarray(t, dtype=np.int8).reshape(-1)
        out = np.zeros((t.size + 3) // 4, dtype=np.uint8)
        self._check(self._fn("ternary_codes")(_p(t, _i8p), C.c_int64(t.size), _p(out, _u8p)), "ternary_codes")
        return out

    def fxb_naive(self, a, b_bin, scale=1.0):
        a = _f32(a)
        b = np.ascontiguousarray(b_bin, dtype=np.uint8)
        M, K = a.shape
        N = b.shape[1]
        out = np.empty((M, N), dtype=np.float32)
        self._check(self._fn("fxb_naive")(_p(a, _f32p), C.c_int64(M), C.c_int64(K), _p(b, _u8p), C.c_int64(N),
                                          C.c_float(scale), _p(out, _f32p)), "fxb_naive")
        return out

    def gemm_f32(self, a, b, c=None, alpha=1.0, beta=0.0, transA=False, transB=False):
        a, b = _f32(a), _f32(b)
        M = a.shape[1] if transA else a.shape[0]
        N = b.shape[0] if transB else b.shape[1]
        out = np.empty((M, N), dtype=np.float32)
        cc = _f32(c) if c is not None else None
        self._check(self._fn("gemm_f32")(_p(a, _f32p), C.c_int64(a.shape[0]), C.c_int64(a.shape[1]),
                                         _p(b, _f32p), C.c_int64(b.shape[0]), C.c_int64(b.shape[1]),
                                         _p(cc, _f32p) if cc is not None else None,
                                         C.c_int(0 if cc is None else cc.ndim), C.c_float(alpha),
                                         C.c_float(beta), C.c_int(transA), C.c_int(transB), _p(out, _f32p)),
                    "gemm_f32")
        return out


class Oracle(_Base):
    """The plain-C restatement."""
    prefix = "orc_"

    def __init__(self):
        build()
        self.lib = C.CDLL(ORACLE_SO)
        self.lib.orc_conv_out_dim.restype = C.c_int64
        self.lib.orc_pool_out_dim.restype = C.c_int64

    def sign_ge0(self, w):
        w = _f32(w)
        out = np.empty(w.shape, dtype=np.int8)
        self._check(self.lib.orc_sign_ge0(_p(w, _f32p), C.c_int64(w.size), _p(out, _i8p)), "sign_ge0")
        return out

    def channel_abs_mean(self, w):
        w = _f32(w)
        ch = w.shape[0]
        out = np.empty(ch, dtype=np.float32)
        self._check(self.lib.orc_channel_abs_mean(_p(w, _f32p), C.c_int64(ch), C.c_int64(w.size // ch),
                                                  _p(out, _f32p)), "channel_abs_mean")
        return out

    def column_abs_mean(self, w):
        w = _f32(w)
        K, N = w.shape
        out = np.empty(N, dtype=np.float32)
        self._check(self.lib.orc_column_abs_mean(_p(w, _f32p), C.c_int64(K), C.c_int64(N), _p(out, _f32p)),
                    "column_abs_mean")
        return out

    def column_abs_mean_nonzero(self, w, lo, hi):
        w = _f32(w)
        K, N = w.shape
        out = np.empty(N, dtype=np.float32)
        self._check(self.lib.orc_column_abs_mean_nonzero(_p(w, _f32p), C.c_int64(K), C.c_int64(N),
                                                         C.c_float(lo), C.c_float(hi), _p(out, _f32p)),
                    "column_abs_mean_nonzero")
        return out

    def binary_pack_padded(self, b_bin):
        """BINARY bytes [K,N] -> uint32 words [ceil8(N), ceil128(K)/32]."""
        b = np.ascontiguousarray(b_bin, dtype=np.uint8)
        K, N = b.shape
        Kp, Np = (K + 127) // 128 * 128, (N + 7) // 8 * 8
        words = np.zeros((Np, Kp // 32), dtype=np.uint32)
        self._check(self.lib.orc_binary_pack_padded(_p(b, _u8p), C.c_uint32(K), C.c_uint32(N), C.c_uint32(Kp),
                                                    C.c_uint32(Np), _p(words, _u32p)), "binary_pack_padded")
        return words

    def gemm_tbn(self, pos, neg, bits, M, K, N):
        out = np.empty((M, N), dtype=np.int32)
        self._check(self.lib.orc_gemm_tbn(_p(pos, _u8p), _p(neg, _u8p), _p(bits, _u8p), C.c_uint32(M),
                                          C.c_uint32(K), C.c_uint32(N), _p(out, _i32p)), "gemm_tbn")
        return out

    def qlinear_matmul_binary(self, a, b_bin, scale=1.0, lo=-0.1, hi=0.1):
        a = _f32(a)
        b = np.ascontiguousarray(b_bin, dtype=np.uint8)
        M, K = a.shape
        N = b.shape[1]
        out = np.empty((M, N), dtype=np.float32)
        self._check(self.lib.orc_qlinear_matmul_binary(_p(a, _f32p), C.c_uint32(M), C.c_uint32(K), _p(b, _u8p),
                                                       C.c_uint32(N), C.c_float(scale), C.c_float(lo),
                                                       C.c_float(hi), _p(out, _f32p)), "qlinear_matmul_binary")
        return out

    def conv_out_shape(self, xshape, wshape, p):
        N, _, H, W = xshape
        M, _, kh, kw = wshape
        oh = self.lib.orc_conv_out_dim(C.c_int64(H), C.c_int64(kh), C.c_int64(p[0]), C.c_int64(p[2]), C.c_int64(p[4]))
        ow = self.lib.orc_conv_out_dim(C.c_int64(W), C.c_int64(kw), C.c_int64(p[1]), C.c_int64(p[3]), C.c_int64(p[5]))
        return (N, M, oh, ow)

    def conv2d_f32(self, x, w, bias, p):
        x, w = _f32(x), _f32(w)
        p = _i64arr(p)
        out = np.empty(self.conv_out_shape(x.shape, w.shape, p), dtype=np.float32)
        b = _f32(bias) if bias is not None else None
        N, Cc, H, W = x.shape
        M, _, kh, kw = w.shape
        self._check(self.lib.orc_conv2d_f32(_p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H), C.c_int64(W),
                                            _p(w, _f32p), C.c_int64(M), C.c_int64(kh), C.c_int64(kw),
                                            _p(b, _f32p) if b is not None else None, _p(p, _i64p),
                                            _p(out, _f32p)), "conv2d_f32")
        return out

    def conv2d_tbn_session(self, x, w, bias, p, use_alpha=True):
        x, w = _f32(x), _f32(w)
        p = _i64arr(p)
        out = np.empty(self.conv_out_shape(x.shape, w.shape, p), dtype=np.float32)
        b = _f32(bias) if bias is not None else None
        N, Cc, H, W = x.shape
        M, _, kh, kw = w.shape
        self._check(self.lib.orc_conv2d_tbn_session(_p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H),
                                                    C.c_int64(W), _p(w, _f32p), C.c_int64(M), C.c_int64(kh),
                                                    C.c_int64(kw), _p(b, _f32p) if b is not None else None,
                                                    _p(p, _i64p), C.c_int(use_alpha), _p(out, _f32p)),
                    "conv2d_tbn_session")
        return out

    def im2col(self, x, kh, kw, p):
        x = _f32(x)
        p = _i64arr(p)
        N, Cc, H, W = x.shape
        _, _, oh, ow = self.conv_out_shape(x.shape, (1, Cc, kh, kw), p)
        out = np.empty((N * oh * ow, Cc * kh * kw), dtype=np.float32)
        self._check(self.lib.orc_im2col(_p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H), C.c_int64(W),
                                        C.c_int64(kh), C.c_int64(kw), _p(p, _i64p), _p(out, _f32p)), "im2col")
        return out

    def im2col_ternary_packed(self, x, kh, kw, p, m_padded, k_padded, lo=-0.1, hi=0.1):
        x = _f32(x)
        p = _i64arr(p)
        N, Cc, H, W = x.shape
        pos = np.zeros(m_padded * k_padded // 8, dtype=np.uint8)
        neg = np.zeros_like(pos)
        self._check(self.lib.orc_im2col_ternary_packed(_p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H),
                                                       C.c_int64(W), C.c_int64(kh), C.c_int64(kw), _p(p, _i64p),
                                                       C.c_uint32(m_padded), C.c_uint32(k_padded), C.c_float(lo),
                                                       C.c_float(hi), _p(pos, _u8p), _p(neg, _u8p)),
                    "im2col_ternary_packed")
        return pos, neg

    def pool2d(self, kind, x, p, ceil_mode=False, count_include_pad=False):
        x = _f32(x)
        N, Cc, H, W = x.shape
        if kind == 2:
            out = np.empty((N, Cc, 1, 1), dtype=np.float32)
            self._check(self.lib.orc_global_avgpool2d(_p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H),
                                                      C.c_int64(W), _p(out, _f32p)), "global_avgpool2d")
            return out
        p = _i64arr(p)
        oh = self.lib.orc_pool_out_dim(C.c_int64(H), C.c_int64(p[0]), C.c_int64(p[2]), C.c_int64(p[4]), C.c_int(ceil_mode))
        ow = self.lib.orc_pool_out_dim(C.c_int64(W), C.c_int64(p[1]), C.c_int64(p[3]), C.c_int64(p[5]), C.c_int(ceil_mode))
        out = np.empty((N, Cc, oh, ow), dtype=np.float32)
        self._check(self.lib.orc_pool2d(C.c_int(kind), _p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H),
                                        C.c_int64(W), _p(p, _i64p), C.c_int(ceil_mode), C.c_int(count_include_pad),
                                        _p(out, _f32p)), "pool2d")
        return out

    def relu(self, x):
        x = _f32(x)
        out = np.empty_like(x)
        self._check(self.lib.orc_relu(_p(x, _f32p), C.c_int64(x.size), _p(out, _f32p)), "relu")
        return out

    def add(self, a, b):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        hw = 1
        if a.size != b.size and a.ndim == 4:
            hw = a.shape[2] * a.shape[3]
        self._check(self.lib.orc_add(_p(a, _f32p), C.c_int64(a.size), _p(b, _f32p), C.c_int64(b.size),
                                     C.c_int64(hw), _p(out, _f32p)), "add")
        return out


class Reference(_Base):
    """The reference's own code (only where oracle/_ref/libtbn_ref.so was built)."""
    prefix = "ref_"

    def __init__(self):
        build()
        if not reference_available():
            raise FileNotFoundError(REF_SO)
        self.lib = C.CDLL(REF_SO)
        self.lib.ref_last_error.restype = C.c_char_p

    def last_error(self):
        return self.lib.ref_last_error().decode()

    @staticmethod
    def _tiling(t):
        return np.asarray(t or REF_TILING, dtype=np.uint32)

    def gemm_engine(self, pos, neg, a_rows, a_cols, bits, b_cols, tiling=None):
        t = self._tiling(tiling)
        out = np.empty((a_rows, b_cols), dtype=np.int32)
        flops = C.c_uint64(0)
        self._check(self.lib.ref_gemm_engine(_p(pos, _u8p), _p(neg, _u8p), C.c_uint32(a_rows), C.c_uint32(a_cols),
                                             _p(bits, _u8p), C.c_uint32(b_cols), _p(t, _u32p), _p(out, _i32p),
                                             C.byref(flops)), "gemm_engine")
        return out, flops.value

    def qlinear_matmul_binary(self, a, b_bin, scale=1.0, tiling=None):
        a = _f32(a)
        b = np.ascontiguousarray(b_bin, dtype=np.uint8)
        t = self._tiling(tiling)
        M, K = a.shape
        N = b.shape[1]
        out = np.empty((M, N), dtype=np.float32)
        self._check(self.lib.ref_qlinear_matmul_binary(_p(a, _f32p), C.c_int64(M), C.c_int64(K), _p(b, _u8p),
                                                       C.c_int64(N), C.c_float(scale), _p(t, _u32p),
                                                       _p(out, _f32p)), "qlinear_matmul_binary")
        return out

    def pack_binary_weights(self, b_bin):
        """BINARY bytes [K,N] -> opaque handle of the reference's packed BinaryMatrix."""
        b = np.ascontiguousarray(b_bin, dtype=np.uint8)
        self.lib.ref_pack_binary_weights.restype = C.c_void_p
        h = self.lib.ref_pack_binary_weights(_p(b, _u8p), C.c_uint32(b.shape[0]), C.c_uint32(b.shape[1]))
        if not h:
            raise RuntimeError("ref_pack_binary_weights failed: " + self.last_error())
        return C.c_void_p(h), b.shape[1]

    def free_binary_weights(self, handle):
        self.lib.ref_free_binary_weights(handle[0])

    def qlinear_matmul_binary_packed(self, a, handle, scale=1.0, tiling=None):
        a = _f32(a)
        t = self._tiling(tiling)
        M, K = a.shape
        N = handle[1]
        out = np.empty((M, N), dtype=np.float32)
        self._check(self.lib.ref_qlinear_matmul_binary_packed(_p(a, _f32p), C.c_int64(M), C.c_int64(K), handle[0],
                                                              C.c_uint32(N), C.c_float(scale), _p(t, _u32p),
                                                              _p(out, _f32p)), "qlinear_matmul_binary_packed")
        return out

    def conv2d_f32(self, x, w, bias, p):
        x, w = _f32(x), _f32(w)
        p = _i64arr(p)
        b = _f32(bias) if bias is not None else None
        N, Cc, H, W = x.shape
        M, _, kh, kw = w.shape
        dims = np.zeros(4, dtype=np.int64)
        args = (_p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H), C.c_int64(W), _p(w, _f32p), C.c_int64(M),
                C.c_int64(kh), C.c_int64(kw), _p(b, _f32p) if b is not None else None, _p(p, _i64p))
        self._check(self.lib.ref_conv2d_f32(*args, None, _p(dims, _i64p)), "conv2d_f32(shape)")
        out = np.empty(tuple(int(d) for d in dims), dtype=np.float32)
        self._check(self.lib.ref_conv2d_f32(*args, _p(out, _f32p), _p(dims, _i64p)), "conv2d_f32")
        return out

    def im2col(self, x, kh, kw, p, rows):
        x = _f32(x)
        p = _i64arr(p)
        N, Cc, H, W = x.shape
        out = np.empty((rows, Cc * kh * kw), dtype=np.float32)
        self._check(self.lib.ref_im2col(_p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H), C.c_int64(W),
                                        C.c_int64(kh), C.c_int64(kw), _p(p, _i64p), _p(out, _f32p)), "im2col")
        return out

    def im2col_ternary_packed(self, x, kh, kw, p, m_padded, k_padded, lo=-0.1, hi=0.1):
        x = _f32(x)
        p = _i64arr(p)
        N, Cc, H, W = x.shape
        pos = np.zeros(m_padded * k_padded // 8, dtype=np.uint8)
        neg = np.zeros_like(pos)
        self._check(self.lib.ref_im2col_ternary_packed(_p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H),
                                                       C.c_int64(W), C.c_int64(kh), C.c_int64(kw), _p(p, _i64p),
                                                       C.c_uint32(m_padded), C.c_uint32(k_padded), C.c_float(lo),
                                                       C.c_float(hi), _p(pos, _u8p), _p(neg, _u8p)),
                    "im2col_ternary_packed")
        return pos, neg

    def pool2d(self, kind, x, p, ceil_mode=False, count_include_pad=False):
        x = _f32(x)
        N, Cc, H, W = x.shape
        pp = _i64arr(p if p is not None else (1, 1, 1, 1, 0, 0))
        dims = np.zeros(4, dtype=np.int64)
        args = (C.c_int(kind), _p(x, _f32p), C.c_int64(N), C.c_int64(Cc), C.c_int64(H), C.c_int64(W), _p(pp, _i64p),
                C.c_int(ceil_mode), C.c_int(count_include_pad))
        self._check(self.lib.ref_pool2d(*args, None, _p(dims, _i64p)), "pool2d(shape)")
        out = np.empty(tuple(int(d) for d in dims), dtype=np.float32)
        self._check(self.lib.ref_pool2d(*args, _p(out, _f32p), _p(dims, _i64p)), "pool2d")
        return out

    def session_run(self, spec, blob, iblob, input_name, x, output_name, out_shape, quantization,
                    tiling=None, repeats=1):
        x = _f32(x)
        blob = _f32(blob)
        iblob = np.ascontiguousarray(iblob, dtype=np.int64)
        t = self._tiling(tiling)
        out = np.empty(out_shape, dtype=np.float32)
        self._check(self.lib.ref_session_run(spec.encode(), _p(blob, _f32p), _p(iblob, _i64p), input_name.encode(),
                                             _p(x, _f32p), output_name.encode(), _p(out, _f32p),
                                             C.c_int64(out.size), C.c_int(bool(quantization)), _p(t, _u32p),
                                             C.c_int(repeats)), "session_run")
        return out
