"""numpy/ctypes bindings for the two checker libraries (test infrastructure only).

`Oracle` wraps oracle/libtq_oracle.so (the C restatement, symbol prefix tqo_);
`Ref` wraps oracle/_ref/libtq_ref.so (the reference's own C++, prefix ref_).
Both expose the same method names so a test can run either.
Only tests/, the smoke check and bench.py's CPU legs may import this module.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def lcg_matrix(rows: int, cols: int, seed: int) -> np.ndarray:
    """The reference tests' matrix generator (tests/integration/test_linear.cpp:26-34):
    state = state*1103515245 + 12345 (mod 2^32); value = float(state >> 16)/32768 - 1."""
    n = rows * cols
    out = np.empty(n, dtype=np.float32)
    state = seed & 0xFFFFFFFF
    for i in range(n):
        state = (state * 1103515245 + 12345) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(state >> 16) / np.float32(32768.0)) - np.float32(1.0)
    return out.reshape(rows, cols)


class _Base:
    prefix = ""

    def __init__(self, path: str):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        self.path = path

    def fn(self, name):
        return getattr(self.lib, self.prefix + name)


class Oracle(_Base):
    prefix = "tqo_"

    def __init__(self, path: str | None = None):
        if path is None:
            path = os.path.join(HERE, "libtq_oracle.so")
            if not os.path.exists(path):
                from . import build as _b  # type: ignore
                _b.build_oracle()
        super().__init__(path)
        L = self.lib
        L.tqo_codebook.argtypes = [C.c_int, _f32p, _f32p]
        L.tqo_fit_codebook.argtypes = [_f32p, C.c_long, C.c_int, C.c_int, _f32p, _f32p]
        L.tqo_codebook_quantize.argtypes = [_f32p, C.c_long, _f32p, C.c_int, _u8p]
        L.tqo_codebook_quantize.restype = None
        L.tqo_sign.argtypes = [C.c_uint32, C.c_uint32]
        L.tqo_sign.restype = C.c_float
        L.tqo_wht.argtypes = [_f32p, C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.c_int, _f32p]
        L.tqo_derive_seed.argtypes = [_f32p, C.c_size_t, C.c_uint32]
        L.tqo_derive_seed.restype = C.c_uint32
        L.tqo_quantize_weight.argtypes = [_f32p, C.c_int, C.c_int, _f32p, C.c_int, _f32p, C.c_int, C.c_int, C.c_int,
                                          C.c_uint32, C.c_int, _u8p, _u8p, _f32p, _u32p]
        L.tqo_dequantize_weight.argtypes = [_u8p, C.c_int, C.c_int, _u8p, C.c_int, _f32p, _u32p, _f32p, C.c_int,
                                            _f32p, C.c_int, C.c_uint32, _f32p]
        L.tqo_linear_from_dequant.argtypes = [_f32p, C.c_int, C.c_int, _f32p, C.c_int, _f32p]
        L.tqo_linear_from_dequant.restype = None
        L.tqo_kv_seed.argtypes = [C.c_uint32, C.c_uint32]
        L.tqo_kv_seed.restype = C.c_uint32
        L.tqo_kv_encode.argtypes = [_f32p, C.c_long, C.c_int, C.c_uint32, C.c_uint32, _u32p, _f32p, C.c_void_p,
                                    C.c_void_p]
        L.tqo_kv_decode_fp16.argtypes = [_u32p, _f32p, C.c_long, C.c_int, C.c_uint32, _u16p]
        L.tqo_attention.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _u32p, _f32p, _u32p,
                                    _f32p, _u32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, _f32p]

    # -- codebooks ---------------------------------------------------------------
    def codebook(self, bits: int):
        c = np.zeros(1 << bits, np.float32)
        b = np.zeros(max((1 << bits) - 1, 1), np.float32)
        if self.lib.tqo_codebook(bits, c, b):
            raise ValueError("unsupported bit width")
        return c, b[: (1 << bits) - 1]

    def fit_codebook(self, data, bits: int, iterations: int = 100):
        data = _c(data, np.float32).ravel()
        c = np.zeros(1 << bits, np.float32)
        b = np.zeros((1 << bits) - 1, np.float32)
        self.lib.tqo_fit_codebook(data, data.size, bits, iterations, c, b)
        return c, b

    def codebook_quantize(self, values, centroids):
        values = _c(values, np.float32).ravel()
        centroids = _c(centroids, np.float32)
        b = ((centroids[:-1] + centroids[1:]) * np.float32(0.5)).astype(np.float32)
        out = np.zeros(values.size, np.uint8)
        self.lib.tqo_codebook_quantize(values, values.size, _c(b, np.float32), centroids.size, out)
        return out

    # -- rotation ----------------------------------------------------------------
    def signs(self, seed: int, n: int):
        return np.array([self.lib.tqo_sign(seed, i) for i in range(n)], np.float32)

    def wht(self, m, seed: int, block: int, inverse: bool = False):
        m = _c(m, np.float32)
        out = np.empty_like(m)
        if self.lib.tqo_wht(m, m.shape[0], m.shape[1], seed, block, int(inverse), out):
            raise ValueError("bad block size")
        return out

    def derive_seed(self, w, salt: int) -> int:
        w = _c(w, np.float32)
        return int(self.lib.tqo_derive_seed(w, w.size, salt))

    # -- weights -----------------------------------------------------------------
    def quantize_weight(self, w, cb_p, cb_r, primary_bits=4, residual_bits=4, block=128, shared_rotation=True):
        w = _c(w, np.float32)
        out, inn = w.shape
        cb_p, cb_r = _c(cb_p, np.float32), _c(cb_r, np.float32)
        pp = np.zeros((out, inn // 2 if primary_bits <= 4 else inn), np.uint8)
        pr = np.zeros((out, inn // 2), np.uint8)
        norms = np.zeros(out, np.float32)
        seeds = np.zeros(3, np.uint32)
        rc = self.fn("quantize_weight")(w, out, inn, cb_p, cb_p.size, cb_r, cb_r.size, primary_bits, residual_bits,
                                        block, int(shared_rotation), pp, pr, norms, seeds)
        if rc:
            raise ValueError("quantize_weight failed")
        return pp, pr, norms, seeds

    def dequantize_weight(self, pp, pr, norms, seeds, cb_p, cb_r, block):
        pp, pr = _c(pp, np.uint8), _c(pr, np.uint8)
        out, p_cols = pp.shape
        r_cols = pr.shape[1]
        inn = p_cols if p_cols == 2 * r_cols else 2 * p_cols
        cb_p, cb_r = _c(cb_p, np.float32), _c(cb_r, np.float32)
        res = np.zeros((out, inn), np.float32)
        rc = self.fn("dequantize_weight")(pp, out, p_cols, pr, r_cols, _c(norms, np.float32), _c(seeds, np.uint32),
                                          cb_p, cb_p.size, cb_r, cb_r.size, block, res)
        if rc:
            raise ValueError("dequantize_weight failed")
        return res

    def linear_from_dequant(self, w, x):
        w, x = _c(w, np.float32), _c(x, np.float32)
        y = np.zeros((x.shape[0], w.shape[0]), np.float32)
        self.lib.tqo_linear_from_dequant(w, w.shape[0], w.shape[1], x, x.shape[0], y)
        return y

    # -- KV ----------------------------------------------------------------------
    def kv_seed(self, layer: int, which: int) -> int:
        return int(self.lib.tqo_kv_seed(layer, which))

    def kv_encode(self, x, wht_seed: int, qjl_seed: int | None = None):
        """x: [..., d] fp32. Returns (words [n, ceil(d/10)], norms [n], qjl_words|None, qjl_norms|None)."""
        x = _c(x, np.float32)
        d = x.shape[-1]
        n = x.size // d
        words = np.zeros((n, (d + 9) // 10), np.uint32)
        norms = np.zeros(n, np.float32)
        if qjl_seed is None:
            rc = self.lib.tqo_kv_encode(x, n, d, wht_seed, 0, words, norms, None, None)
            q = qn = None
        else:
            q = np.zeros((n, (d + 31) // 32), np.uint32)
            qn = np.zeros(n, np.float32)
            rc = self.lib.tqo_kv_encode(x, n, d, wht_seed, qjl_seed, words, norms, q.ctypes.data, qn.ctypes.data)
        if rc:
            raise ValueError("kv_encode failed")
        return words, norms, q, qn

    def kv_decode_fp16(self, words, norms, d: int, wht_seed: int):
        words, norms = _c(words, np.uint32), _c(norms, np.float32)
        n = norms.size
        out = np.zeros((n, d), np.uint16)
        if self.lib.tqo_kv_decode_fp16(words, norms, n, d, wht_seed, out):
            raise ValueError("kv_decode failed")
        return out.view(np.float16)

    def attention(self, q, kv_heads, k_words, k_norms, v_words, v_norms, qjl_words, qjl_norms, layer=0,
                  start=0, end=None, use_qjl=False):
        """q: [q_heads, d]; storage arrays token-major [tokens*kv_heads, ...]. Returns fp32 [q_heads, d]."""
        q = _c(q, np.float32)
        q_heads, d = q.shape
        tokens = _c(k_norms, np.float32).size // kv_heads
        end = tokens if end is None else end
        out = np.zeros((q_heads, d), np.float32)
        rc = self.lib.tqo_attention(q, q_heads, kv_heads, d, tokens, start, end, _c(k_words, np.uint32),
                                    _c(k_norms, np.float32), _c(v_words, np.uint32), _c(v_norms, np.float32),
                                    _c(qjl_words, np.uint32), _c(qjl_norms, np.float32), self.kv_seed(layer, 1),
                                    self.kv_seed(layer, 2), self.kv_seed(layer, 3), int(use_qjl), out)
        if rc:
            raise ValueError("attention failed")
        return out


class Ref(_Base):
    """The reference's own C++ behind ref_glue.cpp.  Present only after oracle/build.py ran
    with the reference source tree available (or a prebuilt copy travelled with the repo)."""
    prefix = "ref_"

    def __init__(self, path: str | None = None):
        super().__init__(path or os.path.join(HERE, "_ref", "libtq_ref.so"))
        L = self.lib
        L.ref_generate_codebook.argtypes = [C.c_int, _f32p, _f32p]
        L.ref_fit_codebook.argtypes = [_f32p, C.c_long, C.c_int, C.c_int, _f32p, _f32p]
        L.ref_codebook_quantize.argtypes = [_f32p, C.c_long, _f32p, C.c_int, _u8p]
        L.ref_wht.argtypes = [_f32p, C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.c_int, _f32p]
        L.ref_quantize_weight.argtypes = [_f32p, C.c_int, C.c_int, _f32p, C.c_int, _f32p, C.c_int, C.c_int, C.c_int,
                                          C.c_uint32, C.c_int, _u8p, _u8p, _f32p, _u32p]
        L.ref_dequantize_weight.argtypes = [_u8p, C.c_int, C.c_int, _u8p, C.c_int, _f32p, _u32p, _f32p, C.c_int,
                                            _f32p, C.c_int, C.c_uint32, _f32p]
        L.ref_dequantize_weight_mt.argtypes = L.ref_dequantize_weight.argtypes + [C.c_int]
        L.ref_kv_create.argtypes = [C.c_int, C.c_int, C.c_int]
        L.ref_kv_create.restype = C.c_void_p
        L.ref_kv_free.argtypes = [C.c_void_p]
        L.ref_kv_free.restype = None
        L.ref_kv_append.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.ref_kv_seq_length.argtypes = [C.c_void_p]
        L.ref_kv_get_fp16.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, _u16p]
        L.ref_kv_export.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 6
        L.ref_kv_snapshot.argtypes = [C.c_void_p, C.c_void_p, C.c_long, C.c_uint32, C.c_uint32]
        L.ref_kv_snapshot.restype = C.c_long
        L.ref_kv_restore.argtypes = [C.c_void_p, C.c_void_p, C.c_long]
        L.ref_kv_delta.argtypes = [C.c_void_p, C.c_void_p, C.c_long, C.c_uint32, C.c_uint32]
        L.ref_kv_delta.restype = C.c_long
        L.ref_kv_apply_delta.argtypes = [C.c_void_p, C.c_void_p, C.c_long]

    def codebook(self, bits: int):
        c = np.zeros(1 << bits, np.float32)
        b = np.zeros(max((1 << bits) - 1, 1), np.float32)
        if self.lib.ref_generate_codebook(bits, c, b):
            raise ValueError("unsupported bit width")
        return c, b[: (1 << bits) - 1]

    def fit_codebook(self, data, bits: int, iterations: int = 100):
        data = _c(data, np.float32).ravel()
        c = np.zeros(1 << bits, np.float32)
        b = np.zeros((1 << bits) - 1, np.float32)
        self.lib.ref_fit_codebook(data, data.size, bits, iterations, c, b)
        return c, b

    def codebook_quantize(self, values, centroids):
        values = _c(values, np.float32).ravel()
        centroids = _c(centroids, np.float32)
        out = np.zeros(values.size, np.uint8)
        self.lib.ref_codebook_quantize(values, values.size, centroids, centroids.size, out)
        return out

    def wht(self, m, seed: int, block: int, inverse: bool = False):
        m = _c(m, np.float32)
        out = np.empty_like(m)
        if self.lib.ref_wht(m, m.shape[0], m.shape[1], seed, block, int(inverse), out):
            raise ValueError("ref wht failed")
        return out

    quantize_weight = Oracle.quantize_weight
    dequantize_weight = Oracle.dequantize_weight

    def dequantize_weight_mt(self, pp, pr, norms, seeds, cb_p, cb_r, block, threads):
        pp, pr = _c(pp, np.uint8), _c(pr, np.uint8)
        out, p_cols = pp.shape
        r_cols = pr.shape[1]
        inn = p_cols if p_cols == 2 * r_cols else 2 * p_cols
        cb_p, cb_r = _c(cb_p, np.float32), _c(cb_r, np.float32)
        res = np.zeros((out, inn), np.float32)
        rc = self.lib.ref_dequantize_weight_mt(pp, out, p_cols, pr, r_cols, _c(norms, np.float32),
                                               _c(seeds, np.uint32), cb_p, cb_p.size, cb_r, cb_r.size, block, res,
                                               threads)
        if rc:
            raise ValueError("ref dequantize_weight_mt failed")
        return res

    # -- KV: the reference's TQKVCache object ------------------------------------
    class KV:
        def __init__(self, ref: "Ref", layers: int, heads: int, dim: int):
            self.ref, self.layers, self.heads, self.dim = ref, layers, heads, dim
            self.h = ref.lib.ref_kv_create(layers, heads, dim)
            if not self.h:
                raise RuntimeError("ref_kv_create failed")

        def __del__(self):
            if getattr(self, "h", None):
                self.ref.lib.ref_kv_free(self.h)
                self.h = None

        def append(self, layer, keys, values):
            """keys/values: [tokens, heads, dim], float32 or float16."""
            if keys.dtype == np.float16:
                k, v, f16 = _c(keys, np.float16), _c(values, np.float16), 1
            else:
                k, v, f16 = _c(keys, np.float32), _c(values, np.float32), 0
            rc = self.ref.lib.ref_kv_append(self.h, layer, k.ctypes.data, v.ctypes.data, k.shape[0], f16)
            if rc:
                raise ValueError("ref append failed (layer out of range?)")

        def seq_length(self):
            return self.ref.lib.ref_kv_seq_length(self.h)

        def get_fp16(self, layer, values, start, end):
            out = np.zeros(((end - start), self.heads, self.dim), np.uint16)
            if self.ref.lib.ref_kv_get_fp16(self.h, layer, int(values), start, end, out):
                raise ValueError("ref get_fp16 failed")
            return out.view(np.float16)

        def export(self, layer):
            n = self.ref.lib.ref_kv_export(self.h, layer, None, None, None, None, None, None)
            wph, qph = (self.dim + 9) // 10, (self.dim + 31) // 32
            kw = np.zeros((n * self.heads, wph), np.uint32)
            vw = np.zeros((n * self.heads, wph), np.uint32)
            kn = np.zeros(n * self.heads, np.float32)
            vn = np.zeros(n * self.heads, np.float32)
            qw = np.zeros((n * self.heads, qph), np.uint32)
            qn = np.zeros(n * self.heads, np.float32)
            self.ref.lib.ref_kv_export(self.h, layer, kw.ctypes.data, vw.ctypes.data, kn.ctypes.data,
                                       vn.ctypes.data, qw.ctypes.data, qn.ctypes.data)
            return dict(k_words=kw, v_words=vw, k_norms=kn, v_norms=vn, qjl_words=qw, qjl_norms=qn, tokens=n)

        def snapshot(self, model_hash=0, codebook_hash=0) -> np.ndarray:
            """The reference's serialized cache snapshot (snapshot() + snapshot_serialize) as bytes."""
            n = self.ref.lib.ref_kv_snapshot(self.h, None, 0, model_hash, codebook_hash)
            if n < 0:
                raise RuntimeError("ref snapshot failed")
            out = np.zeros(n, np.uint8)
            self.ref.lib.ref_kv_snapshot(self.h, out.ctypes.data, n, model_hash, codebook_hash)
            return out

        def restore(self, data: np.ndarray):
            data = np.ascontiguousarray(data, np.uint8)
            if self.ref.lib.ref_kv_restore(self.h, data.ctypes.data, data.size):
                raise ValueError("ref restore failed")

        def delta(self, start: int, end: int) -> np.ndarray:
            """The reference's serialized delta of positions [start, end) (delta() + delta_serialize)."""
            n = self.ref.lib.ref_kv_delta(self.h, None, 0, start, end)
            if n < 0:
                raise RuntimeError("ref delta failed")
            out = np.zeros(n, np.uint8)
            self.ref.lib.ref_kv_delta(self.h, out.ctypes.data, n, start, end)
            return out

        def apply_delta(self, data: np.ndarray):
            data = np.ascontiguousarray(data, np.uint8)
            if self.ref.lib.ref_kv_apply_delta(self.h, data.ctypes.data, data.size):
                raise ValueError("ref apply_delta failed")

    def kv(self, layers, heads, dim):
        return Ref.KV(self, layers, heads, dim)


def have_ref() -> bool:
    return os.path.exists(os.path.join(HERE, "_ref", "libtq_ref.so"))
