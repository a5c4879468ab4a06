"""Host-side mirror of the reference's C++ interface for the hot path, over the C-ABI.

Names follow the reference (include/turboquant/*.h): Codebook / generate_codebook,
apply_wht_rotation / apply_inverse_wht_rotation, quantize_weight -> QuantizedWeight,
dequantize_weight, TurboQuantLinear.forward, TQKVCache.append / get_keys_fp16 /
get_values_fp16 / seq_length, hybrid_attention (compressed branch).

Arguments may be numpy arrays (host memory) or torch CUDA tensors (used in place through
their device pointer).  Everything runs in the CUDA library; nothing here computes.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import TQ_F16, TQ_F32, TQError, check


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


def _ptr(x):
    """Raw address of a numpy array or torch tensor (must be contiguous)."""
    if x is None:
        return None
    if _is_torch(x):
        if not x.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return C.c_void_p(x.data_ptr())
    if not x.flags["C_CONTIGUOUS"]:
        raise ValueError("array must be C-contiguous")
    return C.c_void_p(x.ctypes.data)


def _dtype_tag(x) -> int:
    name = str(x.dtype)
    if name.endswith("float32"):
        return TQ_F32
    if name.endswith("float16"):
        return TQ_F16
    raise TypeError(f"expected float32 or float16, got {x.dtype}")


def _stream_ptr(stream):
    if stream is None:
        return None
    if hasattr(stream, "cuda_stream"):
        return C.c_void_p(stream.cuda_stream)
    return C.c_void_p(int(stream))


def _np(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ---- codebooks -------------------------------------------------------------------------

@dataclass
class Codebook:
    """include/turboquant/codebook.h:25-30."""
    centroids: np.ndarray
    boundaries: np.ndarray
    bits: int


def generate_codebook(bits: int) -> Codebook:
    """generate_codebook (src/codebook.cpp:71-85); raises ValueError for bits outside 1..5."""
    L = _lib.load()
    if not 1 <= bits <= 5:
        raise ValueError("Unsupported bit width; must be 1-5")
    c = np.zeros(1 << bits, np.float32)
    b = np.zeros(max((1 << bits) - 1, 1), np.float32)
    check(L.tq_codebook_generate(bits, c.ctypes.data, b.ctypes.data), "generate_codebook")
    return Codebook(c, b[: (1 << bits) - 1], bits)


def generate_codebook_from_data(data, bits: int, iterations: int = 100, stream=None, return_iterations: bool = False):
    """generate_codebook_from_data (src/codebook.cpp:269-282): Lloyd-Max fit on the device.  data: fp32,
    numpy or a CUDA tensor, any shape."""
    L = _lib.load()
    if not 1 <= bits <= 5:
        raise ValueError("Unsupported bit width; must be 1-5")
    if _is_torch(data):
        data = data.reshape(-1).contiguous().float()
        n = int(data.numel())
    else:
        data = np.ascontiguousarray(data, np.float32).reshape(-1)
        n = int(data.size)
    c = np.zeros(1 << bits, np.float32)
    b = np.zeros(max((1 << bits) - 1, 1), np.float32)
    run = C.c_int(0)
    check(L.tq_codebook_fit(_ptr(data) if n else None, n, bits, int(iterations), c.ctypes.data, b.ctypes.data, C.byref(run),
                            _stream_ptr(stream)), "generate_codebook_from_data")
    cb = Codebook(c, b[: (1 << bits) - 1], bits)
    return (cb, run.value) if return_iterations else cb


def fit_layer_codebooks(weight, block_size: int, primary_bits: int = 4, residual_bits: int = 4, iterations: int = 100, stream=None):
    """Per-layer codebooks as the converter fits them (src/converter.cpp:291-368): (primary, residual);
    residual is None when residual_bits is 0.  weight: fp32 [out, in], numpy or a CUDA tensor."""
    L = _lib.load()
    if _is_torch(weight):
        weight = weight.contiguous().float()
    else:
        weight = np.ascontiguousarray(weight, np.float32)
    out_f, in_f = int(weight.shape[0]), int(weight.shape[1])
    cp = np.zeros(1 << primary_bits, np.float32)
    bp = np.zeros(max((1 << primary_bits) - 1, 1), np.float32)
    cr = np.zeros(1 << max(residual_bits, 1), np.float32)
    br = np.zeros(max((1 << max(residual_bits, 1)) - 1, 1), np.float32)
    check(L.tq_fit_layer_codebooks(_ptr(weight), out_f, in_f, int(block_size), int(primary_bits), int(residual_bits), int(iterations),
                                   cp.ctypes.data, bp.ctypes.data, cr.ctypes.data, br.ctypes.data, _stream_ptr(stream)),
          "fit_layer_codebooks")
    primary = Codebook(cp, bp[: (1 << primary_bits) - 1], primary_bits)
    residual = Codebook(cr, br[: (1 << residual_bits) - 1], residual_bits) if residual_bits > 0 else None
    return primary, residual


def adaptive_block_size(in_features: int, max_block: int) -> int:
    """Largest power of two <= max_block dividing in_features (src/converter.cpp:228-240)."""
    return int(_lib.load().tq_adaptive_block_size(int(in_features), int(max_block)))


def layer_index(name: str) -> int:
    """N of the first ".layers.N." in a tensor name, -1 if none (src/converter.cpp:52-59)."""
    return int(_lib.load().tq_layer_index(name.encode()))


def is_sensitive_layer(index: int, max_index: int, sensitive_start: int, sensitive_end: int) -> bool:
    """Kept at fp16 by the converter (src/converter.cpp:81-93)."""
    return bool(_lib.load().tq_is_sensitive_layer(int(index), int(max_index), int(sensitive_start), int(sensitive_end)))


def qjl_compress(residual, proj_dim: int, proj_seed: int):
    """metal/turboquant_qjl.metal tq_qjl_compress: residual fp32 [tokens, heads, head_dim] (numpy) ->
    (signs uint32 [tokens, heads, ceil(proj_dim / 32)], norms fp32 [tokens, heads])."""
    L = _lib.load()
    r = np.ascontiguousarray(residual, np.float32)
    t, h, d = r.shape
    words = (proj_dim + 31) // 32
    signs = np.zeros((t, h, words), np.uint32)
    norms = np.zeros((t, h), np.float32)
    check(L.tq_qjl_compress(_ptr(r), t, h, d, int(proj_dim), int(proj_seed) & 0xFFFFFFFF, _ptr(signs), _ptr(norms), None), "qjl_compress")
    return signs, norms


def qjl_dot_correction(signs_q, signs_k, norms_k, head_idx: int, proj_dim: int):
    """metal/turboquant_qjl.metal tq_qjl_dot_correction: -> fp32 [num_queries, num_keys] for one head."""
    L = _lib.load()
    sq = np.ascontiguousarray(signs_q, np.uint32)
    sk = np.ascontiguousarray(signs_k, np.uint32)
    nk = np.ascontiguousarray(norms_k, np.float32)
    out = np.zeros((sq.shape[0], sk.shape[0]), np.float32)
    check(L.tq_qjl_dot_correction(_ptr(sq), _ptr(sk), _ptr(nk), sq.shape[0], sk.shape[0], sk.shape[1], int(head_idx), int(proj_dim),
                                  _ptr(out), None), "qjl_dot_correction")
    return out


def codebook_from_centroids(centroids) -> Codebook:
    c = _np(centroids, np.float32)
    b = ((c[:-1] + c[1:]) * np.float32(0.5)).astype(np.float32)
    bits = int(np.ceil(np.log2(max(c.size, 2))))
    return Codebook(c, b, bits)


# ---- rotation ----------------------------------------------------------------------------

def _wht(matrix, seed, block_size, inverse, out, stream):
    L = _lib.load()
    if tuple(matrix.shape)[-1] % block_size:
        raise ValueError("in_features must be divisible by block_size")
    rows = int(np.prod(matrix.shape[:-1])) if len(matrix.shape) > 1 else 1
    cols = matrix.shape[-1]
    if out is None:
        if _is_torch(matrix):
            import torch
            out = torch.empty_like(matrix)
        else:
            matrix = _np(matrix, np.float32)
            out = np.empty_like(matrix)
    check(L.tq_wht_rotate(_ptr(matrix), _ptr(out), rows, cols, seed, block_size, int(inverse), _stream_ptr(stream)),
          "wht_rotate")
    return out


def apply_wht_rotation(matrix, seed: int, block_size: int, out=None, stream=None):
    """apply_wht_rotation (src/rotation.cpp:364-383): fp32 [rows, cols] -> same."""
    return _wht(matrix, seed, block_size, False, out, stream)


def apply_inverse_wht_rotation(matrix, seed: int, block_size: int, out=None, stream=None):
    """apply_inverse_wht_rotation (src/rotation.cpp:385-403)."""
    return _wht(matrix, seed, block_size, True, out, stream)


# ---- weights -------------------------------------------------------------------------------

@dataclass
class QuantizerConfig:
    """include/turboquant/quantizer.h:11-19 (the fields the quantiser reads)."""
    primary_bits: int = 4
    residual_bits: int = 4
    block_size: int = 512
    shared_rotation: bool = False


@dataclass
class QuantizedWeight:
    """include/turboquant/quantizer.h:22-27; norms are fp32 as the reference stores them."""
    packed_primary: np.ndarray
    packed_residual: np.ndarray
    norms: np.ndarray
    seeds: np.ndarray


def quantize_weight(weight, primary_codebook: Codebook, residual_codebook: Codebook,
                    config: QuantizerConfig, seeds=None) -> QuantizedWeight:
    """quantize_weight (src/quantizer.cpp:41-261) on the device; host arrays in and out.  seeds =
    (primary, residual) fixes the rotation seeds instead of deriving them from the weight's bytes."""
    L = _lib.load()
    w = weight if _is_torch(weight) else _np(weight, np.float32)
    out_f, in_f = int(w.shape[0]), int(w.shape[1])
    if in_f % config.block_size:
        raise ValueError("in_features must be divisible by block_size")
    pp = np.zeros((out_f, in_f // 2 if config.primary_bits <= 4 else in_f), np.uint8)
    pr = np.zeros((out_f, in_f // 2), np.uint8)
    norms = np.zeros(out_f, np.float32)
    cp, cr = _np(primary_codebook.centroids, np.float32), _np(residual_codebook.centroids, np.float32)
    out_seeds = np.zeros(3, np.uint32)
    if seeds is None:
        check(L.tq_quantize_weight(_ptr(w), out_f, in_f, _ptr(cp), cp.size, _ptr(cr), cr.size, config.primary_bits,
                                   config.residual_bits, config.block_size, int(config.shared_rotation), _ptr(pp),
                                   _ptr(pr), _ptr(norms), _ptr(out_seeds), None), "quantize_weight")
    else:
        check(L.tq_quantize_weight_seeded(_ptr(w), out_f, in_f, _ptr(cp), cp.size, _ptr(cr), cr.size, config.primary_bits,
                                          config.residual_bits, config.block_size, int(config.shared_rotation),
                                          int(seeds[0]) & 0xFFFFFFFF, int(seeds[1]) & 0xFFFFFFFF, _ptr(pp), _ptr(pr), _ptr(norms),
                                          _ptr(out_seeds), None), "quantize_weight")
    return QuantizedWeight(pp, pr, norms, out_seeds)


class TurboQuantLinear:
    """turboquant::TurboQuantLinear (include/turboquant/linear.h:11-35)."""

    def __init__(self, in_features: int, out_features: int, weights: QuantizedWeight, primary_codebook: Codebook,
                 residual_codebook: Codebook, block_size: int):
        L = _lib.load()
        self._L = L
        pp, pr = _np(weights.packed_primary, np.uint8), _np(weights.packed_residual, np.uint8)
        norms, seeds = _np(weights.norms, np.float32), _np(weights.seeds, np.uint32)
        cp, cr = _np(primary_codebook.centroids, np.float32), _np(residual_codebook.centroids, np.float32)
        if pp.shape[0] != out_features or pr.shape != (out_features, in_features // 2):
            raise ValueError("packed planes do not match in/out features")
        self._h = L.tq_linear_create(in_features, out_features, _ptr(pp), pp.shape[1], _ptr(pr), _ptr(norms),
                                     _ptr(seeds), _ptr(cp), cp.size, _ptr(cr), cr.size, block_size)
        if not self._h:
            raise TQError("TurboQuantLinear: " + _lib.last_error())
        self.in_features_, self.out_features_ = in_features, out_features

    def in_features(self) -> int:
        return self.in_features_

    def out_features(self) -> int:
        return self.out_features_

    @property
    def handle(self):
        return self._h

    def forward(self, x, out=None, stream=None):
        """[batch, in] fp32/fp16 -> fp16 [batch, out] (src/linear.cpp:20-26)."""
        if not _is_torch(x):
            x = np.ascontiguousarray(x)
            if x.dtype not in (np.float32, np.float16):
                x = x.astype(np.float32)
        if x.shape[-1] != self.in_features_:
            raise ValueError("input feature size mismatch")
        batch = int(np.prod(x.shape[:-1])) if len(x.shape) > 1 else 1
        if out is None:
            if _is_torch(x):
                import torch
                out = torch.empty((batch, self.out_features_), dtype=torch.float16, device=x.device)
            else:
                out = np.empty((batch, self.out_features_), np.float16)
        check(self._L.tq_linear_forward(self._h, _ptr(x), _dtype_tag(x), batch, _ptr(out), _stream_ptr(stream)),
              "TurboQuantLinear.forward")
        return out

    def dequantize(self, dtype=np.float32, out=None, stream=None):
        """dequantize_weight_cpu's result (src/dequantizer.cpp:52-256) as fp32, or fp16 (RN cast)."""
        if out is None:
            out = np.empty((self.out_features_, self.in_features_), dtype)
        check(self._L.tq_linear_dequantize(self._h, _ptr(out), _dtype_tag(out), _stream_ptr(stream)), "dequantize")
        return out

    def forward_scatter(self, x, dst_ptrs, dst_row_stride: int, row_offset: int, stream=None, signal_ptrs=None,
                        signal_slot: int = 0, signal_value: int = 0):
        """Decode forward (device fp16 x, at most 8 rows) written straight into several buffers:
        output row r of activation row n lands at dst[d][n * dst_row_stride + row_offset + r] for
        every raw device pointer d in dst_ptrs (this rank's buffer and the peers' mapped ones:
        sharding.SharedBuffer).  Replaces "forward, then all-gather" for row-sharded layers."""
        batch = int(np.prod(x.shape[:-1])) if len(x.shape) > 1 else 1
        arr = (C.c_void_p * len(dst_ptrs))(*[int(d) for d in dst_ptrs])
        if signal_ptrs is None:
            check(self._L.tq_linear_forward_scatter(self._h, _ptr(x), batch, arr, len(dst_ptrs), int(dst_row_stride),
                                                    int(row_offset), _stream_ptr(stream)), "TurboQuantLinear.forward_scatter")
            return
        # with a completion signal: flag `signal_slot` of every destination's flag array is set to
        # signal_value once all results are stored (see wait_peers)
        sig = (C.c_void_p * len(signal_ptrs))(*[int(d) for d in signal_ptrs])
        check(self._L.tq_linear_forward_scatter_signal(self._h, _ptr(x), batch, arr, len(dst_ptrs), int(dst_row_stride),
                                                       int(row_offset), sig, int(signal_slot), int(signal_value) & 0xFFFFFFFF,
                                                       _stream_ptr(stream)), "TurboQuantLinear.forward_scatter")

    def forward_strided(self, x, y_ptr: int, y_row_stride: int, stream=None):
        """Device fp16 x [batch, in]; the fp16 result goes to raw device address y_ptr with
        activation rows y_row_stride elements apart (this layer's rows inside a wider buffer)."""
        batch = int(np.prod(x.shape[:-1])) if len(x.shape) > 1 else 1
        check(self._L.tq_linear_forward_strided(self._h, _ptr(x), batch, C.c_void_p(int(y_ptr)), int(y_row_stride),
                                                _stream_ptr(stream)), "TurboQuantLinear.forward_strided")

    def wait_peers(self, local_flags_ptr: int, n_flags: int, value: int, stream=None):
        """Enqueue the (bounded) wait for the completion flags of n_flags ranks in this rank's own
        flag array to reach `value`; afterwards, on that stream, every rank's scattered results are
        visible here.  A timeout shows up in check_status()."""
        check(self._L.tq_linear_wait_peers(self._h, C.c_void_p(int(local_flags_ptr)), int(n_flags), int(value) & 0xFFFFFFFF,
                                           _stream_ptr(stream)), "TurboQuantLinear.wait_peers")

    def check_status(self):
        """Waits for the device and raises if any kernel launched through this layer refused to
        run or gave up on a bounded wait (calls with host output check this themselves)."""
        check(self._L.tq_linear_status(self._h), "TurboQuantLinear.check_status")

    def close(self):
        if getattr(self, "_h", None):
            self._L.tq_linear_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def forward_group(linears, x, outs=None, stream=None):
    """Several TurboQuantLinear layers on the same device activation x ([batch, in] fp16 torch tensor) in one launch
    of each kernel of the path (tq_linear_forward_group): returns the list of fp16 [batch, out_i] results, each bit-equal
    to linears[i].forward(x).  The layers must share in_features, the WHT block and the rotation mode (q / k / v, gate / up)."""
    import torch
    if not linears or len(linears) > 4:
        raise ValueError("forward_group takes 1..4 layers")
    batch = int(np.prod(x.shape[:-1])) if len(x.shape) > 1 else 1
    if outs is None:
        outs = [torch.empty((batch, lin.out_features_), dtype=torch.float16, device=x.device) for lin in linears]
    hs = (C.c_void_p * len(linears))(*[lin._h for lin in linears])
    ys = (C.c_void_p * len(linears))(*[o.data_ptr() for o in outs])
    check(linears[0]._L.tq_linear_forward_group(hs, len(linears), _ptr(x), batch, ys, _stream_ptr(stream)), "forward_group")
    return outs


def dequantize_weight(qw: QuantizedWeight, primary_codebook: Codebook, residual_codebook: Codebook, block_size: int,
                      dtype=np.float32):
    """dequantize_weight_cpu / _gpu (include/turboquant/dequantizer.h:11-22) -> [out, in]."""
    out_f = qw.packed_primary.shape[0]
    in_f = qw.packed_residual.shape[1] * 2
    lin = TurboQuantLinear(in_f, out_f, qw, primary_codebook, residual_codebook, block_size)
    try:
        return lin.dequantize(dtype)
    finally:
        lin.close()


# ---- KV cache --------------------------------------------------------------------------------

class TQKVCache:
    """turboquant::TQKVCache (include/turboquant/kv_cache.h:42-133): one sequence."""

    def __init__(self, num_layers: int, num_heads: int, head_dim: int, kv_bits: int = 3,
                 max_context: int = 1048576, decode_window: int = 131072):
        L = _lib.load()
        self._L = L
        self.num_layers, self.num_heads, self.head_dim = num_layers, num_heads, head_dim
        self._h = L.tq_kv_cache_create(num_layers, num_heads, head_dim, kv_bits, max_context, decode_window)
        if not self._h:
            raise TQError("TQKVCache: " + _lib.last_error())

    @property
    def handle(self):
        return self._h

    def append(self, layer: int, keys, values, stream=None):
        """[tokens, heads, head_dim] fp32/fp16 (src/kv_cache.cpp:16-61)."""
        if not _is_torch(keys):
            keys, values = np.ascontiguousarray(keys), np.ascontiguousarray(values)
        if tuple(keys.shape) != tuple(values.shape) or tuple(keys.shape[1:]) != (self.num_heads, self.head_dim):
            raise ValueError("keys/values must be [tokens, heads, head_dim]")
        if not 0 <= layer < self.num_layers:
            raise IndexError("Layer index out of range")
        check(self._L.tq_kv_append(self._h, layer, _ptr(keys), _ptr(values), _dtype_tag(keys), int(keys.shape[0]),
                                   _stream_ptr(stream)), "TQKVCache.append")

    def snapshot(self, model_hash: int = 0, codebook_hash: int = 0) -> np.ndarray:
        """The transferable byte stream of the whole cache (TQKVCache::snapshot + snapshot_serialize,
        src/kv_cache.cpp:509-524, src/cache_snapshot.cpp:62-83), as a uint8 array."""
        n = self._L.tq_kv_snapshot(self._h, None, 0, model_hash, codebook_hash)
        if n < 0:
            raise _lib.TQError("TQKVCache.snapshot: " + _lib.last_error())
        out = np.zeros(n, np.uint8)
        if self._L.tq_kv_snapshot(self._h, _ptr(out), n, model_hash, codebook_hash) != n:
            raise _lib.TQError("TQKVCache.snapshot: " + _lib.last_error())
        return out

    def restore(self, data):
        """Replace the contents with a snapshot stream (ours or the reference's)."""
        data = np.ascontiguousarray(data, np.uint8)
        if self._L.tq_kv_restore(self._h, _ptr(data), data.size) != 0:
            raise ValueError("TQKVCache.restore: " + _lib.last_error())

    def delta(self, start: int, end: int) -> np.ndarray:
        """Positions [start, end) of every layer as the reference's delta byte stream (TQKVCache::delta +
        delta_serialize, src/kv_cache.cpp:566-581, src/cache_snapshot.cpp:110-123)."""
        n = self._L.tq_kv_delta(self._h, None, 0, int(start), int(end))
        if n < 0:
            raise _lib.TQError("TQKVCache.delta: " + _lib.last_error())
        out = np.zeros(n, np.uint8)
        if self._L.tq_kv_delta(self._h, _ptr(out), n, int(start), int(end)) != n:
            raise _lib.TQError("TQKVCache.delta: " + _lib.last_error())
        return out

    def apply_delta(self, data):
        """Append a delta stream (ours or the reference's) to every layer."""
        data = np.ascontiguousarray(data, np.uint8)
        if self._L.tq_kv_apply_delta(self._h, _ptr(data), data.size) != 0:
            raise ValueError("TQKVCache.apply_delta: " + _lib.last_error())

    def reserve(self, layer: int, tokens: int, stream=None):
        """Make room for `tokens` tokens of `layer` up front (growth otherwise doubles and copies)."""
        check(self._L.tq_kv_reserve(self._h, layer, int(tokens), _stream_ptr(stream)), "TQKVCache.reserve")

    ATTENTION_AUTO, ATTENTION_LOADS, ATTENTION_PIPELINE, ATTENTION_TENSOR_MEMORY = 0, 1, 2, 3

    def set_attention_kernel(self, kernel: int):
        """Decode-attention kernel for calls that name this cache first: automatic (by job size),
        the load-based kernel, the bulk-copy pipeline, or the tensor-memory kernel (head_dim 128, four KV
        heads; other shapes fall back to the automatic choice)."""
        check(self._L.tq_kv_set_attention_kernel(self._h, int(kernel)), "TQKVCache.set_attention_kernel")

    def check_attention_status(self):
        """Raise if a finished attention call on this cache reported a device-side failure."""
        check(self._L.tq_kv_attention_status(self._h), "TQKVCache.check_attention_status")

    def seq_length(self) -> int:
        return self._L.tq_kv_cache_seq_length(self._h)

    def _get(self, layer, values, start, end, out, stream):
        if not 0 <= layer < self.num_layers:
            raise IndexError("Layer index out of range")
        if out is None:
            out = np.empty((max(end - start, 0), self.num_heads, self.head_dim), np.float16)
        rc = self._L.tq_kv_get_fp16(self._h, layer, int(values), start, end, _ptr(out), _stream_ptr(stream))
        if rc:
            raise IndexError(_lib.last_error())
        return out

    def get_keys_fp16(self, layer, start, end, out=None, stream=None):
        return self._get(layer, False, start, end, out, stream)

    def get_values_fp16(self, layer, start, end, out=None, stream=None):
        return self._get(layer, True, start, end, out, stream)

    def export(self, layer: int) -> dict:
        """Raw storage in the reference's layout (include/turboquant/kv_cache.h:25-36)."""
        n = self._L.tq_kv_export(self._h, layer, None, None, None, None, None, None)
        if n < 0:
            raise TQError(_lib.last_error())
        nv = n * self.num_heads
        wph, qph = (self.head_dim + 9) // 10, (self.head_dim + 31) // 32
        d = dict(k_words=np.zeros((nv, wph), np.uint32), v_words=np.zeros((nv, wph), np.uint32),
                 k_norms=np.zeros(nv, np.float32), v_norms=np.zeros(nv, np.float32),
                 qjl_words=np.zeros((nv, qph), np.uint32), qjl_norms=np.zeros(nv, np.float32))
        self._L.tq_kv_export(self._h, layer, _ptr(d["k_words"]), _ptr(d["v_words"]), _ptr(d["k_norms"]),
                             _ptr(d["v_norms"]), _ptr(d["qjl_words"]), _ptr(d["qjl_norms"]))
        d["tokens"] = n
        return d

    def close(self):
        if getattr(self, "_h", None):
            self._L.tq_kv_cache_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DecodeBuffer:
    """The fp16 decode window (include/turboquant/decode_buffer.h:11-47) in device memory: a ring of
    `window_size` token slots shadowing the most recent tokens of a sequence, so that short contexts
    are attended without touching the compressed cache."""

    def __init__(self, window_size: int, num_heads: int, head_dim: int):
        self._L = _lib.load()
        self.num_heads, self.head_dim = int(num_heads), int(head_dim)
        self._h = self._L.tq_decode_buffer_create(int(window_size), self.num_heads, self.head_dim)
        if not self._h:
            raise TQError("DecodeBuffer: " + _lib.last_error())

    @property
    def handle(self):
        return self._h

    def window_size(self) -> int:
        return self._L.tq_decode_buffer_window_size(self._h)

    def current_length(self) -> int:
        return self._L.tq_decode_buffer_current_length(self._h)

    def _kv(self, keys, values, ndim):
        if not _is_torch(keys):
            keys = np.ascontiguousarray(keys)
            values = np.ascontiguousarray(values)
        if tuple(keys.shape) != tuple(values.shape) or len(keys.shape) != ndim or tuple(keys.shape[-2:]) != (self.num_heads, self.head_dim):
            raise ValueError("keys and values must both be [..., num_heads, head_dim]")
        return keys, values

    def rebuild(self, keys, values, stream=None):
        """keys / values [tokens, heads, head_dim]: fill the window from a decompressed prefix
        (src/decode_buffer.cpp:16-47)."""
        keys, values = self._kv(keys, values, 3)
        check(self._L.tq_decode_buffer_rebuild(self._h, _ptr(keys), _ptr(values), _dtype_tag(keys), int(keys.shape[0]),
                                               _stream_ptr(stream)), "DecodeBuffer.rebuild")

    def append_token(self, key, value, stream=None):
        """One token, [1, heads, head_dim] or [heads, head_dim] (src/decode_buffer.cpp:49-70)."""
        if len(key.shape) == 3:
            key, value = key[0], value[0]
        key, value = self._kv(key, value, 2)
        check(self._L.tq_decode_buffer_append_token(self._h, _ptr(key), _ptr(value), _dtype_tag(key), _stream_ptr(stream)),
              "DecodeBuffer.append_token")

    def slide_window(self, new_keys, new_values, stream=None):
        """Overwrite the oldest slots with [tokens, heads, head_dim] (src/decode_buffer.cpp:72-103)."""
        new_keys, new_values = self._kv(new_keys, new_values, 3)
        check(self._L.tq_decode_buffer_slide_window(self._h, _ptr(new_keys), _ptr(new_values), _dtype_tag(new_keys),
                                                    int(new_keys.shape[0]), _stream_ptr(stream)), "DecodeBuffer.slide_window")

    def _read(self, fn, what, start, end):
        n = max(int(end) - int(start), 0)
        out = np.empty((n, self.num_heads, self.head_dim), np.float16)
        if fn(self._h, int(start), int(end), _ptr(out) if n else None, None) != 0:
            raise IndexError(f"DecodeBuffer.{what}: " + _lib.last_error())
        return out

    def keys(self, start: int, end: int):
        """fp16 [end - start, heads, head_dim]; IndexError unless 0 <= start < end <= current_length()."""
        return self._read(self._L.tq_decode_buffer_keys, "keys", start, end)

    def values(self, start: int, end: int):
        return self._read(self._L.tq_decode_buffer_values, "values", start, end)

    def close(self):
        if self._h:
            self._L.tq_decode_buffer_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def hybrid_attention(cache, buffer, layer: int, queries, out=None, stream=None):
    """hybrid_attention (src/attention_dispatch.cpp:21-74) for one query position: queries
    [q_heads, head_dim] -> fp16 [q_heads, head_dim].  Contexts that fit the decode window are attended
    there, longer ones over the compressed cache."""
    L = _lib.load()
    if not _is_torch(queries):
        queries = np.ascontiguousarray(queries)
    if len(queries.shape) != 2 or queries.shape[-1] != cache.head_dim:
        raise ValueError("queries must be [q_heads, head_dim]")
    if out is None:
        if _is_torch(queries):
            import torch
            out = torch.empty(tuple(queries.shape), dtype=torch.float16, device=queries.device)
        else:
            out = np.empty(queries.shape, np.float16)
    check(L.tq_hybrid_attention(cache.handle, buffer.handle, layer, _ptr(queries), _dtype_tag(queries), int(queries.shape[0]),
                                _ptr(out), _stream_ptr(stream)), "hybrid_attention")
    return out


def append_batch(caches, layer: int, keys, values, stream=None):
    """One decode step of a batch: row i of keys / values ([n_seqs, heads, head_dim], device
    tensors) is appended as one token to caches[i]; two kernel launches per 32 sequences."""
    L = _lib.load()
    n = len(caches)
    if int(keys.shape[0]) != n or int(values.shape[0]) != n:
        raise ValueError("keys and values must have one row per cache")
    arr = (C.c_void_p * n)(*[c.handle for c in caches])
    check(L.tq_kv_append_batch(arr, n, layer, _ptr(keys), _ptr(values), _dtype_tag(keys), _stream_ptr(stream)), "append_batch")


def compressed_attention(caches, layer: int, queries, start: int = 0, end: int = -1, use_qjl: bool = False,
                         out=None, stream=None, return_lse: bool = False):
    """Decode attention over the compressed caches of a batch of sequences: the long-context
    branch of hybrid_attention (src/attention_dispatch.cpp:58-73) without materialising K/V.
    queries: [n_seqs, q_heads, head_dim] -> fp16 of the same shape.  With return_lse the result
    is (out, lse): lse[n_seqs, q_heads] fp32 is the log of each row's softmax denominator, which
    lets results over disjoint token ranges be merged (sharding.merge_attention_parts)."""
    L = _lib.load()
    if isinstance(caches, TQKVCache):
        caches = [caches]
    n = len(caches)
    if not _is_torch(queries):
        queries = np.ascontiguousarray(queries)
    if queries.shape[0] != n or queries.shape[-1] != caches[0].head_dim:
        raise ValueError("queries must be [n_seqs, q_heads, head_dim]")
    q_heads = int(queries.shape[1])
    if out is None:
        if _is_torch(queries):
            import torch
            out = torch.empty(tuple(queries.shape), dtype=torch.float16, device=queries.device)
        else:
            out = np.empty(queries.shape, np.float16)
    arr = (C.c_void_p * n)(*[c.handle for c in caches])
    if not return_lse:
        check(L.tq_kv_attention(arr, n, layer, _ptr(queries), _dtype_tag(queries), q_heads, _ptr(out), start, end,
                                int(use_qjl), _stream_ptr(stream)), "compressed_attention")
        return out
    if _is_torch(queries):
        import torch
        lse = torch.empty((n, q_heads), dtype=torch.float32, device=queries.device)
    else:
        lse = np.empty((n, q_heads), np.float32)
    check(L.tq_kv_attention_lse(arr, n, layer, _ptr(queries), _dtype_tag(queries), q_heads, _ptr(out), _ptr(lse), start,
                                end, int(use_qjl), _stream_ptr(stream)), "compressed_attention")
    return out, lse
