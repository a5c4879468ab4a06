"""CPU restatement of the reference's fp16 decode window and of hybrid_attention's window branch.

TEST INFRASTRUCTURE ONLY: imported by tests/ (and nothing else) as the checker of the CUDA path.

DecodeWindow follows src/decode_buffer.cpp line by line (constructor 9-14, rebuild 16-47,
append_token 49-70, slide_window 72-103, extract_range 105-126, keys / values 128-142): fp32
storage, ring slot = absolute token index % window, fp16 on the way out.  window_attention follows
src/attention_dispatch.cpp:37-56 (fp16 queries, keys and values; scores scaled by 1/sqrt(head_dim);
no mask; grouped-query heads share a KV head in blocks, as MLX's scaled_dot_product_attention does).
The reference's own unit tests for this class (tests/unit/test_decode_buffer.cpp) are restated in
tests/test_decode_window.py and run against this file, which pins it.
"""
import numpy as np


class DecodeWindow:
    def __init__(self, window_size, num_heads, head_dim):
        self.window_size, self.num_heads, self.head_dim = window_size, num_heads, head_dim
        self.k = np.zeros((window_size, num_heads, head_dim), np.float32)
        self.v = np.zeros((window_size, num_heads, head_dim), np.float32)
        self.current_length = 0
        self.window_start = 0

    def rebuild(self, keys, values):
        keys = np.asarray(keys).astype(np.float32)
        values = np.asarray(values).astype(np.float32)
        n = keys.shape[0]
        for t in range(min(n, self.window_size)):
            self.k[t % self.window_size] = keys[t]
            self.v[t % self.window_size] = values[t]
        self.current_length = n
        self.window_start = 0

    def append_token(self, key, value):
        slot = self.current_length % self.window_size
        self.k[slot] = np.asarray(key).astype(np.float32).reshape(self.num_heads, self.head_dim)
        self.v[slot] = np.asarray(value).astype(np.float32).reshape(self.num_heads, self.head_dim)
        self.current_length += 1

    def slide_window(self, new_keys, new_values):
        new_keys = np.asarray(new_keys).astype(np.float32)
        new_values = np.asarray(new_values).astype(np.float32)
        n = new_keys.shape[0]
        for t in range(n):
            slot = (self.window_start + t) % self.window_size
            self.k[slot] = new_keys[t]
            self.v[slot] = new_values[t]
        self.window_start = (self.window_start + n) % self.window_size

    def _extract(self, buf, start, end):
        if start < 0 or end <= start or end > self.current_length:
            raise IndexError("DecodeBuffer: requested range is out of bounds")
        slots = [(start + t) % self.window_size for t in range(end - start)]
        return buf[slots].astype(np.float16)

    def keys(self, start, end):
        return self._extract(self.k, start, end)

    def values(self, start, end):
        return self._extract(self.v, start, end)


def window_attention(queries, keys_fp16, values_fp16):
    """queries [q_heads, d] (rounded to fp16), keys / values [tokens, kv_heads, d] fp16 -> fp32 [q_heads, d]."""
    q = np.asarray(queries).astype(np.float16).astype(np.float64)
    k = np.asarray(keys_fp16).astype(np.float64)
    v = np.asarray(values_fp16).astype(np.float64)
    q_heads, d = q.shape
    kv_heads = k.shape[1]
    group = q_heads // kv_heads
    out = np.zeros((q_heads, d), np.float64)
    for h in range(q_heads):
        kh = h // group
        s = (k[:, kh, :] @ q[h]) / np.sqrt(d)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ v[:, kh, :]
    return out.astype(np.float32)
