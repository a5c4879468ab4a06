"""Generate the golden fixtures in this directory from the REFERENCE's own C++.

Runs only where oracle/_ref/libtq_ref.so could be built (i.e. where the reference source
tree is mounted): `python oracle/build.py && python tests/golden/make_golden.py`.
Every array below is produced by the reference code (quantize_weight,
dequantize_weight_cpu, generate_codebook_from_data_cpu, TQKVCache::append / snapshot /
get_keys_fp16 / get_values_fp16), except the `attn_*` entries, which come from the C
restatement in oracle/tq_oracle.c because the reference has no executable fused
attention.  Inputs are regenerated from seeds by the tests (LCG of the reference's own
tests, or numpy's PCG64), so only outputs are stored.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.pyoracle import Oracle, Ref, lcg_matrix  # noqa: E402

WEIGHT_CASES = [
    # name, rows, cols, block, primary_bits, residual_bits, shared_rotation, lcg seed
    ("w64x128_b128_44s", 64, 128, 128, 4, 4, True, 7),
    ("w32x128_b64_44d", 32, 128, 64, 4, 4, False, 11),
    ("w24x384_b128_40", 24, 384, 128, 4, 0, False, 13),
    ("w16x512_b512_44s", 16, 512, 512, 4, 4, True, 17),
    ("w16x896_b128_44s", 16, 896, 128, 4, 4, True, 19),
    ("w16x896_b128_53s", 16, 896, 128, 5, 3, True, 23),
    ("w8x256_b256_53d", 8, 256, 256, 5, 3, False, 29),
    ("w5x64_b32_44s", 5, 64, 32, 4, 4, True, 31),
    ("w3x1024_b1024_44d", 3, 1024, 1024, 4, 4, False, 37),
]


def kv_inputs(seed, tokens, heads, dim):
    """K, V ~ N(0,1) fp16 with 5 % of the channels (fixed per head) scaled x8."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((tokens, heads, dim)).astype(np.float32)
    v = rng.standard_normal((tokens, heads, dim)).astype(np.float32)
    n_out = max(1, int(round(0.05 * dim)))
    for h in range(heads):
        ch = rng.choice(dim, n_out, replace=False)
        k[:, h, ch] *= 8.0
        v[:, h, ch] *= 8.0
    return k.astype(np.float16), v.astype(np.float16)


def gauss_weight(seed, rows, cols):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((rows, cols)) * 0.02).astype(np.float16).astype(np.float32)


def main():
    ref, ora = Ref(), Oracle()
    out = {}
    for bits in range(1, 6):
        c, b = ref.codebook(bits)
        out[f"codebook{bits}_centroids"], out[f"codebook{bits}_boundaries"] = c, b

    for name, rows, cols, bs, pb, rb, shared, seed in WEIGHT_CASES:
        w = lcg_matrix(rows, cols, seed)
        cbp, _ = ref.codebook(pb)
        cbr, _ = ref.codebook(rb if rb else 4)
        pp, pr, norms, seeds = ref.quantize_weight(w, cbp, cbr, pb, rb, bs, shared)
        deq = ref.dequantize_weight(pp, pr, norms, seeds, cbp, cbr, bs)
        out[name + "_pp"], out[name + "_pr"], out[name + "_norms"], out[name + "_seeds"] = pp, pr, norms, seeds
        out[name + "_deq"] = deq
        for inv in (0, 1):
            out[name + f"_wht{inv}"] = ref.wht(w, 12345 + rows, bs, bool(inv))

    # fitted codebooks on Gaussian weights (the recipe of the headline 4096 x 4096 benchmark layer, small)
    w = gauss_weight(0, 64, 512)
    cb4, _ = ref.codebook(4)
    pp, pr, norms, seeds = ref.quantize_weight(w, cb4, cb4, 4, 4, 128, True)
    nrm = np.sqrt((w * w).sum(1, keepdims=True)).astype(np.float32)
    rot = ref.wht((w / np.maximum(nrm, 1e-10)).astype(np.float32), int(seeds[0]), 128) * np.float32(np.sqrt(np.float32(512)))
    rot = rot.astype(np.float32)
    fit_p, _ = ref.fit_codebook(rot, 4)
    idx = ref.codebook_quantize(rot, fit_p)
    fit_r, _ = ref.fit_codebook(rot.ravel() - fit_p[idx], 4)
    pp, pr, norms, seeds = ref.quantize_weight(w, fit_p, fit_r, 4, 4, 128, True)
    out["fit_cb_p"], out["fit_cb_r"] = fit_p, fit_r
    out["fit_pp"], out["fit_pr"], out["fit_norms"], out["fit_seeds"] = pp, pr, norms, seeds
    out["fit_deq"] = ref.dequantize_weight(pp, pr, norms, seeds, fit_p, fit_r, 128)

    # KV cache: reference TQKVCache
    for name, layers, heads, dim, tokens, seed in [("kv4x128", 2, 4, 128, 24, 5), ("kv2x32", 1, 2, 32, 40, 6),
                                                    ("kv1x64", 1, 1, 64, 9, 8)]:
        k, v = kv_inputs(seed, tokens, heads, dim)
        kv = ref.kv(layers, heads, dim)
        lay = layers - 1
        kv.append(lay, k[: tokens // 2], v[: tokens // 2])
        kv.append(lay, k[tokens // 2:], v[tokens // 2:])
        ex = kv.export(lay)
        for key in ("k_words", "v_words", "k_norms", "v_norms", "qjl_words", "qjl_norms"):
            out[f"{name}_{key}"] = ex[key]
        out[f"{name}_keys_fp16"] = kv.get_fp16(lay, False, 0, tokens).view(np.uint16)
        out[f"{name}_values_fp16"] = kv.get_fp16(lay, True, 0, tokens).view(np.uint16)
        # the reference's serialized snapshot of the whole cache (TQCS stream), with fixed identity hashes
        out[f"{name}_snapshot"] = kv.snapshot(model_hash=0x1234ABCD, codebook_hash=0x0BADF00D)
        # ... and its delta of positions [3, tokens - 2) (TQCD stream)
        out[f"{name}_delta"] = kv.delta(3, tokens - 2)
        # attention (C restatement; GQA group 7 for the 4x128 case, 1 otherwise)
        q_heads = heads * (7 if heads == 4 else 1)
        rng = np.random.default_rng(seed + 100)
        q = rng.standard_normal((q_heads, dim)).astype(np.float16).astype(np.float32)
        for qjl in (0, 1):
            out[f"{name}_attn_qjl{qjl}"] = ora.attention(q, heads, ex["k_words"], ex["k_norms"], ex["v_words"],
                                                         ex["v_norms"], ex["qjl_words"], ex["qjl_norms"], layer=lay,
                                                         use_qjl=bool(qjl))
    path = os.path.join(HERE, "golden_v1.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
