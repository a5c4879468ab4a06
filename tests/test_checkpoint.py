"""TurboQuant safetensors checkpoints: names, dtypes, metadata and loading rules of the reference's
writer and reader (src/serialization.cpp:19-97, src/turboquant_c_dequant.cpp:68-185).  The file
format itself is cross-checked against the `safetensors` package in both directions."""
import os

import numpy as np
import pytest

from tests.conftest import rel_l2


def _layers(oracle, rng):
    cb4, cb5, cb3 = oracle.codebook(4)[0], oracle.codebook(5)[0], oracle.codebook(3)[0]
    out = {}
    for name, rows, cols, bs, pb, rb, shared, cbp, cbr in [
            ("model.layers.0.self_attn.q_proj", 48, 256, 128, 4, 4, True, cb4, cb4),
            ("model.layers.0.mlp.down_proj", 24, 512, 64, 4, 4, False, cb4, cb4),
            ("lm_head", 40, 128, 32, 5, 3, True, cb5, cb3)]:
        w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float16).astype(np.float32)
        pp, pr, norms, seeds = oracle.quantize_weight(w, cbp, cbr, pb, rb, bs, shared)
        out[name] = (pp, pr, norms, seeds, cbp, cbr, bs)
    return out


def _write_model(tq, ckpt, oracle, tmp_path, rng):
    layers = _layers(oracle, rng)
    cb4 = tq.codebook_from_centroids(oracle.codebook(4)[0])
    weights = {n: tq.QuantizedWeight(pp, pr, norms, seeds) for n, (pp, pr, norms, seeds, *_rest) in layers.items()}
    per_layer = {"lm_head": (tq.codebook_from_centroids(layers["lm_head"][4]), tq.codebook_from_centroids(layers["lm_head"][5]))}
    shard = os.path.join(tmp_path, "model-00001-of-00001.safetensors")
    ckpt.write_tq_safetensors(shard, weights, cb4, cb4, per_layer)
    norm_w = rng.standard_normal(256).astype(np.float32)
    ckpt.write_safetensors(os.path.join(tmp_path, "model-00001-of-00001_passthrough.safetensors"),
                           {"model.norm.weight": norm_w})
    return layers, shard, norm_w


def test_writer_matches_the_reference_layout_and_the_safetensors_package(oracle, tmp_path):
    import turboquant_mlx_core_b200 as tq
    from turboquant_mlx_core_b200 import checkpoint as ckpt
    from safetensors import safe_open
    from safetensors.numpy import load_file, save_file
    rng = np.random.default_rng(1)
    layers, shard, _ = _write_model(tq, ckpt, oracle, str(tmp_path), rng)
    # the real package reads what we wrote: names, dtypes, shapes, bytes, metadata
    got = load_file(shard)
    for name, (pp, pr, norms, seeds, *_r) in layers.items():
        assert got[name + ".packed_primary"].dtype == np.uint8 and np.array_equal(got[name + ".packed_primary"], pp)
        assert np.array_equal(got[name + ".packed_residual"], pr)
        assert got[name + ".norms"].dtype == np.float32 and np.array_equal(got[name + ".norms"].view(np.uint32), norms.view(np.uint32))
        assert got[name + ".seeds"].dtype == np.uint32 and got[name + ".seeds"].shape == (3,) and np.array_equal(got[name + ".seeds"], seeds)
    assert got["tq_codebook_primary"].shape == (16,) and got["lm_head.codebook_primary"].shape == (32,)
    assert got["lm_head.codebook_residual"].shape == (8,)
    with safe_open(shard, framework="numpy") as f:
        meta = f.metadata()
    assert meta == {"quantization_method": "turboquant", "tq_version": "1", "tq_primary_bits": "4", "tq_residual_bits": "4",
                    "tq_total_bits": "8", "tq_per_layer_codebooks": "true"}
    assert ckpt.read_tq_metadata(shard) == meta
    # and we read what the real package writes
    other = os.path.join(str(tmp_path), "by_package.safetensors")
    save_file({k: v for k, v in got.items()}, other, metadata=meta)
    a, b = ckpt.read_tq_safetensors(shard), ckpt.read_tq_safetensors(other)
    assert sorted(a.layers) == sorted(b.layers) == sorted(layers)
    for name in layers:
        for field in ("packed_primary", "packed_residual", "norms", "seeds"):
            assert np.array_equal(getattr(a.layers[name].weights, field), getattr(b.layers[name].weights, field))


def test_reader_applies_the_reference_loading_rules(oracle, tmp_path):
    import turboquant_mlx_core_b200 as tq
    from turboquant_mlx_core_b200 import checkpoint as ckpt
    rng = np.random.default_rng(2)
    layers, shard, norm_w = _write_model(tq, ckpt, oracle, str(tmp_path), rng)
    model, passthrough = ckpt.read_tq_model(str(tmp_path))
    assert sorted(model) == sorted(layers) and list(passthrough) == ["model.norm.weight"]
    assert np.array_equal(passthrough["model.norm.weight"], norm_w)
    for name, (pp, pr, norms, seeds, cbp, cbr, bs) in layers.items():
        l = model[name]
        assert (l.out_features, l.in_features, l.block_size) == (pp.shape[0], pr.shape[1] * 2, bs)
        # per-layer codebooks where stored, the model-level ones otherwise
        assert np.array_equal(l.primary_codebook.centroids, cbp) and np.array_equal(l.residual_codebook.centroids, cbr)
        # the loaded layer dequantises to the same weights as the arrays it was written from
        want = oracle.dequantize_weight(pp, pr, norms, seeds, cbp, cbr, bs)
        got = oracle.dequantize_weight(l.weights.packed_primary, l.weights.packed_residual, l.weights.norms, l.weights.seeds,
                                       l.primary_codebook.centroids, l.residual_codebook.centroids, l.block_size)
        assert np.array_equal(want.view(np.uint32), got.view(np.uint32))
    # without the per-layer flag the model-level codebooks win even if per-layer tensors exist
    tensors, meta = ckpt.read_safetensors(shard)
    meta.pop("tq_per_layer_codebooks")
    flat = os.path.join(str(tmp_path), "flat.safetensors")
    ckpt.write_safetensors(flat, tensors, meta)
    assert ckpt.read_tq_safetensors(flat).layers["lm_head"].primary_codebook.centroids.size == 16
    # a file without the TurboQuant marker is not a TQ shard; a layer lacking a tensor is refused
    plain = os.path.join(str(tmp_path), "plain.safetensors")
    ckpt.write_safetensors(plain, {"x": np.zeros(3, np.float32)})
    assert ckpt.read_tq_metadata(plain) == {}
    with pytest.raises(ValueError):
        ckpt.read_tq_safetensors(plain)
    del tensors["lm_head.norms"]
    broken = os.path.join(str(tmp_path), "broken.safetensors")
    ckpt.write_safetensors(broken, tensors, {"quantization_method": "turboquant"})
    with pytest.raises(ValueError):
        ckpt.read_tq_safetensors(broken)
    with pytest.raises(ValueError):
        ckpt.read_tq_model(plain)


@pytest.mark.gpu
def test_load_linears_runs_the_loaded_layers(tq, oracle, tmp_path):
    from turboquant_mlx_core_b200 import checkpoint as ckpt
    rng = np.random.default_rng(3)
    layers, shard, _ = _write_model(tq, ckpt, oracle, str(tmp_path), rng)
    for source in (shard, str(tmp_path)):
        lins = ckpt.load_linears(source)
        assert sorted(lins) == sorted(layers)
        for name, (pp, pr, norms, seeds, cbp, cbr, bs) in layers.items():
            x = rng.standard_normal((3, pr.shape[1] * 2)).astype(np.float16)
            want = oracle.linear_from_dequant(oracle.dequantize_weight(pp, pr, norms, seeds, cbp, cbr, bs), x.astype(np.float32))
            assert rel_l2(lins[name].forward(x), want) < 1e-3, name      # the linear layer's stated tolerance
        for l in lins.values():
            l.close()


@pytest.mark.gpu
def test_c_model_load_uploads_every_layer(tq, oracle, tmp_path):
    """tq_model_load over a model directory (C++ safetensors reader): layer names, shapes, and the
    forward of each loaded handle against the oracle; files written by the `safetensors` package load too."""
    import ctypes as C
    from safetensors.numpy import load_file, save_file
    from turboquant_mlx_core_b200 import checkpoint as ckpt
    rng = np.random.default_rng(4)
    layers, shard, _ = _write_model(tq, ckpt, oracle, str(tmp_path), rng)
    L = tq.load()
    for rewrite in (False, True):
        if rewrite:   # the same shard as the safetensors package lays it out (different header order and padding)
            save_file(load_file(shard), shard, metadata=ckpt.read_tq_metadata(shard))
        m = L.tq_model_load(str(tmp_path).encode())
        assert m, L.tq_last_error()
        n = L.tq_model_layer_count(m)
        names = sorted(L.tq_model_layer_name(m, i).decode() for i in range(n))
        assert names == sorted(layers)
        for name, (pp, pr, norms, seeds, cbp, cbr, bs) in layers.items():
            h = L.tq_model_layer(m, name.encode())
            assert h and L.tq_linear_in_features(h) == pr.shape[1] * 2 and L.tq_linear_out_features(h) == pp.shape[0]
            x = rng.standard_normal((2, pr.shape[1] * 2)).astype(np.float16)
            y = np.zeros((2, pp.shape[0]), np.float16)
            assert L.tq_linear_forward(h, x.ctypes.data_as(C.c_void_p), tq.TQ_F16, 2, y.ctypes.data_as(C.c_void_p), None) == 0
            want = oracle.linear_from_dequant(oracle.dequantize_weight(pp, pr, norms, seeds, cbp, cbr, bs), x.astype(np.float32))
            assert rel_l2(y, want) < 1e-3, name
        assert L.tq_model_layer(m, b"missing") is None
        L.tq_model_free(m)


@pytest.mark.gpu
def test_model_dequant_writes_an_ordinary_model_directory(tq, oracle, tmp_path):
    """tq_model_dequant (src/turboquant_c_dequant.cpp:20-191): side files copied, quantization_config
    stripped from config.json, every quantised layer written as {name}.weight in the passthrough
    tensors' dtype (bfloat16 without any) with the bits of dequantize_weight_cpu + one rounding,
    passthrough tensors merged, foreign shards copied; bad paths give 1."""
    from safetensors.numpy import load_file, save_file
    from turboquant_mlx_core_b200 import checkpoint as ckpt
    rng = np.random.default_rng(6)
    src, dst = os.path.join(str(tmp_path), "tq"), os.path.join(str(tmp_path), "out", "plain")
    os.makedirs(src)
    layers, shard, norm_w = _write_model(tq, ckpt, oracle, src, rng)
    with open(os.path.join(src, "config.json"), "w") as f:
        f.write('{"hidden_size": 256, "quantization_config": {"method": "turboquant", "nested": {"bits": 8}}, "vocab": 40}')
    with open(os.path.join(src, "tokenizer.json"), "w") as f:
        f.write("{}")
    foreign = {"extra.weight": rng.standard_normal((4, 4)).astype(np.float32)}
    save_file(foreign, os.path.join(src, "other.safetensors"))
    L = tq.load()
    assert L.tq_model_dequant(src.encode(), dst.encode()) == 0, L.tq_last_error()
    assert open(os.path.join(dst, "config.json")).read() == '{"hidden_size": 256, "vocab": 40}'
    assert os.path.exists(os.path.join(dst, "tokenizer.json"))
    assert np.array_equal(load_file(os.path.join(dst, "other.safetensors"))["extra.weight"], foreign["extra.weight"])
    got = load_file(os.path.join(dst, os.path.basename(shard)))       # passthrough is fp32 here, so the weights are too
    assert sorted(got) == sorted([n + ".weight" for n in layers] + ["model.norm.weight"])
    assert np.array_equal(got["model.norm.weight"], norm_w)
    for name, (pp, pr, norms, seeds, cbp, cbr, bs) in layers.items():
        want = oracle.dequantize_weight(pp, pr, norms, seeds, cbp, cbr, bs)
        assert got[name + ".weight"].dtype == np.float32
        assert np.array_equal(got[name + ".weight"].view(np.uint32), want.view(np.uint32)), name
    # without a passthrough file the output is bfloat16: the fp32 result rounded to nearest even
    os.remove(os.path.join(src, os.path.basename(shard).replace(".safetensors", "_passthrough.safetensors")))
    dst2 = os.path.join(str(tmp_path), "out2")
    assert L.tq_model_dequant(src.encode(), dst2.encode()) == 0, L.tq_last_error()
    tensors, _ = ckpt.read_safetensors(os.path.join(dst2, os.path.basename(shard)))
    for name, (pp, pr, norms, seeds, cbp, cbr, bs) in layers.items():
        want = oracle.dequantize_weight(pp, pr, norms, seeds, cbp, cbr, bs).view(np.uint32)
        bf = ((want + 0x7FFF + ((want >> 16) & 1)) >> 16).astype(np.uint16)
        assert np.array_equal(np.asarray(tensors[name + ".weight"]).view(np.uint16).reshape(bf.shape), bf), name
    assert L.tq_model_dequant(os.path.join(src, "missing").encode(), dst.encode()) == 1
    assert L.tq_model_dequant(None, dst.encode()) == 1
