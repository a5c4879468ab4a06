"""CPU tests of the C-ABI library: it loads, exports every symbol the two headers declare,
and its host-only entry points behave like the reference's C layer (NULL-safety, error
returns, planner) — mirroring tests/c_api/*.c of the reference.  No GPU work here."""
import ctypes as C
import os
import re
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADERS = [os.path.join(ROOT, "include", "turboquant_c", h) for h in ("turboquant_c.h", "turboquant_b200.h")]


def declared_symbols():
    names = set()
    for h in HEADERS:
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


@pytest.fixture(scope="module")
def lib():
    from turboquant_mlx_core_b200 import _lib
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    syms = declared_symbols()
    assert len(syms) >= 45
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in a header but not exported"


def test_reference_symbol_list_is_complete(lib):
    from turboquant_mlx_core_b200._lib import SYMBOLS_C
    decl = set(declared_symbols())
    for s in SYMBOLS_C:       # the reference's symbols (its turboquant_c.h:25-136)
        assert s in decl and hasattr(lib, s)


def test_version_and_null_safety(lib):
    assert lib.tq_version() == b"0.1.0"
    for fn in ("tq_model_free", "tq_kv_cache_free", "tq_distributed_free", "tq_cluster_free", "tq_array_free",
               "tq_linear_free"):
        getattr(lib, fn)(None)
    assert lib.tq_kv_cache_seq_length(None) == 0
    assert lib.tq_distributed_rank(None) == 0
    assert lib.tq_distributed_world_size(None) == 1
    assert lib.tq_kv_cache_get_keys_fp16(None, 0, 0, 1) is None
    assert lib.tq_kv_cache_attention(None, 0, None, 0, 1) is None
    lib.tq_kv_cache_append(None, 0, None, None)
    # the tensor-level entry points refuse NULL arguments with a message instead of touching the device
    assert lib.tq_linear_forward_group(None, 3, None, 1, None, None) != 0
    assert b"NULL" in lib.tq_last_error()
    assert lib.tq_rope_qk_f16(None, None, None, 1, 1, 1, 128, 1e6, None) != 0
    assert lib.tq_exchange_sum_f16_rmsnorm(None, 1, 0, 1, 8, None, None, None, None, 1e-6, None) != 0


def test_model_handle(lib):
    assert lib.tq_model_load(None) is None
    assert lib.tq_model_load(b"/definitely/not/here") is None
    with tempfile.NamedTemporaryFile() as f:
        assert lib.tq_model_load(f.name.encode()) is None          # a file is not a model directory
    with tempfile.TemporaryDirectory() as d:
        m = lib.tq_model_load(d.encode())
        assert m
        assert lib.tq_model_forward(m, None) is None               # stub in the reference as well
        assert lib.tq_model_layer_count(m) == 0 and lib.tq_model_layer_name(m, 0) is None
        assert lib.tq_model_layer(m, b"nope") is None
        lib.tq_model_free(m)
        # shards that are not TurboQuant shards (or passthrough companions) are skipped; a malformed
        # header is refused with a message, not a crash
        import struct
        with open(os.path.join(d, "plain.safetensors"), "wb") as f:
            h = b'{"x":{"dtype":"F32","shape":[2],"data_offsets":[0,8]}}'
            f.write(struct.pack("<Q", len(h)) + h + b"\0" * 8)
        with open(os.path.join(d, "m_passthrough.safetensors"), "wb") as f:
            f.write(b"garbage that is never parsed")
        m = lib.tq_model_load(d.encode())
        assert m and lib.tq_model_layer_count(m) == 0
        lib.tq_model_free(m)
        for bad in (b"short", struct.pack("<Q", 1 << 40) + b"{}", struct.pack("<Q", 5) + b'{"a":',
                    struct.pack("<Q", 62) + b'{"x":{"dtype":"F32","shape":[2],"data_offsets":[0,800000000]}}'):
            with open(os.path.join(d, "bad.safetensors"), "wb") as f:
                f.write(bad)
            assert lib.tq_model_load(d.encode()) is None
            assert b"tq_model_load" in lib.tq_last_error()
            assert lib.tq_model_dequant(d.encode(), os.path.join(d, "out").encode()) == 1   # a broken shard: 1, as in the reference
        os.remove(os.path.join(d, "bad.safetensors"))
        # a directory without shards: nothing to dequantise, side files are copied (needs no GPU)
        with open(os.path.join(d, "tokenizer.json"), "w") as f:
            f.write("{}")
        assert lib.tq_model_dequant(d.encode(), os.path.join(d, "plain").encode()) == 0
        assert open(os.path.join(d, "plain", "tokenizer.json")).read() == "{}"
        assert lib.tq_model_dequant(os.path.join(d, "missing").encode(), d.encode()) == 1
    assert lib.tq_model_dequant(None, None) != 0


def test_coordinator(lib):
    c = lib.tq_distributed_init_local()
    assert c and lib.tq_distributed_rank(c) == 0 and lib.tq_distributed_world_size(c) == 1
    lib.tq_distributed_free(c)
    assert lib.tq_distributed_init(None, b"auto") is None


def test_cluster_planner(lib):
    assert lib.tq_cluster_create(0, 8, 64) is None
    assert lib.tq_cluster_create(32, -1, 64) is None
    c = lib.tq_cluster_create(32, 8, 128)
    assert c and lib.tq_cluster_node_count(c) == 0
    assert lib.tq_cluster_plan(c) == -1                            # no nodes yet
    assert lib.tq_cluster_get_layer_start(c, 0) == -1
    assert lib.tq_cluster_add_node(c, None, 64.0) == -1
    assert lib.tq_cluster_add_node(c, b"a", 0.0) == -1
    assert lib.tq_cluster_add_node(c, b"a", 96.0) == 0
    assert lib.tq_cluster_add_node(c, b"b", 32.0) == 0
    assert lib.tq_cluster_plan(c) == 0
    assert lib.tq_cluster_plan(c) == -1                            # plan-once
    assert lib.tq_cluster_add_node(c, b"c", 8.0) == -1
    assert (lib.tq_cluster_get_layer_start(c, 0), lib.tq_cluster_get_layer_end(c, 0)) == (0, 24)
    assert (lib.tq_cluster_get_layer_start(c, 1), lib.tq_cluster_get_layer_end(c, 1)) == (24, 32)
    assert lib.tq_cluster_get_layer_end(c, 2) == -1
    lib.tq_cluster_free(c)
    c = lib.tq_cluster_create(5, 1, 32)
    lib.tq_cluster_add_node(c, b"only", 1.0)
    assert lib.tq_cluster_plan(c) == 0 and lib.tq_cluster_get_layer_end(c, 0) == 5
    lib.tq_cluster_free(c)


def test_codebook_entry_point_needs_no_gpu(lib, golden):
    for bits in range(1, 6):
        c = np.zeros(1 << bits, np.float32)
        b = np.zeros(max((1 << bits) - 1, 1), np.float32)
        assert lib.tq_codebook_generate(bits, c.ctypes.data, b.ctypes.data) == 0
        assert np.array_equal(c, golden[f"codebook{bits}_centroids"])
        assert np.array_equal(b[: (1 << bits) - 1], golden[f"codebook{bits}_boundaries"])
    assert lib.tq_codebook_generate(6, c.ctypes.data, b.ctypes.data) != 0
    assert b"bit width" in lib.tq_last_error()


def test_library_is_standalone():
    """The product library must not depend on torch, MLX or the checker libraries."""
    import subprocess
    from turboquant_mlx_core_b200 import LIB_PATH
    r = subprocess.run(["ldd", LIB_PATH], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    # the NAMES of the dependencies (the left-hand side of "name => path"): a directory on the way to a system library
    # may be called anything
    names = [os.path.basename(line.split()[0]) for line in r.stdout.splitlines() if line.strip()]
    assert names, r.stdout
    for banned in ("torch", "mlx", "tq_oracle", "tq_ref", "c10"):
        assert not any(banned in n for n in names), names


def test_headers_are_plain_c(tmp_path):
    """Both public headers compile as C99 with nothing but the standard headers, and a C
    translation unit can take the address of every declared function (the drop-in boundary is
    a C ABI: no C++ and no CUDA types in the signatures)."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    inc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    syms = declared_symbols()
    src = tmp_path / "abi.c"
    src.write_text('#include "turboquant_c/turboquant_c.h"\n#include "turboquant_c/turboquant_b200.h"\n'
                   "const void* table[] = {\n" + "".join(f"    (const void*)&{s},\n" for s in syms) + "};\n"
                   "int n_symbols(void) { return (int)(sizeof table / sizeof table[0]); }\n")
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-Wno-pedantic", "-I", inc, "-c", str(src), "-o",
                        str(tmp_path / "abi.o")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
