"""TurboQuant safetensors checkpoints: the tensor names, dtypes, shapes and metadata keys of the
reference's writer (src/serialization.cpp:19-97) and the loading rules of its dequantising reader
(src/turboquant_c_dequant.cpp:68-185), on the host with numpy.

Per quantised weight `{name}`:
    {name}.packed_primary    uint8   [out, in/2]  (5-bit primary: [out, in], one code per byte)
    {name}.packed_residual   uint8   [out, in/2]
    {name}.norms             float32 [out]
    {name}.seeds             uint32  [3] = {seed_primary, seed_residual, block_size}
model-level `tq_codebook_primary` / `tq_codebook_residual` (float32 centroids), optional per-layer
`{name}.codebook_primary` / `{name}.codebook_residual` (used when the metadata says
tq_per_layer_codebooks = "true"), and a companion `*_passthrough.safetensors` shard per shard for the
tensors that were not quantised.  Metadata: quantization_method = "turboquant", tq_version = "1",
tq_primary_bits, tq_residual_bits, tq_total_bits.

Reading and writing need no GPU; `load_linears` uploads each layer through tq_linear_create.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field

import numpy as np

from . import api

_SUFFIXES = (".packed_primary", ".packed_residual", ".norms", ".seeds")
_DTYPES = {"U8": np.uint8, "F32": np.float32, "U32": np.uint32, "F16": np.float16, "I32": np.int32, "I64": np.int64,
           "U16": np.uint16, "I8": np.int8, "I16": np.int16, "U64": np.uint64, "F64": np.float64, "BOOL": np.bool_}
_NAMES = {np.dtype(v).str: k for k, v in _DTYPES.items()}
DEFAULT_BLOCK_SIZE = 512   # a seeds tensor with fewer than three entries (src/turboquant_c_dequant.cpp:124)


def read_safetensors(path: str) -> tuple[dict[str, np.ndarray], dict[str, str]]:
    """All tensors of one file and its metadata.  bf16 tensors come back as their raw uint16 bits
    (numpy has no bfloat16); everything a TurboQuant shard stores is uint8 / uint32 / float32."""
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: not a safetensors file")
        (n,) = struct.unpack("<Q", raw)
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    meta = {str(k): str(v) for k, v in (header.pop("__metadata__", None) or {}).items()}
    tensors = {}
    for name, info in header.items():
        a, b = info["data_offsets"]
        dt = info["dtype"]
        if b > len(data) or a > b:
            raise ValueError(f"{path}: tensor {name} points outside the file")
        np_dt = np.uint16 if dt == "BF16" else _DTYPES.get(dt)
        if np_dt is None:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {dt}")
        arr = np.frombuffer(data, dtype=np_dt, count=(b - a) // np.dtype(np_dt).itemsize, offset=a)
        tensors[name] = arr.reshape(info["shape"]).copy()
    return tensors, meta


def write_safetensors(path: str, tensors: dict[str, np.ndarray], metadata: dict[str, str] | None = None) -> None:
    header, blobs, pos = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        a = np.ascontiguousarray(tensors[name])
        key = _NAMES.get(a.dtype.str)
        if key is None:
            raise ValueError(f"tensor {name}: dtype {a.dtype} cannot be stored")
        blob = a.tobytes()
        header[name] = {"dtype": key, "shape": list(a.shape), "data_offsets": [pos, pos + len(blob)]}
        blobs.append(blob)
        pos += len(blob)
    h = json.dumps(header, separators=(",", ":")).encode("utf-8")
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for blob in blobs:
            f.write(blob)


def read_tq_metadata(path: str) -> dict[str, str]:
    """read_tq_metadata (src/serialization.cpp:12-15): empty when the file has none."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        return {str(k): str(v) for k, v in (json.loads(f.read(n).decode("utf-8")).get("__metadata__") or {}).items()}


def is_tq_shard(metadata: dict[str, str]) -> bool:
    return metadata.get("quantization_method") == "turboquant"


def write_tq_safetensors(path: str, weights: dict[str, api.QuantizedWeight], primary_codebook: api.Codebook,
                         residual_codebook: api.Codebook,
                         per_layer_codebooks: dict[str, tuple[api.Codebook, api.Codebook]] | None = None) -> None:
    """write_tq_safetensors (src/serialization.cpp:32-97): same tensor names and metadata keys."""
    tensors: dict[str, np.ndarray] = {}
    for name, qw in weights.items():
        tensors[name + ".packed_primary"] = np.asarray(qw.packed_primary, np.uint8)
        tensors[name + ".packed_residual"] = np.asarray(qw.packed_residual, np.uint8)
        tensors[name + ".norms"] = np.asarray(qw.norms, np.float32)
        tensors[name + ".seeds"] = np.asarray(qw.seeds, np.uint32)
    for name, (cp, cr) in (per_layer_codebooks or {}).items():
        tensors[name + ".codebook_primary"] = np.asarray(cp.centroids, np.float32)
        tensors[name + ".codebook_residual"] = np.asarray(cr.centroids, np.float32)
    tensors["tq_codebook_primary"] = np.asarray(primary_codebook.centroids, np.float32)
    tensors["tq_codebook_residual"] = np.asarray(residual_codebook.centroids, np.float32)
    meta = {"quantization_method": "turboquant", "tq_version": "1", "tq_primary_bits": str(primary_codebook.bits),
            "tq_residual_bits": str(residual_codebook.bits),
            "tq_total_bits": str(primary_codebook.bits + residual_codebook.bits)}
    if per_layer_codebooks:
        meta["tq_per_layer_codebooks"] = "true"
    write_safetensors(path, tensors, meta)


@dataclass
class TQLayer:
    """One quantised weight of a shard with the codebooks it decodes with."""
    name: str
    weights: api.QuantizedWeight
    primary_codebook: api.Codebook
    residual_codebook: api.Codebook
    block_size: int

    @property
    def out_features(self) -> int:
        return int(self.weights.packed_primary.shape[0])

    @property
    def in_features(self) -> int:
        return int(self.weights.packed_residual.shape[1]) * 2


@dataclass
class TQShard:
    layers: dict[str, TQLayer] = field(default_factory=dict)
    metadata: dict[str, str] = field(default_factory=dict)
    other: dict[str, np.ndarray] = field(default_factory=dict)   # tensors that are not part of a quantised weight


def read_tq_safetensors(path: str) -> TQShard:
    """One shard.  A layer takes its own codebooks when the metadata announces per-layer
    codebooks and the tensors exist, the model-level ones otherwise; the WHT block size is
    seeds[2] (src/turboquant_c_dequant.cpp:84-150)."""
    tensors, meta = read_safetensors(path)
    if not is_tq_shard(meta):
        raise ValueError(f"{path}: no TurboQuant metadata (quantization_method != turboquant)")
    for key in ("tq_codebook_primary", "tq_codebook_residual"):
        if key not in tensors:
            raise ValueError(f"{path}: missing {key}")
    shared_p = api.codebook_from_centroids(tensors["tq_codebook_primary"])
    shared_r = api.codebook_from_centroids(tensors["tq_codebook_residual"])
    per_layer = meta.get("tq_per_layer_codebooks") == "true"
    shard = TQShard(metadata=meta)
    used = {"tq_codebook_primary", "tq_codebook_residual"}
    for name in sorted(tensors):
        if not name.endswith(".packed_primary"):
            continue
        layer = name[: -len(".packed_primary")]
        parts = []
        for suffix in _SUFFIXES:
            if layer + suffix not in tensors:
                raise ValueError(f"{path}: {layer} lacks {suffix}")
            parts.append(tensors[layer + suffix])
            used.add(layer + suffix)
        pp, pr, norms, seeds = parts
        if pp.dtype != np.uint8 or pr.dtype != np.uint8 or pp.ndim != 2 or pr.ndim != 2 or pp.shape[0] != pr.shape[0] \
                or pp.shape[1] not in (pr.shape[1], 2 * pr.shape[1]) or norms.shape != (pp.shape[0],):
            raise ValueError(f"{path}: {layer} has inconsistent plane shapes")
        seeds = seeds.astype(np.uint32).reshape(-1)
        block = int(seeds[2]) if seeds.size > 2 else DEFAULT_BLOCK_SIZE
        if seeds.size < 3:
            seeds = np.array([seeds[0] if seeds.size > 0 else 0, seeds[1] if seeds.size > 1 else 0, block], np.uint32)
        cp, cr = shared_p, shared_r
        if per_layer:
            if layer + ".codebook_primary" in tensors:
                cp = api.codebook_from_centroids(tensors[layer + ".codebook_primary"])
                used.add(layer + ".codebook_primary")
            if layer + ".codebook_residual" in tensors:
                cr = api.codebook_from_centroids(tensors[layer + ".codebook_residual"])
                used.add(layer + ".codebook_residual")
        shard.layers[layer] = TQLayer(layer, api.QuantizedWeight(pp, pr, norms.astype(np.float32), seeds), cp, cr, block)
    shard.other = {k: v for k, v in tensors.items() if k not in used}
    return shard


def read_tq_model(model_dir: str) -> tuple[dict[str, TQLayer], dict[str, np.ndarray]]:
    """Every shard of a converted model directory: (quantised layers by name, passthrough tensors by
    name).  Shards without TurboQuant metadata and `*_passthrough.safetensors` companions are
    passed through whole, as the reference's dequantiser does (src/turboquant_c_dequant.cpp:68-82, 172-181)."""
    if not os.path.isdir(model_dir):
        raise ValueError(f"{model_dir}: not a model directory")
    layers: dict[str, TQLayer] = {}
    passthrough: dict[str, np.ndarray] = {}
    for fname in sorted(os.listdir(model_dir)):
        if not fname.endswith(".safetensors"):
            continue
        path = os.path.join(model_dir, fname)
        if "_passthrough" in fname or not is_tq_shard(read_tq_metadata(path)):
            passthrough.update(read_safetensors(path)[0])
            continue
        shard = read_tq_safetensors(path)
        layers.update(shard.layers)
        passthrough.update(shard.other)
    return layers, passthrough


def load_linears(model_dir_or_shard: str) -> dict[str, api.TurboQuantLinear]:
    """Upload every quantised layer of a shard or model directory: name -> TurboQuantLinear."""
    if os.path.isdir(model_dir_or_shard):
        layers, _ = read_tq_model(model_dir_or_shard)
    else:
        layers = read_tq_safetensors(model_dir_or_shard).layers
    return {name: api.TurboQuantLinear(l.in_features, l.out_features, l.weights, l.primary_codebook, l.residual_codebook,
                                       l.block_size)
            for name, l in layers.items()}
