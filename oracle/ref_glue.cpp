// Flat C entry points over the reference's own C++ (compiled unmodified from its
// source tree against oracle/mlx_shim).  TEST INFRASTRUCTURE ONLY: used to pin the
// C restatement in tq_oracle.c, to generate the golden fixtures under
// tests/golden/, and as the "reference" CPU baseline that bench.py times.
//
// Every entry point sets the reference's thread-local force-CPU flag first, so no
// Metal route is ever taken (src/rotation.cpp:380, src/codebook.cpp:278).
#include "turboquant/codebook.h"
#include "turboquant/dequantizer.h"
#include "turboquant/kv_cache.h"
#include "turboquant/quantizer.h"

#include <cstring>
#include <thread>
#include <vector>

namespace turboquant {
// External linkage in src/codebook.cpp:99, not declared in its header.
Codebook generate_codebook_from_data_cpu(const std::vector<float>& data, uint8_t bits, int iterations);
}  // namespace turboquant

namespace mx = mlx::core;
using namespace turboquant;

namespace {

Codebook codebook_from_centroids(const float* c, int n) {
    Codebook cb;
    cb.centroids.assign(c, c + n);
    cb.boundaries.resize(n > 0 ? n - 1 : 0);
    // same midpoint rule as src/codebook.cpp:49-57
    for (int i = 0; i + 1 < n; ++i) cb.boundaries[i] = (cb.centroids[i] + cb.centroids[i + 1]) * 0.5f;
    uint8_t bits = 0;
    while ((1 << bits) < n) ++bits;
    cb.bits = bits;
    cb.origin = CodebookOrigin::Empirical;
    return cb;
}

QuantizedWeight make_qw(const uint8_t* pp, int out, int p_cols, const uint8_t* pr, int r_cols,
                        const float* norms, const uint32_t* seeds) {
    return QuantizedWeight{mx::array(pp, {out, p_cols}, mx::uint8), mx::array(pr, {out, r_cols}, mx::uint8),
                           mx::array(norms, {out}, mx::float32), mx::array(seeds, {3}, mx::uint32)};
}

struct KVHandle {
    TQKVCache* cache;
    int layers, heads, dim;
};

}  // namespace

extern "C" {

// generate_codebook (src/codebook.cpp:71-85). Writes 2^bits centroids, 2^bits-1 boundaries.
int ref_generate_codebook(int bits, float* centroids, float* boundaries) {
    try {
        Codebook cb = generate_codebook(static_cast<uint8_t>(bits));
        std::memcpy(centroids, cb.centroids.data(), cb.centroids.size() * 4);
        std::memcpy(boundaries, cb.boundaries.data(), cb.boundaries.size() * 4);
        return 0;
    } catch (...) { return -1; }
}

// generate_codebook_from_data_cpu (src/codebook.cpp:99-143).
int ref_fit_codebook(const float* data, long n, int bits, int iterations, float* centroids, float* boundaries) {
    try {
        set_force_cpu(true);
        std::vector<float> v(data, data + n);
        Codebook cb = generate_codebook_from_data_cpu(v, static_cast<uint8_t>(bits), iterations);
        std::memcpy(centroids, cb.centroids.data(), cb.centroids.size() * 4);
        std::memcpy(boundaries, cb.boundaries.data(), cb.boundaries.size() * 4);
        return 0;
    } catch (...) { return -1; }
}

// quantize (src/codebook.cpp:284-302).
int ref_codebook_quantize(const float* values, long n, const float* centroids, int n_c, uint8_t* out) {
    try {
        Codebook cb = codebook_from_centroids(centroids, n_c);
        auto idx = quantize(mx::array(values, {static_cast<int>(n)}, mx::float32), cb);
        std::memcpy(out, idx.data<uint8_t>(), static_cast<size_t>(n));
        return 0;
    } catch (...) { return -1; }
}

// apply_wht_rotation / apply_inverse_wht_rotation, CPU route (src/rotation.cpp:291-350).
int ref_wht(const float* in, int rows, int cols, uint32_t seed, uint32_t block, int inverse, float* out) {
    try {
        set_force_cpu(true);
        mx::array m(in, {rows, cols}, mx::float32);
        mx::array r = inverse ? apply_inverse_wht_rotation(m, seed, block) : apply_wht_rotation(m, seed, block);
        std::memcpy(out, r.data<float>(), static_cast<size_t>(rows) * cols * 4);
        return 0;
    } catch (...) { return -1; }
}

// quantize_weight (src/quantizer.cpp:41-261). packed_primary is [out, in/2] for
// primary_bits <= 4 and [out, in] for 5; packed_residual is always [out, in/2].
int ref_quantize_weight(const float* w, int out, int in, const float* cb_p, int n_p, const float* cb_r, int n_r,
                        int primary_bits, int residual_bits, uint32_t block, int shared_rotation,
                        uint8_t* packed_primary, uint8_t* packed_residual, float* norms, uint32_t* seeds) {
    try {
        set_force_cpu(true);
        QuantizerConfig cfg;
        cfg.primary_bits = static_cast<uint8_t>(primary_bits);
        cfg.residual_bits = static_cast<uint8_t>(residual_bits);
        cfg.block_size = block;
        cfg.shared_rotation = shared_rotation != 0;
        Codebook p = codebook_from_centroids(cb_p, n_p), r = codebook_from_centroids(cb_r, n_r);
        QuantizedWeight qw = quantize_weight(mx::array(w, {out, in}, mx::float32), p, r, cfg);
        std::memcpy(packed_primary, qw.packed_primary.data<uint8_t>(), qw.packed_primary.size());
        std::memcpy(packed_residual, qw.packed_residual.data<uint8_t>(), qw.packed_residual.size());
        std::memcpy(norms, qw.norms.data<float>(), static_cast<size_t>(out) * 4);
        std::memcpy(seeds, qw.seeds.data<uint32_t>(), 12);
        return 0;
    } catch (...) { return -1; }
}

// dequantize_weight_cpu (src/dequantizer.cpp:52-256) -> fp32 [out, in].
int ref_dequantize_weight(const uint8_t* pp, int out, int p_cols, const uint8_t* pr, int r_cols, const float* norms,
                          const uint32_t* seeds, const float* cb_p, int n_p, const float* cb_r, int n_r,
                          uint32_t block, float* result) {
    try {
        set_force_cpu(true);
        Codebook p = codebook_from_centroids(cb_p, n_p), r = codebook_from_centroids(cb_r, n_r);
        QuantizedWeight qw = make_qw(pp, out, p_cols, pr, r_cols, norms, seeds);
        mx::array w = dequantize_weight_cpu(qw, p, r, block);
        std::memcpy(result, w.data<float>(), w.size() * 4);
        return 0;
    } catch (...) { return -1; }
}

// Row-sliced, multi-threaded driver around dequantize_weight_cpu: rows are
// independent given the codebooks and seeds, so each thread runs the unmodified
// reference routine on its own row range.  One caveat is replicated on purpose: the
// reference decides "residual present" by scanning the plane it is given, so the
// flag is computed once over the whole matrix here and a slice whose own residual
// bytes are all zero gets a non-zero sentinel row appended to keep that decision
// (the sentinel row's output is discarded).
int ref_dequantize_weight_mt(const uint8_t* pp, int out, int p_cols, const uint8_t* pr, int r_cols,
                             const float* norms, const uint32_t* seeds, const float* cb_p, int n_p,
                             const float* cb_r, int n_r, uint32_t block, float* result, int threads) {
    if (threads <= 1) return ref_dequantize_weight(pp, out, p_cols, pr, r_cols, norms, seeds, cb_p, n_p, cb_r, n_r, block, result);
    bool any_res = false;
    for (size_t i = 0, n = static_cast<size_t>(out) * r_cols; i < n; ++i) if (pr[i]) { any_res = true; break; }
    const int in = (p_cols == 2 * r_cols) ? p_cols : p_cols * 2;
    std::vector<std::thread> pool;
    std::vector<int> rc(threads, 0);
    for (int t = 0; t < threads; ++t) {
        pool.emplace_back([&, t]() {
            int r0 = static_cast<int>(static_cast<long>(out) * t / threads);
            int r1 = static_cast<int>(static_cast<long>(out) * (t + 1) / threads);
            int n = r1 - r0;
            if (n <= 0) return;
            bool slice_res = false;
            for (size_t i = 0, m = static_cast<size_t>(n) * r_cols; i < m; ++i)
                if (pr[static_cast<size_t>(r0) * r_cols + i]) { slice_res = true; break; }
            if (slice_res == any_res) {
                rc[t] = ref_dequantize_weight(pp + static_cast<size_t>(r0) * p_cols, n, p_cols,
                                              pr + static_cast<size_t>(r0) * r_cols, r_cols, norms + r0, seeds,
                                              cb_p, n_p, cb_r, n_r, block, result + static_cast<size_t>(r0) * in);
            } else {
                std::vector<uint8_t> p2(static_cast<size_t>(n + 1) * p_cols, 0), r2(static_cast<size_t>(n + 1) * r_cols, 0);
                std::vector<float> n2(n + 1, 0.0f), o2(static_cast<size_t>(n + 1) * in);
                std::memcpy(p2.data(), pp + static_cast<size_t>(r0) * p_cols, static_cast<size_t>(n) * p_cols);
                std::memcpy(r2.data(), pr + static_cast<size_t>(r0) * r_cols, static_cast<size_t>(n) * r_cols);
                std::memcpy(n2.data(), norms + r0, static_cast<size_t>(n) * 4);
                r2[static_cast<size_t>(n) * r_cols] = 1;
                rc[t] = ref_dequantize_weight(p2.data(), n + 1, p_cols, r2.data(), r_cols, n2.data(), seeds, cb_p, n_p,
                                              cb_r, n_r, block, o2.data());
                std::memcpy(result + static_cast<size_t>(r0) * in, o2.data(), static_cast<size_t>(n) * in * 4);
            }
        });
    }
    for (auto& th : pool) th.join();
    for (int v : rc) if (v) return v;
    return 0;
}

// ---- KV cache (src/kv_cache.cpp) -------------------------------------------

void* ref_kv_create(int layers, int heads, int dim) {
    try {
        KVCacheConfig cfg;
        cfg.num_layers = layers;
        cfg.num_heads = heads;
        cfg.head_dim = dim;
        return new KVHandle{new TQKVCache(cfg), layers, heads, dim};
    } catch (...) { return nullptr; }
}

void ref_kv_free(void* h) {
    if (!h) return;
    auto* k = static_cast<KVHandle*>(h);
    delete k->cache;
    delete k;
}

// TQKVCache::append (src/kv_cache.cpp:16-61). keys/values: [tokens, heads, dim];
// is_fp16 != 0 means the buffers hold IEEE half values (cast to fp32 inside, :75,:144).
int ref_kv_append(void* h, int layer, const void* keys, const void* values, int tokens, int is_fp16) {
    try {
        set_force_cpu(true);
        auto* k = static_cast<KVHandle*>(h);
        mx::Shape s{tokens, k->heads, k->dim};
        if (is_fp16) {
            k->cache->append(layer, mx::array(static_cast<const mx::float16_t*>(keys), s, mx::float16),
                             mx::array(static_cast<const mx::float16_t*>(values), s, mx::float16));
        } else {
            k->cache->append(layer, mx::array(static_cast<const float*>(keys), s, mx::float32),
                             mx::array(static_cast<const float*>(values), s, mx::float32));
        }
        return 0;
    } catch (...) { return -1; }
}

int ref_kv_seq_length(void* h) { return static_cast<KVHandle*>(h)->cache->seq_length(); }

// get_keys_fp16 / get_values_fp16 (src/kv_cache.cpp:260-365) -> IEEE half bits [n, heads, dim].
int ref_kv_get_fp16(void* h, int layer, int which_values, int start, int end, uint16_t* out) {
    try {
        set_force_cpu(true);
        auto* k = static_cast<KVHandle*>(h);
        mx::array r = which_values ? k->cache->get_values_fp16(layer, start, end)
                                   : k->cache->get_keys_fp16(layer, start, end);
        std::memcpy(out, r.raw(), r.nbytes());
        return 0;
    } catch (...) { return -1; }
}

// Raw compressed storage of one layer, read back through the reference's public
// snapshot() blob (layout: src/kv_cache.cpp:401-412).  Any output pointer may be
// NULL.  Returns the layer's token count, or -1.
int ref_kv_export(void* h, int layer, uint32_t* key_words, uint32_t* value_words, float* key_norms,
                  float* value_norms, uint32_t* qjl_words, float* qjl_norms) {
    try {
        auto* k = static_cast<KVHandle*>(h);
        TQCacheSnapshot snap = k->cache->snapshot();
        if (layer < 0 || layer >= static_cast<int>(snap.layer_data.size())) return -1;
        const std::vector<uint8_t>& b = snap.layer_data[layer];
        size_t pos = 0;
        uint32_t n;
        std::memcpy(&n, b.data(), 4);
        pos = 4;
        void* dst[6] = {key_words, value_words, key_norms, value_norms, qjl_words, qjl_norms};
        for (int i = 0; i < 6; ++i) {
            uint32_t bytes;
            std::memcpy(&bytes, b.data() + pos, 4);
            pos += 4;
            if (dst[i] && bytes) std::memcpy(dst[i], b.data() + pos, bytes);
            pos += bytes;
        }
        return static_cast<int>(n);
    } catch (...) { return -1; }
}

// TQKVCache::snapshot + snapshot_serialize (src/kv_cache.cpp:509-524, src/cache_snapshot.cpp:62-83):
// the transferable byte stream.  Returns the stream's size; writes it when `out` has room.
long ref_kv_snapshot(void* h, uint8_t* out, long capacity, uint32_t model_hash, uint32_t codebook_hash) {
    try {
        auto* k = static_cast<KVHandle*>(h);
        TQCacheSnapshot snap = k->cache->snapshot();
        snap.model_hash = model_hash;
        snap.codebook_hash = codebook_hash;
        const std::vector<uint8_t> bytes = snapshot_serialize(snap);
        if (out && capacity >= static_cast<long>(bytes.size())) std::memcpy(out, bytes.data(), bytes.size());
        return static_cast<long>(bytes.size());
    } catch (...) { return -1; }
}

// snapshot_deserialize + TQKVCache::restore (src/cache_snapshot.cpp:85-110, src/kv_cache.cpp:526-545).
int ref_kv_restore(void* h, const uint8_t* data, long size) {
    try {
        auto* k = static_cast<KVHandle*>(h);
        const std::vector<uint8_t> bytes(data, data + size);
        const TQCacheSnapshot snap = snapshot_deserialize(bytes);
        if (snap.num_layers == 0) return 1;
        k->cache->restore(snap);
        return 0;
    } catch (...) { return -1; }
}

// TQKVCache::delta + delta_serialize (src/kv_cache.cpp:566-581, src/cache_snapshot.cpp:110-123):
// positions [from, to) of every layer as a byte stream.  Returns its size; writes it when `out` has room.
long ref_kv_delta(void* h, uint8_t* out, long capacity, uint32_t from, uint32_t to) {
    try {
        auto* k = static_cast<KVHandle*>(h);
        const std::vector<uint8_t> bytes = delta_serialize(k->cache->delta(from, to));
        if (out && capacity >= static_cast<long>(bytes.size())) std::memcpy(out, bytes.data(), bytes.size());
        return static_cast<long>(bytes.size());
    } catch (...) { return -1; }
}

// delta_deserialize + TQKVCache::apply_delta (src/cache_snapshot.cpp:125-140, src/kv_cache.cpp:583-594).
int ref_kv_apply_delta(void* h, const uint8_t* data, long size) {
    try {
        auto* k = static_cast<KVHandle*>(h);
        const std::vector<uint8_t> bytes(data, data + size);
        const TQCacheDelta d = delta_deserialize(bytes);
        if (d.num_layers == 0) return 1;
        k->cache->apply_delta(d);
        return 0;
    } catch (...) { return -1; }
}

}  // extern "C"
