// TQKVCache on the device, and its C entry points (the reference's tq_kv_cache_* calls
// plus pointer-level variants and a batched attention over several caches).
//
// Mirrors turboquant::TQKVCache (include/turboquant/kv_cache.h:42-133,
// src/kv_cache.cpp) and hybrid_attention's long-context branch
// (src/attention_dispatch.cpp:58-73).  One cache = one sequence, as in the reference;
// a decode batch is a set of caches attended in one launch.
#include <algorithm>
#include <array>
#include <cmath>
#include <cstring>
#include <string>

#include "tq_attn.cuh"
#include "tq_host.hpp"
#include "tq_kernels.cuh"
#include "turboquant_c/turboquant_b200.h"
#include "turboquant_c/turboquant_c.h"

namespace tq {
// tq_kv_kernels.cu
void launch_kv_encode(const void* x, bool x_is_f16, long n_vec, int head_dim, uint32_t wht_seed, uint32_t qjl_seed,
                      bool with_qjl, uint32_t* words, float* norms, uint32_t* qjl_words, float* qjl_norms,
                      cudaStream_t stream);
void launch_kv_decode_f16(const uint32_t* words, const float* norms, long n_vec, int head_dim, uint32_t wht_seed,
                          __half* out, cudaStream_t stream);
size_t attn_scratch_bytes(int n_seqs, int q_heads, int head_dim, int n_splits);
void launch_kv_attention(const void* d_seqs, int n_seqs, const void* q, bool q_is_f16, int q_heads, int kv_heads,
                         int head_dim, AttnPlan plan, uint32_t k_seed, uint32_t v_seed, uint32_t qjl_seed, bool use_qjl,
                         void* scratch, __half* out, float* lse, unsigned int* status, cudaStream_t stream);
AttnPlan attn_make_plan(int n_seqs, int q_heads, int kv_heads, int head_dim, int max_tok, int sm_count, int kernel);
}  // namespace tq

namespace turboquant {

using tq::DeviceBuffer;
using tq::Error;

// Device image of the kernel-side per-sequence descriptor (tq_kv_kernels.cu: AttnSeq).
struct SeqDesc {
    const uint32_t* k_words;
    const uint32_t* v_words;
    const float* k_norms;
    const float* v_norms;
    const uint32_t* qjl_words;
    const float* qjl_norms;
    int start, end;
};

struct LayerKVStorage {
    DeviceBuffer k_words, v_words, k_norms, v_norms, qjl_words, qjl_norms;
    int num_tokens = 0;
    int capacity = 0;
};

class TQKVCache {
public:
    TQKVCache(int num_layers, int num_heads, int head_dim, int kv_bits, int max_context, int decode_window)
        : layers_n_(num_layers), heads_(num_heads), dim_(head_dim), kv_bits_(kv_bits), max_context_(max_context),
          decode_window_(decode_window) {
        TQ_REQUIRE(num_layers > 0 && num_heads > 0, "TQKVCache: layers and heads must be positive");
        TQ_REQUIRE(tq::is_pow2(static_cast<uint32_t>(head_dim)) && head_dim >= 32 && head_dim <= 512,
                   "TQKVCache: head_dim must be a power of two in [32, 512]");
        device_ = tq::current_device();
        layers_.resize(static_cast<size_t>(num_layers));
    }

    int num_layers() const { return layers_n_; }
    int num_heads() const { return heads_; }
    int head_dim() const { return dim_; }
    int words_per_head() const { return (dim_ + 9) / 10; }
    int qjl_words_per_head() const { return (dim_ + 31) / 32; }
    int seq_length() const { return seq_length_; }  // max over layers, src/kv_cache.cpp:54-60
    int layer_tokens(int layer) const { return layers_.at(static_cast<size_t>(layer)).num_tokens; }

    // keys / values: [tokens, heads, dim], fp32 or fp16, host or device.
    void append(int layer, const void* keys, const void* values, int dtype, int tokens, cudaStream_t st) {
        TQ_REQUIRE(layer >= 0 && layer < layers_n_, "Layer index out of range");
        TQ_REQUIRE(keys && values, "append: NULL argument");
        TQ_REQUIRE(dtype == TQ_F32 || dtype == TQ_F16, "append: keys/values must be fp32 or fp16");
        TQ_REQUIRE(tokens >= 0, "append: negative token count");
        if (tokens == 0) return;
        TQ_CUDA(cudaSetDevice(device_));
        LayerKVStorage& L = layers_[static_cast<size_t>(layer)];
        reserve(L, L.num_tokens + tokens, st);
        const size_t es = dtype == TQ_F32 ? 4 : 2;
        const size_t n_vec = static_cast<size_t>(tokens) * heads_;
        const size_t bytes = n_vec * dim_ * es;
        const void* d_k = keys;
        const void* d_v = values;
        if (!tq::is_device_pointer(keys)) {
            stage_k_.reserve(bytes);
            TQ_CUDA(cudaMemcpyAsync(stage_k_.as<void>(), keys, bytes, cudaMemcpyHostToDevice, st));
            d_k = stage_k_.as<void>();
        }
        if (!tq::is_device_pointer(values)) {
            stage_v_.reserve(bytes);
            TQ_CUDA(cudaMemcpyAsync(stage_v_.as<void>(), values, bytes, cudaMemcpyHostToDevice, st));
            d_v = stage_v_.as<void>();
        }
        const size_t off = static_cast<size_t>(L.num_tokens) * heads_;
        const int wph = words_per_head(), qph = qjl_words_per_head();
        const uint32_t ks = tq::kv_layer_seed(static_cast<uint32_t>(layer), 1);  // src/kv_cache.cpp:40-42
        const uint32_t vs = tq::kv_layer_seed(static_cast<uint32_t>(layer), 2);
        const uint32_t qs = tq::kv_layer_seed(static_cast<uint32_t>(layer), 3);
        const tq::KvEncodeSegment kseg{L.k_words.as<uint32_t>() + off * wph, L.k_norms.as<float>() + off,
                                       L.qjl_words.as<uint32_t>() + off * qph, L.qjl_norms.as<float>() + off};
        const tq::KvEncodeSegment vseg{L.v_words.as<uint32_t>() + off * wph, L.v_norms.as<float>() + off, nullptr, nullptr};
        tq::launch_kv_encode_pair_segments(d_k, d_v, dtype == TQ_F16, static_cast<long>(n_vec), static_cast<long>(n_vec), dim_, ks, vs, qs,
                                           &kseg, &vseg, 1, st);
        L.num_tokens += tokens;
        seq_length_ = std::max(seq_length_, L.num_tokens);
    }

    // Room for `tokens` tokens in `layer` without further allocation (growth otherwise doubles).
    void reserve_tokens(int layer, int tokens, cudaStream_t st) {
        TQ_REQUIRE(layer >= 0 && layer < layers_n_, "Layer index out of range");
        TQ_REQUIRE(tokens >= 0, "reserve: negative token count");
        TQ_CUDA(cudaSetDevice(device_));
        LayerKVStorage& L = layers_[static_cast<size_t>(layer)];
        if (tokens > L.capacity) reserve_exact(L, tokens, st);
    }

    // One decode step of a batch: token i of keys / values ([n, heads, dim], device memory) is
    // appended to caches[i].  All caches must share shape and device; one encoder launch for the
    // keys and one for the values per 32 sequences.
    static void append_batch(TQKVCache* const* caches, int n, int layer, const void* keys, const void* values, int dtype,
                             cudaStream_t st) {
        TQ_REQUIRE(caches && n > 0 && keys && values, "append_batch: bad argument");
        TQ_REQUIRE(dtype == TQ_F32 || dtype == TQ_F16, "append_batch: keys/values must be fp32 or fp16");
        TQ_REQUIRE(tq::is_device_pointer(keys) && tq::is_device_pointer(values), "append_batch: keys and values must be device pointers");
        TQKVCache* c0 = caches[0];
        TQ_REQUIRE(c0, "append_batch: NULL cache");
        TQ_REQUIRE(layer >= 0 && layer < c0->layers_n_, "Layer index out of range");
        TQ_CUDA(cudaSetDevice(c0->device_));
        const int wph = c0->words_per_head(), qph = c0->qjl_words_per_head();
        const uint32_t ks = tq::kv_layer_seed(static_cast<uint32_t>(layer), 1);
        const uint32_t vs = tq::kv_layer_seed(static_cast<uint32_t>(layer), 2);
        const uint32_t qs = tq::kv_layer_seed(static_cast<uint32_t>(layer), 3);
        const size_t es = dtype == TQ_F32 ? 4 : 2;
        const size_t vec_bytes = static_cast<size_t>(c0->heads_) * c0->dim_ * es;
        for (int b0 = 0; b0 < n; b0 += 32) {
            const int nb = std::min(32, n - b0);
            tq::KvEncodeSegment kseg[32], vseg[32];
            for (int i = 0; i < nb; ++i) {
                TQKVCache* c = caches[b0 + i];
                TQ_REQUIRE(c && c->heads_ == c0->heads_ && c->dim_ == c0->dim_ && c->device_ == c0->device_ &&
                               c->layers_n_ == c0->layers_n_,
                           "append_batch: caches of one call must share shape and device");
                LayerKVStorage& L = c->layers_[static_cast<size_t>(layer)];
                c->reserve(L, L.num_tokens + 1, st);
                const size_t off = static_cast<size_t>(L.num_tokens) * c->heads_;
                kseg[i] = {L.k_words.as<uint32_t>() + off * wph, L.k_norms.as<float>() + off,
                           L.qjl_words.as<uint32_t>() + off * qph, L.qjl_norms.as<float>() + off};
                vseg[i] = {L.v_words.as<uint32_t>() + off * wph, L.v_norms.as<float>() + off, nullptr, nullptr};
            }
            const long n_vec = static_cast<long>(nb) * c0->heads_;
            const char* kp = static_cast<const char*>(keys) + static_cast<size_t>(b0) * vec_bytes;
            const char* vp = static_cast<const char*>(values) + static_cast<size_t>(b0) * vec_bytes;
            tq::launch_kv_encode_pair_segments(kp, vp, dtype == TQ_F16, n_vec, c0->heads_, c0->dim_, ks, vs, qs, kseg, vseg, nb, st);
            for (int i = 0; i < nb; ++i) {
                TQKVCache* c = caches[b0 + i];
                LayerKVStorage& L = c->layers_[static_cast<size_t>(layer)];
                L.num_tokens += 1;
                c->seq_length_ = std::max(c->seq_length_, L.num_tokens);
            }
        }
    }

    // fp16 [end-start, heads, dim] into `out` (host or device).
    void get_fp16(int layer, bool values, int start, int end, void* out, cudaStream_t st) {
        TQ_REQUIRE(layer >= 0 && layer < layers_n_, "Layer index out of range");
        LayerKVStorage& L = layers_[static_cast<size_t>(layer)];
        TQ_REQUIRE(start >= 0 && end <= L.num_tokens && start < end, "Invalid token range for dequantization");
        TQ_REQUIRE(out, "get_fp16: NULL output");
        TQ_CUDA(cudaSetDevice(device_));
        const size_t n_vec = static_cast<size_t>(end - start) * heads_;
        const size_t off = static_cast<size_t>(start) * heads_;
        const bool dev = tq::is_device_pointer(out);
        DeviceBuffer stage;
        __half* d_out = static_cast<__half*>(out);
        if (!dev) {
            stage.reserve(n_vec * dim_ * sizeof(__half));
            d_out = stage.as<__half>();
        }
        const uint32_t seed = tq::kv_layer_seed(static_cast<uint32_t>(layer), values ? 2 : 1);
        const DeviceBuffer& W = values ? L.v_words : L.k_words;
        const DeviceBuffer& N = values ? L.v_norms : L.k_norms;
        tq::launch_kv_decode_f16(W.as<uint32_t>() + off * words_per_head(), N.as<float>() + off,
                                 static_cast<long>(n_vec), dim_, seed, d_out, st);
        if (!dev) {
            TQ_CUDA(cudaMemcpyAsync(out, d_out, n_vec * dim_ * sizeof(__half), cudaMemcpyDeviceToHost, st));
            TQ_CUDA(cudaStreamSynchronize(st));
        }
    }

    // Raw storage of a layer in the reference's layout (any pointer may be NULL);
    // destinations are host or device.  Returns the token count.
    int export_layer(int layer, uint32_t* k_words, uint32_t* v_words, float* k_norms, float* v_norms,
                     uint32_t* qjl_words, float* qjl_norms) {
        TQ_REQUIRE(layer >= 0 && layer < layers_n_, "Layer index out of range");
        LayerKVStorage& L = layers_[static_cast<size_t>(layer)];
        TQ_CUDA(cudaSetDevice(device_));
        TQ_CUDA(cudaDeviceSynchronize());
        const size_t n = static_cast<size_t>(L.num_tokens) * heads_;
        auto copy = [&](void* dst, const DeviceBuffer& src, size_t bytes) {
            if (dst && bytes) TQ_CUDA(cudaMemcpy(dst, src.as<void>(), bytes, cudaMemcpyDefault));
        };
        copy(k_words, L.k_words, n * words_per_head() * 4);
        copy(v_words, L.v_words, n * words_per_head() * 4);
        copy(k_norms, L.k_norms, n * 4);
        copy(v_norms, L.v_norms, n * 4);
        copy(qjl_words, L.qjl_words, n * qjl_words_per_head() * 4);
        copy(qjl_norms, L.qjl_norms, n * 4);
        return L.num_tokens;
    }

    // ---- snapshot stream (src/cache_snapshot.cpp:5-31, src/kv_cache.cpp:401-412) ----
    // header: "TQCS", layers, positions, head_dim, heads, kv_bits (as u32), model hash, codebook hash;
    // per layer: blob bytes, then the blob = token count followed by six length-prefixed arrays
    // (key words, value words, key norms, value norms, sign words, sign norms) in storage order.
    size_t snapshot_bytes() const {
        size_t total = 8 * 4;
        for (const LayerKVStorage& L : layers_) total += 4 + layer_blob_bytes(L);
        return total;
    }
    size_t layer_blob_bytes(const LayerKVStorage& L) const {
        const size_t n = static_cast<size_t>(L.num_tokens) * heads_;
        return 4 + 6 * 4 + n * (2 * static_cast<size_t>(words_per_head()) + qjl_words_per_head() + 3) * 4;
    }
    // Writes the stream into host memory `out` (snapshot_bytes() bytes).
    void snapshot_to(uint8_t* out, uint32_t model_hash, uint32_t codebook_hash) {
        TQ_CUDA(cudaSetDevice(device_));
        TQ_CUDA(cudaDeviceSynchronize());
        size_t pos = 0;
        auto put = [&](uint32_t v) { std::memcpy(out + pos, &v, 4); pos += 4; };
        put(0x53435154u);  // 'T','Q','C','S'
        put(static_cast<uint32_t>(layers_n_));
        put(static_cast<uint32_t>(seq_length_));
        put(static_cast<uint32_t>(dim_));
        put(static_cast<uint32_t>(heads_));
        put(static_cast<uint32_t>(kv_bits_) & 0xFFu);
        put(model_hash);
        put(codebook_hash);
        for (const LayerKVStorage& L : layers_) {
            put(static_cast<uint32_t>(layer_blob_bytes(L)));
            put(static_cast<uint32_t>(L.num_tokens));
            const size_t n = static_cast<size_t>(L.num_tokens) * heads_;
            auto span = [&](const DeviceBuffer& src, size_t bytes) {
                put(static_cast<uint32_t>(bytes));
                if (bytes) TQ_CUDA(cudaMemcpy(out + pos, src.as<void>(), bytes, cudaMemcpyDeviceToHost));
                pos += bytes;
            };
            span(L.k_words, n * words_per_head() * 4);
            span(L.v_words, n * words_per_head() * 4);
            span(L.k_norms, n * 4);
            span(L.v_norms, n * 4);
            span(L.qjl_words, n * qjl_words_per_head() * 4);
            span(L.qjl_norms, n * 4);
        }
    }
    // Replaces the cache contents with a stream written by snapshot_to (or by the reference's
    // snapshot_serialize).  The geometry must match this cache; malformed input is refused before
    // anything is changed.
    void restore_from(const uint8_t* data, size_t size) {
        size_t pos = 0;
        auto get = [&](uint32_t& v) {
            TQ_REQUIRE(pos + 4 <= size, "restore: truncated snapshot");
            std::memcpy(&v, data + pos, 4);
            pos += 4;
        };
        uint32_t magic, layers, positions, dim, heads, bits, mh, ch;
        get(magic); get(layers); get(positions); get(dim); get(heads); get(bits); get(mh); get(ch);
        TQ_REQUIRE(magic == 0x53435154u, "restore: not a cache snapshot");
        TQ_REQUIRE(static_cast<int>(layers) == layers_n_ && static_cast<int>(dim) == dim_ && static_cast<int>(heads) == heads_,
                   "restore: snapshot geometry differs from this cache");
        struct Span { size_t off, bytes; };
        std::vector<std::array<Span, 6>> spans(layers);
        std::vector<uint32_t> tokens(layers);
        for (uint32_t l = 0; l < layers; ++l) {
            uint32_t blob;
            get(blob);
            TQ_REQUIRE(pos + blob <= size, "restore: truncated layer blob");
            const size_t end = pos + blob;
            get(tokens[l]);
            const size_t n = static_cast<size_t>(tokens[l]) * heads_;
            const size_t want[6] = {n * words_per_head() * 4, n * words_per_head() * 4, n * 4, n * 4,
                                    n * qjl_words_per_head() * 4, n * 4};
            for (int i = 0; i < 6; ++i) {
                uint32_t bytes;
                get(bytes);
                TQ_REQUIRE(bytes == want[i] && pos + bytes <= end, "restore: array size does not match the token count");
                spans[l][i] = Span{pos, bytes};
                pos += bytes;
            }
            TQ_REQUIRE(pos == end, "restore: trailing bytes in a layer blob");
        }
        TQ_CUDA(cudaSetDevice(device_));
        TQ_CUDA(cudaDeviceSynchronize());
        seq_length_ = 0;
        for (uint32_t l = 0; l < layers; ++l) {
            LayerKVStorage& L = layers_[l];
            L.num_tokens = 0;
            reserve(L, static_cast<int>(tokens[l]), nullptr);
            DeviceBuffer* dst[6] = {&L.k_words, &L.v_words, &L.k_norms, &L.v_norms, &L.qjl_words, &L.qjl_norms};
            for (int i = 0; i < 6; ++i)
                if (spans[l][i].bytes)
                    TQ_CUDA(cudaMemcpy(dst[i]->as<void>(), data + spans[l][i].off, spans[l][i].bytes, cudaMemcpyHostToDevice));
            L.num_tokens = static_cast<int>(tokens[l]);
            seq_length_ = std::max(seq_length_, L.num_tokens);
        }
    }

    // ---- delta stream (src/cache_snapshot.cpp:18-31, 110-140; src/kv_cache.cpp:566-594) ----
    // header: "TQCD", from, to, layers; per layer: blob bytes, then the same blob as in a snapshot
    // holding positions [from, to) clamped to the layer's token count.
    // Positions arrive as uint32 and are narrowed to int first, as the reference does
    // (src/kv_cache.cpp:571-572): values of 2^31 and above turn negative, so such a `to` gives an
    // empty range and such a `from` starts at 0.
    static void clamp_range(const LayerKVStorage& L, uint32_t from_u, uint32_t to_u, int& a, int& b) {
        const int from = static_cast<int>(from_u), to = static_cast<int>(to_u);
        a = std::max(from, 0);
        b = std::min(to, L.num_tokens);
        if (b < a) b = a;
    }
    size_t range_blob_bytes(int tokens) const {
        const size_t n = static_cast<size_t>(tokens) * heads_;
        return 4 + 6 * 4 + n * (2 * static_cast<size_t>(words_per_head()) + qjl_words_per_head() + 3) * 4;
    }
    size_t delta_bytes(uint32_t from, uint32_t to) const {
        size_t total = 4 * 4;
        for (const LayerKVStorage& L : layers_) {
            int a, b;
            clamp_range(L, from, to, a, b);
            total += 4 + range_blob_bytes(b - a);
        }
        return total;
    }
    void delta_to(uint8_t* out, uint32_t from, uint32_t to) {
        TQ_CUDA(cudaSetDevice(device_));
        TQ_CUDA(cudaDeviceSynchronize());
        size_t pos = 0;
        auto put = [&](uint32_t v) { std::memcpy(out + pos, &v, 4); pos += 4; };
        put(0x44435154u);  // 'T','Q','C','D'
        put(from);
        put(to);
        put(static_cast<uint32_t>(layers_n_));
        for (const LayerKVStorage& L : layers_) {
            int a, b;
            clamp_range(L, from, to, a, b);
            put(static_cast<uint32_t>(range_blob_bytes(b - a)));
            put(static_cast<uint32_t>(b - a));
            const size_t n = static_cast<size_t>(b - a) * heads_, first = static_cast<size_t>(a) * heads_;
            auto span = [&](const DeviceBuffer& src, size_t elem_bytes) {
                const size_t bytes = n * elem_bytes;
                put(static_cast<uint32_t>(bytes));
                if (bytes) TQ_CUDA(cudaMemcpy(out + pos, src.as<uint8_t>() + first * elem_bytes, bytes, cudaMemcpyDeviceToHost));
                pos += bytes;
            };
            span(L.k_words, static_cast<size_t>(words_per_head()) * 4);
            span(L.v_words, static_cast<size_t>(words_per_head()) * 4);
            span(L.k_norms, 4);
            span(L.v_norms, 4);
            span(L.qjl_words, static_cast<size_t>(qjl_words_per_head()) * 4);
            span(L.qjl_norms, 4);
        }
    }
    // Appends a delta stream (ours or the reference's delta_serialize) to every layer.  The layer
    // count must match; malformed input is refused before anything is changed.  As in the
    // reference, the positions in the header are not checked against the cache's length.
    void apply_delta_from(const uint8_t* data, size_t size) {
        size_t pos = 0;
        auto get = [&](uint32_t& v) {
            TQ_REQUIRE(pos + 4 <= size, "apply_delta: truncated stream");
            std::memcpy(&v, data + pos, 4);
            pos += 4;
        };
        uint32_t magic, from, to, layers;
        get(magic); get(from); get(to); get(layers);
        TQ_REQUIRE(magic == 0x44435154u, "apply_delta: not a cache delta");
        TQ_REQUIRE(static_cast<int>(layers) == layers_n_, "apply_delta: layer count differs from this cache");
        struct Span { size_t off, bytes; };
        std::vector<std::array<Span, 6>> spans(layers);
        std::vector<uint32_t> tokens(layers);
        for (uint32_t l = 0; l < layers; ++l) {
            uint32_t blob;
            get(blob);
            TQ_REQUIRE(pos + blob <= size, "apply_delta: truncated layer blob");
            const size_t end = pos + blob;
            get(tokens[l]);
            const size_t n = static_cast<size_t>(tokens[l]) * heads_;
            const size_t want[6] = {n * words_per_head() * 4, n * words_per_head() * 4, n * 4, n * 4,
                                    n * qjl_words_per_head() * 4, n * 4};
            for (int i = 0; i < 6; ++i) {
                uint32_t bytes;
                get(bytes);
                TQ_REQUIRE(bytes == want[i] && pos + bytes <= end, "apply_delta: array size does not match the token count");
                spans[l][i] = Span{pos, bytes};
                pos += bytes;
            }
            TQ_REQUIRE(pos == end, "apply_delta: trailing bytes in a layer blob");
        }
        TQ_CUDA(cudaSetDevice(device_));
        TQ_CUDA(cudaDeviceSynchronize());
        for (uint32_t l = 0; l < layers; ++l) {
            LayerKVStorage& L = layers_[l];
            reserve(L, L.num_tokens + static_cast<int>(tokens[l]), nullptr);
            const size_t first = static_cast<size_t>(L.num_tokens) * heads_;
            DeviceBuffer* dst[6] = {&L.k_words, &L.v_words, &L.k_norms, &L.v_norms, &L.qjl_words, &L.qjl_norms};
            const size_t elem[6] = {static_cast<size_t>(words_per_head()) * 4, static_cast<size_t>(words_per_head()) * 4, 4, 4,
                                    static_cast<size_t>(qjl_words_per_head()) * 4, 4};
            for (int i = 0; i < 6; ++i)
                if (spans[l][i].bytes)
                    TQ_CUDA(cudaMemcpy(dst[i]->as<uint8_t>() + first * elem[i], data + spans[l][i].off, spans[l][i].bytes,
                                       cudaMemcpyHostToDevice));
            L.num_tokens += static_cast<int>(tokens[l]);
            seq_length_ = std::max(seq_length_, L.num_tokens);
        }
    }

    SeqDesc describe(int layer, int start, int end) const {
        TQ_REQUIRE(layer >= 0 && layer < layers_n_, "Layer index out of range");
        const LayerKVStorage& L = layers_[static_cast<size_t>(layer)];
        TQ_REQUIRE(start >= 0 && end <= L.num_tokens && start < end, "Invalid token range for attention");
        return SeqDesc{L.k_words.as<uint32_t>(), L.v_words.as<uint32_t>(), L.k_norms.as<float>(), L.v_norms.as<float>(),
                       L.qjl_words.as<uint32_t>(), L.qjl_norms.as<float>(), start, end};
    }

    int device() const { return device_; }
    DeviceBuffer& attn_scratch() { return attn_scratch_; }
    DeviceBuffer& attn_desc() { return attn_desc_; }
    DeviceBuffer& attn_q() { return attn_q_; }
    DeviceBuffer& attn_out() { return attn_out_; }
    DeviceBuffer& attn_lse() { return attn_lse_; }
    int attention_kernel() const { return attention_kernel_; }
    void set_attention_kernel(int k) {
        TQ_REQUIRE(k >= 0 && k <= 3, "attention kernel: 0 (automatic), 1 (load-based), 2 (bulk-copy pipeline) or 3 (tensor memory)");
        attention_kernel_ = k;
    }
    // Status word of the attention kernels: page-locked host memory that the device writes
    // directly (only when a bounded wait ran out), so reading it costs the host nothing.
    unsigned int* attn_status_device() {
        if (!h_attn_status_) {
            TQ_CUDA(cudaMallocHost(&h_attn_status_, sizeof(unsigned int)));
            *h_attn_status_ = 0u;
        }
        void* alias = tq::pinned_host_device_alias(h_attn_status_);
        TQ_REQUIRE(alias != nullptr, "attention: the status word is not mapped for the device");
        return static_cast<unsigned int*>(alias);
    }
    // Device copy of the descriptor table of `layer`; uploaded only when it differs from what is there.
    const void* upload_descriptors(int layer, const void* table, size_t bytes, cudaStream_t st) {
        if (desc_dev_.size() < static_cast<size_t>(layers_n_)) {
            desc_dev_.resize(static_cast<size_t>(layers_n_));
            desc_host_.resize(static_cast<size_t>(layers_n_));
        }
        DeviceBuffer& dev = desc_dev_[static_cast<size_t>(layer)];
        std::vector<uint8_t>& host = desc_host_[static_cast<size_t>(layer)];
        if (bytes == host.size() && bytes > 0 && std::memcmp(host.data(), table, bytes) == 0) return dev.as<void>();
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        TQ_CUDA(cudaStreamIsCapturing(st, &cap));
        TQ_REQUIRE(cap == cudaStreamCaptureStatusNone,
                   "attention: the sequences or ranges of this call differ from the previous call for this layer; run it once "
                   "outside the stream capture first (the descriptor upload cannot be captured)");
        dev.reserve(bytes);
        // from pageable memory: staged by the driver before the call returns, so `table` may die
        TQ_CUDA(cudaMemcpyAsync(dev.as<void>(), table, bytes, cudaMemcpyHostToDevice, st));
        host.assign(static_cast<const uint8_t*>(table), static_cast<const uint8_t*>(table) + bytes);
        return dev.as<void>();
    }
    // Throws when an attention launch that has finished reported a failure (and clears the report).
    ~TQKVCache() {
        if (h_attn_status_) cudaFreeHost(h_attn_status_);
    }
    TQKVCache(const TQKVCache&) = delete;
    TQKVCache& operator=(const TQKVCache&) = delete;
    void check_attention_status() {
        if (h_attn_status_ && *static_cast<volatile unsigned int*>(h_attn_status_) != 0u) {
            const unsigned int code = *h_attn_status_;
            *h_attn_status_ = 0u;
            throw Error("attention: a bounded wait in the kernel ran out (device status " + std::to_string(code) +
                        "); the output of that call is not valid");
        }
    }

private:
    // Grow a layer's buffers to hold `tokens` tokens (capacity doubles; old contents kept).
    void reserve(LayerKVStorage& L, int tokens, cudaStream_t st) {
        if (tokens <= L.capacity) return;
        reserve_exact(L, std::max(L.capacity * 2, std::max(tokens, 256)), st);
    }
    void reserve_exact(LayerKVStorage& L, int cap, cudaStream_t st) {
        // whole 16-token tiles: the attention kernel fetches the cache a tile at a time
        cap = (cap + 15) / 16 * 16;
        const size_t per = static_cast<size_t>(heads_);
        const size_t old_n = static_cast<size_t>(L.num_tokens) * per;
        auto grow = [&](DeviceBuffer& b, size_t elem_bytes_per_vec) {
            DeviceBuffer nb(static_cast<size_t>(cap) * per * elem_bytes_per_vec);
            if (old_n) TQ_CUDA(cudaMemcpyAsync(nb.as<void>(), b.as<void>(), old_n * elem_bytes_per_vec, cudaMemcpyDeviceToDevice, st));
            TQ_CUDA(cudaStreamSynchronize(st));  // the old buffer is freed on return
            b = std::move(nb);
        };
        grow(L.k_words, static_cast<size_t>(words_per_head()) * 4);
        grow(L.v_words, static_cast<size_t>(words_per_head()) * 4);
        grow(L.k_norms, 4);
        grow(L.v_norms, 4);
        grow(L.qjl_words, static_cast<size_t>(qjl_words_per_head()) * 4);
        grow(L.qjl_norms, 4);
        L.capacity = cap;
    }

    int layers_n_, heads_, dim_, kv_bits_, max_context_, decode_window_;
    int device_ = 0;
    int seq_length_ = 0;
    std::vector<LayerKVStorage> layers_;
    DeviceBuffer stage_k_, stage_v_;
    DeviceBuffer attn_scratch_, attn_desc_, attn_q_, attn_out_, attn_lse_;
    unsigned int* h_attn_status_ = nullptr;
    std::vector<DeviceBuffer> desc_dev_;            // per layer: the descriptor table of the last attention call
    std::vector<std::vector<uint8_t>> desc_host_;   // ... and its host copy, to tell whether an upload is needed
    int attention_kernel_ = 0;
};

// Attention of one query position per sequence over [start, end) of each cache.
// q: [n_seqs, q_heads, dim] fp32/fp16, out: fp16 same shape; host or device.
void attention_batched(TQKVCache* const* caches, int n_seqs, int layer, const void* q, int q_dtype, int q_heads,
                       const int* starts, const int* ends, bool use_qjl, void* out, float* lse_out, cudaStream_t st) {
    TQ_REQUIRE(caches && n_seqs > 0 && q && out, "attention: bad argument");
    TQ_REQUIRE(q_dtype == TQ_F32 || q_dtype == TQ_F16, "attention: queries must be fp32 or fp16");
    TQKVCache* c0 = caches[0];
    TQ_REQUIRE(c0, "attention: NULL cache");
    const int heads = c0->num_heads(), dim = c0->head_dim();
    TQ_REQUIRE(q_heads > 0 && q_heads % heads == 0, "attention: query heads must be a multiple of KV heads");
    TQ_REQUIRE(dim <= 256, "attention: head_dim above 256 is not supported");
    TQ_CUDA(cudaSetDevice(c0->device()));
    c0->check_attention_status();   // a failure of an earlier asynchronous call
    std::vector<SeqDesc> desc(static_cast<size_t>(n_seqs));
    int max_tok = 0;
    for (int i = 0; i < n_seqs; ++i) {
        TQ_REQUIRE(caches[i] && caches[i]->num_heads() == heads && caches[i]->head_dim() == dim &&
                       caches[i]->device() == c0->device(),
                   "attention: caches of one call must share shape and device");
        desc[i] = caches[i]->describe(layer, starts[i], ends[i]);
        max_tok = std::max(max_tok, ends[i] - starts[i]);
    }
    const tq::AttnPlan plan = tq::attn_make_plan(n_seqs, q_heads, heads, dim, max_tok, tq::sm_count(c0->device()), c0->attention_kernel());
    const int n_splits = plan.n_splits;

    // The descriptor table goes up only when it differs from the one already on the device: a call
    // that repeats the previous ranges enqueues kernels only (and can then be captured in a graph).
    const void* d_desc = c0->upload_descriptors(layer, desc.data(), desc.size() * sizeof(SeqDesc), st);
    const size_t n_q = static_cast<size_t>(n_seqs) * q_heads * dim;
    const size_t q_es = q_dtype == TQ_F32 ? 4 : 2;
    const void* d_q = q;
    if (!tq::is_device_pointer(q)) {
        c0->attn_q().reserve(n_q * q_es);
        TQ_CUDA(cudaMemcpyAsync(c0->attn_q().as<void>(), q, n_q * q_es, cudaMemcpyHostToDevice, st));
        d_q = c0->attn_q().as<void>();
    }
    const bool out_dev = tq::is_device_pointer(out);
    __half* d_out = static_cast<__half*>(out);
    if (!out_dev) {
        c0->attn_out().reserve(n_q * sizeof(__half));
        d_out = c0->attn_out().as<__half>();
    }
    // optional log-sum-exp per (sequence, query head), fp32, host or device
    const size_t n_lse = static_cast<size_t>(n_seqs) * q_heads;
    float* d_lse = lse_out;
    if (lse_out != nullptr && !tq::is_device_pointer(lse_out)) {
        c0->attn_lse().reserve(n_lse * sizeof(float));
        d_lse = c0->attn_lse().as<float>();
    }
    c0->attn_scratch().reserve(tq::attn_scratch_bytes(n_seqs, q_heads, dim, n_splits));
    tq::launch_kv_attention(d_desc, n_seqs, d_q, q_dtype == TQ_F16, q_heads, heads, dim, plan,
                            tq::kv_layer_seed(static_cast<uint32_t>(layer), 1), tq::kv_layer_seed(static_cast<uint32_t>(layer), 2),
                            tq::kv_layer_seed(static_cast<uint32_t>(layer), 3), use_qjl, c0->attn_scratch().as<void>(), d_out, d_lse,
                            c0->attn_status_device(), st);
    // desc was copied from pageable host memory: the copy has been staged by the time
    // cudaMemcpyAsync returned, so `desc` may die here.
    const bool lse_host = lse_out != nullptr && d_lse != lse_out;
    if (lse_host) TQ_CUDA(cudaMemcpyAsync(lse_out, d_lse, n_lse * sizeof(float), cudaMemcpyDeviceToHost, st));
    if (!out_dev) TQ_CUDA(cudaMemcpyAsync(out, d_out, n_q * sizeof(__half), cudaMemcpyDeviceToHost, st));
    if (!out_dev || lse_host) {
        TQ_CUDA(cudaStreamSynchronize(st));
        c0->check_attention_status();
    }
}

// ---- the fp16 decode window (include/turboquant/decode_buffer.h:11-47, src/decode_buffer.cpp) --------
// A ring of `window` token slots on the device, [slot][head][dim] fp16 per tensor; slot of a token =
// absolute index % window.  Same state machine as the reference: rebuild() fills slots 0.. from a
// decompressed prefix and sets the length to the number of tokens it was given (even beyond the
// window, src/decode_buffer.cpp:45-46), append_token() writes slot length % window, slide_window()
// overwrites from window_start and advances it, keys()/values() gather [start, end) by slot.
class DecodeBuffer {
public:
    DecodeBuffer(int window, int heads, int dim) : window_(window), heads_(heads), dim_(dim), device_(tq::current_device()) {
        TQ_REQUIRE(window > 0 && heads > 0 && dim > 0, "decode buffer: window, heads and head_dim must be positive");
        const size_t bytes = static_cast<size_t>(window) * heads * dim * sizeof(__half);
        k_.resize(bytes);
        v_.resize(bytes);
        TQ_CUDA(cudaMemset(k_.as<void>(), 0, bytes));
        TQ_CUDA(cudaMemset(v_.as<void>(), 0, bytes));
    }
    int window_size() const { return window_; }
    int current_length() const { return current_length_; }
    int num_heads() const { return heads_; }
    int head_dim() const { return dim_; }
    int device() const { return device_; }
    const __half* key_ring() const { return k_.as<__half>(); }
    const __half* value_ring() const { return v_.as<__half>(); }
    DeviceBuffer& scratch() { return scratch_; }
    DeviceBuffer& q_stage() { return q_stage_; }
    DeviceBuffer& out_stage() { return out_stage_; }

    void rebuild(const void* keys, const void* values, int dtype, int num_tokens, cudaStream_t st) {
        TQ_REQUIRE(num_tokens >= 0, "decode buffer: negative token count");
        write(keys, values, dtype, std::min(num_tokens, window_), 0, st);
        current_length_ = num_tokens;
        window_start_ = 0;
    }
    void append_token(const void* key, const void* value, int dtype, cudaStream_t st) {
        write(key, value, dtype, 1, current_length_ % window_, st);
        ++current_length_;
    }
    void slide_window(const void* keys, const void* values, int dtype, int num_tokens, cudaStream_t st) {
        TQ_REQUIRE(num_tokens >= 0, "decode buffer: negative token count");
        write(keys, values, dtype, num_tokens, window_start_, st);
        window_start_ = static_cast<int>((static_cast<long>(window_start_) + num_tokens) % window_);
    }
    void read(bool values, int start, int end, void* out, cudaStream_t st) {
        // src/decode_buffer.cpp:128-141
        TQ_REQUIRE(start >= 0 && end > start && end <= current_length_, "DecodeBuffer: requested range is out of bounds");
        TQ_REQUIRE(out != nullptr, "decode buffer: NULL output");
        TQ_CUDA(cudaSetDevice(device_));
        const long n = end - start;
        const int row = heads_ * dim_;
        const bool dev = tq::is_device_pointer(out);
        __half* d_out = static_cast<__half*>(out);
        if (!dev) {
            out_stage_.reserve(static_cast<size_t>(n) * row * sizeof(__half));
            d_out = out_stage_.as<__half>();
        }
        tq::launch_ring_read(values ? v_.as<__half>() : k_.as<__half>(), n, row, window_, start, d_out, st);
        if (!dev) {
            TQ_CUDA(cudaMemcpyAsync(out, d_out, static_cast<size_t>(n) * row * sizeof(__half), cudaMemcpyDeviceToHost, st));
            TQ_CUDA(cudaStreamSynchronize(st));
        }
    }

private:
    void write(const void* keys, const void* values, int dtype, int n, int slot0, cudaStream_t st) {
        TQ_REQUIRE(dtype == TQ_F32 || dtype == TQ_F16, "decode buffer: keys and values must be fp32 or fp16");
        if (n == 0) return;
        TQ_REQUIRE(keys != nullptr && values != nullptr, "decode buffer: NULL keys or values");
        TQ_CUDA(cudaSetDevice(device_));
        const int row = heads_ * dim_;
        const size_t bytes = static_cast<size_t>(n) * row * (dtype == TQ_F32 ? 4 : 2);
        const void* dk = keys;
        const void* dv = values;
        if (!tq::is_device_pointer(keys)) {
            k_stage_.reserve(bytes);
            TQ_CUDA(cudaMemcpyAsync(k_stage_.as<void>(), keys, bytes, cudaMemcpyHostToDevice, st));
            dk = k_stage_.as<void>();
        }
        if (!tq::is_device_pointer(values)) {
            v_stage_.reserve(bytes);
            TQ_CUDA(cudaMemcpyAsync(v_stage_.as<void>(), values, bytes, cudaMemcpyHostToDevice, st));
            dv = v_stage_.as<void>();
        }
        tq::launch_ring_write(dk, dv, dtype == TQ_F16, n, 0, row, window_, slot0, k_.as<__half>(), v_.as<__half>(), st);
    }

    int window_, heads_, dim_, device_;
    int current_length_ = 0, window_start_ = 0;
    DeviceBuffer k_, v_, k_stage_, v_stage_, out_stage_, q_stage_, scratch_;
};

// hybrid_attention (src/attention_dispatch.cpp:21-74) for one query position.  Nothing cached: zeros.
// A context that fits the window: scaled-dot-product attention over the window's fp16 keys and values
// [0, seq_len).  A longer one: the reference decompresses every key and value (centroids only, the
// residual bits are not read) and runs the same attention; here that is the fused kernel over the
// compressed records, which never materialises them.
void hybrid_attention(TQKVCache* cache, DecodeBuffer* buf, int layer, const void* q, int q_dtype, int q_heads, void* out,
                      cudaStream_t st) {
    TQ_REQUIRE(cache && buf && q && out, "hybrid_attention: bad argument");
    TQ_REQUIRE(q_dtype == TQ_F32 || q_dtype == TQ_F16, "hybrid_attention: queries must be fp32 or fp16");
    const int heads = cache->num_heads(), dim = cache->head_dim();
    TQ_REQUIRE(buf->num_heads() == heads && buf->head_dim() == dim && buf->device() == cache->device(),
               "hybrid_attention: the decode buffer does not match the cache");
    TQ_REQUIRE(q_heads > 0 && q_heads % heads == 0, "hybrid_attention: query heads must be a multiple of KV heads");
    const int seq_len = cache->seq_length();
    const size_t n_q = static_cast<size_t>(q_heads) * dim;
    TQ_CUDA(cudaSetDevice(cache->device()));
    if (seq_len == 0) {
        if (tq::is_device_pointer(out)) TQ_CUDA(cudaMemsetAsync(out, 0, n_q * sizeof(__half), st));
        else std::memset(out, 0, n_q * sizeof(__half));
        return;
    }
    if (seq_len > buf->window_size()) {
        TQKVCache* one[1] = {cache};
        const int start = 0, end = seq_len;
        attention_batched(one, 1, layer, q, q_dtype, q_heads, &start, &end, false, out, nullptr, st);
        return;
    }
    TQ_REQUIRE(seq_len <= buf->current_length(), "DecodeBuffer: requested range is out of bounds");
    const size_t q_es = q_dtype == TQ_F32 ? 4 : 2;
    const void* d_q = q;
    if (!tq::is_device_pointer(q)) {
        buf->q_stage().reserve(n_q * q_es);
        TQ_CUDA(cudaMemcpyAsync(buf->q_stage().as<void>(), q, n_q * q_es, cudaMemcpyHostToDevice, st));
        d_q = buf->q_stage().as<void>();
    }
    const bool out_dev = tq::is_device_pointer(out);
    __half* d_out = static_cast<__half*>(out);
    if (!out_dev) {
        buf->out_stage().reserve(n_q * sizeof(__half));
        d_out = buf->out_stage().as<__half>();
    }
    const int n_splits = tq::dense_attention_splits(seq_len, heads, q_heads, tq::sm_count(cache->device()));
    buf->scratch().reserve(tq::dense_attention_scratch_bytes(q_heads, dim, n_splits));
    tq::launch_dense_attention(buf->key_ring(), buf->value_ring(), seq_len, heads, dim, d_q, q_dtype == TQ_F16, q_heads, n_splits,
                               buf->scratch().as<void>(), d_out, st);
    if (!out_dev) {
        TQ_CUDA(cudaMemcpyAsync(out, d_out, n_q * sizeof(__half), cudaMemcpyDeviceToHost, st));
        TQ_CUDA(cudaStreamSynchronize(st));
    }
}

}  // namespace turboquant

struct tq_kv_cache_s {
    turboquant::TQKVCache* cache;
};
struct tq_decode_buffer_s {
    turboquant::DecodeBuffer* buf;
};

using namespace tq;

namespace {

// [tokens, heads, dim] view of a tq_array for append; returns tokens or -1.
int kv_tokens_of(const tq_array_s* a, int heads, int dim) {
    if (!a || a->ndim != 3 || a->shape[1] != heads || a->shape[2] != dim) return -1;
    if (a->dtype != TQ_F32 && a->dtype != TQ_F16) return -1;
    return a->shape[0];
}

tq_array_s* new_f16_array(int ndim, const int* shape) {
    auto* a = new tq_array_s();
    a->dtype = TQ_F16;
    a->ndim = ndim;
    for (int i = 0; i < ndim; ++i) a->shape[i] = shape[i];
    a->device = current_device();
    a->owns = true;
    if (a->nbytes()) {
        cudaError_t e = cudaMalloc(&a->data, a->nbytes());
        if (e != cudaSuccess) {
            delete a;
            throw Error(std::string("cudaMalloc: ") + cudaGetErrorString(e));
        }
    }
    return a;
}

}  // namespace

extern "C" {

tq_kv_cache_t tq_kv_cache_create(int num_layers, int num_heads, int head_dim, int kv_bits, int max_context,
                                 int decode_window) {
    return guarded<tq_kv_cache_t>(nullptr, nullptr, [&]() -> tq_kv_cache_t {
        auto* c = new turboquant::TQKVCache(num_layers, num_heads, head_dim, kv_bits, max_context, decode_window);
        return new tq_kv_cache_s{c};
    });
}

void tq_kv_cache_append(tq_kv_cache_t cache, int layer, const void* keys_array, const void* values_array) {
    if (!cache || !cache->cache || !keys_array || !values_array) return;
    guarded<int>(0, -1, [&]() {
        const auto* k = static_cast<const tq_array_s*>(keys_array);
        const auto* v = static_cast<const tq_array_s*>(values_array);
        const int tokens = kv_tokens_of(k, cache->cache->num_heads(), cache->cache->head_dim());
        TQ_REQUIRE(tokens >= 0 && tokens == kv_tokens_of(v, cache->cache->num_heads(), cache->cache->head_dim()) &&
                       k->dtype == v->dtype,
                   "tq_kv_cache_append: keys/values must be [tokens, heads, head_dim] of one float type");
        cache->cache->append(layer, k->data, v->data, k->dtype, tokens, nullptr);
        return 0;
    });
}

static void* kv_get(tq_kv_cache_t cache, int layer, int start, int end, bool values) {
    if (!cache || !cache->cache) return nullptr;
    return guarded<void*>(nullptr, nullptr, [&]() -> void* {
        TQ_REQUIRE(start < end, "Invalid token range for dequantization");
        const int shape[3] = {end - start, cache->cache->num_heads(), cache->cache->head_dim()};
        // validate before allocating
        TQ_REQUIRE(layer >= 0 && layer < cache->cache->num_layers(), "Layer index out of range");
        TQ_REQUIRE(start >= 0 && end <= cache->cache->layer_tokens(layer), "Invalid token range for dequantization");
        tq_array_s* a = new_f16_array(3, shape);
        try {
            cache->cache->get_fp16(layer, values, start, end, a->data, nullptr);
        } catch (...) {
            tq_array_free(a);
            throw;
        }
        return a;
    });
}

void* tq_kv_cache_get_keys_fp16(tq_kv_cache_t cache, int layer, int start, int end) {
    return kv_get(cache, layer, start, end, false);
}
void* tq_kv_cache_get_values_fp16(tq_kv_cache_t cache, int layer, int start, int end) {
    return kv_get(cache, layer, start, end, true);
}

void* tq_kv_cache_attention(tq_kv_cache_t cache, int layer, const void* queries_array, int compressed_start,
                            int compressed_end) {
    if (!cache || !cache->cache || !queries_array) return nullptr;
    return guarded<void*>(nullptr, nullptr, [&]() -> void* {
        const auto* q = static_cast<const tq_array_s*>(queries_array);
        const int dim = cache->cache->head_dim();
        TQ_REQUIRE(q->dtype == TQ_F32 || q->dtype == TQ_F16, "tq_kv_cache_attention: queries must be fp32 or fp16");
        int q_heads = 0;
        if (q->ndim == 2 && q->shape[1] == dim) q_heads = q->shape[0];
        else if (q->ndim == 4 && q->shape[0] == 1 && q->shape[2] == 1 && q->shape[3] == dim) q_heads = q->shape[1];
        else if (q->ndim == 3 && q->shape[0] == 1 && q->shape[2] == dim) q_heads = q->shape[1];
        TQ_REQUIRE(q_heads > 0, "tq_kv_cache_attention: queries must be [q_heads, d], [1, q_heads, d] or [1, q_heads, 1, d]");
        tq_array_s* out = new_f16_array(q->ndim, q->shape);
        try {
            turboquant::TQKVCache* one[1] = {cache->cache};
            turboquant::attention_batched(one, 1, layer, q->data, q->dtype, q_heads, &compressed_start, &compressed_end,
                                          false, out->data, nullptr, nullptr);
        } catch (...) {
            tq_array_free(out);
            throw;
        }
        return out;
    });
}

int tq_kv_cache_seq_length(tq_kv_cache_t cache) { return (cache && cache->cache) ? cache->cache->seq_length() : 0; }

void tq_kv_cache_free(tq_kv_cache_t cache) {
    if (!cache) return;
    delete cache->cache;
    delete cache;
}

// ---- pointer-level variants (declared in turboquant_b200.h) --------------------------------------

int tq_kv_append(tq_kv_cache_t cache, int layer, const void* keys, const void* values, int dtype, int tokens,
                 void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(cache && cache->cache, "tq_kv_append: NULL cache");
        cache->cache->append(layer, keys, values, dtype, tokens, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_kv_get_fp16(tq_kv_cache_t cache, int layer, int values, int start, int end, void* out_fp16, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(cache && cache->cache, "tq_kv_get_fp16: NULL cache");
        cache->cache->get_fp16(layer, values != 0, start, end, out_fp16, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_kv_export(tq_kv_cache_t cache, int layer, uint32_t* k_words, uint32_t* v_words, float* k_norms, float* v_norms,
                 uint32_t* qjl_words, float* qjl_norms) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(cache && cache->cache, "tq_kv_export: NULL cache");
        return cache->cache->export_layer(layer, k_words, v_words, k_norms, v_norms, qjl_words, qjl_norms);
    });
}

long tq_kv_snapshot(tq_kv_cache_t cache, void* out, size_t capacity, uint32_t model_hash, uint32_t codebook_hash) {
    return guarded<long>(0, -1, [&]() -> long {
        TQ_REQUIRE(cache && cache->cache, "tq_kv_snapshot: NULL cache");
        const size_t need = cache->cache->snapshot_bytes();
        if (out != nullptr && capacity >= need) {
            TQ_REQUIRE(!tq::is_device_pointer(out), "tq_kv_snapshot: the stream is written to host memory");
            cache->cache->snapshot_to(static_cast<uint8_t*>(out), model_hash, codebook_hash);
        }
        return static_cast<long>(need);
    });
}

int tq_kv_restore(tq_kv_cache_t cache, const void* data, size_t size) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(cache && cache->cache, "tq_kv_restore: NULL cache");
        TQ_REQUIRE(data != nullptr && !tq::is_device_pointer(data), "tq_kv_restore: the stream is read from host memory");
        cache->cache->restore_from(static_cast<const uint8_t*>(data), size);
        return 0;
    });
}

long tq_kv_delta(tq_kv_cache_t cache, void* out, size_t capacity, uint32_t from, uint32_t to) {
    return guarded<long>(0, -1, [&]() -> long {
        TQ_REQUIRE(cache && cache->cache, "tq_kv_delta: NULL cache");
        const size_t need = cache->cache->delta_bytes(from, to);
        if (out != nullptr && capacity >= need) {
            TQ_REQUIRE(!tq::is_device_pointer(out), "tq_kv_delta: the stream is written to host memory");
            cache->cache->delta_to(static_cast<uint8_t*>(out), from, to);
        }
        return static_cast<long>(need);
    });
}

int tq_kv_apply_delta(tq_kv_cache_t cache, const void* data, size_t size) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(cache && cache->cache && data, "tq_kv_apply_delta: NULL argument");
        TQ_REQUIRE(!tq::is_device_pointer(data), "tq_kv_apply_delta: the stream is read from host memory");
        cache->cache->apply_delta_from(static_cast<const uint8_t*>(data), size);
        return 0;
    });
}

int tq_kv_set_attention_kernel(tq_kv_cache_t cache, int kernel) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(cache && cache->cache, "tq_kv_set_attention_kernel: NULL cache");
        cache->cache->set_attention_kernel(kernel);
        return 0;
    });
}

int tq_kv_attention_status(tq_kv_cache_t cache) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(cache && cache->cache, "tq_kv_attention_status: NULL cache");
        cache->cache->check_attention_status();
        return 0;
    });
}

int tq_kv_reserve(tq_kv_cache_t cache, int layer, int tokens, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(cache && cache->cache, "tq_kv_reserve: NULL cache");
        cache->cache->reserve_tokens(layer, tokens, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_kv_append_batch(const tq_kv_cache_t* caches, int n_seqs, int layer, const void* keys, const void* values, int dtype,
                       void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(caches && n_seqs > 0, "tq_kv_append_batch: no caches");
        std::vector<turboquant::TQKVCache*> cs(static_cast<size_t>(n_seqs));
        for (int i = 0; i < n_seqs; ++i) {
            TQ_REQUIRE(caches[i] && caches[i]->cache, "tq_kv_append_batch: NULL cache");
            cs[i] = caches[i]->cache;
        }
        turboquant::TQKVCache::append_batch(cs.data(), n_seqs, layer, keys, values, dtype, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_kv_attention(const tq_kv_cache_t* caches, int n_seqs, int layer, const void* queries, int q_dtype, int q_heads,
                    void* out_fp16, int start, int end, int use_qjl, void* stream) {
    return tq_kv_attention_lse(caches, n_seqs, layer, queries, q_dtype, q_heads, out_fp16, nullptr, start, end, use_qjl, stream);
}

int tq_kv_attention_lse(const tq_kv_cache_t* caches, int n_seqs, int layer, const void* queries, int q_dtype, int q_heads,
                        void* out_fp16, float* lse_out, int start, int end, int use_qjl, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(caches && n_seqs > 0, "tq_kv_attention: no caches");
        std::vector<turboquant::TQKVCache*> cs(static_cast<size_t>(n_seqs));
        std::vector<int> starts(static_cast<size_t>(n_seqs)), ends(static_cast<size_t>(n_seqs));
        for (int i = 0; i < n_seqs; ++i) {
            TQ_REQUIRE(caches[i] && caches[i]->cache, "tq_kv_attention: NULL cache");
            cs[i] = caches[i]->cache;
            starts[i] = start;
            ends[i] = end < 0 ? caches[i]->cache->layer_tokens(layer) : end;
        }
        turboquant::attention_batched(cs.data(), n_seqs, layer, queries, q_dtype, q_heads, starts.data(), ends.data(),
                                      use_qjl != 0, out_fp16, lse_out, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

tq_decode_buffer_t tq_decode_buffer_create(int window_size, int num_heads, int head_dim) {
    return guarded<tq_decode_buffer_t>(nullptr, nullptr, [&]() -> tq_decode_buffer_t {
        auto* b = new turboquant::DecodeBuffer(window_size, num_heads, head_dim);
        return new tq_decode_buffer_s{b};
    });
}

void tq_decode_buffer_free(tq_decode_buffer_t buf) {
    if (!buf) return;
    delete buf->buf;
    delete buf;
}

int tq_decode_buffer_window_size(tq_decode_buffer_t buf) { return (buf && buf->buf) ? buf->buf->window_size() : 0; }
int tq_decode_buffer_current_length(tq_decode_buffer_t buf) { return (buf && buf->buf) ? buf->buf->current_length() : 0; }

int tq_decode_buffer_rebuild(tq_decode_buffer_t buf, const void* keys, const void* values, int dtype, int num_tokens, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(buf && buf->buf, "tq_decode_buffer_rebuild: NULL buffer");
        buf->buf->rebuild(keys, values, dtype, num_tokens, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_decode_buffer_append_token(tq_decode_buffer_t buf, const void* key, const void* value, int dtype, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(buf && buf->buf, "tq_decode_buffer_append_token: NULL buffer");
        buf->buf->append_token(key, value, dtype, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_decode_buffer_slide_window(tq_decode_buffer_t buf, const void* new_keys, const void* new_values, int dtype, int num_tokens,
                                  void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(buf && buf->buf, "tq_decode_buffer_slide_window: NULL buffer");
        buf->buf->slide_window(new_keys, new_values, dtype, num_tokens, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_decode_buffer_keys(tq_decode_buffer_t buf, int start, int end, void* out_fp16, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(buf && buf->buf, "tq_decode_buffer_keys: NULL buffer");
        buf->buf->read(false, start, end, out_fp16, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_decode_buffer_values(tq_decode_buffer_t buf, int start, int end, void* out_fp16, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(buf && buf->buf, "tq_decode_buffer_values: NULL buffer");
        buf->buf->read(true, start, end, out_fp16, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_hybrid_attention(tq_kv_cache_t cache, tq_decode_buffer_t buf, int layer, const void* queries, int q_dtype, int q_heads,
                        void* out_fp16, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(cache && cache->cache && buf && buf->buf, "tq_hybrid_attention: NULL cache or buffer");
        turboquant::hybrid_attention(cache->cache, buf->buf, layer, queries, q_dtype, q_heads, out_fp16, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

}  // extern "C"
