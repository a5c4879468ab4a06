// C-ABI: library/device management, tensor handles, codebooks, rotation, and the
// non-tensor handles of turboquant_c.h (model, coordinator, cluster planner).
#include <sys/stat.h>

#include <cmath>
#include <mutex>

#include "tq_host.hpp"
#include "tq_kernels.cuh"
#include "turboquant_c/turboquant_b200.h"
#include "turboquant_c/turboquant_c.h"

namespace tq {

std::string& last_error_slot() {
    static thread_local std::string slot;
    return slot;
}

int current_device() {
    int d = 0;
    TQ_CUDA(cudaGetDevice(&d));
    return d;
}

int sm_count(int device) {
    static std::mutex mu;
    static int cache[64] = {0};
    std::lock_guard<std::mutex> lock(mu);
    if (device >= 0 && device < 64 && cache[device]) return cache[device];
    int n = 0;
    TQ_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
    if (device >= 0 && device < 64) cache[device] = n;
    return n;
}

// N(0,1) Lloyd-Max centroids for 1..5 bits: the values of src/codebook.cpp:16-45.
static const float kC1[] = {-0.7978845608f, 0.7978845608f};
static const float kC2[] = {-1.510232f, -0.4527800f, 0.4527800f, 1.510232f};
static const float kC3[] = {-2.152176f, -1.344318f, -0.756130f, -0.245379f, 0.245379f, 0.756130f, 1.344318f, 2.152176f};
static const float kC4[] = {-2.732590f, -2.069017f, -1.618046f, -1.256231f, -0.942340f, -0.656759f, -0.388048f, -0.128395f,
                            0.128395f,  0.388048f,  0.656759f,  0.942340f,  1.256231f,  1.618046f,  2.069017f,  2.732590f};
static const float kC5[] = {-3.255544f, -2.685239f, -2.311434f, -2.022174f, -1.780580f, -1.569614f, -1.379896f, -1.205655f,
                            -1.043046f, -0.889350f, -0.742542f, -0.601049f, -0.463598f, -0.329119f, -0.196679f, -0.065429f,
                            0.065429f,  0.196679f,  0.329119f,  0.463598f,  0.601049f,  0.742542f,  0.889350f,  1.043046f,
                            1.205655f,  1.379896f,  1.569614f,  1.780580f,  2.022174f,  2.311434f,  2.685239f,  3.255544f};

const float* analytic_centroids(int bits) {
    switch (bits) {
        case 1: return kC1;
        case 2: return kC2;
        case 3: return kC3;
        case 4: return kC4;
        case 5: return kC5;
        default: return nullptr;
    }
}

}  // namespace tq

using namespace tq;

struct tq_coordinator_s {
    int rank = 0, world = 1;
};
struct tq_cluster_s {
    int num_layers = 0, num_heads = 0, head_dim = 0;
    std::vector<std::pair<std::string, double>> nodes;
    std::vector<std::pair<int, int>> ranges;  // [start, end) per rank
    bool planned = false;
};

extern "C" {

const char* tq_last_error(void) { return last_error_slot().c_str(); }

int tq_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int tq_set_device(int device) {
    return guarded<int>(0, -1, [&]() {
        TQ_CUDA(cudaSetDevice(device));
        return 0;
    });
}

// ---- tq_array ---------------------------------------------------------------------------

tq_array_t tq_array_create(const void* data, int dtype, int ndim, const int* shape) {
    return guarded<tq_array_t>(nullptr, nullptr, [&]() -> tq_array_t {
        TQ_REQUIRE(ndim >= 0 && ndim <= 8 && dtype >= 0 && dtype <= 3, "tq_array_create: bad ndim or dtype");
        TQ_REQUIRE(ndim == 0 || shape, "tq_array_create: NULL shape");
        auto* a = new tq_array_s();
        a->dtype = dtype;
        a->ndim = ndim;
        for (int i = 0; i < ndim; ++i) {
            if (shape[i] < 0) { delete a; throw Error("tq_array_create: negative dimension"); }
            a->shape[i] = shape[i];
        }
        a->device = current_device();
        a->owns = true;
        const size_t nb = a->nbytes();
        try {
            if (nb) {
                TQ_REQUIRE(data, "tq_array_create: NULL data");
                TQ_CUDA(cudaMalloc(&a->data, nb));
                TQ_CUDA(cudaMemcpy(a->data, data, nb, cudaMemcpyDefault));
            }
        } catch (...) {
            if (a->data) cudaFree(a->data);
            delete a;
            throw;
        }
        return a;
    });
}

tq_array_t tq_array_wrap_device(void* device_ptr, int dtype, int ndim, const int* shape) {
    return guarded<tq_array_t>(nullptr, nullptr, [&]() -> tq_array_t {
        TQ_REQUIRE(ndim >= 0 && ndim <= 8 && dtype >= 0 && dtype <= 3, "tq_array_wrap_device: bad ndim or dtype");
        TQ_REQUIRE(is_device_pointer(device_ptr), "tq_array_wrap_device: not a device pointer");
        auto* a = new tq_array_s();
        a->data = device_ptr;
        a->dtype = dtype;
        a->ndim = ndim;
        for (int i = 0; i < ndim; ++i) a->shape[i] = shape[i];
        a->device = current_device();
        a->owns = false;
        return a;
    });
}

int tq_array_ndim(tq_array_t a) { return a ? a->ndim : 0; }
int tq_array_dim(tq_array_t a, int axis) { return (a && axis >= 0 && axis < a->ndim) ? a->shape[axis] : 0; }
int tq_array_dtype(tq_array_t a) { return a ? a->dtype : -1; }
size_t tq_array_nbytes(tq_array_t a) { return a ? a->nbytes() : 0; }
void* tq_array_data(tq_array_t a) { return a ? a->data : nullptr; }

int tq_array_to_host(tq_array_t a, void* dst, size_t dst_bytes) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(a && dst, "tq_array_to_host: NULL argument");
        TQ_REQUIRE(dst_bytes >= a->nbytes(), "tq_array_to_host: destination too small");
        TQ_CUDA(cudaDeviceSynchronize());
        if (a->nbytes()) TQ_CUDA(cudaMemcpy(dst, a->data, a->nbytes(), cudaMemcpyDeviceToHost));
        return 0;
    });
}

void tq_array_free(void* array) {
    if (!array) return;
    auto* a = static_cast<tq_array_s*>(array);
    if (a->owns && a->data) cudaFree(a->data);
    delete a;
}

const char* tq_version(void) { return "0.1.0"; }

// ---- codebook / rotation -------------------------------------------------------------------

int tq_codebook_generate(int bits, float* centroids, float* boundaries) {
    return guarded<int>(0, -1, [&]() {
        const float* c = analytic_centroids(bits);
        TQ_REQUIRE(c, "Unsupported bit width; must be 1-5");
        TQ_REQUIRE(centroids, "tq_codebook_generate: NULL centroids");
        const int n = 1 << bits;
        std::memcpy(centroids, c, sizeof(float) * n);
        if (boundaries)
            for (int i = 0; i + 1 < n; ++i) boundaries[i] = (c[i] + c[i + 1]) * 0.5f;  // src/codebook.cpp:49-57
        return 0;
    });
}

// generate_codebook_from_data (src/codebook.cpp:269-282) on the device, whatever the sample count.
int tq_codebook_fit(const float* data, long n, int bits, int iterations, float* centroids, float* boundaries, int* iterations_run,
                    void* stream) {
    return guarded<int>(0, -1, [&]() {
        const float* c0 = analytic_centroids(bits);
        TQ_REQUIRE(c0, "Unsupported bit width; must be 1-5");
        TQ_REQUIRE(centroids && n >= 0 && (n == 0 || data), "tq_codebook_fit: bad argument");
        auto st = static_cast<cudaStream_t>(stream);
        DeviceBuffer stage;
        const float* d_data = n ? device_view(data, static_cast<size_t>(n), stage, st) : nullptr;
        const int run = launch_codebook_fit(d_data, n, bits, iterations, c0, centroids, boundaries, st);
        if (iterations_run) *iterations_run = run;
        return 0;
    });
}

// The converter's per-layer fit (src/converter.cpp:291-368): samples = sqrt(in) * WHT(row / |row|) with the
// seed the quantiser will derive; the primary codebook is fitted to them, the residual codebook to what the
// SHARED analytic primary codebook leaves of them.
int tq_fit_layer_codebooks(const float* weight, int out_features, int in_features, uint32_t block, int primary_bits, int residual_bits,
                           int iterations, float* primary_centroids, float* primary_boundaries, float* residual_centroids,
                           float* residual_boundaries, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(weight && out_features > 0 && in_features > 0 && primary_centroids, "tq_fit_layer_codebooks: bad argument");
        const float* cp0 = analytic_centroids(primary_bits);
        TQ_REQUIRE(cp0, "Unsupported bit width; must be 1-5");
        const bool need_residual = residual_bits > 0;
        const float* cr0 = need_residual ? analytic_centroids(residual_bits) : nullptr;
        TQ_REQUIRE(!need_residual || (cr0 && residual_centroids), "tq_fit_layer_codebooks: bad residual bit width or NULL output");
        auto st = static_cast<cudaStream_t>(stream);
        const size_t n = static_cast<size_t>(out_features) * in_features;
        DeviceBuffer w_stage, norms(static_cast<size_t>(out_features) * 4), scaled(n * 4), resid(need_residual ? n * 4 : 0);
        const float* d_w = device_view(weight, n, w_stage, st);
        uint32_t seed_p = 0, seed_r = 0;
        derive_seeds(d_w, n, &seed_p, &seed_r, st);
        launch_row_norms(d_w, norms.as<float>(), out_features, in_features, st);
        launch_layer_samples(d_w, norms.as<float>(), out_features, in_features, block, seed_p, cp0, 1 << primary_bits,
                             scaled.as<float>(), need_residual ? resid.as<float>() : nullptr, st);
        launch_codebook_fit(scaled.as<float>(), static_cast<long>(n), primary_bits, iterations, cp0, primary_centroids,
                            primary_boundaries, st);
        if (need_residual)
            launch_codebook_fit(resid.as<float>(), static_cast<long>(n), residual_bits, iterations, cr0, residual_centroids,
                                residual_boundaries, st);
        TQ_CUDA(cudaStreamSynchronize(st));
        return 0;
    });
}

// Largest power of two <= max_block that divides in_features (src/converter.cpp:228-240); 1 when none does.
uint32_t tq_adaptive_block_size(int in_features, uint32_t max_block) {
    uint32_t best = 1;
    for (int p = 1; p < 20; ++p) {
        const uint32_t c = 1u << p;
        if (c > max_block) break;
        if (in_features % static_cast<int>(c) == 0) best = c;
    }
    return best;
}

// Index N of the first ".layers.N." in a tensor name, -1 when there is none (src/converter.cpp:52-59).
int tq_layer_index(const char* name) {
    if (!name) return -1;
    const char* key = ".layers.";
    for (const char* p = std::strstr(name, key); p; p = std::strstr(p + 1, key)) {
        const char* d = p + 8;
        if (*d < '0' || *d > '9') continue;
        long v = 0;
        while (*d >= '0' && *d <= '9') {
            v = v * 10 + (*d - '0');
            if (v > 0x7fffffffL) return -1;
            ++d;
        }
        if (*d == '.') return static_cast<int>(v);
    }
    return -1;
}

// Layers kept at fp16: the first `sensitive_start` and the last `sensitive_end` of the stack (src/converter.cpp:81-93).
int tq_is_sensitive_layer(int layer_index, int max_layer_index, int sensitive_start, int sensitive_end) {
    if (layer_index < 0) return 0;
    if (layer_index < sensitive_start) return 1;
    if (layer_index > max_layer_index - sensitive_end) return 1;
    return 0;
}

// metal/turboquant_qjl.metal:52-137 (tq_qjl_compress)
int tq_qjl_compress(const float* residual, int num_tokens, int num_heads, int head_dim, int proj_dim, uint32_t proj_seed,
                    uint32_t* signs_out, float* norms_out, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(residual && signs_out && norms_out, "tq_qjl_compress: NULL argument");
        auto st = static_cast<cudaStream_t>(stream);
        const size_t n = static_cast<size_t>(num_tokens) * num_heads * head_dim;
        const size_t n_vec = static_cast<size_t>(num_tokens) * num_heads, words = (static_cast<size_t>(proj_dim) + 31) / 32;
        DeviceBuffer in_stage, s_stage, n_stage;
        const float* d_r = device_view(residual, n, in_stage, st);
        const bool s_dev = is_device_pointer(signs_out), n_dev = is_device_pointer(norms_out);
        uint32_t* d_s = signs_out;
        float* d_n = norms_out;
        if (!s_dev) { s_stage.reserve(n_vec * words * 4); d_s = s_stage.as<uint32_t>(); }
        if (!n_dev) { n_stage.reserve(n_vec * 4); d_n = n_stage.as<float>(); }
        launch_qjl_compress(d_r, num_tokens, num_heads, head_dim, proj_dim, proj_seed, d_s, d_n, st);
        if (!s_dev && n_vec) TQ_CUDA(cudaMemcpyAsync(signs_out, d_s, n_vec * words * 4, cudaMemcpyDeviceToHost, st));
        if (!n_dev && n_vec) TQ_CUDA(cudaMemcpyAsync(norms_out, d_n, n_vec * 4, cudaMemcpyDeviceToHost, st));
        if (!s_dev || !n_dev || in_stage.bytes()) TQ_CUDA(cudaStreamSynchronize(st));
        return 0;
    });
}

// metal/turboquant_qjl.metal:163-216 (tq_qjl_dot_correction); corrections[query * num_keys + key]
int tq_qjl_dot_correction(const uint32_t* signs_q, const uint32_t* signs_k, const float* norms_k, int num_queries, int num_keys,
                          int num_heads, int head_idx, int proj_dim, float* corrections, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(signs_q && signs_k && norms_k && corrections && num_queries >= 0 && num_keys >= 0, "tq_qjl_dot_correction: bad argument");
        auto st = static_cast<cudaStream_t>(stream);
        const size_t words = (static_cast<size_t>(proj_dim) + 31) / 32;
        DeviceBuffer q_stage, k_stage, n_stage, c_stage;
        const uint32_t* d_q = device_view(signs_q, static_cast<size_t>(num_queries) * num_heads * words, q_stage, st);
        const uint32_t* d_k = device_view(signs_k, static_cast<size_t>(num_keys) * num_heads * words, k_stage, st);
        const float* d_n = device_view(norms_k, static_cast<size_t>(num_keys) * num_heads, n_stage, st);
        const size_t total = static_cast<size_t>(num_queries) * num_keys;
        const bool c_dev = is_device_pointer(corrections);
        float* d_c = corrections;
        if (!c_dev) { c_stage.reserve(total * 4); d_c = c_stage.as<float>(); }
        launch_qjl_dot_correction(d_q, d_k, d_n, num_queries, num_keys, num_heads, head_idx, proj_dim, d_c, st);
        if (!c_dev && total) TQ_CUDA(cudaMemcpyAsync(corrections, d_c, total * 4, cudaMemcpyDeviceToHost, st));
        TQ_CUDA(cudaStreamSynchronize(st));
        return 0;
    });
}

int tq_wht_rotate(const float* in, float* out, int rows, int cols, uint32_t seed, uint32_t block, int inverse,
                  void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(in && out && rows >= 0 && cols >= 0, "tq_wht_rotate: bad argument");
        auto st = static_cast<cudaStream_t>(stream);
        const size_t n = static_cast<size_t>(rows) * cols;
        DeviceBuffer in_stage, out_stage;
        const float* d_in = device_view(in, n, in_stage, st);
        const bool out_dev = is_device_pointer(out);
        float* d_out = out;
        if (!out_dev) {
            out_stage.reserve(n * sizeof(float));
            d_out = out_stage.as<float>();
        }
        launch_wht_rows(d_in, d_out, rows, cols, seed, block, inverse != 0, st);
        if (!out_dev && n) {
            TQ_CUDA(cudaMemcpyAsync(out, d_out, n * sizeof(float), cudaMemcpyDeviceToHost, st));
        }
        if (!out_dev || in_stage.bytes()) TQ_CUDA(cudaStreamSynchronize(st));  // staging buffers die here
        return 0;
    });
}

// ---- coordinator / cluster (the model handle lives in tq_api_model.cu) ------------------------------------------------------------

tq_coordinator_t tq_distributed_init(const char* hostfile, const char*) {
    (void)hostfile;
    set_last_error("tq_distributed_init: hostfile bring-up is not provided; launch one process per GPU instead");
    return nullptr;
}
tq_coordinator_t tq_distributed_init_local(void) {
    try {
        return new tq_coordinator_s();
    } catch (...) {
        return nullptr;
    }
}
int tq_distributed_rank(tq_coordinator_t c) { return c ? c->rank : 0; }
int tq_distributed_world_size(tq_coordinator_t c) { return c ? c->world : 1; }
void tq_distributed_free(tq_coordinator_t c) { delete c; }

tq_cluster_t tq_cluster_create(int num_layers, int num_heads, int head_dim) {
    if (num_layers <= 0 || num_heads <= 0 || head_dim <= 0) return nullptr;
    try {
        auto* c = new tq_cluster_s();
        c->num_layers = num_layers;
        c->num_heads = num_heads;
        c->head_dim = head_dim;
        return c;
    } catch (...) {
        return nullptr;
    }
}

int tq_cluster_add_node(tq_cluster_t c, const char* hostname, double memory_gb) {
    if (!c || !hostname || !(memory_gb > 0.0) || c->planned) return -1;
    try {
        c->nodes.emplace_back(hostname, memory_gb);
        return 0;
    } catch (...) {
        return -1;
    }
}

// Layers in proportion to usable memory, at least one per node, the last node taking
// the remainder (the rule of src/distributed.cpp:213-253).
int tq_cluster_plan(tq_cluster_t c) {
    if (!c || c->planned || c->nodes.empty()) return -1;
    try {
        const int L = c->num_layers;
        const size_t n = c->nodes.size();
        c->ranges.clear();
        if (n == 1) {
            c->ranges.emplace_back(0, L);
        } else {
            double total = 0.0;
            for (auto& nd : c->nodes) total += nd.second;
            if (total <= 0.0) total = 1.0;
            int assigned = 0;
            for (size_t i = 0; i < n; ++i) {
                int take;
                if (i + 1 == n) {
                    take = L - assigned;
                } else {
                    take = static_cast<int>(std::round(static_cast<double>(L) * c->nodes[i].second / total));
                    if (take < 1) take = 1;
                    if (assigned + take > L) take = L - assigned;
                }
                c->ranges.emplace_back(assigned, assigned + take);
                assigned += take;
            }
        }
        c->planned = true;
        return 0;
    } catch (...) {
        return -1;
    }
}

int tq_cluster_node_count(tq_cluster_t c) { return c ? static_cast<int>(c->nodes.size()) : 0; }
int tq_cluster_get_layer_start(tq_cluster_t c, int rank) {
    if (!c || !c->planned || rank < 0 || rank >= static_cast<int>(c->ranges.size())) return -1;
    return c->ranges[rank].first;
}
int tq_cluster_get_layer_end(tq_cluster_t c, int rank) {
    if (!c || !c->planned || rank < 0 || rank >= static_cast<int>(c->ranges.size())) return -1;
    return c->ranges[rank].second;
}
void tq_cluster_free(tq_cluster_t c) { delete c; }

}  // extern "C"
