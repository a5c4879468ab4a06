// C entry points of the rank-to-rank exchange (tq_peer.cu): the data plane of the sharded paths.
// The reference plans a layer split (src/distributed.cpp:201-253) and ships no collective
// (benchmarks/bench_distributed.cpp:9-12), so these calls have no counterpart there.
#include "tq_host.hpp"
#include "tq_kernels.cuh"
#include "turboquant_c/turboquant_b200.h"

struct tq_exchange_s {
    int rank = 0, world = 1, device = 0;
    tq::DeviceBuffer words;               // [0] CTAs finished, [1] broadcasts completed, [2] waits started
    unsigned int* h_status = nullptr;     // page-locked: a wait that gave up stores 10 here
    unsigned int* d_status = nullptr;
    ~tq_exchange_s() {
        if (h_status) cudaFreeHost(h_status);
    }
};

using namespace tq;

extern "C" {

tq_exchange_t tq_exchange_create(int rank, int world) {
    return guarded<tq_exchange_t>(nullptr, nullptr, [&]() -> tq_exchange_t {
        TQ_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world, "tq_exchange_create: rank / world out of range (1..8 ranks)");
        auto* ex = new tq_exchange_s;
        try {
            ex->rank = rank;
            ex->world = world;
            ex->device = current_device();
            ex->words.resize(256);
            TQ_CUDA(cudaMemset(ex->words.as<void>(), 0, 256));
            TQ_CUDA(cudaMallocHost(&ex->h_status, sizeof(unsigned int)));
            *ex->h_status = 0;
            ex->d_status = static_cast<unsigned int*>(pinned_host_device_alias(ex->h_status));
            TQ_REQUIRE(ex->d_status != nullptr, "tq_exchange_create: the status word is not mapped for the device");
        } catch (...) {
            delete ex;
            throw;
        }
        return ex;
    });
}

int tq_exchange_broadcast(tq_exchange_t ex, const void* src, void* const* dst, int n_dst, int rows, long row_bytes,
                          long src_stride_bytes, long dst_stride_bytes, void* const* flags, int n_flags, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(ex != nullptr, "tq_exchange_broadcast: NULL handle");
        TQ_REQUIRE(flags != nullptr, "tq_exchange_broadcast: NULL flag list");
        unsigned int* sig[8];
        TQ_REQUIRE(n_flags >= 1 && n_flags <= 8, "tq_exchange_broadcast: 1..8 flag arrays");
        for (int d = 0; d < n_flags; ++d) sig[d] = static_cast<unsigned int*>(flags[d]);
        unsigned int* w = ex->words.as<unsigned int>();
        launch_exchange_broadcast(src, dst, n_dst, rows, row_bytes, src_stride_bytes, dst_stride_bytes, sig, n_flags, ex->rank, w, w + 1,
                                  static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_exchange_wait(tq_exchange_t ex, const void* local_flags, int n_flags, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(ex != nullptr, "tq_exchange_wait: NULL handle");
        launch_exchange_wait(static_cast<const unsigned int*>(local_flags), n_flags, ex->words.as<unsigned int>() + 2, ex->d_status,
                             static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_exchange_sum_f16(const void* slots_fp16, int n_slots, long slot_stride, long count, const void* residual_fp16,
                        void* out_fp16, void* stream) {
    return guarded<int>(0, -1, [&]() {
        launch_exchange_sum_f16(static_cast<const __half*>(slots_fp16), n_slots, slot_stride, count,
                                static_cast<const __half*>(residual_fp16), static_cast<__half*>(out_fp16),
                                static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_exchange_sum_f16_rmsnorm(const void* slots_fp16, int n_slots, long slot_stride, long rows, int cols, const void* residual_fp16,
                                void* out_fp16, const void* norm_weight_fp16, void* normed_fp16, float eps, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(norm_weight_fp16 && normed_fp16, "tq_exchange_sum_f16_rmsnorm: NULL argument");
        launch_exchange_sum_f16(static_cast<const __half*>(slots_fp16), n_slots, slot_stride, rows * cols,
                                static_cast<const __half*>(residual_fp16), static_cast<__half*>(out_fp16),
                                static_cast<cudaStream_t>(stream), static_cast<const __half*>(norm_weight_fp16),
                                static_cast<__half*>(normed_fp16), cols, eps);
        return 0;
    });
}

int tq_rope_qk_f16(void* q_fp16, void* k_fp16, const int* positions, long rows, int q_heads, int kv_heads, int head_dim, float theta,
                   void* stream) {
    return guarded<int>(0, -1, [&]() {
        launch_rope_qk_f16(static_cast<__half*>(q_fp16), static_cast<__half*>(k_fp16), positions, rows, q_heads, kv_heads, head_dim, theta,
                           static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_rmsnorm_f16(const void* x_fp16, const void* weight_fp16, void* y_fp16, long rows, int cols, float eps, void* stream) {
    return guarded<int>(0, -1, [&]() {
        launch_rmsnorm_f16(static_cast<const __half*>(x_fp16), static_cast<const __half*>(weight_fp16), static_cast<__half*>(y_fp16),
                           rows, cols, eps, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_rope_f16(void* x_fp16, const int* positions, long rows, int heads, int head_dim, float theta, void* stream) {
    return guarded<int>(0, -1, [&]() {
        launch_rope_f16(static_cast<__half*>(x_fp16), positions, rows, heads, head_dim, theta, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_swiglu_f16(const void* gate_up_fp16, void* act_fp16, long rows, int intermediate, void* stream) {
    return guarded<int>(0, -1, [&]() {
        launch_swiglu_f16(static_cast<const __half*>(gate_up_fp16), static_cast<__half*>(act_fp16), rows, intermediate,
                          static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_exchange_merge_attention(const void* outs_fp16, const void* lses_fp32, int parts, long rows, int head_dim,
                                long part_stride_out, long part_stride_lse, void* out_fp16, void* stream) {
    return guarded<int>(0, -1, [&]() {
        launch_exchange_merge_attention(static_cast<const __half*>(outs_fp16), static_cast<const float*>(lses_fp32), parts, rows,
                                        head_dim, part_stride_out, part_stride_lse, static_cast<__half*>(out_fp16),
                                        static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_exchange_status(tq_exchange_t ex) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(ex != nullptr, "tq_exchange_status: NULL handle");
        TQ_CUDA(cudaSetDevice(ex->device));
        TQ_CUDA(cudaDeviceSynchronize());
        const unsigned int h = *static_cast<volatile unsigned int*>(ex->h_status);
        if (h != 0)
            throw Error("exchange: a rank's completion flag did not arrive within a second (status " + std::to_string(h) + ")");
        return 0;
    });
}

void tq_exchange_free(tq_exchange_t ex) { delete ex; }

// The exchange's device counters for the fused kernels of tq_api_linear.cu:
// [0] CTAs finished, [1] broadcasts completed, [2] waits started.
unsigned int* tq_exchange_words(tq_exchange_t ex, int* rank) {
    if (rank) *rank = ex->rank;
    return ex->words.as<unsigned int>();
}
unsigned int* tq_exchange_words_world(tq_exchange_t ex, int* rank, int* world) {
    if (rank) *rank = ex->rank;
    if (world) *world = ex->world;
    return ex->words.as<unsigned int>();
}

int tq_exchange_wait_packets(tq_exchange_t ex, const void* local_packets, long rows_per_rank, int batch, void* out_fp16, long out_row_stride,
                             void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(ex != nullptr && local_packets && out_fp16, "tq_exchange_wait_packets: NULL argument");
        launch_exchange_wait_packets(static_cast<const uint4*>(local_packets), ex->words.as<unsigned int>() + 1,
                                     ex->words.as<unsigned int>() + 2, ex->rank, ex->world, rows_per_rank, batch, static_cast<__half*>(out_fp16), out_row_stride, ex->d_status,
                                     static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_exchange_sum_packets(tq_exchange_t ex, const void* local_packets, const void* local_partial_fp16, long count,
                            const void* residual_fp16, void* out_fp16, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(ex != nullptr && local_packets && local_partial_fp16 && out_fp16, "tq_exchange_sum_packets: NULL argument");
        launch_exchange_sum_packets(static_cast<const uint4*>(local_packets), ex->words.as<unsigned int>() + 1,
                                    ex->words.as<unsigned int>() + 2, ex->rank, ex->world, count,
                                    static_cast<const __half*>(local_partial_fp16), static_cast<const __half*>(residual_fp16),
                                    static_cast<__half*>(out_fp16), ex->d_status, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_exchange_sum_packets_rmsnorm(tq_exchange_t ex, const void* local_packets, const void* local_partial_fp16, long rows, int cols,
                                    const void* residual_fp16, void* out_fp16, const void* norm_weight_fp16, void* normed_fp16, float eps,
                                    void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(ex != nullptr && local_packets && local_partial_fp16 && out_fp16 && norm_weight_fp16 && normed_fp16,
                   "tq_exchange_sum_packets_rmsnorm: NULL argument");
        launch_exchange_sum_packets(static_cast<const uint4*>(local_packets), ex->words.as<unsigned int>() + 1,
                                    ex->words.as<unsigned int>() + 2, ex->rank, ex->world, rows * cols,
                                    static_cast<const __half*>(local_partial_fp16), static_cast<const __half*>(residual_fp16),
                                    static_cast<__half*>(out_fp16), ex->d_status, static_cast<cudaStream_t>(stream),
                                    static_cast<const __half*>(norm_weight_fp16), static_cast<__half*>(normed_fp16), cols, eps);
        return 0;
    });
}

int tq_exchange_unpack_packets(const void* packets, long n_packets, void* out_fp16, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(packets && out_fp16 && n_packets >= 0, "tq_exchange_unpack_packets: bad argument");
        launch_exchange_unpack_packets(static_cast<const uint4*>(packets), n_packets, static_cast<__half*>(out_fp16),
                                       static_cast<cudaStream_t>(stream));
        return 0;
    });
}

}  // extern "C"
