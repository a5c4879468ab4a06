// TurboQuantLinear on the device, and its C entry points.
//
// Mirrors the reference's turboquant::TurboQuantLinear (include/turboquant/linear.h:11-35)
// and the dequantiser entry points (include/turboquant/dequantizer.h:11-39).  What the
// reference recomputes on every call — packing mode, "residual present" scan, the
// 256-entry centroid-sum table (src/dequantizer.cpp:619-643, 674-688) — is decided once
// when the handle is built.
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "tq_host.hpp"
#include "tq_kernels.cuh"
#include "turboquant_c/turboquant_b200.h"

namespace turboquant {

using tq::DeviceBuffer;
using tq::Error;

class TurboQuantLinear {
public:
    TurboQuantLinear(int in_features, int out_features, const uint8_t* packed_primary, int primary_cols,
                     const uint8_t* packed_residual, const float* norms, const uint32_t* seeds, const float* cb_p,
                     int n_p, const float* cb_r, int n_r, uint32_t block)
        : in_(in_features), out_(out_features), block_(block) {
        TQ_REQUIRE(in_ > 0 && out_ > 0, "TurboQuantLinear: dimensions must be positive");
        TQ_REQUIRE(tq::is_pow2(block) && block >= 32 && block <= 1024,
                   "TurboQuantLinear: block_size must be a power of two in [32, 1024]");
        TQ_REQUIRE(in_ % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
        TQ_REQUIRE(static_cast<long>(in_) * out_ < (1L << 32), "TurboQuantLinear: weight too large for 32-bit offsets");
        TQ_REQUIRE(packed_primary && packed_residual && norms && seeds && cb_p && cb_r, "TurboQuantLinear: NULL argument");
        TQ_REQUIRE(n_p >= 1 && n_p <= 32 && n_r >= 1 && n_r <= 16, "TurboQuantLinear: bad codebook size");
        // packing mode from the plane shapes (src/dequantizer.cpp:72-74)
        if (primary_cols == in_ / 2) primary_5bit_ = false;
        else if (primary_cols == in_) primary_5bit_ = true;
        else throw Error("TurboQuantLinear: packed_primary must have in/2 or in columns");
        device_ = tq::current_device();
        sm_count_ = tq::sm_count(device_);

        cudaStream_t st = nullptr;
        uint32_t h_seeds[3];
        TQ_CUDA(cudaMemcpy(h_seeds, seeds, sizeof h_seeds, cudaMemcpyDefault));
        seed_p_ = h_seeds[0];
        seed_r_ = h_seeds[1];

        // codes: reference planes -> joint bytes
        const size_t n_w = static_cast<size_t>(out_) * in_;
        DeviceBuffer stage_p, stage_r, flags(2 * sizeof(unsigned int));
        const uint8_t* d_pp = tq::device_view(packed_primary, static_cast<size_t>(out_) * primary_cols, stage_p, st);
        const uint8_t* d_pr = tq::device_view(packed_residual, n_w / 2, stage_r, st);
        codes_.resize(tq::code_bytes(out_, in_));
        TQ_CUDA(cudaMemsetAsync(flags.as<void>(), 0, 2 * sizeof(unsigned int), st));
        tq::launch_relayout(d_pp, d_pr, codes_.as<uint8_t>(), out_, in_, primary_5bit_, flags.as<unsigned int>(), st);
        unsigned int h_flags[2];
        TQ_CUDA(cudaMemcpy(h_flags, flags.as<void>(), sizeof h_flags, cudaMemcpyDeviceToHost));
        TQ_REQUIRE(h_flags[1] == 0, "TurboQuantLinear: 5-bit primary needs residual codes below 8 (5+3 mode)");
        has_residual_ = h_flags[0] != 0;                 // src/dequantizer.cpp:118-128
        shared_ = (seed_r_ == 0 && has_residual_);       // src/dequantizer.cpp:133
        dual_ = has_residual_ && !shared_;

        norms_.resize(static_cast<size_t>(out_) * sizeof(float));
        TQ_CUDA(cudaMemcpy(norms_.as<void>(), norms, static_cast<size_t>(out_) * sizeof(float), cudaMemcpyDefault));

        // lookup tables over the joint byte
        std::vector<float> cp(n_p), cr(n_r);
        TQ_CUDA(cudaMemcpy(cp.data(), cb_p, sizeof(float) * n_p, cudaMemcpyDefault));
        TQ_CUDA(cudaMemcpy(cr.data(), cb_r, sizeof(float) * n_r, cudaMemcpyDefault));
        std::vector<float> tables(512, 0.0f);
        const int p_bits = primary_5bit_ ? 5 : 4;
        const int p_mask = (1 << p_bits) - 1;
        auto clamp_p = [&](int i) { return cp[i < n_p ? i : n_p - 1]; };  // src/dequantizer.cpp:92-104
        auto clamp_r = [&](int i) { return cr[i < n_r ? i : n_r - 1]; };
        for (int b = 0; b < 256; ++b) {
            const int pi = b & p_mask, ri = b >> p_bits;
            if (shared_) {
                if (!primary_5bit_) {
                    // the 256-entry table of src/dequantizer.cpp:144-150; entries whose primary
                    // index lies beyond the codebook stay zero there as well
                    tables[b] = (pi < n_p) ? cp[pi] + clamp_r(ri) : 0.0f;
                } else {
                    tables[b] = clamp_p(pi) + clamp_r(ri);  // src/dequantizer.cpp:192-199
                }
            } else {
                tables[b] = clamp_p(pi);
                tables[256 + b] = clamp_r(ri);
            }
        }
        tables_.resize(512 * sizeof(float));
        TQ_CUDA(cudaMemcpy(tables_.as<void>(), tables.data(), 512 * sizeof(float), cudaMemcpyHostToDevice));

        const size_t sb = tq::gemv_scratch_bytes(out_, in_, dual_ ? 2 : 1);
        if (sb) {
            scratch_.resize(sb);
            TQ_CUDA(cudaMemset(scratch_.as<void>(), 0, sb));
        }
        const size_t ssb = tq::gemv_staged_scratch_bytes(out_, in_, dual_ ? 2 : 1, sm_count_);
        staged_scratch_.resize(ssb);
        TQ_CUDA(cudaMemset(staged_scratch_.as<void>(), 0, ssb));
        if (const char* env = std::getenv("TQ_DECODE_KERNEL")) {
            if (std::strcmp(env, "classic") == 0) decode_kernel_ = 1;
            else if (std::strcmp(env, "staged") == 0) decode_kernel_ = 2;
        }
        counter_.resize(sizeof(unsigned int));  // grid completion counter of scattering calls
        TQ_CUDA(cudaMemset(counter_.as<void>(), 0, sizeof(unsigned int)));
        // The kernels' error word is page-locked host memory that they store to directly (only on
        // a failure), so the host checks it after a synchronisation without a copy.
        TQ_CUDA(cudaMallocHost(&h_status_, sizeof(unsigned int)));
        *h_status_ = 0;
        d_status_ = static_cast<unsigned int*>(tq::pinned_host_device_alias(h_status_));
        TQ_REQUIRE(d_status_ != nullptr, "TurboQuantLinear: the status word is not mapped for the device");

        // One launch on a zero activation: proves on this device, now, that the kernel's
        // shared-memory layout holds, instead of failing on the first real forward.
        DeviceBuffer x0(static_cast<size_t>(in_) * sizeof(__half)), y0(static_cast<size_t>(out_) * sizeof(__half));
        TQ_CUDA(cudaMemset(x0.as<void>(), 0, x0.bytes()));
        launch_forward(x0.as<__half>(), 1, y0.as<__half>(), nullptr);
        TQ_CUDA(cudaDeviceSynchronize());
        check_status();
    }

    int in_features() const { return in_; }
    int out_features() const { return out_; }
    bool shared_rotation() const { return shared_; }
    bool has_residual() const { return has_residual_; }

    // x: [batch, in] fp16 or fp32, host or device.  y: [batch, out] fp16, host or device.
    void forward(const void* x, int x_dtype, int batch, void* y, cudaStream_t st) {
        TQ_REQUIRE(x && y, "TurboQuantLinear::forward: NULL argument");
        TQ_REQUIRE(batch >= 0, "TurboQuantLinear::forward: negative batch");
        TQ_REQUIRE(x_dtype == TQ_F32 || x_dtype == TQ_F16, "TurboQuantLinear::forward: x must be fp32 or fp16");
        if (batch == 0) return;
        make_current();
        const size_t nx = static_cast<size_t>(batch) * in_, ny = static_cast<size_t>(batch) * out_;
        const PointerKind kx = classify(x), ky = classify(y);
        const bool x_dev = kx.device, y_dev = ky.device;

        const __half* d_x;
        if (x_dtype == TQ_F16) {
            if (x_dev) d_x = static_cast<const __half*>(x);
            else {
                x_f16_.reserve(nx * sizeof(__half));
                TQ_CUDA(cudaMemcpyAsync(x_f16_.as<void>(), x, nx * sizeof(__half), cudaMemcpyHostToDevice, st));
                d_x = x_f16_.as<__half>();
            }
        } else {
            const float* d_xf;
            if (x_dev) d_xf = static_cast<const float*>(x);
            else {
                x_f32_.reserve(nx * sizeof(float));
                TQ_CUDA(cudaMemcpyAsync(x_f32_.as<void>(), x, nx * sizeof(float), cudaMemcpyHostToDevice, st));
                d_xf = x_f32_.as<float>();
            }
            x_f16_.reserve(nx * sizeof(__half));
            tq::launch_f32_to_f16(d_xf, x_f16_.as<__half>(), static_cast<long>(nx), st);  // src/dequantizer.cpp:691
            d_x = x_f16_.as<__half>();
        }
        // A few rows into page-locked host memory: the decode kernel stores them there itself
        // (8 KB of posted writes cost less than a separate copy); anything larger or pageable is staged.
        void* y_alias = (!y_dev && batch <= 8) ? ky.pinned_alias : nullptr;
        __half* d_y;
        if (y_dev) d_y = static_cast<__half*>(y);
        else if (y_alias) d_y = static_cast<__half*>(y_alias);
        else {
            y_f16_.reserve(ny * sizeof(__half));
            d_y = y_f16_.as<__half>();
        }
        launch_forward(d_x, batch, d_y, st);
        if (!y_dev) {
            if (!y_alias) TQ_CUDA(cudaMemcpyAsync(y, d_y, ny * sizeof(__half), cudaMemcpyDeviceToHost, st));
            TQ_CUDA(cudaStreamSynchronize(st));
            require_ok(*static_cast<volatile unsigned int*>(h_status_));
        }
    }

    // Waits for the device and reports whether any kernel of this handle refused to run or gave
    // up on a bounded wait (the word is sticky).
    // Decode forward (device fp16 in, at most 8 rows) whose result goes to several buffers at
    // once: destination d receives row r of activation row n at dst[d][n * dst_stride + row_offset + r].
    void forward_scatter(const void* x, int batch, void* const* dst, int n_dst, long dst_stride, long row_offset,
                         cudaStream_t st, void* const* signal = nullptr, int signal_slot = 0, unsigned int signal_value = 0) {
        TQ_REQUIRE(x && dst, "forward_scatter: NULL argument");
        TQ_REQUIRE(batch >= 1 && batch <= 8, "forward_scatter: batch must be 1..8");
        TQ_REQUIRE(n_dst >= 1 && n_dst <= 8, "forward_scatter: 1..8 destinations");
        TQ_REQUIRE(row_offset >= 0 && row_offset + out_ <= dst_stride,
                   "forward_scatter: rows [row_offset, row_offset + out) must fit the destination row stride");
        TQ_REQUIRE(tq::is_device_pointer(x), "forward_scatter: x must be a device pointer");
        TQ_CUDA(cudaSetDevice(device_));
        __half* d[8];
        for (int i = 0; i < n_dst; ++i) {
            TQ_REQUIRE(dst[i] != nullptr, "forward_scatter: NULL destination");
            d[i] = static_cast<__half*>(dst[i]) + row_offset;
        }
        unsigned int* sig[8];
        if (signal != nullptr) {
            TQ_REQUIRE(signal_slot >= 0 && signal_slot < 32, "forward_scatter: signal slot must be 0..31");
            for (int i = 0; i < n_dst; ++i) sig[i] = static_cast<unsigned int*>(signal[i]);
        }
        tq::launch_tq8_gemv_scatter(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(),
                                    static_cast<const __half*>(x), d, n_dst, dst_stride, out_, in_, batch, block_,
                                    dual_ ? 2 : 1, seed_p_, seed_r_, scratch_.as<void>(), d_status_,
                                    sm_count_, st, signal ? sig : nullptr, signal_slot, signal_value, counter_.as<unsigned int>());
    }

    // This layer as one matrix of a grouped decode launch (see tq_linear_forward_group).
    tq::GemvGroupItem group_item(void* y) const {
        tq::GemvGroupItem it{};
        it.codes = codes_.as<uint8_t>(); it.norms = norms_.as<float>(); it.table = tables_.as<float>();
        it.y = static_cast<__half*>(y);
        it.out = out_; it.in = in_; it.block = block_; it.n_planes = dual_ ? 2 : 1;
        it.seed_p = seed_p_; it.seed_r = seed_r_;
        it.scratch = scratch_.as<void>(); it.status = d_status_;
        return it;
    }
    // The same for batches that go to the tensor-memory GEMM (scratch for `batch` rows is reserved here).
    tq::GemmGroupItem gemm_group_item(void* y, int batch) {
        const int planes = dual_ ? 2 : 1;
        gemm_scratch_.reserve(tq::gemm_scratch_bytes(out_, in_, batch, planes, sm_count_));
        tq::GemmGroupItem it{};
        it.codes = codes_.as<uint8_t>(); it.norms = norms_.as<float>(); it.table = tables_.as<float>();
        it.y = static_cast<__half*>(y);
        it.out = out_; it.in = in_; it.block = block_; it.n_planes = planes;
        it.seed_p = seed_p_; it.seed_r = seed_r_;
        it.scratch = gemm_scratch_.as<void>(); it.status = d_status_;
        return it;
    }
    bool gemm_path(int batch) const { return batch > kGemmMinBatch && tq::gemm_supported(in_); }
    int block_size() const { return static_cast<int>(block_); }
    int device() const { return device_; }
    int sm_count() const { return sm_count_; }

    // Device fp16 in, device fp16 out whose activation rows are y_stride elements apart (this layer's
    // rows inside a wider buffer, e.g. a rank's shard of the full logits).
    void forward_strided(const void* x, int batch, void* y, long y_stride, cudaStream_t st) {
        TQ_REQUIRE(x && y, "forward_strided: NULL argument");
        TQ_REQUIRE(batch >= 1, "forward_strided: batch must be positive");
        TQ_REQUIRE(y_stride >= out_, "forward_strided: row stride smaller than out_features");
        TQ_REQUIRE(tq::is_device_pointer(x) && tq::is_device_pointer(y), "forward_strided: x and y must be device pointers");
        TQ_CUDA(cudaSetDevice(device_));
        launch_forward(static_cast<const __half*>(x), batch, static_cast<__half*>(y), st, y_stride);
    }

    // Fused all-gather for a row-sharded layer at decode batch sizes (see GemvGather).
    void forward_allgather(const void* x, int batch, void* const* dst, int n_dst, long dst_stride, long row_offset,
                           void* const* flags, int n_flags, int slot, unsigned int* epoch, const void* wait_flags, int n_wait,
                           unsigned int* wait_epoch, cudaStream_t st) {
        TQ_REQUIRE(x && dst && flags, "forward_allgather: NULL argument");
        TQ_REQUIRE(batch >= 1 && batch <= 8, "forward_allgather: batch must be 1..8");
        TQ_REQUIRE(n_dst >= 1 && n_dst <= 8 && n_flags >= 1 && n_flags <= 8, "forward_allgather: 1..8 destinations and flag arrays");
        TQ_REQUIRE(row_offset >= 0 && row_offset + out_ <= dst_stride,
                   "forward_allgather: rows [row_offset, row_offset + out) must fit the destination row stride");
        TQ_REQUIRE(slot >= 0 && slot < 32, "forward_allgather: flag slot must be 0..31");
        TQ_REQUIRE(tq::is_device_pointer(x), "forward_allgather: x must be a device pointer");
        TQ_CUDA(cudaSetDevice(device_));
        __half* d[8];
        for (int i = 0; i < n_dst; ++i) {
            TQ_REQUIRE(dst[i] != nullptr, "forward_allgather: NULL destination");
            d[i] = static_cast<__half*>(dst[i]) + row_offset;
        }
        unsigned int* sig[8];
        for (int i = 0; i < n_flags; ++i) sig[i] = static_cast<unsigned int*>(flags[i]);
        tq::GemvGather g{epoch, static_cast<const unsigned int*>(wait_flags), wait_flags ? n_wait : 0, wait_epoch};
        tq::launch_tq8_gemv_scatter(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(), static_cast<const __half*>(x), d,
                                    n_dst, dst_stride, out_, in_, batch, block_, dual_ ? 2 : 1, seed_p_, seed_r_, scratch_.as<void>(),
                                    d_status_, sm_count_, st, sig, slot, 0u, counter_.as<unsigned int>(), &g, n_flags);
    }

    // The same with the flag-in-data exchange: y (this rank's rows, plain fp16) plus packets to every other rank.
    void forward_allgather_packets(const void* x, int batch, void* y, long y_stride, void* const* packet_bufs, int rank, int world,
                                   unsigned int* epoch, bool wait, unsigned int* wait_epoch, cudaStream_t st) {
        TQ_REQUIRE(x && y && packet_bufs, "forward_allgather_packets: NULL argument");
        TQ_REQUIRE(batch >= 1 && batch <= 8, "forward_allgather_packets: batch must be 1..8");
        TQ_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world, "forward_allgather_packets: bad rank / world");
        TQ_REQUIRE(y_stride >= out_, "forward_allgather_packets: row stride smaller than the layer's rows");
        TQ_REQUIRE(tq::is_device_pointer(x) && tq::is_device_pointer(y), "forward_allgather_packets: x and y must be device pointers");
        TQ_CUDA(cudaSetDevice(device_));
        __half* d[1] = {static_cast<__half*>(y)};
        tq::GemvGather g{epoch, nullptr, wait ? 1 : 0, wait_epoch};
        g.ll_rank = rank;
        g.ll_world = world;
        for (int r = 0; r < world; ++r) g.ll_base[r] = packet_bufs[r];
        tq::launch_tq8_gemv_scatter(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(), static_cast<const __half*>(x), d, 1,
                                    y_stride, out_, in_, batch, block_, dual_ ? 2 : 1, seed_p_, seed_r_, scratch_.as<void>(), d_status_,
                                    sm_count_, st, nullptr, 0, 0u, counter_.as<unsigned int>(), &g, 0);
    }

    void wait_peers(const void* flags, int n, unsigned int value, cudaStream_t st) {
        TQ_CUDA(cudaSetDevice(device_));
        tq::launch_peer_wait(static_cast<const unsigned int*>(flags), n, value, d_status_, st);
    }

    void check_status() {
        TQ_CUDA(cudaSetDevice(device_));
        TQ_CUDA(cudaDeviceSynchronize());
        require_ok(*static_cast<volatile unsigned int*>(h_status_));
    }

    // result: [out, in] fp32 or fp16, host or device.
    void dequantize(void* result, int dtype, cudaStream_t st) {
        TQ_REQUIRE(result, "dequantize: NULL result");
        TQ_REQUIRE(dtype == TQ_F32 || dtype == TQ_F16, "dequantize: result must be fp32 or fp16");
        TQ_CUDA(cudaSetDevice(device_));
        const size_t n = static_cast<size_t>(out_) * in_;
        const size_t es = dtype == TQ_F32 ? 4 : 2;
        const bool dev = tq::is_device_pointer(result);
        DeviceBuffer stage;
        void* d_out = result;
        if (!dev) {
            stage.reserve(n * es);
            d_out = stage.as<void>();
        }
        if (dtype == TQ_F32)
            tq::launch_dequant_f32(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(), static_cast<float*>(d_out),
                                   out_, in_, block_, seed_p_, seed_r_, dual_, st);
        else
            tq::launch_dequant_f16(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(), static_cast<__half*>(d_out),
                                   out_, in_, block_, seed_p_, seed_r_, dual_, st);
        if (!dev) {
            TQ_CUDA(cudaMemcpyAsync(result, d_out, n * es, cudaMemcpyDeviceToHost, st));
            TQ_CUDA(cudaStreamSynchronize(st));
        }
    }

    // Forward that allocates nothing: device fp16 in, device fp16 out, at most 8 rows, scratch
    // from the library's built-in array.
    void forward_static(const void* x, int batch, void* y, cudaStream_t st) {
        TQ_REQUIRE(x && y, "allocation-free forward: NULL argument");
        TQ_REQUIRE(batch >= 1 && batch <= 8, "allocation-free forward: batch must be 1..8");
        TQ_REQUIRE(tq::is_device_pointer(x) && tq::is_device_pointer(y),
                   "allocation-free forward: x and y must be device pointers (copying host memory would need a staging allocation)");
        TQ_CUDA(cudaSetDevice(device_));
        // the kernel forward() would run, when its working set fits the array; else the other one
        if (decode_kernel_ == 2 && tq::gemv_staged_fits_static(out_, in_, batch, dual_ ? 2 : 1, sm_count_))
            tq::launch_tq8_gemv_staged_static(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(),
                                              static_cast<const __half*>(x), static_cast<__half*>(y), out_, in_, batch, block_,
                                              dual_ ? 2 : 1, seed_p_, seed_r_, d_status_, sm_count_, st);
        else
            tq::launch_tq8_gemv_static(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(),
                                       static_cast<const __half*>(x), static_cast<__half*>(y), out_, in_, batch, block_,
                                       dual_ ? 2 : 1, seed_p_, seed_r_, d_status_, sm_count_, st);
    }

    ~TurboQuantLinear() {
        if (h_status_) cudaFreeHost(h_status_);
    }

private:
    // What the driver knows about a caller's pointer.  A decode loop passes the same few buffers on
    // every call, so the last answers are kept (four per handle, round robin): the look-up costs a
    // driver call each time otherwise.  A buffer that is freed and re-created at the same address
    // as another KIND of memory (device / page-locked / pageable) between two calls on one handle
    // would be misjudged; callers that do that use a fresh handle or device pointers.
    struct PointerKind {
        const void* ptr = nullptr;
        bool device = false;
        void* pinned_alias = nullptr;   // device-side address of page-locked host memory, else NULL
    };
    PointerKind classify(const void* p) {
        for (const PointerKind& k : kinds_)
            if (k.ptr == p) return k;
        PointerKind k;
        k.ptr = p;
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
            cudaGetLastError();
        } else {
            k.device = attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
            k.pinned_alias = attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
        }
        kinds_[next_kind_] = k;
        next_kind_ = (next_kind_ + 1) & 3;
        return k;
    }
    // cudaSetDevice only when another device is current (it is not free even as a no-op).
    void make_current() {
        int cur = -1;
        if (cudaGetDevice(&cur) != cudaSuccess || cur != device_) TQ_CUDA(cudaSetDevice(device_));
    }
    PointerKind kinds_[4];
    int next_kind_ = 0;

    static void require_ok(unsigned int h) {
        if (h == 0) return;
        const char* what = h == 1 ? "decode kernel: unexpected shared-memory base address, kernel did not run"
                           : (h == 4 || h == 5) ? "decode kernel: a bounded wait on a partial-sum barrier gave up"
                           : h == 9 ? "prefill kernel: shared-memory layout does not fit, kernel did not run"
                           : h == 10 ? "peer wait: a rank's completion flag did not arrive within a second"
                           : (h >= 6 && h <= 8) ? "prefill kernel: a bounded wait on a pipeline barrier gave up"
                                                : "kernel reported an unknown status";
        throw Error(std::string("TurboQuantLinear: ") + what + " (status " + std::to_string(h) + ")");
    }

    // Device pointers only.  More than kGemmMinBatch rows go to the tensor-core GEMM (when the
    // shape allows); otherwise batches above 8 rows are issued as passes of 8 through the GEMV.
    static constexpr int kGemmMinBatch = 8;
    // y_stride: elements between activation rows of y (0 = out_features: a dense [batch, out] result).
    void launch_forward(const __half* d_x, int batch, __half* d_y, cudaStream_t st, long y_stride = 0) {
        if (y_stride <= 0) y_stride = out_;
        // From 9 rows on the tensor-memory kernel streams the codes once whatever the batch (its
        // activation tile is as narrow as the batch, in steps of 16 rows).
        if (batch > kGemmMinBatch && tq::gemm_supported(in_)) {
            const int planes = dual_ ? 2 : 1;
            gemm_scratch_.reserve(tq::gemm_scratch_bytes(out_, in_, batch, planes, sm_count_));
            tq::launch_tq8_gemm(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(), d_x, d_y, out_, in_, batch,
                                block_, planes, seed_p_, seed_r_, gemm_scratch_.as<void>(), d_status_,
                                sm_count_, st, y_stride);
            return;
        }
        if (y_stride != out_) {
            // rows of a wider buffer: the decode kernel's variant with an explicit destination stride
            for (int b0 = 0; b0 < batch; b0 += 8) {
                const int nb = batch - b0 < 8 ? batch - b0 : 8;
                __half* dst = d_y + static_cast<size_t>(b0) * y_stride;
                tq::launch_tq8_gemv_scatter(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(),
                                            d_x + static_cast<size_t>(b0) * in_, &dst, 1, y_stride, out_, in_, nb, block_,
                                            dual_ ? 2 : 1, seed_p_, seed_r_, scratch_.as<void>(), d_status_, sm_count_, st);
            }
            return;
        }
        for (int b0 = 0; b0 < batch; b0 += 8) {
            const int nb = batch - b0 < 8 ? batch - b0 : 8;
            if (decode_kernel_ == 2)
                tq::launch_tq8_gemv_staged(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(),
                                           d_x + static_cast<size_t>(b0) * in_, d_y + static_cast<size_t>(b0) * out_, out_, in_,
                                           nb, block_, dual_ ? 2 : 1, seed_p_, seed_r_, staged_scratch_.as<void>(), d_status_,
                                           sm_count_, st);
            else
                tq::launch_tq8_gemv(codes_.as<uint8_t>(), norms_.as<float>(), tables_.as<float>(),
                                    d_x + static_cast<size_t>(b0) * in_, d_y + static_cast<size_t>(b0) * out_, out_, in_, nb,
                                    block_, dual_ ? 2 : 1, seed_p_, seed_r_, scratch_.as<void>(),
                                    d_status_, sm_count_, st);
        }
    }

    int in_, out_;
    uint32_t block_;
    int device_ = 0, sm_count_ = 0;
    bool primary_5bit_ = false, has_residual_ = false, shared_ = false, dual_ = false;
    uint32_t seed_p_ = 0, seed_r_ = 0;
    DeviceBuffer codes_, norms_, tables_, scratch_, staged_scratch_, gemm_scratch_, counter_;
    int decode_kernel_ = 0;               // 0 / 1: register-streamed kernel (the default), 2: bulk-copy staged kernel (TQ_DECODE_KERNEL=staged)
    DeviceBuffer x_f16_, x_f32_, y_f16_;  // staging for host-side callers
    unsigned int* h_status_ = nullptr;    // the kernels' error word: page-locked host memory
    unsigned int* d_status_ = nullptr;    // its address for kernels
};

}  // namespace turboquant

struct tq_linear_s {
    turboquant::TurboQuantLinear* impl;
};

using namespace tq;

extern "C" {

tq_linear_t tq_linear_create(int in_features, int out_features, const uint8_t* packed_primary, int primary_cols,
                             const uint8_t* packed_residual, const float* norms, const uint32_t* seeds,
                             const float* primary_centroids, int n_primary, const float* residual_centroids,
                             int n_residual, uint32_t block) {
    return guarded<tq_linear_t>(nullptr, nullptr, [&]() -> tq_linear_t {
        auto* impl = new turboquant::TurboQuantLinear(in_features, out_features, packed_primary, primary_cols,
                                                      packed_residual, norms, seeds, primary_centroids, n_primary,
                                                      residual_centroids, n_residual, block);
        return new tq_linear_s{impl};
    });
}

int tq_linear_forward(tq_linear_t lin, const void* x, int x_dtype, int batch, void* y_fp16, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_forward: NULL handle");
        lin->impl->forward(x, x_dtype, batch, y_fp16, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_linear_forward_strided(tq_linear_t lin, const void* x_fp16_device, int batch, void* y_fp16_device, long y_row_stride,
                              void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_forward_strided: NULL handle");
        lin->impl->forward_strided(x_fp16_device, batch, y_fp16_device, y_row_stride, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_linear_forward_group(const tq_linear_t* lins, int n, const void* x_fp16_device, int batch, void* const* y_fp16_device,
                            void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lins && y_fp16_device && x_fp16_device, "tq_linear_forward_group: NULL argument");
        TQ_REQUIRE(n >= 1 && n <= 4, "tq_linear_forward_group: 1..4 layers");
        TQ_REQUIRE(batch >= 1, "tq_linear_forward_group: batch must be positive");
        TQ_REQUIRE(tq::is_device_pointer(x_fp16_device), "tq_linear_forward_group: x must be a device pointer");
        for (int i = 0; i < n; ++i) {
            TQ_REQUIRE(lins[i] && lins[i]->impl, "tq_linear_forward_group: NULL handle");
            TQ_REQUIRE(y_fp16_device[i] && tq::is_device_pointer(y_fp16_device[i]), "tq_linear_forward_group: y must be device pointers");
            TQ_REQUIRE(lins[i]->impl->device() == lins[0]->impl->device(), "tq_linear_forward_group: layers on different devices");
            TQ_REQUIRE(lins[i]->impl->in_features() == lins[0]->impl->in_features() &&
                       lins[i]->impl->shared_rotation() == lins[0]->impl->shared_rotation() &&
                       lins[i]->impl->block_size() == lins[0]->impl->block_size(),
                       "tq_linear_forward_group: the layers must share in_features, the WHT block and the rotation mode");
        }
        TQ_CUDA(cudaSetDevice(lins[0]->impl->device()));
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        if (lins[0]->impl->gemm_path(batch)) {
            // 9 rows and up: one rotation launch, one tensor-memory GEMM launch and one split-K finish for the group
            tq::GemmGroupItem items[4];
            for (int i = 0; i < n; ++i) items[i] = lins[i]->impl->gemm_group_item(y_fp16_device[i], batch);
            tq::launch_tq8_gemm_group(items, n, static_cast<const __half*>(x_fp16_device), batch, lins[0]->impl->sm_count(), st);
            return 0;
        }
        // the decode kernel takes up to 8 rows per launch
        for (int b0 = 0; b0 < batch; b0 += 8) {
            const int nb = batch - b0 < 8 ? batch - b0 : 8;
            tq::GemvGroupItem items[4];
            for (int i = 0; i < n; ++i)
                items[i] = lins[i]->impl->group_item(static_cast<__half*>(y_fp16_device[i]) + static_cast<size_t>(b0) * lins[i]->impl->out_features());
            tq::launch_tq8_gemv_group(items, n, static_cast<const __half*>(x_fp16_device) + static_cast<size_t>(b0) * lins[0]->impl->in_features(),
                                      nb, lins[0]->impl->sm_count(), st);
        }
        return 0;
    });
}

int tq_linear_forward_noalloc(tq_linear_t lin, const void* x_fp16_device, int batch, void* y_fp16_device, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_forward_noalloc: NULL handle");
        lin->impl->forward_static(x_fp16_device, batch, y_fp16_device, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

size_t tq_linear_noalloc_scratch_limit(void) { return tq::gemv_static_scratch_capacity(); }

int tq_linear_dequantize(tq_linear_t lin, void* result, int result_dtype, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_dequantize: NULL handle");
        lin->impl->dequantize(result, result_dtype, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

static int quantize_weight_impl(const float* weight, int out_features, int in_features, const float* primary_centroids,
                                int n_primary, const float* residual_centroids, int n_residual, int primary_bits,
                                int residual_bits, uint32_t block, int shared_rotation, const uint32_t* given_seeds,
                                uint8_t* packed_primary, uint8_t* packed_residual, float* norms, uint32_t* seeds, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(weight && primary_centroids && residual_centroids && packed_primary && packed_residual && norms && seeds,
                   "tq_quantize_weight: NULL argument");
        TQ_REQUIRE(out_features >= 0 && in_features > 0 && (in_features % 2) == 0, "tq_quantize_weight: bad shape");
        TQ_REQUIRE(n_primary >= 2 && n_primary <= 32 && n_residual >= 2 && n_residual <= 16, "tq_quantize_weight: bad codebook size");
        auto st = static_cast<cudaStream_t>(stream);
        const size_t n = static_cast<size_t>(out_features) * in_features;
        const size_t pp_bytes = primary_bits <= 4 ? n / 2 : n, pr_bytes = n / 2;
        std::vector<float> cp(n_primary), cr(n_residual);
        TQ_CUDA(cudaMemcpy(cp.data(), primary_centroids, sizeof(float) * n_primary, cudaMemcpyDefault));
        TQ_CUDA(cudaMemcpy(cr.data(), residual_centroids, sizeof(float) * n_residual, cudaMemcpyDefault));
        DeviceBuffer w_stage, recon(n * sizeof(float)), orig(static_cast<size_t>(out_features) * sizeof(float) + 4);
        const float* d_w = device_view(weight, n, w_stage, st);
        const bool pp_dev = is_device_pointer(packed_primary), pr_dev = is_device_pointer(packed_residual),
                   nm_dev = is_device_pointer(norms);
        DeviceBuffer pp_stage, pr_stage, nm_stage;
        uint8_t* d_pp = packed_primary;
        uint8_t* d_pr = packed_residual;
        float* d_nm = norms;
        if (!pp_dev) { pp_stage.reserve(pp_bytes + 4); d_pp = pp_stage.as<uint8_t>(); }
        if (!pr_dev) { pr_stage.reserve(pr_bytes + 4); d_pr = pr_stage.as<uint8_t>(); }
        if (!nm_dev) { nm_stage.reserve(static_cast<size_t>(out_features) * 4 + 4); d_nm = nm_stage.as<float>(); }
        uint32_t seed_p = 0, seed_r = 0;
        if (given_seeds != nullptr) {
            seed_p = given_seeds[0];
            seed_r = given_seeds[1];
        } else {
            derive_seeds(d_w, n, &seed_p, &seed_r, st);  // src/quantizer.cpp:69-70
        }
        launch_quantize_weight(d_w, out_features, in_features, cp.data(), n_primary, cr.data(), n_residual, primary_bits,
                               residual_bits, block, shared_rotation != 0, seed_p, seed_r, d_pp, d_pr, d_nm,
                               orig.as<float>(), recon.as<float>(), st);
        if (!pp_dev && pp_bytes) TQ_CUDA(cudaMemcpyAsync(packed_primary, d_pp, pp_bytes, cudaMemcpyDeviceToHost, st));
        if (!pr_dev && pr_bytes) TQ_CUDA(cudaMemcpyAsync(packed_residual, d_pr, pr_bytes, cudaMemcpyDeviceToHost, st));
        if (!nm_dev && out_features) TQ_CUDA(cudaMemcpyAsync(norms, d_nm, static_cast<size_t>(out_features) * 4, cudaMemcpyDeviceToHost, st));
        // seeds = {primary, residual or 0 under shared rotation, block}  (src/quantizer.cpp:255-258)
        const uint32_t h_seeds[3] = {seed_p, (shared_rotation && residual_bits > 0) ? 0u : seed_r, block};
        TQ_CUDA(cudaMemcpyAsync(seeds, h_seeds, sizeof h_seeds, cudaMemcpyDefault, st));
        TQ_CUDA(cudaStreamSynchronize(st));  // scratch and staging buffers die here
        return 0;
    });
}

int tq_quantize_weight(const float* weight, int out_features, int in_features, const float* primary_centroids,
                       int n_primary, const float* residual_centroids, int n_residual, int primary_bits,
                       int residual_bits, uint32_t block, int shared_rotation, uint8_t* packed_primary,
                       uint8_t* packed_residual, float* norms, uint32_t* seeds, void* stream) {
    return quantize_weight_impl(weight, out_features, in_features, primary_centroids, n_primary, residual_centroids, n_residual,
                                primary_bits, residual_bits, block, shared_rotation, nullptr, packed_primary, packed_residual,
                                norms, seeds, stream);
}

int tq_quantize_weight_seeded(const float* weight, int out_features, int in_features, const float* primary_centroids,
                              int n_primary, const float* residual_centroids, int n_residual, int primary_bits,
                              int residual_bits, uint32_t block, int shared_rotation, uint32_t seed_primary,
                              uint32_t seed_residual, uint8_t* packed_primary, uint8_t* packed_residual, float* norms,
                              uint32_t* seeds, void* stream) {
    const uint32_t given[2] = {seed_primary, seed_residual};
    return quantize_weight_impl(weight, out_features, in_features, primary_centroids, n_primary, residual_centroids, n_residual,
                                primary_bits, residual_bits, block, shared_rotation, given, packed_primary, packed_residual, norms,
                                seeds, stream);
}

int tq_linear_forward_scatter(tq_linear_t lin, const void* x_fp16_device, int batch, void* const* dst, int n_dst,
                              long dst_row_stride, long row_offset, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_forward_scatter: NULL handle");
        lin->impl->forward_scatter(x_fp16_device, batch, dst, n_dst, dst_row_stride, row_offset,
                                   static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_linear_forward_scatter_signal(tq_linear_t lin, const void* x_fp16_device, int batch, void* const* dst, int n_dst,
                                     long dst_row_stride, long row_offset, void* const* signal, int signal_slot,
                                     unsigned int signal_value, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_forward_scatter_signal: NULL handle");
        TQ_REQUIRE(signal != nullptr, "tq_linear_forward_scatter_signal: NULL signal list");
        lin->impl->forward_scatter(x_fp16_device, batch, dst, n_dst, dst_row_stride, row_offset,
                                   static_cast<cudaStream_t>(stream), signal, signal_slot, signal_value);
        return 0;
    });
}

// (tq_exchange_s is defined in tq_api_peer.cu; only its counters are needed here)
extern "C" unsigned int* tq_exchange_words(tq_exchange_t ex, int* rank);
extern "C" unsigned int* tq_exchange_words_world(tq_exchange_t ex, int* rank, int* world);

int tq_linear_forward_allgather(tq_linear_t lin, tq_exchange_t ex, const void* x_fp16_device, int batch, void* const* dst,
                                int n_dst, long dst_row_stride, long row_offset, void* const* flags, int n_flags,
                                const void* wait_local_flags, int n_wait, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_forward_allgather: NULL handle");
        TQ_REQUIRE(ex != nullptr, "tq_linear_forward_allgather: NULL exchange");
        int rank = 0;
        unsigned int* w = tq_exchange_words(ex, &rank);
        lin->impl->forward_allgather(x_fp16_device, batch, dst, n_dst, dst_row_stride, row_offset, flags, n_flags, rank, w + 1,
                                     wait_local_flags, n_wait, w + 2, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_linear_forward_allgather_packets(tq_linear_t lin, tq_exchange_t ex, const void* x_fp16_device, int batch, void* y_fp16_device,
                                        long y_row_stride, void* const* packet_buffers, int wait_previous, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_forward_allgather_packets: NULL handle");
        TQ_REQUIRE(ex != nullptr, "tq_linear_forward_allgather_packets: NULL exchange");
        int rank = 0, world = 0;
        unsigned int* w = tq_exchange_words_world(ex, &rank, &world);
        lin->impl->forward_allgather_packets(x_fp16_device, batch, y_fp16_device, y_row_stride, packet_buffers, rank, world, w + 1,
                                             wait_previous != 0, w + 2, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

int tq_linear_wait_peers(tq_linear_t lin, const void* local_flags, int n_flags, unsigned int value, void* stream) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_wait_peers: NULL handle");
        lin->impl->wait_peers(local_flags, n_flags, value, static_cast<cudaStream_t>(stream));
        return 0;
    });
}

void* tq_shared_alloc(size_t bytes) {
    return guarded<void*>(nullptr, nullptr, [&]() -> void* {
        TQ_REQUIRE(bytes > 0, "tq_shared_alloc: zero bytes");
        void* p = nullptr;
        TQ_CUDA(cudaMalloc(&p, bytes));
        TQ_CUDA(cudaMemset(p, 0, bytes));
        return p;
    });
}

void tq_shared_free(void* ptr) {
    if (ptr) cudaFree(ptr);
}

int tq_shared_export(void* ptr, void* handle_out, size_t handle_bytes) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(ptr && handle_out, "tq_shared_export: NULL argument");
        TQ_REQUIRE(handle_bytes >= sizeof(cudaIpcMemHandle_t), "tq_shared_export: handle buffer too small (64 bytes)");
        cudaIpcMemHandle_t h;
        TQ_CUDA(cudaIpcGetMemHandle(&h, ptr));
        std::memcpy(handle_out, &h, sizeof h);
        return 0;
    });
}

void* tq_shared_open(const void* handle, size_t handle_bytes) {
    return guarded<void*>(nullptr, nullptr, [&]() -> void* {
        TQ_REQUIRE(handle && handle_bytes >= sizeof(cudaIpcMemHandle_t), "tq_shared_open: bad handle");
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handle, sizeof h);
        void* p = nullptr;
        TQ_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        return p;
    });
}

int tq_shared_close(void* peer_ptr) {
    return guarded<int>(0, -1, [&]() {
        if (peer_ptr) TQ_CUDA(cudaIpcCloseMemHandle(peer_ptr));
        return 0;
    });
}

int tq_linear_status(tq_linear_t lin) {
    return guarded<int>(0, -1, [&]() {
        TQ_REQUIRE(lin && lin->impl, "tq_linear_status: NULL handle");
        lin->impl->check_status();
        return 0;
    });
}

int tq_linear_in_features(tq_linear_t lin) { return (lin && lin->impl) ? lin->impl->in_features() : 0; }
int tq_linear_out_features(tq_linear_t lin) { return (lin && lin->impl) ? lin->impl->out_features() : 0; }

void tq_linear_free(tq_linear_t lin) {
    if (!lin) return;
    delete lin->impl;
    delete lin;
}

}  // extern "C"
