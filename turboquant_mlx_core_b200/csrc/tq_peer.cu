// Rank-to-rank exchange for the sharded paths, over peer-mapped device memory (one process per
// GPU, buffers shared through CUDA IPC: tq_shared_alloc / tq_shared_open).
//
// The reference has no data plane between devices (src/distributed.cpp plans a layer split and
// nothing else), so there is no counterpart; the shapes come from the partition rules of the sharded
// paths: row-sharded linears exchange fp16 output shards (an all-gather), column-sharded linears
// exchange partial outputs that are then added (an all-reduce), and decode attention split over the
// context exchanges (output, log-sum-exp) parts that are then merged.
//
// One primitive carries all three: exchange_broadcast copies a block of this rank's memory into the
// same place of every rank's buffer with plain 16-byte stores (NVLink for the peers; no multicast,
// no collective library) and then raises this rank's flag on every rank; exchange_wait is a one-warp
// kernel that waits - for at most a second - until every rank's flag has arrived locally.  Flags
// carry an epoch that both sides keep in device memory, so a captured CUDA graph can be replayed:
// nothing in the kernel arguments changes from step to step.  exchange_sum_f16 adds the ranks'
// slots in rank order (fixed order: every rank computes the same bits), exchange_merge_attention
// merges softmax parts.  A kernel only ever waits for kernels running on OTHER GPUs.
#include <cstdint>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

constexpr int kBcastThreads = 256;
constexpr unsigned long long kPeerWaitNs = 1000ull * 1000 * 1000;   // a rank that is a second late is gone

__device__ __forceinline__ unsigned long long p_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

struct BcastArgs {
    const uint8_t* src;        // this rank's block: rows x row_bytes, rows src_stride bytes apart
    uint8_t* dst[8];           // the same block's place in every rank's buffer
    unsigned int* signal[8];   // every rank's flag array (the local one included)
    int n_dst, n_signal;
    int rows;
    long row_bytes, src_stride, dst_stride;   // row_bytes is a multiple of 16
    int slot;                  // which flag this rank raises (its rank)
    unsigned int* done;        // device word, zero between launches: CTAs finished
    unsigned int* epoch;       // device word: how many broadcasts this exchange has completed
};

// grid = (CTAs per destination, destinations)
__global__ void __launch_bounds__(kBcastThreads) exchange_broadcast_kernel(const BcastArgs p) {
    // The data was written by the kernel before this one in the stream.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int d = blockIdx.y;
    const long pieces_per_row = p.row_bytes >> 4;
    const long total = pieces_per_row * p.rows;
    uint8_t* dst = p.dst[d];
    for (long i = static_cast<long>(blockIdx.x) * kBcastThreads + threadIdx.x; i < total;
         i += static_cast<long>(gridDim.x) * kBcastThreads) {
        const long r = i / pieces_per_row, c = i - r * pieces_per_row;
        const uint4 v = *reinterpret_cast<const uint4*>(p.src + r * p.src_stride + (c << 4));
        *reinterpret_cast<uint4*>(dst + r * p.dst_stride + (c << 4)) = v;
    }
    // Order this CTA's (possibly remote) stores system-wide, count in, and let the CTA that completes
    // the grid publish the flag: whoever reads it with acquire semantics sees the whole block.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int n_ctas = gridDim.x * gridDim.y;
        const unsigned int prev = atomicAdd(p.done, 1u);
        if (prev == n_ctas - 1) {
            *p.done = 0u;   // ready for the next launch (stream order)
            const unsigned int e = atomicAdd(p.epoch, 1u) + 1u;
            __threadfence_system();
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < p.n_signal)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.signal[k] + p.slot), "r"(e) : "memory");
        }
    }
}

// One warp: lane i waits until flags[i] has reached the epoch of this wait (kept in *epoch, which
// the kernel advances by one per launch).
__global__ void exchange_wait_kernel(const unsigned int* __restrict__ flags, int n, unsigned int* epoch, unsigned int* status) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x;
    unsigned int want = 0;
    if (lane == 0) want = atomicAdd(epoch, 1u) + 1u;
    want = __shfl_sync(0xffffffffu, want, 0);
    if (lane >= n) return;
    const unsigned long long t0 = p_timer_ns();
    for (unsigned int spin = 0;; ++spin) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
        if (static_cast<int>(v - want) >= 0) return;
        if ((spin & 255u) == 255u && p_timer_ns() - t0 > kPeerWaitNs) {
            raise_status(status, 10u);
            return;
        }
    }
}

// out[i] = fp16( residual[i] + sum over slots s, in slot order, of fp32(slots[s][i]) )   (residual may be NULL)
// With norm_w (one CTA per row of `cols` elements): the CTA then writes normed[row] = RMSNorm(out[row]) * norm_w, the
// bits rmsnorm_kernel would give on out.
__global__ void __launch_bounds__(kRowNormThreads) exchange_sum_f16_kernel(const __half* __restrict__ slots, int n_slots, long slot_stride,
                                                               long count, const __half* __restrict__ residual, __half* __restrict__ out,
                                                               const __half* __restrict__ norm_w, __half* __restrict__ normed, int cols,
                                                               float eps) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const bool by_row = norm_w != nullptr;
    const long first = by_row ? static_cast<long>(blockIdx.x) * cols + threadIdx.x * 2 : (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
    const long last = by_row ? static_cast<long>(blockIdx.x + 1) * cols : count;
    const long step = by_row ? static_cast<long>(blockDim.x) * 2 : static_cast<long>(gridDim.x) * blockDim.x * 2;
    for (long i = first; i < last; i += step) {
        float a = 0.f, b = 0.f;
        if (residual != nullptr) {
            const __half2 h = *reinterpret_cast<const __half2*>(residual + i);
            a = __low2float(h);
            b = __high2float(h);
        }
        for (int s = 0; s < n_slots; ++s) {
            const __half2 h = *reinterpret_cast<const __half2*>(slots + s * slot_stride + i);   // written by other GPUs: plain loads after the acquire of the wait kernel
            a += __low2float(h);
            b += __high2float(h);
        }
        *reinterpret_cast<__half2*>(out + i) = __floats2half2_rn(a, b);
    }
    if (by_row) {
        __syncthreads();   // the row is complete (this CTA wrote all of it)
        rmsnorm_row(out + static_cast<long>(blockIdx.x) * cols, norm_w, normed + static_cast<long>(blockIdx.x) * cols, cols, eps);
    }
}

// Packets of the flag-in-data exchange {2 halves, epoch, 2 halves, epoch} -> contiguous fp16 (4 per packet).
__global__ void __launch_bounds__(256) exchange_unpack_packets_kernel(const uint4* __restrict__ packets, long n, uint2* __restrict__ out) {
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
        const uint4 pk = packets[i];
        out[i] = make_uint2(pk.x, pk.z);
    }
}

// Waits (bounded) for the packets every other rank wrote in the exchange that has just completed on this rank
// (*epoch is its number) and writes their rows into the gathered result: row block `src` of every activation row.
__global__ void __launch_bounds__(256) exchange_wait_packets_kernel(const uint4* __restrict__ base, const unsigned int* __restrict__ epoch,
                                                                    unsigned int* __restrict__ wait_epoch, int rank, int world, long per_row,
                                                                    int batch, long rows, __half* __restrict__ out, long out_stride,
                                                                    unsigned int* status) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const unsigned int want = *reinterpret_cast<const volatile unsigned int*>(epoch);
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(wait_epoch, 1u);   // one wait per exchange, like tq_exchange_wait
    const long packets = static_cast<long>(batch) * per_row;
    const uint4* const half = base + static_cast<size_t>(want & 1u) * world * packets;
    const unsigned long long t0 = p_timer_ns();
    const long total = packets * (world - 1);
    for (long j = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; j < total; j += static_cast<long>(gridDim.x) * blockDim.x) {
        int src = static_cast<int>(j / packets);
        const long i = j - static_cast<long>(src) * packets;
        if (src >= rank) ++src;
        const uint4* at = half + static_cast<size_t>(src) * packets + i;
        uint4 pk;
        for (unsigned int spin = 0;; ++spin) {
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(pk.x), "=r"(pk.y), "=r"(pk.z), "=r"(pk.w) : "l"(at) : "memory");
            if (static_cast<int>(pk.y - want) >= 0 && static_cast<int>(pk.w - want) >= 0) break;
            if ((spin & 255u) == 255u && p_timer_ns() - t0 > kPeerWaitNs) {
                raise_status(status, 10u);
                return;
            }
        }
        const long n = i / per_row, c = i - n * per_row;
        *reinterpret_cast<uint2*>(out + n * out_stride + static_cast<long>(src) * rows + 4 * c) = make_uint2(pk.x, pk.z);
    }
}

// All-reduce tail for partial sums that travelled as packets: out = fp16(residual + sum over ranks, in rank order, fp32),
// this rank's own partial read from `local` ([batch][rows] fp16), the others' polled (bounded) from the packets of the
// exchange that has just completed on this rank.  The arithmetic is exchange_sum_f16_kernel's.
__global__ void __launch_bounds__(kRowNormThreads) exchange_sum_packets_kernel(const uint4* __restrict__ base, const unsigned int* __restrict__ epoch,
                                                                   unsigned int* __restrict__ wait_epoch, int rank, int world, long packets,
                                                                   const __half* __restrict__ local, const __half* __restrict__ residual,
                                                                   __half* __restrict__ out, unsigned int* status,
                                                                   const __half* __restrict__ norm_w, __half* __restrict__ normed, int cols,
                                                                   float eps) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const unsigned int want = *reinterpret_cast<const volatile unsigned int*>(epoch);
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(wait_epoch, 1u);
    const uint4* const half = base + static_cast<size_t>(want & 1u) * world * packets;
    const unsigned long long t0 = p_timer_ns();
    // with norm_w: one CTA per row of cols elements (cols / 4 packets), which it normalises afterwards
    const bool by_row = norm_w != nullptr;
    const long per_row = cols / 4;
    const long first = by_row ? static_cast<long>(blockIdx.x) * per_row + threadIdx.x : static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long last = by_row ? static_cast<long>(blockIdx.x + 1) * per_row : packets;
    const long step = by_row ? static_cast<long>(blockDim.x) : static_cast<long>(gridDim.x) * blockDim.x;
    bool gave_up = false;
    for (long i = first; i < last && !gave_up; i += step) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
        if (residual != nullptr) {
            const uint2 r = *reinterpret_cast<const uint2*>(residual + 4 * i);
            const float2 r0 = __half22float2(*reinterpret_cast<const __half2*>(&r.x)), r1 = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
            a[0] = r0.x; a[1] = r0.y; a[2] = r1.x; a[3] = r1.y;
        }
        // every rank's packet is requested first (one round trip for all of them), then checked, and only what has
        // not arrived yet is polled again; the additions run in rank order afterwards
        uint4 pk[8];
#pragma unroll
        for (int src = 0; src < 8; ++src) {
            if (src < world && src != rank) {
                const uint4* at = half + static_cast<size_t>(src) * packets + i;
                asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(pk[src].x), "=r"(pk[src].y), "=r"(pk[src].z), "=r"(pk[src].w) : "l"(at) : "memory");
            }
        }
#pragma unroll
        for (int src = 0; src < 8; ++src) {
            if (src < world && src != rank && !gave_up) {
                const uint4* at = half + static_cast<size_t>(src) * packets + i;
                for (unsigned int spin = 0; !(static_cast<int>(pk[src].y - want) >= 0 && static_cast<int>(pk[src].w - want) >= 0); ++spin) {
                    if ((spin & 255u) == 255u && p_timer_ns() - t0 > kPeerWaitNs) {   // a peer is gone: stop polling
                        raise_status(status, 10u);
                        gave_up = true;
                        break;
                    }
                    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(pk[src].x), "=r"(pk[src].y), "=r"(pk[src].z), "=r"(pk[src].w) : "l"(at) : "memory");
                }
            }
        }
#pragma unroll
        for (int src = 0; src < 8; ++src) {
            if (src < world) {
                uint2 v;
                if (src == rank) v = *reinterpret_cast<const uint2*>(local + 4 * i);
                else v = make_uint2(pk[src].x, pk[src].z);
                const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), v1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
                a[0] += v0.x; a[1] += v0.y; a[2] += v1.x; a[3] += v1.y;
            }
        }
        if (gave_up) break;
        const __half2 o0 = __floats2half2_rn(a[0], a[1]), o1 = __floats2half2_rn(a[2], a[3]);
        *reinterpret_cast<uint2*>(out + 4 * i) = make_uint2(*reinterpret_cast<const uint32_t*>(&o0), *reinterpret_cast<const uint32_t*>(&o1));
    }
    if (by_row) {
        __syncthreads();   // the row is complete (every thread gets here, also after a timeout)
        rmsnorm_row(out + static_cast<long>(blockIdx.x) * cols, norm_w, normed + static_cast<long>(blockIdx.x) * cols, cols, eps);
    }
}

// Softmax parts over disjoint token ranges of the same rows -> attention over the union:
//   out = sum_p w_p * out_p / sum_p w_p,  w_p = exp(lse_p - max_p lse_p)   (parts in order).
// outs: [parts][rows][dim] fp16 (part_stride_o elements apart), lses: [parts][rows] fp32.
__global__ void __launch_bounds__(128) exchange_merge_attention_kernel(const __half* __restrict__ outs, const float* __restrict__ lses,
                                                                       int parts, long rows, int dim, long part_stride_o,
                                                                       long part_stride_l, __half* __restrict__ out) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const long row = blockIdx.x;
    if (row >= rows) return;
    float m = -INFINITY;
    for (int q = 0; q < parts; ++q) m = fmaxf(m, lses[q * part_stride_l + row]);
    if (!(m > -INFINITY) || !(m < INFINITY)) m = 0.f;
    float den = 0.f;
    for (int q = 0; q < parts; ++q) den += __expf(lses[q * part_stride_l + row] - m);
    den = fmaxf(den, 1e-38f);
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float num = 0.f;
        for (int q = 0; q < parts; ++q)
            num += __expf(lses[q * part_stride_l + row] - m) * __half2float(outs[q * part_stride_o + row * dim + c]);
        out[row * dim + c] = __float2half_rn(num / den);
    }
}

cudaLaunchConfig_t pdl_config(dim3 grid, dim3 block, cudaStream_t stream, cudaLaunchAttribute* attr) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cfg;
}

}  // namespace

void launch_exchange_broadcast(const void* src, void* const* dst, int n_dst, int rows, long row_bytes, long src_stride,
                               long dst_stride, unsigned int* const* signal, int n_signal, int slot, unsigned int* done,
                               unsigned int* epoch, cudaStream_t stream) {
    TQ_REQUIRE(src != nullptr && dst != nullptr && signal != nullptr, "exchange broadcast: NULL argument");
    TQ_REQUIRE(n_dst >= 1 && n_dst <= 8, "exchange broadcast: 1..8 destinations");
    TQ_REQUIRE(n_signal >= 1 && n_signal <= 8, "exchange broadcast: 1..8 flag arrays");
    TQ_REQUIRE(rows >= 1 && row_bytes > 0 && row_bytes % 16 == 0, "exchange broadcast: rows of a multiple of 16 bytes");
    TQ_REQUIRE(reinterpret_cast<uintptr_t>(src) % 16 == 0 && src_stride % 16 == 0 && dst_stride % 16 == 0,
               "exchange broadcast: 16-byte aligned block");
    TQ_REQUIRE(slot >= 0 && slot < 32, "exchange broadcast: flag slot must be 0..31");
    BcastArgs a{};
    a.src = static_cast<const uint8_t*>(src);
    for (int d = 0; d < n_dst; ++d) {
        TQ_REQUIRE(dst[d] != nullptr, "exchange broadcast: NULL destination");
        TQ_REQUIRE(reinterpret_cast<uintptr_t>(dst[d]) % 16 == 0, "exchange broadcast: 16-byte aligned destinations");
        a.dst[d] = static_cast<uint8_t*>(dst[d]);
    }
    for (int d = 0; d < n_signal; ++d) {
        TQ_REQUIRE(signal[d] != nullptr, "exchange broadcast: NULL flag array");
        a.signal[d] = signal[d];
    }
    a.n_signal = n_signal;
    a.n_dst = n_dst; a.rows = rows; a.row_bytes = row_bytes; a.src_stride = src_stride; a.dst_stride = dst_stride;
    a.slot = slot; a.done = done; a.epoch = epoch;
    const long pieces = (row_bytes >> 4) * rows;
    long ctas = (pieces + kBcastThreads * 4 - 1) / (kBcastThreads * 4);   // about four 16-byte pieces per thread
    if (ctas < 1) ctas = 1;
    if (ctas > 16) ctas = 16;
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = pdl_config(dim3(static_cast<unsigned>(ctas), static_cast<unsigned>(n_dst)), dim3(kBcastThreads), stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, exchange_broadcast_kernel, a));
}

void launch_exchange_wait(const unsigned int* flags, int n, unsigned int* epoch, unsigned int* status, cudaStream_t stream) {
    TQ_REQUIRE(flags != nullptr && n >= 1 && n <= 32, "exchange wait: 1..32 flags");
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = pdl_config(dim3(1), dim3(32), stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, exchange_wait_kernel, flags, n, epoch, status));
}

void launch_exchange_sum_f16(const __half* slots, int n_slots, long slot_stride, long count, const __half* residual, __half* out,
                             cudaStream_t stream, const __half* norm_w, __half* normed, int cols, float eps) {
    TQ_REQUIRE(slots != nullptr && out != nullptr && n_slots >= 1, "exchange sum: NULL argument");
    TQ_REQUIRE(count % 2 == 0 && slot_stride % 2 == 0 && reinterpret_cast<uintptr_t>(slots) % 4 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 4 == 0,
               "exchange sum: even element counts and 4-byte aligned buffers");
    if (count == 0) return;
    long blocks = (count / 2 + 255) / 256;
    if (blocks > 296) blocks = 296;
    if (norm_w != nullptr) {
        TQ_REQUIRE(normed != nullptr && cols > 0 && cols % 2 == 0 && count % cols == 0, "exchange sum + RMSNorm: whole rows of an even length");
        blocks = count / cols;
    }
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = pdl_config(dim3(static_cast<unsigned>(blocks)), dim3(norm_w ? kRowNormThreads : 256), stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, exchange_sum_f16_kernel, slots, n_slots, slot_stride, count, residual, out, norm_w, normed, cols, eps));
}

void launch_exchange_unpack_packets(const uint4* packets, long n_packets, __half* out, cudaStream_t stream) {
    TQ_REQUIRE(reinterpret_cast<uintptr_t>(out) % 8 == 0, "packet unpack: the destination must be 8-byte aligned");
    if (n_packets == 0) return;
    const int blocks = static_cast<int>(n_packets + 255 < 296L * 256 ? (n_packets + 255) / 256 : 296);
    exchange_unpack_packets_kernel<<<blocks, 256, 0, stream>>>(packets, n_packets, reinterpret_cast<uint2*>(out));
    TQ_CUDA(cudaGetLastError());
}

void launch_exchange_sum_packets(const uint4* base, const unsigned int* epoch, unsigned int* wait_epoch, int rank, int world, long count,
                                 const __half* local, const __half* residual, __half* out, unsigned int* status, cudaStream_t stream,
                                 const __half* norm_w, __half* normed, int cols, float eps) {
    TQ_REQUIRE(base && epoch && wait_epoch && local && out && world >= 1 && world <= 8 && rank >= 0 && rank < world && count % 4 == 0,
               "packet sum: element counts in groups of four");
    TQ_REQUIRE(reinterpret_cast<uintptr_t>(local) % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0 &&
                   reinterpret_cast<uintptr_t>(residual) % 8 == 0,
               "packet sum: 8-byte aligned buffers");
    if (count == 0) return;
    const long packets = count / 4;
    int blocks = static_cast<int>(packets + 255 < 296L * 256 ? (packets + 255) / 256 : 296);
    if (norm_w != nullptr) {
        TQ_REQUIRE(normed != nullptr && cols > 0 && cols % 4 == 0 && count % cols == 0, "packet sum + RMSNorm: whole rows, a multiple of four long");
        blocks = static_cast<int>(count / cols);
    }
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = pdl_config(dim3(static_cast<unsigned>(blocks)), dim3(norm_w ? kRowNormThreads : 256), stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, exchange_sum_packets_kernel, base, epoch, wait_epoch, rank, world, packets, local, residual, out, status,
                               norm_w, normed, cols, eps));
}

void launch_exchange_wait_packets(const uint4* base, const unsigned int* epoch, unsigned int* wait_epoch, int rank, int world, long rows,
                                  int batch, __half* out, long out_stride, unsigned int* status, cudaStream_t stream) {
    TQ_REQUIRE(base && epoch && out && world >= 1 && rank >= 0 && rank < world && rows % 4 == 0 && out_stride % 4 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 8 == 0,
               "packet wait: rows and strides in groups of four, 8-byte aligned destination");
    if (world == 1 || rows == 0 || batch == 0) return;
    const long total = static_cast<long>(batch) * (rows / 4) * (world - 1);
    const int blocks = static_cast<int>(total + 255 < 296L * 256 ? (total + 255) / 256 : 296);
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = pdl_config(dim3(static_cast<unsigned>(blocks)), dim3(256), stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, exchange_wait_packets_kernel, base, epoch, wait_epoch, rank, world, rows / 4, batch, rows, out, out_stride,
                               status));
}

void launch_exchange_merge_attention(const __half* outs, const float* lses, int parts, long rows, int dim, long part_stride_o,
                                     long part_stride_l, __half* out, cudaStream_t stream) {
    TQ_REQUIRE(outs != nullptr && lses != nullptr && out != nullptr && parts >= 1 && dim >= 1, "attention merge: bad argument");
    if (rows == 0) return;
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = pdl_config(dim3(static_cast<unsigned>(rows)), dim3(128), stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, exchange_merge_attention_kernel, outs, lses, parts, rows, dim, part_stride_o, part_stride_l, out));
}

}  // namespace tq
