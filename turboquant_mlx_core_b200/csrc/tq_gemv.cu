// Fused TQ8 dequantise + GEMV / skinny GEMM for decode (1..8 activation rows per pass).
//
// Replaces the reference's tq_dequant_mm Metal kernel and its host wrapper
// (metal/turboquant_dequant_mm.metal:152-313, src/dequantizer.cpp:606-721):
//   y[b, r] = fp16( norm[r] * sum_j W~[r, j] * fp16(x[b, j]) ),  fp32 accumulate.
//
// Algebra.  A dequantised row block is  norm * (inv_sqrt*sign) o H(table[codes]*inv_scale)
// and H is symmetric, so   <s o H(c), x> = <c, H(s o x)>.   The activation is therefore
// rotated ONCE per call by a small kernel (forward WHT of every block of x) and the
// weight side collapses to a table lookup per code:
//   y[b, r] = norm[r] * inv_scale * sum_j table[code[r, j]] * xrot[b, j].
//
// Two kernels per call, chained with programmatic dependent launch so that the second
// one's set-up overlaps whatever precedes it in the stream:
//   rotate_x_kernel   x fp16 [b, in] -> xrot fp32 (TF32-rounded) [b, in] in scratch
//   tq8_gemv_kernel   persistent, one CTA per SM, 16 warps:
//     HBM --(128-bit loads, 16 codes each)--> registers --(byte -> address, 1 PRMT)-->
//     shared-memory table (lane-private columns: bank-conflict free by construction)
//     --> TF32 A fragments --> mma.sync m16n8k8 against xrot held in registers as B
//     fragments --> fp32 accumulators --> cross-warp sum in shared memory --> y.
//   The table value a thread fetches IS its A-fragment register, so a weight costs one
//   integer op and one shared load; multiply-adds and the row reduction ride on the
//   tensor pipe.  Roofline: HBM; 1 B per weight + 4 B per row (norm).
//
// Shared-memory table.  256 entries, entry stride 256 B, 32 fp32 copies per entry (one
// per lane), placed at the fixed shared-window address 0x10000 so that the address of
// copy `lane` of entry `code` is a pure byte permutation of (code word, per-lane
// constant): no shift, mask or add.
//
// Work split.  A unit is one 4096-column chunk (a "slot") of a 16-row tile; when
// in_features <= 2048 the 16 warps are split over 2, 4, 8 or 16 row tiles instead, so no
// warp idles on narrow matrices.  Units are
// ordered slot-major and dealt to CTAs in contiguous ranges, so a CTA reloads its B
// fragments only when its slot changes.  With more than one slot (in_features > 4096,
// or dual rotation) each unit writes fp32 partial sums to scratch and the CTA that
// completes a row tile (per-tile arrival counter) adds the partials in slot order - a
// fixed order, so results do not depend on scheduling - applies norm*inv_scale and
// writes fp16.
// Dual-rotation weights (separate sign seeds for the primary and residual planes,
// src/dequantizer.cpp:214-246) run as two "planes": plane 0 looks up the primary
// centroid of each joint byte against x rotated with the primary seed, plane 1 the
// residual centroid against x rotated with the residual seed; planes are just further
// partial-sum slots.
#include <cmath>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kSlice = 256;               // columns per warp
constexpr int kChunk = kWarps * kSlice;   // columns per unit
constexpr uint32_t kLutAddr = 0x10000u;   // shared-window address of the table
constexpr uint32_t kLutBytes = 0x10000u;  // 256 entries * 256 B
constexpr int kRedFloats = kWarps * 128;  // one 16x8 tile per warp

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_v4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}
__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Wait for the kernel launched before this one in the stream (no-op without the
// programmatic-serialization launch attribute).
__device__ __forceinline__ void grid_dependency_sync() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Allow the next kernel in the stream to start launching.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// Address of this lane's copy of the table entry selected by byte BYTE of `word`:
//   result byte 0 = lane constant byte 0 (copy offset), byte 1 = the code,
//   bytes 2,3 = lane constant bytes 2,3 (0x0001 -> the 0x10000 base).
template <int BYTE>
__device__ __forceinline__ uint32_t lut_addr(uint32_t word, uint32_t lane_const) {
    return __byte_perm(word, lane_const, 0x7604u | (static_cast<uint32_t>(BYTE) << 4));
}

// ---- activation rotation ---------------------------------------------------------------------
// One warp per (plane, batch row, WHT block): xrot = FWHT(sign o x) / sqrt(bs), rounded to
// TF32 and stored as fp32 [plane][row][in].
template <int E>
__global__ void __launch_bounds__(128) rotate_x_kernel(const __half* __restrict__ x, float* __restrict__ xrot, int in,
                                                       int batch, int n_planes, uint32_t seed_p, uint32_t seed_r,
                                                       float inv_sqrt) {
    // Let the GEMV that follows start its set-up right away; it waits for this grid to
    // finish before it reads xrot.
    grid_launch_dependents();
    // x (and the scratch this kernel overwrites) may still be in use by the previous kernel.
    grid_dependency_sync();
    constexpr int BS = 32 * E;
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = in / BS;
    const int total = n_planes * batch * blocks_per_row;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (warp >= total) return;
    const int plane = warp / (batch * blocks_per_row);
    const int rem = warp - plane * batch * blocks_per_row;
    const int row = rem / blocks_per_row, blk = rem - row * blocks_per_row;
    const uint32_t seed = plane ? seed_r : seed_p;
    const __half* src = x + static_cast<size_t>(row) * in + blk * BS + lane * E;
    float v[E];
#pragma unroll
    for (int j = 0; j < E; ++j) v[j] = __half2float(src[j]) * sign_value(seed, static_cast<uint32_t>(lane * E + j));
    warp_fwht<E>(v, lane);
    float* dst = xrot + (static_cast<size_t>(plane) * batch + row) * in + blk * BS + lane * E;
#pragma unroll
    for (int j = 0; j < E; ++j) dst[j] = to_tf32(v[j] * inv_sqrt);
}

struct GemvArgs {
    const uint8_t* codes;   // [out, in] joint bytes
    const float* norms;     // [out]
    const float* table;     // [n_planes, 256] fp32
    const float* xrot;      // [n_planes, batch, in] fp32 (TF32-rounded)
    __half* y;              // [batch, out]
    float* partial;         // [n_slots, 8, out_pad] (only when n_slots > 1)
    unsigned int* counters; // [n_row_tiles]         (only when n_slots > 1)
    unsigned int* status;   // device error word (0 = ok)
    int out, in, batch;
    int n_row_units, n_chunks, n_slots, out_pad;  // n_slots = n_planes * n_chunks
    int wpt, tpu;           // warps per row tile, row tiles per unit (wpt * tpu = 16)
    float inv_scale;
};

__global__ void __launch_bounds__(kThreads, 1) tq8_gemv_kernel(const GemvArgs p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ unsigned int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;

    // ---- unit range of this CTA: unit = (slot, row tile), slot = plane * n_chunks + chunk ----
    const int n_units = p.n_row_units * p.n_slots;
    const int u_begin = static_cast<int>(static_cast<long>(n_units) * blockIdx.x / gridDim.x);
    const int u_end = static_cast<int>(static_cast<long>(n_units) * (blockIdx.x + 1) / gridDim.x);
    if (u_begin >= u_end) return;

    // ---- shared-memory map: [reduction buffers | ... | table at 0x10000] ----
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t red_addr = (base + 127u) & ~127u;  // 2 buffers of kRedFloats
    if (red_addr + 2u * kRedFloats * 4u > kLutAddr) {  // layout assumption broken: refuse to run
        if (tid == 0) atomicExch(p.status, 1u);
        return;
    }

    // ---- first unit's code loads go out before anything else (weights never depend on
    //      the kernel that runs before this one) ----
    const int tile_in_unit = warp / p.wpt;                 // which of the unit's row tiles this warp works on
    const int slice0 = (warp - tile_in_unit * p.wpt) * kSlice;  // column of this warp's slice inside the chunk
    // byte offset of (row g, this thread's 16 columns) inside a unit; matrices stay below 4 GiB
    const uint32_t thread_off = static_cast<uint32_t>(g) * static_cast<uint32_t>(p.in) + static_cast<uint32_t>(slice0 + 16 * q);
    const uint32_t row8_off = 8u * static_cast<uint32_t>(p.in);
    uint4 a[4][2];
    auto load_step = [&](int s, int kc, int ru) {
        const int c = kc * kChunk + slice0 + 16 * q + 64 * s;
        const int rt = ru * p.tpu + tile_in_unit;
        const int r0 = rt * 16 + g;
        const uint32_t off = static_cast<uint32_t>(rt) * 16u * static_cast<uint32_t>(p.in) +
                             static_cast<uint32_t>(kc * kChunk + 64 * s) + thread_off;
        const bool ok = c < p.in;
        a[s][0] = (ok && r0 < p.out) ? ldg_stream(p.codes + off) : make_uint4(0, 0, 0, 0);
        a[s][1] = (ok && r0 + 8 < p.out) ? ldg_stream(p.codes + off + row8_off) : make_uint4(0, 0, 0, 0);
    };
    {
        const int slot0 = u_begin / p.n_row_units;
        const int rt0 = u_begin - slot0 * p.n_row_units;
#pragma unroll
        for (int s = 0; s < 4; ++s) load_step(s, slot0 % p.n_chunks, rt0);
    }

    const uint32_t lane_const = 0x00010000u | static_cast<uint32_t>(lane * 4);
    auto build_table = [&](int plane) {
        // 256 entries x 32 copies; a thread writes 4 consecutive copies per store
        const int copy4 = (tid & 7) * 4;
        for (int e = tid >> 3; e < 256; e += kThreads / 8) {
            const float v = to_tf32(__ldg(p.table + plane * 256 + e));
            sts_v4(kLutAddr + static_cast<uint32_t>(e) * 256u + static_cast<uint32_t>(copy4) * 4u, v, v, v, v);
        }
    };
    int staged_plane = (u_begin / p.n_row_units) / p.n_chunks;
    build_table(staged_plane);

    // Everything below reads or writes data the preceding kernels produce or still use.
    grid_dependency_sync();
    __syncthreads();  // table visible

    uint32_t bfrag[4][16];
    int staged_slot = -1;
    int buf = 0;

    for (int unit = u_begin; unit < u_end; ++unit) {
        const int slot = unit / p.n_row_units;
        const int rt = unit - slot * p.n_row_units;
        const int plane = slot / p.n_chunks, kc = slot - plane * p.n_chunks;

        if (slot != staged_slot) {
            if (plane != staged_plane) {
                __syncthreads();  // nobody still reads the previous table
                build_table(plane);
                __syncthreads();
                staged_plane = plane;
            }
            // B fragment of MMA (s, m): k = q -> column 64 s + 16 q + 2 m, k = q+4 -> the next column; n = g.
            const int col0 = kc * kChunk + slice0 + 16 * q;
            const float* xr = p.xrot + (static_cast<size_t>(plane) * p.batch + g) * p.in + col0;
            const bool have_row = g < p.batch;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const bool ok = have_row && (col0 + 64 * s) < p.in;
#pragma unroll
                for (int k = 0; k < 16; k += 4) {
                    const float4 t = ok ? *reinterpret_cast<const float4*>(xr + 64 * s + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    bfrag[s][k] = __float_as_uint(t.x);
                    bfrag[s][k + 1] = __float_as_uint(t.y);
                    bfrag[s][k + 2] = __float_as_uint(t.z);
                    bfrag[s][k + 3] = __float_as_uint(t.w);
                }
            }
            staged_slot = slot;
        }

        float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
        const bool has_next = (unit + 1) < u_end;
        int nkc = kc, nrt = rt + 1;
        if (nrt == p.n_row_units) { nrt = 0; nkc = (kc + 1 == p.n_chunks) ? 0 : kc + 1; }
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint32_t lo[4] = {a[s][0].x, a[s][0].y, a[s][0].z, a[s][0].w};
            const uint32_t hi[4] = {a[s][1].x, a[s][1].y, a[s][1].z, a[s][1].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                // bytes 0,1 of the word feed one MMA, bytes 2,3 the next; two accumulator
                // chains keep consecutive MMAs independent
                {
                    const float a0 = lds_f32(lut_addr<0>(lo[w], lane_const));
                    const float a2 = lds_f32(lut_addr<1>(lo[w], lane_const));
                    const float a1 = lds_f32(lut_addr<0>(hi[w], lane_const));
                    const float a3 = lds_f32(lut_addr<1>(hi[w], lane_const));
                    mma_tf32(acc0, __float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3),
                             bfrag[s][4 * w + 0], bfrag[s][4 * w + 1]);
                }
                {
                    const float a0 = lds_f32(lut_addr<2>(lo[w], lane_const));
                    const float a2 = lds_f32(lut_addr<3>(lo[w], lane_const));
                    const float a1 = lds_f32(lut_addr<2>(hi[w], lane_const));
                    const float a3 = lds_f32(lut_addr<3>(hi[w], lane_const));
                    mma_tf32(acc1, __float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3),
                             bfrag[s][4 * w + 2], bfrag[s][4 * w + 3]);
                }
            }
            if (has_next) load_step(s, nkc, nrt);  // registers of step s are dead now: refill from the next unit
        }
        if (!has_next) grid_launch_dependents();  // last unit's codes are in: the next kernel may start setting up

        // ---- cross-warp sum of the 16 per-warp 16x8 tiles ----
        const uint32_t red = red_addr + static_cast<uint32_t>(buf * kRedFloats + warp * 128) * 4u;
        sts_f32(red + static_cast<uint32_t>(g * 8 + 2 * q) * 4u, acc0[0] + acc1[0]);
        sts_f32(red + static_cast<uint32_t>(g * 8 + 2 * q + 1) * 4u, acc0[1] + acc1[1]);
        sts_f32(red + static_cast<uint32_t>((g + 8) * 8 + 2 * q) * 4u, acc0[2] + acc1[2]);
        sts_f32(red + static_cast<uint32_t>((g + 8) * 8 + 2 * q + 1) * 4u, acc0[3] + acc1[3]);
        __syncthreads();
        // thread idx -> (tile of the unit, row in tile, activation row n)
        for (int idx = tid; idx < p.tpu * 128; idx += kThreads) {
            const int t = idx >> 7, e = idx & 127;
            const int n = e & 7;
            const int row = (rt * p.tpu + t) * 16 + (e >> 3);
            const uint32_t src = red_addr + static_cast<uint32_t>(buf * kRedFloats + t * p.wpt * 128 + e) * 4u;
            float sum = 0.f;
            for (int w = 0; w < p.wpt; ++w) sum += lds_f32(src + static_cast<uint32_t>(w * 128) * 4u);
            if (row < p.out) {
                if (p.n_slots == 1) {
                    if (n < p.batch) p.y[static_cast<size_t>(n) * p.out + row] = __float2half_rn(sum * (p.norms[row] * p.inv_scale));
                } else {
                    p.partial[(static_cast<size_t>(slot) * 8 + n) * p.out_pad + row] = sum;
                }
            }
        }
        if (p.n_slots > 1) {
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned int prev = atomicAdd(&p.counters[rt], 1u);
                s_last = (prev == static_cast<unsigned int>(p.n_slots - 1)) ? 1u : 0u;
                if (s_last) p.counters[rt] = 0u;  // ready for the next launch
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                for (int idx = tid; idx < p.tpu * 128; idx += kThreads) {
                    const int t = idx >> 7, e = idx & 127;
                    const int n = e & 7;
                    const int row = (rt * p.tpu + t) * 16 + (e >> 3);
                    if (row < p.out && n < p.batch) {
                        float total = 0.f;
                        for (int c = 0; c < p.n_slots; ++c)
                            total += __ldcg(p.partial + (static_cast<size_t>(c) * 8 + n) * p.out_pad + row);
                        p.y[static_cast<size_t>(n) * p.out + row] = __float2half_rn(total * (p.norms[row] * p.inv_scale));
                    }
                }
            }
        }
        buf ^= 1;
    }
}

constexpr size_t kGemvSmem = kLutAddr + kLutBytes;

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// Warps that share one 16-row tile: enough 256-column slices to cover a chunk, as a power of two.
int warps_per_tile(int in) {
    const int cols = in < kChunk ? in : kChunk;
    int w = 1;
    while (w < kWarps && w * kSlice < cols) w <<= 1;
    return w;
}

}  // namespace

// Scratch layout: [xrot: n_planes*8*in fp32][partials: n_slots*8*out_pad fp32][counters: n_row_tiles u32]
size_t gemv_scratch_bytes(int out, int in, int n_planes) {
    const int n_slots = ((in + kChunk - 1) / kChunk) * n_planes;
    const int n_row_tiles = (out + 15) / 16;
    const size_t out_pad = static_cast<size_t>(n_row_tiles) * 16;
    size_t bytes = align256(static_cast<size_t>(n_planes) * 8 * in * sizeof(float));
    if (n_slots > 1)
        bytes += align256(static_cast<size_t>(n_slots) * 8 * out_pad * sizeof(float)) +
                 align256(static_cast<size_t>(n_row_tiles) * sizeof(unsigned int));
    return bytes;
}

void launch_tq8_gemv(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                     int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                     void* scratch, unsigned int* status, int sm_count, cudaStream_t stream) {
    TQ_REQUIRE(n_planes == 1 || n_planes == 2, "tq8_gemv: one or two rotation planes");
    TQ_REQUIRE(batch >= 1 && batch <= 8, "tq8_gemv handles 1..8 activation rows per launch");
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "WHT block size must be a power of two in [32, 1024]");
    TQ_REQUIRE(in % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    TQ_REQUIRE(scratch != nullptr, "tq8_gemv needs its scratch buffer");
    if (out == 0) return;

    GemvArgs a{};
    a.codes = codes; a.norms = norms; a.table = table; a.y = y; a.status = status;
    a.out = out; a.in = in; a.batch = batch;
    const int n_row_tiles = (out + 15) / 16;
    a.n_chunks = (in + kChunk - 1) / kChunk;
    a.n_slots = a.n_chunks * n_planes;
    a.out_pad = n_row_tiles * 16;
    a.wpt = warps_per_tile(in);
    a.tpu = kWarps / a.wpt;
    a.n_row_units = (n_row_tiles + a.tpu - 1) / a.tpu;
    a.inv_scale = 1.0f / std::sqrt(static_cast<float>(in));
    uint8_t* sp = static_cast<uint8_t*>(scratch);
    float* xrot = reinterpret_cast<float*>(sp);
    a.xrot = xrot;
    if (a.n_slots > 1) {
        sp += align256(static_cast<size_t>(n_planes) * 8 * in * sizeof(float));
        a.partial = reinterpret_cast<float*>(sp);
        sp += align256(static_cast<size_t>(a.n_slots) * 8 * a.out_pad * sizeof(float));
        a.counters = reinterpret_cast<unsigned int*>(sp);
    }

    // the opt-in shared-memory size is a per-device function attribute
    static bool configured[64] = {false};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(tq8_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemvSmem)));
        if (dev < 64) configured[dev] = true;
    }

    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;

    // 1. rotate the activation (one warp per plane x row x block)
    {
        const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(block));
        const int n_warps = n_planes * batch * (in / static_cast<int>(block));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((n_warps + 3) / 4);
        cfg.blockDim = dim3(128);
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
#define TQ_ROT_CASE(EV)                                                                                            \
    case 32 * EV:                                                                                                  \
        TQ_CUDA(cudaLaunchKernelEx(&cfg, rotate_x_kernel<EV>, x, xrot, in, batch, n_planes, seed_p, seed_r, inv_sqrt)); \
        break;
        switch (block) {
            TQ_ROT_CASE(1) TQ_ROT_CASE(2) TQ_ROT_CASE(4) TQ_ROT_CASE(8) TQ_ROT_CASE(16) TQ_ROT_CASE(32)
            default: throw Error("unsupported WHT block size");
        }
#undef TQ_ROT_CASE
    }
    // 2. the GEMV itself
    {
        const int n_units = a.n_row_units * a.n_slots;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(n_units < sm_count ? n_units : sm_count);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kGemvSmem;
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_kernel, a));
    }
}

// ---- allocation-free variant ---------------------------------------------------------------
// Same two kernels, but the scratch (rotated activation, split-K partial sums, arrival
// counters) lives in a fixed array inside the library image instead of a buffer the handle
// allocated.  Every GPU that loads the library carries these bytes until the process exits.
constexpr size_t kStaticScratchBytes = size_t(2) << 20;  // 2 MiB
static __device__ __align__(256) unsigned char g_gemv_static_scratch[kStaticScratchBytes];

size_t gemv_static_scratch_capacity() { return kStaticScratchBytes; }

// Device address of the array on the current device.  In host code the array's name is only
// a handle for the runtime, not an address a kernel could use, so the address is looked up
// once per device (with that device current) and cached.
static void* static_scratch_address() {
    static void* cached[64] = {nullptr};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && cached[dev]) return cached[dev];
    void* ptr = nullptr;
    TQ_CUDA(cudaGetSymbolAddress(&ptr, g_gemv_static_scratch));
    TQ_REQUIRE(ptr != nullptr, "tq8_gemv: static scratch has no device address");
    if (dev >= 0 && dev < 64) cached[dev] = ptr;
    return ptr;
}

void launch_tq8_gemv_static(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                            int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                            unsigned int* status, int sm_count, cudaStream_t stream) {
    const size_t need = gemv_scratch_bytes(out, in, n_planes);
    if (need > kStaticScratchBytes)
        throw Error("allocation-free forward: this layer needs " + std::to_string(need) +
                    " bytes of scratch, the built-in array holds " + std::to_string(kStaticScratchBytes));
    void* scratch = static_scratch_address();
    // The array is shared by every call and keeps what the last one left.  The arrival
    // counters are the only part that must read zero at kernel start; the kernels re-zero
    // them on exit, but a call cut short (device error, aborted process sharing the context)
    // would leave them dirty, so they are cleared here, in stream order.
    const size_t xrot_bytes = align256(static_cast<size_t>(n_planes) * 8 * in * sizeof(float));
    if (need > xrot_bytes) {
        const int n_row_tiles = (out + 15) / 16;
        const size_t counter_bytes = align256(static_cast<size_t>(n_row_tiles) * sizeof(unsigned int));
        TQ_CUDA(cudaMemsetAsync(static_cast<uint8_t*>(scratch) + need - counter_bytes, 0, counter_bytes, stream));
    }
    launch_tq8_gemv(codes, norms, table, x, y, out, in, batch, block, n_planes, seed_p, seed_r, scratch, status, sm_count,
                    stream);
}

}  // namespace tq
