// Fused TQ8 dequantise + GEMV / skinny GEMM for decode (batch 1..8 per pass).
//
// Replaces the reference's tq_dequant_mm Metal kernel and its host wrapper
// (metal/turboquant_dequant_mm.metal:152-313, src/dequantizer.cpp:606-721):
//   y[b, r] = fp16( norm[r] * sum_j W~[r, j] * fp16(x[b, j]) ),  fp32 accumulate.
//
// Algebra.  A dequantised row block is  norm * (inv_sqrt*sign) o H(table[codes]*inv_scale)
// and H is symmetric, so   <s o H(c), x> = <c, H(s o x)>.   The activation is therefore
// rotated ONCE per launch (forward WHT of each block of x, done by every CTA for the
// column chunk it works on) and the weight side collapses to a table lookup per code:
//   y[b, r] = norm[r] * inv_scale * sum_j table[code[r, j]] * xrot[b, j].
//
// Data flow per CTA (persistent, one per SM, 16 warps):
//   HBM --(128-bit loads, 16 codes each)--> registers --(byte -> address, 1 PRMT)-->
//   shared-memory table (lane-private columns, bank-conflict free by construction)
//   --> TF32 A fragments --> mma.sync m16n8k8 against the rotated activation held in
//   registers as B fragments --> fp32 accumulators --> cross-warp sum in shared memory.
// The table value fetched by a thread IS the A-fragment register, so a weight costs one
// integer op and one shared load; the multiply-adds and the reduction over a row ride on
// the tensor pipe.  Roofline: HBM; 1 B per weight + 4 B per row (norm).
//
// Shared-memory table.  256 entries x 64 fp32 copies (entry stride 256 B), placed at
// the fixed shared-window address 0x10000 so that the address of copy `lane` of entry
// `code` is a pure byte permutation of (code word, per-lane constant): no shift, mask
// or add.  Even warps use copies 0..31, odd warps 32..63.
//
// Work split.  A unit is a 16-row tile x one 4096-column chunk.  Units are ordered
// chunk-major and dealt to CTAs in contiguous ranges, so a CTA re-stages the rotated
// activation only when its chunk changes.  With more than one chunk (in_features > 4096)
// each unit writes fp32 partial sums to scratch and the CTA that completes a row tile
// (per-tile arrival counter) adds the partials in chunk order - a fixed order, so
// results do not depend on scheduling - applies norm*inv_scale and writes fp16.
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
constexpr uint32_t kHighAddr = kLutAddr + kLutBytes;
constexpr int kRedFloats = kWarps * 128;  // one 16x8 tile per warp
constexpr int kLowRows = 2;               // activation rows staged below the table

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
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
    asm(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Address of this lane's copy of table entry `byte_index` of `word`.
//   result byte 0 = lane constant byte 0 (copy offset), byte 1 = the code,
//   bytes 2,3 = lane constant bytes 2,3 (0x0001 -> the 0x10000 base).
template <int BYTE>
__device__ __forceinline__ uint32_t lut_addr(uint32_t word, uint32_t lane_const) {
    return __byte_perm(word, lane_const, 0x7604u | (static_cast<uint32_t>(BYTE) << 4));
}

// Shared address of staged activation row r: the first kLowRows rows sit below the
// table, the rest above it.
struct XRow {
    uint32_t low;
    __device__ __forceinline__ uint32_t addr(int r) const {
        return (r < kLowRows) ? low + static_cast<uint32_t>(r) * (kChunk * 4u)
                              : kHighAddr + static_cast<uint32_t>(r - kLowRows) * (kChunk * 4u);
    }
};

// Rotate one chunk of the activation into shared memory: for every batch row and every
// WHT block of the chunk, xrot = FWHT(sign o x) / sqrt(bs), rounded to TF32.
template <int E>
__device__ __forceinline__ void stage_x_blocks(const __half* __restrict__ x, int in, int batch, int col0, int cols,
                                               uint32_t seed, float inv_sqrt, const XRow& rows, int warp, int lane) {
    constexpr int BS = 32 * E;
    const int nb = cols / BS;
    for (int t = warp; t < nb * batch; t += kWarps) {
        const int b = t / nb, blk = t - b * nb;
        const __half* src = x + static_cast<size_t>(b) * in + col0 + blk * BS + lane * E;
        float v[E];
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = __half2float(src[j]) * sign_value(seed, static_cast<uint32_t>(lane * E + j));
        warp_fwht<E>(v, lane);
        const uint32_t dst = rows.addr(b) + static_cast<uint32_t>(blk * BS + lane * E) * 4u;
#pragma unroll
        for (int j = 0; j < E; ++j) sts_f32(dst + 4u * j, to_tf32(v[j] * inv_sqrt));
    }
}

struct GemvArgs {
    const uint8_t* codes;   // [out, in] joint bytes
    const float* norms;     // [out]
    const float* table;     // [n_planes, 256] fp32
    const __half* x;        // [batch, in]
    __half* y;              // [batch, out]
    float* partial;         // [n_slots, 8, out_pad] (only when n_slots > 1)
    unsigned int* counters; // [n_row_tiles]         (only when n_slots > 1)
    unsigned int* status;   // device error word (0 = ok)
    int out, in, batch, block;
    int n_row_tiles, n_chunks, n_slots, out_pad;  // n_slots = n_planes * n_chunks
    uint32_t seed_p, seed_r;
    float inv_sqrt, inv_scale;
};

__global__ void __launch_bounds__(kThreads, 1) tq8_gemv_kernel(const GemvArgs p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ unsigned int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;

    // ---- unit range of this CTA (chunk-major order) ----
    // unit = (slot, row tile), slot = plane * n_chunks + chunk; slot-major order
    const long n_units = static_cast<long>(p.n_row_tiles) * p.n_slots;
    const long u_begin = n_units * blockIdx.x / gridDim.x;
    const long u_end = n_units * (blockIdx.x + 1) / gridDim.x;
    if (u_begin >= u_end) return;

    // ---- shared-memory map ----
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t red_addr = (base + 127u) & ~127u;                   // 2 buffers of kRedFloats
    const uint32_t low_x = red_addr + 2u * kRedFloats * 4u;            // kLowRows activation rows
    if (low_x + kLowRows * kChunk * 4u > kLutAddr) {                   // layout assumption broken
        if (tid == 0) atomicExch(p.status, 1u);
        return;
    }
    const XRow xrows{low_x};

    // ---- first unit's code loads go out before anything else ----
    const int slice0 = warp * kSlice;  // column of this warp's slice inside the chunk
    // Per-thread byte offset of (row g, this thread's 16 columns) inside a unit; code
    // matrices stay below 4 GiB so 32-bit offsets are enough.
    const uint32_t thread_off = static_cast<uint32_t>(g) * static_cast<uint32_t>(p.in) + static_cast<uint32_t>(slice0 + 16 * q);
    const uint32_t row8_off = 8u * static_cast<uint32_t>(p.in);
    uint4 a[4][2];
    auto load_step = [&](int s, int kc, int rt) {
        const int c = kc * kChunk + slice0 + 16 * q + 64 * s;
        const int r0 = rt * 16 + g;
        const uint32_t off = static_cast<uint32_t>(rt) * 16u * static_cast<uint32_t>(p.in) + static_cast<uint32_t>(kc * kChunk + 64 * s) + thread_off;
        const bool ok = c < p.in;
        a[s][0] = (ok && r0 < p.out) ? ldg_stream(p.codes + off) : make_uint4(0, 0, 0, 0);
        a[s][1] = (ok && r0 + 8 < p.out) ? ldg_stream(p.codes + off + row8_off) : make_uint4(0, 0, 0, 0);
    };
    {
        const int slot0 = static_cast<int>(u_begin / p.n_row_tiles);
        const int rt0 = static_cast<int>(u_begin - static_cast<long>(slot0) * p.n_row_tiles);
#pragma unroll
        for (int s = 0; s < 4; ++s) load_step(s, slot0 % p.n_chunks, rt0);
    }

    const uint32_t lane_const = 0x00010000u | static_cast<uint32_t>(((warp & 1) * 32 + lane) * 4);

    uint32_t bfrag[4][16];
    int staged_slot = -1, staged_plane = -1;
    int buf = 0;

    for (long unit = u_begin; unit < u_end; ++unit) {
        const int slot = static_cast<int>(unit / p.n_row_tiles);
        const int rt = static_cast<int>(unit - static_cast<long>(slot) * p.n_row_tiles);
        const int plane = slot / p.n_chunks, kc = slot - plane * p.n_chunks;

        if (slot != staged_slot) {
            // (re)stage the rotated activation for this chunk and refill the B fragments
            __syncthreads();  // nobody still reads the previous rows / table
            if (plane != staged_plane) {
                // build the table: 256 entries x 64 copies, 4 copies per store
                const int copy4 = (tid & 15) * 4;
                for (int e = tid >> 4; e < 256; e += kThreads / 16) {
                    const float v = to_tf32(__ldg(p.table + plane * 256 + e));
                    sts_v4(kLutAddr + static_cast<uint32_t>(e) * 256u + static_cast<uint32_t>(copy4) * 4u, v, v, v, v);
                }
                staged_plane = plane;
            }
            const uint32_t seed = plane ? p.seed_r : p.seed_p;
            const int col0 = kc * kChunk;
            const int cols = min(kChunk, p.in - col0);
            switch (p.block) {
                case 32: stage_x_blocks<1>(p.x, p.in, p.batch, col0, cols, seed, p.inv_sqrt, xrows, warp, lane); break;
                case 64: stage_x_blocks<2>(p.x, p.in, p.batch, col0, cols, seed, p.inv_sqrt, xrows, warp, lane); break;
                case 128: stage_x_blocks<4>(p.x, p.in, p.batch, col0, cols, seed, p.inv_sqrt, xrows, warp, lane); break;
                case 256: stage_x_blocks<8>(p.x, p.in, p.batch, col0, cols, seed, p.inv_sqrt, xrows, warp, lane); break;
                case 512: stage_x_blocks<16>(p.x, p.in, p.batch, col0, cols, seed, p.inv_sqrt, xrows, warp, lane); break;
                default: stage_x_blocks<32>(p.x, p.in, p.batch, col0, cols, seed, p.inv_sqrt, xrows, warp, lane); break;
            }
            __syncthreads();
            // B fragment of MMA (s, m): k = q -> column 64 s + 16 q + 2 m, k = q+4 -> the next column; n = g.
            const bool have_row = g < p.batch;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const int c = slice0 + 64 * s + 16 * q;
                const bool ok = have_row && (col0 + c) < p.in;
#pragma unroll
                for (int k = 0; k < 16; ++k) bfrag[s][k] = ok ? lds_u32(xrows.addr(g) + static_cast<uint32_t>(c + k) * 4u) : 0u;
            }
            staged_slot = slot;
        }

        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const bool has_next = (unit + 1) < u_end;
        int nkc = kc, nrt = rt + 1;
        if (nrt == p.n_row_tiles) { nrt = 0; nkc = (kc + 1 == p.n_chunks) ? 0 : kc + 1; }
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint32_t lo[4] = {a[s][0].x, a[s][0].y, a[s][0].z, a[s][0].w};
            const uint32_t hi[4] = {a[s][1].x, a[s][1].y, a[s][1].z, a[s][1].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                // bytes 0,1 of the word feed one MMA, bytes 2,3 the next
                {
                    const float a0 = lds_f32(lut_addr<0>(lo[w], lane_const));
                    const float a2 = lds_f32(lut_addr<1>(lo[w], lane_const));
                    const float a1 = lds_f32(lut_addr<0>(hi[w], lane_const));
                    const float a3 = lds_f32(lut_addr<1>(hi[w], lane_const));
                    mma_tf32(acc, __float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3),
                             bfrag[s][4 * w + 0], bfrag[s][4 * w + 1]);
                }
                {
                    const float a0 = lds_f32(lut_addr<2>(lo[w], lane_const));
                    const float a2 = lds_f32(lut_addr<3>(lo[w], lane_const));
                    const float a1 = lds_f32(lut_addr<2>(hi[w], lane_const));
                    const float a3 = lds_f32(lut_addr<3>(hi[w], lane_const));
                    mma_tf32(acc, __float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3),
                             bfrag[s][4 * w + 2], bfrag[s][4 * w + 3]);
                }
            }
            if (has_next) load_step(s, nkc, nrt);  // registers of step s are dead now: refill from the next unit
        }

        // ---- cross-warp sum of the 16 per-warp 16x8 tiles ----
        const uint32_t red = red_addr + static_cast<uint32_t>(buf * kRedFloats + warp * 128) * 4u;
        sts_f32(red + static_cast<uint32_t>(g * 8 + 2 * q) * 4u, acc[0]);
        sts_f32(red + static_cast<uint32_t>(g * 8 + 2 * q + 1) * 4u, acc[1]);
        sts_f32(red + static_cast<uint32_t>((g + 8) * 8 + 2 * q) * 4u, acc[2]);
        sts_f32(red + static_cast<uint32_t>((g + 8) * 8 + 2 * q + 1) * 4u, acc[3]);
        __syncthreads();
        const int row_in_tile = tid >> 3, n = tid & 7;
        const int row = rt * 16 + row_in_tile;
        float sum = 0.f;
        if (tid < 128) {
            const uint32_t src = red_addr + static_cast<uint32_t>(buf * kRedFloats + tid) * 4u;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) sum += lds_f32(src + static_cast<uint32_t>(w * 128) * 4u);
        }
        if (p.n_slots == 1) {
            if (tid < 128 && row < p.out && n < p.batch)
                p.y[static_cast<size_t>(n) * p.out + row] = __float2half_rn(sum * (p.norms[row] * p.inv_scale));
        } else {
            if (tid < 128 && row < p.out) p.partial[(static_cast<size_t>(slot) * 8 + n) * p.out_pad + row] = sum;
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
                if (tid < 128 && row < p.out && n < p.batch) {
                    float total = 0.f;
                    for (int c = 0; c < p.n_slots; ++c)
                        total += __ldcg(p.partial + (static_cast<size_t>(c) * 8 + n) * p.out_pad + row);
                    p.y[static_cast<size_t>(n) * p.out + row] = __float2half_rn(total * (p.norms[row] * p.inv_scale));
                }
            }
        }
        buf ^= 1;
    }
}

}  // namespace

size_t gemv_scratch_bytes(int out, int in, int n_planes) {
    const int n_chunks = ((in + kChunk - 1) / kChunk) * n_planes;
    if (n_chunks <= 1) return 0;
    const int n_row_tiles = (out + 15) / 16;
    const size_t out_pad = static_cast<size_t>(n_row_tiles) * 16;
    return static_cast<size_t>(n_chunks) * 8 * out_pad * sizeof(float) + static_cast<size_t>(n_row_tiles) * sizeof(unsigned int);
}

void launch_tq8_gemv(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                     int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                     void* scratch, unsigned int* status, int sm_count, cudaStream_t stream) {
    TQ_REQUIRE(n_planes == 1 || n_planes == 2, "tq8_gemv: one or two rotation planes");
    TQ_REQUIRE(batch >= 1 && batch <= 8, "tq8_gemv handles 1..8 activation rows per launch");
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "WHT block size must be a power of two in [32, 1024]");
    TQ_REQUIRE(in % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    if (out == 0) return;
    GemvArgs a{};
    a.codes = codes; a.norms = norms; a.table = table; a.x = x; a.y = y; a.status = status;
    a.out = out; a.in = in; a.batch = batch; a.block = static_cast<int>(block);
    a.n_row_tiles = (out + 15) / 16;
    a.n_chunks = (in + kChunk - 1) / kChunk;
    a.n_slots = a.n_chunks * n_planes;
    a.out_pad = a.n_row_tiles * 16;
    a.seed_p = seed_p;
    a.seed_r = seed_r;
    a.inv_sqrt = 1.0f / std::sqrt(static_cast<float>(block));
    a.inv_scale = 1.0f / std::sqrt(static_cast<float>(in));
    if (a.n_slots > 1) {
        TQ_REQUIRE(scratch != nullptr, "tq8_gemv needs scratch memory when in_features > 4096 or rotation is dual");
        a.partial = static_cast<float*>(scratch);
        a.counters = reinterpret_cast<unsigned int*>(a.partial + static_cast<size_t>(a.n_slots) * 8 * a.out_pad);
    }
    const int extra_rows = batch > kLowRows ? batch - kLowRows : 0;
    const size_t smem = static_cast<size_t>(kHighAddr) + static_cast<size_t>(extra_rows) * kChunk * 4;
    // the opt-in shared-memory size is a per-device function attribute
    static size_t configured[64] = {0};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && smem > configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(tq8_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured[dev] = smem;
    }
    const long n_units = static_cast<long>(a.n_row_tiles) * a.n_slots;
    int grid = static_cast<int>(n_units < sm_count ? n_units : sm_count);
    tq8_gemv_kernel<<<grid, kThreads, smem, stream>>>(a);
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
