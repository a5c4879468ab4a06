// Fused TQ8 dequantise + GEMV / skinny GEMM for decode (1..8 activation rows per pass).
//
// Replaces the reference's tq_dequant_mm Metal kernel and its host wrapper
// (metal/turboquant_dequant_mm.metal:152-313, src/dequantizer.cpp:606-721):
//   y[b, r] = fp16( norm[r] * sum_j W~[r, j] * fp16(x[b, j]) ),  fp32 accumulate.
//
// Algebra.  A dequantised row block is  norm * (inv_sqrt*sign) o H(table[codes]*inv_scale)
// and H is symmetric, so   <s o H(c), x> = <c, H(s o x)>.   The activation is therefore
// rotated ONCE per call (forward WHT of every block of x) and the weight side collapses
// to a table lookup per code:
//   y[b, r] = norm[r] * inv_scale * sum_j table[code[r, j]] * xrot[b, j].
//
// Where the rotation happens.  A warp multiplies a fixed 256-column slice, so for WHT
// blocks of up to 256 columns it rotates its own slice of x inside the GEMV kernel (16-byte
// loads, butterflies in registers and lane exchanges, a 1 KB strip of shared memory to reach
// the fragment layout): one kernel per call.  Larger blocks span several warps; for those
// rotate_x_kernel writes xrot (fp32, TF32-rounded, [b, in]) to scratch first, chained with
// programmatic dependent launch.  Either way the GEMV is launched with the programmatic
// attribute: its set-up (table, first code loads) overlaps the tail of whatever precedes it.
//   tq8_gemv_kernel   persistent, one CTA per SM, 16 warps:
//     HBM --(128-bit loads, 16 codes each, two 64-column steps ahead)--> registers
//     --(byte -> address, 1 PRMT)-->
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
// Work split.  The 16 warps of a CTA are split into groups of wpt warps (a power of two); a group multiplies one
// 16-row tile against a chunk of wpt * 256 columns, so a unit is 16 / wpt row tiles of one chunk (a "slot").  Up to
// 4096 columns there is one chunk and wpt is the fewest warps that cover the row; above, wpt = 16 unless the last
// chunk would leave more than 15 % of the slices empty (5120 columns: five chunks of 1024 with wpt = 4).  Units are
// ordered slot-major and dealt to CTAs in contiguous ranges, so a CTA reloads its B fragments only when its slot
// changes.  A warp's partial tiles are added across the group through a ring in shared memory, one pass of
// log2(wpt) lane exchanges per unit.  With more than one slot (in_features > 4096, or dual rotation) the sums go
// to scratch as fp32; every warp owns the same rows in every slot and counts its arrivals per (row unit, warp) -
// once per 8 units, since the fence before the count stalls the warp - and the warp that completes a row unit adds
// the slots' partial sums in slot order (a fixed order, so results do not depend on scheduling), applies
// norm*inv_scale and writes fp16.
// Dual-rotation weights (separate sign seeds for the primary and residual planes,
// src/dequantizer.cpp:214-246) run as two "planes": plane 0 looks up the primary
// centroid of each joint byte against x rotated with the primary seed, plane 1 the
// residual centroid against x rotated with the residual seed; planes are just further
// partial-sum slots.
#include <cmath>
#include <cstdint>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kSlice = 256;               // columns per warp
constexpr int kChunk = kWarps * kSlice;   // widest chunk: columns one unit covers with all 16 warps on one row tile
constexpr uint32_t kLutAddr = 0x10000u;   // shared-window address of the table
constexpr uint32_t kLutBytes = 0x10000u;  // 256 entries * 256 B
constexpr int kRedBytes = 32768;           // partial-sum ring: ring * 16 warps * (16 rows * bp + 4) floats
constexpr int kMaxRing = 16;
constexpr int kFlushUnits = 8;             // units a warp finishes between two arrival counts (several slots only)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

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
    const uint8_t* codes;   // joint bytes in 16 x 64 tiles (code_offset)
    const float* norms;     // [out]
    const float* table;     // [n_planes, 256] fp32
    const float* xrot;      // [n_planes, batch, in] fp32 (TF32-rounded); used when x == nullptr
    const __half* x;        // [batch, in] fp16: rotate inside the kernel (WHT block <= 256), else nullptr
    __half* y;              // [batch, y_stride]: row r of activation row n at y[n * y_stride + r]
    float* partial;         // [n_slots, 8, out_pad] (only when n_slots > 1)
    unsigned int* counters; // [n_row_units][16 warps] (only when n_slots > 1)
    unsigned int* status;   // device error word (0 = ok)
    int out, in, batch;
    int n_row_units, n_chunks, n_slots, out_pad;  // n_slots = n_planes * n_chunks
    int wpt, tpu;           // warps per row tile, row tiles per unit (wpt * tpu = 16)
    float inv_scale;
    uint32_t seed_p, seed_r;   // sign seeds of plane 0 / plane 1 (in-kernel rotation)
    int block;                 // WHT block size                  (in-kernel rotation)
    float inv_sqrt_block;
};

// Arguments of scattering calls, a kernel parameter of their own: with these fields inside
// GemvArgs the plain kernel (same code otherwise) needed spills within its 128 registers.
struct ScatterArgs {
    __half* y_peer[7];      // further destinations written with the same values (other GPUs' buffers)
    int n_peer;
    long y_stride;
    // Completion signal of a scattering call (n_signal = 0: none): when the whole grid has
    // stored its results, word `signal_slot` of every destination's flag array is set to
    // `signal_value`.  done_counter is a zero-initialised device word owned by the layer.
    unsigned int* signal[8];
    int n_signal, signal_slot;
    unsigned int signal_value;
    unsigned int* done_counter;
    // Fused all-gather (bulk != 0): results are stored locally only; the CTA that completes the grid
    // copies the whole block to the peers with 16-byte stores and then raises the flags with the value
    // ++(*epoch) (signal_value is not used).  With n_wait > 0 every CTA first waits - bounded - until
    // wait_flags[0..n_wait) have reached *wait_epoch + 1 before it reads the activation (the previous
    // exchange has arrived); the completing CTA then advances *wait_epoch.
    int bulk;
    unsigned int* epoch;
    const unsigned int* wait_flags;
    int n_wait;
    unsigned int* wait_epoch;
    // Flag-in-data exchange (ll != 0, with bulk): instead of data, a fence and a flag, the completing CTA
    // writes 16-byte packets {2 halves, epoch, 2 halves, epoch} - each 8-byte half is written atomically
    // by the one store, so a reader that sees the epoch in both halves holds valid data and nothing has to
    // be fenced.  Every rank's packet buffer is [2 halves of the double buffer][ll_world source ranks]
    // [packets] (ll_base[r] = rank r's buffer, ll_base[ll_rank] this rank's own); the half is the parity of
    // the epoch.  With n_wait > 0 every CTA first polls - bounded - the packets all other ranks wrote for
    // epoch *wait_epoch + 1.
    int ll, ll_rank, ll_world;
    uint4* ll_base[8];
};

// One output element goes to the caller's buffer and, when the call scatters, to the same
// position of up to 7 further buffers (peer GPUs' memory mapped into this process: plain stores
// over NVLink, no multicast).
// SCATTER is a compile-time variant: the plain kernel keeps the register budget it had before the
// scattering code existed (with it in the same instantiation the kernel spilled).
template <bool SCATTER>
__device__ __forceinline__ void store_y(const GemvArgs& p, const ScatterArgs& sc, int n, int row, __half h) {
    if constexpr (SCATTER) {
        const size_t o = static_cast<size_t>(n) * sc.y_stride + row;
        p.y[o] = h;
        if (!sc.bulk) {
#pragma unroll
            for (int d = 0; d < 7; ++d)
                if (d < sc.n_peer) sc.y_peer[d][o] = h;
        }
    } else {
        p.y[static_cast<size_t>(n) * p.out + row] = h;
    }
}

// Shared memory holds only the table and the partial-sum ring: the dynamic allocation ends at
// the end of the table (128 KB).  Asking for much more than that shrinks the L1 side of the
// SM's memory and with it the number of global loads the SM keeps in flight (measured: a
// streaming read drops from 5.8 to 3.4 TB/s when a CTA holds 216 KB), so the codes are never
// staged through shared memory: they go from HBM straight into registers.
constexpr size_t kGemvSmem = kLutAddr + kLutBytes;  // dynamic bytes requested (window end)
constexpr int kConsumerThreads = kThreads;
constexpr int kCtaThreads = kThreads;
constexpr unsigned long long kWaitLimitNs = 200ull * 1000 * 1000;  // bounded waits: give up after 0.2 s and flag it

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// Returns false if the phase did not complete within the spin limit.
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if (spin == 64) t0 = global_timer_ns();
        if (spin > 64 && (spin & 63) == 0 && global_timer_ns() - t0 > kWaitLimitNs) return false;
    }
}
// Streaming 16-byte load that leaves `v` untouched when `pred` is false.  Codes outside the
// matrix are never zero-filled: whatever the registers hold indexes a valid table entry, and it
// meets either a zero activation (columns past in_features) or a row that is never written.
__device__ __forceinline__ void ldg_stream_if(uint4& v, const uint8_t* p, bool pred) {
    asm volatile(
        "{ .reg .pred p; setp.ne.u32 p, %5, 0;\n"
        "  @p ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4]; }"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "l"(p), "r"(static_cast<uint32_t>(pred)));
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Table lookup.  Not volatile: the table is read-only while lookups run, so the compiler may
// batch and reorder these loads freely (the address depends on codes loaded after the
// barrier that publishes the table, which keeps them below it).
__device__ __forceinline__ uint32_t lut_load(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- flag-in-data exchange (see ScatterArgs) ----
__device__ __forceinline__ void ll_wait_packets(const unsigned int* wait_epoch, const uint4* mine, int rank, int world, long packets,
                                                unsigned int* status) {
    const unsigned int want = *reinterpret_cast<const volatile unsigned int*>(wait_epoch) + 1u;
    const uint4* const half = mine + static_cast<size_t>(want & 1u) * world * packets;
    const unsigned long long t0 = global_timer_ns();
    for (int src = 0; src < world; ++src) {
        if (src == rank) continue;
        const uint4* region = half + static_cast<size_t>(src) * packets;
        for (long i = threadIdx.x; i < packets; i += kCtaThreads) {
            for (unsigned int spin = 0;; ++spin) {
                uint4 pk;
                asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(pk.x), "=r"(pk.y), "=r"(pk.z), "=r"(pk.w)
                             : "l"(region + i)
                             : "memory");
                if (static_cast<int>(pk.y - want) >= 0 && static_cast<int>(pk.w - want) >= 0) break;
                if ((spin & 255u) == 255u && global_timer_ns() - t0 > 5ull * kWaitLimitNs) {   // 1 s: a peer is gone
                    raise_status(status, 10u);
                    return;
                }
            }
        }
    }
}
// Packets c0 .. c1 - 1 (groups of four rows) of every activation row, to every other rank: no fence, no flag -
// the epoch travels with the data.
__device__ __forceinline__ void ll_send_packets(const ScatterArgs& sc, const __half* y, int per_row, int batch, int c0, int c1) {
    const unsigned int value = *reinterpret_cast<const volatile unsigned int*>(sc.epoch) + 1u;
    const long packets = static_cast<long>(batch) * per_row;
    const size_t region = (static_cast<size_t>(value & 1u) * sc.ll_world + sc.ll_rank) * packets;
    const int span = c1 - c0;
    for (long i = threadIdx.x; i < static_cast<long>(batch) * span; i += kCtaThreads) {
        const int n = static_cast<int>(i / span), c = c0 + static_cast<int>(i - static_cast<long>(n) * span);
        const uint2 v = __ldcg(reinterpret_cast<const uint2*>(y + static_cast<size_t>(n) * sc.y_stride + static_cast<size_t>(c) * 4));
        const size_t at = region + static_cast<size_t>(n) * per_row + c;
#pragma unroll
        for (int d = 0; d < 8; ++d)
            if (d < sc.ll_world && d != sc.ll_rank)
                asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(sc.ll_base[d] + at), "r"(v.x), "r"(value), "r"(v.y)
                             : "memory");
    }
}

// BP = activation rows padded to 1, 2, 4 or 8 (compile time, so that the partial-sum ring
// geometry and the reduction need no runtime arithmetic).
// MULTI = more than one slot (row units finished through partial sums in scratch); compile time, so that the
// single-slot kernels carry none of that path's state in their 128 registers.
template <int BP, bool SCATTER, bool LL, bool MULTI>
__device__ __forceinline__ void gemv_body(const GemvArgs& p, const ScatterArgs& sargs, const int bid, const int nblk) {
    // columns per chunk, derived here: one more field in GemvArgs made ptxas spill within the 128 registers
    const int chunk_cols = p.wpt * kSlice;
    // A warp's partial tile is [16 rows][BP] floats plus 4 floats of padding: the 16 tiles a
    // reduction reads side by side then start 4 banks apart instead of in the same bank.
    constexpr int kTileFloats = 16 * BP + 4;
    constexpr int kRing = (kRedBytes / (kWarps * kTileFloats * 4)) > kMaxRing ? kMaxRing : (kRedBytes / (kWarps * kTileFloats * 4));
    static_assert(kRing >= 2, "the ring needs a slot to write while another is summed");
    constexpr int kLag = kRing / 2;                       // how many units behind the sums run
    constexpr uint32_t kSlotBytes = kWarps * kTileFloats * 4;  // one ring slot: [warp][16 rows][BP] floats (+ padding)
    constexpr int kPer = BP >= 2 ? BP / 2 : 1;            // floats a lane adds in the reduction

    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ unsigned int s_abort;
    // [0..kRing) "tiles of ring slot written" (one arrival per warp), [kMaxRing..) "slot read"
    __shared__ __align__(8) unsigned long long s_bars[2 * kMaxRing];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // ---- unit range of this CTA: unit = (slot, row unit), slot = plane * n_chunks + chunk ----
    // (the first `rem` CTAs take one unit more; one 32-bit division - the prologue runs once per launch on
    // instructions that are not cached yet, and cannot overlap the preceding kernel, whose CTA fills this SM)
    const int n_units = p.n_row_units * p.n_slots;
    const int u_quot = n_units / nblk, u_rem = n_units - u_quot * nblk;   // bid of nblk CTAs work on this matrix
    const int u_begin = u_quot * bid + (bid < u_rem ? bid : u_rem);
    const int n_local = u_quot + (bid < u_rem ? 1 : 0);
    if (n_local <= 0) return;

    // ---- shared-memory map: [partial-sum ring | rotation strips | unused | table at 0x10000] ----
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t red_addr = (base + 127u) & ~127u;
    const uint32_t strip_addr = red_addr + kRedBytes + static_cast<uint32_t>(warp) * (kSlice * 4u);
    if (red_addr + kRedBytes + kWarps * kSlice * 4u > kLutAddr) {  // layout assumption broken: refuse to run
        if (tid == 0) raise_status(p.status, 1u);
        return;
    }
    const uint32_t bar_written = smem_u32(&s_bars[0]), bar_read = smem_u32(&s_bars[kMaxRing]);
    if (tid < kRing) {   // one pair of barriers per thread: a single thread took 0.45 us for the 32 of them
        mbar_init(bar_written + 8u * tid, kWarps);
        mbar_init(bar_read + 8u * tid, kWarps);
        if (tid == 0) s_abort = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }

    const int g = lane >> 2, q = lane & 3;
    const int wpt_shift = 31 - __clz(p.wpt);                    // wpt is a power of two
    const int tile_in_unit = warp >> wpt_shift;                 // which of the unit's row tiles this warp works on
    const int slice0 = (warp & (p.wpt - 1)) * kSlice;           // column of this warp's slice inside the chunk
    const uint32_t lane_const = 0x00010000u | static_cast<uint32_t>(lane * 4);
    // Codes are stored in 16-row x 64-column tiles of 1 KB (code_offset): a step of a warp is one
    // tile, of which lane (g, q) reads bytes g*64 + 16q (row g) and 512 + g*64 + 16q (row g + 8) -
    // 512 contiguous bytes per warp load.  Consecutive steps are consecutive tiles.
    const size_t tiles_per_row = code_tiles_per_row(p.in);
    const size_t unit_stride = static_cast<size_t>(p.tpu) * tiles_per_row * kCodeTileBytes;  // bytes between consecutive row units

    // ---- position of a unit, kept incrementally (no divisions in the loop) ----
    struct Pos {
        int slot, ru;          // slot and row unit
        const uint8_t* ptr;    // this thread's first 16 codes of the unit (row g)
        uint32_t ok;           // bit s: columns of step s exist; bits 4, 5: the row tile exists (padded rows are stored)
    };
    auto make_pos = [&](int unit) {
        Pos u;
        if constexpr (MULTI) {
            u.slot = unit / p.n_row_units;
            u.ru = unit - u.slot * p.n_row_units;
        } else {
            u.slot = 0;
            u.ru = unit;
        }
        const int c = (MULTI ? (u.slot % p.n_chunks) * chunk_cols : 0) + slice0;  // first column of this warp's slice
        const int tile = u.ru * p.tpu + tile_in_unit;
        u.ptr = p.codes + (static_cast<size_t>(tile) * tiles_per_row + static_cast<size_t>(c >> 6)) * kCodeTileBytes + g * 64 + 16 * q;
        u.ok = 0;
#pragma unroll
        for (int s = 0; s < 4; ++s) u.ok |= (c + 64 * s < p.in) ? (1u << s) : 0u;
        u.ok |= (tile * 16 < p.out) ? 48u : 0u;
        return u;
    };
    auto next_pos = [&](const Pos& u) {
        Pos n = u;
        if (!MULTI || u.ru + 1 < p.n_row_units) {   // same slot, next row unit: only the rows move
            n.ru = u.ru + 1;
            n.ptr = u.ptr + unit_stride;
            n.ok = (u.ok & 15u) | (((n.ru * p.tpu + tile_in_unit) * 16 < p.out) ? 48u : 0u);
            return n;
        }
        return make_pos((u.slot + 1) * p.n_row_units);
    };
    // Codes never depend on the kernel before this one, so the first loads go out before the
    // dependency wait below.  Pieces outside the matrix are simply not loaded.
    auto load_step = [&](const Pos& u, int s, bool live, uint4& lo, uint4& hi) {
        const bool c_ok = live && ((u.ok >> s) & 1u);
        ldg_stream_if(lo, u.ptr + kCodeTileBytes * s, c_ok && (u.ok & 16u));
        ldg_stream_if(hi, u.ptr + kCodeTileBytes * s + 512, c_ok && (u.ok & 32u));
    };
    Pos cur = make_pos(u_begin);
    Pos nxt = (n_local > 1) ? next_pos(cur) : cur;
    // Two register buffers (even / odd step): two steps, 32 KB per SM, in flight.  Four buffers
    // were measured and bought nothing: the kernel is bound by L1 data-pipe wavefronts (table
    // lookups plus the code loads), not by the depth of the load queue.
    uint4 blo[2], bhi[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        blo[s] = make_uint4(0, 0, 0, 0);
        bhi[s] = make_uint4(0, 0, 0, 0);
        load_step(cur, s, true, blo[s], bhi[s]);
    }

    auto build_table = [&](int plane) {
        // 256 entries x 32 copies; a thread writes 4 consecutive copies per store
        const int copy4 = (tid & 7) * 4;
        for (int e = tid >> 3; e < 256; e += kConsumerThreads / 8) {
            const float v = to_tf32(__ldg(p.table + plane * 256 + e));
            sts_v4(kLutAddr + static_cast<uint32_t>(e) * 256u + static_cast<uint32_t>(copy4) * 4u, v, v, v, v);
        }
    };
    // Prologue order: table entries are fetched into registers (they do not depend on the
    // preceding kernel), then comes the dependency wait, then this warp's activation slice of
    // the first unit is requested, and only then are the table entries written to shared
    // memory - so the activation's latency hides behind the table build.
    int staged_plane = MULTI ? cur.slot / p.n_chunks : 0;
    float tab_first[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) tab_first[k] = __ldg(p.table + staged_plane * 256 + (tid >> 3) + 64 * k);

    // Everything below reads or writes data the preceding kernels produce or still use.
    grid_dependency_sync();
    if constexpr (SCATTER) {
        if (LL && sargs.n_wait > 0) {
            // the activation comes out of a flag-in-data exchange: every packet of every other rank must carry the epoch
            if constexpr (LL) {
                ll_wait_packets(sargs.wait_epoch, sargs.ll_base[sargs.ll_rank], sargs.ll_rank, sargs.ll_world,
                                static_cast<long>(p.batch) * (p.out / 4), p.status);
            }
            __syncthreads();
        } else if (sargs.n_wait > 0) {
            // the activation comes out of an exchange: wait until every rank's part has arrived
            if (tid < sargs.n_wait) {
                const unsigned int want = *reinterpret_cast<volatile unsigned int*>(sargs.wait_epoch) + 1u;
                const unsigned long long t0 = global_timer_ns();
                for (unsigned int spin = 0;; ++spin) {
                    unsigned int v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(sargs.wait_flags + tid) : "memory");
                    if (static_cast<int>(v - want) >= 0) break;
                    if ((spin & 255u) == 255u && global_timer_ns() - t0 > 5ull * kWaitLimitNs) {   // 1 s: a peer is gone
                        raise_status(p.status, 10u);
                        break;
                    }
                }
            }
            __syncthreads();
        }
    }
    uint4 x_first = make_uint4(0, 0, 0, 0);
    if (p.x != nullptr) {
        const int cl0 = (MULTI ? (cur.slot - staged_plane * p.n_chunks) * chunk_cols : 0) + slice0 + 8 * lane;
        if (cl0 < p.in) x_first = __ldg(reinterpret_cast<const uint4*>(p.x + cl0));
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float v = to_tf32(tab_first[k]);
        sts_v4(kLutAddr + static_cast<uint32_t>((tid >> 3) + 64 * k) * 256u + static_cast<uint32_t>((tid & 7) * 4) * 4u, v, v, v, v);
    }
    __syncthreads();  // table and barriers visible

    // ---- sum of one unit's per-warp partial tiles ----
    // Ring slot layout: [warp][16 rows][BP] floats (+ 4 floats of padding per warp).  Warp w owns the (tile, row) pairs
    // w*tpu .. w*tpu+tpu-1 of the unit.  The 16 lanes of a half warp cover those tpu pairs times the wpt warps that
    // worked on the pair's row tile (tpu * wpt = 16): lane l reads what warp (l & (wpt - 1)) of the group wrote for pair
    // (l & 15) / wpt, activation columns (l >> 4) * kPer .., and a fixed tree of log2(wpt) lane exchanges adds them
    // (fixed order: results do not depend on timing).  One pass per unit whatever the split.
    const int pw = lane & (p.wpt - 1), hv = lane >> 4;
    const int n0 = BP >= 2 ? hv * kPer : 0;
    const int red_pi = warp * p.tpu + ((lane & 15) >> wpt_shift);       // this lane's pair: row tile red_pi >> 4 of the unit, row red_pi & 15
    const int red_row = (red_pi >> 4) * 16 + (red_pi & 15);      // its row inside the row unit
    const uint32_t red_src = red_addr + static_cast<uint32_t>(((red_pi >> 4) * p.wpt + pw) * kTileFloats + (red_pi & 15) * BP + n0) * 4u;
    const bool red_active = BP >= 2 || hv == 0;
    const bool red_writer = pw == 0 && red_active;
    // Counts this warp's last `pend` units (row units ru_last - pend + 1 .. ru_last of one slot) in and finishes the
    // row units it completes.
    int pend = 0;
    auto flush_pending = [&](int ru_last) {
        __threadfence();
        __syncwarp();
        const int ru0 = ru_last - pend + 1;
        unsigned int prev = 0xffffffffu;
        if (lane < pend) prev = atomicAdd(&p.counters[(ru0 + lane) * kWarps + warp], 1u);
        unsigned int done = __ballot_sync(0xffffffffu, prev == static_cast<unsigned int>(p.n_slots) - 1u);
        pend = 0;
        if (done == 0u) return;
        __threadfence();
        if (prev == static_cast<unsigned int>(p.n_slots) - 1u) p.counters[(ru0 + lane) * kWarps + warp] = 0u;  // ready for the next launch
        // the outputs of all completed row units side by side over the lanes; up to 8 slots' partial sums are requested
        // at once (one round trip to L2) and added in slot order
        const int per_unit = p.tpu * BP;
        const int n_done = __popc(done) * per_unit;
        for (int idx = lane; idx < n_done; idx += 32) {
            const int k = idx / per_unit, e = idx - k * per_unit;
            const int ru = ru0 + static_cast<int>(__fns(done, 0u, k + 1));
            const int n = e % BP, pi = warp * p.tpu + e / BP;
            const int row = (ru * p.tpu + (pi >> 4)) * 16 + (pi & 15);
            if (row < p.out && n < p.batch) {
                const float sc = __ldg(p.norms + row) * p.inv_scale;
                const float* src = p.partial + static_cast<size_t>(n) * p.out_pad + row;
                float total = 0.f;
                for (int c0 = 0; c0 < p.n_slots; c0 += 8) {
                    float t[8];
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        t[c] = (c0 + c < p.n_slots) ? __ldcg(src + static_cast<size_t>(c0 + c) * 8 * p.out_pad) : 0.f;
#pragma unroll
                    for (int c = 0; c < 8; ++c) total += t[c];
                }
                store_y<SCATTER>(p, sargs, n, row, __float2half_rn(total * sc));
            }
        }
    };
    auto reduce_unit = [&](int slot, int ru, int rs, uint32_t parity) {
        if (!mbar_wait(bar_written + 8u * rs, parity)) {
            raise_status(p.status, 5u);
            atomicExch(&s_abort, 1u);
        }
        {
            const int row = ru * p.tpu * 16 + red_row;
            const bool wr = red_writer && row < p.out;
            float sc = 0.f;
            // the norm is fetched first so that its latency hides behind the exchanges
            if constexpr (!MULTI) sc = wr ? __ldg(p.norms + row) * p.inv_scale : 0.f;
            float v[kPer];
#pragma unroll
            for (int k = 0; k < kPer; ++k) v[k] = 0.f;
            if (red_active) {
                const uint32_t src = red_src + static_cast<uint32_t>(rs) * kSlotBytes;
                if constexpr (kPer == 4) asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(src));
                else if constexpr (kPer == 2) asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v[0]), "=f"(v[1]) : "r"(src));
                else asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[0]) : "r"(src));
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) {
                if (o < p.wpt) {
#pragma unroll
                    for (int k = 0; k < kPer; ++k) v[k] += __shfl_xor_sync(0xffffffffu, v[k], o);
                }
            }
            if (wr) {
#pragma unroll
                for (int k = 0; k < kPer; ++k) {
                    const int n = n0 + k;
                    if constexpr (!MULTI) {
                        if (n < p.batch) store_y<SCATTER>(p, sargs, n, row, __float2half_rn(v[k] * sc));
                    } else {
                        p.partial[(static_cast<size_t>(slot) * 8 + n) * p.out_pad + row] = v[k];
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_read + 8u * rs);
        if constexpr (MULTI) {
            // Row units spread over several slots.  A warp owns the same rows of a row unit in every slot, so the
            // arrival count is kept per (row unit, warp): the warp that brings it to n_slots adds the slots' partial
            // sums of its rows in slot order and writes y.  The fence between the partial stores and the count makes
            // the warp wait for its memory traffic, code loads in flight included, so it is paid once per
            // kFlushUnits units (consecutive row units of one slot), not per unit.
            ++pend;
            if (pend == kFlushUnits || ru + 1 == p.n_row_units) flush_pending(ru);
        }
    };
    uint32_t bfrag[4][16];
    int staged_slot = -1;
    // ring bookkeeping: slot / parity for the unit being written and the unit being summed
    int ws = 0;             // write slot = i % kRing
    uint32_t wpar = 0;      // parity of the "read" phase the writer waits for = ((i / kRing) - 1) & 1
    int rs = 0;             // slot of the unit being summed = (i - kLag) % kRing
    uint32_t rpar = 0;      // parity of its "written" phase = ((i - kLag) / kRing) & 1
    Pos red = cur;          // position of the unit being summed

    // Makes `slot` the current one: switches the table when the plane changes and rebuilds this
    // warp's B fragments.  x0 is this lane's first-row activation when the caller has already
    // requested it (have_x0).
    auto stage_slot = [&](int slot, const uint4& x0, bool have_x0) {
        const int plane = MULTI ? slot / p.n_chunks : 0;
            if (plane != staged_plane) {
                named_barrier_sync(1, kConsumerThreads);  // nobody still reads the previous table
                build_table(plane);
                named_barrier_sync(1, kConsumerThreads);
                staged_plane = plane;
            }
            // B fragment of MMA (s, m): k = q -> column 64 s + 16 q + 2 m, k = q+4 -> the next column; n = g.
            const int colw = (MULTI ? (slot - plane * p.n_chunks) * chunk_cols : 0) + slice0;  // first column of this warp's slice
            const int col0 = colw + 16 * q;
            if (BP == 1 && p.x != nullptr) {
                // One activation row (the launcher rotates in here only then): rotate this warp's 256 columns of it.
                // Lane l holds columns 8l..8l+7 of the slice, stages below 8 stay in the lane, the rest are lane
                // exchanges (same add tree as rotate_x_kernel).  A 1 KB strip of shared memory per warp turns the
                // result into the fragment layout.  Every lane loads the row's fragment, so B columns 1..7 repeat
                // column 0 and their results are never read: nothing to clear.
                const uint32_t seed = plane ? p.seed_r : p.seed_p;
                const int cl = colw + 8 * lane;
                uint4 xc = x0;
                if (!have_x0) {
                    xc = make_uint4(0, 0, 0, 0);
                    if (cl < p.in) xc = __ldg(reinterpret_cast<const uint4*>(p.x + cl));
                }
                const uint32_t xw[4] = {xc.x, xc.y, xc.z, xc.w};
                float v[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 h2 = *reinterpret_cast<const __half2*>(&xw[j]);
                    const float lo = __low2float(h2), hi = __high2float(h2);
                    v[2 * j] = sign_is_positive(seed, static_cast<uint32_t>((8 * lane + 2 * j) & (p.block - 1))) ? lo : -lo;
                    v[2 * j + 1] = sign_is_positive(seed, static_cast<uint32_t>((8 * lane + 2 * j + 1) & (p.block - 1))) ? hi : -hi;
                }
#pragma unroll
                for (int h = 1; h < 8; h <<= 1)
#pragma unroll
                    for (int i = 0; i < 8; i += 2 * h)
#pragma unroll
                        for (int j = i; j < i + h; ++j) {
                            const float a = v[j], b = v[j + h];
                            v[j] = __fadd_rn(a, b);
                            v[j + h] = __fsub_rn(a, b);
                        }
                const int lane_steps = p.block >> 3;  // lanes per WHT block
                for (int m = 1; m < lane_steps; m <<= 1) {
                    const bool upper = (lane & m) != 0;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
                        v[j] = upper ? __fsub_rn(o, v[j]) : __fadd_rn(v[j], o);
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = to_tf32(v[j] * p.inv_sqrt_block);
                sts_v4(strip_addr + static_cast<uint32_t>(lane) * 32u, v[0], v[1], v[2], v[3]);
                sts_v4(strip_addr + static_cast<uint32_t>(lane) * 32u + 16u, v[4], v[5], v[6], v[7]);
                __syncwarp();
#pragma unroll
                for (int s = 0; s < 4; ++s)
#pragma unroll
                    for (int k = 0; k < 16; k += 4)
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(bfrag[s][k]), "=r"(bfrag[s][k + 1]), "=r"(bfrag[s][k + 2]), "=r"(bfrag[s][k + 3])
                                     : "r"(strip_addr + static_cast<uint32_t>(64 * s + 16 * q + k) * 4u));
                __syncwarp();
            } else {
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
            }
        staged_slot = slot;
    };
    stage_slot(cur.slot, x_first, p.x != nullptr);

    for (int i = 0; i < n_local; ++i) {
        const int plane = cur.slot / p.n_chunks;
        (void)plane;
        if (cur.slot != staged_slot) stage_slot(cur.slot, make_uint4(0, 0, 0, 0), false);
        const bool has_next = i + 1 < n_local;

        float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            uint4& lo = blo[s & 1];
            uint4& hi = bhi[s & 1];
            // 16 independent lookups, then the 4 MMAs they feed (bytes 0,1 of a word feed one
            // MMA, bytes 2,3 the next); two accumulator chains.  Once the second half's addresses
            // are formed the code registers are free: the step two ahead is loaded into them.
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t l = w == 0 ? lo.x : (w == 1 ? lo.y : (w == 2 ? lo.z : lo.w));
                const uint32_t u = w == 0 ? hi.x : (w == 1 ? hi.y : (w == 2 ? hi.z : hi.w));
                uint32_t ad[8];
                ad[0] = lut_addr<0>(l, lane_const);
                ad[1] = lut_addr<0>(u, lane_const);
                ad[2] = lut_addr<1>(l, lane_const);
                ad[3] = lut_addr<1>(u, lane_const);
                ad[4] = lut_addr<2>(l, lane_const);
                ad[5] = lut_addr<2>(u, lane_const);
                ad[6] = lut_addr<3>(l, lane_const);
                ad[7] = lut_addr<3>(u, lane_const);
                if (w == 3) {
                    if (s < 2) load_step(cur, s + 2, true, lo, hi);
                    else load_step(nxt, s - 2, has_next, lo, hi);
                }
                uint32_t av[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) av[k] = lut_load(ad[k]);
                mma_tf32(acc0, av[0], av[1], av[2], av[3], bfrag[s][4 * w + 0], bfrag[s][4 * w + 1]);
                mma_tf32(acc1, av[4], av[5], av[6], av[7], bfrag[s][4 * w + 2], bfrag[s][4 * w + 3]);
            }
        }
        if (!has_next) grid_launch_dependents();  // the next kernel may start setting up

        // ---- cross-warp sum without a CTA-wide barrier, kLag units behind ----
        // Every warp drops its partial tile of unit i into ring slot i % kRing and signals
        // "written"; the sum is done kLag units later by all warps symmetrically, followed by
        // "read".  With a deep ring (16 slots for one activation row) warps drift apart by
        // several units, so a slow memory response delays one warp, not the CTA.
        if (i >= kLag) {
            reduce_unit(red.slot, red.ru, rs, rpar);
            red = next_pos(red);
            if (++rs == kRing) { rs = 0; rpar ^= 1u; }
        }
        if (i >= kRing && !mbar_wait(bar_read + 8u * ws, wpar)) {
            raise_status(p.status, 4u);
            atomicExch(&s_abort, 1u);
        }
        {
            // C fragment: (row g, columns 2q, 2q+1) and (row g+8, same columns)
            const uint32_t dst = red_addr + static_cast<uint32_t>(ws) * kSlotBytes + static_cast<uint32_t>(warp * kTileFloats) * 4u;
            const int n = 2 * q;
            if (n < BP) {
                sts_f32(dst + static_cast<uint32_t>(g * BP + n) * 4u, acc0[0] + acc1[0]);
                sts_f32(dst + static_cast<uint32_t>((g + 8) * BP + n) * 4u, acc0[2] + acc1[2]);
                if (n + 1 < BP) {
                    sts_f32(dst + static_cast<uint32_t>(g * BP + n + 1) * 4u, acc0[1] + acc1[1]);
                    sts_f32(dst + static_cast<uint32_t>((g + 8) * BP + n + 1) * 4u, acc0[3] + acc1[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_written + 8u * ws);
        if (++ws == kRing) { ws = 0; if (i >= kRing) wpar ^= 1u; }

        cur = nxt;
        if (i + 2 < n_local) nxt = next_pos(nxt);
    }
    // the last kLag units (or all of them, for a short range) are still to be summed
    for (int k = (n_local > kLag ? n_local - kLag : 0); k < n_local; ++k) {
        reduce_unit(red.slot, red.ru, rs, rpar);
        if constexpr (MULTI) if (k + 1 == n_local && pend > 0) flush_pending(red.ru);
        red = next_pos(red);
        if (++rs == kRing) { rs = 0; rpar ^= 1u; }
    }

    // ---- completion signal to the destinations' owners ----
    // Every thread orders its (possibly remote) result stores system-wide, the CTA counts in, and
    // the CTA that completes the grid publishes the flag everywhere.  Whoever then reads the flag
    // with acquire semantics sees all of this launch's results.
    if constexpr (SCATTER) {
    if (sargs.n_signal > 0 || LL) {
        __shared__ unsigned int s_last;
        // Packets, one slot: every row of this CTA's units was stored by this CTA, so it sends its own rows as soon
        // as it is done - the sends of the grid run side by side and nothing waits for the slowest CTA.  (With several
        // slots the CTA that completes a row tile is not known in advance: the completing CTA of the grid sends all.)
        const bool own_rows = LL && !MULTI;
        if constexpr (LL) if (own_rows) {
            __syncthreads();   // this CTA's stores are ordered before the loads below (read back through L2)
            const int per_row = p.out / 4;
            ll_send_packets(sargs, p.y, per_row, p.batch, u_begin * p.tpu * 4, min(per_row, (u_begin + n_local) * p.tpu * 4));
        }
        // results that went to other GPUs need a system-scope fence; with the bulk copy every CTA's
        // results are local and only the copying CTA pays for one
        if (sargs.bulk) __threadfence();
        else __threadfence_system();
        __syncthreads();
        if (tid == 0) {
            const unsigned int prev = atomicAdd(sargs.done_counter, 1u);
            s_last = (prev == static_cast<unsigned int>(nblk) - 1u) ? 1u : 0u;
        }
        __syncthreads();
        if (LL && s_last) {
            __threadfence();
            if constexpr (LL) if (!own_rows) ll_send_packets(sargs, p.y, p.out / 4, p.batch, 0, p.out / 4);
            __syncthreads();
            if (tid == 0) {
                *sargs.done_counter = 0u;  // ready for the next launch (stream order)
                atomicAdd(sargs.epoch, 1u);
                if (sargs.n_wait > 0) atomicAdd(sargs.wait_epoch, 1u);   // every CTA has read it by now
            }
        } else if (s_last) {
            __threadfence();
            if (sargs.bulk && sargs.n_peer > 0) {
                // the whole block (batch rows of `out` halves, y_stride apart) to every peer: 16-byte
                // pieces where the rows allow it
                const bool vec = (p.out % 8 == 0) && (sargs.y_stride % 8 == 0) && (reinterpret_cast<uintptr_t>(p.y) % 16 == 0);
                if (vec) {
                    const int per_row = p.out / 8;
                    for (int i = tid; i < per_row * p.batch; i += kCtaThreads) {
                        const int n = i / per_row, c = i - n * per_row;
                        const size_t o = static_cast<size_t>(n) * sargs.y_stride + static_cast<size_t>(c) * 8;
                        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(p.y + o));
#pragma unroll
                        for (int d = 0; d < 7; ++d)
                            if (d < sargs.n_peer) *reinterpret_cast<uint4*>(sargs.y_peer[d] + o) = v;
                    }
                } else {
                    for (int i = tid; i < p.out * p.batch; i += kCtaThreads) {
                        const int n = i / p.out, c = i - n * p.out;
                        const size_t o = static_cast<size_t>(n) * sargs.y_stride + c;
                        const __half v = __ldcg(p.y + o);
#pragma unroll
                        for (int d = 0; d < 7; ++d)
                            if (d < sargs.n_peer) sargs.y_peer[d][o] = v;
                    }
                }
                __threadfence_system();
                __syncthreads();
            }
            if (tid == 0) {
                *sargs.done_counter = 0u;  // ready for the next launch (stream order)
                unsigned int value = sargs.signal_value;
                if (sargs.bulk) value = atomicAdd(sargs.epoch, 1u) + 1u;
                if (sargs.n_wait > 0) atomicAdd(sargs.wait_epoch, 1u);   // every CTA has read it by now
                __threadfence_system();
#pragma unroll
                for (int d = 0; d < 8; ++d)
                    if (d < sargs.n_signal)
                        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(sargs.signal[d] + sargs.signal_slot), "r"(value) : "memory");
            }
        }
    }
    }
}

template <int BP, bool MULTI>
__global__ void __launch_bounds__(kCtaThreads, 1) tq8_gemv_kernel(const GemvArgs p) {
    gemv_body<BP, false, false, MULTI>(p, ScatterArgs{}, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
}
template <int BP, bool MULTI>
__global__ void __launch_bounds__(kCtaThreads, 1) tq8_gemv_packets_kernel(const GemvArgs p, const ScatterArgs sc) {
    gemv_body<BP, true, true, MULTI>(p, sc, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
}
template <int BP, bool MULTI>
__global__ void __launch_bounds__(kCtaThreads, 1) tq8_gemv_scatter_kernel(const GemvArgs p, const ScatterArgs sc) {
    gemv_body<BP, true, false, MULTI>(p, sc, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
}

// Several matrices that multiply the same activation (q / k / v, gate / up) in one launch: the grid is cut into one
// range of CTAs per matrix, in proportion to the matrices' units, and every CTA runs the ordinary body on its matrix
// with its index inside the range.  A decode layer's small projections then pay the launch and the prologue once.
constexpr int kMaxGroup = 4;
struct GemvGroupArgs {
    GemvArgs m[kMaxGroup];
    int cta_start[kMaxGroup + 1];   // CTAs cta_start[i] .. cta_start[i + 1] - 1 work on matrix i
    int n;
};
template <int BP, bool MULTI>
__global__ void __launch_bounds__(kCtaThreads, 1) tq8_gemv_group_kernel(const __grid_constant__ GemvGroupArgs grp) {
    const int b = static_cast<int>(blockIdx.x);
    int i = 0;
    while (i + 1 < grp.n && b >= grp.cta_start[i + 1]) ++i;
    gemv_body<BP, false, false, MULTI>(grp.m[i], ScatterArgs{}, b - grp.cta_start[i], grp.cta_start[i + 1] - grp.cta_start[i]);
}

// Waits (bounded) until flags[0..n) have all reached `value`: the receiving side of the completion
// signal above.  Runs on the GPU that owns the flags; the writers are kernels on other GPUs.
__global__ void peer_wait_kernel(const unsigned int* __restrict__ flags, int n, unsigned int value, unsigned int* status) {
    const int lane = threadIdx.x;
    if (lane >= n) return;
    const unsigned long long t0 = global_timer_ns();
    for (unsigned int spin = 0;; ++spin) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
        if (static_cast<int>(v - value) >= 0) return;
        if ((spin & 255u) == 255u && global_timer_ns() - t0 > 5ull * kWaitLimitNs) {  // 1 s: a peer is gone
            raise_status(status, 10u);
            return;
        }
    }
}

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// Warps that share one 16-row tile (a power of two up to 16); a chunk is that many 256-column slices, and
// the 16 / wpt row tiles of a unit run side by side.  Up to 4096 columns: the fewest warps that cover the
// row (one chunk).  Above: 16 warps per tile unless the last chunk would leave more than 15 % of the warps'
// slices empty (5120 columns = 20 slices: 16 + 4, i.e. 62 %); then the split with at most 8 chunks that leaves the
// fewest slices empty (5120: 4 warps, five chunks of 1024 columns; 4608: 4 warps, 90 %; 6144: 8 warps, 100 %).
int warps_per_tile(int in) {
    const int slices = (in + kSlice - 1) / kSlice;
    if (in <= kWarps * kSlice) {
        int w = 1;
        while (w < kWarps && w < slices) w <<= 1;
        return w;
    }
    auto fill = [&](int w) { return static_cast<double>(slices) / (static_cast<double>((slices + w - 1) / w) * w); };
    if (fill(kWarps) >= 0.85) return kWarps;
    // otherwise the split (at most 8 chunks) that leaves the fewest slices empty; the wider one when two are close
    int best = kWarps;
    for (int w = kWarps / 2; w >= 1; w >>= 1)
        if ((slices + w - 1) / w <= 8 && fill(w) > fill(best) + 0.02) best = w;
    return best;
}
int chunk_columns(int in) { return warps_per_tile(in) * kSlice; }

}  // namespace

// Scratch layout: [xrot: n_planes*8*in fp32][partials: n_slots*8*out_pad fp32][counters: n_row_tiles*16 u32]
size_t gemv_scratch_bytes(int out, int in, int n_planes) {
    const int chunk = chunk_columns(in);
    const int n_slots = ((in + chunk - 1) / chunk) * n_planes;
    const int n_row_tiles = (out + 15) / 16;
    const size_t out_pad = static_cast<size_t>(n_row_tiles) * 16;
    size_t bytes = align256(static_cast<size_t>(n_planes) * 8 * in * sizeof(float));
    if (n_slots > 1)
        bytes += align256(static_cast<size_t>(n_slots) * 8 * out_pad * sizeof(float)) +
                 align256(static_cast<size_t>(n_row_tiles) * kWarps * sizeof(unsigned int));
    return bytes;
}

// Geometry, rotation mode and scratch pointers of one matrix (codes, norms, table, y and status are the caller's).
// Returns whether the kernel rotates the activation itself; otherwise rotate_x_kernel fills a.xrot first.
static bool fill_gemv_args(GemvArgs& a, const __half* x, int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p,
                           uint32_t seed_r, void* scratch) {
    a.out = out; a.in = in; a.batch = batch;
    const int n_row_tiles = (out + 15) / 16;
    a.wpt = warps_per_tile(in);
    a.tpu = kWarps / a.wpt;
    const int chunk = a.wpt * kSlice;  // columns per chunk
    a.n_chunks = (in + chunk - 1) / chunk;
    a.n_slots = a.n_chunks * n_planes;
    a.out_pad = n_row_tiles * 16;
    a.n_row_units = (n_row_tiles + a.tpu - 1) / a.tpu;
    a.inv_scale = 1.0f / std::sqrt(static_cast<float>(in));
    // Blocks that fit a warp's 256-column slice are rotated inside the GEMV kernel (16-byte
    // activation loads); larger blocks, or an unaligned activation, go through rotate_x_kernel.
    // In-kernel rotation handles one activation row after the other (a chain of lane exchanges per row) in every
    // warp, which costs more than the pre-kernel from two rows on (4096 x 4096: 9.0 / 11.3 / 15.3 us in-kernel
    // against 8.3 / 9.2 / 10.8 us with the pre-kernel at 2 / 4 / 8 rows; the same at one row).
    const bool fused_rotation = block <= static_cast<uint32_t>(kSlice) && in % 8 == 0 &&
                                reinterpret_cast<uintptr_t>(x) % 16 == 0 && batch == 1;
    a.x = fused_rotation ? x : nullptr;
    a.seed_p = seed_p; a.seed_r = seed_r;
    a.block = static_cast<int>(block);
    a.inv_sqrt_block = 1.0f / std::sqrt(static_cast<float>(block));
    uint8_t* sp = static_cast<uint8_t*>(scratch);
    float* xrot = reinterpret_cast<float*>(sp);
    a.xrot = xrot;
    if (a.n_slots > 1) {
        sp += align256(static_cast<size_t>(n_planes) * 8 * in * sizeof(float));
        a.partial = reinterpret_cast<float*>(sp);
        sp += align256(static_cast<size_t>(a.n_slots) * 8 * a.out_pad * sizeof(float));
        a.counters = reinterpret_cast<unsigned int*>(sp);
    }

    return fused_rotation;
}

// Shared-memory opt-in of every instantiation, once per device.
static void configure_gemv_kernels();
static void launch_rotate_x_pdl(const __half* x, float* xrot, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p,
                                uint32_t seed_r, cudaStream_t stream);

void launch_tq8_gemv(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                     int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                     void* scratch, unsigned int* status, int sm_count, cudaStream_t stream) {
    launch_tq8_gemv_scatter(codes, norms, table, x, &y, 1, out, out, in, batch, block, n_planes, seed_p, seed_r, scratch,
                            status, sm_count, stream);
}

void launch_peer_wait(const unsigned int* flags, int n, unsigned int value, unsigned int* status, cudaStream_t stream) {
    TQ_REQUIRE(flags != nullptr && n >= 1 && n <= 32, "peer wait: 1..32 flags");
    peer_wait_kernel<<<1, 32, 0, stream>>>(flags, n, value, status);
    TQ_CUDA(cudaGetLastError());
}

void launch_tq8_gemv_scatter(const uint8_t* codes, const float* norms, const float* table, const __half* x,
                             __half* const* dst, int n_dst, long dst_stride, int out, int in, int batch, uint32_t block,
                             int n_planes, uint32_t seed_p, uint32_t seed_r, void* scratch, unsigned int* status,
                             int sm_count, cudaStream_t stream, unsigned int* const* signal, int signal_slot,
                             unsigned int signal_value, unsigned int* done_counter, const GemvGather* gather, int n_signal) {
    TQ_REQUIRE(dst != nullptr && n_dst >= 1 && n_dst <= 8, "tq8_gemv: 1..8 destinations");
    TQ_REQUIRE(dst_stride >= out, "tq8_gemv: destination row stride smaller than the layer's rows");
    __half* y = dst[0];
    TQ_REQUIRE(n_planes == 1 || n_planes == 2, "tq8_gemv: one or two rotation planes");
    TQ_REQUIRE(batch >= 1 && batch <= 8, "tq8_gemv handles 1..8 activation rows per launch");
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "WHT block size must be a power of two in [32, 1024]");
    TQ_REQUIRE(in % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    TQ_REQUIRE(scratch != nullptr, "tq8_gemv needs its scratch buffer");
    if (out == 0) return;

    GemvArgs a{};
    a.codes = codes; a.norms = norms; a.table = table; a.y = y; a.status = status;
    ScatterArgs sa{};
    sa.n_peer = n_dst - 1;
    for (int d = 1; d < n_dst; ++d) {
        TQ_REQUIRE(dst[d] != nullptr, "tq8_gemv: NULL destination");
        sa.y_peer[d - 1] = dst[d];
    }
    sa.y_stride = dst_stride;
    sa.n_signal = 0;
    if (signal != nullptr) {
        sa.n_signal = n_signal > 0 ? n_signal : n_dst;
        TQ_REQUIRE(sa.n_signal <= 8, "tq8_gemv: at most 8 flag arrays");
        for (int d = 0; d < sa.n_signal; ++d) {
            TQ_REQUIRE(signal[d] != nullptr, "tq8_gemv: NULL signal array");
            sa.signal[d] = signal[d];
        }
        sa.signal_slot = signal_slot;
        sa.signal_value = signal_value;
        TQ_REQUIRE(done_counter != nullptr, "tq8_gemv: signalling needs a completion counter in device memory");
        sa.done_counter = done_counter;
    }
    if (gather != nullptr) {
        TQ_REQUIRE((signal != nullptr || gather->ll_world > 0) && gather->epoch != nullptr,
                   "tq8_gemv: the fused all-gather needs flags (or packet buffers) and an epoch counter");
        TQ_REQUIRE(gather->n_wait >= 0 && gather->n_wait <= 32, "tq8_gemv: 0..32 flags to wait for");
        TQ_REQUIRE(gather->n_wait == 0 || ((gather->wait_flags != nullptr || gather->ll_world > 0) && gather->wait_epoch != nullptr),
                   "tq8_gemv: waiting needs the local flag array and the wait counter");
        sa.bulk = 1;
        if (gather->ll_world > 0) {
            TQ_REQUIRE(gather->ll_world <= 8 && gather->ll_rank >= 0 && gather->ll_rank < gather->ll_world, "tq8_gemv: bad rank / world");
            TQ_REQUIRE(out % 4 == 0 && dst_stride % 4 == 0 && reinterpret_cast<uintptr_t>(y) % 8 == 0,
                       "tq8_gemv: the flag-in-data exchange moves groups of four rows (8-byte aligned)");
            sa.ll = 1;
            sa.ll_rank = gather->ll_rank;
            sa.ll_world = gather->ll_world;
            for (int r = 0; r < gather->ll_world; ++r) {
                TQ_REQUIRE(gather->ll_base[r] != nullptr, "tq8_gemv: NULL packet buffer");
                sa.ll_base[r] = static_cast<uint4*>(gather->ll_base[r]);
            }
            sa.n_peer = 0;   // results are stored locally; the packets carry them to the other ranks
            TQ_REQUIRE(done_counter != nullptr, "tq8_gemv: the exchange needs a completion counter in device memory");
            sa.done_counter = done_counter;
        }
        sa.epoch = gather->epoch;
        sa.wait_flags = gather->wait_flags;
        sa.n_wait = gather->n_wait;
        sa.wait_epoch = gather->wait_epoch;
    }
    const bool fused_rotation = fill_gemv_args(a, x, out, in, batch, block, n_planes, seed_p, seed_r, scratch);
    float* xrot = const_cast<float*>(a.xrot);
    const int bp = batch <= 1 ? 1 : (batch <= 2 ? 2 : (batch <= 4 ? 4 : 8));

    configure_gemv_kernels();

    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    const int n_attr = 1;

    // 1. rotate the activation (one warp per plane x row x block)
    if (!fused_rotation) launch_rotate_x_pdl(x, xrot, in, batch, block, n_planes, seed_p, seed_r, stream);
    // 2. the GEMV itself
    {
        const int n_units = a.n_row_units * a.n_slots;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(n_units < sm_count ? n_units : sm_count);
        cfg.blockDim = dim3(kCtaThreads);
        cfg.dynamicSmemBytes = kGemvSmem;
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = n_attr;
        // one destination with the layer's own row stride and no signal: the plain variant
        const bool scatter = sa.n_peer > 0 || sa.n_signal > 0 || sa.ll != 0 || sa.y_stride != a.out;
#define TQ_GEMV_LAUNCH2(BPV, MV)                                                                  \
    if (sa.ll) TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_packets_kernel<BPV, MV>, a, sa));        \
    else if (scatter) TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_scatter_kernel<BPV, MV>, a, sa)); \
    else TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_kernel<BPV, MV>, a));
#define TQ_GEMV_LAUNCH(BPV)                           \
    if (a.n_slots > 1) { TQ_GEMV_LAUNCH2(BPV, true) } \
    else { TQ_GEMV_LAUNCH2(BPV, false) }
        switch (bp) {
            case 1: TQ_GEMV_LAUNCH(1) break;
            case 2: TQ_GEMV_LAUNCH(2) break;
            case 4: TQ_GEMV_LAUNCH(4) break;
            default: TQ_GEMV_LAUNCH(8) break;
        }
#undef TQ_GEMV_LAUNCH
#undef TQ_GEMV_LAUNCH2
    }
}

static void configure_gemv_kernels() {
    // the opt-in shared-memory size is a per-device function attribute
    static bool configured[64] = {false};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && configured[dev]) return;
#define TQ_GEMV_ATTR1(K) TQ_CUDA(cudaFuncSetAttribute(K, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemvSmem)));
#define TQ_GEMV_ATTR(BPV)                                \
    TQ_GEMV_ATTR1((tq8_gemv_kernel<BPV, false>))         \
    TQ_GEMV_ATTR1((tq8_gemv_kernel<BPV, true>))          \
    TQ_GEMV_ATTR1((tq8_gemv_scatter_kernel<BPV, false>)) \
    TQ_GEMV_ATTR1((tq8_gemv_scatter_kernel<BPV, true>))  \
    TQ_GEMV_ATTR1((tq8_gemv_packets_kernel<BPV, false>)) \
    TQ_GEMV_ATTR1((tq8_gemv_packets_kernel<BPV, true>))  \
    TQ_GEMV_ATTR1((tq8_gemv_group_kernel<BPV, false>))   \
    TQ_GEMV_ATTR1((tq8_gemv_group_kernel<BPV, true>))
    TQ_GEMV_ATTR(1)
    TQ_GEMV_ATTR(2)
    TQ_GEMV_ATTR(4)
    TQ_GEMV_ATTR(8)
#undef TQ_GEMV_ATTR
#undef TQ_GEMV_ATTR1
    if (dev < 64) configured[dev] = true;
}

static void launch_rotate_x_pdl(const __half* x, float* xrot, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p,
                                uint32_t seed_r, cudaStream_t stream) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
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

void launch_tq8_gemv_group(const GemvGroupItem* items, int n, const __half* x, int batch, int sm_count, cudaStream_t stream) {
    TQ_REQUIRE(items != nullptr && n >= 1 && n <= kMaxGroup, "tq8_gemv group: 1..4 matrices");
    TQ_REQUIRE(x != nullptr && batch >= 1 && batch <= 8, "tq8_gemv group: 1..8 activation rows");
    GemvGroupArgs grp{};
    grp.n = n;
    int units[kMaxGroup], total_units = 0;
    bool fused[kMaxGroup];
    for (int i = 0; i < n; ++i) {
        const GemvGroupItem& it = items[i];
        TQ_REQUIRE(it.codes && it.norms && it.table && it.y && it.scratch, "tq8_gemv group: NULL argument");
        TQ_REQUIRE(it.out >= 1 && it.in == items[0].in && it.n_planes == items[0].n_planes,
                   "tq8_gemv group: the matrices must share in_features and the rotation mode");
        TQ_REQUIRE(it.n_planes == 1 || it.n_planes == 2, "n_planes must be 1 or 2");
        TQ_REQUIRE(is_pow2(it.block) && it.block >= 32 && it.block <= 1024, "WHT block size must be a power of two in [32, 1024]");
        TQ_REQUIRE(it.in % static_cast<int>(it.block) == 0, "in_features must be divisible by block_size");
        GemvArgs& a = grp.m[i];
        a.codes = it.codes; a.norms = it.norms; a.table = it.table; a.y = it.y; a.status = it.status;
        fused[i] = fill_gemv_args(a, x, it.out, it.in, batch, it.block, it.n_planes, it.seed_p, it.seed_r, it.scratch);
        units[i] = a.n_row_units * a.n_slots;
        total_units += units[i];
    }
    // CTAs in proportion to the units, at least one per matrix, never more than a matrix has units
    const int total = total_units < sm_count ? total_units : sm_count;
    TQ_REQUIRE(total >= n, "tq8_gemv group: fewer SMs than matrices");
    int ctas[kMaxGroup], given = 0;
    for (int i = 0; i < n; ++i) {
        long c = static_cast<long>(total) * units[i] / total_units;
        ctas[i] = static_cast<int>(c < 1 ? 1 : (c > units[i] ? units[i] : c));
        given += ctas[i];
    }
    while (given > total) {   // the minimum of one pushed the sum over: take from the largest
        int big = 0;
        for (int i = 1; i < n; ++i) if (ctas[i] > ctas[big]) big = i;
        --ctas[big]; --given;
    }
    while (given < total) {   // rounding left CTAs over: to the matrix with the most units per CTA that can still use one
        int best = -1;
        for (int i = 0; i < n; ++i)
            if (ctas[i] < units[i] && (best < 0 || static_cast<long>(units[i]) * ctas[best] > static_cast<long>(units[best]) * ctas[i])) best = i;
        if (best < 0) break;
        ++ctas[best]; ++given;
    }
    grp.cta_start[0] = 0;
    for (int i = 0; i < n; ++i) grp.cta_start[i + 1] = grp.cta_start[i] + ctas[i];
    for (int i = n; i < kMaxGroup; ++i) grp.cta_start[i + 1] = grp.cta_start[n];
    configure_gemv_kernels();
    for (int i = 0; i < n; ++i)
        if (!fused[i])
            launch_rotate_x_pdl(x, const_cast<float*>(grp.m[i].xrot), items[i].in, batch, items[i].block, items[i].n_planes,
                                items[i].seed_p, items[i].seed_r, stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grp.cta_start[n]);
    cfg.blockDim = dim3(kCtaThreads);
    cfg.dynamicSmemBytes = kGemvSmem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int bp = batch <= 1 ? 1 : (batch <= 2 ? 2 : (batch <= 4 ? 4 : 8));
    const bool multi = grp.m[0].n_slots > 1;   // the same for all: same in_features and planes
#define TQ_GROUP_LAUNCH(BPV)                                                              \
    if (multi) TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_group_kernel<BPV, true>, grp)); \
    else TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_group_kernel<BPV, false>, grp));
    switch (bp) {
        case 1: TQ_GROUP_LAUNCH(1) break;
        case 2: TQ_GROUP_LAUNCH(2) break;
        case 4: TQ_GROUP_LAUNCH(4) break;
        default: TQ_GROUP_LAUNCH(8) break;
    }
#undef TQ_GROUP_LAUNCH
}

// The activation rotation alone (the pre-kernel of WHT blocks above 256 columns), for the other
// decode kernels: xrot = [n_planes, batch, in] fp32.
void launch_rotate_x(const __half* x, float* xrot, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p,
                     uint32_t seed_r, cudaStream_t stream) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
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

// The same address for the other decode kernel's allocation-free variant.
void* gemv_static_scratch_address() { return static_scratch_address(); }

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
        const size_t counter_bytes = align256(static_cast<size_t>(n_row_tiles) * kWarps * sizeof(unsigned int));
        TQ_CUDA(cudaMemsetAsync(static_cast<uint8_t*>(scratch) + need - counter_bytes, 0, counter_bytes, stream));
    }
    launch_tq8_gemv(codes, norms, table, x, y, out, in, batch, block, n_planes, seed_p, seed_r, scratch, status, sm_count,
                    stream);
}

}  // namespace tq
