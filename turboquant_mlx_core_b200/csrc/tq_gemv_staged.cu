// Fused TQ8 dequantise + GEMV for decode (1..8 activation rows), codes staged through shared
// memory by bulk copies.
//
// Replaces the reference's tq_dequant_mm Metal kernel and its host wrapper
// (metal/turboquant_dequant_mm.metal:152-313, src/dequantizer.cpp:606-721):
//   y[b, r] = fp16( norm[r] * sum_j W~[r, j] * fp16(x[b, j]) ),  fp32 accumulate.
// Same algebra as tq_gemv.cu: H is symmetric, so the activation is rotated once and a weight
// costs one table lookup:  y[b, r] = norm[r] * inv_scale * sum_j table[code[r, j]] * xrot[b, j].
//
// What is different from tq_gemv.cu is how the bytes move and who owns which of them.
//   * The matrix is a list of 1 KB code tiles (16 rows x 64 columns, tq_common.cuh::code_offset).
//     Four consecutive tiles are a "chunk"; chunks are numbered slot-major (a slot is the range of
//     columns whose rotated activation fits in shared memory at once), then by row tile, then by
//     column.  Every CTA owns a contiguous range of T * b / G chunks: the byte count per SM is
//     balanced to one chunk, whatever the shape.
//   * A chunk comes in by ONE cp.async.bulk (4 KB, contiguous in HBM) completing on an mbarrier.
//     The warps of a CTA form groups of four; group k takes the chunks k, k + groups, ... of the
//     range and owns a private ring of buffers.  A warp copies its tile of a chunk into registers
//     (two 16-byte shared loads), counts in on the buffer's arrival counter, and the warp that
//     completes the count issues the copy that refills the buffer - no producer warp, no CTA-wide
//     barrier.  The first copies are issued before the kernel waits for its predecessor in the
//     stream (programmatic dependent launch), so with one 16-warp CTA per SM per layer the next
//     layer's CTA is already resident and filling its ring while this layer computes.
//   * Codes -> PRMT (address) -> lane-private table in shared memory -> fp16 pair -> A fragment of
//     mma.sync.m16n8k16; the rotated activation is read from shared memory as the B fragment (one
//     16-byte load per 512 weights and activation row), so no warp is tied to a column range.
//   * A warp accumulates over all its tiles of a (slot, row tile) "segment", then drops 16 x BP
//     partial sums into a shared-memory slot; the warp that arrives last adds the slot up in warp
//     order (fixed order: run-to-run identical) and either writes y or, when the segment is shared
//     with other CTAs or other slots, writes a piece to scratch; the last piece's writer adds the
//     pieces in fixed order.
//
// Shared-memory window of a CTA (addresses relative to the CTA's window):
//   [.., 0x4000)        partial-sum slots (16-warp variant)
//   [0x4000, 0x14000)   table: 256 entries x 256 B; bytes 0..127 of an entry hold 32 lane-private
//                       copies of (value, value) as fp16x2, bytes 128..255 hold a 64-column piece
//                       of one rotated activation row (fp16)
//   [0x14000, ...)      chunk buffers, then the partial-sum slots of the 32-warp variant
// The address of a lookup is a byte permutation of (code word, lane constant 0x0001_00_ll) plus a
// fixed negative immediate in the load instruction, which is how the table can start at 0x4000.
// 16 warps, 112 KB and at most 64 registers per thread: two CTAs fit an SM.
//
// Every wait is bounded: on a time-out the warp raises the status word and the CTA's abort flag and
// falls through to the end (copies in flight are left to land in the CTA's own shared memory).
#include <cmath>
#include <cstdint>
#include <cstdlib>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

constexpr uint32_t kLutWin = 0x4000u;        // window address of the table
constexpr uint32_t kLutPrmt = 0x10000u;      // what the byte permutation builds (bytes 2,3 = 0x0001)
constexpr uint32_t kRingWin = 0x14000u;      // window address of the chunk buffers
constexpr int kChunkTiles = 4;
constexpr uint32_t kChunkBytes = kChunkTiles * kCodeTileBytes;
constexpr int kMaxRedSlots = 8;
constexpr unsigned long long kStagedWaitNs = 200ull * 1000 * 1000;

template <int NW> struct StagedCfg;
template <> struct StagedCfg<16> {
    static constexpr int kGroups = 4, kDepth = 2;
    static constexpr uint32_t kRingEnd = kRingWin + kGroups * kDepth * kChunkBytes;   // 0x1C000
    static constexpr uint32_t kRedWin = 0;            // partial sums below the table
    static constexpr uint32_t kEnd = kRingEnd;
    static constexpr int kMinBlocks = 2;
};
template <> struct StagedCfg<32> {
    static constexpr int kGroups = 8, kDepth = 3;
    static constexpr uint32_t kRingEnd = kRingWin + kGroups * kDepth * kChunkBytes;   // 0x2C000
    static constexpr uint32_t kRedWin = kRingEnd;     // partial sums above the ring
    static constexpr uint32_t kEnd = kRedWin + 0xC000u;                               // 0x38000
    static constexpr int kMinBlocks = 1;
};

struct StagedArgs {
    const uint8_t* codes;    // joint bytes in 16 x 64 tiles
    const float* norms;      // [out]
    const float* table;      // [n_planes, 256] fp32
    const float* xrot;       // [n_planes, batch, in] fp32, rotated by rotate_x_kernel (WHT blocks > 256); else nullptr
    const __half* x;         // [batch, in] fp16 (rotated inside the kernel) when xrot == nullptr
    __half* y;               // [batch, out]
    float* partial;          // [RT][n_slots * P][16 * BP] pieces (segments shared between CTAs or slots)
    unsigned int* counters;  // [RT] arrival counters, zero between launches
    unsigned int* status;
    int out, in, batch;
    int RT, CT;              // row tiles, column tiles per row
    int KS, SCT;             // slots per plane, column tiles per full slot
    int n_planes;
    int cps_full, cps_last;  // chunks per segment in the full slots / in the last slot of a plane
    int cpp;                 // chunks per plane
    int T;                   // chunks in all
    int P;                   // piece slots per (row tile, slot)
    float inv_scale;
    uint32_t seed_p, seed_r;
    int block;
    float inv_sqrt_block;
    int ablate;              // measurement only: bit 0 skips lookups and MMAs, bit 1 skips the partial-sum reduction
};

__device__ __forceinline__ uint32_t s_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ unsigned long long s_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void s_griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void s_griddep_launch() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ void s_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool s_mbar_wait(uint32_t bar, uint32_t parity, volatile unsigned int* abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spin & 31) == 31 && *abort_flag) return false;
        if (spin == 64) t0 = s_timer_ns();
        if (spin > 64 && (spin & 63) == 0 && s_timer_ns() - t0 > kStagedWaitNs) return false;
    }
}
// One chunk: `bytes` contiguous bytes of code tiles into a ring buffer, completing on `bar`.
__device__ __forceinline__ void s_bulk_load(uint32_t dst, const uint8_t* src, uint32_t bytes, uint32_t bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint32_t s_atom_inc(uint32_t addr) {
    uint32_t old;
    asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], 1;" : "=r"(old) : "r"(addr) : "memory");
    return old;
}
__device__ __forceinline__ uint32_t s_ld_acquire(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void s_st_release(uint32_t addr, uint32_t v) {
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 s_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void s_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void s_sts32(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float s_lds32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
// Lookup of this lane's copy of the entry selected by byte BYTE of `word`.  The permutation gives
// 0x0001_cc_ll (code in byte 1, lane offset in byte 0); the table starts 0xC000 below 0x10000.
template <int BYTE>
__device__ __forceinline__ uint32_t s_lookup(uint32_t word, uint32_t lane_const) {
    const uint32_t a = __byte_perm(word, lane_const, 0x7604u | (static_cast<uint32_t>(BYTE) << 4));
    uint32_t v;
    asm("ld.shared.b32 %0, [%1 + -49152];" : "=r"(v) : "r"(a));
    return v;
}
static_assert(kLutPrmt - kLutWin == 49152u, "the immediate in s_lookup is the distance between 0x10000 and the table");

__device__ __forceinline__ void s_mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t s_pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Position of a chunk in the matrix.
struct ChunkPos {
    int sidx;   // slot index: plane * KS + slot inside the plane
    int ks;     // slot inside the plane
    int rt;     // row tile
    int cc;     // chunk inside the segment
    int cps;    // chunks per segment of this slot
    int width;  // column tiles of this slot
};

__device__ __forceinline__ ChunkPos s_decode(const StagedArgs& p, int c) {
    ChunkPos u;
    const int plane = c / p.cpp;
    int r = c - plane * p.cpp;
    const int full = (p.KS - 1) * p.RT * p.cps_full;
    int ks;
    if (r < full) {
        ks = r / (p.RT * p.cps_full);
        r -= ks * p.RT * p.cps_full;
        u.cps = p.cps_full;
    } else {
        ks = p.KS - 1;
        r -= full;
        u.cps = p.cps_last;
    }
    u.rt = r / u.cps;
    u.cc = r - u.rt * u.cps;
    u.ks = ks;
    u.sidx = plane * p.KS + ks;
    u.width = ks < p.KS - 1 ? p.SCT : p.CT - (p.KS - 1) * p.SCT;
    return u;
}
__device__ __forceinline__ void s_advance(const StagedArgs& p, ChunkPos& u, int step) {
    u.cc += step;
    while (u.cc >= u.cps) {
        u.cc -= u.cps;
        if (++u.rt == p.RT) {
            u.rt = 0;
            ++u.sidx;
            if (++u.ks == p.KS) u.ks = 0;
            const bool last = u.ks == p.KS - 1;
            u.cps = last ? p.cps_last : p.cps_full;
            u.width = last ? p.CT - (p.KS - 1) * p.SCT : p.SCT;
        }
    }
}
// First chunk of segment (sidx, rt).
__device__ __forceinline__ int s_seg_start(const StagedArgs& p, int sidx, int rt) {
    const int plane = sidx / p.KS, ks = sidx - plane * p.KS;
    const int inside = ks < p.KS - 1 ? (ks * p.RT + rt) * p.cps_full : (p.KS - 1) * p.RT * p.cps_full + rt * p.cps_last;
    return plane * p.cpp + inside;
}
// CTA ranges are [T*b/G, T*(b+1)/G): the CTA that owns chunk c.
__device__ __forceinline__ int s_owner(int c, int T, int G) {
    return static_cast<int>(((static_cast<long long>(c) + 1) * G - 1) / T);
}

template <int BP, int NW>
__global__ void __launch_bounds__(NW * 32, StagedCfg<NW>::kMinBlocks) tq8_gemv_staged_kernel(const StagedArgs p) {
    using Cfg = StagedCfg<NW>;
    constexpr int NG = Cfg::kGroups, D = Cfg::kDepth;
    constexpr uint32_t kTileFloats = 16 * BP;                 // one warp's partial tile
    constexpr uint32_t kRedSlotBytes = NW * kTileFloats * 4;  // one segment's partial tiles
    constexpr int kCapCt = 256 / BP;                          // column tiles of rotated activation the table gaps hold per row

    extern __shared__ __align__(128) uint8_t staged_smem[];
    __shared__ __align__(8) unsigned long long s_full[NG * D];
    __shared__ unsigned int s_ring_cnt[NG * D];
    __shared__ unsigned int s_red_cnt[kMaxRedSlots];
    __shared__ unsigned int s_red_gen[kMaxRedSlots];
    __shared__ unsigned int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int grp = warp & (NG - 1), wi = warp / NG;   // group and position inside it: the group's warps are NG apart
    const int g = lane >> 2, q = lane & 3;

    const int G = gridDim.x;
    const int c0 = static_cast<int>(static_cast<long long>(p.T) * blockIdx.x / G);
    const int c1 = static_cast<int>(static_cast<long long>(p.T) * (blockIdx.x + 1) / G);
    const int n_local = c1 - c0;
    if (n_local <= 0) return;

    // ---- shared-memory map ----
    const uint32_t dyn = s_u32(staged_smem);
    uint32_t dyn_bytes;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    uint32_t red_base, red_bytes;
    if (Cfg::kRedWin == 0) {
        red_base = (dyn + 127u) & ~127u;
        red_bytes = red_base < kLutWin ? kLutWin - red_base : 0u;
    } else {
        red_base = Cfg::kRedWin;
        red_bytes = Cfg::kEnd - Cfg::kRedWin;
    }
    int red_slots = static_cast<int>(red_bytes / kRedSlotBytes);
    if (red_slots > kMaxRedSlots) red_slots = kMaxRedSlots;
    if (dyn > kLutWin || dyn + dyn_bytes < Cfg::kEnd || red_slots < 2) {   // layout assumption broken: refuse to run
        if (tid == 0) raise_status(p.status, 1u);
        return;
    }
    const uint32_t bar_full = s_u32(&s_full[0]);
    const uint32_t ring_cnt = s_u32(&s_ring_cnt[0]);
    const uint32_t red_cnt = s_u32(&s_red_cnt[0]), red_gen = s_u32(&s_red_gen[0]);
    volatile unsigned int* abort_flag = &s_abort;

    if (tid == 0) {
        for (int i = 0; i < NG * D; ++i) {
            s_mbar_init(bar_full + 8u * i, 1);
            s_ring_cnt[i] = 0u;
        }
        for (int i = 0; i < kMaxRedSlots; ++i) {
            s_red_cnt[i] = 0u;
            s_red_gen[i] = 0u;
        }
        s_abort = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // The next kernel in the stream may start its own set-up now (it waits for this grid before it
    // touches anything this grid reads or writes besides the weights).
    s_griddep_launch();

    // ---- chunk addressing ----
    const size_t row_tile_bytes = static_cast<size_t>(p.CT) * kCodeTileBytes;
    auto chunk_src = [&](const ChunkPos& u, uint32_t& bytes) -> const uint8_t* {
        const int t0 = u.cc * kChunkTiles;
        const int nt = u.width - t0 < kChunkTiles ? u.width - t0 : kChunkTiles;
        bytes = static_cast<uint32_t>(nt) * kCodeTileBytes;
        return p.codes + static_cast<size_t>(u.rt) * row_tile_bytes + static_cast<size_t>(u.ks * p.SCT + t0) * kCodeTileBytes;
    };

    // ---- first copies: the group's first D chunks, issued by lane 0 of the group's first warp ----
    // (weights do not depend on the preceding kernel, so this happens before the dependency wait)
    ChunkPos cur = s_decode(p, c0 + grp < c1 ? c0 + grp : c0);
    ChunkPos ahead = cur;   // position of the chunk that will refill the buffer being read
    {
        ChunkPos f = cur;
        for (int m = 0; m < D; ++m) {
            const int i = grp + NG * m;
            if (i < n_local && wi == 0 && lane == 0) {
                uint32_t bytes;
                const uint8_t* src = chunk_src(f, bytes);
                s_bulk_load(kRingWin + static_cast<uint32_t>(grp * D + m) * kChunkBytes, src, bytes, bar_full + 8u * (grp * D + m));
            }
            if (i + NG < n_local) s_advance(p, f, NG);
        }
        ahead = f;   // stands at chunk grp + NG*D when that chunk exists (it is not used otherwise)
    }

    // ---- table ----
    const uint32_t lane_const = kLutPrmt | static_cast<uint32_t>(lane * 4);
    auto build_table = [&](int plane) {
        for (int i = tid; i < 256 * 8; i += NW * 32) {
            const int e = i >> 3, c4 = (i & 7) * 4;
            const __half h = __float2half_rn(__ldg(p.table + plane * 256 + e));
            const uint32_t v = static_cast<uint32_t>(__half_as_ushort(h)) * 0x00010001u;
            s_sts128(kLutWin + static_cast<uint32_t>(e) * 256u + static_cast<uint32_t>(c4) * 4u, v, v, v, v);
        }
    };
    // ---- rotated activation of one slot into the table's gaps ----
    // Row n, column tile t (inside the slot) lives in the upper half of table entry n * kCapCt + t;
    // its eight 16-byte pieces are stored at piece ^ (n & 1), so that the two activation rows a
    // quarter-warp reads side by side fall into different banks.
    auto stage_x = [&](int sidx) {
        const int plane = sidx / p.KS, ks = sidx - plane * p.KS;
        const int col_base = ks * p.SCT * 64;
        const int width = ks < p.KS - 1 ? p.SCT : p.CT - (p.KS - 1) * p.SCT;
        const int groups256 = (width * 64 + 255) / 256;
        const uint32_t seed = plane ? p.seed_r : p.seed_p;
        for (int task = warp; task < p.batch * groups256; task += NW) {
            const int n = task / groups256, gq = task - n * groups256;
            const int cl = gq * 256 + 8 * lane;        // column inside the slot
            const int col = col_base + cl;
            uint32_t h[4] = {0u, 0u, 0u, 0u};
            if (p.xrot != nullptr) {
                if (col < p.in) {
                    const float* src = p.xrot + (static_cast<size_t>(plane) * p.batch + n) * p.in + col;
                    const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
                    h[0] = s_pack_half2(a.x, a.y); h[1] = s_pack_half2(a.z, a.w);
                    h[2] = s_pack_half2(b.x, b.y); h[3] = s_pack_half2(b.z, b.w);
                }
            } else {
                uint4 raw = make_uint4(0u, 0u, 0u, 0u);
                if (col < p.in) raw = __ldg(reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(n) * p.in + col));
                const uint32_t xw[4] = {raw.x, raw.y, raw.z, raw.w};
                float v[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 h2 = *reinterpret_cast<const __half2*>(&xw[j]);
                    const float lo = __low2float(h2), hi = __high2float(h2);
                    v[2 * j] = sign_is_positive(seed, static_cast<uint32_t>((col + 2 * j) & (p.block - 1))) ? lo : -lo;
                    v[2 * j + 1] = sign_is_positive(seed, static_cast<uint32_t>((col + 2 * j + 1) & (p.block - 1))) ? hi : -hi;
                }
#pragma unroll
                for (int hh = 1; hh < 8; hh <<= 1)
#pragma unroll
                    for (int i = 0; i < 8; i += 2 * hh)
#pragma unroll
                        for (int j = i; j < i + hh; ++j) {
                            const float a = v[j], b = v[j + hh];
                            v[j] = __fadd_rn(a, b);
                            v[j + hh] = __fsub_rn(a, b);
                        }
                const int lane_steps = p.block >> 3;   // lanes per WHT block (block <= 256 on this path)
                for (int m = 1; m < lane_steps; m <<= 1) {
                    const bool upper = (lane & m) != 0;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
                        v[j] = upper ? __fsub_rn(o, v[j]) : __fadd_rn(v[j], o);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = s_pack_half2(v[2 * j] * p.inv_sqrt_block, v[2 * j + 1] * p.inv_sqrt_block);
            }
            const int t = cl >> 6, piece = ((cl >> 3) & 7) ^ (n & 1);
            if (t < kCapCt)
                s_sts128(kLutWin + static_cast<uint32_t>(n * kCapCt + t) * 256u + 128u + static_cast<uint32_t>(piece) * 16u, h[0],
                         h[1], h[2], h[3]);
        }
    };

    const int first_sidx = s_decode(p, c0).sidx;
    const int last_sidx = s_decode(p, c1 - 1).sidx;
    int staged_sidx = first_sidx;     // slot whose activation (and plane whose table) is in shared memory
    build_table(first_sidx / p.KS);
    // Everything below reads or writes data the preceding kernels produce or still use.
    s_griddep_wait();
    stage_x(first_sidx);
    __syncthreads();

    // ---- partial sums of one segment ----
    // local segment index j (0 = the segment of chunk c0) -> slot j % red_slots, generation j / red_slots
    const ChunkPos first_pos = s_decode(p, c0);
    const int seg_first = first_pos.sidx * p.RT + first_pos.rt;   // global id of local segment 0
    const int n_slots_total = p.KS * p.n_planes;

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    bool dead = false;

    auto flush_segment = [&](int seg) {
        if (p.ablate & 2) {
            if (acc[0] == 123.f) p.y[0] = __float2half_rn(acc[1]);
            return;
        }
        const int j = seg - seg_first;
        const int rs = j % red_slots;
        const uint32_t gen = static_cast<uint32_t>(j / red_slots);
        // wait until the previous user of the slot has been summed
        if (gen > 0) {
            unsigned long long t0 = 0;
            for (uint32_t spin = 0; s_ld_acquire(red_gen + 4u * rs) < gen; ++spin) {
                if ((spin & 31) == 31 && *abort_flag) { dead = true; break; }
                if (spin == 64) t0 = s_timer_ns();
                if (spin > 64 && (spin & 63) == 0 && s_timer_ns() - t0 > kStagedWaitNs) {
                    raise_status(p.status, 5u);
                    atomicExch(&s_abort, 1u);
                    dead = true;
                    break;
                }
            }
        }
        if (dead) return;
        const uint32_t dst = red_base + static_cast<uint32_t>(rs) * kRedSlotBytes + static_cast<uint32_t>(warp) * (kTileFloats * 4u);
        // C fragment: (row g, columns 2q, 2q+1) and (row g+8, same columns); stored [row][BP]
        if (2 * q < BP) {
            s_sts32(dst + static_cast<uint32_t>(g * BP + 2 * q) * 4u, acc[0]);
            s_sts32(dst + static_cast<uint32_t>((g + 8) * BP + 2 * q) * 4u, acc[2]);
            if (2 * q + 1 < BP) {
                s_sts32(dst + static_cast<uint32_t>(g * BP + 2 * q + 1) * 4u, acc[1]);
                s_sts32(dst + static_cast<uint32_t>((g + 8) * BP + 2 * q + 1) * 4u, acc[3]);
            }
        }
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        __syncwarp();
        uint32_t last = 0;
        if (lane == 0) {
            const uint32_t old = s_atom_inc(red_cnt + 4u * rs);
            last = ((old % NW) == NW - 1) ? 1u : 0u;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) return;

        // ---- this warp completes the segment: add the NW tiles in warp order ----
        const int sidx = seg / p.RT, rt = seg - sidx * p.RT;
        const uint32_t src = red_base + static_cast<uint32_t>(rs) * kRedSlotBytes;
        constexpr int kVals = 16 * BP;                       // sums of the segment
        constexpr int kPer = kVals >= 32 ? kVals / 32 : 1;   // sums per lane
        constexpr int kSplit = kVals >= 32 ? 1 : 32 / kVals; // lanes sharing a sum (each takes NW / kSplit warps)
        float v[kPer];
#pragma unroll
        for (int k = 0; k < kPer; ++k) v[k] = 0.f;
        {
            const int e0 = kVals >= 32 ? lane * kPer : lane % kVals;
            const int part = kVals >= 32 ? 0 : lane / kVals;
            constexpr int kWarpsPer = NW / kSplit;
            for (int w = part * kWarpsPer; w < (part + 1) * kWarpsPer; ++w) {
#pragma unroll
                for (int k = 0; k < kPer; ++k)
                    v[k] += s_lds32(src + static_cast<uint32_t>(w * kTileFloats + e0 + k) * 4u);
            }
            if constexpr (kSplit > 1) {
#pragma unroll
                for (int o = kVals; o < 32; o <<= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
            }
        }
        // the slot may be reused
        __syncwarp();
        if (lane == 0) s_st_release(red_gen + 4u * rs, gen + 1u);

        // Is the whole row tile's sum here?  Yes when there is one slot in all and this CTA owns
        // every chunk of the segment.
        const int seg_c0 = s_seg_start(p, sidx, rt);
        const int seg_cps = ((sidx % p.KS) == p.KS - 1) ? p.cps_last : p.cps_full;
        const bool whole = n_slots_total == 1 && seg_c0 >= c0 && seg_c0 + seg_cps <= c1;
        const int e0 = kVals >= 32 ? lane * kPer : lane % kVals;
        const bool writer = kVals >= 32 || lane < kVals;
        if (whole) {
            if (writer) {
#pragma unroll
                for (int k = 0; k < kPer; ++k) {
                    const int e = e0 + k, r = e / BP, n = e - r * BP;
                    const int row = rt * 16 + r;
                    if (row < p.out && n < p.batch)
                        p.y[static_cast<size_t>(n) * p.out + row] = __float2half_rn(v[k] * (__ldg(p.norms + row) * p.inv_scale));
                }
            }
            return;
        }
        // ---- a piece of the row tile: to scratch, then count in; the last piece's writer adds them up ----
        const int own_first = s_owner(seg_c0, p.T, G);
        const int piece = sidx * p.P + (static_cast<int>(blockIdx.x) - own_first);
        float* dstp = p.partial + (static_cast<size_t>(rt) * n_slots_total * p.P + piece) * kVals;
        if (writer) {
#pragma unroll
            for (int k = 0; k < kPer; ++k) dstp[e0 + k] = v[k];
        }
        __threadfence();
        __syncwarp();
        // pieces of this row tile in all
        int expected = 0;
        for (int s = 0; s < n_slots_total; ++s) {
            const int a = s_seg_start(p, s, rt);
            const int cps = ((s % p.KS) == p.KS - 1) ? p.cps_last : p.cps_full;
            expected += s_owner(a + cps - 1, p.T, G) - s_owner(a, p.T, G) + 1;
        }
        uint32_t fin = 0;
        if (lane == 0) {
            const unsigned int prev = atomicAdd(&p.counters[rt], 1u);
            fin = (prev == static_cast<unsigned int>(expected - 1)) ? 1u : 0u;
            if (fin) p.counters[rt] = 0u;   // ready for the next launch
        }
        fin = __shfl_sync(0xffffffffu, fin, 0);
        if (!fin) return;
        __threadfence();
        if (writer) {
#pragma unroll
            for (int k = 0; k < kPer; ++k) {
                const int e = e0 + k, r = e / BP, n = e - r * BP;
                const int row = rt * 16 + r;
                if (row < p.out && n < p.batch) {
                    float total = 0.f;
                    for (int s = 0; s < n_slots_total; ++s) {
                        const int a = s_seg_start(p, s, rt);
                        const int cps = ((s % p.KS) == p.KS - 1) ? p.cps_last : p.cps_full;
                        const int np = s_owner(a + cps - 1, p.T, G) - s_owner(a, p.T, G) + 1;
                        const float* src_p = p.partial + (static_cast<size_t>(rt) * n_slots_total * p.P + s * p.P) * kVals + e;
                        for (int k2 = 0; k2 < np; ++k2) total += __ldcg(src_p + static_cast<size_t>(k2) * kVals);
                    }
                    p.y[static_cast<size_t>(n) * p.out + row] = __float2half_rn(total * (__ldg(p.norms + row) * p.inv_scale));
                }
            }
        }
    };

    // Makes slot `target` the staged one; every warp of the CTA passes through here once per slot change.
    auto restage = [&](int target) {
        while (staged_sidx < target) {
            const int next = staged_sidx + 1;
            asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");   // nobody reads the old activation / table any more
            if (next / p.KS != staged_sidx / p.KS) build_table(next / p.KS);
            stage_x(next);
            asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
            staged_sidx = next;
        }
    };

    // ---- main loop over the group's chunks ----
    int cur_seg = seg_first;
    int m = 0;
    for (int i = grp; i < n_local && !dead; i += NG, ++m) {
        const int seg = cur.sidx * p.RT + cur.rt;
        while (cur_seg < seg && !dead) flush_segment(cur_seg++);
        if (dead) break;
        if (cur.sidx != staged_sidx) restage(cur.sidx);

        const int tile_ct = cur.cc * kChunkTiles + wi;   // column tile inside the slot
        const bool have_tile = tile_ct < cur.width;
        const int slot = grp * D + (m % D);
        // every warp waits for every fill of its group's buffers, tile or not: the phase parity below
        // is only meaningful for a warp that has seen the previous fill complete
        if (!s_mbar_wait(bar_full + 8u * slot, static_cast<uint32_t>(m / D) & 1u, abort_flag)) {
            raise_status(p.status, 4u);
            atomicExch(&s_abort, 1u);
            dead = true;
            break;
        }
        uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
        if (have_tile) {
            const uint32_t src = kRingWin + static_cast<uint32_t>(slot) * kChunkBytes + static_cast<uint32_t>(wi) * kCodeTileBytes +
                                 static_cast<uint32_t>(g * 64 + 16 * q);
            lo = s_lds128(src);
            hi = s_lds128(src + 512u);
        }
        // the buffer is free once all four warps of the group hold their tile in registers
        __syncwarp();
        if (lane == 0) {
            const uint32_t old = s_atom_inc(ring_cnt + 4u * slot);
            if ((old & 3u) == 3u && i + NG * D < n_local) {
                uint32_t bytes;
                const uint8_t* src = chunk_src(ahead, bytes);
                s_bulk_load(kRingWin + static_cast<uint32_t>(slot) * kChunkBytes, src, bytes, bar_full + 8u * slot);
            }
        }
        if (have_tile && (p.ablate & 1)) {
            acc[0] += __uint_as_float((lo.x ^ lo.y ^ lo.z ^ lo.w ^ hi.x ^ hi.y ^ hi.z ^ hi.w) & 0x3f800000u);
        } else if (have_tile) {
            const int n = g & (BP - 1);
            const uint32_t xb = kLutWin + static_cast<uint32_t>(n * kCapCt + tile_ct) * 256u + 128u;
            const uint4 b01 = s_lds128(xb + static_cast<uint32_t>((2 * q) ^ (n & 1)) * 16u);
            const uint4 b23 = s_lds128(xb + static_cast<uint32_t>((2 * q + 1) ^ (n & 1)) * 16u);
            const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
            const uint32_t bw[8] = {b01.x, b01.y, b01.z, b01.w, b23.x, b23.y, b23.z, b23.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t l0 = s_lookup<0>(lw[j], lane_const), l1 = s_lookup<1>(lw[j], lane_const);
                const uint32_t l2 = s_lookup<2>(lw[j], lane_const), l3 = s_lookup<3>(lw[j], lane_const);
                const uint32_t h0 = s_lookup<0>(hw[j], lane_const), h1 = s_lookup<1>(hw[j], lane_const);
                const uint32_t h2 = s_lookup<2>(hw[j], lane_const), h3 = s_lookup<3>(hw[j], lane_const);
                // every entry holds (v, v): low half of the first, high half of the second
                const uint32_t a0 = __byte_perm(l0, l1, 0x7610u), a1 = __byte_perm(h0, h1, 0x7610u);
                const uint32_t a2 = __byte_perm(l2, l3, 0x7610u), a3 = __byte_perm(h2, h3, 0x7610u);
                s_mma_f16(acc, a0, a1, a2, a3, bw[2 * j], bw[2 * j + 1]);
            }
        }
        if (i + NG < n_local) s_advance(p, cur, NG);
        if (i + NG * (D + 1) < n_local) s_advance(p, ahead, NG);
    }
    // segments up to the CTA's last one (a warp may have had no tile in the trailing ones)
    {
        const ChunkPos lastp = s_decode(p, c1 - 1);
        const int seg_last = lastp.sidx * p.RT + lastp.rt;
        while (cur_seg <= seg_last && !dead) {
            // a warp that skipped a slot change still has to take part in it
            const int need = cur_seg / p.RT;
            if (need != staged_sidx && need <= last_sidx) restage(need);
            flush_segment(cur_seg++);
        }
        if (!dead && staged_sidx < last_sidx) restage(last_sidx);
    }
    // A warp that gave up still matches the CTA barriers of the slot changes it has not reached, so
    // that the others can run to their own end (the result is void anyway: the status word is set).
    if (dead) {
        for (; staged_sidx < last_sidx; ++staged_sidx) {
            asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
            asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
        }
    }
}

size_t s_align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct StagedPlan {
    int bp, nw;
    int RT, CT, KS, SCT, cps_full, cps_last, cpp, T, P, grid;
};

// Geometry of a launch.  The grid is one 16-warp CTA per SM while a launch moves little per SM (so
// that the next layer's CTAs can be resident and prefetching), two per SM for large layers.
StagedPlan staged_plan(int out, int in, int batch, int n_planes, int sm_count) {
    StagedPlan s{};
    s.bp = batch <= 1 ? 1 : (batch <= 2 ? 2 : (batch <= 4 ? 4 : 8));
    s.nw = s.bp == 8 ? 32 : 16;
    s.RT = (out + 15) / 16;
    s.CT = static_cast<int>(code_tiles_per_row(in));
    const int cap = 256 / s.bp;
    s.KS = (s.CT + cap - 1) / cap;
    s.SCT = (s.CT + s.KS - 1) / s.KS;                  // equal slots, rounded up to whole chunks
    s.SCT = (s.SCT + kChunkTiles - 1) / kChunkTiles * kChunkTiles;
    if (s.SCT > cap) s.SCT = cap;
    s.KS = (s.CT + s.SCT - 1) / s.SCT;
    s.cps_full = s.SCT / kChunkTiles;
    const int last_w = s.CT - (s.KS - 1) * s.SCT;
    s.cps_last = (last_w + kChunkTiles - 1) / kChunkTiles;
    s.cpp = s.RT * ((s.KS - 1) * s.cps_full + s.cps_last);
    s.T = s.cpp * n_planes;
    int per_sm = s.nw == 16 ? 2 : 1;
    if (s.nw == 16) {
        static const char* env = std::getenv("TQ_GEMV_CTAS_PER_SM");
        const size_t bytes = static_cast<size_t>(s.T) * kChunkBytes;
        if (env != nullptr && (env[0] == '1' || env[0] == '2')) per_sm = env[0] - '0';
        else per_sm = bytes / static_cast<size_t>(sm_count) >= (256u << 10) ? 2 : 1;
    }
    s.grid = sm_count * per_sm;
    if (s.grid > s.T) s.grid = s.T;
    // pieces per (row tile, slot): a segment of cps chunks over ranges of at least T / grid chunks
    const int min_range = s.T / s.grid;
    const int cps_max = s.cps_full > s.cps_last ? s.cps_full : s.cps_last;
    s.P = (cps_max + min_range - 1) / min_range + 1;
    return s;
}

}  // namespace

// Scratch layout: [xrot fp32: n_planes*8*in][counters: RT u32][pieces: RT * slots * P * 16 * BP fp32].
static size_t staged_xrot_bytes(int in, int n_planes) { return s_align256(static_cast<size_t>(n_planes) * 8 * in * sizeof(float)); }
static size_t staged_counter_bytes(int out) { return s_align256(static_cast<size_t>((out + 15) / 16) * sizeof(unsigned int)); }

size_t gemv_staged_scratch_need(int out, int in, int batch, int n_planes, int sm_count) {
    const StagedPlan s = staged_plan(out, in, batch, n_planes, sm_count);
    const size_t pieces = static_cast<size_t>(s.RT) * s.KS * n_planes * s.P * 16 * s.bp * sizeof(float);
    return staged_xrot_bytes(in, n_planes) + staged_counter_bytes(out) + s_align256(pieces);
}

// Enough for any batch of 1..8 rows.
size_t gemv_staged_scratch_bytes(int out, int in, int n_planes, int sm_count) {
    size_t bytes = 0;
    for (int batch : {1, 2, 4, 8}) {
        const size_t b = gemv_staged_scratch_need(out, in, batch, n_planes, sm_count);
        if (b > bytes) bytes = b;
    }
    return bytes;
}

void launch_tq8_gemv_staged(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                            int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                            void* scratch, unsigned int* status, int sm_count, cudaStream_t stream) {
    TQ_REQUIRE(n_planes == 1 || n_planes == 2, "tq8_gemv: one or two rotation planes");
    TQ_REQUIRE(batch >= 1 && batch <= 8, "tq8_gemv handles 1..8 activation rows per launch");
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "WHT block size must be a power of two in [32, 1024]");
    TQ_REQUIRE(in % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    TQ_REQUIRE(scratch != nullptr, "tq8_gemv needs its scratch buffer");
    if (out == 0) return;

    const StagedPlan s = staged_plan(out, in, batch, n_planes, sm_count);
    StagedArgs a{};
    a.codes = codes; a.norms = norms; a.table = table; a.y = y; a.status = status;
    a.out = out; a.in = in; a.batch = batch;
    a.RT = s.RT; a.CT = s.CT; a.KS = s.KS; a.SCT = s.SCT; a.n_planes = n_planes;
    a.cps_full = s.cps_full; a.cps_last = s.cps_last; a.cpp = s.cpp; a.T = s.T; a.P = s.P;
    a.inv_scale = 1.0f / std::sqrt(static_cast<float>(in));
    a.seed_p = seed_p; a.seed_r = seed_r;
    a.block = static_cast<int>(block);
    a.inv_sqrt_block = 1.0f / std::sqrt(static_cast<float>(block));
    {
        static const char* env = std::getenv("TQ_STAGED_ABLATE");
        a.ablate = env ? std::atoi(env) : 0;
    }
    uint8_t* sp = static_cast<uint8_t*>(scratch);
    float* xrot = reinterpret_cast<float*>(sp);
    sp += staged_xrot_bytes(in, n_planes);
    a.counters = reinterpret_cast<unsigned int*>(sp);
    sp += staged_counter_bytes(out);
    a.partial = reinterpret_cast<float*>(sp);
    // Blocks of up to 256 columns are rotated inside the kernel (16-byte activation loads);
    // larger blocks, or an unaligned activation, go through rotate_x_kernel first.
    const bool fused_rotation = block <= 256u && in % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0;
    a.x = x;
    a.xrot = nullptr;
    if (!fused_rotation) {
        launch_rotate_x(x, xrot, in, batch, block, n_planes, seed_p, seed_r, stream);
        a.xrot = xrot;
    }

    static bool configured[64] = {false};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
#define TQ_STAGED_ATTR(BPV, NWV)                                                                                  \
    TQ_CUDA(cudaFuncSetAttribute(tq8_gemv_staged_kernel<BPV, NWV>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 static_cast<int>(StagedCfg<NWV>::kEnd)));
        TQ_STAGED_ATTR(1, 16)
        TQ_STAGED_ATTR(2, 16)
        TQ_STAGED_ATTR(4, 16)
        TQ_STAGED_ATTR(8, 32)
#undef TQ_STAGED_ATTR
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned int>(s.grid));
    cfg.blockDim = dim3(static_cast<unsigned int>(s.nw * 32));
    // The window must reach kEnd.  The dynamic part starts above the window's first kilobyte
    // (reserved and static shared memory come first), so kEnd - 512 bytes reach it; the kernel
    // checks this and refuses to run otherwise.
    cfg.dynamicSmemBytes = s.nw == 16 ? StagedCfg<16>::kEnd - 512u : StagedCfg<32>::kEnd - 512u;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    switch (s.bp) {
        case 1: TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_staged_kernel<1, 16>, a)); break;
        case 2: TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_staged_kernel<2, 16>, a)); break;
        case 4: TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_staged_kernel<4, 16>, a)); break;
        default: TQ_CUDA(cudaLaunchKernelEx(&cfg, tq8_gemv_staged_kernel<8, 32>, a)); break;
    }
}

// Allocation-free variant: the scratch is the library's built-in array (tq_gemv.cu), shared by every
// call on the device.  Only the arrival counters must read zero at kernel start; the kernel re-zeroes
// them on exit, but a call cut short would leave them dirty, so they are cleared here in stream order.
bool gemv_staged_fits_static(int out, int in, int batch, int n_planes, int sm_count) {
    return gemv_staged_scratch_need(out, in, batch, n_planes, sm_count) <= gemv_static_scratch_capacity();
}

void launch_tq8_gemv_staged_static(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                                   int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                                   unsigned int* status, int sm_count, cudaStream_t stream) {
    const size_t need = gemv_staged_scratch_need(out, in, batch, n_planes, sm_count);
    if (need > gemv_static_scratch_capacity())
        throw Error("allocation-free forward: this layer needs " + std::to_string(need) +
                    " bytes of scratch, the built-in array holds " + std::to_string(gemv_static_scratch_capacity()));
    uint8_t* scratch = static_cast<uint8_t*>(gemv_static_scratch_address());
    TQ_CUDA(cudaMemsetAsync(scratch + staged_xrot_bytes(in, n_planes), 0, staged_counter_bytes(out), stream));
    launch_tq8_gemv_staged(codes, norms, table, x, y, out, in, batch, block, n_planes, seed_p, seed_r, scratch, status, sm_count,
                           stream);
}

}  // namespace tq
