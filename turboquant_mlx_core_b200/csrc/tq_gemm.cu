// Fused TQ8 dequantise + GEMM for prefill (tens to thousands of activation rows) on the
// 5th-generation tensor cores: tcgen05.mma with the accumulator in tensor memory.
//
// Replaces, for large batches, the reference's tq_dequant_mm Metal kernel and its host wrapper
// (metal/turboquant_dequant_mm.metal:152-313, src/dequantizer.cpp:606-721):
//   y[m, r] = fp16( norm[r] * sum_j W~[r, j] * fp16(x[m, j]) ),  fp32 accumulate.
//
// Same algebra as the decode kernel: the activation is rotated once (forward WHT of every block
// of every row, written as fp16 by rotate_rows_f16_kernel), and the weight side is a table
// lookup per code:   y[m, r] = norm[r] * inv_scale * sum_j table[code[r, j]] * xrot[m, j].
// Dual-rotation weights run as two passes over K into the same accumulator (primary table
// against x rotated with the primary seed, residual table against x rotated with the residual
// seed).
//
// One CTA computes a 128 (weight rows) x 256 (activation rows, or fewer) tile of y^T:
//   D[128 x 256] (TMEM, fp32) += A[128 x 64] (weights, fp16, TMEM) . B[256 x 64]^T (xrot, fp16, smem)
// per 64-column K block, as four tcgen05.mma (M 128, N 256, K 16) issued by one thread.
//   A pipeline stage is 128 K columns (two 64-column K blocks), the ring has up to four stages.
//   warps 0-15 producers in two groups of eight; group g takes the stages g, g + 2, ...: codes HBM ->
//              registers (two of the group's stages ahead) -> lookup (lane-private fp16 table in
//              shared memory) -> weight tile in TENSOR memory (tcgen05.st; lane = row, 64 columns of
//              fp16 pairs per stage)
//   warp 17    activation tiles: the rotation kernel stores xrot in operand-tile order, so a K block
//              of a tile is one contiguous bulk copy (cp.async.bulk, mbarrier complete_tx) of 128
//              bytes per activation row of the tile
//   warp 16    one thread: waits for a stage (ONE barrier collects the producers' arrivals and the
//              copies' bytes), issues its eight MMAs, commits to the stage's "empty" barrier.  The
//              serial chain of this thread (wait, fence, issue, commit) is what bounds the kernel when
//              the MMAs are short, hence few and long stages.
//   warps 0-15 epilogue: tcgen05.ld the accumulator, scale by norm * inv_scale, store fp16
// The activation tile is as tall as the rows it really has (in steps of 16): a decode batch of 9..64
// rows costs a short MMA and a short copy, so the codes are streamed once whatever the batch.
// The dequantised weights never touch HBM; a weight tile is looked up once per 256 activation
// rows.  Roofline: tensor pipe (2 * M * out * in flops), with the table lookups (one shared-memory
// load per weight per 256 activation rows) as the competing pipe.
//
// Shared-memory layout of the activation operand (K-major, no swizzle): 8 x 8 fp16 core matrices of
// 128 contiguous bytes (8 rows of 16 bytes); core matrices adjacent in K are 128 bytes apart
// (leading byte offset), 8-row groups are 1024 bytes apart (stride byte offset).
//
// Every wait is bounded: a barrier that does not complete within 0.2 s sets the status word and
// an abort flag, after which all warps fall through to the exit path (which still frees the
// tensor memory).
#include <algorithm>
#include <cmath>
#include <cstdint>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

constexpr int kTileRows = 128;  // weight rows per CTA (MMA M)
constexpr int kTileTok = 256;   // activation rows per CTA (MMA N)
constexpr int kBlockK = 64;     // K columns per stage
constexpr int kSubPerStage = 2; // K blocks per pipeline stage: a stage is 128 K columns
constexpr int kStagesMax = 4;   // ring of stages: weight tiles in tensor memory (4 x 64 columns), activation tiles in shared memory (as many as fit)
constexpr int kGroups = 2;      // producer groups of eight warps: group g dequantises the stages g, g + 2, ...
constexpr int kProducerWarps = 8 * kGroups;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kMmaWarp = kProducerWarps;       // issues the MMAs, owns the tensor-memory allocation
constexpr int kCopyWarp = kProducerWarps + 1;  // issues the activation-tile bulk copies
constexpr int kGemmThreads = kProducerThreads + 64;
constexpr uint32_t kLutBytes = 256 * 32 * 4;           // one plane: 256 entries x 32 lane copies x (fp16, fp16)
constexpr uint32_t kTmemCols = 512;   // accumulator: columns 0..255; weight tiles: 4 stages x 64 columns from 256 on
constexpr uint32_t kTmemAColumn = 256;
constexpr uint32_t kTmemASubCols = kBlockK / 2;                    // one K block: two fp16 per 32-bit column
constexpr uint32_t kTmemAStageCols = kSubPerStage * kTmemASubCols;
constexpr uint32_t kLutWin = 0x800u;  // window address of the lookup tables (an immediate of the lookup's load)
// rings + tables (4 activation stages with one table plane, 3 with two) + worst-case padding in
// front of the 32 KB-aligned tables
// Everything an SM can give one CTA: tables at kLutWin, then three 64 KB stages for a 256-row tile.
constexpr size_t kGemmSmemBytes = 232448 - 512;
constexpr unsigned long long kGemmWaitLimitNs = 200ull * 1000 * 1000;

// instruction descriptor: D fp32, A and B fp16, both K-major, M = 128, N = n (a multiple of 16 up to 256)
__host__ __device__ constexpr uint32_t instr_desc(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | (static_cast<uint32_t>(kTileRows >> 4) << 24);
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait; gives up at once when another thread has already flagged a failure.
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile unsigned int* abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spin & 15) == 15 && *abort_flag) return false;
        if (spin == 64) t0 = timer_ns();
        if (spin > 64 && (spin & 63) == 0 && timer_ns() - t0 > kGemmWaitLimitNs) return false;
    }
}

// shared-memory matrix descriptor: K-major, no swizzle, LBO 128 B, SBO 1024 B, descriptor version 1
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(128u >> 4) << 16) |
           (static_cast<uint64_t>(1024u >> 4) << 32) | (1ull << 46);
}

// Table lookup: `offset` = scaled code | lane offset | plane offset; the table's window address is the immediate.
__device__ __forceinline__ uint32_t lut_load(uint32_t offset) {
    uint32_t v;
    asm("ld.shared.b32 %0, [%1 + 2048];" : "=r"(v) : "r"(offset));
    return v;
}
static_assert(kLutWin == 2048u, "lut_load's immediate is the tables' window address");

// D[tmem_d] (+)= A[tmem_a] . B[desc_b]^T : A from tensor memory (128 lanes x 8 columns of fp16 pairs),
// B from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p; }"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// 16 consecutive 32-bit columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
// Waits for this thread's tensor-memory stores and orders them before the barrier arrival that follows.
__device__ __forceinline__ void tmem_st_publish() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
// Arrives on the barrier once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- activation rotation to fp16, written in operand-tile order --------------------------------
// One warp per (plane, row, WHT block): xrot = fp16( FWHT(sign o fp16(x)) / sqrt(bs) ).
// Output layout: [plane][row tile of 256][K block of 64][32 KB tile], the tile being exactly the
// shared-memory image the GEMM wants (8 x 8 core matrices: [row group 32][core column 8][row 8][8 fp16]),
// so that a CTA fetches an activation tile with ONE contiguous bulk copy.  Rows past the last
// one are left as they are: they only feed accumulator columns that are never stored.
template <int E>
__global__ void __launch_bounds__(128) rotate_rows_f16_kernel(const __half* __restrict__ x, __half* __restrict__ xrot,
                                                              int in, long rows, int n_planes, uint32_t seed_p,
                                                              uint32_t seed_r, float inv_sqrt) {
    pdl_wait_release();   // x, and the scratch this kernel overwrites, belong to the kernels before it until they are done
    constexpr int BS = 32 * E;
    constexpr int V = E < 8 ? E : 8;  // halves per vector store (one core-matrix row holds 8)
    const int lane = threadIdx.x & 31;
    const long blocks_per_row = in / BS;
    const long total = static_cast<long>(n_planes) * rows * blocks_per_row;
    const long warp = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (warp >= total) return;
    // consecutive warps take consecutive rows of the same block: their stores fill whole lines
    const int plane = static_cast<int>(warp / (rows * blocks_per_row));
    const long rem = warp - static_cast<long>(plane) * rows * blocks_per_row;
    const long blk = rem / rows, row = rem - blk * rows;
    const uint32_t seed = plane ? seed_r : seed_p;
    const __half* src = x + row * in + blk * BS + lane * E;
    float v[E];
#pragma unroll
    for (int j = 0; j < E; ++j) v[j] = __half2float(src[j]) * sign_value(seed, static_cast<uint32_t>(lane * E + j));
    warp_fwht<E>(v, lane);
    const long n_row_tiles = (rows + kTileTok - 1) / kTileTok;
    const long kb_per_plane = in / kBlockK;
    const long rt = row / kTileTok, rin = row - rt * kTileTok;
#pragma unroll
    for (int j0 = 0; j0 < E; j0 += V) {
        const long col = blk * BS + lane * E + j0;
        const long kb = col / kBlockK, cin = col - kb * kBlockK;
        const long tile = (static_cast<long>(plane) * n_row_tiles + rt) * kb_per_plane + kb;
        __half* dst = xrot + tile * (kTileTok * kBlockK) + (((rin >> 3) * 8 + (cin >> 3)) * 8 + (rin & 7)) * 8 + (cin & 7);
        __align__(16) __half h[V];
#pragma unroll
        for (int j = 0; j < V; ++j) h[j] = __float2half_rn(v[j0 + j] * inv_sqrt);
        if constexpr (V == 8) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(h);
        else if constexpr (V == 4) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(h);
        else if constexpr (V == 2) *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(h);
        else dst[0] = h[0];
    }
}

// The same for WHT blocks of up to 256 columns, with 16-byte accesses: a warp takes 256 columns
// of one row, lane l the 8 columns 8l..8l+7 (one core-matrix row of the output tile); butterfly
// stages below 8 stay in the lane, the rest are lane exchanges (the add tree of warp_fwht).  The
// 8 warps of a CTA take 8 consecutive rows, so their stores complete whole 128-byte core matrices.
__device__ __forceinline__ void rotate_rows_wide_body(const __half* __restrict__ x, __half* __restrict__ xrot, int in, long rows,
                                                      int n_planes, int block, uint32_t seed_p, uint32_t seed_r, float inv_sqrt) {
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long groups_per_row = (in + 255) / 256;
    const long row_groups = (rows + 7) / 8;
    // blockIdx.x -> (plane, column group, group of 8 rows); warp -> row inside the group
    long b = blockIdx.x;
    const long rg = b % row_groups;
    b /= row_groups;
    const long cg = b % groups_per_row;
    const int plane = static_cast<int>(b / groups_per_row);
    if (plane >= n_planes) return;
    const long row = rg * 8 + wib;
    const int col = static_cast<int>(cg) * 256 + 8 * lane;
    if (row >= rows || col >= in) return;  // in is a multiple of 32 >= block: whole lanes only; exchanges stay inside a block
    const uint32_t seed = plane ? seed_r : seed_p;
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + row * in + col));
    const uint32_t xw[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half2 h2 = *reinterpret_cast<const __half2*>(&xw[j]);
        v[2 * j] = __low2float(h2) * sign_value(seed, static_cast<uint32_t>((col + 2 * j) & (block - 1)));
        v[2 * j + 1] = __high2float(h2) * sign_value(seed, static_cast<uint32_t>((col + 2 * j + 1) & (block - 1)));
    }
#pragma unroll
    for (int h = 1; h < 8; h <<= 1)
#pragma unroll
        for (int i = 0; i < 8; i += 2 * h)
#pragma unroll
            for (int j = i; j < i + h; ++j) {
                const float a0 = v[j], b0 = v[j + h];
                v[j] = __fadd_rn(a0, b0);
                v[j + h] = __fsub_rn(a0, b0);
            }
    // lanes of an incomplete trailing group (in % 256 != 0) have returned: exchange only among the live ones
    const unsigned live = __activemask();
    for (int m = 1; m < (block >> 3); m <<= 1) {
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float o = __shfl_xor_sync(live, v[j], m);
            v[j] = upper ? __fsub_rn(o, v[j]) : __fadd_rn(v[j], o);
        }
    }
    const long n_row_tiles = (rows + kTileTok - 1) / kTileTok;
    const long kb_per_plane = in / kBlockK;
    const long rt = row / kTileTok, rin = row - rt * kTileTok;
    const long kb = col / kBlockK, cin = col - kb * kBlockK;
    const long tile = (static_cast<long>(plane) * n_row_tiles + rt) * kb_per_plane + kb;
    __half* dst = xrot + tile * (kTileTok * kBlockK) + (((rin >> 3) * 8 + (cin >> 3)) * 8 + (rin & 7)) * 8;
    __align__(16) __half hv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) hv[j] = __float2half_rn(v[j] * inv_sqrt);
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(hv);
}
__global__ void __launch_bounds__(256) rotate_rows_f16_wide_kernel(const __half* __restrict__ x, __half* __restrict__ xrot,
                                                                   int in, long rows, int n_planes, int block,
                                                                   uint32_t seed_p, uint32_t seed_r, float inv_sqrt) {
    pdl_wait_release();   // x, and the scratch this kernel overwrites, belong to the kernels before it until they are done
    rotate_rows_wide_body(x, xrot, in, rows, n_planes, block, seed_p, seed_r, inv_sqrt);
}
// The same rows rotated for several matrices at once (their own seeds and destinations): blockIdx.y = matrix.
struct RotateGroupArgs {
    __half* xrot[4];
    uint32_t seed_p[4], seed_r[4];
};
__global__ void __launch_bounds__(256) rotate_rows_f16_wide_group_kernel(const __half* __restrict__ x, const RotateGroupArgs g, int in,
                                                                         long rows, int n_planes, int block, float inv_sqrt) {
    pdl_wait_release();
    rotate_rows_wide_body(x, g.xrot[blockIdx.y], in, rows, n_planes, block, g.seed_p[blockIdx.y], g.seed_r[blockIdx.y], inv_sqrt);
}

struct GemmArgs {
    const uint8_t* codes;   // joint bytes in 16 x 64 tiles (code_offset)
    const float* norms;     // [out]
    const float* table;     // [n_planes, 256] fp32
    const __half* xrot;     // rotated activation in operand-tile order (see rotate_rows_f16_kernel)
    __half* y;              // [m, out], activation rows y_stride elements apart
    long y_stride;
    float* partial;         // [k_splits, m, out] fp32 un-scaled partial sums (only when k_splits > 1)
    unsigned int* status;   // device error word (0 = ok)
    int out, in, m, n_planes;
    int k_splits;           // CTAs along K per output tile (gridDim.z)
    float inv_scale;
};

// One CTA's work: output tile (row tile bx, token tile blockIdx.y), K split bz of matrix p.
__device__ __forceinline__ void gemm_body(const GemmArgs& p, const int bx, const int bz) {
    extern __shared__ __align__(128) uint8_t gemm_smem[];
    __shared__ __align__(8) unsigned long long s_full[kStagesMax], s_empty[kStagesMax], s_accum;
    __shared__ uint32_t s_tmem_base;
    __shared__ unsigned int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = bx * kTileRows;  // first weight row of the tile
    const int tok0 = blockIdx.y * kTileTok;   // first activation row of the tile
    // Activation rows this tile really has, rounded up to the MMA's granularity of 16: a short tile
    // (a decode batch of 9..64 rows, or the tail of a prefill) costs a short MMA and a short copy.
    const int n_tile = min(kTileTok, ((p.m - tok0) + 15) & ~15);
    const uint32_t b_bytes = static_cast<uint32_t>(n_tile) * (kBlockK * 2);   // one 64-column piece: the tile's first n_tile rows are contiguous
    const uint32_t idesc = instr_desc(static_cast<uint32_t>(n_tile));

    // ---- shared-memory map -------------------------------------------------------------------
    // [kLutWin, + 32 KB per plane)  lookup tables, at a fixed window address (it is an immediate of
    //                               the lookup's load instruction)
    // [after the tables, end)       activation stages of 2 * b_bytes (two 64-column pieces), as many
    //                               as fit, at most kStagesMax
    const uint32_t raw = smem_addr(gemm_smem);
    uint32_t dyn_bytes;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    const uint32_t stage0 = kLutWin + kLutBytes * static_cast<uint32_t>(p.n_planes);
    const uint32_t stage_bytes = kSubPerStage * b_bytes;
    const uint32_t smem_end = raw + dyn_bytes;
    int n_st = smem_end > stage0 ? static_cast<int>((smem_end - stage0) / stage_bytes) : 0;
    if (n_st > kStagesMax) n_st = kStagesMax;
    if (raw > kLutWin || n_st < 2) {  // layout does not fit: refuse to run (nothing allocated yet)
        if (tid == 0) raise_status(p.status, 9u);
        return;
    }
    const uint32_t bar_full = smem_addr(&s_full[0]), bar_empty = smem_addr(&s_empty[0]), bar_accum = smem_addr(&s_accum);

    if (tid == 0) {
        for (int s = 0; s < kStagesMax; ++s) {
            bar_init(bar_full + 8u * s, kProducerWarps / kGroups + 1);   // one arrival per producer warp of the group + the copy thread
            bar_init(bar_empty + 8u * s, 1);
        }
        bar_init(bar_accum, 1);
        s_abort = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&s_tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // lookup tables: entry e, lane copy l at kLutWin + plane * 32 KB + e * 128 + l * 4, value (t, t) as fp16
    for (int i = tid; i < 256 * 8 * p.n_planes; i += kGemmThreads) {
        const int e = i >> 3, c4 = (i & 7) * 4;  // e counts across planes
        const __half h = __float2half_rn(__ldg(p.table + e));
        const uint32_t v = static_cast<uint32_t>(__half_as_ushort(h)) * 0x00010001u;
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(kLutWin + static_cast<uint32_t>(e) * 128u + c4 * 4u), "r"(v)
                     : "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = s_tmem_base;
    volatile unsigned int* abort_flag = &s_abort;

    // K blocks (64 columns) of this CTA: a contiguous range of the (plane-major) list of all K blocks.
    // A stage is two consecutive K blocks of the range (the last one may hold a single block).
    const int kb_per_plane = p.in / kBlockK;
    const int n_kb_total = kb_per_plane * p.n_planes;
    const int kb_base = static_cast<int>(static_cast<long>(n_kb_total) * bz / p.k_splits);
    const int n_kb = static_cast<int>(static_cast<long>(n_kb_total) * (bz + 1) / p.k_splits) - kb_base;
    const int n_it = (n_kb + kSubPerStage - 1) / kSubPerStage;

    if (warp < kProducerWarps) {
        // ---- producers ------------------------------------------------------------------------
        // Weight tile in tensor memory: lane = row of the tile, 64 columns per stage (two fp16 per
        // column, 128 K columns).  A warp may touch lanes 32 * (warp % 4) .. + 31.  The 16 producer
        // warps form two groups of eight (warp / 8); inside a group warp w takes the rows of lane
        // quarter w % 4 and the K block (w / 4) % 2 of the stage; group g dequantises the stages g,
        // g + 2, ...  A thread turns the 64 codes of its row and K block into 32 columns.
        const int ar = 32 * (warp & 3) + lane;       // row inside the tile
        const int sub = (warp >> 2) & 1;             // which K block of the stage
        const int grp = warp >> 3;
        const int grow = min(row0 + ar, p.out - 1);  // rows past the matrix repeat the last row (never stored)
        // a row's 64 columns of K block kb are 64 contiguous bytes of code tile (row / 16, kb)
        const uint8_t* code_ptr = p.codes + code_offset(grow, 0, code_tiles_per_row(p.in));
        const uint32_t a_taddr = tmem_d + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + kTmemAColumn + kTmemASubCols * static_cast<uint32_t>(sub);

        // Codes are fetched two of the group's stages ahead into registers.  The second plane reads
        // the same bytes again.
        auto load_codes = [&](int it, uint4 (&c)[4]) {
            const int kb = kSubPerStage * it + sub;
            if (kb < n_kb) {
                const int plane = (kb_base + kb) >= kb_per_plane ? 1 : 0;
                const uint4* src = reinterpret_cast<const uint4*>(
                    code_ptr + static_cast<size_t>(kb_base + kb - plane * kb_per_plane) * kCodeTileBytes);
#pragma unroll
                for (int i = 0; i < 4; ++i) c[i] = __ldg(src + i);
            }
        };
        uint4 c0[4], c1[4], c2[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) c0[i] = c1[i] = c2[i] = make_uint4(0, 0, 0, 0);
        load_codes(grp, c0);
        load_codes(grp + kGroups, c1);
        int slot = grp % n_st, use = grp / n_st;     // ring slot of stage `it` and how often it has been used before
        bool alive = true;
        for (int it = grp; alive && it < n_it; it += kGroups) {
            load_codes(it + 2 * kGroups, c2);
            const int kb = kSubPerStage * it + sub;
            const bool have = kb < n_kb;             // the last stage may lack its second K block
            const int plane = (kb_base + kb) >= kb_per_plane ? 1 : 0;
            // lane offset, plus 32 KB for the second plane's table: bits outside the scaled code (7..14)
            const uint32_t lane_c = static_cast<uint32_t>(lane) * 4u + static_cast<uint32_t>(plane) * kLutBytes;
            const uint32_t st_addr = a_taddr + kTmemAStageCols * static_cast<uint32_t>(slot);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                // 32 codes -> 32 fp16 -> 16 tensor-memory columns of this thread's lane
                const uint32_t w[8] = {c0[2 * half].x, c0[2 * half].y, c0[2 * half].z, c0[2 * half].w,
                                       c0[2 * half + 1].x, c0[2 * half + 1].y, c0[2 * half + 1].z, c0[2 * half + 1].w};
                uint32_t packed[16];
#pragma unroll
                for (int h = 0; h < 16; ++h) {  // codes 2h, 2h + 1 -> column h
                    const uint32_t word = w[h >> 1];
                    const int b0 = (h & 1) * 2;  // bytes b0, b0 + 1 of the word
                    const uint32_t i0 = b0 == 0 ? (word << 7) : (word >> 9);
                    const uint32_t i1 = b0 == 0 ? (word >> 1) : (word >> 17);
                    packed[h] = __byte_perm(lut_load((i0 & (255u << 7)) | lane_c), lut_load((i1 & (255u << 7)) | lane_c), 0x5410);
                }
                // the slot must have been read by the MMAs of its previous stage
                if (half == 0 && use > 0 && !bar_wait(bar_empty + 8u * slot, static_cast<uint32_t>(use - 1) & 1u, abort_flag)) {
                    raise_status(p.status, 6u);
                    atomicExch(&s_abort, 1u);
                    alive = false;
                }
                if (!alive) break;
                if (have) tmem_st16(st_addr + 16u * half, packed);
            }
            if (!alive) break;
            // every lane waits for its own stores, then one arrival per warp
            tmem_st_publish();
            __syncwarp();
            if (lane == 0) bar_arrive(bar_full + 8u * slot);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                c0[i] = c1[i];
                c1[i] = c2[i];
            }
            slot += kGroups;
            if (slot >= n_st) { slot -= n_st; ++use; }
        }
    } else if (warp == kCopyWarp) {
        // ---- activation tiles: one bulk copy per K block of the stage, as far ahead as the ring allows ----
        // One thread runs the whole loop; ring slot and phase are kept incrementally (no divisions on
        // this serial path).
        if (lane == 0) {
            // The rotated activations are the only input the kernel before this one produces (launched with the
            // programmatic-dependency attribute, the CTA has set up its barriers, tensor memory and tables and the
            // producers are already streaming codes meanwhile): wait for that kernel here.
            asm volatile("griddepcontrol.wait;" ::: "memory");
            const size_t n_tok_tiles = (static_cast<size_t>(p.m) + kTileTok - 1) / kTileTok;
            int slot = 0;
            uint32_t par = 1u;   // parity of the "empty" phase to wait for
            for (int it = 0; it < n_it; ++it) {
                if (it >= n_st && !bar_wait(bar_empty + 8u * slot, par, abort_flag)) {
                    raise_status(p.status, 6u);
                    atomicExch(&s_abort, 1u);
                    break;
                }
                const int nsub = min(kSubPerStage, n_kb - kSubPerStage * it);
                const uint32_t bar = bar_full + 8u * slot;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(b_bytes * nsub) : "memory");
                for (int sb = 0; sb < nsub; ++sb) {
                    const int kb = kSubPerStage * it + sb;
                    const int plane = (kb_base + kb) >= kb_per_plane ? 1 : 0;
                    const size_t tile = (static_cast<size_t>(plane) * n_tok_tiles + blockIdx.y) * kb_per_plane + (kb_base + kb - plane * kb_per_plane);
                    const __half* src = p.xrot + tile * (kTileTok * kBlockK);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                     stage0 + static_cast<uint32_t>(slot) * stage_bytes + static_cast<uint32_t>(sb) * b_bytes),
                                 "l"(src), "r"(b_bytes), "r"(bar)
                                 : "memory");
                }
                if (++slot == n_st) { slot = 0; par ^= 1u; }
            }
            // every activation tile of this CTA is on its way: the kernel after this one may start setting up
            asm volatile("griddepcontrol.launch_dependents;");
        }
        __syncwarp();
    } else {
        // ---- MMA issuer (one thread): one wait and one commit per stage ---------------------------------
        if (lane == 0) {
            int slot = 0;
            uint32_t par = 0u;
            bool ok = true;
            for (int it = 0; it < n_it; ++it) {
                if (!bar_wait(bar_full + 8u * slot, par, abort_flag)) {
                    raise_status(p.status, 7u);
                    atomicExch(&s_abort, 1u);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int nsub = min(kSubPerStage, n_kb - kSubPerStage * it);
                const uint32_t a_tmem = tmem_d + kTmemAColumn + kTmemAStageCols * static_cast<uint32_t>(slot);
                const uint32_t b_stage = stage0 + static_cast<uint32_t>(slot) * stage_bytes;
#pragma unroll
                for (int sb = 0; sb < kSubPerStage; ++sb) {
                    if (sb < nsub) {
                        const uint64_t desc0 = smem_desc(b_stage + static_cast<uint32_t>(sb) * b_bytes);
#pragma unroll
                        for (int j = 0; j < kBlockK / 16; ++j)   // 256 bytes further along K per step: +16 in the address field
                            umma_f16_ts(tmem_d, a_tmem + kTmemASubCols * sb + 8u * j, desc0 + static_cast<uint64_t>(16 * j), idesc,
                                        (it | sb | j) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(bar_empty + 8u * slot);   // the slot (weights and activation) may be refilled once these MMAs are done
                if (++slot == n_st) { slot = 0; par ^= 1u; }
            }
            if (ok) umma_commit(bar_accum);
        }
        __syncwarp();
    }

    // ---- epilogue (the producer warps): TMEM lanes 32 * (warp & 3), columns 64 * (warp >> 2) .. +63 ----
    if (warp < kProducerWarps) {
        const bool ok = !*abort_flag && bar_wait(bar_accum, 0, abort_flag);
        if (!ok) {
            raise_status(p.status, 8u);
            atomicExch(&s_abort, 1u);
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int r = row0 + 32 * (warp & 3) + lane;
            const bool r_ok = r < p.out;
            const float scale = r_ok ? __ldg(p.norms + r) * p.inv_scale : 0.f;
#pragma unroll 1
            for (int cb = 0; cb < 2; ++cb) {
                const int col0 = 64 * (warp >> 2) + 32 * cb;
                if (col0 >= n_tile) break;   // warp-uniform: columns the MMA never wrote
                uint32_t v[32];
                tmem_ld32(tmem_d + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + static_cast<uint32_t>(col0), v);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int tok = tok0 + col0 + j;
                    if (r_ok && tok < p.m) {
                        if (p.k_splits == 1) p.y[static_cast<size_t>(tok) * p.y_stride + r] = __float2half_rn(__uint_as_float(v[j]) * scale);
                        else p.partial[(static_cast<size_t>(bz) * p.m + tok) * p.out + r] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kTmemCols) : "memory");
    }
}

__global__ void __launch_bounds__(kGemmThreads, 1) tq8_gemm_kernel(const GemmArgs p) {
    gemm_body(p, static_cast<int>(blockIdx.x), static_cast<int>(blockIdx.z));
}

// Several matrices that multiply the same activation rows (q / k / v, gate / up) in one launch: gridDim.x is cut into
// one range of row tiles per matrix, gridDim.z is the largest K split of the group (CTAs beyond a matrix's own split
// count leave at once).  Every matrix brings its own rotated activations (its own seeds), scratch and status word.
constexpr int kMaxGemmGroup = 4;
struct GemmGroupArgs {
    GemmArgs m[kMaxGemmGroup];
    int tile_start[kMaxGemmGroup + 1];   // row tiles tile_start[i] .. tile_start[i + 1] - 1 belong to matrix i
    int n;
};
__global__ void __launch_bounds__(kGemmThreads, 1) tq8_gemm_group_kernel(const __grid_constant__ GemmGroupArgs grp) {
    const int b = static_cast<int>(blockIdx.x);
    int i = 0;
    while (i + 1 < grp.n && b >= grp.tile_start[i + 1]) ++i;
    if (static_cast<int>(blockIdx.z) >= grp.m[i].k_splits) return;
    gemm_body(grp.m[i], b - grp.tile_start[i], static_cast<int>(blockIdx.z));
}

// y = fp16(norm * inv_scale * sum over K splits, in split order) — fixed order, run-to-run identical.
__global__ void __launch_bounds__(256) gemm_finish_kernel(const float* __restrict__ partial, const float* __restrict__ norms,
                                                          __half* __restrict__ y, long y_stride, long m, int out, int k_splits,
                                                          float inv_scale) {
    pdl_wait_release();
    const long n = m * out;
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
        float acc = 0.f;
        for (int z = 0; z < k_splits; ++z) acc += partial[static_cast<long>(z) * n + i];
        y[(i / out) * y_stride + i % out] = __float2half_rn(acc * (__ldg(norms + i % out) * inv_scale));
    }
}

// The split-K finish of a group: blockIdx.y = matrix (matrices without a split have nothing to finish).
struct FinishGroupArgs {
    const float* partial[4];
    const float* norms[4];
    __half* y[4];
    long y_stride[4];
    int out[4], k_splits[4];
    float inv_scale[4];
};
__global__ void __launch_bounds__(256) gemm_finish_group_kernel(const FinishGroupArgs g, long m) {
    pdl_wait_release();
    const int i = blockIdx.y;
    const int k_splits = g.k_splits[i], out = g.out[i];
    if (k_splits <= 1) return;
    const float* __restrict__ partial = g.partial[i];
    const float* __restrict__ norms = g.norms[i];
    __half* __restrict__ y = g.y[i];
    const long n = m * out;
    for (long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; e < n; e += static_cast<long>(gridDim.x) * blockDim.x) {
        float acc = 0.f;
        for (int z = 0; z < k_splits; ++z) acc += partial[static_cast<long>(z) * n + e];
        y[(e / out) * g.y_stride[i] + e % out] = __float2half_rn(acc * (__ldg(norms + e % out) * g.inv_scale[i]));
    }
}

size_t xrot_bytes(int in, long m, int n_planes) {
    const size_t padded = (static_cast<size_t>(m) + kTileTok - 1) / kTileTok * kTileTok;  // whole operand tiles
    return (static_cast<size_t>(n_planes) * padded * static_cast<size_t>(in) * sizeof(__half) + 255) & ~static_cast<size_t>(255);
}

}  // namespace

// When the output has too few tiles to occupy the SMs (few activation rows on a matrix with few
// rows and many columns), K is split over several CTAs per tile; every split keeps at least 8 K blocks.
int gemm_k_splits(int out, int in, long m, int n_planes, int sm_count) {
    const long tiles = static_cast<long>((out + kTileRows - 1) / kTileRows) * ((m + kTileTok - 1) / kTileTok);
    const int n_kb = in / kBlockK * n_planes;
    long s = sm_count / (tiles > 0 ? tiles : 1);
    if (s > n_kb / 8) s = n_kb / 8;
    return s < 1 ? 1 : static_cast<int>(s);
}

size_t gemm_scratch_bytes(int out, int in, long m, int n_planes, int sm_count) {
    const int splits = gemm_k_splits(out, in, m, n_planes, sm_count);
    size_t bytes = xrot_bytes(in, m, n_planes);
    if (splits > 1) bytes += static_cast<size_t>(splits) * static_cast<size_t>(m) * out * sizeof(float);
    return bytes;
}

bool gemm_supported(int in) { return in % kBlockK == 0; }

void launch_tq8_gemm(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y, int out,
                     int in, long m, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r, void* scratch,
                     unsigned int* status, int sm_count, cudaStream_t stream, long y_stride) {
    if (y_stride <= 0) y_stride = out;
    TQ_REQUIRE(y_stride >= out, "tq8_gemm: output row stride smaller than the layer's rows");
    TQ_REQUIRE(n_planes == 1 || n_planes == 2, "tq8_gemm: one or two rotation planes");
    TQ_REQUIRE(gemm_supported(in), "tq8_gemm: in_features must be a multiple of 64");
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "WHT block size must be a power of two in [32, 1024]");
    TQ_REQUIRE(in % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    TQ_REQUIRE(m >= 1 && m < (1L << 30), "tq8_gemm: bad number of activation rows");
    TQ_REQUIRE(scratch != nullptr, "tq8_gemm needs its scratch buffer");
    if (out == 0) return;
    __half* xrot = static_cast<__half*>(scratch);

    // 1. rotate every activation row (one warp per plane x row x block)
    {
        const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(block));
        const long n_warps = static_cast<long>(n_planes) * m * (in / static_cast<int>(block));
        const unsigned int grid = static_cast<unsigned int>((n_warps + 3) / 4);
        const long wide_blocks = static_cast<long>(n_planes) * ((in + 255) / 256) * ((m + 7) / 8);
        if (block <= 256 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && wide_blocks < (1L << 31)) {
            launch_pdl(rotate_rows_f16_wide_kernel, dim3(static_cast<unsigned int>(wide_blocks)), dim3(256), 0, stream, x, xrot, in, m,
                       n_planes, static_cast<int>(block), seed_p, seed_r, inv_sqrt);
        } else
#define TQ_ROT16_CASE(EV)                                                                                          \
    case 32 * EV:                                                                                                  \
        launch_pdl(rotate_rows_f16_kernel<EV>, dim3(grid), dim3(128), 0, stream, x, xrot, in, m, n_planes, seed_p, seed_r, inv_sqrt); \
        break;
        switch (block) {
            TQ_ROT16_CASE(1) TQ_ROT16_CASE(2) TQ_ROT16_CASE(4) TQ_ROT16_CASE(8) TQ_ROT16_CASE(16) TQ_ROT16_CASE(32)
            default: throw Error("unsupported WHT block size");
        }
#undef TQ_ROT16_CASE
        TQ_CUDA(cudaGetLastError());
    }
    // 2. the GEMM
    GemmArgs a{};
    a.codes = codes; a.norms = norms; a.table = table; a.xrot = xrot; a.y = y; a.y_stride = y_stride; a.status = status;
    a.out = out; a.in = in; a.m = static_cast<int>(m); a.n_planes = n_planes;
    a.inv_scale = 1.0f / std::sqrt(static_cast<float>(in));
    a.k_splits = gemm_k_splits(out, in, m, n_planes, sm_count);
    a.partial = a.k_splits > 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + xrot_bytes(in, m, n_planes)) : nullptr;
    // stages + tables + worst-case padding in front of the 32 KB-aligned tables
    const size_t smem = kGemmSmemBytes;
    static bool configured[64] = {false};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(tq8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kGemmSmemBytes)));
        if (dev < 64) configured[dev] = true;
    }
    const dim3 grid(static_cast<unsigned int>((out + kTileRows - 1) / kTileRows),
                    static_cast<unsigned int>((m + kTileTok - 1) / kTileTok), static_cast<unsigned int>(a.k_splits));
    launch_pdl(tq8_gemm_kernel, grid, dim3(kGemmThreads), smem, stream, a);
    TQ_CUDA(cudaGetLastError());
    if (a.k_splits > 1) {
        const long n = m * out;
        const unsigned int blocks = static_cast<unsigned int>(std::min<long>((n + 255) / 256, 148L * 8));
        launch_pdl(gemm_finish_kernel, dim3(blocks), dim3(256), 0, stream, a.partial, norms, y, y_stride, m, out, a.k_splits, a.inv_scale);
        TQ_CUDA(cudaGetLastError());
    }
}

void launch_tq8_gemm_group(const GemmGroupItem* items, int n, const __half* x, long m, int sm_count, cudaStream_t stream) {
    TQ_REQUIRE(items != nullptr && n >= 1 && n <= kMaxGemmGroup, "tq8_gemm group: 1..4 matrices");
    TQ_REQUIRE(x != nullptr && m >= 1 && m < (1L << 30), "tq8_gemm group: bad number of activation rows");
    const int in = items[0].in, n_planes = items[0].n_planes;
    const uint32_t block = items[0].block;
    TQ_REQUIRE(n_planes == 1 || n_planes == 2, "tq8_gemm: one or two rotation planes");
    TQ_REQUIRE(gemm_supported(in), "tq8_gemm: in_features must be a multiple of 64");
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "WHT block size must be a power of two in [32, 1024]");
    TQ_REQUIRE(in % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    GemmGroupArgs grp{};
    RotateGroupArgs rot{};
    FinishGroupArgs fin{};
    grp.n = n;
    grp.tile_start[0] = 0;
    int max_splits = 1;
    bool any_split = false;
    for (int i = 0; i < n; ++i) {
        const GemmGroupItem& it = items[i];
        TQ_REQUIRE(it.codes && it.norms && it.table && it.y && it.scratch && it.out >= 1, "tq8_gemm group: NULL argument");
        TQ_REQUIRE(it.in == in && it.n_planes == n_planes && it.block == block,
                   "tq8_gemm group: the matrices must share in_features, the WHT block and the rotation mode");
        GemmArgs& a = grp.m[i];
        a.codes = it.codes; a.norms = it.norms; a.table = it.table; a.y = it.y; a.y_stride = it.out; a.status = it.status;
        a.xrot = static_cast<__half*>(it.scratch);
        a.out = it.out; a.in = in; a.m = static_cast<int>(m); a.n_planes = n_planes;
        a.inv_scale = 1.0f / std::sqrt(static_cast<float>(in));
        // the split a matrix would get alone, not one for the group as a whole: with fewer splits the group ran 7-9 %
        // faster (16 / 64 rows) but the fp32 sums changed their order, and results would no longer be bit-equal to
        // separate calls
        a.k_splits = gemm_k_splits(it.out, in, m, n_planes, sm_count);
        a.partial = a.k_splits > 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(it.scratch) + xrot_bytes(in, m, n_planes)) : nullptr;
        grp.tile_start[i + 1] = grp.tile_start[i] + (it.out + kTileRows - 1) / kTileRows;
        max_splits = std::max(max_splits, a.k_splits);
        any_split = any_split || a.k_splits > 1;
        rot.xrot[i] = static_cast<__half*>(it.scratch);
        rot.seed_p[i] = it.seed_p; rot.seed_r[i] = it.seed_r;
        fin.partial[i] = a.partial; fin.norms[i] = it.norms; fin.y[i] = it.y; fin.y_stride[i] = it.out; fin.out[i] = it.out;
        fin.k_splits[i] = a.k_splits; fin.inv_scale[i] = a.inv_scale;
    }
    for (int i = n; i < kMaxGemmGroup; ++i) grp.tile_start[i + 1] = grp.tile_start[n];
    // 1. the rotations: one launch for the group where the wide kernel applies
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(block));
    const long wide_blocks = static_cast<long>(n_planes) * ((in + 255) / 256) * ((m + 7) / 8);
    if (block <= 256 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && wide_blocks < (1L << 31)) {
        launch_pdl(rotate_rows_f16_wide_group_kernel, dim3(static_cast<unsigned int>(wide_blocks), static_cast<unsigned int>(n)), dim3(256), 0,
                   stream, x, rot, in, m, n_planes, static_cast<int>(block), inv_sqrt);
    } else {
        const long n_warps = static_cast<long>(n_planes) * m * (in / static_cast<int>(block));
        const unsigned int grid = static_cast<unsigned int>((n_warps + 3) / 4);
        for (int i = 0; i < n; ++i) {
#define TQ_ROT16G_CASE(EV)                                                                                                              \
    case 32 * EV:                                                                                                                       \
        launch_pdl(rotate_rows_f16_kernel<EV>, dim3(grid), dim3(128), 0, stream, x, rot.xrot[i], in, m, n_planes, rot.seed_p[i], rot.seed_r[i], \
                   inv_sqrt);                                                                                                           \
        break;
            switch (block) {
                TQ_ROT16G_CASE(1) TQ_ROT16G_CASE(2) TQ_ROT16G_CASE(4) TQ_ROT16G_CASE(8) TQ_ROT16G_CASE(16) TQ_ROT16G_CASE(32)
                default: throw Error("unsupported WHT block size");
            }
#undef TQ_ROT16G_CASE
        }
    }
    // 2. the GEMMs
    static bool configured[64] = {false};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(tq8_gemm_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemmSmemBytes)));
        if (dev < 64) configured[dev] = true;
    }
    const dim3 grid(static_cast<unsigned int>(grp.tile_start[n]), static_cast<unsigned int>((m + kTileTok - 1) / kTileTok),
                    static_cast<unsigned int>(max_splits));
    launch_pdl(tq8_gemm_group_kernel, grid, dim3(kGemmThreads), kGemmSmemBytes, stream, grp);
    // 3. the split-K sums
    if (any_split) {
        long biggest = 0;
        for (int i = 0; i < n; ++i) if (fin.k_splits[i] > 1) biggest = std::max<long>(biggest, m * fin.out[i]);
        const unsigned int blocks = static_cast<unsigned int>(std::min<long>((biggest + 255) / 256, 148L * 8));
        launch_pdl(gemm_finish_group_kernel, dim3(blocks, static_cast<unsigned int>(n)), dim3(256), 0, stream, fin, m);
    }
}

}  // namespace tq
