// Decode attention over the compressed KV cache on the 5th-generation tensor cores
// (head_dim 128, four KV heads, up to eight query heads per KV head and CTA).
//
// A tile is 32 tokens x 4 KV heads = 128 cache records, one per worker thread and one per row of
// the MMAs (row r = 4 * token + head, the order the records have in memory):
//   S1[128 rows x 32]  = K~[128 x 128 dims] . Qrot^T      K~ looked up by its thread into TENSOR memory
//   S2[128 rows x 32]  = Sgn[128 x 128]     . Qsgn^T      (the 1-bit residual signs, also tensor memory)
//   O^T[128 dims x 32] += V~^T[128 x 128 rows] . P'[128 rows x 32]
// The 32 columns are (KV head, query head of its group): a row uses the eight columns of its own
// head, and P' is block-diagonal (a row's probabilities sit in its head's columns, zeros elsewhere),
// so one accumulator holds the four heads' value sums.  No operand fragment is assembled per lane:
// a thread looks its record up pair by pair (64-entry table of centroid pairs, replicated per lane)
// and writes 64 registers to its tensor-memory lane (keys, signs) or sixteen 16-byte chunks to the
// value tile in shared memory (MN-major, no swizzle: [8-dim chunk][row][8 fp16]).
//
// Warps: 0-3 key group (keys and signs into tensor memory, upper half of the value tile), 4-7 value
// group (lower half of the value tile, scores, softmax, P'), 8 issues the MMAs (one thread), 9 the
// bulk copies (one thread).  Thread t of either group owns record t of the tile and tensor-memory
// lane t.  The cache records of a tile are fetched with cp.async.bulk into a two-stage ring (six
// arrays, each a contiguous slab because records are token-major with the four heads adjacent).
//
// Softmax: the reference maximum per (head, query head) is shared by the CTA and lazy: it moves
// only when some score exceeds it by more than kAttnSoftmaxSlack; then all workers meet, rescale
// their partial sums and the accumulator in tensor memory.  The usual tile costs one barrier vote.
//
// Every mbarrier wait is bounded (0.2 s): on a time-out the CTA raises *status, sets an abort flag
// that all other waits observe, lets outstanding copies land, frees its tensor memory and returns.
#include <cmath>
#include <cstdint>

#include "tq_attn.cuh"
#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

__constant__ float kTcC3[8] = {-2.152176f, -1.344318f, -0.756130f, -0.245379f, 0.245379f, 0.756130f, 1.344318f, 2.152176f};

constexpr int kTcThreads = 320;
constexpr int kTcGroup = 128;   // threads of a worker group
constexpr int kTcMmaWarp = 8, kTcCopyWarp = 9;
constexpr int kTcTile = 32;     // tokens per tile
constexpr int kTcStages = 2;
constexpr uint32_t kTcTmemCols = 256;
constexpr uint32_t kColAK = 0, kColAS = 64, kColD1 = 128, kColD2 = 160, kColO = 192;
constexpr unsigned long long kTcWaitLimitNs = 200ull * 1000 * 1000;

struct TcSmem {
    static constexpr int kKBytes = kTcTile * 4 * 52;
    static constexpr int kSBytes = kTcTile * 4 * 16;
    static constexpr int kNBytes = kTcTile * 4 * 4;
    static constexpr int kOffV = kKBytes, kOffS = 2 * kKBytes, kOffKN = kOffS + kSBytes, kOffVN = kOffKN + kNBytes,
                         kOffQN = kOffVN + kNBytes;
    static constexpr int kStageBytes = kOffQN + kNBytes;
    static constexpr int kOffVhat = kTcStages * kStageBytes;   // value tile, 16 chunks x 2 KB
    static constexpr int kOffP = kOffVhat + 32768;             // P', 4 chunks x 2 KB
    static constexpr int kOffBq = kOffP + 8192;                // rotated queries, K-major core matrices
    static constexpr int kOffBs = kOffBq + 8192;               // sign-weighted rotated queries
    static constexpr int kOffBars = kOffBs + 8192;             // 9 mbarriers
    static constexpr int kOffM = kOffBars + 128;               // reference maxima [32], log2 domain
    static constexpr int kOffFactor = kOffM + 128;             // rescale factors [32]
    static constexpr int kOffWmax = kOffFactor + 128;          // per-warp maxima / sums [4][32]
    static constexpr int kSmemBytes = kOffWmax + 512;
    static_assert(kStageBytes % 16 == 0 && kKBytes % 32 == 0, "bulk copies move multiples of 16 bytes, also for half a tile");
    static_assert(kOffVhat % 128 == 0, "operand tiles start on 128-byte boundaries");
};

__device__ __forceinline__ uint32_t tc_smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ unsigned long long tc_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  sleep_ns > 0: back off between polls (the threads that only issue copies or MMAs
// wait most of the time; a busy poll loop would take issue slots from the workers).
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile unsigned int* abort_flag, unsigned sleep_ns = 0) {
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (done) return true;
        if (sleep_ns) __nanosleep(sleep_ns);
        if ((spin & 63u) == 63u) {
            if (*abort_flag) return false;
            const unsigned long long now = tc_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kTcWaitLimitNs) return false;
        }
    }
}
// The same for a whole warp: the outcome is made uniform, because the tensor-memory accesses that
// follow a wait are warp-collective.
__device__ __forceinline__ bool tc_wait_warp(uint32_t bar, uint32_t parity, volatile unsigned int* abort_flag) {
    return __all_sync(0xffffffffu, tc_wait(bar, parity, abort_flag) ? 1 : 0) != 0;
}
__device__ __forceinline__ void tc_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint32_t tc_pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float tc_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// instruction descriptor: D fp32, A and B fp16, M 128, N 32; bits 15 / 16: A / B are MN-major
constexpr uint32_t kIdescS = (1u << 4) | ((32u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescPV = kIdescS | (1u << 15) | (1u << 16);
// shared-memory matrix descriptor, no swizzle, version 1
__device__ __forceinline__ uint64_t tc_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(lbo >> 4) << 16) |
           (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p; }"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
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
// Barriers 1 (value group) and 2 (key group), 128 threads each.
__device__ __forceinline__ void tc_group_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
__device__ __forceinline__ bool tc_value_group_or(bool pred) {
    uint32_t out;
    asm volatile("{ .reg .pred p, q; setp.ne.u32 p, %1, 0; bar.red.or.pred q, 1, 128, p; selp.u32 %0, 1, 0, q; }"
                 : "=r"(out)
                 : "r"(pred ? 1u : 0u)
                 : "memory");
    return out != 0u;
}

template <typename QT>
__global__ void __launch_bounds__(kTcThreads, kAttnTcCtasPerSm) attn_tc_kernel(const AttnSeq* __restrict__ seqs, const QT* __restrict__ qv,
                                                                              int q_heads, int n_splits, uint32_t k_seed,
                                                                              uint32_t qjl_seed, int use_qjl, float inv_sqrt,
                                                                              float inv_scale_d, float attn_scale, float gamma,
                                                                              float* __restrict__ part_acc, float* __restrict__ part_ml,
                                                                              unsigned int* __restrict__ status) {
    using LY = TcSmem;
    constexpr int D = 128;
    constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
    extern __shared__ __align__(128) unsigned char tc_smem[];
    __shared__ __align__(16) uint32_t s_lut[64 * 32];   // pair table [pair index][lane]
    __shared__ unsigned int s_abort;
    __shared__ uint32_t s_tmem_base;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = q_heads / 4;
    const int split = blockIdx.x, gchunk = blockIdx.y, seq = blockIdx.z;
    const int g0 = gchunk * 8;
    const int ng = min(8, G - g0);

    const AttnSeq S = seqs[seq];
    const int first_tile = S.start >> 5, end_tile = (S.end + kTcTile - 1) >> 5;
    const int all_tiles = S.end > S.start ? end_tile - first_tile : 0;
    const int tile0 = first_tile + static_cast<int>(static_cast<long>(all_tiles) * split / n_splits);
    const int tile1 = first_tile + static_cast<int>(static_cast<long>(all_tiles) * (split + 1) / n_splits);
    const int n_tiles = tile1 - tile0;
    const int end16 = (S.end + 15) & ~15;   // storage is a multiple of 16 tokens: copies stop here

    unsigned char* const base = tc_smem;
    const uint32_t raw = tc_smem_addr(tc_smem);
    const uint32_t bar0 = raw + LY::kOffBars;
    // full / empty per stage; a_ready: keys and signs of a tile are in tensor memory; s_ready: its scores are;
    // d_free: the scores have been read; vp_ready: value tile and P' are written; v_free: O += V~^T P' is done
    const uint32_t bar_full = bar0, bar_empty = bar0 + 8u * kTcStages, bar_aready = bar0 + 32u, bar_sready = bar0 + 40u,
                   bar_vpready = bar0 + 48u, bar_vfree = bar0 + 56u, bar_dfree = bar0 + 64u;
    static_assert(kTcStages == 2, "barrier offsets above assume two stages");
    float* const s_m = reinterpret_cast<float*>(base + LY::kOffM);
    float* const s_factor = reinterpret_cast<float*>(base + LY::kOffFactor);
    float* const s_wmax = reinterpret_cast<float*>(base + LY::kOffWmax);
    volatile unsigned int* abort_flag = &s_abort;

    if (tid == 0) {
        s_abort = 0u;
        for (int s = 0; s < kTcStages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_full + 8u * s), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_empty + 8u * s), "r"(8) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_aready), "r"(4) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_sready), "r"(1) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_vpready), "r"(8) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_vfree), "r"(1) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_dfree), "r"(4) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 32) s_m[tid] = -INFINITY;
    if (warp == kTcMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_addr(&s_tmem_base)),
                     "r"(kTcTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem_base;

    bool ok = true;
    // one tile of the ring: expected bytes, then the copies (one thread)
    auto issue_tile = [&](int it) {
        const int s = it % kTcStages;
        const int tok0 = (tile0 + it) * kTcTile;
        const uint32_t ntok = end16 - tok0 >= kTcTile ? kTcTile : 16;
        const uint32_t kb = ntok * 4u * 52u, sb = ntok * 4u * 16u, nb = ntok * 4u * 4u;
        const uint32_t total = 2u * kb + 2u * nb + (use_qjl ? sb + nb : 0u);
        const uint32_t bar = bar_full + 8u * s;
        const uint32_t dst = raw + static_cast<uint32_t>(s) * LY::kStageBytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(total) : "memory");
        const size_t rec = static_cast<size_t>(tok0) * 4;
        tc_copy(dst, S.k_words + rec * 13, kb, bar);
        tc_copy(dst + LY::kOffV, S.v_words + rec * 13, kb, bar);
        tc_copy(dst + LY::kOffKN, S.k_norms + rec, nb, bar);
        tc_copy(dst + LY::kOffVN, S.v_norms + rec, nb, bar);
        if (use_qjl) {
            tc_copy(dst + LY::kOffS, S.qjl_words + rec * 4, sb, bar);
            tc_copy(dst + LY::kOffQN, S.qjl_norms + rec, nb, bar);
        }
    };
    // the first tiles start moving while the tables below are set up
    if (warp == kTcCopyWarp && lane == 0)
        for (int it = 0; it < min(kTcStages, n_tiles); ++it) issue_tile(it);

    // ---- set-up: pair table and P' zeros (value group), rotated queries (key group) ------------------
    if (warp >= 4 && warp < 8) {
        for (int i = tid - kTcGroup; i < 64 * 32; i += kTcGroup) {
            const int idx = i >> 5;
            s_lut[i] = tc_pack_half2(kAttnCentroidScale * kTcC3[idx & 7], kAttnCentroidScale * kTcC3[idx >> 3]);
        }
        for (int i = tid - kTcGroup; i < 8192 / 16; i += kTcGroup) reinterpret_cast<uint4*>(base + LY::kOffP)[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    } else if (warp < 4) {
        // warp = KV head: fp16-round, sign, butterfly, 1/sqrt(d), fp16-round; row n = 8 * head + h
        __half* const scratch = reinterpret_cast<__half*>(base + LY::kOffVhat);   // [32][128], natural dim order
        for (int h = 0; h < 8; ++h) {
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float t = 0.f;
                if (h < ng) {
                    const size_t qi = (static_cast<size_t>(seq) * q_heads + warp * G + g0 + h) * D + lane * 4 + j;
                    t = __half2float(__float2half_rn(static_cast<float>(qv[qi])));
                }
                v[j] = t * sign_value(k_seed, static_cast<uint32_t>(lane * 4 + j));
            }
            warp_fwht<4>(v, lane);
            const uint32_t lo = tc_pack_half2(v[0] * inv_sqrt, v[1] * inv_sqrt), hi = tc_pack_half2(v[2] * inv_sqrt, v[3] * inv_sqrt);
            // K-major core matrices: (n / 8) * 2048 + (k / 8) * 128 + (n % 8) * 16 + (k % 8) * 2, k = 4 * lane ..
            *reinterpret_cast<uint2*>(base + LY::kOffBq + warp * 2048 + (lane >> 1) * 128 + h * 16 + (lane & 1) * 8) = make_uint2(lo, hi);
            *reinterpret_cast<uint2*>(scratch + (warp * 8 + h) * D + lane * 4) = make_uint2(lo, hi);
        }
        tc_group_sync(2);
        // sign operand: column c = 16 * j + pp of the sign tile holds dims (32 j + pp, 32 j + pp + 16)
        for (int idx = tid; idx < 32 * 64; idx += kTcGroup) {
            const int n = idx >> 6, c = idx & 63;
            const int e = 32 * (c >> 4) + (c & 15);
            const float s0 = qjl_sign_is_positive(qjl_seed, static_cast<uint32_t>(e)) ? 1.f : -1.f;
            const float s1 = qjl_sign_is_positive(qjl_seed, static_cast<uint32_t>(e + 16)) ? 1.f : -1.f;
            const uint32_t val = tc_pack_half2(__half2float(scratch[n * D + e]) * s0, __half2float(scratch[n * D + e + 16]) * s1);
            *reinterpret_cast<uint32_t*>(base + LY::kOffBs + (n >> 3) * 2048 + (c >> 2) * 128 + (n & 7) * 16 + (c & 3) * 4) = val;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // every worker thread owns record `row` of a tile (= 4 * token-in-tile + head) and tensor-memory lane `row`
    const int row = 32 * (warp & 3) + lane;
    const int hh = lane & 3, tt = row >> 2;
    const uint32_t lane_off = static_cast<uint32_t>(lane) * 4u;
    const uint32_t tm_lane = tmem + (static_cast<uint32_t>(32 * (warp & 3)) << 16);
    auto lut_pair = [&](uint32_t word, int bit) -> uint32_t {
        // byte offset ((word >> bit) & 63) * 128 + lane * 4: one shift, one logic op; the table's address is an immediate
        const uint32_t sh = bit >= 7 ? (word >> (bit - 7)) : (word << (7 - bit));
        return *reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(s_lut) + ((sh & (63u << 7)) | lane_off));
    };
    // 16-byte chunk c of a record's value row (dims 8c .. 8c+7) -> value tile [chunk][row][8 fp16]
    auto value_chunk = [&](const uint32_t (&vw)[13], int c) {
        uint4 o;
        o.x = lut_pair(vw[(4 * c) / 5], 6 * ((4 * c) % 5));
        o.y = lut_pair(vw[(4 * c + 1) / 5], 6 * ((4 * c + 1) % 5));
        o.z = lut_pair(vw[(4 * c + 2) / 5], 6 * ((4 * c + 2) % 5));
        o.w = lut_pair(vw[(4 * c + 3) / 5], 6 * ((4 * c + 3) % 5));
        *reinterpret_cast<uint4*>(base + LY::kOffVhat + c * 2048 + row * 16) = o;
    };

    if (warp == kTcCopyWarp) {
        // ---- copies: one thread keeps the ring full -----------------------------------------------
        if (lane == 0) {
            for (int it = kTcStages; it < n_tiles; ++it) {
                if (!tc_wait(bar_empty + 8u * (it % kTcStages), static_cast<uint32_t>(it / kTcStages - 1) & 1u, abort_flag, 64)) {
                    ok = false;
                    break;
                }
                issue_tile(it);
            }
        }
        __syncwarp();
    } else if (warp == kTcMmaWarp) {
        // ---- MMA issue (one thread) -------------------------------------------------------------------
        if (lane == 0) {
            // no-swizzle descriptors, K-major and MN-major alike: the leading byte offset is the step to the next
            // core matrix along K (8 rows of 16 bytes, stored contiguously here), the stride byte offset the step
            // along M / N (the next 8 rows of a K-major operand, the next 8-element chunk of an MN-major one)
            const uint32_t lbo = 128u, sbo = 2048u;
            const uint64_t desc_q = tc_desc(raw + LY::kOffBq, lbo, sbo), desc_s = tc_desc(raw + LY::kOffBs, lbo, sbo);
            const uint64_t desc_v = tc_desc(raw + LY::kOffVhat, lbo, sbo), desc_p = tc_desc(raw + LY::kOffP, lbo, sbo);
            for (int it = 0; it < n_tiles; ++it) {
                const uint32_t par = static_cast<uint32_t>(it) & 1u;
                if (!tc_wait(bar_aready, par, abort_flag, 32) ||
                    (it > 0 && !tc_wait(bar_dfree, static_cast<uint32_t>(it - 1) & 1u, abort_flag, 32))) {
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    tc_mma_ts(tmem + kColD1, tmem + kColAK + 8u * ks, desc_q + static_cast<uint64_t>(16 * ks), kIdescS, ks ? 1u : 0u);
                if (use_qjl) {
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)
                        tc_mma_ts(tmem + kColD2, tmem + kColAS + 8u * ks, desc_s + static_cast<uint64_t>(16 * ks), kIdescS, ks ? 1u : 0u);
                }
                tc_commit(bar_sready);
                if (!tc_wait(bar_vpready, par, abort_flag, 32)) {
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)   // 16 rows (two 8-row groups of 128 bytes) per step
                    tc_mma_ss(tmem + kColO, desc_v + static_cast<uint64_t>(16 * ks), desc_p + static_cast<uint64_t>(16 * ks), kIdescPV,
                              (it | ks) ? 1u : 0u);
                tc_commit(bar_vfree);
            }
        }
        __syncwarp();
    } else if (warp < 4) {
        // ---- key group: keys and residual signs into tensor memory, value chunks 8..15 -----------------
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % kTcStages;
            if (!tc_wait_warp(bar_full + 8u * s, static_cast<uint32_t>(it / kTcStages) & 1u, abort_flag)) {
                ok = false;
                break;
            }
            const unsigned char* st = base + s * LY::kStageBytes;
            const uint32_t* sk = reinterpret_cast<const uint32_t*>(st) + row * 13;
            const uint32_t* sv = reinterpret_cast<const uint32_t*>(st + LY::kOffV) + row * 13;
            uint32_t kw[13], vw[13];
#pragma unroll
            for (int j = 0; j < 13; ++j) {
                kw[j] = sk[j];
                vw[j] = sv[j];
            }
            uint4 sw = make_uint4(0u, 0u, 0u, 0u);
            if (use_qjl) sw = *reinterpret_cast<const uint4*>(st + LY::kOffS + row * 16);
            __syncwarp();
            if (lane == 0) tc_arrive(bar_empty + 8u * s);
            // the previous tile's score MMAs must have read the key and sign tiles
            if (it > 0 && !tc_wait_warp(bar_sready, static_cast<uint32_t>(it - 1) & 1u, abort_flag)) {
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            {
                uint32_t a[16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int p = 16 * c + i;
                        a[i] = lut_pair(kw[p / 5], 6 * (p % 5));
                    }
                    tc_st16(tm_lane + kColAK + 16u * c, a);
                }
                if (use_qjl) {
                    const uint32_t inv[4] = {~sw.x, ~sw.y, ~sw.z, ~sw.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int pp = 0; pp < 16; ++pp) {
                            const uint32_t sh = pp == 15 ? inv[j] : (inv[j] << (15 - pp));
                            a[pp] = (sh & 0x80008000u) | 0x3C003C00u;
                        }
                        tc_st16(tm_lane + kColAS + 16u * j, a);
                    }
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_arrive(bar_aready);
            // the previous tile's O += V~^T P' must have read the value tile
            if (it > 0 && !tc_wait_warp(bar_vfree, static_cast<uint32_t>(it - 1) & 1u, abort_flag)) {
                ok = false;
                break;
            }
#pragma unroll
            for (int c = 8; c < 16; ++c) value_chunk(vw, c);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_arrive(bar_vpready);
        }
    } else {
        // ---- value group: value chunks 0..7, scores, softmax, P' -----------------------------------------
        const float kscale = inv_scale_d * attn_scale / kAttnCentroidScale * kLog2e;   // scores in the log2 domain
        const float qscale = gamma * kAttnCentroidScale;
        const float slack = kAttnSoftmaxSlack * kLog2e;
        float l_run[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) l_run[g] = 0.f;

        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % kTcStages;
            bool fail = !ok;
            float sc[8];
            bool valid = false, trigger = false;
            float vnq = 0.f;
            if (!fail && !tc_wait_warp(bar_full + 8u * s, static_cast<uint32_t>(it / kTcStages) & 1u, abort_flag)) fail = true;
            if (!fail) {
                const unsigned char* st = base + s * LY::kStageBytes;
                const uint32_t* sv = reinterpret_cast<const uint32_t*>(st + LY::kOffV) + row * 13;
                uint32_t vw[13];
#pragma unroll
                for (int j = 0; j < 13; ++j) vw[j] = sv[j];
                const float qa = use_qjl ? reinterpret_cast<const float*>(st + LY::kOffQN)[row] * qscale : 0.f;
                const float kn = reinterpret_cast<const float*>(st + LY::kOffKN)[row] * kscale;
                const float vn = reinterpret_cast<const float*>(st + LY::kOffVN)[row];
                const int token = (tile0 + it) * kTcTile + tt;
                valid = token >= S.start && token < S.end;
                vnq = valid ? vn * (1.0f / kAttnCentroidScale) : 0.f;
                __syncwarp();
                if (lane == 0) tc_arrive(bar_empty + 8u * s);
                if (it > 0 && !tc_wait_warp(bar_vfree, static_cast<uint32_t>(it - 1) & 1u, abort_flag)) fail = true;
                if (!fail) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) value_chunk(vw, c);
                }
                if (!fail && !tc_wait_warp(bar_sready, static_cast<uint32_t>(it) & 1u, abort_flag)) fail = true;
                if (!fail) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t d1[32];
                    tc_ld32(tm_lane + kColD1, d1);
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const uint32_t a = (hh & 1) ? d1[8 + g] : d1[g], b = (hh & 1) ? d1[24 + g] : d1[16 + g];
                        sc[g] = __uint_as_float((hh & 2) ? b : a);
                    }
                    if (use_qjl) {
                        tc_ld32(tm_lane + kColD2, d1);
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            const uint32_t a = (hh & 1) ? d1[8 + g] : d1[g], b = (hh & 1) ? d1[24 + g] : d1[16 + g];
                            sc[g] = fmaf(qa, __uint_as_float((hh & 2) ? b : a), sc[g]);
                        }
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) tc_arrive(bar_dfree);
                    const float4 m0 = *reinterpret_cast<const float4*>(s_m + hh * 8), m1 = *reinterpret_cast<const float4*>(s_m + hh * 8 + 4);
                    const float mr[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        sc[g] = valid ? sc[g] * kn : -INFINITY;
                        trigger = trigger || sc[g] > mr[g] + slack;
                    }
                }
            }
            if (fail) {
                atomicExch(&s_abort, 1u);
                ok = false;
            }
            // every thread of the group votes once per tile, whatever happened to it
            const bool move = tc_value_group_or(trigger || fail);
            if (*abort_flag) {
                ok = false;
                break;
            }
            if (move) {
                // new reference maxima; rescale the partial sums and the accumulator
                float tm[8];
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    tm[g] = sc[g];
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) tm[g] = fmaxf(tm[g], __shfl_xor_sync(0xffffffffu, tm[g], o));
                }
                if (lane < 4) {
#pragma unroll
                    for (int g = 0; g < 8; ++g) s_wmax[(warp & 3) * 32 + lane * 8 + g] = tm[g];
                }
                tc_group_sync(1);
                const int t = tid - kTcGroup;
                if (t < 32) {
                    const float old = s_m[t];
                    const float nm = fmaxf(fmaxf(old, fmaxf(s_wmax[t], s_wmax[32 + t])), fmaxf(s_wmax[64 + t], s_wmax[96 + t]));
                    s_factor[t] = (nm == -INFINITY) ? 1.f : tc_ex2(old - nm);
                    s_m[t] = nm;
                }
                tc_group_sync(1);
#pragma unroll
                for (int g = 0; g < 8; ++g) l_run[g] *= s_factor[hh * 8 + g];
                if (it > 0) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t o[32];
                    tc_ld32(tm_lane + kColO, o);
#pragma unroll
                    for (int n = 0; n < 32; ++n) o[n] = __float_as_uint(__uint_as_float(o[n]) * s_factor[n]);
                    tc_st16(tm_lane + kColO, o);
                    tc_st16(tm_lane + kColO + 16u, o + 16);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            {
                const float4 m0 = *reinterpret_cast<const float4*>(s_m + hh * 8), m1 = *reinterpret_cast<const float4*>(s_m + hh * 8 + 4);
                const float mr[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
                float p[8];
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    p[g] = valid ? tc_ex2(sc[g] - mr[g]) : 0.f;
                    l_run[g] += p[g];
                }
                uint4 o;
                o.x = tc_pack_half2(p[0] * vnq, p[1] * vnq);
                o.y = tc_pack_half2(p[2] * vnq, p[3] * vnq);
                o.z = tc_pack_half2(p[4] * vnq, p[5] * vnq);
                o.w = tc_pack_half2(p[6] * vnq, p[7] * vnq);
                *reinterpret_cast<uint4*>(base + LY::kOffP + hh * 2048 + row * 16) = o;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_arrive(bar_vpready);
        }

        // ---- publish the partial result -------------------------------------------------------------
        if (ok && n_tiles > 0 && !tc_wait_warp(bar_vfree, static_cast<uint32_t>(n_tiles - 1) & 1u, abort_flag)) ok = false;
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t o[32];
            if (n_tiles > 0) {
                tc_ld32(tm_lane + kColO, o);
            } else {
#pragma unroll
                for (int n = 0; n < 32; ++n) o[n] = 0u;
            }
            const int d = row;   // accumulator lane = dim
#pragma unroll
            for (int n = 0; n < 32; ++n) {
                const int h = n >> 3, g = n & 7;
                if (g < ng) {
                    const size_t slot = (static_cast<size_t>(seq) * q_heads + h * G + g0 + g) * n_splits + split;
                    part_acc[slot * D + d] = __uint_as_float(o[n]);
                }
            }
#pragma unroll
            for (int g = 0; g < 8; ++g) {
#pragma unroll
                for (int off = 4; off < 32; off <<= 1) l_run[g] += __shfl_xor_sync(0xffffffffu, l_run[g], off);
            }
            if (lane < 4) {
#pragma unroll
                for (int g = 0; g < 8; ++g) s_wmax[(warp & 3) * 32 + lane * 8 + g] = l_run[g];
            }
        }
    }
    if (!ok) atomicExch(&s_abort, 1u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (!s_abort && tid < 32) {
        const int h = tid >> 3, g = tid & 7;
        if (g < ng) {
            const size_t slot = (static_cast<size_t>(seq) * q_heads + h * G + g0 + g) * n_splits + split;
            part_ml[slot * 2] = s_m[tid] * kLn2;   // natural-log domain, as attn_combine_kernel expects
            part_ml[slot * 2 + 1] = (s_wmax[tid] + s_wmax[32 + tid]) + (s_wmax[64 + tid] + s_wmax[96 + tid]);
        }
    }
    if (warp == kTcMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTcTmemCols) : "memory");
    }
    if (s_abort) {
        // let whatever was requested land before the shared memory is released
        if (tid == 0) {
            *reinterpret_cast<volatile unsigned int*>(status) = 12u;   // may be host memory: a plain store, then a system fence
            __threadfence_system();
            const unsigned long long t0 = tc_timer_ns();
            while (tc_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        }
        __syncthreads();
    }
}

}  // namespace

void launch_attn_tc(const AttnSeq* seqs, int n_seqs, const void* q, bool q_is_f16, int q_heads, int kv_heads, int n_splits,
                    uint32_t k_seed, uint32_t qjl_seed, bool use_qjl, float inv_sqrt, float inv_scale_d, float attn_scale,
                    float gamma, float* part_acc, float* part_ml, unsigned int* status, cudaStream_t stream) {
    TQ_REQUIRE(kv_heads == 4 && q_heads % 4 == 0, "tensor-memory attention kernel: four KV heads");
    static bool configured[64] = {false};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(attn_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem::kSmemBytes));
        TQ_CUDA(cudaFuncSetAttribute(attn_tc_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem::kSmemBytes));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int gchunks = (q_heads / 4 + 7) / 8;
    const dim3 grid(n_splits, gchunks, n_seqs);
    if (q_is_f16)
        attn_tc_kernel<__half><<<grid, kTcThreads, TcSmem::kSmemBytes, stream>>>(seqs, static_cast<const __half*>(q), q_heads, n_splits, k_seed,
                                                                                qjl_seed, use_qjl ? 1 : 0, inv_sqrt, inv_scale_d, attn_scale,
                                                                                gamma, part_acc, part_ml, status);
    else
        attn_tc_kernel<float><<<grid, kTcThreads, TcSmem::kSmemBytes, stream>>>(seqs, static_cast<const float*>(q), q_heads, n_splits, k_seed,
                                                                               qjl_seed, use_qjl ? 1 : 0, inv_sqrt, inv_scale_d, attn_scale,
                                                                               gamma, part_acc, part_ml, status);
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
