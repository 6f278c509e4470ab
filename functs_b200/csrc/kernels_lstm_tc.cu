// C4, launch 1 on the tensor cores: the hoisted LSTM input projection
//     pre[m, g*H + j] = sum_k x[m, k] * w_ih[g, k, j] + b_ih[g, j] + b_hh[g, j]          (m = t*B + b)
// as a tcgen05 GEMM with fp32-level accuracy.  fp32 operands do not fit the tensor core's TF32 inputs (10 mantissa
// bits), so every operand is split into hi = tf32(v) and lo = tf32(v - hi) and three products are accumulated in
// the fp32 TMEM accumulator: lo*hi + hi*lo + hi*hi (the dropped lo*lo term is ~2^-22 relative).
//
// Two kernels:
//   lstm_tc_split_kernel  writes the split operands PRE-TILED: every [128 rows x 32 k] tile is stored contiguously
//                         in the no-swizzle K-major core-matrix order the MMA reads from shared memory
//                         (8 rows x 16 bytes per core matrix; K-adjacent core matrices 128 B apart, 8-row groups
//                         1024 B apart).  A tile therefore reaches shared memory with ONE bulk (TMA, untiled) copy.
//   lstm_tc_gemm_kernel   one CTA per 128 x 128 output tile, warp-specialised: warp 0 issues the bulk copies into a
//                         3-stage ring, warp 1 owns TMEM and issues tcgen05.mma (one elected lane), warps 2-5 read
//                         the accumulator back with tcgen05.ld, add the biases and store.
// Every mbarrier wait is bounded; a wait that runs out sets FB_STATUS_WAIT_TIMEOUT, and all roles fall through to
// the common teardown (TMEM is always released).
#include "common.cuh"

namespace fb {

constexpr int kTcBM = 128, kTcBN = 128, kTcBK = 32;
constexpr int kTcTileBytes = kTcBM * kTcBK * 4;   // 16 KB: one hi or lo tile
constexpr int kTcStageBytes = 4 * kTcTileBytes;   // A_hi, A_lo, B_hi, B_lo
constexpr int kTcStages = 3;
constexpr int kTcThreads = 192;
constexpr uint32_t kTcWaitLimit = 2000000u;

__device__ __forceinline__ float tf32_round(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}

// byte offset of element (r, c) inside a pre-tiled [128 x 32] fp32 tile
__device__ __forceinline__ int tile_offset(int r, int c) { return (r >> 3) * 1024 + (c >> 2) * 128 + (r & 7) * 16 + (c & 3) * 4; }

// a_tiles: [M/128][K/32][hi, lo][16 KB];  b_tiles: [4H/128][K/32][hi, lo][16 KB]
__global__ void __launch_bounds__(256)
lstm_tc_split_kernel(const float* __restrict__ x, const float* __restrict__ w_ih, int M, int K, int H,
                     unsigned char* __restrict__ a_tiles, unsigned char* __restrict__ b_tiles) {
    const int kchunks = K / 4;
    const int64_t a_items = static_cast<int64_t>(M) * kchunks;
    const int64_t b_items = static_cast<int64_t>(4 * H) * kchunks;
    const int KT = K / kTcBK;
    const int64_t gstride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < a_items + b_items; e += gstride) {
        float v[4];
        int r, c;
        unsigned char* tile;
        if (e < a_items) {
            // consecutive threads: consecutive 16-byte chunks of one row of x (coalesced reads)
            r = static_cast<int>(e / kchunks);
            c = static_cast<int>(e - static_cast<int64_t>(r) * kchunks) * 4;
            const float4 q = __ldg(reinterpret_cast<const float4*>(x + static_cast<int64_t>(r) * K + c));
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
            tile = a_tiles + (static_cast<int64_t>(r / kTcBM) * KT + c / kTcBK) * (2 * kTcTileBytes);
        } else {
            // consecutive threads: consecutive output columns n = g*H + j for one k-chunk (coalesced reads of w_ih rows)
            const int64_t f = e - a_items;
            const int kc = static_cast<int>(f / (4 * H));
            r = static_cast<int>(f - static_cast<int64_t>(kc) * (4 * H));  // n
            c = kc * 4;
            const int g = r / H, j = r - g * H;
            const float* src = w_ih + (static_cast<int64_t>(g) * K + c) * H + j;
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = __ldg(src + static_cast<int64_t>(i) * H);
            tile = b_tiles + (static_cast<int64_t>(r / kTcBN) * KT + c / kTcBK) * (2 * kTcTileBytes);
        }
        float hi[4], lo[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            hi[i] = tf32_round(v[i]);
            lo[i] = tf32_round(__fsub_rn(v[i], hi[i]));
        }
        const int off = tile_offset(r % kTcBM, c % kTcBK);
        *reinterpret_cast<float4*>(tile + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<float4*>(tile + kTcTileBytes + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// ---- tcgen05 helpers ----------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, no swizzle, K-major: start address, leading-dimension byte offset (between core
// matrices adjacent in K), stride-dimension byte offset (between 8-row groups), descriptor version 1.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    return d;
}

// Instruction descriptor for kind::tf32: D = F32, A = B = TF32, both K-major, M = 128, N = 128.
constexpr uint32_t kTcIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((kTcBN >> 3) << 17) | ((kTcBM >> 4) << 24);

__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kTcIdesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_ld_32cols(uint32_t taddr, float* out) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) out[i] = __uint_as_float(r[i]);
}

struct TcShared {
    uint64_t full[kTcStages];
    uint64_t empty[kTcStages];
    uint64_t accum;
    uint32_t tmem_base;
    volatile int abort_flag;
};

// grid = (4H / 128, M / 128).  dynamic smem: kTcStages * 64 KB of operand tiles (1024-byte aligned) + TcShared.
__global__ void __launch_bounds__(kTcThreads, 1)
lstm_tc_gemm_kernel(const unsigned char* __restrict__ a_tiles, const unsigned char* __restrict__ b_tiles,
                    const float* __restrict__ b_ih, const float* __restrict__ b_hh, int K, int H, float* __restrict__ pre,
                    int32_t* status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles = smem_raw;
    TcShared& sh = *reinterpret_cast<TcShared*>(smem_raw + kTcStages * kTcStageBytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = K / kTcBK;
    const int nt = blockIdx.x, mt = blockIdx.y;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; ++s) {
            mbar_init(&sh.full[s], 1);
            mbar_init(&sh.empty[s], 1);
        }
        mbar_init(&sh.accum, 1);
        sh.abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        // 128 fp32 accumulator columns; the allocating warp also frees them at the end
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(128u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            const unsigned char* a_src = a_tiles + static_cast<int64_t>(mt) * KT * (2 * kTcTileBytes);
            const unsigned char* b_src = b_tiles + static_cast<int64_t>(nt) * KT * (2 * kTcTileBytes);
            for (int kt = 0; kt < KT; ++kt) {
                const int s = kt % kTcStages;
                const uint32_t par = ((kt / kTcStages) & 1) ^ 1;  // passes at once on a fresh barrier
                bool ok = false;
                for (uint32_t it = 0; it < kTcWaitLimit && !sh.abort_flag; ++it) {
                    if (mbar_try_wait(&sh.empty[s], par)) { ok = true; break; }
                }
                if (!ok) {
                    sh.abort_flag = 1;
                    if (status != nullptr) atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
                    break;
                }
                unsigned char* dst = tiles + s * kTcStageBytes;
                mbar_arrive_expect_tx(&sh.full[s], kTcStageBytes);
                bulk_copy_g2s(dst, a_src + static_cast<int64_t>(kt) * (2 * kTcTileBytes), 2 * kTcTileBytes, &sh.full[s]);
                bulk_copy_g2s(dst + 2 * kTcTileBytes, b_src + static_cast<int64_t>(kt) * (2 * kTcTileBytes), 2 * kTcTileBytes,
                              &sh.full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // descriptor strides of the pre-tiled layout (tile_offset): core matrices adjacent in K are 128 bytes apart
            // (leading-dimension offset), 8-row groups 1024 bytes apart (stride-dimension offset)
            constexpr uint32_t lbo = 128u, sbo = 1024u;
            uint32_t accumulate = 0;
            bool failed = false;
            for (int kt = 0; kt < KT && !failed; ++kt) {
                const int s = kt % kTcStages;
                const uint32_t par = (kt / kTcStages) & 1;
                bool ok = false;
                for (uint32_t it = 0; it < kTcWaitLimit && !sh.abort_flag; ++it) {
                    if (mbar_try_wait(&sh.full[s], par)) { ok = true; break; }
                }
                if (!ok) {
                    sh.abort_flag = 1;
                    if (status != nullptr) atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
                    failed = true;
                    break;
                }
                tc_fence_after();
                const uint32_t a_hi = smem_u32(tiles + s * kTcStageBytes);
                const uint32_t a_lo = a_hi + kTcTileBytes;
                const uint32_t b_hi = a_hi + 2 * kTcTileBytes;
                const uint32_t b_lo = a_hi + 3 * kTcTileBytes;
#pragma unroll
                for (int kk = 0; kk < kTcBK / 8; ++kk) {
                    const uint32_t ko = kk * 256;  // 8 k-elements = two core matrices of 128 bytes
                    const uint64_t dah = make_smem_desc(a_hi + ko, lbo, sbo), dal = make_smem_desc(a_lo + ko, lbo, sbo);
                    const uint64_t dbh = make_smem_desc(b_hi + ko, lbo, sbo), dbl = make_smem_desc(b_lo + ko, lbo, sbo);
                    tc_mma_tf32(tmem, dal, dbh, accumulate);
                    accumulate = 1;
                    tc_mma_tf32(tmem, dah, dbl, 1);
                    tc_mma_tf32(tmem, dah, dbh, 1);
                }
                tc_commit(&sh.empty[s]);  // the stage is free once these MMAs have read it
            }
            if (!failed) tc_commit(&sh.accum);
        }
    } else {
        // epilogue warps 2..5: TMEM lane quadrant = warp % 4
        bool ok = false;
        for (uint32_t it = 0; it < kTcWaitLimit && !sh.abort_flag; ++it) {
            if (mbar_try_wait(&sh.accum, 0)) { ok = true; break; }
        }
        ok = __all_sync(kFullMask, ok);
        if (ok) {
            tc_fence_after();
            const int q = warp & 3;
            const int m = mt * kTcBM + q * 32 + lane;
            const int n0 = nt * kTcBN;  // column in [0, 4H); a tile lies inside one gate because H % 128 == 0
            float* orow = pre + static_cast<int64_t>(m) * (4 * H) + n0;
#pragma unroll 1
            for (int cb = 0; cb < kTcBN / 32; ++cb) {
                float acc[32];
                tc_ld_32cols(tmem + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(cb * 32), acc);
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const int n = n0 + cb * 32 + i;
                    const float4 bi = __ldg(reinterpret_cast<const float4*>(b_ih + n));
                    const float4 bh = __ldg(reinterpret_cast<const float4*>(b_hh + n));
                    float4 o;
                    o.x = __fadd_rn(acc[i + 0], __fadd_rn(bi.x, bh.x));
                    o.y = __fadd_rn(acc[i + 1], __fadd_rn(bi.y, bh.y));
                    o.z = __fadd_rn(acc[i + 2], __fadd_rn(bi.z, bh.z));
                    o.w = __fadd_rn(acc[i + 3], __fadd_rn(bi.w, bh.w));
                    *reinterpret_cast<float4*>(orow + cb * 32 + i) = o;
                }
            }
        } else if (lane == 0 && status != nullptr) {
            atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
        }
    }
    // ---- teardown: everybody meets, then the allocating warp frees TMEM ----
    tc_fence_before();
    __syncthreads();
    if (sh.abort_flag && threadIdx.x == 0) {
        // give bulk copies that are still in flight time to land before the CTA's shared memory is released
        const unsigned long long t0 = clock64();
        while (clock64() - t0 < 400000ull) {
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
    }
}

// ==== the recurrence on the tensor cores =====================================================================
// Per time step  gates[b, n] = pre[t, b, n] + sum_k h[t-1][b, k] * w_hh[gate(n), k, unit(n)]   (b < 64, n < 4H)
// as a persistent cooperative kernel.  A CTA owns kRtcUnits = 4 hidden units, i.e. N = 16 gate columns (4 gates x 4
// units), and ALL batch rows: per step it runs one [128 x 16] += [128 x H] * [H x 16] tcgen05 GEMM (M = 128 is the
// instruction's tile; rows 64..127 of the A tiles are zero padding that is written once), 3xTF32 like the projection.
//   B operand   the CTA's slice of w_hh, split into hi / lo TF32 parts and pre-tiled, resident in shared memory for all
//               steps (H / 32 k-tiles x 4 KB = 64 KB at H = 512);
//   A operand   h[t-1], hi / lo, pre-tiled: the epilogue of step t-1 (of every CTA) stores its four units of every row
//               as one 16-byte chunk straight into the tiled global buffer (a [64 x 32] half tile is 8 KB contiguous),
//               and step t brings it in with bulk copies through a ring of kRtcStages stages (32 KB each);
//   D           128 lanes x 16 TMEM columns; the epilogue reads rows 0..63 (tcgen05.ld), hands them through shared
//               memory to 256 threads, one (row, unit) each: add the input projection, gate non-linearities,
//               c / h update, hs[t] / cs[t] slice assignment, h hi / lo tiles for the next step.
// Steps are separated by a device-wide arrive / wait counter (the grid is launched cooperatively, one CTA per SM).
// Every wait is bounded; when one runs out the CTA sets FB_STATUS_WAIT_TIMEOUT, raises its abort flag and every role
// falls through to the common teardown, where TMEM is released.
constexpr int kRtcUnits = 4;
constexpr int kRtcN = 16;
constexpr int kRtcATile = 128 * kTcBK * 4;        // 16 KB, rows 64..127 stay zero
constexpr int kRtcAHalf = 64 * kTcBK * 4;         // 8 KB: the rows that exist
constexpr int kRtcBTile = kRtcN * kTcBK * 4;      // 2 KB
constexpr int kRtcStageBytes = 2 * kRtcATile;     // A_hi, A_lo
constexpr int kRtcStages = 4;
constexpr int kRtcThreads = 320;                  // warp 0: copies, warp 1: MMA, warps 2..9: epilogue
constexpr int kRtcEpiThreads = 256;
constexpr int kRtcBatch = 64;
constexpr int kRtcGateStride = kRtcN + 1;
constexpr unsigned long long kRtcWaitCycles = 2000000000ull;  // ~1 s: bound of the inter-step wait
constexpr uint32_t kRtcIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((kRtcN >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void rtc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kRtcIdesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tc_ld_16cols(uint32_t taddr, float* out) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = __uint_as_float(r[i]);
}

struct RtcShared {
    uint64_t full[kRtcStages];
    uint64_t empty[kRtcStages];
    uint64_t accum;
    uint32_t tmem_base;
    volatile int abort_flag;
    float gates[kRtcBatch * kRtcGateStride];
};

__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kRtcEpiThreads) : "memory"); }

// grid = H / 4 CTAs (cooperative).  h_tiles: [2 (step parity)][H / 32][hi, lo][8 KB]; pre: [T * B, 4H].
__global__ void __launch_bounds__(kRtcThreads, 1)
lstm_recurrent_tc_kernel(const float* __restrict__ pre, const float* __restrict__ w_hh, int T, int H, float* hs, float* cs,
                         unsigned char* h_tiles, unsigned int* step_counter, int32_t* status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int KT = H / kTcBK;
    unsigned char* ring = smem_raw;                                   // kRtcStages x 32 KB
    unsigned char* btiles = ring + kRtcStages * kRtcStageBytes;       // KT x (hi 2 KB, lo 2 KB)
    RtcShared& sh = *reinterpret_cast<RtcShared*>(btiles + static_cast<size_t>(KT) * 2 * kRtcBTile);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int j0 = blockIdx.x * kRtcUnits;
    const unsigned int num_ctas = gridDim.x;
    constexpr int B = kRtcBatch;

    // ---- set-up: barriers, zero ring (the padding rows must read as zero), resident w_hh slice, TMEM ----
    if (tid == 0) {
        for (int s = 0; s < kRtcStages; ++s) {
            mbar_init(&sh.full[s], 1);
            mbar_init(&sh.empty[s], 1);
        }
        mbar_init(&sh.accum, 1);
        sh.abort_flag = 0;
        fence_barrier_init();
    }
    for (int i = tid; i < kRtcStages * kRtcStageBytes / 16; i += kRtcThreads) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0, 0, 0, 0);
    for (int e = tid; e < kRtcN * H; e += kRtcThreads) {
        // consecutive threads: the 4 units of one (gate, k): a 16-byte read of w_hh
        const int unit = e & 3, gk = e >> 2;
        const int k = gk % H, gate = gk / H;
        const float v = __ldg(w_hh + (static_cast<int64_t>(gate) * H + k) * H + j0 + unit);
        const float hi = tf32_round(v), lo = tf32_round(__fsub_rn(v, hi));
        const int n = gate * kRtcUnits + unit;
        unsigned char* tile = btiles + static_cast<size_t>(k / kTcBK) * 2 * kRtcBTile;
        const int off = tile_offset(n, k % kTcBK);
        *reinterpret_cast<float*>(tile + off) = hi;
        *reinterpret_cast<float*>(tile + kRtcBTile + off) = lo;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(32u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_proxy_async();  // the generic-proxy writes above are read by the tensor core through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0) {
        // ---- copies: for every step t >= 1, the KT k-tiles of h[t-1] (hi, lo) ----
        if (lane == 0) {
            uint32_t it = 0;
            for (int t = 1; t < T && !sh.abort_flag; ++t) {
                // every CTA has published h[t-1]
                const unsigned int target = num_ctas * static_cast<unsigned int>(t);
                const unsigned long long start = clock64();
                unsigned int seen;
                bool ok = true;
                while (true) {
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(step_counter) : "memory");
                    if (seen >= target) break;
                    if (sh.abort_flag || clock64() - start > kRtcWaitCycles) { ok = false; break; }
                }
                if (!ok) {
                    sh.abort_flag = 1;
                    if (status != nullptr) atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
                    break;
                }
                asm volatile("fence.proxy.async;" ::: "memory");  // the tiles were written by generic stores of other SMs
                const unsigned char* src = h_tiles + static_cast<size_t>((t - 1) & 1) * KT * 2 * kRtcAHalf;
                for (int kt = 0; kt < KT; ++kt, ++it) {
                    const int s = it % kRtcStages;
                    const uint32_t par = ((it / kRtcStages) & 1) ^ 1;
                    bool got = false;
                    for (uint32_t w = 0; w < kTcWaitLimit && !sh.abort_flag; ++w) {
                        if (mbar_try_wait(&sh.empty[s], par)) { got = true; break; }
                    }
                    if (!got) {
                        sh.abort_flag = 1;
                        if (status != nullptr) atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
                        break;
                    }
                    unsigned char* dst = ring + s * kRtcStageBytes;
                    mbar_arrive_expect_tx(&sh.full[s], 2 * kRtcAHalf);
                    bulk_copy_g2s(dst, src + static_cast<size_t>(kt) * 2 * kRtcAHalf, kRtcAHalf, &sh.full[s]);
                    bulk_copy_g2s(dst + kRtcATile, src + static_cast<size_t>(kt) * 2 * kRtcAHalf + kRtcAHalf, kRtcAHalf, &sh.full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ----
        if (lane == 0) {
            constexpr uint32_t lbo = 128u, sbo = 1024u;
            uint32_t it = 0;
            for (int t = 1; t < T && !sh.abort_flag; ++t) {
                uint32_t accumulate = 0;
                bool failed = false;
                for (int kt = 0; kt < KT && !failed; ++kt, ++it) {
                    const int s = it % kRtcStages;
                    const uint32_t par = (it / kRtcStages) & 1;
                    bool got = false;
                    // the first tile of a step only arrives after the inter-step wait: bounded by time, like that wait
                    const unsigned long long wstart = clock64();
                    while (!sh.abort_flag) {
                        if (mbar_try_wait(&sh.full[s], par)) { got = true; break; }
                        if (clock64() - wstart > 2 * kRtcWaitCycles) break;
                    }
                    if (!got) {
                        sh.abort_flag = 1;
                        if (status != nullptr) atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
                        failed = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_hi = smem_u32(ring + s * kRtcStageBytes), a_lo = a_hi + kRtcATile;
                    const uint32_t b_hi = smem_u32(btiles + static_cast<size_t>(kt) * 2 * kRtcBTile), b_lo = b_hi + kRtcBTile;
#pragma unroll
                    for (int kk = 0; kk < kTcBK / 8; ++kk) {
                        const uint32_t ko = kk * 256;
                        const uint64_t dah = make_smem_desc(a_hi + ko, lbo, sbo), dal = make_smem_desc(a_lo + ko, lbo, sbo);
                        const uint64_t dbh = make_smem_desc(b_hi + ko, lbo, sbo), dbl = make_smem_desc(b_lo + ko, lbo, sbo);
                        rtc_mma(tmem, dal, dbh, accumulate);
                        accumulate = 1;
                        rtc_mma(tmem, dah, dbl, 1);
                        rtc_mma(tmem, dah, dbh, 1);
                    }
                    tc_commit(&sh.empty[s]);
                }
                if (failed) break;
                tc_commit(&sh.accum);
            }
        }
    } else {
        // ---- epilogue: 256 threads, one (row, unit) each ----
        const int e = tid - 64;
        const int eb = e >> 2, eu = e & 3;  // row, unit
        float c_state = 0.0f;
        float pre_g[4];
        {
            const float* prow = pre + static_cast<int64_t>(eb) * (4 * H) + j0 + eu;
#pragma unroll
            for (int g = 0; g < 4; ++g) pre_g[g] = __ldg(prow + g * H);
        }
        const int kt_mine = j0 / kTcBK;                 // the k-tile this CTA's units belong to
        const int tile_off = tile_offset(eb, (j0 % kTcBK) + eu);
        for (int t = 0; t < T; ++t) {
            float s_g[4] = {0.f, 0.f, 0.f, 0.f};
            if (t > 0) {
                bool ok = false;
                const unsigned long long start = clock64();
                while (!sh.abort_flag) {
                    if (mbar_try_wait(&sh.accum, static_cast<uint32_t>((t - 1) & 1))) { ok = true; break; }
                    if (clock64() - start > 2 * kRtcWaitCycles) break;
                }
                if (!ok) {
                    sh.abort_flag = 1;
                    if (status != nullptr && lane == 0) atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
                }
                // warps 4 and 5 own the TMEM lane quadrants 0 and 1 (rows 0..31, 32..63)
                if ((warp == 4 || warp == 5) && !sh.abort_flag) {
                    tc_fence_after();
                    const int q = warp & 3;
                    float acc[16];
                    tc_ld_16cols(tmem + (static_cast<uint32_t>(q * 32) << 16), acc);
                    float* grow = sh.gates + (q * 32 + lane) * kRtcGateStride;
#pragma unroll
                    for (int i = 0; i < 16; ++i) grow[i] = acc[i];
                    tc_fence_before();
                }
                epi_barrier();
                if (sh.abort_flag) break;
#pragma unroll
                for (int g = 0; g < 4; ++g) s_g[g] = sh.gates[eb * kRtcGateStride + g * kRtcUnits + eu];
            }
            float gate[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) gate[g] = __fadd_rn(pre_g[g], s_g[g]);
            if (t + 1 < T) {
                const float* prow = pre + (static_cast<int64_t>(t + 1) * B + eb) * (4 * H) + j0 + eu;
#pragma unroll
                for (int g = 0; g < 4; ++g) pre_g[g] = __ldg(prow + g * H);
            }
            const float ig = sigmoid_f32(gate[0]);
            const float fg = sigmoid_f32(gate[1]);
            const float gg = tanhf(gate[2]);
            const float og = sigmoid_f32(gate[3]);
            c_state = __fadd_rn(__fmul_rn(fg, c_state), __fmul_rn(ig, gg));
            const float hval = __fmul_rn(og, tanhf(c_state));
            const int64_t o = (static_cast<int64_t>(t) * B + eb) * H + j0 + eu;
            hs[o] = hval;
            cs[o] = c_state;
            if (t + 1 < T) {
                // h[t] for the next step: hi / lo parts into the pre-tiled buffer of this step's parity
                const float hi = tf32_round(hval), lo = tf32_round(__fsub_rn(hval, hi));
                unsigned char* dst = h_tiles + (static_cast<size_t>(t & 1) * KT + kt_mine) * 2 * kRtcAHalf + tile_off;
                *reinterpret_cast<float*>(dst) = hi;
                *reinterpret_cast<float*>(dst + kRtcAHalf) = lo;
                __threadfence();
                epi_barrier();  // every thread's stores are fenced before the CTA announces the step
                if (e == 0) atomicAdd(step_counter, 1u);
            }
        }
    }
    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (sh.abort_flag && threadIdx.x == 0) {
        const unsigned long long t0 = clock64();
        while (clock64() - t0 < 400000ull) {
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32u) : "memory");
    }
}

bool lstm_rtc_supported(int B, int H) { return B == kRtcBatch && H > 0 && (H % kTcBK) == 0 && (H / kRtcUnits) <= kNumSMs; }

int64_t lstm_rtc_scratch_bytes(int H) { return static_cast<int64_t>(2) * (H / kTcBK) * 2 * kRtcAHalf; }

int launch_lstm_recurrent_tc(const float* pre, const float* w_hh, int T, int B, int H, float* hs, float* cs,
                             void* h_tiles, unsigned int* step_counter, int32_t* status, cudaStream_t st) {
    FB_REQUIRE(lstm_rtc_supported(B, H), "lstm tensor-core recurrence: needs batch 64 and hidden a multiple of 32, <= %d",
               kNumSMs * kRtcUnits);
    FB_REQUIRE(h_tiles != nullptr && (reinterpret_cast<uintptr_t>(h_tiles) & 255) == 0, "lstm tensor-core recurrence: misaligned scratch");
    const int KT = H / kTcBK;
    const size_t smem = static_cast<size_t>(kRtcStages) * kRtcStageBytes + static_cast<size_t>(KT) * 2 * kRtcBTile +
                        sizeof(RtcShared) + 1024;
    FB_TRY(check_cuda(cudaFuncSetAttribute(lstm_recurrent_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)),
                      "lstm_recurrent_tc attr"));
    int occ = 0, dev = 0, sms = 0;
    FB_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
    FB_TRY(check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "sm count"));
    FB_TRY(check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, lstm_recurrent_tc_kernel, kRtcThreads, smem), "occupancy"));
    const int ctas = H / kRtcUnits;
    if (ctas > occ * sms) {
        set_error("lstm tensor-core recurrence: %d CTAs cannot be co-resident on %d SMs", ctas, sms);
        return FB_ERR_UNSUPPORTED;
    }
    unsigned char* tiles = static_cast<unsigned char*>(h_tiles);
    void* args[] = {(void*)&pre, (void*)&w_hh, (void*)&T, (void*)&H, (void*)&hs, (void*)&cs, (void*)&tiles,
                    (void*)&step_counter, (void*)&status};
    FB_TRY(check_cuda(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(&lstm_recurrent_tc_kernel), dim3(ctas),
                                                  dim3(kRtcThreads), args, smem, st),
                      "lstm_recurrent_tc launch"));
    count_launch();
    return check_launch("lstm_recurrent_tc_kernel");
}

bool lstm_tc_supported(int M, int K, int H) {
    return M > 0 && K > 0 && H > 0 && (M % kTcBM) == 0 && (K % kTcBK) == 0 && (H % kTcBN) == 0;
}

int64_t lstm_tc_scratch_bytes(int M, int K, int H) {
    if (!lstm_tc_supported(M, K, H)) return 0;
    const int64_t a = static_cast<int64_t>(M / kTcBM) * (K / kTcBK) * 2 * kTcTileBytes;
    const int64_t b = static_cast<int64_t>(4 * H / kTcBN) * (K / kTcBK) * 2 * kTcTileBytes;
    return a + b;
}

int launch_lstm_input_proj_tc(const float* x, const float* w_ih, const float* b_ih, const float* b_hh, int M, int K,
                              int H, float* pre, void* tc_scratch, int32_t* status, cudaStream_t st) {
    FB_REQUIRE(lstm_tc_supported(M, K, H), "lstm tensor-core projection: shape not supported");
    FB_REQUIRE(tc_scratch != nullptr && (reinterpret_cast<uintptr_t>(tc_scratch) & 255) == 0 &&
                   (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(b_ih) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(b_hh) & 15) == 0 && (reinterpret_cast<uintptr_t>(pre) & 15) == 0,
               "lstm tensor-core projection: misaligned pointer");
    unsigned char* a_tiles = static_cast<unsigned char*>(tc_scratch);
    unsigned char* b_tiles = a_tiles + static_cast<int64_t>(M / kTcBM) * (K / kTcBK) * 2 * kTcTileBytes;
    const int64_t items = (static_cast<int64_t>(M) + 4 * H) * (K / 4);
    int blocks = static_cast<int>((items + 255) / 256);
    if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
    lstm_tc_split_kernel<<<blocks, 256, 0, st>>>(x, w_ih, M, K, H, a_tiles, b_tiles);
    count_launch();
    FB_TRY(check_launch("lstm_tc_split_kernel"));
    const size_t smem = static_cast<size_t>(kTcStages) * kTcStageBytes + sizeof(TcShared) + 1024;
    FB_TRY(check_cuda(cudaFuncSetAttribute(lstm_tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)),
                      "lstm_tc_gemm attr"));
    dim3 grid(4 * H / kTcBN, M / kTcBM);
    lstm_tc_gemm_kernel<<<grid, kTcThreads, smem, st>>>(a_tiles, b_tiles, b_ih, b_hh, K, H, pre, status);
    count_launch();
    return check_launch("lstm_tc_gemm_kernel");
}

}  // namespace fb
