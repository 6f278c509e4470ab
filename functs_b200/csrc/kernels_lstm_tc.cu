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
