// C4: imperative LSTM (functs/benchmark/ai_model/lstm/lstm.py:79-98, 118-133) in two launches.
//
//   launch 1  input projection, hoisted out of the time loop because it does not depend on h:
//             pre[t*B + b, g*H + j] = x[t, b, :] @ w_ih[g, :, j] + b_ih[g, j] + b_hh[g, j]
//             (tensor cores: see kernels_lstm_tc.cu; the fp32 CUDA-core GEMM below is the device-side check)
//   launch 2  one persistent cooperative kernel for the whole recurrence.  A CTA owns 8 hidden units (all four
//             gates: 32 columns of w_hh, kept in REGISTERS for all T steps) and a tile of 32 batch rows.  Per
//             step it stages h[t-1] of its batch rows in shared memory, forms the 32x32 gate pre-activations,
//             applies the gate non-linearities and slice-assigns h and c straight into hs[t] / cs[t] — hs[t] is
//             at the same time the buffer the other CTAs read h from in step t+1.  Steps are separated by a
//             device-wide arrive/wait counter whose wait is bounded (status bit FB_STATUS_WAIT_TIMEOUT).
#include <cstring>

#include "common.cuh"

namespace fb {

int launch_lstm_input_proj_tc(const float* x, const float* w_ih, const float* b_ih, const float* b_hh, int M, int K,
                              int H, float* pre, void* tc_scratch, int32_t* status, cudaStream_t st);  // kernels_lstm_tc.cu
int64_t lstm_tc_scratch_bytes(int M, int K, int H);
bool lstm_tc_supported(int M, int K, int H);
bool lstm_rtc_supported(int B, int H);
int64_t lstm_rtc_scratch_bytes(int H);
int launch_lstm_recurrent_tc(const float* pre, const float* w_hh, int T, int B, int H, float* hs, float* cs, void* h_tiles,
                             unsigned int* step_counter, int32_t* status, cudaStream_t st);

// ---- fp32 CUDA-core GEMM with bias (check path for launch 1) ------------------------------------------------
constexpr int kGemmBM = 64, kGemmBN = 64, kGemmBK = 16;

__global__ void __launch_bounds__(256)
lstm_input_proj_simt_kernel(const float* __restrict__ x, const float* __restrict__ w_ih, const float* __restrict__ b_ih,
                            const float* __restrict__ b_hh, int M, int K, int H, float* __restrict__ pre) {
    __shared__ float As[kGemmBK][kGemmBM + 4];
    __shared__ float Bs[kGemmBK][kGemmBN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * kGemmBM;
    const int n0 = blockIdx.x * kGemmBN;  // column in [0, 4H); a tile never straddles two gates (H % 64 == 0)
    const int g = n0 / H, j0 = n0 - g * H;
    const float* __restrict__ Bg = w_ih + static_cast<int64_t>(g) * K * H;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += kGemmBK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = threadIdx.x + r * 256;  // 0..1023
            const int am = e >> 4, ak = e & 15;   // A tile: 64 rows x 16 k
            const int gm = m0 + am, gk = k0 + ak;
            As[ak][am] = (gm < M && gk < K) ? __ldg(x + static_cast<int64_t>(gm) * K + gk) : 0.0f;
            const int bk = e >> 6, bn = e & 63;   // B tile: 16 k x 64 cols
            const int gk2 = k0 + bk;
            Bs[bk][bn] = (gk2 < K) ? __ldg(Bg + static_cast<int64_t>(gk2) * H + j0 + bn) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kGemmBK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int jj = j0 + tx * 4 + j;
            const float bias = __fadd_rn(__ldg(b_ih + g * H + jj), __ldg(b_hh + g * H + jj));
            pre[static_cast<int64_t>(gm) * (4 * H) + g * H + jj] = __fadd_rn(acc[i][j], bias);
        }
    }
}

// asynchronous 16-byte copy global (L2) -> shared memory, in commit groups
__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most `pending` of this thread's commit groups are still in flight (pending is a compile-time value
// wherever this is called: the switch folds away)
__device__ __forceinline__ void cp_async_wait_pending(int pending) {
    switch (pending) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
        case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
        case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}

// ---- persistent recurrent kernel ----------------------------------------------------------------------------
constexpr int kRecThreads = 512;  // two halves of 256: each takes 16 of the CTA's 32 rows in the multiply phase
constexpr int kRecB = 32;      // batch rows per tile
constexpr int kRecJ = 8;       // hidden units per CTA (4 gates x 8 units = 32 columns, in 16 groups of 2)
constexpr int kRecKS = 16;     // k-slices (threads along K)
constexpr int kPartStride = 40;
constexpr unsigned long long kWaitCycles = 2000000000ull;  // ~1 s: bound of the inter-step wait

template <int KSL>  // k per slice; H == 16 * KSL
__global__ void __launch_bounds__(kRecThreads, 1)
lstm_recurrent_kernel(const float* __restrict__ pre, const float* __restrict__ w_hh, int T, int B, float* hs, float* cs,
                      unsigned int* step_counter, int32_t* status) {
    constexpr int H = 16 * KSL;
    constexpr int HROW = H + 16 * 4;  // 4 floats of padding after every KSL-float slice: slices of one warp hit different banks
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* h_s = reinterpret_cast<float*>(smem_raw);                       // [kRecB][HROW]
    float* part = h_s + kRecB * HROW;                                      // [kRecKS][kRecB][kPartStride]
    __shared__ int s_abort;

    const int tid = threadIdx.x;
    const int half = tid >> 8;        // which 16 rows this thread multiplies
    const int ks = (tid & 255) >> 4;  // 0..15
    const int cg = tid & 15;          // 0..15 -> columns 2cg, 2cg+1
    const int j0 = blockIdx.x * kRecJ;
    const int b0 = blockIdx.y * kRecB;
    const unsigned int num_ctas = gridDim.x * gridDim.y;

    // resident slice of w_hh: column c = gate * 8 + unit  ->  w_hh[gate][k][j0 + unit]
    float w[KSL][2];
    {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            const int c = cg * 2 + cc;
            const int gate = c >> 3, unit = c & 7;
            const float* src = w_hh + (static_cast<int64_t>(gate) * H + ks * KSL) * H + j0 + unit;
#pragma unroll
            for (int kk = 0; kk < KSL; ++kk) w[kk][cc] = __ldg(src + static_cast<int64_t>(kk) * H);
        }
    }
    // epilogue ownership: thread -> (row eb, unit ej); its cell state lives in a register across steps
    const bool epi = tid < kRecB * kRecJ;  // one epilogue thread per (row, unit)
    const int eb = (tid >> 3) & (kRecB - 1), ej = tid & 7;
    float c_state = 0.0f;
    if (tid == 0) s_abort = 0;
    __syncthreads();
    // the input projection of step t does not depend on h: it is fetched one step ahead, before the inter-step wait
    float pre_g[4] = {0.f, 0.f, 0.f, 0.f};
    if (epi && b0 + eb < B) {
        const float* prow = pre + (static_cast<int64_t>(0) * B + b0 + eb) * (4 * H) + j0 + ej;
#pragma unroll
        for (int g = 0; g < 4; ++g) pre_g[g] = __ldg(prow + g * H);
    }

    for (int t = 0; t < T; ++t) {
        // ---- wait until every CTA has published hs[t-1] ----
        if (t > 0) {
            if (tid == 0) {
                const unsigned int target = num_ctas * static_cast<unsigned int>(t);
                const unsigned long long start = clock64();
                unsigned int seen;
                while (true) {
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(step_counter) : "memory");
                    if (seen >= target) break;
                    if (clock64() - start > kWaitCycles) {
                        s_abort = 1;
                        if (status != nullptr) atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
                        break;
                    }
                }
            }
            __syncthreads();
            if (s_abort) return;
        }
        // ---- stage h[t-1] and accumulate, four rows at a time ----
        // A warp holds two k-slices (lanes 0-15: slice 2w, lanes 16-31: slice 2w + 1) and needs, of h[t-1], only their
        // 2 x KSL columns of the CTA's 32 rows: it fetches them itself with asynchronous copies (L2 -> shared memory, one
        // commit group per block of four rows; 16 consecutive lanes write one row's 16 chunks, so the copies do not
        // collide on banks) and starts multiplying as soon as the first block has landed, while the others are still on
        // their way.  No block barrier between staging and arithmetic.  The order of the additions inside every dot
        // product is the slice's k order, as before.
        constexpr int kRowsPerGroup = 4, kGroups = kRecB / 2 / kRowsPerGroup;  // per half
        static_assert(KSL / 4 * 2 == 16 || KSL / 4 * 2 == 8, "a row's chunks of both slices: 16 (H = 512) or 8 (H = 256)");
        constexpr int kChunks = KSL / 4 * 2;  // 16-byte chunks per row and warp
        if (t > 0) {
            const int warp = (tid & 255) >> 5, lane = tid & 31;  // (the k-slices of this warp: 2 * warp, 2 * warp + 1)
            const float* hsrc = hs + (static_cast<int64_t>(t - 1) * B) * H;
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
#pragma unroll
                for (int e = lane; e < kRowsPerGroup * kChunks; e += 32) {
                    const int r = half * (kRecB / 2) + g * kRowsPerGroup + e / kChunks, c = e % kChunks;
                    const int kcol = (2 * warp + c / (KSL / 4)) * KSL + 4 * (c % (KSL / 4));
                    float* dst = h_s + r * HROW + kcol + (kcol / KSL) * 4;
                    if (b0 + r < B) cp_async_16(dst, hsrc + static_cast<int64_t>(b0 + r) * H + kcol);
                    else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                cp_async_commit();
            }
        }
        {
            const float* hrow = h_s + ks * KSL + ks * 4;
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
                if (t > 0) {
                    cp_async_wait_pending(kGroups - 1 - g);  // row blocks 0 .. g have landed
                    __syncwarp();
                }
#pragma unroll
                for (int bb = 0; bb < kRowsPerGroup; ++bb) {
                    const int b = half * (kRecB / 2) + g * kRowsPerGroup + bb;
                    float a0 = 0.0f, a1 = 0.0f;
                    if (t > 0) {
#pragma unroll
                        for (int q = 0; q < KSL / 4; ++q) {
                            const float4 hv = *reinterpret_cast<const float4*>(hrow + b * HROW + q * 4);
                            a0 = fmaf(hv.x, w[4 * q + 0][0], a0);
                            a1 = fmaf(hv.x, w[4 * q + 0][1], a1);
                            a0 = fmaf(hv.y, w[4 * q + 1][0], a0);
                            a1 = fmaf(hv.y, w[4 * q + 1][1], a1);
                            a0 = fmaf(hv.z, w[4 * q + 2][0], a0);
                            a1 = fmaf(hv.z, w[4 * q + 2][1], a1);
                            a0 = fmaf(hv.w, w[4 * q + 3][0], a0);
                            a1 = fmaf(hv.w, w[4 * q + 3][1], a1);
                        }
                    }
                    *reinterpret_cast<float2*>(part + (ks * kRecB + b) * kPartStride + cg * 2) = make_float2(a0, a1);
                }
            }
        }
        __syncthreads();
        // ---- reduce the 16 slices, add the input projection, gates, slice-assign into hs[t], cs[t] ----
        {
            const int gb = b0 + eb;
            if (epi && gb < B) {
                float gate[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float s = 0.0f;
#pragma unroll
                    for (int s16 = 0; s16 < kRecKS; ++s16) s = __fadd_rn(s, part[(s16 * kRecB + eb) * kPartStride + g * 8 + ej]);
                    gate[g] = __fadd_rn(pre_g[g], s);
                }
                if (t + 1 < T) {
                    const float* prow = pre + (static_cast<int64_t>(t + 1) * B + gb) * (4 * H) + j0 + ej;
#pragma unroll
                    for (int g = 0; g < 4; ++g) pre_g[g] = __ldg(prow + g * H);
                }
                const float ig = sigmoid_f32(gate[0]);
                const float fg = sigmoid_f32(gate[1]);
                const float gg = tanhf(gate[2]);
                const float og = sigmoid_f32(gate[3]);
                c_state = __fadd_rn(__fmul_rn(fg, c_state), __fmul_rn(ig, gg));
                const float hval = __fmul_rn(og, tanhf(c_state));
                const int64_t o = (static_cast<int64_t>(t) * B + gb) * H + j0 + ej;
                hs[o] = hval;
                cs[o] = c_state;
            }
        }
        // ---- publish ----
        // the block barrier orders every thread's stores before thread 0's fence, and that fence (cumulative, device
        // scope) orders them before the counter update: one fence per CTA instead of one per thread
        __syncthreads();
        if (tid == 0 && t + 1 < T) {
            __threadfence();
            atomicAdd(step_counter, 1u);
        }
    }
}

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// what mode 0 means: the combination measured fastest at the configured shape (T = 64, B = 64, H = 512)
constexpr int kLstmDefaultMode = 3;

}  // namespace fb

namespace fb {
void yolo_set_prune(int on);
}

extern "C" {

int64_t functs_b200_lstm_scratch_bytes(int32_t seq_len, int32_t batch, int32_t input, int32_t hidden) {
    if (seq_len <= 0 || batch <= 0 || input <= 0 || hidden <= 0) return 0;
    const int64_t M = static_cast<int64_t>(seq_len) * batch;
    int64_t total = 256;                                             // step counter
    total += fb::align_up(M * 4 * hidden * 4, 256);                  // pre-activations from the input projection
    total += fb::align_up(fb::lstm_tc_scratch_bytes(static_cast<int>(M), input, hidden), 256);
    total += fb::align_up(fb::lstm_rtc_scratch_bytes(hidden), 256);  // h tiles of the tensor-core recurrence
    return total;
}

// mode: 0 = default; 1 = fp32 CUDA cores for both GEMMs; 2 = tensor cores for both (where the shapes allow it);
//       3 = tensor-core projection + CUDA-core recurrence
int functs_b200_lstm_forward_mode(const float* x, const float* w_ih, const float* w_hh, const float* b_ih,
                                  const float* b_hh, int32_t seq_len, int32_t batch, int32_t input, int32_t hidden,
                                  float* hs, float* cs, int32_t* status, void* scratch, void* stream, int32_t mode) {
    using namespace fb;
    FB_REQUIRE(x && w_ih && w_hh && b_ih && b_hh && hs && cs && scratch, "lstm_forward: null pointer");
    FB_REQUIRE(seq_len > 0 && batch > 0 && input > 0, "lstm_forward: bad sizes");
    FB_REQUIRE(hidden == 256 || hidden == 512, "lstm_forward: hidden size %d not supported (256 or 512)", hidden);
    FB_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255) == 0 && (reinterpret_cast<uintptr_t>(hs) & 15) == 0,
               "lstm_forward: scratch must be 256-byte aligned and hs 16-byte aligned");
    cudaStream_t st = as_stream(stream);
    const int M = seq_len * batch;
    unsigned char* base = static_cast<unsigned char*>(scratch);
    unsigned int* counter = reinterpret_cast<unsigned int*>(base);
    float* pre = reinterpret_cast<float*>(base + 256);
    void* tc_scratch = base + 256 + align_up(static_cast<int64_t>(M) * 4 * hidden * 4, 256);
    void* rtc_scratch = static_cast<unsigned char*>(tc_scratch) + align_up(lstm_tc_scratch_bytes(M, input, hidden), 256);
    FB_REQUIRE(mode >= 0 && mode <= 3, "lstm_forward: mode %d unknown", mode);
    if (mode == 0) mode = kLstmDefaultMode;
    FB_TRY(check_cuda(cudaMemsetAsync(counter, 0, 256, st), "memset step counter"));

    record_stage_event(0, st);
    if (mode != 1 && lstm_tc_supported(M, input, hidden)) {
        FB_TRY(launch_lstm_input_proj_tc(x, w_ih, b_ih, b_hh, M, input, hidden, pre, tc_scratch, status, st));
    } else {
        dim3 grid(4 * hidden / kGemmBN, (M + kGemmBM - 1) / kGemmBM);
        lstm_input_proj_simt_kernel<<<grid, 256, 0, st>>>(x, w_ih, b_ih, b_hh, M, input, hidden, pre);
        count_launch();
        FB_TRY(check_launch("lstm_input_proj_simt_kernel"));
    }

    record_stage_event(1, st);
    if (mode == 2 && lstm_rtc_supported(batch, hidden)) {
        const int rc = launch_lstm_recurrent_tc(pre, w_hh, seq_len, batch, hidden, hs, cs, rtc_scratch, counter, status, st);
        record_stage_event(2, st);
        return rc;
    }
    const int btiles = (batch + kRecB - 1) / kRecB;
    dim3 rgrid(hidden / kRecJ, btiles);
    const int hrow = hidden + 64;
    const size_t smem = static_cast<size_t>(kRecB) * hrow * 4 + static_cast<size_t>(kRecKS) * kRecB * kPartStride * 4;
    const void* kfn = hidden == 512 ? reinterpret_cast<const void*>(&lstm_recurrent_kernel<32>)
                                    : reinterpret_cast<const void*>(&lstm_recurrent_kernel<16>);
    FB_TRY(check_cuda(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
                      "lstm_recurrent attr"));
    int occ = 0, dev = 0, sms = 0;
    FB_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
    FB_TRY(check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "sm count"));
    FB_TRY(check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kfn, kRecThreads, smem), "occupancy"));
    if (static_cast<int64_t>(rgrid.x) * rgrid.y > static_cast<int64_t>(occ) * sms) {
        set_error("lstm_forward: %u x %u CTAs cannot be co-resident on %d SMs (batch %d too large for one launch)", rgrid.x,
                  rgrid.y, sms, batch);
        return FB_ERR_UNSUPPORTED;
    }
    const float* pre_c = pre;
    int T = seq_len, B = batch;
    void* args[] = {(void*)&pre_c, (void*)&w_hh, (void*)&T, (void*)&B, (void*)&hs, (void*)&cs, (void*)&counter, (void*)&status};
    FB_TRY(check_cuda(cudaLaunchCooperativeKernel(kfn, rgrid, dim3(kRecThreads), args, smem, st), "lstm_recurrent launch"));
    count_launch();
    record_stage_event(2, st);
    return check_launch("lstm_recurrent_kernel");
}

int functs_b200_debug_set(const char* name, int32_t value) {
    if (name != nullptr && std::strcmp(name, "yolo_prune") == 0) {
        fb::yolo_set_prune(value);
        return FB_OK;
    }
    fb::set_error("debug_set: unknown switch");
    return FB_ERR_NOT_FOUND;
}

int functs_b200_lstm_forward(const float* x, const float* w_ih, const float* w_hh, const float* b_ih,
                             const float* b_hh, int32_t seq_len, int32_t batch, int32_t input, int32_t hidden,
                             float* hs, float* cs, int32_t* status, void* scratch, void* stream) {
    return functs_b200_lstm_forward_mode(x, w_ih, w_hh, b_ih, b_hh, seq_len, batch, input, hidden, hs, cs, status,
                                         scratch, stream, 0);
}

}  // extern "C"
