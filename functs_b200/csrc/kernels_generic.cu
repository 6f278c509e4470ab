// Generic fusion group: one precompiled kernel that evaluates, per output element, the postfix program the host made of
// a fusion group's subgraph (program format: include/functs_b200.h).  It stands where the reference JIT-compiles a
// kernel per group (fait/fuser/graph_builder.cpp:259-712, fait/tensorexpr/cuda_codegen_tssa.cpp:1319-1414): the gather
// expression is the same, only it is interpreted instead of generated.  Map iterations and group outputs sit on
// blockIdx.y (the reference puts map iterations there as well, functor_parallization.cpp:83-111).
#include "common.cuh"

namespace fb {

__device__ __forceinline__ float g_load(const functs_b200_gprogram& P, const functs_b200_gload& L, const int* x) {
    int off = L.base;
#pragma unroll
    for (int k = 0; k < FB_G_MAX_TERMS; ++k) {
        if (k < L.nterms) {
            const functs_b200_gterm t = L.term[k];
            int v = t.add;
            if (t.dim >= 0) v += t.mul * x[t.dim];
            if (t.div > 1) v /= t.div;
            off += v * t.stride;
        }
    }
    const void* p = P.in_ptr[L.tensor];
    switch (L.dtype) {
        case 0: return __ldg(static_cast<const float*>(p) + off);
        case 1: return static_cast<float>(__ldg(static_cast<const uint8_t*>(p) + off));
        case 2: return static_cast<float>(__ldg(static_cast<const long long*>(p) + off));
        default: return static_cast<float>(__ldg(static_cast<const int*>(p) + off));
    }
}

__device__ __forceinline__ float g_eval(const functs_b200_gprogram& P, const int* x) {
    float st[FB_G_STACK];
    int sp = 0;
    int pc = 0;
    for (int guard = 0; guard < 4 * FB_G_MAX_INSTR; ++guard) {
        const functs_b200_ginstr I = P.instr[pc];
        ++pc;
        const int op = I.op;
        if (op == FB_G_END) break;
        if (op == FB_G_LOAD) {
            st[sp++] = g_load(P, P.load[I.arg], x);
        } else if (op == FB_G_CONST) {
            st[sp++] = I.imm.f;
        } else if (op == FB_G_COND) {
            const functs_b200_gpred q = P.pred[I.arg];
            const int v = (q.dim >= 0 ? q.mul * x[q.dim] : 0) + q.add;
            const bool ok = v >= q.lo && v < q.hi && (q.step <= 1 || ((v - q.lo) % q.step) == 0);
            if (!ok) pc = I.imm.i;
        } else if (op == FB_G_JUMP) {
            pc = I.arg;
        } else if (op < FB_G_ADD) {
            float a = st[sp - 1];
            switch (op) {
                case FB_G_EXP: a = expf(a); break;
                case FB_G_SIGMOID: a = sigmoid_f32(a); break;
                case FB_G_TANH: a = tanhf(a); break;
                case FB_G_RELU: a = fmaxf(a, 0.0f); break;
                case FB_G_NEG: a = -a; break;
                case FB_G_CLAMP_MIN: a = fmaxf(a, I.imm.f); break;
                case FB_G_CLAMP_MAX: a = fminf(a, I.imm.f); break;
                case FB_G_ABS: a = fabsf(a); break;
                case FB_G_SQRT: a = sqrtf(a); break;
                case FB_G_LOG: a = logf(a); break;
                default: break;
            }
            st[sp - 1] = a;
        } else {
            const float b = st[--sp];
            float a = st[sp - 1];
            switch (op) {
                case FB_G_ADD: a = __fadd_rn(a, b); break;
                case FB_G_SUB: a = __fsub_rn(a, b); break;
                case FB_G_MUL: a = __fmul_rn(a, b); break;
                case FB_G_DIV: a = __fdiv_rn(a, b); break;
                case FB_G_MIN: a = fminf(a, b); break;
                case FB_G_MAX: a = fmaxf(a, b); break;
                case FB_G_GT: a = a > b ? 1.0f : 0.0f; break;
                case FB_G_GE: a = a >= b ? 1.0f : 0.0f; break;
                case FB_G_LT: a = a < b ? 1.0f : 0.0f; break;
                case FB_G_LE: a = a <= b ? 1.0f : 0.0f; break;
                case FB_G_EQ: a = a == b ? 1.0f : 0.0f; break;
                case FB_G_NE: a = a != b ? 1.0f : 0.0f; break;
                default: break;
            }
            st[sp - 1] = a;
        }
    }
    return sp > 0 ? st[sp - 1] : 0.0f;
}

__device__ __forceinline__ void g_run(const functs_b200_gprogram& P) {
    const int stride = gridDim.x * blockDim.x;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < P.numel; e += stride) {
        int x[8];
        int rem = e;
#pragma unroll
        for (int k = 7; k >= 0; --k) {
            x[k] = 0;
            if (k < P.rank) {
                x[k] = rem % P.shape[k];
                rem /= P.shape[k];
            }
        }
        const float v = g_eval(P, x);
        if (P.out_dtype == 0) static_cast<float*>(P.out_ptr)[e] = v;
        else static_cast<uint8_t*>(P.out_ptr)[e] = v != 0.0f ? 1 : 0;
    }
}

// the program travels as a kernel parameter (constant bank): no device memory, no copy
__global__ void __launch_bounds__(256) generic_group_kernel_param(const __grid_constant__ functs_b200_gprogram P) { g_run(P); }

// several programs (map iterations x outputs) in device memory; the CTA stages its own in shared memory
__global__ void __launch_bounds__(256) generic_group_kernel_table(const functs_b200_gprogram* __restrict__ progs) {
    __shared__ functs_b200_gprogram P;
    const int4* src = reinterpret_cast<const int4*>(progs + blockIdx.y);
    int4* dst = reinterpret_cast<int4*>(&P);
    static_assert(sizeof(functs_b200_gprogram) % 16 == 0, "the program is copied in 16-byte pieces");
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(functs_b200_gprogram) / 16); i += blockDim.x) dst[i] = __ldg(src + i);
    __syncthreads();
    g_run(P);
}

static int validate_program(const functs_b200_gprogram& P) {
    FB_REQUIRE(P.rank >= 0 && P.rank <= 8 && P.numel >= 0 && P.ninstr > 0 && P.ninstr <= FB_G_MAX_INSTR && P.out_ptr != nullptr,
               "generic group: bad program header");
    int64_t n = 1;
    for (int k = 0; k < P.rank; ++k) {
        FB_REQUIRE(P.shape[k] > 0, "generic group: empty or negative extent");
        n *= P.shape[k];
    }
    FB_REQUIRE(n == P.numel, "generic group: numel does not match the shape");
    // static stack-depth and slot check, so that the kernel needs no run-time checks
    FB_REQUIRE(P.instr[P.ninstr - 1].op == FB_G_END, "generic group: the program must end with END");
    for (int pc = 0; pc < P.ninstr; ++pc) {
        const functs_b200_ginstr& I = P.instr[pc];
        if (I.op == FB_G_LOAD) {
            FB_REQUIRE(I.arg < FB_G_MAX_LOADS, "generic group: load slot out of range");
            const functs_b200_gload& L = P.load[I.arg];
            FB_REQUIRE(L.tensor >= 0 && L.tensor < FB_G_MAX_INPUTS && P.in_ptr[L.tensor] != nullptr && L.nterms >= 0 &&
                           L.nterms <= FB_G_MAX_TERMS && L.dtype >= 0 && L.dtype <= 3,
                       "generic group: bad load");
            for (int k = 0; k < L.nterms; ++k)
                FB_REQUIRE(L.term[k].dim >= -1 && L.term[k].dim < P.rank && L.term[k].div >= 1, "generic group: bad load term");
        } else if (I.op == FB_G_COND) {
            FB_REQUIRE(I.arg < FB_G_MAX_PREDS && I.imm.i > pc && I.imm.i < P.ninstr && P.pred[I.arg].dim >= -1 &&
                           P.pred[I.arg].dim < P.rank,
                       "generic group: bad COND");
        } else if (I.op == FB_G_JUMP) {
            FB_REQUIRE(I.arg > pc && I.arg < P.ninstr, "generic group: jumps go forward");
        }
    }
    return FB_OK;
}

}  // namespace fb

extern "C" int functs_b200_generic_group_launch(const functs_b200_gprogram* programs, int32_t count, int32_t max_numel,
                                                int32_t on_device, void* stream) {
    using namespace fb;
    FB_REQUIRE(programs != nullptr && count > 0 && count <= 65535 && max_numel >= 0, "generic group: bad arguments");
    if (max_numel == 0) return FB_OK;
    int64_t need = (static_cast<int64_t>(max_numel) + 255) / 256;
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 8;
    if (need > cap) need = cap;
    cudaStream_t st = as_stream(stream);
    if (!on_device) {
        FB_REQUIRE(count == 1, "generic group: %d programs in host memory (only one can travel as a kernel parameter)", count);
        FB_TRY(validate_program(programs[0]));
        generic_group_kernel_param<<<static_cast<unsigned>(need), 256, 0, st>>>(programs[0]);
    } else {
        FB_REQUIRE((reinterpret_cast<uintptr_t>(programs) & 15) == 0, "generic group: the program table must be 16-byte aligned");
        dim3 grid(static_cast<unsigned>(need), static_cast<unsigned>(count));
        generic_group_kernel_table<<<grid, 256, 0, st>>>(programs);
    }
    count_launch();
    return check_launch("generic_group_kernel");
}
