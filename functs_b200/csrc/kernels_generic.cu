// Generic fusion group: one precompiled kernel that evaluates, per output element, the postfix program the host made of
// a fusion group's subgraph (program format: include/functs_b200.h).  It stands where the reference JIT-compiles a
// kernel per group (fait/fuser/graph_builder.cpp:259-712, fait/tensorexpr/cuda_codegen_tssa.cpp:1319-1414): the gather
// expression is the same, only it is interpreted instead of generated.  Map iterations and group outputs sit on
// blockIdx.y (the reference puts map iterations there as well, functor_parallization.cpp:83-111).
#include "common.cuh"

namespace fb {

// the element's multi-index stays in registers: every access to it is unrolled over the eight possible dimensions
struct GIndex {
    int x[8];
};

// R: the largest rank the instantiation serves (coefficients and indices beyond the program's rank are zero)
template <int R>
__device__ __forceinline__ int g_dot(const int32_t (&coef)[8], const GIndex& ix) {
    int v = 0;
#pragma unroll
    for (int k = 0; k < R; ++k) v += coef[k] * ix.x[k];
    return v;
}

template <int R>
__device__ __forceinline__ int g_pick(const GIndex& ix, int dim) {
    int v = 0;
#pragma unroll
    for (int k = 0; k < R; ++k) v = (k == dim) ? ix.x[k] : v;
    return v;
}

template <int R>
__device__ __forceinline__ float g_load(const functs_b200_gprogram& P, const functs_b200_gload& L, const GIndex& ix) {
    int off = L.base;
    if (L.general == 0) {
        off += g_dot<R>(L.coef, ix);
    } else {  // a coordinate is divided (a read below a strided assignment): term by term
        for (int k = 0; k < L.nterms; ++k) {
            const functs_b200_gterm t = L.term[k];
            int v = t.add;
            if (t.dim >= 0) v += t.mul * g_pick<R>(ix, t.dim);
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

__device__ __forceinline__ float g_binary(int op, float a, float b) {
    switch (op) {
        case FB_G_ADD: return __fadd_rn(a, b);
        case FB_G_SUB: return __fsub_rn(a, b);
        case FB_G_MUL: return __fmul_rn(a, b);
        case FB_G_DIV: return __fdiv_rn(a, b);
        case FB_G_MIN: return fminf(a, b);
        case FB_G_MAX: return fmaxf(a, b);
        case FB_G_GT: return a > b ? 1.0f : 0.0f;
        case FB_G_GE: return a >= b ? 1.0f : 0.0f;
        case FB_G_LT: return a < b ? 1.0f : 0.0f;
        case FB_G_LE: return a <= b ? 1.0f : 0.0f;
        case FB_G_EQ: return a == b ? 1.0f : 0.0f;
        case FB_G_NE: return a != b ? 1.0f : 0.0f;
        default: return a;
    }
}

// The value stack: its top lives in a register, the rest in a small local array, so a chain of loads, unary operators and
// scalar (*_IMM) operators never touches memory.
template <int R>
__device__ __forceinline__ float g_eval(const functs_b200_gprogram& P, const GIndex& ix) {
    float st[FB_G_STACK];
    float tos = 0.0f;
    int sp = 0;  // values on the stack, the one in `tos` included
    int pc = 0;
    for (int guard = 0; guard < 4 * FB_G_MAX_INSTR; ++guard) {
        const functs_b200_ginstr I = P.instr[pc];
        ++pc;
        const int op = I.op;
        if (op == FB_G_END) break;
        if (op == FB_G_LOAD || op == FB_G_CONST) {
            const float v = op == FB_G_LOAD ? g_load<R>(P, P.load[I.arg], ix) : I.imm.f;
            if (sp > 0) st[sp - 1] = tos;
            tos = v;
            ++sp;
        } else if (op == FB_G_COND) {
            const functs_b200_gpred& q = P.pred[I.arg];
            const int v = q.add + g_dot<R>(q.coef, ix);
            const bool ok = v >= q.lo && v < q.hi && (q.step <= 1 || ((v - q.lo) % q.step) == 0);
            if (!ok) pc = I.imm.i;
        } else if (op == FB_G_JUMP) {
            pc = I.arg;
        } else if (op < FB_G_ADD) {
            float a = tos;
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
            tos = a;
        } else if (op < FB_G_ADD + FB_G_IMM) {
            const float b = tos;
            --sp;
            tos = g_binary(op, st[sp - 1], b);
        } else if (op == FB_G_RSUB_IMM) {
            tos = __fsub_rn(I.imm.f, tos);
        } else if (op == FB_G_RDIV_IMM) {
            tos = __fdiv_rn(I.imm.f, tos);
        } else {
            tos = g_binary(op - FB_G_IMM, tos, I.imm.f);
        }
    }
    return tos;
}

template <int R>
__device__ __forceinline__ void g_run(const functs_b200_gprogram& P) {
    const int stride = gridDim.x * blockDim.x;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < P.numel; e += stride) {
        GIndex ix;
        uint32_t rem = static_cast<uint32_t>(e);
#pragma unroll
        for (int k = 7; k >= 0; --k) {
            ix.x[k] = 0;
            if (k < R && P.shape[k] > 1) {  // (extents beyond the program's rank are zero)
                // multiply-shift division by the extent (magic and shift come from the host)
                const uint32_t hi = __umulhi(P.div_magic[k], rem);
                const uint32_t q = (((rem - hi) >> 1) + hi) >> P.div_shift[k];
                ix.x[k] = static_cast<int>(rem - q * static_cast<uint32_t>(P.shape[k]));
                rem = q;
            }
        }
        const float v = g_eval<R>(P, ix);
        const int o = g_dot<R>(P.out_coef, ix);
        if (P.out_dtype == 0) static_cast<float*>(P.out_ptr)[o] = v;
        else static_cast<uint8_t*>(P.out_ptr)[o] = v != 0.0f ? 1 : 0;
    }
}

// the program travels as a kernel parameter (constant bank): no device memory, no copy.  R = 2, 4, 8: the instantiation
// for programs of rank <= R (index arithmetic is unrolled over R dimensions)
template <int R>
__global__ void __launch_bounds__(256) generic_group_kernel_param(const __grid_constant__ functs_b200_gprogram P) { g_run<R>(P); }

// several programs (map iterations x outputs) in device memory; the CTA stages its own in shared memory
template <int R>
__global__ void __launch_bounds__(256) generic_group_kernel_table(const functs_b200_gprogram* __restrict__ progs) {
    __shared__ functs_b200_gprogram P;
    const int4* src = reinterpret_cast<const int4*>(progs + blockIdx.y);
    int4* dst = reinterpret_cast<int4*>(&P);
    static_assert(sizeof(functs_b200_gprogram) % 16 == 0, "the program is copied in 16-byte pieces");
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(functs_b200_gprogram) / 16); i += blockDim.x) dst[i] = __ldg(src + i);
    __syncthreads();
    if (P.rank <= R) g_run<R>(P);  // (the launcher passes the largest rank of the table; a wrong value computes nothing)
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
    {
        // out_coef must place the elements one to one into [0, numel): the largest offset is numel - 1 and the
        // coefficients, sorted, are the running products of the extents (a permutation of contiguous strides)
        int64_t top = 0;
        for (int k = 0; k < P.rank; ++k) {
            FB_REQUIRE(P.out_coef[k] >= 0, "generic group: negative output coefficient");
            top += static_cast<int64_t>(P.out_coef[k]) * (P.shape[k] - 1);
        }
        FB_REQUIRE(top == static_cast<int64_t>(P.numel) - 1, "generic group: the output coefficients do not cover the output");
        bool used[8] = {false, false, false, false, false, false, false, false};
        int64_t run = 1;
        for (int step = 0; step < P.rank; ++step) {
            int pick = -1;
            for (int k = 0; k < P.rank && pick < 0; ++k)
                if (!used[k] && (P.shape[k] == 1 || P.out_coef[k] == run)) pick = k;
            FB_REQUIRE(pick >= 0, "generic group: the output coefficients are not a permutation of contiguous strides");
            used[pick] = true;
            run *= P.shape[pick];
        }
    }
    for (int k = 0; k < P.rank; ++k) FB_REQUIRE(P.shape[k] == 1 || P.div_shift[k] < 32, "generic group: bad divisor shift");
    // static slot and stack-depth check, so that the kernel needs no run-time checks: jumps go forward, so one pass
    // over the program carries the depth along (depth_at[pc] = depth on arrival through a jump, -1 = none yet)
    FB_REQUIRE(P.instr[P.ninstr - 1].op == FB_G_END, "generic group: the program must end with END");
    int depth_at[FB_G_MAX_INSTR + 1];
    for (int pc = 0; pc <= FB_G_MAX_INSTR; ++pc) depth_at[pc] = -1;
    int depth = 0;
    bool reachable = true;
    for (int pc = 0; pc < P.ninstr; ++pc) {
        if (depth_at[pc] >= 0) {
            FB_REQUIRE(!reachable || depth == depth_at[pc], "generic group: the branches of a COND leave different stack depths");
            depth = depth_at[pc];
            reachable = true;
        }
        FB_REQUIRE(reachable, "generic group: unreachable instruction");
        const functs_b200_ginstr& I = P.instr[pc];
        const int op = I.op;
        if (op == FB_G_END) {
            FB_REQUIRE(depth == 1, "generic group: the program must leave exactly one value");
            reachable = false;
        } else if (op == FB_G_LOAD || op == FB_G_CONST) {
            if (op == FB_G_LOAD) {
                FB_REQUIRE(I.arg < FB_G_MAX_LOADS, "generic group: load slot out of range");
                const functs_b200_gload& L = P.load[I.arg];
                FB_REQUIRE(L.tensor >= 0 && L.tensor < FB_G_MAX_INPUTS && P.in_ptr[L.tensor] != nullptr && L.nterms >= 0 &&
                               L.nterms <= FB_G_MAX_TERMS && L.dtype >= 0 && L.dtype <= 3,
                           "generic group: bad load");
                for (int k = 0; k < L.nterms; ++k)
                    FB_REQUIRE(L.term[k].dim >= -1 && L.term[k].dim < P.rank && L.term[k].div >= 1, "generic group: bad load term");
            }
            ++depth;
            FB_REQUIRE(depth <= FB_G_STACK, "generic group: value stack too deep");
        } else if (op == FB_G_COND) {
            FB_REQUIRE(I.arg < FB_G_MAX_PREDS && I.imm.i > pc && I.imm.i < P.ninstr, "generic group: bad COND");
            FB_REQUIRE(depth_at[I.imm.i] < 0 || depth_at[I.imm.i] == depth, "generic group: inconsistent stack depth at a jump target");
            depth_at[I.imm.i] = depth;
        } else if (op == FB_G_JUMP) {
            FB_REQUIRE(I.arg > pc && I.arg < P.ninstr, "generic group: jumps go forward");
            FB_REQUIRE(depth_at[I.arg] < 0 || depth_at[I.arg] == depth, "generic group: inconsistent stack depth at a jump target");
            depth_at[I.arg] = depth;
            reachable = false;
        } else if (op >= FB_G_EXP && op <= FB_G_LOG) {
            FB_REQUIRE(depth >= 1, "generic group: unary operator on an empty stack");
        } else if (op >= FB_G_ADD && op <= FB_G_NE) {
            FB_REQUIRE(depth >= 2, "generic group: binary operator needs two values");
            --depth;
        } else if ((op >= FB_G_ADD + FB_G_IMM && op <= FB_G_NE + FB_G_IMM) || op == FB_G_RSUB_IMM || op == FB_G_RDIV_IMM) {
            FB_REQUIRE(depth >= 1, "generic group: scalar operator on an empty stack");
        } else {
            FB_REQUIRE(false, "generic group: unknown instruction %d", op);
        }
    }
    return FB_OK;
}

}  // namespace fb

extern "C" int functs_b200_generic_group_launch(const functs_b200_gprogram* programs, int32_t count, int32_t max_numel,
                                                int32_t max_rank, int32_t on_device, void* stream) {
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
        const int rank = programs[0].rank;
        if (rank <= 2) generic_group_kernel_param<2><<<static_cast<unsigned>(need), 256, 0, st>>>(programs[0]);
        else if (rank <= 4) generic_group_kernel_param<4><<<static_cast<unsigned>(need), 256, 0, st>>>(programs[0]);
        else generic_group_kernel_param<8><<<static_cast<unsigned>(need), 256, 0, st>>>(programs[0]);
    } else {
        FB_REQUIRE((reinterpret_cast<uintptr_t>(programs) & 15) == 0, "generic group: the program table must be 16-byte aligned");
        FB_REQUIRE(max_rank >= 0 && max_rank <= 8, "generic group: bad maximum rank");
        dim3 grid(static_cast<unsigned>(need), static_cast<unsigned>(count));
        if (max_rank <= 2) generic_group_kernel_table<2><<<grid, 256, 0, st>>>(programs);
        else if (max_rank <= 4) generic_group_kernel_table<4><<<grid, 256, 0, st>>>(programs);
        else generic_group_kernel_table<8><<<grid, 256, 0, st>>>(programs);
    }
    count_launch();
    return check_launch("generic_group_kernel");
}
