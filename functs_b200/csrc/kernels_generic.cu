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

__device__ __forceinline__ float g_fetch(const void* p, int dtype, int off) {
    switch (dtype) {
        case 0: return __ldg(static_cast<const float*>(p) + off);
        case 1: return static_cast<float>(__ldg(static_cast<const uint8_t*>(p) + off));
        case 2: return static_cast<float>(__ldg(static_cast<const long long*>(p) + off));
        default: return static_cast<float>(__ldg(static_cast<const int*>(p) + off));
    }
}

// V values of one load: the V elements a thread works on lie kLaneStep apart along the fastest dimension (position
// rank - 1; the lanes of a warp take neighbouring elements, so a warp's load covers one contiguous run), which no
// predicate tests, so their offsets differ by multiples of that dimension's coefficient only.  `last` is the number of
// valid elements minus one (an element beyond the extent re-reads the last valid one; it is never stored).
constexpr int kLaneStep = 32;
template <int R, int V>
__device__ __forceinline__ void g_load(const functs_b200_gprogram& P, const functs_b200_gload& L, const GIndex& ix, int last,
                                       float (&out)[V]) {
    const void* p = P.in_ptr[L.tensor];
    if (L.general == 0) {
        const int off = L.base + g_dot<R>(L.coef, ix);
        int step = 0;
#pragma unroll
        for (int k = 0; k < R; ++k) step = (k == P.rank - 1) ? L.coef[k] : step;
#pragma unroll
        for (int v = 0; v < V; ++v) out[v] = g_fetch(p, L.dtype, off + min(v, last) * (kLaneStep * step));
    } else {  // a coordinate is divided (a read below a strided assignment): term by term, element by element
#pragma unroll
        for (int v = 0; v < V; ++v) {
            GIndex iv = ix;
#pragma unroll
            for (int k = 0; k < R; ++k) iv.x[k] += (k == P.rank - 1) ? kLaneStep * min(v, last) : 0;
            int off = L.base;
            for (int k = 0; k < L.nterms; ++k) {
                const functs_b200_gterm t = L.term[k];
                int c = t.add;
                if (t.dim >= 0) c += t.mul * g_pick<R>(iv, t.dim);
                if (t.div > 1) c /= t.div;
                off += c * t.stride;
            }
            out[v] = g_fetch(p, L.dtype, off);
        }
    }
}

__device__ __forceinline__ float g_unary(int op, float a, float imm) {
    switch (op) {
        case FB_G_EXP: return expf(a);
        case FB_G_SIGMOID: return sigmoid_f32(a);
        case FB_G_TANH: return tanhf(a);
        case FB_G_RELU: return fmaxf(a, 0.0f);
        case FB_G_NEG: return -a;
        case FB_G_CLAMP_MIN: return fmaxf(a, imm);
        case FB_G_CLAMP_MAX: return fminf(a, imm);
        case FB_G_ABS: return fabsf(a);
        case FB_G_SQRT: return sqrtf(a);
        case FB_G_LOG: return logf(a);
        default: return a;
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

// The value stack, V values wide: its top lives in registers, the rest in a small local array, so a chain of loads, unary
// operators and scalar (*_IMM) operators never touches memory.  One pass through the program serves the thread's V
// elements: decoding an instruction and testing a predicate cost the same for one element as for four.
template <int R, int V>
__device__ __forceinline__ void g_eval(const functs_b200_gprogram& P, const GIndex& ix, int last, float (&tos)[V]) {
    float st[FB_G_STACK][V];
#pragma unroll
    for (int v = 0; v < V; ++v) tos[v] = 0.0f;
    int sp = 0;  // values on the stack, the one in `tos` included
    int pc = 0;
    for (int guard = 0; guard < 4 * FB_G_MAX_INSTR; ++guard) {
        const functs_b200_ginstr I = P.instr[pc];
        ++pc;
        const int op = I.op;
        if (op == FB_G_END) break;
        if (op == FB_G_LOAD || op == FB_G_CONST) {
            if (sp > 0) {
#pragma unroll
                for (int v = 0; v < V; ++v) st[sp - 1][v] = tos[v];
            }
            if (op == FB_G_LOAD) {
                g_load<R, V>(P, P.load[I.arg], ix, last, tos);
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) tos[v] = I.imm.f;
            }
            ++sp;
        } else if (op == FB_G_COND) {
            const functs_b200_gpred& q = P.pred[I.arg];
            const int c = q.add + g_dot<R>(q.coef, ix);
            const bool ok = c >= q.lo && c < q.hi && (q.step <= 1 || ((c - q.lo) % q.step) == 0);
            if (!ok) pc = I.imm.i;
        } else if (op == FB_G_JUMP) {
            pc = I.arg;
        } else if (op < FB_G_ADD) {
#pragma unroll
            for (int v = 0; v < V; ++v) tos[v] = g_unary(op, tos[v], I.imm.f);
        } else if (op < FB_G_ADD + FB_G_IMM) {
            --sp;
#pragma unroll
            for (int v = 0; v < V; ++v) tos[v] = g_binary(op, st[sp - 1][v], tos[v]);
        } else if (op == FB_G_RSUB_IMM) {
#pragma unroll
            for (int v = 0; v < V; ++v) tos[v] = __fsub_rn(I.imm.f, tos[v]);
        } else if (op == FB_G_RDIV_IMM) {
#pragma unroll
            for (int v = 0; v < V; ++v) tos[v] = __fdiv_rn(I.imm.f, tos[v]);
        } else {
#pragma unroll
            for (int v = 0; v < V; ++v) tos[v] = g_binary(op - FB_G_IMM, tos[v], I.imm.f);
        }
    }
}

// One work item = V elements of the fastest dimension, kLaneStep apart (V = P.vec): work item q of a row takes elements
// (q / 32) * 32 * V + q % 32 + 32 * v, so the 32 lanes of a warp read and write contiguous runs.  The extent of that
// dimension in `shape` is then the number of work items per row (a multiple of 32), lane_extent the number of elements.
template <int R, int V>
__device__ __forceinline__ void g_run(const functs_b200_gprogram& P) {
    const int stride = gridDim.x * blockDim.x;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < P.work; e += stride) {
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
        int last = 0, ostep = 0;
        if (V > 1) {
            int first = 0;
#pragma unroll
            for (int k = 0; k < R; ++k) {
                if (k == P.rank - 1) {
                    ix.x[k] = (ix.x[k] >> 5) * (kLaneStep * V) + (ix.x[k] & 31);
                    first = ix.x[k];
                    ostep = kLaneStep * P.out_coef[k];
                }
            }
            if (first >= P.lane_extent) continue;  // the row's last block of work items is only partly used
            last = min(V - 1, (P.lane_extent - 1 - first) / kLaneStep);
        }
        float val[V];
        g_eval<R, V>(P, ix, last, val);
        const int o = g_dot<R>(P.out_coef, ix);
#pragma unroll
        for (int v = 0; v < V; ++v) {
            if (v <= last) {
                if (P.out_dtype == 0) static_cast<float*>(P.out_ptr)[o + v * ostep] = val[v];
                else static_cast<uint8_t*>(P.out_ptr)[o + v * ostep] = val[v] != 0.0f ? 1 : 0;
            }
        }
    }
}

// the program travels as a kernel parameter (constant bank): no device memory, no copy.  R = 2, 4, 8: the instantiation
// for programs of rank <= R (index arithmetic is unrolled over R dimensions); V = elements per thread
constexpr int kGenericVec = 4;
template <int R, int V>
__global__ void __launch_bounds__(256) generic_group_kernel_param(const __grid_constant__ functs_b200_gprogram P) { g_run<R, V>(P); }

// several programs (map iterations x outputs) in device memory; the CTA stages its own in shared memory
template <int R>
__global__ void __launch_bounds__(256) generic_group_kernel_table(const functs_b200_gprogram* __restrict__ progs) {
    __shared__ functs_b200_gprogram P;
    const int4* src = reinterpret_cast<const int4*>(progs + blockIdx.y);
    int4* dst = reinterpret_cast<int4*>(&P);
    static_assert(sizeof(functs_b200_gprogram) % 16 == 0, "the program is copied in 16-byte pieces");
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(functs_b200_gprogram) / 16); i += blockDim.x) dst[i] = __ldg(src + i);
    __syncthreads();
    if (P.rank > R) return;  // (the launcher passes the largest rank of the table; a wrong value computes nothing)
    if (P.vec == kGenericVec) g_run<R, kGenericVec>(P);
    else g_run<R, 1>(P);
}

static int validate_program(const functs_b200_gprogram& P) {
    FB_REQUIRE(P.rank >= 0 && P.rank <= 8 && P.numel >= 0 && P.ninstr > 0 && P.ninstr <= FB_G_MAX_INSTR && P.out_ptr != nullptr,
               "generic group: bad program header");
    // `shape` is what the element number is decomposed over; with vec > 1 its last extent counts blocks of vec elements
    // and lane_extent is the true extent of that dimension
    FB_REQUIRE(P.vec == 1 || (P.vec == kGenericVec && P.rank >= 1), "generic group: bad elements-per-thread value");
    int64_t n = 1, w = 1;
    int extent[8] = {1, 1, 1, 1, 1, 1, 1, 1};
    for (int k = 0; k < P.rank; ++k) {
        FB_REQUIRE(P.shape[k] > 0, "generic group: empty or negative extent");
        extent[k] = P.shape[k];
        if (P.vec > 1 && k == P.rank - 1) {
            FB_REQUIRE(P.lane_extent > 0 && P.shape[k] == (P.lane_extent + kLaneStep * P.vec - 1) / (kLaneStep * P.vec) * kLaneStep,
                       "generic group: the work items of the fastest dimension do not match its extent");
            extent[k] = P.lane_extent;
        }
        n *= extent[k];
        w *= P.shape[k];
    }
    FB_REQUIRE(n == P.numel && w == P.work, "generic group: numel / work do not match the shape");
    {
        // out_coef must place the elements one to one into [0, numel): the largest offset is numel - 1 and the
        // coefficients, sorted, are the running products of the extents (a permutation of contiguous strides)
        int64_t top = 0;
        for (int k = 0; k < P.rank; ++k) {
            FB_REQUIRE(P.out_coef[k] >= 0, "generic group: negative output coefficient");
            top += static_cast<int64_t>(P.out_coef[k]) * (extent[k] - 1);
        }
        FB_REQUIRE(top == static_cast<int64_t>(P.numel) - 1, "generic group: the output coefficients do not cover the output");
        bool used[8] = {false, false, false, false, false, false, false, false};
        int64_t run = 1;
        for (int step = 0; step < P.rank; ++step) {
            int pick = -1;
            for (int k = 0; k < P.rank && pick < 0; ++k)
                if (!used[k] && (extent[k] == 1 || P.out_coef[k] == run)) pick = k;
            FB_REQUIRE(pick >= 0, "generic group: the output coefficients are not a permutation of contiguous strides");
            used[pick] = true;
            run *= extent[pick];
        }
    }
    if (P.vec > 1) {  // no predicate may depend on the dimension whose neighbours share one pass through the program
        for (int pc = 0; pc < P.ninstr; ++pc)
            if (P.instr[pc].op == FB_G_COND && P.instr[pc].arg < FB_G_MAX_PREDS)
                FB_REQUIRE(P.pred[P.instr[pc].arg].coef[P.rank - 1] == 0, "generic group: a predicate tests the vectorised dimension");
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

extern "C" int functs_b200_generic_group_launch(const functs_b200_gprogram* programs, int32_t count, int32_t max_work,
                                                int32_t max_rank, int32_t on_device, void* stream) {
    using namespace fb;
    FB_REQUIRE(programs != nullptr && count > 0 && count <= 65535 && max_work >= 0, "generic group: bad arguments");
    if (max_work == 0) return FB_OK;
    int64_t need = (static_cast<int64_t>(max_work) + 255) / 256;
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 8;
    if (need > cap) need = cap;
    cudaStream_t st = as_stream(stream);
    if (!on_device) {
        FB_REQUIRE(count == 1, "generic group: %d programs in host memory (only one can travel as a kernel parameter)", count);
        FB_TRY(validate_program(programs[0]));
        const int rank = programs[0].rank;
        const unsigned g = static_cast<unsigned>(need);
        if (programs[0].vec == kGenericVec) {
            if (rank <= 2) generic_group_kernel_param<2, kGenericVec><<<g, 256, 0, st>>>(programs[0]);
            else if (rank <= 4) generic_group_kernel_param<4, kGenericVec><<<g, 256, 0, st>>>(programs[0]);
            else generic_group_kernel_param<8, kGenericVec><<<g, 256, 0, st>>>(programs[0]);
        } else {
            if (rank <= 2) generic_group_kernel_param<2, 1><<<g, 256, 0, st>>>(programs[0]);
            else if (rank <= 4) generic_group_kernel_param<4, 1><<<g, 256, 0, st>>>(programs[0]);
            else generic_group_kernel_param<8, 1><<<g, 256, 0, st>>>(programs[0]);
        }
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
