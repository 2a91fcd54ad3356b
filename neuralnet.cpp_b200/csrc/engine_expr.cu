// Interpreter for the reference's element-wise expression programs (ExprSpec, expr_spec.hpp:30-180) on
// the device, fp32, reference layout (rows, cols) row-major.  Semantics follow the CPU engine's
// eval_expr_impl (cpu_engine.hpp:1298-1659): reduce views are evaluated first, then every reduce
// instruction in program order (its source replays the element-wise prefix before it over the whole
// grid), then the output pass.  Reductions here combine partial sums in a fixed tree order instead of
// the CPU's ascending loop, so sums agree to fp32 rounding, not bit for bit; Max is exact.
#include "kernels.h"
#include "nnb200.h"

namespace nnb {

enum : int { kOpColSum = 20, kOpColMax = 21, kOpRowSum = 22, kOpRowMax = 23 };
enum : int { kReg = 0, kInput = 1, kConst = 2, kFanout = 3, kReduce = 4 };
enum : int { vLinear = 0, vRotateHalf = 1, vRowMod = 2, vColSum = 3, vColMax = 4, vRowSum = 5, vRowMax = 6, vRowBcast = 7, vColBcast = 8 };

static inline bool op_is_reduce(int op) { return op >= kOpColSum && op <= kOpRowMax; }
static inline bool op_reduces_cols(int op) { return op == kOpColSum || op == kOpColMax; }
static inline int op_operands(int op) { return (op <= 6 || op_is_reduce(op)) ? 1 : (op == 19 ? 3 : 2); }
static inline bool view_is_reduce(int k) { return k >= vColSum && k <= vRowMax; }
static inline bool view_reduces_rows(int k) { return k == vRowSum || k == vRowMax; }

// everything a kernel needs, passed by value (about 1 KB of kernel parameters)
struct DevProg {
    nnb200_expr_program p;
    const float* in[NNB200_EXPR_MAX_INPUTS];
    const float* view_red[NNB200_EXPR_MAX_INPUTS];   // reduce-view vectors (length rows or cols)
    float* reg_red[NNB200_EXPR_MAX_REGS];            // reduce-instruction vectors by destination register
    unsigned char reg_red_cols[NNB200_EXPR_MAX_REGS]; // 1: one scalar per column, 0: one per row
    int rows, cols;
};

__device__ __forceinline__ float read_input(const DevProg& g, int k, int r, int c)
{
    const float* s = g.in[k];
    const size_t cols = g.cols;
    switch (g.p.view_kind[k]) {
    default:
    case vLinear: return s[r * cols + c];
    case vRotateHalf: {
        const int block = static_cast<int>(g.p.view_param[k]), rl = r % block, half = block / 2;
        const int rr = (r / block) * block + (rl < half ? rl + half : rl - half);
        const float v = s[rr * cols + c];
        return (g.p.view_negate[k] && rl < half) ? -v : v;
    }
    case vRowMod: return s[(r % static_cast<int>(g.p.view_param[k])) * cols + c];
    case vRowSum: case vRowMax: return g.view_red[k][r];
    case vColSum: case vColMax: return g.view_red[k][c];
    case vRowBcast: return s[r];
    case vColBcast: return s[c];
    }
}

__device__ __forceinline__ float operand(const DevProg& g, const float* regs, int kind, int idx, int r, int c)
{
    switch (kind) {
    default:
    case kReg: case kFanout: return regs[idx];
    case kConst: return g.p.consts[idx];
    case kInput: return read_input(g, idx, r, c);
    case kReduce: return g.reg_red[idx][g.reg_red_cols[idx] ? c : r];
    }
}

// run the element-wise instructions [0, upto) for element (r, c); reduce instructions are skipped
__device__ __forceinline__ void run_prefix(const DevProg& g, float* regs, int upto, int r, int c)
{
    for (int j = 0; j < upto; ++j) {
        const unsigned char* I = g.p.instrs[j];
        const int op = I[0];
        if (op >= kOpColSum) continue;
        const float a = operand(g, regs, I[2], I[3], r, c);
        float b = 0.f;
        if (op >= 7) b = operand(g, regs, I[4], I[5], r, c);
        float v;
        switch (op) {
        case 0: v = -a; break;
        case 1: v = expf(a); break;
        case 2: v = logf(a); break;
        case 3: v = sqrtf(a); break;
        case 4: v = 1.0f / sqrtf(a); break;
        case 5: v = fabsf(a); break;
        case 6: v = tanhf(a); break;
        case 7: v = a + b; break;
        case 8: v = a - b; break;
        case 9: v = a * b; break;
        case 10: v = a / b; break;
        case 11: v = (a < b) ? b : a; break;          // std::max(a, b)
        case 12: v = (b < a) ? b : a; break;          // std::min(a, b)
        case 13: v = a < b ? 1.f : 0.f; break;
        case 14: v = a <= b ? 1.f : 0.f; break;
        case 15: v = a > b ? 1.f : 0.f; break;
        case 16: v = a >= b ? 1.f : 0.f; break;
        case 17: v = a == b ? 1.f : 0.f; break;
        case 18: v = a != b ? 1.f : 0.f; break;
        case 19: v = (a != 0.f) ? b : operand(g, regs, I[6], I[7], r, c); break;
        default: continue;
        }
        regs[I[1]] = v;
    }
}

// value reduced by pass (mode, idx): mode 0 = reduce view of input idx, mode 1 = reduce instruction idx
__device__ __forceinline__ float reduce_source(const DevProg& g, int mode, int idx, int r, int c)
{
    if (mode == 0) return g.in[idx][static_cast<size_t>(r) * g.cols + c];
    float regs[NNB200_EXPR_MAX_REGS];
#pragma unroll
    for (int i = 0; i < NNB200_EXPR_MAX_REGS; ++i) regs[i] = 0.f;
    run_prefix(g, regs, idx, r, c);
    const unsigned char* I = g.p.instrs[idx];
    return operand(g, regs, I[2], I[3], r, c);
}

constexpr float kLowest = -3.402823466e38f;   // std::numeric_limits<float>::lowest(), the CPU engine's Max seed

// one warp per row: lanes stride the columns, then a butterfly
__global__ void __launch_bounds__(256)
expr_row_reduce_kernel(DevProg g, int mode, int idx, int is_max, float* __restrict__ dst)
{
    const int lane = threadIdx.x & 31, r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= g.rows) return;
    float acc = is_max ? kLowest : 0.f;
    for (int c = lane; c < g.cols; c += 32) {
        const float v = reduce_source(g, mode, idx, r, c);
        acc = is_max ? fmaxf(acc, v) : acc + v;
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, acc, s);
        acc = is_max ? fmaxf(acc, o) : acc + o;
    }
    if (lane == 0) dst[r] = acc;
}

// a block owns 32 columns; 8 row lanes stride the rows and meet in shared memory
__global__ void __launch_bounds__(256)
expr_col_reduce_kernel(DevProg g, int mode, int idx, int is_max, float* __restrict__ dst)
{
    __shared__ float red[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5, c = blockIdx.x * 32 + tx;
    float acc = is_max ? kLowest : 0.f;
    if (c < g.cols)
        for (int r = ty; r < g.rows; r += 8) {
            const float v = reduce_source(g, mode, idx, r, c);
            acc = is_max ? fmaxf(acc, v) : acc + v;
        }
    red[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && c < g.cols) {
        for (int k = 1; k < 8; ++k) acc = is_max ? fmaxf(acc, red[k][tx]) : acc + red[k][tx];
        dst[c] = acc;
    }
}

// output pass.  shape 0: (rows, cols); 1: (rows, 1) evaluated at column 0; 2: (1, cols) evaluated at row 0
__global__ void __launch_bounds__(256)
expr_output_kernel(DevProg g, int shape, float* __restrict__ out)
{
    const long long n = shape == 0 ? static_cast<long long>(g.rows) * g.cols : (shape == 1 ? g.rows : g.cols);
    const int last = static_cast<int>(g.p.num_instrs) - 1;
    const unsigned char* L = g.p.instrs[last];
    const bool last_reduce = L[0] >= kOpColSum;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = shape == 0 ? static_cast<int>(i / g.cols) : (shape == 1 ? static_cast<int>(i) : 0);
        const int c = shape == 0 ? static_cast<int>(i % g.cols) : (shape == 1 ? 0 : static_cast<int>(i));
        float v;
        if (last_reduce) {
            v = g.reg_red[L[1]][g.reg_red_cols[L[1]] ? c : r];
        } else {
            float regs[NNB200_EXPR_MAX_REGS];
#pragma unroll
            for (int k = 0; k < NNB200_EXPR_MAX_REGS; ++k) regs[k] = 0.f;
            run_prefix(g, regs, last + 1, r, c);
            v = regs[L[1]];
        }
        out[i] = v;
    }
}

static int fail(const char* what)
{
    fprintf(stderr, "nnb200_eval_expr: %s\n", what);
    return -1;
}

// the checks of validate_expr_spec (expr_spec.hpp:330-412), on the flat program
static int validate(const nnb200_expr_program& p)
{
    if (p.num_instrs == 0) return fail("empty instruction list");
    if (p.num_instrs > NNB200_EXPR_MAX_INSTRS) return fail("too many instructions");
    if (p.num_regs == 0 || p.num_regs > NNB200_EXPR_MAX_REGS) return fail("invalid num_regs");
    if (p.num_inputs > NNB200_EXPR_MAX_INPUTS) return fail("too many inputs");
    if (p.num_consts > NNB200_EXPR_MAX_CONSTS) return fail("too many constants");
    bool reduce_dst[NNB200_EXPR_MAX_REGS] = {}, elem_dst[NNB200_EXPR_MAX_REGS] = {};
    for (unsigned i = 0; i < p.num_instrs; ++i) {
        const unsigned char* I = p.instrs[i];
        const int op = I[0], dst = I[1];
        if (op > kOpRowMax) return fail("unknown operator");
        if (dst >= static_cast<int>(p.num_regs)) return fail("dst reg out of range");
        const bool red = op_is_reduce(op);
        (red ? reduce_dst : elem_dst)[dst] = true;
        for (int o = 0; o < op_operands(op); ++o) {
            const int kind = I[2 + 2 * o], idx = I[3 + 2 * o];
            if ((kind == kReg || kind == kFanout) && idx >= static_cast<int>(p.num_regs)) return fail("src reg out of range");
            if (kind == kInput && idx >= static_cast<int>(p.num_inputs)) return fail("input index out of range");
            if (kind == kConst && idx >= static_cast<int>(p.num_consts)) return fail("const index out of range");
            if (kind == kReduce) {
                if (idx >= static_cast<int>(p.num_regs)) return fail("reduce ref out of range");
                if (idx == dst) return fail("reduce self-reference");
                if (!reduce_dst[idx] || elem_dst[idx]) return fail("Reduce operand must reference a prior reduce instruction");
            } else if ((kind == kReg || kind == kFanout) && reduce_dst[idx]) {
                return fail("register ref to reduce dst (use Reduce operand)");
            }
        }
    }
    return 0;
}

static int reduce_axis(const nnb200_expr_program& p)
{
    int axis = -1;
    for (unsigned k = 0; k < p.num_inputs; ++k) {
        if (!view_is_reduce(p.view_kind[k])) continue;
        const int a = view_reduces_rows(p.view_kind[k]) ? 0 : 1;
        if (axis == -1) axis = a; else if (axis != a) return -2;
    }
    for (unsigned i = 0; i < p.num_instrs; ++i) {
        if (!op_is_reduce(p.instrs[i][0])) continue;
        const int a = op_reduces_cols(p.instrs[i][0]) ? 1 : 0;
        if (axis == -1) axis = a; else if (axis != a) return -2;
    }
    return axis;
}

// vector output evaluates one representative element per row / column: every input the output chain
// reads directly must be a reduce or broadcast view (cpu_engine.hpp:1590-1630)
static int check_vector_chain(const nnb200_expr_program& p)
{
    bool needed[NNB200_EXPR_MAX_REGS] = {};
    needed[p.instrs[p.num_instrs - 1][1]] = true;
    for (int i = static_cast<int>(p.num_instrs) - 1; i >= 0; --i) {
        const unsigned char* I = p.instrs[i];
        if (!needed[I[1]] || op_is_reduce(I[0])) continue;
        for (int o = 0; o < op_operands(I[0]); ++o) {
            const int kind = I[2 + 2 * o], idx = I[3 + 2 * o];
            if (kind == kInput) {
                const int vk = p.view_kind[idx];
                if (!view_is_reduce(vk) && vk != vRowBcast && vk != vColBcast)
                    return fail("vector output reads an input through a non-reduce view: not constant along the reduced axis");
            } else if (kind == kReg || kind == kFanout || kind == kReduce) {
                needed[idx] = true;
            }
        }
    }
    return 0;
}

}  // namespace nnb

using namespace nnb;

extern "C" {

int nnb200_expr_reduce_axis(const nnb200_expr_program* prog) { return prog ? reduce_axis(*prog) : -2; }

size_t nnb200_eval_expr_scratch_floats(int rows, int cols)
{
    const size_t len = static_cast<size_t>(rows > cols ? rows : cols);
    return (NNB200_EXPR_MAX_INPUTS + NNB200_EXPR_MAX_REGS) * ((len + 63) / 64 * 64);
}

int nnb200_eval_expr(const nnb200_expr_program* prog, const float* const* inputs, const int* input_rows, const int* input_cols,
                     float* out, float* scratch, int rows, int cols, int vector_out, void* stream)
{
    if (!prog || rows < 0 || cols < 0) return fail("bad arguments");
    const nnb200_expr_program& p = *prog;
    if (validate(p)) return -1;
    const int axis = vector_out ? reduce_axis(p) : -1;
    if (vector_out && axis != 0 && axis != 1) return fail("vector output needs a pure row or pure column reduction");
    for (unsigned k = 0; k < p.num_inputs; ++k) {
        const int ir = input_rows[k], ic = input_cols[k];
        const unsigned prm = p.view_param[k];
        switch (p.view_kind[k]) {
        case vRotateHalf:
            if (ir != rows || ic != cols || prm == 0 || rows % prm != 0 || prm % 2 != 0) return fail("RotateHalf shape/param invalid");
            break;
        case vRowMod:
            if (prm == 0 || ir != static_cast<int>(prm) || ic != cols || rows % prm != 0) return fail("RowMod shape/param invalid");
            break;
        case vRowBcast:
            if (ir != rows || ic != 1) return fail("RowBroadcast input must be (rows,1)");
            break;
        case vColBcast:
            if (ir != 1 || ic != cols) return fail("ColBroadcast input must be (1,cols)");
            break;
        default:
            if (ir != rows || ic != cols) return fail("Linear/reduce input shape mismatch");
            break;
        }
    }
    if (static_cast<long long>(rows) * cols == 0) return 0;
    if (vector_out && p.instrs[p.num_instrs - 1][0] < kOpColSum && check_vector_chain(p)) return -1;

    cudaStream_t s = to_stream(stream);
    DevProg g{};
    g.p = p;
    g.rows = rows;
    g.cols = cols;
    const size_t slot = (static_cast<size_t>(rows > cols ? rows : cols) + 63) / 64 * 64;
    for (unsigned k = 0; k < p.num_inputs; ++k) {
        g.in[k] = inputs[k];
        g.view_red[k] = scratch + k * slot;
    }
    for (int r = 0; r < NNB200_EXPR_MAX_REGS; ++r) g.reg_red[r] = scratch + (NNB200_EXPR_MAX_INPUTS + r) * slot;

    auto launch_reduce = [&](int mode, int idx, bool by_cols, bool is_max, float* dst) -> int {
        if (by_cols) expr_col_reduce_kernel<<<static_cast<unsigned>(ceil_div(cols, 32)), 256, 0, s>>>(g, mode, idx, is_max, dst);
        else expr_row_reduce_kernel<<<static_cast<unsigned>(ceil_div(rows, 8)), 256, 0, s>>>(g, mode, idx, is_max, dst);
        NNB_LAUNCH_CHECK();
        return 0;
    };
    for (unsigned k = 0; k < p.num_inputs; ++k) {
        const int vk = p.view_kind[k];
        if (!view_is_reduce(vk)) continue;
        NNB_TRY(launch_reduce(0, static_cast<int>(k), !view_reduces_rows(vk), vk == vColMax || vk == vRowMax, scratch + k * slot));
    }
    for (unsigned i = 0; i < p.num_instrs; ++i) {
        const int op = p.instrs[i][0], dst = p.instrs[i][1];
        if (!op_is_reduce(op)) continue;
        g.reg_red_cols[dst] = op_reduces_cols(op) ? 1 : 0;
        NNB_TRY(launch_reduce(1, static_cast<int>(i), op_reduces_cols(op), op == kOpColMax || op == kOpRowMax, g.reg_red[dst]));
    }
    const int shape = vector_out ? (axis == 0 ? 1 : 2) : 0;
    const long long n = shape == 0 ? static_cast<long long>(rows) * cols : (shape == 1 ? rows : cols);
    expr_output_kernel<<<grid_for(n, 256), 256, 0, s>>>(g, shape, out);
    NNB_LAUNCH_CHECK();
    return 0;
}

}  // extern "C"
