// Token / position embedding forward and its deterministic backward.
//
// Forward fuses what GPTModel::forward builds from transpose + gather_rows + transpose + add
// (compute_layer.hpp:2792-2809, 2535-2548): x[i] = token_emb[id_i] (+ pos_table[i % seq]); an
// out-of-range id gives a zero embedding row (cpu_engine.hpp:150-158).
//
// Backward is scatter_add_rows (compute_layer.hpp:2882-2891): dst[id_i] += g[i].  The CPU engine
// adds rows in ascending i (cpu_engine.hpp:203-214); atomics cannot reproduce that order, so the
// token positions are sorted by (id, i) and each destination row is accumulated by one block that
// walks its segment in ascending i — the fp32 result is bit-identical to the sequential loop.
#include <cmath>

#include "kernels.h"

namespace nnb {

template <typename T>
__global__ void embed_fwd_kernel(const float* __restrict__ tok_emb, const float* __restrict__ pos_table,
                                 const int* __restrict__ tokens, T* __restrict__ x, int n_tok, int seq, int d, int vocab)
{
    const int warps = (gridDim.x * blockDim.x) >> 5, lane = threadIdx.x & 31;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n_tok; i += warps) {
        const int id = tokens[i];
        const bool ok = id >= 0 && id < vocab;
        const float* e = tok_emb + static_cast<size_t>(ok ? id : 0) * d;
        const float* p = pos_table ? pos_table + static_cast<size_t>(i % seq) * d : nullptr;
        T* xr = x + static_cast<size_t>(i) * d;
        if ((d & 3) == 0) {
            for (int c = lane * 4; c < d; c += 128) {
                float4 v = ok ? *reinterpret_cast<const float4*>(e + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                if (p) { const float4 q = *reinterpret_cast<const float4*>(p + c); v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w; }
                xr[c] = from_f32<T>(v.x); xr[c + 1] = from_f32<T>(v.y); xr[c + 2] = from_f32<T>(v.z); xr[c + 3] = from_f32<T>(v.w);
            }
        } else {
            for (int c = lane; c < d; c += 32) xr[c] = from_f32<T>((ok ? e[c] : 0.f) + (p ? p[c] : 0.f));
        }
    }
}


// keys[i] = (id << 32 | i) for valid ids, ~0 for padding / out-of-range ids (ignored by scatter-add)
__global__ void make_keys_kernel(const int* __restrict__ tokens, unsigned long long* __restrict__ keys, int n_tok,
                                 int n_pad, int vocab)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pad) return;
    unsigned long long k = ~0ull;
    if (i < n_tok) { const int id = tokens[i]; if (id >= 0 && id < vocab) k = (static_cast<unsigned long long>(id) << 32) | static_cast<unsigned>(i); }
    keys[i] = k;
}

// one compare-exchange stage of a bitonic sorting network over n_pad (power of two) keys
__global__ void bitonic_stage_kernel(unsigned long long* __restrict__ keys, int n_pad, int k, int j)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pad) return;
    const int partner = i ^ j;
    if (partner > i) {
        const unsigned long long a = keys[i], b = keys[partner];
        const bool up = (i & k) == 0;
        if ((a > b) == up) { keys[i] = b; keys[partner] = a; }
    }
}
// all stages with j < 1024 for one k, inside shared memory (2048 keys per block)
__global__ void __launch_bounds__(1024) bitonic_local_kernel(unsigned long long* __restrict__ keys, int n_pad, int k_begin, int k_end)
{
    __shared__ unsigned long long s[2048];
    const int base = blockIdx.x * 2048;
    for (int t = threadIdx.x; t < 2048; t += 1024) s[t] = (base + t < n_pad) ? keys[base + t] : ~0ull;
    __syncthreads();
    for (int k = k_begin; k <= k_end; k <<= 1) {
        for (int j = min(k >> 1, 1024); j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < 2048; t += 1024) {
                const int partner = t ^ j;
                if (partner > t) {
                    const unsigned long long a = s[t], b = s[partner];
                    const bool up = ((base + t) & k) == 0;
                    if ((a > b) == up) { s[t] = b; s[partner] = a; }
                }
            }
            __syncthreads();
        }
    }
    for (int t = threadIdx.x; t < 2048; t += 1024) if (base + t < n_pad) keys[base + t] = s[t];
}

// Segment heads of the sorted keys.  flags[i] = 0: not the first row of its token id; 1: head of a short segment
// (at most SC_SHORT rows, added by one warp); 2: head of a long segment, whose position is also appended to
// long_list (the order of the list does not matter: each entry is an independent sum).  long_count must be zero.
constexpr int SC_SHORT = 8;
__global__ void segment_heads_kernel(const unsigned long long* __restrict__ keys, int n_pad, int* __restrict__ flags,
                                     int* __restrict__ long_list, int* __restrict__ long_count)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pad) return;
    const unsigned long long k = keys[i];
    const bool valid = k != ~0ull;
    const bool head = valid && (i == 0 || (keys[i - 1] >> 32) != (k >> 32));
    int f = 0;
    if (head) {
        const bool is_long = i + SC_SHORT < n_pad && (keys[i + SC_SHORT] >> 32) == (k >> 32);   // sorted: same id there = more than SC_SHORT rows
        f = is_long ? 2 : 1;
        if (is_long) long_list[atomicAdd(long_count, 1)] = i;
    }
    flags[i] = f;
}

// Short segments: one warp per sorted position; a head's warp adds its at most SC_SHORT rows, in ascending
// position order, into the whole destination row (lanes own 16-byte column chunks).
template <typename T>
__global__ void __launch_bounds__(256)
scatter_short_kernel(float* __restrict__ dst, const unsigned long long* __restrict__ keys, const int* __restrict__ flags,
                     const T* __restrict__ g, int n_pad, int d, int rows_aligned)
{
    constexpr int VN = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int h = static_cast<int>((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5);
    if (h >= n_pad || flags[h] != 1) return;
    const unsigned id = static_cast<unsigned>(keys[h] >> 32);
    unsigned pos[SC_SHORT];
    int count = 0;
#pragma unroll
    for (int r = 0; r < SC_SHORT; ++r) {
        pos[r] = 0;
        if (h + r < n_pad) { const unsigned long long k = keys[h + r]; if (k != ~0ull && static_cast<unsigned>(k >> 32) == id) { pos[r] = static_cast<unsigned>(k); count = r + 1; } }
    }
    float* drow = dst + static_cast<size_t>(id) * d;
    for (int c0 = lane * VN; c0 < d; c0 += 32 * VN) {
        const bool vec_ok = rows_aligned && c0 + VN <= d;
        Vec16<T> v[SC_SHORT];
#pragma unroll
        for (int r = 0; r < SC_SHORT; ++r)
            if (r < count) {
                const T* src = g + static_cast<size_t>(pos[r]) * d + c0;
                if (vec_ok) v[r] = ld16(src);
                else
#pragma unroll
                    for (int k = 0; k < VN; ++k) v[r].v[k] = (c0 + k < d) ? src[k] : from_f32<T>(0.f);
            }
        float acc[VN];
#pragma unroll
        for (int k = 0; k < VN; ++k) acc[k] = (c0 + k < d) ? drow[c0 + k] : 0.f;
#pragma unroll
        for (int r = 0; r < SC_SHORT; ++r)
            if (r < count) {
#pragma unroll
                for (int k = 0; k < VN; ++k) acc[k] += to_f32(v[r].v[k]);
            }
#pragma unroll
        for (int k = 0; k < VN; ++k) if (c0 + k < d) drow[c0 + k] = acc[k];
    }
}

// Long segments.  Work item = (entry of long_list, 128-column slice): a block adds the rows of one token id, in ascending
// position order, into 128 columns of its destination row.  The rows of a segment are fetched 256 at a
// time by all 256 threads (every 16-byte load of the batch in flight together) into shared memory; then
// one thread per column adds the staged values in order, which is the same sequential fp32 sum as the
// CPU loop.  A frequent token (thousands of rows under a Zipf distribution) costs a handful of such
// rounds instead of a serial chain of global-memory round trips.
constexpr int SC_COLS = 128, SC_TILE_BYTES = 65536;   // rows per round = 64 KB / row slice: 256 (bf16) or 128 (fp32)

template <typename T>
__global__ void __launch_bounds__(256)
scatter_segments_kernel(float* __restrict__ dst, const unsigned long long* __restrict__ keys, const int* __restrict__ long_list,
                        const int* __restrict__ long_count, const T* __restrict__ g, int n_pad, int d, int rows_aligned)
{
    constexpr int SC_ROWS = SC_TILE_BYTES / (SC_COLS * static_cast<int>(sizeof(T)));
    constexpr int VN = Vec16<T>::N;                   // elements per 16-byte load
    constexpr int CHUNKS = SC_COLS / VN;              // 16-byte chunks per staged row
    constexpr int ROWS_PER_PASS = 256 / CHUNKS;
    constexpr int PASSES = SC_ROWS / ROWS_PER_PASS;
    extern __shared__ uint8_t sc_smem[];
    T* tile = reinterpret_cast<T*>(sc_smem);          // [SC_ROWS][SC_COLS]
    __shared__ unsigned spos[SC_ROWS];
    __shared__ int s_count;
    static_assert(SC_ROWS <= 256 && SC_ROWS % ROWS_PER_PASS == 0, "one position per thread");
    const int nchunk = (d + SC_COLS - 1) / SC_COLS;
    const long long work_total = static_cast<long long>(*long_count) * nchunk;
    const int my_chunk = threadIdx.x % CHUNKS, my_row = threadIdx.x / CHUNKS;
    for (long long w = blockIdx.x; w < work_total; w += gridDim.x) {
        const int h = long_list[w / nchunk], cc = static_cast<int>(w % nchunk);
        const unsigned id = static_cast<unsigned>(keys[h] >> 32);
        const int c0 = cc * SC_COLS;
        const int c = c0 + threadIdx.x;                            // the column thread t < 128 accumulates
        const bool col_ok = threadIdx.x < SC_COLS && c < d;
        float acc = col_ok ? dst[static_cast<size_t>(id) * d + c] : 0.f;
        const int cv = c0 + my_chunk * VN;                         // first column of the chunk this thread fetches
        const bool vec_ok = rows_aligned && cv + VN <= d;
        for (int base = h;; base += SC_ROWS) {
            __syncthreads();                                       // the previous round's adds are done
            if (threadIdx.x == 0) s_count = SC_ROWS;
            __syncthreads();
            {
                const int pidx = base + threadIdx.x;
                unsigned v = 0xffffffffu;
                if (threadIdx.x < SC_ROWS && pidx < n_pad) { const unsigned long long k = keys[pidx]; if (k != ~0ull && static_cast<unsigned>(k >> 32) == id) v = static_cast<unsigned>(k); }
                if (threadIdx.x < SC_ROWS) {
                    spos[threadIdx.x] = v;
                    // the segment is contiguous in the sorted keys: the first slot that is not ours ends it
                    if (v == 0xffffffffu) atomicMin(&s_count, static_cast<int>(threadIdx.x));
                }
            }
            __syncthreads();
            const int count = s_count;
            Vec16<T> v[PASSES];
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps) {
                const int r = ps * ROWS_PER_PASS + my_row;
                if (r < count) {
                    const T* src = g + static_cast<size_t>(spos[r]) * d + cv;
                    if (vec_ok) v[ps] = ld16(src);
                    else
#pragma unroll
                        for (int k = 0; k < VN; ++k) v[ps].v[k] = (cv + k < d) ? src[k] : from_f32<T>(0.f);
                }
            }
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps) {
                const int r = ps * ROWS_PER_PASS + my_row;
                if (r < count) st16(tile + r * SC_COLS + my_chunk * VN, v[ps]);
            }
            __syncthreads();
            if (col_ok)
                for (int r = 0; r < count; ++r) acc += to_f32(tile[r * SC_COLS + threadIdx.x]);
            if (count < SC_ROWS) break;                            // block-uniform
        }
        if (col_ok) dst[static_cast<size_t>(id) * d + c] = acc;
    }
}

// learned position gradient: pos_grad[t] += g[b*seq + t] for b ascending (scatter_add_rows with the
// cached position indices, compute_layer.hpp:2573-2580)
template <typename T>
__global__ void pos_bwd_kernel(float* __restrict__ pos_grad, const T* __restrict__ g, int batch, int seq, int d)
{
    const size_t n = static_cast<size_t>(seq) * d;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float acc = pos_grad[i];
        for (int b = 0; b < batch; ++b) acc += to_f32(g[static_cast<size_t>(b) * n + i]);
        pos_grad[i] = acc;
    }
}

// Rotary position encoding on the Q and K thirds of a token-major qkv buffer, in place (RotaryEmbedding::apply,
// compute_layer.hpp:926-945): for j < dk/2 of every head, with c, s = table[t][j]
//   forward   x[j] <- x[j] c - x[j+dk/2] s ,  x[j+dk/2] <- x[j+dk/2] c + x[j] s
//   backward  the inverse rotation, applied to the gradients of Q and K
// table: cos (seq, dk/2) then sin (seq, dk/2), fp32, built on the host with the reference's float calls.
template <typename T, int VEC>
__global__ void rope_kernel(T* __restrict__ qkv, const float* __restrict__ table, long long items, int seq, int heads, int dk,
                            long long ld, int backward)
{
    const int half = dk / 2, vph = half / VEC;                 // vectors per half head
    const float* cos_t = table;
    const float* sin_t = table + static_cast<size_t>(seq) * half;
    for (long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; w < items;
         w += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int jv = static_cast<int>(w % vph);
        long long r = w / vph;
        const int h = static_cast<int>(r % heads); r /= heads;
        const int which = static_cast<int>(r % 2);              // 0: Q, 1: K
        const long long tok = r / 2;
        const int t = static_cast<int>(tok % seq), j0 = jv * VEC;
        T* lo = qkv + tok * ld + static_cast<long long>(which) * heads * dk + h * dk + j0;
        T* hi = lo + half;
        float a[VEC], b[VEC];
        if (VEC > 1) {
            const Vec16<T> va = ld16(lo), vb = ld16(hi);
#pragma unroll
            for (int k = 0; k < VEC; ++k) { a[k] = to_f32(va.v[k]); b[k] = to_f32(vb.v[k]); }
        } else { a[0] = to_f32(lo[0]); b[0] = to_f32(hi[0]); }
        Vec16<T> oa, ob;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const float c = cos_t[static_cast<size_t>(t) * half + j0 + k];
            const float sn = backward ? -sin_t[static_cast<size_t>(t) * half + j0 + k] : sin_t[static_cast<size_t>(t) * half + j0 + k];
            oa.v[k] = from_f32<T>(a[k] * c - b[k] * sn);
            ob.v[k] = from_f32<T>(b[k] * c + a[k] * sn);
        }
        if (VEC > 1) { st16(lo, oa); st16(hi, ob); }
        else { lo[0] = oa.v[0]; hi[0] = ob.v[0]; }
    }
}

template <typename T>
int rope_apply(T* qkv, const float* table, int ntok, int seq, int heads, int dk, long long ld, bool backward, cudaStream_t s)
{
    if (ntok == 0) return 0;
    NNB_ARG_CHECK(dk > 0 && dk % 2 == 0, "rotary encoding needs an even head size");      // compute_layer.hpp:929-930
    constexpr int VN = Vec16<T>::N;
    const int half = dk / 2;
    const bool vec = (half % VN) == 0 && (ld % VN) == 0 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0;
    const long long items = static_cast<long long>(ntok) * 2 * heads * (vec ? half / VN : half);
    if (vec) rope_kernel<T, VN><<<grid_for(items, 256), 256, 0, s>>>(qkv, table, items, seq, heads, dk, ld, backward ? 1 : 0);
    else rope_kernel<T, 1><<<grid_for(items, 256), 256, 0, s>>>(qkv, table, items, seq, heads, dk, ld, backward ? 1 : 0);
    NNB_LAUNCH_CHECK();
    return 0;
}
template int rope_apply<float>(float*, const float*, int, int, int, int, long long, bool, cudaStream_t);
template int rope_apply<bf16>(bf16*, const float*, int, int, int, int, long long, bool, cudaStream_t);

// host: the table the kernel reads, computed as RotaryEmbedding::fill_pos_column_ does (compute_layer.hpp:886-902)
void rope_table_host(int seq, int dk, float* out)
{
    const int half = dk / 2;
    for (int pos = 0; pos < seq; ++pos)
        for (int j = 0; j < half; ++j) {
            const float theta = static_cast<float>(pos) / std::pow(10000.0f, static_cast<float>(2 * j) / static_cast<float>(dk));
            out[static_cast<size_t>(pos) * half + j] = std::cos(theta);
            out[static_cast<size_t>(seq) * half + static_cast<size_t>(pos) * half + j] = std::sin(theta);
        }
}

static int next_pow2(int n) { int p = 1; while (p < n) p <<= 1; return p; }

size_t embed_bwd_scratch_bytes(int n_tok)
{
    const size_t n_pad = static_cast<size_t>(next_pow2(n_tok < 2048 ? 2048 : n_tok));
    return n_pad * sizeof(unsigned long long) + 2 * n_pad * sizeof(int) + 16;   // keys, flags, long-segment list, its counter
}

template <typename T>
int embed_fwd(const float* tok_emb, const float* pos_table, const int* tokens, T* x, int n_tok, int seq, int d, int vocab,
              cudaStream_t s)
{
    if (n_tok == 0) return 0;
    embed_fwd_kernel<T><<<grid_for(n_tok, 8), 256, 0, s>>>(tok_emb, pos_table, tokens, x, n_tok, seq, d, vocab);
    NNB_LAUNCH_CHECK();
    return 0;
}


template <typename T>
int embed_bwd(float* tok_grad, float* pos_grad, const int* tokens, const T* g, void* scratch, int batch, int seq, int d,
              int vocab, cudaStream_t s)
{
    const int n_tok = batch * seq;
    if (n_tok == 0) return 0;
    const int n_pad = next_pow2(n_tok < 2048 ? 2048 : n_tok);
    auto* keys = static_cast<unsigned long long*>(scratch);
    int* flags = reinterpret_cast<int*>(keys + n_pad);
    const unsigned blocks = static_cast<unsigned>(ceil_div(n_pad, 256));
    make_keys_kernel<<<blocks, 256, 0, s>>>(tokens, keys, n_tok, n_pad, vocab);
    NNB_LAUNCH_CHECK();
    // bitonic network: k = 2..2048 entirely in shared memory, then global stages for j >= 2048 and
    // a shared-memory tail for j < 2048 of each larger k
    bitonic_local_kernel<<<n_pad / 2048, 1024, 0, s>>>(keys, n_pad, 2, 2048);
    NNB_LAUNCH_CHECK();
    for (int k = 4096; k <= n_pad; k <<= 1) {
        for (int j = k >> 1; j >= 2048; j >>= 1) {
            bitonic_stage_kernel<<<blocks, 256, 0, s>>>(keys, n_pad, k, j);
            NNB_LAUNCH_CHECK();
        }
        bitonic_local_kernel<<<n_pad / 2048, 1024, 0, s>>>(keys, n_pad, k, k);
        NNB_LAUNCH_CHECK();
    }
    int* long_list = flags + n_pad;
    int* long_count = long_list + n_pad;
    NNB_CUDA_CHECK(cudaMemsetAsync(long_count, 0, sizeof(int), s));
    segment_heads_kernel<<<blocks, 256, 0, s>>>(keys, n_pad, flags, long_list, long_count);
    NNB_LAUNCH_CHECK();
    constexpr int sc_smem = SC_TILE_BYTES;
    static PerDeviceOnce sc_attr;
    NNB_TRY(sc_attr.run([] { return cudaFuncSetAttribute(scatter_segments_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, SC_TILE_BYTES); }));
    const int rows_aligned = ((reinterpret_cast<uintptr_t>(g) & 15) == 0 && (static_cast<size_t>(d) * sizeof(T)) % 16 == 0) ? 1 : 0;
    scatter_short_kernel<T><<<static_cast<unsigned>(ceil_div(static_cast<long long>(n_pad) * 32, 256)), 256, 0, s>>>(tok_grad, keys, flags, g, n_pad, d, rows_aligned);
    NNB_LAUNCH_CHECK();
    scatter_segments_kernel<T><<<kSmCount * 3, 256, sc_smem, s>>>(tok_grad, keys, long_list, long_count, g, n_pad, d, rows_aligned);
    NNB_LAUNCH_CHECK();
    if (pos_grad) {
        pos_bwd_kernel<T><<<grid_for(static_cast<long long>(seq) * d, 256), 256, 0, s>>>(pos_grad, g, batch, seq, d);
        NNB_LAUNCH_CHECK();
    }
    return 0;
}

template int embed_fwd<float>(const float*, const float*, const int*, float*, int, int, int, int, cudaStream_t);
template int embed_fwd<bf16>(const float*, const float*, const int*, bf16*, int, int, int, int, cudaStream_t);
template int embed_bwd<float>(float*, float*, const int*, const float*, void*, int, int, int, int, cudaStream_t);
template int embed_bwd<bf16>(float*, float*, const int*, const bf16*, void*, int, int, int, int, cudaStream_t);

// ---------------------------------------------------------------- host-interface helpers
// The reference hands GPTModel::forward its token ids as a (seq, batch) matrix of floats (compute_layer.hpp:2783-2790);
// the fused step wants int32 ids in batch-major order.  out[b*seq + t] = (int) ids[t*batch + b]; a value that is not a
// finite non-negative number becomes -1, which the embedding lookup treats as out of range (zero row).
__global__ void ids_from_float_kernel(const float* __restrict__ ids, int* __restrict__ out, int seq, int batch)
{
    const int n = seq * batch;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int b = i / seq, t = i - b * seq;
        const float v = ids[static_cast<size_t>(t) * batch + b];
        out[i] = (v >= 0.f && v < 2147483520.f) ? static_cast<int>(v) : -1;
    }
}
int ids_from_float(const float* ids, int* out, int seq, int batch, cudaStream_t s)
{
    if (seq <= 0 || batch <= 0) return 0;
    ids_from_float_kernel<<<grid_for(static_cast<long long>(seq) * batch, 256), 256, 0, s>>>(ids, out, seq, batch);
    NNB_LAUNCH_CHECK();
    return 0;
}

// Token-major logits (tokens, vocab) of the fused step -> the reference's (vocab, tokens) fp32 matrix: 32 x 32 tiles
// through shared memory, coalesced on both sides.
template <typename T>
__global__ void logits_to_reference_kernel(const T* __restrict__ in, float* __restrict__ out, int tokens, int vocab)
{
    __shared__ float tile[32][33];
    const int v0 = blockIdx.x * 32, t0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int t = t0 + j, v = v0 + threadIdx.x;
        tile[j][threadIdx.x] = (t < tokens && v < vocab) ? to_f32(in[static_cast<size_t>(t) * vocab + v]) : 0.f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int v = v0 + j, t = t0 + threadIdx.x;
        if (v < vocab && t < tokens) out[static_cast<size_t>(v) * tokens + t] = tile[threadIdx.x][j];
    }
}
template <typename T> int logits_to_reference(const T* in, float* out, int tokens, int vocab, cudaStream_t s)
{
    if (tokens <= 0 || vocab <= 0) return 0;
    const dim3 grid(static_cast<unsigned>(ceil_div(vocab, 32)), static_cast<unsigned>(ceil_div(tokens, 32)));
    NNB_ARG_CHECK(grid.y <= 65535u, "too many token rows for one launch");
    logits_to_reference_kernel<T><<<grid, dim3(32, 8), 0, s>>>(in, out, tokens, vocab);
    NNB_LAUNCH_CHECK();
    return 0;
}
template int logits_to_reference<float>(const float*, float*, int, int, cudaStream_t);
template int logits_to_reference<bf16>(const bf16*, float*, int, int, cudaStream_t);

__global__ void zero_f32_kernel(float4* __restrict__ p4, size_t n4, float* __restrict__ tail, int ntail)
{
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<size_t>(gridDim.x) * blockDim.x) p4[i] = z;
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < ntail) tail[threadIdx.x] = 0.f;
}
// zero_grad over a flat fp32 range (Layer::zero_grad / Optimizer::zero_grad, compute_layer.hpp:57-65): one launch
int zero_f32(float* p, size_t n, cudaStream_t s)
{
    if (n == 0) return 0;
    NNB_ARG_CHECK((reinterpret_cast<uintptr_t>(p) & 15) == 0, "the range must start on a 16-byte boundary");
    const size_t n4 = n / 4;
    zero_f32_kernel<<<grid_for(static_cast<long long>(n4 ? n4 : 1), 256), 256, 0, s>>>(reinterpret_cast<float4*>(p), n4, p + 4 * n4, static_cast<int>(n - 4 * n4));
    NNB_LAUNCH_CHECK();
    return 0;
}

}  // namespace nnb
