// What follows the lm_head GEMV on the decode path: the arg-max of each row of logits, and the 64 best candidates of
// each row with the row's maximum and softmax denominator (what the sampler needs; the rest of the vocabulary never
// leaves the GPU).
//
// Replaces the reference's argmax_rows (Shaders/verify.metal:525-547) and TopK64 (topk64_part + topk64_merge,
// Shaders/zz_sample.metal; contract in Tests/IngotTests/TopK64Tests.swift:8-63): candidates are the logits
// x >= -FLT_MAX, ordered by value descending with ties to the lower id, padded with (id 0xFFFFFFFF, -FLT_MAX); the values
// are the logits' own bits; z[2r] is the row maximum (exact), z[2r+1] = sum_i exp((x_i - max) / T_r).
#include <float.h>
#include <math.h>

#include "internal.h"

namespace iq {
namespace {

constexpr int kTopK = 64;
constexpr int kChunk = 4096;   // logits per part
constexpr int kMaxParts = 64;  // parts per row: up to 262,144 logits
constexpr int kSortThreads = 1024;

// 64-bit sort key: value first (as an unsigned that orders like the float, -0 taken as +0 so that it ties with it),
// then the id inverted, so that one descending sort gives "value descending, lower id first". 0 = not a candidate.
__device__ __forceinline__ unsigned long long make_key(float v, uint32_t id) {
    if (!(v >= -FLT_MAX)) return 0ull;  // -inf and NaN
    uint32_t u = __float_as_uint(v == 0.f ? 0.f : v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - id);
}

// descending bitonic sort of n = 4096 keys in shared memory by 1024 threads
__device__ __forceinline__ void bitonic_desc(unsigned long long* k, int tid) {
    for (int size = 2; size <= kChunk; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int t = tid; t < kChunk / 2; t += kSortThreads) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const unsigned long long a = k[lo], b = k[hi];
                if ((a < b) == desc) { k[lo] = b; k[hi] = a; }
            }
        }
    }
    __syncthreads();
}

struct TopkParams {
    const float* x;
    int64_t ldx;
    int32_t rows, V, parts;
    float inv_t[16];
    unsigned long long* part_keys;  // [rows, parts, 64]
    float* part_mz;                 // [rows, parts, 2] part maximum and sum exp((x - part max) / T)
    uint32_t* idx;                  // [rows, 64]
    float* val;                     // [rows, 64]
    float* z;                       // [rows, 2]
};

__global__ void __launch_bounds__(kSortThreads) topk64_part_kernel(const TopkParams p) {
    __shared__ unsigned long long keys[kChunk];
    __shared__ float red[32];
    const int part = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
    const float* xr = p.x + (size_t)row * p.ldx;
    const int i0 = part * kChunk;
    float m = -INFINITY;
    for (int i = tid; i < kChunk; i += kSortThreads) {
        const int id = i0 + i;
        const float v = id < p.V ? xr[id] : -INFINITY;
        keys[i] = id < p.V ? make_key(v, (uint32_t)id) : 0ull;
        m = fmaxf(m, v);
    }
    // part maximum
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    m = red[0];
    for (int i = 1; i < kSortThreads / 32; i++) m = fmaxf(m, red[i]);
    __syncthreads();
    // sum exp((x - part max) / T) in a fixed order: per thread, warp tree, then the warps in order
    float s = 0.f;
    if (m > -INFINITY) {
        const float it = p.inv_t[row];
        for (int i = tid; i < kChunk; i += kSortThreads) {
            const int id = i0 + i;
            if (id < p.V) s += expf((xr[id] - m) * it);
        }
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((tid & 31) == 0) red[tid >> 5] = s;
    bitonic_desc(keys, tid);  // starts with a barrier
    if (tid == 0) {
        float tot = 0.f;
        for (int i = 0; i < kSortThreads / 32; i++) tot += red[i];
        p.part_mz[((size_t)row * p.parts + part) * 2] = m;
        p.part_mz[((size_t)row * p.parts + part) * 2 + 1] = tot;
    }
    if (tid < kTopK) p.part_keys[((size_t)row * p.parts + part) * kTopK + tid] = keys[tid];
}

__global__ void __launch_bounds__(kSortThreads) topk64_merge_kernel(const TopkParams p) {
    __shared__ unsigned long long keys[kChunk];
    const int row = blockIdx.x, tid = threadIdx.x;
    for (int i = tid; i < kChunk; i += kSortThreads)
        keys[i] = i < p.parts * kTopK ? p.part_keys[(size_t)row * p.parts * kTopK + i] : 0ull;
    bitonic_desc(keys, tid);
    if (tid < kTopK) {
        const unsigned long long k = keys[tid];
        uint32_t id = 0xFFFFFFFFu;
        float v = -FLT_MAX;
        if (k != 0ull) {
            id = 0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull);
            v = p.x[(size_t)row * p.ldx + id];  // the logit's own bits (-0 stays -0)
        }
        p.idx[(size_t)row * kTopK + tid] = id;
        p.val[(size_t)row * kTopK + tid] = v;
    }
    if (tid == 0) {
        float M = -INFINITY;
        for (int q = 0; q < p.parts; q++) M = fmaxf(M, p.part_mz[((size_t)row * p.parts + q) * 2]);
        double Z = 0.0;
        const float it = p.inv_t[row];
        for (int q = 0; q < p.parts; q++) {
            const float mq = p.part_mz[((size_t)row * p.parts + q) * 2];
            if (mq > -INFINITY) Z += (double)p.part_mz[((size_t)row * p.parts + q) * 2 + 1] * exp((double)(mq - M) * (double)it);
        }
        p.z[row * 2] = M;
        p.z[row * 2 + 1] = (float)Z;
    }
}

// arg-max of each row, ties to the lower index (verify.metal:525-547)
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float* __restrict__ x, int64_t ldx, uint32_t* __restrict__ out,
                                                          int N) {
    __shared__ float bv[32];
    __shared__ uint32_t bi[32];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* xr = x + (size_t)row * ldx;
    float m = -INFINITY;
    uint32_t mi = 0;
    for (int i = tid; i < N; i += 1024)
        if (xr[i] > m) { m = xr[i]; mi = (uint32_t)i; }
    float sm = m;
    for (int o = 16; o > 0; o >>= 1) sm = fmaxf(sm, __shfl_xor_sync(0xffffffffu, sm, o));
    uint32_t si = m == sm ? mi : 0xFFFFFFFFu;
    for (int o = 16; o > 0; o >>= 1) si = min(si, __shfl_xor_sync(0xffffffffu, si, o));
    if ((tid & 31) == 0) { bv[tid >> 5] = sm; bi[tid >> 5] = si; }
    __syncthreads();
    if (tid == 0) {
        float b = bv[0];
        uint32_t ix = bi[0];
        for (int i = 1; i < 32; i++)
            if (bv[i] > b || (bv[i] == b && bi[i] < ix)) { b = bv[i]; ix = bi[i]; }
        out[row] = ix;
    }
}

}  // namespace
}  // namespace iq

using namespace iq;

extern "C" int32_t iq_argmax_rows(iq_ctx* ctx, void* stream, const float* x, int64_t ldx, int32_t rows, int32_t n,
                                  uint32_t* out) {
    if (ctx == nullptr) return kErrInvalidArg;
    if (x == nullptr || out == nullptr || rows < 1 || n < 1 || ldx < n) return fail(ctx, kErrInvalidArg, "argmax_rows: arguments");
    argmax_rows_kernel<<<rows, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, ldx, out, n);
    return check_cuda(ctx, cudaGetLastError(), "argmax_rows launch");
}

extern "C" int32_t iq_topk64_scratch_bytes(int32_t rows, int32_t vocab, size_t* bytes) {
    if (bytes == nullptr || rows < 1 || rows > 16 || vocab < 1 || vocab > kChunk * kMaxParts) return kErrInvalidArg;
    const size_t parts = (size_t)(vocab + kChunk - 1) / kChunk;
    *bytes = (size_t)rows * parts * (kTopK * 8 + 2 * 4) + 256;
    return kOk;
}

extern "C" int32_t iq_topk64(iq_ctx* ctx, void* stream, const float* x, int64_t ldx, int32_t rows, int32_t vocab,
                             const float* temperatures, int32_t n_temperatures, uint32_t* idx, float* val, float* z,
                             void* scratch, size_t scratch_bytes) {
    if (ctx == nullptr) return kErrInvalidArg;
    size_t need = 0;
    if (x == nullptr || idx == nullptr || val == nullptr || z == nullptr || temperatures == nullptr || ldx < vocab ||
        (n_temperatures != 1 && n_temperatures != rows) || iq_topk64_scratch_bytes(rows, vocab, &need) != kOk)
        return fail(ctx, kErrInvalidArg, "topk64: arguments (1..16 rows, up to %d logits, one temperature or one per row)",
                    kChunk * kMaxParts);
    if (scratch == nullptr || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 7) != 0)
        return fail(ctx, kErrWorkspace, "topk64: scratch %zu < %zu (8-byte aligned)", scratch_bytes, need);
    TopkParams p;
    p.x = x; p.ldx = ldx; p.rows = rows; p.V = vocab;
    p.parts = (vocab + kChunk - 1) / kChunk;
    for (int r = 0; r < 16; r++) {
        const float t = temperatures[n_temperatures == 1 ? 0 : (r < rows ? r : 0)];
        if (!(t > 0.f)) return fail(ctx, kErrInvalidArg, "topk64: temperature %g", (double)t);
        p.inv_t[r] = 1.0f / t;
    }
    p.part_keys = static_cast<unsigned long long*>(scratch);
    p.part_mz = reinterpret_cast<float*>(p.part_keys + (size_t)rows * p.parts * kTopK);
    p.idx = idx; p.val = val; p.z = z;
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    topk64_part_kernel<<<dim3(p.parts, rows), kSortThreads, 0, cs>>>(p);
    topk64_merge_kernel<<<rows, kSortThreads, 0, cs>>>(p);
    return check_cuda(ctx, cudaGetLastError(), "topk64 launch");
}
