// The rotated ternary format (Bonsai 2): MLX affine 2-bit codes in groups of 128 with an fp16 scale and bias = -scale,
// i.e. w = (q - 1) * s with q in {0, 1, 2}; only the scale is stored. The weights live in a rotated basis: before each
// matrix the activations go through x <- H_1024(x * signs) / 32 per block of 1024 inputs (normalised Sylvester
// Walsh-Hadamard), and the embedding applies the inverse to a table row.
//
// Replaces, on sm_100a, had_rows_h, embed_rows_t and vnax_qmvt* of the reference (Shaders/xc_tern.metal:29-65, 110-230;
// launcher Layers/Linear.swift:298-349). The prefill GEMM of the format is the tcgen05 kernel with a ternary
// dequantiser (csrc/qmm_tc.cuh). The kernels here are small: a 4096 x 4096 ternary matrix is 4 MB.
#include "common.cuh"
#include "internal.h"

namespace iq {
namespace {

// Unnormalised Walsh-Hadamard transform of 1024 floats in shared memory by 256 threads, in the reference's butterfly
// order (span 1, 2, 4, ...: a + b and a - b), so that the fp32 results are the CPU rule's bits
// (Tests/IngotTests/KernelHarness.swift:196-210).
__device__ __forceinline__ void fwht1024(float* sh, int tid) {
    for (int h = 1; h < 1024; h <<= 1) {
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const int pidx = tid + 256 * q;                      // 512 butterflies per stage
            const int j = ((pidx & ~(h - 1)) << 1) | (pidx & (h - 1));
            const float a = sh[j], b = sh[j + h];
            sh[j] = a + b;
            sh[j + h] = a - b;
        }
    }
    __syncthreads();
}

// y[r, block] = half(H(x[r, block] * signs[block]) / 32). Grid (K / 1024, rows), 256 threads.
__global__ void __launch_bounds__(256) had_rows_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx,
                                                      const float* __restrict__ signs, __half* __restrict__ y, int64_t ldy) {
    __shared__ float sh[1024];
    const int tid = threadIdx.x, k0 = blockIdx.x * 1024;
    if (tid < 128) {
        float v[8];
        load_x8(x, x_dtype, (size_t)blockIdx.y * ldx + k0 + tid * 8, v);
#pragma unroll
        for (int e = 0; e < 8; e++) sh[tid * 8 + e] = v[e] * signs[k0 + tid * 8 + e];
    }
    fwht1024(sh, tid);
    for (int i = tid; i < 1024; i += 256) y[(size_t)blockIdx.y * ldy + k0 + i] = __float2half_rn(sh[i] * (1.0f / 32.0f));
}

// Ternary embedding: row tokens[r] dequantised, inverse rotation (H / 32, then the signs), fp32 and / or fp16 out.
// One block of 256 threads per output row; a token outside the table gives a zero row.
__global__ void __launch_bounds__(256) embed_rows_tern_kernel(const uint32_t* __restrict__ tokens, const uint32_t* __restrict__ w,
                                                             const __half* __restrict__ s, const float* __restrict__ signs,
                                                             float* __restrict__ of, __half* __restrict__ oh, int64_t ldo,
                                                             int vocab, int K) {
    __shared__ float sh[1024];
    const int tid = threadIdx.x, row = blockIdx.x;
    const uint32_t t = tokens[row];
    const bool live = t < (uint32_t)vocab;
    const uint32_t* wr = w + (size_t)(live ? t : 0) * (K / 16);
    const __half* sr = s + (size_t)(live ? t : 0) * (K / 128);
    for (int b0 = 0; b0 < K; b0 += 1024) {
        __syncthreads();
        for (int i = tid; i < 1024; i += 256) {
            const int k = b0 + i;
            const float q = (float)((wr[k / 16] >> (2 * (k % 16))) & 3u) - 1.0f;
            sh[i] = live ? q * __half2float(sr[k / 128]) : 0.f;
        }
        fwht1024(sh, tid);
        for (int i = tid; i < 1024; i += 256) {
            const float v = sh[i] * (1.0f / 32.0f) * signs[b0 + i];
            if (of != nullptr) of[(size_t)row * ldo + b0 + i] = v;
            if (oh != nullptr) oh[(size_t)row * ldo + b0 + i] = __float2half_rn(v);
        }
    }
}

// Decode GEMV: Y[m, n] (+)= sum_k x[m, k] * (q[n, k] - 1) * s[n, k / 128] for up to 16 rows of (already rotated) fp16
// activations. One warp per output feature; a lane takes 16-byte pieces of the row (64 codes, half a scale group): the
// weights are -s, 0, +s, so a piece contributes s * sum_k (q_k - 1) x_k, the inner sum with exact products. The
// activations sit in shared memory as floats, the rows of one input side by side and four floats of padding after every
// 64 inputs, so that the 32 lanes' 16-byte loads (64 inputs apart) fall into different banks. A row's bits do not
// depend on the other rows.
constexpr int kTernWarps = 8;
struct TernParams {
    const __half* x;
    int64_t ldx;
    const uint32_t* w;
    const __half* s;
    void* y;
    int32_t y_dtype;
    int64_t ldy;
    int32_t M, N, K, accumulate;
    int32_t kt;  // inputs staged at a time (a multiple of 64)
};

template <int MH>  // activation rows handled per pass: 8 * MH >= M
__global__ void __launch_bounds__(kTernWarps * 32) tern_qmv_kernel(const TernParams p) {
    extern __shared__ __align__(16) float xs[];  // input k, row m at k * MR + (k / 64) * 4 + m
    constexpr int MR = 8 * MH;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = blockIdx.x * kTernWarps + warp;
    const bool n_ok = n < p.N;
    const uint4* wr = reinterpret_cast<const uint4*>(p.w + (size_t)(n_ok ? n : 0) * (p.K / 16));
    const __half* sr = p.s + (size_t)(n_ok ? n : 0) * (p.K / 128);
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; m++) acc[m] = 0.f;
    for (int k0 = 0; k0 < p.K; k0 += p.kt) {  // K in tiles that fit shared memory
    const int klen = min(p.kt, p.K - k0);
    __syncthreads();
    for (int i = tid; i < klen * MR; i += kTernWarps * 32) {
        const int k = i / MR, m = i % MR;
        xs[k * MR + (k >> 6) * 4 + m] = m < p.M ? __half2float(p.x[(size_t)m * p.ldx + k0 + k]) : 0.f;
    }
    __syncthreads();
    if (!n_ok) continue;
    for (int cl = lane; cl < klen / 64; cl += 32) {
        const int c = k0 / 64 + cl;
        const uint4 q4 = ldg_nc_u4(wr + c);
        const float sc = __half2float(sr[c >> 1]);
        const uint32_t words[4] = {q4.x, q4.y, q4.z, q4.w};
        float part[MR];
#pragma unroll
        for (int m = 0; m < MR; m++) part[m] = 0.f;
#pragma unroll
        for (int wi = 0; wi < 4; wi++) {
#pragma unroll
            for (int e = 0; e < 16; e++) {
                const float sgn = (float)((words[wi] >> (2 * e)) & 3u) - 1.0f;  // -1, 0, +1
                const float* xk = xs + (size_t)(cl * 64 + wi * 16 + e) * MR + cl * 4;
#pragma unroll
                for (int m = 0; m < MR; m += 4) {
                    const float4 xv = *reinterpret_cast<const float4*>(xk + m);
                    part[m] = fmaf(sgn, xv.x, part[m]);
                    part[m + 1] = fmaf(sgn, xv.y, part[m + 1]);
                    part[m + 2] = fmaf(sgn, xv.z, part[m + 2]);
                    part[m + 3] = fmaf(sgn, xv.w, part[m + 3]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MR; m++) acc[m] = fmaf(sc, part[m], acc[m]);
    }
    }
    if (!n_ok) return;
#pragma unroll
    for (int m = 0; m < MR; m++) {
        float v = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && m < p.M) {
            const size_t o = (size_t)m * p.ldy + n;
            if (p.y_dtype == kF32) {
                float* yp = reinterpret_cast<float*>(p.y) + o;
                *yp = p.accumulate ? *yp + v : v;
            } else if (p.y_dtype == kF16) {
                __half* yp = reinterpret_cast<__half*>(p.y) + o;
                *yp = __float2half_rn(p.accumulate ? __half2float(*yp) + v : v);
            } else {
                uint16_t* yp = reinterpret_cast<uint16_t*>(p.y) + o;
                *yp = (uint16_t)f32_to_bf16_bits(p.accumulate ? bf16_bits_to_f32(*yp) + v : v);
            }
        }
    }
}

}  // namespace

// The GEMV of the ternary format (called by iq_qmv for bits = 2, group = 128). x must be fp16 (the rotation's output).
int32_t launch_tern_qmv(iq_ctx* ctx, cudaStream_t st, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* m, void* y,
                        int32_t y_dtype, int64_t ldy, int32_t rows, int32_t n, int32_t accumulate) {
    if (x_dtype != kF16)
        return fail(ctx, kErrInvalidArg, "qmv: ternary weights take fp16 activations (the output of iq_had_rows)");
    if (m->k % 128 != 0) return fail(ctx, kErrInvalidArg, "qmv: ternary k = %d must be a multiple of 128", m->k);
    if ((reinterpret_cast<uintptr_t>(m->w) & 15) != 0) return fail(ctx, kErrInvalidArg, "qmv: ternary codes must be 16-byte aligned");
    TernParams p;
    p.x = static_cast<const __half*>(x); p.ldx = ldx;
    p.w = static_cast<const uint32_t*>(m->w); p.s = static_cast<const __half*>(m->scales);
    p.y = y; p.y_dtype = y_dtype; p.ldy = ldy;
    p.M = rows; p.N = n; p.K = m->k; p.accumulate = accumulate;
    const int mh = rows > 8 ? 2 : 1;
    p.kt = m->k < 4096 / mh ? m->k : 4096 / mh;  // 128 KB of staged activations at most (K is a multiple of 128)
    const size_t smem = ((size_t)p.kt * 8 * mh + (size_t)p.kt / 64 * 4) * sizeof(float);
    const unsigned grid = (unsigned)((n + kTernWarps - 1) / kTernWarps);
    if (mh == 1) tern_qmv_kernel<1><<<grid, kTernWarps * 32, smem, st>>>(p);
    else tern_qmv_kernel<2><<<grid, kTernWarps * 32, smem, st>>>(p);
    return check_cuda(ctx, cudaGetLastError(), "tern_qmv launch");
}

int32_t tern_init(iq_ctx* ctx) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(tern_qmv_kernel<1>),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(reinterpret_cast<const void*>(tern_qmv_kernel<2>), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 200 * 1024);
    return check_cuda(ctx, e, "cudaFuncSetAttribute(tern_qmv)");
}

}  // namespace iq

using namespace iq;

extern "C" int32_t iq_had_rows(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const float* signs,
                               void* y_f16, int64_t ldy, int32_t rows, int32_t k) {
    if (ctx == nullptr) return kErrInvalidArg;
    if (x == nullptr || signs == nullptr || y_f16 == nullptr || rows < 1 || k < 1024 || k % 1024 != 0 || ldx < k || ldy < k ||
        ldx % 8 != 0 || x_dtype < 0 || x_dtype > 2 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
        return fail(ctx, kErrInvalidArg, "had_rows: rows = %d, k = %d (a multiple of 1024), ldx / ldy >= k, x 16-byte aligned",
                    rows, k);
    had_rows_kernel<<<dim3(k / 1024, rows), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        x, x_dtype, ldx, signs, static_cast<__half*>(y_f16), ldy);
    return check_cuda(ctx, cudaGetLastError(), "had_rows launch");
}

extern "C" int32_t iq_embed_rows_ternary(iq_ctx* ctx, void* stream, const iq_qlinear* table, const float* signs,
                                         const uint32_t* tokens, int32_t rows, float* out_f32, void* out_f16, int64_t ldo) {
    if (ctx == nullptr) return kErrInvalidArg;
    if (table == nullptr || table->w == nullptr || table->scales == nullptr || signs == nullptr || tokens == nullptr ||
        (out_f32 == nullptr && out_f16 == nullptr))
        return fail(ctx, kErrInvalidArg, "embed_rows_ternary: null pointer");
    if (table->bits != 2 || table->group != 128 || table->mode != IQ_MODE_AFFINE)
        return fail(ctx, kErrUnsupported, "embed_rows_ternary: the table must be 2-bit, group 128");
    if (rows < 1 || table->n < 1 || table->k < 1024 || table->k % 1024 != 0 || ldo < table->k)
        return fail(ctx, kErrInvalidArg, "embed_rows_ternary: rows = %d, k = %d (a multiple of 1024), ldo = %lld", rows, table->k,
                    (long long)ldo);
    embed_rows_tern_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        tokens, static_cast<const uint32_t*>(table->w), static_cast<const __half*>(table->scales), signs, out_f32,
        static_cast<__half*>(out_f16), ldo, table->n, table->k);
    return check_cuda(ctx, cudaGetLastError(), "embed_rows_ternary launch");
}
