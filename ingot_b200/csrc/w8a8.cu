// Rotated W8A8 prefill GEMM (lossy; the serving path's option for dense prefill): per call, the 4-bit weights and the
// activations are rotated along K by an unnormalised Hadamard transform of n = 32 * 2^lb inputs per contiguous block
// (what spreads outlier channels), quantised to int8 per row (scale max / 127, round half to even), and
// Y = (Xq Wq^T) * sx * sw / n runs on the int8 tensor cores (tcgen05 kind::i8, s32 accumulation in tensor memory).
//
// Replaces w4_i8rot, quant_rows_rot_i8g and qmm_i8 of the reference (Shaders/xa_dense_i8.metal; launcher
// DenseQ.encodeQmmI8, Layers/Dense.swift:99-172). The arithmetic of the two conversion kernels is the CPU emulation's
// (Tests/IngotTests/KernelHarness.swift:225-255), fp32 butterflies in the same order, so the int8 rows are its bits.
#include "common.cuh"
#include "internal.h"

namespace iq {
namespace {

// One block per row: the row's K floats in shared memory, the Hadamard transform of every block of n inputs (spans
// 1, 2, ..., n / 2: a + b and a - b), the row's largest magnitude, then the int8 codes.
// SRC 0: 4-bit affine weights (w, scales, biases; group 64 or 32); SRC 1: activations of any dtype.
template <int SRC>
__global__ void __launch_bounds__(256) rot_quant_rows_kernel(const void* __restrict__ src, const uint16_t* __restrict__ sc,
                                                            const uint16_t* __restrict__ bi, int group, int32_t x_dtype,
                                                            int64_t ld, int K, int n, int8_t* __restrict__ q,
                                                            float* __restrict__ scale_out) {
    extern __shared__ float row[];  // [K]
    __shared__ float wmax[8];
    const int tid = threadIdx.x, r = blockIdx.x;
    if (SRC == 0) {
        const uint32_t* w = static_cast<const uint32_t*>(src) + (size_t)r * (K / 8);
        const size_t g0 = (size_t)r * (K / group);
        for (int i = tid; i < K / 8; i += 256) {
            const uint32_t word = w[i];
            const float s = bf16_bits_to_f32(sc[g0 + i * 8 / group]), b = bf16_bits_to_f32(bi[g0 + i * 8 / group]);
#pragma unroll
            for (int e = 0; e < 8; e++) row[i * 8 + e] = fmaf(s, (float)((word >> (4 * e)) & 15u), b);
        }
    } else {
        for (int i = tid; i < K / 8; i += 256) {
            float v[8];
            load_x8(src, x_dtype, (size_t)r * ld + i * 8, v);
#pragma unroll
            for (int e = 0; e < 8; e++) row[i * 8 + e] = v[e];
        }
    }
    for (int h = 1; h < n; h <<= 1) {
        __syncthreads();
        for (int pidx = tid; pidx < K / 2; pidx += 256) {
            const int j = ((pidx & ~(h - 1)) << 1) | (pidx & (h - 1));  // butterflies never cross a block: n divides K
            const float a = row[j], b = row[j + h];
            row[j] = a + b;
            row[j + h] = a - b;
        }
    }
    __syncthreads();
    float amax = 0.f;
    for (int i = tid; i < K; i += 256) amax = fmaxf(amax, fabsf(row[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((tid & 31) == 0) wmax[tid >> 5] = amax;
    __syncthreads();
    amax = wmax[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, wmax[i]);
    const float s = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    if (tid == 0) scale_out[r] = s;
    for (int i = tid; i < K / 4; i += 256) {
        char4 o;
        int c[4];
#pragma unroll
        for (int e = 0; e < 4; e++) c[e] = max(-127, min(127, __float2int_rn(__fdiv_rn(row[i * 4 + e], s))));
        o.x = (signed char)c[0]; o.y = (signed char)c[1]; o.z = (signed char)c[2]; o.w = (signed char)c[3];
        reinterpret_cast<char4*>(q + (size_t)r * K)[i] = o;
    }
}

// Ternary weights (2-bit codes t + 1, one fp16 scale per group of 128) to int8 with ONE scale per row:
// s_row = max_g |s_g| / 127, code = t * rint(s_g / s_row) (tern_i8row, Shaders/xc_tern.metal:213-237). One warp per
// row, four rows per block.
__global__ void __launch_bounds__(128) tern_i8row_kernel(const uint32_t* __restrict__ w, const __half* __restrict__ s, int N, int K,
                                                        int8_t* __restrict__ q, float* __restrict__ scale_out) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (n >= N) return;
    const int G = K / 128;
    const __half* sr = s + (size_t)n * G;
    float m = 0.f;
    for (int g = lane; g < G; g += 32) m = fmaxf(m, fabsf(__half2float(sr[g])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float srow = m > 0.f ? __fdiv_rn(m, 127.0f) : 1.0f;
    if (lane == 0) scale_out[n] = srow;
    const uint32_t* wr = w + (size_t)n * (K / 16);
    uint4* o = reinterpret_cast<uint4*>(q + (size_t)n * K);  // sixteen codes per word of w
    for (int u = lane; u < K / 16; u += 32) {
        const int qg = __float2int_rn(__fdiv_rn(__half2float(sr[u / 8]), srow));
        const uint32_t x = wr[u];
        uint32_t out[4];
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint32_t word = 0;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int t = (int)((x >> (8 * c + 2 * e)) & 3u) - 1;
                word |= (uint32_t)((t * qg) & 0xFF) << (8 * e);
            }
            out[c] = word;
        }
        o[u] = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// Hadamard of 256 along K when K / 32 is a multiple of 32, else of 32 (DenseI8Scratch.lb, Layers/Dense.swift:107-109).
int rot_block(int K) { return (K / 32) % 32 == 0 ? 256 : 32; }

struct W8a8Ws {
    int8_t* wq;
    float* sw;
    int8_t* xq;
    float* sx;
    size_t bytes;
};
W8a8Ws carve_w8a8(void* base, int N, int K, int rows) {
    size_t off = 0;
    auto take = [&](size_t bytes) {
        void* p = base ? static_cast<char*>(base) + off : nullptr;
        off += round_up_sz(bytes, 256);
        return p;
    };
    W8a8Ws w;
    w.wq = static_cast<int8_t*>(take((size_t)N * K));
    w.sw = static_cast<float*>(take((size_t)N * 4));
    w.xq = static_cast<int8_t*>(take((size_t)rows * K));
    w.sx = static_cast<float*>(take((size_t)rows * 4));
    w.bytes = off;
    return w;
}

int32_t check_w8a8(iq_ctx* ctx, const iq_qlinear* m, int rows) {
    if (m == nullptr || m->w == nullptr || m->scales == nullptr || (m->biases == nullptr && m->bits != 2))
        return fail(ctx, kErrInvalidArg, "qmm_w8a8: null pointer");
    // the reference converts from 4 bits (DenseQ.int8OK: 8-bit layers already have int8 precision) and from the ternary
    // format (DenseQ.encodeQmmI8T)
    const bool tern = m->bits == 2 && m->group == 128;
    if (m->mode != IQ_MODE_AFFINE || m->experts > 1 || !(tern || (m->bits == 4 && (m->group == 64 || m->group == 32))))
        return fail(ctx, kErrUnsupported, "qmm_w8a8: %d-bit group %d mode %d (4-bit affine with group 64 or 32, or ternary)", m->bits,
                    m->group, m->mode);
    if (m->k % 128 != 0 || m->n % 64 != 0 || m->k > 49152)
        return fail(ctx, kErrInvalidArg, "qmm_w8a8: k = %d (a multiple of 128, at most 49152), n = %d (a multiple of 64)", m->k, m->n);
    if (rows < 64 || rows % 64 != 0) return fail(ctx, kErrInvalidArg, "qmm_w8a8: rows = %d must be a multiple of 64", rows);
    return kOk;
}

}  // namespace

int32_t w8a8_init(iq_ctx* ctx) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(rot_quant_rows_kernel<0>),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 49152 * 4);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(reinterpret_cast<const void*>(rot_quant_rows_kernel<1>),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 49152 * 4);
    return check_cuda(ctx, e, "cudaFuncSetAttribute(rot_quant_rows)");
}

}  // namespace iq

using namespace iq;

extern "C" int32_t iq_qmm_w8a8_workspace_bytes(iq_ctx* ctx, const iq_qlinear* m, int32_t rows, size_t* bytes) {
    if (ctx == nullptr || bytes == nullptr) return kErrInvalidArg;
    const int32_t st = check_w8a8(ctx, m, rows);
    if (st != kOk) return st;
    *bytes = carve_w8a8(nullptr, m->n, m->k, rows).bytes;
    return kOk;
}

extern "C" int32_t iq_qmm_w8a8(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* m,
                               void* y, int32_t y_dtype, int64_t ldy, int32_t rows, uint32_t flags, void* workspace,
                               size_t workspace_bytes) {
    if (ctx == nullptr) return kErrInvalidArg;
    int32_t st = check_w8a8(ctx, m, rows);
    if (st != kOk) return st;
    if (x == nullptr || y == nullptr || x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2 || ldx < m->k || ldx % 8 != 0 ||
        ldy < m->n || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
        return fail(ctx, kErrInvalidArg, "qmm_w8a8: x must be 16-byte aligned with ldx >= k, ldx %% 8 == 0; ldy >= n");
    W8a8Ws w = carve_w8a8(workspace, m->n, m->k, rows);
    if (workspace == nullptr || workspace_bytes < w.bytes || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return fail(ctx, kErrWorkspace, "qmm_w8a8: workspace %zu < %zu (256-byte aligned)", workspace_bytes, w.bytes);
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    const bool tern = m->bits == 2;
    // ternary: x arrives rotated by the format's own transform (iq_had_rows), so neither side is rotated here (n = 1)
    const int n = tern ? 1 : rot_block(m->k);
    const size_t smem = (size_t)m->k * sizeof(float);
    if (tern)
        tern_i8row_kernel<<<(m->n + 3) / 4, 128, 0, cs>>>(static_cast<const uint32_t*>(m->w), static_cast<const __half*>(m->scales),
                                                          m->n, m->k, w.wq, w.sw);
    else
        rot_quant_rows_kernel<0><<<m->n, 256, smem, cs>>>(m->w, static_cast<const uint16_t*>(m->scales),
                                                          static_cast<const uint16_t*>(m->biases), m->group, 0, 0, m->k, n, w.wq,
                                                          w.sw);
    rot_quant_rows_kernel<1><<<rows, 256, smem, cs>>>(x, nullptr, nullptr, 0, x_dtype, ldx, m->k, n, w.xq, w.sx);
    st = check_cuda(ctx, cudaGetLastError(), "rot_quant_rows launch");
    if (st != kOk) return st;
    QmmCall c;
    c.fmt = kFmtInt8Plain; c.epi = 0; c.bn = rows >= 256 ? 256 : 128;
    c.x16 = w.xq; c.ldx = m->k; c.x_rows = rows;
    c.w[0] = w.wq; c.s[0] = w.sx; c.b[0] = w.sw;
    c.experts = 1;
    c.N = m->n; c.K = m->k; c.M = rows;
    c.y = y; c.y_dtype = y_dtype; c.ldy = ldy;
    c.accumulate = (flags & IQ_FLAG_ACCUMULATE) ? 1 : 0;
    c.limit = 1.0f / (float)n;  // (H x) . (H w) = n x . w with the unnormalised transform of size n
    return launch_qmm(ctx, cs, c);
}
