// Embedding gather: row tokens[r] of a quantized (or bf16) table, dequantised into the residual stream (fp32) and / or
// its fp16 copy. HBM-bound: one CTA per output row, each thread turns one 16-byte piece of the row's codes into 32
// (4-bit) or 16 (8-bit) values and writes them with 16-byte stores.
//
// Replaces embed_rows / embed_rows_g32 / embed_rows_b6 / embed_rows_b8 / embed_rows_bf16 (Shaders/yy_model.metal:12-95,
// Shaders/yw_lfm.metal of the reference;
// its check is bit-exact against the dequantised table, Tests/IngotTests/KernelCaseG32.swift:80-93): the value is
// float(scale) * float(code) + float(bias) in fp32 (the product of a bf16 and a code of at most 8 bits is exact, so a
// fused and an unfused evaluation agree), the fp16 output its round-to-nearest.
#include "common.cuh"
#include "internal.h"

namespace iq {
namespace {

struct EmbedParams {
    const uint32_t* tokens;
    const uint32_t* w;
    const uint16_t* s;  // bf16 bits
    const uint16_t* b;
    float* of;    // [rows, ldo] or null
    __half* oh;   // [rows, ldo] or null
    int64_t ldo;
    int32_t vocab, K, group;
};

__device__ __forceinline__ void store8(const EmbedParams& p, size_t at, const float (&v)[8]) {
    if (p.of != nullptr) {
        *reinterpret_cast<float4*>(p.of + at) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p.of + at + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (p.oh != nullptr) {
        uint4 h;
        h.x = pack_half2(v[0], v[1]); h.y = pack_half2(v[2], v[3]);
        h.z = pack_half2(v[4], v[5]); h.w = pack_half2(v[6], v[7]);
        *reinterpret_cast<uint4*>(p.oh + at) = h;
    }
}

// 6-bit codes (a little-endian bit stream, code j in bits 6j.. of the row; embed_rows_b6 of the reference): one thread
// per three words = sixteen values.
__global__ void __launch_bounds__(256) embed_rows6_kernel(const EmbedParams p) {
    const int row = blockIdx.x;
    const uint32_t t = p.tokens[row];
    const bool live = t < (uint32_t)p.vocab;
    const uint32_t* wr = p.w + (size_t)(live ? t : 0) * (p.K / 16 * 3);
    const size_t g0 = (size_t)(live ? t : 0) * (p.K / 64);
    for (int i = threadIdx.x; i < p.K / 16; i += blockDim.x) {
        const uint32_t w0 = live ? __ldg(wr + 3 * i) : 0u, w1 = live ? __ldg(wr + 3 * i + 1) : 0u;
        const uint32_t w2 = live ? __ldg(wr + 3 * i + 2) : 0u;
        const unsigned long long lo = ((unsigned long long)w1 << 32) | w0;  // codes 0..9 and the low bits of code 10
        const unsigned long long hi = ((unsigned long long)w2 << 28) | (w1 >> 4);  // from bit 36 = code 6 on
        const float sc = live ? bf16_bits_to_f32(p.s[g0 + i / 4]) : 0.f;
        const float bi = live ? bf16_bits_to_f32(p.b[g0 + i / 4]) : 0.f;
        float v[16];
#pragma unroll
        for (int e = 0; e < 16; e++) {
            const uint32_t q = e < 6 ? (uint32_t)(lo >> (6 * e)) & 63u : (uint32_t)(hi >> (6 * (e - 6))) & 63u;
            v[e] = fmaf(sc, (float)q, bi);
        }
        const size_t at = (size_t)row * p.ldo + (size_t)i * 16;
        const float (&va)[8] = *reinterpret_cast<const float (*)[8]>(v);
        const float (&vb)[8] = *reinterpret_cast<const float (*)[8]>(v + 8);
        store8(p, at, va);
        store8(p, at + 8, vb);
    }
}

// BITS: 4 or 8 (affine codes, low bits first), 16 (a plain bf16 table)
template <int BITS>
__global__ void __launch_bounds__(256) embed_rows_kernel(const EmbedParams p) {
    const int row = blockIdx.x;
    const uint32_t t = p.tokens[row];
    const bool live = t < (uint32_t)p.vocab;  // a token outside the table gives a zero row
    constexpr int PER = 128 / BITS;           // values per 16-byte piece
    const uint4* wr = reinterpret_cast<const uint4*>(p.w) + (size_t)(live ? t : 0) * (p.K / PER);
    const size_t g0 = (size_t)(live ? t : 0) * (p.K / (BITS == 16 ? 1 : p.group));
    for (int i = threadIdx.x; i < p.K / PER; i += blockDim.x) {
        const uint4 q = live ? __ldg(wr + i) : make_uint4(0, 0, 0, 0);
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
        const size_t at = (size_t)row * p.ldo + (size_t)i * PER;
        if (BITS == 16) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                v[2 * j] = live ? __uint_as_float(words[j] << 16) : 0.f;
                v[2 * j + 1] = live ? __uint_as_float(words[j] & 0xFFFF0000u) : 0.f;
            }
            store8(p, at, v);
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                constexpr int VW = 32 / BITS;  // values per word
                const int k = i * PER + j * VW;
                const float sc = live ? bf16_bits_to_f32(p.s[g0 + k / p.group]) : 0.f;
                const float bi = live ? bf16_bits_to_f32(p.b[g0 + k / p.group]) : 0.f;
                if (BITS == 4) {
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = fmaf(sc, (float)((words[j] >> (4 * e)) & 15u), bi);
                    store8(p, at + j * 8, v);
                } else {
                    float v[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) v[e] = fmaf(sc, (float)((words[j] >> (8 * e)) & 255u), bi);
                    if (p.of != nullptr) *reinterpret_cast<float4*>(p.of + at + j * 4) = make_float4(v[0], v[1], v[2], v[3]);
                    if (p.oh != nullptr)
                        *reinterpret_cast<uint2*>(p.oh + at + j * 4) = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
                }
            }
        }
    }
}

}  // namespace
}  // namespace iq

using namespace iq;

extern "C" int32_t iq_embed_rows(iq_ctx* ctx, void* stream, const iq_qlinear* table, const uint32_t* tokens, int32_t rows,
                                 float* out_f32, void* out_f16, int64_t ldo) {
    if (ctx == nullptr) return kErrInvalidArg;
    if (table == nullptr || table->w == nullptr || tokens == nullptr || (out_f32 == nullptr && out_f16 == nullptr))
        return fail(ctx, kErrInvalidArg, "embed_rows: null pointer");
    if (rows < 1 || table->n < 1 || table->k < 64 || table->k % 64 != 0 || ldo < table->k || ldo % 8 != 0)
        return fail(ctx, kErrInvalidArg, "embed_rows: rows = %d, k = %d (a multiple of 64), ldo = %lld (>= k, a multiple of 8)",
                    rows, table->k, (long long)ldo);
    if ((reinterpret_cast<uintptr_t>(table->w) & 15) || (reinterpret_cast<uintptr_t>(out_f32) & 15) ||
        (reinterpret_cast<uintptr_t>(out_f16) & 15))
        return fail(ctx, kErrInvalidArg, "embed_rows: table and outputs must be 16-byte aligned");
    const bool plain = table->bits == 16;
    if (!plain) {
        if (table->mode != IQ_MODE_AFFINE || !((table->bits == 4 && (table->group == 64 || table->group == 32)) ||
                                               ((table->bits == 8 || table->bits == 6) && table->group == 64)))
            return fail(ctx, kErrUnsupported, "embed_rows: %d-bit group %d mode %d (affine 4-bit g64/g32, 6/8-bit g64, or bf16)",
                        table->bits, table->group, table->mode);
        if (table->scales == nullptr || table->biases == nullptr) return fail(ctx, kErrInvalidArg, "embed_rows: scales/biases");
    }
    EmbedParams p;
    p.tokens = tokens;
    p.w = static_cast<const uint32_t*>(table->w);
    p.s = static_cast<const uint16_t*>(table->scales);
    p.b = static_cast<const uint16_t*>(table->biases);
    p.of = out_f32;
    p.oh = static_cast<__half*>(out_f16);
    p.ldo = ldo;
    p.vocab = table->n; p.K = table->k; p.group = plain ? 1 : table->group;
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    if (plain) embed_rows_kernel<16><<<rows, 256, 0, cs>>>(p);
    else if (table->bits == 4) embed_rows_kernel<4><<<rows, 256, 0, cs>>>(p);
    else if (table->bits == 6) embed_rows6_kernel<<<rows, 256, 0, cs>>>(p);
    else embed_rows_kernel<8><<<rows, 256, 0, cs>>>(p);
    return check_cuda(ctx, cudaGetLastError(), "embed_rows launch");
}
