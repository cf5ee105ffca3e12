// Shared device helpers for the quantized-matmul kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace iq {

// Status codes returned through the C ABI (negative = error). Kept in sync with include/ingot_qmm.h.
enum : int32_t {
    kOk = 0,
    kErrInvalidArg = -1,
    kErrUnsupported = -2,
    kErrCuda = -3,
    kErrWorkspace = -4,
    kErrNoKernel = -5,
    kErrTimeout = -6,
    kErrComm = -7,
};

// Element types of activations / outputs at the ABI.
enum : int32_t { kF32 = 0, kF16 = 1, kBF16 = 2 };

// Weight formats.
// kFmtAffine4G32: 4-bit affine with groups of 32 (dense matrices); kFmtAffine6: 6-bit affine, groups of 64 (decode GEMV)
// kFmtBf16Plain: not a quantized format: a bf16 matrix used as it is (the router's approximate logits on the tensor cores)
// kFmtTernary: 2-bit codes in groups of 128 with an fp16 scale, w = (q - 1) * s (the rotated ternary format)
// kFmtInt8Plain: not a stored format: int8 rows with a scale per row on both sides (the rotated W8A8 prefill GEMM)
enum : int32_t {
    kFmtAffine4 = 0, kFmtAffine8 = 1, kFmtMxfp4 = 2, kFmtAffine4G32 = 3, kFmtAffine6 = 4, kFmtBf16Plain = 5, kFmtTernary = 6,
    kFmtInt8Plain = 7
};

// FFN activations, numbered as the reference's lab_glu (qmm.metal:9-31): 0 SiLU gate, 1 GELU (tanh form) gate,
// 2 gpt-oss's swiglu_oai, 3 relu^2 of the up projection alone (no gate).
enum : int32_t { kActSilu = 0, kActGelu = 1, kActSwigluOai = 2, kActRelu2 = 3 };

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t u16) { return __uint_as_float(u16 << 16); }

__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    // round to nearest even (Loader/Quant.swift:121-125 of the reference)
    uint32_t u = __float_as_uint(f);
    return (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b),
                        *reinterpret_cast<__half2*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

// Loads 8 consecutive activations starting at element index `i` (a multiple of 8) and returns them as fp32.
__device__ __forceinline__ void load_x8(const void* x, int32_t dtype, size_t i, float (&v)[8]) {
    if (dtype == kBF16) {
        uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + i);
        uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            v[2 * j] = __uint_as_float(w[j] << 16);
            v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
    } else if (dtype == kF16) {
        uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(x) + i);
        uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float2 f = __half22float2(*reinterpret_cast<__half2*>(&w[j]));
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        }
    } else {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + i);
        float4 a = p[0], b = p[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

// Gated FFN activation on fp32 values.
template <int ACT>
__device__ __forceinline__ float glu(float g, float u, float limit) {
    // __expf / __fdividef: a few ulp, far inside the fp16 rounding that follows; the IEEE division alone was a
    // noticeable share of the grouped GEMM's epilogue
    if (ACT == kActSilu) {
        return __fdividef(g, 1.0f + __expf(-g)) * u;
    } else if (ACT == kActGelu) {
        // g * sigmoid(2z), z = sqrt(2/pi) (g + 0.044715 g^3): 0.5 g (1 + tanh z) without the cancellation in the tail
        const float z2 = 1.5957691216057308f * (g + 0.044715f * g * g * g);
        return __fdividef(g, 1.0f + __expf(-z2)) * u;
    } else if (ACT == kActRelu2) {
        const float r = fmaxf(u, 0.f);
        return r * r;
    } else {
        const float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
        return __fdividef(gc, 1.0f + __expf(-1.702f * gc)) * (uc + 1.0f);
    }
}

// The same with the activation chosen at run time (uniform over a launch).
__device__ __forceinline__ float glu_rt(int32_t act, float g, float u, float limit) {
    if (act == kActSilu) return glu<kActSilu>(g, u, 0.f);
    if (act == kActSwigluOai) return glu<kActSwigluOai>(g, u, limit);
    if (act == kActGelu) return glu<kActGelu>(g, u, 0.f);
    return glu<kActRelu2>(g, u, 0.f);
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_nc_u4(const void* p) {
    uint4 r;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

__device__ __forceinline__ uint32_t ldg_nc_u16(const void* p) {
    unsigned short r;
    asm("ld.global.nc.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
}

// Prefetching variants: volatile, so the compiler keeps them where they are written (ahead of a barrier wait) instead
// of sinking them to the first use.
__device__ __forceinline__ uint32_t ldg_nc_u16_early(const void* p) {
    unsigned short r;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ldg_nc_u8_early(const void* p) {
    uint32_t r;
    asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}

__device__ __forceinline__ uint32_t ldg_nc_u8(const void* p) {
    uint32_t r;
    asm("ld.global.nc.u8 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}

}  // namespace iq
