// Bandwidth-bound quantized GEMV family ("qmv" / decode "gather_qmv"): Y[M<=16, N] = X[M, K] * W^T with W in MLX affine
// 4/8-bit (group 64) or MXFP4 (group 32) format, read once from HBM with 128-bit loads and dequantised in registers.
//
// One warp owns 16 consecutive output rows of W and a slice of K. Each lane streams 16-byte pieces ("chunks") of two
// rows (r = lane/4 and r + 8): the four lanes of a row take four adjacent chunks, so every load instruction covers
// 64 contiguous bytes of 8 (x2) rows. The codes become fp16 weights with one logic op, one exact half2 subtraction
// and one half2 FMA per pair (the 0x6400 "1024 + q" trick, then w = fma(q, s, b) rounded once: the fp16 rounding of
// the exact s*q + b, which is the reference kernels' arithmetic), and the multiply-accumulate runs on m16n8k16
// tensor-core fragments with W as the A operand and up to 8 (or 16) activation rows as B, accumulating in fp32.
// (Rounding s*q alone and adding the bias separately was measured at 1.2e-3 on a small MoE layer: over the parity
// bound; the single rounding of s*q + b measures ~0.) Activations are staged once per CTA into shared memory as fp16 in the
// fragment order the B operand wants, so the inner loop has no shuffles. Partial sums of the K-slices are added in a
// fixed warp order, which makes a row's bits independent of the other rows (the reference's row-invariance property,
// Tests/IngotTests/KernelCaseTests.swift:68-86).
//
// Replaces the reference's decode kernels vnax_qmv_nf1_sg32 / fn_qmv8_nf1 / vqmv_* (Shaders/verify_nax.metal:105-209,
// Shaders/verify.metal:89-155) and, through the tile list, vnax_moe_gateup* / vnax_moe_down_split*
// (Shaders/verify_nax.metal:258-509).
#pragma once

#include "common.cuh"

namespace iq {

// One unit of MoE work: rows [start, start + count) of the expert-sorted pair list belong to `expert`
// (the reference's uint4(expert, start, rows, 0) tile descriptor, Shaders/qmm_nax_moe.metal:139-217).
struct Tile {
    uint32_t expert, start, count, pad;
};

enum : int { kModePlain = 0, kModeGateUp = 1, kModeDown = 2 };

struct GqmvParams {
    // weights: [0] = the matrix (plain / down) or gate; [1] = up (gate/up mode only)
    const uint32_t* w[2];
    const void* s[2];
    const void* b[2];
    int64_t w_estride;  // uint32 words between experts
    int64_t s_estride;  // scale elements between experts
    int32_t N, K;       // output rows per expert, inputs
    // activations
    const void* x;
    int32_t x_dtype;
    int64_t ldx;
    const uint32_t* row_map;  // gate/up: sorted position -> pair id (token = pair / topk); null: rows are in place
    int32_t topk;
    // work list
    const Tile* tiles;       // null: one tile {0, 0, M}
    const uint32_t* ntiles;  // device count of valid tiles
    int32_t M;
    // outputs
    void* y;
    int32_t y_dtype;
    int64_t ldy;
    int32_t accumulate;
    const float* ebias[2];  // expert biases fp32 [E, N] (gate/up: gate and up; down: [0]) or null
    float limit;            // swiglu_oai clamp
    int32_t act;            // gate/up mode: activation (kAct*)
    // K tiling (host-chosen): K is walked in tiles of `kt` inputs, kt a multiple of 512
    int32_t kt;
    int32_t xs_bytes;    // bytes of the staged-x region (sized for the largest tile)
};

template <int FMT>
struct FmtTraits;
template <>
struct FmtTraits<kFmtAffine4> {
    static constexpr int CK = 32, QU = 4, CPG = 2, GROUP = 64;
    static constexpr bool PERM = true, BIAS = true;  // BIAS: the format carries a per-group bias tensor
};
template <>
struct FmtTraits<kFmtAffine8> {
    static constexpr int CK = 16, QU = 2, CPG = 4, GROUP = 64;
    static constexpr bool PERM = false, BIAS = true;
};
template <>
struct FmtTraits<kFmtAffine4G32> {  // one scale and bias per 16-byte chunk
    static constexpr int CK = 32, QU = 4, CPG = 1, GROUP = 32;
    static constexpr bool PERM = true, BIAS = true;
};
template <>
struct FmtTraits<kFmtMxfp4> {
    static constexpr int CK = 32, QU = 4, CPG = 1, GROUP = 32;
    static constexpr bool PERM = false, BIAS = false;
};

__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// Two e2m1 codes per byte -> four half2 (natural order) for one 32-bit word.
__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t (&h)[4]) {
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}\n"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w));
}

// Per-chunk dequantisation constants of one weight row: scale, scale / 16 and bias as half2 pairs.
struct DqConst {
    uint32_t s2, s16, b2;
};

// raw_scale / raw_bias: bf16 bit patterns (affine) or the e8m0 byte (mxfp4, no bias).
template <int FMT>
__device__ __forceinline__ DqConst make_dq(uint32_t raw_scale, uint32_t raw_bias = 0) {
    DqConst d;
    if (FMT == kFmtMxfp4) {
        // e8m0: 2^(s - 127), 255 = NaN (Loader/Quant.swift:198-202 of the reference)
        float f = raw_scale == 255u ? __uint_as_float(0x7FC00000u)
                                    : (raw_scale == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(raw_scale << 23));
        d.s2 = pack_half2(f, f);
        d.s16 = d.b2 = 0;
    } else {
        const float s = bf16_bits_to_f32(raw_scale), b = bf16_bits_to_f32(raw_bias);
        d.s2 = pack_half2(s, s);
        d.s16 = hmul2_u32(d.s2, 0x2C002C00u);  // s / 16 (exact)
        d.b2 = pack_half2(b, b);
    }
    return d;
}

// (1024 + v, 1024 + v') -> fma(v, s, b) with one rounding: the subtraction is exact, so the weight is the fp16
// rounding of the exact s * q + b — the reference kernels' own arithmetic (Shaders/qmm_nax.metal:77-95).
__device__ __forceinline__ uint32_t dq_pair(uint32_t magic_plus_v, uint32_t s2, uint32_t b2) {
    const uint32_t k1024 = 0x64006400u;
    __half2 q = __hsub2(*reinterpret_cast<__half2*>(&magic_plus_v), *reinterpret_cast<const __half2*>(&k1024));
    __half2 r = __hfma2(q, *reinterpret_cast<__half2*>(&s2), *reinterpret_cast<__half2*>(&b2));
    return *reinterpret_cast<uint32_t*>(&r);
}

// Dequantises word `wd` of a chunk into the A-operand halves it feeds:
// 4-bit / mxfp4: two MMAs (k-slot pairs p[0], p[1] then p[2], p[3]); 8-bit: one MMA (p[0], p[1]).
template <int FMT>
__device__ __forceinline__ void dequant_word(uint32_t w, const DqConst& d, uint32_t (&p)[4]) {
    if (FMT == kFmtAffine4 || FMT == kFmtAffine4G32) {
        const uint32_t w8 = w >> 8;
        p[0] = dq_pair((w & 0x000F000Fu) | 0x64006400u, d.s2, d.b2);    // (n0, n4)
        p[1] = dq_pair((w & 0x00F000F0u) | 0x64006400u, d.s16, d.b2);   // (n1, n5): the codes sit 16x up
        p[2] = dq_pair((w8 & 0x000F000Fu) | 0x64006400u, d.s2, d.b2);   // (n2, n6)
        p[3] = dq_pair((w8 & 0x00F000F0u) | 0x64006400u, d.s16, d.b2);  // (n3, n7)
    } else if (FMT == kFmtAffine8) {
        p[0] = dq_pair(__byte_perm(w, 0x64646464u, 0x4140), d.s2, d.b2);  // (c0, c1)
        p[1] = dq_pair(__byte_perm(w, 0x64646464u, 0x4342), d.s2, d.b2);  // (c2, c3)
        p[2] = p[3] = 0;
    } else {
        uint32_t h[4];
        cvt_e2m1x8(w, h);
#pragma unroll
        for (int i = 0; i < 4; i++) p[i] = hmul2_u32(h[i], d.s2);
    }
}

template <int FMT, int NW>
struct Batch {
    uint4 v[NW][2];       // codes of rows r and r + 8
    uint32_t sc[NW][2];   // raw scale of the chunk's group
    uint32_t bi[NW][2];   // raw bias of the chunk's group (affine)
};

template <int FMT, int MH, int NW, int MODE, int RG, int WK>
__global__ void __launch_bounds__(RG* WK * 32) gqmv_kernel(const GqmvParams p) {
    using F = FmtTraits<FMT>;
    constexpr int NT = RG * WK * 32;
    constexpr int U = NW == 2 ? 1 : 2;  // steps per register batch
    extern __shared__ __align__(16) unsigned char smem[];

    // ---- which tile ------------------------------------------------------------------------------------------
    Tile tile;
    if (p.tiles != nullptr) {
        if (blockIdx.y >= *p.ntiles) return;
        tile = p.tiles[blockIdx.y];
    } else {
        tile.expert = 0; tile.start = 0; tile.count = (uint32_t)p.M; tile.pad = 0;
    }
    const int M = (int)tile.count;  // live activation rows (1 .. 8 * MH)
    const int MR = M;               // rows of the staged x block

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rg = warp / WK, wk = warp % WK;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = (blockIdx.x * RG + rg) * 16;  // first output row of this warp
    const bool rows_ok = n0 < p.N;               // N is a multiple of 16

    uint4* xs = reinterpret_cast<uint4*>(smem);
    float* red = reinterpret_cast<float*>(smem + p.xs_bytes);

    const int row_words = p.K / 32 * (FMT == kFmtAffine8 ? 8 : 4);  // uint32 per weight row
    const int row_groups = p.K / F::GROUP;

    const uint4* wrow[NW][2];
    const unsigned char* srow[NW][2];
    const unsigned char* brow[NW][2];
#pragma unroll
    for (int i = 0; i < NW; i++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int64_t r = rows_ok ? (n0 + g + 8 * h) : 0;
            wrow[i][h] = reinterpret_cast<const uint4*>(p.w[i] + tile.expert * p.w_estride + r * row_words);
            srow[i][h] = reinterpret_cast<const unsigned char*>(p.s[i]) +
                         (tile.expert * p.s_estride + r * row_groups) * (FMT == kFmtMxfp4 ? 1 : 2);
            brow[i][h] = FMT == kFmtMxfp4 ? srow[i][h]
                                          : reinterpret_cast<const unsigned char*>(p.b[i]) +
                                                (tile.expert * p.s_estride + r * row_groups) * 2;
        }

    float acc[NW][MH][4];
#pragma unroll
    for (int i = 0; i < NW; i++)
#pragma unroll
        for (int h = 0; h < MH; h++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][h][e] = 0.f;

    auto load_batch = [&](Batch<FMT, NW>(&bt)[U], int j, int c_base, int nch_tile) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int cl = 4 * (j + u) + t;
            const bool ok = rows_ok && cl < nch_tile;
            const int c = c_base + cl;
#pragma unroll
            for (int i = 0; i < NW; i++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    if (ok) {
                        bt[u].v[i][h] = ldg_nc_u4(wrow[i][h] + c);
                        bt[u].sc[i][h] = FMT == kFmtMxfp4 ? ldg_nc_u8(srow[i][h] + c / F::CPG)
                                                         : ldg_nc_u16(srow[i][h] + 2 * (c / F::CPG));
                        bt[u].bi[i][h] = FMT == kFmtMxfp4 ? 0u : ldg_nc_u16(brow[i][h] + 2 * (c / F::CPG));
                    } else {
                        bt[u].v[i][h] = make_uint4(0, 0, 0, 0);
                        bt[u].sc[i][h] = FMT == kFmtMxfp4 ? 127u : 0u;
                        bt[u].bi[i][h] = 0u;
                    }
                }
        }
    };

    int nch_cur = 0;  // chunks in the K tile being consumed
    auto compute_batch = [&](Batch<FMT, NW>(&bt)[U], int j) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            DqConst dq[NW][2];
#pragma unroll
            for (int i = 0; i < NW; i++)
#pragma unroll
                for (int h = 0; h < 2; h++) dq[i][h] = make_dq<FMT>(bt[u].sc[i][h], bt[u].bi[i][h]);
#pragma unroll
            for (int q = 0; q < F::QU; q++) {
                // x fragments of this 8-input unit for rows g (and g + 8)
                uint4 xf[MH];
#pragma unroll
                for (int h = 0; h < MH; h++) {
                    const int m = g + 8 * h;
                    const bool live = m < M && 4 * (j + u) + t < nch_cur;
                    xf[h] = live ? xs[(((j + u) * F::QU + q) * MR + m) * 4 + t] : make_uint4(0, 0, 0, 0);
                }
                constexpr int WPQ = FMT == kFmtAffine8 ? 2 : 1;  // words per x unit
#pragma unroll
                for (int ww = 0; ww < WPQ; ww++) {
                    const int wd = q * WPQ + ww;
#pragma unroll
                    for (int i = 0; i < NW; i++) {
                        uint32_t pa[4], pb[4];
                        dequant_word<FMT>(word_of(bt[u].v[i][0], wd), dq[i][0], pa);
                        dequant_word<FMT>(word_of(bt[u].v[i][1], wd), dq[i][1], pb);
#pragma unroll
                        for (int h = 0; h < MH; h++) {
                            if (FMT == kFmtAffine8) {
                                const uint32_t b0 = ww == 0 ? xf[h].x : xf[h].z, b1 = ww == 0 ? xf[h].y : xf[h].w;
                                mma16816(acc[i][h], pa[0], pb[0], pa[1], pb[1], b0, b1);
                            } else {
                                mma16816(acc[i][h], pa[0], pb[0], pa[1], pb[1], xf[h].x, xf[h].y);
                                mma16816(acc[i][h], pa[2], pb[2], pa[3], pb[3], xf[h].z, xf[h].w);
                            }
                        }
                    }
                }
            }
        }
    };

    // ---- K tiles -----------------------------------------------------------------------------------------------
    Batch<FMT, NW> cur[U], nxt[U];
    for (int k0 = 0; k0 < p.K; k0 += p.kt) {
        const int klen = min(p.kt, p.K - k0);
        const int nch_tile = klen / F::CK;
        nch_cur = nch_tile;
        const int c_base = k0 / F::CK;
        const int nsteps = (nch_tile + 3) / 4;
        const int spw = ((nsteps + WK - 1) / WK + U - 1) / U * U;  // steps per warp, a multiple of U
        const int jb = wk * spw, je = min(nsteps, jb + spw);

        // first batch of weight loads goes out before the activations are staged
        if (jb < je) load_batch(cur, jb, c_base, nch_tile);

        if (k0 > 0) __syncthreads();  // previous tile fully consumed
        // ---- stage x[:, k0 : k0 + klen] as fp16 in fragment order, and the per-group sums --------------------------
        {
            const int units_per_row = klen / 8;
            const int total = M * units_per_row;
            for (int uidx = tid; uidx < (total + 31) / 32 * 32; uidx += NT) {
                const int m = uidx / units_per_row, ku = uidx % units_per_row;
                float v[8];
                const bool live = uidx < total;
                if (live) {
                    size_t row;
                    if (MODE == kModeGateUp && p.row_map != nullptr) row = p.row_map[tile.start + m] / (uint32_t)p.topk;
                    else row = (size_t)tile.start + m;
                    load_x8(p.x, p.x_dtype, row * p.ldx + k0 + ku * 8, v);
                } else {
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = 0.f;
                }
                uint4 o;
                if (F::PERM) {
                    o.x = pack_half2(v[0], v[4]); o.y = pack_half2(v[1], v[5]);
                    o.z = pack_half2(v[2], v[6]); o.w = pack_half2(v[3], v[7]);
                } else {
                    o.x = pack_half2(v[0], v[1]); o.y = pack_half2(v[2], v[3]);
                    o.z = pack_half2(v[4], v[5]); o.w = pack_half2(v[6], v[7]);
                }
                if (uidx < total) {
                    const int kl = ku * 8, cl = kl / F::CK, q = (kl % F::CK) / 8;
                    xs[(((cl >> 2) * F::QU + q) * MR + m) * 4 + (cl & 3)] = o;
                }
            }
        }
        __syncthreads();

        // ---- stream this warp's K slice ------------------------------------------------------------------------
        for (int j = jb; j < je; j += U) {
            const bool more = j + U < je;
            if (more) load_batch(nxt, j + U, c_base, nch_tile);
            compute_batch(cur, j);
            if (more) {
#pragma unroll
                for (int u = 0; u < U; u++) cur[u] = nxt[u];
            }
        }

    }

    // ---- reduce the K slices in warp order -------------------------------------------------------------------------
    if (WK > 1) {
        __syncthreads();
        float* mine = red + (size_t)(rg * WK + wk) * (NW * MH * 4 * 32);
#pragma unroll
        for (int i = 0; i < NW; i++)
#pragma unroll
            for (int h = 0; h < MH; h++)
#pragma unroll
                for (int e = 0; e < 4; e++) mine[((i * MH + h) * 4 + e) * 32 + lane] = acc[i][h][e];
        __syncthreads();
        if (wk != 0) return;
#pragma unroll
        for (int i = 0; i < NW; i++)
#pragma unroll
            for (int h = 0; h < MH; h++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    float s = 0.f;
                    for (int k = 0; k < WK; k++)
                        s += red[(size_t)(rg * WK + k) * (NW * MH * 4 * 32) + ((i * MH + h) * 4 + e) * 32 + lane];
                    acc[i][h][e] = s;
                }
    }
    if (!rows_ok) return;

    // ---- epilogue: lane holds rows n0 + g (+8) x activation rows 2t, 2t + 1 (+8) ---------------------------------------
#pragma unroll
    for (int h = 0; h < MH; h++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int n = n0 + g + 8 * (e >> 1);
            const int m = 2 * t + (e & 1) + 8 * h;
            if (m >= M) continue;
            float v = acc[0][h][e];
            if (MODE == kModeGateUp) {
                float u = acc[NW - 1][h][e];
                if (p.ebias[0] != nullptr) {
                    v += p.ebias[0][(size_t)tile.expert * p.N + n];
                    u += p.ebias[1][(size_t)tile.expert * p.N + n];
                }
                v = glu_rt(p.act, v, u, p.limit);
            } else if (MODE == kModeDown) {
                if (p.ebias[0] != nullptr) v += p.ebias[0][(size_t)tile.expert * p.N + n];
            }
            const size_t o = (size_t)(tile.start + m) * p.ldy + n;
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

}  // namespace iq
