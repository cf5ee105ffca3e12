// Prefill quantized GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory), dense and grouped (MoE).
//
//   D[128 weight rows, BN tokens] += Wd[128, 64] * X[BN, 64]^T      per K step of 64 inputs
//
// The weight tile is the M = 128 side of the MMA and the tokens are its N side (16..256 in steps of 16), so a ragged
// number of tokens per expert costs no padding rows and every weight byte is dequantised once per token tile.
// Warp roles inside one persistent CTA (448 threads):
//   warp 0      TMA producer: per stage, the fp16 activation tile X[BN, 64] (128-byte swizzle, the layout the MMA
//               reads) and the packed codes of the weight tile(s) ([128, 64 inputs] as raw bytes)
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane), commits stages and accumulators
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulator, apply bias / activation, store (coalesced along the
//               weight-row dimension, which is the fast dimension of Y)
//   warps 6-13  dequantisers: packed codes (shared memory) -> fp16 w = fma(q, s, b) -> swizzled K-major tile
// Stages are recycled by tcgen05.commit on an mbarrier; two accumulators in tensor memory let the epilogue of one
// tile overlap the main loop of the next (one accumulator when a tile needs all 512 columns: gate+up on 256 tokens). Every wait is bounded: on a timeout the kernel writes a status word, all
// roles drain and tensor memory is released.
//
// Replaces qmm_t_nax3* (Shaders/qmm_nax_v3.metal:107-256) and, with a tile list, moe_gateup_swiglu2* / moe_down2*
// (Shaders/qmm_nax_moe.metal:442-717) of the reference.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "gqmv.cuh"
#include "ptx.cuh"

namespace iq {

constexpr int kQmmThreads = 448;
constexpr int kQmmGatherThreads = 544;  // + three warps that help the producer fetch gathered activation rows
constexpr int kBK = 64;              // inputs per K step (= one affine group, two mxfp4 groups)
constexpr int kWRows = 128;          // weight rows per tile (MMA M)

enum : int { kEpiStore = 0, kEpiGateUp = 1 };

struct QmmParams {
    // scales / biases are read straight from global memory by the dequantisers
    const void* s[2];
    const void* b[2];
    int32_t expert_lo;       // first expert held here: tile.expert - expert_lo indexes the stacked tensors
    int32_t N, K;            // weight rows per expert, inputs
    int32_t M;               // token rows (dense) / total sorted rows (grouped)
    // work list: null = dense tiling over (N / 128) x (M / BN)
    const Tile* tiles;
    const uint32_t* ntiles;
    // output
    void* y;
    int32_t y_dtype;
    int64_t ldy;
    int32_t accumulate;
    const float* ebias[2];   // fp32 [E, N] or null
    float limit;
    // Gathered activations (grouped gate/up): row r of a tile is row gather_map[tile.start + r] / gather_div of xg (fp16
    // [*, ldxg]) instead of row tile.start + r of the tensor map's matrix: the producer warp fetches the rows itself with
    // 16-byte asynchronous copies, so the rows never have to be packed in expert order first. Null: the tensor map.
    const __half* xg;
    const uint32_t* gather_map;
    int64_t ldxg;
    uint32_t gather_div;
    int32_t* status;         // device status word (0 = ok)
    int32_t reserved;        // keeps the parameter block off an exact 512 bytes: at that size the fused gate/up kernel
                             // measured a quarter slower (487 against 386 us on the 4096-token layer), same code otherwise
};

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes
// apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;              // leading byte offset (unused with a swizzled K-major tile)
    d |= (uint64_t)(1024 >> 4) << 32;    // stride byte offset
    d |= (uint64_t)1 << 46;              // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;              // SWIZZLE_128B
    return d;
}
// Instruction descriptor, kind::f16: D = f32, A and B both f16 or both bf16 (the two format fields must agree: fp16
// weights with bf16 activations raised "illegal instruction" on sm_100a), both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(int n, bool bf16) {
    return (1u << 4) | (bf16 ? (1u << 7) | (1u << 10) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kWRows >> 4) << 24);
}
// kind::i8: D = s32, A = B = signed 8-bit, both K-major (32 inputs per MMA), M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc_i8(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kWRows >> 4) << 24);
}

// ---- dequantisation of 32 consecutive inputs of one weight row into four 16-byte chunks --------------------------
template <int FMT>
__device__ __forceinline__ void dequant32(uint32_t packed_row_half, uint32_t sc_raw, uint32_t bi_raw, uint4 (&out)[4]) {
    // packed_row_half: shared-memory address (explicit shared-space loads: a generic load here costs the long latency
    // path and showed up as the dequantisers' main stall)
    if (FMT == kFmtAffine4 || FMT == kFmtAffine4G32) {
        const uint4 v = lds128(packed_row_half);
        const float s = bf16_bits_to_f32(sc_raw), b = bf16_bits_to_f32(bi_raw);
        const uint32_t s2 = pack_half2(s, s * 0.0625f), b2 = pack_half2(b, b);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                // byte j of the word holds inputs 2j (low nibble) and 2j + 1: (1024 + q_lo, 1024 + 16 q_hi)
                const uint32_t t = (__byte_perm(w[i], 0u, 0x4040 + 0x0101 * j) & 0x00F0000Fu) | 0x64006400u;
                __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&t), __half2half2(__ushort_as_half(0x6400)));
                __half2 r = __hfma2(q, *reinterpret_cast<const __half2*>(&s2), *reinterpret_cast<const __half2*>(&b2));
                o[j] = *reinterpret_cast<uint32_t*>(&r);
            }
            out[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    } else if (FMT == kFmtAffine8) {
        const uint4 v0 = lds128(packed_row_half);
        const uint4 v1 = lds128(packed_row_half + 16);
        const float s = bf16_bits_to_f32(sc_raw), b = bf16_bits_to_f32(bi_raw);
        const uint32_t s2 = pack_half2(s, s), b2 = pack_half2(b, b);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t t = __byte_perm(w[2 * i + (j >> 1)], 0x64646464u, (j & 1) ? 0x4342 : 0x4140);
                __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&t), __half2half2(__ushort_as_half(0x6400)));
                __half2 r = __hfma2(q, *reinterpret_cast<const __half2*>(&s2), *reinterpret_cast<const __half2*>(&b2));
                o[j] = *reinterpret_cast<uint32_t*>(&r);
            }
            out[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    } else if (FMT == kFmtTernary) {
        // 32 codes of two bits in eight bytes; w = (q - 1) * s with the fp16 scale as it is stored: exact in fp16
        const uint2 v = lds64(packed_row_half);
        const uint32_t s2 = (sc_raw & 0xFFFFu) | (sc_raw << 16);
        const uint32_t k1025 = 0x64016401u;
        const uint32_t w[2] = {v.x, v.y};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t h16 = w[i >> 1] >> ((i & 1) * 16);  // eight codes in the low 16 bits
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t t = ((h16 >> (4 * j)) & 3u) | (((h16 >> (4 * j + 2)) & 3u) << 16) | 0x64006400u;  // 1024 + q
                __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&t), *reinterpret_cast<const __half2*>(&k1025));
                __half2 r = __hmul2(q, *reinterpret_cast<const __half2*>(&s2));
                o[j] = *reinterpret_cast<uint32_t*>(&r);
            }
            out[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    } else {
        const uint4 v = lds128(packed_row_half);
        const DqConst d = make_dq<kFmtMxfp4>(sc_raw);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t h[4];
            cvt_e2m1x8(w[i], h);
            out[i] = make_uint4(hmul2_u32(h[0], d.s2), hmul2_u32(h[1], d.s2), hmul2_u32(h[2], d.s2),
                                hmul2_u32(h[3], d.s2));
        }
    }
}

template <int FMT, int BN, int EPI>
struct QmmSmem {
    static constexpr int NWT = EPI == kEpiGateUp ? 2 : 1;                 // weight tiles per stage
    static constexpr bool I8 = FMT == kFmtInt8Plain;                      // int8 x int8 -> s32, a scale per row on both sides
    static constexpr bool PLAIN = FMT == kFmtBf16Plain || I8;             // weights used as they are: no packed tile
    static constexpr int BKE = I8 ? 128 : kBK;                            // inputs per K step (128 bytes of a row either way)
    static constexpr int PACK_ROW = PLAIN ? 0 : (FMT == kFmtAffine8 ? 64 : (FMT == kFmtTernary ? 16 : 32));  // packed bytes per row per K step
    static constexpr int X_BYTES = BN * 128;
    static constexpr int WD_BYTES = kWRows * 128;
    static constexpr int WP_BYTES = kWRows * PACK_ROW;
    static constexpr int STAGE_BYTES = X_BYTES + NWT * (WD_BYTES + WP_BYTES);
    static constexpr int kMaxDyn = 232448 - 1280;                         // opt-in limit minus alignment + barriers
    static constexpr int STAGES = kMaxDyn / STAGE_BYTES > 6 ? 6 : kMaxDyn / STAGE_BYTES;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
    static constexpr int ACC_COLS = NWT * BN;                             // tensor-memory columns per accumulator
    static constexpr int NACC = 2 * ACC_COLS <= 512 ? 2 : 1;              // accumulators in tensor memory (512 columns)
    static_assert(ACC_COLS <= 512, "the accumulator must fit tensor memory");
    static_assert(STAGES >= 2, "need at least two stages");
};

// ACT: activation of the gate/up epilogue (kAct*), fixed at compile time: the epilogue is on the critical path when gate
// and up fill tensor memory, and a run-time choice in its inner loop measured a quarter slower.
// GATHER: the activation rows of a tile are fetched by row index (three more warps help the producer); a variant of
// its own because more than 448 threads cap the registers at 96 per thread, which costs the dense kernels 4-8 %.
template <int FMT, int BN, int EPI, int ACT = kActSilu, bool GATHER = false>
__global__ void __launch_bounds__(GATHER ? kQmmGatherThreads : kQmmThreads, 1)
    qmm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w0,
                  const __grid_constant__ CUtensorMap map_w1, const QmmParams p) {
    using S = QmmSmem<FMT, BN, EPI>;
    constexpr int NWT = S::NWT, STAGES = S::STAGES;
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES);
    // barrier slots: full[STAGES], ready[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
    const uint32_t bar_full = smem_u32(bars), bar_ready = bar_full + 8 * STAGES, bar_empty = bar_ready + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    constexpr bool gather = GATHER;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            // the producer's arrive.expect_tx; gathered rows: plus one arrival per lane when its copies have landed
            mbar_init(bar_full + 8 * s, gather ? 129 : 1);
            mbar_init(bar_ready + 8 * s, 4);  // the four warps of the dequantiser group that owns the step
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // ---- work list --------------------------------------------------------------------------------------------
    const int n_tiles_n = (p.N + kWRows - 1) / kWRows;
    int total_work;
    int m_tiles = 0;
    if (p.tiles != nullptr) {
        total_work = (int)(*p.ntiles) * n_tiles_n;
    } else {
        m_tiles = (p.M + BN - 1) / BN;
        total_work = m_tiles * n_tiles_n;
    }
    const int ksteps = p.K / S::BKE;
    const int row_groups = p.K / ((FMT == kFmtMxfp4 || FMT == kFmtAffine4G32) ? 32 : (FMT == kFmtTernary ? 128 : 64));

    // Decodes work item `wi` into (expert, first token row, live token rows, first weight row).
    auto decode = [&](int wi, uint32_t& expert, int& row0, int& rows, int& n0) {
        if (p.tiles != nullptr) {
            const Tile t = p.tiles[wi / n_tiles_n];
            expert = t.expert - (uint32_t)p.expert_lo; row0 = (int)t.start; rows = (int)t.count;  // local slot
            n0 = (wi % n_tiles_n) * kWRows;
        } else {
            const int tm = wi % m_tiles;
            expert = 0; row0 = tm * BN; rows = min(BN, p.M - row0);
            n0 = (wi / m_tiles) * kWRows;
        }
    };

    if (gather && (warp == 0 || warp >= 14)) {
        // ================= producers, gathered activation rows: warps 0, 14, 15, 16 =================
        // Producer warp pw copies rows [pw * BN / 4, (pw + 1) * BN / 4) of every tile: a lane takes 16-byte chunk c of rows
        // rq, rq + 4, ... of that range (eight lanes cover one row's 128 bytes), with the rows' indices in registers for
        // the whole tile. Warp 0's first lane also issues the tensor copies of the packed weight tiles.
        constexpr int RPL = BN / 16;  // rows per lane
        const int pw = warp == 0 ? 0 : warp - 13;
        const int c = lane & 7, rq = lane >> 3;
        uint32_t it = 0;
        bool ok = true;
        for (int wi = blockIdx.x; wi < total_work && ok; wi += gridDim.x) {
            uint32_t expert; int row0, rows, n0;
            decode(wi, expert, row0, rows, n0);
            uint32_t g[RPL];
#pragma unroll
            for (int i = 0; i < RPL; i++) {
                const int r = pw * (BN / 4) + 4 * i + rq;
                g[i] = r < rows ? p.gather_map[row0 + r] / p.gather_div : 0xFFFFFFFFu;
            }
            const int wrow = (int)expert * p.N + n0;
            for (int ks = 0; ks < ksteps; ks++, it++) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                ok = mbar_wait_relaxed(bar_empty + 8 * s, ph ^ 1, abort_flag);
                if (!(ok = __all_sync(0xffffffffu, ok))) break;
                unsigned char* st = smem + s * S::STAGE_BYTES;
                if (warp == 0 && lane == 0) {
                    mbar_arrive_expect_tx(bar_full + 8 * s, NWT * S::WP_BYTES);
                    tma_load_2d(smem_u32(st + S::X_BYTES + NWT * S::WD_BYTES), &map_w0, bar_full + 8 * s, ks * S::PACK_ROW, wrow);
                    if (NWT == 2)
                        tma_load_2d(smem_u32(st + S::X_BYTES + NWT * S::WD_BYTES + S::WP_BYTES), &map_w1, bar_full + 8 * s,
                                    ks * S::PACK_ROW, wrow);
                }
                // row r of the tile lands where the tensor copy would have put it: 128-byte rows, eight-row groups of
                // 1024 bytes, the 16-byte chunks of a row XORed with the row's index in its group. Rows beyond the
                // tile's keep whatever the stage held: a column of B only feeds its own column of D, which is not stored.
                const __half* src0 = p.xg + (size_t)ks * kBK + c * 8;
                const uint32_t dst0 = smem_u32(st);
#pragma unroll
                for (int i = 0; i < RPL; i++) {
                    const int r = pw * (BN / 4) + 4 * i + rq;
                    if (g[i] != 0xFFFFFFFFu)
                        cp_async16(dst0 + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4), src0 + (size_t)g[i] * p.ldxg);
                }
                cp_async_arrive_noinc(bar_full + 8 * s);
            }
        }
    } else if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int wi = blockIdx.x; wi < total_work && ok; wi += gridDim.x) {
                uint32_t expert; int row0, rows, n0;
                decode(wi, expert, row0, rows, n0);
                for (int ks = 0; ks < ksteps; ks++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!(ok = mbar_wait_relaxed(bar_empty + 8 * s, ph ^ 1, abort_flag))) break;
                    unsigned char* st = smem + s * S::STAGE_BYTES;
                    if (S::PLAIN) {  // the bf16 weight tile goes straight where the MMA reads it (128-byte swizzle)
                        mbar_arrive_expect_tx(bar_full + 8 * s, S::X_BYTES + S::WD_BYTES);
                        tma_load_2d(smem_u32(st), &map_x, bar_full + 8 * s, ks * S::BKE, row0);
                        tma_load_2d(smem_u32(st + S::X_BYTES), &map_w0, bar_full + 8 * s, ks * S::BKE, (int)expert * p.N + n0);
                        continue;
                    }
                    mbar_arrive_expect_tx(bar_full + 8 * s, S::X_BYTES + NWT * S::WP_BYTES);
                    tma_load_2d(smem_u32(st), &map_x, bar_full + 8 * s, ks * kBK, row0);
                    const int wrow = (int)expert * p.N + n0;
                    tma_load_2d(smem_u32(st + S::X_BYTES + NWT * S::WD_BYTES), &map_w0, bar_full + 8 * s,
                                ks * S::PACK_ROW, wrow);
                    if (NWT == 2)
                        tma_load_2d(smem_u32(st + S::X_BYTES + NWT * S::WD_BYTES + S::WP_BYTES), &map_w1,
                                    bar_full + 8 * s, ks * S::PACK_ROW, wrow);
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int wi = blockIdx.x; wi < total_work && ok; wi += gridDim.x, tcount++) {
                uint32_t expert; int row0, rows, n0;
                decode(wi, expert, row0, rows, n0);
                const int nmma = min(BN, (rows + 15) & ~15);
                const uint32_t idesc = S::I8 ? make_idesc_i8(nmma) : make_idesc(nmma, S::PLAIN);
                const int a = tcount % S::NACC;
                const uint32_t aph = (tcount / S::NACC) & 1;
                if (!(ok = mbar_wait(bar_tempty + 8 * a, aph ^ 1, abort_flag))) break;
                tc_fence_after();
                const uint32_t tacc = tmem_base + a * S::ACC_COLS;
                for (int ks = 0; ks < ksteps; ks++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!(ok = mbar_wait(bar_full + 8 * s, ph, abort_flag))) break;
                    if (!S::PLAIN && !(ok = mbar_wait(bar_ready + 8 * s, ph, abort_flag))) break;
                    tc_fence_after();
                    unsigned char* st = smem + s * S::STAGE_BYTES;
                    const uint64_t bdesc = make_sw128_desc(smem_u32(st));
#pragma unroll
                    for (int wt = 0; wt < NWT; wt++) {
                        const uint64_t adesc = make_sw128_desc(smem_u32(st + S::X_BYTES + wt * S::WD_BYTES));
#pragma unroll
                        for (int kk = 0; kk < kBK / 16; kk++) {  // four MMAs of 32 bytes of K each
                            if (S::I8) umma_i8(tacc + wt * BN, adesc + 2 * kk, bdesc + 2 * kk, idesc, (ks | kk) ? 1u : 0u);
                            else umma_f16(tacc + wt * BN, adesc + 2 * kk, bdesc + 2 * kk, idesc, (ks | kk) ? 1u : 0u);
                        }
                    }
                    umma_commit(bar_empty + 8 * s);  // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(bar_tfull + 8 * a);
            }
        }
    } else if (warp < 6) {
        // ================= epilogue =================
        const int q = warp & 3;  // tensor-memory lane quadrant this warp may read
        uint32_t tcount = 0;
        bool ok = true;
        for (int wi = blockIdx.x; wi < total_work && ok; wi += gridDim.x, tcount++) {
            uint32_t expert; int row0, rows, n0;
            decode(wi, expert, row0, rows, n0);
            const int a = tcount % S::NACC;
            const uint32_t aph = (tcount / S::NACC) & 1;
            if (!(ok = mbar_wait_relaxed(bar_tfull + 8 * a, aph, abort_flag))) break;
            tc_fence_after();
            const int n = n0 + 32 * q + lane;  // weight row = output feature of this thread
            const bool n_ok = n < p.N;
            float bias0 = 0.f, bias1 = 0.f;
            if (n_ok && p.ebias[0] != nullptr) bias0 = p.ebias[0][(size_t)expert * p.N + n];
            if (EPI == kEpiGateUp && n_ok && p.ebias[1] != nullptr) bias1 = p.ebias[1][(size_t)expert * p.N + n];
            const uint32_t tbase = tmem_base + ((uint32_t)(32 * q) << 16) + a * S::ACC_COLS;
            for (int c0 = 0; c0 < rows; c0 += 32) {
                uint32_t r0[32], r1[32];
                tmem_ld32(tbase + c0, r0);
                if (EPI == kEpiGateUp) tmem_ld32(tbase + BN + c0, r1);
                tmem_ld_wait();
                if (!n_ok) continue;
                if (EPI == kEpiStore && p.tiles == nullptr) {
                    // Dense tiling: two accumulators, the epilogue runs under the next tile's main loop and has time
                    // to spare. Element after element with the exit test between them, its stores trickle out; issued
                    // as a burst of 32 (the branch-free form below) they got in the way of the dequantisers' shared-
                    // memory traffic and cost the dense GEMM 4-8 % (253.8 -> 265 us at M = 2048, 85 -> 93 at M = 512).
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (c0 + j >= rows) break;
                        // int8: ((sum * sx[token]) * sw[feature]) / n, in the order of the CPU emulation
                        const float v = S::I8 ? ((float)(int)r0[j] * reinterpret_cast<const float*>(p.s[0])[row0 + c0 + j]) *
                                                    reinterpret_cast<const float*>(p.b[0])[n] * p.limit
                                              : __uint_as_float(r0[j]) + bias0;
                        const size_t o = (size_t)(row0 + c0 + j) * p.ldy + n;
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
                    continue;
                }
                // The 32 token columns of this thread's output feature. No early exit inside the loops: an exit test
                // between the elements serialises them (each then pays the whole dependent chain of the activation,
                // about a hundred cycles) and made the epilogue a third of the grouped GEMM's time; the columns beyond
                // the tile's rows are computed and dropped by the stores' predicates.
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    v[j] = __uint_as_float(r0[j]) + bias0;
                    // gate and up stay fp32 up to the activation (the reference's prefill kernels round them to half
                    // first, GU_HALF, Shaders/qmm_nax_moe.metal:491-505: a storage choice, not needed here)
                    if (EPI == kEpiGateUp) v[j] = glu<ACT>(v[j], __uint_as_float(r1[j]) + bias1, p.limit);
                }
                const int live = rows - c0;  // columns j < live exist
                const size_t o0 = (size_t)(row0 + c0) * p.ldy + n;
                if (p.y_dtype == kF16) {
                    __half* yp = reinterpret_cast<__half*>(p.y) + o0;
                    if (p.accumulate) {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (j < live) yp[(size_t)j * p.ldy] = __float2half_rn(__half2float(yp[(size_t)j * p.ldy]) + v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (j < live) yp[(size_t)j * p.ldy] = __float2half_rn(v[j]);
                    }
                } else if (p.y_dtype == kF32) {
                    float* yp = reinterpret_cast<float*>(p.y) + o0;
                    if (p.accumulate) {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (j < live) yp[(size_t)j * p.ldy] += v[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (j < live) yp[(size_t)j * p.ldy] = v[j];
                    }
                } else {
                    uint16_t* yp = reinterpret_cast<uint16_t*>(p.y) + o0;
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (j < live)
                            yp[(size_t)j * p.ldy] =
                                (uint16_t)f32_to_bf16_bits(p.accumulate ? bf16_bits_to_f32(yp[(size_t)j * p.ldy]) + v[j] : v[j]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * a);
        }
    } else if (!S::PLAIN && warp < 14) {
        // ================= dequantisers (256 threads, two groups of four warps) =================
        // Group g takes the K steps with (global step index) % 2 == g: one thread per weight row, both halves of the
        // step. While one group waits for its stage, converts and publishes it, the other is half a period ahead, so the
        // fixed latencies (barrier wait, shared-memory round trip, proxy fence) overlap instead of adding up.
        const int dt = threadIdx.x - 6 * 32;      // 0..255
        const int grp = dt >> 7;                  // which half of the steps
        const int row = dt & 127;                 // weight row inside the tile
        const int sw = row & 7;
        bool ok = true;
        // mxfp4: two scale bytes per step; affine g64: one scale and bias; affine g32: two of each
        constexpr int NB = FMT == kFmtAffine4G32 ? 2 : 1;
        struct SB { uint32_t sc[NWT][2], bi[NWT][NB]; };
        struct Cursor { int wi, ks; uint32_t lin; size_t srow; bool live; };
        auto locate = [&](Cursor& c) {  // srow / live of the item c.wi
            c.live = false;
            c.srow = 0;
            if (c.wi < total_work) {
                uint32_t expert; int row0, rows, n0;
                decode(c.wi, expert, row0, rows, n0);
                c.live = n0 + row < p.N;
                c.srow = ((size_t)expert * p.N + (c.live ? n0 + row : 0)) * row_groups;
            }
        };
        auto advance = [&](Cursor& c) {  // two global steps forward
            c.ks += 2;
            c.lin += 2;
            bool moved = false;
            while (c.ks >= ksteps && c.wi < total_work) { c.ks -= ksteps; c.wi += gridDim.x; moved = true; }
            if (moved) locate(c);
        };
        auto fetch = [&](const Cursor& c, SB& v) {
            const bool live = c.live && c.wi < total_work;
#pragma unroll
            for (int wt = 0; wt < NWT; wt++) {
                if (FMT == kFmtMxfp4) {
                    const unsigned char* sp = reinterpret_cast<const unsigned char*>(p.s[wt]) + c.srow + 2 * c.ks;
                    v.sc[wt][0] = live ? ldg_nc_u8_early(sp) : 127u;
                    v.sc[wt][1] = live ? ldg_nc_u8_early(sp + 1) : 127u;
                    v.bi[wt][0] = 0;
                } else if (FMT == kFmtTernary) {  // one fp16 scale per 128 inputs = two K steps, no bias tensor
                    v.sc[wt][0] = v.sc[wt][1] = live ? ldg_nc_u16_early(reinterpret_cast<const uint16_t*>(p.s[wt]) + c.srow + (c.ks >> 1)) : 0u;
                    v.bi[wt][0] = 0;
                } else if (FMT == kFmtAffine4G32) {
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        v.sc[wt][h] = live ? ldg_nc_u16_early(reinterpret_cast<const uint16_t*>(p.s[wt]) + c.srow + 2 * c.ks + h) : 0u;
                        v.bi[wt][h % NB] = live ? ldg_nc_u16_early(reinterpret_cast<const uint16_t*>(p.b[wt]) + c.srow + 2 * c.ks + h) : 0u;
                    }
                } else {
                    v.sc[wt][0] = v.sc[wt][1] = live ? ldg_nc_u16_early(reinterpret_cast<const uint16_t*>(p.s[wt]) + c.srow + c.ks) : 0u;
                    v.bi[wt][0] = live ? ldg_nc_u16_early(reinterpret_cast<const uint16_t*>(p.b[wt]) + c.srow + c.ks) : 0u;
                }
            }
        };
        auto process = [&](const Cursor& c, const SB& v) -> bool {
            const int s = c.lin % STAGES;
            const uint32_t ph = (c.lin / STAGES) & 1;
            if (!mbar_wait(bar_full + 8 * s, ph, abort_flag)) return false;       // packed codes landed
            if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag)) return false;  // fp16 tile no longer read
            const uint32_t st = smem_u32(smem + s * S::STAGE_BYTES);
#pragma unroll
            for (int wt = 0; wt < NWT; wt++) {
                const uint32_t wd = st + S::X_BYTES + wt * S::WD_BYTES + (row >> 3) * 1024 + sw * 128;
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    const uint32_t pk = st + S::X_BYTES + NWT * S::WD_BYTES + wt * S::WP_BYTES + row * S::PACK_ROW +
                                        half * (S::PACK_ROW / 2);
                    uint4 o[4];
                    dequant32<FMT>(pk, v.sc[wt][half], v.bi[wt][half % NB], o);
#pragma unroll
                    for (int j = 0; j < 4; j++) sts128(wd + (((half * 4 + j) ^ sw) << 4), o[j]);
                }
            }
            fence_async_smem();  // generic-proxy writes -> visible to the tensor core's async-proxy reads
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_ready + 8 * s);
            return true;
        };
        // cursor of the step being converted and of the step whose scales are being fetched (two of this group's steps
        // ahead); three register sets rotate between them
        Cursor cur;
        cur.wi = blockIdx.x; cur.ks = grp; cur.lin = grp;
        {
            bool moved = false;
            while (cur.ks >= ksteps && cur.wi < total_work) { cur.ks -= ksteps; cur.wi += gridDim.x; moved = true; }
            (void)moved;
            locate(cur);
        }
        Cursor pf = cur;
        SB A, B, C;
        fetch(pf, A); advance(pf);
        fetch(pf, B); advance(pf);
        while (ok && cur.wi < total_work) {
            fetch(pf, C); advance(pf);
            ok = process(cur, A); advance(cur);
            if (!ok || cur.wi >= total_work) break;
            fetch(pf, A); advance(pf);
            ok = process(cur, B); advance(cur);
            if (!ok || cur.wi >= total_work) break;
            fetch(pf, B); advance(pf);
            ok = process(cur, C); advance(cur);
        }
    }

    // ---- teardown ------------------------------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, kErrTimeout);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// fp32 / bf16 activations -> fp16, row-major [rows, k] contiguous (the MMA's B operand type)
__global__ void convert_x_f16_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx, __half* __restrict__ out,
                                     int rows, int k) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= (size_t)rows * k) return;
    const size_t r = i / k, c = i % k;
    float v[8];
    load_x8(x, x_dtype, r * ldx + c, v);
    uint4 o;
    o.x = pack_half2(v[0], v[1]); o.y = pack_half2(v[2], v[3]); o.z = pack_half2(v[4], v[5]); o.w = pack_half2(v[6], v[7]);
    *reinterpret_cast<uint4*>(out + i) = o;
}

}  // namespace iq
