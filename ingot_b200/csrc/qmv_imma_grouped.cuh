// MoE decode on the int8 tensor-core path: the expert tiles' gate + up + activation and down projections for tiles of
// up to 16 routed rows (affine 4-bit experts). Same arithmetic as qmv_imma.cuh: codes enter m16n8k32 u8 x s8 MMAs
// unconverted, the tile's activation rows are converted once per tile to block fixed point (two signed 7-bit digits per
// group of 64 inputs), per group y += s * 2^(e-13) * (128 * acc_hi + acc_lo) + b * sum(x); a row's bits do not depend on
// the other rows of its tile.
//
// Work items are (tile, block of R = 16 * rgs weight rows); a CTA takes a contiguous range of items, so a tile's
// activations are converted once per CTA that touches it. Warp 8 streams the blocks (both matrices in gate/up mode)
// through a ring of bulk copies; the eight consumer warps are rgs row blocks x wk K slices, and the K slices meet in
// shared memory in a fixed order.
//
// Replaces the reference's vnax_moe_gateup* / vnax_moe_down_split* decode kernels (Shaders/verify_nax.metal:258-509)
// where the fp16 tile kernels of qmv_stream.cuh ran before; those still serve MXFP4 experts and odd shapes.
#pragma once

#include "common.cuh"
#include "gqmv.cuh"
#include "ptx.cuh"
#include "qmv_imma.cuh"

namespace iq {

constexpr int kQgThreads = 288;  // 8 consumer warps + 1 producer warp

struct QgParams {
    const unsigned char* w[2];
    const unsigned char* s[2];
    const unsigned char* b[2];
    int64_t w_ebytes, s_ebytes;  // bytes between experts (codes; scales = biases)
    int32_t N, K;
    const void* x;
    int32_t x_dtype;
    int64_t ldx;
    const uint32_t* row_map;     // gate/up: sorted position -> pair id (token = pair / topk); null: rows are in place
    int32_t topk;
    const Tile* tiles;
    const uint32_t* ntiles;
    void* y;
    int32_t y_dtype;
    int64_t ldy;
    const float* ebias[2];
    float limit;
    int32_t act;
    int32_t rgs, wk;             // row blocks of 16 per item x K slices = 8 consumer warps
    int32_t NB;                  // items per tile
    int32_t row_bytes, row_pitch, srow_bytes;
    int32_t mat_bytes, stage_bytes, nstages;
    int32_t expert_lo;           // tensor-copy staging: the first expert the stacked tensors (and the maps) hold
    int32_t xq_bytes, xsc_bytes, red_bytes;
    int32_t* status;
};

// MODE: kModeGateUp (two matrices, h = act(gate, up)) or kModeDown; MS: sets of four activation rows per tile (2 or 4).
// TM: a block of R rows of a matrix arrives as one swizzled tensor copy, laid out [128-byte column][row][128] (see
// qmv_imma.cuh), instead of one bulk copy per row: expert rows are 384 to 1024 bytes, and copies that short are bound by
// their issue rate (one producer warp sustains about one per 60 ns), not by their bytes.
template <int MODE, int MS, bool TM>
__global__ void __launch_bounds__(kQgThreads, 1)
    qmv_imma_grouped_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1, const QgParams p) {
    constexpr int NW = MODE == kModeGateUp ? 2 : 1;
    constexpr int GB = 32;  // code bytes per group of 64 inputs (4-bit)
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* xq = smem;                                            // [groups][MS][32 lanes] uint4: B fragments
    float2* xsc = reinterpret_cast<float2*>(smem + p.xq_bytes);          // [groups][MS * 4 rows] {2^(e-13), sum x}
    float* red = reinterpret_cast<float*>(smem + p.xq_bytes + p.xsc_bytes);  // [2][8 warps][NW * MS][32 lanes][2]
    unsigned char* stages = smem + p.xq_bytes + p.xsc_bytes + p.red_bytes;
    if (TM) stages += (1024u - (smem_u32(stages) & 1023u)) & 1023u;  // the swizzle pattern is a function of the address
    uint64_t* bars = reinterpret_cast<uint64_t*>(stages + (size_t)p.nstages * p.stage_bytes);
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * p.nstages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * p.nstages);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (TM && tid == 256) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map0) : "memory");
        if (NW == 2) asm volatile("prefetch.tensormap [%0];" ::"l"(&map1) : "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < p.nstages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 8);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();  // the tile list, the activations and y come from earlier kernels of the stream

    const int R = 16 * p.rgs;
    const int G = p.K / 64;
    const int codes_bytes = R * p.row_pitch;
    const int sc_bytes = R * p.srow_bytes;
    const int total = (int)(*p.ntiles) * p.NB;
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int lo = min(total, (int)blockIdx.x * per), hi = min(total, lo + per);

    if (warp == 8) {
        // ================= producer =================
        bool ok = true;
        for (int item = lo, it = 0; item < hi && ok; item++, it++) {
            const int s = it % p.nstages;
            const uint32_t ph = (it / p.nstages) & 1;
            const int ti = item / p.NB, blk = item % p.NB;
            const uint32_t expert = p.tiles[ti].expert;
            const int r0 = blk * R;
            const int rows = min(R, p.N - r0);
            ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            // (a tensor copy counts its whole box; rows past the block belong to the next expert or arrive as zeros)
            if (lane == 0)
                mbar_arrive_expect_tx(bar_full + 8 * s, NW * ((TM ? R : rows) * p.row_bytes + 2 * rows * p.srow_bytes));
            __syncwarp();
            const uint32_t st = smem_u32(stages + (size_t)s * p.stage_bytes);
            if (TM) {
                // per matrix: one tensor copy of the codes, one bulk copy of the scales, one of the biases
                if (lane < NW * 3) {
                    const int i = lane / 3, q = lane % 3;
                    const uint32_t dst = st + i * p.mat_bytes;
                    if (q == 0) {
                        tma_load_3d(dst, i == 0 ? &map0 : &map1, bar_full + 8 * s, 0,
                                    (int)(expert - (uint32_t)p.expert_lo) * p.N + r0, 0);
                    } else {
                        const unsigned char* src = (q == 1 ? p.s[i] : p.b[i]) + expert * p.s_ebytes + (int64_t)r0 * p.srow_bytes;
                        bulk_g2s(dst + codes_bytes + (q == 2 ? sc_bytes : 0), src, rows * p.srow_bytes, bar_full + 8 * s);
                    }
                }
            } else {
                // per matrix: one copy per row of codes (into padded rows), one for the scales, one for the biases
                for (int j = lane; j < NW * (rows + 2); j += 32) {
                    const int i = j / (rows + 2), q = j % (rows + 2);
                    const uint32_t dst = st + i * p.mat_bytes;
                    if (q < rows) {
                        bulk_g2s(dst + q * p.row_pitch, p.w[i] + expert * p.w_ebytes + (int64_t)(r0 + q) * p.row_bytes, p.row_bytes,
                                 bar_full + 8 * s);
                    } else if (q == rows) {
                        bulk_g2s(dst + codes_bytes, p.s[i] + expert * p.s_ebytes + (int64_t)r0 * p.srow_bytes, rows * p.srow_bytes,
                                 bar_full + 8 * s);
                    } else {
                        bulk_g2s(dst + codes_bytes + sc_bytes, p.b[i] + expert * p.s_ebytes + (int64_t)r0 * p.srow_bytes,
                                 rows * p.srow_bytes, bar_full + 8 * s);
                    }
                }
            }
        }
        if (!ok) {  // give copies in flight time to land before the CTA's shared memory is released
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {}
        }
    } else {
        // ================= consumers =================
        const int g = lane >> 2, t = lane & 3;
        const int rb = warp / p.wk, ks = warp % p.wk;
        const int gw = G / p.wk, g0 = ks * gw;
        const uint32_t xq32 = smem_u32(xq) + lane * 16, xsc32 = smem_u32(xsc) + t * 8;
        int cur_tile = -1, M = 0;
        uint32_t xtok = 0;
        Tile tile;
        tile.expert = 0; tile.start = 0; tile.count = 0; tile.pad = 0;
        for (int item = lo, it = 0; item < hi; item++, it++) {
            const int s = it % p.nstages;
            const uint32_t ph = (it / p.nstages) & 1;
            const int ti = item / p.NB, blk = item % p.NB;
            if (ti != cur_tile) {
                // ---- this tile's activation rows -> block fixed point in B-fragment order (see qmv_imma.cuh) -----------
                if (cur_tile >= 0) qi_consumer_barrier(256);
                cur_tile = ti;
                tile = p.tiles[ti];
                M = min((int)tile.count, 4 * MS);
                for (int u = tid; u < G * 8 * (4 * MS - M); u += 256) {
                    const int m = M + u / (G * 8), j = (u >> 3) % G, w8 = u & 7;
                    const int fb = ((j * MS + (m >> 2)) * 32 + 8 * (m & 3)) * 16 + (w8 & 1) * 8 + (w8 >> 1) * 16;
                    *reinterpret_cast<uint2*>(xq + fb) = make_uint2(0, 0);
                    *reinterpret_cast<uint2*>(xq + fb + 64) = make_uint2(0, 0);
                    if (w8 == 0) xsc[j * 4 * MS + m] = make_float2(0.f, 0.f);
                }
                for (int u = tid; u < (G * 8 * M + 31) / 32 * 32; u += 256) {
                    const bool live = u < G * 8 * M;
                    const int m = live ? u / (G * 8) : 0, j = (u >> 3) % G, w8 = u & 7;
                    size_t row;
                    if (MODE == kModeGateUp && p.row_map != nullptr) row = p.row_map[tile.start + m] / (uint32_t)p.topk;
                    else row = (size_t)tile.start + m;
                    float v[8];
                    load_x8(p.x, p.x_dtype, row * p.ldx + j * 64 + w8 * 8, v);
                    float amax = 0.f, sum = 0.f;
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        amax = fmaxf(amax, fabsf(v[k]));
                        sum += v[k];
                    }
#pragma unroll
                    for (int o = 1; o < 8; o <<= 1) {
                        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                        sum += __shfl_xor_sync(0xffffffffu, sum, o);
                    }
                    float scale, inv;
                    qi_group_scale(amax, sum, scale, inv);
                    if (!live) continue;
                    if (w8 == 0) xsc[j * 4 * MS + m] = make_float2(scale, sum);
                    uint32_t hi_w[2] = {0, 0}, lo_w[2] = {0, 0};
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const int X = __float2int_rn(v[k] * inv);
                        const int hi_d = (X + 64) >> 7, lo_d = X - (hi_d << 7);
                        const int half = k & 1, i = k >> 1;  // even inputs: low nibbles (b0), odd: high nibbles (b1)
                        hi_w[half] |= (uint32_t)(hi_d & 0xFF) << (8 * i);
                        lo_w[half] |= (uint32_t)(lo_d & 0xFF) << (8 * i);
                    }
                    const int tt = w8 >> 1, mm = w8 & 1;
                    const int fb = ((j * MS + (m >> 2)) * 32 + 8 * (m & 3)) * 16 + mm * 8;
                    *reinterpret_cast<uint2*>(xq + fb + tt * 16) = make_uint2(hi_w[0], hi_w[1]);
                    *reinterpret_cast<uint2*>(xq + fb + (4 + tt) * 16) = make_uint2(lo_w[0], lo_w[1]);
                }
                xtok = qi_consumer_barrier(256) + (uint32_t)ti;
            }
            const int r0 = blk * R;
            const int rows = min(R, p.N - r0);
            const bool rows_ok = rb * 16 < rows;
            const bool ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
            const uint32_t tok = (uint32_t)it + (ok ? 0u : 0x80000000u);
            float acc[NW][MS][2];
#pragma unroll
            for (int i = 0; i < NW; i++)
#pragma unroll
                for (int c = 0; c < MS; c++) acc[i][c][0] = acc[i][c][1] = 0.f;
            if (ok && rows_ok) {
                const uint32_t st = smem_u32(stages + (size_t)s * p.stage_bytes);
                for (int q = 0; q < gw; q++) {
                    const int grp = g0 + q;
                    uint4 xb[MS];
                    float2 xs[MS];
#pragma unroll
                    for (int c = 0; c < MS; c++) {
                        xb[c] = lds128_after(xq32 + (grp * MS + c) * 512, xtok);
                        xs[c] = lds64f_after(xsc32 + (grp * MS + c) * 32, xtok);
                    }
#pragma unroll
                    for (int i = 0; i < NW; i++) {
                        // TM: column grp / 4 of the block, row rb * 16 + g, 16-byte piece ((grp % 4) * 2 + t / 2) ^ g
                        const uint32_t wa0 = st + i * p.mat_bytes +
                                             (TM ? (grp >> 2) * (R * 128) + (rb * 16 + g) * 128 +
                                                       (((((grp & 3) << 1) + (t >> 1)) ^ g) << 4) + ((t & 1) << 3)
                                                 : (rb * 16 + g) * p.row_pitch + t * 8 + grp * GB);
                        const uint32_t wa1 = wa0 + (TM ? 1024 : 8 * p.row_pitch);
                        const uint32_t sa0 = st + i * p.mat_bytes + codes_bytes + (rb * 16 + g) * p.srow_bytes + grp * 2;
                        const uint32_t sa1 = sa0 + 8 * p.srow_bytes;
                        const uint2 w0 = lds64_after(wa0, tok), w1 = lds64_after(wa1, tok);
                        const float sc0 = __uint_as_float(lds_u16_after(sa0, tok) << 16);
                        const float sc1 = __uint_as_float(lds_u16_after(sa1, tok) << 16);
                        const float bi0 = __uint_as_float(lds_u16_after(sa0 + sc_bytes, tok) << 16);
                        const float bi1 = __uint_as_float(lds_u16_after(sa1 + sc_bytes, tok) << 16);
                        constexpr uint32_t MSK = 0x0F0F0F0Fu;
                        const uint32_t a00 = w0.x & MSK, a01 = w1.x & MSK, a02 = (w0.x >> 4) & MSK, a03 = (w1.x >> 4) & MSK;
                        const uint32_t a10 = w0.y & MSK, a11 = w1.y & MSK, a12 = (w0.y >> 4) & MSK, a13 = (w1.y >> 4) & MSK;
                        const int z[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int c = 0; c < MS; c++) {
                            int d[4];
                            imma16832_u8s8(d, a00, a01, a02, a03, xb[c].x, xb[c].y, z);
                            imma16832_u8s8(d, a10, a11, a12, a13, xb[c].z, xb[c].w, d);
                            const float v0 = (float)(d[0] * 128 + d[1]), v1 = (float)(d[2] * 128 + d[3]);
                            acc[i][c][0] = fmaf(v0, sc0 * xs[c].x, acc[i][c][0]);
                            acc[i][c][0] = fmaf(bi0, xs[c].y, acc[i][c][0]);
                            acc[i][c][1] = fmaf(v1, sc1 * xs[c].x, acc[i][c][1]);
                            acc[i][c][1] = fmaf(bi1, xs[c].y, acc[i][c][1]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(bar_empty + 8 * s);

            // ---- the K slices meet in shared memory; the slice-0 warp of each row block adds them in order ----------
            float* mine = red + ((it & 1) * 8 + warp) * (NW * MS * 64);
            if (p.wk > 1) {
#pragma unroll
                for (int i = 0; i < NW; i++)
#pragma unroll
                    for (int c = 0; c < MS; c++) {
                        mine[(i * MS + c) * 64 + lane * 2] = acc[i][c][0];
                        mine[(i * MS + c) * 64 + lane * 2 + 1] = acc[i][c][1];
                    }
            }
            if (qi_consumer_barrier_or(256, !ok)) break;  // a wait gave up somewhere: everybody leaves together
            if (ks != 0 || !rows_ok) continue;
            if (p.wk > 1) {
#pragma unroll
                for (int i = 0; i < NW; i++)
#pragma unroll
                    for (int c = 0; c < MS; c++) {
                        float y0 = 0.f, y1 = 0.f;
                        for (int k = 0; k < p.wk; k++) {
                            const float* r = red + ((it & 1) * 8 + warp + k) * (NW * MS * 64) + (i * MS + c) * 64 + lane * 2;
                            y0 += r[0];
                            y1 += r[1];
                        }
                        acc[i][c][0] = y0;
                        acc[i][c][1] = y1;
                    }
            }
#pragma unroll
            for (int c = 0; c < MS; c++) {
                const int m = 4 * c + t;
                if (m >= M) continue;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int n = r0 + rb * 16 + g + 8 * h;
                    float v = acc[0][c][h];
                    if (MODE == kModeGateUp) {
                        float u = acc[NW - 1][c][h];
                        if (p.ebias[0] != nullptr) {
                            v += p.ebias[0][(size_t)tile.expert * p.N + n];
                            u += p.ebias[1][(size_t)tile.expert * p.N + n];
                        }
                        v = glu_rt(p.act, v, u, p.limit);
                    } else {
                        if (p.ebias[0] != nullptr) v += p.ebias[0][(size_t)tile.expert * p.N + n];
                    }
                    const size_t o = (size_t)(tile.start + m) * p.ldy + n;
                    if (p.y_dtype == kF32) reinterpret_cast<float*>(p.y)[o] = v;
                    else if (p.y_dtype == kF16) reinterpret_cast<__half*>(p.y)[o] = __float2half_rn(v);
                    else reinterpret_cast<uint16_t*>(p.y)[o] = (uint16_t)f32_to_bf16_bits(v);
                }
            }
        }
    }
    __syncthreads();
    if (*abort_flag && tid == 0 && p.status != nullptr) atomicExch(p.status, kErrTimeout);
}

}  // namespace iq
