// MoE decode on the int8 tensor-core path: the expert tiles' gate + up + activation and down projections for tiles of
// up to 16 routed rows (affine 4-bit experts). Same arithmetic as qmv_imma.cuh: codes enter m16n8k32 u8 x s8 MMAs
// unconverted, the tile's activation rows are converted once per tile to block fixed point (two signed 7-bit digits per
// group of 64 inputs), per group y += s * 2^(e-13) * (128 * acc_hi + acc_lo) + b * sum(x); a row's bits do not depend on
// the other rows of its tile.
//
// Work items are (tile, block of R = 16 * rgs weight rows); a CTA takes a contiguous range of items, so a tile's
// activations are converted once per CTA that touches it. Warp 8 streams the blocks (both matrices in gate/up mode)
// through a ring of bulk copies; the eight consumer warps are rgs row blocks x wk K slices, and the K slices meet in
// shared memory in a fixed order: the consumer warps leave their partial sums in one of two buffers and go on to the
// next item, and four epilogue warps add them up, apply the activation and store, one item behind (hand-over through
// named barriers: buffer full, buffer free), so that no item waits for a barrier of the whole CTA.
//
// Replaces the reference's vnax_moe_gateup* / vnax_moe_down_split* decode kernels (Shaders/verify_nax.metal:258-509)
// where the fp16 tile kernels of qmv_stream.cuh ran before; those still serve MXFP4 experts and odd shapes. The down
// projection of a narrow expert (K = 768) runs here as 128-row blocks without a K split.
#pragma once

#include <type_traits>

#include "common.cuh"
#include "gqmv.cuh"
#include "ptx.cuh"
#include "qmv_imma.cuh"

namespace iq {

constexpr int kQgWarps = 8;      // consumer warps (row blocks x K slices); one producer warp follows them
constexpr int kQgEpiWarps = 4;  // epilogue warps: add the K slices, apply the activation, store
constexpr int kQgThreads = (kQgWarps + 1 + kQgEpiWarps) * 32;

__device__ __forceinline__ void qg_bar_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
__device__ __forceinline__ void qg_bar_arrive(int id, int threads) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

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
    int32_t rgs, wk;             // row blocks of 16 per item x K slices = kQgWarps consumer warps
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
// GW: groups of 64 inputs per consumer warp when fixed at compile time (4), else 0. A warp's K slice does not change from
// item to item, so with GW > 0 its activation fragments stay in registers between tile changes: read from shared
// memory per item they are as many bytes as the codes themselves, and the kernel runs at the shared-memory port's rate.
template <int MODE, int MS, bool TM, int GW>
__global__ void __launch_bounds__(kQgThreads, 1)
    qmv_imma_grouped_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1, const QgParams p) {
    constexpr int NW = MODE == kModeGateUp ? 2 : 1;
    constexpr int GB = 32;  // code bytes per group of 64 inputs (4-bit)
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* xq = smem;                                            // [groups][MS][32 lanes] uint4: B fragments
    float2* xsc = reinterpret_cast<float2*>(smem + p.xq_bytes);          // [groups][MS * 4 rows] {2^(e-13), sum x}
    float* red = reinterpret_cast<float*>(smem + p.xq_bytes + p.xsc_bytes);  // [2][kQgWarps][NW * MS][32 lanes][2]
    unsigned char* stages = smem + p.xq_bytes + p.xsc_bytes + p.red_bytes;
    if (TM) stages += (1024u - (smem_u32(stages) & 1023u)) & 1023u;  // the swizzle pattern is a function of the address
    uint64_t* bars = reinterpret_cast<uint64_t*>(stages + (size_t)p.nstages * p.stage_bytes);
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * p.nstages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * p.nstages);
    uint32_t* srow = reinterpret_cast<uint32_t*>(bars + 2 * p.nstages + 2);  // [16] the tile's activation rows
    volatile int* cut = reinterpret_cast<volatile int*>(srow + 16);           // [2] this CTA's range of items

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NCT = kQgWarps * 32;     // consumer threads
    constexpr int NET = kQgEpiWarps * 32;  // epilogue threads
    if (TM && tid == NCT) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map0) : "memory");
        if (NW == 2) asm volatile("prefetch.tensormap [%0];" ::"l"(&map1) : "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < p.nstages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, kQgWarps);
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
    // This CTA's contiguous range of items. An item of a tile with more live row sets costs more (about 3 + sets in
    // units of issue slots), so the ranges are cut by cost, not by count: warp 0 adds up the tiles' costs (a lane per run
    // of consecutive tiles) and finds where this CTA's share begins and ends. Lists too long for that are cut evenly.
    const int ntl = (int)(*p.ntiles);
    const int total = ntl * p.NB;
    {
        const int per = (total + gridDim.x - 1) / gridDim.x;
        if (tid == 0) {
            cut[0] = min(total, (int)blockIdx.x * per);
            cut[1] = min(total, cut[0] + per);
        }
        __syncwarp();
        constexpr int TPL = 16;  // tiles per lane
        if (warp == 0 && ntl <= 32 * TPL && ntl > 0) {
            const int tpl = (ntl + 31) / 32;
            int w[TPL];
            int mine = 0;
#pragma unroll
            for (int j = 0; j < TPL; j++) {
                const int ti = lane * tpl + j;
                w[j] = 0;
                if (j < tpl && ti < ntl) {
                    const int sets = (min((int)p.tiles[ti].count, 4 * MS) + 3) >> 2;
                    w[j] = 3 + (sets > 2 ? 4 : sets);
                }
                mine += w[j];
            }
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const long long all = (long long)__shfl_sync(0xffffffffu, incl, 31) * p.NB;  // cost of the whole list
            const int before = incl - mine;                                               // tiles before this lane's run
#pragma unroll
            for (int e = 0; e < 2; e++) {
                // first item whose cost prefix reaches the target
                const long long target = all * (long long)(blockIdx.x + e) / gridDim.x;
                const bool here = (long long)before * p.NB <= target && target < (long long)incl * p.NB;
                if (here) {
                    long long acc = (long long)before * p.NB;
                    int ti = lane * tpl, found = total;
#pragma unroll
                    for (int j = 0; j < TPL; j++) {
                        if (found == total && w[j] > 0) {
                            const long long span = (long long)w[j] * p.NB;
                            if (target < acc + span) found = (ti + j) * p.NB + (int)((target - acc + w[j] - 1) / w[j]);
                            acc += span;
                        }
                    }
                    cut[e] = found;
                } else if (target >= all && lane == 0) {
                    cut[e] = total;
                }
            }
        }
        __syncthreads();
    }
    const int lo = cut[0], hi = cut[1];

    if (warp == kQgWarps) {
        // ================= producer =================
        bool ok = true;
        int s = 0, ti = lo / p.NB, blk = lo % p.NB;
        uint32_t ph = 0;
        uint32_t expert = lo < hi ? p.tiles[ti].expert : 0;
        for (int item = lo; item < hi && ok; item++) {
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
            if (++s == p.nstages) { s = 0; ph ^= 1; }
            if (++blk == p.NB) {
                blk = 0;
                ti++;
                if (item + 1 < hi) expert = p.tiles[ti].expert;
            }
        }
        if (!ok) {  // give copies in flight time to land before the CTA's shared memory is released
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {}
        }
    } else if (warp < kQgWarps) {
        // ================= consumers =================
        const int g = lane >> 2, t = lane & 3;
        const int rb = warp / p.wk, ks = warp % p.wk;
        const int gw = GW > 0 ? GW : G / p.wk, g0 = ks * gw;
        const uint32_t xq32 = smem_u32(xq) + lane * 16, xsc32 = smem_u32(xsc) + t * 8;
        int cur_tile = -1, M = 0, sets = 0;  // sets: row sets of four that hold a live row
        uint32_t xtok = 0;
        Tile tile;
        tile.expert = 0; tile.start = 0; tile.count = 0; tile.pad = 0;
        uint4 xbr[GW > 0 ? GW : 1][MS];
        float2 xsr[GW > 0 ? GW : 1][MS];
        int s = 0, ti = lo / p.NB, blk = lo % p.NB;
        uint32_t ph = 0;
        for (int item = lo, it = 0; item < hi; item++, it++) {
            if (ti != cur_tile) {
                // ---- this tile's activation rows -> block fixed point in B-fragment order (see qmv_imma.cuh) -----------
                if (cur_tile >= 0) qi_consumer_barrier(NCT);
                cur_tile = ti;
                tile = p.tiles[ti];
                M = min((int)tile.count, 4 * MS);
                sets = (M + 3) >> 2;
                for (int u = tid; u < G * 8 * (4 * sets - M); u += NCT) {  // dead rows of the live sets
                    const int m = M + u / (G * 8), j = (u >> 3) % G, w8 = u & 7;
                    const int fb = ((j * MS + (m >> 2)) * 32 + 8 * (m & 3)) * 16 + (w8 & 1) * 8 + (w8 >> 1) * 16;
                    *reinterpret_cast<uint2*>(xq + fb) = make_uint2(0, 0);
                    *reinterpret_cast<uint2*>(xq + fb + 64) = make_uint2(0, 0);
                    if (w8 == 0) xsc[j * 4 * MS + m] = make_float2(0.f, 0.f);
                }
                // the rows' places in x first (one round trip to memory for all of them), then the values, four units
                // of eight inputs per thread in flight
                if (tid < M) {
                    srow[tid] = (MODE == kModeGateUp && p.row_map != nullptr) ? p.row_map[tile.start + tid] / (uint32_t)p.topk
                                                                             : tile.start + (uint32_t)tid;
                }
                qi_consumer_barrier(NCT);
                const int units = G * 8 * M, upad = (units + 31) / 32 * 32;
                for (int u0 = tid; u0 < upad; u0 += 4 * NCT) {
                    float v[4][8];
#pragma unroll
                    for (int k4 = 0; k4 < 4; k4++) {
                        const int u = u0 + k4 * NCT;
                        const bool live = u < units;
                        const int m = live ? u / (G * 8) : 0, j = (u >> 3) % G, w8 = u & 7;
                        if (u < upad) load_x8(p.x, p.x_dtype, (size_t)srow[m] * p.ldx + j * 64 + w8 * 8, v[k4]);
                    }
#pragma unroll
                    for (int k4 = 0; k4 < 4; k4++) {
                        const int u = u0 + k4 * NCT;
                        if (u >= upad) break;  // whole warps leave together: upad and NCT are multiples of 32
                        const bool live = u < units;
                        const int m = live ? u / (G * 8) : 0, j = (u >> 3) % G, w8 = u & 7;
                        float amax = 0.f, sum = 0.f;
#pragma unroll
                        for (int k = 0; k < 8; k++) {
                            amax = fmaxf(amax, fabsf(v[k4][k]));
                            sum += v[k4][k];
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
                            const int X = __float2int_rn(v[k4][k] * inv);
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
                }
                xtok = qi_consumer_barrier(NCT) + (uint32_t)ti;
                if (GW > 0) {
#pragma unroll
                    for (int q = 0; q < (GW > 0 ? GW : 1); q++)
#pragma unroll
                        for (int c = 0; c < MS; c++) {  // sets without live rows hold leftovers nobody uses
                            xbr[q][c] = lds128_after(xq32 + ((g0 + q) * MS + c) * 512, xtok);
                            xsr[q][c] = lds64f_after(xsc32 + ((g0 + q) * MS + c) * 32, xtok);
                        }
                }
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
            // NS: the tile's live row sets, as a compile-time bound (no branches between the MMAs of a group)
            auto body = [&](auto ns_c) {
                constexpr int NS = decltype(ns_c)::value;
                const uint32_t st = smem_u32(stages + (size_t)s * p.stage_bytes);
                // Scales and biases: lane L fetches four groups of row L % 16 of the warp's row block with one 8-byte load
                // (lanes 0-15 the scales, 16-31 the biases) and the MMA lanes pick theirs up by shuffle: the rows of these
                // tensors are 2 * G bytes apart, so a load per (row, group) from every lane meets four-way bank conflicts.
                const uint32_t sl = st + codes_bytes + (lane >> 4) * sc_bytes + (rb * 16 + (lane & 15)) * p.srow_bytes + g0 * 2;
#pragma unroll
                for (int q4 = 0; q4 < gw; q4 += 4) {
                    uint2 sw[NW];
#pragma unroll
                    for (int i = 0; i < NW; i++) sw[i] = lds64_after(sl + i * p.mat_bytes + q4 * 2, tok);
#pragma unroll
                    for (int q2 = 0; q2 < 2; q2++) {
                        uint32_t s0w[NW], s1w[NW], b0w[NW], b1w[NW];  // two groups each: bf16 pairs
#pragma unroll
                        for (int i = 0; i < NW; i++) {
                            const uint32_t word = q2 ? sw[i].y : sw[i].x;
                            s0w[i] = __shfl_sync(0xffffffffu, word, g);
                            s1w[i] = __shfl_sync(0xffffffffu, word, g + 8);
                            b0w[i] = __shfl_sync(0xffffffffu, word, g + 16);
                            b1w[i] = __shfl_sync(0xffffffffu, word, g + 24);
                        }
#pragma unroll
                        for (int q1 = 0; q1 < 2; q1++) {
                            const int ql = q4 + q2 * 2 + q1, grp = g0 + ql;
                            uint4 xb[NS];
                            float2 xs[NS];
#pragma unroll
                            for (int c = 0; c < NS; c++) {
                                xb[c] = GW > 0 ? xbr[GW > 0 ? ql : 0][c] : lds128_after(xq32 + (grp * MS + c) * 512, xtok);
                                xs[c] = GW > 0 ? xsr[GW > 0 ? ql : 0][c] : lds64f_after(xsc32 + (grp * MS + c) * 32, xtok);
                            }
                            uint32_t a[NW][8];
#pragma unroll
                            for (int i = 0; i < NW; i++) {
                                // TM: column grp / 4 of the block, row rb * 16 + g, 16-byte piece ((grp % 4) * 2 + t / 2) ^ g
                                const uint32_t wa0 = st + i * p.mat_bytes +
                                                     (TM ? (grp >> 2) * (R * 128) + (rb * 16 + g) * 128 +
                                                               (((((grp & 3) << 1) + (t >> 1)) ^ g) << 4) + ((t & 1) << 3)
                                                         : (rb * 16 + g) * p.row_pitch + t * 8 + grp * GB);
                                const uint32_t wa1 = wa0 + (TM ? 1024 : 8 * p.row_pitch);
                                const uint2 w0 = lds64_after(wa0, tok), w1 = lds64_after(wa1, tok);
                                constexpr uint32_t MSK = 0x0F0F0F0Fu;
                                a[i][0] = w0.x & MSK; a[i][1] = w1.x & MSK; a[i][2] = (w0.x >> 4) & MSK; a[i][3] = (w1.x >> 4) & MSK;
                                a[i][4] = w0.y & MSK; a[i][5] = w1.y & MSK; a[i][6] = (w0.y >> 4) & MSK; a[i][7] = (w1.y >> 4) & MSK;
                            }
                            // the group's 2 * NW * NS MMAs, independent ones next to each other
                            int d[NW][NS][4];
                            const int z[4] = {0, 0, 0, 0};
#pragma unroll
                            for (int i = 0; i < NW; i++)
#pragma unroll
                                for (int c = 0; c < NS; c++)
                                    imma16832_u8s8(d[i][c], a[i][0], a[i][1], a[i][2], a[i][3], xb[c].x, xb[c].y, z);
#pragma unroll
                            for (int i = 0; i < NW; i++)
#pragma unroll
                                for (int c = 0; c < NS; c++)
                                    imma16832_u8s8(d[i][c], a[i][4], a[i][5], a[i][6], a[i][7], xb[c].z, xb[c].w, d[i][c]);
#pragma unroll
                            for (int i = 0; i < NW; i++) {
                                const float sc0 = __uint_as_float(q1 ? (s0w[i] & 0xFFFF0000u) : (s0w[i] << 16));
                                const float sc1 = __uint_as_float(q1 ? (s1w[i] & 0xFFFF0000u) : (s1w[i] << 16));
                                const float bi0 = __uint_as_float(q1 ? (b0w[i] & 0xFFFF0000u) : (b0w[i] << 16));
                                const float bi1 = __uint_as_float(q1 ? (b1w[i] & 0xFFFF0000u) : (b1w[i] << 16));
#pragma unroll
                                for (int c = 0; c < NS; c++) {
                                    const float v0 = (float)(d[i][c][0] * 128 + d[i][c][1]);
                                    const float v1 = (float)(d[i][c][2] * 128 + d[i][c][3]);
                                    acc[i][c][0] = fmaf(v0, sc0 * xs[c].x, acc[i][c][0]);
                                    acc[i][c][0] = fmaf(bi0, xs[c].y, acc[i][c][0]);
                                    acc[i][c][1] = fmaf(v1, sc1 * xs[c].x, acc[i][c][1]);
                                    acc[i][c][1] = fmaf(bi1, xs[c].y, acc[i][c][1]);
                                }
                            }
                        }
                    }
                }
            };
            if (ok && rows_ok) {
                if (MS == 4 && sets > 2) body(std::integral_constant<int, MS>{});
                else if (sets > 1) body(std::integral_constant<int, 2>{});
                else body(std::integral_constant<int, 1>{});
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(bar_empty + 8 * s);

            // ---- the K slices meet in shared memory: slab (row block, slice) holds [matrix][set][half][t][g], so that the
            // threads of the epilogue, one per (weight row, activation row), read consecutive words. After a wait gave up
            // the loop goes on without computing, so that every barrier keeps its count and nobody is left waiting.
            const int buf = it & 1;
            if (it >= 2) qg_bar_sync(4 + buf, NCT + NET);  // the epilogue of two items ago has read this buffer
            if (MODE == kModeDown && p.wk == 1) {
                // one K slice: the warp's sums are the outputs, stored from here (the epilogue warps only keep step)
                if (ok && rows_ok) {
#pragma unroll
                    for (int c = 0; c < MS; c++) {
                        const int m = 4 * c + t;
                        if (m >= M) continue;
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const int n = r0 + rb * 16 + g + 8 * h;
                            float v = acc[0][c][h];
                            if (p.ebias[0] != nullptr) v += p.ebias[0][(size_t)tile.expert * p.N + n];
                            const size_t oy = (size_t)(tile.start + m) * p.ldy + n;
                            if (p.y_dtype == kF32) reinterpret_cast<float*>(p.y)[oy] = v;
                            else if (p.y_dtype == kF16) reinterpret_cast<__half*>(p.y)[oy] = __float2half_rn(v);
                            else reinterpret_cast<uint16_t*>(p.y)[oy] = (uint16_t)f32_to_bf16_bits(v);
                        }
                    }
                }
            } else {
                float* mine = red + (buf * kQgWarps + warp) * (NW * MS * 64);
#pragma unroll
                for (int i = 0; i < NW; i++)
#pragma unroll
                    for (int c = 0; c < MS; c++) {
                        mine[(i * MS + c) * 64 + t * 8 + g] = acc[i][c][0];
                        mine[(i * MS + c) * 64 + 32 + t * 8 + g] = acc[i][c][1];
                    }
            }
            qg_bar_arrive(2 + buf, NCT + NET);
            if (++s == p.nstages) { s = 0; ph ^= 1; }
            if (++blk == p.NB) { blk = 0; ti++; }
        }
    } else {
        // ================= epilogue =================
        const int et = tid - (kQgWarps + 1) * 32;
        const int rsh = 31 - __clz(R);  // R is a power of two
        int ti = lo / p.NB, blk = lo % p.NB, cur_tile = -1, M = 0;
        Tile tile;
        tile.expert = 0; tile.start = 0; tile.count = 0; tile.pad = 0;
        for (int item = lo, it = 0; item < hi; item++, it++) {
            if (ti != cur_tile) {
                cur_tile = ti;
                tile = p.tiles[ti];
                M = min((int)tile.count, 4 * MS);
            }
            const int r0 = blk * R;
            const int rows = min(R, p.N - r0);
            const int buf = it & 1;
            qg_bar_sync(2 + buf, NCT + NET);
            const bool good = *abort_flag == 0;
            // Outputs (weight row n, activation row m), n fastest; with two matrices a pair of neighbouring lanes takes one
            // output, one matrix each, and the even lane gets the other's sum by shuffle. Slices are added in slice order.
            // Two outputs per thread and pass, all their loads first.
            // live row sets only; a multiple of 32: whole warps stay together. Nothing to add up with one K slice of a down
            // projection: the consumers stored the outputs themselves.
            const int total = (MODE == kModeDown && p.wk == 1) ? 0 : NW * (R * 4 * ((M + 3) >> 2));
            for (int u0 = et; u0 < total; u0 += 2 * NET) {
                float part[2][kQgWarps];
                int nl[2], m[2];
                bool live[2];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int u = u0 + h * NET;
                    const int i = NW == 2 ? (u & 1) : 0, o = NW == 2 ? (u >> 1) : u;
                    nl[h] = o & (R - 1);
                    m[h] = o >> rsh;
                    live[h] = good && u < total && m[h] < M && nl[h] < rows;
                    const float* r = red + (buf * kQgWarps + (nl[h] >> 4) * p.wk) * (NW * MS * 64) + (i * MS + (m[h] >> 2)) * 64 +
                                     ((nl[h] >> 3) & 1) * 32 + (m[h] & 3) * 8 + (nl[h] & 7);
#pragma unroll
                    for (int k = 0; k < kQgWarps; k++) part[h][k] = (live[h] && k < p.wk) ? r[k * (NW * MS * 64)] : 0.f;
                }
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    if (u0 + h * NET >= total) break;  // warp-uniform
                    float v = 0.f;
#pragma unroll
                    for (int k = 0; k < kQgWarps; k++) v += part[h][k];  // absent slices add +0
                    float uu = 0.f;
                    if (NW == 2) uu = __shfl_down_sync(0xffffffffu, v, 1);
                    if (!live[h] || (NW == 2 && (lane & 1))) continue;
                    const int n = r0 + nl[h];
                    if (MODE == kModeGateUp) {
                        if (p.ebias[0] != nullptr) {
                            v += p.ebias[0][(size_t)tile.expert * p.N + n];
                            uu += p.ebias[1][(size_t)tile.expert * p.N + n];
                        }
                        v = glu_rt(p.act, v, uu, p.limit);
                    } else {
                        if (p.ebias[0] != nullptr) v += p.ebias[0][(size_t)tile.expert * p.N + n];
                    }
                    const size_t oy = (size_t)(tile.start + m[h]) * p.ldy + n;
                    if (p.y_dtype == kF32) reinterpret_cast<float*>(p.y)[oy] = v;
                    else if (p.y_dtype == kF16) reinterpret_cast<__half*>(p.y)[oy] = __float2half_rn(v);
                    else reinterpret_cast<uint16_t*>(p.y)[oy] = (uint16_t)f32_to_bf16_bits(v);
                }
            }
            if (item + 2 < hi) qg_bar_arrive(4 + buf, NCT + NET);  // the buffer may be written again
            if (++blk == p.NB) { blk = 0; ti++; }
        }
    }
    __syncthreads();
    if (*abort_flag && tid == 0 && p.status != nullptr) atomicExch(p.status, kErrTimeout);
}

}  // namespace iq
