// Streaming quantized GEMV: the weight stream goes HBM -> shared memory through a ring of bulk (TMA) copies, so the
// bytes in flight per SM are set by the ring (3-6 stages of 24-64 KB), not by registers. One persistent CTA per SM:
//   warp 8       producer: per stage one block of R consecutive weight rows over the whole K (codes, scales and biases
//                are each one contiguous range of the MLX layout, so a block is 2-3 bulk copies per matrix)
//   warps 0..7   consumers: RGS row groups of 16 rows x WK K-slices; dequantise from shared memory and multiply on
//                m16n8k16 fragments exactly as gqmv_kernel does (same fragment order, same fixed-order K reduction,
//                hence the same row-invariant bits)
// Work items are (tile, row block); a CTA takes a contiguous range of items so that the activations of a tile are
// staged once. With programmatic dependent launch the producer of the dense form starts streaming weights while the
// previous kernel of the stream is still draining; activations are only read after the dependency wait.
//
// Same operators as gqmv.cuh (the reference's vnax_qmv* / vnax_moe_gateup* / vnax_moe_down_split*,
// Shaders/verify_nax.metal:105-509); this is the path taken when a block of 16+ rows over the whole K fits a stage.
#pragma once

#include "common.cuh"
#include "gqmv.cuh"
#include <type_traits>

#include "ptx.cuh"

namespace iq {

constexpr int kQsConsumers = 256;
constexpr int kQsThreads = 288;
constexpr int kQsPiece = 8192;  // bytes per bulk copy

struct QsParams {
    const unsigned char* w[2];
    const unsigned char* s[2];
    const unsigned char* b[2];
    int64_t w_ebytes, s_ebytes;  // bytes between experts (codes; scales = biases)
    int32_t N, K;
    const void* x;
    int32_t x_dtype;
    int64_t ldx;
    const uint32_t* row_map;
    int32_t topk;
    const Tile* tiles;
    const uint32_t* ntiles;
    int32_t M;
    void* y;
    int32_t y_dtype;
    int64_t ldy;
    int32_t accumulate;
    const float* ebias[2];
    float limit;
    int32_t act;
    // blocking
    int32_t R;          // weight rows per block (16 * rgs)
    int32_t NB;         // blocks per expert
    int32_t rgs, wk;    // row groups x K slices = 8 consumer warps
    int32_t row_bytes;  // code bytes per weight row
    int32_t srow_bytes; // scale bytes per weight row
    int32_t mat_bytes;  // bytes of one matrix inside a stage (codes + scales (+ biases) of R rows)
    int32_t stage_bytes;
    int32_t nstages;
    // shared-memory layout
    int32_t xs_bytes, red_bytes;
    int32_t* status;
};

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ bool consumer_barrier_or(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.or.pred q, 1, 256, p;\nselp.u32 %0, 1, 0, q;\n}\n"
        : "=r"(r)
        : "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}

template <int FMT, int MH, int MODE>
__global__ void __launch_bounds__(kQsThreads, (MH == 1 && MODE != kModeGateUp) ? 2 : 1) qmv_stream_kernel(const QsParams p) {
    using F = FmtTraits<FMT>;
    constexpr int NW = MODE == kModeGateUp ? 2 : 1;
    extern __shared__ __align__(128) unsigned char smem[];
    uint4* xs = reinterpret_cast<uint4*>(smem);
    float* red = reinterpret_cast<float*>(smem + p.xs_bytes);
    unsigned char* stages = smem + p.xs_bytes + p.red_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(stages + (size_t)p.nstages * p.stage_bytes);
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * p.nstages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * p.nstages);
    uint4* zero16 = reinterpret_cast<uint4*>(bars + 2 * p.nstages + 2);  // 16 bytes of zeros for idle fragment lanes

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < p.nstages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 8);
        }
        *abort_flag = 0;
        *zero16 = make_uint4(0, 0, 0, 0);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    __syncthreads();
    pdl_launch_dependents();

    const int sc_bytes = p.R * p.srow_bytes;       // scales (and biases) of a block
    const int codes_bytes = p.R * p.row_bytes;
    const int row_groups = p.K / F::GROUP;
    const int nch = p.row_bytes / 16;              // 16-byte chunks per weight row
    const int nsteps = (nch + 3) / 4;

    // the work list may come from the previous kernel: only the dense form may look at its work before the wait
    if (MODE != kModePlain) pdl_wait();
    const int total = (p.tiles != nullptr ? (int)(*p.ntiles) : 1) * p.NB;
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int lo = min(total, (int)blockIdx.x * per), hi = min(total, lo + per);

    if (warp == 8) {
        // ================= producer =================
        bool ok = true;
        for (int item = lo, it = 0; item < hi && ok; item++, it++) {
            const int s = it % p.nstages;
            const uint32_t ph = (it / p.nstages) & 1;
            const int ti = item / p.NB, blk = item % p.NB;
            const uint32_t expert = p.tiles != nullptr ? p.tiles[ti].expert : 0;
            const int r0 = blk * p.R;
            const int rows = min(p.R, p.N - r0);
            ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t cb = rows * p.row_bytes, sb = rows * p.srow_bytes;
            if (lane == 0) mbar_arrive_expect_tx(bar_full + 8 * s, NW * (cb + sb * (F::BIAS ? 2 : 1)));
            __syncwarp();
            const uint32_t st = smem_u32(stages + (size_t)s * p.stage_bytes);
            const int npc = (cb + kQsPiece - 1) / kQsPiece;  // code pieces per matrix
            const int per_mat = npc + (F::BIAS ? 2 : 1);
            for (int pc = lane; pc < NW * per_mat; pc += 32) {
                const int i = pc / per_mat, j = pc % per_mat;
                const uint32_t dst = st + i * p.mat_bytes;
                if (j < npc) {
                    const uint32_t off = j * kQsPiece;
                    bulk_g2s(dst + off, p.w[i] + expert * p.w_ebytes + (int64_t)r0 * p.row_bytes + off,
                             min((uint32_t)kQsPiece, cb - off), bar_full + 8 * s);
                } else if (j == npc) {
                    bulk_g2s(dst + codes_bytes, p.s[i] + expert * p.s_ebytes + (int64_t)r0 * p.srow_bytes, sb,
                             bar_full + 8 * s);
                } else {
                    bulk_g2s(dst + codes_bytes + sc_bytes, p.b[i] + expert * p.s_ebytes + (int64_t)r0 * p.srow_bytes, sb,
                             bar_full + 8 * s);
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
        const int rg = warp / p.wk, wk = warp % p.wk;
        const int spw = (nsteps + p.wk - 1) / p.wk;
        const int jb = wk * spw, je = min(nsteps, jb + spw);
        if (MODE == kModePlain) pdl_wait();  // activations (and y) belong to the previous kernel until here
        int cur_tile = -1;
        int M = 0;
        Tile tile;
        tile.expert = 0; tile.start = 0; tile.count = 0; tile.pad = 0;
        for (int item = lo, it = 0; item < hi; item++, it++) {
            const int s = it % p.nstages;
            const uint32_t ph = (it / p.nstages) & 1;
            const int ti = item / p.NB, blk = item % p.NB;
            if (ti != cur_tile) {
                // ---- stage the activations of this tile (fp16, fragment order) and the per-group sums ----------------
                if (cur_tile >= 0) consumer_barrier();
                cur_tile = ti;
                if (p.tiles != nullptr) tile = p.tiles[ti];
                else tile.count = (uint32_t)p.M;
                M = (int)tile.count;
                const int units_per_row = p.K / 8;
                const int total_units = M * units_per_row;
                for (int uidx = tid; uidx < (total_units + 31) / 32 * 32; uidx += kQsConsumers) {
                    const int m = uidx / units_per_row, ku = uidx % units_per_row;
                    float v[8];
                    if (uidx < total_units) {
                        size_t row;
                        if (MODE == kModeGateUp && p.row_map != nullptr) row = p.row_map[tile.start + m] / (uint32_t)p.topk;
                        else row = (size_t)tile.start + m;
                        load_x8(p.x, p.x_dtype, row * p.ldx + ku * 8, v);
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
                    if (uidx < total_units) {
                        const int kl = ku * 8, cl = kl / F::CK, q = (kl % F::CK) / 8;
                        xs[(((cl >> 2) * F::QU + q) * M + m) * 4 + (cl & 3)] = o;
                    }
                }
                consumer_barrier();
            }
            const int r0 = blk * p.R;
            const int rows = min(p.R, p.N - r0);
            const bool rows_ok = rg * 16 < rows;
            const unsigned char* st = stages + (size_t)s * p.stage_bytes;

            // two independent accumulation chains per output (even / odd MMAs), added at the end in a fixed order
            float acc2[NW][MH][2][4];
#pragma unroll
            for (int i = 0; i < NW; i++)
#pragma unroll
                for (int h = 0; h < MH; h++)
#pragma unroll
                    for (int c2 = 0; c2 < 2; c2++)
#pragma unroll
                        for (int e = 0; e < 4; e++) acc2[i][h][c2][e] = 0.f;
            float acc[NW][MH][4];

            const bool ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
            const int lr = rg * 16 + g;  // this lane's first row inside the block
            if (ok && rows_ok) {
                const uint32_t st32 = smem_u32(st);
                // per-lane shared-memory addresses of the codes and scales of rows lr and lr + 8
                uint32_t ca[NW][2], sa[NW][2];
#pragma unroll
                for (int i = 0; i < NW; i++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        ca[i][h] = st32 + i * p.mat_bytes + (lr + 8 * h) * p.row_bytes + t * 16;
                        sa[i][h] = st32 + i * p.mat_bytes + codes_bytes + (lr + 8 * h) * p.srow_bytes +
                                   (FMT == kFmtAffine4 ? 2 * (t >> 1) : (FMT == kFmtMxfp4 ? t : 0));
                    }
                constexpr int SSTEP = FMT == kFmtAffine8 ? 2 : 4;  // scale bytes per step of four chunks
                // activation fragments: live lanes walk the staged x, the others keep reading one block of zeros
                uint32_t xa[MH], xstep[MH];
#pragma unroll
                for (int h = 0; h < MH; h++) {
                    const int m = g + 8 * h;
                    xa[h] = m < M ? smem_u32(xs) + (m * 4 + t) * 16 : smem_u32(zero16);
                    xstep[h] = m < M ? M * 64 : 0;
                }
                auto step = [&](int j, auto full_tag) {
                    constexpr bool FULL = decltype(full_tag)::value;
                    const bool c_ok = FULL || 4 * j + t < nch;
                    uint4 cv[NW][2];
                    DqConst dq[NW][2];
#pragma unroll
                    for (int i = 0; i < NW; i++)
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (c_ok) {
                                cv[i][h] = lds128(ca[i][h] + j * 64);
                                dq[i][h] = FMT == kFmtMxfp4 ? make_dq<FMT>(lds_u8(sa[i][h] + j * SSTEP))
                                                            : make_dq<FMT>(lds_u16(sa[i][h] + j * SSTEP),
                                                                           lds_u16(sa[i][h] + sc_bytes + j * SSTEP));
                            } else {
                                cv[i][h] = make_uint4(0, 0, 0, 0);
                                dq[i][h] = make_dq<FMT>(FMT == kFmtMxfp4 ? 127u : 0u);
                            }
                        }
#pragma unroll
                    for (int q = 0; q < F::QU; q++) {
                        uint4 xf[MH];
#pragma unroll
                        for (int h = 0; h < MH; h++)
                            xf[h] = c_ok ? lds128(xa[h] + (j * F::QU + q) * xstep[h]) : make_uint4(0, 0, 0, 0);
                        constexpr int WPQ = FMT == kFmtAffine8 ? 2 : 1;
#pragma unroll
                        for (int ww = 0; ww < WPQ; ww++) {
                            const int wd = q * WPQ + ww;
#pragma unroll
                            for (int i = 0; i < NW; i++) {
                                uint32_t pa[4], pb[4];
                                dequant_word<FMT>(word_of(cv[i][0], wd), dq[i][0], pa);
                                dequant_word<FMT>(word_of(cv[i][1], wd), dq[i][1], pb);
#pragma unroll
                                for (int h = 0; h < MH; h++) {
                                    if (FMT == kFmtAffine8) {
                                        const uint32_t b0 = ww == 0 ? xf[h].x : xf[h].z, b1 = ww == 0 ? xf[h].y : xf[h].w;
                                        mma16816(acc2[i][h][ww], pa[0], pb[0], pa[1], pb[1], b0, b1);
                                    } else {
                                        mma16816(acc2[i][h][0], pa[0], pb[0], pa[1], pb[1], xf[h].x, xf[h].y);
                                        mma16816(acc2[i][h][1], pa[2], pb[2], pa[3], pb[3], xf[h].z, xf[h].w);
                                    }
                                }
                            }
                        }
                    }
                };
                const int jfull = min(je, nch / 4);  // steps whose four chunks all exist
#pragma unroll 2
                for (int j = jb; j < jfull; j++) step(j, std::true_type{});
                for (int j = max(jb, jfull); j < je; j++) step(j, std::false_type{});
            }
#pragma unroll
            for (int i = 0; i < NW; i++)
#pragma unroll
                for (int h = 0; h < MH; h++)
#pragma unroll
                    for (int e = 0; e < 4; e++) acc[i][h][e] = acc2[i][h][0][e] + acc2[i][h][1][e];
            // the stage is free as soon as every warp has read its part
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(bar_empty + 8 * s);

            // ---- fixed-order reduction over the K slices, then the epilogue in the slice-0 warps ---------------------
            float* mine = red + (size_t)((it & 1) * 8 + warp) * (NW * MH * 4 * 32);
            if (p.wk > 1) {
#pragma unroll
                for (int i = 0; i < NW; i++)
#pragma unroll
                    for (int h = 0; h < MH; h++)
#pragma unroll
                        for (int e = 0; e < 4; e++) mine[((i * MH + h) * 4 + e) * 32 + lane] = acc[i][h][e];
            }
            if (consumer_barrier_or(!ok)) break;  // a wait gave up somewhere: everybody leaves together
            if (wk != 0 || !rows_ok) continue;
            if (p.wk > 1) {
#pragma unroll
                for (int i = 0; i < NW; i++)
#pragma unroll
                    for (int h = 0; h < MH; h++)
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float sum = 0.f;
                            for (int k = 0; k < p.wk; k++)
                                sum += red[(size_t)((it & 1) * 8 + warp + k) * (NW * MH * 4 * 32) + ((i * MH + h) * 4 + e) * 32 + lane];
                            acc[i][h][e] = sum;
                        }
            }
            const int n0 = r0 + rg * 16;
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
    }
    __syncthreads();
    if (*abort_flag && tid == 0 && p.status != nullptr) atomicExch(p.status, kErrTimeout);
}

}  // namespace iq
