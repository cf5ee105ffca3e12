// MoE routing, token->expert permutation and combine kernels.
//
// Replaces, on sm_100a, the reference's router/group/combine kernels:
//   router logits   MoE.swift:359-361 (router qmv) and MoEPrefill.swift:176-186 (router qmm)
//   route_topk      Shaders/verify.metal:181-260 (decode) and Shaders/qmm_nax_moe.metal:26-126 (prefill)
//   count/scatter   Shaders/qmm_nax_moe.metal:139-217 (moe_group) and the union build of Shaders/verify.metal:282-318
//   combine         Shaders/qmm_nax_moe.metal:371-396, Shaders/yy_model.metal:129-149
#pragma once

#include "common.cuh"
#include "gqmv.cuh"
#include "ptx.cuh"

namespace iq {

// ---------------------------------------------------------------------------------------------------------------------
// Router logits with a float64 accumulator: logits[t, e] = fp32( sum_k x[t,k] * w[e,k] ).
//
// The inputs are bf16/fp16/fp32 values, so each product is exact in float64 and the sum does not depend on the order
// at fp32 resolution. That is what makes the top-k indices reproducible bit for bit whatever the tiling, the batch
// size or the number of GPUs. Columns E..ld-1 of the output are written as zero (the reference pads the router to a
// multiple of 64 rows, MoE.swift:258-273).
//
// Block: TT tokens (x staged in shared memory as doubles), thread = (expert, k-slice).
constexpr int kRouterTT = 4;

template <int WFMT>  // 0: bf16 dense router; 1: 8-bit affine g64 router
__global__ void __launch_bounds__(256) router_logits_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx,
                                                            const void* __restrict__ wr, const void* __restrict__ ws,
                                                            const void* __restrict__ wb, float* __restrict__ logits,
                                                            int T, int E, int D, int ld, int eb) {
    // eb: experts per block (a power of two, at most 256); blockIdx.y picks the expert range. Few tokens take small
    // ranges so that the dot products spread over many blocks and K slices.
    extern __shared__ __align__(16) unsigned char smem[];
    double* xs = reinterpret_cast<double*>(smem);                      // [TT][D]
    double* part = xs + (size_t)kRouterTT * D;                         // [slices][TT][ee]
    const int tid = threadIdx.x;
    const int t0 = blockIdx.x * kRouterTT;
    const int nt = min(kRouterTT, T - t0);
    const int ee = eb;                          // experts handled by this block
    const int slices = 256 / ee;                // k-slices per expert
    for (int i = tid; i < kRouterTT * D / 8; i += 256) {
        const int tt = i / (D / 8), ku = i % (D / 8);
        float v[8];
        if (tt < nt) load_x8(x, x_dtype, (size_t)(t0 + tt) * ldx + ku * 8, v);
        else {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; e++) xs[(size_t)tt * D + ku * 8 + e] = (double)v[e];
    }
    __syncthreads();
    const int el = tid % ee, sl = tid / ee;
    const int units = D / 8;                                  // 8-input units per row
    const int upw = (units + slices - 1) / slices;            // units per slice
    {
        const int e = blockIdx.y * ee + el;
        double acc[kRouterTT];
#pragma unroll
        for (int tt = 0; tt < kRouterTT; tt++) acc[tt] = 0.0;
        if (e < E && sl < slices) {
            for (int u = sl * upw; u < min(units, (sl + 1) * upw); u++) {
                double w[8];
                if (WFMT == 0) {
                    const uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(wr) +
                                                                    (size_t)e * D + u * 8);
                    const uint32_t q[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        w[2 * j] = (double)__uint_as_float(q[j] << 16);
                        w[2 * j + 1] = (double)__uint_as_float(q[j] & 0xFFFF0000u);
                    }
                } else {
                    const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint32_t*>(wr) +
                                                                    (size_t)e * (D / 4) + u * 2);
                    const int gi = e * (D / 64) + u / 8;
                    // the weight value is the fp32 s*q + b of the reference's CPU dequantisation
                    const float sc = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(ws)[gi]);
                    const float bi = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(wb)[gi]);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        w[j] = (double)__fadd_rn(__fmul_rn(sc, (float)((r.x >> (8 * j)) & 0xFFu)), bi);
                        w[4 + j] = (double)__fadd_rn(__fmul_rn(sc, (float)((r.y >> (8 * j)) & 0xFFu)), bi);
                    }
                }
#pragma unroll
                for (int tt = 0; tt < kRouterTT; tt++) {
                    if (tt >= nt) break;
                    const double2* xp = reinterpret_cast<const double2*>(xs + (size_t)tt * D + u * 8);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const double2 xv = xp[j];
                        acc[tt] = fma(xv.x, w[2 * j], acc[tt]);
                        acc[tt] = fma(xv.y, w[2 * j + 1], acc[tt]);
                    }
                }
            }
        }
        if (slices > 1) {
            __syncthreads();
#pragma unroll
            for (int tt = 0; tt < kRouterTT; tt++) part[((size_t)sl * kRouterTT + tt) * ee + el] = acc[tt];
            __syncthreads();
            if (sl == 0) {
#pragma unroll
                for (int tt = 0; tt < kRouterTT; tt++) {
                    double s = 0.0;
                    for (int k = 0; k < slices; k++) s += part[((size_t)k * kRouterTT + tt) * ee + el];
                    acc[tt] = s;
                }
            }
        }
        if (sl == 0 && e < E) {
#pragma unroll
            for (int tt = 0; tt < kRouterTT; tt++)
                if (tt < nt) logits[(size_t)(t0 + tt) * ld + e] = (float)acc[tt];
        }
    }
    if (blockIdx.y == 0) {
        for (int i = tid; i < kRouterTT * (ld - E); i += 256) {
            const int tt = i / (ld - E), c = E + i % (ld - E);
            if (tt < nt) logits[(size_t)(t0 + tt) * ld + c] = 0.f;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// The same logits for many tokens: a register-tiled float64 GEMM. Block = BM tokens x 64 experts, 128 threads, each
// thread a (BM/8) x 4 tile of accumulators (32 DFMA per six 16-byte shared loads at BM = 64), operands converted to
// float64 on their way into shared memory ([k][row] layout, double-buffered, next chunk's global loads in flight during
// the math). The K range is split over the gridDim.z blocks of a thread-block cluster; their partial tiles are summed
// through distributed shared memory in rank order, so the result does not depend on timing.
constexpr int kRtBN = 64, kRtBK = 32;
constexpr size_t router_tiled_smem(int BM) { return (size_t)2 * kRtBK * (BM + kRtBN) * 8; }

template <int WFMT>
__device__ __forceinline__ void router_w8(const void* __restrict__ wr, const void* __restrict__ ws,
                                          const void* __restrict__ wb, int e, int k, int D, float (&w)[8]) {
    if (WFMT == 0) {
        const uint4 r = ldg_nc_u4(reinterpret_cast<const uint16_t*>(wr) + (size_t)e * D + k);
        const uint32_t q[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            w[2 * j] = __uint_as_float(q[j] << 16);
            w[2 * j + 1] = __uint_as_float(q[j] & 0xFFFF0000u);
        }
    } else {
        const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint32_t*>(wr) + (size_t)e * (D / 4) + k / 4);
        const int gi = e * (D / 64) + k / 64;
        // the weight value is the fp32 s*q + b of the reference's CPU dequantisation
        const float sc = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(ws)[gi]);
        const float bi = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(wb)[gi]);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            w[j] = __fadd_rn(__fmul_rn(sc, (float)((r.x >> (8 * j)) & 0xFFu)), bi);
            w[4 + j] = __fadd_rn(__fmul_rn(sc, (float)((r.y >> (8 * j)) & 0xFFu)), bi);
        }
    }
}

template <int WFMT, int BM>
__global__ void __launch_bounds__(128) router_logits_tiled_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx,
                                                                  const void* __restrict__ wr, const void* __restrict__ ws,
                                                                  const void* __restrict__ wb, float* __restrict__ logits,
                                                                  int T, int E, int D, int ld, int chunks_per_split) {
    constexpr int TM = BM / 8;   // tokens per thread: TM/2 pairs, 16 rows apart
    constexpr int XU = BM / 32;  // 8-value units of x per thread and chunk
    extern __shared__ __align__(16) unsigned char smem_raw[];
    double (*xs)[kRtBK][BM] = reinterpret_cast<double (*)[kRtBK][BM]>(smem_raw);
    double (*wsm)[kRtBK][kRtBN] = reinterpret_cast<double (*)[kRtBK][kRtBN]>(smem_raw + (size_t)2 * kRtBK * BM * 8);
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int t0 = blockIdx.x * BM, e0 = blockIdx.y * kRtBN;
    const int nchunks = D / kRtBK;
    const int c_lo = blockIdx.z * chunks_per_split, c_hi = min(nchunks, c_lo + chunks_per_split);
    // fill roles: consecutive lanes take consecutive rows, so the transposed float64 stores are free of bank conflicts
    const int xrow = tid & (BM - 1), xku = tid / BM;   // BM = 32: four k-units by tid; BM = 64: two, twice
    const int wrow = tid & 63, wku = tid >> 6;
    float xv[XU][8], wv[2][8];
    auto fetch = [&](int c) {
        const int k0 = c * kRtBK;
#pragma unroll
        for (int i = 0; i < XU; i++) {
            if (t0 + xrow < T) load_x8(x, x_dtype, (size_t)(t0 + xrow) * ldx + k0 + (xku + (128 / BM) * i) * 8, xv[i]);
            else {
#pragma unroll
                for (int j = 0; j < 8; j++) xv[i][j] = 0.f;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (e0 + wrow < E) router_w8<WFMT>(wr, ws, wb, e0 + wrow, k0 + (wku + 2 * i) * 8, D, wv[i]);
            else {
#pragma unroll
                for (int j = 0; j < 8; j++) wv[i][j] = 0.f;
            }
        }
    };
    auto stash = [&](int b) {
#pragma unroll
        for (int i = 0; i < XU; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) xs[b][(xku + (128 / BM) * i) * 8 + j][xrow] = (double)xv[i][j];
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) wsm[b][(wku + 2 * i) * 8 + j][wrow] = (double)wv[i][j];
    };
    // thread tile: tokens {16p + 2ty, 16p + 2ty + 1 : p < TM/2} x experts {2tx, 2tx+1, 32+2tx, 33+2tx}
    double acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0;
    int b = 0;
    if (c_lo < c_hi) {
        fetch(c_lo);
        stash(0);
    }
    __syncthreads();
    for (int c = c_lo; c < c_hi; c++) {
        const bool more = c + 1 < c_hi;
        if (more) fetch(c + 1);
#pragma unroll 4
        for (int k = 0; k < kRtBK; k++) {
            double xr[TM];
#pragma unroll
            for (int p = 0; p < TM / 2; p++) {
                const double2 v = *reinterpret_cast<const double2*>(&xs[b][k][16 * p + 2 * ty]);
                xr[2 * p] = v.x;
                xr[2 * p + 1] = v.y;
            }
            const double2 wa = *reinterpret_cast<const double2*>(&wsm[b][k][2 * tx]);
            const double2 wc = *reinterpret_cast<const double2*>(&wsm[b][k][32 + 2 * tx]);
            const double wq[4] = {wa.x, wa.y, wc.x, wc.y};
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fma(xr[i], wq[j], acc[i][j]);
        }
        if (more) stash(b ^ 1);
        __syncthreads();
        b ^= 1;
    }
    const int ecol[4] = {2 * tx, 2 * tx + 1, 32 + 2 * tx, 33 + 2 * tx};
    if (gridDim.z == 1) {
#pragma unroll
        for (int i = 0; i < TM; i++) {
            const int tr = 16 * (i >> 1) + 2 * ty + (i & 1);
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (t0 + tr < T && e0 + ecol[j] < E) logits[(size_t)(t0 + tr) * ld + e0 + ecol[j]] = (float)acc[i][j];
        }
    } else {
        // partial tiles meet in the cluster: every block parks its tile in its own shared memory, then sums a slice of
        // the rows over all blocks, in rank order
        double* red = reinterpret_cast<double*>(smem_raw);  // [BM][kRtBN], free after the last barrier of the loop
#pragma unroll
        for (int i = 0; i < TM; i++) {
            const int tr = 16 * (i >> 1) + 2 * ty + (i & 1);
#pragma unroll
            for (int j = 0; j < 4; j++) red[tr * kRtBN + ecol[j]] = acc[i][j];
        }
        cluster_sync_all();
        const int S = gridDim.z, z = blockIdx.z;
        const int rows = BM / S;  // S is a power of two, at most 8
        for (int i = tid; i < rows * kRtBN; i += 128) {
            const int r = z * rows + i / kRtBN, cidx = i % kRtBN;
            double sum = 0.0;
            for (int q = 0; q < S; q++) sum += ld_dsmem_f64(red + r * kRtBN + cidx, q);
            if (t0 + r < T && e0 + cidx < E) logits[(size_t)(t0 + r) * ld + e0 + cidx] = (float)sum;
        }
        cluster_sync_all();  // no block leaves while its shared memory may still be read
    }
    if (blockIdx.y == 0 && blockIdx.z == 0) {
        for (int i = tid; i < BM * (ld - E); i += 128) {
            const int tt = i / (ld - E), cidx = E + i % (ld - E);
            if (t0 + tt < T) logits[(size_t)(t0 + tt) * ld + cidx] = 0.f;
        }
    }
}

// Largest Euclidean norm of a router row (bf16 [E, D]), rounded up a little: one block per expert, the maximum taken
// over the bit patterns (positive floats order like their bits). Feeds the error bound of the approximate logits.
__global__ void __launch_bounds__(256) router_wnorm_max_kernel(const uint16_t* __restrict__ wr, int D, uint32_t* __restrict__ out) {
    __shared__ float wsum[8];
    const uint16_t* row = wr + (size_t)blockIdx.x * D;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += 256) {
        const float f = bf16_bits_to_f32(row[i]);
        s = fmaf(f, f, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < 8; i++) tot += wsum[i];
        atomicMax(out, __float_as_uint(sqrtf(tot) * 1.001f));
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Top-k routing of softmax-family routers. One warp per token. The rule (KernelCaseRouter.swift:57-80 of the
// reference): add the router bias to the logits, NaN counts as -inf, pick the maximum k times with ties going to the
// lower index (when everything left is -inf the lowest index not yet taken wins), weights exp(l_k - l_top1) / sum in
// k order, then x routed scale and x the per-expert scale of the chosen expert.
struct RouteParams {
    const float* logits;       // [T, ld]
    // Refinement (route_topk_kernel<VPL, true>): `logits` then holds approximate values, each within
    // err_coef * ||x_t||_2 of the exact one. The kernel recomputes, exactly (float64 sums of exact products, rounded once
    // to fp32), every logit that could still belong to the top k, writes them back and selects among those.
    float* logits_rw;          // the same array, writable
    const uint16_t* x;         // bf16 activations [T, ldx]
    int64_t ldx;
    const uint16_t* wr;        // bf16 router [E, D]
    int32_t D;
    float err_coef;
    const float* logit_bias;   // [E] or null
    const float* pes;          // per-expert scale [E] or null
    uint32_t* inds;            // [T, topk]
    float* wts;                // [T, topk]
    int32_t T, E, ld, topk;
    float scale;
    int32_t sigmoid;           // 0: softmax over the chosen logits; 1: sigmoid scores
    const float* select_bias;  // sigmoid: [E] added to the scores for the selection only, or null
    float eps;                 // sigmoid: added to the sum of the chosen scores
};

// One exact logit: sum_k x[k] * w[k] over bf16 inputs. Every product is exact in fp32 (two 8-bit significands); the sum
// runs in float64 in a fixed order (lane-strided chunks, then a butterfly over the lanes), so its fp32 rounding is the
// correctly rounded dot product whatever the order. All lanes get the result.
__device__ __forceinline__ float exact_dot_bf16(const uint16_t* __restrict__ xrow, const uint16_t* __restrict__ wrow, int D,
                                                int lane) {
    double a4[4] = {0.0, 0.0, 0.0, 0.0};  // four independent chains (the float64 adds would otherwise wait for each other)
    for (int u = lane; u < D / 8; u += 32) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xrow + u * 8);
        const uint4 wv = ldg_nc_u4(wrow + u * 8);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            a4[j] += (double)(__uint_as_float(xw[j] << 16) * __uint_as_float(ww[j] << 16));
            a4[j] += (double)(__uint_as_float(xw[j] & 0xFFFF0000u) * __uint_as_float(ww[j] & 0xFFFF0000u));
        }
    }
    double acc = (a4[0] + a4[1]) + (a4[2] + a4[3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    return (float)acc;
}

// WPT: warps per token. 1: a block takes four tokens. 4 (refinement only): a block takes one token and its warps share
// the exact dot products (candidate c goes to warp c % 4, results meet in shared memory); everything else runs in all
// four warps alike. With few tokens per GPU the refinement is one dependent chain per warp, so four warps per token
// cut it to a quarter; with thousands of tokens the GPU is full either way.
template <int VPL, bool REFINE = false, int WPT = 1>
__global__ void __launch_bounds__(128) route_topk_kernel(const RouteParams p) {
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int t = WPT == 1 ? blockIdx.x * 4 + wib : blockIdx.x;
    if (t >= p.T) return;  // WPT = 4: the whole block leaves
    __shared__ float sx[WPT > 1 ? VPL * 32 : 1];  // WPT = 4: exact logits of the candidates
    const float* lr = p.logits + (size_t)t * p.ld;
    float v[VPL];   // what the selection compares
    float pv[VPL];  // sigmoid: the unbiased score the weight is made of
    uint32_t taken = 0;
#pragma unroll
    for (int j = 0; j < VPL; j++) {
        const int e = j * 32 + lane;
        float f = e < p.E ? lr[e] : -INFINITY;
        if (e < p.E && p.logit_bias != nullptr) f += p.logit_bias[e];
        pv[j] = 0.f;
        if (p.sigmoid) {
            // the fp32 score is the correctly rounded sigmoid (evaluated in float64), so that the selection does not
            // depend on an exp implementation
            f = (float)(1.0 / (1.0 + exp(-(double)f)));
            pv[j] = f;
            if (e < p.E && p.select_bias != nullptr) f += p.select_bias[e];
        }
        if (f != f) f = -INFINITY;
        v[j] = f;
        if (e >= p.E) taken |= 1u << j;
    }
    if (REFINE) {
        // ---- which experts can still be among the k largest? Those within 2 eps of the k-th largest approximate value:
        // with |approx - exact| <= eps everywhere, at least k experts have an exact value >= kth - eps, so a true member of
        // the top k has exact >= kth - eps and approx >= kth - 2 eps. The exact values of these candidates decide.
        uint32_t tk = taken;
        float kth = -INFINITY;
        for (int k = 0; k < p.topk; k++) {
            float bv = -INFINITY;
            int bj = -1;
#pragma unroll
            for (int j = 0; j < VPL; j++)
                if (!((tk >> j) & 1u) && (bj < 0 || v[j] > bv)) { bv = v[j]; bj = j; }
            float gv = bj >= 0 ? bv : -INFINITY;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) gv = fmaxf(gv, __shfl_xor_sync(0xffffffffu, gv, o));
            // one holder of the maximum drops out (the lowest lane; which one is irrelevant for the k-th value)
            const uint32_t holders = __ballot_sync(0xffffffffu, bj >= 0 && bv == gv);
            if (holders == 0u) { gv = -INFINITY; }
            else if (lane == __ffs(holders) - 1) tk |= 1u << bj;
            kth = gv;
        }
        const uint16_t* xrow = p.x + (size_t)t * p.ldx;
        float ss = 0.f;
        for (int u = lane; u < p.D / 8; u += 32) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xrow + u * 8);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float a = __uint_as_float(xw[j] << 16), b = __uint_as_float(xw[j] & 0xFFFF0000u);
                ss = fmaf(a, a, ss);
                ss = fmaf(b, b, ss);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float eps = p.err_coef * sqrtf(ss) * 1.001f;
        // anything not finite (an infinity or NaN among the inputs): every expert is recomputed
        float thr = kth - 2.f * eps;
        if (!(fabsf(kth) <= 3.0e38f) || !(eps <= 3.0e38f)) thr = -INFINITY;
        int cidx = 0;  // candidates so far, the same count in every warp of the token
#pragma unroll
        for (int j = 0; j < VPL; j++) {
            const bool mine = !((taken >> j) & 1u) && v[j] >= thr;
            uint32_t bal = __ballot_sync(0xffffffffu, mine);
            while (bal != 0u) {
                const int src = __ffs(bal) - 1;
                bal &= bal - 1u;
                const int e = j * 32 + src;
                if (WPT == 1 || (cidx & (WPT - 1)) == wib) {
                    const float exact = exact_dot_bf16(xrow, p.wr + (size_t)e * p.D, p.D, lane);
                    if (lane == src) {
                        p.logits_rw[(size_t)t * p.ld + e] = exact;
                        if (WPT > 1) {
                            sx[e] = exact;
                        } else {
                            float f = exact;
                            if (p.logit_bias != nullptr) f += p.logit_bias[e];
                            if (f != f) f = -INFINITY;
                            v[j] = f;
                        }
                    }
                }
                cidx++;
            }
            if (!mine) taken |= 1u << j;  // out of the running
        }
        if (WPT > 1) {
            __syncthreads();
#pragma unroll
            for (int j = 0; j < VPL; j++) {
                if ((taken >> j) & 1u) continue;
                float f = sx[j * 32 + lane];
                if (p.logit_bias != nullptr) f += p.logit_bias[j * 32 + lane];
                if (f != f) f = -INFINITY;
                v[j] = f;
            }
        }
    }
    float myv = -INFINITY, myp = 0.f;
    uint32_t myi = 0;
    for (int k = 0; k < p.topk; k++) {
        float bv = -INFINITY;
        uint32_t bi = 0xFFFFFFFFu;
#pragma unroll
        for (int j = 0; j < VPL; j++) {
            if (!((taken >> j) & 1u) && (bi == 0xFFFFFFFFu || v[j] > bv)) {
                bv = v[j];
                bi = j * 32 + lane;
            }
        }
        // warp maximum over the lanes that still have a candidate, then the lowest index among the equal ones
        float gv = bv;
        uint32_t any = bi != 0xFFFFFFFFu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, gv, o);
            const uint32_t oa = __shfl_xor_sync(0xffffffffu, any, o);
            if (oa && (!any || ov > gv)) gv = ov;
            any |= oa;
        }
        uint32_t gi = (bi != 0xFFFFFFFFu && bv == gv) ? bi : 0xFFFFFFFFu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) gi = min(gi, __shfl_xor_sync(0xffffffffu, gi, o));
        float gp = 0.f;  // the chosen expert's unbiased score, from the lane that holds it
#pragma unroll
        for (int j = 0; j < VPL; j++)
            if ((uint32_t)(j * 32 + lane) == gi) {
                taken |= 1u << j;
                gp = pv[j];
            }
        gp = __shfl_sync(0xffffffffu, gp, gi & 31u);
        if (lane == k) { myv = gv; myi = gi; myp = gp; }
    }
    if (p.sigmoid) {
        float sum = 0.f;
        for (int k = 0; k < p.topk; k++) sum += __shfl_sync(0xffffffffu, myp, k);
        sum += p.eps;
        if (lane < p.topk && (WPT == 1 || wib == 0)) {
            float w = myp / sum * p.scale;
            if (p.pes != nullptr) w *= p.pes[myi];
            p.inds[(size_t)t * p.topk + lane] = myi;
            p.wts[(size_t)t * p.topk + lane] = w;
        }
        return;
    }
    const float top1 = __shfl_sync(0xffffffffu, myv, 0);
    const float ex = lane < p.topk ? expf(myv - top1) : 0.f;
    float sum = 0.f;
    for (int k = 0; k < p.topk; k++) sum += __shfl_sync(0xffffffffu, ex, k);
    if (lane < p.topk && (WPT == 1 || wib == 0)) {
        float w = ex / sum * p.scale;
        if (p.pes != nullptr) w *= p.pes[myi];
        p.inds[(size_t)t * p.topk + lane] = myi;
        p.wts[(size_t)t * p.topk + lane] = w;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Token->expert permutation, deterministic: inside an expert the pairs keep ascending pair id.
// count: one block per expert counts its pairs. scatter: one block per expert places them, writes the tile
// descriptors for two tile heights and, in the last block, the totals.
struct GroupParams {
    const uint32_t* inds;   // [P] expert of each pair
    uint32_t* counts;       // [E]
    uint32_t* offsets;      // [E + 1]
    uint32_t* row_map;      // [P] sorted position -> pair
    uint32_t* pos;          // [P] pair -> sorted position
    Tile* tiles_a;          // tile height bm_a
    Tile* tiles_b;          // tile height bm_b
    uint32_t* ntiles;       // [2]
    int32_t P, E, bm_a, bm_b;
    int32_t e_lo, e_hi;     // experts owned here (expert parallel); tiles are emitted only for these
    uint32_t* chunk_hist;   // [chunks, E] scratch of the chunked form (many pairs)
    int32_t chunks;
};

__global__ void __launch_bounds__(256) moe_count_kernel(const GroupParams p) {
    __shared__ uint32_t wsum[8];
    const uint32_t e = blockIdx.x;
    uint32_t c = 0;
    for (int i = threadIdx.x; i < p.P; i += 256) c += p.inds[i] == e;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t s = 0;
        for (int i = 0; i < 8; i++) s += wsum[i];
        p.counts[e] = s;
    }
}

__global__ void __launch_bounds__(256) moe_scatter_kernel(const GroupParams p) {
    __shared__ uint32_t sh[3][8];
    __shared__ uint32_t base[4];
    const uint32_t e = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // exclusive prefixes over the experts before this one: pairs, tiles of height a, tiles of height b
    uint32_t c0 = 0, ta = 0, tb = 0;
    for (int i = tid; i < (int)e; i += 256) {
        const uint32_t c = p.counts[i];
        c0 += c;
        if (i >= p.e_lo && i < p.e_hi) {
            ta += (c + p.bm_a - 1) / p.bm_a;
            tb += (c + p.bm_b - 1) / p.bm_b;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        c0 += __shfl_xor_sync(0xffffffffu, c0, o);
        ta += __shfl_xor_sync(0xffffffffu, ta, o);
        tb += __shfl_xor_sync(0xffffffffu, tb, o);
    }
    if (lane == 0) { sh[0][warp] = c0; sh[1][warp] = ta; sh[2][warp] = tb; }
    __syncthreads();
    if (tid == 0) {
        uint32_t a = 0, b = 0, c = 0;
        for (int i = 0; i < 8; i++) { a += sh[0][i]; b += sh[1][i]; c += sh[2][i]; }
        base[0] = a; base[1] = b; base[2] = c;
    }
    __syncthreads();
    const uint32_t off = base[0], tile_a0 = base[1], tile_b0 = base[2];
    const uint32_t cnt = p.counts[e];
    if (tid == 0) {
        p.offsets[e] = off;
        if ((int)e == p.E - 1) {
            p.offsets[p.E] = off + cnt;
            const bool own = (int)e >= p.e_lo && (int)e < p.e_hi;
            p.ntiles[0] = tile_a0 + (own ? (cnt + p.bm_a - 1) / p.bm_a : 0);
            p.ntiles[1] = tile_b0 + (own ? (cnt + p.bm_b - 1) / p.bm_b : 0);
        }
    }
    if ((int)e >= p.e_lo && (int)e < p.e_hi) {
        for (uint32_t j = tid; j * p.bm_a < cnt; j += 256)
            p.tiles_a[tile_a0 + j] = Tile{e, off + j * p.bm_a, min((uint32_t)p.bm_a, cnt - j * p.bm_a), 0};
        for (uint32_t j = tid; j * p.bm_b < cnt; j += 256)
            p.tiles_b[tile_b0 + j] = Tile{e, off + j * p.bm_b, min((uint32_t)p.bm_b, cnt - j * p.bm_b), 0};
    }
    // ordered placement: walk the pairs 256 at a time, rank the matches with a block-wide prefix
    uint32_t placed = 0;
    for (int i0 = 0; i0 < p.P; i0 += 256) {
        const int i = i0 + tid;
        const bool hit = i < p.P && p.inds[i] == e;
        const uint32_t bal = __ballot_sync(0xffffffffu, hit);
        __syncthreads();  // sh[0] reuse
        if (lane == 0) sh[0][warp] = __popc(bal);
        __syncthreads();
        uint32_t before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const uint32_t c = sh[0][w];
            if (w < warp) before += c;
            total += c;
        }
        if (hit) {
            const uint32_t r = off + placed + before + __popc(bal & ((1u << lane) - 1u));
            p.row_map[r] = (uint32_t)i;
            p.pos[i] = r;
        }
        placed += total;
    }
}

// The same grouping for many pairs, as a stable counting sort over chunks of kGroupChunk pairs: every kernel touches
// each pair once instead of once per expert. (1) per-chunk histograms; (2) one block turns them into per-chunk bases,
// expert offsets and the tile lists; (3) every chunk places its pairs: position = expert offset + pairs of that expert
// in earlier chunks + in earlier warps of the chunk + earlier in the warp's walk. Nothing depends on timing.
constexpr int kGroupChunk = 1024;

__global__ void __launch_bounds__(256) moe_hist_kernel(const GroupParams p) {
    extern __shared__ uint32_t hist[];
    for (int e = threadIdx.x; e < p.E; e += 256) hist[e] = 0;
    __syncthreads();
    const int i0 = blockIdx.x * kGroupChunk, i1 = min(p.P, i0 + kGroupChunk);
    for (int i = i0 + threadIdx.x; i < i1; i += 256) atomicAdd(&hist[p.inds[i]], 1u);
    __syncthreads();
    for (int e = threadIdx.x; e < p.E; e += 256) p.chunk_hist[(size_t)blockIdx.x * p.E + e] = hist[e];
}

__global__ void __launch_bounds__(256) moe_scan_kernel(const GroupParams p) {
    __shared__ uint32_t sc[256], sa[256], sb[256];
    const int tid = threadIdx.x;
    // experts handled by this thread: a contiguous run, so that a block-wide scan over threads orders the experts
    const int per = (p.E + 255) / 256;
    const int e0 = tid * per, e1 = min(p.E, e0 + per);
    uint32_t c_sum = 0, a_sum = 0, b_sum = 0;
    for (int e = e0; e < e1; e++) {
        uint32_t run = 0;
        for (int c0 = 0; c0 < p.chunks; c0 += 8) {  // histogram -> exclusive prefix over the chunks, eight loads in flight
            uint32_t t[8];
#pragma unroll
            for (int k = 0; k < 8; k++) t[k] = c0 + k < p.chunks ? p.chunk_hist[(size_t)(c0 + k) * p.E + e] : 0u;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                if (c0 + k < p.chunks) p.chunk_hist[(size_t)(c0 + k) * p.E + e] = run;
                run += t[k];
            }
        }
        p.counts[e] = run;
        c_sum += run;
        if (e >= p.e_lo && e < p.e_hi) {
            a_sum += (run + p.bm_a - 1) / p.bm_a;
            b_sum += (run + p.bm_b - 1) / p.bm_b;
        }
    }
    sc[tid] = c_sum; sa[tid] = a_sum; sb[tid] = b_sum;
    __syncthreads();
    uint32_t off = 0, ta = 0, tb = 0;
    for (int i = 0; i < tid; i++) { off += sc[i]; ta += sa[i]; tb += sb[i]; }
    for (int e = e0; e < e1; e++) {
        const uint32_t cnt = p.counts[e];
        p.offsets[e] = off;
        if (e >= p.e_lo && e < p.e_hi) {
            for (uint32_t j = 0; j * p.bm_a < cnt; j++)
                p.tiles_a[ta++] = Tile{(uint32_t)e, off + j * p.bm_a, min((uint32_t)p.bm_a, cnt - j * p.bm_a), 0};
            for (uint32_t j = 0; j * p.bm_b < cnt; j++)
                p.tiles_b[tb++] = Tile{(uint32_t)e, off + j * p.bm_b, min((uint32_t)p.bm_b, cnt - j * p.bm_b), 0};
        }
        off += cnt;
    }
    if (tid == 255) {
        p.offsets[p.E] = off;
        p.ntiles[0] = ta;
        p.ntiles[1] = tb;
    }
}

__global__ void __launch_bounds__(256) moe_place_kernel(const GroupParams p) {
    extern __shared__ uint32_t sm[];  // [8 warps][E] pairs of each expert in each warp's share, then running counts
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < 8 * p.E; i += 256) sm[i] = 0;
    __syncthreads();
    // warp w walks pairs [i0 + 128 w, i0 + 128 w + 128) of the chunk, 32 at a time
    const int i0 = blockIdx.x * kGroupChunk + warp * (kGroupChunk / 8);
    uint32_t* mine = sm + warp * p.E;
    uint32_t ev[4];
#pragma unroll
    for (int st = 0; st < 4; st++) {
        const int i = i0 + st * 32 + lane;
        ev[st] = i < p.P ? p.inds[i] : 0xFFFFFFFFu;
        const uint32_t same = __match_any_sync(0xffffffffu, ev[st]);
        if (ev[st] != 0xFFFFFFFFu && lane == __ffs(same) - 1) mine[ev[st]] += __popc(same);
        __syncwarp();
    }
    __syncthreads();
    // per expert: exclusive prefix over the warps, on top of the expert's offset and its pairs in earlier chunks
    for (int e = tid; e < p.E; e += 256) {
        uint32_t run = p.offsets[e] + p.chunk_hist[(size_t)blockIdx.x * p.E + e];
        for (int w = 0; w < 8; w++) {
            const uint32_t t = sm[w * p.E + e];
            sm[w * p.E + e] = run;
            run += t;
        }
    }
    __syncthreads();
#pragma unroll
    for (int st = 0; st < 4; st++) {
        const int i = i0 + st * 32 + lane;
        const uint32_t same = __match_any_sync(0xffffffffu, ev[st]);
        if (ev[st] != 0xFFFFFFFFu) {
            const uint32_t r = mine[ev[st]] + __popc(same & ((1u << lane) - 1u));
            p.row_map[r] = (uint32_t)i;
            p.pos[i] = r;
        }
        __syncwarp();
        if (ev[st] != 0xFFFFFFFFu && lane == __ffs(same) - 1) mine[ev[st]] += __popc(same);
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Combine: out[t, :] (+)= sum_k wts[t, k] * Yd[pos[t*topk + k], :] in router rank order k = 0..topk-1, fp32
// (Shaders/qmm_nax_moe.metal:371-396 of the reference). One block per token.
struct CombineParams {
    const void* yd;         // [P, D] expert outputs at sorted positions, fp32 or fp16
    int32_t yd_dtype;
    const uint32_t* pos;    // [P]
    const float* wts;       // [T, topk]
    void* out;              // [T, ldo]
    int32_t out_dtype;
    int64_t ldo;
    int32_t T, D, topk, accumulate;
};

__global__ void __launch_bounds__(256) moe_combine_kernel(const CombineParams p) {
    const int t = blockIdx.x;
    __shared__ uint32_t spos[32];
    __shared__ float sw[32];
    if (threadIdx.x < p.topk) {
        spos[threadIdx.x] = p.pos[(size_t)t * p.topk + threadIdx.x];
        sw[threadIdx.x] = p.wts[(size_t)t * p.topk + threadIdx.x];
    }
    __syncthreads();
    for (int d = threadIdx.x * 4; d < p.D; d += 1024) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < p.topk; k++) {
            float4 y;
            if (p.yd_dtype == kF32) {
                y = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.yd) + (size_t)spos[k] * p.D + d);
            } else {
                const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(p.yd) + (size_t)spos[k] * p.D + d);
                const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
                const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
                y = make_float4(lo.x, lo.y, hi.x, hi.y);
            }
            const float w = sw[k];
            a.x = fmaf(w, y.x, a.x); a.y = fmaf(w, y.y, a.y); a.z = fmaf(w, y.z, a.z); a.w = fmaf(w, y.w, a.w);
        }
        const size_t o = (size_t)t * p.ldo + d;
        if (p.out_dtype == kF32) {
            float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o);
            if (p.accumulate) {
                const float4 c = *op;
                a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
            }
            *op = a;
        } else if (p.out_dtype == kBF16) {
            uint16_t* op = reinterpret_cast<uint16_t*>(p.out) + o;
            float r[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; j++)
                op[j] = (uint16_t)f32_to_bf16_bits(p.accumulate ? bf16_bits_to_f32(op[j]) + r[j] : r[j]);
        } else {
            __half* op = reinterpret_cast<__half*>(p.out) + o;
            float r[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; j++) op[j] = __float2half_rn(p.accumulate ? __half2float(op[j]) + r[j] : r[j]);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Expert-parallel helpers.
//
// pack: rows[pos[pair], :] = fp16(x[pair / topk, :]) — the activations in expert-sorted order, i.e. one contiguous
// segment per destination rank when experts are sharded in contiguous ranges.
__global__ void __launch_bounds__(256) moe_pack_rows_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx,
                                                           const uint32_t* __restrict__ pos, __half* __restrict__ rows,
                                                           int P, int D, int topk) {
    const int pair = blockIdx.x;
    if (pair >= P) return;
    const size_t src = (size_t)(pair / topk) * ldx;
    __half* dst = rows + (size_t)pos[pair] * D;
    for (int u = threadIdx.x; u < D / 8; u += 256) {
        float v[8];
        load_x8(x, x_dtype, src + u * 8, v);
        uint4 o;
        o.x = pack_half2(v[0], v[1]); o.y = pack_half2(v[2], v[3]); o.z = pack_half2(v[4], v[5]); o.w = pack_half2(v[6], v[7]);
        *reinterpret_cast<uint4*>(dst + u * 8) = o;
    }
}

// Tile list of the rows a rank received, by source then by local expert; counts[s * E + e] rows from source s for
// expert e. region_rows == 0: the sources' rows follow each other (packed); region_rows > 0: the rows of source s start
// at s * region_rows (every source owns a fixed region of the receive buffer). One block; at most 4096 entries.
constexpr int kMaxEpSources = 16;  // source ranks of one tile list (the per-source totals live in shared memory)

__global__ void __launch_bounds__(512) ep_tiles_kernel(const uint32_t* __restrict__ counts, int sources, int E, int e_lo,
                                                       int e_cnt, int bm, uint32_t region_rows, Tile* __restrict__ tiles,
                                                       uint32_t* __restrict__ ntiles) {
    __shared__ uint32_t rstart[4096];
    __shared__ uint32_t stot[kMaxEpSources];
    __shared__ uint32_t stiles[512];
    const int n = sources * e_cnt;
    if ((int)threadIdx.x < sources) {
        uint32_t t = 0;
        for (int j = 0; j < e_cnt; j++) t += counts[threadIdx.x * E + e_lo + j];
        stot[threadIdx.x] = t;
    }
    __syncthreads();
    if ((int)threadIdx.x < sources) {
        const int s = threadIdx.x;
        uint32_t r = 0;
        if (region_rows > 0) r = s * region_rows;
        else for (int s2 = 0; s2 < s; s2++) r += stot[s2];
        for (int j = 0; j < e_cnt; j++) {
            rstart[s * e_cnt + j] = r;
            r += counts[s * E + e_lo + j];
        }
    }
    __syncthreads();
    const int per = (n + 511) / 512;
    const int b = threadIdx.x * per, e_end = min(n, b + per);
    uint32_t tl = 0;
    for (int i = b; i < e_end; i++) {
        const uint32_t c = counts[(i / e_cnt) * E + e_lo + i % e_cnt];
        tl += (c + bm - 1) / bm;
    }
    stiles[threadIdx.x] = tl;
    __syncthreads();
    uint32_t t0 = 0;
    for (int i = 0; i < (int)threadIdx.x; i++) t0 += stiles[i];
    for (int i = b; i < e_end; i++) {
        const uint32_t e = e_lo + i % e_cnt;
        const uint32_t c = counts[(i / e_cnt) * E + e];
        const uint32_t r0 = rstart[i];
        for (uint32_t j = 0; j * bm < c; j++) tiles[t0++] = Tile{e, r0 + j * bm, min((uint32_t)bm, c - j * bm), 0};
    }
    if (threadIdx.x == 511) ntiles[0] = t0;
}

// Row r of src (row_bytes each, a multiple of 16) copied to the address row_ptr[r]; rows whose address is 0 stay.
// Four rows per block, 64 threads per row.
__global__ void __launch_bounds__(256) moe_scatter_rows_kernel(const void* __restrict__ src, const uint64_t* __restrict__ row_ptr,
                                                              int rows, int row_bytes) {
    // most slots are empty when the table is sized for the worst case: a fixed grid walks them
    for (int r = blockIdx.x * 4 + (threadIdx.x >> 6); r < rows; r += gridDim.x * 4) {
        const uint64_t dptr = row_ptr[r];
        if (dptr == 0) continue;
        const uint4* s = reinterpret_cast<const uint4*>(static_cast<const char*>(src) + (size_t)r * row_bytes);
        uint4* d = reinterpret_cast<uint4*>(dptr);
        for (int u = threadIdx.x & 63; u < row_bytes / 16; u += 64) d[u] = ldg_nc_u4(s + u);
    }
}

// Shared expert: the per-token weight sigmoid(x . w) with w an 8-bit affine g64 row (verify.metal:262-277), or 1 without
// a gate tensor. One warp per token, fixed lane order.
__global__ void __launch_bounds__(128) shared_gate_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx,
                                                         const uint32_t* __restrict__ gw, const uint16_t* __restrict__ gs,
                                                         const uint16_t* __restrict__ gb, float* __restrict__ sg, int T,
                                                         int D) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= T) return;
    float w = 1.f;
    if (gw != nullptr) {
        float acc = 0.f;
        for (int u = lane; u < D / 8; u += 32) {
            float v[8];
            load_x8(x, x_dtype, (size_t)t * ldx + u * 8, v);
            const uint2 q = *reinterpret_cast<const uint2*>(gw + u * 2);
            const float sc = bf16_bits_to_f32(gs[u / 8]), bi = bf16_bits_to_f32(gb[u / 8]);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                acc = fmaf(v[j], fmaf(sc, (float)((q.x >> (8 * j)) & 0xFFu), bi), acc);
                acc = fmaf(v[4 + j], fmaf(sc, (float)((q.y >> (8 * j)) & 0xFFu), bi), acc);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        w = 1.0f / (1.0f + expf(-acc));
    }
    if (lane == 0) sg[t] = w;
}

// fp16 copy of x [T, D] (rows in place), the tensor-core GEMM's operand type
__global__ void __launch_bounds__(256) rows_to_f16_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx,
                                                         __half* __restrict__ out, int T, int D) {
    const size_t i = ((size_t)blockIdx.x * 256 + threadIdx.x) * 8;
    if (i >= (size_t)T * D) return;
    const size_t r = i / D, c = i % D;
    float v[8];
    load_x8(x, x_dtype, r * ldx + c, v);
    uint4 o;
    o.x = pack_half2(v[0], v[1]); o.y = pack_half2(v[2], v[3]); o.z = pack_half2(v[4], v[5]); o.w = pack_half2(v[6], v[7]);
    *reinterpret_cast<uint4*>(out + i) = o;
}

// Tile list of the shared expert: all T rows in place, tiles of bm rows, expert id `expert`.
__global__ void shared_tiles_kernel(int T, int bm, uint32_t expert, Tile* __restrict__ tiles, uint32_t* __restrict__ ntiles) {
    const int n = (T + bm - 1) / bm;
    for (int j = threadIdx.x; j < n; j += blockDim.x)
        tiles[j] = Tile{expert, (uint32_t)(j * bm), (uint32_t)min(bm, T - j * bm), 0};
    if (threadIdx.x == 0) ntiles[0] = (uint32_t)n;
}

// out[t, :] += sg[t] * ys[t, :] (the shared expert's contribution)
__global__ void __launch_bounds__(256) shared_add_kernel(const void* __restrict__ ys, int32_t ys_dtype, const float* __restrict__ sg,
                                                        void* __restrict__ out, int32_t out_dtype, int64_t ldo, int T, int D) {
    const int t = blockIdx.x;
    const float w = sg[t];
    for (int d = threadIdx.x; d < D; d += 256) {
        const float y = ys_dtype == kF32 ? reinterpret_cast<const float*>(ys)[(size_t)t * D + d]
                                         : __half2float(reinterpret_cast<const __half*>(ys)[(size_t)t * D + d]);
        const size_t o = (size_t)t * ldo + d;
        if (out_dtype == kF32) reinterpret_cast<float*>(out)[o] += w * y;
        else if (out_dtype == kF16) reinterpret_cast<__half*>(out)[o] = __float2half_rn(__half2float(reinterpret_cast<__half*>(out)[o]) + w * y);
        else reinterpret_cast<uint16_t*>(out)[o] = (uint16_t)f32_to_bf16_bits(bf16_bits_to_f32(reinterpret_cast<uint16_t*>(out)[o]) + w * y);
    }
}

// Unit-weight RMSNorm of fp32 rows (the layer-stack skeleton's input normalisation; Shaders/verify.metal:503-523 of
// the reference): out = x / sqrt(mean(x^2) + eps), written as bf16 / fp16 / fp32. One block per row.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* __restrict__ x, int64_t ldx, void* __restrict__ out,
                                                     int32_t out_dtype, int64_t ldo, int d, float eps) {
    __shared__ float wsum[8];
    const float* xr = x + (size_t)blockIdx.x * ldx;
    float s = 0.f;
    for (int i = threadIdx.x * 4; i < d; i += 1024) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += wsum[i];
    const float r = rsqrtf(tot / (float)d + eps);
    for (int i = threadIdx.x * 4; i < d; i += 1024) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        const float o4[4] = {v.x * r, v.y * r, v.z * r, v.w * r};
        const size_t o = (size_t)blockIdx.x * ldo + i;
        if (out_dtype == kF32) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o) = make_float4(o4[0], o4[1], o4[2], o4[3]);
        } else if (out_dtype == kBF16) {
            uint2 w;
            w.x = f32_to_bf16_bits(o4[0]) | (f32_to_bf16_bits(o4[1]) << 16);
            w.y = f32_to_bf16_bits(o4[2]) | (f32_to_bf16_bits(o4[3]) << 16);
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(out) + o) = w;
        } else {
            uint2 w;
            w.x = pack_half2(o4[0], o4[1]);
            w.y = pack_half2(o4[2], o4[3]);
            *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + o) = w;
        }
    }
}

}  // namespace iq
