// Launchers of the GEMV family and the iq_qmv entry point.
#include <stdarg.h>
#include <stdio.h>

#include "gqmv.cuh"
#include "internal.h"

namespace iq {

namespace {

typedef void (*GqmvKernel)(const GqmvParams);

// (RG, WK) pairs: RG row groups of 16 rows and WK K-slices per CTA, always 8 warps.
template <int FMT, int MH, int MODE, int RG, int WK>
constexpr GqmvKernel kernel_of() {
    return gqmv_kernel<FMT, MH, (MODE == kModeGateUp ? 2 : 1), MODE, RG, WK>;
}

template <int FMT, int MH, int MODE>
GqmvKernel pick_cfg(int wk) {
    switch (wk) {
        case 8: return kernel_of<FMT, MH, MODE, 1, 8>();
        case 4: return kernel_of<FMT, MH, MODE, 2, 4>();
        default: return kernel_of<FMT, MH, MODE, 4, 2>();
    }
}

template <int FMT, int MH>
GqmvKernel pick_mode(int mode, int wk) {
    switch (mode) {
        case kModeGateUp: return pick_cfg<FMT, MH, kModeGateUp>(wk);
        case kModeDown: return pick_cfg<FMT, MH, kModeDown>(wk);
        default: return pick_cfg<FMT, MH, kModePlain>(wk);
    }
}

template <int FMT>
GqmvKernel pick_mh(int mh, int mode, int wk) {
    return mh == 2 ? pick_mode<FMT, 2>(mode, wk) : pick_mode<FMT, 1>(mode, wk);
}

GqmvKernel pick(int32_t fmt, int mh, int mode, int wk) {
    switch (fmt) {
        case kFmtAffine4: return pick_mh<kFmtAffine4>(mh, mode, wk);
        case kFmtAffine8: return pick_mh<kFmtAffine8>(mh, mode, wk);
        case kFmtMxfp4: return pick_mh<kFmtMxfp4>(mh, mode, wk);
        default: return nullptr;
    }
}

constexpr int kSmemBudget = 200 * 1024;

}  // namespace

int32_t gqmv_init(iq_ctx* ctx) {
    for (int fmt = 0; fmt < 3; fmt++)
        for (int mh = 1; mh <= 2; mh++)
            for (int mode = 0; mode < 3; mode++)
                for (int wk = 2; wk <= 8; wk *= 2) {
                    GqmvKernel k = pick(fmt, mh, mode, wk);
                    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k),
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 20480);
                    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(gqmv)");
                }
    return kOk;
}

int32_t launch_gqmv(iq_ctx* ctx, cudaStream_t st, const GqmvCall& c) {
    const int ck = c.fmt == kFmtAffine8 ? 16 : 32;  // inputs per 16-byte chunk
    const int mh = c.max_rows > 8 ? 2 : 1;
    const int nw = c.mode == kModeGateUp ? 2 : 1;
    const bool has_bias = c.fmt != kFmtMxfp4;
    // K tile: everything at once when the staged activations fit, else the largest multiple of 1024 that does
    int kt = c.K;
    auto smem_for = [&](int ktile, int* xs_bytes, int* xsum_bytes, int* gp) {
        const int nsteps = (ktile / ck + 3) / 4;
        const int qu = ck == 32 ? 4 : 2;
        *xs_bytes = nsteps * qu * c.max_rows * 4 * 16;
        *gp = round_up(ktile / 64, 16);
        *xsum_bytes = has_bias ? 2 * c.max_rows * (*gp) * 2 : 0;
        const int red_bytes = 8 * nw * mh * 4 * 32 * 4;
        return *xs_bytes + *xsum_bytes + red_bytes;
    };
    int xs_bytes, xsum_bytes, gp;
    while (smem_for(kt, &xs_bytes, &xsum_bytes, &gp) > kSmemBudget) {
        kt = kt > 1024 ? (kt - 1) / 1024 * 1024 : 0;
        if (kt == 0) return fail(ctx, kErrInvalidArg, "qmv: activations do not fit shared memory");
    }
    const int smem = smem_for(kt, &xs_bytes, &xsum_bytes, &gp);

    // K slices per CTA: the fewest that still fill the GPU, keeping at least two steps per warp
    const int nsteps = (kt / ck + 3) / 4;
    const int64_t row_groups = (int64_t)(c.N / 16) * c.grid_tiles;
    const int64_t target = (int64_t)ctx->sms * 24;
    int wk = 2;
    while (wk < 8 && row_groups * wk < target && nsteps / (wk * 2) >= 2) wk *= 2;
    const int rg = 8 / wk;

    GqmvKernel k = pick(c.fmt, mh, c.mode, wk);
    if (k == nullptr) return fail(ctx, kErrNoKernel, "qmv: no kernel for format %d", c.fmt);

    GqmvParams p;
    for (int i = 0; i < 2; i++) {
        p.w[i] = c.w[i] ? c.w[i] : c.w[0];
        p.s[i] = c.s[i] ? c.s[i] : c.s[0];
        p.b[i] = c.b[i] ? c.b[i] : c.b[0];
        p.ebias[i] = c.ebias[i];
    }
    p.w_estride = c.w_estride; p.s_estride = c.s_estride;
    p.N = c.N; p.K = c.K;
    p.x = c.x; p.x_dtype = c.x_dtype; p.ldx = c.ldx;
    p.row_map = c.row_map; p.topk = c.topk;
    p.tiles = c.tiles; p.ntiles = c.ntiles; p.M = c.rows;
    p.y = c.y; p.y_dtype = c.y_dtype; p.ldy = c.ldy; p.accumulate = c.accumulate;
    p.limit = c.limit;
    p.kt = kt; p.xs_bytes = xs_bytes; p.xsum_bytes = xsum_bytes; p.gp = gp;

    dim3 grid((c.N / 16 + rg - 1) / rg, c.grid_tiles, 1);
    k<<<grid, 256, smem, st>>>(p);
    return check_cuda(ctx, cudaGetLastError(), "gqmv launch");
}

int32_t format_of(const iq_qlinear* m) {
    if (m->mode == IQ_MODE_MXFP4) return (m->bits == 4 && m->group == 32) ? kFmtMxfp4 : -1;
    if (m->mode != IQ_MODE_AFFINE || m->group != 64) return -1;
    if (m->bits == 4) return kFmtAffine4;
    if (m->bits == 8) return kFmtAffine8;
    return -1;
}

}  // namespace iq

using namespace iq;

extern "C" int32_t iq_qmv(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* m,
                          void* y, int32_t y_dtype, int64_t ldy, int32_t rows, uint32_t flags, int32_t n_prefix) {
    if (ctx == nullptr) return kErrInvalidArg;
    if (x == nullptr || y == nullptr || m == nullptr || m->w == nullptr || m->scales == nullptr)
        return fail(ctx, kErrInvalidArg, "qmv: null pointer");
    const int32_t fmt = format_of(m);
    if (fmt < 0)
        return fail(ctx, kErrUnsupported, "qmv: %d-bit group %d mode %d has no kernel (affine 4/8-bit g64, mxfp4 g32)",
                    m->bits, m->group, m->mode);
    if (fmt != kFmtMxfp4 && m->biases == nullptr) return fail(ctx, kErrInvalidArg, "qmv: affine layer without biases");
    if (rows < 1 || rows > 16) return fail(ctx, kErrInvalidArg, "qmv: rows = %d (1..16)", rows);
    if (m->n % 16 != 0 || m->k % 64 != 0 || m->n <= 0 || m->k <= 0)
        return fail(ctx, kErrInvalidArg, "qmv: n = %d must be a multiple of 16 and k = %d of 64", m->n, m->k);
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return fail(ctx, kErrInvalidArg, "qmv: dtype");
    if (ldx < m->k || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
        return fail(ctx, kErrInvalidArg, "qmv: x must be 16-byte aligned with ldx >= k and ldx %% 8 == 0");
    int32_t n = m->n;
    if (n_prefix > 0) {
        if (n_prefix % 16 != 0 || n_prefix > m->n) return fail(ctx, kErrInvalidArg, "qmv: n_prefix = %d", n_prefix);
        n = n_prefix;
    }
    if (ldy < n) return fail(ctx, kErrInvalidArg, "qmv: ldy = %lld < n", (long long)ldy);
    GqmvCall c;
    c.mode = kModePlain;
    c.fmt = fmt;
    c.w[0] = reinterpret_cast<const uint32_t*>(m->w);
    c.s[0] = m->scales;
    c.b[0] = m->biases;
    c.N = n;
    c.K = m->k;
    c.x = x; c.x_dtype = x_dtype; c.ldx = ldx;
    c.rows = rows; c.max_rows = rows; c.grid_tiles = 1;
    c.y = y; c.y_dtype = y_dtype; c.ldy = ldy;
    c.accumulate = (flags & IQ_FLAG_ACCUMULATE) ? 1 : 0;
    return launch_gqmv(ctx, reinterpret_cast<cudaStream_t>(stream), c);
}
