// Launchers of the GEMV family and the iq_qmv entry point.
#include <stdarg.h>
#include <stdio.h>

#include <stdlib.h>
#include <string.h>

#include "gqmv.cuh"
#include "internal.h"
#include "qmv_imma.cuh"
#include "qmv_imma_grouped.cuh"
#include "qmv_stream.cuh"

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
        case kFmtAffine4G32: return pick_mh<kFmtAffine4G32>(mh, mode, wk);
        default: return nullptr;
    }
}

constexpr int kSmemBudget = 200 * 1024;

// ---- streaming (TMA ring) path --------------------------------------------------------------------------------------
typedef void (*QsKernel)(const QsParams);

template <int FMT, int MH>
QsKernel qs_pick_mode(int mode) {
    switch (mode) {
        case kModeGateUp: return qmv_stream_kernel<FMT, MH, kModeGateUp>;
        case kModeDown: return qmv_stream_kernel<FMT, MH, kModeDown>;
        default: return qmv_stream_kernel<FMT, MH, kModePlain>;
    }
}
QsKernel qs_pick(int32_t fmt, int mh, int mode) {
    switch (fmt) {
        case kFmtAffine4: return mh == 2 ? qs_pick_mode<kFmtAffine4, 2>(mode) : qs_pick_mode<kFmtAffine4, 1>(mode);
        case kFmtAffine8: return mh == 2 ? qs_pick_mode<kFmtAffine8, 2>(mode) : qs_pick_mode<kFmtAffine8, 1>(mode);
        case kFmtMxfp4: return mh == 2 ? qs_pick_mode<kFmtMxfp4, 2>(mode) : qs_pick_mode<kFmtMxfp4, 1>(mode);
        default: return nullptr;
    }
}
constexpr int kQsSmemMax = 226 * 1024;

constexpr int kQiCtasPerSm = 2;  // up to four rows: two CTAs per SM (one CTA with a deeper ring measured 10.7 against 10.0 us)

// Returns kOk after a launch, 1 when the shape does not fit this path (the caller falls back), or an error.
int32_t launch_qmv_stream(iq_ctx* ctx, cudaStream_t st, const GqmvCall& c) {
    if (c.fmt == kFmtAffine4G32 || c.fmt == kFmtAffine6) return 1;  // not this kernel's formats
    const bool has_bias = c.fmt != kFmtMxfp4;
    const int nw = c.mode == kModeGateUp ? 2 : 1;
    const int mh = c.max_rows > 8 ? 2 : 1;
    const int ck = c.fmt == kFmtAffine8 ? 16 : 32;
    const int qu = ck == 32 ? 4 : 2;
    const int row_bytes = c.fmt == kFmtAffine8 ? c.K : c.K / 2;
    const int srow_bytes = c.fmt == kFmtMxfp4 ? c.K / 32 : c.K / 64 * 2;
    const int per_row = row_bytes + srow_bytes * (has_bias ? 2 : 1);
    for (int i = 0; i < nw; i++) {
        if ((reinterpret_cast<uintptr_t>(c.w[i] ? c.w[i] : c.w[0]) & 15) || (reinterpret_cast<uintptr_t>(c.s[i] ? c.s[i] : c.s[0]) & 15) ||
            (has_bias && (reinterpret_cast<uintptr_t>(c.b[i] ? c.b[i] : c.b[0]) & 15)))
            return 1;
    }
    int rgs = 1;
    while (rgs < 8 && 16 * rgs * per_row * nw < 24 * 1024 && 16 * rgs * 2 <= c.N) rgs *= 2;
    const int R = 16 * rgs;
    const int mat_bytes = round_up(R * per_row, 128);
    const int stage_bytes = nw * mat_bytes;
    const int nsteps = (row_bytes / 16 + 3) / 4;
    const int xs_bytes = round_up(nsteps * qu * c.max_rows * 4 * 16, 128);
    const int red_bytes = 2 * 8 * nw * mh * 4 * 32 * 4;
    const int fixed = xs_bytes + red_bytes + 256;  // + barriers, abort flag, zero block
    if (stage_bytes > 80 * 1024) return 1;
    // two CTAs per SM when the activations are small: twice the warps to hide dependency and barrier stalls
    int ctas_per_sm = 1;
    int nstages = (kQsSmemMax - fixed) / stage_bytes;
    if (mh == 1 && nw == 1 && (kQsSmemMax / 2 - 1024 - fixed) / stage_bytes >= 2) {
        ctas_per_sm = 2;
        nstages = (kQsSmemMax / 2 - 1024 - fixed) / stage_bytes;
    }
    if (nstages < 2) return 1;
    if (nstages > 8) nstages = 8;
    QsKernel k = qs_pick(c.fmt, mh, c.mode);
    if (k == nullptr) return 1;

    QsParams p;
    memset(&p, 0, sizeof(p));
    for (int i = 0; i < 2; i++) {
        p.w[i] = reinterpret_cast<const unsigned char*>(c.w[i] ? c.w[i] : c.w[0]);
        p.s[i] = reinterpret_cast<const unsigned char*>(c.s[i] ? c.s[i] : c.s[0]);
        p.b[i] = reinterpret_cast<const unsigned char*>(c.b[i] ? c.b[i] : c.b[0]);
        p.ebias[i] = c.ebias[i];
    }
    p.w_ebytes = c.w_estride * 4;
    p.s_ebytes = c.s_estride * (c.fmt == kFmtMxfp4 ? 1 : 2);
    p.N = c.N; p.K = c.K;
    p.x = c.x; p.x_dtype = c.x_dtype; p.ldx = c.ldx;
    p.row_map = c.row_map; p.topk = c.topk;
    p.tiles = c.tiles; p.ntiles = c.ntiles; p.M = c.rows;
    p.y = c.y; p.y_dtype = c.y_dtype; p.ldy = c.ldy; p.accumulate = c.accumulate;
    p.limit = c.limit;
    p.act = c.act;
    p.R = R; p.NB = (c.N + R - 1) / R; p.rgs = rgs; p.wk = 8 / rgs;
    p.row_bytes = row_bytes; p.srow_bytes = srow_bytes; p.mat_bytes = mat_bytes; p.stage_bytes = stage_bytes;
    p.nstages = nstages;
    p.xs_bytes = xs_bytes; p.red_bytes = red_bytes;
    p.status = ctx->d_status;

    const int64_t items = (int64_t)p.NB * c.grid_tiles;
    const int64_t slots = (int64_t)ctx->sms * ctas_per_sm;
    const int grid = (int)(items < slots ? items : slots);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kQsThreads, 1, 1);
    cfg.dynamicSmemBytes = fixed + nstages * stage_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(ctx, cudaLaunchKernelEx(&cfg, k, p), "qmv_stream launch");
}

// The tail split's scratch slot of a stream: launches of one stream run in series (a dependent launch waits for its
// predecessor before it touches the scratch), so a stream keeps one slot for good; streams may overlap, so each gets its
// own, and a context serves at most kQmvTailSlots of them. -1 when they are used up.
int tail_slot_of(iq_ctx* ctx, cudaStream_t st) {
    std::lock_guard<std::mutex> hold(ctx->qmv_tail_lock);
    for (int i = 0; i < ctx->qmv_tail_stream_count; i++)
        if (ctx->qmv_tail_streams[i] == static_cast<void*>(st)) return i;
    if (ctx->qmv_tail_stream_count >= kQmvTailSlots) return -1;
    ctx->qmv_tail_streams[ctx->qmv_tail_stream_count] = static_cast<void*>(st);
    return ctx->qmv_tail_stream_count++;
}

// ---- int8 tensor-core path (decode, up to four rows, affine codes) -----------------------------------------------
// Returns kOk after a launch, 1 when the shape does not fit this path (the caller falls back), or an error.
int32_t launch_qmv_imma(iq_ctx* ctx, cudaStream_t st, const GqmvCall& c) {
    if (c.mode != kModePlain || c.tiles != nullptr || c.rows > 16 || c.rows < 1) return 1;
    if (c.fmt != kFmtAffine4 && c.fmt != kFmtAffine8 && c.fmt != kFmtAffine6) return 1;
    if (c.K % 2048 != 0 || c.N < kQiRows) return 1;
    if ((reinterpret_cast<uintptr_t>(c.w[0]) & 15) || (reinterpret_cast<uintptr_t>(c.s[0]) & 15) ||
        (reinterpret_cast<uintptr_t>(c.b[0]) & 15))
        return 1;
    const bool w8 = c.fmt == kFmtAffine8, w6 = c.fmt == kFmtAffine6;
    const int G = c.K / 64;
    QiParams p;
    memset(&p, 0, sizeof(p));
    p.row_bytes = w8 ? c.K : (w6 ? c.K / 4 * 3 : c.K / 2);
    // 4-bit codes with rows of 1 KB (K = 2048): one swizzled tensor copy per block of 16 rows, no padding (the swizzle
    // spreads the rows over the banks). Otherwise one bulk copy per row (4-bit) or per pair of rows (6- and 8-bit), padded apart by a quad's piece.
    const bool tm = c.fmt == kFmtAffine4 && p.row_bytes <= 1024 && ctx->encode_tiled != nullptr;
    p.pair = (w8 || w6) ? 1 : 0;  // two rows per bulk copy
    p.row_pitch = tm ? p.row_bytes : (p.pair ? 2 : 1) * p.row_bytes + (w8 ? 64 : (w6 ? 48 : 32));
    p.srow_bytes = G * 2;
    p.srow_pitch = p.srow_bytes;
    p.stage_bytes = (tm ? kQiRows * p.row_bytes : (p.pair ? kQiRows / 2 : kQiRows) * p.row_pitch) + 2 * kQiRows * p.srow_pitch;
    // The path is chosen on what eight rows need, whatever the row count of this call: a row must see the same
    // arithmetic alone and among sixteen.
    const int ncw = 8;  // consumer warps (16 measured slower: 11.3 against 10.0 us on the 14336 x 4096 layer)
    // (+ 1024: the stages of the tensor copies start on a 1024-byte boundary)
    auto fixed_bytes = [&](int ms) { return G * 512 * ms + G * 32 * ms + 512 * ms * ncw + 256 + (tm ? 1024 : 0); };
    if ((kQsSmemMax - fixed_bytes(2)) / p.stage_bytes < 2) return 1;
    p.w = reinterpret_cast<const unsigned char*>(c.w[0]);
    p.s = reinterpret_cast<const unsigned char*>(c.s[0]);
    p.b = reinterpret_cast<const unsigned char*>(c.b[0]);
    p.N = c.N; p.K = c.K;
    p.x_dtype = c.x_dtype; p.ldx = c.ldx;
    p.y_dtype = c.y_dtype; p.ldy = c.ldy; p.accumulate = c.accumulate;
    p.status = ctx->d_status;
    CUtensorMap wmap = {};
    const CUtensorMap* map = &wmap;
    if (tm) {
        // the matrix as the kernel sees it: all rows of W, whatever prefix of them this call computes (one cached map
        // per matrix, not one per prefix)
        const int32_t r = cached_rowblock_map(ctx, p.w, c.n_full > c.N ? c.n_full : c.N, p.row_bytes, kQiRows, &wmap);
        if (r != kOk) return r;
    }
    const int blocks = c.N / kQiRows;
    // Tail split, decided from the output features this call computes and the GPU alone (not from the activation row
    // count, so an activation row sees the same arithmetic alone and among sixteen; a call with n_prefix may split
    // differently from a call over the whole matrix): when the blocks do not divide over two CTAs per SM and few are
    // left over, the left-over blocks are cut into K slices and dealt out one piece per CTA.
    const int slots = 2 * ctx->sms;
    const int per2 = blocks / slots, tail = blocks - per2 * slots;
    int tail_slices = 0;
    if (c.N % kQiRows == 0 && per2 >= 1 && tail > 0 && tail * 8 <= slots && tail <= kQmvTailBlocks) {
        tail_slices = 1;
        while (tail_slices * 2 * tail <= slots && tail_slices * 2 <= 32 && G % (tail_slices * 2) == 0) tail_slices *= 2;
        if (tail_slices < 8 || tail * tail_slices > kQmvTailPieces) tail_slices = 0;
    }
    const size_t xes = c.x_dtype == kF32 ? 4 : 2, yes = c.y_dtype == kF32 ? 4 : 2;
    for (int m0 = 0; m0 < c.rows; m0 += 8) {  // nine to sixteen rows: two launches of up to eight
        const int m = c.rows - m0 < 8 ? c.rows - m0 : 8;
        const int ms = m > 4 ? 2 : 1;
        p.M = m;
        p.x = static_cast<const char*>(c.x) + (size_t)m0 * c.ldx * xes;
        p.y = static_cast<char*>(c.y) + (size_t)m0 * c.ldy * yes;
        p.xq_bytes = G * 512 * ms;
        p.xsc_bytes = G * 32 * ms;
        p.red_bytes = 512 * ms * ncw;
        p.ncw = ncw;
        // up to four rows: two CTAs per SM when each still gets two stages (twice the warps to hide latencies behind)
        int ctas = 1;
        if (ms == 1 && kQiCtasPerSm == 2 && (kQsSmemMax / 2 - 1024 - fixed_bytes(ms)) / p.stage_bytes >= 2) ctas = 2;
        int nstages = ((ctas == 2 ? kQsSmemMax / 2 - 1024 : kQsSmemMax) - fixed_bytes(ms)) / p.stage_bytes;
        if (nstages > 8) nstages = 8;
        p.nstages = nstages;
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(blocks < ctx->sms * ctas ? blocks : ctx->sms * ctas, 1, 1);
        p.tail_blocks = 0;
        if (tail_slices > 0) {
            const int slot = tail_slot_of(ctx, st);
            if (slot < 0)
                return fail(ctx, kErrInvalidArg, "qmv: more than %d streams launch GEMVs with a tail split on this context",
                            kQmvTailSlots);
            p.tail_blocks = tail;
            p.tail_slices = tail_slices;
            p.blocks_per_cta = per2 * (2 / ctas);
            p.tail_scratch = ctx->qmv_tail_scratch + (size_t)slot * kQmvTailPieces * 2 * 64;
            p.tail_counters = ctx->qmv_tail_counters + (size_t)slot * kQmvTailBlocks;
            cfg.gridDim = dim3(ctx->sms * ctas, 1, 1);
        }
        cfg.blockDim = dim3(32 * (ncw + 2), 1, 1);
        cfg.dynamicSmemBytes = fixed_bytes(ms) + nstages * p.stage_bytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        // up to four rows and eight or four groups per warp (K = 4096, 2048): the activation fragments stay in registers
        const int gwh = ms == 1 ? G / ncw : 0;
        cudaError_t e;
#define IQ_QI_LAUNCH(F)                                                                             \
    (ms == 2 ? cudaLaunchKernelEx(&cfg, qmv_imma_kernel<F, 2, 0>, *map, p)                          \
             : gwh == 8 ? cudaLaunchKernelEx(&cfg, qmv_imma_kernel<F, 1, 8>, *map, p)               \
                        : gwh == 4 ? cudaLaunchKernelEx(&cfg, qmv_imma_kernel<F, 1, 4>, *map, p)    \
                                   : cudaLaunchKernelEx(&cfg, qmv_imma_kernel<F, 1, 0>, *map, p))
        if (tm) e = ms == 2 ? cudaLaunchKernelEx(&cfg, qmv_imma_kernel<kFmtAffine4, 2, 0, true>, *map, p)
                            : cudaLaunchKernelEx(&cfg, qmv_imma_kernel<kFmtAffine4, 1, 4, true>, *map, p);
        else if (w6) e = IQ_QI_LAUNCH(kFmtAffine6);
        else if (w8) e = IQ_QI_LAUNCH(kFmtAffine8);
        else e = IQ_QI_LAUNCH(kFmtAffine4);
#undef IQ_QI_LAUNCH
        const int32_t r = check_cuda(ctx, e, "qmv_imma launch");
        if (r != kOk) return r;
    }
    return kOk;
}

// ---- int8 tensor-core path for the MoE decode tiles (gate/up + activation, down; affine 4-bit experts) ---------------
typedef void (*QgKernel)(const CUtensorMap, const CUtensorMap, const QgParams);
// gw4: each consumer warp's K slice is four groups, its activation fragments stay in registers (8-row tiles only)
template <int MODE, bool TM>
QgKernel qg_pick_mt(int ms, bool gw4) {
    if (ms == 4) return qmv_imma_grouped_kernel<MODE, 4, TM, 0>;
    return gw4 ? qmv_imma_grouped_kernel<MODE, 2, TM, 4> : qmv_imma_grouped_kernel<MODE, 2, TM, 0>;
}
QgKernel qg_pick(int mode, int ms, bool tm, bool gw4) {
    if (mode == kModeGateUp) return tm ? qg_pick_mt<kModeGateUp, true>(ms, gw4) : qg_pick_mt<kModeGateUp, false>(ms, gw4);
    return tm ? qg_pick_mt<kModeDown, true>(ms, gw4) : qg_pick_mt<kModeDown, false>(ms, gw4);
}
// Returns kOk after a launch, 1 when the shape does not fit this path (the caller falls back), or an error.
int32_t launch_qmv_imma_grouped(iq_ctx* ctx, cudaStream_t st, const GqmvCall& c) {
    if ((c.mode != kModeGateUp && c.mode != kModeDown) || c.tiles == nullptr || c.fmt != kFmtAffine4) return 1;
    if (c.K % 64 != 0 || c.N % 16 != 0 || c.max_rows > 16 || c.accumulate) return 1;
    const int nw = c.mode == kModeGateUp ? 2 : 1;
    for (int i = 0; i < nw; i++)
        if ((reinterpret_cast<uintptr_t>(c.w[i]) & 15) || (reinterpret_cast<uintptr_t>(c.s[i]) & 15) ||
            (reinterpret_cast<uintptr_t>(c.b[i]) & 15))
            return 1;
    const int G = c.K / 64;
    QgParams p;
    memset(&p, 0, sizeof(p));
    p.row_bytes = c.K / 2;
    // Tensor-copy staging: the stacked tensors must be known (which experts they hold) and dense, rows whole 128-byte
    // columns. Short weight rows (the down projection's K = d_ff, 384 bytes) take this path only with tensor copies: one
    // bulk copy per row measured 61.9 against 49.6 us on the fp16 tile kernels at 64 tokens; with tensor copies, 128-row
    // blocks and no K split (12 groups of 64 inputs do not divide into runs of four over more than one slice) it
    // measures 37.3 us (16 tokens: 23.9 against 30.6; 256 tokens: 79.8 against 121).
    const bool tm = ctx->encode_tiled != nullptr && c.expert_count > 0 && p.row_bytes % 128 == 0 && p.row_bytes / 128 <= 256 &&
                    c.w_estride * 4 == (int64_t)c.N * p.row_bytes;
    if (c.K < 2048 && !tm) return 1;
    const int ms = c.max_rows > 8 ? 4 : 2;
    p.row_pitch = tm ? p.row_bytes : p.row_bytes + 32;
    p.srow_bytes = G * 2;
    p.xq_bytes = G * ms * 512;
    p.xsc_bytes = G * ms * 32;
    p.red_bytes = 2 * kQgWarps * nw * ms * 64 * 4;
    const int fixed = p.xq_bytes + p.xsc_bytes + p.red_bytes + 256 + (tm ? 1024 : 0);
    // K slices per block of rows. 8-row tiles: one slice of four groups per warp when K allows it (the activation
    // fragments then live in registers: 69 against 83 us on the 64-token layer); else four slices (32-row blocks: half as
    // many hand-overs per byte) when two stages of that size fit, else eight.
    int ctas = 1, nstages = 0;
    const bool gw4 = ms == 2 && G == 4 * kQgWarps;
    const int cand[4] = {gw4 ? kQgWarps : kQgWarps / 2, kQgWarps, kQgWarps / 4, kQgWarps / 8};
    for (int ci = 0; ci < 4 && nstages < 2; ci++) {
        const int wk = cand[ci];
        if (G % wk != 0 || (G / wk) % 4 != 0) continue;  // a warp's K slice: runs of four groups
        const int R = 16 * (kQgWarps / wk);
        if ((R * p.srow_bytes) % 16 != 0) continue;
        p.wk = wk; p.rgs = kQgWarps / wk;
        p.NB = (c.N + R - 1) / R;
        p.mat_bytes = round_up(R * p.row_pitch + 2 * R * p.srow_bytes, tm ? 1024 : 16);
        p.stage_bytes = nw * p.mat_bytes;
        nstages = (kQsSmemMax - fixed) / p.stage_bytes;
    }
    if (nstages < 2) return 1;
    if (nstages > 8) nstages = 8;
    p.nstages = nstages;
    for (int i = 0; i < 2; i++) {
        p.w[i] = reinterpret_cast<const unsigned char*>(c.w[i] ? c.w[i] : c.w[0]);
        p.s[i] = reinterpret_cast<const unsigned char*>(c.s[i] ? c.s[i] : c.s[0]);
        p.b[i] = reinterpret_cast<const unsigned char*>(c.b[i] ? c.b[i] : c.b[0]);
        p.ebias[i] = c.ebias[i];
    }
    p.w_ebytes = c.w_estride * 4;
    p.s_ebytes = c.s_estride * 2;
    p.expert_lo = c.expert_lo;
    CUtensorMap wmaps[2] = {};
    const CUtensorMap* maps[2] = {&wmaps[0], &wmaps[1]};
    if (tm) {
        for (int i = 0; i < nw; i++) {
            const int32_t r = cached_rowblock_map(ctx, p.w[i] + (int64_t)c.expert_lo * p.w_ebytes, (int64_t)c.expert_count * c.N,
                                                  p.row_bytes, 16 * p.rgs, &wmaps[i]);
            if (r != kOk) return r;
        }
    }
    p.N = c.N; p.K = c.K;
    p.x = c.x; p.x_dtype = c.x_dtype; p.ldx = c.ldx;
    p.row_map = c.row_map; p.topk = c.topk;
    p.tiles = c.tiles; p.ntiles = c.ntiles;
    p.y = c.y; p.y_dtype = c.y_dtype; p.ldy = c.ldy;
    p.limit = c.limit;
    p.act = c.act;
    p.status = ctx->d_status;
    const int64_t items = (int64_t)p.NB * c.grid_tiles;
    const int64_t slots = (int64_t)ctx->sms * ctas;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(items < slots ? items : slots), 1, 1);
    cfg.blockDim = dim3(kQgThreads, 1, 1);
    cfg.dynamicSmemBytes = fixed + nstages * p.stage_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(ctx, cudaLaunchKernelEx(&cfg, qg_pick(c.mode, ms, tm, gw4 && p.wk == kQgWarps), *maps[0], *maps[1], p), "qmv_imma_grouped launch");
}

}  // namespace

int32_t gqmv_init(iq_ctx* ctx) {
#define IQ_QI_ALL(F)                                                                                           \
    reinterpret_cast<const void*>(qmv_imma_kernel<F, 1, 0>), reinterpret_cast<const void*>(qmv_imma_kernel<F, 1, 4>), \
        reinterpret_cast<const void*>(qmv_imma_kernel<F, 1, 8>), reinterpret_cast<const void*>(qmv_imma_kernel<F, 2, 0>)
    const void* qi[14] = {IQ_QI_ALL(kFmtAffine4), IQ_QI_ALL(kFmtAffine8), IQ_QI_ALL(kFmtAffine6),
                          reinterpret_cast<const void*>(qmv_imma_kernel<kFmtAffine4, 1, 4, true>),
                          reinterpret_cast<const void*>(qmv_imma_kernel<kFmtAffine4, 2, 0, true>)};
#undef IQ_QI_ALL
    for (int i = 0; i < 14; i++) {
        cudaError_t e = cudaFuncSetAttribute(qi[i], cudaFuncAttributeMaxDynamicSharedMemorySize, kQsSmemMax);
        if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(qmv_imma)");
    }
    for (int mode = kModeGateUp; mode <= kModeDown; mode++)
        for (int v = 0; v < 6; v++) {  // 4 row sets, 2, 2 with register-resident activations; bulk or tensor copies
            cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(qg_pick(mode, v % 3 == 0 ? 4 : 2, v >= 3, v % 3 == 2)),
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kQsSmemMax);
            if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(qmv_imma_grouped)");
        }
    for (int fmt = 0; fmt < 4; fmt++)
        for (int mh = 1; mh <= 2; mh++)
            for (int mode = 0; mode < 3; mode++)
                for (int wk = 2; wk <= 8; wk *= 2) {
                    GqmvKernel k = pick(fmt, mh, mode, wk);
                    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k),
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 20480);
                    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(gqmv)");
                }
    for (int fmt = 0; fmt < 3; fmt++)
        for (int mh = 1; mh <= 2; mh++)
            for (int mode = 0; mode < 3; mode++) {
                cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(qs_pick(fmt, mh, mode)),
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kQsSmemMax);
                if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(qmv_stream)");
            }
    return kOk;
}

int32_t launch_gqmv(iq_ctx* ctx, cudaStream_t st, const GqmvCall& c) {
    // One kernel per (format, shape), chosen from the matrix alone: the int8 tensor-core kernels for affine codes whose
    // K fits their staging, the streaming fp16 kernel for MXFP4 and the remaining affine shapes, the register-staged
    // fp16 kernel where a 16-row block over the whole K does not fit a stage.
    int32_t r = launch_qmv_imma(ctx, st, c);
    if (r != 1) return r;
    r = launch_qmv_imma_grouped(ctx, st, c);
    if (r != 1) return r;
    r = launch_qmv_stream(ctx, st, c);
    if (r != 1) return r;
    if (c.fmt == kFmtAffine6)
        return fail(ctx, kErrUnsupported, "qmv: 6-bit weights run on the int8 kernel only (a plain GEMV, k a multiple of 2048, n >= 16)");
    const int ck = c.fmt == kFmtAffine8 ? 16 : 32;  // inputs per 16-byte chunk
    const int mh = c.max_rows > 8 ? 2 : 1;
    const int nw = c.mode == kModeGateUp ? 2 : 1;
    // K tile: everything at once when the staged activations fit, else the largest multiple of 1024 that does
    int kt = c.K;
    auto smem_for = [&](int ktile, int* xs_bytes) {
        const int nsteps = (ktile / ck + 3) / 4;
        const int qu = ck == 32 ? 4 : 2;
        *xs_bytes = nsteps * qu * c.max_rows * 4 * 16;
        const int red_bytes = 8 * nw * mh * 4 * 32 * 4;
        return *xs_bytes + red_bytes;
    };
    int xs_bytes;
    while (smem_for(kt, &xs_bytes) > kSmemBudget) {
        kt = kt > 1024 ? (kt - 1) / 1024 * 1024 : 0;
        if (kt == 0) return fail(ctx, kErrInvalidArg, "qmv: activations do not fit shared memory");
    }
    const int smem = smem_for(kt, &xs_bytes);

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
    p.act = c.act;
    p.kt = kt; p.xs_bytes = xs_bytes;

    dim3 grid((c.N / 16 + rg - 1) / rg, c.grid_tiles, 1);
    k<<<grid, 256, smem, st>>>(p);
    return check_cuda(ctx, cudaGetLastError(), "gqmv launch");
}

int32_t format_of(const iq_qlinear* m) {
    if (m->mode == IQ_MODE_MXFP4) return (m->bits == 4 && m->group == 32) ? kFmtMxfp4 : -1;
    if (m->mode != IQ_MODE_AFFINE) return -1;
    if (m->group == 32) return m->bits == 4 ? kFmtAffine4G32 : -1;
    if (m->group == 128) return m->bits == 2 ? kFmtTernary : -1;
    if (m->group != 64) return -1;
    if (m->bits == 6) return kFmtAffine6;
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
        return fail(ctx, kErrUnsupported, "qmv: %d-bit group %d mode %d has no kernel (affine 4/6/8-bit g64, 4-bit g32, ternary 2-bit g128, mxfp4 g32)",
                    m->bits, m->group, m->mode);
    if (fmt != kFmtMxfp4 && fmt != kFmtTernary && m->biases == nullptr)
        return fail(ctx, kErrInvalidArg, "qmv: affine layer without biases");
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
    if (fmt == kFmtTernary)  // the rotated ternary format has kernels of its own (csrc/tern.cu)
        return launch_tern_qmv(ctx, reinterpret_cast<cudaStream_t>(stream), x, x_dtype, ldx, m, y, y_dtype, ldy, rows, n,
                               (flags & IQ_FLAG_ACCUMULATE) ? 1 : 0);
    GqmvCall c;
    c.mode = kModePlain;
    c.fmt = fmt;
    c.w[0] = reinterpret_cast<const uint32_t*>(m->w);
    c.s[0] = m->scales;
    c.b[0] = m->biases;
    c.N = n;
    c.n_full = m->n;
    c.K = m->k;
    c.x = x; c.x_dtype = x_dtype; c.ldx = ldx;
    c.rows = rows; c.max_rows = rows; c.grid_tiles = 1;
    c.y = y; c.y_dtype = y_dtype; c.ldy = ldy;
    c.accumulate = (flags & IQ_FLAG_ACCUMULATE) ? 1 : 0;
    return launch_gqmv(ctx, reinterpret_cast<cudaStream_t>(stream), c);
}
