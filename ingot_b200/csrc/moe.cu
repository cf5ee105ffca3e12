// MoE layer and dense gated FFN entry points.
#include <string.h>

#include <new>

#include "internal.h"
#include "moe_aux.cuh"

struct iq_moe {
    iq_ctx* ctx = nullptr;
    iq_moe_desc d;
    int32_t fmt = 0;
    int32_t ld = 0;  // logits row stride
    const uint32_t* ext_inds = nullptr;
    const float* ext_wts = nullptr;
    // largest row norm of a bf16 router (0: not computed), for the error bound of the tensor-core logits
    float router_wnorm_max = 0.f;
};

namespace iq {

namespace {

struct MoeWs {
    float* logits;
    uint32_t* inds;
    float* wts;
    uint32_t* counts;
    uint32_t* offsets;
    uint32_t* row_map;
    uint32_t* pos;
    uint32_t* ntiles;
    uint32_t* chunk_hist;
    Tile* tiles_a;
    Tile* tiles_b;
    __half* h;
    void* yd;
    __half* xs;  // activations in expert order, fp16 [P, d_model] (tensor-core path)
    // shared expert (only when the layer has one): fp16 copy of x, h, output, per-token weight, tile list
    __half* s_x16;
    __half* s_h;
    void* s_yd;
    float* s_w;
    Tile* s_tiles;
    uint32_t* s_ntiles;
    size_t bytes;
};

// Height of the tiles of the GEMV-style expert kernels: 8 rows while experts see few rows, else 16.
int decode_tile_rows(const iq_moe* l, int tokens) {
    const int64_t pairs = (int64_t)tokens * l->d.top_k;
    return pairs <= (int64_t)l->d.experts * 6 ? 8 : 16;
}
constexpr int kPrefillTileRows = 128;      // token rows per tensor-core tile while experts see few rows
constexpr int kPrefillTileRowsBig = 256;   // ... and once they see many: every weight tile is dequantised half as often
constexpr int kTensorPathRowsPerExpert = 24;
constexpr int kBigTileRowsPerExpert = 96;
constexpr int kRouterSmemMax = 200 * 1024;
constexpr int kGroupChunkedMinPairs = 4096;  // from here on the permutation runs as a chunked counting sort
constexpr int kRouterTiledMinTokens = 64;  // above this the router runs as a tiled float64 GEMM

// Expert outputs between the down projection and the combine: fp16 for affine experts, fp32 for MXFP4 ones, whose
// outputs can pass half's range (the reference makes the same choice, MoEPrefill.swift:159-160).
int32_t yd_dtype_of(const iq_moe* l) { return l->fmt == kFmtMxfp4 ? kF32 : kF16; }

MoeWs carve(const iq_moe* l, void* base, int tokens) {
    const iq_moe_desc& d = l->d;
    const size_t P = (size_t)tokens * d.top_k;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        void* p = base ? static_cast<char*>(base) + off : nullptr;
        off += round_up_sz(bytes, 256);
        return p;
    };
    MoeWs w;
    w.logits = static_cast<float*>(take((size_t)tokens * l->ld * 4));
    w.inds = static_cast<uint32_t*>(take(P * 4));
    w.wts = static_cast<float*>(take(P * 4));
    w.counts = static_cast<uint32_t*>(take((size_t)d.experts * 4));
    w.offsets = static_cast<uint32_t*>(take((size_t)(d.experts + 1) * 4));
    w.row_map = static_cast<uint32_t*>(take(P * 4));
    w.pos = static_cast<uint32_t*>(take(P * 4));
    w.ntiles = static_cast<uint32_t*>(take(16));
    w.chunk_hist = static_cast<uint32_t*>(take((P / kGroupChunk + 1) * (size_t)d.experts * 4));
    w.tiles_a = static_cast<Tile*>(take((d.experts + P / 8 + 1) * sizeof(Tile)));
    w.tiles_b = static_cast<Tile*>(take((d.experts + P / kPrefillTileRows + 1) * sizeof(Tile)));
    w.h = static_cast<__half*>(take(P * d.d_ff * 2));
    w.yd = take(P * d.d_model * (yd_dtype_of(l) == kF16 ? 2 : 4));
    w.xs = static_cast<__half*>(take(P * d.d_model * 2));
    w.s_x16 = nullptr; w.s_h = nullptr; w.s_yd = nullptr; w.s_w = nullptr; w.s_tiles = nullptr; w.s_ntiles = nullptr;
    if (d.shared != IQ_SHARED_NONE) {
        const size_t T = (size_t)tokens;
        w.s_x16 = static_cast<__half*>(take(T * d.d_model * 2));
        w.s_h = static_cast<__half*>(take(T * d.shared_up.n * 2));
        w.s_yd = take(T * d.d_model * 4);
        w.s_w = static_cast<float*>(take(T * 4));
        w.s_tiles = static_cast<Tile*>(take((T / 16 + 2) * sizeof(Tile)));
        w.s_ntiles = static_cast<uint32_t*>(take(16));
    }
    w.bytes = off;
    return w;
}

typedef void (*RouteKernel)(const RouteParams);
template <bool REFINE, int WPT>
RouteKernel route_kernel_of(int experts) {
    switch ((experts + 31) / 32) {
        case 1: return route_topk_kernel<1, REFINE, WPT>;
        case 2: return route_topk_kernel<2, REFINE, WPT>;
        case 3: return route_topk_kernel<3, REFINE, WPT>;
        case 4: return route_topk_kernel<4, REFINE, WPT>;
        case 5: case 6: return route_topk_kernel<6, REFINE, WPT>;
        case 7: case 8: return route_topk_kernel<8, REFINE, WPT>;
        case 9: case 10: case 11: case 12: return route_topk_kernel<12, REFINE, WPT>;
        default: return route_topk_kernel<16, REFINE, WPT>;
    }
}
// wide: four warps per token share the refinement's exact dot products (few tokens: the chain per token is the time)
RouteKernel route_kernel_for(int experts, bool refine, bool wide) {
    if (!refine) return route_kernel_of<false, 1>(experts);
    return wide ? route_kernel_of<true, 4>(experts) : route_kernel_of<true, 1>(experts);
}
constexpr int kRouteWideMaxTokens = 2048;

// Many tokens with a bf16 router and bf16 activations: the logits come from the tensor cores (bf16 products are exact,
// the fp32 accumulation is not), and the route kernel recomputes exactly, in float64, the few logits per token that
// can still be among the k largest. Indices and weights are then the same bits as with float64 logits throughout, at
// a fifth of the time: the float64 GEMM was 135 us of a 4096-token layer.
// Error bound of an approximate logit: K accumulations, each assumed to lose at most 2^-21 of the running magnitude
// (eight times what round-to-nearest fp32 would), over sum_k |x_k w_k| <= ||x||_2 ||w||_2.
bool tensor_router(const iq_moe* l, int tokens, int32_t x_dtype) {
    const iq_moe_desc& d = l->d;
    return l->router_wnorm_max > 0.f && l->ext_inds == nullptr && d.router_kind == IQ_ROUTER_BF16 &&
           d.router_score == IQ_SCORE_SOFTMAX && x_dtype == kBF16 && tokens > kRouterTiledMinTokens && d.experts % 64 == 0 &&
           d.d_model % 64 == 0;
}
float router_err_coef(const iq_moe* l) { return (float)l->d.d_model * 4.76837158e-7f * 1.05f * l->router_wnorm_max; }

int32_t launch_route(iq_moe* l, cudaStream_t st, const float* logits, int ld, int tokens, uint32_t* inds, float* wts,
                     const void* refine_x = nullptr, int64_t ldx = 0) {
    RouteParams rp;
    rp.logits = logits;
    rp.logits_rw = const_cast<float*>(logits);
    rp.x = static_cast<const uint16_t*>(refine_x);
    rp.ldx = ldx;
    rp.wr = static_cast<const uint16_t*>(l->d.router_w);
    rp.D = l->d.d_model;
    rp.err_coef = router_err_coef(l);
    rp.logit_bias = l->d.router_logit_bias;
    rp.pes = l->d.per_expert_scale;
    rp.inds = inds;
    rp.wts = wts;
    rp.T = tokens; rp.E = l->d.experts; rp.ld = ld; rp.topk = l->d.top_k;
    rp.scale = l->d.routed_scale;
    rp.sigmoid = l->d.router_score == IQ_SCORE_SIGMOID ? 1 : 0;
    rp.select_bias = l->d.router_select_bias;
    rp.eps = l->d.route_eps;
    const bool wide = refine_x != nullptr && tokens <= kRouteWideMaxTokens;
    route_kernel_for(l->d.experts, refine_x != nullptr, wide)<<<wide ? tokens : (tokens + 3) / 4, 128, 0, st>>>(rp);
    return check_cuda(l->ctx, cudaGetLastError(), "route_topk launch");
}

// Gate + up + activation of every tile: h[row, :] = half(act(x W_gate^T + b_g, x W_up^T + b_u)). Expert e's weights live
// at local slot e - expert_lo: the offset is folded into the base pointers. row_map == nullptr: x rows are in place.
int32_t run_gateup(iq_moe* l, cudaStream_t cs, const void* x, int32_t x_dtype, int64_t ldx, const uint32_t* row_map,
                   const Tile* tiles, const uint32_t* ntiles, int max_tiles, int bm, __half* h, int row_map_div = 0) {
    const iq_moe_desc& d = l->d;
    const int64_t lo = d.expert_lo;
    GqmvCall c;
    c.mode = kModeGateUp;
    c.fmt = l->fmt;
    c.w_estride = (int64_t)d.d_ff * (d.d_model / 8);
    c.s_estride = (int64_t)d.d_ff * (d.d_model / d.gate.group);
    const size_t sb = l->fmt == kFmtMxfp4 ? 1 : 2;
    c.w[0] = static_cast<const uint32_t*>(d.gate.w) - lo * c.w_estride;
    c.w[1] = static_cast<const uint32_t*>(d.up.w) - lo * c.w_estride;
    c.s[0] = static_cast<const char*>(d.gate.scales) - lo * c.s_estride * (int64_t)sb;
    c.s[1] = static_cast<const char*>(d.up.scales) - lo * c.s_estride * (int64_t)sb;
    if (d.gate.biases) {
        c.b[0] = static_cast<const char*>(d.gate.biases) - lo * c.s_estride * 2;
        c.b[1] = static_cast<const char*>(d.up.biases) - lo * c.s_estride * 2;
    }
    c.expert_lo = d.expert_lo; c.expert_count = d.expert_count;
    c.N = d.d_ff; c.K = d.d_model;
    c.x = x; c.x_dtype = x_dtype; c.ldx = ldx;
    c.row_map = row_map; c.topk = row_map_div > 0 ? row_map_div : d.top_k;  // x row = row_map[sorted position] / divisor
    c.tiles = tiles; c.ntiles = ntiles; c.grid_tiles = max_tiles;
    c.rows = 0; c.max_rows = bm;
    c.y = h; c.y_dtype = kF16; c.ldy = d.d_ff;
    if (d.gate_bias) {
        c.ebias[0] = d.gate_bias - lo * d.d_ff;
        c.ebias[1] = d.up_bias - lo * d.d_ff;
    }
    c.limit = d.act == IQ_ACT_SWIGLU_OAI ? d.act_limit : 0.f;
    c.act = d.act;
    return launch_gqmv(l->ctx, cs, c);
}

// Down projection of every tile: yd[row, :] = h[row, :] W_down^T + b_d.
int32_t run_down(iq_moe* l, cudaStream_t cs, const __half* h, const Tile* tiles, const uint32_t* ntiles, int max_tiles,
                 int bm, void* yd, int32_t yd_dtype) {
    const iq_moe_desc& d = l->d;
    const int64_t lo = d.expert_lo;
    GqmvCall c;
    c.mode = kModeDown;
    c.fmt = l->fmt;
    c.w_estride = (int64_t)d.d_model * (d.d_ff / 8);
    c.s_estride = (int64_t)d.d_model * (d.d_ff / d.down.group);
    const size_t sb = l->fmt == kFmtMxfp4 ? 1 : 2;
    c.w[0] = static_cast<const uint32_t*>(d.down.w) - lo * c.w_estride;
    c.s[0] = static_cast<const char*>(d.down.scales) - lo * c.s_estride * (int64_t)sb;
    if (d.down.biases) c.b[0] = static_cast<const char*>(d.down.biases) - lo * c.s_estride * 2;
    c.expert_lo = d.expert_lo; c.expert_count = d.expert_count;
    c.N = d.d_model; c.K = d.d_ff;
    c.x = h; c.x_dtype = kF16; c.ldx = d.d_ff;
    c.tiles = tiles; c.ntiles = ntiles; c.grid_tiles = max_tiles;
    c.rows = 0; c.max_rows = bm;
    c.y = yd; c.y_dtype = yd_dtype; c.ldy = d.d_model;
    if (d.down_bias) c.ebias[0] = d.down_bias - lo * d.d_model;
    return launch_gqmv(l->ctx, cs, c);
}

// The experts run on the tcgen05 grouped GEMM once they see enough rows each for 128-row MMA tiles to pay; below
// that the layer is bandwidth-bound and the GEMV-style tile kernels read each touched expert once.
bool use_tensor_path(int64_t rows, int64_t expert_slots) { return rows >= expert_slots * kTensorPathRowsPerExpert; }
int tensor_tile_rows(int64_t rows, int64_t expert_slots) {
    return rows >= expert_slots * kBigTileRowsPerExpert ? kPrefillTileRowsBig : kPrefillTileRows;
}

// rows16: fp16 rows [n_rows, ld16] in tile order, or (gather_map given) the tokens' rows in place, fetched through
// gather_map[sorted position] / gather_div.
int32_t run_gateup_tc(iq_moe* l, cudaStream_t cs, const __half* rows16, int64_t n_rows, const Tile* tiles,
                      const uint32_t* ntiles, __half* h, int bn, const uint32_t* gather_map = nullptr, uint32_t gather_div = 1,
                      int64_t ld16 = 0, int64_t x_rows = 0) {
    const iq_moe_desc& d = l->d;
    QmmCall c;
    c.fmt = l->fmt; c.epi = 1; c.bn = bn;
    c.x16 = rows16; c.ldx = ld16 > 0 ? ld16 : d.d_model; c.x_rows = x_rows > 0 ? x_rows : n_rows;
    c.gather_map = gather_map; c.gather_div = gather_div;
    c.w[0] = d.gate.w; c.w[1] = d.up.w;
    c.s[0] = d.gate.scales; c.s[1] = d.up.scales;
    c.b[0] = d.gate.biases; c.b[1] = d.up.biases;
    c.experts = d.expert_count; c.expert_lo = d.expert_lo;
    c.N = d.d_ff; c.K = d.d_model; c.M = (int32_t)n_rows;
    c.tiles = tiles; c.ntiles = ntiles;
    c.y = h; c.y_dtype = kF16; c.ldy = d.d_ff;
    c.ebias[0] = d.gate_bias; c.ebias[1] = d.up_bias;
    c.limit = d.act == IQ_ACT_SWIGLU_OAI ? d.act_limit : 0.f;
    c.act = d.act;
    return launch_qmm(l->ctx, cs, c);
}

int32_t run_down_tc(iq_moe* l, cudaStream_t cs, const __half* h, int64_t n_rows, const Tile* tiles, const uint32_t* ntiles,
                    void* yd, int32_t yd_dtype, int bn) {
    const iq_moe_desc& d = l->d;
    QmmCall c;
    c.fmt = l->fmt; c.epi = 0; c.bn = bn;
    c.x16 = h; c.ldx = d.d_ff; c.x_rows = n_rows;
    c.w[0] = d.down.w; c.s[0] = d.down.scales; c.b[0] = d.down.biases;
    c.experts = d.expert_count; c.expert_lo = d.expert_lo;
    c.N = d.d_model; c.K = d.d_ff; c.M = (int32_t)n_rows;
    c.tiles = tiles; c.ntiles = ntiles;
    c.y = yd; c.y_dtype = yd_dtype; c.ldy = d.d_model;
    c.ebias[0] = d.down_bias;
    return launch_qmm(l->ctx, cs, c);
}

// The shared expert (MoE.swift:140-154; the reference runs it as expert id E of the same kernels): one more FFN over all
// tokens, rows in place, through the same tile kernels with a copy of the layer whose expert tensors are the shared
// expert's; out += w_s * y_s with w_s = sigmoid(x . shared_gate) or 1.
int32_t run_shared_expert(iq_moe* l, cudaStream_t cs, const void* x, int32_t x_dtype, int64_t ldx, int tokens, const MoeWs& w,
                          void* out, int32_t out_dtype, int64_t ldo) {
    const iq_moe_desc& d = l->d;
    iq_ctx* ctx = l->ctx;
    iq_moe tmp = *l;
    tmp.d.gate = d.shared_gate_proj; tmp.d.up = d.shared_up; tmp.d.down = d.shared_down;
    tmp.d.d_ff = d.shared_up.n;
    tmp.d.expert_lo = 0; tmp.d.expert_count = 1;
    tmp.d.gate_bias = nullptr; tmp.d.up_bias = nullptr; tmp.d.down_bias = nullptr;
    const bool gated = d.shared == IQ_SHARED_GATED;
    shared_gate_kernel<<<(tokens + 3) / 4, 128, 0, cs>>>(
        x, x_dtype, ldx, gated ? static_cast<const uint32_t*>(d.shared_gate.w) : nullptr,
        static_cast<const uint16_t*>(d.shared_gate.scales), static_cast<const uint16_t*>(d.shared_gate.biases), w.s_w, tokens,
        d.d_model);
    int32_t st = check_cuda(ctx, cudaGetLastError(), "shared_gate launch");
    if (st != kOk) return st;
    const int32_t ydt = yd_dtype_of(l);
    if (use_tensor_path(tokens, 1)) {
        const int bn = tensor_tile_rows(tokens, 1);
        const size_t units = (size_t)tokens * d.d_model / 8;
        rows_to_f16_kernel<<<(unsigned)((units + 255) / 256), 256, 0, cs>>>(x, x_dtype, ldx, w.s_x16, tokens, d.d_model);
        shared_tiles_kernel<<<1, 128, 0, cs>>>(tokens, bn, 0u, w.s_tiles, w.s_ntiles);
        st = check_cuda(ctx, cudaGetLastError(), "shared tiles launch");
        if (st == kOk) st = run_gateup_tc(&tmp, cs, w.s_x16, tokens, w.s_tiles, w.s_ntiles, w.s_h, bn);
        if (st == kOk) st = run_down_tc(&tmp, cs, w.s_h, tokens, w.s_tiles, w.s_ntiles, w.s_yd, ydt, bn);
    } else {
        const int bm = 16;
        shared_tiles_kernel<<<1, 128, 0, cs>>>(tokens, bm, 0u, w.s_tiles, w.s_ntiles);
        st = check_cuda(ctx, cudaGetLastError(), "shared tiles launch");
        const int max_tiles = (tokens + bm - 1) / bm;
        if (st == kOk) st = run_gateup(&tmp, cs, x, x_dtype, ldx, nullptr, w.s_tiles, w.s_ntiles, max_tiles, bm, w.s_h);
        if (st == kOk) st = run_down(&tmp, cs, w.s_h, w.s_tiles, w.s_ntiles, max_tiles, bm, w.s_yd, ydt);
    }
    if (st != kOk) return st;
    shared_add_kernel<<<tokens, 256, 0, cs>>>(w.s_yd, ydt, w.s_w, out, out_dtype, ldo, tokens, d.d_model);
    return check_cuda(ctx, cudaGetLastError(), "shared_add launch");
}

// The experts' kernels wrote yd; the rows then go where the caller's table points (peer memory included).
int32_t scatter_rows(iq_ctx* ctx, cudaStream_t cs, const void* yd, void* const* yd_rows, int max_rows, int d_model,
                     int32_t yd_dtype) {
    const int row_bytes = d_model * (yd_dtype == kF32 ? 4 : 2);
    const int want = (max_rows + 3) / 4, cap = ctx->sms * 8;
    moe_scatter_rows_kernel<<<want < cap ? want : cap, 256, 0, cs>>>(yd, reinterpret_cast<const uint64_t*>(yd_rows), max_rows, row_bytes);
    return check_cuda(ctx, cudaGetLastError(), "moe_scatter_rows launch");
}

}  // namespace

int32_t moe_init(iq_ctx* ctx) {
    cudaFuncSetAttribute(reinterpret_cast<const void*>(router_logits_tiled_kernel<0, 64>),
                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)router_tiled_smem(64));
    cudaFuncSetAttribute(reinterpret_cast<const void*>(router_logits_tiled_kernel<1, 64>),
                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)router_tiled_smem(64));
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(router_logits_kernel<0>),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kRouterSmemMax);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(reinterpret_cast<const void*>(router_logits_kernel<1>),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kRouterSmemMax);
    return check_cuda(ctx, e, "cudaFuncSetAttribute(router)");
}

// ---------------------------------------------------------------------------------------------------------------------
// Elementwise gated activation of the dense FFN GEMM path: h[r, i] = half(act(gu[r, i], gu[r, d_ff + i]))
// (dswiglu_hh of the reference, Shaders/yy_model.metal:187-227).
__global__ void dswiglu_kernel(const float* __restrict__ gu, __half* __restrict__ h, int rows, int d_ff, int act,
                               float limit) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * d_ff) return;
    const size_t r = i / d_ff, c = i % d_ff;
    const float g = gu[r * 2 * d_ff + c], u = gu[r * 2 * d_ff + d_ff + c];
    h[i] = __float2half_rn(glu_rt(act, g, u, limit));
}

}  // namespace iq

using namespace iq;

// ---------------------------------------------------------------------------------------------------------------------
// dense FFN

extern "C" int32_t iq_dense_ffn_workspace_bytes(iq_ctx* ctx, const iq_qlinear* gate_up, const iq_qlinear* down,
                                                int32_t rows, int32_t x_dtype, size_t* bytes) {
    if (ctx == nullptr || gate_up == nullptr || down == nullptr || bytes == nullptr) return kErrInvalidArg;
    if (gate_up->n % 2 != 0 || gate_up->n / 2 != down->k || gate_up->k != down->n)
        return fail(ctx, kErrInvalidArg, "dense_ffn: gate|up [%d, %d] and down [%d, %d] do not chain", gate_up->n,
                    gate_up->k, down->n, down->k);
    const size_t d_ff = down->k;
    size_t total = round_up_sz((size_t)rows * d_ff * 2, 256);  // h fp16
    if (rows > 16) {
        size_t q = 0;
        int32_t st = iq_qmm_workspace_bytes(ctx, gate_up, rows, x_dtype, &q);
        if (st != kOk) return st;
        total += round_up_sz((size_t)rows * 2 * d_ff * 4, 256) + round_up_sz(q, 256);  // gate|up fp32 + qmm scratch
    }
    *bytes = total;
    return kOk;
}

extern "C" int32_t iq_dense_ffn(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx,
                                const iq_qlinear* gate_up, const iq_qlinear* down, int32_t act, float act_limit, void* out,
                                int32_t out_dtype, int64_t ldo, int32_t rows, uint32_t flags, void* workspace,
                                size_t workspace_bytes) {
    size_t need = 0;
    int32_t st = iq_dense_ffn_workspace_bytes(ctx, gate_up, down, rows, x_dtype, &need);
    if (st != kOk) return st;
    if (workspace == nullptr || workspace_bytes < need)
        return fail(ctx, kErrWorkspace, "dense_ffn: workspace %zu < %zu", workspace_bytes, need);
    if (act < IQ_ACT_SILU || act > IQ_ACT_RELU2) return fail(ctx, kErrUnsupported, "dense_ffn: activation %d", act);
    const int32_t fmt = format_of(gate_up);
    if (fmt < 0 || format_of(down) < 0) return fail(ctx, kErrUnsupported, "dense_ffn: weight format");
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    const int d_ff = down->k;
    __half* h = static_cast<__half*>(workspace);
    if (rows <= 16) {
        if (rows < 1) return fail(ctx, kErrInvalidArg, "dense_ffn: rows = %d", rows);
        if (d_ff % 16 != 0 || gate_up->k % 64 != 0 || ldx % 8 != 0)
            return fail(ctx, kErrInvalidArg, "dense_ffn: shapes (d_ff %% 16, d %% 64, ldx %% 8)");
        // gate and up rows of the concatenated matrix feed one fused gate+up+activation launch
        const size_t row_words = (size_t)gate_up->k / 32 * gate_up->bits;
        const size_t row_groups = (size_t)gate_up->k / gate_up->group;
        const size_t sbytes = fmt == kFmtMxfp4 ? 1 : 2;
        GqmvCall c;
        c.mode = kModeGateUp;
        c.fmt = fmt;
        c.w[0] = static_cast<const uint32_t*>(gate_up->w);
        c.w[1] = c.w[0] + (size_t)d_ff * row_words;
        c.s[0] = gate_up->scales;
        c.s[1] = static_cast<const char*>(gate_up->scales) + (size_t)d_ff * row_groups * sbytes;
        c.b[0] = gate_up->biases;
        c.b[1] = gate_up->biases ? static_cast<const char*>(gate_up->biases) + (size_t)d_ff * row_groups * 2 : nullptr;
        c.N = d_ff; c.K = gate_up->k;
        c.x = x; c.x_dtype = x_dtype; c.ldx = ldx;
        c.rows = rows; c.max_rows = rows;
        c.y = h; c.y_dtype = kF16; c.ldy = d_ff;
        c.limit = act == IQ_ACT_SWIGLU_OAI ? act_limit : 0.f;
        c.act = act;
        st = launch_gqmv(ctx, cs, c);
        if (st != kOk) return st;
        return iq_qmv(ctx, stream, h, IQ_F16, d_ff, down, out, out_dtype, ldo, rows, flags, 0);
    }
    if (fmt == kFmtAffine4 || fmt == kFmtMxfp4) {
        // GEMM path, fused: the gate and the up rows of the concatenated matrix are the two weight tiles of one stage of
        // the tcgen05 kernel, whose epilogue applies the activation and writes h = half(act(gate x, up x)) directly
        // (dswiglu_hh of the reference, Shaders/yy_model.metal:187-227, without the fp32 gate|up round trip: at
        // rows = 2048, d_ff = 14336 that is 235 MB not written and read back); then the down GEMM.
        if (rows % 64 != 0 || d_ff % 64 != 0 || gate_up->k % 64 != 0)
            return fail(ctx, kErrInvalidArg, "dense_ffn: rows = %d, d_ff = %d, d = %d must be multiples of 64", rows, d_ff, gate_up->k);
        char* q = static_cast<char*>(workspace) + round_up_sz((size_t)rows * d_ff * 2, 256);
        const void* x16 = x;
        int64_t ld16 = ldx;
        if (x_dtype != IQ_F16) {
            if (ldx < gate_up->k || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
                return fail(ctx, kErrInvalidArg, "dense_ffn: x must be 16-byte aligned with ldx >= d and ldx %% 8 == 0");
            const size_t units = (size_t)rows * gate_up->k / 8;
            rows_to_f16_kernel<<<(unsigned)((units + 255) / 256), 256, 0, cs>>>(x, x_dtype, ldx, reinterpret_cast<__half*>(q), rows,
                                                                               gate_up->k);
            st = check_cuda(ctx, cudaGetLastError(), "rows_to_f16 launch");
            if (st != kOk) return st;
            x16 = q;
            ld16 = gate_up->k;
        }
        const size_t row_words = (size_t)gate_up->k / 32 * gate_up->bits;
        const size_t row_groups = (size_t)gate_up->k / gate_up->group;
        const size_t sbytes = fmt == kFmtMxfp4 ? 1 : 2;
        QmmCall c;
        c.fmt = fmt; c.epi = 1; c.bn = rows >= 256 ? 256 : 128;
        c.x16 = x16; c.ldx = ld16; c.x_rows = rows;
        c.w[0] = gate_up->w;
        c.w[1] = static_cast<const uint32_t*>(gate_up->w) + (size_t)d_ff * row_words;
        c.s[0] = gate_up->scales;
        c.s[1] = static_cast<const char*>(gate_up->scales) + (size_t)d_ff * row_groups * sbytes;
        c.b[0] = gate_up->biases;
        c.b[1] = gate_up->biases ? static_cast<const char*>(gate_up->biases) + (size_t)d_ff * row_groups * 2 : nullptr;
        c.experts = 1;
        c.N = d_ff; c.K = gate_up->k; c.M = rows;
        c.y = h; c.y_dtype = kF16; c.ldy = d_ff;
        c.limit = act == IQ_ACT_SWIGLU_OAI ? act_limit : 0.f;
        c.act = act;
        st = launch_qmm(ctx, cs, c);
        if (st != kOk) return st;
        return iq_qmm(ctx, stream, h, IQ_F16, d_ff, down, out, out_dtype, ldo, rows, flags, nullptr, 0);
    }
    // other formats (8-bit, 4-bit g32): gate|up GEMM -> activation -> down GEMM
    char* p = static_cast<char*>(workspace) + round_up_sz((size_t)rows * d_ff * 2, 256);
    float* gu = reinterpret_cast<float*>(p);
    p += round_up_sz((size_t)rows * 2 * d_ff * 4, 256);
    const size_t qbytes = workspace_bytes - (p - static_cast<char*>(workspace));
    st = iq_qmm(ctx, stream, x, x_dtype, ldx, gate_up, gu, IQ_F32, 2 * d_ff, rows, 0, p, qbytes);
    if (st != kOk) return st;
    const size_t total = (size_t)rows * d_ff;
    dswiglu_kernel<<<(unsigned)((total + 255) / 256), 256, 0, cs>>>(gu, h, rows, d_ff, act, act_limit);
    st = check_cuda(ctx, cudaGetLastError(), "dswiglu launch");
    if (st != kOk) return st;
    return iq_qmm(ctx, stream, h, IQ_F16, d_ff, down, out, out_dtype, ldo, rows, flags, p, qbytes);
}

// ---------------------------------------------------------------------------------------------------------------------
// MoE

extern "C" int32_t iq_moe_create(iq_ctx* ctx, const iq_moe_desc* d, iq_moe** out) {
    if (ctx == nullptr || d == nullptr || out == nullptr) return kErrInvalidArg;
    *out = nullptr;
    // the reference's load guards (Layers/MoE.swift:186-219, Layers/MoEPrefill.swift:129-142)
    if (d->experts <= 0 || d->experts % 32 != 0 || d->experts > 512)
        return fail(ctx, kErrUnsupported, "moe: experts = %d (a multiple of 32, at most 512)", d->experts);
    if (d->top_k < 1 || d->top_k > 16 || d->top_k > d->experts)
        return fail(ctx, kErrUnsupported, "moe: top_k = %d (1..16)", d->top_k);
    if (d->d_ff <= 0 || d->d_ff % 64 != 0) return fail(ctx, kErrUnsupported, "moe: d_ff = %d (a multiple of 64)", d->d_ff);
    if (d->d_model < 128 || d->d_model % 64 != 0)
        return fail(ctx, kErrUnsupported, "moe: d_model = %d (a multiple of 64, at least 128)", d->d_model);
    if (d->act < IQ_ACT_SILU || d->act > IQ_ACT_RELU2) return fail(ctx, kErrUnsupported, "moe: activation %d", d->act);
    if (d->router_score != IQ_SCORE_SOFTMAX && d->router_score != IQ_SCORE_SIGMOID)
        return fail(ctx, kErrUnsupported, "moe: router score %d", d->router_score);
    if (d->router_kind != IQ_ROUTER_BF16 && d->router_kind != IQ_ROUTER_Q8)
        return fail(ctx, kErrUnsupported, "moe: router kind %d (bf16 or 8-bit g64; a 4-bit router is not supported)",
                    d->router_kind);
    if (d->router_w == nullptr || (d->router_kind == IQ_ROUTER_Q8 && (!d->router_scales || !d->router_biases)))
        return fail(ctx, kErrInvalidArg, "moe: router tensors missing");
    const int32_t fg = format_of(&d->gate), fu = format_of(&d->up), fd = format_of(&d->down);
    if (fg != fu || fg != fd || (fg != kFmtAffine4 && fg != kFmtMxfp4))
        return fail(ctx, kErrUnsupported, "moe: experts must be all affine 4-bit g64 or all mxfp4");
    if (d->gate.n != d->d_ff || d->gate.k != d->d_model || d->up.n != d->d_ff || d->up.k != d->d_model ||
        d->down.n != d->d_model || d->down.k != d->d_ff)
        return fail(ctx, kErrInvalidArg, "moe: expert tensor shapes do not match d_model/d_ff");
    if (d->expert_lo < 0 || d->expert_count < 1 || d->expert_lo + d->expert_count > d->experts ||
        d->gate.experts != d->expert_count || d->up.experts != d->expert_count || d->down.experts != d->expert_count)
        return fail(ctx, kErrInvalidArg, "moe: expert range [%d, %d) vs %d stacked experts", d->expert_lo,
                    d->expert_lo + d->expert_count, d->gate.experts);
    if (!d->gate.w || !d->up.w || !d->down.w || !d->gate.scales || !d->up.scales || !d->down.scales)
        return fail(ctx, kErrInvalidArg, "moe: expert tensors missing");
    if (fg != kFmtMxfp4 && (!d->gate.biases || !d->up.biases || !d->down.biases))
        return fail(ctx, kErrInvalidArg, "moe: affine experts without biases");
    if ((d->gate_bias != nullptr) != (d->up_bias != nullptr))
        return fail(ctx, kErrInvalidArg, "moe: gate and up expert biases go together");
    if (d->shared != IQ_SHARED_NONE) {
        // the reference's load guards (MoE.swift:186-219, MoEPrefill.swift:129-141): 4-bit affine shared expert, 8-bit
        // gate, width a multiple of 64, no shared expert beside MXFP4 experts
        if (d->shared != IQ_SHARED_GATED && d->shared != IQ_SHARED_UNGATED)
            return fail(ctx, kErrUnsupported, "moe: shared expert kind %d", d->shared);
        if (fg == kFmtMxfp4) return fail(ctx, kErrUnsupported, "moe: MXFP4 experts have no shared expert");
        if (format_of(&d->shared_gate_proj) != kFmtAffine4 || format_of(&d->shared_up) != kFmtAffine4 ||
            format_of(&d->shared_down) != kFmtAffine4)
            return fail(ctx, kErrUnsupported, "moe: the shared expert must be 4-bit affine g64 (got %d/%d/%d bits)",
                        d->shared_gate_proj.bits, d->shared_up.bits, d->shared_down.bits);
        const int si = d->shared_up.n;
        if (si < 64 || si % 64 != 0 || d->shared_gate_proj.n != si || d->shared_up.k != d->d_model ||
            d->shared_gate_proj.k != d->d_model || d->shared_down.n != d->d_model || d->shared_down.k != si ||
            d->shared_up.experts != 1 || d->shared_gate_proj.experts != 1 || d->shared_down.experts != 1)
            return fail(ctx, kErrInvalidArg, "moe: shared expert shapes (width %d)", si);
        if (!d->shared_gate_proj.w || !d->shared_up.w || !d->shared_down.w || !d->shared_gate_proj.biases ||
            !d->shared_up.biases || !d->shared_down.biases)
            return fail(ctx, kErrInvalidArg, "moe: shared expert tensors missing");
        if (d->shared == IQ_SHARED_GATED &&
            (format_of(&d->shared_gate) != kFmtAffine8 || d->shared_gate.n != 1 || d->shared_gate.k != d->d_model ||
             !d->shared_gate.w || !d->shared_gate.scales || !d->shared_gate.biases))
            return fail(ctx, kErrUnsupported, "moe: the shared expert's gate must be 8-bit affine g64 [1, d_model]");
    }
    iq_moe* l = new (std::nothrow) iq_moe();
    if (l == nullptr) return kErrCuda;
    l->ctx = ctx;
    l->d = *d;
    l->fmt = fg;
    l->ld = round_up(d->experts, 64);
    if (d->router_kind == IQ_ROUTER_BF16 && d->router_score == IQ_SCORE_SOFTMAX && d->experts % 64 == 0) {
        // set-up time (this call takes no stream): the largest row norm of the router, for the error bound of the
        // tensor-core logits. The router tensor must be complete on the device when the layer is created.
        uint32_t* dmax = nullptr;
        cudaError_t e = cudaMalloc(&dmax, 4);
        if (e == cudaSuccess) e = cudaMemset(dmax, 0, 4);
        if (e == cudaSuccess) {
            router_wnorm_max_kernel<<<d->experts, 256>>>(static_cast<const uint16_t*>(d->router_w), d->d_model, dmax);
            e = cudaGetLastError();
        }
        uint32_t bits = 0;
        if (e == cudaSuccess) e = cudaMemcpy(&bits, dmax, 4, cudaMemcpyDeviceToHost);
        if (dmax) cudaFree(dmax);
        if (e != cudaSuccess) {
            delete l;
            return check_cuda(ctx, e, "moe: router norm");
        }
        float f;
        memcpy(&f, &bits, 4);
        if (f > 0.f && f < 3.0e38f) l->router_wnorm_max = f;  // otherwise (zero or non-finite router): the float64 path
    }
    *out = l;
    return kOk;
}

extern "C" void iq_moe_destroy(iq_moe* l) { delete l; }

extern "C" int32_t iq_moe_workspace_bytes(const iq_moe* l, int32_t max_tokens, size_t* bytes) {
    if (l == nullptr || bytes == nullptr || max_tokens < 1) return kErrInvalidArg;
    *bytes = carve(l, nullptr, max_tokens).bytes;
    return kOk;
}

extern "C" int32_t iq_moe_get_views(const iq_moe* l, void* workspace, int32_t tokens, iq_moe_views* v) {
    if (l == nullptr || workspace == nullptr || v == nullptr || tokens < 1) return kErrInvalidArg;
    MoeWs w = carve(l, workspace, tokens);
    v->logits = w.logits; v->ld = l->ld;
    v->inds = l->ext_inds ? const_cast<uint32_t*>(l->ext_inds) : w.inds;
    v->wts = l->ext_wts ? const_cast<float*>(l->ext_wts) : w.wts;
    v->offsets = w.offsets; v->row_map = w.row_map; v->pos = w.pos;
    v->h = w.h; v->yd = w.yd; v->yd_dtype = yd_dtype_of(l);
    return kOk;
}

extern "C" int32_t iq_moe_set_external_routing(iq_moe* l, const uint32_t* inds, const float* wts) {
    if (l == nullptr || ((inds == nullptr) != (wts == nullptr))) return kErrInvalidArg;
    l->ext_inds = inds;
    l->ext_wts = wts;
    return kOk;
}

extern "C" int32_t iq_moe_route(iq_moe* l, void* stream, const float* logits, int32_t ld, int32_t tokens, uint32_t* inds,
                                float* wts) {
    if (l == nullptr) return kErrInvalidArg;
    if (logits == nullptr || inds == nullptr || wts == nullptr || tokens < 1 || ld < l->d.experts)
        return fail(l->ctx, kErrInvalidArg, "moe_route: arguments");
    return launch_route(l, reinterpret_cast<cudaStream_t>(stream), logits, ld, tokens, inds, wts);
}

extern "C" int32_t iq_moe_forward(iq_moe* l, void* stream, const void* x, int32_t x_dtype, int64_t ldx, void* out,
                                  int32_t out_dtype, int64_t ldo, int32_t tokens, uint32_t flags, uint32_t pieces,
                                  void* workspace, size_t workspace_bytes) {
    if (l == nullptr) return kErrInvalidArg;
    iq_ctx* ctx = l->ctx;
    const iq_moe_desc& d = l->d;
    if (tokens < 1) return fail(ctx, kErrInvalidArg, "moe: tokens = %d", tokens);
    if (x_dtype < 0 || x_dtype > 2 || out_dtype < 0 || out_dtype > 2) return fail(ctx, kErrInvalidArg, "moe: dtype");
    if ((pieces & (IQ_PIECE_ROUTER | IQ_PIECE_ROUTE | IQ_PIECE_GATEUP)) && (x != nullptr || (pieces & (IQ_PIECE_ROUTER | IQ_PIECE_GATEUP))) &&
        (x == nullptr || ldx < d.d_model || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0))
        return fail(ctx, kErrInvalidArg, "moe: x must be 16-byte aligned with ldx >= d_model and ldx %% 8 == 0");
    if ((pieces & IQ_PIECE_COMBINE) && (out == nullptr || ldo < d.d_model || ldo % 4 != 0))
        return fail(ctx, kErrInvalidArg, "moe: out / ldo");
    MoeWs w = carve(l, workspace, tokens);
    if (workspace == nullptr || workspace_bytes < w.bytes)
        return fail(ctx, kErrWorkspace, "moe: workspace %zu < %zu", workspace_bytes, w.bytes);
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    const int P = tokens * d.top_k;
    const uint32_t* inds = l->ext_inds ? l->ext_inds : w.inds;
    const float* wts = l->ext_wts ? l->ext_wts : w.wts;
    int32_t st;

    const bool fast_router = tensor_router(l, tokens, x_dtype);
    if ((pieces & IQ_PIECE_ROUTER) && fast_router) {
        QmmCall c;
        c.fmt = kFmtBf16Plain; c.epi = 0; c.bn = 128;
        // one CTA per (token tile, 128 experts): narrower token tiles until the grid covers the GPU (4096 tokens and 128
        // experts: 32 CTAs of 128 tokens took 21 us, the K loop's latency; 128 CTAs of 32 tokens run it side by side)
        while (c.bn > 32 && ((tokens + c.bn - 1) / c.bn) * ((d.experts + 127) / 128) < ctx->sms) c.bn /= 2;
        c.x16 = x; c.ldx = ldx; c.x_rows = tokens;
        c.w[0] = d.router_w;
        c.experts = 1;
        c.N = d.experts; c.K = d.d_model; c.M = tokens;
        c.y = w.logits; c.y_dtype = kF32; c.ldy = l->ld;
        st = launch_qmm(ctx, cs, c);
        if (st != kOk) return st;
    } else if ((pieces & IQ_PIECE_ROUTER) && l->ext_inds == nullptr) {
        if (tokens > kRouterTiledMinTokens && d.d_model % 64 == 0) {
            // register-tiled float64 GEMM; the K range is split over a cluster until the grid fills the GPU several
            // times over (the blocks of one SM share its float64 pipe, so balance comes from many small blocks)
            const int bm = tokens >= 1024 ? 64 : 32;
            const int tiles = ((tokens + bm - 1) / bm) * ((d.experts + kRtBN - 1) / kRtBN);
            const int nchunks = d.d_model / kRtBK;
            int S = 1;
            while (tiles * S < 4 * ctx->sms && S < 8 && nchunks / (2 * S) >= 2) S *= 2;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((tokens + bm - 1) / bm, (d.experts + kRtBN - 1) / kRtBN, S);
            cfg.blockDim = dim3(128);
            cfg.dynamicSmemBytes = router_tiled_smem(bm);
            cfg.stream = cs;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = S;
            cfg.attrs = at; cfg.numAttrs = 1;
            const int cps = (nchunks + S - 1) / S;
            const bool q8 = d.router_kind != IQ_ROUTER_BF16;
            const void* rw = d.router_w;
            const void* rs = q8 ? d.router_scales : nullptr;
            const void* rb = q8 ? d.router_biases : nullptr;
            auto kern = bm == 64 ? (q8 ? router_logits_tiled_kernel<1, 64> : router_logits_tiled_kernel<0, 64>)
                                 : (q8 ? router_logits_tiled_kernel<1, 32> : router_logits_tiled_kernel<0, 32>);
            st = check_cuda(ctx, cudaLaunchKernelEx(&cfg, kern, x, x_dtype, ldx, rw, rs, rb, w.logits, tokens, d.experts,
                                                    d.d_model, l->ld, cps),
                            "router_logits_tiled launch");
            if (st != kOk) return st;
        } else {
        // experts per block: small ranges for few tokens (more blocks, shorter dot products per thread)
        int eb = d.experts < 256 ? d.experts : 256;
        if (tokens <= 64) eb = 8;  // a decode batch: 256 blocks of 8 experts x 32 K slices fill the GPU (20 -> 10 us at 64 tokens)
        else if (tokens <= 256 && eb > 32) eb = 32;
        while (d.experts % eb != 0) eb /= 2;
        const size_t smem = (size_t)kRouterTT * d.d_model * 8 + (size_t)256 * kRouterTT * 8;
        if (smem > (size_t)kRouterSmemMax) return fail(ctx, kErrUnsupported, "moe: d_model = %d is too wide for the router kernel", d.d_model);
        const dim3 grid((tokens + kRouterTT - 1) / kRouterTT, d.experts / eb);
        if (d.router_kind == IQ_ROUTER_BF16)
            router_logits_kernel<0><<<grid, 256, smem, cs>>>(x, x_dtype, ldx, d.router_w, nullptr, nullptr, w.logits,
                                                              tokens, d.experts, d.d_model, l->ld, eb);
        else
            router_logits_kernel<1><<<grid, 256, smem, cs>>>(x, x_dtype, ldx, d.router_w, d.router_scales,
                                                              d.router_biases, w.logits, tokens, d.experts, d.d_model,
                                                              l->ld, eb);
        }
        st = check_cuda(ctx, cudaGetLastError(), "router_logits launch");
        if (st != kOk) return st;
    }
    if ((pieces & IQ_PIECE_ROUTE) && l->ext_inds == nullptr) {
        if (fast_router && x == nullptr) return fail(ctx, kErrInvalidArg, "moe: the route piece needs x (it recomputes logits)");
        st = launch_route(l, cs, w.logits, l->ld, tokens, w.inds, w.wts, fast_router ? x : nullptr, ldx);
        if (st != kOk) return st;
    }
    const int bm = decode_tile_rows(l, tokens);
    if (pieces & IQ_PIECE_GROUP) {
        GroupParams gp;
        gp.inds = inds; gp.counts = w.counts; gp.offsets = w.offsets; gp.row_map = w.row_map; gp.pos = w.pos;
        gp.tiles_a = w.tiles_a; gp.tiles_b = w.tiles_b; gp.ntiles = w.ntiles;
        gp.P = P; gp.E = d.experts; gp.bm_a = bm; gp.bm_b = tensor_tile_rows(P, d.expert_count);
        gp.e_lo = d.expert_lo; gp.e_hi = d.expert_lo + d.expert_count;
        gp.chunk_hist = w.chunk_hist;
        gp.chunks = (P + kGroupChunk - 1) / kGroupChunk;
        if (P >= kGroupChunkedMinPairs && d.experts * 8 * 4 <= 48 * 1024) {
            // many pairs: a chunked counting sort touches each pair once per kernel instead of once per expert
            moe_hist_kernel<<<gp.chunks, 256, d.experts * 4, cs>>>(gp);
            moe_scan_kernel<<<1, 256, 0, cs>>>(gp);
            moe_place_kernel<<<gp.chunks, 256, d.experts * 8 * 4, cs>>>(gp);
        } else {
            moe_count_kernel<<<d.experts, 256, 0, cs>>>(gp);
            moe_scatter_kernel<<<d.experts, 256, 0, cs>>>(gp);
        }
        st = check_cuda(ctx, cudaGetLastError(), "moe_group launch");
        if (st != kOk) return st;
    }
    const int64_t max_tiles64 = (int64_t)d.expert_count + P / bm;
    const int max_tiles = (int)(max_tiles64 < P ? max_tiles64 : P);
    if (max_tiles > 65535 && !use_tensor_path(P, d.expert_count))
        return fail(ctx, kErrInvalidArg, "moe: %d tokens give too many tiles for one launch", tokens);
    const bool tc = use_tensor_path(P, d.expert_count);
    if (pieces & IQ_PIECE_GATEUP) {
        if (tc) {
            // The GEMM's producer fetches each tile's token rows through row_map (the reference gathers through rowMap
            // too, Shaders/qmm_nax_moe.metal:512-586): nothing is packed in expert order. It needs fp16 rows: fp16
            // activations are used in place, others are converted once per token (not once per routed pair).
            const __half* x16 = static_cast<const __half*>(x);
            int64_t ld16 = ldx;
            st = kOk;
            if (x_dtype != kF16) {
                const size_t units = (size_t)tokens * d.d_model / 8;
                rows_to_f16_kernel<<<(unsigned)((units + 255) / 256), 256, 0, cs>>>(x, x_dtype, ldx, w.xs, tokens, d.d_model);
                st = check_cuda(ctx, cudaGetLastError(), "rows_to_f16 launch");
                x16 = w.xs;
                ld16 = d.d_model;
            }
            if (st == kOk)
                st = run_gateup_tc(l, cs, x16, P, w.tiles_b, w.ntiles + 1, w.h, tensor_tile_rows(P, d.expert_count), w.row_map,
                                   (uint32_t)d.top_k, ld16, tokens);
        } else {
            st = run_gateup(l, cs, x, x_dtype, ldx, w.row_map, w.tiles_a, w.ntiles, max_tiles, bm, w.h);
        }
        if (st != kOk) return st;
    }
    if (pieces & IQ_PIECE_DOWN) {
        st = tc ? run_down_tc(l, cs, w.h, P, w.tiles_b, w.ntiles + 1, w.yd, yd_dtype_of(l), tensor_tile_rows(P, d.expert_count))
                : run_down(l, cs, w.h, w.tiles_a, w.ntiles, max_tiles, bm, w.yd, yd_dtype_of(l));
        if (st != kOk) return st;
    }
    if (pieces & IQ_PIECE_COMBINE) {
        CombineParams cp;
        cp.yd = w.yd; cp.yd_dtype = yd_dtype_of(l); cp.pos = w.pos; cp.wts = wts;
        cp.out = out; cp.out_dtype = out_dtype; cp.ldo = ldo;
        cp.T = tokens; cp.D = d.d_model; cp.topk = d.top_k;
        cp.accumulate = (flags & IQ_FLAG_ACCUMULATE) ? 1 : 0;
        moe_combine_kernel<<<tokens, 256, 0, cs>>>(cp);
        st = check_cuda(ctx, cudaGetLastError(), "moe_combine launch");
        if (st != kOk) return st;
        if (d.shared != IQ_SHARED_NONE) {
            st = run_shared_expert(l, cs, x, x_dtype, ldx, tokens, w, out, out_dtype, ldo);
            if (st != kOk) return st;
        }
    }
    return kOk;
}

// ---------------------------------------------------------------------------------------------------------------------
// Expert-parallel pieces and the stack helper

extern "C" int32_t iq_moe_pack_rows(iq_moe* l, void* stream, const void* x, int32_t x_dtype, int64_t ldx, int32_t tokens,
                                    void* workspace, size_t workspace_bytes, void* rows_f16) {
    if (l == nullptr) return kErrInvalidArg;
    iq_ctx* ctx = l->ctx;
    const iq_moe_desc& d = l->d;
    if (tokens < 1 || x == nullptr || rows_f16 == nullptr || x_dtype < 0 || x_dtype > 2 || ldx < d.d_model || ldx % 8 != 0 ||
        (reinterpret_cast<uintptr_t>(x) & 15) != 0 || (reinterpret_cast<uintptr_t>(rows_f16) & 15) != 0)
        return fail(ctx, kErrInvalidArg, "moe_pack_rows: arguments");
    MoeWs w = carve(l, workspace, tokens);
    if (workspace == nullptr || workspace_bytes < w.bytes)
        return fail(ctx, kErrWorkspace, "moe_pack_rows: workspace %zu < %zu", workspace_bytes, w.bytes);
    const int P = tokens * d.top_k;
    moe_pack_rows_kernel<<<P, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, x_dtype, ldx, w.pos,
                                                                                static_cast<__half*>(rows_f16), P,
                                                                                d.d_model, d.top_k);
    return check_cuda(ctx, cudaGetLastError(), "moe_pack_rows launch");
}

namespace {
struct ExpertsWs {
    Tile* tiles;
    uint32_t* ntiles;
    __half* h;
    size_t bytes;
};
ExpertsWs carve_experts(const iq_moe* l, void* base, int max_rows, int sources) {
    size_t off = 0;
    auto take = [&](size_t bytes) {
        void* p = base ? static_cast<char*>(base) + off : nullptr;
        off += round_up_sz(bytes, 256);
        return p;
    };
    ExpertsWs w;
    w.tiles = static_cast<Tile*>(take(((size_t)max_rows / 8 + (size_t)sources * l->d.expert_count + 1) * sizeof(Tile)));
    w.ntiles = static_cast<uint32_t*>(take(16));
    w.h = static_cast<__half*>(take((size_t)max_rows * l->d.d_ff * 2));
    w.bytes = off;
    return w;
}
}  // namespace

extern "C" int32_t iq_moe_experts_workspace_bytes(const iq_moe* l, int32_t max_rows, int32_t sources, size_t* bytes) {
    if (l == nullptr || bytes == nullptr || max_rows < 1 || sources < 1 || sources > kMaxEpSources) return kErrInvalidArg;
    *bytes = carve_experts(l, nullptr, max_rows, sources).bytes;
    return kOk;
}

namespace {
int32_t moe_experts_impl(iq_moe* l, void* stream, const void* rows_f16, const uint32_t* row_index, int32_t total_rows,
                         int32_t max_rows, const uint32_t* counts, int32_t sources, int32_t region_rows, void* yd, int32_t yd_dtype,
                         void* const* yd_rows, void* workspace, size_t workspace_bytes);
}

extern "C" int32_t iq_moe_experts(iq_moe* l, void* stream, const void* rows_f16, int32_t total_rows, int32_t max_rows,
                                  const uint32_t* counts, int32_t sources, int32_t region_rows, void* yd, int32_t yd_dtype,
                                  void* const* yd_rows, void* workspace, size_t workspace_bytes) {
    return moe_experts_impl(l, stream, rows_f16, nullptr, total_rows, max_rows, counts, sources, region_rows, yd, yd_dtype, yd_rows,
                            workspace, workspace_bytes);
}

extern "C" int32_t iq_moe_experts_indexed(iq_moe* l, void* stream, const void* rows_f16, const uint32_t* row_index,
                                          int32_t total_rows, int32_t max_rows, const uint32_t* counts, void* yd, int32_t yd_dtype,
                                          void* const* yd_rows, void* workspace, size_t workspace_bytes) {
    if (l != nullptr && row_index == nullptr) return fail(l->ctx, kErrInvalidArg, "moe_experts_indexed: row_index");
    return moe_experts_impl(l, stream, rows_f16, row_index, total_rows, max_rows, counts, 1, 0, yd, yd_dtype, yd_rows, workspace,
                            workspace_bytes);
}

namespace {
int32_t moe_experts_impl(iq_moe* l, void* stream, const void* rows_f16, const uint32_t* row_index, int32_t total_rows,
                         int32_t max_rows, const uint32_t* counts, int32_t sources, int32_t region_rows, void* yd, int32_t yd_dtype,
                         void* const* yd_rows, void* workspace, size_t workspace_bytes) {
    if (l == nullptr) return kErrInvalidArg;
    iq_ctx* ctx = l->ctx;
    const iq_moe_desc& d = l->d;
    if (rows_f16 == nullptr || counts == nullptr || yd == nullptr || sources < 1 || sources > kMaxEpSources ||
        sources * d.expert_count > 4096 ||
        total_rows < 0 || total_rows > max_rows || (yd_dtype != kF32 && yd_dtype != kF16) || region_rows < 0 ||
        (int64_t)region_rows * sources > max_rows ||
        (reinterpret_cast<uintptr_t>(rows_f16) & 15) != 0)
        return fail(ctx, kErrInvalidArg, "moe_experts: arguments");
    if (total_rows == 0) return kOk;
    ExpertsWs w = carve_experts(l, workspace, max_rows, sources);
    if (workspace == nullptr || workspace_bytes < w.bytes)
        return fail(ctx, kErrWorkspace, "moe_experts: workspace %zu < %zu", workspace_bytes, w.bytes);
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    const int64_t slots = (int64_t)sources * d.expert_count;
    if (use_tensor_path(total_rows, slots)) {
        const int bn = tensor_tile_rows(total_rows, slots);
        ep_tiles_kernel<<<1, 512, 0, cs>>>(counts, sources, d.experts, d.expert_lo, d.expert_count, bn, (uint32_t)region_rows, w.tiles,
                                           w.ntiles);
        int32_t st2 = check_cuda(ctx, cudaGetLastError(), "ep_tiles launch");
        // the row count is only known on the device: bounds come from the capacity, total_rows picks the kernels
        if (st2 == kOk)
            st2 = run_gateup_tc(l, cs, static_cast<const __half*>(rows_f16), max_rows, w.tiles, w.ntiles, w.h, bn, row_index, 1,
                                d.d_model, max_rows);
        if (st2 == kOk) st2 = run_down_tc(l, cs, w.h, max_rows, w.tiles, w.ntiles, yd, yd_dtype, bn);
        if (st2 == kOk && yd_rows != nullptr) st2 = scatter_rows(ctx, cs, yd, yd_rows, max_rows, d.d_model, yd_dtype);
        return st2;
    }
    const int bm = total_rows <= slots * 6 ? 8 : 16;
    ep_tiles_kernel<<<1, 512, 0, cs>>>(counts, sources, d.experts, d.expert_lo, d.expert_count, bm, (uint32_t)region_rows, w.tiles,
                                       w.ntiles);
    int32_t st = check_cuda(ctx, cudaGetLastError(), "ep_tiles launch");
    if (st != kOk) return st;
    const int64_t mt = max_rows / bm + slots;
    const int max_tiles = (int)(mt < max_rows ? mt : max_rows);
    if (max_tiles > 65535) return fail(ctx, kErrInvalidArg, "moe_experts: too many tiles for one launch");
    st = run_gateup(l, cs, rows_f16, kF16, d.d_model, row_index, w.tiles, w.ntiles, max_tiles, bm, w.h, 1);
    if (st != kOk) return st;
    st = run_down(l, cs, w.h, w.tiles, w.ntiles, max_tiles, bm, yd, yd_dtype);
    if (st != kOk || yd_rows == nullptr) return st;
    return scatter_rows(ctx, cs, yd, yd_rows, max_rows, d.d_model, yd_dtype);
}
}  // namespace

extern "C" int32_t iq_moe_combine_rows(iq_moe* l, void* stream, const void* yd_rows, int32_t yd_dtype, int32_t tokens,
                                       void* out, int32_t out_dtype, int64_t ldo, uint32_t flags, void* workspace,
                                       size_t workspace_bytes) {
    if (l == nullptr) return kErrInvalidArg;
    iq_ctx* ctx = l->ctx;
    const iq_moe_desc& d = l->d;
    if (yd_rows == nullptr || out == nullptr || tokens < 1 || (yd_dtype != kF32 && yd_dtype != kF16) || out_dtype < 0 ||
        out_dtype > 2 || ldo < d.d_model || ldo % 4 != 0)
        return fail(ctx, kErrInvalidArg, "moe_combine_rows: arguments");
    MoeWs w = carve(l, workspace, tokens);
    if (workspace == nullptr || workspace_bytes < w.bytes)
        return fail(ctx, kErrWorkspace, "moe_combine_rows: workspace %zu < %zu", workspace_bytes, w.bytes);
    CombineParams cp;
    cp.yd = yd_rows; cp.yd_dtype = yd_dtype; cp.pos = w.pos; cp.wts = l->ext_wts ? l->ext_wts : w.wts;
    cp.out = out; cp.out_dtype = out_dtype; cp.ldo = ldo;
    cp.T = tokens; cp.D = d.d_model; cp.topk = d.top_k;
    cp.accumulate = (flags & IQ_FLAG_ACCUMULATE) ? 1 : 0;
    moe_combine_kernel<<<tokens, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(cp);
    return check_cuda(ctx, cudaGetLastError(), "moe_combine launch");
}

extern "C" int32_t iq_rmsnorm(iq_ctx* ctx, void* stream, const float* x, int64_t ldx, void* out, int32_t out_dtype,
                              int64_t ldo, int32_t rows, int32_t d, float eps) {
    if (ctx == nullptr) return kErrInvalidArg;
    if (x == nullptr || out == nullptr || rows < 1 || d < 4 || d % 4 != 0 || ldx < d || ldo < d || ldx % 4 != 0 ||
        ldo % 4 != 0 || out_dtype < 0 || out_dtype > 2)
        return fail(ctx, kErrInvalidArg, "rmsnorm: arguments");
    rmsnorm_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, ldx, out, out_dtype, ldo, d, eps);
    return check_cuda(ctx, cudaGetLastError(), "rmsnorm launch");
}
