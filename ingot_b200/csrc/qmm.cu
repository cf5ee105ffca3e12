// Host side of the tcgen05 GEMM: tensor maps, kernel selection, the iq_qmm entry point.
#include "internal.h"
#include "qmm_tc.cuh"

namespace iq {

namespace {

typedef void (*QmmKernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const QmmParams);

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct KernelEntry {
    int32_t fmt;
    int bn;
    int epi;
    int act;
    bool gather;
    QmmKernel fn;
    int smem;
};

template <int FMT, int BN, int EPI, int ACT = kActSilu, bool GATHER = false>
KernelEntry entry() {
    return KernelEntry{FMT, BN, EPI, ACT, GATHER, qmm_tc_kernel<FMT, BN, EPI, ACT, GATHER>, QmmSmem<FMT, BN, EPI>::TOTAL};
}
// gate/up with the activation rows gathered by row index, both tile heights
template <int FMT, int ACT>
void gather_entries(KernelEntry* t, int* n) {
    t[(*n)++] = entry<FMT, 128, kEpiGateUp, ACT, true>();
    t[(*n)++] = entry<FMT, 256, kEpiGateUp, ACT, true>();
}

const KernelEntry* table(int* n) {
    static const KernelEntry fixed[] = {
        entry<kFmtAffine4, 256, kEpiStore>(), entry<kFmtAffine4, 128, kEpiStore>(),
        entry<kFmtAffine8, 256, kEpiStore>(), entry<kFmtAffine8, 128, kEpiStore>(),
        entry<kFmtMxfp4, 256, kEpiStore>(),   entry<kFmtMxfp4, 128, kEpiStore>(),
        entry<kFmtAffine4G32, 256, kEpiStore>(), entry<kFmtAffine4G32, 128, kEpiStore>(),
        entry<kFmtAffine4, 128, kEpiGateUp>(), entry<kFmtMxfp4, 128, kEpiGateUp>(),
        entry<kFmtAffine4, 256, kEpiGateUp>(), entry<kFmtMxfp4, 256, kEpiGateUp>(),
        entry<kFmtAffine4, 128, kEpiGateUp, kActSwigluOai>(), entry<kFmtMxfp4, 128, kEpiGateUp, kActSwigluOai>(),
        entry<kFmtAffine4, 256, kEpiGateUp, kActSwigluOai>(), entry<kFmtMxfp4, 256, kEpiGateUp, kActSwigluOai>(),
        entry<kFmtAffine4, 128, kEpiGateUp, kActGelu>(), entry<kFmtAffine4, 256, kEpiGateUp, kActGelu>(),
        entry<kFmtAffine4, 128, kEpiGateUp, kActRelu2>(), entry<kFmtAffine4, 256, kEpiGateUp, kActRelu2>(),
        entry<kFmtMxfp4, 128, kEpiGateUp, kActGelu>(), entry<kFmtMxfp4, 256, kEpiGateUp, kActGelu>(),
        entry<kFmtMxfp4, 128, kEpiGateUp, kActRelu2>(), entry<kFmtMxfp4, 256, kEpiGateUp, kActRelu2>(),
        // bf16 x bf16 (the router's approximate logits); the small token tiles spread few experts over many CTAs
        entry<kFmtBf16Plain, 128, kEpiStore>(), entry<kFmtBf16Plain, 64, kEpiStore>(), entry<kFmtBf16Plain, 32, kEpiStore>(),
        entry<kFmtTernary, 256, kEpiStore>(), entry<kFmtTernary, 128, kEpiStore>(),
        entry<kFmtInt8Plain, 256, kEpiStore>(), entry<kFmtInt8Plain, 128, kEpiStore>(),  // rotated W8A8
    };
    constexpr int kFixed = (int)(sizeof(fixed) / sizeof(fixed[0]));
    static KernelEntry t[kFixed + 16];
    static int count = 0;
    static std::once_flag once;
    std::call_once(once, [] {
        for (int i = 0; i < kFixed; i++) t[count++] = fixed[i];
        gather_entries<kFmtAffine4, kActSilu>(t, &count);
        gather_entries<kFmtAffine4, kActGelu>(t, &count);
        gather_entries<kFmtAffine4, kActSwigluOai>(t, &count);
        gather_entries<kFmtAffine4, kActRelu2>(t, &count);
        gather_entries<kFmtMxfp4, kActSilu>(t, &count);
        gather_entries<kFmtMxfp4, kActGelu>(t, &count);
        gather_entries<kFmtMxfp4, kActSwigluOai>(t, &count);
        gather_entries<kFmtMxfp4, kActRelu2>(t, &count);
    });
    *n = count;
    return t;
}

const KernelEntry* find(int32_t fmt, int bn, int epi, int act, bool gather) {
    int n;
    const KernelEntry* t = table(&n);
    if (epi != kEpiGateUp) act = kActSilu;
    for (int i = 0; i < n; i++)
        if (t[i].fmt == fmt && t[i].bn == bn && t[i].epi == epi && t[i].act == act && t[i].gather == gather) return &t[i];
    return nullptr;
}

}  // namespace

int32_t qmm_init(iq_ctx* ctx) {
    int n;
    const KernelEntry* t = table(&n);
    for (int i = 0; i < n; i++) {
        cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(t[i].fn),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, t[i].smem);
        if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(qmm)");
    }
    return kOk;
}

// 2-D tensor map over a row-major matrix: `inner` elements per row, `rows` rows, `row_bytes` between rows.
// elem: 0 = bytes, 1 = fp16, 2 = bf16 elements
int32_t make_map_2d(iq_ctx* ctx, CUtensorMap* map, const void* base, int elem, uint64_t inner, uint64_t rows,
                    uint64_t row_bytes, uint32_t box_inner, uint32_t box_rows, bool swizzle128) {
    if (ctx->encode_tiled == nullptr) return fail(ctx, kErrCuda, "cuTensorMapEncodeTiled is not available");
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || row_bytes % 16 != 0)
        return fail(ctx, kErrInvalidArg, "qmm: TMA needs a 16-byte aligned base and row pitch");
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
        map, elem == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : (elem == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8),
        2, const_cast<void*>(base), dims,
        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, kErrCuda, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return kOk;
}

int32_t make_map_rowblock(iq_ctx* ctx, CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                          uint32_t box_rows) {
    if (ctx->encode_tiled == nullptr) return fail(ctx, kErrCuda, "cuTensorMapEncodeTiled is not available");
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || row_bytes % 128 != 0 || row_bytes / 128 > 256 || rows < 1 || box_rows < 8 ||
        box_rows > 256 || box_rows % 8 != 0)
        return fail(ctx, kErrInvalidArg, "qmv: TMA needs a 16-byte aligned base and rows of 128..32768 bytes in 128-byte steps");
    const cuuint64_t dims[3] = {128, rows, row_bytes / 128};
    const cuuint64_t strides[2] = {row_bytes, 128};
    const cuuint32_t box[3] = {128, box_rows, (cuuint32_t)(row_bytes / 128)};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
        map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, kErrCuda, "cuTensorMapEncodeTiled (row block) failed (%d)", (int)r);
    return kOk;
}

int32_t cached_rowblock_map(iq_ctx* ctx, const void* base, int64_t rows, int32_t row_bytes, int32_t box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> hold(ctx->qmv_maps_lock);
    if (ctx->qmv_maps == nullptr) ctx->qmv_maps = new iq_ctx::QmvMap[iq_ctx::kQmvMaps];
    const uintptr_t key = reinterpret_cast<uintptr_t>(base);
    iq_ctx::QmvMap& e = ctx->qmv_maps[((key >> 8) ^ (key >> 20) ^ (uintptr_t)rows ^ (uintptr_t)box_rows) % iq_ctx::kQmvMaps];
    if (e.base != base || e.rows != rows || e.row_bytes != row_bytes || e.box_rows != box_rows) {
        e.base = nullptr;
        const int32_t r = make_map_rowblock(ctx, &e.map, base, (uint64_t)rows, (uint64_t)row_bytes, (uint32_t)box_rows);
        if (r != kOk) return r;
        e.base = base; e.rows = (int32_t)rows; e.row_bytes = row_bytes; e.box_rows = box_rows;
    }
    *out = e.map;
    return kOk;
}

int32_t launch_qmm(iq_ctx* ctx, cudaStream_t st, const QmmCall& c) {
    const KernelEntry* ke = find(c.fmt, c.bn, c.epi, c.act, c.gather_map != nullptr);
    if (ke == nullptr) return fail(ctx, kErrNoKernel, "qmm: no kernel for format %d, tile %d, epilogue %d", c.fmt, c.bn, c.epi);
    const bool i8 = c.fmt == kFmtInt8Plain;     // int8 rows on both sides, 128 inputs per K step
    const bool plain = c.fmt == kFmtBf16Plain;  // bf16 activations and bf16 weights, both copied as they are
    if (i8) {
        CUtensorMap ax, aw;
        int32_t ri = make_map_2d(ctx, &ax, c.x16, 0, (uint64_t)c.K, (uint64_t)c.x_rows, (uint64_t)c.ldx, 128, c.bn, true);
        if (ri == kOk) ri = make_map_2d(ctx, &aw, c.w[0], 0, (uint64_t)c.K, (uint64_t)c.N, (uint64_t)c.K, 128, kWRows, true);
        if (ri != kOk) return ri;
        QmmParams q = {};
        q.s[0] = q.s[1] = c.s[0]; q.b[0] = q.b[1] = c.b[0];
        q.N = c.N; q.K = c.K; q.M = c.M;
        q.y = c.y; q.y_dtype = c.y_dtype; q.ldy = c.ldy; q.accumulate = c.accumulate;
        q.limit = c.limit;
        q.status = ctx->d_status;
        const int work = ((c.M + c.bn - 1) / c.bn) * ((c.N + kWRows - 1) / kWRows);
        ke->fn<<<work < ctx->sms ? work : ctx->sms, kQmmThreads, ke->smem, st>>>(ax, aw, aw, q);
        return check_cuda(ctx, cudaGetLastError(), "qmm_i8 launch");
    }
    const int pack_row = c.fmt == kFmtAffine8 ? 64 : (c.fmt == kFmtTernary ? 16 : 32);
    const uint64_t row_bytes = (uint64_t)c.K / kBK * pack_row;
    CUtensorMap mx, mw0, mw1;
    int32_t r = make_map_2d(ctx, &mx, c.x16, plain ? 2 : 1, (uint64_t)c.K, (uint64_t)c.x_rows, (uint64_t)c.ldx * 2, kBK, c.bn, true);
    if (r != kOk) return r;
    if (plain) {
        r = make_map_2d(ctx, &mw0, c.w[0], 2, (uint64_t)c.K, (uint64_t)c.experts * c.N, (uint64_t)c.K * 2, kBK, kWRows, true);
        mw1 = mw0;
    } else {
        r = make_map_2d(ctx, &mw0, c.w[0], 0, row_bytes, (uint64_t)c.experts * c.N, row_bytes, pack_row, kWRows, false);
        if (r != kOk) return r;
        r = make_map_2d(ctx, &mw1, c.w[1] ? c.w[1] : c.w[0], 0, row_bytes, (uint64_t)c.experts * c.N, row_bytes, pack_row,
                        kWRows, false);
    }
    if (r != kOk) return r;
    QmmParams p;
    for (int i = 0; i < 2; i++) {
        p.s[i] = c.s[i] ? c.s[i] : c.s[0];
        p.b[i] = c.b[i] ? c.b[i] : c.b[0];
        p.ebias[i] = c.ebias[i];
    }
    p.expert_lo = c.expert_lo;
    p.N = c.N; p.K = c.K; p.M = c.M;
    p.tiles = c.tiles; p.ntiles = c.ntiles;
    p.y = c.y; p.y_dtype = c.y_dtype; p.ldy = c.ldy; p.accumulate = c.accumulate;
    p.limit = c.limit;
    p.xg = c.gather_map != nullptr ? static_cast<const __half*>(c.x16) : nullptr;
    p.gather_map = c.gather_map;
    p.ldxg = c.ldx;
    p.gather_div = c.gather_div;
    p.status = ctx->d_status;
    p.reserved = 0;
    int grid = ctx->sms;
    if (c.tiles == nullptr) {
        const int work = ((c.M + c.bn - 1) / c.bn) * ((c.N + kWRows - 1) / kWRows);
        if (work < grid) grid = work;
    }
    ke->fn<<<grid, c.gather_map != nullptr ? kQmmGatherThreads : kQmmThreads, ke->smem, st>>>(mx, mw0, mw1, p);
    return check_cuda(ctx, cudaGetLastError(), "qmm launch");
}

}  // namespace iq

using namespace iq;

extern "C" int32_t iq_qmm_workspace_bytes(iq_ctx* ctx, const iq_qlinear* m, int32_t rows, int32_t x_dtype, size_t* bytes) {
    if (ctx == nullptr || m == nullptr || bytes == nullptr || rows < 1) return kErrInvalidArg;
    // The MMA takes fp16 weights with fp16 activations only (a bf16 B operand beside an fp16 A operand is an illegal
    // instruction on sm_100a: kind::f16 wants both operands of one type), so bf16 and fp32 activations are converted
    *bytes = x_dtype == IQ_F16 ? 0 : round_up_sz((size_t)rows * m->k * 2, 256);
    return kOk;
}

extern "C" int32_t iq_qmm(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* m,
                          void* y, int32_t y_dtype, int64_t ldy, int32_t rows, uint32_t flags, void* workspace,
                          size_t workspace_bytes) {
    if (ctx == nullptr) return kErrInvalidArg;
    if (x == nullptr || y == nullptr || m == nullptr || m->w == nullptr || m->scales == nullptr)
        return fail(ctx, kErrInvalidArg, "qmm: null pointer");
    const int32_t fmt = format_of(m);
    if (fmt < 0 || fmt == kFmtAffine6)
        return fail(ctx, kErrUnsupported,
                    "qmm: %d-bit group %d mode %d has no kernel (affine 4/8-bit g64, 4-bit g32, ternary 2-bit g128, mxfp4 g32)",
                    m->bits, m->group, m->mode);
    if (fmt != kFmtMxfp4 && fmt != kFmtTernary && m->biases == nullptr)
        return fail(ctx, kErrInvalidArg, "qmm: affine layer without biases");
    if (fmt == kFmtTernary && m->k % 128 != 0) return fail(ctx, kErrInvalidArg, "qmm: ternary k = %d must be a multiple of 128", m->k);
    // the reference's preconditions (Layers/Linear.swift:695)
    if (rows < 64 || rows % 64 != 0) return fail(ctx, kErrInvalidArg, "qmm: rows = %d must be a multiple of 64", rows);
    if (m->n % 64 != 0 || m->k % 64 != 0 || m->n <= 0 || m->k <= 0)
        return fail(ctx, kErrInvalidArg, "qmm: n = %d and k = %d must be multiples of 64", m->n, m->k);
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return fail(ctx, kErrInvalidArg, "qmm: dtype");
    if (ldx < m->k || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0 || ldy < m->n)
        return fail(ctx, kErrInvalidArg, "qmm: x must be 16-byte aligned with ldx >= k, ldx %% 8 == 0; ldy >= n");
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    const void* x16 = x;
    int64_t ld16 = ldx;
    if (x_dtype != IQ_F16) {
        size_t need = 0;
        iq_qmm_workspace_bytes(ctx, m, rows, x_dtype, &need);
        if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
            return fail(ctx, kErrWorkspace, "qmm: workspace %zu < %zu (256-byte aligned)", workspace_bytes, need);
        const size_t units = (size_t)rows * m->k / 8;
        convert_x_f16_kernel<<<(unsigned)((units + 255) / 256), 256, 0, cs>>>(x, x_dtype, ldx, static_cast<__half*>(workspace),
                                                                             rows, m->k);
        int32_t st = check_cuda(ctx, cudaGetLastError(), "convert_x launch");
        if (st != kOk) return st;
        x16 = workspace;
        ld16 = m->k;
    }
    QmmCall c;
    c.fmt = fmt;
    c.epi = kEpiStore;
    c.bn = rows >= 256 ? 256 : 128;
    c.x16 = x16; c.ldx = ld16; c.x_rows = rows;
    c.w[0] = m->w; c.s[0] = m->scales; c.b[0] = m->biases;
    c.experts = 1;
    c.N = m->n; c.K = m->k; c.M = rows;
    c.y = y; c.y_dtype = y_dtype; c.ldy = ldy;
    c.accumulate = (flags & IQ_FLAG_ACCUMULATE) ? 1 : 0;
    return launch_qmm(ctx, cs, c);
}

// ---------------------------------------------------------------------------------------------------------------------
// Prefill GEMM for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all: a plugin loaded into an engine whose memory pool owns
// every device byte and forbids side allocations, a call site that runs after the pool has been sealed, or code under
// a "no allocation after start-up" rule (real-time serving paths, sandboxes that filter the allocator entry points).
// iq_qmm needs a scratch buffer when the activations are bf16 or fp32 (they are converted to fp16 first) and expects the
// caller to bring it. This variant brings its own: a fixed array that is part of the library image, so it exists on
// every GPU that loads the library, from load until the process exits, and costs that GPU kNoAllocBytes of memory.
constexpr size_t kNoAllocBytes = 8u << 20;  // 8 MiB: rows * k <= 4,194,304 activations (e.g. 1024 x 4096)
static __device__ __align__(256) unsigned char g_qmm_noalloc_scratch[kNoAllocBytes];

namespace {
constexpr int kMaxDevices = 64;
std::atomic<void*> g_noalloc_ptr[kMaxDevices];  // device address of the array, per device, resolved on first use (zero-initialised)
}  // namespace

extern "C" int32_t iq_qmm_noalloc(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx,
                                  const iq_qlinear* m, void* y, int32_t y_dtype, int64_t ldy, int32_t rows,
                                  uint32_t flags) {
    if (ctx == nullptr) return kErrInvalidArg;
    if (m == nullptr) return fail(ctx, kErrInvalidArg, "qmm_noalloc: null pointer");
    if (rows < 1 || m->k < 1) return fail(ctx, kErrInvalidArg, "qmm_noalloc: rows = %d, k = %d", rows, m->k);
    const size_t need = (size_t)rows * (size_t)m->k * 2;
    if (need > kNoAllocBytes)
        return fail(ctx, kErrWorkspace,
                    "qmm_noalloc: rows * k = %zu activations exceed the built-in scratch (%zu); use iq_qmm with a "
                    "caller-provided workspace", (size_t)rows * (size_t)m->k, kNoAllocBytes / 2);
    const int dev = ctx->device;
    if (dev < 0 || dev >= kMaxDevices) return fail(ctx, kErrInvalidArg, "qmm_noalloc: device %d", dev);
    void* scratch = g_noalloc_ptr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {
        // The array's name is only a host-side handle here; the kernels need its address on this device. Resolved once
        // per device with that device current (it is: the context selected it, and the caller runs on it).
        int cur = -1;
        cudaError_t e = cudaGetDevice(&cur);
        if (e != cudaSuccess) return check_cuda(ctx, e, "cudaGetDevice");
        if (cur != dev) return fail(ctx, kErrInvalidArg, "qmm_noalloc: device %d is current, the context is on %d", cur, dev);
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_qmm_noalloc_scratch);
        if (e != cudaSuccess) return check_cuda(ctx, e, "cudaGetSymbolAddress(scratch)");
        g_noalloc_ptr[dev].store(p, std::memory_order_release);  // two first callers store the same address
        scratch = p;
    }
    // Every byte the GEMM reads from the scratch is written by this call's own conversion pass first, so nothing has
    // to be cleared; what the previous call left behind is simply overwritten.
    return iq_qmm(ctx, stream, x, x_dtype, ldx, m, y, y_dtype, ldy, rows, flags, scratch, kNoAllocBytes);
}
