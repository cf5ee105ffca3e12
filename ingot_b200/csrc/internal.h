// Internal declarations shared by the translation units of libingot_qmm.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

#include "../../include/ingot_qmm.h"
#include "common.cuh"

struct iq_ctx {
    int device = 0;
    int sms = 0;
    int smem_optin = 0;
    // cuTensorMapEncodeTiled, resolved through the runtime so that the library does not link libcuda directly
    void* encode_tiled = nullptr;
    int32_t* d_status = nullptr;  // device status word written by kernels whose bounded waits gave up
    // bound, in SM clock cycles, of the waits on another GPU (the flag barrier of the expert-parallel exchange and of the
    // column-split linear); iq_ctx_set_wait_cycles changes it
    unsigned long long wait_cycles = 4000000000ull;
    // scratch of the GEMV's tail split (csrc/qmv_imma.cuh): kQmvTailSlots slots
    float* qmv_tail_scratch = nullptr;
    uint32_t* qmv_tail_counters = nullptr;
    // one slot of the ring per stream that has launched a tail-split GEMV (launches of one stream run in series, so they
    // can share a slot; different streams may overlap and must not)
    static constexpr int kTailSlots = 16;
    void* qmv_tail_streams[kTailSlots] = {nullptr};
    int qmv_tail_stream_count = 0;
    std::mutex qmv_tail_lock;
    // tensor maps of the GEMV's weight matrices (csrc/qmv.cu), keyed by (base, rows, row bytes): encoding one costs a
    // driver call, a decode step launches the same matrices over and over
    struct QmvMap {
        const void* base = nullptr;
        int32_t rows = 0, row_bytes = 0, box_rows = 0;
        CUtensorMap map;
    };
    static constexpr int kQmvMaps = 256;
    QmvMap* qmv_maps = nullptr;  // host array [kQmvMaps], allocated on first use
    std::mutex qmv_maps_lock;    // several host threads may launch on one context
    char last_error[256] = {0};
};

namespace iq {

constexpr int kQmvTailSlots = iq_ctx::kTailSlots;  // streams whose tail-split launches may overlap
constexpr int kQmvTailPieces = 512;       // at most this many (block, K slice) pieces per launch
constexpr int kQmvTailBlocks = 64;        // ... over at most this many 16-row blocks

int32_t fail(iq_ctx* ctx, int32_t code, const char* fmt, ...);
int32_t check_cuda(iq_ctx* ctx, cudaError_t e, const char* what);

inline bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }
inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
inline size_t round_up_sz(size_t v, size_t m) { return (v + m - 1) / m * m; }
inline int dtype_size(int32_t dt) { return dt == kF32 ? 4 : 2; }

// format id from (bits, group, mode) or -1
int32_t format_of(const iq_qlinear* m);

// 3-D tensor map over a row-major byte matrix [rows, row_bytes] (row_bytes a multiple of 128) seen as
// [row_bytes / 128 columns of 128 bytes][rows][128 bytes], box = all columns of box_rows rows, 128-byte swizzle: one copy
// brings a block of rows into shared memory as [column][row][128 bytes] with the rows of a column in different banks.
int32_t make_map_rowblock(iq_ctx* ctx, CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                          uint32_t box_rows);
// The same through the context's cache, copied into *out; an error code (with the message recorded) when the encoding fails.
int32_t cached_rowblock_map(iq_ctx* ctx, const void* base, int64_t rows, int32_t row_bytes, int32_t box_rows, CUtensorMap* out);

struct Tile;
// One launch of the gqmv family. mode: 0 plain, 1 gate/up, 2 down. `max_rows` bounds the rows of any tile (<= 16).
// tiles == nullptr means a single tile of `rows` rows. grid_tiles = upper bound of the tile count for the launch.
struct GqmvCall {
    int mode = 0;
    int32_t fmt = 0;
    const uint32_t* w[2] = {nullptr, nullptr};
    const void* s[2] = {nullptr, nullptr};
    const void* b[2] = {nullptr, nullptr};
    int64_t w_estride = 0, s_estride = 0;
    // which experts the stacked tensors hold (w[] is offset so that a global expert id indexes it); 0 experts: not known
    int32_t expert_lo = 0, expert_count = 0;
    int32_t N = 0, K = 0;
    int32_t n_full = 0;  // rows of the whole matrix when N is a prefix of it (0: N)
    const void* x = nullptr;
    int32_t x_dtype = 0;
    int64_t ldx = 0;
    const uint32_t* row_map = nullptr;
    int32_t topk = 1;
    const Tile* tiles = nullptr;
    const uint32_t* ntiles = nullptr;
    int32_t grid_tiles = 1;
    int32_t rows = 1;
    int32_t max_rows = 1;
    void* y = nullptr;
    int32_t y_dtype = 0;
    int64_t ldy = 0;
    int32_t accumulate = 0;
    const float* ebias[2] = {nullptr, nullptr};
    float limit = 0.f;
    int32_t act = 0;  // gate/up mode: activation (kAct*)
};
int32_t launch_gqmv(iq_ctx* ctx, cudaStream_t st, const GqmvCall& c);

// One launch of the tensor-core GEMM (csrc/qmm.cu). x16: fp16 activations [x_rows, ldx] (bf16 with the plain bf16 format); w[i]: stacked
// [experts * N, K] codes (w[1]: the up matrix of the gate/up epilogue). tiles == nullptr: dense tiling over M x N.
struct QmmCall {
    int32_t fmt = 0;
    int epi = 0;   // 0 store, 1 gate/up + activation
    int bn = 256;  // token rows per tile (MMA N): 128 or 256
    const void* x16 = nullptr;
    int64_t ldx = 0;
    int64_t x_rows = 0;
    // gathered activation rows (grouped gate/up): row r of a tile is row gather_map[tile.start + r] / gather_div of x16
    const uint32_t* gather_map = nullptr;
    uint32_t gather_div = 1;
    const void* w[2] = {nullptr, nullptr};
    const void* s[2] = {nullptr, nullptr};
    const void* b[2] = {nullptr, nullptr};
    int32_t experts = 1;
    int32_t expert_lo = 0;
    int32_t N = 0, K = 0, M = 0;
    const Tile* tiles = nullptr;
    const uint32_t* ntiles = nullptr;
    void* y = nullptr;
    int32_t y_dtype = 0;
    int64_t ldy = 0;
    int32_t accumulate = 0;
    const float* ebias[2] = {nullptr, nullptr};
    float limit = 0.f;
    int32_t act = 0;  // gate/up epilogue: activation (kAct*)
};
int32_t launch_qmm(iq_ctx* ctx, cudaStream_t st, const QmmCall& c);
int32_t launch_tern_qmv(iq_ctx* ctx, cudaStream_t st, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* m, void* y,
                        int32_t y_dtype, int64_t ldy, int32_t rows, int32_t n, int32_t accumulate);
int32_t tern_init(iq_ctx* ctx);
int32_t w8a8_init(iq_ctx* ctx);
int32_t gqmv_init(iq_ctx* ctx);
int32_t qmm_init(iq_ctx* ctx);
int32_t moe_init(iq_ctx* ctx);

}  // namespace iq
