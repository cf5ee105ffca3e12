// Column-split dense linear over the GPUs of one box: rank r holds output features [r*n/G, (r+1)*n/G) of the weight
// matrix (a contiguous range of rows of w / scales / biases, the layout being row-major by output feature), x is
// replicated, and every rank ends up with the whole y. The slices are exchanged by this library's own kernels over
// peer-addressable memory: each rank computes its slice straight into its own y, stores it into the same columns of
// every peer's y with 16-byte peer stores and meets the others at a flag barrier. No host synchronisation and no
// library collective, so a decode step can keep the call inside a CUDA graph; for one activation row the exchange is a
// single small kernel (enter barrier, push, exit barrier), which a host-launched all-gather cannot match when the
// slice is a few kilobytes.
//
// The reference runs on one GPU and has no counterpart; its nearest analogue is the row concatenation of matrices that
// share their input and the nPrefix call that computes a prefix of the rows (Layers/Linear.swift:107-183, 350-366): a
// shard is exactly such a row range.
#include <new>

#include "internal.h"
#include "peer.cuh"

namespace iq {

namespace {

// rows x n_local elements of `esz` bytes at column c0 of this rank's y (row pitch ldy elements) stored into the same
// place of every other rank's y. 16-byte units: c0 * esz and n_local * esz are multiples of 16.
__device__ __forceinline__ void push_slice(const PeerPtrs& y, int rank, int world, int rows, int64_t ldy, int c0, int n_local,
                                           int esz, int tid, int nthreads) {
    const int upr = n_local * esz / 16;  // 16-byte units per row of the slice
    const char* mine = static_cast<const char*>(y.p[rank]);
    const int64_t total = (int64_t)rows * upr;
    for (int64_t i = tid; i < total; i += nthreads) {
        const int r = (int)(i / upr), u = (int)(i % upr);
        const size_t off = ((size_t)r * ldy + c0) * esz + (size_t)u * 16;
        const uint4 v = *reinterpret_cast<const uint4*>(mine + off);
        for (int q = 1; q < world; q++) {
            const int d = (rank + q) % world;  // every rank starts with another peer: the links fill evenly
            *reinterpret_cast<uint4*>(static_cast<char*>(y.p[d]) + off) = v;
        }
    }
}

// Small slices (decode): one block does the whole exchange. Enter barrier: every rank has reached this call, so nothing
// of the previous call's y is still being read there; push; exit barrier: every slice has landed everywhere.
__global__ void __launch_bounds__(256) colsplit_exchange_kernel(PeerPtrs y, PeerPtrs flags, uint32_t* epoch, int rank, int world,
                                                                int rows, int64_t ldy, int n_local, int esz, int barriers,
                                                                int32_t* status, unsigned long long wait_cycles) {
    __shared__ uint32_t e;
    if (threadIdx.x == 0) {
        e = *epoch;
        if (barriers) *epoch = e + 2;
    }
    __syncthreads();
    if (barriers) peer_flag_barrier(flags, e + 1, rank, world, status, wait_cycles);
    push_slice(y, rank, world, rows, ldy, rank * n_local, n_local, esz, threadIdx.x, blockDim.x);
    if (barriers) peer_flag_barrier(flags, e + 2, rank, world, status, wait_cycles);
}

// Large slices (prefill): the barrier and the push as kernels of their own, the push over many blocks.
__global__ void __launch_bounds__(32) colsplit_barrier_kernel(PeerPtrs flags, uint32_t* epoch, int rank, int world,
                                                              int32_t* status, unsigned long long wait_cycles) {
    __shared__ uint32_t e;
    if (threadIdx.x == 0) {
        e = *epoch + 1;
        *epoch = e;
    }
    __syncthreads();
    peer_flag_barrier(flags, e, rank, world, status, wait_cycles);
}

__global__ void __launch_bounds__(256) colsplit_push_kernel(PeerPtrs y, int rank, int world, int rows, int64_t ldy, int n_local,
                                                            int esz) {
    push_slice(y, rank, world, rows, ldy, rank * n_local, n_local, esz, blockIdx.x * blockDim.x + threadIdx.x,
               gridDim.x * blockDim.x);
}

}  // namespace
}  // namespace iq

using namespace iq;

struct iq_colsplit {
    iq_ctx* ctx = nullptr;
    int32_t rank = 0, world = 1, n_total = 0, max_rows = 0, y_dtype = 0;
    PeerPtrs y, flags;
    uint32_t* epoch = nullptr;  // device
};

extern "C" int32_t iq_colsplit_create(iq_ctx* ctx, int32_t rank, int32_t world, int32_t n_total, int32_t max_rows,
                                      int32_t y_dtype, void* const* peer_y, void* const* peer_flags, iq_colsplit** out) {
    if (ctx == nullptr || out == nullptr) return kErrInvalidArg;
    *out = nullptr;
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || max_rows < 1 || y_dtype < 0 || y_dtype > 2 ||
        peer_y == nullptr || peer_flags == nullptr)
        return fail(ctx, kErrInvalidArg, "colsplit_create: rank %d of %d", rank, world);
    // every slice is a whole number of 16-row blocks (the GEMV's unit) and of 16-byte units
    if (n_total < 16 * world || n_total % (16 * world) != 0)
        return fail(ctx, kErrInvalidArg, "colsplit_create: n = %d must be a multiple of 16 * %d ranks", n_total, world);
    iq_colsplit* cs = new (std::nothrow) iq_colsplit();
    if (cs == nullptr) return kErrCuda;
    cs->ctx = ctx; cs->rank = rank; cs->world = world; cs->n_total = n_total; cs->max_rows = max_rows; cs->y_dtype = y_dtype;
    for (int i = 0; i < world; i++) {
        if (!peer_y[i] || !peer_flags[i] || (reinterpret_cast<uintptr_t>(peer_y[i]) & 15) != 0) {
            delete cs;
            return fail(ctx, kErrInvalidArg, "colsplit_create: null or unaligned peer pointer");
        }
        cs->y.p[i] = peer_y[i];
        cs->flags.p[i] = peer_flags[i];
    }
    // set-up time: the one allocation (the epoch counter); never in the enqueue path
    void* blk = nullptr;
    cudaError_t e = cudaMalloc(&blk, 256);
    if (e == cudaSuccess) e = cudaMemset(blk, 0, 256);
    if (e != cudaSuccess) {
        delete cs;
        return check_cuda(ctx, e, "colsplit_create: cudaMalloc");
    }
    cs->epoch = static_cast<uint32_t*>(blk);
    *out = cs;
    return kOk;
}

extern "C" void iq_colsplit_destroy(iq_colsplit* cs) {
    if (cs == nullptr) return;
    if (cs->epoch) cudaFree(cs->epoch);
    delete cs;
}

extern "C" int32_t iq_linear_colsplit_workspace_bytes(iq_colsplit* cs, const iq_qlinear* shard, int32_t rows, int32_t x_dtype,
                                                      size_t* bytes) {
    if (cs == nullptr || shard == nullptr || bytes == nullptr || rows < 1) return kErrInvalidArg;
    *bytes = 0;
    if (rows <= 16) return kOk;
    return iq_qmm_workspace_bytes(cs->ctx, shard, rows, x_dtype, bytes);
}

extern "C" int32_t iq_linear_colsplit(iq_colsplit* cs, void* stream, const void* x, int32_t x_dtype, int64_t ldx,
                                      const iq_qlinear* shard, int32_t rows, uint32_t flags, void* workspace,
                                      size_t workspace_bytes) {
    if (cs == nullptr) return kErrInvalidArg;
    iq_ctx* ctx = cs->ctx;
    if (shard == nullptr || x == nullptr) return fail(ctx, kErrInvalidArg, "linear_colsplit: null pointer");
    if (rows < 1 || rows > cs->max_rows)
        return fail(ctx, kErrInvalidArg, "linear_colsplit: rows = %d (1..%d)", rows, cs->max_rows);
    const int n_local = cs->n_total / cs->world;
    if (shard->n != n_local || shard->experts > 1)
        return fail(ctx, kErrInvalidArg, "linear_colsplit: the shard has %d output features, %d / %d ranks = %d expected",
                    shard->n, cs->n_total, cs->world, n_local);
    if (flags & ~(uint32_t)(IQ_FLAG_ACCUMULATE | IQ_FLAG_NO_BARRIER))
        return fail(ctx, kErrInvalidArg, "linear_colsplit: flags");
    if (flags & IQ_FLAG_ACCUMULATE)
        return fail(ctx, kErrUnsupported, "linear_colsplit: accumulate is not offered (y is overwritten on every rank)");
    const int esz = dtype_size(cs->y_dtype);
    const int64_t ldy = cs->n_total;
    // this rank's slice, computed straight into its place in this rank's y
    char* y_mine = static_cast<char*>(cs->y.p[cs->rank]) + (size_t)cs->rank * n_local * esz;
    int32_t st;
    if (rows <= 16) {
        st = iq_qmv(ctx, stream, x, x_dtype, ldx, shard, y_mine, cs->y_dtype, ldy, rows, 0, 0);
    } else {
        st = iq_qmm(ctx, stream, x, x_dtype, ldx, shard, y_mine, cs->y_dtype, ldy, rows, 0, workspace, workspace_bytes);
    }
    if (st != kOk) return st;
    if (cs->world == 1) return kOk;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int barriers = (flags & IQ_FLAG_NO_BARRIER) ? 0 : 1;
    const int64_t slice_bytes = (int64_t)rows * n_local * esz;
    if (slice_bytes <= 256 * 1024) {
        colsplit_exchange_kernel<<<1, 256, 0, s>>>(cs->y, cs->flags, cs->epoch, cs->rank, cs->world, rows, ldy, n_local, esz,
                                                   barriers, ctx->d_status, ctx->wait_cycles);
        return check_cuda(ctx, cudaGetLastError(), "colsplit_exchange launch");
    }
    if (barriers) colsplit_barrier_kernel<<<1, 32, 0, s>>>(cs->flags, cs->epoch, cs->rank, cs->world, ctx->d_status, ctx->wait_cycles);
    const int64_t units = slice_bytes / 16;
    const int64_t want = (units + 1023) / 1024, cap = (int64_t)ctx->sms * 4;
    colsplit_push_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, s>>>(cs->y, cs->rank, cs->world, rows, ldy, n_local, esz);
    if (barriers) colsplit_barrier_kernel<<<1, 32, 0, s>>>(cs->flags, cs->epoch, cs->rank, cs->world, ctx->d_status, ctx->wait_cycles);
    return check_cuda(ctx, cudaGetLastError(), "colsplit push launch");
}
