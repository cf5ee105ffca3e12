// Expert-parallel exchange over NVLink peer memory: the dispatch and the return of the rows are plain peer stores
// issued by this library's kernels, ordered by a flag barrier in peer memory, with every size read on the device.
// Nothing in a layer touches the host, so a whole multi-layer step can be captured in a CUDA graph.
//
// The reference engine runs on one GPU and has nothing to compare with; the nearest notion is its expert -> slot table
// (Layers/MoE.swift:104). Buffers: every rank owns a receive buffer (rows it computes for others), a return buffer
// (expert outputs coming back, in its own expert order) and a flag array, all allocated by the host in memory the
// peers can address (cudaIpc, cuMem, torch symmetric memory, ...) and passed here as arrays of device pointers.
// No TMA and no multicast is involved: rows move with 16-byte peer stores.
#include <new>

#include "internal.h"
#include "peer.cuh"
#include "ptx.cuh"

namespace iq {

namespace {

constexpr int kMaxSegs = kMaxRanks * 512;

// Receive-buffer layout: every source rank owns a fixed region of region_rows rows in each peer's receive buffer, so a
// rank can push its rows without knowing what the other sources send. Inside region s the rows are in local-expert
// order. Per-layer plan of rank `rank`, derived from counts[s * E + e] (rows rank s routes to expert e):
//   from[s]                 rows received from source s
//   seg_recv[s * El + j]    first row of (source s, local expert j) in this rank's receive buffer
//   seg_src[s * El + j]     position of that segment in source s's expert-sorted list
//   seg_dst[s * El + j]     where that segment goes when the rows are compacted expert-major (all sources' rows of one
//                           expert next to each other, so that the grouped GEMM sees one run of rows per expert)
//   merged[e]               rows of expert e over all sources (global expert index; zero outside this rank's range)
struct EpPlan {
    uint32_t from[kMaxRanks];
    uint32_t seg_recv[kMaxSegs];
    uint32_t seg_src[kMaxSegs];
    uint32_t seg_dst[kMaxSegs];
    uint32_t merged[kMaxSegs];
};

// One block of any size.
__device__ __forceinline__ void ep_plan_body(const uint32_t* __restrict__ counts, int rank, int world, int E,
                                             uint32_t region_rows, EpPlan* __restrict__ plan) {
    const int El = E / world;
    if ((int)threadIdx.x < world) {
        const int s = threadIdx.x;
        uint32_t r = s * region_rows, src = 0;
        for (int e = 0; e < rank * El; e++) src += counts[s * E + e];
        for (int j = 0; j < El; j++) {
            plan->seg_recv[s * El + j] = r;
            plan->seg_src[s * El + j] = src;
            const uint32_t c = counts[s * E + rank * El + j];
            r += c;
            src += c;
        }
        plan->from[s] = r - s * region_rows;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        uint32_t m = 0;
        if (e / El == rank)
            for (int s = 0; s < world; s++) m += counts[s * E + e];
        plan->merged[e] = m;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < El; j += blockDim.x) {
        uint32_t o = 0;
        for (int j2 = 0; j2 < j; j2++) o += plan->merged[rank * El + j2];
        for (int s = 0; s < world; s++) {
            plan->seg_dst[s * El + j] = o;
            o += counts[s * E + rank * El + j];
        }
    }
}

__global__ void __launch_bounds__(32) ep_plan_kernel(const uint32_t* __restrict__ counts, int rank, int world, int E,
                                                     uint32_t region_rows, EpPlan* __restrict__ plan) {
    ep_plan_body(counts, rank, world, E, region_rows, plan);
}

// Rows of this rank, packed as fp16 in expert order, written straight into region `rank` of the owners' receive
// buffers; the first `world` blocks also write this rank's per-expert counts into row `rank` of every peer's count
// matrix. Nothing here depends on what the peers do in the same layer.
__global__ void __launch_bounds__(256) ep_pack_push_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx,
                                                          const uint32_t* __restrict__ inds, const uint32_t* __restrict__ pos,
                                                          const uint32_t* __restrict__ offsets, PeerPtrs recv, PeerPtrs counts,
                                                          int rank, int world, int E, uint32_t region_rows, int P, int D,
                                                          int topk) {
    const int El = E / world;
    if ((int)blockIdx.x < world) {
        uint32_t* c = static_cast<uint32_t*>(counts.p[blockIdx.x]) + rank * E;
        for (int e = threadIdx.x; e < E; e += 256) c[e] = offsets[e + 1] - offsets[e];
    }
    const int pair = blockIdx.x;
    if (pair >= P) return;
    const uint32_t e = inds[pair];
    const int d = e / El;
    const uint32_t row = rank * region_rows + (pos[pair] - offsets[d * El]);
    __half* dst = static_cast<__half*>(recv.p[d]) + (size_t)row * D;
    const size_t src = (size_t)(pair / topk) * ldx;
    for (int u = threadIdx.x; u < D / 8; u += 256) {
        float v[8];
        load_x8(x, x_dtype, src + u * 8, v);
        uint4 o;
        o.x = pack_half2(v[0], v[1]); o.y = pack_half2(v[2], v[3]); o.z = pack_half2(v[4], v[5]); o.w = pack_half2(v[6], v[7]);
        *reinterpret_cast<uint4*>(dst + u * 8) = o;
    }
}

// The same dispatch with every token row sent ONCE per destination rank, however many of its experts live there (with
// top-8 routing over 2 / 4 / 8 ranks a token has on average 4 / 2.2 / 1.5 pairs per rank it reaches). Layout of a
// receive buffer in this mode: fp16 rows [world * tok_rows, D], row s * tok_rows + t = token t of source s (rows of
// tokens that do not come here are simply not written), followed at byte ep_tokmap_offset() by uint32
// [world * region_rows]: entry s * region_rows + q = the token of the q-th pair source s routes here, in its
// local-expert order. One block per (token, destination); the first `world` blocks also push the counts.
__host__ __device__ inline size_t ep_tokmap_offset(int world, int tok_rows, int D) {
    return ((size_t)world * tok_rows * D * 2 + 255) / 256 * 256;
}
__global__ void __launch_bounds__(256) ep_pack_push_tokens_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx,
                                                                 const uint32_t* __restrict__ inds, const uint32_t* __restrict__ pos,
                                                                 const uint32_t* __restrict__ offsets, PeerPtrs recv, PeerPtrs counts,
                                                                 int rank, int world, int E, uint32_t region_rows, int T, int D,
                                                                 int topk, int tok_rows) {
    const int El = E / world;
    const int lin = blockIdx.y * gridDim.x + blockIdx.x;
    if (lin < world) {
        uint32_t* c = static_cast<uint32_t*>(counts.p[lin]) + rank * E;
        for (int e = threadIdx.x; e < E; e += 256) c[e] = offsets[e + 1] - offsets[e];
    }
    const int t = blockIdx.x, d = blockIdx.y;
    __shared__ int here;
    if (threadIdx.x == 0) here = 0;
    __syncthreads();
    char* base = static_cast<char*>(recv.p[d]);
    if ((int)threadIdx.x < topk) {
        const int pair = t * topk + threadIdx.x;
        const uint32_t e = inds[pair];
        if ((int)(e / El) == d) {
            uint32_t* tokmap = reinterpret_cast<uint32_t*>(base + ep_tokmap_offset(world, tok_rows, D));
            tokmap[(size_t)rank * region_rows + (pos[pair] - offsets[d * El])] = (uint32_t)t;
            here = 1;
        }
    }
    __syncthreads();
    if (!here) return;
    __half* dst = reinterpret_cast<__half*>(base) + ((size_t)rank * tok_rows + t) * D;
    const size_t src = (size_t)t * ldx;
    for (int u = threadIdx.x; u < D / 8; u += 256) {
        float v[8];
        load_x8(x, x_dtype, src + u * 8, v);
        uint4 o;
        o.x = pack_half2(v[0], v[1]); o.y = pack_half2(v[2], v[3]); o.z = pack_half2(v[4], v[5]); o.w = pack_half2(v[6], v[7]);
        *reinterpret_cast<uint4*>(dst + u * 8) = o;
    }
}

// Expert outputs of the rows this rank computed, written back into each source's return buffer at the source's own
// expert-sorted positions. Four rows per block, 64 threads per row, four 16-byte loads in flight per thread.
__global__ void __launch_bounds__(256) ep_return_push_kernel(const void* __restrict__ yd, int elem_bytes,
                                                            const EpPlan* __restrict__ plan, PeerPtrs back, int D, int world,
                                                            int El, uint32_t region_rows) {
    const uint32_t j = blockIdx.x * 4 + (threadIdx.x >> 6);
    const int t = threadIdx.x & 63;
    const uint32_t s = j / region_rows;
    if ((int)s >= world) return;
    if (j - s * region_rows >= plan->from[s]) return;
    // the segment of source s that holds row j: binary search over that source's segment starts
    int lo = s * El, hi = (s + 1) * El;  // seg_recv[lo] <= j, seg_recv[hi] > j (hi may be one past the source's last)
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (plan->seg_recv[mid] <= j) lo = mid; else hi = mid;
    }
    const uint32_t drow = plan->seg_src[lo] + (j - plan->seg_recv[lo]);
    const size_t row_bytes = (size_t)D * elem_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(yd) + (size_t)j * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(back.p[s]) + (size_t)drow * row_bytes);
    const int n16 = (int)(row_bytes / 16);
    int u = t;
    for (; u + 192 < n16; u += 256) {
        const uint4 a = ldg_nc_u4(src + u), b = ldg_nc_u4(src + u + 64), c = ldg_nc_u4(src + u + 128), d = ldg_nc_u4(src + u + 192);
        dst[u] = a; dst[u + 64] = b; dst[u + 128] = c; dst[u + 192] = d;
    }
    for (; u < n16; u += 64) dst[u] = ldg_nc_u4(src + u);
}

// Received rows gathered from their per-source regions into expert-major order (xc), with the table of return addresses
// in the same order: table[i] = where the output of compacted row i goes in its source rank's return buffer (0 past the
// rows received). Four rows per block, 64 threads per row.
__global__ void __launch_bounds__(256) ep_compact_kernel(const __half* __restrict__ recv, const EpPlan* __restrict__ plan,
                                                        PeerPtrs back, int D, int row_bytes_back, int world, int El,
                                                        uint32_t region_rows, __half* __restrict__ xc,
                                                        uint64_t* __restrict__ table) {
    // rows past the total keep a zero in the table (j runs over the capacity; the total is small next to it)
    uint32_t total = 0;
    for (int q = 0; q < world; q++) total += plan->from[q];
    const int t = threadIdx.x & 63;
    // the capacity is many times what arrives: a fixed grid walks the row slots instead of one block per four slots
    for (uint32_t j = blockIdx.x * 4 + (threadIdx.x >> 6); j < (uint32_t)world * region_rows; j += gridDim.x * 4) {
    const uint32_t s = j / region_rows;
    if (j >= total && t == 0) table[j] = 0;
    if (j - s * region_rows >= plan->from[s]) continue;
    int lo = s * El, hi = (s + 1) * El;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (plan->seg_recv[mid] <= j) lo = mid; else hi = mid;
    }
    const uint32_t idx = j - plan->seg_recv[lo];
    const uint32_t dst = plan->seg_dst[lo] + idx;
    if (t == 0)
        table[dst] = reinterpret_cast<uint64_t>(static_cast<char*>(back.p[s]) + (size_t)(plan->seg_src[lo] + idx) * row_bytes_back);
    const uint4* src = reinterpret_cast<const uint4*>(recv + (size_t)j * D);
    uint4* out = reinterpret_cast<uint4*>(xc + (size_t)dst * D);
    const int n16 = D / 8;
    int u = t;
    for (; u + 192 < n16; u += 256) {
        const uint4 a = ldg_nc_u4(src + u), b = ldg_nc_u4(src + u + 64), c = ldg_nc_u4(src + u + 128), d = ldg_nc_u4(src + u + 192);
        out[u] = a; out[u + 64] = b; out[u + 128] = c; out[u + 192] = d;
    }
    for (; u < n16; u += 64) out[u] = ldg_nc_u4(src + u);
    }
}

// The expert-major order without moving a row: index[i] = the receive-buffer row that position i of the expert-major
// order holds, table[i] = where its output goes in its source rank's return buffer (0 past the rows received). The
// experts' kernels then fetch their rows through `index` (the grouped GEMM's producer gathers by row index).
// tokmap: null, or (token mode, see ep_pack_push_tokens_kernel) the token of every received pair: the row of pair j of
// source s is then s * tok_rows + tokmap[j].
__global__ void __launch_bounds__(256) ep_index_kernel(const EpPlan* __restrict__ plan, PeerPtrs back, int row_bytes_back, int world,
                                                      int El, uint32_t region_rows, uint32_t* __restrict__ index,
                                                      uint64_t* __restrict__ table, const uint32_t* __restrict__ tokmap = nullptr,
                                                      uint32_t tok_rows = 0) {
    uint32_t total = 0;
    for (int q = 0; q < world; q++) total += plan->from[q];
    for (uint32_t j = blockIdx.x * 256 + threadIdx.x; j < (uint32_t)world * region_rows; j += gridDim.x * 256) {
        if (j >= total) {
            table[j] = 0;
            index[j] = 0;
        }
        const uint32_t s = j / region_rows;
        if (j - s * region_rows >= plan->from[s]) continue;
        int lo = s * El, hi = (s + 1) * El;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (plan->seg_recv[mid] <= j) lo = mid; else hi = mid;
        }
        const uint32_t idx = j - plan->seg_recv[lo];
        const uint32_t dst = plan->seg_dst[lo] + idx;
        index[dst] = tokmap != nullptr ? s * tok_rows + tokmap[j] : j;
        table[dst] = reinterpret_cast<uint64_t>(static_cast<char*>(back.p[s]) + (size_t)(plan->seg_src[lo] + idx) * row_bytes_back);
    }
}

// The same mapping as a table: table[j] = address, in the source rank's return buffer, of the output of received row j
// (0 for rows nobody sent). A GEMM epilogue that stores through this table returns the rows without a copy kernel.
__global__ void __launch_bounds__(256) ep_return_rows_kernel(const EpPlan* __restrict__ plan, PeerPtrs back, int row_bytes, int world,
                                                            int El, uint32_t region_rows, uint64_t* __restrict__ table) {
    const uint32_t j = blockIdx.x * 256 + threadIdx.x;
    const uint32_t s = j / region_rows;
    if ((int)s >= world) return;
    uint64_t out = 0;
    if (j - s * region_rows < plan->from[s]) {
        int lo = s * El, hi = (s + 1) * El;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (plan->seg_recv[mid] <= j) lo = mid; else hi = mid;
        }
        const uint32_t drow = plan->seg_src[lo] + (j - plan->seg_recv[lo]);
        out = reinterpret_cast<uint64_t>(static_cast<char*>(back.p[s]) + (size_t)drow * row_bytes);
    }
    table[j] = out;
}

// this rank's per-expert row counts (from its expert offsets) written into row `rank` of every peer's count matrix
__global__ void ep_share_counts_kernel(const uint32_t* __restrict__ offsets, PeerPtrs counts, int rank, int world, int E) {
    for (int i = threadIdx.x; i < E * world; i += blockDim.x) {
        const int d = i / E, e = i % E;
        static_cast<uint32_t*>(counts.p[d])[rank * E + e] = offsets[e + 1] - offsets[e];
    }
}

// Barrier over the ranks of the box. Each rank bumps its own epoch, publishes it into slot `rank` of every peer's flag
// array and waits until every slot of its own array has reached the epoch. Counters only grow, so the kernel can be
// replayed from a CUDA graph. The wait is bounded: on a timeout the status word is set and the kernel returns.
// With plan != nullptr the kernel goes on to derive this rank's plan from the count matrix the peers have just completed.
__global__ void ep_barrier_kernel(PeerPtrs flags, uint32_t* epoch, int rank, int world, int32_t* status,
                                  const uint32_t* counts, int E, uint32_t region_rows, EpPlan* plan,
                                  unsigned long long wait_cycles) {
    __shared__ uint32_t e;
    if (threadIdx.x == 0) {
        e = *epoch + 1;
        *epoch = e;
    }
    __syncthreads();
    peer_flag_barrier(flags, e, rank, world, status, wait_cycles);
    if (plan != nullptr) ep_plan_body(counts, rank, world, E, region_rows, plan);
}

}  // namespace
}  // namespace iq

using namespace iq;

// Opaque per-rank state of the exchange: the peers' buffers and a small device block (plan, epoch).
struct iq_ep {
    iq_ctx* ctx = nullptr;
    int32_t rank = 0, world = 1, experts = 0, region_rows = 0;
    PeerPtrs recv, back, flags, counts;
    EpPlan* plan = nullptr;   // device
    uint32_t* epoch = nullptr;  // device
};

extern "C" int32_t iq_ep_create(iq_ctx* ctx, int32_t rank, int32_t world, int32_t experts, int32_t region_rows, void* const* peer_recv,
                                void* const* peer_back, void* const* peer_flags, void* const* peer_counts, iq_ep** out) {
    if (ctx == nullptr || out == nullptr) return kErrInvalidArg;
    *out = nullptr;
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || experts < world || experts % world != 0 || region_rows < 1 ||
        world * (experts / world) > kMaxSegs || peer_recv == nullptr || peer_back == nullptr || peer_flags == nullptr || peer_counts == nullptr)
        return fail(ctx, kErrInvalidArg, "ep_create: rank %d of %d, %d experts", rank, world, experts);
    iq_ep* ep = new (std::nothrow) iq_ep();
    if (ep == nullptr) return kErrCuda;
    ep->ctx = ctx; ep->rank = rank; ep->world = world; ep->experts = experts; ep->region_rows = region_rows;
    for (int i = 0; i < world; i++) {
        if (!peer_recv[i] || !peer_back[i] || !peer_flags[i] || !peer_counts[i]) {
            delete ep;
            return fail(ctx, kErrInvalidArg, "ep_create: null peer pointer");
        }
        ep->recv.p[i] = peer_recv[i]; ep->back.p[i] = peer_back[i]; ep->flags.p[i] = peer_flags[i];
        ep->counts.p[i] = peer_counts[i];
    }
    // set-up time: the one allocation of the exchange (plan + epoch); never in the enqueue path
    void* blk = nullptr;
    cudaError_t e = cudaMalloc(&blk, sizeof(EpPlan) + 256);
    if (e == cudaSuccess) e = cudaMemset(blk, 0, sizeof(EpPlan) + 256);
    if (e != cudaSuccess) {
        delete ep;
        return check_cuda(ctx, e, "ep_create: cudaMalloc");
    }
    ep->plan = static_cast<EpPlan*>(blk);
    ep->epoch = reinterpret_cast<uint32_t*>(static_cast<char*>(blk) + sizeof(EpPlan));
    *out = ep;
    return kOk;
}

extern "C" void iq_ep_destroy(iq_ep* ep) {
    if (ep == nullptr) return;
    if (ep->plan) cudaFree(ep->plan);
    delete ep;
}

extern "C" int32_t iq_ep_share_counts(iq_ep* ep, void* stream, const uint32_t* offsets) {
    if (ep == nullptr || offsets == nullptr) return kErrInvalidArg;
    ep_share_counts_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(offsets, ep->counts, ep->rank, ep->world,
                                                                                ep->experts);
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_share_counts launch");
}

extern "C" int32_t iq_ep_plan(iq_ep* ep, void* stream) {
    if (ep == nullptr) return kErrInvalidArg;
    const uint32_t* counts_all = static_cast<const uint32_t*>(ep->counts.p[ep->rank]);
    ep_plan_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(counts_all, ep->rank, ep->world, ep->experts,
                                                                         (uint32_t)ep->region_rows, ep->plan);
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_plan launch");
}

extern "C" int32_t iq_ep_barrier(iq_ep* ep, void* stream, int32_t then_plan) {
    if (ep == nullptr) return kErrInvalidArg;
    ep_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        ep->flags, ep->epoch, ep->rank, ep->world, ep->ctx->d_status, static_cast<const uint32_t*>(ep->counts.p[ep->rank]),
        ep->experts, (uint32_t)ep->region_rows, then_plan ? ep->plan : nullptr, ep->ctx->wait_cycles);
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_barrier launch");
}

extern "C" int32_t iq_ep_pack_push(iq_ep* ep, void* stream, const void* x, int32_t x_dtype, int64_t ldx, int32_t tokens,
                                   int32_t top_k, int32_t d_model, const uint32_t* inds, const uint32_t* pos,
                                   const uint32_t* offsets) {
    if (ep == nullptr) return kErrInvalidArg;
    if (x == nullptr || inds == nullptr || pos == nullptr || offsets == nullptr || tokens < 1 || top_k < 1 || d_model % 8 != 0 ||
        ldx < d_model || ldx % 8 != 0 || x_dtype < 0 || x_dtype > 2)
        return fail(ep->ctx, kErrInvalidArg, "ep_pack_push: arguments");
    const int P = tokens * top_k;
    if (P > ep->region_rows)
        return fail(ep->ctx, kErrInvalidArg, "ep_pack_push: %d rows exceed the region of %d rows", P, ep->region_rows);
    const int grid = P > ep->world ? P : ep->world;
    ep_pack_push_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        x, x_dtype, ldx, inds, pos, offsets, ep->recv, ep->counts, ep->rank, ep->world, ep->experts, (uint32_t)ep->region_rows, P,
        d_model, top_k);
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_pack_push launch");
}

extern "C" int32_t iq_ep_return_push(iq_ep* ep, void* stream, const void* yd, int32_t yd_dtype, int32_t d_model) {
    if (ep == nullptr) return kErrInvalidArg;
    if (yd == nullptr || (yd_dtype != kF32 && yd_dtype != kF16) || d_model % 8 != 0)
        return fail(ep->ctx, kErrInvalidArg, "ep_return_push: arguments");
    const int64_t rows = (int64_t)ep->world * ep->region_rows;
    ep_return_push_kernel<<<(unsigned)((rows + 3) / 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        yd, yd_dtype == kF32 ? 4 : 2, ep->plan, ep->back, d_model, ep->world, ep->experts / ep->world, (uint32_t)ep->region_rows);
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_return_push launch");
}

extern "C" int32_t iq_ep_return_rows(iq_ep* ep, void* stream, int32_t yd_dtype, int32_t d_model, void** table) {
    if (ep == nullptr) return kErrInvalidArg;
    if (table == nullptr || (yd_dtype != kF32 && yd_dtype != kF16) || d_model % 8 != 0)
        return fail(ep->ctx, kErrInvalidArg, "ep_return_rows: arguments");
    const int64_t rows = (int64_t)ep->world * ep->region_rows;
    ep_return_rows_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        ep->plan, ep->back, d_model * (yd_dtype == kF32 ? 4 : 2), ep->world, ep->experts / ep->world, (uint32_t)ep->region_rows,
        reinterpret_cast<uint64_t*>(table));
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_return_rows launch");
}

extern "C" int32_t iq_ep_compact(iq_ep* ep, void* stream, const void* recv_rows, int32_t d_model, int32_t yd_dtype,
                                 void* rows_out, void** table, const uint32_t** merged_counts) {
    if (ep == nullptr) return kErrInvalidArg;
    if (recv_rows == nullptr || rows_out == nullptr || table == nullptr || (yd_dtype != kF32 && yd_dtype != kF16) ||
        d_model % 8 != 0)
        return fail(ep->ctx, kErrInvalidArg, "ep_compact: arguments");
    const int64_t rows = (int64_t)ep->world * ep->region_rows;
    const int64_t want = (rows + 3) / 4, cap = (int64_t)ep->ctx->sms * 8;
    ep_compact_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(recv_rows), ep->plan, ep->back, d_model, d_model * (yd_dtype == kF32 ? 4 : 2), ep->world,
        ep->experts / ep->world, (uint32_t)ep->region_rows, static_cast<__half*>(rows_out), reinterpret_cast<uint64_t*>(table));
    if (merged_counts != nullptr) *merged_counts = ep->plan->merged;
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_compact launch");
}

extern "C" int32_t iq_ep_index(iq_ep* ep, void* stream, int32_t d_model, int32_t yd_dtype, uint32_t* row_index, void** table,
                               const uint32_t** merged_counts) {
    if (ep == nullptr) return kErrInvalidArg;
    if (row_index == nullptr || table == nullptr || (yd_dtype != kF32 && yd_dtype != kF16) || d_model % 8 != 0)
        return fail(ep->ctx, kErrInvalidArg, "ep_index: arguments");
    const int64_t rows = (int64_t)ep->world * ep->region_rows;
    const int64_t want = (rows + 255) / 256, cap = (int64_t)ep->ctx->sms * 4;
    ep_index_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        ep->plan, ep->back, d_model * (yd_dtype == kF32 ? 4 : 2), ep->world, ep->experts / ep->world, (uint32_t)ep->region_rows,
        row_index, reinterpret_cast<uint64_t*>(table));
    if (merged_counts != nullptr) *merged_counts = ep->plan->merged;
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_index launch");
}

extern "C" int32_t iq_ep_pack_push_tokens(iq_ep* ep, void* stream, const void* x, int32_t x_dtype, int64_t ldx, int32_t tokens,
                                          int32_t top_k, int32_t d_model, const uint32_t* inds, const uint32_t* pos,
                                          const uint32_t* offsets, int32_t tok_rows) {
    if (ep == nullptr) return kErrInvalidArg;
    if (x == nullptr || inds == nullptr || pos == nullptr || offsets == nullptr || tokens < 1 || top_k < 1 || top_k > 256 ||
        d_model % 8 != 0 || ldx < d_model || ldx % 8 != 0 || x_dtype < 0 || x_dtype > 2 || tok_rows < tokens)
        return fail(ep->ctx, kErrInvalidArg, "ep_pack_push_tokens: arguments");
    if (tokens * top_k > ep->region_rows)
        return fail(ep->ctx, kErrInvalidArg, "ep_pack_push_tokens: %d pairs exceed the region of %d rows", tokens * top_k,
                    ep->region_rows);
    // the token rows and the pair -> token map share the receive buffer (fp16 [world * region_rows, d_model] as created)
    if (ep_tokmap_offset(ep->world, tok_rows, d_model) + (size_t)ep->world * ep->region_rows * 4 >
        (size_t)ep->world * ep->region_rows * d_model * 2)
        return fail(ep->ctx, kErrInvalidArg, "ep_pack_push_tokens: %d token rows per source do not fit the receive buffer", tok_rows);
    if ((int64_t)tokens * ep->world < ep->world) return kErrInvalidArg;
    ep_pack_push_tokens_kernel<<<dim3(tokens, ep->world), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        x, x_dtype, ldx, inds, pos, offsets, ep->recv, ep->counts, ep->rank, ep->world, ep->experts, (uint32_t)ep->region_rows, tokens,
        d_model, top_k, tok_rows);
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_pack_push_tokens launch");
}

extern "C" int32_t iq_ep_index_tokens(iq_ep* ep, void* stream, int32_t d_model, int32_t yd_dtype, int32_t tok_rows,
                                      uint32_t* row_index, void** table, const uint32_t** merged_counts) {
    if (ep == nullptr) return kErrInvalidArg;
    if (row_index == nullptr || table == nullptr || (yd_dtype != kF32 && yd_dtype != kF16) || d_model % 8 != 0 || tok_rows < 1)
        return fail(ep->ctx, kErrInvalidArg, "ep_index_tokens: arguments");
    const int64_t rows = (int64_t)ep->world * ep->region_rows;
    const int64_t want = (rows + 255) / 256, cap = (int64_t)ep->ctx->sms * 4;
    const uint32_t* tokmap = reinterpret_cast<const uint32_t*>(static_cast<const char*>(ep->recv.p[ep->rank]) +
                                                               ep_tokmap_offset(ep->world, tok_rows, d_model));
    ep_index_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        ep->plan, ep->back, d_model * (yd_dtype == kF32 ? 4 : 2), ep->world, ep->experts / ep->world, (uint32_t)ep->region_rows,
        row_index, reinterpret_cast<uint64_t*>(table), tokmap, (uint32_t)tok_rows);
    if (merged_counts != nullptr) *merged_counts = ep->plan->merged;
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_index_tokens launch");
}
