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
#include "ptx.cuh"

namespace iq {

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxSegs = kMaxRanks * 512;

// Per-layer plan derived from counts[s * E + e] (rows rank s routes to expert e), for rank `rank`:
//   send_off[d]   first row of this rank's segment inside rank d's receive buffer
//   recv_off[s]   first row of source s's segment inside this rank's receive buffer; recv_off[world] = total
//   seg_recv[s * El + j] / seg_src[s * El + j]: where the rows of (source s, local expert j) start in this rank's
//   receive buffer and in source s's expert-sorted list
struct EpPlan {
    uint32_t send_off[kMaxRanks];
    uint32_t recv_off[kMaxRanks + 1];
    uint32_t seg_recv[kMaxSegs + 1];
    uint32_t seg_src[kMaxSegs];
};

__global__ void __launch_bounds__(256) ep_plan_kernel(const uint32_t* __restrict__ counts, int rank, int world, int E,
                                                      EpPlan* __restrict__ plan) {
    const int El = E / world;
    __shared__ uint32_t tot[kMaxRanks][kMaxRanks];  // tot[s][d] = rows s -> d
    for (int i = threadIdx.x; i < world * world; i += 256) {
        const int s = i / world, d = i % world;
        uint32_t t = 0;
        for (int e = d * El; e < (d + 1) * El; e++) t += counts[s * E + e];
        tot[s][d] = t;
    }
    __syncthreads();
    if (threadIdx.x < world) {
        const int d = threadIdx.x;
        uint32_t o = 0;
        for (int s = 0; s < rank; s++) o += tot[s][d];
        plan->send_off[d] = o;
    }
    if (threadIdx.x == 0) {
        uint32_t o = 0;
        for (int s = 0; s < world; s++) {
            plan->recv_off[s] = o;
            o += tot[s][rank];
        }
        plan->recv_off[world] = o;
    }
    // segments (source, local expert): one thread per source walks its local experts
    if (threadIdx.x < world) {
        const int s = threadIdx.x;
        uint32_t r = 0;
        for (int s2 = 0; s2 < s; s2++) r += tot[s2][rank];
        uint32_t src = 0;
        for (int e = 0; e < rank * El; e++) src += counts[s * E + e];
        for (int j = 0; j < El; j++) {
            plan->seg_recv[s * El + j] = r;
            plan->seg_src[s * El + j] = src;
            const uint32_t c = counts[s * E + rank * El + j];
            r += c;
            src += c;
        }
        if (s == world - 1) plan->seg_recv[world * El] = r;
    }
}

struct PeerPtrs {
    void* p[kMaxRanks];
};

// rows of this rank, packed as fp16 in expert order, written straight into the owners' receive buffers
__global__ void __launch_bounds__(256) ep_pack_push_kernel(const void* __restrict__ x, int32_t x_dtype, int64_t ldx,
                                                          const uint32_t* __restrict__ inds, const uint32_t* __restrict__ pos,
                                                          const uint32_t* __restrict__ offsets, const EpPlan* __restrict__ plan,
                                                          PeerPtrs recv, int P, int D, int topk, int El) {
    const int pair = blockIdx.x;
    if (pair >= P) return;
    const uint32_t e = inds[pair];
    const int d = e / El;
    const uint32_t row = plan->send_off[d] + (pos[pair] - offsets[d * El]);
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

// expert outputs of the rows this rank computed, written back into each source's return buffer at the source's own
// expert-sorted positions
__global__ void __launch_bounds__(256) ep_return_push_kernel(const void* __restrict__ yd, int elem_bytes,
                                                            const EpPlan* __restrict__ plan, PeerPtrs back, int D, int world,
                                                            int El) {
    __shared__ uint32_t s_dst, s_src;
    const uint32_t j = blockIdx.x;
    if (j >= plan->recv_off[world]) return;
    if (threadIdx.x == 0) {
        // the segment that holds row j: binary search over the segment starts
        int lo = 0, hi = world * El;  // seg_recv[lo] <= j < seg_recv[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (plan->seg_recv[mid] <= j) lo = mid; else hi = mid;
        }
        s_src = lo / El;
        s_dst = plan->seg_src[lo] + (j - plan->seg_recv[lo]);
    }
    __syncthreads();
    const size_t row_bytes = (size_t)D * elem_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(yd) + (size_t)j * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(back.p[s_src]) + (size_t)s_dst * row_bytes);
    for (int u = threadIdx.x; u < (int)(row_bytes / 16); u += 256) dst[u] = src[u];
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
__global__ void ep_barrier_kernel(PeerPtrs flags, uint32_t* epoch, int rank, int world, int32_t* status) {
    __shared__ uint32_t e;
    if (threadIdx.x == 0) {
        e = *epoch + 1;
        *epoch = e;
        __threadfence_system();  // everything this rank wrote to its peers before the barrier is ordered before the flag
    }
    __syncthreads();
    if ((int)threadIdx.x < world) {
        volatile uint32_t* remote = static_cast<volatile uint32_t*>(flags.p[threadIdx.x]) + rank;
        *remote = e;
    }
    if ((int)threadIdx.x < world) {
        volatile uint32_t* mine = static_cast<volatile uint32_t*>(flags.p[rank]) + threadIdx.x;
        const long long t0 = clock64();
        while ((int32_t)(*mine - e) < 0) {
            if ((unsigned long long)(clock64() - t0) > kWaitCycles) {
                atomicExch(status, kErrTimeout);
                break;
            }
        }
    }
    __syncthreads();
    __threadfence_system();
}

}  // namespace
}  // namespace iq

using namespace iq;

// Opaque per-rank state of the exchange: the peers' buffers and a small device block (plan, epoch).
struct iq_ep {
    iq_ctx* ctx = nullptr;
    int32_t rank = 0, world = 1, experts = 0;
    PeerPtrs recv, back, flags, counts;
    EpPlan* plan = nullptr;   // device
    uint32_t* epoch = nullptr;  // device
};

extern "C" int32_t iq_ep_create(iq_ctx* ctx, int32_t rank, int32_t world, int32_t experts, void* const* peer_recv,
                                void* const* peer_back, void* const* peer_flags, void* const* peer_counts, iq_ep** out) {
    if (ctx == nullptr || out == nullptr) return kErrInvalidArg;
    *out = nullptr;
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || experts < world || experts % world != 0 ||
        world * (experts / world) > kMaxSegs || peer_recv == nullptr || peer_back == nullptr || peer_flags == nullptr || peer_counts == nullptr)
        return fail(ctx, kErrInvalidArg, "ep_create: rank %d of %d, %d experts", rank, world, experts);
    iq_ep* ep = new (std::nothrow) iq_ep();
    if (ep == nullptr) return kErrCuda;
    ep->ctx = ctx; ep->rank = rank; ep->world = world; ep->experts = experts;
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
    ep_plan_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(counts_all, ep->rank, ep->world, ep->experts, ep->plan);
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_plan launch");
}

extern "C" int32_t iq_ep_barrier(iq_ep* ep, void* stream) {
    if (ep == nullptr) return kErrInvalidArg;
    ep_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(ep->flags, ep->epoch, ep->rank, ep->world,
                                                                           ep->ctx->d_status);
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
    ep_pack_push_kernel<<<P, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, x_dtype, ldx, inds, pos, offsets, ep->plan,
                                                                             ep->recv, P, d_model, top_k,
                                                                             ep->experts / ep->world);
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_pack_push launch");
}

extern "C" int32_t iq_ep_return_push(iq_ep* ep, void* stream, const void* yd, int32_t yd_dtype, int32_t max_rows,
                                     int32_t d_model) {
    if (ep == nullptr) return kErrInvalidArg;
    if (yd == nullptr || max_rows < 1 || (yd_dtype != kF32 && yd_dtype != kF16) || d_model % 8 != 0)
        return fail(ep->ctx, kErrInvalidArg, "ep_return_push: arguments");
    ep_return_push_kernel<<<max_rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        yd, yd_dtype == kF32 ? 4 : 2, ep->plan, ep->back, d_model, ep->world, ep->experts / ep->world);
    return check_cuda(ep->ctx, cudaGetLastError(), "ep_return_push launch");
}
