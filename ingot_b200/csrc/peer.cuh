// Pieces shared by the kernels that talk to other GPUs of the box through peer-addressable memory (the expert-parallel
// exchange, the column-split linear): the array of per-rank pointers and the flag barrier. Plain loads and stores only:
// no TMA and no multicast touches a peer's memory.
#pragma once

#include <stdint.h>

#include "common.cuh"

namespace iq {

constexpr int kMaxRanks = 8;

struct PeerPtrs {
    void* p[kMaxRanks];
};

// Barrier over the ranks of the box, run by the first `world` threads of one block (call it from all threads of the
// block: it ends with __syncthreads). Every rank publishes epoch `e` into slot `rank` of every peer's flag array and
// waits until every slot of its own array has reached `e`. Epochs only grow, so a kernel that uses it can be replayed
// from a CUDA graph. Everything this rank stored to its peers before the call is visible to them once they have seen
// the flag. The wait is bounded: after wait_cycles the status word is set to kErrTimeout and the block goes on.
__device__ __forceinline__ void peer_flag_barrier(const PeerPtrs& flags, uint32_t e, int rank, int world, int32_t* status,
                                                  unsigned long long wait_cycles) {
    __syncthreads();  // every thread's peer stores are done; the fence below, by the flag writers, covers them
    if ((int)threadIdx.x < world) {
        __threadfence_system();
        volatile uint32_t* remote = static_cast<volatile uint32_t*>(flags.p[threadIdx.x]) + rank;
        *remote = e;
        volatile uint32_t* mine = static_cast<volatile uint32_t*>(flags.p[rank]) + threadIdx.x;
        const long long t0 = clock64();
        while ((int32_t)(*mine - e) < 0) {
            if ((unsigned long long)(clock64() - t0) > wait_cycles) {
                atomicExch(status, kErrTimeout);
                break;
            }
        }
        __threadfence_system();  // what the peers stored before their flags is read after this point
    }
    __syncthreads();
}

}  // namespace iq
