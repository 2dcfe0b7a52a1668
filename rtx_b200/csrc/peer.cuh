// Barrier among the ranks of one node through flag words in peer-mapped memory: one launch per rank (each on its own
// GPU), thread t of the single CTA deals with rank t.  It publishes this rank's epoch (the count of barriers it has
// run, kept in device memory) in rank t's flag array (a
// release store at system scope: everything this rank's earlier kernels on the stream wrote, also into peer
// memory, is visible to whoever acquires the flag) and then waits, with the bounded wait every kernel here uses,
// until rank t's epoch has arrived in this rank's own array.  A rank that never arrives makes the wait run out:
// the kernel records kStatusWaitPeer in the status word and returns; nothing traps.  Replaces a one-word NCCL
// all-reduce (20-40 us on the stream) where only the ordering is wanted.  No counterpart in the reference.
#pragma once

#include "common.cuh"

namespace rtxb {

constexpr int kMaxPeers = 8;

struct PeerFlags {
  int* rank_flags[kMaxPeers];   // rank_flags[t]: rank t's array of kMaxPeers words (peer-mapped), [this rank] is ours to write
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerFlags flags, int world, int rank, int* epoch_counter,
                                                          uint64_t limit_ns, int* status) {
  // The epoch lives on the device (this rank's own counter, advanced by every barrier it runs): the launch carries
  // no per-call number, so the same launch can sit in a captured CUDA graph and be replayed.
  __shared__ int epoch_now;
  if (threadIdx.x == 0) epoch_now = atomicAdd(epoch_counter, 1) + 1;
  __syncwarp();
  const int epoch = epoch_now;
  const int t = threadIdx.x;
  if (t >= world) return;
  int* theirs = flags.rank_flags[t] + rank;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const int* mine = flags.rank_flags[rank] + t;
  uint64_t start = 0;
  uint32_t polls = 0;
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (seen - epoch >= 0) break;          // epochs only grow; the difference form survives wrap-around
    if ((++polls & 0x3F) == 0) {
      const uint64_t now = global_timer_ns();
      if (start == 0) start = now;
      else if (now - start > limit_ns) {
        if (status) atomicCAS(status, 0, kStatusWaitPeer);
        break;
      }
    }
  }
}

}  // namespace rtxb
