// Two tiny kernels that make a bounded wait run out, for the test of the tear-down path that every
// tensor-core kernel of this folder shares: a wait on an mbarrier that nobody arrives on gives up
// after the library's limit, sets the block's abort flag, the block leaves in order and the error
// word in global memory tells the host.  Nothing here copies, uses tensor memory, traps or spins
// without limit: the kernels return by themselves.
//
//   probe_single:  one block; one thread waits (tc::mbar_wait, the helper the kernels use), the
//                  other warps poll the abort flag as the kernels' other roles do.
//   probe_cluster: a cluster of two blocks shaped like the decode attention's merge: block 0 waits
//                  (tc::mbar_wait_cluster) for a signal that block 1 never sends; block 1 spends a
//                  bounded number of clock cycles and exits.  Block 0 gives up, reports, and leaves
//                  through the cluster's hardware barrier, which completes once block 1 has exited.
//
// The reference has no counterpart: its kernels wait on nothing (one launch per operation).
#include "common.cuh"
#include "tc_common.cuh"

namespace {

__global__ void probe_single(int* err, int* trace) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    abort_flag = 0;
    tc::mbar_fence_init();
  }
  __syncthreads();
  volatile int* af = &abort_flag;
  bool ok = true;
  if (threadIdx.x == 0) {
    ok = tc::mbar_wait(&bar, 0, af);               // nobody arrives
    trace[0] = ok ? 1 : 2;
  } else {
    // the other roles: bounded polling of the abort flag
    const uint32_t limit = tc::c_wait_limit;
    for (uint32_t i = 0; i < 4u * limit && !*af; ++i) __nanosleep(64);
    if (threadIdx.x == 32) trace[1] = *af ? 2 : 1;
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && err) atomicExch(err, 1);
}

__global__ void __cluster_dims__(2, 1, 1) probe_cluster(int* err, int* trace, int peer_cycles) {
  __shared__ uint64_t merge_bar;
  __shared__ int abort_flag;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  if (threadIdx.x == 0) {
    tc::mbar_init(&merge_bar, 1);
    abort_flag = 0;
    tc::mbar_fence_init();
  }
  __syncthreads();
  tc::cluster_arrive();
  tc::cluster_wait();                               // both blocks' barriers exist
  if (rank != 0) {
    // the peer: works for a bounded while, never signals, exits
    const long long t0 = clock64();
    while (clock64() - t0 < (long long)peer_cycles) {}
    if (threadIdx.x == 0) trace[3] = 1;
    return;
  }
  volatile int* af = &abort_flag;
  const bool ok = tc::mbar_wait_cluster(&merge_bar, 0, af);
  if (threadIdx.x == 0) trace[2] = ok ? 1 : 2;
  if (!ok) {
    if (threadIdx.x == 0 && err) atomicExch(err, 1);
    tc::cluster_arrive();                           // completes when the peer has arrived or exited
    tc::cluster_wait();
    if (threadIdx.x == 0) trace[4] = 1;
  }
}

}  // namespace

SGLC_DEFINE_ERROR_STRING()

// Runs both probes with a wait limit of `polls` (then puts the library's default back).
// err: the error word the tensor-core kernels report in; trace: 5 ints
// [waiter's outcome, other warps' outcome, cluster waiter's outcome, peer left, waiter left]
// (1 = the wait succeeded / the peer ran, 2 = the wait ran out).
SGLC_API int sglc_wait_probe(int* err, int* trace, unsigned polls, int peer_cycles, cudaStream_t stream) {
  int e = tc::set_wait_limit(polls);
  if (e != 0) return e;
  probe_single<<<1, 128, 0, stream>>>(err, trace);
  e = (int)cudaGetLastError();
  if (e == 0) {
    probe_cluster<<<2, 64, 0, stream>>>(err, trace, peer_cycles);
    e = (int)cudaGetLastError();
  }
  cudaStreamSynchronize(stream);
  const int e2 = tc::set_wait_limit(1u << 22);
  return e ? e : e2;
}
