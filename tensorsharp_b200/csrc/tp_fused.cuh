// Tensor-parallel exchange through peer-mapped memory (one process per GPU, NVLink / NVSwitch).
//
// A row-parallel projection leaves every rank with a partial sum of the same [M, D] output.
// Instead of handing that tensor to a collective library, the producing kernel stores its
// partial straight into a mailbox in every rank's memory and raises a flag there; the kernel
// that consumes the sum (residual add + RMSNorm + activation quantisation) waits for the flags
// of all ranks, adds the partials in rank order (so every rank computes bit-identical hidden
// states) and goes on.  A decode step therefore contains no collective call and no extra
// launch for the reduction.  The reference has no multi-GPU path at all.
//
// Protocol.  Exchanges are numbered by an epoch that both sides keep in device memory (so a
// CUDA-graph replay needs no new arguments).  Exchange e uses mailbox slot e % TP_SLOTS.  A
// rank cannot send e+1 before it has consumed e, and cannot consume e+1 before every rank has
// sent it, so no rank is ever more than one exchange ahead and two slots would suffice.
// Producer CTAs: store partials to all ranks, fence at system scope, take a ticket; the last
// CTA publishes flag[rank] = e+1 on every rank with a release store.  Consumer: acquire-load
// its own flags until all are >= e+1, bounded by TP_WAIT_NS; on expiry it records the rank it
// was waiting for in `status` and carries on with what is there (nothing traps or hangs).
#pragma once
#include "common.cuh"

#define TP_MAX_RANKS 8
#define TP_SLOTS 4
#define TP_WAIT_NS 2000000000ull

struct TpPush {
    float* mailbox[TP_MAX_RANKS];      // rank r's mailbox base as mapped here: [TP_SLOTS][size][max_rows * max_d]
    unsigned* flags[TP_MAX_RANKS];     // rank r's flag array as mapped here: [size] last epoch sent by each source
    unsigned* epoch_send;              // local counters
    unsigned* epoch_recv;
    unsigned* ticket_send;
    unsigned* ticket_recv;
    int* status;                       // 0, or 1 + the rank whose flag never arrived
    int rank, size;
    long src_stride;                   // floats between two sources inside a slot (= max_rows * max_d)
    long slot_stride;                  // floats between two slots (= size * src_stride)
};

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Call from every thread of the CTA after its stores to peer memory.  The last CTA of the
// grid publishes the epoch on every rank and advances the local send counter.
__device__ __forceinline__ void tp_publish(const TpPush* tp, unsigned epoch, unsigned n_ctas) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(tp->ticket_send, 1u);
        if (t == n_ctas - 1) {
            __threadfence_system();
            for (int r = 0; r < tp->size; ++r) st_release_sys(tp->flags[r] + tp->rank, epoch + 1);
            *tp->ticket_send = 0;
            *tp->epoch_send = epoch + 1;
        }
    }
}
#endif
