// Tensor-parallel exchange through peer-mapped memory (one process per GPU, NVLink / NVSwitch).
//
// A row-parallel projection leaves every rank with a partial sum of the same [M, D] output.
// Instead of handing that tensor to a collective library, the producing kernel stores its
// partial straight into a mailbox in every rank's memory; the kernel that consumes the sum
// (residual add + RMSNorm + activation quantisation) polls its own mailbox, adds the partials in
// rank order (so every rank computes bit-identical hidden states) and goes on.  A decode step
// therefore contains no collective call, no fence and no extra launch for the reduction.  The
// reference has no multi-GPU path at all.
//
// Protocol: every value travels as an 8-byte word {float value, uint32 tag} written with one
// aligned 8-byte store, which the memory system never splits, so a reader that sees the expected
// tag also sees the value: no flag, no memory fence, no ordering between stores is needed (the
// scheme low-latency collectives use for small messages).  Exchanges are numbered by an epoch
// kept in device memory (so a CUDA-graph replay needs no new arguments); exchange e is tagged
// e + 1 and uses mailbox slot e % TP_SLOTS.  A rank cannot send e + 1 before it has consumed e,
// and cannot consume e + 1 before every rank has sent it, so no rank is ever more than one
// exchange ahead: a slot is rewritten at the earliest TP_SLOTS - 1 exchanges after it was read.
// The consumer's polling is bounded by TP_WAIT_NS; on expiry it records the rank it was waiting
// for in `status`, treats the missing values as zero and carries on (nothing traps or hangs).
#pragma once
#include "common.cuh"

#define TP_MAX_RANKS 8
#define TP_SLOTS 4
#define TP_WAIT_NS 2000000000ull

struct TpPush {
    float2* mailbox[TP_MAX_RANKS];     // rank r's mailbox as mapped here: [TP_SLOTS][size][max_rows * max_d] words
    unsigned* epoch;                   // local: number of exchanges completed (advanced by the consumer)
    unsigned* ticket;                  // local: consumer CTAs that have finished the current exchange
    int* status;                       // local: 0, or 1 + the rank whose data never arrived
    int rank, size;
    long src_stride;                   // words between two sources inside a slot (= max_rows * max_d)
    long slot_stride;                  // words between two slots (= size * src_stride)
};

// Sequence-parallel prefill: tokens are dealt to ranks in contiguous shards of `shard` rows.
//  * GEMM -> reduce-scatter: the epilogue of a row-parallel GEMM stores each output tile (rounded
//    to bf16 to halve the NVLink bytes; the owner adds in f32) into this rank's slot of the accumulator of the rank that owns
//    the tile's tokens, then bumps that rank's arrival counter (one release per CTA).
//  * The owner waits for `size x tiles` arrivals, adds the slots in rank order (so the sum does not
//    depend on arrival order) into its shard of the residual stream, normalises, and stores the
//    bf16 rows into every rank's gathered buffer (all-gather), bumping the per-source arrival
//    counter there.
//  * All-gather -> GEMM: the TMA producer of the next (column-parallel) GEMM waits, per token
//    tile, only for the shard that tile belongs to, so tiles of early shards start at once.
// Counters only ever grow; the targets to wait for live in local device memory and are advanced
// by the kernel that precedes the waiter in stream order, so graph replays need no new arguments.
// Two accumulators alternate, so a fast rank's next reduction never lands in rows being read.
//
// Expert-parallel dispatch / combine on the same buffers and counters (mixture-of-experts layers whose experts are
// dealt to the ranks in equal ranges): the owner normalises its rows locally, routes them, and stores each row only
// into the gathered buffers of the ranks that hold one of its chosen experts, while the small routing records (expert
// ids and weights of every token) go to every rank; arrivals are counted as for the full all-gather, so the waiters do
// not change.  On the way back a rank stores partial sums only for the tokens it computed, and the owner adds only the
// slots of the ranks its routing record names.
#define TP_ROUTE_KMAX 8
struct TpSeq {
    bf16* acc[TP_MAX_RANKS];             // rank r's accumulators as mapped here: [2][size][shard * ld] bf16, one slot per source
    unsigned* rs_arrive[TP_MAX_RANKS];   // rank r's reduce-scatter arrival counter (one word)
    bf16* xfull[TP_MAX_RANKS];           // rank r's gathered activations: [size * shard, ld] bf16
    unsigned* ag_arrive[TP_MAX_RANKS];   // rank r's all-gather arrival counters: [size], one per source
    int* route_ids[TP_MAX_RANKS];        // rank r's routing records: expert ids [size * shard * k] (row stride k <= TP_ROUTE_KMAX)
    float* route_w[TP_MAX_RANKS];        // ... and their weights
    unsigned* rs_target;                 // local: arrivals the next consumer must see
    unsigned* ag_target;                 // local: per-source arrivals the next GEMM must see
    unsigned* rs_phase;                  // local: reductions consumed so far (parity picks the accumulator)
    unsigned* ticket;                    // local: [0] GEMM CTAs done, [1] consumer CTAs done
    int* status;                         // local: 0, or a code telling which wait ran out
    int rank, size, shard;
    long ld;                             // row length of acc / xfull (the hidden size)
};

#ifdef __CUDACC__
__device__ __forceinline__ void red_release_inc_sys(unsigned* p) {
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns();
// Spin until *p - target >= 0 (wrap-safe) or TP_WAIT_NS has passed; false on expiry.
__device__ __forceinline__ bool tp_wait_counter(const unsigned* p, unsigned target);
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Two neighbouring {value, tag} words in one 16-byte load that bypasses L1 (the words are written
// by other GPUs, so a cached line could be stale for ever).
__device__ __forceinline__ uint4 ld_words2(const float2* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool tp_wait_counter(const unsigned* p, unsigned target) {
    if ((int)(ld_acquire_sys_u32(p) - target) >= 0) return true;
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    while ((int)(ld_acquire_sys_u32(p) - target) < 0) {
        __nanosleep(64);
        if ((++spins & 63u) == 0 && global_timer_ns() - t0 > TP_WAIT_NS) return false;
    }
    return true;
}
__device__ __forceinline__ void st_word(float2* p, float value, unsigned tag) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(__float_as_uint(value)), "r"(tag) : "memory");
}
#endif
