// Context-parallel prefill attention: the sequence is dealt to ranks in contiguous shards, every rank
// keeps the K / V of its own shard, and a rank's queries attend to the shards of all lower ranks plus
// (causally) their own.  A remote shard crosses NVLink once: the owner publishes it in a peer-mapped
// staging buffer, the consumer pulls it into local memory with plain peer loads and runs the ordinary
// flash-attention kernel on the local copy, and the per-shard partial results are merged with their
// log-sum-exp weights.  The reference has no multi-device attention.
//
// Hand-shake (counters only grow, all waits are bounded, nothing traps):
//   ready[dst][src]  bumped by `src` on every higher rank `dst` once its staging holds call e's shard
//   done[src]        bumped on `src` by every higher rank once it has pulled call e's shard
// A source reuses its two staging halves alternately and waits, before overwriting a half, until all
// readers of the call that last used it have pulled (a low rank never waits for anything else, so
// without this it could run several calls ahead of a slow high rank).
#include "tp_fused.cuh"

struct CpRing {
    bf16* stage[TP_MAX_RANKS];          // rank r's staging as mapped here: [2 halves][2 (K, V)][max_shard * kv_row]
    unsigned* ready[TP_MAX_RANKS];      // rank r's ready counters: [size], one per source
    unsigned* done[TP_MAX_RANKS];       // rank r's done counter (one word)
    unsigned* epoch;                    // local: calls published so far
    int* status;                        // local: 0, or a code telling which wait ran out
    int rank, size;
    long half_stride;                   // elements between the two staging halves (= 2 * max_shard * kv_row)
    long kv_stride;                     // elements between K and V inside a half (= max_shard * kv_row)
};

extern "C" int tsb_cp_struct_bytes() { return (int)sizeof(CpRing); }
// Symmetric region of one rank: counters in the first 256 bytes (ready[size] at +0, done at +128), then staging.
extern "C" long tsb_cp_region_bytes(long max_shard, long kv_row) { return 256 + 4L * max_shard * kv_row * 2; }

extern "C" int tsb_cp_init(void* dev_struct, void* const* regions, void* local, int rank, int size, long max_shard, long kv_row) {
    TSB_CHECK_ARG(dev_struct && regions && local, "cp_init: null argument");
    TSB_CHECK_ARG(size >= 1 && size <= TP_MAX_RANKS && rank >= 0 && rank < size, "cp_init: rank %d of %d", rank, size);
    TSB_CHECK_ARG(max_shard > 0 && kv_row > 0 && kv_row % 8 == 0, "cp_init: bad sizes");
    CpRing h = {};
    for (int r = 0; r < size; ++r) {
        unsigned char* base = (unsigned char*)regions[r];
        h.ready[r] = (unsigned*)base;
        h.done[r] = (unsigned*)(base + 128);
        h.stage[r] = (bf16*)(base + 256);
    }
    unsigned* c = (unsigned*)local;
    h.epoch = c; h.status = (int*)(c + 4);
    h.rank = rank; h.size = size;
    h.kv_stride = max_shard * kv_row;
    h.half_stride = 2 * h.kv_stride;
    TSB_CHECK_CUDA(cudaMemset(local, 0, 8 * sizeof(unsigned)));
    TSB_CHECK_CUDA(cudaMemcpy(dev_struct, &h, sizeof(h), cudaMemcpyHostToDevice));
    TSB_CHECK_CUDA(cudaDeviceSynchronize());
    return TSB_OK;
}

// Copy this rank's K and V shard ([n, kv_row] each) into its staging half and tell the higher ranks.
__global__ void __launch_bounds__(256) cp_publish_kernel(const CpRing* g, const bf16* k, const bf16* v, long n_elems) {
    __shared__ int s_ok;
    pdl_wait();
    pdl_trigger();
    const unsigned e = *g->epoch;
    const int readers = g->size - 1 - g->rank;
    if (threadIdx.x == 0) {
        // the half was last used by call e - 2: all its readers must have pulled
        s_ok = 1;
        if (e >= 2 && readers > 0 && !tp_wait_counter(g->done[g->rank], (e - 1) * (unsigned)readers)) {
            s_ok = 0;
            atomicCAS(g->status, 0, 30);
        }
    }
    __syncthreads();
    if (!s_ok) return;                  // a reader may still be inside this half: leave it alone, the status word says why
    bf16* dst = g->stage[g->rank] + (long)(e & 1u) * g->half_stride;
    const long vecs = n_elems / 8;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (long)gridDim.x * blockDim.x) {
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(k)[i];
        reinterpret_cast<uint4*>(dst + g->kv_stride)[i] = reinterpret_cast<const uint4*>(v)[i];
    }
}
// Runs after cp_publish_kernel in the same stream: everything is in local memory by then, so one
// thread raises the flags and advances the call counter.
__global__ void cp_signal_kernel(const CpRing* g) {
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int d = g->rank + 1; d < g->size; ++d) red_release_inc_sys(g->ready[d] + g->rank);
        *g->epoch = *g->epoch + 1;
    }
}

// Pull rank `src`'s shard of the current call into local memory and release the source.
__global__ void __launch_bounds__(256) cp_pull_kernel(const CpRing* g, int src, bf16* k_out, bf16* v_out, long n_elems,
                                                      unsigned* ticket) {
    __shared__ int s_ok;
    pdl_wait();
    pdl_trigger();
    const unsigned e = *g->epoch - 1;                       // cp_signal already advanced it for this call
    if (threadIdx.x == 0) {
        s_ok = tp_wait_counter(g->ready[g->rank] + src, e + 1) ? 1 : 0;
        if (!s_ok) atomicCAS(g->status, 0, 40 + src);
    }
    __syncthreads();
    const bf16* from = g->stage[src] + (long)(e & 1u) * g->half_stride;
    const long vecs = n_elems / 8;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (long)gridDim.x * blockDim.x) {
        uint4 a, b;                                          // peer memory: keep it out of L1
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w)
                     : "l"(reinterpret_cast<const uint4*>(from) + i) : "memory");
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
                     : "l"(reinterpret_cast<const uint4*>(from + g->kv_stride) + i) : "memory");
        reinterpret_cast<uint4*>(k_out)[i] = a;
        reinterpret_cast<uint4*>(v_out)[i] = b;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(ticket, 1u);
        if (t == gridDim.x - 1) {                            // every block has finished reading the source
            *ticket = 0;
            red_release_inc_sys(g->done[src]);
        }
    }
}

// out[t, h, :] = sum_s exp(lse_s - M) * o_s / sum_s exp(lse_s - M); parts are [S][T, H, Dh] bf16 and [S][T, H] f32.
__global__ void __launch_bounds__(128) cp_merge_kernel(const bf16* parts, const float* lse, bf16* out, int S, long TH, int Dh) {
    pdl_wait();
    pdl_trigger();
    const long th = blockIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < S; ++s) M = fmaxf(M, lse[(long)s * TH + th]);
    float wsum = 0.f;
    for (int s = 0; s < S; ++s) {
        const float l = lse[(long)s * TH + th];
        wsum += (l == -INFINITY) ? 0.f : __expf(l - M);
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    for (int d = threadIdx.x; d < Dh; d += 128) {
        float acc = 0.f;
        for (int s = 0; s < S; ++s) {
            const float l = lse[(long)s * TH + th];
            if (l != -INFINITY) acc += __expf(l - M) * __bfloat162float(parts[((long)s * TH + th) * Dh + d]);
        }
        out[th * Dh + d] = __float2bfloat16(acc * inv);
    }
}

extern "C" int tsb_cp_publish(const void* g, const void* k, const void* v, long n_elems, void* stream) {
    TSB_CHECK_ARG(g && k && v && n_elems > 0 && n_elems % 8 == 0, "cp_publish: bad arguments");
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (int)((n_elems / 8 + 255) / 256 < 592 ? (n_elems / 8 + 255) / 256 : 592);
    TSB_CHECK_CUDA(tsb_launch(cp_publish_kernel, dim3(blocks), dim3(256), 0, s, (const CpRing*)g, (const bf16*)k, (const bf16*)v, n_elems));
    TSB_CHECK_CUDA(tsb_launch(cp_signal_kernel, dim3(1), dim3(32), 0, s, (const CpRing*)g));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}
extern "C" int tsb_cp_pull(const void* g, int src, void* k_out, void* v_out, long n_elems, void* ticket, void* stream) {
    TSB_CHECK_ARG(g && k_out && v_out && ticket && n_elems > 0 && n_elems % 8 == 0, "cp_pull: bad arguments");
    const int blocks = (int)((n_elems / 8 + 255) / 256 < 592 ? (n_elems / 8 + 255) / 256 : 592);
    TSB_CHECK_CUDA(tsb_launch(cp_pull_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const CpRing*)g, src,
                              (bf16*)k_out, (bf16*)v_out, n_elems, (unsigned*)ticket));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}
extern "C" int tsb_cp_merge(const void* parts, const float* lse, void* out, int S, long TH, int Dh, void* stream) {
    TSB_CHECK_ARG(parts && lse && out && S >= 1 && TH > 0 && Dh > 0, "cp_merge: bad arguments");
    TSB_CHECK_CUDA(tsb_launch(cp_merge_kernel, dim3((unsigned)TH), dim3(128), 0, (cudaStream_t)stream, (const bf16*)parts, lse,
                              (bf16*)out, S, TH, Dh));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}
