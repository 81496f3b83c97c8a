// Peer-memory plumbing and the consumer side of the tensor-parallel exchange (see tp_fused.cuh).
#include "tp_fused.cuh"

// ------------------------------------------------------------------------------------------
// Symmetric allocation: plain cudaMalloc memory exported with CUDA IPC.  The caller exchanges the
// 64-byte handles between ranks (any transport) and opens each peer's handle once.
// ------------------------------------------------------------------------------------------
extern "C" int tsb_symm_alloc(size_t bytes, void** out) {
    TSB_CHECK_ARG(bytes > 0 && out, "symm_alloc: bad arguments");
    TSB_CHECK_CUDA(cudaMalloc(out, bytes));
    TSB_CHECK_CUDA(cudaMemset(*out, 0, bytes));
    TSB_CHECK_CUDA(cudaDeviceSynchronize());
    return TSB_OK;
}
extern "C" int tsb_symm_free(void* p) {
    if (p) TSB_CHECK_CUDA(cudaFree(p));
    return TSB_OK;
}
extern "C" int tsb_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }
extern "C" int tsb_ipc_get_handle(void* p, void* handle_out) {
    TSB_CHECK_ARG(p && handle_out, "ipc_get_handle: bad arguments");
    TSB_CHECK_CUDA(cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle_out, p));
    return TSB_OK;
}
extern "C" int tsb_ipc_open(const void* handle, void** out) {
    TSB_CHECK_ARG(handle && out, "ipc_open: bad arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    TSB_CHECK_CUDA(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
    return TSB_OK;
}
extern "C" int tsb_ipc_close(void* p) {
    if (p) TSB_CHECK_CUDA(cudaIpcCloseMemHandle(p));
    return TSB_OK;
}
extern "C" int tsb_tp_struct_bytes() { return (int)sizeof(TpPush); }

// Fill a device-resident TpPush.  `mailboxes` holds `size` device addresses (the local one at
// index `rank`, peers as opened through IPC); `counters` is local memory of >= 8 words:
// [epoch, ticket, -, -, status].
extern "C" int tsb_tp_init(void* tp_dev, void* const* mailboxes, void* counters, int rank, int size, long max_rows,
                           long max_d) {
    TSB_CHECK_ARG(tp_dev && mailboxes && counters, "tp_init: null argument");
    TSB_CHECK_ARG(size >= 1 && size <= TP_MAX_RANKS && rank >= 0 && rank < size, "tp_init: rank %d of %d", rank, size);
    TpPush h = {};
    for (int r = 0; r < size; ++r) h.mailbox[r] = (float2*)mailboxes[r];
    unsigned* c = (unsigned*)counters;
    h.epoch = c; h.ticket = c + 1; h.status = (int*)(c + 4);
    h.rank = rank; h.size = size;
    h.src_stride = max_rows * max_d;
    h.slot_stride = h.src_stride * size;
    TSB_CHECK_CUDA(cudaMemset(counters, 0, 8 * sizeof(unsigned)));
    TSB_CHECK_CUDA(cudaMemcpy(tp_dev, &h, sizeof(h), cudaMemcpyHostToDevice));
    TSB_CHECK_CUDA(cudaDeviceSynchronize());
    return TSB_OK;
}
extern "C" long tsb_tp_mailbox_bytes(int size, long max_rows, long max_d) {
    return (long)TP_SLOTS * size * max_rows * max_d * (long)sizeof(float2);
}

// ------------------------------------------------------------------------------------------
// Consumer: h[m, :] += sum over ranks of partial_r[m, :]  (rank order), then optionally
// y = RMSNorm(h) * w as bf16 and / or as int8 groups of 32 with (scale, sum), the form the
// quantised GEMV kernels read.  One CTA per row; the last CTA advances the epoch.
// ------------------------------------------------------------------------------------------
// `parts` > 1: every source delivers `parts` partial rows per token (the top-k slots of a mixture of
// experts), laid out token-major, which are all added.
template <int NT>
__global__ void __launch_bounds__(NT) tp_reduce_norm_kernel(const TpPush* tp, float* h, const float* w, float eps, int D,
                                                            int rows, int parts, bf16* yb, int8_t* yq, float2* yds) {
    __shared__ float red[32];
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x;
    const unsigned epoch = *tp->epoch;              // written only by the last CTA of the previous exchange
    const unsigned tag = epoch + 1;
    const int size = tp->size;
    const float2* box = tp->mailbox[tp->rank] + (long)(epoch % TP_SLOTS) * tp->slot_stride + (long)m * parts * D;
    float* hr = h + (long)m * D;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < D; i += NT * 4) {
        float4 v = *reinterpret_cast<const float4*>(hr + i);
        for (int rp = 0; rp < size * parts; ++rp) {
            const int r = rp / parts;
            const float2* src = box + (long)r * tp->src_stride + (long)(rp % parts) * D + i;
            uint4 a = ld_words2(src), b = ld_words2(src + 2);
            if (a.y != tag || a.w != tag || b.y != tag || b.w != tag) {
                const unsigned long long t0 = global_timer_ns();
                unsigned spins = 0;
                bool late = false;
                do {
                    __nanosleep(32);
                    a = ld_words2(src);
                    b = ld_words2(src + 2);
                    // a wait that already ran out anywhere on this GPU ends all the others at once
                    if ((++spins & 63u) == 0 &&
                        (global_timer_ns() - t0 > TP_WAIT_NS || *(volatile int*)tp->status != 0)) { late = true; break; }
                } while (a.y != tag || a.w != tag || b.y != tag || b.w != tag);
                if (late) {
                    atomicCAS(tp->status, 0, 1 + r);
                    if (a.y != tag) a.x = 0u;
                    if (a.w != tag) a.z = 0u;
                    if (b.y != tag) b.x = 0u;
                    if (b.w != tag) b.z = 0u;
                }
            }
            v.x += __uint_as_float(a.x); v.y += __uint_as_float(a.z);
            v.z += __uint_as_float(b.x); v.w += __uint_as_float(b.z);
        }
        *reinterpret_cast<float4*>(hr + i) = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (w != nullptr || yb != nullptr || yq != nullptr) {
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)D + eps);
        // each thread re-reads the values it wrote itself: no barrier needed.  The loop bound is
        // uniform across the warp because the q8 group reduction shuffles over all 32 lanes.
        for (int base = 0; base < D; base += NT * 4) {
            const int i = base + threadIdx.x * 4;
            const bool ok = i < D;
            float4 n = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ok) {
                const float4 v = *reinterpret_cast<const float4*>(hr + i);
                n = make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv);
                if (w) {
                    const float4 g = *reinterpret_cast<const float4*>(w + i);
                    n.x *= g.x; n.y *= g.y; n.z *= g.z; n.w *= g.w;
                }
                if (yb) {
                    uint2 o;
                    *reinterpret_cast<bf162*>(&o.x) = __floats2bfloat162_rn(n.x, n.y);
                    *reinterpret_cast<bf162*>(&o.y) = __floats2bfloat162_rn(n.z, n.w);
                    *reinterpret_cast<uint2*>(yb + (long)m * D + i) = o;
                }
            }
            if (yq) {
                // a group of 32 values is 8 neighbouring lanes; same convention as the RMSNorm
                // kernel: int8 = round(n * 127 / amax), stored with (amax / 127, unrounded sum)
                float amax = fmaxf(fmaxf(fabsf(n.x), fabsf(n.y)), fmaxf(fabsf(n.z), fabsf(n.w)));
                float sum = n.x + n.y + n.z + n.w;
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                    sum += __shfl_xor_sync(0xffffffffu, sum, o);
                }
                if (ok) {
                    const float qi = amax > 0.f ? 127.f / amax : 0.f;
                    char4 q;
                    q.x = (signed char)__float2int_rn(n.x * qi);
                    q.y = (signed char)__float2int_rn(n.y * qi);
                    q.z = (signed char)__float2int_rn(n.z * qi);
                    q.w = (signed char)__float2int_rn(n.w * qi);
                    *reinterpret_cast<char4*>(yq + (long)m * D + i) = q;
                    if ((threadIdx.x & 7) == 0) yds[(long)m * (D >> 5) + (i >> 5)] = make_float2(amax / 127.f, sum);
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(tp->ticket, 1u);
        if (t == (unsigned)rows - 1) {
            *tp->ticket = 0;
            __threadfence();
            *tp->epoch = epoch + 1;
        }
    }
}

extern "C" int tsb_tp_reduce_norm(const void* tp, float* h, const float* w, float eps, int rows, int D, int parts,
                                  void* y_bf16, void* yq, void* yds, void* stream) {
    TSB_CHECK_ARG(tp && h && rows > 0 && D > 0 && parts >= 1, "tp_reduce_norm: bad arguments");
    TSB_CHECK_ARG(D % 32 == 0, "tp_reduce_norm: D=%d must be a multiple of 32", D);
    TSB_CHECK_ARG(!yq || yds, "tp_reduce_norm: q8 output needs the scale buffer");
    // NT*4 must cover whole groups of 32 per 8 lanes; D % 32 == 0 keeps all 8 lanes of a group in range together
    TSB_CHECK_CUDA(tsb_launch(tp_reduce_norm_kernel<256>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (const TpPush*)tp, h,
                              w, eps, D, rows, parts, (bf16*)y_bf16, (int8_t*)yq, (float2*)yds));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// All-reduce of a small tensor y [rows, D] (f32, in place) over the same mailboxes: every CTA first stores
// its row to every peer (tagged words), then polls its own mailbox and adds the ranks' rows in rank order, its
// own row taken from registers.  A CTA waits only for stores that the peers issue before their own waits, so
// CTAs need not be resident together.  The drop-in form of the exchange for model graphs that have no fused
// projection + norm pair (sandwich norms, recurrent layers, shared experts).
// ------------------------------------------------------------------------------------------
template <int NT>
__global__ void __launch_bounds__(NT) tp_all_reduce_kernel(const TpPush* tp, float* y, int D, int rows) {
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x;
    const unsigned epoch = *tp->epoch;
    const unsigned tag = epoch + 1;
    const int size = tp->size, rank = tp->rank;
    const long slot = (long)(epoch % TP_SLOTS) * tp->slot_stride;
    float* yr = y + (long)m * D;
    for (int i = threadIdx.x * 4; i < D; i += NT * 4) {
        const float4 v = *reinterpret_cast<const float4*>(yr + i);
        for (int r = 0; r < size; ++r) {
            if (r == rank) continue;
            float2* dst = tp->mailbox[r] + slot + (long)rank * tp->src_stride + (long)m * D + i;
            st_word(dst, v.x, tag); st_word(dst + 1, v.y, tag); st_word(dst + 2, v.z, tag); st_word(dst + 3, v.w, tag);
        }
    }
    const float2* box = tp->mailbox[rank] + slot + (long)m * D;
    for (int i = threadIdx.x * 4; i < D; i += NT * 4) {
        const float4 own = *reinterpret_cast<const float4*>(yr + i);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < size; ++r) {
            if (r == rank) { acc.x += own.x; acc.y += own.y; acc.z += own.z; acc.w += own.w; continue; }
            const float2* src = box + (long)r * tp->src_stride + i;
            uint4 a = ld_words2(src), b = ld_words2(src + 2);
            if (a.y != tag || a.w != tag || b.y != tag || b.w != tag) {
                const unsigned long long t0 = global_timer_ns();
                unsigned spins = 0;
                bool late = false;
                do {
                    __nanosleep(32);
                    a = ld_words2(src);
                    b = ld_words2(src + 2);
                    if ((++spins & 63u) == 0 &&
                        (global_timer_ns() - t0 > TP_WAIT_NS || *(volatile int*)tp->status != 0)) { late = true; break; }
                } while (a.y != tag || a.w != tag || b.y != tag || b.w != tag);
                if (late) {
                    atomicCAS(tp->status, 0, 1 + r);
                    if (a.y != tag) a.x = 0u;
                    if (a.w != tag) a.z = 0u;
                    if (b.y != tag) b.x = 0u;
                    if (b.w != tag) b.z = 0u;
                }
            }
            acc.x += __uint_as_float(a.x); acc.y += __uint_as_float(a.z);
            acc.z += __uint_as_float(b.x); acc.w += __uint_as_float(b.z);
        }
        *reinterpret_cast<float4*>(yr + i) = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(tp->ticket, 1u);
        if (t == (unsigned)rows - 1) {
            *tp->ticket = 0;
            __threadfence();
            *tp->epoch = epoch + 1;
        }
    }
}

extern "C" int tsb_tp_all_reduce(const void* tp, float* y, int rows, int D, void* stream) {
    TSB_CHECK_ARG(tp && y && rows > 0 && D > 0, "tp_all_reduce: bad arguments");
    TSB_CHECK_ARG(D % 4 == 0, "tp_all_reduce: D=%d must be a multiple of 4", D);
    TSB_CHECK_ARG(((uintptr_t)y & 15) == 0, "tp_all_reduce: y must be 16-byte aligned");
    TSB_CHECK_CUDA(tsb_launch(tp_all_reduce_kernel<256>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (const TpPush*)tp, y, D, rows));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// Host-visible status word: 0 = every wait was satisfied.
extern "C" int tsb_tp_status(void* counters, int* out) {
    TSB_CHECK_ARG(counters && out, "tp_status: bad arguments");
    TSB_CHECK_CUDA(cudaMemcpy(out, (unsigned*)counters + 4, sizeof(int), cudaMemcpyDeviceToHost));
    return TSB_OK;
}

// ==========================================================================================
// Sequence-parallel prefill (TpSeq, tp_fused.cuh)
// ==========================================================================================
extern "C" int tsb_tpseq_struct_bytes() { return (int)sizeof(TpSeq); }

// Layout of one rank's symmetric region, in bytes from its base:
//   [0, 256)                      counters: rs_arrive at +0, ag_arrive[size] at +64
//   [256, 256 + 2*size*shard*ld*2)  the two bf16 accumulators, one slot per source rank
//   then                            xfull: size*shard*ld bf16
//   then                            routing records: size*shard*TP_ROUTE_KMAX expert ids (int32), then as many weights (f32)
extern "C" long tsb_tpseq_region_bytes(int size, int shard, long ld) {
    return 256 + 2L * size * shard * ld * 2 + (long)size * shard * ld * 2 + 2L * size * shard * TP_ROUTE_KMAX * 4;
}
extern "C" long tsb_tpseq_route_offset(int size, int shard, long ld) {
    return 256 + 2L * size * shard * ld * 2 + (long)size * shard * ld * 2;
}
extern "C" int tsb_tpseq_route_kmax() { return TP_ROUTE_KMAX; }

// `regions` holds `size` device addresses of the symmetric regions (local one at index rank);
// `local` is private device memory of >= 16 words: [rs_target, ag_target, rs_phase, -, ticket0,
// ticket1, -, -, status].
extern "C" int tsb_tpseq_init(void* dev_struct, void* const* regions, void* local, int rank, int size, int shard, long ld) {
    TSB_CHECK_ARG(dev_struct && regions && local, "tpseq_init: null argument");
    TSB_CHECK_ARG(size >= 1 && size <= TP_MAX_RANKS && rank >= 0 && rank < size, "tpseq_init: rank %d of %d", rank, size);
    TSB_CHECK_ARG(shard > 0 && shard % 128 == 0 && ld > 0 && ld % 8 == 0, "tpseq_init: shard=%d ld=%ld", shard, ld);
    // the arrival counters are bumped with reductions on peer memory: refuse to set up where the
    // link does not execute atomics natively
    int me = 0;
    TSB_CHECK_CUDA(cudaGetDevice(&me));
    for (int r = 0; r < size; ++r) {
        if (r == rank) continue;
        cudaPointerAttributes pa;
        TSB_CHECK_CUDA(cudaPointerGetAttributes(&pa, regions[r]));
        int native_atomics = 0;
        if (pa.device != me) TSB_CHECK_CUDA(cudaDeviceGetP2PAttribute(&native_atomics, cudaDevP2PAttrNativeAtomicSupported, me, pa.device));
        TSB_CHECK_ARG(pa.device == me || native_atomics, "tpseq_init: no native peer atomics between device %d and %d", me, pa.device);
    }
    TpSeq h = {};
    for (int r = 0; r < size; ++r) {
        unsigned char* base = (unsigned char*)regions[r];
        h.rs_arrive[r] = (unsigned*)base;
        h.ag_arrive[r] = (unsigned*)(base + 64);
        h.acc[r] = (bf16*)(base + 256);
        h.xfull[r] = (bf16*)(base + 256 + 2L * size * shard * ld * 2);
        h.route_ids[r] = (int*)(base + tsb_tpseq_route_offset(size, shard, ld));
        h.route_w[r] = (float*)(h.route_ids[r] + (long)size * shard * TP_ROUTE_KMAX);
    }
    unsigned* c = (unsigned*)local;
    h.rs_target = c; h.ag_target = c + 1; h.rs_phase = c + 2; h.ticket = c + 4; h.status = (int*)(c + 8);
    h.rank = rank; h.size = size; h.shard = shard; h.ld = ld;
    TSB_CHECK_CUDA(cudaMemset(local, 0, 16 * sizeof(unsigned)));
    TSB_CHECK_CUDA(cudaMemcpy(dev_struct, &h, sizeof(h), cudaMemcpyHostToDevice));
    TSB_CHECK_CUDA(cudaDeviceSynchronize());
    return TSB_OK;
}

// One CTA per row of this rank's shard:
//   has_acc: wait for the reduce-scatter arrivals, h[r] += sum over sources of acc[phase][src][r]
//   then     y = RMSNorm(h[r]) * w  (bf16) stored into row (rank * shard + r) of every rank's gathered
//            buffer, and one arrival per destination.
// The last CTA advances the all-gather target (and the reduction phase).
//   local_only: the normalised rows go to this rank's own gathered buffer and nothing is announced (the expert
//               dispatch that follows sends them on and counts the arrivals);
//   acc_k > 0:  the accumulators hold the expert combine: only the slots of the ranks that own one of the row's acc_k
//               chosen experts (its routing record; `epr` experts per rank) were written, and only those are added.
template <int NT>
__global__ void __launch_bounds__(NT) tp_seq_norm_gather_kernel(const TpSeq* g, float* h, const float* w, float eps,
                                                                int has_acc, int local_only, int acc_k, int epr) {
    __shared__ float red[32];
    __shared__ int s_ok;
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, D = (int)g->ld;
    const unsigned phase = *g->rs_phase;
    if (has_acc) {
        if (threadIdx.x == 0) {
            s_ok = tp_wait_counter(g->rs_arrive[g->rank], *g->rs_target) ? 1 : 0;
            if (!s_ok) atomicCAS(g->status, 0, 10);
        }
        __syncthreads();
    }
    float* hr = h + (long)r * D;
    const long slot = (long)g->shard * D;
    const bf16* ar = g->acc[g->rank] + (long)(phase & 1u) * g->size * slot + (long)r * D;
    unsigned srcs = 0xffffffffu;                        // sources whose slot of this row was written
    if (has_acc && acc_k > 0) {
        srcs = 0u;
        const int* rid = g->route_ids[g->rank] + ((long)g->rank * g->shard + r) * acc_k;
        for (int j = 0; j < acc_k; ++j) {
            const int e = rid[j];
            if (e >= 0) srcs |= 1u << (e / epr);
        }
    }
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < D; i += NT * 4) {
        float4 v = *reinterpret_cast<const float4*>(hr + i);
        if (has_acc) {
            for (int src = 0; src < g->size; ++src) {
                if (!((srcs >> src) & 1u)) continue;
                const uint2 a = __ldcg(reinterpret_cast<const uint2*>(ar + src * slot + i));   // remote stores: skip L1
                const float2 lo = __bfloat1622float2(*reinterpret_cast<const bf162*>(&a.x));
                const float2 hi = __bfloat1622float2(*reinterpret_cast<const bf162*>(&a.y));
                v.x += lo.x; v.y += lo.y; v.z += hi.x; v.w += hi.y;
            }
            *reinterpret_cast<float4*>(hr + i) = v;
        }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)D + eps);
    const long grow = (long)g->rank * g->shard + r;
    for (int i = threadIdx.x * 8; i < D; i += NT * 8) {
        const float4 a = *reinterpret_cast<const float4*>(hr + i), b = *reinterpret_cast<const float4*>(hr + i + 4);
        float4 ga = make_float4(1.f, 1.f, 1.f, 1.f), gb = ga;
        if (w) { ga = *reinterpret_cast<const float4*>(w + i); gb = *reinterpret_cast<const float4*>(w + i + 4); }
        uint4 o;
        *reinterpret_cast<bf162*>(&o.x) = __floats2bfloat162_rn(a.x * inv * ga.x, a.y * inv * ga.y);
        *reinterpret_cast<bf162*>(&o.y) = __floats2bfloat162_rn(a.z * inv * ga.z, a.w * inv * ga.w);
        *reinterpret_cast<bf162*>(&o.z) = __floats2bfloat162_rn(b.x * inv * gb.x, b.y * inv * gb.y);
        *reinterpret_cast<bf162*>(&o.w) = __floats2bfloat162_rn(b.z * inv * gb.z, b.w * inv * gb.w);
        if (local_only) *reinterpret_cast<uint4*>(g->xfull[g->rank] + grow * D + i) = o;
        else for (int p = 0; p < g->size; ++p) *reinterpret_cast<uint4*>(g->xfull[p] + grow * D + i) = o;
    }
    if (!local_only) __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!local_only)
            for (int p = 0; p < g->size; ++p) red_release_inc_sys(g->ag_arrive[p] + g->rank);
        const unsigned done = atomicAdd(g->ticket + 1, 1u);
        if (done == gridDim.x - 1) {
            g->ticket[1] = 0;
            __threadfence();
            if (!local_only) *g->ag_target += gridDim.x;
            if (has_acc) *g->rs_phase = phase + 1;
        }
    }
}

static int tpseq_norm_launch(const void* g, float* h_shard, const float* w, float eps, int shard, int D, int has_acc,
                             int local_only, int acc_k, int epr, void* stream) {
    TSB_CHECK_ARG(g && h_shard && shard > 0 && D > 0 && D % 8 == 0, "tpseq_norm_gather: bad arguments");
    TSB_CHECK_ARG(acc_k >= 0 && acc_k <= TP_ROUTE_KMAX && (acc_k == 0 || epr > 0), "tpseq_norm_gather: acc_k=%d epr=%d", acc_k, epr);
    TSB_CHECK_CUDA(tsb_launch(tp_seq_norm_gather_kernel<256>, dim3(shard), dim3(256), 0, (cudaStream_t)stream,
                              (const TpSeq*)g, h_shard, w, eps, has_acc, local_only, acc_k, epr));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

extern "C" int tsb_tpseq_norm_gather(const void* g, float* h_shard, const float* w, float eps, int shard, int D, int has_acc,
                                     void* stream) {
    return tpseq_norm_launch(g, h_shard, w, eps, shard, D, has_acc, 0, 0, 0, stream);
}

// The same kernel with the expert-parallel options (see the kernel's comment).
extern "C" int tsb_tpseq_norm_ep(const void* g, float* h_shard, const float* w, float eps, int shard, int D, int has_acc,
                                 int local_only, int acc_k, int epr, void* stream) {
    return tpseq_norm_launch(g, h_shard, w, eps, shard, D, has_acc, local_only, acc_k, epr, stream);
}

// Expert dispatch: one CTA per row of this rank's shard.  The row (already normalised, in this rank's own gathered
// buffer) is stored into the gathered buffer of every other rank that owns one of its k chosen experts; its routing
// record goes to every rank (rows at or past T carry id -1 and are sent nowhere); then one arrival per destination, as
// after the full all-gather, and the last CTA advances the all-gather target.
__global__ void __launch_bounds__(256) tp_seq_dispatch_kernel(const TpSeq* g, const int* ids, const float* wts, int k, int epr,
                                                              int T) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, D = (int)g->ld;
    const long grow = (long)g->rank * g->shard + r;
    const bool live = grow < T;
    unsigned dests = 0u;
    if (live)
        for (int j = 0; j < k; ++j) {
            const int e = ids[(long)r * k + j];
            if (e >= 0) dests |= 1u << (e / epr);
        }
    if ((int)threadIdx.x < k) {
        const int e = live ? ids[(long)r * k + threadIdx.x] : -1;
        const float wv = live ? wts[(long)r * k + threadIdx.x] : 0.f;
        for (int p = 0; p < g->size; ++p) {
            g->route_ids[p][grow * k + threadIdx.x] = e;
            g->route_w[p][grow * k + threadIdx.x] = wv;
        }
    }
    dests &= ~(1u << g->rank);
    if (dests != 0u) {
        const bf16* src = g->xfull[g->rank] + grow * D;
        for (int i = threadIdx.x * 8; i < D; i += 256 * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + i);
            for (int p = 0; p < g->size; ++p)
                if ((dests >> p) & 1u) *reinterpret_cast<uint4*>(g->xfull[p] + grow * D + i) = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int p = 0; p < g->size; ++p) red_release_inc_sys(g->ag_arrive[p] + g->rank);
        const unsigned done = atomicAdd(g->ticket + 1, 1u);
        if (done == gridDim.x - 1) {
            g->ticket[1] = 0;
            __threadfence();
            *g->ag_target += gridDim.x;
        }
    }
}

extern "C" int tsb_tpseq_dispatch(const void* g, const int* ids, const float* wts, int k, int epr, int T, int shard, void* stream) {
    TSB_CHECK_ARG(g && ids && wts && k >= 1 && k <= TP_ROUTE_KMAX && epr >= 1 && shard > 0, "tpseq_dispatch: bad arguments (k=%d epr=%d)", k, epr);
    TSB_CHECK_CUDA(tsb_launch(tp_seq_dispatch_kernel, dim3(shard), dim3(256), 0, (cudaStream_t)stream, (const TpSeq*)g, ids, wts, k,
                              epr, T));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// Wait (bounded) until every rank's gathered rows have arrived: for consumers of the gathered
// buffer that are not the GEMM above (for example the vocabulary projection of the last row).
__global__ void tp_seq_wait_all_kernel(const TpSeq* g) {
    pdl_wait();
    pdl_trigger();
    if ((int)threadIdx.x < g->size && !tp_wait_counter(g->ag_arrive[g->rank] + threadIdx.x, *g->ag_target))
        atomicCAS(g->status, 0, 20 + (int)threadIdx.x);
}
extern "C" int tsb_tpseq_wait_all(const void* g, void* stream) {
    TSB_CHECK_ARG(g, "tpseq_wait_all: null descriptor");
    TSB_CHECK_CUDA(tsb_launch(tp_seq_wait_all_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, (const TpSeq*)g));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// Reduce-scatter of a partial sum that no GEMM epilogue produced (the expert outputs of this rank's
// experts, already summed over its experts): row t of `partial` goes, as bf16, into this rank's slot of
// the accumulator of the rank that owns token t, exactly where the GEMM epilogue would have put it, and
// the arrival counters advance the same way, so tp_seq_norm_gather consumes it unchanged.
#define TPS_PUSH_ROWS 8
// k > 0 (expert combine): only the rows of tokens with one of their k chosen experts in [e0, e1) are stored; the
// owner skips this rank's slot for the others (tp_seq_norm_gather_kernel, acc_k).
__global__ void __launch_bounds__(256) tp_seq_push_rows_kernel(const TpSeq* g, const float* partial, int T, int k, int e0, int e1) {
    pdl_wait();
    pdl_trigger();
    const int D = (int)g->ld;
    const int row0 = blockIdx.x * TPS_PUSH_ROWS;                    // global token index; a block never straddles shards
    const int owner = row0 / g->shard;
    bf16* dst = g->acc[owner] + ((long)(*g->rs_phase & 1u) * g->size + g->rank) * g->shard * D - (long)owner * g->shard * D;
    for (int r = 0; r < TPS_PUSH_ROWS; ++r) {
        const int t = row0 + r;
        if (k > 0) {
            bool mine = false;
            const int* rid = g->route_ids[g->rank] + (long)t * k;
            for (int j = 0; j < k; ++j) mine = mine || (rid[j] >= e0 && rid[j] < e1);
            if (!mine) continue;                                   // uniform over the block
        }
        for (int i = threadIdx.x * 8; i < D; i += 256 * 8) {
            uint4 o = make_uint4(0u, 0u, 0u, 0u);
            if (t < T) {
                const float4 a = *reinterpret_cast<const float4*>(partial + (long)t * D + i);
                const float4 b = *reinterpret_cast<const float4*>(partial + (long)t * D + i + 4);
                *reinterpret_cast<bf162*>(&o.x) = __floats2bfloat162_rn(a.x, a.y);
                *reinterpret_cast<bf162*>(&o.y) = __floats2bfloat162_rn(a.z, a.w);
                *reinterpret_cast<bf162*>(&o.z) = __floats2bfloat162_rn(b.x, b.y);
                *reinterpret_cast<bf162*>(&o.w) = __floats2bfloat162_rn(b.z, b.w);
            }
            *reinterpret_cast<uint4*>(dst + (long)t * D + i) = o;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        red_release_inc_sys(g->rs_arrive[owner]);
        const unsigned done = atomicAdd(g->ticket, 1u);
        if (done == gridDim.x - 1) {
            *g->ticket = 0;
            __threadfence();
            *g->rs_target += (unsigned)g->size * (unsigned)(g->shard / TPS_PUSH_ROWS);
        }
    }
}

static int tpseq_push_launch(const void* g, const float* partial, int T, int shard, int size, int D, int k, int e0, int e1,
                             void* stream) {
    TSB_CHECK_ARG(g && partial && T >= 0 && shard % TPS_PUSH_ROWS == 0 && D % 8 == 0, "tpseq_push_rows: bad arguments");
    TSB_CHECK_ARG(k >= 0 && k <= TP_ROUTE_KMAX, "tpseq_push_rows: k=%d", k);
    TSB_CHECK_CUDA(tsb_launch(tp_seq_push_rows_kernel, dim3((unsigned)(shard * size / TPS_PUSH_ROWS)), dim3(256), 0,
                              (cudaStream_t)stream, (const TpSeq*)g, partial, T, k, e0, e1));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

extern "C" int tsb_tpseq_push_rows(const void* g, const float* partial, int T, int shard, int size, int D, void* stream) {
    return tpseq_push_launch(g, partial, T, shard, size, D, 0, 0, 0, stream);
}

// The expert combine: rows of tokens that chose none of this rank's experts [e0, e1) are not sent.
extern "C" int tsb_tpseq_push_rows_ep(const void* g, const float* partial, int T, int shard, int size, int D, int k, int e0,
                                      int e1, void* stream) {
    return tpseq_push_launch(g, partial, T, shard, size, D, k, e0, e1, stream);
}
