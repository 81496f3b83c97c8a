// Attention over a paged bf16 KV cache: flash prefill (varlen, causal, sliding window,
// sinks, soft-cap, GQA) and split-KV decode with a combine pass.
//
// Cache layout: k_cache / v_cache are [n_slots, Hkv, Dh] bf16 with slot = page * page_size +
// offset; block_table[b, i] is the page that holds tokens [i*page_size, (i+1)*page_size) of
// sequence b.  A query at position p attends to cache positions j with j <= p and, when
// window > 0, j > p - window.
//
// Replaces in the reference: flash_attn_ext_f16 (ggml-cuda/fattn-mma-f16.cuh:1354),
// flash_attn_ext_vec (fattn-vec.cuh:21), flash_attn_combine_results (fattn-common.cuh:721),
// flash_attn_mask_to_KV_max (:576), soft_max_f32 with sinks (softmax.cu:47), the batched
// cuBLAS QK^T / PV of the non-flash prefill path (ggml-cuda.cu:2084) and the host-built masks
// of TensorSharp.GGML.Native/ggml_ops_norm_attn.cpp:1699-1884.  Scores are never materialised.
#include <cstdlib>
#include <mutex>
#include "common.cuh"
#include "attn_args.cuh"
#include "attn_mma.cuh"
#include "tsb_noalloc.h"


__device__ __forceinline__ long kv_slot(const AttnArgs& a, int b, int j) {
    const int page = a.block_table[(long)b * a.max_pages + j / a.page_size];
    return (long)page * a.page_size + j % a.page_size;
}

// ------------------------------------------------------------------------------------------
// Decode: grid (splits, Hkv * chunks, B), 128 threads.  A CTA serves G query heads of one KV head, which share the
// K / V traffic; the Hq / Hkv heads of a KV head are dealt to `chunks` CTAs of G heads each (one chunk when the
// group size is 1, 2, 4 or 8; other group sizes and head size 512 take several).  Lane = token for QK^T,
// lane = dim slice for PV.
// ------------------------------------------------------------------------------------------
// LEAN: the variant for batches.  With one sequence a CTA has an SM to itself and spends registers on having every K and
// V row of its chunk in flight at once; with many sequences there are several CTAs per SM to hide latency with, so the
// V rows are fetched eight at a time and the register budget is capped for four CTAs per SM.
template <int DH, int G, bool LEAN>
__device__ __forceinline__ void attn_decode_body(const AttnArgs& a);

// (two entry points so that the one-sequence kernel keeps exactly the launch bounds it was tuned with: giving it an
// explicit "one block per SM" as well measured 16.2 against 12.0 us per launch)
template <int DH, int G, bool LEAN = false>
__global__ void __launch_bounds__(128) attn_decode_kernel(AttnArgs a) { attn_decode_body<DH, G, false>(a); }
template <int DH, int G>
__global__ void __launch_bounds__(128, 4) attn_decode_lean_kernel(AttnArgs a) { attn_decode_body<DH, G, true>(a); }

template <int DH, int G, bool LEAN>
__device__ __forceinline__ void attn_decode_body(const AttnArgs& a) {
    constexpr int DPL = DH / 32;             // output dims per lane
    pdl_wait();
    pdl_trigger();
    const int split = blockIdx.x, b = blockIdx.z;
    const int heads_per_kv = a.Hq / a.Hkv, chunks = heads_per_kv / G;
    const int hk = blockIdx.y / chunks, h0 = hk * heads_per_kv + (blockIdx.y % chunks) * G;     // first query head of this CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ __align__(16) bf16 qs[G][DH];
    __shared__ float red_m[4][G], red_l[4][G];
    __shared__ float red_o[4][G][DH];
    // the query rows and the sequence length are requested together (the G heads of a KV head are contiguous)
    constexpr int QV = G * DH / 8;                     // 16-byte pieces of the query rows
    const uint4* qsrc = reinterpret_cast<const uint4*>(a.q + ((long)b * a.Hq + h0) * DH);
    uint4 qreg[(QV + 127) / 128];
#pragma unroll
    for (int i = 0; i < (QV + 127) / 128; ++i)
        if (threadIdx.x + i * 128 < QV) qreg[i] = qsrc[threadIdx.x + i * 128];
    // With a caller-fixed split length and no window, the first chunk's cache slot does not depend on the
    // sequence length either: its block-table entry is requested now (the table row is max_pages long and
    // zero beyond the reserved pages, so the read is always in bounds) and validated against the length later.
    const bool fixed = a.split_len > 0 && a.window == 0;
    long slot_first = 0;
    if (fixed) {
        const int j0 = split * a.split_len + warp * 32 + lane;
        const int page = min(j0 / a.page_size, a.max_pages - 1);
        slot_first = (long)a.block_table[(long)b * a.max_pages + page] * a.page_size + j0 % a.page_size;
    }
    const int len = a.kv_lens[b];
#pragma unroll
    for (int i = 0; i < (QV + 127) / 128; ++i)
        if (threadIdx.x + i * 128 < QV) reinterpret_cast<uint4*>(&qs[0][0])[threadIdx.x + i * 128] = qreg[i];
    const int lo = (a.window > 0 && len > a.window) ? len - a.window : 0;
    const int span = len - lo;
    const int per = a.split_len > 0 ? a.split_len : ((((span + a.splits - 1) / a.splits) + 31) & ~31);
    const int s0 = lo + split * per, s1 = min(len, s0 + per);
    __syncthreads();

    float m[G], l[G], acc[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[g][d] = 0.f;
    }
    for (int base = s0 + warp * 32; base < s1; base += 128) {
        const int j = base + lane;
        const bool valid = j < s1;
        const long slot = !valid ? 0 : ((fixed && base == s0 + warp * 32) ? slot_first : kv_slot(a, b, j));
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = 0.f;
        // All of this chunk's K rows (one per lane) and, for head sizes up to 128, all of its V rows are
        // requested before anything is used: a CTA has the SM to itself (the grid is about one CTA per SM),
        // so registers are free and the chunk costs one DRAM round trip instead of six.
        constexpr bool PREFETCH_V = DPL <= 4 && !LEAN;
        constexpr int KCH = DH / 8;
        uint4 kreg[KCH <= 16 ? KCH : 1];
        uint2 vreg[PREFETCH_V ? 32 : 1];
        const int cnt = min(32, s1 - base);
        if (KCH <= 16) {
            const uint4* kp = reinterpret_cast<const uint4*>(a.k_cache + (slot * a.Hkv + hk) * DH);
#pragma unroll
            for (int c = 0; c < KCH; ++c) kreg[c] = valid ? kp[c] : make_uint4(0u, 0u, 0u, 0u);
        }
        if (PREFETCH_V) {
#pragma unroll
            for (int u = 0; u < 32; ++u) {
                const long sl = __shfl_sync(0xffffffffu, slot, u);
                const bf16* vp = a.v_cache + (sl * a.Hkv + hk) * DH + lane * DPL;
                if (DPL == 4) vreg[u] = u < cnt ? *reinterpret_cast<const uint2*>(vp) : make_uint2(0u, 0u);
                else if (DPL == 2) vreg[u] = u < cnt ? make_uint2(*reinterpret_cast<const unsigned*>(vp), 0u) : make_uint2(0u, 0u);
                else vreg[u] = u < cnt ? make_uint2((unsigned)*reinterpret_cast<const unsigned short*>(vp), 0u) : make_uint2(0u, 0u);
            }
        }
        auto dot_chunk = [&](const uint4 kv, int c) {
            const bf162* k2 = reinterpret_cast<const bf162*>(&kv);
            float kf[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(k2[i]);
                kf[2 * i] = f.x;
                kf[2 * i + 1] = f.y;
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const uint4 qv = *reinterpret_cast<const uint4*>(&qs[g][c * 8]);
                const bf162* q2 = reinterpret_cast<const bf162*>(&qv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(q2[i]);
                    s[g] += f.x * kf[2 * i] + f.y * kf[2 * i + 1];
                }
            }
        };
        if (valid) {
            if (KCH <= 16) {
#pragma unroll
                for (int c = 0; c < (KCH <= 16 ? KCH : 1); ++c) dot_chunk(kreg[c], c);     // fully unrolled: kreg stays in registers
            } else {
                const uint4* kp = reinterpret_cast<const uint4*>(a.k_cache + (slot * a.Hkv + hk) * DH);
#pragma unroll 8
                for (int c = 0; c < KCH; ++c) dot_chunk(kp[c], c);
            }
        }
        float p[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float sv = s[g] * a.scale;
            if (a.softcap > 0.f) sv = a.softcap * tanhf(sv / a.softcap);
            sv = valid ? sv : -INFINITY;
            const float mx = fmaxf(m[g], warp_max(sv));
            const float corr = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mx);
            p[g] = valid ? __expf(sv - mx) : 0.f;
            l[g] = l[g] * corr + warp_sum(p[g]);
            m[g] = mx;
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[g][d] *= corr;
        }
        if (PREFETCH_V) {
#pragma unroll
            for (int u = 0; u < 32; ++u) {
                float vf[DPL];                          // bf16 -> f32 is a 16-bit shift; no address of the register array is taken
                vf[0] = __uint_as_float(vreg[u].x << 16);
                if (DPL >= 2) vf[1 % DPL] = __uint_as_float(vreg[u].x & 0xffff0000u);
                if (DPL >= 4) {
                    vf[2 % DPL] = __uint_as_float(vreg[u].y << 16);
                    vf[3 % DPL] = __uint_as_float(vreg[u].y & 0xffff0000u);
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pg = __shfl_sync(0xffffffffu, p[g], u);
#pragma unroll
                    for (int d = 0; d < DPL; ++d) acc[g][d] += pg * vf[d];
                }
            }
        } else {
        // P V: eight value rows are fetched before any of them is used, so the loads overlap
        constexpr int VB = DPL > 8 ? 4 : 8;             // value rows in flight (fewer for the widest heads: registers)
        for (int t0 = 0; t0 < cnt; t0 += VB) {
            float vf[VB][DPL];
#pragma unroll
            for (int u = 0; u < VB; ++u) {
                const long sl = __shfl_sync(0xffffffffu, slot, (t0 + u) & 31);
                const bf16* vp = a.v_cache + (sl * a.Hkv + hk) * DH + lane * DPL;
                if (t0 + u < cnt) {
                    if (DPL % 8 == 0) {
#pragma unroll
                        for (int c8 = 0; c8 < DPL / 8; ++c8) {
                            const uint4 vv = reinterpret_cast<const uint4*>(vp)[c8];
                            const bf162* v2 = reinterpret_cast<const bf162*>(&vv);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 f = __bfloat1622float2(v2[i]);
                                vf[u][(c8 * 8 + 2 * i) % DPL] = f.x;
                                vf[u][(c8 * 8 + 2 * i + 1) % DPL] = f.y;
                            }
                        }
                    } else {
#pragma unroll
                        for (int d = 0; d < DPL; ++d) vf[u][d] = bf2f(vp[d]);
                    }
                } else {
#pragma unroll
                    for (int d = 0; d < DPL; ++d) vf[u][d] = 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < VB; ++u) {
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pg = __shfl_sync(0xffffffffu, p[g], (t0 + u) & 31);
#pragma unroll
                    for (int d = 0; d < DPL; ++d) acc[g][d] += pg * vf[u][d];
                }
            }
        }
        }
    }
    // merge the four warps
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) { red_m[warp][g] = m[g]; red_l[warp][g] = l[g]; }
#pragma unroll
        for (int d = 0; d < DPL; ++d) red_o[warp][g][lane * DPL + d] = acc[g][d];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * DH; i += 128) {
        const int g = i / DH, d = i % DH;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red_m[w][g]);
        float ll = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float c = (red_m[w][g] == -INFINITY) ? 0.f : __expf(red_m[w][g] - mm);
            ll += red_l[w][g] * c;
            o += red_o[w][g][d] * c;
        }
        const long pi = ((long)b * a.Hq + h0 + g) * a.splits + split;
        a.part_o[pi * DH + d] = o;
        if (d == 0) { a.part_ml[pi * 2] = mm; a.part_ml[pi * 2 + 1] = ll; }
    }
    if (a.ticket == nullptr) return;
    // The CTA that finishes this (sequence, KV head) last merges the splits: no combine launch.
    __shared__ bool last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(&a.ticket[b * a.Hkv + hk], 1u) == (unsigned)a.splits - 1u;
    __syncthreads();
    if (!last) return;
    __threadfence();
    for (int i = threadIdx.x; i < G * DH; i += 128) {
        const int g = i / DH, d = i % DH, h = h0 + g;       // (the in-kernel merge runs with one chunk per KV head only)
        const long pb = ((long)b * a.Hq + h) * a.splits;
        float mm = a.sinks ? a.sinks[h] : -INFINITY;
        for (int sp = 0; sp < a.splits; ++sp) mm = fmaxf(mm, __ldcg(&a.part_ml[(pb + sp) * 2]));
        float ll = a.sinks ? __expf(a.sinks[h] - mm) : 0.f, o = 0.f;
        for (int sp = 0; sp < a.splits; ++sp) {
            const float ms = __ldcg(&a.part_ml[(pb + sp) * 2]);
            const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
            ll += __ldcg(&a.part_ml[(pb + sp) * 2 + 1]) * c;
            o += __ldcg(&a.part_o[(pb + sp) * DH + d]) * c;
        }
        const bf16 ob = f2bf(ll > 0.f ? o / ll : 0.f);
        const long e = ((long)b * a.Hq + h) * DH + d;
        a.out[e] = ob;
        if (a.out_q != nullptr) {                      // a warp holds one group of 32 dims; arithmetic of quantize_q8_kernel
            const float v = bf2f(ob);
            const float amax = warp_max(fabsf(v));
            const float sum = warp_sum(v);
            const float dq = amax / 127.f;
            a.out_q[e] = (int8_t)__float2int_rn(amax > 0.f ? v / dq : 0.f);
            if ((d & 31) == 0) a.out_ds[e >> 5] = make_float2(dq, sum);
        }
    }
    if (threadIdx.x == 0) a.ticket[b * a.Hkv + hk] = 0u;     // ready for the next launch on this stream
}

// grid (Hq, B), DH threads (rounded up to 32): merge split partials, apply the sink, normalise.
// Latency is all that matters here (a few KB per block), so nothing is read in a dependent loop: each
// lane fetches the (max, sum) of two splits at once, the warp reduces them, and the partial outputs
// are fetched thirty-two splits at a time before any is used.  At most 64 splits.
__global__ void attn_combine_kernel(AttnArgs a) {
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x, lane = threadIdx.x & 31;
    const long base = ((long)b * a.Hq + h) * a.splits;
    const bool in0 = lane < a.splits, in1 = lane + 32 < a.splits;
    const float2 ml0 = in0 ? *reinterpret_cast<const float2*>(a.part_ml + (base + lane) * 2) : make_float2(-INFINITY, 0.f);
    const float2 ml1 = in1 ? *reinterpret_cast<const float2*>(a.part_ml + (base + lane + 32) * 2) : make_float2(-INFINITY, 0.f);
    const float sink = a.sinks ? a.sinks[h] : -INFINITY;
    const float mm = fmaxf(sink, warp_max(fmaxf(ml0.x, ml1.x)));
    const float c0 = (ml0.x == -INFINITY) ? 0.f : __expf(ml0.x - mm), c1 = (ml1.x == -INFINITY) ? 0.f : __expf(ml1.x - mm);
    const float ll = warp_sum(ml0.y * c0 + ml1.y * c1) + (a.sinks ? __expf(sink - mm) : 0.f);
    float o = 0.f;
    const int dd = d < a.Dh ? d : 0;
    for (int s0 = 0; s0 < a.splits; s0 += 32) {
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) pv[i] = (s0 + i < a.splits) ? a.part_o[(base + s0 + i) * a.Dh + dd] : 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int sp = s0 + i;
            const float c = __shfl_sync(0xffffffffu, sp < 32 ? c0 : c1, sp & 31);
            o += pv[i] * c;
        }
    }
    const bf16 ob = f2bf(ll > 0.f ? o / ll : 0.f);
    if (d < a.Dh) a.out[((long)b * a.Hq + h) * a.Dh + d] = ob;
    if (a.out_q != nullptr) {
        // a warp holds 32 consecutive dims = one group (Dh is a multiple of 32); same arithmetic as quantize_q8_kernel
        const float v = d < a.Dh ? bf2f(ob) : 0.f;
        const float amax = warp_max(fabsf(v));
        const float sum = warp_sum(v);
        const float dq = amax / 127.f;
        const long e = ((long)b * a.Hq + h) * a.Dh + d;
        if (d < a.Dh) {
            a.out_q[e] = (int8_t)__float2int_rn(amax > 0.f ? v / dq : 0.f);
            if ((d & 31) == 0) a.out_ds[e >> 5] = make_float2(dq, sum);
        }
    }
}

// Heads of a KV head that one CTA serves: the largest of 8, 4, 2, 1 that divides the group (at most 2 for head size
// 512, whose accumulators and merge buffers are four times those of head size 128).
static int attn_decode_chunk(int heads_per_kv, int Dh) {
    const int cap = Dh > 256 ? 2 : 8;
    for (int g = cap; g > 1; g >>= 1)
        if (heads_per_kv % g == 0) return g;
    return 1;
}

template <int DH>
static int launch_decode_g(const AttnArgs& a, cudaStream_t s) {
    const int G = attn_decode_chunk(a.Hq / a.Hkv, DH);
    dim3 grid(a.splits, a.Hkv * ((a.Hq / a.Hkv) / G), a.B);
    if constexpr (DH <= 128) {
        // more CTAs than four per SM: the lean variant (batches)
        if ((long)grid.x * grid.y * grid.z > 4L * 148) {
            switch (G) {
            case 1: return tsb_launch(attn_decode_lean_kernel<DH, 1>, grid, dim3(128), 0, s, a) == cudaSuccess ? TSB_OK : TSB_ERR_CUDA;
            case 2: return tsb_launch(attn_decode_lean_kernel<DH, 2>, grid, dim3(128), 0, s, a) == cudaSuccess ? TSB_OK : TSB_ERR_CUDA;
            case 4: return tsb_launch(attn_decode_lean_kernel<DH, 4>, grid, dim3(128), 0, s, a) == cudaSuccess ? TSB_OK : TSB_ERR_CUDA;
            default: return tsb_launch(attn_decode_lean_kernel<DH, 8>, grid, dim3(128), 0, s, a) == cudaSuccess ? TSB_OK : TSB_ERR_CUDA;
            }
        }
    }
    switch (G) {
    case 1: if (tsb_launch(attn_decode_kernel<DH, 1>, grid, dim3(128), 0, s, a) != cudaSuccess) return TSB_ERR_CUDA; break;
    case 2: if (tsb_launch(attn_decode_kernel<DH, 2>, grid, dim3(128), 0, s, a) != cudaSuccess) return TSB_ERR_CUDA; break;
    case 4:
        if constexpr (DH <= 256) {
            if (tsb_launch(attn_decode_kernel<DH, 4>, grid, dim3(128), 0, s, a) != cudaSuccess) return TSB_ERR_CUDA;
        }
        break;
    default:
        if constexpr (DH <= 256) {
            if (tsb_launch(attn_decode_kernel<DH, 8>, grid, dim3(128), 0, s, a) != cudaSuccess) return TSB_ERR_CUDA;
        }
        break;
    }
    return TSB_OK;
}

// Arrival counters of the fused split merge: one per (sequence, KV head), zero between launches (the
// merging CTA resets its counter).  Launches that share a device must be ordered, as a decode loop's are.
#define ATTN_MAX_TICKETS 65536
static __device__ unsigned g_attn_ticket[ATTN_MAX_TICKETS];
static unsigned* g_attn_ticket_ptr[64] = {nullptr};
static std::once_flag g_attn_ticket_once[64];

static unsigned* attn_ticket_for_current_device() {
    // Off unless TSB_ATTN_FUSED_COMBINE=1: inside the decode step the in-kernel merge measured slower than the
    // separate combine launch (2.57 ms against 2.23 ms per step on Qwen3-4B): the fences and the serial merge by
    // one CTA sit on the critical path, while the combine kernel's launch overlaps the attention kernel's tail.
    static const bool on = []() { const char* e = getenv("TSB_ATTN_FUSED_COMBINE"); return e && atoi(e) != 0; }();
    if (!on) return nullptr;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    // once per device, whichever host thread gets here first (the device is current in that thread)
    std::call_once(g_attn_ticket_once[dev], [dev]() {
        unsigned* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_attn_ticket) == cudaSuccess) g_attn_ticket_ptr[dev] = p;
    });
    return g_attn_ticket_ptr[dev];
}

// `allow_fused`: whether this call may use the in-kernel split merge (and with it the shared arrival tickets).
static int attn_decode_impl(const AttnArgs* args, void* stream, bool allow_fused) {
    AttnArgs a = *args;
    TSB_CHECK_ARG(a.Hkv > 0 && a.Hq % a.Hkv == 0, "attn_decode: Hq=%d not a multiple of Hkv=%d", a.Hq, a.Hkv);
    // the in-kernel merge counts arrivals per KV head: only when one CTA serves the whole head group
    const bool one_chunk = attn_decode_chunk(a.Hq / a.Hkv, a.Dh) == a.Hq / a.Hkv;
    a.ticket = (allow_fused && one_chunk && a.splits >= 1 && (long)a.B * a.Hkv <= ATTN_MAX_TICKETS) ? attn_ticket_for_current_device() : nullptr;
    TSB_CHECK_ARG(a.splits >= 1 && a.part_o && a.part_ml, "attn_decode: scratch for %d splits missing", a.splits);
    TSB_CHECK_ARG(a.splits <= 64, "attn_decode: %d splits (limit 64)", a.splits);
    if (a.B == 0) return TSB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    // Head sizes 64 / 128 with up to 16 query heads per KV head: Q K^T and P V on the tensor cores, the query heads of a
    // KV head as the rows of one tile (attention_decode_mma.cu).  Measured on the Qwen3-4B shape: one sequence 2.015 ->
    // 1.750 ms per step, 16 sequences 5.76 -> 4.48 ms.  TSB_ATTN_MMA=0 keeps the CUDA-core kernels for every shape,
    // TSB_ATTN_MMA_MIN_CTAS=n for grids of fewer than n CTAs.
    static const bool mma_on = []() { const char* e = getenv("TSB_ATTN_MMA"); return !e || atoi(e) != 0; }();
    static const long mma_min_ctas = []() { const char* e = getenv("TSB_ATTN_MMA_MIN_CTAS"); return e ? atol(e) : 1L; }();
    if (mma_on && (long)a.splits * a.Hkv * a.B >= mma_min_ctas && tsb_attn_decode_mma_supported(a)) {
        a.ticket = nullptr;
        bool merged = false;
        rc = tsb_attn_decode_mma_launch(a, s, &merged);
        if (rc != TSB_OK) return rc;
        TSB_CHECK_LAUNCH();
        if (!merged) {
            TSB_CHECK_CUDA(tsb_launch(attn_combine_kernel, dim3(a.Hq, a.B), dim3((a.Dh + 31) & ~31), 0, s, a));
            TSB_CHECK_LAUNCH();
        }
        return TSB_OK;
    }
    switch (a.Dh) {
    case 64: rc = launch_decode_g<64>(a, s); break;
    case 128: rc = launch_decode_g<128>(a, s); break;
    case 256: rc = launch_decode_g<256>(a, s); break;
    case 512: rc = launch_decode_g<512>(a, s); break;
    default:
        tsb_set_error("attn_decode: unsupported head dim %d (supported 64, 128, 256, 512)", a.Dh);
        return TSB_ERR_UNSUPPORTED;
    }
    if (rc != TSB_OK) return rc;
    TSB_CHECK_LAUNCH();
    if (a.ticket == nullptr) {
        TSB_CHECK_CUDA(tsb_launch(attn_combine_kernel, dim3(a.Hq, a.B), dim3((a.Dh + 31) & ~31), 0, s, a));
        TSB_CHECK_LAUNCH();
    }
    return TSB_OK;
}

extern "C" int tsb_attn_decode(const AttnArgs* args, void* stream) { return attn_decode_impl(args, stream, true); }

// The merge of the split partials on its own, for split kernels that live in other translation units.
extern "C" int tsb_attn_combine(const AttnArgs* args, void* stream) {
    const AttnArgs& a = *args;
    TSB_CHECK_ARG(a.splits >= 1 && a.splits <= 64 && a.part_o && a.part_ml, "attn_combine: scratch for %d splits (limit 64)", a.splits);
    if (a.B == 0) return TSB_OK;
    TSB_CHECK_CUDA(tsb_launch(attn_combine_kernel, dim3(a.Hq, a.B), dim3((a.Dh + 31) & ~31), 0, (cudaStream_t)stream, a));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant (see tsb_noalloc.h): the split-KV partials live in a file-scope
// device array instead of caller scratch.  In host code the array's name is only a handle
// for the runtime, not a device address, so its address is fetched once per device with
// cudaGetSymbolAddress and that pointer is what the kernels receive.
// ------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_attn_noalloc_scratch[TSB_ATTN_NOALLOC_MAX_FLOATS];

static float* g_attn_noalloc_ptr[64] = {nullptr};
static cudaError_t g_attn_noalloc_err[64];
static std::once_flag g_attn_noalloc_once[64];

extern "C" long tsb_attn_decode_noalloc_capacity(void) { return (long)TSB_ATTN_NOALLOC_MAX_FLOATS; }

extern "C" int tsb_attn_decode_noalloc(const AttnArgs* args, void* stream) {
    TSB_CHECK_ARG(args != nullptr, "attn_decode_noalloc: null arguments");
    AttnArgs a = *args;
    TSB_CHECK_ARG(a.B >= 0 && a.Hq > 0 && a.Dh > 0 && a.splits >= 1, "attn_decode_noalloc: bad sizes B=%d Hq=%d Dh=%d splits=%d",
                  a.B, a.Hq, a.Dh, a.splits);
    TSB_CHECK_ARG(a.splits <= 64, "attn_decode_noalloc: %d splits (limit 64)", a.splits);
    const long slots = (long)a.B * a.Hq * a.splits;
    const long need = slots * (a.Dh + 2);
    TSB_CHECK_ARG(need <= (long)TSB_ATTN_NOALLOC_MAX_FLOATS,
                  "attn_decode_noalloc: B*Hq*splits*(Dh+2) = %ld floats exceeds the built-in scratch of %ld floats; "
                  "use fewer splits or a smaller batch", need, (long)TSB_ATTN_NOALLOC_MAX_FLOATS);
    int dev = -1;
    TSB_CHECK_CUDA(cudaGetDevice(&dev));
    TSB_CHECK_ARG(dev >= 0 && dev < 64, "attn_decode_noalloc: device ordinal %d out of range", dev);
    // one-time set-up for this device (current device == dev): resolve the array's device address.  call_once makes
    // two host threads that reach their first call on one device together agree on one lookup.
    std::call_once(g_attn_noalloc_once[dev], [dev]() {
        float* p = nullptr;
        g_attn_noalloc_err[dev] = cudaGetSymbolAddress((void**)&p, g_attn_noalloc_scratch);
        if (g_attn_noalloc_err[dev] == cudaSuccess) g_attn_noalloc_ptr[dev] = p;
    });
    TSB_CHECK_CUDA(g_attn_noalloc_err[dev]);
    float* base = g_attn_noalloc_ptr[dev];
    a.part_o = base;                       // [B, Hq, splits, Dh]
    a.part_ml = base + slots * a.Dh;       // [B, Hq, splits, 2]
    // always the two-kernel form: the in-kernel split merge would bring in a second shared array (its arrival tickets)
    return attn_decode_impl(&a, stream, false);
}

// ------------------------------------------------------------------------------------------
// Prefill: flash attention on mma.sync m16n8k16 bf16, 64 queries x one head per CTA, 64-token
// KV tiles streamed with cp.async double buffering from the paged cache.
// ------------------------------------------------------------------------------------------
// DS > 1 (head size 512): DS sets of four warps share the tiles and the score arithmetic, each set keeps DH / DS of the
// output columns, so that a thread's accumulators stay at the head-size-256 count.
template <int DH, int BN, int DS>
__global__ void __launch_bounds__(128 * DS) attn_prefill_kernel(AttnArgs a) {
    constexpr int BM = 64, CH = DH / 8;   // CH = 16-byte chunks per row
    constexpr int NT = 128 * DS, DO = DH / DS;     // threads; output columns per warp set
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
    bf16* sK = sQ + BM * DH;         // 2 stages
    bf16* sV = sK + 2 * BN * DH;     // 2 stages

    const int b = blockIdx.z, h = blockIdx.y, hk = h / (a.Hq / a.Hkv);
    const int q0 = a.cu_q[b], qlen = a.cu_q[b + 1] - q0;
    const int m0 = (int)(gridDim.x - 1 - blockIdx.x) * BM;      // last query tiles first: under a causal mask they have the most keys
    if (m0 >= qlen) return;
    const int kvlen = a.kv_lens[b];
    const int pos0 = a.q_pos0 ? a.q_pos0[b] : kvlen - qlen;   // cache position of the sequence's first query
    const int warp = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31, dset = threadIdx.x >> 7;
    const int rows = min(BM, qlen - m0);

    // KV range needed by this query tile
    const int p_last = pos0 + m0 + rows - 1;
    int j_lo = 0;
    if (a.window > 0) j_lo = max(0, pos0 + m0 - a.window + 1);
    const int j_hi = min(p_last + 1, kvlen);       // exclusive
    const int t_lo = j_lo / BN, t_hi = (j_hi + BN - 1) / BN;

    // Q tile -> shared (rows beyond the sequence are zero)
    for (int i = threadIdx.x; i < BM * CH; i += NT) {
        const int r = i / CH, c = i % CH;
        bf16* dst = tile_ptr<DH>(sQ, r, c);
        if (r < rows) cp_async16(dst, a.q + ((long)(q0 + m0 + r) * a.Hq + h) * DH + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    auto load_kv = [&](int t, int stage) {
        bf16* dk = sK + stage * BN * DH;
        bf16* dv = sV + stage * BN * DH;
        for (int i = threadIdx.x; i < BN * CH; i += NT) {
            const int r = i / CH, c = i % CH;
            const int j = t * BN + r;
            bf16* pk = tile_ptr<DH>(dk, r, c);
            bf16* pv = tile_ptr<DH>(dv, r, c);
            if (j < kvlen) {
                const long off = (kv_slot(a, b, j) * a.Hkv + hk) * DH + c * 8;
                cp_async16(pk, a.k_cache + off);
                cp_async16(pv, a.v_cache + off);
            } else {
                *reinterpret_cast<uint4*>(pk) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(pv) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    load_kv(t_lo, 0);
    cp_async_commit();

    float o[DO / 8][4];
#pragma unroll
    for (int i = 0; i < DO / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const int r_lo = warp * 16 + (lane >> 2);      // this thread's two query rows: r_lo, r_lo + 8
    const int qpos_a = pos0 + m0 + r_lo, qpos_b = qpos_a + 8;

    for (int t = t_lo; t < t_hi; ++t) {
        const int stage = (t - t_lo) & 1;
        if (t + 1 < t_hi) load_kv(t + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* tK = sK + stage * BN * DH;
        const bf16* tV = sV + stage * BN * DH;

        // S = Q K^T  (16 x 64 per warp)
        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
            uint32_t qa[4];
            ldsm_x4(qa, tile_ptr<DH>(sQ, warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
            for (int nt = 0; nt < BN / 16; ++nt) {
                uint32_t kb[4];
                const int tok = nt * 16 + ((lane >> 4) << 3) + (lane & 7);
                ldsm_x4(kb, tile_ptr<DH>(const_cast<bf16*>(tK), tok, kk * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[2 * nt], qa, kb[0], kb[1]);
                mma_bf16(s[2 * nt + 1], qa, kb[2], kb[3]);
            }
        }
        // soft-cap, mask, online softmax.  The scores stay unscaled: with f = scale (or 1 after the soft-cap, which needs
        // the scaled value) the row maximum is max(x) * f and p = 2^(x * f * log2 e - max * log2 e), one multiply-add and
        // one exponential per score.  The mask compares run only in tiles that touch the diagonal, the end of the cache
        // or the window's edge (uniform per warp); interior tiles skip them.
        constexpr float LOG2E = 1.4426950408889634f;
        float f = a.scale;
        if (a.softcap > 0.f) {
            const float inv_cap = a.scale / a.softcap;
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = a.softcap * tanhf(s[nt][e] * inv_cap);
            f = 1.f;
        }
        const int q_first = pos0 + m0 + warp * 16;               // cache position of this warp's first query row
        const bool need_mask = (t * BN + BN - 1 > q_first) || ((t + 1) * BN > kvlen) ||
                               (a.window > 0 && t * BN <= q_first + 15 - a.window);
        if (need_mask) {
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = t * BN + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int qp = (e < 2) ? qpos_a : qpos_b;
                    const bool ok = j <= qp && j < kvlen && (a.window <= 0 || j > qp - a.window);
                    s[nt][e] = ok ? s[nt][e] : -INFINITY;
                }
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
            mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            mx[r] = fmaxf(mrow[r], mx[r] * f);                   // running maximum, in scaled units
        }
        float corr[2], rsum[2] = {0.f, 0.f}, mneg[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            corr[r] = (mrow[r] == -INFINITY) ? 0.f : exp2f((mrow[r] - mx[r]) * LOG2E);
            mrow[r] = mx[r];
            mneg[r] = (mx[r] == -INFINITY) ? 0.f : -mx[r] * LOG2E;
        }
        const float fl = f * LOG2E;
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = exp2f(fmaf(s[nt][e], fl, mneg[e >> 1]));
                s[nt][e] = p;
                rsum[e >> 1] += p;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) lrow[r] = lrow[r] * corr[r] + rsum[r];
#pragma unroll
        for (int i = 0; i < DO / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // O += P V
#pragma unroll
        for (int kt = 0; kt < BN / 16; ++kt) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
            pa[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
            pa[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            pa[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
            for (int dt = 0; dt < DO / 16; ++dt) {
                uint32_t vb[4];
                const int tok = kt * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
                ldsm_x4_t(vb, tile_ptr<DH>(const_cast<bf16*>(tV), tok, (dset * (DO / 16) + dt) * 2 + (lane >> 4)));
                mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
                mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    // row sums across the four lanes that share a row
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
    }
    float inv[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float mm = mrow[r], ll = lrow[r], oc = 1.f;
        if (a.sinks) {
            const float sk = a.sinks[h];
            const float mn = fmaxf(mm, sk);
            oc = (mm == -INFINITY) ? 0.f : __expf(mm - mn);
            ll = ll * oc + __expf(sk - mn);
        }
        inv[r] = ll > 0.f ? oc / ll : 0.f;
    }
    const int ra = warp * 16 + (lane >> 2), rb = ra + 8;
    if (a.lse_out != nullptr && (lane & 3) == 0 && dset == 0) {
        if (ra < rows) a.lse_out[(long)(q0 + m0 + ra) * a.Hq + h] = lrow[0] > 0.f ? mrow[0] + __logf(lrow[0]) : -INFINITY;
        if (rb < rows) a.lse_out[(long)(q0 + m0 + rb) * a.Hq + h] = lrow[1] > 0.f ? mrow[1] + __logf(lrow[1]) : -INFINITY;
    }
#pragma unroll
    for (int i = 0; i < DO / 8; ++i) {
        const int d = dset * DO + i * 8 + (lane & 3) * 2;
        if (ra < rows)
            *reinterpret_cast<uint32_t*>(a.out + ((long)(q0 + m0 + ra) * a.Hq + h) * DH + d) =
                pack_bf16(o[i][0] * inv[0], o[i][1] * inv[0]);
        if (rb < rows)
            *reinterpret_cast<uint32_t*>(a.out + ((long)(q0 + m0 + rb) * a.Hq + h) * DH + d) =
                pack_bf16(o[i][2] * inv[1], o[i][3] * inv[1]);
    }
}

template <int DH>
static int launch_prefill(const AttnArgs& a, int max_q, cudaStream_t s) {
    // head size 512: 32-key tiles (query tile 64 KB + two stages of K and V 128 KB) and two warp sets
    constexpr int BN = DH > 256 ? 32 : 64, DS = DH > 256 ? 2 : 1;
    const size_t smem = (size_t)(64 + 4 * BN) * DH * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<DH, BN, DS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)smem));
        configured = true;
    }
    dim3 grid((max_q + 63) / 64, a.Hq, a.B);
    TSB_CHECK_CUDA(tsb_launch(attn_prefill_kernel<DH, BN, DS>, grid, dim3(128 * DS), smem, s, a));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

extern "C" int tsb_attn_prefill(const AttnArgs* args, int max_q_len, void* stream) {
    const AttnArgs& a = *args;
    TSB_CHECK_ARG(a.Hkv > 0 && a.Hq % a.Hkv == 0, "attn_prefill: Hq=%d not a multiple of Hkv=%d", a.Hq, a.Hkv);
    TSB_CHECK_ARG(a.cu_q != nullptr, "attn_prefill: cu_q is required");
    if (a.B == 0 || max_q_len == 0) return TSB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    switch (a.Dh) {
    case 64: return launch_prefill<64>(a, max_q_len, s);
    case 128: return launch_prefill<128>(a, max_q_len, s);
    case 256: return launch_prefill<256>(a, max_q_len, s);
    case 512: return launch_prefill<512>(a, max_q_len, s);
    default:
        tsb_set_error("attn_prefill: unsupported head dim %d (supported 64, 128, 256, 512)", a.Dh);
        return TSB_ERR_UNSUPPORTED;
    }
}
