// One decode step of a dense decoder (Qwen3 / Llama family, one sequence) as ONE persistent kernel.
//
// The per-op decode step is a chain of about ten dependent launches per layer, each at its latency
// floor (launch, first-load round trip, tail), so the step streams 2.4 GB of weights at under a fifth
// of the HBM rate and dividing the weights over tensor-parallel ranks buys nothing.  Here the whole
// step runs as one cooperative grid of one CTA per SM:
//
//   * Weights never wait for activations.  In every CTA a producer thread walks the step's weight
//     schedule (this CTA's rows of every matrix of every layer, in order) and keeps a ring of shared
//     memory stages full with bulk asynchronous copies (cp.async.bulk + mbarrier transaction counts,
//     no multicast).  The ring runs ahead across phase and layer boundaries, so HBM keeps streaming
//     while the consumers sit in a dependency.
//   * Twelve consumer warps per CTA (three groups that take tasks in turn) take rows out of the ring, up to
//     four rows per warp at a time: Q4_K / Q6_K blocks against int8 activations with one scale per 256
//     values (the contract of ggml's K-quant dot products on the CPU: ggml-quants.c, q8_K), so the 6-bit
//     block scales multiply integer partial sums and one float multiply-add finishes 64 weights.  The
//     activations stay in shared memory and the loop body is one compact copy per block type: with nearly
//     all of the SM's memory configured as shared, neither spilled registers nor a large instruction
//     footprint are affordable.
//   * There is no grid barrier.  Every value that crosses CTAs (q/k/v rows, attention partials,
//     projection outputs, gated activations) travels as an 8-byte word {f32 value, u32 tag} written
//     with one store; a consumer polls exactly the words it needs until their tag is this step's tag
//     for that phase.  A dependency therefore costs one L2 round trip after the last producer's store.
//   * The residual stream lives in every CTA's shared memory; each CTA adds the same partial sums in
//     the same (rank) order, so all CTAs and all ranks hold bit-identical hidden states.
//   * Tensor parallelism costs no launch and no collective: the row-parallel projections (o_proj,
//     down) store their tagged partial sums straight into every rank's buffer over NVLink (plain peer
//     stores through CUDA-IPC mappings), and the next phase's gather simply waits for `size` parts.
//
// Phases of a layer (tags are unique per step, layer and phase):
//   QKV   h -> RMSNorm -> int8 -> rows of wq / wk / wv               -> qkv words
//   ATT   per (KV head, split): per-head norm + RoPE, new K / V row into the paged cache, split-KV
//         attention over the cache                                    -> partial (o, m, l) words
//   CMB   per query head: merge of the splits                         -> attention output words
//   OPR   attention output -> int8 -> rows of wo                      -> o_proj partial words (all ranks)
//   GUP   h += sum of parts; RMSNorm -> int8 -> gate / up rows, GLU   -> activation words
//   DWN   activations -> int8 -> rows of w_down                       -> down partial words (all ranks)
// and after the last layer the output norm and the lm_head rows, written as plain f32 logits.
//
// Every wait is bounded (2 s on %globaltimer); on expiry the kernel records a code in `status`, raises
// a flag that makes every later wait return at once, lets the copies in flight land and returns.
//
// Replaces the reference's whole-model decode graph (TensorSharp.GGML.Native/ggml_ops_transformer.cpp
// :1012-1298, TSGgml_TransformerModelDecode), which is rebuilt on the host for every token.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include "gemv_core.cuh"
#include "tcgen05.cuh"

#define MG_GW 4                              // warps per consumer group (a group takes every MG_GROUPS-th task)
#define MG_GROUPS 3
#define MG_CWARPS (MG_GW * MG_GROUPS)        // consumer warps
#define MG_CTHREADS (MG_CWARPS * 32)
#define MG_THREADS (MG_CTHREADS + 32)        // + the producer warp
#define MG_MAX_RANKS 8
#define MG_MAX_STAGES 8
#define MG_MAX_G 8                           // query heads per KV head
#define MG_WAIT_NS 2000000000ull

enum { PH_QKV = 0, PH_ATT = 1, PH_CMB = 2, PH_OPR = 3, PH_GUP = 4, PH_DWN = 5, PH_MAX = 6, PH_STRIDE = 8 };

typedef QW MegaMat;

struct MegaLayer {
    MegaMat qkv[3];                // wq, wk, wv; or the fused matrix in [0] and N = 0 in the others
    MegaMat wo, gate_up, down;     // gate_up: gate rows [0, ffn), up rows [ffn, 2 ffn)
    const float* attn_norm;
    const float* ffn_norm;
    const float* q_norm;           // [Dh] or null
    const float* k_norm;
    const float* qkv_bias;         // [(Hq + 2 Hkv) Dh] or null
    bf16* k_cache;
    bf16* v_cache;
};

struct MegaArgs {
    const MegaLayer* layers;
    int n_layers;
    MegaMat embed;                 // token embedding (any GGUF type dequant8 knows)
    MegaMat lm_head;               // this rank's vocabulary rows
    const float* out_norm;
    float embed_scale;
    int hidden, Hq, Hkv, Dh, ffn;  // sizes on this rank (heads and FFN width are the rank's share)
    float eps, attn_scale;
    const float* rope_freq;        // [rot_dim / 2] angle per position and pair (scaling folded in)
    float rope_mscale;
    int rot_dim, rope_mode;        // mode 0: NeoX pairs (i, i + rot/2); 1: adjacent pairs
    int act;                       // GLU activation (ACT_SWIGLU, ACT_GEGLU_*)
    // the sequence (batch of one): all device memory, so that graph replays follow the bookkeeping kernels
    const int* tokens;
    const int* positions;
    const int* kv_lens;
    const long* slots;
    const int* block_table;
    int max_pages, page_size;
    float* logits;                 // [lm_head.N]
    // exchange buffers: rank r's buffer as mapped in this process; word offsets of the regions
    float2* xbuf[MG_MAX_RANKS];
    int rank, size;
    long off_qkv, off_part, off_attn, off_opr, off_act, off_dwn;
    unsigned* step;                // local: steps completed (advanced by CTA 0 at the end)
    int* status;                   // local: 0, or the code of the wait that ran out
    unsigned long long* prof;      // null, or [grid][24] nanoseconds spent per phase by each CTA (diagnostics)
    int debug;                     // diagnostics: 1 = rows are fetched but not multiplied; 2 = rows are multiplied without waiting for their stage
    int splits;                    // attention splits per KV head
    // filled by tsb_mega_plan
    int grid, stage_bytes, n_stages;
    int off_h, off_xq, off_xds, off_bsum_words, off_qs, off_red, off_ring, smem_bytes;
};

// status codes: 100 + phase: a tagged word never arrived; 200: weight stage never filled; 201: stage never freed
#ifdef __CUDACC__

struct Ctl {
    volatile int* dead;            // shared: set once any wait of this CTA gave up (or another CTA's did)
    int* status;
};

__device__ __forceinline__ uint2 ld_word(const float2* p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// True when the grid is going down (a wait gave up here or elsewhere); called every few hundred polls.
__device__ __noinline__ bool wait_expired(const Ctl& c, unsigned long long t0, int code) {
    if (*c.dead) return true;
    if (*reinterpret_cast<volatile int*>(c.status) != 0) { *c.dead = 1; return true; }
    if (global_timer_ns() - t0 > MG_WAIT_NS) {
        atomicCAS(c.status, 0, code);
        *c.dead = 1;
        return true;
    }
    return false;
}

// N tagged words at once: all loads are issued before any tag is looked at, so the common case (everything has
// arrived) costs one round trip, not N; while some are stale, the stale ones are re-read together.  `addr(u)` gives
// the address of word u, or null for a slot that is not used (its value reads as 0).
template <int N, class Addr>
__device__ __forceinline__ void wait_words(Addr addr, float (&out)[N], unsigned tag, const Ctl& c, int code) {
    uint2 w[N];
    bool all = true;
#pragma unroll
    for (int u = 0; u < N; ++u) {
        const float2* p = addr(u);
        w[u] = p ? ld_word(p) : make_uint2(0u, tag);
    }
#pragma unroll
    for (int u = 0; u < N; ++u) all = all && (w[u].y == tag);
    if (!all && !*c.dead) {
        const unsigned long long t0 = global_timer_ns();
        unsigned spins = 0;
        for (;;) {
#pragma unroll
            for (int u = 0; u < N; ++u)
                if (w[u].y != tag) w[u] = ld_word(addr(u));
            all = true;
#pragma unroll
            for (int u = 0; u < N; ++u) all = all && (w[u].y == tag);
            if (all) break;
            if ((++spins & 63u) == 0 && wait_expired(c, t0, code)) break;
        }
    }
#pragma unroll
    for (int u = 0; u < N; ++u) out[u] = (w[u].y == tag) ? __uint_as_float(w[u].x) : 0.f;
}

// The same for N pairs of neighbouring words, one 16-byte load per pair (addresses 16-byte aligned).
template <int N, class Addr>
__device__ __forceinline__ void wait_pairs(Addr addr, float (&out)[2 * N], unsigned tag, const Ctl& c, int code) {
    uint4 w[N];
    bool all = true;
#pragma unroll
    for (int u = 0; u < N; ++u) {
        const float2* p = addr(u);
        w[u] = p ? ld_words2(p) : make_uint4(0u, tag, 0u, tag);
    }
#pragma unroll
    for (int u = 0; u < N; ++u) all = all && (w[u].y == tag) && (w[u].w == tag);
    if (!all && !*c.dead) {
        const unsigned long long t0 = global_timer_ns();
        unsigned spins = 0;
        for (;;) {
#pragma unroll
            for (int u = 0; u < N; ++u)
                if (w[u].y != tag || w[u].w != tag) w[u] = ld_words2(addr(u));
            all = true;
#pragma unroll
            for (int u = 0; u < N; ++u) all = all && (w[u].y == tag) && (w[u].w == tag);
            if (all) break;
            if ((++spins & 63u) == 0 && wait_expired(c, t0, code)) break;
        }
    }
#pragma unroll
    for (int u = 0; u < N; ++u) {
        out[2 * u] = (w[u].y == tag) ? __uint_as_float(w[u].x) : 0.f;
        out[2 * u + 1] = (w[u].w == tag) ? __uint_as_float(w[u].z) : 0.f;
    }
}

__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(MG_CTHREADS) : "memory"); }
__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(MG_GW * 32) : "memory"); }

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc::smem_u32(dst)), "l"(src), "r"(bytes), "r"(tc::smem_u32(bar)) : "memory");
}

// unsigned bytes of a times signed bytes of b
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Warps of a group that share a row (each takes a range of its 256-value blocks): rows longer than 4096 values are
// shared by 2 or 4 warps, and so are shorter ones when four rows per warp would not fit a ring stage otherwise.
__host__ __device__ __forceinline__ int ks_of(bool q6, int K, int stage_bytes, bool glu) {
    const int nb = K >> 8, rowbytes = q6 ? nb * 210 + 8 : nb * 144;
    int ks = K <= 4096 ? 1 : K <= 8192 ? 2 : 4;
    // a gated pair of matrices needs four rows (two gate / up pairs) per warp: share the rows rather than take fewer
    while (glu && ks < MG_GW && (MG_GW / ks) * 4 * rowbytes + 64 > stage_bytes) ks *= 2;
    return ks;
}

// Rows per warp and task: as many of 4, 2, 1 as fit a ring stage (`rowsets` warps of a group take different rows).
__host__ __device__ __forceinline__ int rw_of(bool q6, int nb, int rowsets, int stage_bytes) {
    const int rowbytes = q6 ? nb * 210 + 8 : nb * 144;               // Q6_K: plus its share of the super-scale padding
    for (int rw = 4; rw > 1; rw >>= 1)
        if (rowsets * rw * rowbytes + 64 <= stage_bytes) return rw;
    return 1;
}

// This CTA's share [lo, hi) of `total` items.
__device__ __forceinline__ void cta_range(int total, int& lo, int& hi) {
    lo = (int)((unsigned)total * blockIdx.x / gridDim.x);              // total * grid stays far below 2^32 (checked by the plan)
    hi = (int)((unsigned)total * (blockIdx.x + 1) / gridDim.x);
}

// Layout of one task inside a ring stage.  A task is `n` rows starting at row0 and, for a gated pair of matrices,
// the `n` rows glu_F further down behind them (local rows [0, n) and [n, 2n)).
//   Q4_K: the rows' GGUF blocks, contiguous per run of rows.
//   Q6_K: the four planes one after the other, each holding all local rows; the 2-byte super-scales of each run are
//         copied from the 16-byte boundary at or below their first byte (`lead` = distance from there to that byte).
struct TaskGeo { uint32_t b0, b1, b2, d0, d1, lead0, lead1; };

__device__ __forceinline__ TaskGeo task_geo(int type, int nb, int row0, int n, int glu_F) {
    TaskGeo g;
    const uint32_t nloc = glu_F > 0 ? 2u * n : (uint32_t)n;
    g.d0 = g.d1 = g.lead0 = g.lead1 = 0;
    if (type == TSB_Q4_K) {
        g.b0 = nloc * nb * 144u; g.b1 = g.b2 = 0;
    } else {
        g.b0 = nloc * nb * 128u; g.b1 = nloc * nb * 64u; g.b2 = nloc * nb * 16u;
        const long s0 = (long)row0 * nb * 2, e0 = s0 + (long)n * nb * 2;
        g.lead0 = (uint32_t)(s0 & 15);
        g.d0 = (uint32_t)(((e0 + 15) & ~15L) - (s0 & ~15L));
        if (glu_F > 0) {
            const long s1 = (long)(row0 + glu_F) * nb * 2, e1 = s1 + (long)n * nb * 2;
            g.lead1 = (uint32_t)(s1 & 15);
            g.d1 = (uint32_t)(((e1 + 15) & ~15L) - (s1 & ~15L));
        }
    }
    return g;
}

__device__ __forceinline__ void mg_mbar_wait(uint64_t* bar, uint32_t parity, const Ctl& c, int code) {
    const uint32_t addr = tc::smem_u32(bar);
    if (tc::mbar_try(addr, parity)) return;
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    for (;;) {
        if (tc::mbar_try(addr, parity)) return;
        if ((++spins & 15u) == 0 && wait_expired(c, t0, code)) return;
    }
}

// ------------------------------------------------------------------------------------------------
// Producer: one thread per CTA.  Mirrors the consumers' task order exactly.
// ------------------------------------------------------------------------------------------------
struct Producer {
    uint8_t* ring;
    uint64_t* full;
    uint64_t* empty;
    int stage_bytes, n_stages;
    unsigned t;                    // tasks issued
    Ctl ctl;
    int stage, round;              // stage of the next task and how many times the ring has wrapped
    __device__ bool task(const MegaMat& m, int row0, int n, int glu_F) {
        if (*ctl.dead) return false;
        const int s = stage;
        if (round > 0) {
            mg_mbar_wait(&empty[s], (uint32_t)(round - 1) & 1u, ctl, 201);
            if (*ctl.dead) return false;
        }
        if (++stage == n_stages) { stage = 0; ++round; }
        const int nb = m.K >> 8;
        const TaskGeo g = task_geo(m.type, nb, row0, n, glu_F);
        uint8_t* dst = ring + (long)s * stage_bytes;
        tc::mbar_expect_tx(&full[s], g.b0 + g.b1 + g.b2 + g.d0 + g.d1);
        for (int run = 0; run < (glu_F > 0 ? 2 : 1); ++run) {
            const long r = row0 + (long)run * glu_F;
            const uint32_t lr = (uint32_t)run * n;                       // first local row of this run
            if (m.type == TSB_Q4_K) {
                bulk_g2s(dst + lr * nb * 144u, m.p0 + r * nb * 144, (uint32_t)n * nb * 144u, &full[s]);
            } else {
                bulk_g2s(dst + lr * nb * 128u, m.p0 + r * nb * 128, (uint32_t)n * nb * 128u, &full[s]);
                bulk_g2s(dst + g.b0 + lr * nb * 64u, m.p1 + r * nb * 64, (uint32_t)n * nb * 64u, &full[s]);
                bulk_g2s(dst + g.b0 + g.b1 + lr * nb * 16u, m.p2 + r * nb * 16, (uint32_t)n * nb * 16u, &full[s]);
                bulk_g2s(dst + g.b0 + g.b1 + g.b2 + (run ? g.d0 : 0u), m.p3 + ((r * nb * 2) & ~15L), run ? g.d1 : g.d0, &full[s]);
            }
        }
        ++t;
        return true;
    }

    // rows [r0, r1) of m, one task per 16 / KS rows (or per 8 / KS gate / up pairs)
    __device__ void segment(const MegaMat& m, int r0, int r1, int glu_F) {
        const int rowsets = MG_GW / ks_of(m.type == TSB_Q6_K, m.K, stage_bytes, glu_F > 0);
        const int rt = rowsets * rw_of(m.type == TSB_Q6_K, m.K >> 8, rowsets, stage_bytes), step = glu_F > 0 ? rt / 2 : rt;
        for (int r = r0; r < r1; r += step)
            if (!task(m, r, min(step, r1 - r), glu_F)) return;
    }
};

// ------------------------------------------------------------------------------------------------
// Consumers: MG_GROUPS groups of MG_GW warps; task t belongs to group t % MG_GROUPS.  Inside a group a warp takes
// four rows of the task (or, for rows longer than 4096 values, a range of blocks of the four rows its warps share).
// ------------------------------------------------------------------------------------------------
struct Consumer {
    uint32_t ring;                 // shared-space address of the ring
    uint32_t full, empty;          // shared-space addresses of the mbarrier arrays
    int stage_bytes, n_stages;
    int stage, round;              // stage of the next task and how many times the ring has wrapped
    int turn;                      // which group takes the next task
    Ctl ctl;
    const int8_t* xq;              // shared: int8 activations of the current matrix
    const float* xd;               // shared: scale per 256 activations
    const int* bsum;               // shared: sum of the int8 activations per 16
    float* part;                   // shared: [2][MG_CWARPS][4] partial sums of rows shared by several warps
    int warp, lane;
    int debug;
    bool prof;                     // diagnostics: time spent waiting for stages, hoisting activations, computing
    unsigned long long wait_ns;
    unsigned tasks;
    unsigned hoist_ns, comp_ns;
};

// Stage loads.  Not volatile, so that the compiler may interleave the loads and the arithmetic of the four rows a
// warp works on; the row loop pins them between the stage's "full" wait and its release by data dependencies (the
// stage address passes through a volatile statement after the wait, the four sums through one before the release).
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint16_t lds16(uint32_t addr) {
    uint16_t v;
    asm("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ void mg_mbar_wait_addr(uint32_t addr, uint32_t parity, const Ctl& c, int code) {
    if (tc::mbar_try(addr, parity)) return;
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    for (;;) {
        if (tc::mbar_try(addr, parity)) return;
        if ((++spins & 15u) == 0 && wait_expired(c, t0, code)) return;
    }
}

// Shared-space addresses of a local row's data inside the stage.
struct RowPtr { uint32_t p0, p1, p2, p3; };

// The activation vector in shared memory: int8 values, one scale per 256, sums of the int8 values per 16.  The
// values are stored in 16-byte chunks, chunk (block b, c) at ((c & 3) * 4 nb + 4 b + (c >> 2)) * 16: the lanes of a
// warp work on neighbouring 64-value units, and this way their 16-byte loads fall on different banks.
struct ActMem { uint32_t xq, xd, bsum, plane; };                   // plane = 4 nb * 16 bytes

// Dot product of one 64-value unit of a row with the activations, scaled by the activation scale of its block.
//   Q4_K unit = (block b, pair sub): sub-blocks 2 sub and 2 sub + 1; the low nibbles go with the first 32
//               activations of the pair, the high nibbles with the other 32.
//   Q6_K unit = (block b, half n = sub >> 1, l-range 16 h, h = sub & 1): four groups of 16 values 32 apart.
template <bool Q6>
__device__ __forceinline__ float unit_dot(const ActMem& am, const RowPtr& r, int b, int sub) {
    const float xd = __uint_as_float(lds32(am.xd + 4u * b));
    if (!Q6) {
        const uint32_t xo = am.xq + 64u * b + 16u * sub;
        const uint4 hdr = lds128(r.p0 + 144u * b);
        const uint4 qa = lds128(r.p0 + 144u * b + 16u + 32u * sub);
        const uint4 qb = lds128(r.p0 + 144u * b + 32u + 32u * sub);
        const uint4 x0 = lds128(xo), x1 = lds128(xo + am.plane), x2 = lds128(xo + 2u * am.plane), x3 = lds128(xo + 3u * am.plane);
        const uint4 bq = lds128(am.bsum + 64u * b + 16u * sub);
        int s0 = 0, s1 = 0;
        s0 = dp4a_us(qa.x & 0x0F0F0F0Fu, (int)x0.x, s0); s0 = dp4a_us(qa.y & 0x0F0F0F0Fu, (int)x0.y, s0);
        s0 = dp4a_us(qa.z & 0x0F0F0F0Fu, (int)x0.z, s0); s0 = dp4a_us(qa.w & 0x0F0F0F0Fu, (int)x0.w, s0);
        s0 = dp4a_us(qb.x & 0x0F0F0F0Fu, (int)x1.x, s0); s0 = dp4a_us(qb.y & 0x0F0F0F0Fu, (int)x1.y, s0);
        s0 = dp4a_us(qb.z & 0x0F0F0F0Fu, (int)x1.z, s0); s0 = dp4a_us(qb.w & 0x0F0F0F0Fu, (int)x1.w, s0);
        // 16 x the sum over the high nibbles
        s1 = dp4a_us(qa.x & 0xF0F0F0F0u, (int)x2.x, s1); s1 = dp4a_us(qa.y & 0xF0F0F0F0u, (int)x2.y, s1);
        s1 = dp4a_us(qa.z & 0xF0F0F0F0u, (int)x2.z, s1); s1 = dp4a_us(qa.w & 0xF0F0F0F0u, (int)x2.w, s1);
        s1 = dp4a_us(qb.x & 0xF0F0F0F0u, (int)x3.x, s1); s1 = dp4a_us(qb.y & 0xF0F0F0F0u, (int)x3.y, s1);
        s1 = dp4a_us(qb.z & 0xF0F0F0F0u, (int)x3.z, s1); s1 = dp4a_us(qb.w & 0xF0F0F0F0u, (int)x3.w, s1);
        // 6-bit scales / minimums of the two sub-blocks as packed byte pairs, both encodings, then select
        const unsigned sh = 16u * (sub & 1);
        const uint32_t Y = hdr.y >> sh, Z = hdr.z >> sh, W = hdr.w >> sh;
        const uint32_t p_lo = Y & 0x3F3Fu, q_lo = Z & 0x3F3Fu;
        const uint32_t p_hi = (W & 0x0F0Fu) | ((Y >> 2) & 0x3030u), q_hi = ((W >> 4) & 0x0F0Fu) | ((Z >> 2) & 0x3030u);
        const uint32_t P = sub >= 2 ? p_hi : p_lo, Q = sub >= 2 ? q_hi : q_lo;
        const int iS = (int)((P & 0xFFu) << 4) * s0 + (int)(P >> 8) * s1;             // 16 x sum of scale x dot
        const int iM = (int)(Q & 0xFFu) * (int)(bq.x + bq.y) + (int)(Q >> 8) * (int)(bq.z + bq.w);
        const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
        return xd * (dd.x * 0.0625f * (float)iS - dd.y * (float)iM);
    } else {
        const int n = sub >> 1, h = sub & 1;
        const uint32_t xo = am.xq + 64u * b + 32u * n + h * am.plane;          // group k: chunk 8 n + 2 k + h
        const uint32_t o0 = 128u * b + 64u * n + 16u * h;
        const uint4 A = lds128(r.p0 + o0);
        const uint4 B = lds128(r.p0 + o0 + 32);
        const uint4 H = lds128(r.p1 + 64u * b + 32u * n + 16u * h);
        const uint2 sc8 = lds64(r.p2 + 16u * b + 8u * n);
        const float d = __half2float(__ushort_as_half(lds16(r.p3 + 2u * b)));
        const uint4 x0 = lds128(xo), x1 = lds128(xo + 2u * am.plane), x2 = lds128(xo + 16u), x3 = lds128(xo + 16u + 2u * am.plane);
        const uint4 ba = lds128(am.bsum + 64u * b + 32u * n), bb = lds128(am.bsum + 64u * b + 32u * n + 16u);
        const uint32_t a[4] = {A.x, A.y, A.z, A.w}, bw[4] = {B.x, B.y, B.z, B.w}, hw[4] = {H.x, H.y, H.z, H.w};
        const int xa[4] = {(int)x0.x, (int)x0.y, (int)x0.z, (int)x0.w}, xb[4] = {(int)x1.x, (int)x1.y, (int)x1.z, (int)x1.w};
        const int xc[4] = {(int)x2.x, (int)x2.y, (int)x2.z, (int)x2.w}, xe[4] = {(int)x3.x, (int)x3.y, (int)x3.z, (int)x3.w};
        int t0 = 0, t1 = 0, t2 = 0, t3 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t q0 = (a[i] & 0x0F0F0F0Fu) | ((hw[i] & 0x03030303u) << 4);
            const uint32_t q1 = (bw[i] & 0x0F0F0F0Fu) | ((hw[i] & 0x0C0C0C0Cu) << 2);
            const uint32_t q2 = ((a[i] >> 4) & 0x0F0F0F0Fu) | (hw[i] & 0x30303030u);
            const uint32_t q3 = ((bw[i] >> 4) & 0x0F0F0F0Fu) | ((hw[i] >> 2) & 0x30303030u);
            t0 = dp4a_us(q0, xa[i], t0);
            t1 = dp4a_us(q1, xb[i], t1);
            t2 = dp4a_us(q2, xc[i], t2);
            t3 = dp4a_us(q3, xe[i], t3);
        }
        // sums of the activations of the four groups: entries h, h + 2, h + 4, h + 6 of the half's eight
        const int b0 = h ? (int)ba.y : (int)ba.x, b1 = h ? (int)ba.w : (int)ba.z;
        const int b2 = h ? (int)bb.y : (int)bb.x, b3 = h ? (int)bb.w : (int)bb.z;
        // the stored value is q - 32: the offset goes through the activation sums
        const unsigned sel = 8u * h;
        const int c0 = (int)(int8_t)(sc8.x >> sel), c1 = (int)(int8_t)(sc8.x >> (sel + 16u));
        const int c2 = (int)(int8_t)(sc8.y >> sel), c3 = (int)(int8_t)(sc8.y >> (sel + 16u));
        const int iS = c0 * (t0 - 32 * b0) + c1 * (t1 - 32 * b1) + c2 * (t2 - 32 * b2) + c3 * (t3 - 32 * b3);
        return xd * d * (float)iS;
    }
}

// Where a finished row goes.
struct Emit {
    int mode;                      // 0: q/k/v word (+ bias); 1: partial sum to every rank; 2: activation word (bf16-rounded); 3: f32 logit
    float2* local;                 // modes 0, 2: destination words in this rank's buffer
    const float* bias;             // mode 0: or null
    float* logits;                 // mode 3
    float2* const* peers;          // mode 1: every rank's buffer (shared-memory copy of the argument array)
    long off;                      // mode 1: word offset of this rank's row block inside a buffer
    int ranks;
    unsigned tag;
};

// Up to four finished rows of a warp: row < 0 = nothing.  All lanes hold all four values.
__device__ __forceinline__ void emit_rows(const Emit& e, int r0, int r1, int r2, int r3, float v0, float v1, float v2, float v3, int lane) {
    if (e.mode == 1) {
        const int i = lane >> 3, r = lane & 7;                       // lane = (row slot, rank)
        const float val = i == 0 ? v0 : i == 1 ? v1 : i == 2 ? v2 : v3;
        const int rw = i == 0 ? r0 : i == 1 ? r1 : i == 2 ? r2 : r3;
        if (r < e.ranks && rw >= 0) st_word(e.peers[r] + e.off + rw, val, e.tag);
    } else if (e.mode == 2) {
        // gated activations travel as bf16, two to a word: rows (r0, r1) and (r2, r3) are even / odd neighbours
        if (lane < 2) {
            const int ra = lane == 0 ? r0 : r2, rb = lane == 0 ? r1 : r3;
            const float va = lane == 0 ? v0 : v2, vb = lane == 0 ? v1 : v3;
            if (ra >= 0) {
                const uint32_t w = (uint32_t)__bfloat16_as_ushort(f2bf(va)) | ((uint32_t)__bfloat16_as_ushort(f2bf(rb >= 0 ? vb : 0.f)) << 16);
                st_word(e.local + (ra >> 1), __uint_as_float(w), e.tag);
            }
        }
    } else if (lane < 4) {
        const float val = lane == 0 ? v0 : lane == 1 ? v1 : lane == 2 ? v2 : v3;
        const int rw = lane == 0 ? r0 : lane == 1 ? r1 : lane == 2 ? r2 : r3;
        if (rw >= 0) {
            if (e.mode == 0) st_word(e.local + rw, e.bias ? val + e.bias[rw] : val, e.tag);
            else e.logits[rw] = val;
        }
    }
}

// Rows [r0, r1) of a matrix with rows of K values against the activations in shared memory.  With glu_F > 0, rows
// r and r + glu_F are a gate / up pair and the emitted value is act(gate, up) for row r.  A warp's share of a task
// is a list of (row, unit) items; a lane takes every 32nd, two at a time.  Inlined at exactly one place per block
// type (the phase loop of the kernel): a call would have to save its caller's live registers to local memory, and
// with nearly all of the SM's memory configured as shared, local memory misses L1.
template <bool Q6>
__device__ __forceinline__ void run_rows(Consumer& c, int K, int r0, int r1, int glu_F, int act, const Emit& e) {
    if (r0 >= r1) return;
    const int nb = K >> 8, ks = ks_of(Q6, K, c.stage_bytes, glu_F > 0), rowsets = MG_GW / ks;
    const int rw = rw_of(Q6, nb, rowsets, c.stage_bytes), rt = rowsets * rw, half = rw >> 1;
    const int wg = c.warp & (MG_GW - 1), grp = c.warp / MG_GW, part = wg % ks, rowset = wg / ks;
    const int bs = (nb * part) / ks, be = (nb * (part + 1)) / ks;
    const int up = (be - bs) * 4;                                    // units per row part, <= 64
    const int total = rw * up;                                       // items of a warp's share of a task, <= 256
    const unsigned inv = (65536u + up - 1) / up;                     // (it * inv) >> 16 == it / up for it < 256
    const ActMem am{tc::smem_u32(c.xq), tc::smem_u32(c.xd), tc::smem_u32(c.bsum), (uint32_t)nb * 64u};
    const int step = glu_F > 0 ? rt / 2 : rt;
    const uint32_t rb0 = Q6 ? nb * 128u : nb * 144u, rb1 = nb * 64u, rb2 = nb * 16u, rb3 = nb * 2u;
    for (int r = r0; r < r1; r += step) {
        const bool take = c.turn == grp;
        const int s = c.stage;
        const uint32_t par = (uint32_t)c.round & 1u;
        c.turn = c.turn + 1 == MG_GROUPS ? 0 : c.turn + 1;
        if (++c.stage == c.n_stages) { c.stage = 0; ++c.round; }
        ++c.tasks;
        if (!take) continue;
        const int n = min(step, r1 - r);
        // the stage of this task.  Once a wait anywhere has given up, nothing waits any more: every warp still walks
        // the whole schedule (so that the barriers inside it stay matched) over whatever the stages hold, and the
        // step's result is discarded by the host, which sees the status word.
        unsigned long long tp0 = 0;
        if (c.prof) tp0 = global_timer_ns();
        if (!*c.ctl.dead && !(c.debug & 2)) mg_mbar_wait_addr(c.full + 8u * s, par, c.ctl, 200);
        uint32_t st = c.ring + (uint32_t)s * c.stage_bytes;
        asm volatile("" : "+r"(st) : : "memory");                    // the stage is read only after the wait above
        if (c.prof) { const unsigned long long t1 = global_timer_ns(); c.wait_ns += t1 - tp0; tp0 = t1; }
        const int lim = glu_F > 0 ? 2 * n : n;                       // local rows present in the stage
        TaskGeo g;
        if (Q6) g = task_geo(TSB_Q6_K, nb, r, n, glu_F);
        // value of item `it` (row ri of this warp's rows, unit u of the row part) and the row it belongs to.
        // Local rows: plain: rowset * rw + ri; gated: the warp's rw / 2 pairs, gate rows first, then up rows.  Rows
        // beyond the task are clamped to its last row: their sums are computed and never emitted.
        auto item = [&](int it, int& ri) -> float {
            ri = (int)(((unsigned)it * inv) >> 16);
            const int u = it - ri * up;
            int lr = glu_F > 0 ? (ri < half ? rowset * half + ri : n + rowset * half + ri - half) : rowset * rw + ri;
            lr = min(lr, lim - 1);
            RowPtr rp;
            rp.p0 = st + (uint32_t)lr * rb0;
            rp.p1 = rp.p2 = rp.p3 = 0;
            if (Q6) {
                rp.p1 = st + g.b0 + (uint32_t)lr * rb1;
                rp.p2 = st + g.b0 + g.b1 + (uint32_t)lr * rb2;
                const bool second = glu_F > 0 && lr >= n;
                rp.p3 = st + g.b0 + g.b1 + g.b2 + (second ? g.d0 + g.lead1 + (uint32_t)(lr - n) * rb3 : g.lead0 + (uint32_t)lr * rb3);
            }
            return unit_dot<Q6>(am, rp, bs + (u >> 2), u & 3);
        };
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (int it = c.lane; it < ((c.debug & 1) ? 0 : total); it += 64) {
            int ra, rb;
            const float va = item(it, ra);
            const bool second = it + 32 < total;
            float vb = item(second ? it + 32 : it, rb);
            vb = second ? vb : 0.f;
            a0 += (ra == 0 ? va : 0.f) + (rb == 0 ? vb : 0.f);
            a1 += (ra == 1 ? va : 0.f) + (rb == 1 ? vb : 0.f);
            a2 += (ra == 2 ? va : 0.f) + (rb == 2 ? vb : 0.f);
            a3 += (ra == 3 ? va : 0.f) + (rb == 3 ? vb : 0.f);
        }
        a0 = warp_sum(a0); a1 = warp_sum(a1); a2 = warp_sum(a2); a3 = warp_sum(a3);
        asm volatile("" : "+f"(a0), "+f"(a1), "+f"(a2), "+f"(a3) : : "memory");    // every read of the stage is behind us
        if (c.prof) c.comp_ns += (unsigned)(global_timer_ns() - tp0);
        __syncwarp();
        if (c.lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(c.empty + 8u * s) : "memory");
        if (ks > 1) {
            // the warps that share these rows add their parts through shared memory (double-buffered by task parity)
            float* pp = c.part + ((c.tasks / MG_GROUPS) & 1) * MG_CWARPS * 4;
            if (c.lane < 4) pp[c.warp * 4 + c.lane] = c.lane == 0 ? a0 : c.lane == 1 ? a1 : c.lane == 2 ? a2 : a3;
            group_sync(2 + grp);
            if (part == 0) {
                a0 = a1 = a2 = a3 = 0.f;
                for (int k = 0; k < ks; ++k) {
                    a0 += pp[(c.warp + k) * 4]; a1 += pp[(c.warp + k) * 4 + 1]; a2 += pp[(c.warp + k) * 4 + 2]; a3 += pp[(c.warp + k) * 4 + 3];
                }
            }
        }
        if (part != 0) continue;
        if (glu_F > 0) {
            // sums: [gate pairs 0 .. half), [up pairs 0 .. half)
            const int pb = rowset * half;
            emit_rows(e, pb < n ? r + pb : -1, pb + 1 < n ? r + pb + 1 : -1, -1, -1, act_glu(act, a0, a2), act_glu(act, a1, a3), 0.f, 0.f, c.lane);
        } else {
            const int b4 = rowset * rw;
            emit_rows(e, b4 < n ? r + b4 : -1, (rw > 1 && b4 + 1 < n) ? r + b4 + 1 : -1, (rw > 2 && b4 + 2 < n) ? r + b4 + 2 : -1,
                      (rw > 2 && b4 + 3 < n) ? r + b4 + 3 : -1, a0, a1, a2, a3, c.lane);
        }
    }
}

// 256 values (8 consecutive per lane) -> one int8 block: scale amax / 127, sums of the int8 values per 16.
__device__ __forceinline__ void quant_block(const float (&v)[8], int8_t* xq, float* xd, int* bsum, int block, int nblk, int lane) {
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(v[i]));
    am = warp_max(am);
    const float id = am > 0.f ? 127.f / am : 0.f;
    int q[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { q[i] = __float2int_rn(v[i] * id); s += q[i]; }
    uint2 pk;
    pk.x = (uint32_t)(q[0] & 0xFF) | ((uint32_t)(q[1] & 0xFF) << 8) | ((uint32_t)(q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
    pk.y = (uint32_t)(q[4] & 0xFF) | ((uint32_t)(q[5] & 0xFF) << 8) | ((uint32_t)(q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
    const int cb = lane >> 1;                                          // chunk within the block; see ActMem for the layout
    *reinterpret_cast<uint2*>(xq + (((cb & 3) * 4 * nblk + 4 * block + (cb >> 2)) << 4) + (lane & 1) * 8) = pk;
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if (!(lane & 1)) bsum[block * 16 + (lane >> 1)] = s;
    if (lane == 0) xd[block] = am / 127.f;
}

// Sum over the consumer threads; `red` is shared scratch of 32 floats.
__device__ __forceinline__ float cons_sum(float v, float* red, int warp, int lane) {
    v = warp_sum(v);
    cons_sync();
    if (lane == 0) red[warp] = v;
    cons_sync();
    float r = lane < MG_CWARPS ? red[lane] : 0.f;
    return warp_sum(r);
}

template <int DH, int G>
__device__ __forceinline__ void attention_item(const MegaArgs& a, const MegaLayer& L, const Ctl& ctl, unsigned tag_qkv, unsigned tag_part,
                                               float* qs, float* red, const float2* rope_cs, int item, int warp, int lane, float2* mine,
                                               unsigned (&at)[4], bool prof) {
    unsigned long long tl = prof ? global_timer_ns() : 0ull;
#define AT_MARK(i) do { if (prof) { const unsigned long long n_ = global_timer_ns(); at[i] += (unsigned)(n_ - tl); tl = n_; } } while (0)
    // red: [MG_CWARPS][G][DH] partial outputs, then [MG_CWARPS][G][2] (m, l), then a [MG_CWARPS][DH] rope stage
    constexpr int NJ = DH / 32, DPL = DH / 32, QD = DH / 4;
    float* red_o = red;
    float* red_ml = red + MG_CWARPS * G * DH;
    float* stage = red_ml + MG_CWARPS * G * 2;
    const int S = a.splits;
    const int kvh = item / S, split = item % S;
    const int pos = a.positions[0], len = a.kv_lens[0];
    const int per = (((len + S - 1) / S) + 7) & ~7;
    const int s0 = split * per, s1 = min(len, s0 + per);
    const bool owner = pos >= s0 && pos < s1;
    const float2* xw = mine + a.off_qkv;
    // ---- per-head RMSNorm + RoPE of the G query heads (and of the new K row; V as it is) ----
    for (int job = warp; job < G + 2; job += MG_CWARPS) {
        if (job >= G && !owner) continue;
        const int kind = job < G ? 0 : job - G + 1;          // 0 q, 1 k, 2 v
        const long row = kind == 0 ? (long)(kvh * G + job) * DH : kind == 1 ? (long)(a.Hq + kvh) * DH : (long)(a.Hq + a.Hkv + kvh) * DH;
        float v[NJ], ss = 0.f;
        wait_words<NJ>([&](int j) { return xw + row + lane + 32 * j; }, v, tag_qkv, ctl, 100 + PH_QKV);
        AT_MARK(0);
#pragma unroll
        for (int j = 0; j < NJ; ++j) ss += v[j] * v[j];
        const float* nw = kind == 0 ? L.q_norm : (kind == 1 ? L.k_norm : nullptr);
        if (nw) {
            ss = warp_sum(ss);
            const float rs = rsqrtf(ss / (float)DH + a.eps);
#pragma unroll
            for (int j = 0; j < NJ; ++j) v[j] *= rs * nw[lane + 32 * j];
        }
        const int rot = a.rot_dim, half = rot >> 1;
        float o[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) o[j] = v[j];
        if (kind != 2 && rot > 0) {
            if (a.rope_mode == 0) {
                float* st = stage + warp * DH;
                __syncwarp();
#pragma unroll
                for (int j = 0; j < NJ; ++j) st[lane + 32 * j] = v[j];
                __syncwarp();
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const int e = lane + 32 * j;
                    if (e < rot) {
                        const int pair = e < half ? e : e - half;
                        const float cs = rope_cs[pair].x, sn = rope_cs[pair].y;
                        const float x0 = st[pair], x1 = st[pair + half];
                        o[j] = e < half ? x0 * cs - x1 * sn : x0 * sn + x1 * cs;
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const int e = lane + 32 * j;
                    const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
                    if (e < rot) {
                        const float cs = rope_cs[e >> 1].x, sn = rope_cs[e >> 1].y;
                        o[j] = (e & 1) ? other * sn + v[j] * cs : v[j] * cs - other * sn;
                    }
                }
            }
        }
        if (kind == 0) {
#pragma unroll
            for (int j = 0; j < NJ; ++j) qs[job * DH + lane + 32 * j] = bf2f(f2bf(o[j]));     // the cache holds bf16; so does q
        } else {
            bf16* dst = (kind == 1 ? L.k_cache : L.v_cache) + (a.slots[0] * a.Hkv + kvh) * DH;
#pragma unroll
            for (int j = 0; j < NJ; ++j) dst[lane + 32 * j] = f2bf(o[j]);
        }
    }
    cons_sync();                                   // q in shared memory; the new K / V row visible to this CTA
    AT_MARK(1);
    // ---- split-KV attention: lane = (position p of a chunk of 8, quarter c of the head dims) ----
    float m[G], l[G], acc[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[g][d] = 0.f;
    }
    const int p = lane >> 2, cq = lane & 3;
    // the block-table entries of the first two passes are requested together, ahead of the loop
    int page_pre[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int j = s0 + warp * 8 + k * MG_CWARPS * 8 + p;
        page_pre[k] = j < s1 ? a.block_table[j / a.page_size] : 0;
    }
    int pass = 0;
    for (int base = s0 + warp * 8; base < s1; base += MG_CWARPS * 8, ++pass) {
        const int j = base + p;
        const bool valid = j < s1;
        long slot = 0;
        if (valid) slot = (long)(pass == 0 ? page_pre[0] : pass == 1 ? page_pre[1] : a.block_table[j / a.page_size]) * a.page_size + j % a.page_size;
        uint4 kreg[QD / 8];
        {
            const uint4* kp = reinterpret_cast<const uint4*>(L.k_cache + (slot * a.Hkv + kvh) * DH + cq * QD);
#pragma unroll
            for (int i = 0; i < QD / 8; ++i) kreg[i] = valid ? kp[i] : make_uint4(0u, 0u, 0u, 0u);
        }
        uint32_t vreg[8][(DPL + 1) / 2];
        const int cnt = min(8, s1 - base);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const long sl = __shfl_sync(0xffffffffu, slot, u * 4);
            const bf16* vp = L.v_cache + (sl * a.Hkv + kvh) * DH + lane * DPL;
#pragma unroll
            for (int i = 0; i < (DPL + 1) / 2; ++i)
                vreg[u][i] = u < cnt ? (DPL >= 2 ? reinterpret_cast<const uint32_t*>(vp)[i] : (uint32_t)*reinterpret_cast<const unsigned short*>(vp)) : 0u;
        }
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = 0.f;
#pragma unroll
        for (int i = 0; i < QD / 8; ++i) {
            const uint32_t kw[4] = {kreg[i].x, kreg[i].y, kreg[i].z, kreg[i].w};
            float kf[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                kf[2 * e] = __uint_as_float(kw[e] << 16);
                kf[2 * e + 1] = __uint_as_float(kw[e] & 0xffff0000u);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4 q0 = *reinterpret_cast<const float4*>(qs + g * DH + cq * QD + i * 8);
                const float4 q1 = *reinterpret_cast<const float4*>(qs + g * DH + cq * QD + i * 8 + 4);
                s[g] += q0.x * kf[0] + q0.y * kf[1] + q0.z * kf[2] + q0.w * kf[3] + q1.x * kf[4] + q1.y * kf[5] + q1.z * kf[6] + q1.w * kf[7];
            }
        }
        float pr[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float sv = s[g];
            sv += __shfl_xor_sync(0xffffffffu, sv, 1);
            sv += __shfl_xor_sync(0xffffffffu, sv, 2);
            sv = valid ? sv * a.attn_scale : -INFINITY;
            float mx = sv;
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            mx = fmaxf(m[g], mx);
            const float corr = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mx);
            pr[g] = valid ? __expf(sv - mx) : 0.f;
            float ps = pr[g];
            ps += __shfl_xor_sync(0xffffffffu, ps, 4);
            ps += __shfl_xor_sync(0xffffffffu, ps, 8);
            ps += __shfl_xor_sync(0xffffffffu, ps, 16);
            l[g] = l[g] * corr + ps;
            m[g] = mx;
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[g][d] *= corr;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            float vf[DPL];
#pragma unroll
            for (int d = 0; d < DPL; ++d) {
                const uint32_t w = vreg[u][d >> 1];
                vf[d] = (d & 1) ? __uint_as_float(w & 0xffff0000u) : __uint_as_float(w << 16);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float pg = __shfl_sync(0xffffffffu, pr[g], u * 4);
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[g][d] += pg * vf[d];
            }
        }
    }
    AT_MARK(2);
    // ---- merge the warps, publish the partial ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) { red_ml[(warp * G + g) * 2] = m[g]; red_ml[(warp * G + g) * 2 + 1] = l[g]; }
#pragma unroll
        for (int d = 0; d < DPL; ++d) red_o[(warp * G + g) * DH + lane * DPL + d] = acc[g][d];
    }
    cons_sync();
    float2* out = mine + a.off_part;
    for (int i = warp * 32 + lane; i < G * DH; i += MG_CTHREADS) {
        const int g = i / DH, d = i % DH;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < MG_CWARPS; ++w) mm = fmaxf(mm, red_ml[(w * G + g) * 2]);
        float ll = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < MG_CWARPS; ++w) {
            const float mw = red_ml[(w * G + g) * 2];
            const float cw = (mw == -INFINITY) ? 0.f : __expf(mw - mm);
            ll += red_ml[(w * G + g) * 2 + 1] * cw;
            o += red_o[(w * G + g) * DH + d] * cw;
        }
        const long pb = ((long)(kvh * G + g) * S + split) * (DH + 2);
        st_word(out + pb + d, o, tag_part);
        if (d == 0) { st_word(out + pb + DH, mm, tag_part); st_word(out + pb + DH + 1, ll, tag_part); }
    }
    AT_MARK(3);
#undef AT_MARK
}

template <int DH, int G>
__global__ void __launch_bounds__(MG_THREADS, 1) mega_decode_kernel(const MegaArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t full[MG_MAX_STAGES], empty[MG_MAX_STAGES];
    __shared__ int dead_flag;
    __shared__ float red32[32];
    __shared__ float part_s[2 * MG_CWARPS * 4];
    __shared__ float2* peers_s[MG_MAX_RANKS];
    __shared__ float2 rope_s[64];                       // rot_dim / 2 <= 64 (head sizes up to 128)
    __shared__ __align__(16) MegaLayer layer_s[2];     // this layer's and the next layer's descriptors (global reads cost a round trip each)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < MG_MAX_RANKS) peers_s[tid] = a.xbuf[tid];
    if (tid == 0) {
        dead_flag = 0;
        for (int s = 0; s < a.n_stages; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], MG_GW); }
        tc::fence_barrier_init();
    }
    __syncthreads();
    Ctl ctl{&dead_flag, a.status};
    const int R = a.size, D = a.hidden;
    const int nq = a.Hq * DH;

    if (warp == MG_CWARPS) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            Producer pr{smem + a.off_ring, full, empty, a.stage_bytes, a.n_stages, 0u, ctl, 0, 0};
            int lo, hi;
            for (int l = 0; l < a.n_layers && !dead_flag; ++l) {
                const MegaLayer& L = a.layers[l];
                const int tot = L.qkv[0].N + L.qkv[1].N + L.qkv[2].N;
                cta_range(tot, lo, hi);
                int o = 0;
                for (int i = 0; i < 3; ++i) {
                    const int n = L.qkv[i].N;
                    if (n > 0) pr.segment(L.qkv[i], max(lo, o) - o, min(hi, o + n) - o, 0);
                    o += n;
                }
                cta_range(L.wo.N, lo, hi);
                pr.segment(L.wo, lo, hi, 0);
                cta_range(a.ffn >> 1, lo, hi);
                pr.segment(L.gate_up, 2 * lo, 2 * hi, a.ffn);
                cta_range(L.down.N, lo, hi);
                pr.segment(L.down, lo, hi, 0);
            }
            cta_range(a.lm_head.N, lo, hi);
            pr.segment(a.lm_head, lo, hi, 0);
            if (dead_flag) {
                // going down: let the copies already issued land before the CTA's shared memory goes away
                const unsigned t1 = pr.t, t0 = t1 > (unsigned)a.n_stages ? t1 - a.n_stages : 0u;
                for (unsigned t = t0; t < t1; ++t) tc::mbar_wait(&full[t % a.n_stages], (t / a.n_stages) & 1, 200000000ull);
            }
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
    float* h = reinterpret_cast<float*>(smem + a.off_h);
    int8_t* xq = reinterpret_cast<int8_t*>(smem + a.off_xq);
    float* xd = reinterpret_cast<float*>(smem + a.off_xds);
    int* bsum = reinterpret_cast<int*>(smem + a.off_xds) + (a.off_bsum_words);
    float* qs = reinterpret_cast<float*>(smem + a.off_qs);
    float* red = reinterpret_cast<float*>(smem + a.off_red);
    Consumer c{tc::smem_u32(smem + a.off_ring), tc::smem_u32(full), tc::smem_u32(empty), a.stage_bytes, a.n_stages, 0, 0, 0, ctl,
               xq, xd, bsum, part_s, warp, lane, a.debug, a.prof != nullptr, 0ull, 0u, 0u, 0u};
    const unsigned step = *reinterpret_cast<volatile unsigned*>(a.step);
    const unsigned tag0 = step * (unsigned)((a.n_layers + 1) * PH_STRIDE) + 1u;
    float2* mine = peers_s[a.rank];

    // cos / sin of this step's position for every rotated pair (all layers and heads use the same)
    if (tid < (a.rot_dim >> 1)) {
        float sn, cs;
        sincosf((float)a.positions[0] * a.rope_freq[tid], &sn, &cs);
        rope_s[tid] = make_float2(cs * a.rope_mscale, sn * a.rope_mscale);
    }
    // token embedding -> residual stream
    {
        const long tok = a.tokens[0];
        for (int k8 = tid; k8 < (D >> 3); k8 += MG_CTHREADS) {
            float o[8];
            dequant8(a.embed, tok, k8, o);
#pragma unroll
            for (int i = 0; i < 8; ++i) h[8 * k8 + i] = o[i] * a.embed_scale;
        }
    }
    cons_sync();

    // h += sum over ranks of the tagged partial sums at word offset `off` (when `gather`), then RMSNorm of h with
    // weight w into the int8 activation buffers.  A warp owns whole 256-value blocks (lane = 8 consecutive values),
    // so the residual update, the sum of squares and the quantisation stay in registers; the norm weights are
    // requested before the partial sums are waited for, and the words come two per 16-byte load.
    auto gather_norm = [&](bool gather, long off, unsigned tag, int code, const float* w) {
        const int nblk = D >> 8;
        float ss = 0.f;
        if (nblk <= 2 * MG_CWARPS) {
            float hv[2][8], wv[2][8];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int b = warp + MG_CWARPS * j;
                const bool ok = b < nblk;
                const int i = (ok ? b : 0) * 256 + lane * 8;
                const float4 w0 = ok ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 w1 = ok ? *reinterpret_cast<const float4*>(w + i + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 h0 = ok ? *reinterpret_cast<const float4*>(h + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 h1 = ok ? *reinterpret_cast<const float4*>(h + i + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                wv[j][0] = w0.x; wv[j][1] = w0.y; wv[j][2] = w0.z; wv[j][3] = w0.w; wv[j][4] = w1.x; wv[j][5] = w1.y; wv[j][6] = w1.z; wv[j][7] = w1.w;
                hv[j][0] = h0.x; hv[j][1] = h0.y; hv[j][2] = h0.z; hv[j][3] = h0.w; hv[j][4] = h1.x; hv[j][5] = h1.y; hv[j][6] = h1.z; hv[j][7] = h1.w;
            }
            if (gather && nblk <= MG_CWARPS) {
                // one block per warp: the words of two ranks are requested together (the registers the two-block form
                // uses for its second block), so eight ranks cost four round trips through L2 instead of eight; the
                // parts are still added in rank order
                for (int r0 = 0; r0 < R; r0 += 2) {
                    float v[16];
                    wait_pairs<8>([&](int u) -> const float2* {
                        const int r = r0 + (u >> 2);
                        return (warp < nblk && r < R) ? mine + off + (long)r * D + warp * 256 + lane * 8 + 2 * (u & 3) : nullptr;
                    }, v, tag, ctl, code);
#pragma unroll
                    for (int u = 0; u < 16; ++u) hv[0][u & 7] += v[u];            // (an absent rank reads as 0)
                }
            } else if (gather) {
                for (int r = 0; r < R; ++r) {                              // parts are added in rank order
                    float v[16];
                    wait_pairs<8>([&](int u) -> const float2* {
                        const int b = warp + MG_CWARPS * (u >> 2);
                        return b < nblk ? mine + off + (long)r * D + b * 256 + lane * 8 + 2 * (u & 3) : nullptr;
                    }, v, tag, ctl, code);
#pragma unroll
                    for (int u = 0; u < 16; ++u) hv[u >> 3][u & 7] += v[u];
                }
            }
            if (gather) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int b = warp + MG_CWARPS * j;
                    if (b < nblk) {
                        float* hp = h + b * 256 + lane * 8;
                        *reinterpret_cast<float4*>(hp) = make_float4(hv[j][0], hv[j][1], hv[j][2], hv[j][3]);
                        *reinterpret_cast<float4*>(hp + 4) = make_float4(hv[j][4], hv[j][5], hv[j][6], hv[j][7]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += hv[j][i] * hv[j][i];
            ss = cons_sum(ss, red32, warp, lane);                      // (its barriers also fence the previous readers of xq)
            const float rs = rsqrtf(ss / (float)D + a.eps);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int b = warp + MG_CWARPS * j;
                if (b < nblk) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = hv[j][i] * rs * wv[j][i];
                    quant_block(v, xq, xd, bsum, b, nblk, lane);
                }
            }
        } else {
            if (gather) {
                for (int b = warp; b < nblk; b += MG_CWARPS)
                    for (int r = 0; r < R; ++r) {
                        float v[8];
                        wait_pairs<4>([&](int u) { return mine + off + (long)r * D + b * 256 + lane * 8 + 2 * u; }, v, tag, ctl, code);
#pragma unroll
                        for (int i = 0; i < 8; ++i) h[b * 256 + lane * 8 + i] += v[i];
                    }
            }
            for (int b = warp; b < nblk; b += MG_CWARPS)
#pragma unroll
                for (int i = 0; i < 8; ++i) { const float x = h[b * 256 + lane * 8 + i]; ss += x * x; }
            ss = cons_sum(ss, red32, warp, lane);
            const float rs = rsqrtf(ss / (float)D + a.eps);
            for (int b = warp; b < nblk; b += MG_CWARPS) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = h[b * 256 + lane * 8 + i] * rs * w[b * 256 + lane * 8 + i];
                quant_block(v, xq, xd, bsum, b, nblk, lane);
            }
        }
        cons_sync();
    };
    // n tagged values at `off` -> int8 activation buffers.  The values are bf16, two per word; a warp takes whole
    // 256-value blocks (a lane's 8 values are two 16-byte loads), four blocks of loads in flight.
    auto gather_quant = [&](long off, int n, unsigned tag, int code) {
        cons_sync();                                // nobody still reads the previous contents of the activation buffers
        const int nblk = n >> 8;
        for (int b0 = warp; b0 < nblk; b0 += 4 * MG_CWARPS) {
            float v[16];
            wait_pairs<8>([&](int u) -> const float2* {
                const int b = b0 + MG_CWARPS * (u >> 1);
                return b < nblk ? mine + off + b * 128 + lane * 4 + 2 * (u & 1) : nullptr;
            }, v, tag, ctl, code);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int b = b0 + MG_CWARPS * j;
                if (b < nblk) {
                    float x[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t w = __float_as_uint(v[4 * j + i]);
                        x[2 * i] = __uint_as_float(w << 16);
                        x[2 * i + 1] = __uint_as_float(w & 0xffff0000u);
                    }
                    quant_block(x, xq, xd, bsum, b, nblk, lane);
                }
            }
        }
        cons_sync();
    };

    unsigned pt[24];
    unsigned long long plast = 0;
#pragma unroll
    for (int i = 0; i < 24; ++i) pt[i] = 0u;
    const bool prof = a.prof != nullptr;
    unsigned at4[4] = {0u, 0u, 0u, 0u};
    if (prof) plast = global_timer_ns();
    // time since the previous mark goes to slot i (thread 0's view of its CTA)
#define MG_MARK(i) do { if (prof) { const unsigned long long now_ = global_timer_ns(); pt[i] += (unsigned)(now_ - plast); plast = now_; } } while (0)
    // One loop over (layer, phase): every helper above is inlined at a single place.  Phases: 0 QKV, 1 o_proj,
    // 2 gate / up, 3 down; the pass after the last layer is the output norm and the lm_head rows.
    // descriptor of layer 0 now, of layer l + 1 while layer l runs (the copy is fenced by the barriers of the phases)
    auto fetch_layer = [&](int l) {
        if (l < a.n_layers && tid < (int)(sizeof(MegaLayer) / 4))
            reinterpret_cast<uint32_t*>(&layer_s[l & 1])[tid] = reinterpret_cast<const uint32_t*>(&a.layers[l])[tid];
    };
    fetch_layer(0);
    cons_sync();
    for (int l = 0; l <= a.n_layers; ++l) {
        const bool last = l == a.n_layers;
        const MegaLayer& L = layer_s[last ? 0 : (l & 1)];
        const unsigned tg = tag0 + (unsigned)l * PH_STRIDE;
        fetch_layer(l + 1);
        for (int ph = 0; ph < (last ? 1 : 4); ++ph) {
            // ---------------- what the phase's rows need ----------------
            if (ph == 0) {
                gather_norm(l > 0, a.off_dwn, tg - PH_STRIDE + PH_DWN, 100 + PH_DWN, last ? a.out_norm : L.attn_norm);
                MG_MARK(1);
            } else if (ph == 2) {
                gather_norm(true, a.off_opr, tg + PH_OPR, 100 + PH_OPR, L.ffn_norm);
                MG_MARK(8);
            } else if (ph == 1) {
                // attention: splits, then the merge per head
                if ((int)blockIdx.x < a.Hkv * a.splits)
                    attention_item<DH, G>(a, L, ctl, tg + PH_QKV, tg + PH_ATT, qs, red, rope_s, blockIdx.x, warp, lane, mine, at4, prof);
                MG_MARK(3);
                const int hd = (int)gridDim.x - 1 - (int)blockIdx.x;        // heads are merged by the CTAs at the far end of the grid
                if (hd < a.Hq && warp < DH / 32) {
                    // one warp per 32 dims; lanes fetch the (max, sum) of two splits each, the warp reduces them; the
                    // partial outputs come twelve splits at a time (everything of up to 12 splits in one round trip)
                    const int S = a.splits, d = warp * 32 + lane;
                    const float2* pp = mine + a.off_part + (long)hd * S * (DH + 2);
                    float ml[4], pv[12];
                    float c0 = 0.f, c1 = 0.f, ll = 0.f, o = 0.f;
                    for (int s0 = 0; s0 < S; s0 += 12) {
                        if (s0 == 0) {
                            float both[16];
                            wait_words<16>([&](int u) -> const float2* {
                                if (u < 4) { const int sp = lane + 32 * (u >> 1); return sp < S ? pp + (long)sp * (DH + 2) + DH + (u & 1) : nullptr; }
                                return u - 4 < S ? pp + (long)(u - 4) * (DH + 2) + d : nullptr;
                            }, both, tg + PH_ATT, ctl, 100 + PH_ATT);
#pragma unroll
                            for (int u = 0; u < 4; ++u) ml[u] = both[u];
#pragma unroll
                            for (int u = 0; u < 12; ++u) pv[u] = both[4 + u];
                            const float m0 = lane < S ? ml[0] : -INFINITY, m1 = lane + 32 < S ? ml[2] : -INFINITY;
                            const float mm = warp_max(fmaxf(m0, m1));
                            c0 = (m0 == -INFINITY) ? 0.f : __expf(m0 - mm);
                            c1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - mm);
                            ll = warp_sum((lane < S ? ml[1] : 0.f) * c0 + (lane + 32 < S ? ml[3] : 0.f) * c1);
                        } else {
                            wait_words<12>([&](int u) -> const float2* { return s0 + u < S ? pp + (long)(s0 + u) * (DH + 2) + d : nullptr; },
                                           pv, tg + PH_ATT, ctl, 100 + PH_ATT);
                        }
#pragma unroll
                        for (int u = 0; u < 12; ++u) {
                            const int sp = s0 + u;
                            const float cw = __shfl_sync(0xffffffffu, sp < 32 ? c0 : c1, sp & 31);
                            if (sp < S) o += pv[u] * cw;
                        }
                    }
                    // bf16, two dims to a word
                    const float val = ll > 0.f ? o / ll : 0.f, nb_ = __shfl_down_sync(0xffffffffu, val, 1);
                    if (!(lane & 1)) {
                        const uint32_t w = (uint32_t)__bfloat16_as_ushort(f2bf(val)) | ((uint32_t)__bfloat16_as_ushort(f2bf(nb_)) << 16);
                        st_word(mine + a.off_attn + (((long)hd * DH + d) >> 1), __uint_as_float(w), tg + PH_CMB);
                    }
                }
                MG_MARK(4);
            }
            if (ph == 1 || ph == 3) {
                gather_quant(ph == 1 ? a.off_attn : a.off_act, ph == 1 ? nq : a.ffn, tg + (ph == 1 ? PH_CMB : PH_GUP), 100 + (ph == 1 ? PH_CMB : PH_GUP));
                MG_MARK(ph == 1 ? 5 : 10);
            }
            // ---------------- the phase's rows ----------------
            const int nseg = (ph == 0 && !last) ? 3 : 1;
            int lo, hi, o = 0;
            if (last) cta_range(a.lm_head.N, lo, hi);
            else if (ph == 0) cta_range(L.qkv[0].N + L.qkv[1].N + L.qkv[2].N, lo, hi);
            else if (ph == 1) cta_range(L.wo.N, lo, hi);
            else if (ph == 2) { cta_range(a.ffn >> 1, lo, hi); lo *= 2; hi *= 2; }     // even bounds: activations are stored two to a word
            else cta_range(L.down.N, lo, hi);
            for (int si = 0; si < nseg; ++si) {
                const MegaMat* mp = last ? &a.lm_head : ph == 0 ? &L.qkv[si] : ph == 1 ? &L.wo : ph == 2 ? &L.gate_up : &L.down;
                const int mN = mp->N, mK = mp->K, mtype = mp->type;
                if (mN <= 0) continue;
                Emit e;
                e.ranks = R;
                e.peers = peers_s;
                e.logits = a.logits;
                e.bias = nullptr;
                e.local = mine;
                e.off = 0;
                int r0 = lo, r1 = hi, glu = 0;
                if (last) { e.mode = 3; e.tag = 0u; }
                else if (ph == 0) {
                    e.mode = 0; e.tag = tg + PH_QKV; e.local = mine + a.off_qkv + o; e.bias = L.qkv_bias ? L.qkv_bias + o : nullptr;
                    r0 = max(lo, o) - o; r1 = min(hi, o + mN) - o;
                    o += mN;
                } else if (ph == 2) { e.mode = 2; e.tag = tg + PH_GUP; e.local = mine + a.off_act; glu = a.ffn; }
                else { e.mode = 1; e.tag = tg + (ph == 1 ? PH_OPR : PH_DWN); e.off = (ph == 1 ? a.off_opr : a.off_dwn) + (long)a.rank * D; }
                if (mtype == TSB_Q4_K) run_rows<false>(c, mK, r0, r1, glu, a.act, e);
                else run_rows<true>(c, mK, r0, r1, glu, a.act, e);
            }
            MG_MARK(last ? 13 : ph == 0 ? 2 : ph == 1 ? 6 : ph == 2 ? 9 : 11);
        }
    }
    cons_sync();
    if (prof && tid == 0) {
#pragma unroll
        for (int i = 0; i < 24; ++i) a.prof[(long)blockIdx.x * 24 + i] = i == 14 ? c.wait_ns : i == 15 ? (unsigned long long)c.tasks : i == 0 ? (unsigned long long)c.hoist_ns : i == 7 ? (unsigned long long)c.comp_ns : i >= 16 && i < 20 ? (unsigned long long)at4[i - 16] : (unsigned long long)pt[i];
    }
#undef MG_MARK
    if (blockIdx.x == 0 && tid == 0) *a.step = step + 1u;
}

#endif  // __CUDACC__

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
#define MG_STAGE_BYTES 25600        // one ring stage; a task is as many rows as fit (rw_of)

// Bytes a task of this matrix occupies in a stage (with the padding of the Q6_K super-scale runs).
static int mg_task_bytes(int type, int K, bool glu) {
    const int nb = K >> 8, rowsets = MG_GW / ks_of(type == TSB_Q6_K, K, MG_STAGE_BYTES, glu), rt = rowsets * rw_of(type == TSB_Q6_K, nb, rowsets, MG_STAGE_BYTES);
    if (type == TSB_Q4_K) return rt * nb * 144;
    const int runs = glu ? 2 : 1;
    return rt * nb * 208 + runs * (((rt / runs * nb * 2 + 15) & ~15) + 16);
}

static bool mg_mat_ok(const MegaMat& m) {
    return (m.type == TSB_Q4_K || m.type == TSB_Q6_K) && m.K % 256 == 0 && m.K >= 256 && m.K <= 16384 && m.N > 0;
}

template <int DH, int G>
static int mg_launch(const MegaArgs& a, cudaStream_t s) {
    // dynamic shared memory above the default limit has to be allowed per kernel; the static part (about 1 KB)
    // counts against the same 227 KB, so the attribute follows what the plans actually ask for
    static std::mutex mu;
    static int allowed = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (a.smem_bytes > allowed) {
            TSB_CHECK_CUDA(cudaFuncSetAttribute(mega_decode_kernel<DH, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, a.smem_bytes));
            allowed = a.smem_bytes;
        }
    }
    void* params[] = {(void*)&a};
    TSB_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)mega_decode_kernel<DH, G>, dim3(a.grid), dim3(MG_THREADS), params,
                                               (size_t)a.smem_bytes, s));
    return TSB_OK;
}

// Checks the configuration and fills the launch plan (grid, ring geometry, shared-memory layout).  `layers` is a
// HOST copy of the layer table here (the kernel gets the device copy through args->layers).
extern "C" int tsb_mega_plan(MegaArgs* args, const MegaLayer* host_layers, int sm_count) {
    MegaArgs& a = *args;
    TSB_CHECK_ARG(a.n_layers >= 1 && a.size >= 1 && a.size <= MG_MAX_RANKS, "mega_plan: bad layer count %d or rank count %d", a.n_layers, a.size);
    TSB_CHECK_ARG(a.Dh == 64 || a.Dh == 128, "mega_plan: head dim %d (supported 64, 128)", a.Dh);
    TSB_CHECK_ARG(a.Hkv > 0 && a.Hq % a.Hkv == 0, "mega_plan: Hq=%d Hkv=%d", a.Hq, a.Hkv);
    const int G = a.Hq / a.Hkv;
    TSB_CHECK_ARG(G == 1 || G == 2 || G == 4 || G == 8, "mega_plan: %d query heads per KV head (supported 1, 2, 4, 8)", G);
    TSB_CHECK_ARG(a.hidden % 32 == 0 && a.ffn % 32 == 0 && a.hidden <= 16384 && a.ffn <= 65536, "mega_plan: hidden %d / ffn %d", a.hidden, a.ffn);
    TSB_CHECK_ARG(a.rot_dim % 2 == 0 && a.rot_dim <= a.Dh, "mega_plan: rot_dim %d", a.rot_dim);
    int kmax = a.hidden, min_rows = a.hidden;
    auto mat = [&](const MegaMat& m, const char* what, bool glu = false) -> bool {
        if (!mg_mat_ok(m)) { tsb_set_error("mega_plan: %s has type %d, K %d (needs Q4_K / Q6_K, K a multiple of 256 up to 16384)", what, m.type, m.K); return false; }
        kmax = m.K > kmax ? m.K : kmax;
        const int rowsets = MG_GW / ks_of(m.type == TSB_Q6_K, m.K, MG_STAGE_BYTES, glu);
        // (a gated pair needs its two gate / up pairs per warp: the activations are stored two to a word)
        if (mg_task_bytes(m.type, m.K, glu) > MG_STAGE_BYTES || (glu && rw_of(m.type == TSB_Q6_K, m.K >> 8, rowsets, MG_STAGE_BYTES) < 4)) {
            tsb_set_error("mega_plan: rows of %s (K %d) do not fit a ring stage", what, m.K);
            return false;
        }
        return true;
    };
    for (int l = 0; l < a.n_layers; ++l) {
        const MegaLayer& L = host_layers[l];
        int tot = 0;
        for (int i = 0; i < 3; ++i)
            if (L.qkv[i].N > 0) {
                if (!mat(L.qkv[i], "attn_q/k/v")) return TSB_ERR_UNSUPPORTED;
                TSB_CHECK_ARG(L.qkv[i].K == a.hidden, "mega_plan: qkv K %d != hidden %d", L.qkv[i].K, a.hidden);
                tot += L.qkv[i].N;
            }
        TSB_CHECK_ARG(tot == (a.Hq + 2 * a.Hkv) * a.Dh, "mega_plan: qkv rows %d != (Hq + 2 Hkv) Dh", tot);
        if (!mat(L.wo, "attn_output") || !mat(L.gate_up, "ffn_gate_up", true) || !mat(L.down, "ffn_down")) return TSB_ERR_UNSUPPORTED;
        TSB_CHECK_ARG(L.wo.N == a.hidden && L.wo.K == a.Hq * a.Dh && L.gate_up.N == 2 * a.ffn && L.gate_up.K == a.hidden &&
                      L.down.N == a.hidden && L.down.K == a.ffn, "mega_plan: layer %d matrix shapes do not fit the model sizes", l);
        min_rows = tot < min_rows ? tot : min_rows;
    }
    if (!mat(a.lm_head, "lm_head")) return TSB_ERR_UNSUPPORTED;
    TSB_CHECK_ARG(a.lm_head.K == a.hidden, "mega_plan: lm_head K %d", a.lm_head.K);
    min_rows = a.ffn < min_rows ? a.ffn : min_rows;
    min_rows = a.lm_head.N < min_rows ? a.lm_head.N : min_rows;
    // every CTA must own rows in every all-to-all phase (see the file comment): grid <= the smallest row count
    int grid = sm_count < min_rows ? sm_count : min_rows;
    TSB_CHECK_ARG(grid >= a.Hq && grid >= a.Hkv, "mega_plan: %d CTAs cannot hold %d heads", grid, a.Hq);
    a.grid = grid;
    a.splits = grid / a.Hkv;
    if (a.splits > 64) a.splits = 64;
    int off = 0;
    auto take = [&](int bytes) { const int o = off; off += (bytes + 127) & ~127; return o; };
    a.off_h = take(a.hidden * 4);
    a.off_xq = take(kmax);
    a.off_bsum_words = (kmax / 256 + 3) & ~3;               // scales per 256 first, then (16-byte aligned) the sums per 16
    a.off_xds = take((a.off_bsum_words + kmax / 16) * 4);
    a.off_qs = take(G * a.Dh * 4);
    a.off_red = take((MG_CWARPS * G * a.Dh + MG_CWARPS * G * 2 + MG_CWARPS * a.Dh) * 4);
    a.stage_bytes = MG_STAGE_BYTES;
    a.off_ring = take(0);
    const int avail = 227 * 1024 - 3072 - off;            // static shared memory of the kernel stays under 3 KB
    int ns = avail / a.stage_bytes;
    if (ns > MG_MAX_STAGES) ns = MG_MAX_STAGES;
    TSB_CHECK_ARG(ns > MG_GROUPS, "mega_plan: a stage of %d bytes leaves room for %d ring stages", a.stage_bytes, ns);
    a.n_stages = ns;
    a.smem_bytes = off + ns * a.stage_bytes;
    return TSB_OK;
}

// Words of one rank's exchange buffer for these sizes (regions in the order of the off_* fields); fills the offsets.
extern "C" long tsb_mega_xbuf_words(MegaArgs* args) {
    MegaArgs& a = *args;
    long off = 0;
    auto take = [&](long words) { const long o = off; off += (words + 15) & ~15L; return o; };
    a.off_qkv = take((long)(a.Hq + 2 * a.Hkv) * a.Dh);
    a.off_part = take((long)a.Hq * 64 * (a.Dh + 2));
    a.off_attn = take((long)a.Hq * a.Dh);
    a.off_opr = take((long)a.size * a.hidden);
    a.off_act = take(a.ffn);
    a.off_dwn = take((long)a.size * a.hidden);
    return off;
}

extern "C" int tsb_mega_args_bytes(void) { return (int)sizeof(MegaArgs); }
extern "C" int tsb_mega_layer_bytes(void) { return (int)sizeof(MegaLayer); }

extern "C" int tsb_mega_decode(const MegaArgs* args, void* stream) {
    const MegaArgs& a = *args;
    TSB_CHECK_ARG(a.grid > 0 && a.n_stages >= 2 && a.smem_bytes > 0, "mega_decode: the plan is missing (call tsb_mega_plan)");
    cudaStream_t s = (cudaStream_t)stream;
    const int G = a.Hq / a.Hkv;
#define MG_CASE(DHV, GV) if (a.Dh == DHV && G == GV) return mg_launch<DHV, GV>(a, s)
    MG_CASE(128, 1); MG_CASE(128, 2); MG_CASE(128, 4); MG_CASE(128, 8);
    MG_CASE(64, 1); MG_CASE(64, 2); MG_CASE(64, 4); MG_CASE(64, 8);
#undef MG_CASE
    tsb_set_error("mega_decode: unsupported head dim %d / group %d", a.Dh, G);
    return TSB_ERR_UNSUPPORTED;
}
