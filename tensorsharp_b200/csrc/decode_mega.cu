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
//   * Eight consumer warps per CTA (two groups that alternate tasks) take rows out of the ring, four rows
//     per warp at a time: Q4_K / Q6_K blocks against int8 activations with one scale per 256 values (the
//     contract of ggml's K-quant dot products on the CPU: ggml-quants.c, q8_K), so the 6-bit block scales
//     multiply integer partial sums and one float multiply-add finishes 64 weights; the lane's activation
//     words live in registers for the whole matrix.
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
#define MG_GROUPS 2
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
    unsigned long long* prof;      // null, or [grid][16] nanoseconds spent per phase by each CTA (diagnostics)
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

// A row longer than 4096 values is shared by 2 or 4 warps of a group (each takes a range of 256-value blocks).
__host__ __device__ __forceinline__ int ks_of(int K) { return K <= 4096 ? 1 : K <= 8192 ? 2 : 4; }

// This CTA's share [lo, hi) of `total` items.
__device__ __forceinline__ void cta_range(int total, int& lo, int& hi) {
    lo = (int)((long)total * blockIdx.x / gridDim.x);
    hi = (int)((long)total * (blockIdx.x + 1) / gridDim.x);
}

// Layout of one task inside a ring stage.  A task is `n` rows starting at row0 and, for a gated pair of matrices,
// the `n` rows glu_F further down behind them (local rows [0, n) and [n, 2n)).
//   Q4_K: the rows' GGUF blocks, contiguous per run of rows.
//   Q6_K: the four planes one after the other, each holding all local rows; the 2-byte super-scales of each run are
//         copied from the 16-byte boundary at or below their first byte (`lead` = distance from there to that byte).
struct TaskGeo { uint32_t b0, b1, b2, d_bytes[2], lead[2]; int nloc; };

__device__ __forceinline__ TaskGeo task_geo(const MegaMat& m, int row0, int n, int glu_F) {
    TaskGeo g;
    const int nb = m.K >> 8;
    g.nloc = glu_F > 0 ? 2 * n : n;
    g.d_bytes[0] = g.d_bytes[1] = g.lead[0] = g.lead[1] = 0;
    if (m.type == TSB_Q4_K) {
        g.b0 = (uint32_t)g.nloc * nb * 144u; g.b1 = g.b2 = 0;
    } else {
        g.b0 = (uint32_t)g.nloc * nb * 128u; g.b1 = (uint32_t)g.nloc * nb * 64u; g.b2 = (uint32_t)g.nloc * nb * 16u;
        for (int run = 0; run < (glu_F > 0 ? 2 : 1); ++run) {
            const long s = (long)(row0 + run * glu_F) * nb * 2, e = s + (long)n * nb * 2;
            g.lead[run] = (uint32_t)(s & 15);
            g.d_bytes[run] = (uint32_t)(((e + 15) & ~15L) - (s & ~15L));
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

    __device__ bool task(const MegaMat& m, int row0, int n, int glu_F) {
        if (*ctl.dead) return false;
        const int s = t % n_stages;
        if (t >= (unsigned)n_stages) {
            mg_mbar_wait(&empty[s], ((t / n_stages) - 1) & 1, ctl, 201);
            if (*ctl.dead) return false;
        }
        const TaskGeo g = task_geo(m, row0, n, glu_F);
        uint8_t* dst = ring + (long)s * stage_bytes;
        const int nb = m.K >> 8, runs = glu_F > 0 ? 2 : 1;
        tc::mbar_expect_tx(&full[s], g.b0 + g.b1 + g.b2 + g.d_bytes[0] + g.d_bytes[1]);
        uint32_t d_off = g.b0 + g.b1 + g.b2;
        for (int run = 0; run < runs; ++run) {
            const long r = row0 + (long)run * glu_F;
            const uint32_t lr = (uint32_t)run * n;                       // first local row of this run
            if (m.type == TSB_Q4_K) {
                bulk_g2s(dst + lr * nb * 144u, m.p0 + r * nb * 144, (uint32_t)n * nb * 144u, &full[s]);
            } else {
                bulk_g2s(dst + lr * nb * 128u, m.p0 + r * nb * 128, (uint32_t)n * nb * 128u, &full[s]);
                bulk_g2s(dst + g.b0 + lr * nb * 64u, m.p1 + r * nb * 64, (uint32_t)n * nb * 64u, &full[s]);
                bulk_g2s(dst + g.b0 + g.b1 + lr * nb * 16u, m.p2 + r * nb * 16, (uint32_t)n * nb * 16u, &full[s]);
                bulk_g2s(dst + d_off, m.p3 + ((r * nb * 2) & ~15L), g.d_bytes[run], &full[s]);
                d_off += g.d_bytes[run];
            }
        }
        ++t;
        return true;
    }

    // rows [r0, r1) of m, one task per 16 / KS rows (or per 8 / KS gate / up pairs)
    __device__ void segment(const MegaMat& m, int r0, int r1, int glu_F) {
        const int rt = (MG_GW / ks_of(m.K)) * 4, step = glu_F > 0 ? rt / 2 : rt;
        for (int r = r0; r < r1; r += step)
            if (!task(m, r, min(step, r1 - r), glu_F)) return;
    }
};

// ------------------------------------------------------------------------------------------------
// Consumers: MG_GROUPS groups of MG_GW warps; task t belongs to group t % MG_GROUPS.  Inside a group a warp takes
// four rows of the task (or, for rows longer than 4096 values, a range of blocks of the four rows its warps share).
// ------------------------------------------------------------------------------------------------
struct Consumer {
    uint8_t* ring;
    uint64_t* full;
    uint64_t* empty;
    int stage_bytes, n_stages;
    unsigned t;                    // tasks passed (all groups count every task)
    Ctl ctl;
    const int8_t* xq;              // shared: int8 activations of the current matrix
    const float* xd;               // shared: scale per 256 activations
    const int* bsum;               // shared: sum of the int8 activations per 16
    float* part;                   // shared: [MG_CWARPS][4] partial sums of rows shared by several warps
    int warp, lane;
    bool prof;                     // diagnostics: time spent waiting for stages
    unsigned long long wait_ns;
};

// The stage of the task the caller's group takes next.  Once a wait anywhere has given up, nothing waits any more:
// every warp still walks the whole schedule (so that the barriers inside it stay matched) over whatever the stages
// hold, and the step's result is discarded by the host, which sees the status word.
__device__ __forceinline__ const uint8_t* cons_acquire(Consumer& c) {
    const int s = c.t % c.n_stages;
    if (c.prof) {
        const unsigned long long t0 = global_timer_ns();
        if (!*c.ctl.dead) mg_mbar_wait(&c.full[s], (c.t / c.n_stages) & 1, c.ctl, 200);
        c.wait_ns += global_timer_ns() - t0;
    } else if (!*c.ctl.dead) {
        mg_mbar_wait(&c.full[s], (c.t / c.n_stages) & 1, c.ctl, 200);
    }
    return c.ring + (long)s * c.stage_bytes;
}
__device__ __forceinline__ void cons_release(Consumer& c) {
    __syncwarp();
    if (c.lane == 0) tc::mbar_arrive(&c.empty[c.t % c.n_stages]);
}

// One 64-value unit of the activation vector as a lane holds it while it streams rows.
//   Q4_K unit = (block b, pair c): sub-blocks 2c and 2c + 1; x[0..7] go with the low nibbles, x[8..15] with the high.
//   Q6_K unit = (block b, half n, l-range 16 h): four groups of 16 values 32 apart; x[4k..4k+3] go with group k.
struct ActSet {
    int x[16];
    int bs[4];                     // sums of the int8 activations (Q4_K: per sub-block in [0], [1]; Q6_K: per group)
    float xd;                      // activation scale of the unit's 256-block; 0 when the lane has no unit in this set
    int o0, o1, o2, o3;            // byte offsets inside a row (Q4_K: header, quants; Q6_K: ql, qh, scales, super-scale)
    unsigned sel;                  // Q4_K: 16 * (c & 1) | (c >= 2) << 8;  Q6_K: 8 * h
};

template <bool Q6>
__device__ __forceinline__ void hoist_set(ActSet& S, const Consumer& c, int b, int sub, bool valid) {
    const int* xw = reinterpret_cast<const int*>(c.xq);
    if (!valid) { b = 0; sub = 0; }        // a lane without a unit reads block 0 (finite data) and scales it by zero
    if (!Q6) {
        const int base = b * 256 + 64 * sub;
#pragma unroll
        for (int i = 0; i < 16; ++i) S.x[i] = valid ? xw[(base >> 2) + i] : 0;
        S.bs[0] = valid ? c.bsum[(base >> 4)] + c.bsum[(base >> 4) + 1] : 0;
        S.bs[1] = valid ? c.bsum[(base >> 4) + 2] + c.bsum[(base >> 4) + 3] : 0;
        S.bs[2] = S.bs[3] = 0;
        S.o0 = b * 144; S.o1 = b * 144 + 16 + 32 * sub; S.o2 = S.o3 = 0;
        S.sel = 16u * (sub & 1) | ((sub >= 2) ? 256u : 0u);
    } else {
        const int n = sub >> 1, h = sub & 1;
        const int base = b * 256 + 128 * n + 16 * h;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
#pragma unroll
            for (int i = 0; i < 4; ++i) S.x[4 * k + i] = valid ? xw[((base + 32 * k) >> 2) + i] : 0;
            S.bs[k] = valid ? c.bsum[(base + 32 * k) >> 4] : 0;
        }
        S.o0 = b * 128 + 64 * n + 16 * h; S.o1 = b * 64 + 32 * n + 16 * h; S.o2 = b * 16 + 8 * n; S.o3 = b * 2;
        S.sel = 8u * h;
    }
    S.xd = valid ? c.xd[b] : 0.f;
}

// Pointers to a local row's data inside the stage.
struct RowPtr { const uint8_t* p0; const uint8_t* p1; const uint8_t* p2; const uint8_t* p3; };

// Dot product of one unit of a row with the lane's activations (scaled by the activation scale).
template <bool Q6>
__device__ __forceinline__ float unit_dot(const ActSet& S, const RowPtr& r) {
    if (!Q6) {
        const uint4 hdr = *reinterpret_cast<const uint4*>(r.p0 + S.o0);
        const uint4 qa = *reinterpret_cast<const uint4*>(r.p0 + S.o1);
        const uint4 qb = *reinterpret_cast<const uint4*>(r.p0 + S.o1 + 16);
        const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            s0 = dp4a_us(q[i] & 0x0F0F0F0Fu, S.x[i], s0);
            s1 = dp4a_us(q[i] & 0xF0F0F0F0u, S.x[8 + i], s1);          // 16 x the sum over the high nibbles
        }
        // 6-bit scales / minimums of sub-blocks 2c, 2c + 1 as packed byte pairs, both encodings, then select
        const unsigned sh = S.sel & 0xFFu;
        const uint32_t Y = hdr.y >> sh, Z = hdr.z >> sh, W = hdr.w >> sh;
        const uint32_t p_lo = Y & 0x3F3Fu, q_lo = Z & 0x3F3Fu;
        const uint32_t p_hi = (W & 0x0F0Fu) | ((Y >> 2) & 0x3030u), q_hi = ((W >> 4) & 0x0F0Fu) | ((Z >> 2) & 0x3030u);
        const uint32_t P = (S.sel & 256u) ? p_hi : p_lo, Q = (S.sel & 256u) ? q_hi : q_lo;
        const int iS = (int)((P & 0xFFu) << 4) * s0 + (int)(P >> 8) * s1;             // 16 x sum of scale x dot
        const int iM = (int)(Q & 0xFFu) * S.bs[0] + (int)(Q >> 8) * S.bs[1];
        const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
        return S.xd * (dd.x * 0.0625f * (float)iS - dd.y * (float)iM);
    } else {
        const uint4 A = *reinterpret_cast<const uint4*>(r.p0 + S.o0);
        const uint4 B = *reinterpret_cast<const uint4*>(r.p0 + S.o0 + 32);
        const uint4 H = *reinterpret_cast<const uint4*>(r.p1 + S.o1);
        const uint2 sc8 = *reinterpret_cast<const uint2*>(r.p2 + S.o2);
        const float d = __half2float(*reinterpret_cast<const __half*>(r.p3 + S.o3));
        const uint32_t a[4] = {A.x, A.y, A.z, A.w}, b[4] = {B.x, B.y, B.z, B.w}, h[4] = {H.x, H.y, H.z, H.w};
        int t0 = 0, t1 = 0, t2 = 0, t3 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t q0 = (a[i] & 0x0F0F0F0Fu) | ((h[i] & 0x03030303u) << 4);
            const uint32_t q1 = (b[i] & 0x0F0F0F0Fu) | ((h[i] & 0x0C0C0C0Cu) << 2);
            const uint32_t q2 = ((a[i] >> 4) & 0x0F0F0F0Fu) | (h[i] & 0x30303030u);
            const uint32_t q3 = ((b[i] >> 4) & 0x0F0F0F0Fu) | ((h[i] >> 2) & 0x30303030u);
            t0 = dp4a_us(q0, S.x[i], t0);
            t1 = dp4a_us(q1, S.x[4 + i], t1);
            t2 = dp4a_us(q2, S.x[8 + i], t2);
            t3 = dp4a_us(q3, S.x[12 + i], t3);
        }
        // the stored value is q - 32: the offset goes through the activation sums
        const int c0 = (int)(int8_t)(sc8.x >> S.sel), c1 = (int)(int8_t)(sc8.x >> (S.sel + 16u));
        const int c2 = (int)(int8_t)(sc8.y >> S.sel), c3 = (int)(int8_t)(sc8.y >> (S.sel + 16u));
        const int iS = c0 * (t0 - 32 * S.bs[0]) + c1 * (t1 - 32 * S.bs[1]) + c2 * (t2 - 32 * S.bs[2]) + c3 * (t3 - 32 * S.bs[3]);
        return S.xd * d * (float)iS;
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

// Up to four finished rows of a warp: row[i] < 0 = nothing.  All lanes hold all four values.
__device__ __forceinline__ void emit_rows(const Emit& e, const int (&row)[4], const float (&v)[4], int lane) {
    if (e.mode == 1) {
        const int i = lane >> 3, r = lane & 7;                       // lane = (row slot, rank)
        const float val = i == 0 ? v[0] : i == 1 ? v[1] : i == 2 ? v[2] : v[3];
        const int rw = i == 0 ? row[0] : i == 1 ? row[1] : i == 2 ? row[2] : row[3];
        if (r < e.ranks && rw >= 0) st_word(e.peers[r] + e.off + rw, val, e.tag);
    } else if (lane < 4) {
        const float val = lane == 0 ? v[0] : lane == 1 ? v[1] : lane == 2 ? v[2] : v[3];
        const int rw = lane == 0 ? row[0] : lane == 1 ? row[1] : lane == 2 ? row[2] : row[3];
        if (rw >= 0) {
            if (e.mode == 0) st_word(e.local + rw, e.bias ? val + e.bias[rw] : val, e.tag);
            else if (e.mode == 2) st_word(e.local + rw, bf2f(f2bf(val)), e.tag);
            else e.logits[rw] = val;
        }
    }
}

// Rows [r0, r1) of matrix m against the activations in shared memory.  With glu_F > 0, rows r and r + glu_F are a
// gate / up pair and the emitted value is act(gate, up) for row r.  One copy of this code per block type.
template <bool Q6>
__device__ __noinline__ void run_rows(Consumer& c, const MegaMat& m, int r0, int r1, int glu_F, int act, const Emit& e) {
    if (r0 >= r1) return;
    const int nb = m.K >> 8, ks = ks_of(m.K), rowsets = MG_GW / ks, rt = rowsets * 4;
    const int wg = c.warp & (MG_GW - 1), grp = c.warp / MG_GW, part = wg % ks, rowset = wg / ks;
    const int bs = (nb * part) / ks, be = (nb * (part + 1)) / ks;
    const int units = (be - bs) * 4;                                 // <= 64
    // lanes take unit `lane` (set A) and `32 + lane` (set B) of every row; what is left of a row (fewer than 32
    // units) is packed: 4, 2 or 1 rows side by side in one pass, lane = (row within the pass, unit)
    const int full = units >> 5, rem = units & 31;
    const int pack = rem == 0 ? 0 : rem <= 8 ? 4 : rem <= 16 ? 2 : 1, lp = pack ? 32 / pack : 32;
    const int rsub = c.lane / lp, ru = c.lane % lp;
    ActSet SA, SB, SR;
    hoist_set<Q6>(SA, c, bs + (c.lane >> 2), c.lane & 3, full >= 1);
    hoist_set<Q6>(SB, c, bs + 8 + (c.lane >> 2), c.lane & 3, full >= 2);
    hoist_set<Q6>(SR, c, bs + 8 * full + (ru >> 2), ru & 3, pack > 0 && ru < rem);
    const int step = glu_F > 0 ? rt / 2 : rt;
    for (int r = r0; r < r1; r += step, ++c.t) {
        if ((int)(c.t % MG_GROUPS) != grp) continue;
        const int n = min(step, r1 - r);
        const uint8_t* st = cons_acquire(c);
        const TaskGeo g = task_geo(m, r, n, glu_F);
        // the four local rows of this warp: plain: rowset * 4 + i; gated: pairs rowset * 2 + {0, 1}, gate rows then up rows
        auto local_row = [&](int i) { return glu_F > 0 ? (i >> 1) * n + rowset * 2 + (i & 1) : rowset * 4 + i; };
        auto row_ptr = [&](int lr) {
            RowPtr rp;
            if (!Q6) {
                rp.p0 = st + (long)lr * nb * 144; rp.p1 = rp.p2 = rp.p3 = nullptr;
            } else {
                rp.p0 = st + (long)lr * nb * 128;
                rp.p1 = st + g.b0 + (long)lr * nb * 64;
                rp.p2 = st + g.b0 + g.b1 + (long)lr * nb * 16;
                const int run = (glu_F > 0 && lr >= n) ? 1 : 0;
                rp.p3 = st + g.b0 + g.b1 + g.b2 + (run ? g.d_bytes[0] : 0u) + g.lead[run] + (long)(lr - run * n) * nb * 2;
            }
            return rp;
        };
        const int lim = glu_F > 0 ? 2 * n : n;                       // local rows present in the stage
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (full >= 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (local_row(i) < lim) acc[i] += unit_dot<Q6>(SA, row_ptr(local_row(i)));
        }
        if (full >= 2) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (local_row(i) < lim) acc[i] += unit_dot<Q6>(SB, row_ptr(local_row(i)));
        }
        if (pack > 0) {
            for (int j = 0; j < 4; j += pack) {
                const int i = j + rsub, lr = local_row(i);
                const float v = (i < 4 && lr < lim) ? unit_dot<Q6>(SR, row_ptr(lr)) : 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] += (k == i) ? v : 0.f;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = warp_sum(acc[i]);
        cons_release(c);
        if (ks > 1) {
            // the warps that share these rows add their parts through shared memory (double-buffered by task parity)
            float* pp = c.part + ((c.t / MG_GROUPS) & 1) * MG_CWARPS * 4;
            if (c.lane < 4) pp[c.warp * 4 + c.lane] = c.lane == 0 ? acc[0] : c.lane == 1 ? acc[1] : c.lane == 2 ? acc[2] : acc[3];
            group_sync(2 + grp);
            if (part == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[i] = 0.f;
                    for (int k = 0; k < ks; ++k) acc[i] += pp[(c.warp + k) * 4 + i];
                }
            }
        }
        if (part != 0) continue;
        int rows[4];
        float vals[4];
        if (glu_F > 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                rows[i] = rowset * 2 + i < n ? r + rowset * 2 + i : -1;
                vals[i] = act_glu(act, acc[i], acc[2 + i]);
            }
            rows[2] = rows[3] = -1; vals[2] = vals[3] = 0.f;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) { rows[i] = rowset * 4 + i < n ? r + rowset * 4 + i : -1; vals[i] = acc[i]; }
        }
        emit_rows(e, rows, vals, c.lane);
    }
}

__device__ __forceinline__ void run_segment(Consumer& c, const MegaMat& m, int r0, int r1, int glu_F, int act, const Emit& e) {
    if (m.type == TSB_Q4_K) run_rows<false>(c, m, r0, r1, glu_F, act, e);
    else run_rows<true>(c, m, r0, r1, glu_F, act, e);
}

// 256 values (8 consecutive per lane) -> one int8 block: scale amax / 127, sums of the int8 values per 16.
__device__ __forceinline__ void quant_block(const float (&v)[8], int8_t* xq, float* xd, int* bsum, int block, int lane) {
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
    *reinterpret_cast<uint2*>(xq + block * 256 + lane * 8) = pk;
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
                                               float* qs, float* red, int item, int warp, int lane) {
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
    const float2* xw = a.xbuf[a.rank] + a.off_qkv;
    // ---- per-head RMSNorm + RoPE of the G query heads (and of the new K row; V as it is) ----
    for (int job = warp; job < G + 2; job += MG_CWARPS) {
        if (job >= G && !owner) continue;
        const int kind = job < G ? 0 : job - G + 1;          // 0 q, 1 k, 2 v
        const long row = kind == 0 ? (long)(kvh * G + job) * DH : kind == 1 ? (long)(a.Hq + kvh) * DH : (long)(a.Hq + a.Hkv + kvh) * DH;
        float v[NJ], ss = 0.f;
        wait_words<NJ>([&](int j) { return xw + row + lane + 32 * j; }, v, tag_qkv, ctl, 100 + PH_QKV);
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
                        float sn, cs;
                        sincosf((float)pos * a.rope_freq[pair], &sn, &cs);
                        cs *= a.rope_mscale; sn *= a.rope_mscale;
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
                        float sn, cs;
                        sincosf((float)pos * a.rope_freq[e >> 1], &sn, &cs);
                        cs *= a.rope_mscale; sn *= a.rope_mscale;
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
    // ---- split-KV attention: lane = (position p of a chunk of 8, quarter c of the head dims) ----
    float m[G], l[G], acc[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[g][d] = 0.f;
    }
    const int p = lane >> 2, cq = lane & 3;
    for (int base = s0 + warp * 8; base < s1; base += MG_CWARPS * 8) {
        const int j = base + p;
        const bool valid = j < s1;
        long slot = 0;
        if (valid) slot = (long)a.block_table[j / a.page_size] * a.page_size + j % a.page_size;
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
    // ---- merge the warps, publish the partial ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) { red_ml[(warp * G + g) * 2] = m[g]; red_ml[(warp * G + g) * 2 + 1] = l[g]; }
#pragma unroll
        for (int d = 0; d < DPL; ++d) red_o[(warp * G + g) * DH + lane * DPL + d] = acc[g][d];
    }
    cons_sync();
    float2* out = a.xbuf[a.rank] + a.off_part;
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
}

template <int DH, int G>
__global__ void __launch_bounds__(MG_THREADS, 1) mega_decode_kernel(const MegaArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t full[MG_MAX_STAGES], empty[MG_MAX_STAGES];
    __shared__ int dead_flag;
    __shared__ float red32[32];
    __shared__ float part_s[2 * MG_CWARPS * 4];
    __shared__ float2* peers_s[MG_MAX_RANKS];
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
            Producer pr{smem + a.off_ring, full, empty, a.stage_bytes, a.n_stages, 0u, ctl};
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
                cta_range(a.ffn, lo, hi);
                pr.segment(L.gate_up, lo, hi, a.ffn);
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
    Consumer c{smem + a.off_ring, full, empty, a.stage_bytes, a.n_stages, 0u, ctl, xq, xd, bsum, part_s, warp, lane, a.prof != nullptr, 0ull};
    const unsigned step = *reinterpret_cast<volatile unsigned*>(a.step);
    const unsigned tag0 = step * (unsigned)((a.n_layers + 1) * PH_STRIDE) + 1u;
    float2* mine = a.xbuf[a.rank];

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
    int dbg_layer = 0;
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
            if (gather) {
                for (int r = 0; r < R; ++r) {                              // parts are added in rank order
                    float v[16];
                    wait_pairs<8>([&](int u) -> const float2* {
                        const int b = warp + MG_CWARPS * (u >> 2);
                        return b < nblk ? mine + off + (long)r * D + b * 256 + lane * 8 + 2 * (u & 3) : nullptr;
                    }, v, tag, ctl, code);
#pragma unroll
                    for (int u = 0; u < 16; ++u) hv[u >> 3][u & 7] += v[u];
                }
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
            if (!(fabsf(ss) < 1e30f)) atomicCAS(a.status + 1, 0, code * 1000 + dbg_layer);
            const float rs = rsqrtf(ss / (float)D + a.eps);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int b = warp + MG_CWARPS * j;
                if (b < nblk) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = hv[j][i] * rs * wv[j][i];
                    quant_block(v, xq, xd, bsum, b, lane);
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
                quant_block(v, xq, xd, bsum, b, lane);
            }
        }
        cons_sync();
    };
    // n tagged values at `off` -> int8 activation buffers (a warp per 256-value block, two blocks of loads in flight)
    auto gather_quant = [&](long off, int n, unsigned tag, int code) {
        cons_sync();                                // every warp has hoisted what it needed from the previous contents
        const int nblk = n >> 8;
        for (int b0 = warp; b0 < nblk; b0 += 2 * MG_CWARPS) {
            float v[16];
            wait_pairs<8>([&](int u) -> const float2* {
                const int b = b0 + MG_CWARPS * (u >> 2);
                return b < nblk ? mine + off + b * 256 + lane * 8 + 2 * (u & 3) : nullptr;
            }, v, tag, ctl, code);
            float v0[8], v1[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { v0[i] = v[i]; v1[i] = v[8 + i]; }
#pragma unroll
            for (int i = 0; i < 16; ++i) if (!(fabsf(v[i]) < 1e30f)) atomicCAS(a.status + 1, 0, code * 1000 + dbg_layer + 500);
            quant_block(v0, xq, xd, bsum, b0, lane);
            if (b0 + MG_CWARPS < nblk) quant_block(v1, xq, xd, bsum, b0 + MG_CWARPS, lane);
        }
        cons_sync();
    };

    unsigned long long pt[16], plast = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) pt[i] = 0;
    const bool prof = a.prof != nullptr;
    if (prof) plast = global_timer_ns();
    // time since the previous mark goes to slot i (thread 0's view of its CTA)
#define MG_MARK(i) do { if (prof) { const unsigned long long now_ = global_timer_ns(); pt[i] += now_ - plast; plast = now_; } } while (0)
    for (int l = 0; l < a.n_layers; ++l) {
        const MegaLayer& L = a.layers[l];
        const unsigned tg = tag0 + (unsigned)l * PH_STRIDE;
        int lo, hi;
        dbg_layer = l;
        // ---------------- QKV ----------------
        gather_norm(l > 0, a.off_dwn, tg - PH_STRIDE + PH_DWN, 100 + PH_DWN, L.attn_norm);
        MG_MARK(1);
        {
            const int tot = L.qkv[0].N + L.qkv[1].N + L.qkv[2].N;
            cta_range(tot, lo, hi);
            int o = 0;
            for (int i = 0; i < 3; ++i) {
                const int n = L.qkv[i].N;
                if (n > 0) {
                    const Emit e{0, mine + a.off_qkv + o, L.qkv_bias ? L.qkv_bias + o : nullptr, nullptr, nullptr, 0, R, tg + PH_QKV};
                    run_segment(c, L.qkv[i], max(lo, o) - o, min(hi, o + n) - o, 0, 0, e);
                }
                o += n;
            }
        }
        MG_MARK(2);
        // ---------------- attention: splits, then the merge per head ----------------
        if ((int)blockIdx.x < a.Hkv * a.splits)
            attention_item<DH, G>(a, L, ctl, tg + PH_QKV, tg + PH_ATT, qs, red, blockIdx.x, warp, lane);
        MG_MARK(3);
        {
            const int hd = (int)gridDim.x - 1 - (int)blockIdx.x;        // heads are merged by the CTAs at the far end of the grid
            if (hd < a.Hq && warp < DH / 32) {
                // one warp per 32 dims; lanes fetch the (max, sum) of two splits each, the warp reduces them; the
                // partial outputs come eight splits at a time
                const int S = a.splits, d = warp * 32 + lane;
                const float2* pp = mine + a.off_part + (long)hd * S * (DH + 2);
                float ml[4];
                wait_words<4>([&](int u) -> const float2* {
                    const int sp = lane + 32 * (u >> 1);
                    return sp < S ? pp + (long)sp * (DH + 2) + DH + (u & 1) : nullptr;
                }, ml, tg + PH_ATT, ctl, 100 + PH_ATT);
                const float m0 = lane < S ? ml[0] : -INFINITY, m1 = lane + 32 < S ? ml[2] : -INFINITY;
                const float mm = warp_max(fmaxf(m0, m1));
                const float c0 = (m0 == -INFINITY) ? 0.f : __expf(m0 - mm), c1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - mm);
                const float ll = warp_sum((lane < S ? ml[1] : 0.f) * c0 + (lane + 32 < S ? ml[3] : 0.f) * c1);
                float o = 0.f;
                for (int s0 = 0; s0 < S; s0 += 8) {
                    float pv[8];
                    wait_words<8>([&](int u) -> const float2* { return s0 + u < S ? pp + (long)(s0 + u) * (DH + 2) + d : nullptr; },
                                  pv, tg + PH_ATT, ctl, 100 + PH_ATT);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int sp = s0 + u;
                        const float cw = __shfl_sync(0xffffffffu, sp < 32 ? c0 : c1, sp & 31);
                        if (sp < S) o += pv[u] * cw;
                    }
                }
                st_word(mine + a.off_attn + (long)hd * DH + d, bf2f(f2bf(ll > 0.f ? o / ll : 0.f)), tg + PH_CMB);
            }
        }
        MG_MARK(4);
        // ---------------- o_proj (row-parallel: partial sums to every rank) ----------------
        gather_quant(a.off_attn, nq, tg + PH_CMB, 100 + PH_CMB);
        MG_MARK(5);
        cta_range(L.wo.N, lo, hi);
        {
            const Emit e{1, nullptr, nullptr, nullptr, peers_s, a.off_opr + (long)a.rank * D, R, tg + PH_OPR};
            run_segment(c, L.wo, lo, hi, 0, 0, e);
        }
        MG_MARK(6);
        // ---------------- gate / up ----------------
        gather_norm(true, a.off_opr, tg + PH_OPR, 100 + PH_OPR, L.ffn_norm);
        MG_MARK(8);
        cta_range(a.ffn, lo, hi);
        {
            const Emit e{2, mine + a.off_act, nullptr, nullptr, nullptr, 0, R, tg + PH_GUP};
            run_segment(c, L.gate_up, lo, hi, a.ffn, a.act, e);
        }
        MG_MARK(9);
        // ---------------- down (row-parallel) ----------------
        gather_quant(a.off_act, a.ffn, tg + PH_GUP, 100 + PH_GUP);
        MG_MARK(10);
        cta_range(L.down.N, lo, hi);
        {
            const Emit e{1, nullptr, nullptr, nullptr, peers_s, a.off_dwn + (long)a.rank * D, R, tg + PH_DWN};
            run_segment(c, L.down, lo, hi, 0, 0, e);
        }
        MG_MARK(11);
    }
    // ---------------- output norm + lm_head ----------------
    {
        int lo, hi;
        gather_norm(true, a.off_dwn, tag0 + (unsigned)(a.n_layers - 1) * PH_STRIDE + PH_DWN, 100 + PH_DWN, a.out_norm);
        cta_range(a.lm_head.N, lo, hi);
        MG_MARK(12);
        {
            const Emit e{3, nullptr, nullptr, a.logits, nullptr, 0, R, 0u};
            run_segment(c, a.lm_head, lo, hi, 0, 0, e);
        }
        MG_MARK(13);
    }
    cons_sync();
    if (prof && tid == 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) a.prof[(long)blockIdx.x * 16 + i] = i == 14 ? c.wait_ns : i == 15 ? (unsigned long long)c.t : pt[i];
    }
#undef MG_MARK
    if (blockIdx.x == 0 && tid == 0) *a.step = step + 1u;
}

#endif  // __CUDACC__

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
static int mg_task_bytes(int type, int K) {
    const int nb = K >> 8, rt = (MG_GW / ks_of(K)) * 4;
    if (type == TSB_Q4_K) return rt * nb * 144;
    return rt * nb * 208 + 2 * (((rt / 2 * nb * 2 + 15) & ~15) + 16);      // two runs of super-scales (gate rows, up rows)
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
    int kmax = a.hidden, task = 0, min_rows = a.hidden;
    auto mat = [&](const MegaMat& m, const char* what) -> bool {
        if (!mg_mat_ok(m)) { tsb_set_error("mega_plan: %s has type %d, K %d (needs Q4_K / Q6_K, K a multiple of 256)", what, m.type, m.K); return false; }
        kmax = m.K > kmax ? m.K : kmax;
        const int tb = mg_task_bytes(m.type, m.K);
        task = tb > task ? tb : task;
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
        if (!mat(L.wo, "attn_output") || !mat(L.gate_up, "ffn_gate_up") || !mat(L.down, "ffn_down")) return TSB_ERR_UNSUPPORTED;
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
    a.off_bsum_words = kmax / 256;                          // scales per 256 first, then the sums per 16
    a.off_xds = take((kmax / 256 + kmax / 16) * 4);
    a.off_qs = take(G * a.Dh * 4);
    a.off_red = take((MG_CWARPS * G * a.Dh + MG_CWARPS * G * 2 + MG_CWARPS * a.Dh) * 4);
    a.stage_bytes = (task + 127) & ~127;
    a.off_ring = take(0);
    const int avail = 227 * 1024 - 2048 - off;            // static shared memory of the kernel stays under 2 KB
    int ns = avail / a.stage_bytes;
    if (ns > MG_MAX_STAGES) ns = MG_MAX_STAGES;
    TSB_CHECK_ARG(ns >= 2, "mega_plan: a stage of %d bytes leaves room for %d ring stages", a.stage_bytes, ns);
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
