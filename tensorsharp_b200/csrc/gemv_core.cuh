// Device-side building blocks of the weight-streaming GEMV kernels: the GLU activations, the
// per-type "load one unit of a row" / "multiply it with the int8 activations" pairs, and the
// two-deep pipelined row loop that joins them (dot_row).  Included by every kernel file that
// streams GGUF block-quantised weights against a handful of activation rows.
#pragma once
#include "quant_blocks.cuh"
#include "tp_fused.cuh"

enum { ACT_NONE = 0, ACT_SWIGLU = 1, ACT_GEGLU_TANH = 2, ACT_GEGLU_ERF = 3, ACT_SWIGLU_OAI = 4,
       ACT_RELU2 = 5, ACT_SILU = 6 };

__device__ __forceinline__ float act_glu(int act, float g, float u) {
    switch (act) {
    case ACT_SWIGLU: return g / (1.f + __expf(-g)) * u;
    case ACT_GEGLU_TANH: {
        const float c = 0.7978845608028654f;
        float t = tanhf(c * (g + 0.044715f * g * g * g));
        return 0.5f * g * (1.f + t) * u;
    }
    case ACT_GEGLU_ERF: return 0.5f * g * (1.f + erff(g * 0.7071067811865476f)) * u;
    case ACT_SWIGLU_OAI: {
        float x = fminf(g, 7.f), y = fminf(fmaxf(u, -7.f), 7.f);
        return x / (1.f + __expf(-1.702f * x)) * (y + 1.f);
    }
    default: return g * u;
    }
}

struct GemvArgs {
    QW w;
    const int8_t* xq;      // [Mx, K] int8
    const float2* xds;     // [Mx, K/32] (scale, sum of x)
    const bf16* xb;        // [Mx, K] bf16 (used by float-weight types)
    void* out;             // [P or M, N_out]
    const float* bias;     // [E, N] or null
    const void* residual;  // same shape/dtype as out, or null
    const int* ids;        // [P] expert per problem, or null
    const float* row_scale;  // [P] multiply the result (before residual) or null
    int M;                 // activation rows handled per problem (1 when ids != null)
    int x_div;             // activation row of problem p is p / x_div
    int out_f32;           // 1: float output, 0: bf16
    int act;               // GLU activation; rows [0,N/2) are gate, [N/2,N) are up
    int n_out;             // N, or N/2 with GLU
    const TpPush* push;    // tensor-parallel exchange: store the f32 result into every rank's mailbox
                           // instead of `out` (see tp_fused.cuh); null for an ordinary GEMV
};

// Each quantised type is split into a weight *load* (global, streaming, independent of the
// activations) and a *compute* step, so that a lane can have the loads of two units in
// flight before it touches either, and so that the first loads can be issued before the
// kernel waits for its predecessor (weights never change between kernels).

__device__ __forceinline__ void k4_scales(const uint4& hdr, int c, int& sc0, int& sc1, int& mn0, int& mn1) {
    if (c < 2) {
        const int s0 = 16 * c;
        sc0 = (hdr.y >> s0) & 63; sc1 = (hdr.y >> (s0 + 8)) & 63;
        mn0 = (hdr.z >> s0) & 63; mn1 = (hdr.z >> (s0 + 8)) & 63;
    } else {
        const int s0 = 16 * (c - 2);
        sc0 = ((hdr.w >> s0) & 0xF) | (((hdr.y >> (s0 + 6)) & 3) << 4);
        sc1 = ((hdr.w >> (s0 + 8)) & 0xF) | (((hdr.y >> (s0 + 14)) & 3) << 4);
        mn0 = ((hdr.w >> (s0 + 4)) & 0xF) | (((hdr.z >> (s0 + 6)) & 3) << 4);
        mn1 = ((hdr.w >> (s0 + 12)) & 0xF) | (((hdr.z >> (s0 + 14)) & 3) << 4);
    }
}

struct WQ4K { uint4 hdr, qv, hv; };

template <bool Q5>
__device__ __forceinline__ void load_q45k(const QW& w, long row, int u, WQ4K& o) {
    const int nb = w.K >> 8, b = u >> 3, uu = u & 7, c = uu >> 1, h = uu & 1;
    const uint8_t* blk = w.p0 + (row * nb + b) * (Q5 ? 176 : 144);
    o.hdr = ld_stream_u4(blk);
    if (Q5) {
        o.hv = ld_stream_u4(blk + 16 + 16 * h);
        o.qv = ld_stream_u4(blk + 48 + 32 * c + 16 * h);
    } else {
        o.qv = ld_stream_u4(blk + 16 + 32 * c + 16 * h);
    }
}

template <int M, bool Q5>
__device__ __forceinline__ void comp_q45k(const QW& w, const WQ4K& t, int u, const int8_t* xq, const float2* xds,
                                          float* acc, int mv) {
    const int K = w.K, kb = K >> 5, b = u >> 3, uu = u & 7, c = uu >> 1, h = uu & 1;
    const float d = h2f_bits(t.hdr.x & 0xffff), dmin = h2f_bits(t.hdr.x >> 16);
    int sc0, sc1, mn0, mn1;
    k4_scales(t.hdr, c, sc0, sc1, mn0, mn1);
    const float ds0 = d * sc0, ds1 = d * sc1, dm0 = dmin * mn0, dm1 = dmin * mn1;
    const uint32_t q[4] = {t.qv.x, t.qv.y, t.qv.z, t.qv.w};
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        lo[i] = q[i] & 0x0F0F0F0Fu;
        hi[i] = (q[i] >> 4) & 0x0F0F0F0Fu;
    }
    if (Q5) {
        const uint32_t hq[4] = {t.hv.x, t.hv.y, t.hv.z, t.hv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo[i] |= ((hq[i] >> (2 * c)) & 0x01010101u) << 4;
            hi[i] |= ((hq[i] >> (2 * c + 1)) & 0x01010101u) << 4;
        }
    }
    const int xoff = b * 256 + 64 * c + 16 * h;
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const int mr = m < mv ? m : 0;
        const int4 xa = *reinterpret_cast<const int4*>(xq + (long)mr * K + xoff);
        const int4 xb = *reinterpret_cast<const int4*>(xq + (long)mr * K + xoff + 32);
        const int xai[4] = {xa.x, xa.y, xa.z, xa.w}, xbi[4] = {xb.x, xb.y, xb.z, xb.w};
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s0 = __dp4a((int)lo[i], xai[i], s0);
            s1 = __dp4a((int)hi[i], xbi[i], s1);
        }
        const float2 e0 = xds[(long)mr * kb + b * 8 + 2 * c], e1 = xds[(long)mr * kb + b * 8 + 2 * c + 1];
        float v = ds0 * e0.x * (float)s0 + ds1 * e1.x * (float)s1;
        if (h == 0) v -= dm0 * e0.y + dm1 * e1.y;
        acc[m] += v;
    }
}

// Q6_K planes.  Unit = (block b, half n, l-range 16*h): 64 values in four quarters of 16.
struct WQ6K { uint4 la, lb, hv; float s0, s1, s2, s3; };

__device__ __forceinline__ void load_q6k(const QW& w, long row, int u, WQ6K& o) {
    const int nb = w.K >> 8, b = u >> 2, n = (u >> 1) & 1, h = u & 1;
    const long blk = row * nb + b;
    o.la = ld_stream_u4(w.p0 + blk * 128 + 64 * n + 16 * h);
    o.lb = ld_stream_u4(w.p0 + blk * 128 + 64 * n + 32 + 16 * h);
    o.hv = ld_stream_u4(w.p1 + blk * 64 + 32 * n + 16 * h);
    const float d = __half2float(reinterpret_cast<const __half*>(w.p3)[blk]);
    const int8_t* scp = reinterpret_cast<const int8_t*>(w.p2) + blk * 16 + 8 * n + h;
    o.s0 = d * scp[0]; o.s1 = d * scp[2]; o.s2 = d * scp[4]; o.s3 = d * scp[6];
}

template <int M>
__device__ __forceinline__ void comp_q6k(const QW& w, const WQ6K& t, int u, const int8_t* xq, const float2* xds,
                                         float* acc, int mv) {
    const int K = w.K, kb = K >> 5, b = u >> 2, n = (u >> 1) & 1, h = u & 1;
    const uint32_t a[4] = {t.la.x, t.la.y, t.la.z, t.la.w}, bb[4] = {t.lb.x, t.lb.y, t.lb.z, t.lb.w};
    const uint32_t hh[4] = {t.hv.x, t.hv.y, t.hv.z, t.hv.w};
    int q0[4], q1[4], q2[4], q3[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        q0[i] = __vsub4((a[i] & 0x0F0F0F0Fu) | ((hh[i] & 0x03030303u) << 4), 0x20202020u);
        q1[i] = __vsub4((bb[i] & 0x0F0F0F0Fu) | (((hh[i] >> 2) & 0x03030303u) << 4), 0x20202020u);
        q2[i] = __vsub4(((a[i] >> 4) & 0x0F0F0F0Fu) | (((hh[i] >> 4) & 0x03030303u) << 4), 0x20202020u);
        q3[i] = __vsub4(((bb[i] >> 4) & 0x0F0F0F0Fu) | (((hh[i] >> 6) & 0x03030303u) << 4), 0x20202020u);
    }
    const int xoff = b * 256 + 128 * n + 16 * h;
    const int g0 = b * 8 + 4 * n;
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const int mr = m < mv ? m : 0;
        const int8_t* xp = xq + (long)mr * K + xoff;
        const int4 x0 = *reinterpret_cast<const int4*>(xp);
        const int4 x1 = *reinterpret_cast<const int4*>(xp + 32);
        const int4 x2 = *reinterpret_cast<const int4*>(xp + 64);
        const int4 x3 = *reinterpret_cast<const int4*>(xp + 96);
        const int a0[4] = {x0.x, x0.y, x0.z, x0.w}, a1[4] = {x1.x, x1.y, x1.z, x1.w};
        const int a2[4] = {x2.x, x2.y, x2.z, x2.w}, a3[4] = {x3.x, x3.y, x3.z, x3.w};
        int t0 = 0, t1 = 0, t2 = 0, t3 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            t0 = __dp4a(q0[i], a0[i], t0);
            t1 = __dp4a(q1[i], a1[i], t1);
            t2 = __dp4a(q2[i], a2[i], t2);
            t3 = __dp4a(q3[i], a3[i], t3);
        }
        const float2* e = xds + (long)mr * kb + g0;
        acc[m] += t.s0 * e[0].x * (float)t0 + t.s1 * e[1].x * (float)t1 + t.s2 * e[2].x * (float)t2 +
                  t.s3 * e[3].x * (float)t3;
    }
}

// Q8_0 planes.  Unit = one 32-value block (two 16-byte loads).
struct WQ80 { uint4 qa, qb; float d; };

__device__ __forceinline__ void load_q8_0(const QW& w, long row, int u, WQ80& o) {
    const int kb = w.K >> 5;
    const int8_t* wr = reinterpret_cast<const int8_t*>(w.p0) + row * w.K;
    o.qa = ld_stream_u4(wr + u * 32);
    o.qb = ld_stream_u4(wr + u * 32 + 16);
    o.d = __half2float(reinterpret_cast<const __half*>(w.p1)[row * kb + u]);
}

template <int M>
__device__ __forceinline__ void comp_q8_0(const QW& w, const WQ80& t, int u, const int8_t* xq, const float2* xds,
                                          float* acc, int mv) {
    const int K = w.K, kb = K >> 5;
    const int q[8] = {(int)t.qa.x, (int)t.qa.y, (int)t.qa.z, (int)t.qa.w, (int)t.qb.x, (int)t.qb.y, (int)t.qb.z, (int)t.qb.w};
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const int mr = m < mv ? m : 0;
        const int4 x0 = *reinterpret_cast<const int4*>(xq + (long)mr * K + u * 32);
        const int4 x1 = *reinterpret_cast<const int4*>(xq + (long)mr * K + u * 32 + 16);
        const int xi[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = __dp4a(q[i], xi[i], s);
        acc[m] += t.d * xds[(long)mr * kb + u].x * (float)s;
    }
}

// Four 4-bit MXFP4 codes (one per byte, low nibble) -> four int8 values (2 x e2m1 value).
__device__ __forceinline__ int mxfp4_lut4(uint32_t idx) {
    const uint32_t m = idx & 0x07070707u;
    const uint32_t t = m | (m >> 4);
    const uint32_t sel = (t & 0xFFu) | ((t >> 8) & 0xFF00u);
    const uint32_t mag = __byte_perm(0x03020100u, 0x0C080604u, sel);
    const uint32_t neg = ((idx >> 3) & 0x01010101u) * 0xFFu;
    return (int)__vsub4(mag ^ neg, neg);
}

// Eight MXFP4 codes of one 32-bit word (byte i = code of element i in the low nibble, of element i + 16 in the
// high nibble) -> `lo`: the four low-nibble values, `hi`: the four high-nibble values, as int8 (2 x e2m1 value).
// Byte-permute does all of it: the masked word itself is the selector into the magnitude table (and into the
// table of negated magnitudes), the sign bits become byte masks through the permute's sign-replicate mode, and
// two more permutes separate the low- from the high-nibble results.  13 instructions for 8 values, no
// per-byte arithmetic (the table-per-nibble form with a per-byte subtract took about 30).
// prmt.b32 in its default mode: selector nibble n picks byte (n & 7) of {a, b}; with bit 3 set the result byte is
// that byte's sign bit replicated (0x00 / 0xFF).  Written as PTX because the sign-replicate bit is part of the
// instruction, not of the 3-bit selector that the byte-permute intrinsic documents.
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ void mxfp4_decode8(uint32_t w, int& lo, int& hi) {
    const uint32_t s = w & 0x77777777u, s2 = s >> 16, w4 = w << 4;
    const uint32_t p1 = prmt_b32(0x03020100u, 0x0C080604u, s), p2 = prmt_b32(0x03020100u, 0x0C080604u, s2);
    const uint32_t n1 = prmt_b32(0xFDFEFF00u, 0xF4F8FAFCu, s), n2 = prmt_b32(0xFDFEFF00u, 0xF4F8FAFCu, s2);
    const uint32_t m1 = prmt_b32(w4, w, 0xD9C8u), m2 = prmt_b32(w4, w, 0xFBEAu);         // 0xFF where the code's sign bit is set
    const uint32_t v1 = (p1 & ~m1) | (n1 & m1), v2 = (p2 & ~m2) | (n2 & m2);             // [lo0, hi0, lo1, hi1], [lo2, hi2, lo3, hi3]
    lo = (int)prmt_b32(v1, v2, 0x6420u);
    hi = (int)prmt_b32(v1, v2, 0x7531u);
}

// MXFP4 / Q4_0 planes.  Unit = one 32-value block (one 16-byte load).
struct WQ432 { uint4 qv; float d; };

template <bool MX>
__device__ __forceinline__ void load_q4_32(const QW& w, long row, int u, WQ432& o) {
    const int kb = w.K >> 5;
    o.qv = ld_stream_u4(w.p0 + row * (w.K >> 1) + u * 16);
    if (MX) o.d = e8m0_half_scale(w.p1[row * kb + u]);
    else o.d = __half2float(reinterpret_cast<const __half*>(w.p1)[row * kb + u]);
}

template <int M, bool MX>
__device__ __forceinline__ void comp_q4_32(const QW& w, const WQ432& t, int u, const int8_t* xq, const float2* xds,
                                           float* acc, int mv) {
    const int K = w.K, kb = K >> 5;
    const uint32_t q[4] = {t.qv.x, t.qv.y, t.qv.z, t.qv.w};
    int lo[4], hi[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (MX) {
            mxfp4_decode8(q[i], lo[i], hi[i]);
        } else {
            lo[i] = (int)__vsub4(q[i] & 0x0F0F0F0Fu, 0x08080808u);
            hi[i] = (int)__vsub4((q[i] >> 4) & 0x0F0F0F0Fu, 0x08080808u);
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const int mr = m < mv ? m : 0;
        const int4 x0 = *reinterpret_cast<const int4*>(xq + (long)mr * K + u * 32);
        const int4 x1 = *reinterpret_cast<const int4*>(xq + (long)mr * K + u * 32 + 16);
        const int xl[4] = {x0.x, x0.y, x0.z, x0.w}, xh[4] = {x1.x, x1.y, x1.z, x1.w};
        int s = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s = __dp4a(lo[i], xl[i], s);
            s = __dp4a(hi[i], xh[i], s);
        }
        acc[m] += t.d * xds[(long)mr * kb + u].x * (float)s;
    }
}

// Generic two-deep software pipeline over the units of one row; `pre()` sits between the first
// load and the first use of the activations.
#define TSB_ROW_LOOP(WT, LOAD, COMP, UNITS)                                        \
    {                                                                             \
        const int units = (UNITS), step = 32 * parts;                             \
        WT cur, nxt;                                                              \
        int u = lane + 32 * part;                                                 \
        if (u < units) LOAD(w, row, u, cur);                                      \
        pre();                                                                    \
        for (; u < units; u += step) {                                            \
            const bool more = u + step < units;                                   \
            if (more) LOAD(w, row, u + step, nxt);                                \
            COMP(w, cur, u, xq, xds, acc, mv);                                    \
            if (more) cur = nxt;                                                  \
        }                                                                         \
    }

// Float-weight types (BF16 / F16 / F32) against bf16 activations.
template <int M, class Pre>
__device__ __forceinline__ void dot_float(const QW& w, long row, int lane, const bf16* xb, float* acc, int mv,
                                          Pre pre, int part = 0, int parts = 1) {
    const int K = w.K, units = K >> 3;
    pre();
    for (int u = lane + 32 * part; u < units; u += 32 * parts) {
        float wv[8];
        dequant8(w, row, u, wv);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const int mr = m < mv ? m : 0;
            const uint4 xv = *reinterpret_cast<const uint4*>(xb + (long)mr * K + 8 * u);
            const bf16* xe = reinterpret_cast<const bf16*>(&xv);
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s += wv[i] * bf2f(xe[i]);
            acc[m] += s;
        }
    }
}

// `pre` runs exactly once per calling thread, after the first weight loads of the row have been
// issued and before any activation is read: the place for the kernel's dependency wait and for
// an in-CTA activation prologue (it may contain __syncthreads: every thread of the CTA calls
// dot_row with the same weight type).  With `parts` > 1 the row is shared by that many warps, warp
// `part` taking every parts-th group of 32 units; the caller adds the partial sums.
template <int M, class Pre>
__device__ __forceinline__ void dot_row(const QW& w, long row, int lane, const int8_t* xq, const float2* xds,
                                        const bf16* xb, float* acc, int mv, Pre pre, int part = 0, int parts = 1) {
    switch (w.type) {
    case TSB_Q4_K: TSB_ROW_LOOP(WQ4K, load_q45k<false>, (comp_q45k<M, false>), (w.K >> 8) << 3) break;
    case TSB_Q5_K: TSB_ROW_LOOP(WQ4K, load_q45k<true>, (comp_q45k<M, true>), (w.K >> 8) << 3) break;
    case TSB_Q6_K: TSB_ROW_LOOP(WQ6K, load_q6k, comp_q6k<M>, (w.K >> 8) << 2) break;
    case TSB_Q8_0: TSB_ROW_LOOP(WQ80, load_q8_0, comp_q8_0<M>, w.K >> 5) break;
    case TSB_MXFP4: TSB_ROW_LOOP(WQ432, load_q4_32<true>, (comp_q4_32<M, true>), w.K >> 5) break;
    case TSB_Q4_0: TSB_ROW_LOOP(WQ432, load_q4_32<false>, (comp_q4_32<M, false>), w.K >> 5) break;
    default: dot_float<M>(w, row, lane, xb, acc, mv, pre, part, parts); break;
    }
}


// Lane q of the calling warp stores `v`, tagged with the current exchange number, at word `index`
// of this rank's region in rank q's mailbox.
__device__ __forceinline__ void gemv_push_store(const TpPush* tp, int lane, long index, float v) {
    const unsigned epoch = *tp->epoch;
    if (lane < tp->size)
        st_word(tp->mailbox[lane] + (long)(epoch % TP_SLOTS) * tp->slot_stride + (long)tp->rank * tp->src_stride + index, v,
                epoch + 1);
}

struct PdlWait {
    bool on;
    __device__ __forceinline__ void operator()() const {
        if (on) { pdl_wait(); pdl_trigger(); }
    }
};

// Two rows of the same matrix against the same activations (the gate and up rows of a GLU pair) in
// one loop: both rows' loads are in flight together, so the pair costs one latency chain, not two.
#define TSB_ROW_LOOP2(WT, LOAD, COMP, UNITS)                                       \
    {                                                                             \
        const int units = (UNITS);                                                \
        WT ca, cb, na, nb;                                                        \
        int u = lane;                                                             \
        if (u < units) { LOAD(w, row_a, u, ca); LOAD(w, row_b, u, cb); }          \
        pre();                                                                    \
        for (; u < units; u += 32) {                                              \
            const bool more = u + 32 < units;                                     \
            if (more) { LOAD(w, row_a, u + 32, na); LOAD(w, row_b, u + 32, nb); } \
            COMP(w, ca, u, xq, xds, acc_a, mv);                                   \
            COMP(w, cb, u, xq, xds, acc_b, mv);                                   \
            if (more) { ca = na; cb = nb; }                                       \
        }                                                                         \
    }

template <int M, class Pre>
__device__ __forceinline__ void dot_row2(const QW& w, long row_a, long row_b, int lane, const int8_t* xq, const float2* xds,
                                         const bf16* xb, float* acc_a, float* acc_b, int mv, Pre pre) {
    switch (w.type) {
    case TSB_Q4_K: TSB_ROW_LOOP2(WQ4K, load_q45k<false>, (comp_q45k<M, false>), (w.K >> 8) << 3) break;
    case TSB_Q5_K: TSB_ROW_LOOP2(WQ4K, load_q45k<true>, (comp_q45k<M, true>), (w.K >> 8) << 3) break;
    case TSB_Q6_K: TSB_ROW_LOOP2(WQ6K, load_q6k, comp_q6k<M>, (w.K >> 8) << 2) break;
    case TSB_Q8_0: TSB_ROW_LOOP2(WQ80, load_q8_0, comp_q8_0<M>, w.K >> 5) break;
    case TSB_MXFP4: TSB_ROW_LOOP2(WQ432, load_q4_32<true>, (comp_q4_32<M, true>), w.K >> 5) break;
    case TSB_Q4_0: TSB_ROW_LOOP2(WQ432, load_q4_32<false>, (comp_q4_32<M, false>), w.K >> 5) break;
    default:
        dot_float<M>(w, row_a, lane, xb, acc_a, mv, pre);
        dot_float<M>(w, row_b, lane, xb, acc_b, mv, PdlWait{false});
        break;
    }
}
