// Chunked GatedDeltaNet prefill: the part that has to run chunk after chunk, as one kernel.
//
// In the chunked (WY) form of the delta rule the work inside a chunk of 64 tokens is batched matrix algebra over
// (heads x chunks) that has no dependency between chunks (the decay mask, K K^T, the unit-triangular solve, Q K^T);
// what remains sequential is carrying the state S [Dv, Dk] of each head across the chunks:
//
//     U_c   = U0_c - W_c S^T                     [64, Dv]   the chunk's value updates, corrected by the state
//     O_c   = Qd_c S^T + P_c U_c                 [64, Dv]   outputs: state term + intra-chunk term
//     S    <- gamma_c S + U_c^T Kd_c             [Dv, Dk]
//
// The reference builds a ggml graph of about forty nodes per chunk for this
// (TensorSharp.GGML.Native/ggml_ops_gated_delta_net.cpp:178-615); as tensor ops it is three small batched products per
// chunk, launch-bound.  Here a CTA owns one head and a slice of 32 value dimensions, keeps its slice of S in shared
// memory for the whole prompt, and walks the chunks: the three products run on the tensor cores (mma.sync m16n8k8,
// tf32 operands, f32 accumulation; the state itself stays f32), the operands of the next chunk stream in with cp.async
// while the current one is multiplied (each operand buffer is refilled as soon as its product is done).
#include "common.cuh"

struct GdnCarryArgs {
    const float* U0;      // [Hv, nc, 64, Dv]
    const float* W;       // [Hv, nc, 64, Dk]
    const float* Qd;      // [Hv, nc, 64, Dk]
    const float* Kd;      // [Hv, nc, 64, Dk]
    const float* P;       // [Hv, nc, 64, 64]
    const float* gamma;   // [Hv, nc]
    float* state;         // [Hv, Dv, Dk], updated in place
    float* out;           // [Hv, nc, 64, Dv]
    int Hv, nc, Dk, Dv;
};

namespace {
constexpr int GC = 64;        // tokens per chunk
constexpr int DVS = 32;       // value dimensions per CTA

__device__ __forceinline__ uint32_t tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;"); }
__device__ __forceinline__ void cp_wait2() { asm volatile("cp.async.wait_group 2;"); }

// rows x cols f32 from global (row stride gs) into shared (row stride ss), 16 bytes per copy, all 256 threads
__device__ __forceinline__ void stage(float* dst, int ss, const float* src, int gs, int rows, int cols) {
    const int per = cols / 4;
    for (int i = threadIdx.x; i < rows * per; i += 256) {
        const int r = i / per, c = (i % per) * 4;
        cp16(dst + r * ss + c, src + (long)r * gs + c);
    }
}

// Shared-memory row strides (floats), chosen so that the fragment loads below touch 32 different banks:
// operands read as A[row g][k t] or B[n g][k t] want stride = 4 (mod 32); operands read as [k t][n g] want 8 (mod 32).
template <int DK> struct Lay {
    static constexpr int LW = DK + 4;      // W, Qd, S: [row][k]
    static constexpr int LK = DK + 8;      // Kd: [t][k] read as B[k = t][n = k]
    static constexpr int LP = GC + 4;      // P: [t][j]
    static constexpr int LU = DVS + 8;     // U: [j][v] read as B[k = j][n = v] and as A[m = v][k = j]
    static constexpr int floats = DVS * LW + 2 * GC * LW + GC * LK + GC * LP + GC * LU;
};
}  // namespace

// HASW = false: nothing to correct (W = 0, the Mamba2 form): U = U0, and neither W's tiles nor its product exist.
template <int DK, bool HASW>
__global__ void __launch_bounds__(256) gdn_chunk_carry_kernel(GdnCarryArgs a) {
    using L = Lay<DK>;
    extern __shared__ __align__(16) float sm[];
    float* sS = sm;                       // [DVS][LW]   state slice
    float* sW = sS + DVS * L::LW;         // [64][LW]
    float* sQ = sW + GC * L::LW;          // [64][LW]
    float* sK = sQ + GC * L::LW;          // [64][LK]
    float* sP = sK + GC * L::LK;          // [64][LP]
    float* sU = sP + GC * L::LP;          // [64][LU]
    const int h = blockIdx.y, dv0 = blockIdx.x * DVS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int Dv = a.Dv, nc = a.nc;
    float* Sg = a.state + ((long)h * Dv + dv0) * DK;
    const long hc = (long)h * nc;
    // prologue: the state slice and the first chunk's operands, in the commit order W | Qd + P | Kd kept below
    stage(sS, L::LW, Sg, DK, DVS, DK);
    if (HASW) stage(sW, L::LW, a.W + hc * GC * DK, DK, GC, DK);
    cp_commit();
    stage(sQ, L::LW, a.Qd + hc * GC * DK, DK, GC, DK);
    stage(sP, L::LP, a.P + hc * GC * GC, GC, GC, GC);
    cp_commit();
    stage(sK, L::LK, a.Kd + hc * GC * DK, DK, GC, DK);
    cp_commit();

    // tiles of the [64, 32] products: warp -> 16 rows (mt) x 16 columns (two n-tiles of 8)
    const int mt = warp >> 1, nb = (warp & 1) * 2;
    for (int c = 0; c < nc; ++c) {
        const long ch = hc + c;
        const bool more = c + 1 < nc;
        // U0 fragments straight from global (requested before the wait)
        float u[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float* p0 = a.U0 + (ch * GC + mt * 16 + g) * Dv + dv0 + (nb + j) * 8 + 2 * t;
            const float2 lo = *reinterpret_cast<const float2*>(p0), hi = *reinterpret_cast<const float2*>(p0 + 8L * Dv);
            u[j][0] = lo.x; u[j][1] = lo.y; u[j][2] = hi.x; u[j][3] = hi.y;
        }
        const float gam = a.gamma[ch];
        cp_wait2();                       // W of this chunk (and, for c = 0, the state) has landed
        __syncthreads();
        // ---- U = U0 - W S^T
        {
            float acc[2][4] = {};
#pragma unroll 4
            for (int k0 = 0; HASW && k0 < DK; k0 += 8) {
                uint32_t af[4];
                const float* ap = sW + (mt * 16 + g) * L::LW + k0 + t;
                af[0] = tf32(ap[0]); af[1] = tf32(ap[8 * L::LW]); af[2] = tf32(ap[4]); af[3] = tf32(ap[8 * L::LW + 4]);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float* bp = sS + ((nb + j) * 8 + g) * L::LW + k0 + t;
                    mma_tf32(acc[j], af, tf32(bp[0]), tf32(bp[4]));
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float* up = sU + (mt * 16 + g) * L::LU + (nb + j) * 8 + 2 * t;
                up[0] = u[j][0] - acc[j][0]; up[1] = u[j][1] - acc[j][1];
                up[8 * L::LU] = u[j][2] - acc[j][2]; up[8 * L::LU + 1] = u[j][3] - acc[j][3];
            }
        }
        __syncthreads();                  // U complete, W free
        if (more && HASW) stage(sW, L::LW, a.W + (ch + 1) * GC * DK, DK, GC, DK);
        cp_commit();
        cp_wait2();                       // Qd and P of this chunk
        __syncthreads();
        // ---- O = Qd S^T + P U
        {
            float acc[2][4] = {};
#pragma unroll 4
            for (int k0 = 0; k0 < DK; k0 += 8) {
                uint32_t af[4];
                const float* ap = sQ + (mt * 16 + g) * L::LW + k0 + t;
                af[0] = tf32(ap[0]); af[1] = tf32(ap[8 * L::LW]); af[2] = tf32(ap[4]); af[3] = tf32(ap[8 * L::LW + 4]);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float* bp = sS + ((nb + j) * 8 + g) * L::LW + k0 + t;
                    mma_tf32(acc[j], af, tf32(bp[0]), tf32(bp[4]));
                }
            }
#pragma unroll 4
            for (int k0 = 0; k0 < GC; k0 += 8) {
                uint32_t af[4];
                const float* ap = sP + (mt * 16 + g) * L::LP + k0 + t;
                af[0] = tf32(ap[0]); af[1] = tf32(ap[8 * L::LP]); af[2] = tf32(ap[4]); af[3] = tf32(ap[8 * L::LP + 4]);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float* bp = sU + (k0 + t) * L::LU + (nb + j) * 8 + g;
                    mma_tf32(acc[j], af, tf32(bp[0]), tf32(bp[4 * L::LU]));
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float* op = a.out + (ch * GC + mt * 16 + g) * Dv + dv0 + (nb + j) * 8 + 2 * t;
                *reinterpret_cast<float2*>(op) = make_float2(acc[j][0], acc[j][1]);
                *reinterpret_cast<float2*>(op + 8L * Dv) = make_float2(acc[j][2], acc[j][3]);
            }
        }
        __syncthreads();                  // Qd, P free; every read of the old state is done
        if (more) {
            stage(sQ, L::LW, a.Qd + (ch + 1) * GC * DK, DK, GC, DK);
            stage(sP, L::LP, a.P + (ch + 1) * GC * GC, GC, GC, GC);
        }
        cp_commit();
        cp_wait2();                       // Kd of this chunk
        __syncthreads();
        // ---- S = gamma S + U^T Kd: [32, DK] as 2 x (DK / 8) tiles, warp -> one 16-row half and DK / 32 column tiles
        {
            constexpr int NT = DK / 32;                   // n-tiles per warp
            const int m2 = warp & 1, n0 = (warp >> 1) * NT;
            float acc[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const float* sp = sS + (m2 * 16 + g) * L::LW + (n0 + j) * 8 + 2 * t;
                acc[j][0] = gam * sp[0]; acc[j][1] = gam * sp[1];
                acc[j][2] = gam * sp[8 * L::LW]; acc[j][3] = gam * sp[8 * L::LW + 1];
            }
#pragma unroll 2
            for (int k0 = 0; k0 < GC; k0 += 8) {
                uint32_t af[4];                           // A[m = v][k = token] = U[token][v]
                const float* ap = sU + (k0 + t) * L::LU + m2 * 16 + g;
                af[0] = tf32(ap[0]); af[1] = tf32(ap[8]); af[2] = tf32(ap[4 * L::LU]); af[3] = tf32(ap[4 * L::LU + 8]);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const float* bp = sK + (k0 + t) * L::LK + (n0 + j) * 8 + g;
                    mma_tf32(acc[j], af, tf32(bp[0]), tf32(bp[4 * L::LK]));
                }
            }
            // each warp reads only the state rows and columns it writes, so no barrier between the read above and this
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float* sp = sS + (m2 * 16 + g) * L::LW + (n0 + j) * 8 + 2 * t;
                sp[0] = acc[j][0]; sp[1] = acc[j][1];
                sp[8 * L::LW] = acc[j][2]; sp[8 * L::LW + 1] = acc[j][3];
            }
        }
        __syncthreads();                  // new state visible, Kd and U free
        if (more) stage(sK, L::LK, a.Kd + (ch + 1) * GC * DK, DK, GC, DK);
        cp_commit();
    }
    asm volatile("cp.async.wait_group 0;");
    for (int i = threadIdx.x; i < DVS * (DK / 4); i += 256) {
        const int r = i / (DK / 4), c4 = (i % (DK / 4)) * 4;
        *reinterpret_cast<float4*>(Sg + (long)r * DK + c4) = *reinterpret_cast<const float4*>(sS + r * L::LW + c4);
    }
}

template <int DK, bool HASW>
static int launch_carry_w(const GdnCarryArgs& a, cudaStream_t s) {
    const size_t smem = (size_t)Lay<DK>::floats * sizeof(float);
    static bool configured = false;
    if (!configured) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(gdn_chunk_carry_kernel<DK, HASW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    gdn_chunk_carry_kernel<DK, HASW><<<dim3(a.Dv / DVS, a.Hv), 256, smem, s>>>(a);
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

template <int DK>
static int launch_carry(const GdnCarryArgs& a, cudaStream_t s) {
    return a.W != nullptr ? launch_carry_w<DK, true>(a, s) : launch_carry_w<DK, false>(a, s);
}

// One sequence: carries `state` through `nc` chunks of 64 tokens and writes the chunk outputs.
extern "C" int tsb_gdn_chunk_carry(const GdnCarryArgs* args, void* stream) {
    TSB_CHECK_ARG(args != nullptr, "gdn_chunk_carry: null arguments");
    const GdnCarryArgs& a = *args;
    TSB_CHECK_ARG(a.Hv > 0 && a.nc > 0, "gdn_chunk_carry: Hv=%d chunks=%d", a.Hv, a.nc);
    TSB_CHECK_ARG(a.Dv % DVS == 0 && a.Dv > 0, "gdn_chunk_carry: value head size %d is not a multiple of %d", a.Dv, DVS);
    switch (a.Dk) {
    case 64: return launch_carry<64>(a, (cudaStream_t)stream);
    case 128: return launch_carry<128>(a, (cudaStream_t)stream);
    default:
        tsb_set_error("gdn_chunk_carry: key head size %d unsupported (64, 128)", a.Dk);
        return TSB_ERR_UNSUPPORTED;
    }
}

// ==========================================================================================
// The chunk-parallel part: everything the carry kernel consumes, from the layer's packed projections.
//
// One CTA per (sequence, value head, chunk of 64 tokens).  With k, q the L2-normalised key / query rows (q also times
// Dv^-1/2), g the log-decay and b the write strength of each token, c_i the running sum of g inside the chunk:
//     A[i][j]  = b_i (k_i . k_j) exp(c_i - c_j)        j <  i      (strictly lower triangular)
//     P[i][j]  =     (q_i . k_j) exp(c_i - c_j)        j <= i
//     (I + A) [U0 | W] = [b v | b exp(c) k]            forward substitution, one right-hand-side column per thread
//     Qd = q exp(c),   Kd = k exp(c_last - c),   gamma = exp(c_last)
// The two Gram products run on the tensor cores with split tf32 operands (hi + lo parts, three products), which keeps
// f32-level accuracy in the matrix that the substitution then inverts.  Tokens past a sequence's end are zero rows
// (b = 0, g = 0): they leave state and outputs untouched, so ragged batches share one launch.
// ==========================================================================================
struct GdnPrepArgs {
    const float* qkv; long qkv_s;          // [T, 2 Hk Dk + Hv Dv] rows: q heads | k heads | v heads
    const void* beta; const void* alpha; long ba_s; int ba_f32;      // [T, Hv]
    const float* dt_bias; const float* a_log;                        // [Hv]
    const int* cu_q;                       // [B + 1] first row of each sequence
    float* U0; float* W; float* Qd; float* Kd; float* P; float* gamma;
    int Hk, Hv, Dk, Dv, B, nc;
    float eps;
};

namespace {
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    hi = tf32(x);
    lo = tf32(x - __uint_as_float(hi));
}
__device__ __forceinline__ float ld_ba(const void* p, long i, int f32) {
    return f32 ? reinterpret_cast<const float*>(p)[i] : bf2f(reinterpret_cast<const bf16*>(p)[i]);
}
}  // namespace

template <int DK>
__global__ void __launch_bounds__(256) gdn_chunk_prep_kernel(GdnPrepArgs a) {
    constexpr int LQ = DK + 4;             // row stride of the q / k tiles (fragment loads hit 32 banks)
    constexpr int LA = GC + 1;
    extern __shared__ __align__(16) float sm[];
    const int Dv = a.Dv, NX = Dv + DK, LX = NX + 4;
    float* sK = sm;                        // [64][LQ] normalised keys
    float* sQ = sK + GC * LQ;              // [64][LQ] normalised, scaled queries
    float* sX = sQ + GC * LQ;              // [64][LX] right-hand sides [b v | b exp(c) k]
    float* sA = sX + GC * LX;              // [64][LA] strictly lower triangular A
    float* sc = sA + GC * LA;              // [64] running log-decay
    float* sb = sc + GC;                   // [64] write strength
    const int c = blockIdx.x, bh = blockIdx.y, b = bh / a.Hv, h = bh % a.Hv, hk = h % a.Hk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = a.cu_q[b], len = a.cu_q[b + 1] - row0;
    const int valid = max(0, min(GC, len - c * GC));           // tokens of this chunk that exist
    const long tok0 = (long)row0 + (long)c * GC;
    const float qscale = rsqrtf((float)Dv);
    // ---- rows: normalise q and k, stage v, per-token scalars
    for (int r = warp; r < GC; r += 8) {
        const bool ok = r < valid;
        const float* row = a.qkv + (tok0 + r) * a.qkv_s;
        float qs = 0.f, ks = 0.f;
        float qv[DK / 32], kv[DK / 32];
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) {
            qv[i] = ok ? row[hk * DK + lane + 32 * i] : 0.f;
            kv[i] = ok ? row[(long)a.Hk * DK + hk * DK + lane + 32 * i] : 0.f;
            qs += qv[i] * qv[i];
            ks += kv[i] * kv[i];
        }
        qs = warp_sum(qs);
        ks = warp_sum(ks);
        const float qn = ok ? qscale * rsqrtf(qs + a.eps) : 0.f, kn = ok ? rsqrtf(ks + a.eps) : 0.f;
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) {
            sQ[r * LQ + lane + 32 * i] = qv[i] * qn;
            sK[r * LQ + lane + 32 * i] = kv[i] * kn;
        }
        for (int d = lane; d < Dv; d += 32) sX[r * LX + d] = ok ? row[2L * a.Hk * DK + (long)h * Dv + d] : 0.f;
        if (lane == 0) {
            float g = 0.f, be = 0.f;
            if (ok) {
                const float al = ld_ba(a.alpha, (tok0 + r) * a.ba_s + h, a.ba_f32) + a.dt_bias[h];
                g = (al > 20.f ? al : log1pf(__expf(al))) * a.a_log[h];
                be = 1.f / (1.f + __expf(-ld_ba(a.beta, (tok0 + r) * a.ba_s + h, a.ba_f32)));
            }
            sc[r] = g;
            sb[r] = be;
        }
    }
    __syncthreads();
    if (warp == 0) {                       // inclusive running sum over the 64 tokens
        float x0 = sc[lane], x1 = sc[lane + 32];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y0 = __shfl_up_sync(0xffffffffu, x0, o), y1 = __shfl_up_sync(0xffffffffu, x1, o);
            if (lane >= o) { x0 += y0; x1 += y1; }
        }
        x1 += __shfl_sync(0xffffffffu, x0, 31);
        sc[lane] = x0;
        sc[lane + 32] = x1;
    }
    __syncthreads();
    const float c_last = sc[GC - 1];
    const long ch = (long)bh * a.nc + c;
    // ---- Gram products k k^T and q k^T: warp -> rows mt * 16 .. + 15, columns nq * 32 .. + 31 of both
    {
        const int g = lane >> 2, t = lane & 3, mt = warp & 3, nq = warp >> 2;
        float kk[4][4] = {}, qk[4][4] = {};
#pragma unroll 2
        for (int k0 = 0; k0 < DK; k0 += 8) {
            uint32_t ah[4], al[4], qh[4], ql[4];
            const float* ap = sK + (mt * 16 + g) * LQ + k0 + t;
            const float* qp = sQ + (mt * 16 + g) * LQ + k0 + t;
            split_tf32(ap[0], ah[0], al[0]); split_tf32(ap[8 * LQ], ah[1], al[1]);
            split_tf32(ap[4], ah[2], al[2]); split_tf32(ap[8 * LQ + 4], ah[3], al[3]);
            split_tf32(qp[0], qh[0], ql[0]); split_tf32(qp[8 * LQ], qh[1], ql[1]);
            split_tf32(qp[4], qh[2], ql[2]); split_tf32(qp[8 * LQ + 4], qh[3], ql[3]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* bp = sK + ((nq * 4 + j) * 8 + g) * LQ + k0 + t;
                uint32_t b0h, b0l, b1h, b1l;
                split_tf32(bp[0], b0h, b0l);
                split_tf32(bp[4], b1h, b1l);
                mma_tf32(kk[j], al, b0h, b1h); mma_tf32(kk[j], ah, b0l, b1l); mma_tf32(kk[j], ah, b0h, b1h);
                mma_tf32(qk[j], ql, b0h, b1h); mma_tf32(qk[j], qh, b0l, b1l); mma_tf32(qk[j], qh, b0h, b1h);
            }
        }
        float* Pg = a.P + ch * GC * GC;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = mt * 16 + g + (e >> 1) * 8, jj = (nq * 4 + j) * 8 + 2 * t + (e & 1);
                const float m = jj <= i ? __expf(fminf(sc[i] - sc[jj], 0.f)) : 0.f;
                sA[i * LA + jj] = jj < i ? sb[i] * kk[j][e] * m : 0.f;
                Pg[i * GC + jj] = qk[j][e] * m;
            }
        }
    }
    // ---- right-hand sides (the v part is staged already), Qd, Kd, gamma
    for (int r = warp; r < GC; r += 8) {
        const float be = sb[r], dec = __expf(sc[r]), tail = __expf(c_last - sc[r]);
        for (int d = lane; d < Dv; d += 32) sX[r * LX + d] *= be;
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) {
            const int d = lane + 32 * i;
            const float kv = sK[r * LQ + d];
            sX[r * LX + Dv + d] = be * dec * kv;
            a.Kd[(ch * GC + r) * DK + d] = kv * tail;
            a.Qd[(ch * GC + r) * DK + d] = sQ[r * LQ + d] * dec;
        }
    }
    if (threadIdx.x == 0) a.gamma[ch] = __expf(c_last);
    __syncthreads();
    // ---- (I + A) X = RHS by forward substitution; a thread owns one column and keeps its solution in registers
    for (int col = threadIdx.x; col < NX; col += 256) {
        float x[GC];
#pragma unroll
        for (int i = 0; i < GC; ++i) {
            float acc = sX[i * LX + col];
#pragma unroll
            for (int j = 0; j < i; ++j) acc -= sA[i * LA + j] * x[j];
            x[i] = acc;
            if (col < Dv) a.U0[(ch * GC + i) * Dv + col] = acc;
            else a.W[(ch * GC + i) * DK + col - Dv] = acc;
        }
    }
}

// Gated output: core [B * Hv, nc, 64, Dv] -> out[t, h * Dv + d] = rmsnorm(core) * norm_w[d] * silu(z[t, h * Dv + d]) (bf16).
struct GdnFinishArgs {
    const float* core; const void* z; long z_s; int z_f32;
    const float* norm_w; const int* cu_q;
    bf16* out; long out_s;
    int Hv, Dv, B, nc;
    float eps;
};

__global__ void __launch_bounds__(256) gdn_chunk_finish_kernel(GdnFinishArgs a) {
    const int c = blockIdx.x, bh = blockIdx.y, b = bh / a.Hv, h = bh % a.Hv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = a.cu_q[b], len = a.cu_q[b + 1] - row0;
    const int Dv = a.Dv;
    for (int r = warp; r < GC; r += 8) {
        const int pos = c * GC + r;
        if (pos >= len) break;
        const float* src = a.core + (((long)bh * a.nc + c) * GC + r) * Dv;
        float v[8], ss = 0.f;                                  // Dv <= 256
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            v[i] = d < Dv ? src[d] : 0.f;
            ss += v[i] * v[i];
        }
        ss = warp_sum(ss);
        const float rs = rsqrtf(ss / (float)Dv + a.eps);
        const long t = (long)row0 + pos;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            if (d < Dv) {
                const long zi = t * a.z_s + (long)h * Dv + d;
                const float zz = a.z_f32 ? reinterpret_cast<const float*>(a.z)[zi] : bf2f(reinterpret_cast<const bf16*>(a.z)[zi]);
                a.out[t * a.out_s + (long)h * Dv + d] = f2bf(v[i] * rs * a.norm_w[d] * (zz / (1.f + __expf(-zz))));
            }
        }
    }
}

template <int DK>
static int launch_prep(const GdnPrepArgs& a, cudaStream_t s) {
    const size_t smem = sizeof(float) * ((size_t)2 * GC * (DK + 4) + (size_t)GC * (a.Dv + DK + 4) + (size_t)GC * (GC + 1) + 2 * GC);
    static size_t configured = 0;
    if (smem > configured) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(gdn_chunk_prep_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    gdn_chunk_prep_kernel<DK><<<dim3(a.nc, a.B * a.Hv), 256, smem, s>>>(a);
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

extern "C" int tsb_gdn_chunk_prep(const GdnPrepArgs* args, void* stream) {
    TSB_CHECK_ARG(args != nullptr, "gdn_chunk_prep: null arguments");
    const GdnPrepArgs& a = *args;
    TSB_CHECK_ARG(a.B > 0 && a.nc > 0 && a.Hv > 0 && a.Hk > 0, "gdn_chunk_prep: B=%d chunks=%d heads=%d/%d", a.B, a.nc, a.Hk, a.Hv);
    TSB_CHECK_ARG(a.Dv % 32 == 0 && a.Dv > 0 && a.Dv <= 128, "gdn_chunk_prep: value head size %d (multiples of 32 up to 128)", a.Dv);
    TSB_CHECK_ARG((long)a.B * a.Hv <= 65535, "gdn_chunk_prep: %d x %d sequence-heads exceed the grid", a.B, a.Hv);
    switch (a.Dk) {
    case 64: return launch_prep<64>(a, (cudaStream_t)stream);
    case 128: return launch_prep<128>(a, (cudaStream_t)stream);
    default:
        tsb_set_error("gdn_chunk_prep: key head size %d unsupported (64, 128)", a.Dk);
        return TSB_ERR_UNSUPPORTED;
    }
}

// ------------------------------------------------------------------------------------------
// Mamba2 in chunked (state-space duality) form: the chunk-parallel part for one (sequence, head, chunk).  With
// d = softplus(dt + bias), log-decay c = cumsum(d * A) inside the chunk, inputs X = d * x, and the group's B / C rows:
//   U0 = X                       what a token writes
//   Qd = C * exp(c)              reads of the state entering the chunk
//   Kd = B * exp(c_last - c)     writes that survive to the chunk's end
//   P  = (C B^T) * exp(c_i - c_j) for j <= i, else 0        contributions inside the chunk
//   gamma = exp(c_last)
// which is exactly what gdn_chunk_carry_kernel consumes with W = 0: out = Qd S^T + P U0, S <- gamma S + U0^T Kd.
// Reference: the ssm_scan path of ggml (ggml-cuda/ssm-scan.cu) is a token-by-token scan; the chunked form is this
// framework's own.
// ------------------------------------------------------------------------------------------
struct MambaPrepArgs {
    const float* xbc; long xbc_s;          // [T, H Pd + 2 G N] rows: x heads | B groups | C groups
    const void* dt; long dt_s; int dt_f32; // [T, H]
    const float* dt_bias; const float* A;  // [H] (dt_bias may be null)
    const int* cu_q;                       // [B + 1]
    float* U0; float* Qd; float* Kd; float* P; float* gamma;
    int H, Pd, G, N, B, nc;
};

template <int DK>
__global__ void __launch_bounds__(256) mamba2_chunk_prep_kernel(MambaPrepArgs a) {
    constexpr int LQ = DK + 4;
    extern __shared__ __align__(16) float sm[];
    float* sK = sm;                        // [64][LQ] B rows
    float* sQ = sK + GC * LQ;              // [64][LQ] C rows
    float* sc = sQ + GC * LQ;              // [64] running log-decay
    float* sd = sc + GC;                   // [64] step size d
    const int c = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H, grp = h / (a.H / a.G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = a.cu_q[b], len = a.cu_q[b + 1] - row0;
    const int valid = max(0, min(GC, len - c * GC));
    const long tok0 = (long)row0 + (long)c * GC;
    const long ch = (long)bh * a.nc + c;
    const int Pd = a.Pd;
    const long offB = (long)a.H * Pd + (long)grp * DK, offC = offB + (long)a.G * DK;
    for (int r = warp; r < GC; r += 8) {
        const bool ok = r < valid;
        const float* row = a.xbc + (tok0 + r) * a.xbc_s;
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) {
            sK[r * LQ + lane + 32 * i] = ok ? row[offB + lane + 32 * i] : 0.f;
            sQ[r * LQ + lane + 32 * i] = ok ? row[offC + lane + 32 * i] : 0.f;
        }
        float d = 0.f;
        if (ok) {
            const long di = (tok0 + r) * a.dt_s + h;
            const float v = (a.dt_f32 ? reinterpret_cast<const float*>(a.dt)[di] : bf2f(reinterpret_cast<const bf16*>(a.dt)[di])) +
                            (a.dt_bias ? a.dt_bias[h] : 0.f);
            d = v > 20.f ? v : log1pf(__expf(v));
        }
        for (int e = lane; e < Pd; e += 32) a.U0[(ch * GC + r) * Pd + e] = ok ? row[(long)h * Pd + e] * d : 0.f;
        if (lane == 0) {
            sd[r] = d;
            sc[r] = d * a.A[h];
        }
    }
    __syncthreads();
    if (warp == 0) {                       // inclusive running sum over the 64 tokens
        float x0 = sc[lane], x1 = sc[lane + 32];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y0 = __shfl_up_sync(0xffffffffu, x0, o), y1 = __shfl_up_sync(0xffffffffu, x1, o);
            if (lane >= o) { x0 += y0; x1 += y1; }
        }
        x1 += __shfl_sync(0xffffffffu, x0, 31);
        sc[lane] = x0;
        sc[lane + 32] = x1;
    }
    __syncthreads();
    const float c_last = sc[GC - 1];
    // ---- C B^T: warp -> rows mt * 16 .. + 15, columns nq * 32 .. + 31 (split tf32: three products per term)
    {
        const int g = lane >> 2, t = lane & 3, mt = warp & 3, nq = warp >> 2;
        float qk[4][4] = {};
#pragma unroll 2
        for (int k0 = 0; k0 < DK; k0 += 8) {
            uint32_t qh[4], ql[4];
            const float* qp = sQ + (mt * 16 + g) * LQ + k0 + t;
            split_tf32(qp[0], qh[0], ql[0]); split_tf32(qp[8 * LQ], qh[1], ql[1]);
            split_tf32(qp[4], qh[2], ql[2]); split_tf32(qp[8 * LQ + 4], qh[3], ql[3]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* bp = sK + ((nq * 4 + j) * 8 + g) * LQ + k0 + t;
                uint32_t b0h, b0l, b1h, b1l;
                split_tf32(bp[0], b0h, b0l);
                split_tf32(bp[4], b1h, b1l);
                mma_tf32(qk[j], ql, b0h, b1h); mma_tf32(qk[j], qh, b0l, b1l); mma_tf32(qk[j], qh, b0h, b1h);
            }
        }
        float* Pg = a.P + ch * GC * GC;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = mt * 16 + g + (e >> 1) * 8, jj = (nq * 4 + j) * 8 + 2 * t + (e & 1);
                Pg[i * GC + jj] = jj <= i ? qk[j][e] * __expf(fminf(sc[i] - sc[jj], 0.f)) : 0.f;
            }
        }
    }
    for (int r = warp; r < GC; r += 8) {
        const float dec = __expf(sc[r]), tail = __expf(c_last - sc[r]);
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) {
            const int d = lane + 32 * i;
            a.Kd[(ch * GC + r) * DK + d] = sK[r * LQ + d] * tail;
            a.Qd[(ch * GC + r) * DK + d] = sQ[r * LQ + d] * dec;
        }
    }
    if (threadIdx.x == 0) a.gamma[ch] = __expf(c_last);
}

template <int DK>
static int launch_mamba_prep(const MambaPrepArgs& a, cudaStream_t s) {
    const size_t smem = ((size_t)2 * GC * (DK + 4) + 2 * GC) * sizeof(float);
    static size_t configured = 0;
    if (smem > configured) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(mamba2_chunk_prep_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    mamba2_chunk_prep_kernel<DK><<<dim3(a.nc, a.B * a.H), 256, smem, s>>>(a);
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

extern "C" int tsb_mamba2_chunk_prep(const MambaPrepArgs* args, void* stream) {
    TSB_CHECK_ARG(args != nullptr, "mamba2_chunk_prep: null arguments");
    const MambaPrepArgs& a = *args;
    TSB_CHECK_ARG(a.B > 0 && a.nc > 0 && a.H > 0 && a.G > 0 && a.H % a.G == 0, "mamba2_chunk_prep: B=%d chunks=%d heads=%d groups=%d", a.B, a.nc,
                  a.H, a.G);
    TSB_CHECK_ARG(a.Pd > 0, "mamba2_chunk_prep: head size %d", a.Pd);
    TSB_CHECK_ARG((long)a.B * a.H <= 65535, "mamba2_chunk_prep: %d x %d sequence-heads exceed the grid", a.B, a.H);
    switch (a.N) {
    case 64: return launch_mamba_prep<64>(a, (cudaStream_t)stream);
    case 128: return launch_mamba_prep<128>(a, (cudaStream_t)stream);
    default:
        tsb_set_error("mamba2_chunk_prep: state size %d unsupported (64, 128)", a.N);
        return TSB_ERR_UNSUPPORTED;
    }
}

extern "C" int tsb_gdn_chunk_finish(const GdnFinishArgs* args, void* stream) {
    TSB_CHECK_ARG(args != nullptr, "gdn_chunk_finish: null arguments");
    const GdnFinishArgs& a = *args;
    TSB_CHECK_ARG(a.Dv > 0 && a.Dv <= 256 && a.B > 0 && a.nc > 0, "gdn_chunk_finish: Dv=%d B=%d chunks=%d", a.Dv, a.B, a.nc);
    TSB_CHECK_ARG((long)a.B * a.Hv <= 65535, "gdn_chunk_finish: %d x %d sequence-heads exceed the grid", a.B, a.Hv);
    gdn_chunk_finish_kernel<<<dim3(a.nc, a.B * a.Hv), 256, 0, (cudaStream_t)stream>>>(a);
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}
