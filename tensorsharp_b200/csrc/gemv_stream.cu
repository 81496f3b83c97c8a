// Decode GEMV for Q4_K / Q5_K weights with a deep asynchronous row pipeline.
//
// The one-warp-per-row GEMV keeps two 16-byte loads per lane in flight; with rows of 1.4 KB (K = 2560)
// a warp's whole life is three such round trips, and the launch runs as four waves of short-lived
// CTAs: measured 17.7 us for the 28 MB gate/up matrix of a Qwen3-4B layer (4.3 us at the copy rate).
// Here a warp owns a contiguous range of row pairs and streams them through a ring of D row buffers
// in shared memory filled by cp.async (coalesced 16-byte copies of the row's contiguous GGUF blocks),
// so D - 1 whole rows per warp are in flight all the time (about 10 KB per warp, 150 KB per SM), the
// first rows are requested before the kernel waits for its predecessor, and the grid is one wave.
// The block arithmetic is the same comp_q45k as the plain kernel, fed from shared memory.
//
// Same contract as gemv_kernel without expert ids and without the tensor-parallel push: bias, gated
// activation over (row r, row r + N/2), ReLU^2, row scale, residual, f32 or bf16 output; M <= 4.
// Replaces mul_mat_vec_q + quantize_q8_1 of the reference (ggml-cuda/mmvq.cu:143) for these types.
#include <cstdlib>
#include "gemv_core.cuh"

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int M, bool GLU, bool Q5, int D>
__global__ void __launch_bounds__(128) gemv_stream_kernel(GemvArgs a, int ppw) {
    extern __shared__ uint4 stream_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = a.w.K, nb = K >> 8;
    constexpr int BLK16 = Q5 ? 11 : 9;                 // 16-byte chunks per 256-value block
    const int chunks = nb * BLK16;                     // per row
    uint4* ring = stream_smem + (long)warp * D * chunks;
    const int N = a.w.N, n_out = a.n_out;
    const int n_pairs = GLU ? n_out : (N + 1) / 2;
    const int p0 = (blockIdx.x * 4 + warp) * ppw, p1 = min(n_pairs, p0 + ppw);
    const int ntask = p1 > p0 ? 2 * (p1 - p0) : 0;

    auto task_row = [&](int i) -> int {                // weight row of task i, or -1
        const int pair = p0 + (i >> 1), which = i & 1;
        if (GLU) return which ? pair + n_out : pair;
        const int r = 2 * pair + which;
        return r < N ? r : -1;
    };
    auto issue = [&](int i) {
        if (i < ntask) {
            const int r = task_row(i);
            if (r >= 0) {
                const uint4* src = reinterpret_cast<const uint4*>(a.w.p0) + (long)r * chunks;
                uint4* dst = ring + (long)(i % D) * chunks;
                for (int c = lane; c < chunks; c += 32) cp_async16(dst + c, src + c);
            }
        }
        cp_async_commit();                             // one group per task, empty or not: the wait below counts groups
    };
#pragma unroll
    for (int i = 0; i < D - 1; ++i) issue(i);          // weights never change: requested before the dependency wait
    pdl_wait();
    pdl_trigger();

    float keep[M];                                     // gate result (GLU) while the up row is computed
#pragma unroll
    for (int m = 0; m < M; ++m) keep[m] = 0.f;
    const int mv = min(M, a.M);
    const int units = nb << 3;
    for (int i = 0; i < ntask; ++i) {
        issue(i + D - 1);
        cp_async_wait<D - 1>();
        __syncwarp();
        const int r = task_row(i);
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        if (r >= 0) {
            const uint4* st = ring + (long)(i % D) * chunks;
            for (int u = lane; u < units; u += 32) {
                const int b = u >> 3, uu = u & 7;
                WQ4K t;
                t.hdr = st[b * BLK16];
                if (Q5) {
                    t.hv = st[b * BLK16 + 1 + (uu & 1)];
                    t.qv = st[b * BLK16 + 3 + uu];
                } else {
                    t.qv = st[b * BLK16 + 1 + uu];
                }
                comp_q45k<M, Q5>(a.w, t, u, a.xq, a.xds, acc, mv);
            }
#pragma unroll
            for (int m = 0; m < M; ++m) acc[m] = warp_sum(acc[m]);
        }
        __syncwarp();                                  // every lane is done with this buffer before it is refilled
        if (GLU && !(i & 1)) {
#pragma unroll
            for (int m = 0; m < M; ++m) keep[m] = acc[m];
            continue;
        }
        if (lane != 0 || r < 0) continue;
        const int orow_col = GLU ? p0 + (i >> 1) : r;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m >= mv) break;
            float v;
            if (GLU) {
                float g = keep[m], up = acc[m];
                if (a.bias) { g += a.bias[orow_col]; up += a.bias[orow_col + n_out]; }
                v = act_glu(a.act, g, up);
            } else {
                v = acc[m];
                if (a.bias) v += a.bias[orow_col];
                if (a.act == ACT_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
            }
            if (a.row_scale) v *= a.row_scale[m];
            const long o = (long)m * n_out + orow_col;
            if (a.out_f32) {
                if (a.residual) v += reinterpret_cast<const float*>(a.residual)[o];
                reinterpret_cast<float*>(a.out)[o] = v;
            } else {
                if (a.residual) v += bf2f(reinterpret_cast<const bf16*>(a.residual)[o]);
                reinterpret_cast<bf16*>(a.out)[o] = f2bf(v);
            }
        }
    }
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// Single-token Q4_K rows of up to 4096 values: the instruction diet.  The generic block arithmetic
// spends about 150 instructions per 64 weights (measured: 8.7 M warp instructions for a 28 MB
// matrix, issue slots 47 % busy, DRAM 16 %), most of it on things that do not depend on the row.
// A lane's units (u = lane + 32 j) are the same for every row its warp streams, so the activation
// words, their scales and sums, the shared-memory offsets and the scale-field selectors are
// computed once per kernel and kept in registers; per row and unit what remains is two shared
// loads, the nibble split, eight dp4a, a branch-free 6-bit scale extraction on packed pairs, and
// int -> float by the magic-constant add instead of conversion instructions.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float i2f_small(int n) { return __int_as_float(0x4B400000 + n) - 12582912.f; }        // |n| < 2^22
__device__ __forceinline__ float u2f_small(unsigned n) { return __int_as_float(0x4B000000 | n) - 8388608.f; }   // n < 2^23

// KS = 1: a warp owns whole rows.  KS = 4 (rows longer than 4096 values, e.g. the FFN down projection):
// the four warps of a CTA split every row by 256-value blocks, each streams and hoists only its
// quarter, and the partial sums meet in shared memory (one barrier per row, double-buffered).
template <bool GLU, int D, int NJ, int KS>
__global__ void __launch_bounds__(128) gemv_stream_q4k_m1_kernel(GemvArgs a, int ppw) {
    extern __shared__ uint4 stream_smem[];
    __shared__ float part[2][4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = a.w.K, nb = K >> 8;
    const int bs = KS == 1 ? 0 : (nb * warp) / KS, be = KS == 1 ? nb : (nb * (warp + 1)) / KS;   // this warp's blocks
    const int max_blocks = KS == 1 ? nb : (nb + KS - 1) / KS;
    const int chunks = (be - bs) * 9, stage_chunks = max_blocks * 9, row_chunks = nb * 9;
    uint4* ring = stream_smem + (long)warp * D * stage_chunks;
    const int N = a.w.N, n_out = a.n_out;
    const int n_pairs = GLU ? n_out : (N + 1) / 2;
    const int owner = KS == 1 ? blockIdx.x * 4 + warp : blockIdx.x;          // rows belong to a warp, or to the CTA
    const int p0 = owner * ppw, p1 = min(n_pairs, p0 + ppw);
    const int ntask = p1 > p0 ? 2 * (p1 - p0) : 0;
    auto task_row = [&](int i) -> int {
        const int pair = p0 + (i >> 1), which = i & 1;
        if (GLU) return which ? pair + n_out : pair;
        const int r = 2 * pair + which;
        return r < N ? r : -1;
    };
    auto issue = [&](int i) {
        if (i < ntask) {
            const int r = task_row(i);
            if (r >= 0) {
                const uint4* src = reinterpret_cast<const uint4*>(a.w.p0) + (long)r * row_chunks + bs * 9;
                uint4* dst = ring + (long)(i % D) * stage_chunks;
                for (int c = lane; c < chunks; c += 32) cp_async16(dst + c, src + c);
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < D - 1; ++i) issue(i);
    pdl_wait();
    pdl_trigger();

    // row-independent state of this lane's units
    const int units = (be - bs) << 3;
    int xa[NJ][4], xb[NJ][4], offh[NJ], offq[NJ];
    float fx0[NJ], fx1[NJ], fm0[NJ], fm1[NJ];
    unsigned sh[NJ];
    bool hi[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int u = lane + 32 * j;
        const bool ok = u < units;
        const int uc = ok ? u : 0;
        const int bl = uc >> 3, b = bs + bl, uu = uc & 7, c = uu >> 1, h = uu & 1;
        const int xoff = b * 256 + 64 * c + 16 * h;
        const int4 va = *reinterpret_cast<const int4*>(a.xq + xoff);
        const int4 vb = *reinterpret_cast<const int4*>(a.xq + xoff + 32);
        xa[j][0] = va.x; xa[j][1] = va.y; xa[j][2] = va.z; xa[j][3] = va.w;
        xb[j][0] = vb.x; xb[j][1] = vb.y; xb[j][2] = vb.z; xb[j][3] = vb.w;
        const float2 e0 = a.xds[b * 8 + 2 * c], e1 = a.xds[b * 8 + 2 * c + 1];
        fx0[j] = ok ? e0.x : 0.f;
        fx1[j] = ok ? e1.x : 0.f;
        fm0[j] = (ok && h == 0) ? e0.y : 0.f;           // the minimum term is counted once per 32 values, by the h = 0 unit
        fm1[j] = (ok && h == 0) ? e1.y : 0.f;
        offh[j] = bl * 9;
        offq[j] = bl * 9 + 1 + uu;
        sh[j] = 16u * (c & 1);
        hi[j] = c >= 2;
    }

    float keep = 0.f;
    for (int i = 0; i < ntask; ++i) {
        issue(i + D - 1);
        cp_async_wait<D - 1>();
        __syncwarp();
        const int r = task_row(i);
        float acc = 0.f;
        if (r >= 0) {
            const uint4* st = ring + (long)(i % D) * stage_chunks;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const uint4 hdr = st[offh[j]];
                const uint4 q = st[offq[j]];
                const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
                int s0 = 0, s1 = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    s0 = __dp4a((int)(qq[k] & 0x0F0F0F0Fu), xa[j][k], s0);
                    s1 = __dp4a((int)((qq[k] >> 4) & 0x0F0F0F0Fu), xb[j][k], s1);
                }
                // 6-bit scales / minimums of sub-blocks 2c, 2c + 1 as packed byte pairs, both encodings, then select
                const uint32_t Y = hdr.y >> sh[j], Z = hdr.z >> sh[j], W = hdr.w >> sh[j];
                const uint32_t p_lo = Y & 0x3F3Fu, q_lo = Z & 0x3F3Fu;
                const uint32_t p_hi = (W & 0x0F0Fu) | ((Y >> 2) & 0x3030u), q_hi = ((W >> 4) & 0x0F0Fu) | ((Z >> 2) & 0x3030u);
                const uint32_t P = hi[j] ? p_hi : p_lo, Q = hi[j] ? q_hi : q_lo;
                const float t0 = i2f_small(s0 * (int)(P & 0xFFu)), t1 = i2f_small(s1 * (int)(P >> 8));
                const float A = t0 * fx0[j] + t1 * fx1[j];
                const float Bm = u2f_small(Q & 0xFFu) * fm0[j] + u2f_small(Q >> 8) * fm1[j];
                const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
                acc += dd.x * A - dd.y * Bm;
            }
            acc = warp_sum(acc);
        }
        __syncwarp();
        if (KS > 1) {
            if (lane == 0) part[i & 1][warp] = acc;
            __syncthreads();
            acc = part[i & 1][0] + part[i & 1][1] + part[i & 1][2] + part[i & 1][3];
            if (warp != 0) continue;
        }
        if (GLU && !(i & 1)) { keep = acc; continue; }
        if (!GLU && a.push != nullptr) {
            // row-parallel projection of a tensor-parallel layer: every lane holds the sum; lane q stores it,
            // tagged with the exchange number, into rank q's mailbox
            if (r >= 0) gemv_push_store(a.push, lane, r, (a.bias && a.push->rank == 0) ? acc + a.bias[r] : acc);
            continue;
        }
        if (lane != 0 || r < 0) continue;
        const int col = GLU ? p0 + (i >> 1) : r;
        float v;
        if (GLU) {
            float g = keep, up = acc;
            if (a.bias) { g += a.bias[col]; up += a.bias[col + n_out]; }
            v = act_glu(a.act, g, up);
        } else {
            v = acc;
            if (a.bias) v += a.bias[col];
            if (a.act == ACT_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
        }
        if (a.row_scale) v *= a.row_scale[0];
        if (a.out_f32) {
            if (a.residual) v += reinterpret_cast<const float*>(a.residual)[col];
            reinterpret_cast<float*>(a.out)[col] = v;
        } else {
            if (a.residual) v += bf2f(reinterpret_cast<const bf16*>(a.residual)[col]);
            reinterpret_cast<bf16*>(a.out)[col] = f2bf(v);
        }
    }
    cp_async_wait<0>();
}

template <bool GLU, int NJ, int KS>
static int launch_stream_fast(const GemvArgs& a, int ppw, int ctas, size_t smem, cudaStream_t s) {
    static bool attr = false;
    if (!attr) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(gemv_stream_q4k_m1_kernel<GLU, 4, NJ, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr = true;
    }
    TSB_CHECK_CUDA(tsb_launch(gemv_stream_q4k_m1_kernel<GLU, 4, NJ, KS>, dim3(ctas), dim3(128), smem, s, a, ppw));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

template <bool GLU, int KS>
static int launch_stream_fast_nj(const GemvArgs& a, int nj, int ppw, int ctas, size_t smem, cudaStream_t s) {
    switch (nj) {
    case 1: return launch_stream_fast<GLU, 1, KS>(a, ppw, ctas, smem, s);
    case 2: return launch_stream_fast<GLU, 2, KS>(a, ppw, ctas, smem, s);
    case 3: return launch_stream_fast<GLU, 3, KS>(a, ppw, ctas, smem, s);
    default: return launch_stream_fast<GLU, 4, KS>(a, ppw, ctas, smem, s);
    }
}

// Single-token Q4_K: whole rows per warp up to 4096 values, rows split over the CTA's warps up to 16384.
static int launch_fast(const GemvArgs& a, bool glu, cudaStream_t s) {
    const int nb = a.w.K >> 8;
    const int ks = nb * 8 <= 128 ? 1 : 4;
    const int max_blocks = ks == 1 ? nb : (nb + ks - 1) / ks;
    const int nj = (max_blocks * 8 + 31) / 32;
    const size_t smem = (size_t)max_blocks * 144 * 4 * 4;               // 4 warps x ring of 4
    int per_sm = (int)((220 * 1024) / (smem + 1024));
    per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
    const int n_pairs = glu ? a.n_out : (a.w.N + 1) / 2;
    const int owners = 148 * per_sm * (ks == 1 ? 4 : 1);
    const int ppw = (n_pairs + owners - 1) / owners;
    const int ctas = ks == 1 ? (n_pairs + 4 * ppw - 1) / (4 * ppw) : (n_pairs + ppw - 1) / ppw;
    if (ks == 1) return glu ? launch_stream_fast_nj<true, 1>(a, nj, ppw, ctas, smem, s) : launch_stream_fast_nj<false, 1>(a, nj, ppw, ctas, smem, s);
    return glu ? launch_stream_fast_nj<true, 4>(a, nj, ppw, ctas, smem, s) : launch_stream_fast_nj<false, 4>(a, nj, ppw, ctas, smem, s);
}

template <int M, bool GLU, bool Q5, int D>
static int launch_stream(const GemvArgs& a, int ppw, int ctas, size_t smem, cudaStream_t s) {
    static bool attr = false;
    if (!attr) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(gemv_stream_kernel<M, GLU, Q5, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr = true;
    }
    TSB_CHECK_CUDA(tsb_launch(gemv_stream_kernel<M, GLU, Q5, D>, dim3(ctas), dim3(128), smem, s, a, ppw));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

template <bool GLU, bool Q5, int D>
static int launch_stream_m(const GemvArgs& a, int ppw, int ctas, size_t smem, cudaStream_t s) {
    if (a.M <= 1) return launch_stream<1, GLU, Q5, D>(a, ppw, ctas, smem, s);
    if (a.M <= 2) return launch_stream<2, GLU, Q5, D>(a, ppw, ctas, smem, s);
    return launch_stream<4, GLU, Q5, D>(a, ppw, ctas, smem, s);
}

// ---------------------------------------------------------------------------------------------
// Single-token Q6_K (the V projection, half of the down projections and the output matrix of a
// Q4_K_M file).  The weight lives in four planes (low nibbles, high bit pairs, int8 scales, half
// super-scales); a ring buffer holds the four row segments back to back.  A unit is 32 values
// (8 bytes of each of la / lb / hv), so that a quarter row splits evenly over a warp.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}

template <int NJ, int KS>
__global__ void __launch_bounds__(128) gemv_stream_q6k_m1_kernel(GemvArgs a, int ppw) {
    extern __shared__ uint4 stream_smem[];
    __shared__ float part[2][4];
    constexpr int D = 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = a.w.K, nb = K >> 8;
    // even block boundaries keep the 2-byte super-scales 4-byte aligned for cp.async
    const int bs = KS == 1 ? 0 : ((nb * warp) / KS) & ~1, be = KS == 1 ? nb : (warp == KS - 1 ? nb : ((nb * (warp + 1)) / KS) & ~1);
    const int nblk = be - bs;
    const int max_blocks = KS == 1 ? nb : ((nb + KS - 1) / KS + 2);
    const int stage_bytes = max_blocks * 208 + ((max_blocks * 2 + 15) & ~15);
    uint8_t* ring = reinterpret_cast<uint8_t*>(stream_smem) + (long)warp * D * stage_bytes;
    const int N = a.w.N;
    const int owner = KS == 1 ? blockIdx.x * 4 + warp : blockIdx.x;
    const int r0 = owner * ppw, r1 = min(N, r0 + ppw);
    const int ntask = r1 > r0 ? r1 - r0 : 0;
    const int off_qh = nblk * 128, off_sc = nblk * 192, off_d = nblk * 208;
    auto issue = [&](int i) {
        if (i < ntask) {
            const long blk0 = (long)(r0 + i) * nb + bs;
            uint8_t* dst = ring + (long)(i % D) * stage_bytes;
            const uint8_t* ql = a.w.p0 + blk0 * 128;
            const uint8_t* qh = a.w.p1 + blk0 * 64;
            const uint8_t* sc = a.w.p2 + blk0 * 16;
            const uint8_t* dd = a.w.p3 + blk0 * 2;
            for (int c = lane; c < nblk * 8; c += 32) cp_async16(dst + c * 16, ql + c * 16);
            for (int c = lane; c < nblk * 4; c += 32) cp_async16(dst + off_qh + c * 16, qh + c * 16);
            for (int c = lane; c < nblk; c += 32) cp_async16(dst + off_sc + c * 16, sc + c * 16);
            for (int c = lane; c < nblk / 2; c += 32) cp_async4(dst + off_d + c * 4, dd + c * 4);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < D - 1; ++i) issue(i);
    pdl_wait();
    pdl_trigger();

    const int units = nblk << 3;
    int xr[NJ][8], o_la[NJ], o_hv[NJ], o_sc[NJ], o_d[NJ];
    float xd[NJ][4];
    unsigned bsel[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int u = lane + 32 * j;
        const bool ok = u < units;
        const int uc = ok ? u : 0;
        const int bl = uc >> 3, b = bs + bl, rem = uc & 7, n = rem >> 2, h = (rem >> 1) & 1, hh = rem & 1;
        const int xoff = b * 256 + 128 * n + 16 * h + 8 * hh;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int2 xv = *reinterpret_cast<const int2*>(a.xq + xoff + 32 * k);
            xr[j][2 * k] = xv.x;
            xr[j][2 * k + 1] = xv.y;
            xd[j][k] = ok ? a.xds[b * 8 + 4 * n + k].x : 0.f;
        }
        o_la[j] = bl * 128 + 64 * n + 16 * h + 8 * hh;
        o_hv[j] = off_qh + bl * 64 + 32 * n + 16 * h + 8 * hh;
        o_sc[j] = off_sc + bl * 16 + 8 * n;
        o_d[j] = off_d + bl * 2;
        bsel[j] = 8u * h;                                 // scales of this unit: bytes h, h + 2, h + 4, h + 6 of the 8
    }

    for (int i = 0; i < ntask; ++i) {
        issue(i + D - 1);
        cp_async_wait<D - 1>();
        __syncwarp();
        const uint8_t* st = ring + (long)(i % D) * stage_bytes;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const uint2 la = *reinterpret_cast<const uint2*>(st + o_la[j]);
            const uint2 lb = *reinterpret_cast<const uint2*>(st + o_la[j] + 32);
            const uint2 hv = *reinterpret_cast<const uint2*>(st + o_hv[j]);
            const uint2 sc8 = *reinterpret_cast<const uint2*>(st + o_sc[j]);
            const float d = __half2float(*reinterpret_cast<const __half*>(st + o_d[j]));
            const uint32_t A[2] = {la.x, la.y}, B[2] = {lb.x, lb.y}, H[2] = {hv.x, hv.y};
            int t0 = 0, t1 = 0, t2 = 0, t3 = 0;
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                const int q0 = __vsub4((A[w] & 0x0F0F0F0Fu) | ((H[w] & 0x03030303u) << 4), 0x20202020u);
                const int q1 = __vsub4((B[w] & 0x0F0F0F0Fu) | (((H[w] >> 2) & 0x03030303u) << 4), 0x20202020u);
                const int q2 = __vsub4(((A[w] >> 4) & 0x0F0F0F0Fu) | (((H[w] >> 4) & 0x03030303u) << 4), 0x20202020u);
                const int q3 = __vsub4(((B[w] >> 4) & 0x0F0F0F0Fu) | (((H[w] >> 6) & 0x03030303u) << 4), 0x20202020u);
                t0 = __dp4a(q0, xr[j][w], t0);
                t1 = __dp4a(q1, xr[j][2 + w], t1);
                t2 = __dp4a(q2, xr[j][4 + w], t2);
                t3 = __dp4a(q3, xr[j][6 + w], t3);
            }
            // int8 scales: bytes h and h + 2 of the low word, h and h + 2 of the high word
            const int s0 = (int)(int8_t)(sc8.x >> bsel[j]), s1 = (int)(int8_t)(sc8.x >> (bsel[j] + 16u));
            const int s2 = (int)(int8_t)(sc8.y >> bsel[j]), s3 = (int)(int8_t)(sc8.y >> (bsel[j] + 16u));
            const float A4 = i2f_small(t0 * s0) * xd[j][0] + i2f_small(t1 * s1) * xd[j][1] + i2f_small(t2 * s2) * xd[j][2] +
                             i2f_small(t3 * s3) * xd[j][3];
            acc += d * A4;
        }
        acc = warp_sum(acc);
        __syncwarp();
        if (KS > 1) {
            if (lane == 0) part[i & 1][warp] = acc;
            __syncthreads();
            acc = part[i & 1][0] + part[i & 1][1] + part[i & 1][2] + part[i & 1][3];
            if (warp != 0) continue;
        }
        if (a.push != nullptr) {
            gemv_push_store(a.push, lane, r0 + i, (a.bias && a.push->rank == 0) ? acc + a.bias[r0 + i] : acc);
            continue;
        }
        if (lane != 0) continue;
        const int col = r0 + i;
        float v = acc;
        if (a.bias) v += a.bias[col];
        if (a.act == ACT_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
        if (a.row_scale) v *= a.row_scale[0];
        if (a.out_f32) {
            if (a.residual) v += reinterpret_cast<const float*>(a.residual)[col];
            reinterpret_cast<float*>(a.out)[col] = v;
        } else {
            if (a.residual) v += bf2f(reinterpret_cast<const bf16*>(a.residual)[col]);
            reinterpret_cast<bf16*>(a.out)[col] = f2bf(v);
        }
    }
    cp_async_wait<0>();
}

template <int NJ, int KS>
static int launch_q6k(const GemvArgs& a, int ppw, int ctas, size_t smem, cudaStream_t s) {
    static bool attr = false;
    if (!attr) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(gemv_stream_q6k_m1_kernel<NJ, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr = true;
    }
    TSB_CHECK_CUDA(tsb_launch(gemv_stream_q6k_m1_kernel<NJ, KS>, dim3(ctas), dim3(128), smem, s, a, ppw));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

static bool q6k_ok(const GemvArgs& a, bool glu) {
    const int nb = a.w.K >> 8;
    return a.w.type == TSB_Q6_K && !glu && a.M == 1 && nb >= 2 && nb % 2 == 0 && nb <= 64 && a.w.N >= 64;
}

static int launch_q6k_any(const GemvArgs& a, cudaStream_t s) {
    const int nb = a.w.K >> 8;
    const int ks = nb * 8 <= 128 ? 1 : 4;
    const int max_blocks = ks == 1 ? nb : ((nb + ks - 1) / ks + 2);
    const int nj = (max_blocks * 8 + 31) / 32;
    const size_t stage = (size_t)max_blocks * 208 + (((size_t)max_blocks * 2 + 15) & ~(size_t)15);
    const size_t smem = stage * 4 * 4;
    int per_sm = (int)((220 * 1024) / (smem + 1024));
    per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
    const int owners = 148 * per_sm * (ks == 1 ? 4 : 1);
    const int ppw = (a.w.N + owners - 1) / owners;
    const int ctas = ks == 1 ? (a.w.N + 4 * ppw - 1) / (4 * ppw) : (a.w.N + ppw - 1) / ppw;
#define TSB_Q6(NJV, KSV) return launch_q6k<NJV, KSV>(a, ppw, ctas, smem, s)
    if (ks == 1) { if (nj <= 1) TSB_Q6(1, 1); if (nj == 2) TSB_Q6(2, 1); if (nj == 3) TSB_Q6(3, 1); TSB_Q6(4, 1); }
    if (nj <= 2) TSB_Q6(2, 4); if (nj == 3) TSB_Q6(3, 4); if (nj == 4) TSB_Q6(4, 4); TSB_Q6(5, 4);
#undef TSB_Q6
}

// Whether the row pipeline takes this GEMV (called by tsb_gemv_push before the plain launch).  By default
// only the single-token Q4_K form runs here; the generic form (M <= 4, Q5_K, any row length) measured
// slower than the plain kernel inside the decode step and is kept behind TSB_GEMV_STREAM=2.
// TSB_GEMV_STREAM=0 turns the pipeline off altogether.
static int stream_mode() {
    static const int mode = []() { const char* e = getenv("TSB_GEMV_STREAM"); return e ? atoi(e) : 1; }();
    return mode;
}

static bool fast_ok(const GemvArgs& a) {
    const int nb = a.w.K >> 8;
    return a.w.type == TSB_Q4_K && a.M == 1 && nb >= 1 && nb * 8 <= 512 && a.w.N >= 64;
}

bool tsb_gemv_stream_eligible(const GemvArgs& a) {
    const int mode = stream_mode();
    if (!mode || a.ids || a.M > 4 || a.M < 1) return false;
    const bool glu = a.act >= ACT_SWIGLU && a.act <= ACT_SWIGLU_OAI;
    if (fast_ok(a) && !(glu && a.push)) return true;
    if (q6k_ok(a, glu)) return true;
    if (a.push || mode < 2 || (a.w.type != TSB_Q4_K && a.w.type != TSB_Q5_K)) return false;
    const size_t rowbytes = (size_t)(a.w.K >> 8) * (a.w.type == TSB_Q5_K ? 176 : 144);
    return rowbytes * 4 * 4 <= 200 * 1024 && a.w.N >= 64;           // four warps x four buffers must fit
}

int tsb_gemv_stream_launch(const GemvArgs& a, bool glu, cudaStream_t s) {
    if (fast_ok(a)) return launch_fast(a, glu, s);
    if (q6k_ok(a, glu)) return launch_q6k_any(a, s);
    const bool q5 = a.w.type == TSB_Q5_K;
    const size_t rowbytes = (size_t)(a.w.K >> 8) * (q5 ? 176 : 144);
    const size_t smem = rowbytes * 4 * 4;
    int per_sm = (int)((220 * 1024) / (smem + 1024));
    per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
    const int n_pairs = glu ? a.n_out : (a.w.N + 1) / 2;
    const int warps = 148 * per_sm * 4;
    const int ppw = (n_pairs + warps - 1) / warps;
    const int ctas = (n_pairs + 4 * ppw - 1) / (4 * ppw);
    if (glu) return q5 ? launch_stream_m<true, true, 4>(a, ppw, ctas, smem, s) : launch_stream_m<true, false, 4>(a, ppw, ctas, smem, s);
    return q5 ? launch_stream_m<false, true, 4>(a, ppw, ctas, smem, s) : launch_stream_m<false, false, 4>(a, ppw, ctas, smem, s);
}
