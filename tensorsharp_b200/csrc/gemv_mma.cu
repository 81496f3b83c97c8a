// Batched-decode GEMV (5 to 16 activation rows) for Q4_K weights on the tensor cores.
//
// The dp4a GEMV repeats its whole block arithmetic for every activation row: at 8 rows it spends about
// five times the instructions of the single-row case on the same weights (measured: 12.5 us per launch
// for the projections of a batch-8 decode step of a 35 B MoE model, 311 launches per step).  One
// Q4_K sub-block of 32 values is exactly the K of an int8 m16n8k32 MMA, its 4-bit codes are already
// valid int8 values (0..15, no table), and 8 activation rows are exactly the MMA's N: a warp gets
// 16 weight rows x 8 activation rows per sub-block from one instruction, and the 6-bit scale, the
// activation scale and the minimum term are applied to the 16 x 8 int32 result in the epilogue.
//
//   CTA (128 threads) = 16 output rows (for a gated pair: 16 gate rows + the matching 16 up rows);
//   its four warps take every fourth 64-value chunk of the rows and add up through shared memory,
//   so even a 2560-row projection is 160 CTAs.  Lane (g, t) loads the 4 bytes holding values
//   4t..4t+3 and 16+4t..16+4t+3 of a chunk's two sub-blocks (low / high nibbles) for rows g and g+8:
//   these words are the A fragments as they stand.
//
// Same contract as gemv_kernel without expert ids and without the tensor-parallel push.
// Replaces mul_mat_vec_q / mul_mat_q for small batches (ggml-cuda/mmvq.cu:143, mmq.cu) of the reference.
#include <cstdlib>
#include "gemv_core.cuh"

__device__ __forceinline__ void mma_s8(int (&c)[4], int a0, int a1, int a2, int a3, int b0, int b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float i2f_fast(int n) { return __int_as_float(0x4B400000 + n) - 12582912.f; }   // |n| < 2^22

// NT: n-tiles of 8 activation rows (1 or 2).
template <bool GLU, int NT>
__global__ void __launch_bounds__(128) gemv_mma_q4k_kernel(GemvArgs a) {
    constexpr int S = GLU ? 2 : 1;
    __shared__ float red[3][S * NT * 4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int K = a.w.K, nb = K >> 8, kb = K >> 5, n_out = a.n_out, M = a.M;
    const int r0 = blockIdx.x * 16;
    // weight rows of this lane, clamped at the edge (surplus rows are never stored)
    long wrow[S][2];
#pragma unroll
    for (int s = 0; s < S; ++s) {
        wrow[s][0] = (long)s * n_out + min(r0 + g, n_out - 1);
        wrow[s][1] = (long)s * n_out + min(r0 + g + 8, n_out - 1);
    }
    float acc[S][NT][4];
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[s][n][i] = 0.f;
    // activation rows this lane feeds (B fragment: column g of each n-tile) and reads scales for (columns 2t, 2t+1)
    const int8_t* xb_row[NT];
    bool xb_on[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        xb_on[n] = 8 * n + g < M;
        xb_row[n] = a.xq + (long)(xb_on[n] ? 8 * n + g : 0) * K + 4 * t;
    }
    pdl_wait();
    pdl_trigger();
    const int nchunks = nb * 4;
    for (int cc = warp; cc < nchunks; cc += 4) {
        const int b = cc >> 2, c = cc & 3;
        // ---- loads: code words and block headers of rows g, g + 8; activation words and scales
        uint32_t w0[S][2], w1[S][2];
        uint4 hdr[S][2];
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint8_t* blk = a.w.p0 + (wrow[s][h] * nb + b) * 144;
                hdr[s][h] = __ldg(reinterpret_cast<const uint4*>(blk));
                w0[s][h] = __ldg(reinterpret_cast<const uint32_t*>(blk + 16 + 32 * c + 4 * t));
                w1[s][h] = __ldg(reinterpret_cast<const uint32_t*>(blk + 16 + 32 * c + 16 + 4 * t));
            }
        int bl0[NT], bl1[NT], bh0[NT], bh1[NT];
        float2 e_lo[NT][2], e_hi[NT][2];
        const int sub = b * 8 + 2 * c;                   // 32-value group index of the low-nibble sub-block
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int8_t* xp = xb_row[n] + sub * 32;
            bl0[n] = xb_on[n] ? *reinterpret_cast<const int*>(xp) : 0;
            bl1[n] = xb_on[n] ? *reinterpret_cast<const int*>(xp + 16) : 0;
            bh0[n] = xb_on[n] ? *reinterpret_cast<const int*>(xp + 32) : 0;
            bh1[n] = xb_on[n] ? *reinterpret_cast<const int*>(xp + 48) : 0;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int col = 8 * n + 2 * t + j;
                const bool on = col < M;
                e_lo[n][j] = on ? a.xds[(long)col * kb + sub] : make_float2(0.f, 0.f);
                e_hi[n][j] = on ? a.xds[(long)col * kb + sub + 1] : make_float2(0.f, 0.f);
            }
        }
        // ---- arithmetic
#pragma unroll
        for (int s = 0; s < S; ++s) {
            float ds_lo[2], ds_hi[2], dm_lo[2], dm_hi[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                int sc0, sc1, mn0, mn1;
                k4_scales(hdr[s][h], c, sc0, sc1, mn0, mn1);
                const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr[s][h].x));
                ds_lo[h] = dd.x * (float)sc0; ds_hi[h] = dd.x * (float)sc1;
                dm_lo[h] = dd.y * (float)mn0; dm_hi[h] = dd.y * (float)mn1;
            }
            const int a_lo0 = (int)(w0[s][0] & 0x0F0F0F0Fu), a_lo1 = (int)(w0[s][1] & 0x0F0F0F0Fu);
            const int a_lo2 = (int)(w1[s][0] & 0x0F0F0F0Fu), a_lo3 = (int)(w1[s][1] & 0x0F0F0F0Fu);
            const int a_hi0 = (int)((w0[s][0] >> 4) & 0x0F0F0F0Fu), a_hi1 = (int)((w0[s][1] >> 4) & 0x0F0F0F0Fu);
            const int a_hi2 = (int)((w1[s][0] >> 4) & 0x0F0F0F0Fu), a_hi3 = (int)((w1[s][1] >> 4) & 0x0F0F0F0Fu);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
                mma_s8(cl, a_lo0, a_lo1, a_lo2, a_lo3, bl0[n], bl1[n]);
                mma_s8(ch, a_hi0, a_hi1, a_hi2, a_hi3, bh0[n], bh1[n]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int h = i >> 1, j = i & 1;     // row g + 8 h, column 2 t + j
                    acc[s][n][i] += ds_lo[h] * e_lo[n][j].x * i2f_fast(cl[i]) + ds_hi[h] * e_hi[n][j].x * i2f_fast(ch[i]) -
                                    dm_lo[h] * e_lo[n][j].y - dm_hi[h] * e_hi[n][j].y;
                }
            }
        }
    }
    // ---- the four warps hold partial sums over disjoint chunks: add them up in warp 0
    if (warp > 0) {
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) red[warp - 1][(s * NT + n) * 4 + i][lane] = acc[s][n][i];
    }
    __syncthreads();
    if (warp > 0) return;
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                acc[s][n][i] += red[0][(s * NT + n) * 4 + i][lane] + red[1][(s * NT + n) * 4 + i][lane] +
                                red[2][(s * NT + n) * 4 + i][lane];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + g + 8 * (i >> 1), col = 8 * n + 2 * t + (i & 1);
            if (r >= n_out || col >= M) continue;
            float v = acc[0][n][i];
            if (a.bias) v += a.bias[r];
            if (GLU) {
                float up = acc[S - 1][n][i];
                if (a.bias) up += a.bias[r + n_out];
                v = act_glu(a.act, v, up);
            } else if (a.act == ACT_RELU2) {
                v = fmaxf(v, 0.f);
                v = v * v;
            }
            if (a.row_scale) v *= a.row_scale[col];
            const long o = (long)col * n_out + r;
            if (a.out_f32) {
                if (a.residual) v += reinterpret_cast<const float*>(a.residual)[o];
                reinterpret_cast<float*>(a.out)[o] = v;
            } else {
                if (a.residual) v += bf2f(reinterpret_cast<const bf16*>(a.residual)[o]);
                reinterpret_cast<bf16*>(a.out)[o] = f2bf(v);
            }
        }
}

// TSB_GEMV_MMA=0 keeps the dp4a kernel for these batches.
bool tsb_gemv_mma_eligible(const GemvArgs& a) {
    static const int on = []() { const char* e = getenv("TSB_GEMV_MMA"); return e ? atoi(e) : 1; }();
    return on && a.w.type == TSB_Q4_K && !a.ids && !a.push && a.M >= 5 && a.M <= 16 && a.w.N >= 16;
}

int tsb_gemv_mma_launch(const GemvArgs& a, bool glu, cudaStream_t s) {
    const dim3 grid((a.n_out + 15) / 16), block(128);
    if (a.M <= 8) {
        if (glu) TSB_CHECK_CUDA(tsb_launch(gemv_mma_q4k_kernel<true, 1>, grid, block, 0, s, a));
        else TSB_CHECK_CUDA(tsb_launch(gemv_mma_q4k_kernel<false, 1>, grid, block, 0, s, a));
    } else {
        if (glu) TSB_CHECK_CUDA(tsb_launch(gemv_mma_q4k_kernel<true, 2>, grid, block, 0, s, a));
        else TSB_CHECK_CUDA(tsb_launch(gemv_mma_q4k_kernel<false, 2>, grid, block, 0, s, a));
    }
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}
