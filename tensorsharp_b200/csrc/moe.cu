// Mixture-of-experts routing and grouped expert projections that never leave the device, so a whole
// MoE layer is a fixed sequence of launches (CUDA-graph capturable) whatever the routing turns out
// to be:
//
//   moe_route_kernel    router logits -> top-k expert ids + weights (softmax over the selected k, or
//                       sigmoid + selection bias, optional renormalisation and scale)
//   moe_group_kernel    stable counting sort of the (token, slot) pairs by local expert; emits the
//                       sorted position of every pair, a list of tiles {expert, first row, rows} of
//                       at most 8 rows, and the tile count
//   moe_gather_kernel   activation rows (int8 groups + scales, or bf16) and routing weights into
//                       sorted order
//   gemv_tiles_kernel   weight-streaming projection of one tile: the expert's rows are streamed once
//                       for up to 8 activation rows; grid.y is a host-side upper bound on the tile
//                       count, surplus CTAs leave at once
//   moe_combine_kernel  out[t] = sum over the token's slots of the sorted result rows
//
// Replaces in the reference: topk_moe / argsort + mm_ids_helper (ggml-cuda/topk-moe.cu,
// mmid.cu), ggml_cuda_mul_mat_id and the host-side routing loops of GptOssModel.cs:814-865,
// Qwen35Model.cs:1931-2402 and NemotronModel.cs:822-856, which read the router output back to the
// host for every layer.
#include <cstdlib>
#include "gemv_core.cuh"

#define MOE_TILE_ROWS 8
#define MOE_MAX_E 1024
#define MOE_MAX_K 16

// ---------------------------------------------------------------------------------------------
// Router: one warp per token.
// mode 0: top-k of the logits, weights = softmax over the selected logits.
// mode 1: p = sigmoid(logit); select on p + sel_bias; weights = p, optionally / max(sum, 6.1e-5); * scale.
// ---------------------------------------------------------------------------------------------
template <int PER>
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ sel_bias,
                                                        int T, int E, int k, int mode, int normalize, float scale,
                                                        int* __restrict__ ids, float* __restrict__ wts) {
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    pdl_trigger();
    if (t >= T) return;
    float sel[PER], val[PER];                   // PER = ceil(E / 32) rounded up to an instantiated size
    const float* row = logits + (long)t * E;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        if (e < E) {
            const float x = row[e];
            if (mode == 1) {
                const float p = 1.f / (1.f + __expf(-x));
                val[i] = p;
                sel[i] = sel_bias ? p + sel_bias[e] : p;
            } else {
                val[i] = x;
                sel[i] = x;
            }
        } else {
            val[i] = 0.f;
            sel[i] = -INFINITY;
        }
    }
    float wk = 0.f;                       // lane j keeps the j-th selected weight
    int ik = 0;
    for (int j = 0; j < k; ++j) {
        // warp arg-max, ties to the lower expert index (the order torch.topk and the reference's sort give)
        float best = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * 32 + lane;
            if (sel[i] > best || (sel[i] == best && e < bi)) { best = sel[i]; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        // the owner lane hands over the value and retires the entry
        float v = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (i * 32 + lane == bi) { v = val[i]; sel[i] = -INFINITY; }
        v = __shfl_sync(0xffffffffu, v, bi & 31);
        if (lane == j) { wk = v; ik = bi; }
    }
    const bool on = lane < k;
    if (mode == 0) {
        const float m = warp_max(on ? wk : -INFINITY);
        const float ex = on ? __expf(wk - m) : 0.f;
        const float s = warp_sum(ex);
        wk = ex / s;
    } else {
        if (normalize) {
            const float s = warp_sum(on ? wk : 0.f);
            wk = wk / fmaxf(s, 6.103515625e-5f);
        }
        wk *= scale;
    }
    if (on) {
        ids[(long)t * k + lane] = ik;
        wts[(long)t * k + lane] = wk;
    }
}

extern "C" int tsb_moe_route(const float* logits, const float* sel_bias, int T, int E, int k, int mode, int normalize,
                             float scale, int* ids, float* wts, void* stream) {
    TSB_CHECK_ARG(E > 0 && E <= MOE_MAX_E, "moe_route: %d experts (limit %d)", E, MOE_MAX_E);
    TSB_CHECK_ARG(k > 0 && k <= MOE_MAX_K && k <= E, "moe_route: top-%d of %d", k, E);
    if (T == 0) return TSB_OK;
    const dim3 grid((T + 3) / 4), block(128);
    cudaStream_t st = (cudaStream_t)stream;
#define TSB_ROUTE(P) TSB_CHECK_CUDA(tsb_launch(moe_route_kernel<P>, grid, block, 0, st, logits, sel_bias, T, E, k, mode, normalize, scale, ids, wts))
    if (E <= 32) TSB_ROUTE(1);
    else if (E <= 128) TSB_ROUTE(4);
    else if (E <= 256) TSB_ROUTE(8);
    else TSB_ROUTE(MOE_MAX_E / 32);
#undef TSB_ROUTE
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ---------------------------------------------------------------------------------------------
// Grouping: one CTA.  Thread e owns local expert e and walks the id list in order, so positions
// inside an expert keep the original (token, slot) order: the sort is stable and deterministic.
// meta[0] = tile count, meta[1] = rows held by local experts.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ ids, int P, int e0, int E_local,
                                                         int* __restrict__ pos, int4* __restrict__ tiles, int* __restrict__ meta) {
    extern __shared__ int sm[];
    int* sid = sm;                         // [P] local expert or -1
    int* cnt = sm + P;                     // [E_local + 1]
    int* toff = cnt + E_local + 1;         // [E_local + 1]
    pdl_wait();
    pdl_trigger();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p] - e0;
        sid[p] = (e >= 0 && e < E_local) ? e : -1;
        pos[p] = -1;
    }
    __syncthreads();
    const int e = threadIdx.x;
    int c = 0;
    if (e < E_local)
        for (int p = 0; p < P; ++p) c += sid[p] == e;
    if (e < E_local) cnt[e] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int rows = 0, nt = 0;
        for (int i = 0; i < E_local; ++i) {
            const int ci = cnt[i];
            cnt[i] = rows;
            toff[i] = nt;
            rows += ci;
            nt += (ci + MOE_TILE_ROWS - 1) / MOE_TILE_ROWS;
        }
        cnt[E_local] = rows;
        toff[E_local] = nt;
        meta[0] = nt;
        meta[1] = rows;
    }
    __syncthreads();
    if (e < E_local) {
        const int start = cnt[e];
        int n = 0;
        for (int p = 0; p < P; ++p)
            if (sid[p] == e) pos[p] = start + n++;
        int ti = toff[e];
        for (int r = 0; r < n; r += MOE_TILE_ROWS) tiles[ti++] = make_int4(e, start + r, min(MOE_TILE_ROWS, n - r), 0);
    }
}

extern "C" int tsb_moe_group(const int* ids, int P, int e0, int E_local, int* pos, void* tiles, int* meta, void* stream) {
    TSB_CHECK_ARG(E_local > 0 && E_local <= 1024, "moe_group: %d local experts (limit 1024)", E_local);
    const size_t smem = sizeof(int) * ((size_t)P + 2 * (E_local + 1));
    TSB_CHECK_ARG(smem <= 200 * 1024, "moe_group: %d routed pairs do not fit one CTA's shared memory", P);
    if (P == 0) return TSB_OK;
    static bool attr = false;
    if (!attr) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(moe_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr = true;
    }
    TSB_CHECK_CUDA(tsb_launch(moe_group_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, ids, P, e0, E_local, pos,
                              (int4*)tiles, meta));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// Upper bound on the tile count for P routed pairs over E_local experts (the grid.y of the tile GEMV).
extern "C" int tsb_moe_max_tiles(int P, int E_local) {
    const int full = P / MOE_TILE_ROWS;
    return full + (E_local < P ? E_local : P);
}

// ---------------------------------------------------------------------------------------------
// Gather into sorted order.  One warp per routed pair; 16-byte copies.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_gather_kernel(const int* __restrict__ pos, int P, int x_div, int K,
                                                         const int8_t* __restrict__ xq, const float2* __restrict__ xds,
                                                         const bf16* __restrict__ xb, const float* __restrict__ w,
                                                         int8_t* __restrict__ sq, float2* __restrict__ sds, bf16* __restrict__ sb,
                                                         float* __restrict__ sw) {
    const int p = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    pdl_trigger();
    if (p >= P) return;
    const int d = pos[p];
    if (d < 0) return;
    const long src = p / x_div;
    if (xq) {
        const uint4* s = reinterpret_cast<const uint4*>(xq + src * K);
        uint4* o = reinterpret_cast<uint4*>(sq + (long)d * K);
        for (int i = lane; i < K / 16; i += 32) o[i] = s[i];
        const int kb = K >> 5;
        for (int i = lane; i < kb; i += 32) sds[(long)d * kb + i] = xds[src * kb + i];
    }
    if (xb) {
        const uint4* s = reinterpret_cast<const uint4*>(xb + src * K);
        uint4* o = reinterpret_cast<uint4*>(sb + (long)d * K);
        for (int i = lane; i < K / 8; i += 32) o[i] = s[i];
    }
    if (w && lane == 0) sw[d] = w[p];
}

extern "C" int tsb_moe_gather(const int* pos, int P, int x_div, int K, const void* xq, const void* xds, const void* xb,
                              const float* w, void* sq, void* sds, void* sb, float* sw, void* stream) {
    TSB_CHECK_ARG(K % 32 == 0 && x_div > 0, "moe_gather: K=%d x_div=%d", K, x_div);
    if (P == 0) return TSB_OK;
    TSB_CHECK_CUDA(tsb_launch(moe_gather_kernel, dim3((P + 7) / 8), dim3(256), 0, (cudaStream_t)stream, pos, P, x_div, K,
                              (const int8_t*)xq, (const float2*)xds, (const bf16*)xb, w, (int8_t*)sq, (float2*)sds, (bf16*)sb, sw));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ---------------------------------------------------------------------------------------------
// Tile GEMV: CTA (x, y) computes four output rows (one per warp) of tile y.
// ---------------------------------------------------------------------------------------------
struct TileArgs {
    QW w;
    const int8_t* xq;
    const float2* xds;
    const bf16* xb;
    void* out;               // [rows, n_out] in sorted order
    const float* bias;       // [E_local, N] or null
    const float* row_scale;  // [rows] in sorted order or null
    const int4* tiles;
    const int* meta;
    int out_f32, act, n_out;
};

template <bool GLU>
__global__ void __launch_bounds__(128) gemv_tiles_kernel(TileArgs a) {
    constexpr int M = MOE_TILE_ROWS;
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    pdl_wait();
    pdl_trigger();
    if ((int)blockIdx.y >= a.meta[0] || r >= a.n_out) return;
    const int4 t = a.tiles[blockIdx.y];
    const int expert = t.x, row0 = t.y, mv = t.z;
    const int K = a.w.K, kb = K >> 5;
    const int8_t* xq = a.xq ? a.xq + (long)row0 * K : nullptr;
    const float2* xds = a.xds ? a.xds + (long)row0 * kb : nullptr;
    const bf16* xb = a.xb ? a.xb + (long)row0 * K : nullptr;
    const long wrow = (long)expert * a.w.N + r;
    float acc[M], acc2[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { acc[m] = 0.f; acc2[m] = 0.f; }
    dot_row<M>(a.w, wrow, lane, xq, xds, xb, acc, mv, PdlWait{false});
    if (GLU) dot_row<M>(a.w, wrow + a.n_out, lane, xq, xds, xb, acc2, mv, PdlWait{false});
#pragma unroll
    for (int m = 0; m < M; ++m) {
        acc[m] = warp_sum(acc[m]);
        if (GLU) acc2[m] = warp_sum(acc2[m]);
    }
    if (lane != 0) return;
#pragma unroll
    for (int m = 0; m < M; ++m) {
        if (m >= mv) break;
        float v = acc[m];
        if (a.bias) v += a.bias[(long)expert * a.w.N + r];
        if (GLU) {
            float u = acc2[m];
            if (a.bias) u += a.bias[(long)expert * a.w.N + r + a.n_out];
            v = act_glu(a.act, v, u);
        } else if (a.act == ACT_RELU2) {
            v = fmaxf(v, 0.f);
            v = v * v;
        } else if (a.act == ACT_SILU) {
            v = v / (1.f + __expf(-v));
        }
        if (a.row_scale) v *= a.row_scale[row0 + m];
        const long o = (long)(row0 + m) * a.n_out + r;
        if (a.out_f32) reinterpret_cast<float*>(a.out)[o] = v;
        else reinterpret_cast<bf16*>(a.out)[o] = f2bf(v);
    }
}

// ---------------------------------------------------------------------------------------------
// Tensor-core tile GEMV for 4-bit blocks of 32 (MXFP4, Q4_0).  The 8 activation rows of a tile are
// exactly the N of an int8 m16n8k32 MMA and one quant block is exactly its K, so a warp computes
// 16 output rows x 8 pairs per block with one instruction: A = the block's codes decoded to int8
// (lane (g, t) loads the 4 bytes that hold elements 4t..4t+3 and 16+4t..16+4t+3 of rows g and g+8,
// which is the A fragment as it stands), B = the int8 activations, and the int32 result is scaled by
// weight scale x activation scale into float accumulators.  Activations are read once per 16 rows
// instead of once per row, which is what bounds the dp4a version at 8 rows per tile.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_s8_16x8x32(int (&c)[4], const int (&a)[4], int b0, int b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool MX>
__device__ __forceinline__ void decode_q4_words(uint32_t wg, uint32_t wg8, int (&a)[4]) {
    if (MX) {
        mxfp4_decode8(wg, a[0], a[2]);
        mxfp4_decode8(wg8, a[1], a[3]);
    } else {
        a[0] = (int)__vsub4(wg & 0x0F0F0F0Fu, 0x08080808u);
        a[1] = (int)__vsub4(wg8 & 0x0F0F0F0Fu, 0x08080808u);
        a[2] = (int)__vsub4((wg >> 4) & 0x0F0F0F0Fu, 0x08080808u);
        a[3] = (int)__vsub4((wg8 >> 4) & 0x0F0F0F0Fu, 0x08080808u);
    }
}

template <bool MX>
__device__ __forceinline__ float q4_block_scale(const QW& w, long row, int kb, int u) {
    if (MX) return e8m0_half_scale(w.p1[row * kb + u]);
    return __half2float(reinterpret_cast<const __half*>(w.p1)[row * kb + u]);
}

#ifndef MOE_MMA_BLOCKS_IN_FLIGHT
#define MOE_MMA_BLOCKS_IN_FLIGHT 2
#endif

template <bool GLU, bool MX>
__global__ void __launch_bounds__(128) gemv_tiles_mma_kernel(TileArgs a) {
    constexpr int S = GLU ? 2 : 1;               // weight row sets per warp: gate (+ up)
    constexpr int U = MOE_MMA_BLOCKS_IN_FLIGHT;    // k-blocks in flight per iteration
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int r0 = (blockIdx.x * 4 + (threadIdx.x >> 5)) * 16;
    pdl_wait();
    pdl_trigger();
    if ((int)blockIdx.y >= a.meta[0] || r0 >= a.n_out) return;
    const int4 tile = a.tiles[blockIdx.y];
    const int expert = tile.x, row0 = tile.y, mv = tile.z;
    const int K = a.w.K, kb = K >> 5;
    // weight rows of this lane (clamped at the edge; surplus rows are never stored)
    long wr[S][2];
#pragma unroll
    for (int s = 0; s < S; ++s) {
        wr[s][0] = (long)expert * a.w.N + s * a.n_out + min(r0 + g, a.n_out - 1);
        wr[s][1] = (long)expert * a.w.N + s * a.n_out + min(r0 + g + 8, a.n_out - 1);
    }
    const bool bact = g < mv;
    const int8_t* xrow = a.xq + (long)(row0 + (bact ? g : 0)) * K + 4 * t;
    const int c0 = 2 * t, c1 = 2 * t + 1;
    const float2* xs0 = a.xds + (long)(row0 + (c0 < mv ? c0 : 0)) * kb;
    const float2* xs1 = a.xds + (long)(row0 + (c1 < mv ? c1 : 0)) * kb;
    float acc[S][4];
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[s][i] = 0.f;
    for (int u0 = 0; u0 < kb; u0 += U) {
        uint32_t wq[U][S][2];
        float ws[U][S][2];
        int b0[U], b1[U];
        float xd0[U], xd1[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int u = min(u0 + j, kb - 1);
#pragma unroll
            for (int s = 0; s < S; ++s)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    wq[j][s][h] = __ldg(reinterpret_cast<const uint32_t*>(a.w.p0 + wr[s][h] * (K >> 1) + u * 16 + 4 * t));
                    ws[j][s][h] = q4_block_scale<MX>(a.w, wr[s][h], kb, u);
                }
            b0[j] = bact ? *reinterpret_cast<const int*>(xrow + u * 32) : 0;
            b1[j] = bact ? *reinterpret_cast<const int*>(xrow + u * 32 + 16) : 0;
            xd0[j] = xs0[u].x;
            xd1[j] = xs1[u].x;
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (u0 + j >= kb) break;
#pragma unroll
            for (int s = 0; s < S; ++s) {
                int af[4], c[4] = {0, 0, 0, 0};
                decode_q4_words<MX>(wq[j][s][0], wq[j][s][1], af);
                mma_s8_16x8x32(c, af, b0[j], b1[j]);
                acc[s][0] += ws[j][s][0] * xd0[j] * (float)c[0];
                acc[s][1] += ws[j][s][0] * xd1[j] * (float)c[1];
                acc[s][2] += ws[j][s][1] * xd0[j] * (float)c[2];
                acc[s][3] += ws[j][s][1] * xd1[j] * (float)c[3];
            }
        }
    }
    // thread (g, t) holds rows r0 + g, r0 + g + 8 for pairs 2t, 2t + 1
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + g + (i >> 1) * 8, col = 2 * t + (i & 1);
        if (r >= a.n_out || col >= mv) continue;
        float v = acc[0][i];
        if (a.bias) v += a.bias[(long)expert * a.w.N + r];
        if (GLU) {
            float up = acc[S - 1][i];
            if (a.bias) up += a.bias[(long)expert * a.w.N + r + a.n_out];
            v = act_glu(a.act, v, up);
        } else if (a.act == ACT_RELU2) {
            v = fmaxf(v, 0.f);
            v = v * v;
        } else if (a.act == ACT_SILU) {
            v = v / (1.f + __expf(-v));
        }
        if (a.row_scale) v *= a.row_scale[row0 + col];
        const long o = (long)(row0 + col) * a.n_out + r;
        if (a.out_f32) reinterpret_cast<float*>(a.out)[o] = v;
        else reinterpret_cast<bf16*>(a.out)[o] = f2bf(v);
    }
}

// The same tile GEMV with 8-byte weight loads.  In the kernel above a lane reads 4 bytes per block and row, so a warp
// has about 1 KB of weights in flight and every request uses half a sector; at four CTAs per SM that is a third of the
// bytes in flight the memory system needs.  Here lane t of a row's four lanes reads half (t & 1) of block ub + (t >> 1):
// one request covers two whole blocks (a full sector), twice the bytes in flight for the same registers, and the word a
// lane needs for a block's MMA fragment (word t) comes from lane 2q + (t >> 1) by shuffle.  The scales of a block pair
// are one 2-byte (MXFP4) or 4-byte (Q4_0) load.  Needs an even number of blocks per row.
template <bool GLU, bool MX>
__global__ void __launch_bounds__(128) gemv_tiles_mma_wide_kernel(TileArgs a) {
    constexpr int S = GLU ? 2 : 1;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int r0 = (blockIdx.x * 4 + (threadIdx.x >> 5)) * 16;
    pdl_wait();
    pdl_trigger();
    if ((int)blockIdx.y >= a.meta[0] || r0 >= a.n_out) return;
    const int4 tile = a.tiles[blockIdx.y];
    const int expert = tile.x, row0 = tile.y, mv = tile.z;
    const int K = a.w.K, kb = K >> 5;
    long wr[S][2];
#pragma unroll
    for (int s = 0; s < S; ++s) {
        wr[s][0] = (long)expert * a.w.N + s * a.n_out + min(r0 + g, a.n_out - 1);
        wr[s][1] = (long)expert * a.w.N + s * a.n_out + min(r0 + g + 8, a.n_out - 1);
    }
    const bool bact = g < mv;
    const int8_t* xrow = a.xq + (long)(row0 + (bact ? g : 0)) * K + 4 * t;
    const int c0 = 2 * t, c1 = 2 * t + 1;
    const float2* xs0 = a.xds + (long)(row0 + (c0 < mv ? c0 : 0)) * kb;
    const float2* xs1 = a.xds + (long)(row0 + (c1 < mv ? c1 : 0)) * kb;
    const int src_base = lane & ~3;
    float acc[S][4];
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[s][i] = 0.f;
    for (int u0 = 0; u0 < kb; u0 += 4) {
        uint2 wv[2][S][2];
        uint32_t sc[2][S][2];
        int b0[4], b1[4];
        float xd0[4], xd1[4];
#pragma unroll
        for (int P = 0; P < 2; ++P) {
            const int ub = min(u0 + 2 * P, kb - 2);                 // (a pair past the end re-reads the last one; not used)
#pragma unroll
            for (int s = 0; s < S; ++s)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    wv[P][s][h] = __ldg(reinterpret_cast<const uint2*>(a.w.p0 + wr[s][h] * (K >> 1) + (ub + (t >> 1)) * 16 + (t & 1) * 8));
                    if (MX) sc[P][s][h] = __ldg(reinterpret_cast<const unsigned short*>(a.w.p1 + wr[s][h] * kb + ub));
                    else sc[P][s][h] = __ldg(reinterpret_cast<const uint32_t*>(a.w.p1 + 2 * (wr[s][h] * kb + ub)));
                }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int u = min(u0 + j, kb - 1);
            b0[j] = bact ? *reinterpret_cast<const int*>(xrow + u * 32) : 0;
            b1[j] = bact ? *reinterpret_cast<const int*>(xrow + u * 32 + 16) : 0;
            xd0[j] = xs0[u].x;
            xd1[j] = xs1[u].x;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int P = j >> 1, q = j & 1;
            const bool live = u0 + j < kb;                          // uniform over the warp
            const int src = src_base | (2 * q + (t >> 1));
#pragma unroll
            for (int s = 0; s < S; ++s) {
                uint32_t wd[2];
                float ws[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t x = __shfl_sync(0xffffffffu, wv[P][s][h].x, src), y = __shfl_sync(0xffffffffu, wv[P][s][h].y, src);
                    wd[h] = (t & 1) ? y : x;
                    if (MX) ws[h] = e8m0_half_scale((uint8_t)(sc[P][s][h] >> (8 * q)));
                    else ws[h] = __half2float(__ushort_as_half((unsigned short)(sc[P][s][h] >> (16 * q))));
                }
                if (live) {
                    int af[4], c[4] = {0, 0, 0, 0};
                    decode_q4_words<MX>(wd[0], wd[1], af);
                    mma_s8_16x8x32(c, af, b0[j], b1[j]);
                    acc[s][0] += ws[0] * xd0[j] * (float)c[0];
                    acc[s][1] += ws[0] * xd1[j] * (float)c[1];
                    acc[s][2] += ws[1] * xd0[j] * (float)c[2];
                    acc[s][3] += ws[1] * xd1[j] * (float)c[3];
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + g + (i >> 1) * 8, col = 2 * t + (i & 1);
        if (r >= a.n_out || col >= mv) continue;
        float v = acc[0][i];
        if (a.bias) v += a.bias[(long)expert * a.w.N + r];
        if (GLU) {
            float up = acc[S - 1][i];
            if (a.bias) up += a.bias[(long)expert * a.w.N + r + a.n_out];
            v = act_glu(a.act, v, up);
        } else if (a.act == ACT_RELU2) {
            v = fmaxf(v, 0.f);
            v = v * v;
        } else if (a.act == ACT_SILU) {
            v = v / (1.f + __expf(-v));
        }
        if (a.row_scale) v *= a.row_scale[row0 + col];
        const long o = (long)(row0 + col) * a.n_out + r;
        if (a.out_f32) reinterpret_cast<float*>(a.out)[o] = v;
        else reinterpret_cast<bf16*>(a.out)[o] = f2bf(v);
    }
}

extern "C" int tsb_moe_gemv_tiles(const void* p0, const void* p1, const void* p2, const void* p3, int type, int N, int K,
                                  const void* xq, const void* xds, const void* xb, void* out, const float* bias,
                                  const float* row_scale, const void* tiles, const int* meta, int max_tiles, int out_f32,
                                  int act, void* stream) {
    TSB_CHECK_ARG(N > 0 && K > 0 && max_tiles >= 0, "moe_gemv_tiles: bad shape N=%d K=%d tiles=%d", N, K, max_tiles);
    const bool q8 = type == TSB_Q4_K || type == TSB_Q5_K || type == TSB_Q6_K || type == TSB_Q8_0 || type == TSB_MXFP4 ||
                    type == TSB_Q4_0;
    TSB_CHECK_ARG(!q8 || (xq && xds), "moe_gemv_tiles: quantised weight type %d needs int8 activations", type);
    TSB_CHECK_ARG(q8 || xb, "moe_gemv_tiles: float weight type %d needs bf16 activations", type);
    const bool kq = type == TSB_Q4_K || type == TSB_Q5_K || type == TSB_Q6_K;
    TSB_CHECK_ARG(K % (kq ? 256 : 32) == 0, "moe_gemv_tiles: K=%d not a whole number of blocks for type %d", K, type);
    const bool glu = act >= ACT_SWIGLU && act <= ACT_SWIGLU_OAI;
    TSB_CHECK_ARG(!glu || N % 2 == 0, "moe_gemv_tiles: GLU needs an even row count, got %d", N);
    TSB_CHECK_ARG(max_tiles <= 65535, "moe_gemv_tiles: %d tiles exceed the grid limit", max_tiles);
    if (max_tiles == 0) return TSB_OK;
    TileArgs a;
    a.w = QW{(const uint8_t*)p0, (const uint8_t*)p1, (const uint8_t*)p2, (const uint8_t*)p3, type, N, K};
    a.xq = (const int8_t*)xq; a.xds = (const float2*)xds; a.xb = (const bf16*)xb;
    a.out = out; a.bias = bias; a.row_scale = row_scale; a.tiles = (const int4*)tiles; a.meta = meta;
    a.out_f32 = out_f32; a.act = act; a.n_out = glu ? N / 2 : N;
    static const bool use_mma = []() { const char* e = getenv("TSB_MOE_MMA"); return !e || atoi(e) != 0; }();
    if (use_mma && (type == TSB_MXFP4 || type == TSB_Q4_0)) {
        dim3 grid((a.n_out + 63) / 64, max_tiles), block(128);
        cudaStream_t st = (cudaStream_t)stream;
        static const bool wide_loads = []() { const char* e = getenv("TSB_MOE_WIDE_LOADS"); return !e || atoi(e) != 0; }();
        if (wide_loads && (K >> 5) % 2 == 0 && (K >> 5) >= 2) {
            if (type == TSB_MXFP4) {
                if (glu) TSB_CHECK_CUDA(tsb_launch(gemv_tiles_mma_wide_kernel<true, true>, grid, block, 0, st, a));
                else TSB_CHECK_CUDA(tsb_launch(gemv_tiles_mma_wide_kernel<false, true>, grid, block, 0, st, a));
            } else {
                if (glu) TSB_CHECK_CUDA(tsb_launch(gemv_tiles_mma_wide_kernel<true, false>, grid, block, 0, st, a));
                else TSB_CHECK_CUDA(tsb_launch(gemv_tiles_mma_wide_kernel<false, false>, grid, block, 0, st, a));
            }
            TSB_CHECK_LAUNCH();
            return TSB_OK;
        }
        if (type == TSB_MXFP4) {
            if (glu) TSB_CHECK_CUDA(tsb_launch(gemv_tiles_mma_kernel<true, true>, grid, block, 0, st, a));
            else TSB_CHECK_CUDA(tsb_launch(gemv_tiles_mma_kernel<false, true>, grid, block, 0, st, a));
        } else {
            if (glu) TSB_CHECK_CUDA(tsb_launch(gemv_tiles_mma_kernel<true, false>, grid, block, 0, st, a));
            else TSB_CHECK_CUDA(tsb_launch(gemv_tiles_mma_kernel<false, false>, grid, block, 0, st, a));
        }
        TSB_CHECK_LAUNCH();
        return TSB_OK;
    }
    dim3 grid((a.n_out + 3) / 4, max_tiles), block(128);
    if (glu) TSB_CHECK_CUDA(tsb_launch(gemv_tiles_kernel<true>, grid, block, 0, (cudaStream_t)stream, a));
    else TSB_CHECK_CUDA(tsb_launch(gemv_tiles_kernel<false>, grid, block, 0, (cudaStream_t)stream, a));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ---------------------------------------------------------------------------------------------
// Combine: out[t, :] = sum_j w[t * k + j] * y[pos[t * k + j], :]  (pairs held by other ranks have pos < 0; w null = 1).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos,
                                                          const float* __restrict__ w, int k, int D, float* __restrict__ out) {
    const int t = blockIdx.x;
    pdl_wait();
    pdl_trigger();
    for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < k; ++j) {
            const int p = pos[t * k + j];
            if (p < 0) continue;
            const float4 v = *reinterpret_cast<const float4*>(y + (long)p * D + c);
            const float wj = w ? w[t * k + j] : 1.f;
            s.x += wj * v.x; s.y += wj * v.y; s.z += wj * v.z; s.w += wj * v.w;
        }
        *reinterpret_cast<float4*>(out + (long)t * D + c) = s;
    }
}

extern "C" int tsb_moe_combine(const float* y, const int* pos, int T, int k, int D, float* out, void* stream) {
    TSB_CHECK_ARG(D % 4 == 0, "moe_combine: D=%d is not a multiple of 4", D);
    if (T == 0) return TSB_OK;
    TSB_CHECK_CUDA(tsb_launch(moe_combine_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, y, pos, (const float*)nullptr, k, D, out));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// The same with a weight per (token, slot), for projections that did not scale their rows themselves.
extern "C" int tsb_moe_combine_weighted(const float* y, const int* pos, const float* w, int T, int k, int D, float* out, void* stream) {
    TSB_CHECK_ARG(D % 4 == 0 && y && pos && w && out, "moe_combine_weighted: D=%d or a null argument", D);
    if (T == 0) return TSB_OK;
    TSB_CHECK_CUDA(tsb_launch(moe_combine_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, y, pos, w, k, D, out));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}
