// Decode attention on the bf16 tensor cores: the query heads that share a KV head (up to 16) are the rows of one m16
// tile, so Q K^T and P V of a 32-key chunk are 2 x 32 mma.sync m16n8k16 instead of the thousand multiply-adds per lane
// the CUDA-core kernels (attention.cu: attn_decode_body) spend on it.  Serves head sizes 64 and 128, one sequence or a
// batch; the CUDA-core kernels keep the other shapes.  Measured on the Qwen3-4B shape at context 2048: one sequence 12.0
// -> 5.3 us per launch inside the decode step, 16 sequences 77.9 -> 40.0 us (51 % of the measured copy rate).
//
// grid (splits, Hkv, B), 128 threads.  Each warp walks its own 32-key chunks of the split (stride 128 keys): the chunk's
// K and V rows come through cp.async into the warp's own swizzled tiles, ldmatrix feeds the fragments, the online
// softmax runs in registers on the accumulator layout (two rows per lane), P goes back in as the A operand of P V.
// The four warps' partial results are merged through shared memory and written as this split's partial; the combine
// kernel of attention.cu finishes (sinks, normalisation, int8 form).
//
// Replaces in the reference: flash_attn_ext_vec (ggml-cuda/fattn-vec.cuh:21).
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "attn_args.cuh"
#include "attn_mma.cuh"
#include "common.cuh"

namespace cg = cooperative_groups;

// The e4m3 cache (FP8 = true): the tiles hold half values (the hardware converts two e4m3 bytes to a half pair in one
// instruction, exactly), the query rows are converted from bf16 to half as they are staged, and the products are the
// f16 form of the same mma.  K / V pieces are fetched with plain 16-byte loads (16 values each), all of a chunk's
// requests issued before the first conversion.
__device__ __forceinline__ void mma_f16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t e4m3x2_to_half2(uint32_t two_bytes) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two_bytes, __NV_E4M3);
    return (uint32_t)h.x | ((uint32_t)h.y << 16);
}
// 16 e4m3 bytes -> two 16-byte pieces of 8 halves each
__device__ __forceinline__ void e4m3x16_to_half(const uint4& raw, uint4& lo, uint4& hi) {
    lo.x = e4m3x2_to_half2(raw.x & 0xffffu); lo.y = e4m3x2_to_half2(raw.x >> 16);
    lo.z = e4m3x2_to_half2(raw.y & 0xffffu); lo.w = e4m3x2_to_half2(raw.y >> 16);
    hi.x = e4m3x2_to_half2(raw.z & 0xffffu); hi.y = e4m3x2_to_half2(raw.z >> 16);
    hi.z = e4m3x2_to_half2(raw.w & 0xffffu); hi.w = e4m3x2_to_half2(raw.w >> 16);
}

// CS > 0: the CS splits of a (sequence, KV head) are one thread-block cluster, and instead of writing partials for a
// second kernel every CTA leaves its partial in its own shared memory, the cluster synchronises, and each CTA reads the
// others' partials through distributed shared memory to finish 1 / CS of the group's output columns (sinks,
// normalisation, bf16 and int8 forms: the arithmetic of attn_combine_kernel).  No CTA returns before the second
// cluster barrier, so no shared memory disappears under a reader.
template <int DH, int CS, bool FP8 = false>
__global__ void __launch_bounds__(128) attn_decode_mma_kernel(AttnArgs a) {
    constexpr int CH = DH / 8;                     // 16-byte pieces per row
    constexpr int KT = 32;                         // keys per chunk
    constexpr float LOG2E = 1.4426950408889634f;
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);                          // [16][DH]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    bf16* sK = sQ + 16 * DH + warp * (2 * KT * DH);                         // this warp's [32][DH] K tile
    bf16* sV = sK + KT * DH;                                                // and V tile
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int G = a.Hq / a.Hkv, h0 = hk * G;

    // query rows of the group -> rows 0 .. G - 1 of a 16-row tile, the rest zero
    for (int i = threadIdx.x; i < 16 * CH; i += 128) {
        const int r = i / CH, c = i % CH;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < G) v = *reinterpret_cast<const uint4*>(a.q + ((long)b * a.Hq + h0 + r) * DH + c * 8);
        if constexpr (FP8) {                                // bf16 -> half, pair by pair
            const bf162* p2 = reinterpret_cast<const bf162*>(&v);
            uint4 hv;
            uint32_t* hp = reinterpret_cast<uint32_t*>(&hv);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const float2 f = __bfloat1622float2(p2[q4]);
                hp[q4] = pack_f16(f.x, f.y);
            }
            v = hv;
        }
        *reinterpret_cast<uint4*>(tile_ptr<DH>(sQ, r, c)) = v;
    }
    const int len = a.kv_lens[b];
    const int lo = (a.window > 0 && len > a.window) ? len - a.window : 0;
    const int span = len - lo;
    const int per = a.split_len > 0 ? a.split_len : ((((span + a.splits - 1) / a.splits) + 31) & ~31);
    const int s0 = lo + split * per, s1 = min(len, s0 + per);
    __syncthreads();
    uint32_t qa[DH / 16][4];
#pragma unroll
    for (int kk = 0; kk < DH / 16; ++kk) ldsm_x4(qa[kk], tile_ptr<DH>(sQ, lane & 15, kk * 2 + (lane >> 4)));

    float o[DH / 8][4];
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};          // rows lane / 4 and lane / 4 + 8

    for (int base = s0 + warp * KT; base < s1; base += 4 * KT) {
        const int j = base + lane;
        long slot = 0;
        if (j < s1) {
            const int page = a.block_table[(long)b * a.max_pages + j / a.page_size];
            slot = (long)page * a.page_size + j % a.page_size;
        }
        // the chunk's K and V rows -> this warp's tiles (rows past the split's end are zero: 0 x garbage would poison P V)
        if constexpr (FP8) {
            constexpr int PC = DH / 16;                 // 16-byte pieces (16 values) per e4m3 row
            constexpr int NP = KT * PC / 32;            // pieces per lane and matrix
            const uint8_t* kc8 = reinterpret_cast<const uint8_t*>(a.k_cache);
            const uint8_t* vc8 = reinterpret_cast<const uint8_t*>(a.v_cache);
            uint4 kr[NP], vr[NP];
#pragma unroll
            for (int r = 0; r < NP; ++r) {
                const int i = lane + 32 * r, key = i / PC, pc = i % PC;
                const long sl = __shfl_sync(0xffffffffu, slot, key);
                const long off = (sl * a.Hkv + hk) * DH + pc * 16;
                const bool ok = base + key < s1;
                kr[r] = ok ? *reinterpret_cast<const uint4*>(kc8 + off) : make_uint4(0u, 0u, 0u, 0u);
                vr[r] = ok ? *reinterpret_cast<const uint4*>(vc8 + off) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int r = 0; r < NP; ++r) {
                const int i = lane + 32 * r, key = i / PC, pc = i % PC;
                uint4 lo, hi;
                e4m3x16_to_half(kr[r], lo, hi);
                *reinterpret_cast<uint4*>(tile_ptr<DH>(sK, key, 2 * pc)) = lo;
                *reinterpret_cast<uint4*>(tile_ptr<DH>(sK, key, 2 * pc + 1)) = hi;
                e4m3x16_to_half(vr[r], lo, hi);
                *reinterpret_cast<uint4*>(tile_ptr<DH>(sV, key, 2 * pc)) = lo;
                *reinterpret_cast<uint4*>(tile_ptr<DH>(sV, key, 2 * pc + 1)) = hi;
            }
        } else {
#pragma unroll 4
        for (int i = lane; i < KT * CH; i += 32) {
            const int key = i / CH, c = i % CH;
            const long sl = __shfl_sync(0xffffffffu, slot, key);
            bf16* pk = tile_ptr<DH>(sK, key, c);
            bf16* pv = tile_ptr<DH>(sV, key, c);
            if (base + key < s1) {
                const long off = (sl * a.Hkv + hk) * DH + c * 8;
                cp_async16(pk, a.k_cache + off);
                cp_async16(pv, a.v_cache + off);
            } else {
                *reinterpret_cast<uint4*>(pk) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(pv) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        }
        __syncwarp();

        // S = Q K^T: 16 rows x 32 keys
        float s[KT / 8][4];
#pragma unroll
        for (int i = 0; i < KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
#pragma unroll
            for (int nt = 0; nt < KT / 16; ++nt) {
                uint32_t kb[4];
                const int tok = nt * 16 + ((lane >> 4) << 3) + (lane & 7);
                ldsm_x4(kb, tile_ptr<DH>(sK, tok, kk * 2 + ((lane >> 3) & 1)));
                if constexpr (FP8) {
                    mma_f16(s[2 * nt], qa[kk], kb[0], kb[1]);
                    mma_f16(s[2 * nt + 1], qa[kk], kb[2], kb[3]);
                } else {
                    mma_bf16(s[2 * nt], qa[kk], kb[0], kb[1]);
                    mma_bf16(s[2 * nt + 1], qa[kk], kb[2], kb[3]);
                }
            }
        }
        // scale, soft-cap, mask the keys past the end, online softmax (scores in natural-log units, as the combine expects)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sv = s[nt][e] * a.scale;
                if (a.softcap > 0.f) sv = a.softcap * tanhf(sv / a.softcap);
                const int key = base + nt * 8 + (lane & 3) * 2 + (e & 1);
                sv = key < s1 ? sv : -INFINITY;
                s[nt][e] = sv;
                mx[e >> 1] = fmaxf(mx[e >> 1], sv);
            }
        }
        float corr[2], rsum[2] = {0.f, 0.f}, mneg[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            mx[r] = fmaxf(mrow[r], mx[r]);
            corr[r] = (mrow[r] == -INFINITY) ? 0.f : exp2f((mrow[r] - mx[r]) * LOG2E);
            mrow[r] = mx[r];
            mneg[r] = (mx[r] == -INFINITY) ? 0.f : -mx[r] * LOG2E;
        }
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = exp2f(fmaf(s[nt][e], LOG2E, mneg[e >> 1]));
                s[nt][e] = p;
                rsum[e >> 1] += p;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) lrow[r] = lrow[r] * corr[r] + rsum[r];
#pragma unroll
        for (int i = 0; i < DH / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // O += P V
#pragma unroll
        for (int kt = 0; kt < KT / 16; ++kt) {
            uint32_t pa[4];
            if constexpr (FP8) {
                pa[0] = pack_f16(s[2 * kt][0], s[2 * kt][1]);
                pa[1] = pack_f16(s[2 * kt][2], s[2 * kt][3]);
                pa[2] = pack_f16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
                pa[3] = pack_f16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
            } else {
                pa[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
                pa[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
                pa[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
                pa[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
            }
#pragma unroll
            for (int dt = 0; dt < DH / 16; ++dt) {
                uint32_t vb[4];
                const int tok = kt * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
                ldsm_x4_t(vb, tile_ptr<DH>(sV, tok, dt * 2 + (lane >> 4)));
                if constexpr (FP8) {
                    mma_f16(o[2 * dt], pa, vb[0], vb[1]);
                    mma_f16(o[2 * dt + 1], pa, vb[2], vb[3]);
                } else {
                    mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
                    mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
                }
            }
        }
        __syncwarp();                                   // every lane is done with the tiles before the next chunk lands
    }
    // row sums over the four lanes that share a row
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
    }
    // merge the four warps through shared memory (over the staging tiles, which are free now)
    __syncthreads();
    float* red_m = reinterpret_cast<float*>(smem_raw);                      // [4][16]
    float* red_l = red_m + 64;                                              // [4][16]
    float* red_o = red_l + 64;                                              // [4][G][DH]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + 8 * r;
        if (row < G) {
            if ((lane & 3) == 0) { red_m[warp * 16 + row] = mrow[r]; red_l[warp * 16 + row] = lrow[r]; }
#pragma unroll
            for (int i = 0; i < DH / 8; ++i) {
                float* dst = red_o + ((long)(warp * G + row)) * DH + i * 8 + (lane & 3) * 2;
                dst[0] = o[i][2 * r];
                dst[1] = o[i][2 * r + 1];
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * DH; i += 128) {
        const int g = i / DH, d = i % DH;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red_m[w * 16 + g]);
        float ll = 0.f, ov = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float c = (red_m[w * 16 + g] == -INFINITY) ? 0.f : __expf(red_m[w * 16 + g] - mm);
            ll += red_l[w * 16 + g] * c;
            ov += red_o[((long)(w * G + g)) * DH + d] * c;
        }
        if constexpr (CS == 0) {
            const long pi = ((long)b * a.Hq + h0 + g) * a.splits + split;
            a.part_o[pi * DH + d] = ov;
            if (d == 0) { a.part_ml[pi * 2] = mm; a.part_ml[pi * 2 + 1] = ll; }
        } else {
            float* fin = red_o + 4 * 16 * DH;                               // [16] max | [16] sum | [G][DH] partial output
            fin[32 + i] = ov;
            if (d == 0) { fin[g] = mm; fin[16 + g] = ll; }
        }
    }
    if constexpr (CS > 0) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                                                     // every split's partial is in place
        float* fin = red_o + 4 * 16 * DH;
        const int per = G * DH / CS;                                        // output columns this CTA finishes (a multiple of 32)
        const int rank = (int)cluster.block_rank();
        for (int i0 = threadIdx.x; i0 < per; i0 += 128) {
            const int i = rank * per + i0, g = i / DH, d = i % DH, h = h0 + g;
            float ms[CS], mm = a.sinks ? a.sinks[h] : -INFINITY;
#pragma unroll
            for (int sp = 0; sp < CS; ++sp) {
                ms[sp] = cluster.map_shared_rank(fin, sp)[g];
                mm = fmaxf(mm, ms[sp]);
            }
            float ll = a.sinks ? __expf(a.sinks[h] - mm) : 0.f, ov = 0.f;
#pragma unroll
            for (int sp = 0; sp < CS; ++sp) {
                const float* rf = cluster.map_shared_rank(fin, sp);
                const float c = (ms[sp] == -INFINITY) ? 0.f : __expf(ms[sp] - mm);
                ll += rf[16 + g] * c;
                ov += rf[32 + i] * c;
            }
            const bf16 ob = f2bf(ll > 0.f ? ov / ll : 0.f);
            const long e = ((long)b * a.Hq + h) * DH + d;
            a.out[e] = ob;
            if (a.out_q != nullptr) {                   // a warp holds one group of 32 columns; arithmetic of quantize_q8_kernel
                const float v = bf2f(ob);
                const float amax = warp_max(fabsf(v));
                const float sum = warp_sum(v);
                const float dq = amax / 127.f;
                a.out_q[e] = (int8_t)__float2int_rn(amax > 0.f ? v / dq : 0.f);
                if ((d & 31) == 0) a.out_ds[e >> 5] = make_float2(dq, sum);
            }
        }
        cluster.sync();                                                     // nobody leaves while its partial is being read
    }
}

template <int DH, int CS, bool FP8 = false>
static int launch_decode_mma(const AttnArgs& a, cudaStream_t s) {
    // the query tile, four warps' K and V tiles; the merge buffers reuse them (4 * 16 * DH floats, and with a cluster
    // this CTA's finished partial behind them)
    const size_t stage = (size_t)(16 + 4 * 2 * 32) * DH * sizeof(bf16);
    const size_t merge = (size_t)(128 + 4 * 16 * DH + 32 + 16 * DH) * sizeof(float);
    const size_t smem = stage > merge ? stage : merge;
    static bool configured = false;
    if (!configured) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(attn_decode_mma_kernel<DH, CS, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (CS > 8) TSB_CHECK_CUDA(cudaFuncSetAttribute(attn_decode_mma_kernel<DH, CS, FP8>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        configured = true;
    }
    if constexpr (CS == 0) {
        TSB_CHECK_CUDA(tsb_launch(attn_decode_mma_kernel<DH, 0, FP8>, dim3(a.splits, a.Hkv, a.B), dim3(128), smem, s, a));
    } else {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(a.splits, a.Hkv, a.B);
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute at[2];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = CS;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = tsb_pdl_enabled() ? 2 : 1;
        TSB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, attn_decode_mma_kernel<DH, CS, FP8>, a));
    }
    return TSB_OK;
}

// Whether this kernel serves the shape (the caller decides whether the grid is large enough to prefer it).
bool tsb_attn_decode_mma_supported(const AttnArgs& a) {
    return (a.Dh == 64 || a.Dh == 128) && a.Hkv > 0 && a.Hq % a.Hkv == 0 && a.Hq / a.Hkv <= 16;
}

// Whether the splits are merged inside the kernel by a thread-block cluster: only with TSB_ATTN_CLUSTER=1 (read at every
// call), 8 or 16 splits, and whole groups of 32 output columns per CTA.  Off by default: inside the decode step of the
// Qwen3-4B shape it measured 1.801 ms against 1.757 ms with the separate combine launch, whose start overlaps this
// kernel's tail, while the merge after two cluster barriers sits on the critical path.
bool tsb_attn_decode_mma_cluster(const AttnArgs& a) {
    const char* e = getenv("TSB_ATTN_CLUSTER");
    const bool on = e != nullptr && atoi(e) != 0;
    if (!on || (a.splits != 8 && a.splits != 16)) return false;
    const int cols = (a.Hq / a.Hkv) * a.Dh;
    return cols % (a.splits * 32) == 0;
}

// Returns TSB_OK; `*merged` tells whether the outputs are final (cluster form) or the caller has to launch the combine.
int tsb_attn_decode_mma_launch(const AttnArgs& a, cudaStream_t s, bool* merged) {
    const bool cl = tsb_attn_decode_mma_cluster(a);
    *merged = cl;
    if (cl && a.splits == 8) return a.Dh == 64 ? launch_decode_mma<64, 8>(a, s) : launch_decode_mma<128, 8>(a, s);
    if (cl) return a.Dh == 64 ? launch_decode_mma<64, 16>(a, s) : launch_decode_mma<128, 16>(a, s);
    return a.Dh == 64 ? launch_decode_mma<64, 0>(a, s) : launch_decode_mma<128, 0>(a, s);
}

// The same split kernel on e4m3 pages (`k_cache` / `v_cache` point at bytes); the caller launches the combine.
int tsb_attn_decode_mma_fp8_launch(const AttnArgs& a, cudaStream_t s) {
    return a.Dh == 64 ? launch_decode_mma<64, 0, true>(a, s) : launch_decode_mma<128, 0, true>(a, s);
}
