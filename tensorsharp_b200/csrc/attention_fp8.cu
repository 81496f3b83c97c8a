// An 8-bit KV cache: pages of e4m3 bytes, [n_slots, Hkv, Dh] one byte per value, half the bytes of the bf16 cache and
// twice the context per GB.  Three entry points:
//
//   tsb_kv_store_fp8     rows of K and V (bf16, as the norm / RoPE kernel leaves them) -> e4m3 at their cache slots
//   tsb_kv_load_fp8      cache slots -> dense bf16 rows (what the prefill kernel reads: a prompt's keys are converted
//                        once per layer instead of once per query tile)
//   tsb_attn_decode_fp8  split-KV decode attention that reads the e4m3 pages directly; the partial results go
//                        through the same merge kernel as the bf16 cache's (tsb_attn_combine)
//
// Values are stored unscaled with saturation (e4m3 reaches +-448; keys after the per-head norm and values of the
// supported models stay far inside that).  The reference keeps its KV cache in f16 / f32 (KVCache.cs); the 8-bit form
// is this framework's own.
#include <cuda_fp8.h>

#include "attn_args.cuh"
#include "common.cuh"

extern "C" int tsb_attn_combine(const AttnArgs* args, void* stream);

__device__ __forceinline__ void fp8x4_to_float(uint32_t w, float* f) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

__device__ __forceinline__ uint32_t float4_to_fp8x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// ------------------------------------------------------------------------------------------
// store: one thread per 8 values (a 16-byte bf16 read, an 8-byte write); rows [T, Hkv * Dh] dense
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) kv_store_fp8_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                           uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache,
                                                           const long* __restrict__ slots, long T, int row) {
    pdl_wait();
    pdl_trigger();
    const int per_row = row / 8;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * per_row) return;
    const long t = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const long dst = slots[t] * row + c;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
        const uint4 raw = *reinterpret_cast<const uint4*>((which ? v : k) + t * row + c);
        const bf162* p = reinterpret_cast<const bf162*>(&raw);
        const float2 f0 = __bfloat1622float2(p[0]), f1 = __bfloat1622float2(p[1]);
        const float2 f2 = __bfloat1622float2(p[2]), f3 = __bfloat1622float2(p[3]);
        uint2 o;
        o.x = float4_to_fp8x4(f0.x, f0.y, f1.x, f1.y);
        o.y = float4_to_fp8x4(f2.x, f2.y, f3.x, f3.y);
        *reinterpret_cast<uint2*>((which ? v_cache : k_cache) + dst) = o;
    }
}

extern "C" int tsb_kv_store_fp8(const void* k, const void* v, void* k_cache, void* v_cache, const long* slots, long T,
                                int Hkv, int Dh, void* stream) {
    TSB_CHECK_ARG(T >= 0 && Hkv > 0 && Dh > 0 && Dh % 8 == 0, "kv_store_fp8: bad shape T=%ld Hkv=%d Dh=%d", T, Hkv, Dh);
    if (T == 0) return TSB_OK;
    const int row = Hkv * Dh;
    const long n = T * (row / 8);
    TSB_CHECK_CUDA(tsb_launch(kv_store_fp8_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                              (const bf16*)k, (const bf16*)v, (uint8_t*)k_cache, (uint8_t*)v_cache, slots, T, row));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// load: out[i] = cache[idx[i]] as bf16, for K and V in one launch; one thread per 8 values
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) kv_load_fp8_kernel(const uint8_t* __restrict__ k_cache, const uint8_t* __restrict__ v_cache,
                                                          const long* __restrict__ idx, bf16* __restrict__ k_out,
                                                          bf16* __restrict__ v_out, long n_rows, int row) {
    pdl_wait();
    pdl_trigger();
    const int per_row = row / 8;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * per_row) return;
    const long t = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const long src = idx[t] * row + c;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
        const uint2 raw = *reinterpret_cast<const uint2*>((which ? v_cache : k_cache) + src);
        float f[8];
        fp8x4_to_float(raw.x, f);
        fp8x4_to_float(raw.y, f + 4);
        uint4 o;
        bf162* p = reinterpret_cast<bf162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) p[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
        *reinterpret_cast<uint4*>((which ? v_out : k_out) + t * row + c) = o;
    }
}

extern "C" int tsb_kv_load_fp8(const void* k_cache, const void* v_cache, const long* idx, void* k_out, void* v_out,
                               long n_rows, int Hkv, int Dh, void* stream) {
    TSB_CHECK_ARG(n_rows >= 0 && Hkv > 0 && Dh > 0 && Dh % 8 == 0, "kv_load_fp8: bad shape n=%ld Hkv=%d Dh=%d", n_rows, Hkv, Dh);
    if (n_rows == 0) return TSB_OK;
    const int row = Hkv * Dh;
    const long n = n_rows * (row / 8);
    TSB_CHECK_CUDA(tsb_launch(kv_load_fp8_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                              (const uint8_t*)k_cache, (const uint8_t*)v_cache, idx, (bf16*)k_out, (bf16*)v_out, n_rows, row));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// Decode: grid (splits, Hkv * chunks, B), 128 threads; a CTA serves G query heads of one KV head.  Each warp takes 32
// cache positions at a time: lane = position for Q K^T (its K row is Dh bytes, read 16 at a time), lane = slice of
// Dh / 32 output columns for P V (a V row is one coalesced Dh-byte request of the warp), eight V rows in flight.
// ------------------------------------------------------------------------------------------
template <int DH, int G>
__global__ void __launch_bounds__(128) attn_decode_fp8_kernel(AttnArgs a) {
    constexpr int DPL = DH / 32;             // output columns (= V bytes) per lane
    pdl_wait();
    pdl_trigger();
    const uint8_t* k_cache = reinterpret_cast<const uint8_t*>(a.k_cache);
    const uint8_t* v_cache = reinterpret_cast<const uint8_t*>(a.v_cache);
    const int split = blockIdx.x, b = blockIdx.z;
    const int heads_per_kv = a.Hq / a.Hkv, chunks = heads_per_kv / G;
    const int hk = blockIdx.y / chunks, h0 = hk * heads_per_kv + (blockIdx.y % chunks) * G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ __align__(16) float qs[G][DH];
    __shared__ float red_m[4][G], red_l[4][G];
    __shared__ float red_o[4][G][DH];
    for (int i = threadIdx.x; i < G * DH; i += 128) qs[i / DH][i % DH] = bf2f(a.q[((long)b * a.Hq + h0) * DH + i]);
    const int len = a.kv_lens[b];
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
        long slot = 0;
        if (valid) {
            const int page = a.block_table[(long)b * a.max_pages + j / a.page_size];
            slot = (long)page * a.page_size + j % a.page_size;
        }
        const int cnt = min(32, s1 - base);
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = 0.f;
        if (valid) {
            const uint4* kp = reinterpret_cast<const uint4*>(k_cache + (slot * a.Hkv + hk) * DH);
#pragma unroll 4
            for (int c = 0; c < DH / 16; ++c) {
                const uint4 kv = kp[c];
                float kf[16];
                fp8x4_to_float(kv.x, kf);
                fp8x4_to_float(kv.y, kf + 4);
                fp8x4_to_float(kv.z, kf + 8);
                fp8x4_to_float(kv.w, kf + 12);
#pragma unroll
                for (int g = 0; g < G; ++g) {
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) {
                        const float4 qv = *reinterpret_cast<const float4*>(&qs[g][c * 16 + i4 * 4]);     // same address in every lane
                        s[g] += qv.x * kf[i4 * 4] + qv.y * kf[i4 * 4 + 1] + qv.z * kf[i4 * 4 + 2] + qv.w * kf[i4 * 4 + 3];
                    }
                }
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
        constexpr int VB = DPL > 8 ? 4 : 8;
        for (int t0 = 0; t0 < cnt; t0 += VB) {
            float vf[VB][DPL];
#pragma unroll
            for (int u = 0; u < VB; ++u) {
                const long sl = __shfl_sync(0xffffffffu, slot, (t0 + u) & 31);
                const uint8_t* vp = v_cache + (sl * a.Hkv + hk) * DH + lane * DPL;
                if (t0 + u < cnt) {
                    if constexpr (DPL == 2) {
                        const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(*reinterpret_cast<const __nv_fp8x2_storage_t*>(vp), __NV_E4M3);
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
                        vf[u][0] = f.x;
                        vf[u][1] = f.y;
                    } else {
#pragma unroll
                        for (int w = 0; w < DPL / 4; ++w) fp8x4_to_float(reinterpret_cast<const uint32_t*>(vp)[w], &vf[u][w * 4]);
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
    // merge the four warps, write this split's partial
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
}

static int fp8_decode_chunk(int heads_per_kv, int Dh) {
    const int cap = Dh > 256 ? 2 : (Dh > 128 ? 4 : 8);
    for (int g = cap; g > 1; g >>= 1)
        if (heads_per_kv % g == 0) return g;
    return 1;
}

template <int DH, int G>
static int launch_fp8(const AttnArgs& a, cudaStream_t s) {
    dim3 grid(a.splits, a.Hkv * ((a.Hq / a.Hkv) / G), a.B);
    return tsb_launch(attn_decode_fp8_kernel<DH, G>, grid, dim3(128), 0, s, a) == cudaSuccess ? TSB_OK : TSB_ERR_CUDA;
}

template <int DH>
static int launch_fp8_g(const AttnArgs& a, cudaStream_t s) {
    switch (fp8_decode_chunk(a.Hq / a.Hkv, DH)) {
    case 1: return launch_fp8<DH, 1>(a, s);
    case 2: return launch_fp8<DH, 2>(a, s);
    case 4:
        if constexpr (DH <= 256) return launch_fp8<DH, 4>(a, s);
        return TSB_ERR_UNSUPPORTED;
    default:
        if constexpr (DH <= 128) return launch_fp8<DH, 8>(a, s);
        return TSB_ERR_UNSUPPORTED;
    }
}

// `k_cache` / `v_cache` of the argument block point at e4m3 bytes here.
extern "C" int tsb_attn_decode_fp8(const AttnArgs* args, void* stream) {
    AttnArgs a = *args;
    a.ticket = nullptr;
    TSB_CHECK_ARG(a.Hkv > 0 && a.Hq % a.Hkv == 0, "attn_decode_fp8: Hq=%d not a multiple of Hkv=%d", a.Hq, a.Hkv);
    TSB_CHECK_ARG(a.splits >= 1 && a.splits <= 64 && a.part_o && a.part_ml, "attn_decode_fp8: scratch for %d splits (limit 64)", a.splits);
    if (a.B == 0) return TSB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    // head sizes 64 / 128 with up to 16 query heads per KV head: the tensor-core split kernel (attention_decode_mma.cu)
    static const bool mma_on = []() { const char* e = getenv("TSB_ATTN_MMA"); return !e || atoi(e) != 0; }();
    if (mma_on && tsb_attn_decode_mma_supported(a)) {
        rc = tsb_attn_decode_mma_fp8_launch(a, s);
        if (rc != TSB_OK) return rc;
        TSB_CHECK_LAUNCH();
        return tsb_attn_combine(&a, stream);
    }
    switch (a.Dh) {
    case 64: rc = launch_fp8_g<64>(a, s); break;
    case 128: rc = launch_fp8_g<128>(a, s); break;
    case 256: rc = launch_fp8_g<256>(a, s); break;
    case 512: rc = launch_fp8_g<512>(a, s); break;
    default:
        tsb_set_error("attn_decode_fp8: unsupported head dim %d (supported 64, 128, 256, 512)", a.Dh);
        return TSB_ERR_UNSUPPORTED;
    }
    if (rc != TSB_OK) {
        if (rc == TSB_ERR_CUDA) tsb_set_error("attn_decode_fp8: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        return rc;
    }
    TSB_CHECK_LAUNCH();
    return tsb_attn_combine(&a, stream);
}
