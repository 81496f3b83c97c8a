// Fused normalisation, rotary embedding + KV-cache write, gated activations, embedding
// gather, row dequantisation and arg-max.
//
// Replaces in the reference: rms_norm_f32 (+mul, +add) (ggml-cuda/norm.cu:108, :358-435),
// l2_norm_f32 (:287), rope_neox / rope_norm with YaRN and freq factors (rope.cu:44, :111),
// the rope + view + set_rows fusion (ggml-cuda.cu:3359-3790 item 2), k_set_rows
// (set-rows.cu:113), unary_gated_op_kernel / swiglu_oai_kernel (unary.cu:255, :352),
// k_get_rows* (getrows.cu:6-225), dequantize_block_* (convert.cu), argmax_f32 (argmax.cu:8),
// softcap_f32 (softcap.cu:3), quantize_q8_1 fused into the producer.
#include "quant_blocks.cuh"

// ------------------------------------------------------------------------------------------
// RMSNorm family.  One block per row.
//   v      = x (+ delta)                       (delta optional; when given, v is also stored
//                                               back to x, which is the residual stream)
//   n      = v * rsqrt(mean(v^2) + eps) * w    (w optional)
//   y_bf16 = n            y_f32 = (add ? add : 0) + n         yq/yds = q8(n)
// ------------------------------------------------------------------------------------------
template <typename TX>
__global__ void __launch_bounds__(256) rmsnorm_kernel(TX* x, const bf16* delta, const float* w, float eps,
                                                      int D, bf16* y_bf16, float* y_f32, const float* add,
                                                      int8_t* yq, float2* yds, int l2_mode) {
    __shared__ float red[32];
    pdl_wait();
    pdl_trigger();
    const long row = blockIdx.x;
    TX* xr = x + row * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = (float)xr[i];
        if (delta) {
            v += bf2f(delta[row * D + i]);
            xr[i] = (TX)v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    // l2_mode: x / max(||x||, eps) (ggml l2_norm); otherwise RMS.
    const float rs = l2_mode ? 1.f / fmaxf(sqrtf(ss), eps) : rsqrtf(ss / (float)D + eps);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int dpad = (D + 31) & ~31;
    for (int i = threadIdx.x; i < dpad; i += blockDim.x) {
        float n = 0.f;
        if (i < D) {
            n = (float)xr[i] * rs;
            if (w) n *= w[i];
            if (y_bf16) y_bf16[row * D + i] = f2bf(n);
            if (y_f32) y_f32[row * D + i] = (add ? add[row * D + i] : 0.f) + n;
        }
        if (yq) {
            // whole warps iterate together because blockDim.x and dpad are multiples of 32
            const float amax = warp_max(fabsf(n));
            const float sum = warp_sum(n);
            const float d = amax / 127.f;
            if (i < D) yq[row * D + i] = (int8_t)__float2int_rn(amax > 0.f ? n / d : 0.f);
            if (lane == 0 && i < D) yds[row * (D / 32) + i / 32] = make_float2(d, sum);
        }
    }
}

// Vectorised variant (D % 4 == 0): each thread keeps up to VMAX float4 chunks of the row in
// registers, so every global load is issued before the first reduction and the row is read
// exactly once.  A q8 group of 32 values is 8 neighbouring lanes.
template <typename TX, int VMAX>
__global__ void __launch_bounds__(1024) rmsnorm_vec_kernel(TX* x, const bf16* delta, const float* w, float eps, int D,
                                                           bf16* y_bf16, float* y_f32, const float* add, int8_t* yq,
                                                           float2* yds, int l2_mode) {
    __shared__ float red[32];
    const long row = blockIdx.x;
    const int nvec = D >> 2, tid = threadIdx.x, nt = blockDim.x;
    float4 wv[VMAX];
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {          // weights do not depend on the previous kernel
        const int i = tid + j * nt;
        wv[j] = (w && i < nvec) ? reinterpret_cast<const float4*>(w)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
    }
    pdl_wait();
    pdl_trigger();
    float4 v[VMAX];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
        const int i = tid + j * nt;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nvec) {
            if (sizeof(TX) == 4) {
                t = reinterpret_cast<const float4*>(x + row * D)[i];
            } else {
                const uint2 r = reinterpret_cast<const uint2*>(x + row * D)[i];
                const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(&r.x));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(&r.y));
                t = make_float4(a.x, a.y, b.x, b.y);
            }
            if (delta) {
                const uint2 r = reinterpret_cast<const uint2*>(delta + row * D)[i];
                const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(&r.x));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(&r.y));
                t.x += a.x; t.y += a.y; t.z += b.x; t.w += b.y;
                if (sizeof(TX) == 4) {
                    reinterpret_cast<float4*>(x + row * D)[i] = t;
                } else {
                    uint2 o;
                    *reinterpret_cast<bf162*>(&o.x) = __floats2bfloat162_rn(t.x, t.y);
                    *reinterpret_cast<bf162*>(&o.y) = __floats2bfloat162_rn(t.z, t.w);
                    reinterpret_cast<uint2*>(x + row * D)[i] = o;
                }
            }
        }
        v[j] = t;
        ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
    }
    ss = block_sum(ss, red);
    const float rs = l2_mode ? 1.f / fmaxf(sqrtf(ss), eps) : rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
        const int i = tid + j * nt;
        const bool ok = i < nvec;
        float4 n = make_float4(v[j].x * rs * wv[j].x, v[j].y * rs * wv[j].y, v[j].z * rs * wv[j].z, v[j].w * rs * wv[j].w);
        if (ok) {
            if (y_bf16) {
                uint2 o;
                *reinterpret_cast<bf162*>(&o.x) = __floats2bfloat162_rn(n.x, n.y);
                *reinterpret_cast<bf162*>(&o.y) = __floats2bfloat162_rn(n.z, n.w);
                reinterpret_cast<uint2*>(y_bf16 + row * D)[i] = o;
            }
            if (y_f32) {
                float4 o = n;
                if (add) {
                    const float4 ad = reinterpret_cast<const float4*>(add + row * D)[i];
                    o.x += ad.x; o.y += ad.y; o.z += ad.z; o.w += ad.w;
                }
                reinterpret_cast<float4*>(y_f32 + row * D)[i] = o;
            }
        }
        if (yq) {
            float amax = fmaxf(fmaxf(fabsf(n.x), fabsf(n.y)), fmaxf(fabsf(n.z), fabsf(n.w)));
            float sum = n.x + n.y + n.z + n.w;
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                sum += __shfl_xor_sync(0xffffffffu, sum, o);
            }
            if (ok) {
                const float inv = amax > 0.f ? 127.f / amax : 0.f;
                char4 q;
                q.x = (signed char)__float2int_rn(n.x * inv);
                q.y = (signed char)__float2int_rn(n.y * inv);
                q.z = (signed char)__float2int_rn(n.z * inv);
                q.w = (signed char)__float2int_rn(n.w * inv);
                reinterpret_cast<char4*>(yq + row * D)[i] = q;
                if ((i & 7) == 0) yds[row * (D / 32) + (i >> 3)] = make_float2(amax / 127.f, sum);
            }
        }
    }
}

template <typename TX>
static cudaError_t launch_rmsnorm(TX* x, const bf16* delta, const float* w, float eps, long rows, int D, bf16* yb,
                                  float* yf, const float* add, int8_t* yq, float2* yds, int l2, cudaStream_t s) {
    if (D % 4 == 0 && D <= 16384) {
        const int nvec = D / 4;
        if (nvec <= 1024) {
            const int nt = (nvec + 31) & ~31;
            return tsb_launch(rmsnorm_vec_kernel<TX, 1>, dim3((unsigned)rows), dim3(nt), 0, s, x, delta, w, eps, D, yb,
                              yf, add, yq, yds, l2);
        }
        const int nt = (((nvec + 3) / 4) + 31) & ~31;
        return tsb_launch(rmsnorm_vec_kernel<TX, 4>, dim3((unsigned)rows), dim3(nt), 0, s, x, delta, w, eps, D, yb, yf,
                          add, yq, yds, l2);
    }
    return tsb_launch(rmsnorm_kernel<TX>, dim3((unsigned)rows), dim3(256), 0, s, x, delta, w, eps, D, yb, yf, add, yq,
                      yds, l2);
}

extern "C" int tsb_rmsnorm(void* x, int x_f32, const void* delta, const float* w, float eps, long rows, int D,
                           void* y_bf16, float* y_f32, const float* add, void* yq, void* yds, int l2_mode,
                           void* stream) {
    TSB_CHECK_ARG(D > 0 && rows >= 0, "rmsnorm: bad shape rows=%ld D=%d", rows, D);
    TSB_CHECK_ARG(!yq || D % 32 == 0, "rmsnorm: q8 output needs D %% 32 == 0, got %d", D);
    if (rows == 0) return TSB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (x_f32)
        TSB_CHECK_CUDA(launch_rmsnorm<float>((float*)x, (const bf16*)delta, w, eps, rows, D, (bf16*)y_bf16, y_f32, add,
                                             (int8_t*)yq, (float2*)yds, l2_mode, s));
    else
        TSB_CHECK_CUDA(launch_rmsnorm<bf16>((bf16*)x, (const bf16*)delta, w, eps, rows, D, (bf16*)y_bf16, y_f32, add,
                                            (int8_t*)yq, (float2*)yds, l2_mode, s));
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// Per-head norm + RoPE + KV-cache write.  One warp per (token, head); heads are laid out
// q[0..Hq), k[0..Hkv), v[0..Hkv).  Head dim <= 512.
// ------------------------------------------------------------------------------------------
struct RopeParams {
    float theta_base;      // rope.freq_base
    float freq_scale;      // 1 / rope.scaling.factor
    float ext_factor;      // YaRN mix (0 = plain)
    float attn_factor;     // magnitude scale
    float corr_lo, corr_hi;  // YaRN ramp bounds (already computed on the host)
    int rot_dim;           // number of rotated dims (<= head dim); 0 disables RoPE
    int mode;              // 0 = NeoX (pairs i, i + rot/2), 1 = adjacent pairs (2i, 2i+1)
};

struct QkvArgs {
    const void* q; const void* k; const void* v;   // inputs (same dtype), may alias one buffer
    long q_tok, q_head, k_tok, k_head, v_tok, v_head;  // element strides
    int in_f32;
    const float* qn; const float* kn;   // per-head RMSNorm weights [Dh] or null
    int v_norm;                         // 1: unweighted RMSNorm on V
    float eps;
    const int* pos;                     // [T]
    const long* slot;                   // [T] flat slot in the KV cache (page * page_size + offset), <0 = skip
    const float* freq_factors;          // [rot_dim/2] or null
    const float2* cs_table;             // [T, rot_dim/2] (cos, sin) precomputed per token, or null
    bf16* q_out;                        // [T, Hq, Dh]
    bf16* k_cache; bf16* v_cache;       // [slots, Hkv, Dh]
    float q_scale;                      // multiplied into q after RoPE (1 = none)
    int T, Hq, Hkv, Dh;
    RopeParams rp;
};

__device__ __forceinline__ void rope_cs(const RopeParams& rp, const float* ff, int pair, float pos, float& c, float& s) {
    float theta = pos * powf(rp.theta_base, -2.f * (float)pair / (float)rp.rot_dim);
    if (ff) theta /= ff[pair];
    float th = rp.freq_scale * theta;
    float ms = rp.attn_factor;
    if (rp.ext_factor != 0.f) {
        const float y = ((float)pair - rp.corr_lo) / fmaxf(0.001f, rp.corr_hi - rp.corr_lo);
        const float ramp = (1.f - fminf(1.f, fmaxf(0.f, y))) * rp.ext_factor;
        th = th * (1.f - ramp) + theta * ramp;
        ms *= 1.f + 0.1f * logf(1.f / rp.freq_scale);
    }
    sincosf(th, &s, &c);
    c *= ms;
    s *= ms;
}

// (cos, sin) of every (token, pair): computed once per forward and shared by all layers and heads.
__global__ void rope_table_kernel(const int* pos, RopeParams rp, const float* ff, float2* out, int T) {
    pdl_wait();
    pdl_trigger();
    const int half = rp.rot_dim >> 1;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)T * half) return;
    const int t = (int)(i / half), pair = (int)(i % half);
    float c, s;
    rope_cs(rp, ff, pair, (float)pos[t], c, s);
    out[i] = make_float2(c, s);
}

extern "C" int tsb_rope_table(const int* pos, const RopeParams* rp, const float* ff, void* out, int T, void* stream) {
    TSB_CHECK_ARG(rp->rot_dim > 0 && rp->rot_dim % 2 == 0, "rope_table: bad rot_dim %d", rp->rot_dim);
    const long n = (long)T * (rp->rot_dim / 2);
    if (n == 0) return TSB_OK;
    TSB_CHECK_CUDA(tsb_launch(rope_table_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, (cudaStream_t)stream, pos,
                              *rp, ff, (float2*)out, T));
    return TSB_OK;
}

__device__ __forceinline__ void rope_lookup(const QkvArgs& a, int t, int pair, float pos, float& c, float& s) {
    if (a.cs_table) {
        const float2 cs = a.cs_table[(long)t * (a.rp.rot_dim >> 1) + pair];
        c = cs.x;
        s = cs.y;
    } else {
        rope_cs(a.rp, a.freq_factors, pair, pos, c, s);
    }
}

// NJ = 32-element slices a lane holds (head size up to 32 * NJ): the loops below run NJ times, not 16.
template <int NJ>
__global__ void __launch_bounds__(128) qkv_rope_kernel(QkvArgs a) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const long wid = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int H = a.Hq + 2 * a.Hkv;
    if (wid >= (long)a.T * H) return;
    const int t = (int)(wid / H), h = (int)(wid % H);
    const int Dh = a.Dh;
    const void* src;
    long off;
    int kind;  // 0 q, 1 k, 2 v
    if (h < a.Hq) { kind = 0; src = a.q; off = t * a.q_tok + h * a.q_head; }
    else if (h < a.Hq + a.Hkv) { kind = 1; src = a.k; off = t * a.k_tok + (h - a.Hq) * a.k_head; }
    else { kind = 2; src = a.v; off = t * a.v_tok + (h - a.Hq - a.Hkv) * a.v_head; }
    const long slot = a.slot ? a.slot[t] : -1;
    if (kind != 0 && slot < 0) return;
    // each lane holds up to NJ values: element e = lane + 32 * j
    float v[NJ];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        float x = 0.f;
        if (e < Dh) x = a.in_f32 ? reinterpret_cast<const float*>(src)[off + e]
                                  : bf2f(reinterpret_cast<const bf16*>(src)[off + e]);
        v[j] = x;
        ss += x * x;
    }
    const float* nw = kind == 0 ? a.qn : (kind == 1 ? a.kn : nullptr);
    // Everything else this warp will read (norm weights, cos / sin of its pairs) is requested here, next to
    // the inputs, so the kernel is one memory round trip deep instead of three.
    const int rot = a.rp.rot_dim;
    const bool tab = a.cs_table != nullptr && kind != 2 && rot > 0;
    float nwv[NJ];
    float2 csv[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        nwv[j] = (nw && e < Dh) ? nw[e] : 1.f;
        csv[j] = make_float2(1.f, 0.f);
        if (tab && e < rot) {
            const int pair = a.rp.mode == 0 ? (e < (rot >> 1) ? e : e - (rot >> 1)) : (e >> 1);
            csv[j] = a.cs_table[(long)t * (rot >> 1) + pair];
        }
    }
    if (nw || (kind == 2 && a.v_norm)) {
        ss = warp_sum(ss);
        const float rs = rsqrtf(ss / (float)Dh + a.eps);
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int e = lane + 32 * j;
            if (e < Dh) v[j] *= rs * nwv[j];
        }
    }
    bf16* dst;
    if (kind == 0) dst = a.q_out + ((long)t * a.Hq + h) * Dh;
    else if (kind == 1) dst = a.k_cache + (slot * a.Hkv + (h - a.Hq)) * Dh;
    else dst = a.v_cache + (slot * a.Hkv + (h - a.Hq - a.Hkv)) * Dh;
    if (kind == 2 || rot == 0) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int e = lane + 32 * j;
            if (e < Dh) dst[e] = f2bf(kind == 0 ? v[j] * a.q_scale : v[j]);
        }
        return;
    }
    const float pos = (float)a.pos[t];
    const float qs = kind == 0 ? a.q_scale : 1.f;
    if (a.rp.mode == 0) {
        // NeoX: element e pairs with e + rot/2.  The partner lives in another register or lane;
        // stage through shared memory (one row of 512 floats per warp).
        __shared__ float stage[4][512];
        float* st = stage[threadIdx.x >> 5];
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int e = lane + 32 * j;
            if (e < Dh) st[e] = v[j];
        }
        __syncwarp();
        const int half = rot >> 1;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int e = lane + 32 * j;
            if (e >= Dh) continue;
            float o = v[j];
            if (e < rot) {
                const int pair = e < half ? e : e - half;
                float c = csv[j].x, s = csv[j].y;
                if (!tab) rope_lookup(a, t, pair, pos, c, s);
                const float x0 = st[pair], x1 = st[pair + half];
                o = e < half ? x0 * c - x1 * s : x0 * s + x1 * c;
            }
            dst[e] = f2bf(o * qs);
        }
    } else {
        // adjacent pairs (2i, 2i+1): the partner is in the neighbouring lane
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int e = lane + 32 * j;
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
            if (e >= Dh) continue;
            float o = v[j];
            if (e < rot) {
                float c = csv[j].x, s = csv[j].y;
                if (!tab) rope_lookup(a, t, e >> 1, pos, c, s);
                o = (e & 1) ? other * s + v[j] * c : v[j] * c - other * s;
            }
            dst[e] = f2bf(o * qs);
        }
    }
}

extern "C" int tsb_qkv_rope(const QkvArgs* args, void* stream) {
    const QkvArgs& a = *args;
    TSB_CHECK_ARG(a.Dh > 0 && a.Dh <= 512, "qkv_rope: head dim %d out of range (1..512)", a.Dh);
    TSB_CHECK_ARG(a.rp.rot_dim <= a.Dh && a.rp.rot_dim % 2 == 0, "qkv_rope: bad rot_dim %d", a.rp.rot_dim);
    const long warps = (long)a.T * (a.Hq + 2 * a.Hkv);
    if (warps == 0) return TSB_OK;
    const dim3 grid((unsigned)((warps + 3) / 4)), block(128);
    cudaStream_t st = (cudaStream_t)stream;
    if (a.Dh <= 64) TSB_CHECK_CUDA(tsb_launch(qkv_rope_kernel<2>, grid, block, 0, st, a));
    else if (a.Dh <= 128) TSB_CHECK_CUDA(tsb_launch(qkv_rope_kernel<4>, grid, block, 0, st, a));
    else if (a.Dh <= 256) TSB_CHECK_CUDA(tsb_launch(qkv_rope_kernel<8>, grid, block, 0, st, a));
    else TSB_CHECK_CUDA(tsb_launch(qkv_rope_kernel<16>, grid, block, 0, st, a));
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// Gated activation: out[t, f] = act(gate[t, f] (+bg[f])) * (up[t, f] (+bu[f])), optional q8 output.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float glu_apply(int act, float g, float u) {
    switch (act) {
    case 1: return g / (1.f + __expf(-g)) * u;
    case 2: {
        const float c = 0.7978845608028654f;
        return 0.5f * g * (1.f + tanhf(c * (g + 0.044715f * g * g * g))) * u;
    }
    case 3: return 0.5f * g * (1.f + erff(g * 0.7071067811865476f)) * u;
    case 4: {
        const float x = fminf(g, 7.f), y = fminf(fmaxf(u, -7.f), 7.f);
        return x / (1.f + __expf(-1.702f * x)) * (y + 1.f);
    }
    case 5: { const float r = fmaxf(g, 0.f); return r * r; }             // ReLU^2 (no gate)
    case 6: return g / (1.f + __expf(-g));                                // SiLU (no gate)
    case 7: return u / (1.f + __expf(-g));                                // sigmoid(g) * u
    default: return g * u;
    }
}

template <typename T>
__global__ void glu_kernel(const T* gate, const T* up, long g_stride, long u_stride, int F, int act, bf16* out,
                           int8_t* yq, float2* yds, long rows) {
    pdl_wait();
    pdl_trigger();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int fpad = (F + 31) & ~31;
    const long total = rows * fpad;
    if (idx >= total) return;
    const long t = idx / fpad;
    const int f = (int)(idx % fpad);
    float r = 0.f;
    if (f < F) {
        const float g = (float)gate[t * g_stride + f];
        const float u = up ? (float)up[t * u_stride + f] : 0.f;
        r = glu_apply(act, g, u);
        if (out) out[t * F + f] = f2bf(r);
    }
    if (yq) {
        const float amax = warp_max(fabsf(r));
        const float sum = warp_sum(r);
        const float d = amax / 127.f;
        if (f < F) yq[t * F + f] = (int8_t)__float2int_rn(amax > 0.f ? r / d : 0.f);
        if ((threadIdx.x & 31) == 0 && f < F) yds[t * (F / 32) + f / 32] = make_float2(d, sum);
    }
}

extern "C" int tsb_glu(const void* gate, const void* up, int in_f32, long g_stride, long u_stride, long rows, int F,
                       int act, void* out, void* yq, void* yds, void* stream) {
    TSB_CHECK_ARG(!yq || F % 32 == 0, "glu: q8 output needs F %% 32 == 0, got %d", F);
    if (rows == 0 || F == 0) return TSB_OK;
    const long total = rows * ((F + 31) & ~31);
    dim3 grid((unsigned)((total + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    if (in_f32)
        TSB_CHECK_CUDA(tsb_launch(glu_kernel<float>, grid, dim3(256), 0, s, (const float*)gate, (const float*)up, g_stride,
                                  u_stride, F, act, (bf16*)out, (int8_t*)yq, (float2*)yds, rows));
    else
        TSB_CHECK_CUDA(tsb_launch(glu_kernel<bf16>, grid, dim3(256), 0, s, (const bf16*)gate, (const bf16*)up, g_stride,
                                  u_stride, F, act, (bf16*)out, (int8_t*)yq, (float2*)yds, rows));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// Row gather with dequantisation (embedding lookup when ids != null, whole-matrix decode to
// bf16 when ids == null).  One thread per 8 output values.
// ------------------------------------------------------------------------------------------
template <typename TO>
__global__ void gather_rows_kernel(QW w, const int* ids, long n_rows, float scale, TO* out) {
    pdl_wait();
    pdl_trigger();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int k8n = w.K >> 3;
    if (idx >= n_rows * k8n) return;
    const long r = idx / k8n;
    const int k8 = (int)(idx % k8n);
    long src = ids ? (long)ids[r] : r;
    if (src < 0 || src >= w.N) src = 0;
    float v[8];
    dequant8(w, src, k8, v);
    TO* o = out + r * w.K + 8 * k8;
    if (sizeof(TO) == 2) {
        bf16 b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = f2bf(v[i] * scale);
        *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(b);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (TO)(v[i] * scale);
    }
}

extern "C" int tsb_gather_rows(const void* p0, const void* p1, const void* p2, const void* p3, int type, int N, int K,
                               const int* ids, long n_rows, float scale, void* out, int out_f32, void* stream) {
    TSB_CHECK_ARG(K % 8 == 0, "gather_rows: K=%d must be a multiple of 8", K);
    if (n_rows == 0) return TSB_OK;
    QW w{(const uint8_t*)p0, (const uint8_t*)p1, (const uint8_t*)p2, (const uint8_t*)p3, type, N, K};
    const long total = n_rows * (K / 8);
    dim3 grid((unsigned)((total + 255) / 256));
    if (out_f32)
        TSB_CHECK_CUDA(tsb_launch(gather_rows_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, w, ids, n_rows, scale, (float*)out));
    else
        TSB_CHECK_CUDA(tsb_launch(gather_rows_kernel<bf16>, grid, dim3(256), 0, (cudaStream_t)stream, w, ids, n_rows, scale, (bf16*)out));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// Row arg-max over float logits with optional soft-cap (cap * tanh(x / cap)).  One block per row.
// Ties resolve to the lowest index, like the host sampler.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) argmax_kernel(const float* logits, long stride, int V, int* out_idx,
                                                      float* out_val) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_wait();
    pdl_trigger();
    const float* row = logits + blockIdx.x * stride;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = best; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            out_idx[blockIdx.x] = bi;
            if (out_val) out_val[blockIdx.x] = best;
        }
    }
}

// Large vocabularies: the row is cut into chunks of 4096 logits, one CTA each; every CTA leaves its
// best (value, index) in a per-device scratch and takes a ticket, and the CTA that draws the last
// ticket of a row merges the chunk results and resets the ticket counter for the next call.  Calls
// on one device share the scratch, so they must be ordered (same stream), as the decode loop's are.
#define ARGMAX_CHUNK 4096
#define ARGMAX_MAX_CHUNKS 128
#define ARGMAX_MAX_ROWS 1024
static __device__ float g_argmax_val[ARGMAX_MAX_ROWS * ARGMAX_MAX_CHUNKS];
static __device__ int g_argmax_idx[ARGMAX_MAX_ROWS * ARGMAX_MAX_CHUNKS];
static __device__ unsigned g_argmax_ticket[ARGMAX_MAX_ROWS];

__global__ void __launch_bounds__(256) argmax_chunk_kernel(const float* logits, long stride, int V, int chunks, int* out_idx,
                                                           float* out_val) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ bool last;
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.y, ch = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const float* r = logits + row * stride;
    const int i0 = ch * ARGMAX_CHUNK, i1 = min(V, i0 + ARGMAX_CHUNK);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = i0 + threadIdx.x * 4; i < i1; i += 1024) {
        if (i + 3 < i1 && ((reinterpret_cast<size_t>(r + i) & 15) == 0)) {
            const float4 v = *reinterpret_cast<const float4*>(r + i);
            const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (vv[j] > best) { best = vv[j]; bi = i + j; }
        } else {
            for (int j = i; j < min(i + 4, i1); ++j)
                if (r[j] > best) { best = r[j]; bi = j; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sv[w] = best; si[w] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i)
            if (sv[i] > best || (sv[i] == best && si[i] < bi)) { best = sv[i]; bi = si[i]; }
        g_argmax_val[row * ARGMAX_MAX_CHUNKS + ch] = best;
        g_argmax_idx[row * ARGMAX_MAX_CHUNKS + ch] = bi;
        __threadfence();
        last = atomicAdd(&g_argmax_ticket[row], 1u) == (unsigned)chunks - 1u;
    }
    __syncthreads();
    if (!last || w != 0) return;
    __threadfence();
    best = -INFINITY;
    bi = 0x7fffffff;
    for (int c = lane; c < chunks; c += 32) {
        const float v = __ldcg(&g_argmax_val[row * ARGMAX_MAX_CHUNKS + c]);
        const int i = __ldcg(&g_argmax_idx[row * ARGMAX_MAX_CHUNKS + c]);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
        out_idx[row] = bi == 0x7fffffff ? 0 : bi;
        if (out_val) out_val[row] = best;
        g_argmax_ticket[row] = 0u;
    }
}

extern "C" int tsb_argmax(const float* logits, long stride, long rows, int V, int* out_idx, float* out_val,
                          void* stream) {
    if (rows == 0) return TSB_OK;
    TSB_CHECK_ARG(V > 0, "argmax: empty vocabulary");
    const int chunks = (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    if (chunks >= 4 && chunks <= ARGMAX_MAX_CHUNKS && rows <= ARGMAX_MAX_ROWS) {
        TSB_CHECK_CUDA(tsb_launch(argmax_chunk_kernel, dim3(chunks, (unsigned)rows), dim3(256), 0, (cudaStream_t)stream, logits,
                                  stride, V, chunks, out_idx, out_val));
        TSB_CHECK_LAUNCH();
        return TSB_OK;
    }
    TSB_CHECK_CUDA(tsb_launch(argmax_kernel, dim3((unsigned)rows), dim3(1024), 0, (cudaStream_t)stream, logits, stride, V, out_idx, out_val));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// Decode bookkeeping on the device, so that a captured decode graph can run step after step
// without the host: feed the sampled ids back as the next inputs, advance positions and
// cache lengths, and look up the KV slot of the new position in the block table.
// ------------------------------------------------------------------------------------------
__global__ void decode_advance_kernel(const int* sampled, int* tokens, int* positions, int* kv_lens, long* slots,
                                      const int* block_table, int max_pages, int page_size, int B) {
    pdl_wait();
    pdl_trigger();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    tokens[b] = sampled[b];
    const int p = positions[b] + 1;
    positions[b] = p;
    kv_lens[b] = p + 1;
    int page = p / page_size;
    if (page >= max_pages) page = max_pages - 1;   // out of reserved pages: stay inside the table
    slots[b] = (long)block_table[(long)b * max_pages + page] * page_size + p % page_size;
}

extern "C" int tsb_decode_advance(const int* sampled, int* tokens, int* positions, int* kv_lens, long* slots,
                                  const int* block_table, int max_pages, int page_size, int B, void* stream) {
    if (B == 0) return TSB_OK;
    TSB_CHECK_CUDA(tsb_launch(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, (cudaStream_t)stream, sampled,
                              tokens, positions, kv_lens, slots, block_table, max_pages, page_size, B));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}
