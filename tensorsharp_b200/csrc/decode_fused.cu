// Decode-path GEMV with the activation prologue inside the kernel.
//
// A decode step is a chain of small dependent kernels, each costing a few microseconds of launch
// and first-load latency however little it computes.  This kernel removes two links per
// projection: the RMSNorm (or plain cast) and the int8 quantisation of the activations run in
// every CTA, into shared memory, while the CTA's first weight loads are already in flight; the
// weights are then streamed against the shared-memory copy.  Re-doing a 2560..9728-element norm
// in each of a few hundred CTAs costs L2 reads only (the row is tiny), no extra DRAM traffic.
//
//   y[m, n] = act( W[n, :] . q8( RMSNorm(x[m, :]) * g ) + bias[n] ) + residual[m, n]
//
// x is the f32 residual stream (norm mode) or a bf16 activation (cast mode).  Eight rows per CTA,
// one warp per row (a gate / up row pair with GLU).  The arithmetic contract is that of the
// separate kernels (tsb_rmsnorm with q8 output, then tsb_gemv), so results match them bit for bit.
//
// Replaces in the reference: rms_norm_f32 + mul fusion, quantize_q8_1 and mul_mat_vec_q as three
// launches (ggml-cuda/norm.cu, quantize.cu:5, mmvq.cu:143).
#include "gemv_core.cuh"

struct FusedGemvArgs {
    QW w;
    const float* xf;       // [M, K] f32 input, or null
    const bf16* xb;        // [M, K] bf16 input when xf is null
    const float* norm_w;   // [K] RMSNorm weight or null
    float eps;
    int do_norm;           // apply RMSNorm (weighted when norm_w != null) before quantising
    void* out;             // [M, n_out]
    const float* bias;     // [N] or null
    const void* residual;  // [M, n_out] in the output dtype, or null
    int M, out_f32, act, n_out;
    const TpPush* push;    // tensor-parallel partial-sum exchange instead of `out` (tp_fused.cuh)
};

#define FG_THREADS 256
#define FG_ROWS 8

// Stage row m of the input into shared memory: int8 groups of 32 with (scale, sum) for quantised
// weight types, bf16 for float weight types.  A group of 32 values is 8 neighbouring lanes.
template <bool FLOATW>
__device__ __forceinline__ void stage_row(const FusedGemvArgs& a, int m, int8_t* sq, float2* sds, bf16* sb, float* red) {
    const int K = a.w.K, nvec = K >> 2, tid = threadIdx.x;
    constexpr int VMAX = 10;                         // K <= 10240
    float4 v[VMAX];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
        const int i = tid + j * FG_THREADS;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nvec) {
            if (a.xf) {
                t = reinterpret_cast<const float4*>(a.xf + (long)m * K)[i];
            } else {
                const uint2 r = reinterpret_cast<const uint2*>(a.xb + (long)m * K)[i];
                const float2 p = __bfloat1622float2(*reinterpret_cast<const bf162*>(&r.x));
                const float2 q = __bfloat1622float2(*reinterpret_cast<const bf162*>(&r.y));
                t = make_float4(p.x, p.y, q.x, q.y);
            }
        }
        v[j] = t;
        ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
    }
    float rs = 1.f;
    if (a.do_norm) {
        ss = block_sum(ss, red);
        rs = rsqrtf(ss / (float)K + a.eps);
    }
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
        const int i = tid + j * FG_THREADS;
        if (j * FG_THREADS >= nvec) break;           // uniform across the CTA
        const bool ok = i < nvec;
        float4 n = v[j];
        if (a.do_norm) {
            float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
            if (a.norm_w && ok) g = reinterpret_cast<const float4*>(a.norm_w)[i];
            n = make_float4(n.x * rs * g.x, n.y * rs * g.y, n.z * rs * g.z, n.w * rs * g.w);
        }
        if (FLOATW) {
            if (ok) {
                uint2 o;
                *reinterpret_cast<bf162*>(&o.x) = __floats2bfloat162_rn(n.x, n.y);
                *reinterpret_cast<bf162*>(&o.y) = __floats2bfloat162_rn(n.z, n.w);
                reinterpret_cast<uint2*>(sb + (long)m * K)[i] = o;
            }
        } else {
            if (!a.do_norm && a.xf == nullptr) {
                // cast mode quantises what a bf16 tensor holds (already exact in n)
            }
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
                reinterpret_cast<char4*>(sq + (long)m * K)[i] = q;
                if ((i & 7) == 0) sds[(long)m * (K >> 5) + (i >> 3)] = make_float2(amax / 127.f, sum);
            }
        }
    }
}

template <int M, bool FLOATW>
struct StagePrologue {
    const FusedGemvArgs& a;
    int8_t* sq; float2* sds; bf16* sb; float* red;
    __device__ __forceinline__ void operator()() const {
        pdl_wait();
        pdl_trigger();
#pragma unroll
        for (int m = 0; m < M; ++m)
            if (m < a.M) stage_row<FLOATW>(a, m, sq, sds, sb, red);
        __syncthreads();
    }
};

template <int M, bool GLU, bool FLOATW>
__device__ __forceinline__ void fused_epilogue(const FusedGemvArgs& a, int r, int lane, int mv, float* acc, float* acc2) {
    const int n_out = a.n_out;
#pragma unroll
    for (int m = 0; m < M; ++m) {
        acc[m] = warp_sum(acc[m]);
        if (GLU) acc2[m] = warp_sum(acc2[m]);
    }
    if (r >= n_out) return;                          // shadow row of an idle warp
    if (a.push != nullptr) {
        const TpPush* tp = a.push;
        const unsigned epoch = *tp->epoch;
        if (lane < tp->size) {
            float2* dst = tp->mailbox[lane] + (long)(epoch % TP_SLOTS) * tp->slot_stride + (long)tp->rank * tp->src_stride;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                if (m >= mv) break;
                float v = acc[m];
                if (a.bias && tp->rank == 0) v += a.bias[r];
                st_word(dst + (long)m * n_out + r, v, epoch + 1);
            }
        }
        return;
    }
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m >= mv) break;
            float v = acc[m];
            if (a.bias) v += a.bias[r];
            if (GLU) {
                float u = acc2[m];
                if (a.bias) u += a.bias[r + n_out];
                v = act_glu(a.act, v, u);
            } else if (a.act == ACT_RELU2) {
                v = fmaxf(v, 0.f);
                v = v * v;
            }
            const long o = (long)m * n_out + r;
            if (a.out_f32) {
                if (a.residual) v += reinterpret_cast<const float*>(a.residual)[o];
                reinterpret_cast<float*>(a.out)[o] = v;
            } else {
                if (a.residual) v += bf2f(reinterpret_cast<const bf16*>(a.residual)[o]);
                reinterpret_cast<bf16*>(a.out)[o] = f2bf(v);
            }
        }
    }
}

// The grid is sized so that every warp owns `rows_per_warp` rows, strided by the number of warps
// in the grid: the prologue is paid once per CTA and all CTAs are resident in one wave.
template <int M, bool GLU, bool FLOATW>
__global__ void __launch_bounds__(FG_THREADS) fused_gemv_kernel(FusedGemvArgs a, int rows_per_warp) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float red[32];
    const int K = a.w.K;
    int8_t* sq = reinterpret_cast<int8_t*>(smem);
    float2* sds = reinterpret_cast<float2*>(smem + (size_t)M * K);
    bf16* sb = reinterpret_cast<bf16*>(smem);
    const int lane = threadIdx.x & 31;
    const int stride = gridDim.x * FG_ROWS;
    int r = blockIdx.x * FG_ROWS + (threadIdx.x >> 5);
    const int n_out = a.n_out;
    const int mv = min(M, a.M);
    float acc[M], acc2[M];
    {
        const int row = r < n_out ? r : n_out - 1;   // idle warps shadow a valid row: the prologue needs every thread
#pragma unroll
        for (int m = 0; m < M; ++m) { acc[m] = 0.f; acc2[m] = 0.f; }
        StagePrologue<M, FLOATW> pro{a, sq, sds, sb, red};
        dot_row<M>(a.w, row, lane, sq, sds, sb, acc, mv, pro);
        if (GLU) dot_row<M>(a.w, (long)row + n_out, lane, sq, sds, sb, acc2, mv, PdlWait{false});
        fused_epilogue<M, GLU, FLOATW>(a, r, lane, mv, acc, acc2);
    }
    for (int j = 1; j < rows_per_warp; ++j) {
        r += stride;
        if (r >= n_out) break;
#pragma unroll
        for (int m = 0; m < M; ++m) { acc[m] = 0.f; acc2[m] = 0.f; }
        dot_row<M>(a.w, r, lane, sq, sds, sb, acc, mv, PdlWait{false});
        if (GLU) dot_row<M>(a.w, (long)r + n_out, lane, sq, sds, sb, acc2, mv, PdlWait{false});
        fused_epilogue<M, GLU, FLOATW>(a, r, lane, mv, acc, acc2);
    }
}

static int fused_max_ctas() {
    static int n = 0;
    if (n == 0) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        n = 2 * sms;
    }
    return n;
}

template <int M, bool GLU, bool FLOATW>
static int launch_fused(const FusedGemvArgs& a, cudaStream_t s) {
    const size_t smem = FLOATW ? (size_t)M * a.w.K * 2 : (size_t)M * a.w.K + (size_t)M * (a.w.K >> 5) * 8;
    auto kern = fused_gemv_kernel<M, GLU, FLOATW>;
    if (smem > 48 * 1024) TSB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int blocks = (a.n_out + FG_ROWS - 1) / FG_ROWS;
    const int rpw = (blocks + fused_max_ctas() - 1) / fused_max_ctas();
    dim3 grid((blocks + rpw - 1) / rpw);
    TSB_CHECK_CUDA(tsb_launch(kern, grid, dim3(FG_THREADS), smem, s, a, rpw));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

template <bool GLU, bool FLOATW>
static int launch_fused_m(const FusedGemvArgs& a, cudaStream_t s) {
    switch (a.M) {
    case 1: return launch_fused<1, GLU, FLOATW>(a, s);
    case 2: return launch_fused<2, GLU, FLOATW>(a, s);
    case 3:
    case 4: return launch_fused<4, GLU, FLOATW>(a, s);
    default: tsb_set_error("fused_gemv: M=%d (at most 4 rows)", a.M); return TSB_ERR_ARG;
    }
}

// y = act(W . stage(x) + bias) + residual, where stage(x) is RMSNorm(x) * norm_w (do_norm) or x,
// quantised in the kernel.  Exactly one of x_f32 / x_bf16 is given.  With `push` the f32 result
// goes to the tensor-parallel mailboxes instead of `out` (no act / residual then).
extern "C" int tsb_fused_gemv(const void* p0, const void* p1, const void* p2, const void* p3, int type, int N, int K,
                              const float* x_f32, const void* x_bf16, const float* norm_w, float eps, int do_norm,
                              void* out, const float* bias, const void* residual, int M, int out_f32, int act,
                              const void* push, void* stream) {
    TSB_CHECK_ARG(N > 0 && K > 0 && M >= 1 && M <= 4, "fused_gemv: bad shape N=%d K=%d M=%d", N, K, M);
    TSB_CHECK_ARG((x_f32 != nullptr) != (x_bf16 != nullptr), "fused_gemv: give exactly one of x_f32 / x_bf16");
    TSB_CHECK_ARG(K % 32 == 0 && K <= 10240, "fused_gemv: K=%d must be a multiple of 32 and at most 10240", K);
    const bool kq = type == TSB_Q4_K || type == TSB_Q5_K || type == TSB_Q6_K;
    TSB_CHECK_ARG(!kq || K % 256 == 0, "fused_gemv: K=%d not a whole number of super-blocks for type %d", K, type);
    const bool glu = act >= ACT_SWIGLU && act <= ACT_SWIGLU_OAI;
    TSB_CHECK_ARG(!glu || N % 2 == 0, "fused_gemv: GLU needs an even row count, got %d", N);
    TSB_CHECK_ARG(!push || (!residual && act == 0), "fused_gemv: push mode takes no residual / act");
    TSB_CHECK_ARG(push || out, "fused_gemv: no output");
    FusedGemvArgs a;
    a.w = QW{(const uint8_t*)p0, (const uint8_t*)p1, (const uint8_t*)p2, (const uint8_t*)p3, type, N, K};
    a.xf = x_f32; a.xb = (const bf16*)x_bf16; a.norm_w = norm_w; a.eps = eps; a.do_norm = do_norm;
    a.out = out; a.bias = bias; a.residual = residual; a.M = M; a.out_f32 = out_f32; a.act = act;
    a.n_out = glu ? N / 2 : N;
    a.push = (const TpPush*)push;
    const bool floatw = !(type == TSB_Q4_K || type == TSB_Q5_K || type == TSB_Q6_K || type == TSB_Q8_0 ||
                          type == TSB_MXFP4 || type == TSB_Q4_0);
    cudaStream_t s = (cudaStream_t)stream;
    if (floatw) return glu ? launch_fused_m<true, true>(a, s) : launch_fused_m<false, true>(a, s);
    return glu ? launch_fused_m<true, false>(a, s) : launch_fused_m<false, false>(a, s);
}
