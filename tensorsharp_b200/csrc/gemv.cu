// Weight-streaming GEMV / small-batch GEMM over GGUF-quantised weights (decode path).
//
//   out[m, n] = sum_k W[n, k] * x[m, k]  (+ bias[n]) (+ residual[m, n])      m < M <= 8 per pass
//
// One warp owns one output row (or a gate/up row pair when a GLU epilogue is requested) and
// streams that row's blocks with 16-byte loads; activations are pre-quantised to int8 in
// groups of 32 with a float scale and the group's float sum (same arithmetic contract as
// ggml's q8_1 activations), so the inner product is dp4a.  Weights are read exactly once
// per call; activations come from L1.  The optional `ids` argument turns the launch into a
// mixture-of-experts GEMV: problem p uses expert ids[p], activation row p / x_div and
// output row p.
//
// Replaces in the reference: mul_mat_vec_q + quantize_q8_1 (ggml-cuda/mmvq.cu:143,
// quantize.cu:5), mul_mat_vec_f (mmvf.cu:8), the bias / GLU fusion of
// ggml-cuda.cu:3359-3790 item (5), and the per-expert unrolled graphs of
// TensorSharp.GGML.Native/ggml_ops_fused.cpp:1766 for the single-token case.
#include <cstdlib>
#include "gemv_core.cuh"

// Row-parallel projection of a tensor-parallel layer: the result is this rank's partial sum, so
// instead of writing it to a local tensor the warp stores it, tagged with the exchange number,
// into the mailbox of every rank (tp_fused.cuh).  GEMM -> reduce in one kernel: the NVLink stores
// of early rows overlap the weight streaming of later rows, and nothing waits or fences.
template <int M, bool GLU>
__device__ __forceinline__ void gemv_push_body(const GemvArgs& a, int r, int lane) {
    const TpPush* tp = a.push;
    const int n_out = a.n_out;
    if (r >= n_out) return;
    const int orow = blockIdx.y * M;
    const int mv = min(M, a.M - orow);
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    const int K = a.w.K, kb = K >> 5;
    const int8_t* xq = a.xq ? a.xq + (long)orow * K : nullptr;
    const float2* xds = a.xds ? a.xds + (long)orow * kb : nullptr;
    const bf16* xb = a.xb ? a.xb + (long)orow * K : nullptr;
    dot_row<M>(a.w, r, lane, xq, xds, xb, acc, mv, PdlWait{true});
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = warp_sum(acc[m]);
    const unsigned epoch = *tp->epoch;              // stable: the consumer of this exchange runs after this kernel
    if (lane < tp->size) {
        // lane q stores to rank q, so all peers are written in parallel
        float2* dst = tp->mailbox[lane] + (long)(epoch % TP_SLOTS) * tp->slot_stride + (long)tp->rank * tp->src_stride;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m >= mv) break;
            float v = acc[m];
            if (a.bias && tp->rank == 0) v += a.bias[r];
            st_word(dst + (long)(orow + m) * n_out + r, v, epoch + 1);
        }
    }
}

template <int M, bool GLU>
__global__ void __launch_bounds__(128) gemv_kernel(GemvArgs a) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int n_out = a.n_out;
    if (a.push != nullptr && a.ids == nullptr) {
        gemv_push_body<M, GLU>(a, r, lane);
        return;
    }
    if (r >= n_out) return;
    const int p = blockIdx.y;                       // problem (MoE slot) or M-chunk
    int expert = 0, xrow, orow;
    if (a.ids) {
        pdl_wait();                                 // expert ids come from the router kernel
        pdl_trigger();
        expert = a.ids[p];
        if (expert < 0) {
            // expert-parallel combine: a slot whose expert lives on another rank still has to
            // arrive (as zero) in every mailbox, or the consumer would wait for it
            if (a.push != nullptr) gemv_push_store(a.push, lane, (long)p * n_out + r, 0.f);
            return;
        }
        xrow = p / a.x_div;
        orow = p;
    } else {
        xrow = p * M;
        orow = p * M;
    }
    const int K = a.w.K, kb = K >> 5;
    const int8_t* xq = a.xq ? a.xq + (long)xrow * K : nullptr;
    const float2* xds = a.xds ? a.xds + (long)xrow * kb : nullptr;
    const bf16* xb = a.xb ? a.xb + (long)xrow * K : nullptr;
    const long wrow = (long)expert * a.w.N + r;
    float acc[M], acc2[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { acc[m] = 0.f; acc2[m] = 0.f; }
    const int mv = a.ids ? 1 : min(M, a.M - orow);
    if (GLU && M <= 4) dot_row2<M>(a.w, wrow, wrow + n_out, lane, xq, xds, xb, acc, acc2, mv, PdlWait{a.ids == nullptr});
    else {
        dot_row<M>(a.w, wrow, lane, xq, xds, xb, acc, mv, PdlWait{a.ids == nullptr});
        if (GLU) dot_row<M>(a.w, wrow + n_out, lane, xq, xds, xb, acc2, mv, PdlWait{false});
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        acc[m] = warp_sum(acc[m]);
        if (GLU) acc2[m] = warp_sum(acc2[m]);
    }
    if (lane == 0) {
        const int mrows = mv;
        for (int m = 0; m < M; ++m) {
            if (m >= mrows) break;
            float v = acc[m];
            if (a.bias) v += a.bias[(long)expert * a.w.N + r];
            if (GLU) {
                float u = acc2[m];
                if (a.bias) u += a.bias[(long)expert * a.w.N + r + n_out];
                v = act_glu(a.act, v, u);
            } else if (a.act == ACT_RELU2) {
                v = fmaxf(v, 0.f);
                v = v * v;
            }
            if (a.row_scale) v *= a.row_scale[orow + m];
            const long o = (long)(orow + m) * n_out + r;
            if (a.push != nullptr) {                // MoE down projection: the weighted slot row goes to every rank
                acc[m] = v;
                continue;
            }
            if (a.out_f32) {
                if (a.residual) v += reinterpret_cast<const float*>(a.residual)[o];
                reinterpret_cast<float*>(a.out)[o] = v;
            } else {
                if (a.residual) v += bf2f(reinterpret_cast<const bf16*>(a.residual)[o]);
                reinterpret_cast<bf16*>(a.out)[o] = f2bf(v);
            }
        }
    }
    if (a.push != nullptr) {
        const float v = __shfl_sync(0xffffffffu, acc[0], 0);          // ids mode runs one row per problem
        gemv_push_store(a.push, lane, (long)orow * n_out + r, v);
    }
}

// Few output rows, long rows (o_proj, down, K / V projections at batch 1): one warp per row leaves
// most of the GPU's warp slots empty and each warp walks its row as a chain of dependent DRAM
// round trips.  Here the four warps of a CTA share one row (every fourth group of 32 units each)
// and add their partial sums through shared memory, so four times as many loads are in flight.
template <int M, bool PUSH>
__global__ void __launch_bounds__(128) gemv_split_kernel(GemvArgs a) {
    __shared__ float part_sum[4][M];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x;
    const int n_out = a.n_out;
    const int orow = blockIdx.y * M;
    const int mv = min(M, a.M - orow);
    const int K = a.w.K, kb = K >> 5;
    const int8_t* xq = a.xq ? a.xq + (long)orow * K : nullptr;
    const float2* xds = a.xds ? a.xds + (long)orow * kb : nullptr;
    const bf16* xb = a.xb ? a.xb + (long)orow * K : nullptr;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    dot_row<M>(a.w, r, lane, xq, xds, xb, acc, mv, PdlWait{true}, warp, 4);
#pragma unroll
    for (int m = 0; m < M; ++m) {
        acc[m] = warp_sum(acc[m]);
        if (lane == 0) part_sum[warp][m] = acc[m];
    }
    __syncthreads();
    if (warp != 0) return;
    if (PUSH) {
        const TpPush* tp = a.push;
        const unsigned epoch = *tp->epoch;
        if (lane < tp->size) {
            float2* dst = tp->mailbox[lane] + (long)(epoch % TP_SLOTS) * tp->slot_stride + (long)tp->rank * tp->src_stride;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                if (m >= mv) break;
                float v = part_sum[0][m] + part_sum[1][m] + part_sum[2][m] + part_sum[3][m];
                if (a.bias && tp->rank == 0) v += a.bias[r];
                st_word(dst + (long)(orow + m) * n_out + r, v, epoch + 1);
            }
        }
        return;
    }
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m >= mv) break;
            float v = part_sum[0][m] + part_sum[1][m] + part_sum[2][m] + part_sum[3][m];
            if (a.bias) v += a.bias[r];
            if (a.act == ACT_RELU2) {
                v = fmaxf(v, 0.f);
                v = v * v;
            }
            if (a.row_scale) v *= a.row_scale[orow + m];
            const long o = (long)(orow + m) * n_out + r;
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

// Up to three weight matrices that share one input (Q, K and V projections kept apart in the file
// because their quantisation types differ) in one launch: the rows of all matrices form one row
// space, a warp looks up which matrix its row belongs to, and the results land side by side in one
// [M, N0 + N1 + N2] output.  Saves two launches per layer in the latency-bound decode step.
struct GemvMultiArgs {
    QW w[3];
    int n_w;
    int row_end[3];          // cumulative row counts
    const int8_t* xq;
    const float2* xds;
    const bf16* xb;
    void* out;
    int M, out_f32, n_total;
};

template <int M>
__global__ void __launch_bounds__(128) gemv_multi_kernel(GemvMultiArgs a) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= a.n_total) return;
    const int wi = r < a.row_end[0] ? 0 : (r < a.row_end[1] ? 1 : 2);
    const QW w = a.w[wi];
    const int lr = r - (wi ? a.row_end[wi - 1] : 0);
    const int orow = blockIdx.y * M;
    const int mv = min(M, a.M - orow);
    const int K = w.K, kb = K >> 5;
    const int8_t* xq = a.xq ? a.xq + (long)orow * K : nullptr;
    const float2* xds = a.xds ? a.xds + (long)orow * kb : nullptr;
    const bf16* xb = a.xb ? a.xb + (long)orow * K : nullptr;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    dot_row<M>(w, lr, lane, xq, xds, xb, acc, mv, PdlWait{true});
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = warp_sum(acc[m]);
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m >= mv) break;
            const long o = (long)(orow + m) * a.n_total + r;
            if (a.out_f32) reinterpret_cast<float*>(a.out)[o] = acc[m];
            else reinterpret_cast<bf16*>(a.out)[o] = f2bf(acc[m]);
        }
    }
}

// x [M, K] (bf16 or f32) -> int8 groups of 32 with (scale, float sum).  One warp per group.
template <typename T>
__global__ void quantize_q8_kernel(const T* x, int8_t* xq, float2* xds, long n_groups) {
    const long g = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_wait();
    pdl_trigger();
    if (g >= n_groups) return;
    const int lane = threadIdx.x & 31;
    const float v = (float)x[g * 32 + lane];
    const float amax = warp_max(fabsf(v));
    const float sum = warp_sum(v);
    const float d = amax / 127.f;
    const float q = (amax > 0.f) ? v / d : 0.f;
    xq[g * 32 + lane] = (int8_t)__float2int_rn(q);
    if (lane == 0) xds[g] = make_float2(d, sum);
}

static bool type_uses_q8(int t) {
    return t == TSB_Q4_K || t == TSB_Q5_K || t == TSB_Q6_K || t == TSB_Q8_0 || t == TSB_MXFP4 || t == TSB_Q4_0;
}

extern "C" int tsb_quantize_q8(const void* x, int x_is_f32, void* xq, void* xds, long rows, int K, void* stream) {
    TSB_CHECK_ARG(K % 32 == 0, "quantize_q8: K=%d is not a multiple of 32", K);
    const long groups = rows * (K / 32);
    if (groups == 0) return TSB_OK;
    const int wpb = 8;
    dim3 grid((unsigned)((groups + wpb - 1) / wpb)), block(32 * wpb);
    cudaStream_t s = (cudaStream_t)stream;
    if (x_is_f32)
        TSB_CHECK_CUDA(tsb_launch(quantize_q8_kernel<float>, grid, block, 0, s, (const float*)x, (int8_t*)xq, (float2*)xds, groups));
    else
        TSB_CHECK_CUDA(tsb_launch(quantize_q8_kernel<bf16>, grid, block, 0, s, (const bf16*)x, (int8_t*)xq, (float2*)xds, groups));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

bool tsb_gemv_stream_eligible(const GemvArgs& a);                     // gemv_stream.cu
int tsb_gemv_stream_launch(const GemvArgs& a, bool glu, cudaStream_t s);
bool tsb_gemv_mma_eligible(const GemvArgs& a);                        // gemv_mma.cu
int tsb_gemv_mma_launch(const GemvArgs& a, bool glu, cudaStream_t s);

template <bool GLU>
static int launch_gemv(const GemvArgs& a, int problems, cudaStream_t s) {
    const int rows = a.n_out;
    dim3 block(128);
    // One row per CTA (4 warps share it).  Off unless TSB_GEMV_SPLIT=1 (K >= 4096) or 2 (K >= 2048):
    // inside the graph-replayed decode step it measured slower than one warp per row (2.68 ms
    // against 2.60 ms per step on Qwen3-4B), although each kernel alone has more loads in flight.
    static const int split_mode = []() { const char* e = getenv("TSB_GEMV_SPLIT"); return e ? atoi(e) : 0; }();
    if (split_mode && !GLU && !a.ids && a.M <= 4 && rows <= 4096 && a.w.K >= (split_mode == 2 ? 2048 : 4096)) {
        dim3 grid(rows, 1);
        const bool push = a.push != nullptr;
        if (a.M <= 1) TSB_CHECK_CUDA(push ? tsb_launch(gemv_split_kernel<1, true>, grid, block, 0, s, a) : tsb_launch(gemv_split_kernel<1, false>, grid, block, 0, s, a));
        else if (a.M <= 2) TSB_CHECK_CUDA(push ? tsb_launch(gemv_split_kernel<2, true>, grid, block, 0, s, a) : tsb_launch(gemv_split_kernel<2, false>, grid, block, 0, s, a));
        else TSB_CHECK_CUDA(push ? tsb_launch(gemv_split_kernel<4, true>, grid, block, 0, s, a) : tsb_launch(gemv_split_kernel<4, false>, grid, block, 0, s, a));
        TSB_CHECK_LAUNCH();
        return TSB_OK;
    }
    if (a.ids) {
        dim3 grid((rows + 3) / 4, problems);
        TSB_CHECK_CUDA(tsb_launch(gemv_kernel<1, GLU>, grid, block, 0, s, a));
    } else {
        const int M = a.M;
        if (M <= 1) { dim3 grid((rows + 3) / 4, 1); TSB_CHECK_CUDA(tsb_launch(gemv_kernel<1, GLU>, grid, block, 0, s, a)); }
        else if (M <= 2) { dim3 grid((rows + 3) / 4, 1); TSB_CHECK_CUDA(tsb_launch(gemv_kernel<2, GLU>, grid, block, 0, s, a)); }
        else if (M <= 4) { dim3 grid((rows + 3) / 4, 1); TSB_CHECK_CUDA(tsb_launch(gemv_kernel<4, GLU>, grid, block, 0, s, a)); }
        else { dim3 grid((rows + 3) / 4, (M + 7) / 8); TSB_CHECK_CUDA(tsb_launch(gemv_kernel<8, GLU>, grid, block, 0, s, a)); }
    }
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}

extern "C" int tsb_gemv_push(const void* p0, const void* p1, const void* p2, const void* p3, int type, int N, int K,
                             const void* xq, const void* xds, const void* xb, void* out, const float* bias,
                             const void* residual, const int* ids, const float* row_scale, int M, int problems,
                             int x_div, int out_f32, int act, const void* push, void* stream);

// out = act(W x + bias) * row_scale + residual.  See GemvArgs for the meaning of each field.
extern "C" int tsb_gemv(const void* p0, const void* p1, const void* p2, const void* p3, int type, int N, int K,
                        const void* xq, const void* xds, const void* xb, void* out, const float* bias,
                        const void* residual, const int* ids, const float* row_scale, int M, int problems,
                        int x_div, int out_f32, int act, void* stream) {
    return tsb_gemv_push(p0, p1, p2, p3, type, N, K, xq, xds, xb, out, bias, residual, ids, row_scale, M, problems, x_div,
                         out_f32, act, nullptr, stream);
}

// Same as tsb_gemv; with `push` != null the result goes to the tensor-parallel mailboxes (f32
// partial sums, bias added by rank 0 only) and `out`, `residual`, `ids`, `row_scale` and GLU must
// not be given.  The row length of the mailbox layout is N.
extern "C" int tsb_gemv_push(const void* p0, const void* p1, const void* p2, const void* p3, int type, int N, int K,
                             const void* xq, const void* xds, const void* xb, void* out, const float* bias,
                             const void* residual, const int* ids, const float* row_scale, int M, int problems,
                             int x_div, int out_f32, int act, const void* push, void* stream) {
    TSB_CHECK_ARG(N > 0 && K > 0 && M >= 0, "gemv: bad shape N=%d K=%d M=%d", N, K, M);
    TSB_CHECK_ARG(!push || (!residual && act == 0), "gemv: push mode takes no residual / act");
    TSB_CHECK_ARG(!push || ids || !row_scale, "gemv: push mode takes a row scale only with expert ids");
    const bool q8 = type_uses_q8(type);
    TSB_CHECK_ARG(!q8 || (xq && xds), "gemv: quantised weight type %d needs int8 activations", type);
    TSB_CHECK_ARG(q8 || xb, "gemv: float weight type %d needs bf16 activations", type);
    const bool kq = type == TSB_Q4_K || type == TSB_Q5_K || type == TSB_Q6_K;
    TSB_CHECK_ARG(K % (kq ? 256 : 32) == 0, "gemv: K=%d not a whole number of blocks for type %d", K, type);
    const bool glu = act >= ACT_SWIGLU && act <= ACT_SWIGLU_OAI;
    TSB_CHECK_ARG(!glu || N % 2 == 0, "gemv: GLU needs an even row count, got %d", N);
    if (M == 0 || (ids && problems == 0)) return TSB_OK;
    GemvArgs a;
    a.w = QW{(const uint8_t*)p0, (const uint8_t*)p1, (const uint8_t*)p2, (const uint8_t*)p3, type, N, K};
    a.xq = (const int8_t*)xq; a.xds = (const float2*)xds; a.xb = (const bf16*)xb;
    a.out = out; a.bias = bias; a.residual = residual; a.ids = ids; a.row_scale = row_scale;
    a.M = M; a.x_div = x_div > 0 ? x_div : 1; a.out_f32 = out_f32; a.act = act;
    a.n_out = glu ? N / 2 : N;
    a.push = (const TpPush*)push;
    if (tsb_gemv_mma_eligible(a)) return tsb_gemv_mma_launch(a, glu, (cudaStream_t)stream);
    if (tsb_gemv_stream_eligible(a)) return tsb_gemv_stream_launch(a, glu, (cudaStream_t)stream);
    return glu ? launch_gemv<true>(a, problems, (cudaStream_t)stream)
               : launch_gemv<false>(a, problems, (cudaStream_t)stream);
}

// out[:, cumulative rows] = W_i x for i < n_w (2 or 3 matrices with the same K and the same kind of
// activations).  `planes` holds 4 plane pointers per matrix, `types` and `rows` one entry each.
extern "C" int tsb_gemv_multi(const void* const* planes, const int* types, const int* rows, int n_w, int K, const void* xq,
                              const void* xds, const void* xb, void* out, int M, int out_f32, void* stream) {
    TSB_CHECK_ARG(n_w >= 1 && n_w <= 3 && K > 0 && M >= 0, "gemv_multi: bad arguments n_w=%d K=%d M=%d", n_w, K, M);
    if (M == 0) return TSB_OK;
    GemvMultiArgs a;
    int total = 0;
    for (int i = 0; i < 3; ++i) {
        const int j = i < n_w ? i : n_w - 1;
        const bool q8 = type_uses_q8(types[j]);
        TSB_CHECK_ARG(!q8 || (xq && xds), "gemv_multi: quantised weight type %d needs int8 activations", types[j]);
        TSB_CHECK_ARG(q8 || xb, "gemv_multi: float weight type %d needs bf16 activations", types[j]);
        const bool kq = types[j] == TSB_Q4_K || types[j] == TSB_Q5_K || types[j] == TSB_Q6_K;
        TSB_CHECK_ARG(K % (kq ? 256 : 32) == 0, "gemv_multi: K=%d not a whole number of blocks for type %d", K, types[j]);
        a.w[i] = QW{(const uint8_t*)planes[4 * j], (const uint8_t*)planes[4 * j + 1], (const uint8_t*)planes[4 * j + 2],
                    (const uint8_t*)planes[4 * j + 3], types[j], rows[j], K};
        if (i < n_w) total += rows[i];
        a.row_end[i] = total;
    }
    a.n_w = n_w; a.xq = (const int8_t*)xq; a.xds = (const float2*)xds; a.xb = (const bf16*)xb; a.out = out;
    a.M = M; a.out_f32 = out_f32; a.n_total = total;
    dim3 block(128);
    cudaStream_t s = (cudaStream_t)stream;
    if (M <= 1) TSB_CHECK_CUDA(tsb_launch(gemv_multi_kernel<1>, dim3((total + 3) / 4, 1), block, 0, s, a));
    else if (M <= 2) TSB_CHECK_CUDA(tsb_launch(gemv_multi_kernel<2>, dim3((total + 3) / 4, 1), block, 0, s, a));
    else if (M <= 4) TSB_CHECK_CUDA(tsb_launch(gemv_multi_kernel<4>, dim3((total + 3) / 4, 1), block, 0, s, a));
    else TSB_CHECK_CUDA(tsb_launch(gemv_multi_kernel<8>, dim3((total + 3) / 4, (M + 7) / 8), block, 0, s, a));
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}
