// Recurrent / linear-attention layers on the device: causal depth-wise conv1d (+SiLU) with a
// carried tail, the GatedDeltaNet delta-rule recurrence and the Mamba2 selective scan.
//
// The reference runs all three on the host, token by token (GatedDeltaNet step and conv:
// TensorSharp.Models/Models/Qwen35/Qwen35Model.GatedDeltaNet.cs:1341-1500; Mamba2:
// Models/Nemotron/NemotronModel.cs:1103-1331), and its chunked GatedDeltaNet prefill is a ggml
// graph of ~40 nodes per chunk (TensorSharp.GGML.Native/ggml_ops_gated_delta_net.cpp:178-615).
// Here one kernel per (head, sequence) walks the tokens with the state matrix held in
// registers, so prefill and decode share one code path and the state never leaves the chip
// between tokens.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// Causal depth-wise conv1d.  x: [T, *] rows with C channels at stride xs; w: [C, K]; the tail
// state holds the last K-1 inputs of each sequence slot, oldest first: [slot, K-1, C].
//   out[t, c] = act(bias[c] + sum_k w[c, k] * in(t - (K-1) + k, c))
// ------------------------------------------------------------------------------------------
struct ConvArgs {
    const void* x; long xs; int x_f32;
    const float* w; const float* bias;
    float* state;
    const int* cu_q; const long* seq_slots;
    float* out; long os;          // f32 output rows
    int C, K, B, act;             // act: 1 = SiLU
};

__global__ void conv1d_kernel(ConvArgs a) {
    pdl_wait();
    pdl_trigger();
    const int b = blockIdx.y;
    const int q0 = a.cu_q[b], n = a.cu_q[b + 1] - q0;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n * a.C) return;
    const int i = (int)(idx / a.C), c = (int)(idx % a.C);
    const int K = a.K;
    const float* st = a.state + a.seq_slots[b] * (long)(K - 1) * a.C;
    float acc = a.bias ? a.bias[c] : 0.f;
    for (int k = 0; k < K; ++k) {
        const int j = i - (K - 1) + k;
        float v;
        if (j >= 0) {
            const long o = (long)(q0 + j) * a.xs + c;
            v = a.x_f32 ? reinterpret_cast<const float*>(a.x)[o] : bf2f(reinterpret_cast<const bf16*>(a.x)[o]);
        } else {
            v = st[(long)(K - 1 + j) * a.C + c];
        }
        acc += a.w[(long)c * K + k] * v;
    }
    if (a.act == 1) acc = acc / (1.f + __expf(-acc));
    a.out[(long)(q0 + i) * a.os + c] = acc;
}

// One thread per (sequence, channel): shift the tail so that it ends with this call's inputs.
__global__ void conv1d_state_kernel(ConvArgs a) {
    pdl_wait();
    pdl_trigger();
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int q0 = a.cu_q[b], n = a.cu_q[b + 1] - q0;
    const int Km = a.K - 1;
    float* st = a.state + a.seq_slots[b] * (long)Km * a.C;
    float nv[8];
    for (int j = 0; j < Km; ++j) {
        const int src = n - Km + j;              // index into this call's inputs (negative: old tail)
        if (src >= 0) {
            const long o = (long)(q0 + src) * a.xs + c;
            nv[j] = a.x_f32 ? reinterpret_cast<const float*>(a.x)[o] : bf2f(reinterpret_cast<const bf16*>(a.x)[o]);
        } else {
            nv[j] = st[(long)(Km + src) * a.C + c];
        }
    }
    for (int j = 0; j < Km; ++j) st[(long)j * a.C + c] = nv[j];
}

extern "C" int tsb_causal_conv1d(const ConvArgs* args, int max_q, void* stream) {
    const ConvArgs& a = *args;
    TSB_CHECK_ARG(a.K >= 1 && a.K <= 9, "conv1d: kernel size %d out of range (1..9)", a.K);
    if (a.B == 0 || max_q == 0) return TSB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long per = (long)max_q * a.C;
    TSB_CHECK_CUDA(tsb_launch(conv1d_kernel, dim3((unsigned)((per + 255) / 256), a.B), dim3(256), 0, s, a));
    if (a.K > 1)
        TSB_CHECK_CUDA(tsb_launch(conv1d_state_kernel, dim3((a.C + 127) / 128, a.B), dim3(128), 0, s, a));
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// GatedDeltaNet recurrence.  Grid (Hv, B), Dv threads; thread r owns row r of the head's
// [Dv, Dk] state in registers.  Per token (Qwen35Model.GatedDeltaNet.cs:1449-1490):
//   q, k <- L2-normalised head (K heads are tiled onto V heads: src = h % Hk); q *= 1/sqrt(Dv)
//   g = softplus(alpha + dt_bias[h]) * a[h];  S *= exp(g);  beta = sigmoid(beta_raw)
//   delta = (v - S k) * beta;  S += delta (x) k;  core = S q
//   out = RMSNorm(core) * norm_w * silu(z)
// ------------------------------------------------------------------------------------------
struct GdnArgs {
    const float* qkv; long qkv_s;     // conv output rows: [q (Hk*Dk) | k (Hk*Dk) | v (Hv*Dv)]
    const void* z; long z_s; int z_f32;
    const void* beta; const void* alpha; long ba_s; int ba_f32;   // [T, Hv] raw
    const float* dt_bias; const float* a; const float* norm_w;
    float* state;                     // [slot, Hv, Dv, Dk]
    const int* cu_q; const long* seq_slots;
    bf16* out; long out_s;            // [T, Hv*Dv]
    float eps;
    int Hk, Hv, Dk, Dv, B;
};

__device__ __forceinline__ float ld_f(const void* p, long i, int f32) {
    return f32 ? reinterpret_cast<const float*>(p)[i] : bf2f(reinterpret_cast<const bf16*>(p)[i]);
}

template <int DK>
__global__ void __launch_bounds__(256) gdn_kernel(GdnArgs a) {
    pdl_wait();
    pdl_trigger();
    __shared__ float sq[DK], sk[DK];
    __shared__ float red[32];
    const int h = blockIdx.x, b = blockIdx.y, r = threadIdx.x;
    const int Dv = a.Dv;
    const int q0 = a.cu_q[b], n = a.cu_q[b + 1] - q0;
    const int hk = h % a.Hk;
    float S[DK];
    float* sp = a.state + ((a.seq_slots[b] * a.Hv + h) * (long)Dv + r) * DK;
#pragma unroll
    for (int c = 0; c < DK; c += 4) {
        const float4 v = *reinterpret_cast<const float4*>(sp + c);
        S[c] = v.x; S[c + 1] = v.y; S[c + 2] = v.z; S[c + 3] = v.w;
    }
    const float qscale = rsqrtf((float)Dv);
    const float nw = a.norm_w[r];
    for (int i = 0; i < n; ++i) {
        const long t = q0 + i;
        const float* row = a.qkv + t * a.qkv_s;
        // stage the K-head's q and k, L2-normalised (threads stride over DK)
        float qs = 0.f, ks = 0.f;
        for (int c = r; c < DK; c += Dv) {
            const float qv = row[hk * DK + c], kv = row[(long)a.Hk * DK + hk * DK + c];
            sq[c] = qv;
            sk[c] = kv;
            qs += qv * qv;
            ks += kv * kv;
        }
        qs = block_sum(qs, red);
        ks = block_sum(ks, red);
        const float qn = qscale * rsqrtf(qs + a.eps), kn = rsqrtf(ks + a.eps);
        __syncthreads();
        const float v = row[2L * a.Hk * DK + (long)h * Dv + r];
        const float al = ld_f(a.alpha, t * a.ba_s + h, a.ba_f32) + a.dt_bias[h];
        const float sp_al = al > 20.f ? al : log1pf(__expf(al));
        const float eg = __expf(sp_al * a.a[h]);
        const float beta = 1.f / (1.f + __expf(-ld_f(a.beta, t * a.ba_s + h, a.ba_f32)));
        float kv_mem = 0.f;
#pragma unroll
        for (int c = 0; c < DK; ++c) {
            S[c] *= eg;
            kv_mem += S[c] * sk[c];
        }
        const float delta = (v - kv_mem * kn) * beta;
        float core = 0.f;
        const float dk = delta * kn;
#pragma unroll
        for (int c = 0; c < DK; ++c) {
            S[c] += sk[c] * dk;
            core += S[c] * sq[c];
        }
        core *= qn;
        const float ms = block_sum(core * core, red);
        const float rs = rsqrtf(ms / (float)Dv + a.eps);
        const float zz = ld_f(a.z, t * a.z_s + (long)h * Dv + r, a.z_f32);
        a.out[t * a.out_s + (long)h * Dv + r] = f2bf(core * rs * nw * (zz / (1.f + __expf(-zz))));
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < DK; c += 4)
        *reinterpret_cast<float4*>(sp + c) = make_float4(S[c], S[c + 1], S[c + 2], S[c + 3]);
}

extern "C" int tsb_gdn_recurrent(const GdnArgs* args, void* stream) {
    const GdnArgs& a = *args;
    TSB_CHECK_ARG(a.Dv >= 32 && a.Dv <= 256 && a.Dv % 32 == 0, "gdn: value head dim %d unsupported", a.Dv);
    TSB_CHECK_ARG(a.Hk > 0 && a.Hv % a.Hk == 0, "gdn: Hv=%d not a multiple of Hk=%d", a.Hv, a.Hk);
    if (a.B == 0) return TSB_OK;
    dim3 grid(a.Hv, a.B), block(a.Dv);
    cudaStream_t s = (cudaStream_t)stream;
    switch (a.Dk) {
    case 64: TSB_CHECK_CUDA(tsb_launch(gdn_kernel<64>, grid, block, 0, s, a)); break;
    case 128: TSB_CHECK_CUDA(tsb_launch(gdn_kernel<128>, grid, block, 0, s, a)); break;
    default:
        tsb_set_error("gdn: key head dim %d unsupported (64, 128)", a.Dk);
        return TSB_ERR_UNSUPPORTED;
    }
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
// Mamba2 selective scan.  Grid (H, B), P (= head dim) threads; thread p owns state[h, p, :].
//   dt = softplus(dt_raw + dt_bias[h]);  dA = exp(dt * A[h])
//   state = state * dA + x[h, p] * dt * B[g, :];   y = state . C[g, :] + D[h] * x[h, p]
// xBC rows (after conv + SiLU): [x (H*P) | B (G*N) | C (G*N)].  (NemotronModel.cs:1103-1331)
// ------------------------------------------------------------------------------------------
struct MambaArgs {
    const float* xbc; long xbc_s;
    const void* dt; long dt_s; int dt_f32;          // [T, H] raw
    const float* dt_bias; const float* A; const float* D;
    float* state;                                   // [slot, H, P, N]
    const int* cu_q; const long* seq_slots;
    float* y; long y_s;                             // [T, H*P]
    int H, P, G, N, B;
};

template <int NS>
__global__ void __launch_bounds__(256) mamba2_kernel(MambaArgs a) {
    pdl_wait();
    pdl_trigger();
    __shared__ float sB[NS], sC[NS];
    const int h = blockIdx.x, b = blockIdx.y, p = threadIdx.x;
    const int P = a.P;
    const int q0 = a.cu_q[b], n = a.cu_q[b + 1] - q0;
    const int g = h / (a.H / a.G);
    float S[NS];
    float* sp = a.state + ((a.seq_slots[b] * a.H + h) * (long)P + p) * NS;
#pragma unroll
    for (int c = 0; c < NS; c += 4) {
        const float4 v = *reinterpret_cast<const float4*>(sp + c);
        S[c] = v.x; S[c + 1] = v.y; S[c + 2] = v.z; S[c + 3] = v.w;
    }
    const float Ah = a.A[h], Dh = a.D ? a.D[h] : 0.f, dtb = a.dt_bias ? a.dt_bias[h] : 0.f;
    const long xdim = (long)a.H * P;
    for (int i = 0; i < n; ++i) {
        const long t = q0 + i;
        const float* row = a.xbc + t * a.xbc_s;
        for (int c = p; c < NS; c += P) {
            sB[c] = row[xdim + (long)g * NS + c];
            sC[c] = row[xdim + (long)a.G * NS + (long)g * NS + c];
        }
        __syncthreads();
        const float x = row[(long)h * P + p];
        float dt = ld_f(a.dt, t * a.dt_s + h, a.dt_f32) + dtb;
        dt = dt > 20.f ? dt : log1pf(__expf(dt));
        const float dA = __expf(dt * Ah), xdt = x * dt;
        float y = 0.f;
#pragma unroll
        for (int c = 0; c < NS; ++c) {
            S[c] = S[c] * dA + xdt * sB[c];
            y += S[c] * sC[c];
        }
        a.y[t * a.y_s + (long)h * P + p] = y + Dh * x;
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < NS; c += 4)
        *reinterpret_cast<float4*>(sp + c) = make_float4(S[c], S[c + 1], S[c + 2], S[c + 3]);
}

extern "C" int tsb_mamba2_recurrent(const MambaArgs* args, void* stream) {
    const MambaArgs& a = *args;
    TSB_CHECK_ARG(a.P >= 32 && a.P <= 256 && a.P % 32 == 0, "mamba2: head dim %d unsupported", a.P);
    TSB_CHECK_ARG(a.G > 0 && a.H % a.G == 0, "mamba2: H=%d not a multiple of G=%d", a.H, a.G);
    if (a.B == 0) return TSB_OK;
    dim3 grid(a.H, a.B), block(a.P);
    cudaStream_t s = (cudaStream_t)stream;
    switch (a.N) {
    case 64: TSB_CHECK_CUDA(tsb_launch(mamba2_kernel<64>, grid, block, 0, s, a)); break;
    case 128: TSB_CHECK_CUDA(tsb_launch(mamba2_kernel<128>, grid, block, 0, s, a)); break;
    default:
        tsb_set_error("mamba2: state size %d unsupported (64, 128)", a.N);
        return TSB_ERR_UNSUPPORTED;
    }
    return TSB_OK;
}
