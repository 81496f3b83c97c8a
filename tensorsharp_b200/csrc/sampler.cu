// Token sampling on the device, one CTA per sequence, in the reference's order
// (TensorSharp.Runtime/TokenSampler.cs:36-61): penalties over the ids generated so far (repetition:
// divide a positive logit, multiply a negative one; presence: subtract once; frequency: subtract per
// occurrence) -> arg-max when temperature <= 0 -> / temperature -> softmax -> min-p -> top-k ->
// top-p (smallest prefix of the descending order whose mass reaches p) -> draw in proportion.
// The logits never leave the device and the step needs no host decision, so sampled decoding is
// captured in the same CUDA graph as the model.  Occurrence counts live in a [B, V] table that the
// kernel itself updates; the random stream is Philox-4x32-10 keyed by the seed and counted by
// (sequence, tokens generated so far), so a seed reproduces a run whatever the batch composition.
//
// Exact for 1 <= top_k <= 1024 with any top_p / min_p, and for top_k <= 0 with top_p >= 1 (plain
// multinomial over the whole vocabulary); other settings are left to the host sampler.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define SAMPLE_MAX_K 1024

struct SampleArgs {
    const float* logits;     // [B, V]
    int* counts;             // [B, V] occurrences of each id among the generated tokens, or null
    int* ngen;               // [B] tokens generated so far (advanced here)
    int* out;                // [B]
    int B, V;
    float temperature, top_p, min_p, rep, pres, freq;
    int top_k;
    unsigned long long seed;
};

__device__ __forceinline__ unsigned f2key(float f) {
    const unsigned b = __float_as_uint(f);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

__device__ __forceinline__ void philox4x32(unsigned long long seed, unsigned c0, unsigned c1, unsigned* r) {
    unsigned k0 = (unsigned)seed, k1 = (unsigned)(seed >> 32);
    unsigned x0 = c0, x1 = c1, x2 = 0x243F6A88u, x3 = 0x85A308D3u;
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        const unsigned long long p0 = (unsigned long long)0xD2511F53u * x0, p1 = (unsigned long long)0xCD9E8D57u * x2;
        const unsigned y0 = (unsigned)(p1 >> 32) ^ x1 ^ k0, y1 = (unsigned)p1;
        const unsigned y2 = (unsigned)(p0 >> 32) ^ x3 ^ k1, y3 = (unsigned)p0;
        x0 = y0; x1 = y1; x2 = y2; x3 = y3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    r[0] = x0; r[1] = x1; r[2] = x2; r[3] = x3;
}

__device__ __forceinline__ float penalised(const SampleArgs& a, const float* lg, const int* cnt, int i, float inv_t) {
    float v = lg[i];
    if (cnt) {
        const int c = cnt[i];
        if (c > 0) {
            if (a.rep != 1.f) v = v > 0.f ? v / a.rep : v * a.rep;
            v -= a.pres;
            v -= a.freq * (float)c;
        }
    }
    return v * inv_t;
}

__device__ __forceinline__ float cta_max(float v, float* red) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = red[0];
    for (int w = 1; w < SAMPLE_THREADS / 32; ++w) m = fmaxf(m, red[w]);
    return m;
}

__device__ __forceinline__ float cta_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
    for (int w = 0; w < SAMPLE_THREADS / 32; ++w) s += red[w];      // fixed order: identical on every thread
    return s;
}

// Inclusive scan of one float per thread over the CTA, in thread order.
__device__ __forceinline__ float cta_scan(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) red[w] = x;
    __syncthreads();
    float base = 0.f;
    for (int i = 0; i < w; ++i) base += red[i];
    return base + x;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(SampleArgs a) {
    __shared__ float red[SAMPLE_THREADS / 32];
    __shared__ unsigned hist[256];
    __shared__ float cv[SAMPLE_MAX_K];
    __shared__ int ci[SAMPLE_MAX_K];
    __shared__ unsigned s_prefix, s_krem, s_n;
    __shared__ int s_pick;
    const int b = blockIdx.x, tid = threadIdx.x, V = a.V;
    const float* lg = a.logits + (long)b * V;
    int* cnt = a.counts ? a.counts + (long)b * V : nullptr;
    const bool pen = cnt && (a.rep != 1.f || a.pres != 0.f || a.freq != 0.f);
    const int* pc = pen ? cnt : nullptr;
    const bool greedy = a.temperature <= 0.f;
    const float inv_t = greedy ? 1.f : 1.f / a.temperature;

    // ---- maximum (and arg-max, lowest index on ties)
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = penalised(a, lg, pc, i, inv_t);
        if (v > m) { m = v; mi = i; }
    }
    const float gmax = cta_max(m, red);
    if (greedy) {
        if (tid == 0) s_pick = 0x7fffffff;
        __syncthreads();
        if (m == gmax) atomicMin(&s_pick, mi);
        __syncthreads();
    } else {
        float z = 0.f;
        for (int i = tid; i < V; i += SAMPLE_THREADS) z += __expf(penalised(a, lg, pc, i, inv_t) - gmax);
        const float Z = cta_sum(z, red);
        const float cut = a.min_p > 0.f ? __logf(a.min_p) : -INFINITY;      // keep s - max >= log(min_p)
        unsigned rnd[4];
        philox4x32(a.seed, (unsigned)b, (unsigned)a.ngen[b], rnd);
        const float u = (float)(rnd[0] >> 8) * (1.f / 16777216.f);
        if (a.top_k <= 0) {
            // plain multinomial over the survivors of min-p: total mass, then the first index whose
            // running mass reaches u * total (chunks of the vocabulary scanned in order)
            float t = 0.f;
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const float s = penalised(a, lg, pc, i, inv_t) - gmax;
                t += s >= cut ? __expf(s) : 0.f;
            }
            const float total = cta_sum(t, red);
            const float target = u * total;
            if (tid == 0) s_pick = V - 1;
            __syncthreads();
            float base = 0.f;
            for (int i0 = 0; i0 < V; i0 += SAMPLE_THREADS) {
                const int i = i0 + tid;
                float p = 0.f;
                if (i < V) {
                    const float s = penalised(a, lg, pc, i, inv_t) - gmax;
                    p = s >= cut ? __expf(s) : 0.f;
                }
                const float inc = cta_scan(p, red) + base;
                if (i < V && p > 0.f && inc >= target) atomicMin(&s_pick, i);
                __syncthreads();
                if (tid == SAMPLE_THREADS - 1) red[0] = inc;
                __syncthreads();
                base = red[0];
                if (s_pick != V - 1) break;             // uniform: every thread reads it after the barrier
            }
            __syncthreads();
        } else {
            // ---- k-th largest score by radix select on the order-preserving key
            const unsigned k = (unsigned)min(min(a.top_k, SAMPLE_MAX_K), V);
            if (tid == 0) { s_prefix = 0u; s_krem = k; }
            unsigned mask = 0u;
            for (int pass = 3; pass >= 0; --pass) {
                if (tid < 256) hist[tid] = 0u;
                __syncthreads();
                const unsigned prefix = s_prefix;
                const int sh = pass * 8;
                for (int i = tid; i < V; i += SAMPLE_THREADS) {
                    const unsigned key = f2key(penalised(a, lg, pc, i, inv_t));
                    if ((key & mask) == prefix) atomicAdd(&hist[(key >> sh) & 255u], 1u);
                }
                __syncthreads();
                if (tid == 0) {
                    unsigned rem = s_krem, bin = 255u;
                    for (;; --bin) {
                        if (hist[bin] >= rem || bin == 0u) break;
                        rem -= hist[bin];
                    }
                    s_krem = rem;
                    s_prefix = prefix | (bin << sh);
                }
                mask |= 0xffu << sh;
                __syncthreads();
            }
            const unsigned kth = s_prefix;
            // ---- gather everything above the k-th key, then ties with it while room remains
            if (tid == 0) s_n = 0u;
            for (int i = tid; i < SAMPLE_MAX_K; i += SAMPLE_THREADS) { cv[i] = -INFINITY; ci[i] = 0x7fffffff; }
            __syncthreads();
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const float s = penalised(a, lg, pc, i, inv_t);
                if (f2key(s) > kth) {
                    const unsigned d = atomicAdd(&s_n, 1u);
                    if (d < SAMPLE_MAX_K) { cv[d] = s; ci[d] = i; }
                }
            }
            __syncthreads();
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const float s = penalised(a, lg, pc, i, inv_t);
                if (f2key(s) == kth) {
                    const unsigned d = atomicAdd(&s_n, 1u);
                    if (d < SAMPLE_MAX_K) { cv[d] = s; ci[d] = i; }
                }
            }
            __syncthreads();
            // ---- bitonic sort, descending by score then ascending by index
            for (int size = 2; size <= SAMPLE_MAX_K; size <<= 1) {
                for (int stride = size >> 1; stride > 0; stride >>= 1) {
                    const int j = tid ^ stride;
                    if (j > tid) {
                        const bool desc = (tid & size) == 0;
                        const float va = cv[tid], vb = cv[j];
                        const int ia = ci[tid], ib = ci[j];
                        const bool a_first = va > vb || (va == vb && ia < ib);
                        if (a_first != desc) { cv[tid] = vb; cv[j] = va; ci[tid] = ib; ci[j] = ia; }
                    }
                    __syncthreads();
                }
            }
            // ---- probabilities of the first k, top-p cut, draw
            const float s = cv[tid] - gmax;
            const float p = ((unsigned)tid < k && ci[tid] < V && s >= cut) ? __expf(s) / Z : 0.f;
            const float cum = cta_scan(p, red);
            if (tid == 0) s_pick = (int)k - 1;
            __syncthreads();
            if (a.top_p < 1.f && (unsigned)tid < k && cum >= a.top_p) atomicMin(&s_pick, tid);
            __syncthreads();
            const int last = s_pick;                    // candidates [0, last] survive
            __syncthreads();
            if (tid == last) red[0] = cum;
            __syncthreads();
            const float target = u * red[0];
            __syncthreads();
            if (tid == 0) s_pick = last;
            __syncthreads();
            if (tid <= last && p > 0.f && cum >= target) atomicMin(&s_pick, tid);
            __syncthreads();
            if (tid == 0) s_pick = ci[s_pick] < V ? ci[s_pick] : ci[0];
            __syncthreads();
        }
    }
    if (tid == 0) {
        const int tok = min(max(s_pick, 0), V - 1);
        a.out[b] = tok;
        if (cnt) atomicAdd(&cnt[tok], 1);
        a.ngen[b] += 1;
    }
}

extern "C" int tsb_sample(const float* logits, int* counts, int* ngen, int* out, int B, int V, float temperature, int top_k,
                          float top_p, float min_p, float rep, float pres, float freq, unsigned long long seed, void* stream) {
    TSB_CHECK_ARG(B >= 0 && V > 0, "sample: bad shape B=%d V=%d", B, V);
    TSB_CHECK_ARG(top_k <= SAMPLE_MAX_K, "sample: top_k=%d exceeds the device sampler's limit %d", top_k, SAMPLE_MAX_K);
    TSB_CHECK_ARG(top_k > 0 || top_p >= 1.f || temperature <= 0.f, "sample: top_p=%g without top_k needs the host sampler", top_p);
    if (B == 0) return TSB_OK;
    SampleArgs a{logits, counts, ngen, out, B, V, temperature, top_p, min_p, rep, pres, freq, top_k, seed};
    sample_kernel<<<B, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(a);
    TSB_CHECK_LAUNCH();
    return TSB_OK;
}
