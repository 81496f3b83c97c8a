// Device-side views of quantised weight matrices and element decoders.
//
// A weight matrix W[N, K] arrives from GGUF as rows of blocks.  Block types whose size is
// a multiple of 16 bytes (Q4_K 144 B, Q5_K 176 B) are used exactly as stored.  The others
// (Q8_0 34 B, Q6_K 210 B, MXFP4 17 B, Q4_0 18 B) are split once at load time into planes
// so that every kernel load is 16-byte aligned:
//   Q8_0 : p0 = int8 qs[N][K]            p1 = half d[N][K/32]
//   Q4_0 : p0 = u8 qs[N][K/2] (per 32-block: 16 bytes, value j low nibble, j+16 high)
//          p1 = half d[N][K/32]
//   MXFP4: p0 = u8 qs[N][K/2] (same nibble order as Q4_0)   p1 = u8 e8m0[N][K/32]
//   Q6_K : p0 = u8 ql[N][K/2]  p1 = u8 qh[N][K/4]  p2 = int8 sc[N][K/16]  p3 = half d[N][K/256]
//   Q4_K / Q5_K : p0 = the GGUF blocks, unchanged
//   BF16 / F16  : p0 = the values
// Block layouts follow ggml-quants.c (reference: TensorSharp.Models/ManagedQuantizedOps.cs
// :411 Q8_0, :447-479 Q4_K, :520 Q6_K, :579-598 MXFP4).
#pragma once
#include "common.cuh"

struct QW {
    const uint8_t* p0;
    const uint8_t* p1;
    const uint8_t* p2;
    const uint8_t* p3;
    int type;   // TsbGgmlType
    int N, K;   // rows (output features), row length
};

__device__ __forceinline__ float e8m0_half_scale(uint32_t e) {
    uint32_t bits = (e < 2) ? (0x00200000u << e) : ((e - 1u) << 23);
    return __uint_as_float(bits);
}

// 6-bit scale / min of sub-block j (0..7) from the 12-byte Q4_K / Q5_K scale field.
__device__ __forceinline__ void k4_scale_min(const uint8_t* s, int j, int& sc, int& mn) {
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

__constant__ int8_t c_mxfp4_tab[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

// Decode values [8*k8, 8*k8+8) of row `row` into o[0..7] (float).
__device__ __forceinline__ void dequant8(const QW& w, long row, int k8, float* o) {
    const int K = w.K;
    switch (w.type) {
    case TSB_BF16: {
        const bf16* p = reinterpret_cast<const bf16*>(w.p0) + row * K + 8 * k8;
        uint4 v = *reinterpret_cast<const uint4*>(p);
        const bf16* e = reinterpret_cast<const bf16*>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = bf2f(e[i]);
        break;
    }
    case TSB_F16: {
        const __half* p = reinterpret_cast<const __half*>(w.p0) + row * K + 8 * k8;
        uint4 v = *reinterpret_cast<const uint4*>(p);
        const __half* e = reinterpret_cast<const __half*>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __half2float(e[i]);
        break;
    }
    case TSB_F32: {
        const float* p = reinterpret_cast<const float*>(w.p0) + row * K + 8 * k8;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = p[i];
        break;
    }
    case TSB_Q8_0: {
        const int8_t* q = reinterpret_cast<const int8_t*>(w.p0) + row * K + 8 * k8;
        const float d = __half2float(reinterpret_cast<const __half*>(w.p1)[row * (K / 32) + k8 / 4]);
        uint2 v = *reinterpret_cast<const uint2*>(q);
        const int8_t* e = reinterpret_cast<const int8_t*>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = d * (float)e[i];
        break;
    }
    case TSB_Q4_0:
    case TSB_MXFP4: {
        const int blk = k8 / 4, sub = k8 % 4;
        const uint8_t* q = w.p0 + row * (K / 2) + blk * 16 + (sub & 1) * 8;
        uint2 v = *reinterpret_cast<const uint2*>(q);
        const uint8_t* e = reinterpret_cast<const uint8_t*>(&v);
        const int sh = (sub >> 1) * 4;
        if (w.type == TSB_Q4_0) {
            const float d = __half2float(reinterpret_cast<const __half*>(w.p1)[row * (K / 32) + blk]);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = d * (float)(((e[i] >> sh) & 0xF) - 8);
        } else {
            const float d = e8m0_half_scale(w.p1[row * (K / 32) + blk]);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = d * (float)c_mxfp4_tab[(e[i] >> sh) & 0xF];
        }
        break;
    }
    case TSB_Q4_K:
    case TSB_Q5_K: {
        const int bsz = (w.type == TSB_Q4_K) ? 144 : 176;
        const int sb = k8 / 32, v0 = (k8 % 32) * 8;
        const int s = v0 / 32, c = s >> 1, hi = s & 1, l0 = v0 % 32;
        const uint8_t* b = w.p0 + (row * (K / 256) + sb) * bsz;
        const float d = h2f_bits(*reinterpret_cast<const uint16_t*>(b));
        const float dmin = h2f_bits(*reinterpret_cast<const uint16_t*>(b + 2));
        int sc, mn;
        k4_scale_min(b + 4, s, sc, mn);
        const float ds = d * sc, dm = dmin * mn;
        const uint8_t* q = b + ((w.type == TSB_Q4_K) ? 16 : 48) + 32 * c + l0;
        uint2 v = *reinterpret_cast<const uint2*>(q);
        const uint8_t* e = reinterpret_cast<const uint8_t*>(&v);
        if (w.type == TSB_Q4_K) {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = ds * (float)((e[i] >> (4 * hi)) & 0xF) - dm;
        } else {
            uint2 hv = *reinterpret_cast<const uint2*>(b + 16 + l0);
            const uint8_t* h = reinterpret_cast<const uint8_t*>(&hv);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                o[i] = ds * (float)(((e[i] >> (4 * hi)) & 0xF) + (((h[i] >> (2 * c + hi)) & 1) << 4)) - dm;
        }
        break;
    }
    case TSB_Q6_K: {
        const int sb = k8 / 32, v0 = (k8 % 32) * 8;
        const int n = v0 / 128, r = v0 % 128, k = r / 32, l0 = r % 32, is = l0 / 16;
        const long blk = row * (K / 256) + sb;
        const uint8_t* ql = w.p0 + blk * 128 + 64 * n + (k & 1) * 32 + l0;
        const uint8_t* qh = w.p1 + blk * 64 + 32 * n + l0;
        const float d = __half2float(reinterpret_cast<const __half*>(w.p3)[blk]);
        const float s = d * (float)reinterpret_cast<const int8_t*>(w.p2)[blk * 16 + 8 * n + 2 * k + is];
        uint2 lv = *reinterpret_cast<const uint2*>(ql);
        uint2 hv = *reinterpret_cast<const uint2*>(qh);
        const uint8_t* le = reinterpret_cast<const uint8_t*>(&lv);
        const uint8_t* he = reinterpret_cast<const uint8_t*>(&hv);
        const int lsh = (k >> 1) * 4, hsh = 2 * k;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            o[i] = s * (float)((int)(((le[i] >> lsh) & 0xF) | (((he[i] >> hsh) & 3) << 4)) - 32);
        break;
    }
    default:
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = 0.f;
    }
}
