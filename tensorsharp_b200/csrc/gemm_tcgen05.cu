// bf16 GEMM on the 5th-generation tensor cores:  Y[t, n] = sum_k X[t, k] * W[n, k]
//   (+ bias[n]) (+ residual[t, n]),  f32 accumulation in tensor memory.
//
// The problem is run "weights as the M operand": each CTA owns 128 rows of W (output
// features) and BN tokens, so that a small token count still fills the 128-lane MMA and the
// same kernel serves batched decode (BN = 32) and prefill (BN = 256).
//
//   warp 0    : TMA producer - W and X tiles (64-element K slabs, 128-byte swizzle) into a
//               STAGES-deep shared-memory ring, completion on mbarriers
//   warp 1    : allocates tensor memory, one thread issues tcgen05.mma (128 x BN x 16) and
//               commits each stage back to the producer
//   warps 2-5 : epilogue - tcgen05.ld the accumulator (lane = feature, column = token),
//               add bias / residual, store coalesced along the feature dimension
//
// Replaces in the reference: mul_mat_q + stream-k fixup + quantize_mmq_q8_1
// (ggml-cuda/mmq.cuh:3301, :3542, quantize.cu:51), mul_mat_f (mmf.cuh:25) and the cuBLAS
// fallback (ggml-cuda.cu:1361-1497): quantised weights are decoded once into an L2-resident
// bf16 scratch by tsb_gather_rows and consumed here.
#include <cudaTypedefs.h>
#include <mutex>
#include <cstdlib>
#include "tcgen05.cuh"
#include "tp_fused.cuh"

struct GemmEpi {
    void* out;              // [T, ldo]
    const float* bias;      // [N] or null
    const void* residual;   // same dtype / layout as out, or null
    long ldo;
    int T, N;               // valid tokens, valid features
    int out_f32;
    // Tensor-parallel prefill (tp_fused.cuh); both null for an ordinary GEMM.
    const TpSeq* rs;        // GEMM -> reduce-scatter: store the tile into the token owner's accumulator over NVLink
    const TpSeq* ag;        // all-gather -> GEMM: X is the gathered buffer; wait for the tile's shard to arrive
    int rs_rows;            // size * shard (host copy, for the grid)
    int tile_rot;           // token tiles are visited starting from this one (see tsb_gemm_bf16_tp)
    // Grouped mode (mixture of experts): W is a stack of matrices of N rows each, X holds the rows of all groups sorted
    // by group, and token tile y of the grid is described by groups[3 * y .. 3 * y + 2] = {matrix index or -1 for an
    // unused tile, first row, end row}.  The list is built on the device, so the host never learns the group sizes.
    const int* groups;
    // Split-K (one-tile-per-CTA kernel, few tiles and a long K: decode batches of 9 to 64 rows): blockIdx.z takes a
    // range of k-blocks and stores its raw partial tile into ws[z][t][n]; splitk_reduce_kernel adds the parts in order
    // with bias and residual.  Null for an ordinary launch.
    float* ws;
    int kb_per_split;
};

// Epilogue of one thread for 16 consecutive tokens of its feature n: out[t, n] = acc + bias (+ residual[t, n]).
// The residual values are all requested before the first store: with the load and the store of one token back to back
// (the residual may be the output buffer itself, so the compiler keeps their order) every token would cost a full
// memory round trip, 16 in a row per chunk.  Each element is read and written by the same thread, so reading ahead is
// safe for an in-place residual too.
__device__ __forceinline__ void gemm_store16(const GemmEpi& ep, const uint32_t (&r)[16], int n, int t0, int t_end, float bias) {
    float res[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) res[j] = 0.f;
    if (ep.residual != nullptr) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int t = t0 + j;
            if (t < t_end) {
                const long o = (long)t * ep.ldo + n;
                res[j] = ep.out_f32 ? reinterpret_cast<const float*>(ep.residual)[o] : bf2f(reinterpret_cast<const bf16*>(ep.residual)[o]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int t = t0 + j;
        if (t < t_end) {
            const float v = __uint_as_float(r[j]) + bias + res[j];
            const long o = (long)t * ep.ldo + n;
            if (ep.out_f32) reinterpret_cast<float*>(ep.out)[o] = v;
            else reinterpret_cast<bf16*>(ep.out)[o] = f2bf(v);
        }
    }
}

// MT = 1: a CTA owns 128 features; MT = 2: 256 features as two accumulators that share every token slab, which halves
// the bytes a CTA pulls from L2 per FLOP (the limiter of the 128 x 256 tile) at the price of coarser tiles.
template <int BN, int STAGES, int MT = 1>
struct GemmSmem {
    static constexpr int A_BYTES = MT * 128 * 64 * 2;
    static constexpr int B_BYTES = BN * 64 * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BAR_OFF + (2 * STAGES + 1) * 8 + 16 + 1024;  // + alignment slack
};

template <int BN, int STAGES, int MT = 1>
__global__ void __launch_bounds__(192) gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmW,
                                                        const __grid_constant__ CUtensorMap tmX, GemmEpi ep, int K,
                                                        int* status) {
    using L = GemmSmem<BN, STAGES, MT>;
    constexpr int TMEM_COLS = MT * BN < 32 ? 32 : MT * BN;
    static_assert(MT == 1 || (MT == 2 && BN == 256), "two accumulators fill the 512 columns of tensor memory");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * (128 * MT);       // first feature (row of W)
    int n0 = (int)((blockIdx.y + (unsigned)ep.tile_rot) % gridDim.y) * BN;        // first token
    int t_end = ep.T;                      // tokens at or past this row are not stored
    int w_row0 = m0;                       // row of the (stacked) weight matrix where this tile's features start
    bool active = true;
    const int kb_all = (K + 63) / 64;
    const int kb_first = ep.ws != nullptr ? (int)blockIdx.z * ep.kb_per_split : 0;
    const int kblocks = ep.ws != nullptr ? min(kb_all - kb_first, ep.kb_per_split) : kb_all;     // this CTA's share (>= 1)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        tc::mbar_init(acc_bar, 1);
        tc::fence_barrier_init();
    }
    if (warp == 1) tc::tmem_alloc<TMEM_COLS>(tmem_slot);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();        // barrier set-up and the TMEM allocation above overlap the previous kernel's tail
    pdl_trigger();
    int group = 0;
    if (ep.groups != nullptr) {
        const int* gt = ep.groups + 3 * blockIdx.y;
        group = gt[0];
        active = group >= 0;
        n0 = gt[1];
        t_end = gt[2];
        w_row0 = group * ep.N + m0;
    }

    if (!active) {
        // an unused entry of the tile list: nothing to load, multiply or store
    } else if (warp == 0) {
        if (lane == 0) {
            tc::tma_prefetch_desc(&tmW);
            tc::tma_prefetch_desc(&tmX);
            if (ep.ag != nullptr) {
                // the rows of this token tile come from one rank; its stores are complete once its
                // arrival counter here has reached the target left by the preceding gather kernel
                const TpSeq* g = ep.ag;
                const int owner = n0 / g->shard;
                if (owner < g->size && !tp_wait_counter(g->ag_arrive[g->rank] + owner, *g->ag_target))
                    atomicExch(status, 4);
            }
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!tc::mbar_wait(&empty_bar[s], ph ^ 1)) { atomicExch(status, 1); break; }
                unsigned char* a = smem + s * L::STAGE_BYTES;
                tc::mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
                tc::tma_load_2d(a, &tmW, &full_bar[s], (kb_first + kb) * 64, w_row0);
                tc::tma_load_2d(a + L::A_BYTES, &tmX, &full_bar[s], (kb_first + kb) * 64, n0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::make_idesc_bf16(128, BN);
            bool ok = true;
            for (int kb = 0; kb < kblocks && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!tc::mbar_wait(&full_bar[s], ph)) { atomicExch(status, 2); ok = false; break; }
                tc::fence_after_sync();
                const uint32_t a = tc::smem_u32(smem + s * L::STAGE_BYTES);
                const uint64_t da = tc::make_desc_sw128(a), db = tc::make_desc_sw128(a + L::A_BYTES);
#pragma unroll
                for (int k = 0; k < 4; ++k) {   // 4 x (K = 16) per 64-element slab: +32 bytes = +2 descriptor units
                    tc::mma_f16_ss(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    if (MT == 2) {              // the second 128 features: next 16 KB of the stage, next BN columns
                        const uint64_t da2 = tc::make_desc_sw128(a + 128 * 64 * 2);
                        tc::mma_f16_ss(tmem_base + BN, da2 + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    }
                }
                tc::mma_commit(&empty_bar[s]);
            }
            if (ok) tc::mma_commit(acc_bar);
        }
        __syncwarp();
    } else {
        const int q = warp & 3;                       // TMEM lane quadrant this warp may read
        if (tc::mbar_wait(acc_bar, 0)) {
            tc::fence_after_sync();
#pragma unroll 1
          for (int half = 0; half < MT; ++half) {
            const int n = m0 + half * 128 + q * 32 + lane;             // feature owned by this thread
            const float bias = (ep.bias && n < ep.N && (ep.rs == nullptr || ep.rs->rank == 0)) ? ep.bias[(long)group * ep.N + n] : 0.f;
            bf16* rs_dst = nullptr;
            if (ep.rs != nullptr) {
                const TpSeq* g = ep.rs;
                const int owner = n0 / g->shard;                    // a token tile never straddles two shards
                if (owner < g->size)       // this rank's slot of the current accumulator, rebased to global token indices
                    rs_dst = g->acc[owner] + ((long)(*g->rs_phase & 1u) * g->size + g->rank) * g->shard * g->ld -
                             (long)owner * g->shard * g->ld;
            }
#pragma unroll 1
            for (int c = 0; c < BN / 16; ++c) {
                uint32_t r[16];
                tc::tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + half * BN + c * 16, r);
                tc::tmem_ld_wait();
                if (rs_dst != nullptr) {
                    if (n < ep.N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int t = n0 + c * 16 + j;
                            // a warp covers 32 consecutive features of one token: one 64-byte packet.  Rows
                            // past T are written too (zeros from the zero-filled X tile) so the owner
                            // never reads a stale slot row.
                            rs_dst[(long)t * ep.rs->ld + n] = f2bf(__uint_as_float(r[j]) + (t < ep.T ? bias : 0.f));
                        }
                    }
                } else if (ep.ws != nullptr) {
                    if (n < ep.N) {
                        float* part = ep.ws + (long)blockIdx.z * ep.T * ep.N;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int t = n0 + c * 16 + j;
                            if (t < ep.T) part[(long)t * ep.N + n] = __uint_as_float(r[j]);
                        }
                    }
                } else if (n < ep.N) {
                    gemm_store16(ep, r, n, n0 + c * 16, t_end, bias);
                }
            }
          }
        } else {
            atomicExch(status, 3);
        }
        if (ep.rs != nullptr) __threadfence_system();               // reductions visible before the arrival below
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc<TMEM_COLS>(tmem_base);
    }
    if (ep.rs != nullptr && threadIdx.x == 0) {
        const TpSeq* g = ep.rs;
        const int owner = n0 / g->shard;
        if (owner < g->size) red_release_inc_sys(g->rs_arrive[owner]);
        const unsigned done = atomicAdd(g->ticket, 1u);
        if (done == gridDim.x * gridDim.y - 1) {
            // every owner receives (feature tiles) x (token tiles per shard) arrivals from each rank
            *g->ticket = 0;
            __threadfence();
            *g->rs_target += (unsigned)g->size * gridDim.x * (unsigned)(g->shard / BN);
        }
    }
}

// out[t, n] = sum over the splits (in order) of ws[z][t][n] + bias[n] + residual[t, n]
__global__ void __launch_bounds__(256) splitk_reduce_kernel(GemmEpi ep, int splits) {
    pdl_wait();
    pdl_trigger();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)ep.T * ep.N) return;
    const int t = (int)(i / ep.N), n = (int)(i % ep.N);
    float v = ep.bias ? ep.bias[n] : 0.f;
    for (int z = 0; z < splits; ++z) v += ep.ws[((long)z * ep.T + t) * ep.N + n];
    const long o = (long)t * ep.ldo + n;
    if (ep.out_f32) {
        if (ep.residual) v += reinterpret_cast<const float*>(ep.residual)[o];
        reinterpret_cast<float*>(ep.out)[o] = v;
    } else {
        if (ep.residual) v += bf2f(reinterpret_cast<const bf16*>(ep.residual)[o]);
        reinterpret_cast<bf16*>(ep.out)[o] = f2bf(v);
    }
}

// ------------------------------------------------------------------------------------------
// Persistent form for plain GEMMs (no tensor-parallel hooks, no tile list): one CTA per SM walks the tiles
// (feature tile fastest, so CTAs that run together share a token slab in L2), the TMA producer keeps filling the
// shared-memory ring across tile boundaries, and tensor memory holds two accumulators: the epilogue warps drain tile i
// while the MMA warp already multiplies tile i + 1.  With short K (the gate / up and QKV projections) the epilogue is
// about half of a tile's time in the one-tile-per-CTA kernel above; here it disappears behind the next main loop.
// ------------------------------------------------------------------------------------------
template <int BN, int STAGES>
__global__ void __launch_bounds__(192) gemm_bf16_persistent_kernel(const __grid_constant__ CUtensorMap tmW,
                                                                   const __grid_constant__ CUtensorMap tmX, GemmEpi ep, int K,
                                                                   int m_tiles, int total_tiles, int n_fast, int* status) {
    using L = GemmSmem<BN, STAGES>;
    constexpr int TMEM_COLS = 2 * BN;
    static_assert(TMEM_COLS >= 32 && TMEM_COLS <= 512, "two accumulators must fit tensor memory");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;          // [2] accumulator complete (one commit by the MMA thread)
    uint64_t* acc_empty = acc_full + 2;               // [2] accumulator drained (one arrival per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    // reduce-scatter epilogue: two buffers of 16 tokens x 128 features (bf16) in which the four epilogue warps turn
    // their feature-per-lane fragments into whole token rows, so that a peer store covers 256 contiguous bytes
    bf16* rs_stage = reinterpret_cast<bf16*>(smem + L::BAR_OFF + 256);      // past the barriers (at most 2 * 8 + 4 words) and the TMEM slot
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (K + 63) / 64;
    const int n_tiles = total_tiles / m_tiles;
    // Tile order.  Feature tile fastest: the CTAs that run together share one token slab.  Token tile fastest (plain
    // GEMMs whose weight matrix is the larger operand): the CTAs that run together share a few weight tiles, so the
    // weights come from DRAM once instead of once per token tile.
    auto tile_m = [&](int tile) { return n_fast ? tile / n_tiles : tile % m_tiles; };
    auto tile_n = [&](int tile) { return n_fast ? tile % n_tiles : tile / m_tiles; };
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], 4);
        }
        tc::fence_barrier_init();
    }
    if (warp == 1) tc::tmem_alloc<TMEM_COLS>(tmem_slot);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();
    pdl_trigger();

    if (warp == 0) {
        if (lane == 0) {
            tc::tma_prefetch_desc(&tmW);
            tc::tma_prefetch_desc(&tmX);
            long it = 0;                               // k-blocks issued so far, over all tiles of this CTA
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int w_row0 = tile_m(tile) * 128, n0 = (int)((tile_n(tile) + (unsigned)ep.tile_rot) % n_tiles) * BN;
                if (ep.ag != nullptr) {
                    // the rows of this token tile come from one rank; its stores are complete once its arrival counter
                    // here has reached the target left by the preceding gather kernel
                    const TpSeq* g = ep.ag;
                    const int owner = n0 / g->shard;
                    if (owner < g->size && !tp_wait_counter(g->ag_arrive[g->rank] + owner, *g->ag_target)) atomicExch(status, 4);
                }
                if (ep.groups != nullptr) {            // grouped mode: the token tile comes from the device-built list
                    const int* gt = ep.groups + 3 * tile_n(tile);
                    if (gt[0] < 0) continue;
                    w_row0 += gt[0] * ep.N;
                    n0 = gt[1];
                }
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    if (!tc::mbar_wait(&empty_bar[s], ph ^ 1)) { atomicExch(status, 1); ok = false; break; }
                    unsigned char* a = smem + s * L::STAGE_BYTES;
                    tc::mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
                    tc::tma_load_2d(a, &tmW, &full_bar[s], kb * 64, w_row0);
                    tc::tma_load_2d(a + L::A_BYTES, &tmX, &full_bar[s], kb * 64, n0);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::make_idesc_bf16(128, BN);
            long it = 0;
            int j = 0;                                 // tiles done by this CTA
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (ep.groups != nullptr && ep.groups[3 * tile_n(tile)] < 0) continue;
                const int buf = j & 1;
                const uint32_t aph = (uint32_t)(j >> 1) & 1u;
                if (!tc::mbar_wait(&acc_empty[buf], aph ^ 1)) { atomicExch(status, 5); ok = false; break; }
                tc::fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t)buf * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    if (!tc::mbar_wait(&full_bar[s], ph)) { atomicExch(status, 2); ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t a = tc::smem_u32(smem + s * L::STAGE_BYTES);
                    const uint64_t da = tc::make_desc_sw128(a), db = tc::make_desc_sw128(a + L::A_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k) tc::mma_f16_ss(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    tc::mma_commit(&empty_bar[s]);
                }
                if (ok) tc::mma_commit(&acc_full[buf]);
                ++j;
            }
        }
        __syncwarp();
    } else {
        const int q = warp & 3;
        int j = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            int n0 = (int)((tile_n(tile) + (unsigned)ep.tile_rot) % n_tiles) * BN, t_end = ep.T, group = 0;
            if (ep.groups != nullptr) {
                const int* gt = ep.groups + 3 * tile_n(tile);
                group = gt[0];
                if (group < 0) continue;
                n0 = gt[1];
                t_end = gt[2];
            }
            const int buf = j & 1;
            const uint32_t aph = (uint32_t)(j >> 1) & 1u;
            const int m0 = tile_m(tile) * 128;
            const int n = m0 + q * 32 + lane;
            if (!tc::mbar_wait(&acc_full[buf], aph)) { atomicExch(status, 3); break; }
            tc::fence_after_sync();
            const float bias = (ep.bias && n < ep.N && (ep.rs == nullptr || ep.rs->rank == 0)) ? ep.bias[(long)group * ep.N + n] : 0.f;
            if (ep.rs == nullptr) {
#pragma unroll 1
                for (int c = 0; c < BN / 16; ++c) {
                    uint32_t r[16];
                    tc::tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)buf * BN + c * 16, r);
                    tc::tmem_ld_wait();
                    if (n < ep.N) gemm_store16(ep, r, n, n0 + c * 16, t_end, bias);
                }
                tc::fence_before_sync();              // this warp's reads of the accumulator are complete
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
            } else {
                // GEMM -> reduce-scatter: this rank's slot of the token owner's accumulator, over NVLink.  Rows past T
                // are written too (zeros from the zero-filled X tile) so the owner never reads a stale slot row.
                const TpSeq* g = ep.rs;
                const int owner = n0 / g->shard;                    // a token tile never straddles two shards
                bf16* rs_dst = nullptr;
                if (owner < g->size)
                    rs_dst = g->acc[owner] + ((long)(*g->rs_phase & 1u) * g->size + g->rank) * g->shard * g->ld -
                             (long)owner * g->shard * g->ld;
                const int et = threadIdx.x - 64;                    // 0..127 among the epilogue threads
#pragma unroll 1
                for (int c = 0; c < BN / 16; ++c) {
                    uint32_t r[16];
                    tc::tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)buf * BN + c * 16, r);
                    tc::tmem_ld_wait();
                    bf16* st = rs_stage + (c & 1) * (16 * 128);
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj)
                        st[jj * 128 + q * 32 + lane] = f2bf(__uint_as_float(r[jj]) + (n0 + c * 16 + jj < ep.T ? bias : 0.f));
                    asm volatile("bar.sync 1, 128;" ::: "memory");  // the 16 x 128 chunk is complete
                    if (rs_dst != nullptr) {
                        // thread -> tokens et / 16 and et / 16 + 8, eight features: 16 threads cover one 256-byte row
#pragma unroll
                        for (int rr = 0; rr < 2; ++rr) {
                            const int tok = (et >> 4) + rr * 8, f0 = (et & 15) * 8;
                            const int nn = m0 + f0;
                            if (nn < ep.N) {                        // N is a multiple of 8 (checked by the host)
                                const uint4 v = *reinterpret_cast<const uint4*>(st + tok * 128 + f0);
                                *reinterpret_cast<uint4*>(rs_dst + (long)(n0 + c * 16 + tok) * g->ld + nn) = v;
                            }
                        }
                    }
                    // the other buffer is written next; this one again two chunks on, after the next barrier
                }
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
                __threadfence_system();                             // this thread's peer stores are visible before the arrival
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (et == 0) {
                    if (owner < g->size) red_release_inc_sys(g->rs_arrive[owner]);
                    const unsigned done = atomicAdd(g->ticket, 1u);
                    if (done == (unsigned)total_tiles - 1u) {
                        // every owner receives (feature tiles) x (token tiles per shard) arrivals from each rank
                        *g->ticket = 0;
                        __threadfence();
                        *g->rs_target += (unsigned)g->size * (unsigned)m_tiles * (unsigned)(g->shard / BN);
                    }
                }
            }
            ++j;
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc<TMEM_COLS>(tmem_base);
    }
}

template <int BN, int STAGES>
static int launch_gemm_persistent(const CUtensorMap& tw, const CUtensorMap& tx, const GemmEpi& ep, int K, int sms, int* status,
                                  cudaStream_t s) {
    using L = GemmSmem<BN, STAGES>;
    constexpr int SMEM = L::TOTAL + 256 + 2 * 16 * 128 * 2;      // more barriers than the one-tile kernel + the reduce-scatter staging rows
    static bool configured = false;
    if (!configured) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(gemm_bf16_persistent_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        configured = true;
    }
    // with a reduce-scatter epilogue the tiles also cover the padding rows of the last shard, so that every owner sees
    // the same number of arrivals
    const int t_cover = ep.rs != nullptr ? ep.rs_rows : ep.T;
    const int m_tiles = (ep.N + 127) / 128, n_tiles = (t_cover + BN - 1) / BN, total = m_tiles * n_tiles;
    const int grid = total < sms ? total : sms;
    static const int order_mode = []() { const char* e = getenv("TSB_GEMM_ORDER"); return e ? atoi(e) : -1; }();
    int n_fast = (ep.rs == nullptr && ep.ag == nullptr && ep.groups == nullptr && ep.N > t_cover) ? 1 : 0;
    if (order_mode >= 0 && ep.rs == nullptr && ep.ag == nullptr) n_fast = order_mode;
    TSB_CHECK_CUDA(tsb_launch(gemm_bf16_persistent_kernel<BN, STAGES>, dim3(grid), dim3(192), (size_t)SMEM, s, tw, tx, ep, K, m_tiles,
                              total, n_fast, status));
    return TSB_OK;
}

// ------------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static void resolve_encode() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
}

int tsb_make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                          uint32_t box_rows, uint32_t box_cols) {
    std::call_once(g_encode_once, resolve_encode);
    if (!g_encode) {
        tsb_set_error("cuTensorMapEncodeTiled is not available from the driver");
        return TSB_ERR_CUDA;
    }
    TSB_CHECK_ARG((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor map base %p is not 16-byte aligned", base);
    TSB_CHECK_ARG((row_stride_elems * 2) % 16 == 0, "tensor map row stride %llu elements is not a multiple of 16 bytes",
                  (unsigned long long)row_stride_elems);
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {row_stride_elems * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tsb_set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu box=%ux%u)", (int)r,
                      (unsigned long long)rows, (unsigned long long)cols, box_rows, box_cols);
        return TSB_ERR_CUDA;
    }
    return TSB_OK;
}

template <int BN, int STAGES, int MT = 1>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmEpi& ep, int K, int* status,
                       cudaStream_t s) {
    using L = GemmSmem<BN, STAGES, MT>;
    static bool configured = false;
    if (!configured) {
        TSB_CHECK_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            L::TOTAL));
        configured = true;
    }
    // with a reduce-scatter epilogue the grid also covers the padding rows of the last shard, so
    // that every owner sees the same number of arrivals
    const int t_cover = ep.rs != nullptr ? ep.rs_rows : ep.T;
    const int kb_all = (K + 63) / 64;
    const int splits = ep.ws != nullptr ? (kb_all + ep.kb_per_split - 1) / ep.kb_per_split : 1;
    dim3 grid((ep.N + 128 * MT - 1) / (128 * MT), (t_cover + BN - 1) / BN, splits);
    TSB_CHECK_CUDA(tsb_launch(gemm_bf16_kernel<BN, STAGES, MT>, grid, dim3(192), (size_t)L::TOTAL, s, tw, tx, ep, K, status));
    if (ep.ws != nullptr) {
        const long n = (long)ep.T * ep.N;
        TSB_CHECK_CUDA(tsb_launch(splitk_reduce_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, ep, splits));
    }
    return TSB_OK;
}

// W: [N, K] bf16 row-major (ldw elements per row); X: [T, K] bf16 (ldx); out: [T, ldo].
// `status` is a device int the kernel sets non-zero if one of its bounded waits gave up.
static int gemm_bf16_impl(const void* W, long ldw, const void* X, long ldx, void* out, long ldo, int out_f32,
                          const float* bias, const void* residual, int T, int N, int K, const void* rs, const void* ag, int shard,
                          int size, int rank, int* status, void* stream, void* splitk_ws, long splitk_ws_bytes);

extern "C" int tsb_gemm_bf16(const void* W, long ldw, const void* X, long ldx, void* out, long ldo, int out_f32,
                             const float* bias, const void* residual, int T, int N, int K, int* status, void* stream) {
    return gemm_bf16_impl(W, ldw, X, ldx, out, ldo, out_f32, bias, residual, T, N, K, nullptr, nullptr, 0, 1, 0, status, stream,
                          nullptr, 0);
}

// The plain GEMM with a caller-provided float32 workspace, which lets launches with few tiles and a long K split K.
extern "C" int tsb_gemm_bf16_ws(const void* W, long ldw, const void* X, long ldx, void* out, long ldo, int out_f32,
                                const float* bias, const void* residual, int T, int N, int K, int* status, void* stream,
                                void* ws, long ws_bytes) {
    return gemm_bf16_impl(W, ldw, X, ldx, out, ldo, out_f32, bias, residual, T, N, K, nullptr, nullptr, 0, 1, 0, status, stream,
                          ws, ws_bytes);
}

extern "C" int tsb_gemm_bf16_tp(const void* W, long ldw, const void* X, long ldx, void* out, long ldo, int out_f32,
                                const float* bias, const void* residual, int T, int N, int K, const void* rs,
                                const void* ag, int shard, int size, int rank, int* status, void* stream) {
    return gemm_bf16_impl(W, ldw, X, ldx, out, ldo, out_f32, bias, residual, T, N, K, rs, ag, shard, size, rank, status, stream,
                          nullptr, 0);
}

// The GEMM with the tensor-parallel prefill hooks: `rs` (device TpSeq*) sends the result to the token
// owners' accumulators instead of `out`; `ag` makes the producer wait for X's shards.  `shard` and
// `size` repeat the descriptor's values for the host-side launch arithmetic; the token tile is
// 128 rows so that it divides the shard.
static int gemm_bf16_impl(const void* W, long ldw, const void* X, long ldx, void* out, long ldo, int out_f32,
                          const float* bias, const void* residual, int T, int N, int K, const void* rs, const void* ag, int shard,
                          int size, int rank, int* status, void* stream, void* splitk_ws, long splitk_ws_bytes) {
    TSB_CHECK_ARG(T >= 0 && N > 0 && K > 0, "gemm_bf16: bad shape T=%d N=%d K=%d", T, N, K);
    TSB_CHECK_ARG((!rs && !ag) || (shard > 0 && shard % 128 == 0 && size >= 1), "gemm_bf16: shard=%d must be a multiple of 128", shard);
    TSB_CHECK_ARG(!rs || !residual, "gemm_bf16: reduce-scatter mode takes no residual");
    TSB_CHECK_ARG(K % 8 == 0 && ldw % 8 == 0 && ldx % 8 == 0, "gemm_bf16: K, ldw, ldx must be multiples of 8");
    TSB_CHECK_ARG(status != nullptr, "gemm_bf16: status word is required");
    if (T == 0) return TSB_OK;
    int bn = T <= 32 ? 32 : (T <= 64 ? 64 : (T <= 128 ? 128 : 256));
    if (bn == 256) {
        // 128 x 256 tiles run one per SM; when the tile count is just over a multiple of the SM count
        // the last wave is nearly empty (N = 2560, T = 2048: 160 tiles on 148 SMs).  Compare the two
        // tile widths by waves x per-tile cost (a 128-token tile re-reads the weight slab, hence +64).
        static int sms = 0;
        if (sms == 0) {
            int dev = 0;
            sms = 148;
            if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        }
        const long mt = (N + 127) / 128;
        const long w256 = (mt * ((T + 255) / 256) + sms - 1) / sms, w128 = (mt * ((T + 127) / 128) + sms - 1) / sms;
        if (w128 * (128 + 64) < w256 * (256 + 64)) bn = 128;
    }
    if (rs || ag) bn = shard % 256 == 0 ? 256 : 128;          // a token tile must not straddle two shards
    // Reduce-scatter epilogues stall on NVLink stores; with 128-token tiles and a 3-deep ring two
    // CTAs fit on an SM, so one CTA's epilogue overlaps the other's main loop.
    static const int rs_small = []() { const char* e = getenv("TSB_TP_RS_TILE"); return e ? atoi(e) : 256; }();
    const bool two_per_sm = rs && rs_small == 128;
    if (two_per_sm) bn = 128;
    // 256 x 256 tiles (two accumulators per CTA): two thirds of the L2 bytes per FLOP of the 128 x 256 tile.  Measured
    // on 8192 x 19456 x 2560: 652 against 623 TFLOP/s, and nothing at 2048 tokens, so it is opt-in (TSB_GEMM_WIDE=1: when
    // there are at least three waves of such tiles; 2: always); the persistent kernel below is what the default takes.
    static const int wide_mode = []() { const char* e = getenv("TSB_GEMM_WIDE"); return e ? atoi(e) : 0; }();
    bool wide = false;
    if (bn == 256 && !rs && !ag && wide_mode != 0) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long tiles = (long)((N + 255) / 256) * ((T + 255) / 256);
        wide = tiles >= 3L * sms || wide_mode == 2;
    }
    CUtensorMap tw, tx;
    int rc = tsb_make_tmap_2d_bf16(&tw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, wide ? 256 : 128, 64);
    if (rc) return rc;
    rc = tsb_make_tmap_2d_bf16(&tx, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)bn, 64);
    if (rc) return rc;
    // Visit order of the token tiles.  all-gather -> GEMM starts with this rank's own shard (already
    // here) so that waiting for remote shards overlaps useful work; GEMM -> reduce-scatter starts with
    // the next rank's shard and ends with its own, so remote owners receive their tiles first.
    int rot = 0;
    if (ag) rot = rank * (shard / bn);
    if (rs) rot = ((rank + 1) % size) * (shard / bn);
    GemmEpi ep{out, bias, residual, ldo, T, N, out_f32, (const TpSeq*)rs, (const TpSeq*)ag, shard * size, rot};
    cudaStream_t s = (cudaStream_t)stream;
    // Few tiles and a long K (decode batches): split K over CTAs so that the weight stream uses the whole GPU.
    if (!rs && !ag && splitk_ws != nullptr && bn <= 64) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int tiles = ((N + 127) / 128) * ((T + bn - 1) / bn), kb_all = (K + 63) / 64;
        int want = sms / (tiles > 0 ? tiles : 1);
        if (want > 8) want = 8;
        if (want > kb_all / 4) want = kb_all / 4;
        if (want >= 2 && (long)want * T * N * 4 <= splitk_ws_bytes) {
            ep.kb_per_split = (kb_all + want - 1) / want;
            ep.ws = (float*)splitk_ws;
        }
    }
    // plain GEMMs with more tiles than SMs: the persistent kernel (epilogue of a tile under the next tile's main loop)
    static const int persist_mode = []() { const char* e = getenv("TSB_GEMM_PERSISTENT"); return e ? atoi(e) : 1; }();
    if (!wide && persist_mode != 0 && (bn == 256 || bn == 128) && !two_per_sm && (!rs || N % 8 == 0)) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long tiles = (long)((N + 127) / 128) * (((rs ? shard * size : T) + bn - 1) / bn);
        if (tiles > sms || persist_mode == 2)
            return bn == 256 ? launch_gemm_persistent<256, 4>(tw, tx, ep, K, sms, status, s)
                             : launch_gemm_persistent<128, 6>(tw, tx, ep, K, sms, status, s);
    }
    switch (bn) {
    case 32: return launch_gemm<32, 8>(tw, tx, ep, K, status, s);
    case 64: return launch_gemm<64, 8>(tw, tx, ep, K, status, s);
    case 128: return two_per_sm ? launch_gemm<128, 3>(tw, tx, ep, K, status, s) : launch_gemm<128, 6>(tw, tx, ep, K, status, s);
    default: return wide ? launch_gemm<256, 3, 2>(tw, tx, ep, K, status, s) : launch_gemm<256, 4>(tw, tx, ep, K, status, s);
    }
}

// Grouped GEMM over a stack of matrices (mixture-of-experts prefill): W [E * N, K] bf16, X [P, K] bf16 with the rows of
// each group contiguous, `groups` a device list of `n_tiles` entries {matrix index or -1, first row, end row} whose
// tiles hold at most `bn` rows (32, 64, 128 or 256).  out [P, ldo]; bias [E, N] or null.  Rows that no tile covers are
// left as they are.  The host passes only upper bounds (P, n_tiles): the list itself is built by device code.
extern "C" int tsb_gemm_bf16_grouped(const void* W, long ldw, int E, const void* X, long ldx, void* out, long ldo, int out_f32,
                                     const float* bias, int P, int N, int K, const int* groups, int n_tiles, int bn,
                                     int* status, void* stream) {
    TSB_CHECK_ARG(P >= 0 && N > 0 && K > 0 && E > 0 && n_tiles >= 0, "gemm_bf16_grouped: bad shape P=%d N=%d K=%d E=%d", P, N, K, E);
    TSB_CHECK_ARG(K % 8 == 0 && ldw % 8 == 0 && ldx % 8 == 0, "gemm_bf16_grouped: K, ldw, ldx must be multiples of 8");
    TSB_CHECK_ARG(bn == 32 || bn == 64 || bn == 128 || bn == 256, "gemm_bf16_grouped: tile of %d rows", bn);
    TSB_CHECK_ARG(status != nullptr && groups != nullptr, "gemm_bf16_grouped: status word and tile list are required");
    if (P == 0 || n_tiles == 0) return TSB_OK;
    CUtensorMap tw, tx;
    int rc = tsb_make_tmap_2d_bf16(&tw, W, (uint64_t)E * N, (uint64_t)K, (uint64_t)ldw, 128, 64);
    if (rc) return rc;
    rc = tsb_make_tmap_2d_bf16(&tx, X, (uint64_t)P, (uint64_t)K, (uint64_t)ldx, (uint32_t)bn, 64);
    if (rc) return rc;
    GemmEpi ep{out, bias, nullptr, ldo, n_tiles * bn, N, out_f32, nullptr, nullptr, 0, 0, groups};
    cudaStream_t s = (cudaStream_t)stream;
    static const int persist_mode = []() { const char* e = getenv("TSB_GEMM_PERSISTENT"); return e ? atoi(e) : 1; }();
    if (persist_mode != 0 && (bn == 256 || bn == 128)) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if ((long)((N + 127) / 128) * n_tiles > sms)
            return bn == 256 ? launch_gemm_persistent<256, 4>(tw, tx, ep, K, sms, status, s)
                             : launch_gemm_persistent<128, 6>(tw, tx, ep, K, sms, status, s);
    }
    switch (bn) {
    case 32: return launch_gemm<32, 8>(tw, tx, ep, K, status, s);
    case 64: return launch_gemm<64, 8>(tw, tx, ep, K, status, s);
    case 128: return launch_gemm<128, 6>(tw, tx, ep, K, status, s);
    default: return launch_gemm<256, 4>(tw, tx, ep, K, status, s);
    }
}
