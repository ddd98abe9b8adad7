// The kernels of the decode chain (batches of at most 8 tokens):
//
//   embed -> per layer: wqkv -> attention -> wo -> w13 (+ gate) -> w2 -> ... -> output head -> argmax
//
// A BitLinear at batch 1 moves 1.6-8.8 MB of packed weights: about a microsecond of HBM time,
// as much as one kernel boundary costs (0.9 us measured on B200 with programmatic dependent
// launch).  The step is therefore bound by the latency of its chain of dependent phases and by
// the number of instructions each phase executes on every SM, and these kernels are built to
// keep both small:
//  * every kernel lets its successor start at once (griddepcontrol.launch_dependents first);
//    the successor's CTAs bring their share of the weight matrix into shared memory with bulk
//    asynchronous copies - weights do not depend on the predecessor - and only then wait for it;
//  * a CTA owns whole 16-row groups of the weight matrix, so no partial sums cross CTAs: no
//    atomics on sums in global memory, no scratch buffer, no tickets;
//  * every CTA needs the whole quantised input vector, so the prologue is work that all SMs
//    repeat: it is cut to the bone.  The producer of a vector x stores, next to x, the products
//    t = x * g with the weight g of the RMSNorm in front of the NEXT BitLinear, and accumulates
//    the statistics of x (sum of squares, max |t|) in one slot per token; the consumer's prologue
//    is then one load of the slot, one rsqrt, and per element a multiply, a bf16 rounding, a
//    multiply and a rounding to int8 - no reduction over the vector, no norm weight
//    (gpu/model.py:68-71 behind the norms of :159-160, :195-196, :237-242);
//  * the gate of the feed-forward block (gpu/model.py:193-195) is applied by w13's epilogue: a
//    CTA owns gate row group u together with up row group u + F/16, so w2 reads a vector of F
//    gated values instead of 2 F.
#include <cuda.h>

#include "common.cuh"
#include "decode_fused.h"
#include "prologue.cuh"
#include "decode_device.cuh"

namespace bitnet {

namespace {

constexpr int kCStageTiles = 32;
constexpr int kCStageBytes = kCStageTiles * kTileBytes;     // 16 KB
constexpr int kCWarps = 8;                                  // consumer warps
constexpr int kCThreads = kCWarps * 32;
constexpr int kCLinearThreads = kCThreads + 32;             // + one producer warp
constexpr int kCMaxStages = 8;

#ifdef BITNET_TRACE
#define CHAIN_STAMP(i)                                                   \
    if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) {                \
        unsigned long long t_;                                           \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));           \
        p.trace[i] = t_;                                                 \
    }
#else
#define CHAIN_STAMP(i)
#endif

__device__ __forceinline__ void chain_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kCThreads) : "memory"); }

// Adds a CTA's share to a statistics slot (device scope, or system scope for a slot in another
// rank's memory).
__device__ __forceinline__ void stat_add(StatPart* slot, double ss, float mx, bool system_scope) {
    unsigned long long* mxp = reinterpret_cast<unsigned long long*>(&slot->mx);
    const unsigned long long bits = (unsigned long long)__double_as_longlong((double)mx);   // mx >= 0: bit patterns order like values
    if (system_scope) {
        atomicAdd_system(&slot->ss, ss);
        atomicMax_system(mxp, bits);
    } else {
        atomicAdd(&slot->ss, ss);
        atomicMax(mxp, bits);
    }
}

// Tensor parallel, last CTA of a grid: this GPU's total of token m in `local` goes to its packets in
// every rank's area, and `local` is cleared for its next use.
__device__ __forceinline__ void stat_forward(const TpPeers& tp, size_t off, int M, int m, StatPart* local, unsigned int tag) {
    const double ss = __ldcg(&local[m].ss);
    const double mxd = __ldcg(&local[m].mx);
    local[m].ss = 0.0;
    local[m].mx = 0.0;
    tp_put_stats(tp, off, M, m, ss, (float)mxd, tag);
}

struct ChainSmem {
    uint8_t* ring;
    uint64_t *full_bar, *empty_bar;
    float *a_s, *stat_f;
    int *ysum_s, *flag_s, *sacc;
    double* stat_d;
    int8_t* ys;
};
// Shared-memory layout (host and device use the same arithmetic).
__host__ __device__ inline size_t chain_carve(const ChainLinearParams& p, uint8_t* base, ChainSmem* s) {
    const size_t k_pad = (size_t)p.k_tiles * kTileCols;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 15) / 16 * 16; return o; };
    const size_t o_ring = take((size_t)p.ring_stages * kCStageBytes);
    const size_t o_bar = take(2 * kCMaxStages * sizeof(uint64_t));
    const size_t o_misc = take(32 * sizeof(float));
    const size_t o_statd = take((size_t)8 * p.units_max * sizeof(double));
    const size_t o_statf = take((size_t)8 * p.units_max * sizeof(float));
    const size_t o_sacc = take((size_t)p.units_max * p.n_sub * 128 * sizeof(int));
    const size_t o_ys = take((size_t)p.M * (k_pad + 16));
    if (s) {
        s->ring = base + o_ring;
        s->full_bar = reinterpret_cast<uint64_t*>(base + o_bar);
        s->empty_bar = s->full_bar + kCMaxStages;
        float* misc = reinterpret_cast<float*>(base + o_misc);
        s->a_s = misc;
        s->ysum_s = reinterpret_cast<int*>(misc + 8);
        s->flag_s = reinterpret_cast<int*>(misc + 16);
        s->stat_d = reinterpret_cast<double*>(base + o_statd);
        s->stat_f = reinterpret_cast<float*>(base + o_statf);
        s->sacc = reinterpret_cast<int*>(base + o_sacc);
        s->ys = reinterpret_cast<int8_t*>(base + o_ys);
    }
    return off;
}

// ---------------------------------------------------------------------------------------
// BitLinear of the chain.  288 threads: 8 consumer warps and one producer warp; two CTAs fit an SM, so
// that the successor kernel's CTAs are resident, and past their set-up, while this kernel still runs.
// ---------------------------------------------------------------------------------------
// kTp: the tensor-parallel paths (packets from and to other ranks) exist only in the instantiations
// that a tensor-parallel decoder launches, so that they cost the single-GPU kernels nothing.
template <bool kOneToken, bool kTp>
__global__ void __launch_bounds__(kCLinearThreads, 2) chain_linear_kernel(const ChainLinearParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    ChainSmem sm;
    chain_carve(p, smem, &sm);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    CHAIN_STAMP(0)

    // this CTA's units and the tile sequence they make: for each of the n_sub row-group sets,
    // the tiles of row groups u0 .. u1-1 (+ set * sub_stride), one contiguous range of the matrix
    const int u0 = cta * p.units_base + min(cta, p.units_rem);      // the first units_rem CTAs take one unit more
    const int nu = p.units_base + (cta < p.units_rem ? 1 : 0);
    const int seg_tiles = nu * p.k_tiles;                  // tiles per contiguous range
    const int n_tiles = seg_tiles * p.n_sub;
    const int n_chunks = (n_tiles + kCStageTiles - 1) / kCStageTiles;
    const int s_mask = p.ring_stages - 1;                  // ring_stages is a power of two

    if (tid == 0) {
#pragma unroll 1
        for (int s = 0; s <= s_mask; ++s) {
            mbar_init(&sm.full_bar[s], 1);
            mbar_init(&sm.empty_bar[s], kCWarps);
        }
        sm.flag_s[0] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kCWarps) {
        // ---- producer: streams the weight tiles; independent of the predecessor kernel ----
        if (lane == 0) {
            const uint64_t policy = l2_evict_first_policy();
#pragma unroll 1
            for (int c = 0; c < n_chunks; ++c) {
                const int s = c & s_mask;
                if (c > s_mask && !mbar_wait(&sm.empty_bar[s], ((c / p.ring_stages) - 1) & 1)) {
                    atomicExch(p.error_flag, kErrProducerWait);
                    break;
                }
                int t = c * kCStageTiles;
                const int end = min(t + kCStageTiles, n_tiles);
                mbar_expect_tx(&sm.full_bar[s], (uint32_t)(end - t) * kTileBytes);
#pragma unroll 1
                while (t < end) {    // a chunk may straddle the boundary between two ranges
                    const int set = t / seg_tiles, off = t - set * seg_tiles;
                    const int n = min(end - t, seg_tiles - off);
                    const uint8_t* src = p.w2t + ((int64_t)(u0 + set * p.sub_stride) * p.k_tiles + off) * kTileBytes;
                    bulk_g2s(sm.ring + s * kCStageBytes + (t - c * kCStageTiles) * kTileBytes, src, (uint32_t)n * kTileBytes,
                             &sm.full_bar[s], policy);
                    t += n;
                }
            }
        }
        return;
    }

    // ---- consumers ---------------------------------------------------------------------
    const int K = p.K, n_vec = K / 8;                      // K is a multiple of 8
    const int k_pad = p.k_tiles * kTileCols;
    const int y_stride = k_pad + 16;
    const int n_lg = nu * p.n_sub;                         // local row groups
#pragma unroll 1
    for (int i = tid; i < n_lg * 128; i += kCThreads) sm.sacc[i] = 0;
    if (tid < 8) sm.ysum_s[tid] = 0;
    // the padding of the token rows
    if (k_pad > K) {
#pragma unroll 1
        for (int i = tid; i < p.M * ((k_pad - K) / 8); i += kCThreads) {
            const int m = i / ((k_pad - K) / 8), v = i - m * ((k_pad - K) / 8);
            *reinterpret_cast<uint2*>(sm.ys + (size_t)m * y_stride + K + v * 8) = make_uint2(0, 0);
        }
    }
    // What the epilogue needs and the predecessor does not produce: this thread's first output
    // (consecutive threads -> consecutive rows), its weight scales and the next norm's weight.
    const int total_out = nu * 16 * p.M;
    const int n_out_rows = p.out_kind == kOutGlu ? p.N / 2 : p.N;
    int e_m = 0, e_lu = 0, e_r = 0;
    if (tid < total_out) {
        e_m = tid / (nu * 16);
        const int rem = tid - e_m * (nu * 16);
        e_lu = rem >> 4;
        e_r = rem & 15;
    }
    const int e_row = (u0 + e_lu) * 16 + e_r;
    const bool e_live = tid < total_out && e_row < n_out_rows;
    float e_ws0 = 0.f, e_ws1 = 0.f, e_g = 1.f;
    if (e_live) {
        e_ws0 = p.ws[segment_of(p.seg, e_row)];
        if (p.out_kind == kOutGlu) e_ws1 = p.ws[segment_of(p.seg, e_row + p.sub_stride * 16)];
        if (p.gamma_out) e_g = __bfloat162float(p.gamma_out[e_row]);
    }

    float e_h = 0.f;
    constexpr bool real = true;
    {
    if (real) {
        CHAIN_STAMP(1)
        pdl_wait();   // the predecessor's results are visible from here on
        CHAIN_STAMP(2)
        if (e_live && p.out_kind == kOutResidual)
            e_h = __bfloat162float(__ldcg(reinterpret_cast<const __nv_bfloat16*>(p.out) + (int64_t)e_m * p.ldo + e_row));
        if (p.zero_slot && cta == 0 && tid < p.M) {
            p.zero_slot[tid].ss = 0.0;
            p.zero_slot[tid].mx = 0.0;
        }
    }

    // ---- prologue: int8 activations of every token into shared memory ----------------------
    // A thread takes 8 consecutive values of t (two 16-byte loads) and the token's statistics
    // (one 16-byte load, the same for all threads), derives the factors itself and writes 8 bytes.
#pragma unroll 1
    for (int m = 0; m < p.M; ++m) {
        double2 st = make_double2(0.0, 0.0);
        if (!kTp || !p.tp_stats_in) st = __ldcg(reinterpret_cast<const double2*>(p.stats_in + m));
        const float* tm = p.t + (int64_t)m * p.ldt;
        constexpr int kIt = 1024 / kCThreads;               // 8192 values per pass: all of a pass's loads in flight at once
        float4 lo[kIt], hi[kIt];
        auto fetch = [&](int v0) {
#pragma unroll
            for (int it = 0; it < kIt; ++it) {
                const int v = v0 + tid + it * kCThreads;
                if (v < n_vec) {
                    lo[it] = __ldcg(reinterpret_cast<const float4*>(tm + v * 8));
                    hi[it] = __ldcg(reinterpret_cast<const float4*>(tm + v * 8 + 4));
                }
            }
        };
        fetch(0);
        if (kTp && p.tp_stats_in) {
            // tensor parallel: the statistics are the sum over all ranks' packets; lane 0 of every warp
            // gathers them (this rank's own vector is already on its way: the loads above)
            double ss = 0.0;
            float mx = 0.f;
            // (a step that has already given up somewhere does not wait again)
            if (lane == 0 && !tp_get_stats(p.tp_stats_in, p.tp.size, p.M, m, tp_tag(p.tp_tag_in),
                                           __ldcg(p.error_flag) ? 0 : p.tp_tag_in.limit_cycles, ss, mx))
                atomicExch(p.error_flag, kErrPeerWait);
            st.x = __shfl_sync(0xffffffffu, ss, 0);
            st.y = (double)__shfl_sync(0xffffffffu, mx, 0);
        }
        float rinv, a;
        finish_stats(st.x, (float)st.y, p.k_norm, p.eps, true, rinv, a);
        int8_t* ym = sm.ys + (size_t)m * y_stride;
        int sy = 0;
        auto quantise = [&](const float4 (&cl)[kIt], const float4 (&ch)[kIt], int v0) {
#pragma unroll
            for (int it = 0; it < kIt; ++it) {
                const int v = v0 + tid + it * kCThreads;
                if (v < n_vec) {
                    const float f[8] = {cl[it].x, cl[it].y, cl[it].z, cl[it].w, ch[it].x, ch[it].y, ch[it].z, ch[it].w};
                    int q[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) q[e] = quant_s8(bf16_round(f[e] * rinv) * a);
                    const uint32_t w0 = pack_bytes(q[0], q[1], q[2], q[3]), w1 = pack_bytes(q[4], q[5], q[6], q[7]);
                    sy = __dp4a((int)w0, 0x01010101, sy);
                    sy = __dp4a((int)w1, 0x01010101, sy);
                    *reinterpret_cast<uint2*>(ym + v * 8) = make_uint2(w0, w1);
                }
            }
        };
        if (n_vec <= kIt * kCThreads) {
            quantise(lo, hi, 0);             // the usual case: one pass
        } else {
#pragma unroll 1
            for (int v0 = 0; v0 < n_vec; v0 += kIt * kCThreads) {
                float4 cl[kIt], ch[kIt];
#pragma unroll
                for (int it = 0; it < kIt; ++it) { cl[it] = lo[it]; ch[it] = hi[it]; }
                if (v0 + kIt * kCThreads < n_vec) fetch(v0 + kIt * kCThreads);     // the next pass, in flight during this one
                quantise(cl, ch, v0);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sy += __shfl_xor_sync(0xffffffffu, sy, o);
        if (lane == 0 && real) atomicAdd(&sm.ysum_s[m], sy);
        if (tid == 0) sm.a_s[m] = a;
    }
    if (real) { CHAIN_STAMP(8) }
    chain_sync();   // ys, ysum_s, a_s complete
    if (real) { CHAIN_STAMP(3) }

    // ---- matmul over the staged tiles ----------------------------------------------------
    // Per tile a lane holds the weights of rows g, g+8 in columns 32q .. 32q+31: four words whose
    // four 2-bit fields are separated by AND masks alone (field j stays scaled by 4^j and has its
    // own accumulator, folded by exact shifts at the end).  One token: eight dp4a per field pair
    // against the lane's 32 activation bytes (cheaper than tensor-core MMAs that would leave seven
    // of eight columns empty).  Two to eight tokens: four m16n8k32 MMAs per tile with the tokens as
    // the MMA's columns, so that any such M costs the same.
    const int g = lane >> 2, q = lane & 3;
    constexpr bool one_token = kOneToken;                  // the launcher picks the instantiation by M
    // MMA column g is token g; lanes whose column has no token feed zeros and load nothing
    const bool has_token = one_token || g < p.M;
    const int8_t* y_lane = sm.ys + (size_t)((!one_token && has_token) ? g : 0) * y_stride + 32 * q;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    int acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0;
    bool gave_up = false;
#ifdef BITNET_TRACE
    long long tr_wait = 0, tr_flush = 0, tr_t0 = clock64(), tr_a;
#define TR_BEGIN tr_a = clock64();
#define TR_END(x) x += clock64() - tr_a;
#else
#define TR_BEGIN
#define TR_END(x)
#endif
    // The warp's sums of one row group into the CTA's accumulator.
    auto flush = [&](int lg) {
        TR_BEGIN
        int* dst = sm.sacc + lg * 128;
        if (one_token) {
            int v0 = acc[0][0] + (acc[1][0] >> 2) + (acc[2][0] >> 4) + (acc[3][0] >> 6);
            int v1 = acc[0][1] + (acc[1][1] >> 2) + (acc[2][1] >> 4) + (acc[3][1] >> 6);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1); v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2); v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            if (q == 0) {
                atomicAdd(&dst[g * 8], v0);
                atomicAdd(&dst[(g + 8) * 8], v1);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) { acc[j][0] = 0; acc[j][1] = 0; }
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int tok = 2 * q + (e & 1);
                const int v = acc[0][e] + (acc[1][e] >> 2) + (acc[2][e] >> 4) + (acc[3][e] >> 6);
                if (tok < p.M) atomicAdd(&dst[(g + 8 * (e >> 1)) * 8 + tok], v);
                acc[0][e] = 0; acc[1][e] = 0; acc[2][e] = 0; acc[3][e] = 0;
            }
        }
        TR_END(tr_flush)
    };
    // One tile: the lane's 16 weight bytes against its 32 activation bytes.
    auto one_tile = [&](const uint4 wc, const uint4 y0, const uint4 y1) {
        const uint32_t b[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
        const uint32_t w[4] = {wc.x, wc.y, wc.z, wc.w};
        if (one_token) {
            // acc[j][0], acc[j][1]: rows g, g+8 of field j, summed over this lane's columns
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t msk = 0x03030303u << (2 * j);
                acc[j][0] = dp4a_u8s8(w[0] & msk, b[2 * j], acc[j][0]);
                acc[j][1] = dp4a_u8s8(w[1] & msk, b[2 * j], acc[j][1]);
                acc[j][0] = dp4a_u8s8(w[2] & msk, b[2 * j + 1], acc[j][0]);
                acc[j][1] = dp4a_u8s8(w[3] & msk, b[2 * j + 1], acc[j][1]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t msk = 0x03030303u << (2 * j);
                mma_u8s8(acc[j], w[0] & msk, w[1] & msk, w[2] & msk, w[3] & msk, b[2 * j], b[2 * j + 1]);
            }
        }
    };
    // n consecutive tiles, the first one local tile number t_first at `tile` (this lane's 16 bytes).
    // The run is cut where a row group ends; within a piece four tiles are loaded before any is used.
    auto run_tiles = [&](const uint8_t* tile, int n, int t_first) {
        int lg = t_first / p.k_tiles, kt = t_first - lg * p.k_tiles;
#pragma unroll 1
        while (n > 0) {
            const int piece = min(n, p.k_tiles - kt);
            const uint8_t* yk = reinterpret_cast<const uint8_t*>(y_lane) + kt * kTileCols;
            int i = 0;
#pragma unroll 1
            for (; i + 4 <= piece; i += 4, tile += 4 * kTileBytes, yk += 4 * kTileCols) {
                uint4 wc[4], y0[4], y1[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    wc[u] = *reinterpret_cast<const uint4*>(tile + u * kTileBytes);
                    y0[u] = has_token ? *reinterpret_cast<const uint4*>(yk + u * kTileCols) : zero4;
                    y1[u] = has_token ? *reinterpret_cast<const uint4*>(yk + u * kTileCols + 16) : zero4;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) one_tile(wc[u], y0[u], y1[u]);
            }
            if (i < piece) {     // up to three tiles left: again all loads first
                uint4 wc[3], y0[3], y1[3];
#pragma unroll
                for (int u = 0; u < 3; ++u) {
                    if (i + u < piece) {
                        wc[u] = *reinterpret_cast<const uint4*>(tile + u * kTileBytes);
                        y0[u] = has_token ? *reinterpret_cast<const uint4*>(yk + u * kTileCols) : zero4;
                        y1[u] = has_token ? *reinterpret_cast<const uint4*>(yk + u * kTileCols + 16) : zero4;
                    }
                }
#pragma unroll
                for (int u = 0; u < 3; ++u)
                    if (i + u < piece) one_tile(wc[u], y0[u], y1[u]);
                tile += (piece - i) * kTileBytes;
            }
            flush(lg);
            n -= piece;
            kt += piece;
            if (kt == p.k_tiles) {
                kt = 0;
                ++lg;
            }
        }
    };
    if (kOneToken || n_chunks <= p.ring_stages) {     // (the one-token form is only launched for resident shares)
        // The CTA's whole share sits in the ring (the usual case up to a few billion parameters):
        // every warp takes one contiguous run of it, nothing is released or refilled.
        const int lo_t = n_tiles * warp / kCWarps, hi_t = n_tiles * (warp + 1) / kCWarps;
        if (hi_t > lo_t) {
            bool ok = true;
            TR_BEGIN
#pragma unroll 1
            for (int c = lo_t / kCStageTiles; c <= (hi_t - 1) / kCStageTiles; ++c) ok = ok && mbar_wait(&sm.full_bar[c], 0);
            TR_END(tr_wait)
            CHAIN_STAMP(9)
            if (ok) {
                run_tiles(sm.ring + lo_t * kTileBytes + lane * 16, hi_t - lo_t, lo_t);
            } else if (lane == 0) {
                atomicExch(p.error_flag, kErrConsumerWait);
                sm.flag_s[0] = 1;
            }
        }
    } else {
        // Larger shares stream through the ring in rounds of two stages (up to 64 tiles); within
        // a round each warp takes one contiguous run.
        const int round_stages = p.ring_stages >> 1;         // half of the ring is worked on, the other half in flight
        const int kRoundTiles = round_stages * kCStageTiles;
        const int n_rounds = (n_tiles + kRoundTiles - 1) / kRoundTiles;
#pragma unroll 1
        for (int r = 0; r < n_rounds && !gave_up; ++r) {
            const int nr_t = min(kRoundTiles, n_tiles - r * kRoundTiles);
            const int lo_t = nr_t * warp / kCWarps, hi_t = nr_t * (warp + 1) / kCWarps;
            const int c0 = r * round_stages;                     // first chunk of the round
            if (hi_t > lo_t) {
                bool ok = true;
                TR_BEGIN
#pragma unroll 1
                for (int ls = lo_t / kCStageTiles; ls <= (hi_t - 1) / kCStageTiles; ++ls)
                    ok = ok && mbar_wait(&sm.full_bar[(c0 + ls) & s_mask], ((c0 + ls) / p.ring_stages) & 1);
                TR_END(tr_wait)
                if (!ok) {   // gave up: flag it, leave together below
                    if (lane == 0) {
                        atomicExch(p.error_flag, kErrConsumerWait);
                        sm.flag_s[0] = 1;
                    }
                    gave_up = true;
                }
            }
            if (r == 0) { CHAIN_STAMP(9) }
            // the two stages of a round are adjacent in the ring (ring_stages is even)
            if (!gave_up && hi_t > lo_t)
                run_tiles(sm.ring + (c0 & s_mask) * kCStageBytes + lo_t * kTileBytes + lane * 16, hi_t - lo_t, r * kRoundTiles + lo_t);
            __syncwarp();
            if (lane == 0 && !gave_up) {
                // This warp is done with every stage of the round.  It releases a stage only after
                // having seen that stage's copy complete (usually it has, long ago), so that no warp
                // ever waits for a later fill of a stage whose earlier fill it has not observed.
#pragma unroll 1
                for (int ls = 0; ls < round_stages; ++ls) {
                    const int c = c0 + ls;
                    if (c < n_chunks && mbar_wait(&sm.full_bar[c & s_mask], (c / p.ring_stages) & 1)) mbar_arrive(&sm.empty_bar[c & s_mask]);
                }
            }
        }
    }
#ifdef BITNET_TRACE
    if (real && p.trace && blockIdx.x == 0 && threadIdx.x == 0) {
        p.trace[11] = (unsigned long long)tr_wait;
        p.trace[12] = (unsigned long long)tr_flush;
        p.trace[13] = (unsigned long long)(clock64() - tr_t0);
        p.trace[14] = (unsigned long long)n_tiles;
    }
#endif
    if (real) { CHAIN_STAMP(4) }
    chain_sync();
    if (real) { CHAIN_STAMP(10) }
    if (real && (sm.flag_s[0] || n_tiles == 0)) return;

    // ---- epilogue --------------------------------------------------------------------------
    // Thread idx finalises output r of unit lu for token m; 16 consecutive threads hold the 16
    // outputs of one unit and token, and reduce their statistics by shuffles.
    const bool want_stats = p.stats_out != nullptr;
    const unsigned int part_tag = (kTp && p.out_kind == kOutTpPartial) ? tp_tag(p.tp_tag_out) : 0u;
#pragma unroll 1
    for (int base = 0; base < total_out; base += kCThreads) {
        const int idx = base + tid;
        const bool valid = idx < total_out;
        int m = e_m, lu = e_lu, r = e_r;
        float ws0 = e_ws0, ws1 = e_ws1, gq = e_g, h_old = e_h;
        bool live = e_live;
        if (base > 0) {            // more than 512 outputs per CTA: the general form
            m = 0; lu = 0; r = 0; live = false;
            if (valid) {
                m = idx / (nu * 16);
                const int rem = idx - m * (nu * 16);
                lu = rem >> 4;
                r = rem & 15;
                const int row = (u0 + lu) * 16 + r;
                live = row < n_out_rows;
                if (live) {
                    ws0 = p.ws[segment_of(p.seg, row)];
                    if (p.out_kind == kOutGlu) ws1 = p.ws[segment_of(p.seg, row + p.sub_stride * 16)];
                    gq = p.gamma_out ? __bfloat162float(p.gamma_out[row]) : 1.f;
                    if (p.out_kind == kOutResidual)
                        h_old = __bfloat162float(__ldcg(reinterpret_cast<const __nv_bfloat16*>(p.out) + (int64_t)m * p.ldo + row));
                }
            }
        }
        const int row = (u0 + lu) * 16 + r;                 // output index (glu: index of the gated value)
        float o = 0.f;
        if (live) {
            const float a = sm.a_s[m];
            const int ys_m = sm.ysum_s[m];                  // fields hold weight + 1: take sum(y) off once per row
            const int v0 = sm.sacc[lu * 128 + r * 8 + m] - ys_m;
            if (kTp && p.out_kind == kOutTpPartial) {
                // this rank's exact partial sums, as packets [rank][m][row] of every rank's area
                const size_t at = p.tp_part_off + (((size_t)p.tp.rank * p.M + m) * p.N + row) * sizeof(uint2);
#pragma unroll 1
                for (int pr = 0; pr < p.tp.size && real; ++pr) tp_put(p.tp.area[pr] + at, (unsigned int)v0, part_tag);
            } else {
                if (p.out_kind == kOutGlu) {
                    const int v1 = sm.sacc[(nu + lu) * 128 + r * 8 + m] - ys_m;
                    const float x1 = lin_out(v0, a, ws0), x3 = lin_out(v1, a, ws1);
                    const float tt = fmaxf(x1, 0.f);
                    o = bf16_round(bf16_round(tt * tt) * x3);   // rounded after each step, as bf16 tensor operations round
                } else {
                    const float lin = lin_out(v0, a, ws0);
                    o = p.out_kind == kOutResidual ? bf16_round(h_old + lin) : lin;
                    if (real) p.out[(int64_t)m * p.ldo + row] = __float2bfloat16_rn(o);
                }
                if (p.t_out && real) p.t_out[(int64_t)m * p.ldt_out + row] = o * gq;    // exact: both factors are bf16 values
            }
        }
        if (want_stats) {
            double ss = (double)o * (double)o;
            float mx = fabsf(o * gq);
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) {
                ss += __shfl_xor_sync(0xffffffffu, ss, off);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            }
            if (valid && (lane & 15) == 0) {      // the unit's share, to be added up per token below
                sm.stat_d[m * p.units_max + lu] = ss;
                sm.stat_f[m * p.units_max + lu] = mx;
            }
        }
    }
    if (want_stats) {
        // one share per token and CTA: the units' shares added in their order, then one atomic pair
        chain_sync();
        if (tid < p.M && real) {
            double ss = 0.0;
            float mx = 0.f;
#pragma unroll 1
            for (int lu = 0; lu < nu; ++lu) {
                ss += sm.stat_d[tid * p.units_max + lu];
                mx = fmaxf(mx, sm.stat_f[tid * p.units_max + lu]);
            }
            stat_add(p.stats_out + tid, ss, mx, false);
        }
        if (kTp && p.tp.size > 1 && real && warp == 0) {
            // Every rank normalises over the whole vector.  This GPU's CTAs add up in its own slot;
            // the last of them forwards the total to its packets in every rank's area.
            __syncwarp();            // the M adding threads are lanes of this warp
            int last = 0;
            if (lane == 0) last = tp_last_cta(p.tp_ticket, (unsigned int)gridDim.x) ? 1 : 0;
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last && lane < p.M) stat_forward(p.tp, p.tp_stats_off, p.M, lane, p.stats_out, tp_tag(p.tp_tag_out));
        }
    }
    if (kTp && p.out_kind == kOutTpPartial && real && cta == 0 && tid < p.M) p.a_out[tid] = sm.a_s[tid];
    CHAIN_STAMP(5)
    }
}

// ---------------------------------------------------------------------------------------
// First kernel of a step: the embedding rows of the new tokens start the residual stream; their
// products with layer 0's attention_norm weight and their statistics go where wqkv expects them.
// One CTA of 256 threads per token.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embed_kernel(const EmbedParams p) {
    __shared__ double sd[8];
    __shared__ float sf[8];
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x;
    if (p.zero_slot && tid == 0) {
        p.zero_slot[m].ss = 0.0;
        p.zero_slot[m].mx = 0.0;
    }
    int64_t tok = p.tokens[m];
    if (tok < 0 || tok >= p.vocab) {      // outside the vocabulary: flag it, use token 0
        if (tid == 0) atomicExch(p.error_flag, kErrToken);
        tok = 0;
    }
    const __nv_bfloat16* row = p.emb + tok * (int64_t)p.K;
    double ss = 0.0;
    float mx = 0.f;
#pragma unroll 1
    for (int v = tid; v < p.K / 8; v += 256) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + v * 8);
        const Vec8 x = unpack_bf16x8(raw), g = unpack_bf16x8(*reinterpret_cast<const uint4*>(p.gamma + v * 8));
        *reinterpret_cast<uint4*>(p.h + (int64_t)m * p.K + v * 8) = raw;
        float t[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            t[e] = x.v[e] * g.v[e];
            ss = fma((double)x.v[e], (double)x.v[e], ss);
            mx = fmaxf(mx, fabsf(t[e]));
        }
        *reinterpret_cast<float4*>(p.t + (int64_t)m * p.K + v * 8) = make_float4(t[0], t[1], t[2], t[3]);
        *reinterpret_cast<float4*>(p.t + (int64_t)m * p.K + v * 8 + 4) = make_float4(t[4], t[5], t[6], t[7]);
    }
    reduce_stats<256>(ss, mx, sd, sf, tid, [] { __syncthreads(); });
    if (tid == 0) {
        p.stats_out[m].ss = ss;
        p.stats_out[m].mx = (double)mx;
    }
}

// ---------------------------------------------------------------------------------------
// Second half of a row-parallel BitLinear under tensor parallelism: adds up the ranks' exact
// int32 partial sums, rescales, adds the residual, and hands h, t = h * g and the statistics of h
// to the next BitLinear.  Every rank does the whole vector (it needs all of h).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) tp_reduce_kernel(const TpReduceParams p) {
    __shared__ double sd[8];
    __shared__ float sf[8];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const unsigned int tag = tp_tag(p.tag);
    long long limit = __ldcg(p.error_flag) ? 0 : p.tag.limit_cycles;    // a step that has already given up does not wait again
    const int row = blockIdx.x * 256 + tid;
    const float gq = row < p.N ? __bfloat162float(p.gamma_out[row]) : 0.f;
#pragma unroll 1
    for (int m = 0; m < p.M; ++m) {
        float o = 0.f;
        if (row < p.N) {
            int v = 0;
            bool ok = true;
            // every thread takes its own packets: a pass that requests them all without waiting, then -
            // only if one was missing - a pass that waits packet by packet; integer sums: any order
            bool all = true;
#pragma unroll
            for (int r = 0; r < kMaxTp; ++r) {
                if (r < p.T) {
                    unsigned int x, t;
                    tp_peek(p.part + ((size_t)r * p.M + m) * p.N + row, x, t);
                    all = all && t == tag;
                    v += (int)x;
                }
            }
            if (!all) {
                v = 0;
#pragma unroll 1
                for (int r = 0; r < p.T; ++r) {
                    unsigned int x;
                    ok = tp_get(p.part + ((size_t)r * p.M + m) * p.N + row, tag, limit, x) && ok;
                    v += (int)x;
                }
            }
            if (!ok) {
                atomicExch(p.error_flag, kErrPeerWait);
                limit = 0;
            }
            const float h_old = __bfloat162float(p.out[(int64_t)m * p.ldo + row]);
            o = bf16_round(h_old + lin_out(v, p.a[m], p.ws));
            p.out[(int64_t)m * p.ldo + row] = __float2bfloat16_rn(o);
            p.t_out[(int64_t)m * p.ldo + row] = o * gq;
        }
        double ss = (double)o * (double)o;
        float mx = fabsf(o * gq);
        reduce_stats<256>(ss, mx, sd, sf, tid, [] { __syncthreads(); });
        if (tid == 0) stat_add(p.stats_out + m, ss, mx, false);
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------
// Attention of the chain.  One new token per sequence: RoPE on q and k, append k, v to the
// cache, softmax(q k^T / sqrt(D)) v (gpu/model.py:121-158).  Up to a context of 384 keys with
// few sequences every query head gets its own CTA and runs the short form below: all 512
// threads fetch keys and values at once - 16 lanes per key, 16 bytes per lane, up to 256 keys
// per pass with every load in flight before the first score is computed - so that the phase
// costs one memory latency instead of one per step of a key loop.  Longer contexts, larger
// batches and head sizes that are not a multiple of 8 take the split-KV body of
// decode_device.cuh.  Either way the CTA that writes a head's output also publishes the
// statistics for the RMSNorm + quantisation in front of wo.
// ---------------------------------------------------------------------------------------
constexpr int kAttnThreads = 512;
constexpr int kKeyRounds = 8;                     // keys per half-warp and pass

__device__ __forceinline__ void unpack8(const uint4& r, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        f[2 * e] = __low2float(h[e]);
        f[2 * e + 1] = __high2float(h[e]);
    }
}

// Statistics of one head's output for the next prologue: thread d < D holds value `val` of
// dimension d (others hold 0); the head's share goes to the sequence's slot.  `sd`/`sf` hold 16
// entries; every thread of the CTA must call.
template <class Sync>
__device__ __forceinline__ void publish_head_stats(const AttentionParams& p, int b, float val, float gq, int tid, double* sd,
                                                   float* sf, Sync sync) {
    double ss = (double)val * (double)val;
    float mx = fabsf(val * gq);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    sync();
    if ((tid & 31) == 0 && tid < 128) {
        sd[tid >> 5] = ss;
        sf[tid >> 5] = mx;
    }
    sync();
    if (tid == 0) {
        ss = sd[0] + sd[1] + sd[2] + sd[3];          // D <= 128: the values sit in the first four warps
        mx = fmaxf(fmaxf(sf[0], sf[1]), fmaxf(sf[2], sf[3]));
        stat_add(p.stats_out + b, ss, mx, false);
        // Tensor parallel: every rank's wo normalises over all heads.  This GPU's heads add up in its
        // own slots; the CTA that delivers the last head forwards the totals of all sequences to the
        // packets in every rank's area.
        if (p.tp.size > 1 && tp_last_cta(p.tp_ticket, (unsigned int)(gridDim.y * p.H))) {
            const unsigned int tag = tp_tag(p.tp_tag_out);
#pragma unroll 1
            for (int m = 0; m < (int)gridDim.y; ++m) stat_forward(p.tp, p.tp_stats_off, (int)gridDim.y, m, p.stats_out, tag);
        }
    }
}

// The short form: query head h of sequence b, D a multiple of 8.  Called after the dependency
// wait by all 512 threads.  Returns false (having stored nothing) when the context is too long
// for it; the caller then takes the split-KV body.
// Everything this kernel reads that an earlier kernel of the stream wrote - the position, the
// new token's q, k, v, and the cache rows - is read after the wait: with programmatic dependent
// launch a kernel's code in front of its wait may run while kernels further back in the stream
// are still running, so only true constants may be touched there.  To keep the phase at about
// one memory latency all the same, the first 256 cache rows are requested before the position
// has arrived (rows beyond it exist - the cache is allocated to its full length - and are
// masked out afterwards).
__device__ __forceinline__ bool attention_short(const AttentionParams& p, uint8_t* smem, int b, int h, int tid) {
    const int D = p.D, G = p.H / p.Hkv, kvh = h / G;
    const int hw = tid >> 4, l16 = tid & 15, d0 = 8 * l16;
    const bool live = d0 < D;
    float* red_m = reinterpret_cast<float*>(smem);      // [32] (16 used)
    float* red_l = red_m + 32;                          // [32]: 16 sums, 16 normalised weights
    float* sf = red_l + 32;                             // [16]
    double* sd = reinterpret_cast<double*>(sf + 16);    // [16]
    float* red_o = reinterpret_cast<float*>(sd + 16);   // [16][D]
    const int64_t key_stride = (int64_t)p.Hkv * D;
    const __nv_bfloat16* ck = p.cache_k + ((int64_t)b * p.L * p.Hkv + kvh) * D + d0;
    const __nv_bfloat16* cv = p.cache_v + ((int64_t)b * p.L * p.Hkv + kvh) * D + d0;
    const int P = (int)__ldcg(p.pos + b);
    uint4 kr[kKeyRounds], vr[kKeyRounds];
    const uint64_t keep = l2_evict_last_policy();
    auto load_block = [&](int j0, int j_end) {   // cache rows j0 + 32 r + hw, r < 8, below j_end
#pragma unroll
        for (int r = 0; r < kKeyRounds; ++r) {
            const int j = j0 + r * 32 + hw;
            kr[r] = make_uint4(0, 0, 0, 0);
            vr[r] = make_uint4(0, 0, 0, 0);
            if (j < j_end && live) {
                kr[r] = ldcg_keep(reinterpret_cast<const uint4*>(ck + j * key_stride), keep);   // L2: rows appended by earlier steps
                vr[r] = ldcg_keep(reinterpret_cast<const uint4*>(cv + j * key_stride), keep);
            }
        }
    };
    load_block(0, p.L);       // requested before P is known; rows >= P are masked below
    const __nv_bfloat16* x = p.xqkv + (int64_t)b * p.ld_qkv;
    uint4 q_raw = make_uint4(0, 0, 0, 0), k_raw = make_uint4(0, 0, 0, 0), v_new = make_uint4(0, 0, 0, 0);
    if (live) {      // L2: written by other SMs.  Every half-warp takes the new token's k and v: which one owns key P is not known yet
        q_raw = __ldcg(reinterpret_cast<const uint4*>(x + h * D + d0));
        k_raw = __ldcg(reinterpret_cast<const uint4*>(x + (p.H + kvh) * D + d0));
        v_new = __ldcg(reinterpret_cast<const uint4*>(x + (p.H + p.Hkv + kvh) * D + d0));
    }
    if (P < 0 || P >= p.L) {      // outside the cache: flag it, touch nothing
        if (tid == 0) atomicExch(p.error_flag, kErrPosition);
        return true;
    }
    if (attention_slices(p.S, P) != 1) return false;
    CHAIN_STAMP(1)
    // rotation of position P for this lane's pairs d0/2 .. d0/2+3
    const float* rope = p.rope + (int64_t)P * D + d0;
    float cs[8] = {1.f, 0.f, 1.f, 0.f, 1.f, 0.f, 1.f, 0.f};
    if (live) {
        const float4 r0 = *reinterpret_cast<const float4*>(rope), r1 = *reinterpret_cast<const float4*>(rope + 4);
        cs[0] = r0.x; cs[1] = r0.y; cs[2] = r0.z; cs[3] = r0.w; cs[4] = r1.x; cs[5] = r1.y; cs[6] = r1.z; cs[7] = r1.w;
    }
    auto rotate = [&](const uint4& raw, float (&out)[8]) {   // pairs (2i, 2i+1), products rounded separately, result to bf16
        float f[8];
        unpack8(raw, f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = bf16_round(__fmul_rn(f[2 * i], cs[2 * i]) - __fmul_rn(f[2 * i + 1], cs[2 * i + 1]));
            out[2 * i + 1] = bf16_round(__fmul_rn(f[2 * i], cs[2 * i + 1]) + __fmul_rn(f[2 * i + 1], cs[2 * i]));
        }
    };
    // q of this head, rotated and scaled; every half-warp holds a copy, lane l16 dims d0 .. d0+7
    float qv[8];
    {
        rotate(q_raw, qv);
        const float qscale = rsqrtf((float)D);
#pragma unroll
        for (int e = 0; e < 8; ++e) qv[e] *= qscale;
    }
    // the new token is key P: its owner half-warp takes k (rotated) and v from xqkv, and the CTA
    // of the kv head's first query head appends them to the cache
    const bool own_new = (P & 31) == hw;
    uint4 k_new = make_uint4(0, 0, 0, 0);
    if (own_new && live) {
        float kf[8];
        rotate(k_raw, kf);
        Vec8 kv8;
#pragma unroll
        for (int e = 0; e < 8; ++e) kv8.v[e] = kf[e];
        k_new = pack_bf16x8(kv8);
        if (h == kvh * G) {
            *reinterpret_cast<uint4*>(p.cache_k + (((int64_t)b * p.L + P) * p.Hkv + kvh) * D + d0) = k_new;
            *reinterpret_cast<uint4*>(p.cache_v + (((int64_t)b * p.L + P) * p.Hkv + kvh) * D + d0) = v_new;
        }
    }

    float m_run = -INFINITY, l_run = 0.f, o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = 0.f;
    const int n_keys = P + 1;
    CHAIN_STAMP(2)
#pragma unroll 1
    for (int j0 = 0; j0 < n_keys; j0 += 32 * kKeyRounds) {
        if (j0 > 0) load_block(j0, P);
        float sc[kKeyRounds];
        float m_blk = -INFINITY;
#pragma unroll
        for (int r = 0; r < kKeyRounds; ++r) {
            const int j = j0 + r * 32 + hw;
            if (j == P) {
                kr[r] = k_new;
                vr[r] = v_new;
            } else if (j > P) {       // requested before P was known: whatever the row holds must not count
                kr[r] = make_uint4(0, 0, 0, 0);
                vr[r] = make_uint4(0, 0, 0, 0);
            }
            float kf[8];
            unpack8(kr[r], kf);
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) s = fmaf(qv[e], kf[e], s);
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            sc[r] = j < n_keys ? s : -INFINITY;
            m_blk = fmaxf(m_blk, sc[r]);
        }
        if (m_blk > -INFINITY) {
            const float m_new = fmaxf(m_run, m_blk);
            const float corr = m_run > -INFINITY ? __expf(m_run - m_new) : 0.f;
            l_run *= corr;
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] *= corr;
#pragma unroll
            for (int r = 0; r < kKeyRounds; ++r) {
                const float pr = sc[r] > -INFINITY ? __expf(sc[r] - m_new) : 0.f;
                float vf[8];
                unpack8(vr[r], vf);
                l_run += pr;
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = fmaf(pr, vf[e], o[e]);
            }
            m_run = m_new;
        }
    }
    CHAIN_STAMP(3)
    // combine: first the two half-warps of a warp by shuffles, then the 16 warps through shared memory
    {
        const float m_o = __shfl_xor_sync(0xffffffffu, m_run, 16), l_o = __shfl_xor_sync(0xffffffffu, l_run, 16);
        const float m_n = fmaxf(m_run, m_o);
        const float f_me = m_run > -INFINITY ? __expf(m_run - m_n) : 0.f, f_ot = m_o > -INFINITY ? __expf(m_o - m_n) : 0.f;
        l_run = l_run * f_me + l_o * f_ot;
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = o[e] * f_me + __shfl_xor_sync(0xffffffffu, o[e], 16) * f_ot;
        m_run = m_n;
    }
    const int wp = tid >> 5;
    if ((tid & 31) == 0) {
        red_m[wp] = m_run;
        red_l[wp] = l_run;
    }
    if ((tid & 16) == 0 && live) {
        *reinterpret_cast<float4*>(red_o + wp * D + d0) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4*>(red_o + wp * D + d0 + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
    __syncthreads();
    if (tid < 32) {      // the warps' weights, normalised: exp(m_w - max) / sum
        const float mw = tid < 16 ? red_m[tid] : -INFINITY, lw = tid < 16 ? red_l[tid] : 0.f;
        float mx = mw;
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float f = mw > -INFINITY ? __expf(mw - mx) : 0.f;
        float l = lw * f;
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
        if (tid < 16) red_l[16 + tid] = l > 0.f ? f / l : 0.f;
    }
    __syncthreads();
    float val = 0.f, gq = 1.f;
    if (tid < D) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 16; ++w) acc = fmaf(red_o[w * D + tid], red_l[16 + w], acc);
        const __nv_bfloat16 ob = __float2bfloat16_rn(acc);
        const int64_t oi = (int64_t)b * p.H * D + h * D + tid;
        p.out[oi] = ob;
        if (p.tap) p.tap[oi] = ob;
        val = __bfloat162float(ob);
        if (p.stats_out) {
            gq = __bfloat162float(p.gamma_out[h * D + tid]);
            p.t_out[oi] = val * gq;                  // exact: both factors are bf16 values
        }
    }
    CHAIN_STAMP(4)
    if (p.stats_out) publish_head_stats(p, b, val, gq, tid, sd, sf, [] { __syncthreads(); });
    CHAIN_STAMP(5)
    return true;
}

// The 8-row tensor-core split-KV body of the 512-thread kernel, out of line: its register
// allocation (and what it spills at 128 registers) must not touch the short form's code.
__device__ __noinline__ bool attention_groups8(const AttentionParams& p, uint8_t* smem, int* is_last, int b, int kvh, int h0, int G,
                                               int split, int S, int P, int tid) {
    auto sync = [] { asm volatile("bar.sync 2, 512;\n" ::: "memory"); };
    return attention_body<8, 16, true>(p, smem, is_last, b, kvh, h0, G, split, S, P, tid, sync, [] {});
}

// NTHREADS = 512 (grouped-query ratios up to 4: short form and split-KV body share the CTA) or
// the split-KV body's own thread count (larger ratios: its register budget rules out 512
// threads, and the short form is left out).
template <int GMAX, int NTHREADS>
__global__ void __launch_bounds__(NTHREADS) chain_attention_kernel(const __grid_constant__ AttentionParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int is_last;
    static_assert(AttnCfg<GMAX>::kThreads <= NTHREADS, "the split-KV body uses a prefix of the CTA's warps");
    pdl_launch_dependents();
    pdl_wait();
    CHAIN_STAMP(0)
    const int b = blockIdx.y, tid = threadIdx.x;
    if (p.zero_slot && blockIdx.x == 0 && tid == 0) {
        p.zero_slot[b].ss = 0.0;
        p.zero_slot[b].mx = 0.0;
    }
    if constexpr (NTHREADS == kAttnThreads) {
        // candidates for the short form: one CTA per query head (see attention_item)
        if ((int)blockIdx.x < p.H && p.S >= p.H / p.Hkv && (p.D & 7) == 0 && attention_short(p, smem, b, blockIdx.x, tid)) return;
    }
    const int P = (int)__ldcg(p.pos + b);
    if (P < 0 || P >= p.L) {      // outside the cache: flag it, touch nothing
        if (tid == 0 && blockIdx.x == 0) atomicExch(p.error_flag, kErrPosition);
        return;
    }
    const AttnItem it = attention_item(p, blockIdx.x, P);
    if (it.G == 0) return;
    // the split-KV body runs on the first AttnCfg<GMAX>::kThreads threads
    constexpr int NT = AttnCfg<GMAX>::kThreads, NW = AttnCfg<GMAX>::kWarps;
    bool wrote = false;
    if (GMAX > 4 && it.G > 1 && p.D == 128) {
        // whole groups of more than four query heads at head_dim 128: the key loop on tensor cores, by
        // four warps (the 512-thread form of this kernel leaves a thread too few registers for it)
        if (tid < 128) {
            auto sync = [] { asm volatile("bar.sync 3, 128;\n" ::: "memory"); };
            wrote = attention_body<16, 4, true>(p, smem, &is_last, b, it.kvh, it.h0, it.G, it.split, it.S, P, tid, sync, [] {});
        }
    } else if (GMAX <= 4 && it.G > 1 && p.D == 128) {
        // whole groups of up to four query heads (long contexts, or many sequences): the 8-row form of
        // the tensor-core key loop, which fits this 512-thread kernel's 128 registers, on all 16 warps
        static_assert(GMAX > 4 || NT == 512, "attention_groups8 synchronises 512 threads");
        if (tid < NT) wrote = attention_groups8(p, smem, &is_last, b, it.kvh, it.h0, it.G, it.split, it.S, P, tid);
    } else if (tid < NT) {
        auto sync = [] { asm volatile("bar.sync 2, %0;\n" ::"n"(NT) : "memory"); };
        if (it.G == 1)
            wrote = attention_body<1, NW>(p, smem, &is_last, b, it.kvh, it.h0, 1, it.split, it.S, P, tid, sync, [] {});
        else
            wrote = attention_body<GMAX, NW>(p, smem, &is_last, b, it.kvh, it.h0, it.G, it.split, it.S, P, tid, sync, [] {});
    }
    if (!p.stats_out) return;
    // statistics of the heads this CTA wrote, read back from its own output
    __shared__ int wrote_s;
    if (tid == 0) wrote_s = wrote ? 1 : 0;
    __syncthreads();
    if (!wrote_s) return;
    float* sf = reinterpret_cast<float*>(smem);
    double* sd = reinterpret_cast<double*>(sf + 16);
    const int Gfull = p.H / p.Hkv;
#pragma unroll 1
    for (int hh = 0; hh < it.G; ++hh) {
        const int head = it.kvh * Gfull + it.h0 + hh;
        float val = 0.f, gq = 1.f;
        if (tid < p.D) {
            const int64_t oi = (int64_t)b * p.H * p.D + head * p.D + tid;
            val = __bfloat162float(p.out[oi]);
            gq = __bfloat162float(p.gamma_out[head * p.D + tid]);
            p.t_out[oi] = val * gq;
        }
        publish_head_stats(p, b, val, gq, tid, sd, sf, [] { __syncthreads(); });
    }
}

template <class Params>
cudaError_t launch_chain_k(void (*kernel)(Params), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const Params& p,
                           bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

}  // namespace

void plan_chain_linear(ChainLinearParams& p, int n_sm) {
    p.k_tiles = (p.K + kTileCols - 1) / kTileCols;
    const int n_rg = (p.N + 15) / 16;
    if (p.out_kind == kOutGlu) {      // gate rows [0, N/2), up rows [N/2, N); N/2 a multiple of 16
        p.n_sub = 2;
        p.n_units = n_rg / 2;
        p.sub_stride = n_rg / 2;
    } else {
        p.n_sub = 1;
        p.n_units = n_rg;
        p.sub_stride = 0;
    }
    p.grid = p.n_units < n_sm ? p.n_units : n_sm;
    p.units_base = p.n_units / p.grid;
    p.units_rem = p.n_units % p.grid;
    p.units_max = (p.n_units + p.grid - 1) / p.grid;
    if (p.ring_stages != 2 && p.ring_stages != 4 && p.ring_stages != 8) p.ring_stages = 8;   // a power of two
    // A share that passes through the ring more than once is bound by instruction throughput, not by
    // latency: it takes the tensor-core form of the tile loop whatever M (16 logic operations and 4
    // MMAs per tile instead of 16 + 16 on the integer pipe, which issues two warp instructions per clock).
    p.big_share = p.units_max * p.n_sub * p.k_tiles > p.ring_stages * kCStageTiles;
    if (p.k_norm == 0) p.k_norm = p.K;
}

size_t chain_linear_smem(const ChainLinearParams& p) { return chain_carve(p, nullptr, nullptr) + 128; }

size_t chain_attention_smem(const AttentionParams& p) {
    const size_t short_form = sizeof(float) * (32 + 32 + 16 + 32 + (size_t)32 * p.D) + 64;
    const size_t split_form = attention_smem(p);
    return short_form > split_form ? short_form : split_form;
}

int prepare_chain_kernels(size_t smem_optin) {
    cudaError_t e = cudaFuncSetAttribute(chain_linear_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(chain_linear_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(chain_linear_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(chain_linear_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_optin);
    if (e != cudaSuccess) return check_cuda(e);
    const int attn = 96 * 1024;
    if ((e = cudaFuncSetAttribute(chain_attention_kernel<4, kAttnThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(chain_attention_kernel<8, AttnCfg<8>::kThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(chain_attention_kernel<16, AttnCfg<16>::kThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn)) != cudaSuccess)
        return check_cuda(e);
    return kOk;
}

int launch_chain_linear(const ChainLinearParams& p, cudaStream_t stream, bool pdl) {
    const bool one = p.M == 1 && !p.big_share, tp = p.tp.size > 1;
    const size_t smem = chain_linear_smem(p);
    cudaError_t e;
    if (one && !tp) e = launch_chain_k(chain_linear_kernel<true, false>, p.grid, kCLinearThreads, smem, stream, p, pdl);
    else if (!tp) e = launch_chain_k(chain_linear_kernel<false, false>, p.grid, kCLinearThreads, smem, stream, p, pdl);
    else if (one) e = launch_chain_k(chain_linear_kernel<true, true>, p.grid, kCLinearThreads, smem, stream, p, pdl);
    else e = launch_chain_k(chain_linear_kernel<false, true>, p.grid, kCLinearThreads, smem, stream, p, pdl);
    return check_cuda(e);
}

int launch_embed(const EmbedParams& p, cudaStream_t stream, bool pdl) {
    return check_cuda(launch_chain_k(embed_kernel, p.M, 256, 0, stream, p, pdl));
}

int launch_tp_reduce(const TpReduceParams& p, cudaStream_t stream, bool pdl) {
    return check_cuda(launch_chain_k(tp_reduce_kernel, (p.N + 255) / 256, 256, 0, stream, p, pdl));
}

int launch_chain_attention(const AttentionParams& p, int batch, cudaStream_t stream, bool pdl) {
    const int G = p.H / p.Hkv;
    const dim3 grid(p.Hkv * p.S, batch);
    const size_t smem = chain_attention_smem(p);
    cudaError_t e;
    if (G <= 4) e = launch_chain_k(chain_attention_kernel<4, kAttnThreads>, grid, kAttnThreads, smem, stream, p, pdl);
    else if (G <= 8) e = launch_chain_k(chain_attention_kernel<8, AttnCfg<8>::kThreads>, grid, AttnCfg<8>::kThreads, smem, stream, p, pdl);
    else e = launch_chain_k(chain_attention_kernel<16, AttnCfg<16>::kThreads>, grid, AttnCfg<16>::kThreads, smem, stream, p, pdl);
    return check_cuda(e);
}

}  // namespace bitnet
