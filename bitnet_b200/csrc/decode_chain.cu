// The BitLinear and attention kernels of the decode chain (batches of at most 8 tokens):
//
//   per layer:  wqkv -> attention -> wo -> w13 (+ gate) -> w2          then:  output head -> argmax
//
// A BitLinear at batch 1 moves 1.6-8.8 MB of packed weights: about a microsecond of HBM time,
// as much as one kernel boundary costs (0.9 us measured on B200 with programmatic dependent
// launch).  The step is therefore bound by the latency of its chain of dependent phases, and
// these kernels are built to make each phase short:
//  * every kernel lets its successor start at once (griddepcontrol.launch_dependents first);
//    the successor's CTAs bring their share of the weight matrix into shared memory with bulk
//    asynchronous copies - weights do not depend on the predecessor - and only then wait for it;
//  * a CTA owns whole 16-row groups of the weight matrix, so no partial sums cross CTAs: no
//    atomics on global memory, no scratch buffer, no tickets;
//  * the statistics that the RMSNorm + absmax quantisation in front of the NEXT BitLinear needs
//    (sum of squares, max |x * g|) are published by the kernel that produces the vector - one
//    partial per 16 outputs, computed by the threads that hold those outputs anyway - so the
//    consumer's prologue is one fetch of the vector and one pass over it, with no reduction over
//    the vector (gpu/model.py:68-71 behind the norms of :159-160, :195-196, :237-242);
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
constexpr int kCRoundStages = 2;                            // stages a round of the consumers spans
constexpr int kCWarps = 8;                                  // consumer warps
constexpr int kCThreads = kCWarps * 32;
constexpr int kCLinearThreads = kCThreads + 32;             // + one producer warp
constexpr int kCMaxStages = 8;
constexpr int kXvRows = 2;                                  // tokens whose source rows are staged together

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
struct ChainSync {
    __device__ __forceinline__ void operator()() const { chain_sync(); }
};
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

struct ChainSmem {
    uint8_t* ring;
    uint64_t *full_bar, *empty_bar;
    float *rinv_s, *a_s, *red_f;
    int *ysum_s, *flag_s, *sacc;
    double* red_d;
    __nv_bfloat16 *gs, *xv;
    int8_t* ys;
};
// Shared-memory layout (host and device use the same arithmetic).
__host__ __device__ inline size_t chain_carve(const ChainLinearParams& p, uint8_t* base, ChainSmem* s) {
    const size_t k_even = (size_t)(p.K + 7) / 8 * 8;
    const size_t k_pad = (size_t)p.k_tiles * kTileCols;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 15) / 16 * 16; return o; };
    const size_t o_ring = take((size_t)p.ring_stages * kCStageBytes);
    const size_t o_bar = take(2 * kCMaxStages * sizeof(uint64_t));
    const size_t o_misc = take(64 * sizeof(float));
    const size_t o_redd = take(8 * sizeof(double));
    const size_t o_sacc = take((size_t)p.units_max * p.n_sub * 128 * sizeof(int));
    const size_t o_gs = take(p.gamma ? k_even * 2 : 0);
    const size_t o_xv = take((size_t)(p.M < kXvRows ? p.M : kXvRows) * k_even * 2);
    const size_t o_ys = take((size_t)(p.M + 1) * (k_pad + 16));
    if (s) {
        s->ring = base + o_ring;
        s->full_bar = reinterpret_cast<uint64_t*>(base + o_bar);
        s->empty_bar = s->full_bar + kCMaxStages;
        float* misc = reinterpret_cast<float*>(base + o_misc);
        s->rinv_s = misc;
        s->a_s = misc + 8;
        s->ysum_s = reinterpret_cast<int*>(misc + 16);
        s->red_f = misc + 24;
        s->flag_s = reinterpret_cast<int*>(misc + 32);
        s->red_d = reinterpret_cast<double*>(base + o_redd);
        s->sacc = reinterpret_cast<int*>(base + o_sacc);
        s->gs = reinterpret_cast<__nv_bfloat16*>(base + o_gs);
        s->xv = reinterpret_cast<__nv_bfloat16*>(base + o_xv);
        s->ys = reinterpret_cast<int8_t*>(base + o_ys);
    }
    return off;
}

// ---------------------------------------------------------------------------------------
// BitLinear of the chain.  288 threads: 8 consumer warps and one producer warp.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kCLinearThreads, 2) chain_linear_kernel(const ChainLinearParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    ChainSmem sm;
    chain_carve(p, smem, &sm);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    CHAIN_STAMP(0)

    // this CTA's units and the tile sequence they make: for each of the n_sub row-group sets,
    // the tiles of row groups u0 .. u1-1 (+ set * sub_stride), one contiguous range of the matrix
    const int u0 = (int)((int64_t)p.n_units * cta / p.grid), u1 = (int)((int64_t)p.n_units * (cta + 1) / p.grid);
    const int nu = u1 - u0;
    const int seg_tiles = nu * p.k_tiles;                  // tiles per contiguous range
    const int n_tiles = seg_tiles * p.n_sub;
    const int n_chunks = (n_tiles + kCStageTiles - 1) / kCStageTiles;
    const int S = p.ring_stages;

    if (tid == 0) {
#pragma unroll 1
        for (int s = 0; s < S; ++s) {
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
#pragma unroll 1
            for (int c = 0; c < n_chunks; ++c) {
                const int s = c % S;
                if (c >= S && !mbar_wait(&sm.empty_bar[s], ((c / S) - 1) & 1)) {
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
                             &sm.full_bar[s]);
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
    const bool use_g = p.gamma != nullptr;
    if (use_g) {   // the norm weight is a constant: stage it before the wait
#pragma unroll 1
        for (int v = tid; v < n_vec; v += kCThreads) cp_async16(sm.gs + v * 8, p.gamma + v * 8);
    }
    // the row of zeros that MMA columns without a token read
#pragma unroll 1
    for (int v = tid; v < y_stride / 16; v += kCThreads)
        *reinterpret_cast<uint4*>(sm.ys + (size_t)p.M * y_stride + v * 16) = make_uint4(0, 0, 0, 0);
    // epilogue inputs that do not depend on the predecessor: the next norm's weight for the
    // first batch of outputs this thread finalises
    const int total_out = nu * 16 * p.M;
    const int n_out_rows = p.out_kind == kOutGlu ? p.N / 2 : p.N;
    auto out_index = [&](int idx, int& m, int& lu, int& r) {   // consecutive threads -> consecutive rows
        m = idx / (nu * 16);
        const int rem = idx - m * (nu * 16);
        lu = rem >> 4;
        r = rem & 15;
    };
    float g_pre = 1.f, h_pre = 0.f;
    {
        int m, lu, r;
        out_index(tid, m, lu, r);
        const int row = (u0 + lu) * 16 + r;
        if (tid < total_out && row < n_out_rows && p.stats_out) g_pre = __bfloat162float(p.gamma_out[row]);
    }

    CHAIN_STAMP(1)
    pdl_wait();   // the predecessor's results are visible from here on
    CHAIN_STAMP(2)
    {
        int m, lu, r;
        out_index(tid, m, lu, r);
        const int row = (u0 + lu) * 16 + r;
        if (tid < total_out && row < n_out_rows && p.out_kind == kOutResidual)
            h_pre = __bfloat162float(__ldcg(reinterpret_cast<const __nv_bfloat16*>(p.out) + (int64_t)m * p.ldo + row));
    }

    // ---- prologue: int8 activations of every token into shared memory ----------------------
#pragma unroll 1
    for (int m0 = 0; m0 < p.M; m0 += kXvRows) {
        const int nr = min(kXvRows, p.M - m0);
        // source rows: asynchronous 16-byte copies, all in flight at once
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            const __nv_bfloat16* row;
            if (p.src == kSrcEmbedding) {
                int64_t tok = p.tokens[m0 + r];
                if (tok < 0 || tok >= p.vocab) {
                    if (tid == 0) atomicExch(p.error_flag, kErrToken);
                    tok = 0;
                }
                row = p.emb + tok * (int64_t)K;
            } else {
                row = p.x + (int64_t)(m0 + r) * p.ldx;
            }
#pragma unroll 1
            for (int v = tid; v < n_vec; v += kCThreads) cp_async16(sm.xv + (size_t)r * K + v * 8, row + v * 8);
        }
        if (p.stats_in && warp < nr) {
            // warp w adds up the producer's partial statistics of token m0 + w
            const StatPart* sp = p.stats_in + (size_t)(m0 + warp) * p.n_stats_in;
            double ss = 0.0, mx = 0.0;
#pragma unroll 1
            for (int i = lane; i < p.n_stats_in; i += 32) {
                const double2 v = __ldcg(reinterpret_cast<const double2*>(sp + i));
                ss += v.x;
                mx = fmax(mx, v.y);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                ss += __shfl_xor_sync(0xffffffffu, ss, o);
                mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            }
            if (lane == 0) {
                float rinv, a;
                finish_stats(ss, (float)mx, K, p.eps, use_g, rinv, a);
                sm.rinv_s[m0 + warp] = rinv;
                sm.a_s[m0 + warp] = a;
            }
        }
        cp_async_wait_all();
        chain_sync();
        if (!p.stats_in) {
            // no producer statistics (first layer: the source is an embedding row): reduce here
#pragma unroll 1
            for (int r = 0; r < nr; ++r) {
                double ss = 0.0;
                float mt = 0.f;
#pragma unroll 1
                for (int v = tid; v < n_vec; v += kCThreads)
                    group_stats(unpack_bf16x8(*reinterpret_cast<const uint4*>(sm.xv + (size_t)r * K + v * 8)),
                                use_g ? unpack_bf16x8(*reinterpret_cast<const uint4*>(sm.gs + v * 8)) : Vec8{}, use_g, ss, mt);
                reduce_stats_256(ss, mt, sm.red_d, sm.red_f, tid, ChainSync());
                if (tid == 0) {
                    float rinv, a;
                    finish_stats(ss, mt, K, p.eps, use_g, rinv, a);
                    sm.rinv_s[m0 + r] = rinv;
                    sm.a_s[m0 + r] = a;
                }
            }
            chain_sync();
        }
        if (p.src == kSrcEmbedding && p.h_copy && cta == 0) {   // the residual stream starts as the embedding row
#pragma unroll 1
            for (int r = 0; r < nr; ++r)
#pragma unroll 1
                for (int v = tid; v < n_vec; v += kCThreads)
                    *reinterpret_cast<uint4*>(p.h_copy + (int64_t)(m0 + r) * K + v * 8) =
                        *reinterpret_cast<const uint4*>(sm.xv + (size_t)r * K + v * 8);
        }
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            const float rinv = sm.rinv_s[m0 + r], a = sm.a_s[m0 + r];
            int8_t* ym = sm.ys + (size_t)(m0 + r) * y_stride;
            int sy = 0;
#pragma unroll 1
            for (int v = tid; v < k_pad / 8; v += kCThreads) {
                uint2 w = make_uint2(0, 0);
                if (v < n_vec)
                    w = quant_group(unpack_bf16x8(*reinterpret_cast<const uint4*>(sm.xv + (size_t)r * K + v * 8)),
                                    use_g ? unpack_bf16x8(*reinterpret_cast<const uint4*>(sm.gs + v * 8)) : Vec8{}, use_g, rinv, a, sy);
                *reinterpret_cast<uint2*>(ym + v * 8) = w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sy += __shfl_xor_sync(0xffffffffu, sy, o);
            if (lane == 0) atomicAdd(&sm.ysum_s[m0 + r], sy);
        }
        chain_sync();   // ys and ysum_s complete; xv may be overwritten by the next tokens
    }
    CHAIN_STAMP(3)

    // ---- matmul over the staged tiles ----------------------------------------------------
    // Per tile a lane holds the A fragments of rows g, g+8 for four m16n8k32 MMAs: each of its
    // four words is split into its four 2-bit fields by AND masks alone (field j stays scaled by
    // 4^j and has its own accumulator).  Tokens are the MMA's 8 columns, so any M <= 8 costs the
    // same.  Two tiles are in flight per warp on separate accumulators, so that the second
    // tile's MMAs do not wait for the first one's.
    const int g = lane >> 2, q = lane & 3;
    const int8_t* y_lane = sm.ys + (size_t)(g < p.M ? g : p.M) * y_stride + 32 * q;
    constexpr int kRoundTiles = kCRoundStages * kCStageTiles;
    const int n_rounds = (n_tiles + kRoundTiles - 1) / kRoundTiles;
    int acc[2][4][4];
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[s2][j][e] = 0;
    auto flush = [&](int lg) {   // this warp's sums of local row group lg into the CTA's accumulator
        int* dst = sm.sacc + lg * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int tok = 2 * q + (i & 1);
            const int v = acc[0][0][i] + acc[1][0][i] + ((acc[0][1][i] + acc[1][1][i]) >> 2) + ((acc[0][2][i] + acc[1][2][i]) >> 4) +
                          ((acc[0][3][i] + acc[1][3][i]) >> 6);
            if (tok < p.M) atomicAdd(&dst[(g + 8 * (i >> 1)) * 8 + tok], v);
        }
#pragma unroll
        for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[s2][j][e] = 0;
    };
    auto tile_mma = [&](int (&a4)[4][4], const uint4& wc, const uint4& y0, const uint4& y1) {
        const uint32_t b[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
        const uint32_t w[4] = {wc.x, wc.y, wc.z, wc.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t msk = 0x03030303u << (2 * j);
            mma_u8s8(a4[j], w[0] & msk, w[1] & msk, w[2] & msk, w[3] & msk, b[2 * j], b[2 * j + 1]);
        }
    };
    bool gave_up = false;
#pragma unroll 1
    for (int r = 0; r < n_rounds && !gave_up; ++r) {
        const int nr_t = min(kRoundTiles, n_tiles - r * kRoundTiles);
        const int lo = nr_t * warp / kCWarps, hi = nr_t * (warp + 1) / kCWarps;
        if (hi > lo) {
            bool ok = true;
#pragma unroll 1
            for (int ls = lo / kCStageTiles; ls <= (hi - 1) / kCStageTiles; ++ls) {
                const int c = r * kCRoundStages + ls;        // chunk number of the CTA's tile sequence
                ok = ok && mbar_wait(&sm.full_bar[c % S], (c / S) & 1);
            }
            if (!ok) {   // gave up: flag it, leave together below
                if (lane == 0) {
                    atomicExch(p.error_flag, kErrConsumerWait);
                    sm.flag_s[0] = 1;
                }
                gave_up = true;
            }
        }
        if (!gave_up && hi > lo) {
            int t = r * kRoundTiles + lo;                    // local tile number
            const int t_end = r * kRoundTiles + hi;
            int lg = t / p.k_tiles, kt = t - lg * p.k_tiles;
            // the ring slot of a tile: chunk c = t / 32 sits in stage c % S
            auto tile_ptr = [&](int tt) -> const uint8_t* {
                const int c = tt / kCStageTiles;
                return sm.ring + (c % S) * kCStageBytes + (tt - c * kCStageTiles) * kTileBytes + lane * 16;
            };
#pragma unroll 1
            while (t < t_end) {
                const int n_here = min(t_end - t, p.k_tiles - kt);   // tiles of this row group in the run
                int j = 0;
#pragma unroll 1
                for (; j + 2 <= n_here; j += 2) {
                    const uint4 w0 = *reinterpret_cast<const uint4*>(tile_ptr(t + j));
                    const uint4 w1 = *reinterpret_cast<const uint4*>(tile_ptr(t + j + 1));
                    const uint4* yp0 = reinterpret_cast<const uint4*>(y_lane + (kt + j) * kTileCols);
                    const uint4* yp1 = reinterpret_cast<const uint4*>(y_lane + (kt + j + 1) * kTileCols);
                    const uint4 y00 = yp0[0], y01 = yp0[1], y10 = yp1[0], y11 = yp1[1];
                    tile_mma(acc[0], w0, y00, y01);
                    tile_mma(acc[1], w1, y10, y11);
                }
                if (j < n_here) {
                    const uint4 w0 = *reinterpret_cast<const uint4*>(tile_ptr(t + j));
                    const uint4* yp0 = reinterpret_cast<const uint4*>(y_lane + (kt + j) * kTileCols);
                    const uint4 y00 = yp0[0], y01 = yp0[1];
                    tile_mma(acc[0], w0, y00, y01);
                }
                flush(lg);
                t += n_here;
                kt += n_here;
                if (kt == p.k_tiles) {
                    kt = 0;
                    ++lg;
                }
            }
        }
        __syncwarp();
        if (lane == 0 && !gave_up) {
            // This warp is done with every stage of the round.  It releases a stage only after
            // having seen that stage's copy complete (usually it has, long ago), so that no warp
            // ever waits for a later fill of a stage whose earlier fill it has not observed.
#pragma unroll 1
            for (int ls = 0; ls < kCRoundStages; ++ls) {
                const int c = r * kCRoundStages + ls;
                if (c < n_chunks && mbar_wait(&sm.full_bar[c % S], (c / S) & 1)) mbar_arrive(&sm.empty_bar[c % S]);
            }
        }
    }
    CHAIN_STAMP(4)
    chain_sync();
    if (sm.flag_s[0] || n_tiles == 0) return;

    // ---- epilogue --------------------------------------------------------------------------
    // Thread idx finalises output r of unit lu for token m; 16 consecutive threads hold the 16
    // outputs of one unit and token, and reduce their statistics by shuffles.
#pragma unroll 1
    for (int base = 0; base < total_out; base += kCThreads) {
        const int idx = base + tid;
        const bool valid = idx < total_out;
        int m = 0, lu = 0, r = 0;
        if (valid) out_index(idx, m, lu, r);
        const int row = (u0 + lu) * 16 + r;                 // output index (glu: index of the gated value)
        const bool live = valid && row < n_out_rows;
        float o = 0.f, gq = 1.f;
        if (live) {
            const float a = sm.a_s[m];
            const int ys_m = sm.ysum_s[m];                  // fields hold weight + 1: take sum(y) off once per row
            const int v0 = sm.sacc[lu * 128 + r * 8 + m] - ys_m;
            if (p.out_kind == kOutGlu) {
                const int v1 = sm.sacc[(nu + lu) * 128 + r * 8 + m] - ys_m;
                const int row_up = row + p.sub_stride * 16;
                const float x1 = lin_out(v0, a, p.ws[segment_of(p.seg, row)]);
                const float x3 = lin_out(v1, a, p.ws[segment_of(p.seg, row_up)]);
                const float t = fmaxf(x1, 0.f);
                o = bf16_round(bf16_round(t * t) * x3);     // rounded after each step, as bf16 tensor operations round
            } else {
                const float lin = lin_out(v0, a, p.ws[segment_of(p.seg, row)]);
                if (p.out_kind == kOutResidual) {
                    const float h_old = base == 0 ? h_pre : __bfloat162float(__ldcg(reinterpret_cast<const __nv_bfloat16*>(p.out) + (int64_t)m * p.ldo + row));
                    o = bf16_round(h_old + lin);
                } else {
                    o = lin;
                }
            }
            p.out[(int64_t)m * p.ldo + row] = __float2bfloat16_rn(o);
            if (p.stats_out) gq = base == 0 ? g_pre : __bfloat162float(p.gamma_out[row]);
        }
        if (p.stats_out) {
            double ss = (double)o * (double)o;
            float mx = fabsf(o * gq);
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) {
                ss += __shfl_xor_sync(0xffffffffu, ss, off);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            }
            if (valid && (lane & 15) == 0) {
                StatPart sp;
                sp.ss = ss;
                sp.mx = (double)mx;
                p.stats_out[(size_t)m * p.n_units + u0 + lu] = sp;
            }
        }
    }
    CHAIN_STAMP(5)
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
// dimension d (others hold 0).  `sd`/`sf` hold 16 entries; every thread of the CTA must call.
template <class Sync>
__device__ __forceinline__ void publish_head_stats(const AttentionParams& p, int b, int head, float val, float gq, int tid,
                                                   double* sd, float* sf, Sync sync) {
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
        StatPart sp;
        sp.ss = sd[0] + sd[1] + sd[2] + sd[3];      // D <= 128: the values sit in the first four warps
        sp.mx = (double)fmaxf(fmaxf(sf[0], sf[1]), fmaxf(sf[2], sf[3]));
        p.stats_out[(size_t)b * p.H + head] = sp;
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
    float* red_m = reinterpret_cast<float*>(smem);      // [32]
    float* red_l = red_m + 32;                          // [32]
    float* sf = red_l + 32;                             // [16]
    double* sd = reinterpret_cast<double*>(sf + 16);    // [16]
    float* red_o = reinterpret_cast<float*>(sd + 16);   // [32][D]
    const int64_t key_stride = (int64_t)p.Hkv * D;
    const __nv_bfloat16* ck = p.cache_k + ((int64_t)b * p.L * p.Hkv + kvh) * D + d0;
    const __nv_bfloat16* cv = p.cache_v + ((int64_t)b * p.L * p.Hkv + kvh) * D + d0;
    const int P = (int)__ldcg(p.pos + b);
    uint4 kr[kKeyRounds], vr[kKeyRounds];
    auto load_block = [&](int j0, int j_end) {   // cache rows j0 + 32 r + hw, r < 8, below j_end
#pragma unroll
        for (int r = 0; r < kKeyRounds; ++r) {
            const int j = j0 + r * 32 + hw;
            kr[r] = make_uint4(0, 0, 0, 0);
            vr[r] = make_uint4(0, 0, 0, 0);
            if (j < j_end && live) {
                kr[r] = __ldcg(reinterpret_cast<const uint4*>(ck + j * key_stride));   // L2: rows appended by earlier steps
                vr[r] = __ldcg(reinterpret_cast<const uint4*>(cv + j * key_stride));
            }
        }
    };
    load_block(0, p.L);       // requested before P is known; rows >= P are masked below
    const __nv_bfloat16* x = p.xqkv + (int64_t)b * p.ld_qkv;
    uint4 q_raw = make_uint4(0, 0, 0, 0);
    if (live) q_raw = __ldcg(reinterpret_cast<const uint4*>(x + h * D + d0));   // L2: written by other SMs
    if (P < 0 || P >= p.L) {      // outside the cache: flag it, touch nothing
        if (tid == 0) atomicExch(p.error_flag, kErrPosition);
        return true;
    }
    if (attention_slices(p.S, P) != 1) return false;
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
    uint4 k_new = make_uint4(0, 0, 0, 0), v_new = make_uint4(0, 0, 0, 0);
    if (own_new && live) {
        const uint4 kraw = __ldcg(reinterpret_cast<const uint4*>(x + (p.H + kvh) * D + d0));
        v_new = __ldcg(reinterpret_cast<const uint4*>(x + (p.H + p.Hkv + kvh) * D + d0));
        float kf[8];
        rotate(kraw, kf);
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
    // combine the 32 half-warps
    if (l16 == 0) {
        red_m[hw] = m_run;
        red_l[hw] = l_run;
    }
    if (live) {
        *reinterpret_cast<float4*>(red_o + hw * D + d0) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4*>(red_o + hw * D + d0 + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
    __syncthreads();
    float val = 0.f, gq = 1.f;
    if (tid < D) {
        float mx = -INFINITY;
#pragma unroll 1
        for (int w = 0; w < 32; ++w) mx = fmaxf(mx, red_m[w]);
        float l = 0.f, acc = 0.f;
#pragma unroll 1
        for (int w = 0; w < 32; ++w) {
            const float lw = red_l[w];
            if (lw > 0.f) {
                const float f = __expf(red_m[w] - mx);
                l = fmaf(lw, f, l);
                acc = fmaf(red_o[w * D + tid], f, acc);
            }
        }
        const __nv_bfloat16 ob = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        const int64_t oi = (int64_t)b * p.H * D + h * D + tid;
        p.out[oi] = ob;
        if (p.tap) p.tap[oi] = ob;
        val = __bfloat162float(ob);
        if (p.stats_out) gq = __bfloat162float(p.gamma_out[h * D + tid]);
    }
    if (p.stats_out) publish_head_stats(p, b, h, val, gq, tid, sd, sf, [] { __syncthreads(); });
    return true;
}

// NTHREADS = 512 (grouped-query ratios up to 4: short form and split-KV body share the CTA) or
// the split-KV body's own thread count (larger ratios: its register budget rules out 512
// threads, and the short form is left out).
template <int GMAX, int NTHREADS>
__global__ void __launch_bounds__(NTHREADS) chain_attention_kernel(const AttentionParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int is_last;
    static_assert(AttnCfg<GMAX>::kThreads <= NTHREADS, "the split-KV body uses a prefix of the CTA's warps");
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y, tid = threadIdx.x;
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
    if (tid < NT) {
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
            val = __bfloat162float(p.out[(int64_t)b * p.H * p.D + head * p.D + tid]);
            gq = __bfloat162float(p.gamma_out[head * p.D + tid]);
        }
        publish_head_stats(p, b, head, val, gq, tid, sd, sf, [] { __syncthreads(); });
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
    p.units_max = (p.n_units + p.grid - 1) / p.grid;
    if (p.ring_stages < 2 || p.ring_stages > kCMaxStages) p.ring_stages = 4;
    p.ring_stages = p.ring_stages / kCRoundStages * kCRoundStages;
}

size_t chain_linear_smem(const ChainLinearParams& p) { return chain_carve(p, nullptr, nullptr) + 128; }

size_t chain_attention_smem(const AttentionParams& p) {
    const size_t short_form = sizeof(float) * (32 + 32 + 16 + 32 + (size_t)32 * p.D) + 64;
    const size_t split_form = attention_smem(p);
    return short_form > split_form ? short_form : split_form;
}

int prepare_chain_kernels(size_t smem_optin) {
    cudaError_t e = cudaFuncSetAttribute(chain_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_optin);
    if (e != cudaSuccess) return check_cuda(e);
    const int attn = 96 * 1024;
    if ((e = cudaFuncSetAttribute(chain_attention_kernel<4, kAttnThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(chain_attention_kernel<8, AttnCfg<8>::kThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(chain_attention_kernel<16, AttnCfg<16>::kThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn)) != cudaSuccess)
        return check_cuda(e);
    return kOk;
}

int launch_chain_linear(const ChainLinearParams& p, cudaStream_t stream, bool pdl) {
    return check_cuda(launch_chain_k(chain_linear_kernel, p.grid, kCLinearThreads, chain_linear_smem(p), stream, p, pdl));
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
