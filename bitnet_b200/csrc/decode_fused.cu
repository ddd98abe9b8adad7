// The stand-alone fused BitLinear for batches of at most 8 tokens on caller-quantised
// activations, the decode attention of the op-by-op path, the output head and the greedy
// choice.  (The BitLinear and attention kernels of the decode chain live in decode_chain.cu.)
//
// fused_linear_kernel: the matrix is a flat sequence of 16x128 tiles (row-group major); CTA c
// of G takes a contiguous range of total/G tiles, so the load is even for every shape.  A
// producer warp streams the range through a ring of 16 KB stages with cp.async.bulk; eight
// consumer warps unpack with masks only and multiply with mma.sync m16n8k32 (u8 x s8).
// Ranges cut through row groups, so a CTA that holds only part of a row group's K range adds
// its int32 sums and a ticket to a 64-bit scratch slot in one atomic; the contributor that
// completes the count rescales the finished sums to bf16, then clears the slot.  Nobody waits.
#include <cuda.h>
#include <stdlib.h>

#include <mutex>

#include "../../include/bitnet_b200.h"
#include "common.cuh"
#include "decode_fused.h"
#include "prologue.cuh"
#include "decode_device.cuh"

namespace bitnet {

namespace {

// Ring of 6 x 16 KB.  Its size also keeps two of these CTAs from sharing an SM: the CTAs of the
// next kernel of the chain, launched early, then start when a CTA of the running kernel leaves
// instead of competing with it (measured on the 2B decode step: 1.48 ms with a 64 KB ring, 1.39
// with the same ring and 32 KB of unused shared memory, 1.36 with this one).
constexpr int kStages = 6;
constexpr int kRoundStages = 2;                           // stages a round of the consumers spans
constexpr int kStageTiles = 32;
constexpr int kStageBytes = kStageTiles * kTileBytes;     // 16 KB
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kLinearThreads = kConsumerThreads + 32;     // + one producer warp

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumerThreads) : "memory"); }

struct ConsumerSync {
    __device__ __forceinline__ void operator()() const { consumer_sync(); }
};
// CTA that owns tile t under the even split (tiles_base + 1 tiles for the first tiles_rem CTAs).
__device__ __forceinline__ int cta_of_tile(const FusedLinearParams& p, int t) {
    const int big = p.tiles_rem * (p.tiles_base + 1);
    return t < big ? t / (p.tiles_base + 1) : p.tiles_rem + (t - big) / p.tiles_base;
}

// ---------------------------------------------------------------------------------------
// Fused BitLinear.  One kernel for all source kinds and token counts, with rolled loops:
// the kernels of the chain run for a few microseconds each, so their code has to stay
// resident in the instruction cache from launch to launch.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

__global__ void __launch_bounds__(kLinearThreads, 2) fused_linear_kernel(const FusedLinearParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* empty_bar = full_bar + kStages;
    int* sy_part = reinterpret_cast<int*>(empty_bar + kStages);                // [8 tokens][8 warps]
    int* ysum_s = sy_part + 64;                                                // 8 ints
    float* a_s = reinterpret_cast<float*>(ysum_s + 8);                         // 8 floats
    int* flag_s = reinterpret_cast<int*>(a_s + 8);                             // 8 ints (1 used)
    int* sacc = flag_s + 8;                                                    // [r_max][16][8]
    const int k_pad = p.k_tiles * kTileCols;
    const int y_stride = k_pad + 16;
    int8_t* ys = reinterpret_cast<int8_t*>(sacc + p.r_max * 128);              // [M + 1][y_stride]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;

    const int t0 = cta * p.tiles_base + min(cta, p.tiles_rem);
    const int n_tiles = p.tiles_base + (cta < p.tiles_rem ? 1 : 0);
    const int n_chunks = (n_tiles + kStageTiles - 1) / kStageTiles;

    if (tid == 0) {
#pragma unroll 1
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kConsumerWarps);
        }
        flag_s[0] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kConsumerWarps) {
        // ---- producer: streams the weight tiles; independent of the predecessor kernel ----
        if (lane == 0) {
            const uint8_t* src = p.w2t + (int64_t)t0 * kTileBytes;
#pragma unroll 1
            for (int c = 0; c < n_chunks; ++c) {
                const int s = c % kStages;
                if (c >= kStages && !mbar_wait(&empty_bar[s], ((c / kStages) - 1) & 1)) {
                    atomicExch(p.error_flag, kErrProducerWait);
                    break;
                }
                const int tiles = min(kStageTiles, n_tiles - c * kStageTiles);
                mbar_expect_tx(&full_bar[s], tiles * kTileBytes);
                bulk_g2s(ring + s * kStageBytes, src + (int64_t)c * kStageBytes, tiles * kTileBytes, &full_bar[s]);
            }
        }
        return;
    }

    // ---- consumers ---------------------------------------------------------------------
#pragma unroll 1
    for (int i = tid; i < p.r_max * 128; i += kConsumerThreads) sacc[i] = 0;
    pdl_wait();   // the predecessor's results are visible from here on

    // the int8 activations of every token, in shared memory (plus one row of zeros)
#pragma unroll 1
    for (int v = tid; v < y_stride / 16; v += kConsumerThreads)
        *reinterpret_cast<uint4*>(ys + (size_t)p.M * y_stride + v * 16) = make_uint4(0, 0, 0, 0);
#pragma unroll 1
    for (int m = 0; m < p.M; ++m) {
        int8_t* ym = ys + (size_t)m * y_stride;
        const int8_t* row = p.yq + (int64_t)m * p.ldy;
        const bool vec_ok = aligned16(p.yq, p.ldy, 1);
        int sy = 0;
#pragma unroll 1
        for (int v = tid; v < k_pad / 16; v += kConsumerThreads) {
            uint4 u = make_uint4(0, 0, 0, 0);
            const int k = v * 16;
            if (vec_ok && k + 16 <= p.K) {
                u = *reinterpret_cast<const uint4*>(row + k);
            } else {
                uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll 1
                for (int e = 0; e < 16; ++e)
                    if (k + e < p.K) w[e >> 2] |= (uint32_t)(uint8_t)row[k + e] << (8 * (e & 3));
                u = make_uint4(w[0], w[1], w[2], w[3]);
            }
            *reinterpret_cast<uint4*>(ym + k) = u;
            sy += __dp4a((int)u.x, 0x01010101, 0) + __dp4a((int)u.y, 0x01010101, 0) + __dp4a((int)u.z, 0x01010101, 0) +
                  __dp4a((int)u.w, 0x01010101, 0);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sy += __shfl_xor_sync(0xffffffffu, sy, o);
        const int sy_warp = p.ysum_q ? (warp == 0 ? p.ysum_q[m] : 0) : sy;
        const float a = p.a_q ? p.a_q[m] : (p.a_q_bf16 ? __bfloat162float(p.a_q_bf16[m]) : 1.f);
        if (lane == 0) sy_part[m * 8 + warp] = sy_warp;
        if (tid == 0) a_s[m] = a;
        consumer_sync();   // xv is reused by the next token; ys, sy_part, a_s are complete
    }
    if (tid < p.M) {       // sum(y) per token
        int t = 0;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) t += sy_part[tid * 8 + w];
        ysum_s[tid] = t;
    }
    consumer_sync();
    // ---- matmul over the staged tiles ----------------------------------------------------
    // Per tile a lane holds the A fragments of rows g, g+8 for four m16n8k32 MMAs: each of its
    // four words is split into its four 2-bit fields by AND masks alone (field j stays scaled
    // by 4^j and has its own accumulator).  Tokens are the MMA's 8 columns, so any M <= 8
    // costs the same.  Measured on B200: 0.52 such MMAs per clock per SM against 2 integer
    // warp-instructions per clock, so the 16 ANDs per tile, not the MMAs, bound the loop.
    const int g = lane >> 2, q = lane & 3;
    const int rg_first = t0 / p.k_tiles;
    // A round spans two of the ring's six stages: while the warps work on one round, the copies
    // of the next two rounds are in flight (64 KB per SM, what the HBM latency asks for).
    constexpr int kRoundTiles = kRoundStages * kStageTiles;
    int cur_rg = -1;
    int acc[4][4];
    auto flush = [&]() {
        if (cur_rg >= 0) {
            int* dst = sacc + (cur_rg - rg_first) * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = 2 * q + (i & 1);
                if (tok < p.M) {
                    const int v = acc[0][i] + (acc[1][i] >> 2) + (acc[2][i] >> 4) + (acc[3][i] >> 6);
                    atomicAdd(&dst[(g + 8 * (i >> 1)) * 8 + tok], v);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][e] = 0;
    };
    flush();
    // MMA column g multiplies token g; columns beyond M read the zero row behind the last token
    const int8_t* y_lane = ys + (size_t)(g < p.M ? g : p.M) * y_stride + 32 * q;
    const int ysub0 = (2 * q < p.M) ? ysum_s[2 * q] : 0, ysub1 = (2 * q + 1 < p.M) ? ysum_s[2 * q + 1] : 0;
    // Within a round (up to 64 tiles) each warp takes one contiguous run, so that it flushes
    // rarely and its loop reaches a steady state.
    const int n_rounds = (n_tiles + kRoundTiles - 1) / kRoundTiles;
#pragma unroll 1
    for (int r = 0; r < n_rounds; ++r) {
        const int nr = min(kRoundTiles, n_tiles - r * kRoundTiles);
        const int lo = nr * warp / kConsumerWarps, hi = nr * (warp + 1) / kConsumerWarps;
        if (hi > lo) {
            bool ok = true;
#pragma unroll 1
            for (int ls = lo / kStageTiles; ls <= (hi - 1) / kStageTiles; ++ls) {
                const int c = r * kRoundStages + ls;     // chunk number of the CTA's tile range
                ok = ok && mbar_wait(&full_bar[c % kStages], (c / kStages) & 1);
            }
            if (!ok) {   // gave up: flag it, leave together below
                if (lane == 0) {
                    atomicExch(p.error_flag, kErrConsumerWait);
                    flag_s[0] = 1;
                }
                break;
            }
        }
        const int t_first = t0 + r * kRoundTiles + lo;
        int rg = t_first / p.k_tiles, kt = t_first - rg * p.k_tiles;
        const uint8_t* tile = ring + ((r * kRoundStages) % kStages) * kStageBytes + lo * kTileBytes + lane * 16;
#pragma unroll 1
        for (int i = lo; i < hi; ++i, tile += kTileBytes) {
            if (rg != cur_rg) {
                flush();
                cur_rg = rg;
            }
            const uint4 wc = *reinterpret_cast<const uint4*>(tile);
            const uint4* yp = reinterpret_cast<const uint4*>(y_lane + kt * kTileCols);
            const uint4 y0 = yp[0], y1 = yp[1];
            const uint32_t b[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
            const uint32_t w[4] = {wc.x, wc.y, wc.z, wc.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t msk = 0x03030303u << (2 * j);
                mma_u8s8(acc[j], w[0] & msk, w[1] & msk, w[2] & msk, w[3] & msk, b[2 * j], b[2 * j + 1]);
            }
            if (kt == 0) {   // fields hold weight + 1: take sum(y) off once per row
                acc[0][0] -= ysub0; acc[0][1] -= ysub1; acc[0][2] -= ysub0; acc[0][3] -= ysub1;
            }
            if (++kt == p.k_tiles) {
                kt = 0;
                ++rg;
            }
        }
        __syncwarp();
        if (lane == 0) {   // this warp is done with every stage of the round
#pragma unroll 1
            for (int ls = 0; ls < kRoundStages; ++ls) mbar_arrive(&empty_bar[(r * kRoundStages + ls) % kStages]);
        }
    }
    flush();
    consumer_sync();
    if (flag_s[0] || n_tiles == 0) return;

    // ---- epilogue --------------------------------------------------------------------------
    const int n_rg = (t0 + n_tiles - 1) / p.k_tiles - rg_first + 1;
    const int rg_last = rg_first + n_rg - 1;
    // only the first and the last row group of the range can be partial
    const bool part_first = t0 > rg_first * p.k_tiles || (t0 + n_tiles) < (rg_first + 1) * p.k_tiles;
    const bool part_last = n_rg > 1 && (t0 + n_tiles) < (rg_last + 1) * p.k_tiles;
#pragma unroll 1
    for (int idx = tid; idx < n_rg * 16 * p.M; idx += kConsumerThreads) {
        const int m = idx / (n_rg * 16), rem = idx - m * (n_rg * 16);      // consecutive threads -> consecutive rows
        const int li = rem >> 4, r = rem & 15;
        const int rgi = rg_first + li, row = rgi * 16 + r;
        const bool partial = (li == 0 && part_first) || (li == n_rg - 1 && li > 0 && part_last);
        if (row >= p.N && !partial) continue;
        int v = sacc[rem * 8 + m];
        if (partial) {
            // Row group shared with other CTAs: add this CTA's sum and a ticket to the 64-bit
            // slot in one atomic (sum in the low 40 bits, tickets above).  The contributor
            // whose atomic completes the ticket count sees the finished sum in the returned
            // value, finalises the element and clears the slot.  Nobody waits.
            const int lo_t = rgi * p.k_tiles, hi_t = lo_t + p.k_tiles - 1;
            const long long expected = cta_of_tile(p, hi_t) - cta_of_tile(p, lo_t) + 1;
            unsigned long long* slot = &p.acc_scratch[(int64_t)rgi * 128 + r * 8 + m];
            const unsigned long long add = (unsigned long long)((long long)v + (1LL << 40));
            const long long tot = (long long)(atomicAdd(slot, add) + add);
            const long long cnt = (tot + (1LL << 39)) >> 40;
            if (cnt != expected) continue;
            v = (int)(tot - (cnt << 40));
            *slot = 0ull;
        }
        if (row >= p.N) continue;
        if (p.acc_out) p.acc_out[(int64_t)m * p.N + row] = v;
        if (p.out) {
            const int sg = segment_of(p.seg, row);
            const float ws = p.ws_dev_f32 ? p.ws_dev_f32[sg] : (p.ws_dev_bf16 ? __bfloat162float(p.ws_dev_bf16[sg]) : 1.f);
            p.out[(int64_t)m * p.ldo + row] = __float2bfloat16_rn(lin_out(v, a_s[m], ws));
        }
    }
}

// ---------------------------------------------------------------------------------------
// Attention for one new token per sequence: RoPE on q and k, append k, v to the cache,
// softmax(q k^T) v over one slice of the cache per CTA (flash-decoding split); the CTA that
// finishes a (sequence, kv head) last combines the slices.  grid (n_kv_heads * S, batch),
// 4 to 16 warps; a warp walks keys four at a time, a lane owns 4 dims.  With many sequences
// (at least two CTAs per SM without any split) the 4-warp form runs: several CTAs share an SM
// and hide each other's latencies, where one wide CTA per SM would run wave after wave.
// ---------------------------------------------------------------------------------------
template <int GMAX, int NW = AttnCfg<GMAX>::kWarps>
__global__ void __launch_bounds__(NW * 32) attention_decode_kernel(const AttentionParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int is_last;
    pdl_launch_dependents();
    pdl_wait();
    const int P = (int)p.pos[blockIdx.y];
    if (P < 0 || P >= p.L) {      // outside the cache: flag it, touch nothing
        if (threadIdx.x == 0 && blockIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, kErrPosition);
        return;
    }
    const AttnItem it = attention_item(p, blockIdx.x, P);
    if (it.G == 0) return;
    if (it.G == 1)
        attention_body<1, NW>(p, smem, &is_last, blockIdx.y, it.kvh, it.h0, 1, it.split, it.S, P, threadIdx.x,
                              [] { __syncthreads(); }, [] {});
    else
        attention_body<GMAX, NW>(p, smem, &is_last, blockIdx.y, it.kvh, it.h0, it.G, it.split, it.S, P, threadIdx.x,
                                 [] { __syncthreads(); }, [] {});
}

// The same for whole groups of 2 to 16 query heads at head_dim 128, with the key loop on tensor
// cores (attention_keys_mma / attention_keys_mma8): four warps, 16 keys per warp and step.  Groups
// of up to 8 heads take the 8-row loop with all loads of a step in flight, three CTAs to an SM (with
// hundreds of (sequence, kv head) pairs the number of CTAs in flight sets the pace).
template <int ROWS>
__global__ void __launch_bounds__(128, ROWS == 8 ? 3 : 1) attention_decode_mma_kernel(const AttentionParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int is_last;
    pdl_launch_dependents();
    pdl_wait();
    const int P = (int)p.pos[blockIdx.y];
    if (P < 0 || P >= p.L) {      // outside the cache: flag it, touch nothing
        if (threadIdx.x == 0 && blockIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, kErrPosition);
        return;
    }
    const AttnItem it = attention_item(p, blockIdx.x, P);
    if (it.G == 0) return;
    attention_body<ROWS, 4, true, true>(p, smem, &is_last, blockIdx.y, it.kvh, it.h0, it.G, it.split, it.S, P, threadIdx.x,
                                  [] { __syncthreads(); }, [] {});
}

// ---------------------------------------------------------------------------------------
// Output head: final RMSNorm, then logits = x . E^T over this CTA's slice of the vocabulary
// (bf16 weights, f32 accumulation, bf16-rounded result as gpu/model.py:280-281) and the
// slice's argmax.  One warp per vocabulary row, all loads of a row in flight.
// ---------------------------------------------------------------------------------------
template <bool kCompact, bool kOne>
__global__ void __launch_bounds__(kHeadThreads, 1) output_head_kernel(const HeadParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    pdl_wait();
    head_body<kCompact, false, kOne>(p, smem, blockIdx.x, gridDim.x, threadIdx.x, [] { __syncthreads(); });
}

// The same with the projection's rows brought into shared memory by bulk copies: every warp owns
// two row slots, requests its first two rows before the dependency wait (weights are constants) and
// refills a slot as soon as it has used it up.  Bulk copies keep two rows per warp in flight with a
// handful of instructions, which 512 threads issuing 16-byte loads do not.  For hidden sizes whose
// 32 row slots fit shared memory beside the activations.
template <bool kCompact, bool kOne>
__global__ void __launch_bounds__(kHeadThreads, 1) output_head_ring_kernel(const HeadParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const size_t x_bytes = (kCompact ? 2 : 4) * (size_t)p.M * p.K + sizeof(float) * (32 + 16 * 8 * 2) + 64;
    const size_t ring_off = (x_bytes + 127) / 128 * 128;
    const size_t row_bytes = (size_t)p.K * sizeof(__nv_bfloat16);
    uint8_t* ring = smem + ring_off;
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + 2 * kHeadRingRows * row_bytes);     // [warp][2]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (lane == 0) {
        mbar_init(&bars[2 * warp], 1);
        mbar_init(&bars[2 * warp + 1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        const int cta = blockIdx.x, n_cta = gridDim.x;
        const int r0 = (int)((int64_t)p.V * cta / n_cta), r1 = (int)((int64_t)p.V * (cta + 1) / n_cta);
        const uint64_t policy = l2_evict_first_policy();
        for (int k = 0; k < 2; ++k) {
            const int row = r0 + warp + k * (kHeadThreads / 32);
            if (row < r1) head_request_row(p, row, ring + ((size_t)warp * 2 + k) * row_bytes, &bars[2 * warp + k], policy);
        }
    }
    __syncwarp();
    pdl_launch_dependents();
    pdl_wait();
    head_body<kCompact, true, kOne>(p, smem, blockIdx.x, gridDim.x, tid, [] { __syncthreads(); }, ring, bars);
}

// Greedy choice over the per-CTA maxima; writes the chosen ids, feeds them back as the next
// input and advances the positions.
__global__ void __launch_bounds__(256) argmax_kernel(const ArgmaxParams p) {
    __shared__ float sv[256];
    __shared__ int si[256];
    pdl_launch_dependents();
    pdl_wait();
    const bool packets = p.tag.step != nullptr;     // tensor parallel: the maxima of all ranks' vocabulary slices
    const unsigned int tag = packets ? tp_tag(p.tag) : 0u;
    long long limit = (packets && __ldcg(p.error_flag) == 0) ? p.tag.limit_cycles : 0;
    for (int m = 0; m < p.M; ++m) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int c = threadIdx.x; c < p.n_part; c += 256) {
            float cv;
            int ci;
            if (packets) {
                unsigned int vb, ib;
                const bool ok = tp_get(reinterpret_cast<const uint2*>(p.part_val) + c * 8 + m, tag, limit, vb) &&
                                tp_get(reinterpret_cast<const uint2*>(p.part_idx) + c * 8 + m, tag, limit, ib);
                if (!ok) {
                    atomicExch(p.error_flag, kErrPeerWait);
                    limit = 0;
                }
                cv = __uint_as_float(vb);
                ci = (int)ib;
            } else {
                cv = __ldcg(&p.part_val[c * 8 + m]);
                ci = __ldcg(&p.part_idx[c * 8 + m]);
            }
            if (cv > v || (cv == v && ci < i)) { v = cv; i = ci; }
        }
        sv[threadIdx.x] = v; si[threadIdx.x] = i;
        __syncthreads();
        for (int s = 128; s > 0; s >>= 1) {
            if (threadIdx.x < s) {
                const float ov = sv[threadIdx.x + s];
                const int oi = si[threadIdx.x + s];
                if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) {
                    sv[threadIdx.x] = ov; si[threadIdx.x] = oi;
                }
            }
            __syncthreads();
        }
        if (threadIdx.x == 0) {
            p.out[m] = si[0];
            p.tokens[m] = si[0];
            p.pos[m] += 1;
        }
        __syncthreads();
    }
    if (p.step && threadIdx.x == 0) *p.step += 1;
}

// ---------------------------------------------------------------------------------------
// launch helpers
// ---------------------------------------------------------------------------------------
template <class Params>
cudaError_t launch_k(void (*kernel)(Params), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const Params& p,
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

void plan_linear(FusedLinearParams& p, int n_sm) {
    p.k_tiles = (p.K + kTileCols - 1) / kTileCols;
    p.K_even = (p.K + 7) / 8 * 8;
    p.total_tiles = ((p.N + 15) / 16) * p.k_tiles;
    p.grid = p.total_tiles < n_sm ? p.total_tiles : n_sm;
    p.tiles_base = p.total_tiles / p.grid;
    p.tiles_rem = p.total_tiles % p.grid;
    p.r_max = (p.tiles_base + 1 + p.k_tiles - 1) / p.k_tiles + 1;
}

size_t fused_linear_smem(const FusedLinearParams& p) {
    const size_t y_stride = (size_t)p.k_tiles * kTileCols + 16;
    return (size_t)kStages * kStageBytes + 2 * kStages * sizeof(uint64_t) + (64 + 8 * 3) * 4 + (size_t)p.r_max * 128 * 4 +
           (size_t)(p.M + 1) * y_stride + 128;
}

int prepare_fused_kernels(size_t max_linear_smem, size_t max_attn_smem, size_t max_head_smem) {
    cudaError_t e;
#define SET_SMEM(k, n)                                                                              \
    if ((n) > 0) {                                                                                  \
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(n));         \
        if (e != cudaSuccess) return check_cuda(e);                                                 \
    }
    SET_SMEM(fused_linear_kernel, max_linear_smem)
    SET_SMEM(attention_decode_kernel<4>, max_attn_smem)
    SET_SMEM(attention_decode_kernel<8>, max_attn_smem)
    SET_SMEM(attention_decode_kernel<16>, max_attn_smem)
    SET_SMEM(attention_decode_mma_kernel<8>, max_attn_smem)
    SET_SMEM(attention_decode_mma_kernel<16>, max_attn_smem)
    SET_SMEM((output_head_kernel<false, false>), max_head_smem)
    SET_SMEM((output_head_kernel<true, false>), max_head_smem)
    SET_SMEM((output_head_kernel<false, true>), max_head_smem)
    SET_SMEM((output_head_kernel<true, true>), max_head_smem)
    SET_SMEM((output_head_ring_kernel<false, false>), max_head_smem)
    SET_SMEM((output_head_ring_kernel<true, false>), max_head_smem)
    SET_SMEM((output_head_ring_kernel<false, true>), max_head_smem)
    SET_SMEM((output_head_ring_kernel<true, true>), max_head_smem)
#undef SET_SMEM
    return kOk;
}

int launch_fused_linear(const FusedLinearParams& p, cudaStream_t stream, bool pdl) {
    return check_cuda(launch_k(fused_linear_kernel, p.grid, kLinearThreads, fused_linear_smem(p), stream, p, pdl));
}

static size_t attention_smem_nw(const AttentionParams& p, int nw) {
    const int G = p.H / p.Hkv, gmax = G <= 4 ? 8 : 16;     // the tensor-core key loops keep 8 or 16 rows per warp
    return sizeof(float) * ((size_t)(G + 2) * p.D + 2 * nw * gmax + (size_t)nw * G * p.D) + 64;
}
size_t attention_smem(const AttentionParams& p) {
    const int G = p.H / p.Hkv;
    return attention_smem_nw(p, G <= 4 ? 16 : 4);
}

int launch_attention(const AttentionParams& p, int batch, cudaStream_t stream, bool pdl, bool many_sequences) {
    const int G = p.H / p.Hkv;
    const dim3 grid(p.Hkv * p.S, batch);
    const size_t smem = attention_smem(p);
    cudaError_t e;
    if (many_sequences && p.S < G && G > 1 && p.D == 128) {     // whole groups per CTA (and slice), tensor cores
        const size_t sm = sizeof(float) * ((size_t)(G + 2) * p.D + 2 * 4 * 16 + (size_t)4 * G * p.D) + 64;
        e = G <= 8 ? launch_k(attention_decode_mma_kernel<8>, grid, 128, sm, stream, p, pdl)
                   : launch_k(attention_decode_mma_kernel<16>, grid, 128, sm, stream, p, pdl);
    }
    else if (many_sequences && G <= 4)
        e = launch_k(attention_decode_kernel<4, 4>, grid, 4 * 32, attention_smem_nw(p, 4), stream, p, pdl);
    else if (many_sequences && G <= 8)
        e = launch_k(attention_decode_kernel<8, 4>, grid, 4 * 32, attention_smem_nw(p, 4), stream, p, pdl);
    else if (G <= 4) e = launch_k(attention_decode_kernel<4>, grid, AttnCfg<4>::kThreads, smem, stream, p, pdl);
    else if (G <= 8) e = launch_k(attention_decode_kernel<8>, grid, AttnCfg<8>::kThreads, smem, stream, p, pdl);
    else e = launch_k(attention_decode_kernel<16>, grid, AttnCfg<16>::kThreads, smem, stream, p, pdl);
    return check_cuda(e);
}

// Shared memory of the output head.  The activations of all tokens are kept as f32 where that
// fits, else as bf16; the two 16-row stages of the ring-fed form are added where they fit too.
static size_t head_x_bytes(const HeadParams& p, bool compact) {
    return (compact ? 2 : 4) * (size_t)p.M * p.K + sizeof(float) * (32 + 16 * 8 * 2) + 64;
}
static size_t head_ring_bytes(const HeadParams& p, bool compact) {
    return (head_x_bytes(p, compact) + 127) / 128 * 128 + 2 * (size_t)kHeadRingRows * p.K * sizeof(__nv_bfloat16) + 2 * kHeadRingRows * 8 + 64;
}
struct HeadPlan {
    bool compact, ring;
    size_t smem;
};
static HeadPlan head_plan(const HeadParams& p) {
    const size_t cap = 227 * 1024;       // opt-in shared memory per CTA on sm_100
    if (p.K % 8 == 0) {
        for (bool compact : {false, true})
            if (head_ring_bytes(p, compact) <= cap) return {compact, true, head_ring_bytes(p, compact)};
    }
    const bool compact = head_x_bytes(p, false) > 160 * 1024;
    return {compact, false, head_x_bytes(p, compact)};
}
size_t head_smem(const HeadParams& p) { return head_plan(p).smem; }

int launch_head(const HeadParams& p, int grid, cudaStream_t stream, bool pdl) {
    const HeadPlan h = head_plan(p);
    const bool one = p.M == 1;
    auto go = [&](auto kernel) { return check_cuda(launch_k(kernel, grid, kHeadThreads, h.smem, stream, p, pdl)); };
    if (h.ring) {
        if (h.compact) return one ? go(output_head_ring_kernel<true, true>) : go(output_head_ring_kernel<true, false>);
        return one ? go(output_head_ring_kernel<false, true>) : go(output_head_ring_kernel<false, false>);
    }
    if (h.compact) return one ? go(output_head_kernel<true, true>) : go(output_head_kernel<true, false>);
    return one ? go(output_head_kernel<false, true>) : go(output_head_kernel<false, false>);
}

int launch_argmax(const ArgmaxParams& p, cudaStream_t stream, bool pdl) {
    return check_cuda(launch_k(argmax_kernel, 1, 256, 0, stream, p, pdl));
}

}  // namespace bitnet

// ---------------------------------------------------------------------------------------
// BitLinear without any allocation: the scratch of the split-K epilogue lives in a fixed
// device array inside the library image.
// ---------------------------------------------------------------------------------------
namespace bitnet {

namespace {

constexpr int kStaticRowGroups = 1024;                      // outputs of up to 16384 rows
constexpr int kStaticSlots = kStaticRowGroups * 128;        // one 64-bit slot per (row, token)
// 1 MB of slots plus one word for the kernel's error code.  Every GPU that loads the library
// holds this array until the process exits.
static __device__ __align__(256) unsigned long long g_static_scratch[kStaticSlots + 32];

struct StaticSetup {
    bool ready = false;                      // written last, under the mutex
    unsigned long long* scratch = nullptr;   // device address of g_static_scratch on this device
    int n_sm = 0;
    int smem_optin = 0;
};
StaticSetup g_static_setup[64];
std::mutex g_static_mutex;

// The set-up of the calling thread's current device (done once per device, under a lock).
StaticSetup* static_setup() {
    int dev = 0;
    if (check_cuda(cudaGetDevice(&dev))) return nullptr;
    if (dev < 0 || dev >= 64) return set_status(kUnsupported), nullptr;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticSetup& st = g_static_setup[dev];
    if (st.ready) return &st;
    // With that device current: the array's name is only a host-side handle, the kernel needs
    // the address the runtime reports for it on this device.
    void* ptr = nullptr;
    int n_sm = 0, smem_optin = 0;
    if (check_cuda(cudaGetSymbolAddress(&ptr, g_static_scratch))) return nullptr;
    if (check_cuda(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev)) ||
        check_cuda(cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) ||
        check_cuda(cudaFuncSetAttribute(fused_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin)))
        return nullptr;
    st.scratch = static_cast<unsigned long long*>(ptr);
    st.n_sm = n_sm;
    st.smem_optin = smem_optin;
    st.ready = true;
    return &st;
}

}  // namespace

}  // namespace bitnet

extern "C" int bitlinear_int8xint2_noalloc(int8_t* input0, int8_t* input1, void* output0, void* s, void* ws, int M,
                                           int N, int K, void* stream) {
    using namespace bitnet;
    set_status(kOk);
    if (!input0 || !input1 || !output0 || !s || !ws || M < 1 || N < 1 || K < 1) return set_status(kBadArgument), kBadArgument;
    if (N % 16 != 0 || K % 128 != 0) return set_status(kUnsupported), kUnsupported;
    if (M > 8 || N / 16 > kStaticRowGroups) return set_status(kTooLarge), kTooLarge;   // beyond the fixed scratch
    StaticSetup* st = static_setup();
    if (!st) return bitnet_last_status();
    FusedLinearParams p{};
    p.w2t = reinterpret_cast<const uint8_t*>(input1);
    p.N = N; p.K = K; p.M = M;
    plan_linear(p, st->n_sm);
    if (fused_linear_smem(p) > (size_t)st->smem_optin) return set_status(kTooLarge), kTooLarge;
    p.yq = input0; p.ldy = K;
    p.a_q_bf16 = static_cast<const __nv_bfloat16*>(s);
    p.out = static_cast<__nv_bfloat16*>(output0); p.ldo = N;
    p.ws_dev_bf16 = static_cast<const __nv_bfloat16*>(ws);
    // row segments of the reference's shape ladder (gpu/bitnet_kernels/bitnet_kernels.cu:4-33)
    // for the shapes this entry point can take (N <= 16384)
    int ws_num = 1;
    if (N == 3840 && K == 2560) ws_num = 3;
    else if (N == 13824 && K == 2560) ws_num = 2;
    else if (N == 4800 && K == 3200) ws_num = 6;
    p.seg.n_seg = ws_num;
    for (int i = 0; i < 8; ++i) p.seg.end[i] = i < ws_num ? (N / ws_num) * (i + 1) : N;
    p.acc_scratch = st->scratch;
    p.error_flag = reinterpret_cast<int*>(st->scratch + kStaticSlots);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the last call left (after a call that gave up on a wait: partly
    // filled slots): the slots this call uses must start at zero.  The error word is not
    // cleared here, so that bitlinear_int8xint2_noalloc_error can still report an earlier call.
    if (check_cuda(cudaMemsetAsync(st->scratch, 0, (size_t)(N / 16) * 128 * sizeof(unsigned long long), cs)))
        return kCudaError;
    return launch_fused_linear(p, cs, false);
}

extern "C" int bitlinear_int8xint2_noalloc_error(int clear) {
    using namespace bitnet;
    set_status(kOk);
    StaticSetup* st = static_setup();
    if (!st) return -1;
    int v = 0;
    if (check_cuda(cudaMemcpy(&v, st->scratch + kStaticSlots, sizeof(int), cudaMemcpyDeviceToHost))) return -1;
    if (v != 0 && clear && check_cuda(cudaMemset(st->scratch + kStaticSlots, 0, sizeof(unsigned long long)))) return -1;
    return v;
}
