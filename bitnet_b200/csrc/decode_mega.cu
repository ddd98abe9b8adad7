// One decode step (batch <= 8) as a single persistent kernel: one CTA per SM walks the
// layers' phases - wqkv, attention, wo, w13, w2 - and the output head, with a grid-wide
// barrier between phases instead of a kernel boundary.  The packed weight tiles of all
// BitLinears stream, in order, through a shared-memory ring of two rounds; as soon as a
// round has been consumed, thread 0 issues the bulk copies of the round after next - weights
// are constants, so the copies run ahead of the barriers and the next phase's weights are
// already on the SM when its activations become visible.  Arithmetic and reduction orders are those of the
// chained kernels (decode_fused.cu), so both produce the same bits.
//
// All CTAs must be resident at once: the kernel is launched cooperatively with at most one
// CTA per SM.  Every wait is bounded; a wait that gives up sets the error flag and the CTA
// leaves after draining its own copies.
#include <stdlib.h>

#include <new>

#include "common.cuh"
#include "decode_device.cuh"
#include "decode_fused.h"
#include "prologue.cuh"

namespace bitnet {

namespace {

constexpr int kStageTiles = 32;
constexpr int kStageBytes = kStageTiles * kTileBytes;     // 16 KB
constexpr int kMaxHalfStages = 4;                         // a round: up to 4 stages = 128 tiles
constexpr int kMegaWarps = 16;                            // consumer warps
constexpr int kMegaConsumers = kMegaWarps * 32;           // 512
constexpr int kMegaThreads = kMegaConsumers;
constexpr int kMiscBytes = 1024;                          // barriers and small arrays behind the ring

__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kMegaConsumers) : "memory"); }
__device__ __forceinline__ void psync() { asm volatile("bar.sync 2, %0;\n" ::"n"(kPrologueThreads) : "memory"); }
struct CSync {
    __device__ __forceinline__ void operator()() const { csync(); }
};
struct PSync {
    __device__ __forceinline__ void operator()() const { psync(); }
};

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct Range {
    int t0, n_tiles;
};
__device__ __forceinline__ Range cta_range(const FusedLinearParams* d, int cta) {
    if (cta >= d->grid) return Range{0, 0};
    return Range{cta * d->tiles_base + min(cta, d->tiles_rem), d->tiles_base + (cta < d->tiles_rem ? 1 : 0)};
}
__device__ __forceinline__ int cta_of_tile(const FusedLinearParams* d, int t) {
    const int big = d->tiles_rem * (d->tiles_base + 1);
    return t < big ? t / (d->tiles_base + 1) : d->tiles_rem + (t - big) / d->tiles_base;
}

struct MegaParams {
    const FusedLinearParams* lin;    // [n_layers][4]: wqkv, wo, w13, w2 (device memory)
    const AttentionParams* att;      // [n_layers]
    HeadParams head;
    int n_layers, M, half_stages;
    int64_t* tokens;                 // [M] in: this step's ids; out: the chosen ids
    int64_t* pos;                    // [M] advanced by one
    int64_t* out;                    // [M]
    unsigned int* bar;               // [0] barrier arrivals, [1] exit tickets; zero between steps
    int* error_flag;
};

struct Shared {          // views into the dynamic shared memory
    uint8_t* ring;
    uint64_t* full_bar;  // [2 * hs]
    uint64_t* empty_bar; // [2]
    float* scratch;      // [16]
    float* sy_part;      // [8][8]
    int* ysum_s;         // [8]
    float* a_s;          // [8]
    int* flag_s;         // [0] abort, [1] attention is_last, [2] exit ticket is last
    uint8_t* u;          // phase-private region
};

// Position of the copy stream: the next round to issue is round `r` of BitLinear `ph`; `gr`
// rounds have been issued so far.  Only thread 0 uses it.
struct Cursor {
    int ph, r;
    unsigned int gr;
};
// Issues the bulk copies of the next round of the step, if there is one.
__device__ __noinline__ void issue_round(const MegaParams& P, const Shared& sh, int cta, Cursor& c) {
    const int hs = P.half_stages, round_tiles = hs * kStageTiles, n_lin = P.n_layers * 4;
    while (c.ph < n_lin) {
        const FusedLinearParams* d = P.lin + c.ph;
        const Range rng = cta_range(d, cta);
        const int n_rounds = (rng.n_tiles + round_tiles - 1) / round_tiles;
        if (c.r >= n_rounds) {
            ++c.ph;
            c.r = 0;
            continue;
        }
        const int half = c.gr & 1;
        const int nr = min(round_tiles, rng.n_tiles - c.r * round_tiles);
        const uint8_t* src = d->w2t + ((int64_t)rng.t0 + (int64_t)c.r * round_tiles) * kTileBytes;
#pragma unroll 1
        for (int s = 0; s < hs; ++s) {
            uint64_t* bar = &sh.full_bar[half * hs + s];
            const int tiles = min(kStageTiles, nr - s * kStageTiles);
            if (tiles > 0) {
                mbar_expect_tx(bar, tiles * kTileBytes);
                bulk_g2s(sh.ring + (size_t)(half * hs + s) * kStageBytes, src + (int64_t)s * kStageBytes, tiles * kTileBytes, bar);
            } else {
                mbar_arrive(bar);   // unused stage: keep its phase in step with the round count
            }
        }
        ++c.r;
        ++c.gr;
        return;
    }
}
// Before an early exit: see the copies of the last two issued rounds land (bounded), so that
// nothing is in flight into shared memory when the CTA leaves.
__device__ __noinline__ void drain_rounds(const Shared& sh, int hs, const Cursor& c) {
#pragma unroll 1
    for (unsigned int back = 1; back <= 2 && back <= c.gr; ++back) {
        const unsigned int g2 = c.gr - back;
#pragma unroll 1
        for (int s = 0; s < hs; ++s) mbar_wait(&sh.full_bar[(g2 & 1) * hs + s], (g2 >> 1) & 1);
    }
}

// Arrival at grid barrier number `k` of the step (counted from 0): everything this CTA wrote
// is visible to whoever later sees the count.
__device__ __forceinline__ void grid_arrive(unsigned int* ctr, int tid) {
    csync();
    if (tid == 0) {
        __threadfence();
        atomicAdd(ctr, 1u);
    }
}
// Wait until all n_cta CTAs have arrived at barrier k.  False when the wait gave up.
__device__ __forceinline__ bool grid_wait(unsigned int* ctr, unsigned int target, int tid, const Shared& sh, int* error_flag) {
    if (tid == 0) {
        const long long t0 = clock64();
        while ((int)(ld_acquire(ctr) - target) < 0) {
            if (clock64() - t0 > kWaitCycles) {
                atomicExch(error_flag, 3);
                sh.flag_s[0] = 1;
                break;
            }
        }
    }
    csync();
    return sh.flag_s[0] == 0;
}

// Layout of the phase-private region during a BitLinear.
struct LinLayout {
    int* sacc;
    __nv_bfloat16 *xv, *xb, *gs;
    int8_t* ys;
    int k_pad, y_stride;
};
__device__ __forceinline__ LinLayout lin_layout(const FusedLinearParams* d, uint8_t* u, int M) {
    LinLayout l;
    l.sacc = reinterpret_cast<int*>(u);
    l.xv = reinterpret_cast<__nv_bfloat16*>(l.sacc + d->r_max * 128);
    l.xb = l.xv + d->K_even;
    l.gs = l.xb + d->K_even;
    l.ys = reinterpret_cast<int8_t*>(l.gs + d->K_even);
    l.k_pad = d->k_tiles * kTileCols;
    l.y_stride = l.k_pad + 16;
    (void)M;
    return l;
}

// Work of a BitLinear phase that does not depend on other CTAs: clear the row sums, stage the
// norm weight, write the row of zeros that the unused MMA columns read.
__device__ __forceinline__ void linear_pre(const FusedLinearParams* d, const Shared& sh, int M, int tid) {
    const LinLayout l = lin_layout(d, sh.u, M);
#pragma unroll 1
    for (int i = tid; i < d->r_max * 128; i += kMegaConsumers) l.sacc[i] = 0;
    if (d->gamma && tid < kPrologueThreads) {   // each prologue thread stages the pieces it will read itself
#pragma unroll 1
        for (int v = tid; v < d->K_even / 8; v += kPrologueThreads) cp_async16(l.gs + v * 8, d->gamma + v * 8);
    }
#pragma unroll 1
    for (int v = tid; v < l.y_stride / 16; v += kMegaConsumers)
        *reinterpret_cast<uint4*>(l.ys + (size_t)M * l.y_stride + v * 16) = make_uint4(0, 0, 0, 0);
}

// The BitLinear itself.  `gr` counts this CTA's ring rounds over the whole step.
__device__ __forceinline__ bool linear_phase(const MegaParams& P, const FusedLinearParams* d, const Shared& sh, int cta,
                                             int tid, unsigned int& gr, Cursor& cur) {
    const int64_t* tokens = P.tokens;
    const int M = P.M, hs = P.half_stages;
    int* error_flag = P.error_flag;
    const int warp = tid >> 5, lane = tid & 31;
    const LinLayout l = lin_layout(d, sh.u, M);
    const int K = d->K, k_tiles = d->k_tiles, src = d->src;
    const int n_vec = d->K_even / 8;
    const Range rng = cta_range(d, cta);
    const int t0 = rng.t0, n_tiles = rng.n_tiles;

    // ---- prologue: int8 activations of every token, by warps 0-7 -------------------------
    if (warp < 8) {
#pragma unroll 1
        for (int m = 0; m < M; ++m) {
            const __nv_bfloat16* row = src == kSrcEmbedding ? d->emb + tokens[m] * (int64_t)K : d->x + (int64_t)m * d->ldx;
#pragma unroll 1
            for (int v = tid; v < n_vec; v += kPrologueThreads) {
                cp_async16(l.xv + v * 8, row + v * 8);
                if (src == kSrcGlu) cp_async16(l.xb + v * 8, row + K + v * 8);
            }
            cp_async_wait_all();   // also covers the norm weight staged before the barrier
            if (src == kSrcGlu) {
#pragma unroll 1
                for (int v = tid; v < n_vec; v += kPrologueThreads) {
                    Vec8 x1 = unpack_bf16x8(*reinterpret_cast<const uint4*>(l.xv + v * 8));
                    const Vec8 x3 = unpack_bf16x8(*reinterpret_cast<const uint4*>(l.xb + v * 8));
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float t = fmaxf(x1.v[e], 0.f);
                        x1.v[e] = bf16_round(bf16_round(t * t) * x3.v[e]);
                    }
                    *reinterpret_cast<uint4*>(l.xv + v * 8) = pack_bf16x8(x1);
                }
            } else if (src == kSrcEmbedding && d->h_copy && cta == 0) {
#pragma unroll 1
                for (int v = tid; v < n_vec; v += kPrologueThreads)
                    *reinterpret_cast<uint4*>(d->h_copy + (int64_t)m * K + v * 8) = *reinterpret_cast<const uint4*>(l.xv + v * 8);
            }
            float a, sy_warp;
            norm_quant_row(l.xv, K, l.k_pad, d->gamma ? l.gs : nullptr, d->eps, l.ys + (size_t)m * l.y_stride, sh.scratch,
                           tid, PSync(), a, sy_warp);
            if (lane == 0) sh.sy_part[m * 8 + warp] = sy_warp;
            if (tid == 0) sh.a_s[m] = a;
            psync();
        }
        if (tid < M) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += sh.sy_part[tid * 8 + w];
            sh.ysum_s[tid] = (int)t;
        }
    }
    csync();

    // ---- matmul over the staged tiles (see fused_linear_kernel for the scheme) ------------
    const int g = lane >> 2, q = lane & 3;
    const int rg_first = t0 / k_tiles;
    const int round_tiles = hs * kStageTiles;
    int cur_rg = -1;
    int acc[4][4];
    auto flush = [&]() {
        if (cur_rg >= 0) {
            int* dst = l.sacc + (cur_rg - rg_first) * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = 2 * q + (i & 1);
                if (tok < M) {
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
    const int8_t* y_lane = l.ys + (size_t)(g < M ? g : M) * l.y_stride + 32 * q;
    const int ysub0 = (2 * q < M) ? sh.ysum_s[2 * q] : 0, ysub1 = (2 * q + 1 < M) ? sh.ysum_s[2 * q + 1] : 0;
    const int n_rounds = (n_tiles + round_tiles - 1) / round_tiles;
    bool ok = true;
#pragma unroll 1
    for (int r = 0; r < n_rounds; ++r, ++gr) {
        const int half = gr & 1;
        const uint32_t parity = (gr >> 1) & 1;
        const int nr = min(round_tiles, n_tiles - r * round_tiles);
        const int lo = nr * warp / kMegaWarps, hi = nr * (warp + 1) / kMegaWarps;
        if (hi > lo) {
#pragma unroll 1
            for (int s = lo / kStageTiles; s <= (hi - 1) / kStageTiles; ++s)
                ok = ok && mbar_wait(&sh.full_bar[half * hs + s], parity);
            if (!ok) {
                if (lane == 0) {
                    atomicExch(error_flag, 2);
                    sh.flag_s[0] = 1;
                }
                break;
            }
        }
        const int t_first = t0 + r * round_tiles + lo;
        int rg = t_first / k_tiles, kt = t_first - rg * k_tiles;
        const uint8_t* tile = sh.ring + (size_t)half * hs * kStageBytes + lo * kTileBytes + lane * 16;
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
            if (kt == 0) {
                acc[0][0] -= ysub0; acc[0][1] -= ysub1; acc[0][2] -= ysub0; acc[0][3] -= ysub1;
            }
            if (++kt == k_tiles) {
                kt = 0;
                ++rg;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.empty_bar[half]);
        if (tid == 0 && r + 1 < n_rounds) {
            // more rounds of this BitLinear follow: refill this half as soon as all warps left it
            if (mbar_wait(&sh.empty_bar[half], parity)) {
                issue_round(P, sh, cta, cur);
            } else {
                atomicExch(error_flag, 1);
                sh.flag_s[0] = 1;
            }
        }
    }
    flush();
    csync();
    if (sh.flag_s[0]) return false;
    if (n_tiles == 0) return true;
    if (tid == 0) issue_round(P, sh, cta, cur);   // every warp has left the last round's half

    // ---- epilogue: rows whose sums are complete here are finalised here; row groups shared
    // with other CTAs go through the 64-bit ticket slots, the last contributor finalises ----
    const int n_rg = (t0 + n_tiles - 1) / k_tiles - rg_first + 1;
    const int rg_last = rg_first + n_rg - 1;
    const bool part_first = t0 > rg_first * k_tiles || (t0 + n_tiles) < (rg_first + 1) * k_tiles;
    const bool part_last = n_rg > 1 && (t0 + n_tiles) < (rg_last + 1) * k_tiles;
    __nv_bfloat16* out = d->out;
    const int64_t ldo = d->ldo;
    const int N = d->N;
    const bool residual = d->out_kind == kOutResidual;
#pragma unroll 1
    for (int idx = tid; idx < n_rg * 16 * M; idx += kMegaConsumers) {
        const int m = idx / (n_rg * 16), rem = idx - m * (n_rg * 16);
        const int li = rem >> 4, r = rem & 15;
        const int rgi = rg_first + li, row = rgi * 16 + r;
        const bool partial = (li == 0 && part_first) || (li == n_rg - 1 && li > 0 && part_last);
        if (row >= N && !partial) continue;
        float h_old = 0.f;
        if (residual && row < N)   // written by another SM in an earlier phase: read it from L2
            h_old = __uint_as_float((unsigned int)__ldcg(reinterpret_cast<const unsigned short*>(out + (int64_t)m * ldo + row)) << 16);
        int v = l.sacc[rem * 8 + m];
        if (partial) {
            const int lo_t = rgi * k_tiles, hi_t = lo_t + k_tiles - 1;
            const long long expected = cta_of_tile(d, hi_t) - cta_of_tile(d, lo_t) + 1;
            unsigned long long* slot = &d->acc_scratch[(int64_t)rgi * 128 + r * 8 + m];
            const unsigned long long add = (unsigned long long)((long long)v + (1LL << 40));
            const long long tot = (long long)(atomicAdd(slot, add) + add);
            const long long cnt = (tot + (1LL << 39)) >> 40;
            if (cnt != expected) continue;
            v = (int)(tot - (cnt << 40));
            *slot = 0ull;
        }
        if (row >= N) continue;
        const float lin = lin_out(v, sh.a_s[m], d->ws[segment_of(d->seg, row)]);
        out[(int64_t)m * ldo + row] = __float2bfloat16_rn(residual ? h_old + lin : lin);
    }
    return true;
}


__global__ void __launch_bounds__(kMegaThreads, 1) decode_mega_kernel(const MegaParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int hs = P.half_stages;
    Shared sh;
    sh.ring = smem;
    uint8_t* misc = smem + (size_t)2 * hs * kStageBytes;
    sh.full_bar = reinterpret_cast<uint64_t*>(misc);
    sh.empty_bar = sh.full_bar + 2 * kMaxHalfStages;
    sh.scratch = reinterpret_cast<float*>(sh.empty_bar + 2);
    sh.sy_part = sh.scratch + 16;
    sh.ysum_s = reinterpret_cast<int*>(sh.sy_part + 64);
    sh.a_s = reinterpret_cast<float*>(sh.ysum_s + 8);
    sh.flag_s = reinterpret_cast<int*>(sh.a_s + 8);
    sh.u = misc + kMiscBytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, n_cta = gridDim.x;
    const int M = P.M;
    if (tid == 0) {
#pragma unroll 1
        for (int s = 0; s < 2 * hs; ++s) mbar_init(&sh.full_bar[s], 1);
        mbar_init(&sh.empty_bar[0], kMegaWarps);
        mbar_init(&sh.empty_bar[1], kMegaWarps);
        sh.flag_s[0] = 0;
        sh.flag_s[1] = 0;
        sh.flag_s[2] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    Cursor cur{0, 0, 0u};
    if (tid == 0) {   // the first two rounds of the step
        issue_round(P, sh, cta, cur);
        issue_round(P, sh, cta, cur);
    }

    unsigned int gr = 0, barrier_no = 0;
    auto wait_prev = [&]() -> bool {   // all CTAs have finished the previous phase
        const bool ok = grid_wait(&P.bar[0], (unsigned int)n_cta * barrier_no, tid, sh, P.error_flag);
        if (!ok && tid == 0) drain_rounds(sh, hs, cur);
        return ok;
    };
    auto linear = [&](const FusedLinearParams* d) -> bool {
        const bool ok = linear_phase(P, d, sh, cta, tid, gr, cur);
        if (!ok && tid == 0) drain_rounds(sh, hs, cur);
        return ok;
    };
#pragma unroll 1
    for (int layer = 0; layer < P.n_layers; ++layer) {
        const FusedLinearParams* lin = P.lin + layer * 4;
        // wqkv
        linear_pre(lin, sh, M, tid);
        if (barrier_no > 0 && !wait_prev()) return;
        if (!linear(lin)) return;
        grid_arrive(&P.bar[0], tid);
        ++barrier_no;
        // attention: one (sequence, kv head, slice) per CTA and turn
        if (!wait_prev()) return;
        {
            AttentionParams ap = P.att[layer];
            ap.pos = P.pos;
            const int items = M * ap.Hkv * ap.S;
#pragma unroll 1
            for (int item = cta; item < items; item += n_cta) {
                const int b = item / (ap.Hkv * ap.S), rem = item - b * (ap.Hkv * ap.S);
                attention_body<4, kMegaWarps>(ap, sh.u, &sh.flag_s[1], b, rem / ap.S, rem % ap.S, tid, CSync());
                csync();
            }
        }
        grid_arrive(&P.bar[0], tid);
        ++barrier_no;
        // wo, w13, w2
#pragma unroll 1
        for (int j = 1; j < 4; ++j) {
            linear_pre(lin + j, sh, M, tid);
            if (!wait_prev()) return;
            if (!linear(lin + j)) return;
            grid_arrive(&P.bar[0], tid);
            ++barrier_no;
        }
    }
    if (!wait_prev()) return;

    // ---- output head over this CTA's slice of the vocabulary, then the greedy choice by the
    // CTA that finishes last -------------------------------------------------------------------
    head_body(P.head, sh.u, cta, n_cta, tid, CSync());
    csync();
    if (tid == 0) {
        __threadfence();
        sh.flag_s[2] = atomicAdd(&P.bar[1], 1u) == (unsigned int)n_cta - 1;
    }
    csync();
    if (!sh.flag_s[2]) return;
    __threadfence();
    float* sv = reinterpret_cast<float*>(sh.u);
    int* si = reinterpret_cast<int*>(sv + kMegaWarps);
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int c = tid; c < n_cta; c += kMegaConsumers) {
            const float cv = __ldcg(&P.head.part_val[c * 8 + m]);
            const int ci = __ldcg(&P.head.part_idx[c * 8 + m]);
            if (cv > v || (cv == v && ci < i)) { v = cv; i = ci; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, i, o);
            if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
        }
        if (lane == 0) { sv[warp] = v; si[warp] = i; }
        csync();
        if (tid == 0) {
            for (int w = 1; w < kMegaWarps; ++w)
                if (sv[w] > v || (sv[w] == v && si[w] < i)) { v = sv[w]; i = si[w]; }
            P.out[m] = i;
            P.tokens[m] = i;
            P.pos[m] += 1;
        }
        csync();
    }
    if (tid == 0) {   // every CTA has left its last barrier: the counters restart at zero
        P.bar[0] = 0;
        P.bar[1] = 0;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
struct MegaPlan {
    FusedLinearParams* lin_dev = nullptr;
    AttentionParams* att_dev = nullptr;
    unsigned int* bar = nullptr;
    int n_layers = 0, M = 0, half_stages = 0, grid = 0;
    size_t smem = 0;
};

// Shared memory the phase-private region needs for these phases.
static size_t mega_union_bytes(const FusedLinearParams* lin, int n_lin, const AttentionParams& ap, const HeadParams& hp,
                               int M) {
    size_t u = attention_smem(ap) > head_smem(hp) ? attention_smem(ap) : head_smem(hp);
    for (int i = 0; i < n_lin; ++i) {
        const FusedLinearParams& p = lin[i];
        const size_t y_stride = (size_t)p.k_tiles * kTileCols + 16;
        const size_t b = (size_t)p.r_max * 128 * 4 + (size_t)p.K_even * 6 + (size_t)(M + 1) * y_stride;
        u = b > u ? b : u;
    }
    return u + 128;
}

// Builds the device-side tables of a step.  lin: [n_layers * 4] fully filled parameter blocks
// (planned for `grid` CTAs), att: [n_layers].  Returns null (status set) when the step does
// not fit the kernel: grouped-query ratio above 4, head_dim other than what the attention
// body supports, or shared memory.
void* mega_create(const FusedLinearParams* lin, const AttentionParams* att, const HeadParams& hp, int n_layers, int M,
                  int grid, size_t smem_optin) {
    const int G = att[0].H / att[0].Hkv;
    if (G > 4 || M < 1 || M > 8) return set_status(kUnsupported), nullptr;
    const size_t u = mega_union_bytes(lin, n_layers * 4, att[0], hp, M);
    int hs = kMaxHalfStages;
    while (hs >= 1 && (size_t)2 * hs * kStageBytes + kMiscBytes + u > smem_optin) --hs;
    if (hs < 1) return set_status(kTooLarge), nullptr;
    MegaPlan* mp = new (std::nothrow) MegaPlan();
    if (!mp) return set_status(kBadArgument), nullptr;
    mp->n_layers = n_layers; mp->M = M; mp->half_stages = hs; mp->grid = grid;
    mp->smem = (size_t)2 * hs * kStageBytes + kMiscBytes + u;
    const size_t lin_bytes = sizeof(FusedLinearParams) * n_layers * 4, att_bytes = sizeof(AttentionParams) * n_layers;
    uint8_t* base = nullptr;
    int occ = 0;
    if (check_cuda(cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mp->smem)) ||
        check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, decode_mega_kernel, kMegaThreads, mp->smem))) {
        delete mp;
        return nullptr;
    }
    if (occ < 1) {
        delete mp;
        return set_status(kTooLarge), nullptr;
    }
    const size_t lin_al = (lin_bytes + 255) / 256 * 256, att_al = (att_bytes + 255) / 256 * 256;
    if (check_cuda(cudaMalloc(&base, lin_al + att_al + 256)) || check_cuda(cudaMemset(base, 0, lin_al + att_al + 256)) ||
        check_cuda(cudaMemcpy(base, lin, lin_bytes, cudaMemcpyHostToDevice)) ||
        check_cuda(cudaMemcpy(base + lin_al, att, att_bytes, cudaMemcpyHostToDevice))) {
        if (base) cudaFree(base);
        delete mp;
        return nullptr;
    }
    mp->lin_dev = reinterpret_cast<FusedLinearParams*>(base);
    mp->att_dev = reinterpret_cast<AttentionParams*>(base + lin_al);
    mp->bar = reinterpret_cast<unsigned int*>(base + lin_al + att_al);
    return mp;
}

void mega_destroy(void* plan) {
    MegaPlan* mp = static_cast<MegaPlan*>(plan);
    if (!mp) return;
    if (mp->lin_dev) cudaFree(mp->lin_dev);
    delete mp;
}

int mega_launch(void* plan, const HeadParams& hp, int64_t* tokens, int64_t* pos, int64_t* out, int* error_flag,
                cudaStream_t stream) {
    MegaPlan* mp = static_cast<MegaPlan*>(plan);
    MegaParams P{};
    P.lin = mp->lin_dev; P.att = mp->att_dev; P.head = hp;
    P.n_layers = mp->n_layers; P.M = mp->M; P.half_stages = mp->half_stages;
    P.tokens = tokens; P.pos = pos; P.out = out; P.bar = mp->bar; P.error_flag = error_flag;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(mp->grid);
    cfg.blockDim = dim3(kMegaThreads);
    cfg.dynamicSmemBytes = mp->smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs resident at once, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, decode_mega_kernel, P));
}

}  // namespace bitnet
