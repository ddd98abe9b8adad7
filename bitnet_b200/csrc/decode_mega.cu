// One decode step (batch <= 8) as a single persistent kernel: one CTA per SM walks the
// layers' phases - wqkv, attention, wo, w13, w2 - and the output head, with a grid-wide
// barrier between phases instead of a kernel boundary.  The packed weight tiles of all
// BitLinears stream, in order, through a shared-memory ring of two rounds; once a round has
// been consumed, one thread issues the bulk copies of the round after next while the CTA waits
// at the next grid barrier - weights are constants, so the copies run ahead of the barriers and
// the next phase's weights are already on the SM when its activations become visible.  Every
// CTA owns whole 16-row groups of each BitLinear, so no partial sums cross CTAs.  Arithmetic
// and reduction orders are those of the chained kernels (decode_fused.cu), so both produce the
// same bits.
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
constexpr int kIssueTid = 256;                            // lane 0 of warp 8 issues the weight copies (thread 0 polls the barrier)
constexpr int kMiscBytes = 1024;                          // barriers and small arrays behind the ring
constexpr int kLinBlockBytes = (sizeof(FusedLinearParams) + 127) / 128 * 128;
constexpr int kAttBlockBytes = (sizeof(AttentionParams) + 127) / 128 * 128;
constexpr int kMaxLinears = 1024;                         // BitLinears per step the issue table holds

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
    unsigned long long* trace;       // optional: [n_layers * 5][16] cycle stamps of one CTA (a measurement aid)
    int trace_cta;                   // which CTA writes them (BITNET_TRACE_CTA, default 0)
};

__device__ __forceinline__ void stamp(const MegaParams& P, int cta, int tid, int phase, int i) {
    if (P.trace && cta == P.trace_cta && tid == 0) {
        P.trace[phase * 16 + i] = (unsigned long long)clock64();   // SM cycles: a CTA stays on one SM
    }
}

__device__ __forceinline__ void cstamp(const MegaParams& P, int cta, int tid, int phase, int i) {
    if (P.trace && cta == P.trace_cta && tid == 0) P.trace[phase * 16 + i] = (unsigned long long)clock64();
}

// What the copy stream needs to know of a BitLinear: this CTA's tiles.
struct LinIssue {
    const uint8_t* src;
    int n_tiles, pad;
};

// Whole row groups per CTA: row group rg belongs to CTA floor(rg * n_cta / row_groups)'s range,
// so every output row is summed inside one CTA and nothing is exchanged between CTAs.
struct Range {
    int rg0, n_rg;
};
__device__ __forceinline__ Range cta_range(int row_groups, int cta, int n_cta) {   // row_groups * n_cta < 2^32
    const unsigned int rg0 = (unsigned int)row_groups * (unsigned int)cta / (unsigned int)n_cta,
                       rg1 = (unsigned int)row_groups * (unsigned int)(cta + 1) / (unsigned int)n_cta;
    return Range{(int)rg0, (int)(rg1 - rg0)};
}

struct Shared {          // views into the dynamic shared memory
    uint8_t* ring;
    uint64_t* full_bar;  // [2 * hs]
    uint64_t* empty_bar; // [2]
    float* scratch;      // [16]
    float* sy_part;      // [8 tokens][8 warps]
    int* ysum_s;         // [8]
    float* a_s;          // [8]
    int* flag_s;         // [0] abort, [1] attention is_last, [2] exit ticket is last
    int64_t* pos_s;      // [8] positions at the start of the step
    LinIssue* issue;     // [n_layers * 4]
    FusedLinearParams* lin_s;   // [2] parameter blocks of the current and the next BitLinear
    AttentionParams* att_s;     // [2] same for the attention
    uint8_t* u;          // phase-private region
};

// Position of the copy stream: the next round to issue is round `r` of BitLinear `ph`; `gr`
// rounds have been issued so far; `pending` consumed rounds still wait for their successor to
// be issued.  Only thread kIssueTid uses it.
struct Cursor {
    int ph, r;
    unsigned int gr;
    int pending;
};
// Issues the bulk copies of the next round of the step, if there is one.
__device__ __noinline__ void issue_round(const MegaParams& P, const Shared& sh, Cursor& c) {
    const int hs = P.half_stages, round_tiles = hs * kStageTiles, n_lin = P.n_layers * 4;
    while (c.ph < n_lin) {
        const LinIssue li = sh.issue[c.ph];
        if (c.r * round_tiles >= li.n_tiles) {
            ++c.ph;
            c.r = 0;
            continue;
        }
        const int half = c.gr & 1;
        const int nr = min(round_tiles, li.n_tiles - c.r * round_tiles);
        const uint8_t* src = li.src + (int64_t)c.r * round_tiles * kTileBytes;
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

// Copies a parameter block from global to shared memory with `n_threads` threads starting at
// thread `first`; visible to the CTA after its next barrier.
template <class T>
__device__ __forceinline__ void fetch_block(T* dst, const T* src, int tid, int first) {
    static_assert(sizeof(T) % 8 == 0, "parameter blocks are copied in 8-byte words");
    const int i = tid - first;
    if (i >= 0 && i < (int)(sizeof(T) / 8))
        reinterpret_cast<unsigned long long*>(dst)[i] = __ldg(reinterpret_cast<const unsigned long long*>(src) + i);
}

// Arrival at a grid barrier: everything this CTA wrote is visible to whoever later sees the count.
__device__ __forceinline__ void grid_arrive(unsigned int* ctr, int tid) {
    csync();
    if (tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(ctr) : "memory");
}
// Wait until the arrivals reach `target`.  False when the wait gave up.
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
__device__ __host__ __forceinline__ int rg_cap(int N, int n_cta) { return ((N + 15) / 16 + n_cta - 1) / n_cta; }
__device__ __forceinline__ LinLayout lin_layout(const FusedLinearParams* d, uint8_t* u, int n_cta, int M) {
    LinLayout l;
    l.sacc = reinterpret_cast<int*>(u);
    l.xv = reinterpret_cast<__nv_bfloat16*>(l.sacc + rg_cap(d->N, n_cta) * 128);
    l.xb = l.xv + d->K_even;
    l.gs = l.xb + d->K_even;
    l.ys = reinterpret_cast<int8_t*>(l.gs + d->K_even);
    l.k_pad = d->k_tiles * kTileCols;
    l.y_stride = l.k_pad + 16;
    return l;
}

// Work of a BitLinear phase that does not depend on other CTAs: clear the row sums, stage the
// norm weight, write the row of zeros that the unused MMA columns read, and read the old
// residual value of the output element this thread will finalise (the residual stream was
// completed two phases ago).  `d` is the block in shared memory.
__device__ __forceinline__ float linear_pre(const FusedLinearParams* d, const Shared& sh, int M, int cta, int n_cta, int tid) {
    const LinLayout l = lin_layout(d, sh.u, n_cta, M);
    const int cap = rg_cap(d->N, n_cta) * 128;
#pragma unroll 1
    for (int i = tid; i < cap; i += kMegaConsumers) l.sacc[i] = 0;
    if (d->gamma && tid < kPrologueThreads) {   // each prologue thread stages the pieces it will read itself
#pragma unroll 1
        for (int v = tid; v < d->K_even / 8; v += kPrologueThreads) cp_async16(l.gs + v * 8, d->gamma + v * 8);
    }
#pragma unroll 1
    for (int v = tid; v < l.y_stride / 16; v += kMegaConsumers)
        *reinterpret_cast<uint4*>(l.ys + (size_t)M * l.y_stride + v * 16) = make_uint4(0, 0, 0, 0);
    float h_old = 0.f;
    if (d->out_kind == kOutResidual) {
        const Range rng = cta_range((d->N + 15) / 16, cta, n_cta);
        if (tid < rng.n_rg * 16 * M) {
            const int m = tid / (rng.n_rg * 16), row = rng.rg0 * 16 + (tid - m * (rng.n_rg * 16));
            if (row < d->N)
                h_old = __uint_as_float((unsigned int)__ldcg(reinterpret_cast<const unsigned short*>(d->out + (int64_t)m * d->ldo + row)) << 16);
        }
    }
    return h_old;
}

// The BitLinear itself.  `gr` counts this CTA's ring rounds over the whole step; `h_pre` is the
// value linear_pre returned.
__device__ __forceinline__ bool linear_phase(const MegaParams& P, const FusedLinearParams* d, const Shared& sh, int cta,
                                             int n_cta, int tid, unsigned int& gr, Cursor& cur, int phase_no, float h_pre) {
    const int64_t* tokens = P.tokens;
    const int M = P.M, hs = P.half_stages;
    int* error_flag = P.error_flag;
    const int warp = tid >> 5, lane = tid & 31;
    const LinLayout l = lin_layout(d, sh.u, n_cta, M);
    const int K = d->K, k_tiles = d->k_tiles, src = d->src;
    const int n_vec = d->K_even / 8;
    const Range rng = cta_range((d->N + 15) / 16, cta, n_cta);
    const int n_tiles = rng.n_rg * k_tiles;

    // ---- prologue: int8 activations of every token, by warps 0-7; meanwhile the copies that
    // refill the ring half the previous BitLinear left are issued -----------------------------
    cstamp(P, cta, tid, phase_no, 6);
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
            cstamp(P, cta, tid, phase_no, 7);
            if (src == kSrcGlu) {          // relu(x1)^2 * x3 with bf16 rounding after each step
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
            } else if (src == kSrcEmbedding && d->h_copy && cta == 0) {   // the residual stream starts as the embedding row
#pragma unroll 1
                for (int v = tid; v < n_vec; v += kPrologueThreads)
                    *reinterpret_cast<uint4*>(d->h_copy + (int64_t)m * K + v * 8) = *reinterpret_cast<const uint4*>(l.xv + v * 8);
            }
            float a, sy_warp;
            norm_quant_row<true>(l.xv, K, l.k_pad, d->gamma ? l.gs : nullptr, d->eps, l.ys + (size_t)m * l.y_stride,
                                 sh.scratch, tid, PSync(), a, sy_warp);
            cstamp(P, cta, tid, phase_no, 8);
            if (lane == 0) sh.sy_part[m * 8 + warp] = sy_warp;
            if (tid == 0) sh.a_s[m] = a;
            psync();   // xv is reused by the next token
        }
        if (tid < M) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += sh.sy_part[tid * 8 + w];
            sh.ysum_s[tid] = (int)t;
        }
    }
    cstamp(P, cta, tid, phase_no, 9);
    csync();
    cstamp(P, cta, tid, phase_no, 10);

    // ---- matmul over the staged tiles (see fused_linear_kernel for the scheme) ------------
    const int g = lane >> 2, q = lane & 3;
    const int round_tiles = hs * kStageTiles;
    int cur_rg = -1;
    int acc[4][4];
    auto flush = [&]() {
        if (cur_rg >= 0) {
            int* dst = l.sacc + cur_rg * 128;
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
    cstamp(P, cta, tid, phase_no, 2);
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
        cstamp(P, cta, tid, phase_no, 11);
        const int t_first = r * round_tiles + lo;          // tile index within this CTA's range
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
        cstamp(P, cta, tid, phase_no, 12);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.empty_bar[half]);
        if (tid == kIssueTid && r + 1 < n_rounds) {
            // more rounds of this BitLinear follow: refill this half as soon as all warps left it
            if (mbar_wait(&sh.empty_bar[half], parity)) {
                issue_round(P, sh, cur);
            } else {
                atomicExch(error_flag, 1);
                sh.flag_s[0] = 1;
            }
        }
    }
    flush();
    cstamp(P, cta, tid, phase_no, 13);
    csync();
    cstamp(P, cta, tid, phase_no, 14);
    if (sh.flag_s[0]) return false;
    if (n_tiles == 0) return true;
    ++cur.pending;   // every warp has left the last round's half: refilled during the next barrier wait
    cstamp(P, cta, tid, phase_no, 15);

    // ---- epilogue: every row of this CTA's row groups is complete --------------------------
    __nv_bfloat16* out = d->out;
    const int64_t ldo = d->ldo;
    const int N = d->N;
    const bool residual = d->out_kind == kOutResidual;
    const int per_m = rng.n_rg * 16;
#pragma unroll 1
    for (int idx = tid; idx < per_m * M; idx += kMegaConsumers) {
        const int m = idx / per_m, rem = idx - m * per_m;      // consecutive threads -> consecutive rows
        const int row = rng.rg0 * 16 + rem;
        if (row >= N) continue;
        float h_old = h_pre;
        if (residual && idx >= kMegaConsumers)   // beyond the element read ahead; written by another SM: read from L2
            h_old = __uint_as_float((unsigned int)__ldcg(reinterpret_cast<const unsigned short*>(out + (int64_t)m * ldo + row)) << 16);
        const float lin = lin_out(l.sacc[rem * 8 + m], sh.a_s[m], d->ws[segment_of(d->seg, row)]);
        out[(int64_t)m * ldo + row] = __float2bfloat16_rn(residual ? h_old + lin : lin);
    }
    stamp(P, cta, tid, phase_no, 4);
    return true;
}

__global__ void __launch_bounds__(kMegaThreads, 1) decode_mega_kernel(const MegaParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int hs = P.half_stages;
    const int n_lin = P.n_layers * 4;
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
    sh.pos_s = reinterpret_cast<int64_t*>(sh.flag_s + 8);
    sh.lin_s = reinterpret_cast<FusedLinearParams*>(misc + kMiscBytes);
    sh.att_s = reinterpret_cast<AttentionParams*>(misc + kMiscBytes + 2 * kLinBlockBytes);
    sh.issue = reinterpret_cast<LinIssue*>(misc + kMiscBytes + 2 * kLinBlockBytes + 2 * kAttBlockBytes);
    sh.u = reinterpret_cast<uint8_t*>(sh.issue) + (size_t)(n_lin * sizeof(LinIssue) + 127) / 128 * 128;

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
    // the step's constants: what the copy stream needs of every BitLinear, the first two
    // parameter blocks, the positions
#pragma unroll 1
    for (int i = tid; i < n_lin; i += kMegaThreads) {
        const FusedLinearParams* d = P.lin + i;
        const Range rng = cta_range((d->N + 15) / 16, cta, n_cta);
        sh.issue[i] = LinIssue{d->w2t + (int64_t)rng.rg0 * d->k_tiles * kTileBytes, rng.n_rg * d->k_tiles, 0};
    }
    fetch_block(&sh.lin_s[0], P.lin, tid, 0);
    if (n_lin > 1) fetch_block(&sh.lin_s[1], P.lin + 1, tid, 64);
    fetch_block(&sh.att_s[0], P.att, tid, 128);
    if (tid >= 256 && tid < 256 + M) sh.pos_s[tid - 256] = P.pos[tid - 256];
    __syncthreads();

    Cursor cur{0, 0, 0u, 0};
    if (tid == kIssueTid) {   // the first two rounds of the step
        issue_round(P, sh, cur);
        issue_round(P, sh, cur);
    }

    unsigned int gr = 0, barrier_no = 0;
    auto wait_prev = [&]() -> bool {   // all CTAs have finished the previous phase
        if (tid == kIssueTid) {        // meanwhile: the copies that refill the ring half the last BitLinear left
#pragma unroll 1
            for (; cur.pending > 0; --cur.pending) issue_round(P, sh, cur);
        }
        const bool ok = grid_wait(&P.bar[0], (unsigned int)n_cta * barrier_no, tid, sh, P.error_flag);
        if (!ok && tid == kIssueTid) drain_rounds(sh, hs, cur);
        return ok;
    };
    // BitLinear number li of the step; its block is in lin_s[li & 1], the next one's is fetched
    // into the other slot (free since the barrier that ended BitLinear li - 1).
    auto linear = [&](int li, int phase_no) -> bool {
        const FusedLinearParams* d = &sh.lin_s[li & 1];
        stamp(P, cta, tid, phase_no, 0);
        if (li >= 1 && li + 1 < n_lin) fetch_block(&sh.lin_s[(li + 1) & 1], P.lin + li + 1, tid, 448);
        const float h_pre = linear_pre(d, sh, M, cta, n_cta, tid);
        if (barrier_no > 0) {
            if (!wait_prev()) return false;
        } else {
            csync();
        }
        stamp(P, cta, tid, phase_no, 1);
        const bool ok = linear_phase(P, d, sh, cta, n_cta, tid, gr, cur, phase_no, h_pre);
        if (!ok) {
            if (tid == kIssueTid) drain_rounds(sh, hs, cur);
            return false;
        }
        grid_arrive(&P.bar[0], tid);
        stamp(P, cta, tid, phase_no, 5);
        ++barrier_no;
        return true;
    };
#pragma unroll 1
    for (int layer = 0; layer < P.n_layers; ++layer) {
        if (!linear(layer * 4, layer * 5)) return;   // wqkv
        // attention: one (sequence, kv head, slice) per CTA and turn; the slice's first keys are
        // requested before the barrier
        {
            const AttentionParams& ap = sh.att_s[layer & 1];
            const int per_seq = ap.Hkv * ap.S, items = M * per_seq;
            bool waited = false, ok = true;
            auto wait_once = [&]() {
                if (!waited) ok = wait_prev();
                waited = true;
            };
            stamp(P, cta, tid, layer * 5 + 1, 0);
#pragma unroll 1
            for (int item = cta; item < items && ok; item += n_cta) {
                const int b = item / per_seq;
                const int pos_b = (int)sh.pos_s[b];
                const AttnItem it = attention_item(ap, item - b * per_seq, pos_b);
                if (it.G == 0) continue;
                if (P.trace && tid == 0)   // cycle stamps of the traced CTA's attention go behind its phase stamps
                    sh.att_s[layer & 1].trace = cta == P.trace_cta ? P.trace + (layer * 5 + 1) * 16 : nullptr;
                csync();
                if (it.G == 1)
                    attention_body<1, kMegaWarps>(ap, sh.u, &sh.flag_s[1], b, it.kvh, it.h0, 1, it.split, it.S, pos_b, tid,
                                                  CSync(), wait_once);
                else
                    attention_body<4, kMegaWarps>(ap, sh.u, &sh.flag_s[1], b, it.kvh, it.h0, it.G, it.split, it.S, pos_b,
                                                  tid, CSync(), wait_once);
                csync();
            }
            wait_once();
            if (!ok) return;
            if (layer + 1 < P.n_layers) fetch_block(&sh.att_s[(layer + 1) & 1], P.att + layer + 1, tid, 448);
        }
        stamp(P, cta, tid, layer * 5 + 1, 4);
        grid_arrive(&P.bar[0], tid);
        stamp(P, cta, tid, layer * 5 + 1, 5);
        ++barrier_no;
#pragma unroll 1
        for (int j = 1; j < 4; ++j)   // wo, w13, w2
            if (!linear(layer * 4 + j, layer * 5 + 1 + j)) return;
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
    bool single_round = false;   // every BitLinear's tiles of a CTA fit one ring round
    size_t smem = 0;
};

// Shared memory the phase-private region needs for these phases.
static size_t mega_union_bytes(const FusedLinearParams* lin, int n_lin, const AttentionParams& ap, const HeadParams& hp,
                               int M, int grid) {
    size_t u = attention_smem(ap) > head_smem(hp) ? attention_smem(ap) : head_smem(hp);
    for (int i = 0; i < n_lin; ++i) {
        const FusedLinearParams& p = lin[i];
        const size_t y_stride = (size_t)p.k_tiles * kTileCols + 16;
        const size_t b = (size_t)rg_cap(p.N, grid) * 128 * 4 + (size_t)p.K_even * 6 + (size_t)(M + 1) * y_stride;
        u = b > u ? b : u;
    }
    // plus what sits between the ring and the phase-private region
    return u + 128 + kMiscBytes + 2 * kLinBlockBytes + 2 * kAttBlockBytes + ((size_t)n_lin * sizeof(LinIssue) + 127) / 128 * 128;
}

// Builds the device-side tables of a step.  lin: [n_layers * 4] fully filled parameter blocks
// (planned for `grid` CTAs), att: [n_layers].  Returns null (status set) when the step does
// not fit the kernel: grouped-query ratio above 4, head_dim other than what the attention
// body supports, or shared memory.
void* mega_create(const FusedLinearParams* lin, const AttentionParams* att, const HeadParams& hp, int n_layers, int M,
                  int grid, size_t smem_optin) {
    const int G = att[0].H / att[0].Hkv;
    if (G > 4 || M < 1 || M > 8 || n_layers * 4 > kMaxLinears) return set_status(kUnsupported), nullptr;
    const size_t u = mega_union_bytes(lin, n_layers * 4, att[0], hp, M, grid);
    int hs = kMaxHalfStages;
    while (hs >= 1 && (size_t)2 * hs * kStageBytes + u > smem_optin) --hs;
    if (hs < 1) return set_status(kTooLarge), nullptr;
    MegaPlan* mp = new (std::nothrow) MegaPlan();
    if (!mp) return set_status(kBadArgument), nullptr;
    mp->n_layers = n_layers; mp->M = M; mp->half_stages = hs; mp->grid = grid;
    mp->single_round = true;
    for (int i = 0; i < n_layers * 4; ++i)
        mp->single_round = mp->single_round && rg_cap(lin[i].N, grid) * lin[i].k_tiles <= hs * kStageTiles;
    mp->smem = (size_t)2 * hs * kStageBytes + u;
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

// True when every BitLinear's share of a CTA fits one round of the ring, so that all its weights
// are on the SM before the phase starts: the condition under which the persistent kernel comes
// within a few per cent of the chain of kernels (2B architecture; 3B and 8B need several rounds
// per phase and lose more).
bool mega_single_round(const void* plan) { return plan && static_cast<const MegaPlan*>(plan)->single_round; }

void mega_destroy(void* plan) {
    MegaPlan* mp = static_cast<MegaPlan*>(plan);
    if (!mp) return;
    if (mp->lin_dev) cudaFree(mp->lin_dev);
    delete mp;
}

int mega_launch(void* plan, const HeadParams& hp, int64_t* tokens, int64_t* pos, int64_t* out, int* error_flag,
                unsigned long long* trace, cudaStream_t stream) {
    MegaPlan* mp = static_cast<MegaPlan*>(plan);
    MegaParams P{};
    P.lin = mp->lin_dev; P.att = mp->att_dev; P.head = hp;
    P.n_layers = mp->n_layers; P.M = mp->M; P.half_stages = mp->half_stages;
    P.tokens = tokens; P.pos = pos; P.out = out; P.bar = mp->bar; P.error_flag = error_flag; P.trace = trace;
    P.trace_cta = getenv("BITNET_TRACE_CTA") ? atoi(getenv("BITNET_TRACE_CTA")) : 0;
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
