// W2A8 BitLinear for M >= 16 tokens (batched decode, prefill) on the 5th-generation tensor
// cores: tcgen05.mma kind::i8 with the accumulators in tensor memory.  The reference has no
// counterpart (its GPU kernel takes M == 1 only, gpu/bitnet_kernels/bitnet_kernels.cu:4-36,
// and its prefill runs in bf16, gpu/generate.py:56-57).
//
// D[128 weight rows, TN tokens] += A[128 x 32, u8, K-major] * B[TN x 32, s8, K-major].
// One CTA owns a 128-row block of the weight matrix and a block of TN tokens and walks K in
// tiles of 128 columns, two per pipeline step.  Roles (18 warps):
//   warp 16    - producer: packed 2-bit weight tiles, global -> shared ring (cp.async.bulk)
//   warps 0-15 - unpack: warp w turns row group w & 7 (16 rows) of K tile w >> 3 of the step
//                into int8 operands in the canonical no-swizzle K-major layout, and all of
//                them stage the int8 activations of the step in the same layout
//   warp 17    - issues the MMAs (one elected lane) and commits them to mbarriers
//   warps 0-7  - epilogue: tcgen05.ld, fold, rescale, store
// The 2-bit fields are separated by AND masks only, as in the decode kernel: field j of every
// byte stays scaled by 4^j and gets its own accumulator (TMEM columns j*TN..), which the
// epilogue folds with exact shifts.  In the W2T layout field j of lane chunk q covers columns
// 32q+8j..32q+8j+7 of a K tile, so operand slab j holds those 4 x 8 = 32 columns of A, and
// the activations are staged with the same column selection.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace bitnet {

namespace {

constexpr int kRows = 128;                       // weight rows per CTA (UMMA M)
constexpr int kWorkerWarps = 16;                 // warp w: row group w & 7 of K tile w >> 3 of the stage
constexpr int kWorkerThreads = kWorkerWarps * 32;
constexpr int kProducerWarp = kWorkerWarps, kMmaWarp = kWorkerWarps + 1;
constexpr int kThreadsTc = (kWorkerWarps + 2) * 32;
constexpr int kPackStages = 3;                   // packed-weight ring
constexpr int kPackTiles = 4;                    // K tiles per packed stage
constexpr int kPackStageBytes = 8 * kPackTiles * kTileBytes;   // 16 KB
constexpr int kOpStages = 2;                     // unpacked operand buffers
constexpr int kOpTiles = 2;                      // K tiles per operand buffer
constexpr int kSlabA = 4096;                     // 128 rows x 32 int8, canonical K-major
constexpr long long kWaitCyclesTc = 2000000000LL;

struct TcParams {
    const uint8_t* w2t;
    const int8_t* y;
    int64_t ldy;
    const int32_t* ysum;         // [M] or null (then computed from y on the fly is not offered: required)
    int32_t* acc_out;            // [M, N] or null
    __nv_bfloat16* out;          // [M, ldo] or null
    int64_t ldo;
    const float* a_f32;
    const __nv_bfloat16* a_bf16;
    const float* ws_f32;
    const __nv_bfloat16* ws_bf16;
    ScaleSegments seg;
    int M, N, K, k_tiles, n_rowgroups;
    int k_splits;                // grid.z: CTAs that share an output tile and add into acc_ws
    int32_t* acc_ws;             // [M, N] zero-initialised int32 work space (k_splits > 1)
    int* error_flag;
    unsigned long long* trace;   // optional cycle counters (measurement aid)
    // Optional: the activations already in the tensor core's operand layout (restage_kernel):
    // for K tile kt and field j, m_groups blocks of 8 tokens x 32 selected int8 (256 bytes each,
    // two 8 x 16-byte core matrices), so that the slab of TN tokens is one contiguous piece
    // that a bulk copy drops into the operand buffer.  Null: worker warps stage them from y.
    const uint8_t* ycanon;
    int m_groups;
    bool defer_finalize;         // split K: no second pass here, the caller's next kernel finalises acc_ws
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool bar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded: gives up after about a second; `abort_flag` (shared) makes everybody else give up too.
__device__ __noinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (bar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!bar_try(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCyclesTc) {
            *abort_flag = 1;
            return false;
        }
    }
    return true;
}
// The same with an L2 eviction policy: packed weights are read once per call and leave L2 first.
__device__ __forceinline__ void bulk_load_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::"r"(
            smem_addr(dst)),
        "l"(src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// Shared memory operand descriptor: K-major, no swizzle.  Core matrices (8 rows x 16 bytes)
// are 128 contiguous bytes; the two core matrices along K are `lbo` bytes apart, 8-row
// groups `sbo` bytes apart.  Bits: [0,14) address >> 4, [16,30) lbo >> 4, [32,46) sbo >> 4,
// [46,48) descriptor version 1 (sm_100), [61,64) swizzle mode 0.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
// Instruction descriptor for kind::i8: D s32 (bits 4-5 = 2), A u8 (bits 7-9 = 0), B s8
// (bits 10-12 = 1), both K-major (bits 15, 16 = 0), N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc_i8(int m, int n) {
    return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr));
}

template <int TN>
struct TcSmem {
    static constexpr int kSlabB = TN * 32;                              // TN tokens x 32 int8
    static constexpr int kOpBytes = 4 * kSlabA + 4 * kSlabB;            // operands of one K tile (4 fields)
    static constexpr int kPackOff = 0;
    static constexpr int kOpOff = kPackStages * kPackStageBytes;
    static constexpr int kBarOff = kOpOff + kOpStages * kOpTiles * kOpBytes;
    static constexpr int kBytes = kBarOff + 256;
};

template <int TN>
__global__ void __launch_bounds__(kThreadsTc, 1) w2a8_gemm_tc_kernel(const TcParams p) {
    using S = TcSmem<TN>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* pack = smem + S::kPackOff;
    uint8_t* ops = smem + S::kOpOff;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBarOff);
    uint64_t* wfull = bars;                       // [kPackStages] packed stage filled (tx bytes)
    uint64_t* wempty = bars + kPackStages;        // [kPackStages] packed stage consumed (8 warps)
    uint64_t* ofull = bars + 2 * kPackStages;     // [kOpStages] operands written (8 warps)
    uint64_t* oempty = ofull + kOpStages;         // [kOpStages] operands consumed (tcgen05.commit)
    uint64_t* accfull = oempty + kOpStages;       // accumulators complete
    uint64_t* bfull = accfull + 1;                // [kOpStages] activation slabs landed (tx bytes; ycanon only)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bfull + kOpStages);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rb = blockIdx.x;                    // 128-row block
    const int tok0 = blockIdx.y * TN;
    const int k_tiles = p.k_tiles;
    const int rg0 = rb * 8;                       // first row group of the block
    const int n_rg = min(8, p.n_rowgroups - rg0); // row groups that exist
    // this CTA's share of K: tiles [kt_lo, kt_lo + nk)
    const int kt_lo = (int)((int64_t)p.k_tiles * blockIdx.z / p.k_splits);
    const int nk = (int)((int64_t)p.k_tiles * (blockIdx.z + 1) / p.k_splits) - kt_lo;

    if (tid == 0) {
        for (int s = 0; s < kPackStages; ++s) {
            bar_init(&wfull[s], 1);
            bar_init(&wempty[s], kWorkerWarps);
        }
        for (int s = 0; s < kOpStages; ++s) {
            bar_init(&ofull[s], kWorkerWarps);
            bar_init(&oempty[s], 1);
            bar_init(&bfull[s], 1);
        }
        bar_init(accfull, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == kMmaWarp) {   // the MMA warp owns the tensor memory: 4 fields x TN columns
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(tmem_slot)),
                     "r"(4 * TN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // Launched as a programmatic dependent: the set-up above and the producer's weight stream
    // (weights are constants) overlap the tail of the preceding kernel; everything that reads
    // or writes activations, sums or outputs waits for that kernel to finish.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    if (warp != kProducerWarp) asm volatile("griddepcontrol.wait;\n" ::: "memory");

    const int n_pack = (nk + kPackTiles - 1) / kPackTiles;
    const int n_os = (nk + kOpTiles - 1) / kOpTiles;      // pipeline steps

    if (warp == kProducerWarp) {
        // ---- producer ---------------------------------------------------------------------
        if (lane == 0) {
            uint64_t w_policy;
            asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(w_policy));
            for (int c = 0; c < n_pack; ++c) {
                const int s = c % kPackStages;
                if (c >= kPackStages && !bar_wait(&wempty[s], ((c / kPackStages) - 1) & 1, abort_flag)) break;
                const int i0 = c * kPackTiles, nt = min(kPackTiles, nk - i0);
                bar_expect_tx(&wfull[s], (uint32_t)(n_rg * nt * kTileBytes));
                for (int r = 0; r < n_rg; ++r)
                    bulk_load_hint(pack + s * kPackStageBytes + r * kPackTiles * kTileBytes,
                                   p.w2t + ((int64_t)(rg0 + r) * k_tiles + kt_lo + i0) * kTileBytes,
                                   (uint32_t)(nt * kTileBytes), &wfull[s], w_policy);
            }
        } else if (lane == 1 && p.ycanon) {
            // the activation slabs of every pipeline step, straight into the operand buffers
            asm volatile("griddepcontrol.wait;\n" ::: "memory");   // written by the preceding kernel
            for (int os = 0; os < n_os; ++os) {
                const int b = os % kOpStages;
                if (os >= kOpStages && !bar_wait(&oempty[b], ((os / kOpStages) - 1) & 1, abort_flag)) break;
                const int tiles = min(kOpTiles, nk - os * kOpTiles);
                bar_expect_tx(&bfull[b], (uint32_t)(tiles * 4 * S::kSlabB));
                for (int kw = 0; kw < tiles; ++kw)
                    for (int j = 0; j < 4; ++j)
                        bulk_load(ops + (b * kOpTiles + kw) * S::kOpBytes + 4 * kSlabA + j * S::kSlabB,
                                  p.ycanon + (((int64_t)(kt_lo + os * kOpTiles + kw) * 4 + j) * p.m_groups + (tok0 >> 3)) * 256,
                                  (uint32_t)S::kSlabB, &bfull[b]);
            }
        }
    } else if (warp == kMmaWarp) {
        // ---- MMA issue ----------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(kRows, TN);
            for (int os = 0; os < n_os; ++os) {
                const int b = os % kOpStages;
                if (!bar_wait(&ofull[b], (os / kOpStages) & 1, abort_flag)) break;
                if (p.ycanon && !bar_wait(&bfull[b], (os / kOpStages) & 1, abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const int tiles = min(kOpTiles, nk - os * kOpTiles);
                for (int kw = 0; kw < tiles; ++kw) {
                    const uint32_t base = smem_addr(ops + (b * kOpTiles + kw) * S::kOpBytes);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t da = umma_desc(base + j * kSlabA, 128, 256);
                        const uint64_t db = umma_desc(base + 4 * kSlabA + j * S::kSlabB, 128, 256);
                        umma_i8(tmem_base + j * TN, da, db, idesc, os > 0 || kw > 0);
                    }
                }
                umma_commit(&oempty[b]);           // frees the operand buffer when these MMAs retire
            }
            umma_commit(accfull);
        }
    } else {
        // ---- unpack + activation staging ------------------------------------------------------
        const int g = lane >> 2, q = lane & 3;
        const int wtid = tid;                      // 0..511 among the workers
        const int rgw = warp & 7, kw_mine = warp >> 3;
        // activations of a step: 2 K tiles x TN tokens x 128 bytes in 16-byte pieces, one step ahead
        constexpr int kPieces = (TN * 8 * kOpTiles) / kWorkerThreads;
        uint4 ynext[kPieces];
        auto load_y = [&](int os) {
#pragma unroll
            for (int i = 0; i < kPieces; ++i) {
                const int piece = wtid + i * kWorkerThreads;
                const int kw = piece / (TN * 8), rest = piece - kw * (TN * 8);
                const int t = rest >> 3, c16 = rest & 7;
                const int kt = os * kOpTiles + kw;
                ynext[i] = make_uint4(0, 0, 0, 0);
                if (tok0 + t < p.M && kt < nk)
                    ynext[i] = *reinterpret_cast<const uint4*>(p.y + (int64_t)(tok0 + t) * p.ldy +
                                                               (int64_t)(kt_lo + kt) * kTileCols + c16 * 16);
            }
        };
        const bool stage_y = p.ycanon == nullptr;
        if (stage_y) load_y(0);
        // cycle counters of warp 0 of CTA (0,0,0) in builds with BITNET_TRACE: a measurement aid behind error_flag
#ifdef BITNET_TRACE
        const bool tracing = p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid == 0;
#else
        constexpr bool tracing = false;
#endif
        long long c_wfull = 0, c_oempty = 0, c_unpack = 0, c_stage = 0, c_fence = 0, c_t = clock64();
        auto lap = [&](long long& acc) {
            if (tracing) {
                const long long t = clock64();
                acc += t - c_t;
                c_t = t;
            }
        };
        for (int os = 0; os < n_os; ++os) {
            const int kt = os * kOpTiles + kw_mine;                // this warp's K tile of the step
            const int c = (os * kOpTiles) / kPackTiles, s = c % kPackStages;
            const int ktl = kt - c * kPackTiles;
            const int b = os % kOpStages;
            uint4 ycur[kPieces];
#pragma unroll
            for (int i = 0; i < kPieces; ++i) ycur[i] = ynext[i];
            if (stage_y) load_y(os + 1);
            lap(c_stage);
            if ((os * kOpTiles) % kPackTiles == 0 && !bar_wait(&wfull[s], (c / kPackStages) & 1, abort_flag)) break;
            lap(c_wfull);
            if (os >= kOpStages && !bar_wait(&oempty[b], ((os / kOpStages) - 1) & 1, abort_flag)) break;
            lap(c_oempty);
            if (rgw < n_rg && kt < nk) {
                uint8_t* opb = ops + (b * kOpTiles + kw_mine) * S::kOpBytes;
                const uint4 wv = *reinterpret_cast<const uint4*>(pack + s * kPackStageBytes +
                                                                 (rgw * kPackTiles + ktl) * kTileBytes + lane * 16);
                const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t msk = 0x03030303u << (2 * j);
#pragma unroll
                    for (int rs = 0; rs < 2; ++rs) {
                        // row 16*rgw + g + 8*rs, field-j columns 8q + 4h + b: words rs (h=0), rs+2 (h=1)
                        const uint2 v = make_uint2(w[rs] & msk, w[rs + 2] & msk);
                        *reinterpret_cast<uint2*>(opb + j * kSlabA + (2 * rgw + rs) * 256 + (q >> 1) * 128 + g * 16 +
                                                  (q & 1) * 8) = v;
                    }
                }
            }
            lap(c_unpack);
#pragma unroll
            for (int i = 0; i < kPieces && stage_y; ++i) {
                const int piece = wtid + i * kWorkerThreads;
                const int kw = piece / (TN * 8), rest = piece - kw * (TN * 8);
                const int t = rest >> 3, c16 = rest & 7;
                const uint4 v = ycur[i];
                const int qq = c16 >> 1, j0 = (c16 & 1) * 2;   // bytes 0-7: field j0, bytes 8-15: field j0+1
                uint8_t* dst = ops + (b * kOpTiles + kw) * S::kOpBytes + 4 * kSlabA + (t >> 3) * 256 + (qq >> 1) * 128 +
                               (t & 7) * 16 + (qq & 1) * 8;
                *reinterpret_cast<uint2*>(dst + j0 * S::kSlabB) = make_uint2(v.x, v.y);
                *reinterpret_cast<uint2*>(dst + (j0 + 1) * S::kSlabB) = make_uint2(v.z, v.w);
            }
            lap(c_stage);
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> tensor core reads
            __syncwarp();
            lap(c_fence);
            if (lane == 0) {
                bar_arrive(&ofull[b]);
                // last step that reads this packed stage
                if (((os + 1) * kOpTiles) % kPackTiles == 0 || os == n_os - 1) bar_arrive(&wempty[s]);
            }
        }

        if (tracing) {
            p.trace[0] = c_wfull; p.trace[1] = c_oempty; p.trace[2] = c_unpack; p.trace[3] = c_stage; p.trace[4] = c_fence;
            p.trace[5] = n_os;
        }
        const long long c_ep0 = clock64();
        // ---- epilogue: all 16 warps; warp w reads TMEM lanes 32*(w%4).., token quarter w/4 ------
        if (bar_wait(accfull, 0, abort_flag)) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int lane_blk = warp & 3, quarter = warp >> 2;
            const int row = rb * kRows + lane_blk * 32 + lane;
            const int sg = segment_of(p.seg, row < p.N ? row : 0);
            const float ws = p.ws_f32 ? p.ws_f32[sg] : (p.ws_bf16 ? __bfloat162float(p.ws_bf16[sg]) : 1.f);
            constexpr int kCols = TN / 4;                 // tokens per warp: 8, 16 or 32
            constexpr int kChunk = kCols < 16 ? 8 : 16;
            // per-token sum(y) and scale of this warp's tokens: lane t holds token t's, shuffles hand them round
            int ys_l = 0;
            float as_l = 1.f;
            {
                const int tok = tok0 + quarter * kCols + lane;
                if (lane < kCols && tok < p.M) {
                    ys_l = p.ysum[tok];
                    as_l = p.a_f32 ? p.a_f32[tok] : (p.a_bf16 ? __bfloat162float(p.a_bf16[tok]) : 1.f);
                }
            }
            // bf16 results leave through shared memory (the operand buffers are free by now): the warp's
            // 32 rows x kCols tokens are written row by row and stored as 16-byte pieces, 64 contiguous
            // bytes per token, instead of one 2-byte store per value.
            const bool vec_out = p.k_splits == 1 && p.out && (p.ldo & 7) == 0 &&
                                 (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 && rb * kRows + kRows <= p.N;
            __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(ops) + warp * (kCols * 32);
#pragma unroll 1
            for (int cb = quarter * kCols; cb < (quarter + 1) * kCols; cb += kChunk) {
                int c0[16], c1[16], c2[16], c3[16];
                const uint32_t ta = tmem_base + ((uint32_t)(lane_blk * 32) << 16) + cb;
                if (kChunk == 16) {
                    tmem_ld16(ta, c0); tmem_ld16(ta + TN, c1); tmem_ld16(ta + 2 * TN, c2); tmem_ld16(ta + 3 * TN, c3);
                } else {
                    tmem_ld8(ta, c0); tmem_ld8(ta + TN, c1); tmem_ld8(ta + 2 * TN, c2); tmem_ld8(ta + 3 * TN, c3);
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                for (int e = 0; e < kChunk; ++e) {
                    const int tl = cb - quarter * kCols + e;          // token within the warp's share
                    const int tok = tok0 + cb + e;
                    const int ysum_e = __shfl_sync(0xffffffffu, ys_l, tl);
                    const float a_e = __shfl_sync(0xffffffffu, as_l, tl);
                    int v = c0[e] + (c1[e] >> 2) + (c2[e] >> 4) + (c3[e] >> 6);
                    if (p.k_splits > 1) {      // partial sum over this CTA's K share
                        if (tok < p.M && row < p.N) atomicAdd(&p.acc_ws[(int64_t)tok * p.N + row], v);
                        continue;
                    }
                    v -= ysum_e;
                    const __nv_bfloat16 o = __float2bfloat16_rn((float)v / a_e * ws);
                    if (vec_out) {
                        stg[tl * 32 + lane] = o;
                    } else if (tok < p.M && row < p.N) {
                        if (p.out) p.out[(int64_t)tok * p.ldo + row] = o;
                    }
                    if (p.acc_out && tok < p.M && row < p.N) p.acc_out[(int64_t)tok * p.N + row] = v;
                }
            }
            if (vec_out) {
                __syncwarp();
#pragma unroll
                for (int it = 0; it < kCols / 8; ++it) {
                    const int tl = it * 8 + (lane >> 2), part = lane & 3;
                    const int tok = tok0 + quarter * kCols + tl;
                    if (tok < p.M) {
                        const uint4 v = *reinterpret_cast<const uint4*>(stg + tl * 32 + part * 8);
                        *reinterpret_cast<uint4*>(p.out + (int64_t)tok * p.ldo + rb * kRows + lane_blk * 32 + part * 8) = v;
                    }
                }
            }
        }
        if (tracing) p.trace[6] = clock64() - c_ep0;
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(4 * TN) : "memory");
    }
    if (tid == 0 && *abort_flag) atomicExch(p.error_flag, 3);
}

// Second pass of a split-K launch: subtract sum(y), rescale, store, and clear the work space.
// blockIdx.y = token; a thread takes four consecutive rows (one 16-byte load of sums, one
// 8-byte store of results) when the row count and the pointers allow it.
__global__ void __launch_bounds__(256) tc_finalize_kernel(const TcParams p) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");   // the partial sums of the preceding kernel
    const int tok = blockIdx.y;
    const int ysum = p.ysum[tok];
    // (the scales may be absent when only the integer sums are wanted)
    const float a = !p.out ? 1.f : (p.a_f32 ? p.a_f32[tok] : (p.a_bf16 ? __bfloat162float(p.a_bf16[tok]) : 1.f));
    int32_t* acc = p.acc_ws + (int64_t)tok * p.N;
    auto scale_of = [&](int row) -> float {
        const int sg = segment_of(p.seg, row);
        return p.ws_f32 ? p.ws_f32[sg] : (p.ws_bf16 ? __bfloat162float(p.ws_bf16[sg]) : 1.f);
    };
    const bool vec = p.N % 4 == 0 && (!p.out || (p.ldo % 4 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 7) == 0)) &&
                     (reinterpret_cast<uintptr_t>(p.acc_ws) & 15) == 0 &&
                     (!p.acc_out || (reinterpret_cast<uintptr_t>(p.acc_out) & 15) == 0);
    if (vec) {
        for (int row = (blockIdx.x * 256 + threadIdx.x) * 4; row < p.N; row += gridDim.x * 256 * 4) {
            int4 v = *reinterpret_cast<const int4*>(acc + row);
            *reinterpret_cast<int4*>(acc + row) = make_int4(0, 0, 0, 0);
            v.x -= ysum; v.y -= ysum; v.z -= ysum; v.w -= ysum;
            if (p.acc_out) *reinterpret_cast<int4*>(p.acc_out + (int64_t)tok * p.N + row) = v;
            if (p.out) {
                const float w0 = scale_of(row), w3 = scale_of(row + 3);
                const float w1 = w0 == w3 ? w0 : scale_of(row + 1), w2 = w0 == w3 ? w0 : scale_of(row + 2);
                const __nv_bfloat162 lo = __floats2bfloat162_rn((float)v.x / a * w0, (float)v.y / a * w1);
                const __nv_bfloat162 hi = __floats2bfloat162_rn((float)v.z / a * w2, (float)v.w / a * w3);
                uint2 o;
                o.x = *reinterpret_cast<const unsigned int*>(&lo);
                o.y = *reinterpret_cast<const unsigned int*>(&hi);
                *reinterpret_cast<uint2*>(p.out + (int64_t)tok * p.ldo + row) = o;
            }
        }
        return;
    }
    for (int row = blockIdx.x * 256 + threadIdx.x; row < p.N; row += gridDim.x * 256) {
        const int v = acc[row] - ysum;
        acc[row] = 0;
        if (p.acc_out) p.acc_out[(int64_t)tok * p.N + row] = v;
        if (p.out) p.out[(int64_t)tok * p.ldo + row] = __float2bfloat16_rn((float)v / a * scale_of(row));
    }
}

// Activations [M, ldy] (rows zero filled up to a multiple of 128 columns) into the operand
// layout described at TcParams::ycanon.  One thread per 16-byte piece of a row.
__global__ void __launch_bounds__(256) restage_kernel(const int8_t* __restrict__ y, int64_t ldy, uint8_t* __restrict__ out,
                                                      int M, int k_tiles, int m_groups) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int64_t n = (int64_t)M * k_tiles * 8;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
        const int c16 = (int)(i & 7);
        const int64_t r = i >> 3;
        const int kt = (int)(r % k_tiles), t = (int)(r / k_tiles);
        const uint4 v = *reinterpret_cast<const uint4*>(y + (int64_t)t * ldy + (int64_t)kt * kTileCols + c16 * 16);
        const int qq = c16 >> 1, j0 = (c16 & 1) * 2;   // bytes 0-7: field j0, bytes 8-15: field j0 + 1
        uint8_t* dst = out + (((int64_t)kt * 4 + j0) * m_groups + (t >> 3)) * 256 + (qq >> 1) * 128 + (t & 7) * 16 + (qq & 1) * 8;
        *reinterpret_cast<uint2*>(dst) = make_uint2(v.x, v.y);
        *reinterpret_cast<uint2*>(dst + (int64_t)m_groups * 256) = make_uint2(v.z, v.w);
    }
}

template <int TN>
cudaError_t launch_tc(const TcParams& p, cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(w2a8_gemm_tc_kernel<TN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TcSmem<TN>::kBytes + 1024);
    if (e != cudaSuccess) return e;
    if (p.ycanon) {
        const int64_t pieces = (int64_t)p.M * p.k_tiles * 8;
        const int blocks = (int)((pieces + 255) / 256 < 4736 ? (pieces + 255) / 256 : 4736);
        restage_kernel<<<blocks, 256, 0, stream>>>(p.y, p.ldy, const_cast<uint8_t*>(p.ycanon), p.M, p.k_tiles, p.m_groups);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    // Both kernels are launched as programmatic dependents of whatever precedes them in the stream.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((p.N + kRows - 1) / kRows), (unsigned)((p.M + TN - 1) / TN), (unsigned)p.k_splits);
    cfg.blockDim = dim3(kThreadsTc);
    cfg.dynamicSmemBytes = TcSmem<TN>::kBytes + 1024;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, w2a8_gemm_tc_kernel<TN>, p);
    if (e != cudaSuccess) return e;
    if (p.k_splits > 1 && !p.defer_finalize) {
        const int bx = (p.N + 1023) / 1024;   // four rows per thread
        cfg.gridDim = dim3((unsigned)(bx < 64 ? bx : 64), (unsigned)p.M);
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = 0;
        e = cudaLaunchKernelEx(&cfg, tc_finalize_kernel, p);
        if (e != cudaSuccess) return e;
    }
    return cudaGetLastError();
}

}  // namespace

// y must be 16-byte aligned with ldy % 16 == 0 and readable up to ceil128(K) columns (zero
// filled beyond K); ysum is required.
int w2a8_gemm_tc(const LinearArgs& a, int* error_flag, int32_t* acc_ws, size_t acc_ws_ints, int n_sm,
                 cudaStream_t stream) {
    TcParams p{};
    p.w2t = static_cast<const uint8_t*>(a.w2t);
    p.y = a.y; p.ldy = a.ldy; p.ysum = a.ysum;
    p.acc_out = a.acc_out; p.out = a.out; p.ldo = a.ldo;
    p.a_f32 = a.a_f32; p.a_bf16 = a.a_bf16; p.ws_f32 = a.ws_f32; p.ws_bf16 = a.ws_bf16;
    p.seg = a.seg;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.k_tiles = (a.K + kTileCols - 1) / kTileCols;
    p.n_rowgroups = (a.N + 15) / 16;
    p.error_flag = error_flag;
#ifdef BITNET_TRACE
    p.trace = reinterpret_cast<unsigned long long*>(error_flag + 16);   // spare words behind the flag
#endif
    // Few output tiles (decode-sized M): split K over enough CTAs to occupy the SMs.
    const int tn = a.M <= 32 ? 32 : (a.M <= 64 ? 64 : 128);
    const int tiles = ((a.N + kRows - 1) / kRows) * ((a.M + tn - 1) / tn);
    int ks = n_sm / (tiles > 0 ? tiles : 1);
    if (ks > p.k_tiles / 2) ks = p.k_tiles / 2;          // at least two K tiles per CTA
    if (ks < 1 || !acc_ws || (size_t)a.M * a.N > acc_ws_ints) ks = 1;
    p.k_splits = ks;
    p.acc_ws = acc_ws;
    if (a.sums) {
        // the caller finalises: the sums stay in the work space (raw partial sums with split K; with
        // one CTA per output tile the epilogue stores them there with sum(y) already taken off)
        if (!acc_ws || (size_t)a.M * a.N > acc_ws_ints) return set_status(kTooLarge), kTooLarge;
        p.defer_finalize = true;
        p.out = nullptr;
        p.acc_out = ks > 1 ? nullptr : acc_ws;
        *a.sums = acc_ws;
        *a.sums_raw = ks > 1;
    }
    // Many tokens: lay the activations out for the tensor core once, instead of in every CTA.
    if (a.M >= 128) {
        p.m_groups = (a.M + 127) / 128 * 16;
        p.ycanon = workspace_tc_activations((size_t)p.m_groups * 8 * p.k_tiles * kTileCols, stream);
    }
    cudaError_t e;
    if (a.M <= 32) e = launch_tc<32>(p, stream);
    else if (a.M <= 64) e = launch_tc<64>(p, stream);
    else e = launch_tc<128>(p, stream);
    return check_cuda(e);
}

}  // namespace bitnet
