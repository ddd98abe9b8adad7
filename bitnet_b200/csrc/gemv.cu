// W2A8 BitLinear for decode-sized batches: ternary 2-bit weights (W2T layout) times int8
// activations, int32 accumulation, rescale to bf16.  Replaces the reference's
// ladder_int8xint2_kernel (gpu/bitnet_kernels/bitnet_kernels.h:46-83), which covers M == 1
// and ten fixed shapes; this kernel takes any M, any N and K.
//
// The kernel is bound by HBM traffic on the packed weights.  Per 16 weights a thread
// spends one AND per 32-bit operand word and one quarter of an integer tensor-core MMA
// (mma.sync m16n8k32 u8 x s8): the four 2-bit fields of a byte are separated by masks
// only, without shifts, by accumulating field j in its own accumulator (which then holds
// 4^j times the true sum) and folding the four with exact arithmetic shifts at the end.
#include "common.cuh"
#include "kernels.h"

namespace bitnet {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

struct GemvParams {
    const uint4* w;          // W2T tiles
    const int8_t* y;         // [M, ldy] int8 activations
    int64_t ldy;
    const int32_t* ysum;     // [M] sum of each token's int8 activations, or null (computed here)
    int32_t* acc_out;        // [M, N] int32 sum (weight * y), or null
    __nv_bfloat16* out;      // [M, ldo] bf16, or null
    int64_t ldo;
    const float* a_f32;      // [M] activation scales (127/absmax) as f32, or null
    const __nv_bfloat16* a_bf16;  // same as bf16 (the reference's `s`); used when a_f32 is null
    int a_stride;            // 1, or 0 to apply a[0] to every token (the reference reads s[0] only)
    const float* ws_f32;     // weight scale per segment as f32, or null
    const __nv_bfloat16* ws_bf16;
    ScaleSegments seg;
    int M, N, K;
    int k_tiles;             // ceil(K / 128)
};

// Loads the 32 activation bytes [k0, k0+32) of one token as eight words, zero beyond K.
__device__ __forceinline__ void load_act32(const int8_t* row, int k0, int K, bool vec_ok, uint32_t (&b)[8]) {
    if (vec_ok && k0 + 32 <= K) {
        const uint4 v0 = *reinterpret_cast<const uint4*>(row + k0);
        const uint4 v1 = *reinterpret_cast<const uint4*>(row + k0 + 16);
        b[0] = v0.x; b[1] = v0.y; b[2] = v0.z; b[3] = v0.w;
        b[4] = v1.x; b[5] = v1.y; b[6] = v1.z; b[7] = v1.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t w = 0;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int k = k0 + 4 * i + c;
                if (k < K) w |= (uint32_t)(uint8_t)row[k] << (8 * c);
            }
            b[i] = w;
        }
    }
}

// MB = number of 8-token blocks a CTA covers.  FOUR = keep one accumulator per 2-bit field
// (mask-only unpack); otherwise shift each field down and use one accumulator.
template <int MB, bool FOUR, bool COMPUTE_YSUM>
__global__ void __launch_bounds__(kThreads) w2a8_gemv_kernel(const GemvParams p) {
    constexpr int NC = FOUR ? 4 : 1;
    __shared__ int red[kWarps][16][8 * MB + 1];
    __shared__ int red_ysum[kWarps][8 * MB];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int row_group = blockIdx.x;
    const int tok0 = blockIdx.y * (8 * MB);
    // Launched as a programmatic dependent: the activations may be the predecessor's output, the
    // weights are constants.  The first tiles of every warp (most of a row group for K up to a few
    // thousand) are therefore requested before the wait, while the predecessor still runs.
    constexpr int U = 4;   // weight tiles in flight per warp
    const uint4* wrow = p.w + (int64_t)row_group * p.k_tiles * 32 + lane;
    uint4 wv[U];
    uint64_t w_policy;      // weights are read once per call: first out of L2
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(w_policy));
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int kt = warp + u * kWarps;
        if (kt < p.k_tiles) wv[u] = ldg_stream_hint(wrow + (int64_t)kt * 32, w_policy);
    }
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");

    int acc[NC][MB][4];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int nb = 0; nb < MB; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[c][nb][i] = 0;
    int ys[MB];
#pragma unroll
    for (int nb = 0; nb < MB; ++nb) ys[nb] = 0;

    const bool vec_ok = (p.ldy % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0);

    for (int kt0 = warp; kt0 < p.k_tiles; kt0 += kWarps * U) {
        if (kt0 != warp) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int kt = kt0 + u * kWarps;
                if (kt < p.k_tiles) wv[u] = ldg_stream_hint(wrow + (int64_t)kt * 32, w_policy);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kt = kt0 + u * kWarps;
            if (kt >= p.k_tiles) continue;
            const uint32_t w[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
#pragma unroll
            for (int nb = 0; nb < MB; ++nb) {
                const int tok = tok0 + 8 * nb + g;
                uint32_t b[8];
                if (tok < p.M) {
                    load_act32(p.y + (int64_t)tok * p.ldy, kt * kTileCols + 32 * q, p.K, vec_ok, b);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) b[i] = 0;
                }
                if (COMPUTE_YSUM) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) ys[nb] = __dp4a((int)b[i], 0x01010101, ys[nb]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (FOUR) {
                        const uint32_t m = 0x03030303u << (2 * j);
                        mma_u8s8(acc[j][nb], w[0] & m, w[1] & m, w[2] & m, w[3] & m, b[2 * j], b[2 * j + 1]);
                    } else {
                        mma_u8s8(acc[0][nb], (w[0] >> (2 * j)) & 0x03030303u, (w[1] >> (2 * j)) & 0x03030303u,
                                 (w[2] >> (2 * j)) & 0x03030303u, (w[3] >> (2 * j)) & 0x03030303u, b[2 * j],
                                 b[2 * j + 1]);
                    }
                }
            }
        }
    }

    // Fold the per-field accumulators (exact: accumulator j is a multiple of 4^j), then
    // reduce over the four warps that split K.
#pragma unroll
    for (int nb = 0; nb < MB; ++nb) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int v = acc[0][nb][i];
            if (FOUR) v += (acc[1][nb][i] >> 2) + (acc[2][nb][i] >> 4) + (acc[3][nb][i] >> 6);
            const int r = g + 8 * (i >> 1), t = 8 * nb + 2 * q + (i & 1);
            red[warp][r][t] = v;
        }
        if (COMPUTE_YSUM) {
            int v = ys[nb];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (q == 0) red_ysum[warp][8 * nb + g] = v;
        }
    }
    __syncthreads();

    for (int idx = threadIdx.x; idx < 16 * 8 * MB; idx += kThreads) {
        const int t = idx / 16, r = idx % 16;          // consecutive threads -> consecutive rows
        const int tok = tok0 + t, row = row_group * 16 + r;
        if (tok >= p.M || row >= p.N) continue;
        int v = red[0][r][t] + red[1][r][t] + red[2][r][t] + red[3][r][t];
        int s;
        if (COMPUTE_YSUM) s = red_ysum[0][t] + red_ysum[1][t] + red_ysum[2][t] + red_ysum[3][t];
        else s = p.ysum[tok];
        v -= s;                                        // fields hold weight + 1
        if (p.acc_out) p.acc_out[(int64_t)tok * p.N + row] = v;
        if (p.out) {
            const float a = p.a_f32 ? p.a_f32[tok * p.a_stride] : __bfloat162float(p.a_bf16[tok * p.a_stride]);
            const int sg = segment_of(p.seg, row);
            const float ws = p.ws_f32 ? p.ws_f32[sg] : __bfloat162float(p.ws_bf16[sg]);
            // same operation order as gpu/bitnet_kernels/bitnet_kernels.h:82
            p.out[(int64_t)tok * p.ldo + row] = __float2bfloat16_rn((float)v / a * ws);
        }
    }
}

// Both kernels of this file are launched as programmatic dependents of whatever precedes them
// in the stream: the launch and the set-up overlap the predecessor's tail.
template <class Kernel, class Params>
cudaError_t launch_pdl(Kernel kernel, dim3 grid, dim3 block, cudaStream_t stream, const Params& p) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

template <int MB, bool FOUR>
cudaError_t launch(const GemvParams& p, cudaStream_t stream) {
    const dim3 grid((unsigned)((p.N + 15) / 16), (unsigned)((p.M + 8 * MB - 1) / (8 * MB)));
    if (p.ysum) return launch_pdl(w2a8_gemv_kernel<MB, FOUR, false>, grid, dim3(kThreads), stream, p);
    return launch_pdl(w2a8_gemv_kernel<MB, FOUR, true>, grid, dim3(kThreads), stream, p);
}

// sum_k y[m, k] per token, one warp per token: for callers of the tensor-core kernel that hand
// over plain int8 rows without their sums (the reference's bitlinear_int8xint2 arguments).
struct RowSumParams {
    const int8_t* y;
    int64_t ldy;
    int32_t* ysum;
    int M, K;
};
__global__ void __launch_bounds__(256) row_sum_kernel(const RowSumParams p) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int tok = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (tok >= p.M) return;
    const uint4* row = reinterpret_cast<const uint4*>(p.y + (int64_t)tok * p.ldy);   // 16-byte aligned, K % 16 == 0
    int s = 0;
    for (int v = lane; v < p.K / 16; v += 32) {
        const uint4 u = row[v];
        s = __dp4a((int)u.x, 0x01010101, s);
        s = __dp4a((int)u.y, 0x01010101, s);
        s = __dp4a((int)u.z, 0x01010101, s);
        s = __dp4a((int)u.w, 0x01010101, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) p.ysum[tok] = s;
}

}  // namespace

int w2a8_gemv(const LinearArgs& a, cudaStream_t stream) {
    // Decode-sized batches of already quantised activations: measured on B200, the direct-load
    // kernel below is the faster one for almost every shape (13824 x 2560: 5.2 vs 8.4 us at M = 1,
    // 5.4 vs 13.7 us at M = 8; 65536 x 10240: 43 vs 68 us, 61 % of the measured copy bandwidth) -
    // the fused kernel earns its keep inside the decode chain, where it also does the prologue and
    // overlaps its predecessor.  It stays ahead for one or two tokens on short, wide matrices
    // (2560 x 6912: 6.7 vs 8.2 us), where the direct kernel has too few row groups to fill the SMs.
    if (a.M <= 2 && a.K % 8 == 0 && a.K >= 2 * a.N && a.N <= 4096) {
        const int rc = fused_linear_quantized(a, stream);
        if (rc != kTooLarge) return rc;
        set_status(kOk);   // does not fit the fused kernel's shared memory: the direct kernel takes it
    }
    // Larger batches go to the tcgen05 kernel when the activations are laid out for it.
    const int64_t k_pad = (a.K + kTileCols - 1) / kTileCols * kTileCols;
    if (a.M >= 16 && a.ldy % 16 == 0 && a.ldy >= k_pad && (reinterpret_cast<uintptr_t>(a.y) & 15) == 0) {
        WorkspaceView ws;
        if (!workspace_view(&ws)) return kCudaError;
        if (a.ysum) return w2a8_gemm_tc(a, ws.error_flag, ws.tc_acc, ws.tc_acc_ints, ws.n_sm, stream);
        if ((size_t)a.M <= ws.ysum_ints) {
            // plain int8 rows without their sums (the arguments of the reference's symbol): one
            // small kernel adds them up into the workspace, then the same tensor-core path
            const RowSumParams rp{a.y, a.ldy, ws.ysum, a.M, (int)k_pad};
            if (check_cuda(launch_pdl(row_sum_kernel, dim3((unsigned)((a.M + 7) / 8)), dim3(256), stream, rp)))
                return kCudaError;
            LinearArgs b = a;
            b.ysum = ws.ysum;
            return w2a8_gemm_tc(b, ws.error_flag, ws.tc_acc, ws.tc_acc_ints, ws.n_sm, stream);
        }
    }
    GemvParams p;
    p.w = reinterpret_cast<const uint4*>(a.w2t);
    p.y = a.y; p.ldy = a.ldy; p.ysum = a.ysum;
    p.acc_out = a.acc_out; p.out = a.out; p.ldo = a.ldo;
    p.a_f32 = a.a_f32; p.a_bf16 = a.a_bf16; p.a_stride = a.a_stride;
    p.ws_f32 = a.ws_f32; p.ws_bf16 = a.ws_bf16; p.seg = a.seg;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.k_tiles = (a.K + kTileCols - 1) / kTileCols;
    cudaError_t e;
    // The mask-only unpack scales the top field by 64: |sum| stays below 2^31 for K <= 65536.
    const bool four_ok = a.K <= 65536;
    if (a.M <= 8 && four_ok) e = launch<1, true>(p, stream);
    else if (a.M <= 8) e = launch<1, false>(p, stream);
    else if (a.M <= 16 && four_ok) e = launch<2, true>(p, stream);
    else if (a.M <= 16) e = launch<2, false>(p, stream);
    else if (a.M <= 32) e = launch<4, false>(p, stream);
    else e = launch<8, false>(p, stream);
    return check_cuda(e);
}

}  // namespace bitnet
