// Stand-alone activation prologue of a BitLinear: optional gating (squared ReLU times the
// second half of the row), optional RMSNorm, then per-token absmax int8 quantisation (gpu/model.py:68-71 behind the norms of :159-160, :195-196, :237-242).
// One CTA of 256 threads per token; the arithmetic lives in prologue.cuh, shared with the
// fused decode kernels.
#include "common.cuh"
#include "kernels.h"
#include "prologue.cuh"

namespace bitnet {

namespace {

__global__ void __launch_bounds__(kPrologueThreads) act_quant_kernel(const QuantArgs p) {
    extern __shared__ __align__(16) uint8_t smem_q[];
    __shared__ double red_d[8];
    __shared__ float red_f[8];
    __shared__ int sy_part[kPrologueThreads / 32];
    __nv_bfloat16* xv = reinterpret_cast<__nv_bfloat16*>(smem_q);
    const int tok = blockIdx.x, tid = threadIdx.x;
    // launched as a programmatic dependent: the launch overlaps the tail of the kernel that
    // produces x
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const __nv_bfloat16* row = p.x_bf16 + (int64_t)tok * p.ldx;
    const bool vec_ok = aligned16(p.x_bf16, p.ldx, 2);
    const int K = p.K;
    float a;
    int sy_warp;
    if (p.lin_acc) {
        // x += rescaled sums of the preceding BitLinear (K % 8 == 0 and aligned rows: checked by the host)
        int32_t* acc = p.lin_acc + (int64_t)tok * K;
        const int ys = p.lin_ysum ? p.lin_ysum[tok] : 0;
        const float la = p.lin_a[tok];
        __nv_bfloat16* hrow = const_cast<__nv_bfloat16*>(row);
#pragma unroll 1
        for (int v = tid; v < K / 8; v += kPrologueThreads) {
            const int4 s0 = *reinterpret_cast<const int4*>(acc + v * 8), s1 = *reinterpret_cast<const int4*>(acc + v * 8 + 4);
            *reinterpret_cast<int4*>(acc + v * 8) = make_int4(0, 0, 0, 0);
            *reinterpret_cast<int4*>(acc + v * 8 + 4) = make_int4(0, 0, 0, 0);
            const int sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            Vec8 x = unpack_bf16x8(*reinterpret_cast<const uint4*>(hrow + v * 8));
#pragma unroll
            for (int e = 0; e < 8; ++e) x.v[e] = bf16_round(x.v[e] + bf16_round((float)(sv[e] - ys) / la * p.lin_ws));
            const uint4 packed = pack_bf16x8(x);
            *reinterpret_cast<uint4*>(hrow + v * 8) = packed;
            *reinterpret_cast<uint4*>(xv + v * 8) = packed;
        }
        if (!p.y) return;
        __syncthreads();
    }
#pragma unroll 1
    for (int v = tid; v < (K + 7) / 8 && !p.lin_acc; v += kPrologueThreads) {
        Vec8 x = load_bf16x8(row, v * 8, K, vec_ok);
        if (p.glu) {   // relu(x1)^2 * x3 with bf16 rounding after each step, as the bf16 tensor ops round
            const Vec8 x3 = load_bf16x8(row + K, v * 8, K, vec_ok && K % 8 == 0);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float t = fmaxf(x.v[e], 0.f);
                x.v[e] = bf16_round(bf16_round(t * t) * x3.v[e]);
            }
        }
        *reinterpret_cast<uint4*>(xv + v * 8) = pack_bf16x8(x);
    }
    norm_quant_row(xv, K, (int)p.ldy, p.gamma, p.eps, p.y + (int64_t)tok * p.ldy, red_d, red_f, tid,
                   [] { __syncthreads(); }, a, sy_warp);
    if ((tid & 31) == 0) sy_part[tid >> 5] = sy_warp;
    __syncthreads();
    int ysum = 0;
    for (int i = 0; i < kPrologueThreads / 32; ++i) ysum += sy_part[i];
    if (tid == 0) {
        if (p.a_f32) p.a_f32[tok] = a;
        if (p.a_bf16) p.a_bf16[tok] = __float2bfloat16_rn(a);
        if (p.ysum) p.ysum[tok] = ysum;
    }
}

}  // namespace

int act_quant(const QuantArgs& a, cudaStream_t stream) {
    const size_t smem = (size_t)((a.K + 7) / 8) * 16;
    if (smem > 200 * 1024) {
        set_status(kTooLarge);
        return kTooLarge;
    }
    if (smem > 48 * 1024) {   // per device, so set whenever it is needed
        cudaError_t e = cudaFuncSetAttribute(act_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return check_cuda(e);
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.M);
    cfg.blockDim = dim3(kPrologueThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, act_quant_kernel, a));
}

}  // namespace bitnet
