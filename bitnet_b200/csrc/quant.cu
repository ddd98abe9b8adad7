// Activation prologue of a BitLinear: optional RMSNorm, then per-token absmax int8
// quantisation (gpu/model.py:68-71 with the norms of :159-160, :195-196, :237-242 in
// front).  One CTA per token.  Arithmetic is f32; the normalised value is rounded to bf16
// before quantising because the reference's norm returns bf16.
//     a = 127 / max(absmax, 1e-5);  y = clamp(rint(x * a), -128, 127);  ysum = sum(y)
#include "common.cuh"
#include "kernels.h"

namespace bitnet {

namespace {

constexpr int kQThreads = 256;

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, t) : v + t;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float r = sh[0];
    for (int i = 1; i < kQThreads / 32; ++i) r = is_max ? fmaxf(r, sh[i]) : r + sh[i];
    return r;
}

__device__ __forceinline__ int block_reduce_int(int v, int* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    int r = 0;
    for (int i = 0; i < kQThreads / 32; ++i) r += sh[i];
    return r;
}

__global__ void __launch_bounds__(kQThreads) act_quant_kernel(const QuantArgs p) {
    __shared__ float sh[kQThreads / 32];
    __shared__ int shi[kQThreads / 32];
    const int tok = blockIdx.x;
    const __nv_bfloat16* xb = p.x_bf16 ? p.x_bf16 + (int64_t)tok * p.ldx : nullptr;
    const float* xf = p.x_f32 ? p.x_f32 + (int64_t)tok * p.ldx : nullptr;
    auto load = [&](int k) -> float { return xb ? __bfloat162float(xb[k]) : xf[k]; };

    float rinv = 1.f;
    if (p.gamma) {
        float ss = 0.f;
        for (int k = threadIdx.x; k < p.K; k += kQThreads) {
            const float v = load(k);
            ss += v * v;
        }
        ss = block_reduce(ss, false, sh);
        rinv = rsqrtf(ss / (float)p.K + p.eps);
    }
    auto value = [&](int k) -> float {
        float v = load(k);
        if (p.gamma) v = bf16_round(v * rinv * __bfloat162float(p.gamma[k]));
        return v;
    };

    float mx = 0.f;
    for (int k = threadIdx.x; k < p.K; k += kQThreads) mx = fmaxf(mx, fabsf(value(k)));
    mx = block_reduce(mx, true, sh);
    const float a = 127.0f / fmaxf(mx, 1e-5f);

    int8_t* y = p.y + (int64_t)tok * p.ldy;
    int s = 0;
    for (int k = threadIdx.x; k < p.ldy; k += kQThreads) {
        int v = 0;
        if (k < p.K) {
            float f = rintf(value(k) * a);
            f = fminf(fmaxf(f, -128.f), 127.f);
            v = (int)f;
        }
        y[k] = (int8_t)v;
        s += v;
    }
    s = block_reduce_int(s, shi);
    if (threadIdx.x == 0) {
        if (p.a_f32) p.a_f32[tok] = a;
        if (p.a_bf16) p.a_bf16[tok] = __float2bfloat16_rn(a);
        if (p.ysum) p.ysum[tok] = s;
    }
}

}  // namespace

int act_quant(const QuantArgs& a, cudaStream_t stream) {
    act_quant_kernel<<<a.M, kQThreads, 0, stream>>>(a);
    return check_cuda(cudaGetLastError());
}

}  // namespace bitnet
