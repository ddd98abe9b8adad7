// Activation prologue of a BitLinear, shared by the stand-alone quantisation kernel and
// the fused decode kernels so that both produce bit-identical int8 activations:
// (optional) RMSNorm -> round to bf16 -> absmax -> a = 127 / max(absmax, 1e-5)
// -> y = clamp(rint(x * a), -128, 127), following gpu/model.py:68-71 behind the norms of
// gpu/model.py:159-160, 195-196, 237-242.  Executed by exactly 256 threads per token;
// thread t owns the 8-element groups t, t + 256, ... in every pass, so the result does not
// depend on which kernel runs it.
#pragma once
#include "common.cuh"

namespace bitnet {

constexpr int kPrologueThreads = 256;

struct Vec8 {
    float v[8];
};

__device__ __forceinline__ Vec8 unpack_bf16x8(const uint4& u) {
    Vec8 r;
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        r.v[2 * e] = __low2float(h[e]);
        r.v[2 * e + 1] = __high2float(h[e]);
    }
    return r;
}

__device__ __forceinline__ uint4 pack_bf16x8(const Vec8& x) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(x.v[2 * e], x.v[2 * e + 1]);
    return u;
}

// Eight consecutive bf16 values starting at element k of a row of length K (zero beyond K).
__device__ __forceinline__ Vec8 load_bf16x8(const __nv_bfloat16* row, int k, int K, bool vec_ok) {
    if (vec_ok && k + 8 <= K) return unpack_bf16x8(*reinterpret_cast<const uint4*>(row + k));
    Vec8 r;
#pragma unroll
    for (int e = 0; e < 8; ++e) r.v[e] = (k + e < K) ? __bfloat162float(row[k + e]) : 0.f;
    return r;
}

__device__ __forceinline__ bool aligned16(const void* p, int64_t ld_elems, int elem_bytes) {
    return ((reinterpret_cast<uintptr_t>(p) & 15) == 0) && ((ld_elems * elem_bytes) % 16 == 0);
}

// Sum or max over the 256 threads.  `sync` is a barrier over exactly those threads.
template <class Sync>
__device__ __forceinline__ float reduce_256(float v, bool is_max, float* scratch, int tid, Sync sync) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, t) : v + t;
    }
    sync();
    if ((tid & 31) == 0) scratch[tid >> 5] = v;
    sync();
    float r = scratch[0];
#pragma unroll
    for (int i = 1; i < kPrologueThreads / 32; ++i) r = is_max ? fmaxf(r, scratch[i]) : r + scratch[i];
    return r;
}

// Sum of `ss` and max of `mx` over the 256 threads in one round (two barriers).  `scratch`
// holds 16 floats.
template <class Sync>
__device__ __forceinline__ void reduce2_256(float& ss, float& mx, float* scratch, int tid, Sync sync) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    sync();
    if ((tid & 31) == 0) {
        scratch[tid >> 5] = ss;
        scratch[8 + (tid >> 5)] = mx;
    }
    sync();
    ss = scratch[0];
    mx = scratch[8];
#pragma unroll
    for (int i = 1; i < kPrologueThreads / 32; ++i) {
        ss += scratch[i];
        mx = fmaxf(mx, scratch[8 + i]);
    }
}

// One token whose source values already sit in shared memory: xv holds ceil8(K) bf16 values
// (zero beyond K).  y: destination row of k_pad bytes (shared or global), zero filled beyond
// K.  Arithmetic, in f32: t = x * g; r = rsqrt(mean(x^2) + eps); xn = bf16(t * r);
// a = 127 / max(max|xn|, 1e-5); y = clamp(rint(xn * a), -128, 127).  Because rounding and
// multiplication by r > 0 are monotone, max|xn| = bf16(max|t| * r), so one reduction round
// (sum of squares and max|t| together) and two passes suffice.  On return every thread holds
// the activation scale; `sy_warp` is the sum of y over the calling warp's elements (exact in
// f32), which the caller adds up over the eight warps.  The loops are deliberately not
// unrolled: these kernels run for microseconds, and code that does not fit the instruction
// cache costs more than the loop overhead saves.
template <class Sync>
__device__ __forceinline__ void norm_quant_row(const __nv_bfloat16* xv, int K, int k_pad, const __nv_bfloat16* gamma,
                                               float eps, int8_t* y, float* scratch, int tid, Sync sync, float& a_out,
                                               float& sy_warp) {
    const int n_vec = (K + 7) / 8;
    const bool g_vec = gamma && aligned16(gamma, 8, 2);
    float ss = 0.f, mt = 0.f;
#pragma unroll 1
    for (int v = tid; v < n_vec; v += kPrologueThreads) {
        const Vec8 x = unpack_bf16x8(*reinterpret_cast<const uint4*>(xv + v * 8));
        Vec8 g;
        if (gamma) g = load_bf16x8(gamma, v * 8, K, g_vec);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            ss += x.v[e] * x.v[e];
            mt = fmaxf(mt, fabsf(gamma ? x.v[e] * g.v[e] : x.v[e]));
        }
    }
    reduce2_256(ss, mt, scratch, tid, sync);
    const float rinv = gamma ? rsqrtf(ss / (float)K + eps) : 1.f;
    const float amax = gamma ? bf16_round(mt * rinv) : mt;
    const float a = 127.0f / fmaxf(amax, 1e-5f);
    float sy = 0.f;
#pragma unroll 1
    for (int v = tid; v < k_pad / 8; v += kPrologueThreads) {
        uint32_t lo = 0, hi = 0;
        if (v < n_vec) {
            const Vec8 x = unpack_bf16x8(*reinterpret_cast<const uint4*>(xv + v * 8));
            Vec8 g;
            if (gamma) g = load_bf16x8(gamma, v * 8, K, g_vec);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float xn = gamma ? bf16_round(x.v[e] * g.v[e] * rinv) : x.v[e];
                float f = rintf(xn * a);
                f = fminf(fmaxf(f, -128.f), 127.f);
                sy += f;
                const uint32_t b = (uint32_t)(uint8_t)(int8_t)(int)f;
                if (e < 4) lo |= b << (8 * e);
                else hi |= b << (8 * (e - 4));
            }
        }
        *reinterpret_cast<uint2*>(y + v * 8) = make_uint2(lo, hi);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sy += __shfl_xor_sync(0xffffffffu, sy, o);
    a_out = a;
    sy_warp = sy;
}

}  // namespace bitnet
