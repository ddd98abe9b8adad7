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

// One token whose source values already sit in shared memory: xv holds ceil8(K) bf16
// values (zero beyond K).  y: destination row of k_pad bytes (shared or global), zero filled
// beyond K.  On return every thread holds the token's activation scale and sum(y).  The
// loops are deliberately not unrolled: these kernels run for microseconds, and code that
// does not fit the instruction cache costs more than the loop overhead saves.
// reduce(v, is_max, scratch, tid) must return the sum / max of v over the 256 threads, in
// the order reduce_256 defines.
template <class Reduce>
__device__ __forceinline__ void norm_quant_row(__nv_bfloat16* xv, int K, int k_pad, const __nv_bfloat16* gamma,
                                               float eps, int8_t* y, float* scratch, int tid, Reduce reduce,
                                               float& a_out, int& ysum_out) {
    const int n_vec = (K + 7) / 8;
    const bool g_vec = gamma && aligned16(gamma, 8, 2);
    float ss = 0.f, mx = 0.f;
#pragma unroll 1
    for (int v = tid; v < n_vec; v += kPrologueThreads) {
        const Vec8 x = unpack_bf16x8(*reinterpret_cast<const uint4*>(xv + v * 8));
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            ss += x.v[e] * x.v[e];
            mx = fmaxf(mx, fabsf(x.v[e]));
        }
    }
    if (gamma) {
        ss = reduce(ss, false, scratch, tid);
        const float rinv = rsqrtf(ss / (float)K + eps);
        mx = 0.f;
#pragma unroll 1
        for (int v = tid; v < n_vec; v += kPrologueThreads) {
            Vec8 x = unpack_bf16x8(*reinterpret_cast<const uint4*>(xv + v * 8));
            const Vec8 g = load_bf16x8(gamma, v * 8, K, g_vec);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                x.v[e] = bf16_round(x.v[e] * rinv * g.v[e]);
                mx = fmaxf(mx, fabsf(x.v[e]));
            }
            *reinterpret_cast<uint4*>(xv + v * 8) = pack_bf16x8(x);
        }
    }
    mx = reduce(mx, true, scratch, tid);
    const float a = 127.0f / fmaxf(mx, 1e-5f);
    float sy = 0.f;
#pragma unroll 1
    for (int v = tid; v < k_pad / 8; v += kPrologueThreads) {
        uint32_t lo = 0, hi = 0;
        if (v < n_vec) {
            const Vec8 x = unpack_bf16x8(*reinterpret_cast<const uint4*>(xv + v * 8));
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float f = rintf(x.v[e] * a);
                f = fminf(fmaxf(f, -128.f), 127.f);
                sy += f;
                const uint32_t b = (uint32_t)(uint8_t)(int8_t)(int)f;
                if (e < 4) lo |= b << (8 * e);
                else hi |= b << (8 * (e - 4));
            }
        }
        *reinterpret_cast<uint2*>(y + v * 8) = make_uint2(lo, hi);
    }
    sy = reduce(sy, false, scratch, tid);   // exact: |sum| < 2^24
    a_out = a;
    ysum_out = (int)sy;
}

}  // namespace bitnet
