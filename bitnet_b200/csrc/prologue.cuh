// Activation prologue of a BitLinear, shared by the stand-alone quantisation kernel and
// the fused decode kernels so that both produce bit-identical int8 activations:
// (optional) RMSNorm -> round to bf16 -> absmax -> a = 127 / max(absmax, 1e-5)
// -> y = clamp(rint(x * a), -128, 127), following gpu/model.py:68-71 behind the norms of
// gpu/model.py:159-160, 195-196, 237-242.
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

// clamp(rint(f), -128, 127) as one conversion: round to nearest even, saturate to int8
// (the low byte of the result is the quantised value; NaN gives 0).
__device__ __forceinline__ int quant_s8(float f) {
    int q;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(f));
    return q;
}
// The low bytes of four integers as one word (a in the lowest byte).
__device__ __forceinline__ uint32_t pack_bytes(int a, int b, int c, int d) {
    return __byte_perm(__byte_perm((uint32_t)a, (uint32_t)b, 0x0040), __byte_perm((uint32_t)c, (uint32_t)d, 0x0040), 0x5410);
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

// Sum of `ss` (double) and max of `mx` over NT threads in one round (two barriers).
// `sd` holds NT / 32 doubles, `sf` NT / 32 floats.
template <int NT, class Sync>
__device__ __forceinline__ void reduce_stats(double& ss, float& mx, double* sd, float* sf, int tid, Sync sync) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    sync();
    if ((tid & 31) == 0) {
        sd[tid >> 5] = ss;
        sf[tid >> 5] = mx;
    }
    sync();
    ss = sd[0];
    mx = sf[0];
#pragma unroll
    for (int i = 1; i < NT / 32; ++i) {
        ss += sd[i];
        mx = fmaxf(mx, sf[i]);
    }
}

// ---- the arithmetic of one token, shared by every kernel that quantises activations ----------
// t = x * g (f32); r = 1 / sqrt(sum(x^2) / K + eps) with the sum accumulated in double precision,
// rounded to f32 once, and the rest in correctly rounded f32 operations; xn = bf16(t * r);
// a = 127 / max(max|xn|, 1e-5); y = clamp(rint(xn * a), -128, 127).
// Because rounding and multiplication by r > 0 are monotone, max|xn| = bf16(max|t| * r), so one
// reduction round (sum of squares and max|t| together) and two passes over the values suffice.
//
// The sum of squares is accumulated in double precision (B200 runs it at half the f32 rate, and
// a token has a few thousand values): its f32 rounding then does not depend on the order of the
// additions, so every kernel - whatever its thread count, and however a producer kernel cut the
// vector into slices - derives the same r, and r equals what the CPU checker derives from a
// double-precision sum.  A quantiser turns a last-bit difference in r into different int8 values; this removes
// that source of divergence between kernels, between GPUs of a tensor-parallel group, and
// between the GPU and the CPU checker.

// Adds the squares of a group to ss and folds max |x * g| (max |x| without norm weight) into m.
__device__ __forceinline__ void group_stats(const Vec8& x, const Vec8& g, bool use_g, double& ss, float& m) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        ss = fma((double)x.v[e], (double)x.v[e], ss);
        m = fmaxf(m, fabsf(use_g ? x.v[e] * g.v[e] : x.v[e]));
    }
}
// From the reduced statistics to the normalisation factor and the activation scale.
__device__ __forceinline__ void finish_stats(double ss, float mt, int K, float eps, bool use_g, float& rinv, float& a) {
    // the sum rounded to f32 once, then IEEE f32 operations (each correctly rounded, so a CPU
    // evaluation in f32 gives the same bits): r = 1 / sqrt(sum / K + eps)
    rinv = use_g ? __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn((float)ss, (float)K), eps))) : 1.f;
    const float amax = use_g ? bf16_round(mt * rinv) : mt;
    a = 127.0f / fmaxf(amax, 1e-5f);
}
// The eight int8 values of a group (two words) and their sum added to sy.
__device__ __forceinline__ uint2 quant_group(const Vec8& x, const Vec8& g, bool use_g, float rinv, float a, int& sy) {
    int q[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float xn = use_g ? bf16_round(x.v[e] * g.v[e] * rinv) : x.v[e];
        q[e] = quant_s8(xn * a);
    }
    const uint32_t lo = pack_bytes(q[0], q[1], q[2], q[3]), hi = pack_bytes(q[4], q[5], q[6], q[7]);
    sy = __dp4a((int)lo, 0x01010101, sy);
    sy = __dp4a((int)hi, 0x01010101, sy);
    return make_uint2(lo, hi);
}

// One token whose source values already sit in shared memory, by 256 threads: xv holds ceil8(K)
// bf16 values (zero beyond K).  y: destination row of k_pad bytes (shared or global), zero
// filled beyond K.  On return every thread holds the activation scale; `sy_warp` is the sum of
// y over the calling warp's elements, which the caller adds up over the eight warps.  `sd` holds
// 8 doubles, `sf` 8 floats.  The loops are deliberately not unrolled: these kernels run for
// microseconds, and code that does not fit the instruction cache costs more than the loop
// overhead saves.
// GVEC: gamma is 16-byte aligned and padded to whole groups of 8 (e.g. staged in shared memory),
// so the element-wise fallback is left out of the code.
template <bool GVEC = false, class Sync>
__device__ __forceinline__ void norm_quant_row(const __nv_bfloat16* xv, int K, int k_pad, const __nv_bfloat16* gamma,
                                               float eps, int8_t* y, double* sd, float* sf, int tid, Sync sync,
                                               float& a_out, int& sy_warp) {
    const int n_vec = (K + 7) / 8;
    const bool use_g = gamma != nullptr;
    const bool g_vec = GVEC || (use_g && aligned16(gamma, 8, 2));
    auto load_g = [&](int v) -> Vec8 {
        if (!use_g) return Vec8{};
        return GVEC ? unpack_bf16x8(*reinterpret_cast<const uint4*>(gamma + v * 8)) : load_bf16x8(gamma, v * 8, K, g_vec);
    };
    double ss = 0.0;
    float mt = 0.f;
#pragma unroll 1
    for (int v = tid; v < n_vec; v += kPrologueThreads)
        group_stats(unpack_bf16x8(*reinterpret_cast<const uint4*>(xv + v * 8)), load_g(v), use_g, ss, mt);
    reduce_stats<kPrologueThreads>(ss, mt, sd, sf, tid, sync);
    float rinv, a;
    finish_stats(ss, mt, K, eps, use_g, rinv, a);
    int sy_i = 0;
#pragma unroll 1
    for (int v = tid; v < k_pad / 8; v += kPrologueThreads) {
        uint2 w = make_uint2(0, 0);
        if (v < n_vec) w = quant_group(unpack_bf16x8(*reinterpret_cast<const uint4*>(xv + v * 8)), load_g(v), use_g, rinv, a, sy_i);
        *reinterpret_cast<uint2*>(y + v * 8) = w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sy_i += __shfl_xor_sync(0xffffffffu, sy_i, o);
    a_out = a;
    sy_warp = sy_i;
}

}  // namespace bitnet
