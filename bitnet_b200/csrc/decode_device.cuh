// Device code shared by the decode kernels (decode_fused.cu, decode_chain.cu): PTX helpers,
// the split-KV attention body and the output-head body.
#pragma once
#include <type_traits>
#include "common.cuh"
#include "decode_fused.h"
#include "prologue.cuh"

namespace bitnet {

namespace {

constexpr long long kWaitCycles = 2000000000LL;           // about one second: then give up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and the caller abandons the kernel) after about a second.
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > kWaitCycles) return false;
    }
    return true;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    return mbar_test_wait(bar, parity) || mbar_wait_slow(bar, parity);   // usually complete already
}
// Weight tiles are read once per step and a step's weights are many times the L2: they are marked
// evict-first so that what is read again soon (KV cache rows, activations, statistics) stays.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_evict_last_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(pol));
    return pol;
}
// 16-byte load through L2 (the data was written by other SMs) that asks L2 to keep the line:
// KV cache rows, which every step reads again.
__device__ __forceinline__ uint4 ldcg_keep(const uint4* p, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.cg.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(policy)
                 : "memory");
    return v;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// ---- tensor-parallel exchange (see TpPeers and TpTag in decode_fused.h) ------------------------
constexpr long long kPeerWaitCycles = 600000000LL;       // default limit of a wait for another rank: about 0.3 s

__device__ __forceinline__ unsigned int tp_tag(const TpTag& t) {
    return (unsigned int)(__ldcg(t.step) * t.mul + t.add);
}
// One packet into (possibly another rank's) memory: a single 8-byte store, nothing to follow it.
__device__ __forceinline__ void tp_put(void* addr, unsigned int value, unsigned int tag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};\n" ::"l"(addr), "r"(value), "r"(tag) : "memory");
}
// Reads a packet of this rank's area once it carries `tag`.  False after the time limit (the caller
// records kErrPeerWait and carries on with whatever is there, so that the kernel ends and the host
// can read the error word).
__device__ __forceinline__ bool tp_get(const void* addr, unsigned int tag, long long limit_cycles, unsigned int& value) {
    unsigned int v, t;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];\n" : "=r"(v), "=r"(t) : "l"(addr) : "memory");
    if (t != tag) {
        const long long t0 = clock64();
        do {
            if (clock64() - t0 > limit_cycles) { value = v; return false; }
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];\n" : "=r"(v), "=r"(t) : "l"(addr) : "memory");
        } while (t != tag);
    }
    value = v;
    return true;
}
// A rank's statistics of one token to slot [rank][m] of every rank's area.
__device__ __forceinline__ void tp_put_stats(const TpPeers& tp, size_t off, int M, int m, double ss, float mx, unsigned int tag) {
    const unsigned long long b = (unsigned long long)__double_as_longlong(ss);
#pragma unroll 1
    for (int pr = 0; pr < tp.size; ++pr) {
        TpStatPackets* dst = reinterpret_cast<TpStatPackets*>(tp.area[pr] + off) + (size_t)tp.rank * M + m;
        tp_put(&dst->w[0], (unsigned int)b, tag);
        tp_put(&dst->w[2], (unsigned int)(b >> 32), tag);
        tp_put(&dst->w[4], __float_as_uint(mx), tag);
    }
}
// One volatile 8-byte load of a packet (no waiting).
__device__ __forceinline__ void tp_peek(const void* addr, unsigned int& value, unsigned int& tag) {
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];\n" : "=r"(value), "=r"(tag) : "l"(addr) : "memory");
}
// All ranks' statistics of token m from this rank's area, added in the order of the ranks (the same
// sum on every rank).  First a pass that requests every packet without waiting - one memory
// latency when they have all arrived, the usual case for all but the last rank to finish - and,
// only if a tag was missing, a second pass that waits packet by packet.  False if a packet did not
// arrive in time.
__device__ __forceinline__ bool tp_get_stats(const TpStatPackets* slots, int size, int M, int m, unsigned int tag,
                                             long long limit_cycles, double& ss, float& mx) {
    bool all = true;
    ss = 0.0;
    mx = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxTp; ++r) {
        if (r < size) {
            const TpStatPackets* src = slots + (size_t)r * M + m;
            unsigned int lo, hi, mb, t0, t1, t2;
            tp_peek(&src->w[0], lo, t0);
            tp_peek(&src->w[2], hi, t1);
            tp_peek(&src->w[4], mb, t2);
            all = all && t0 == tag && t1 == tag && t2 == tag;
            ss += __longlong_as_double((long long)(((unsigned long long)hi << 32) | lo));
            mx = fmaxf(mx, __uint_as_float(mb));
        }
    }
    if (all) return true;
    bool ok = true;
    ss = 0.0;
    mx = 0.f;
#pragma unroll 1
    for (int r = 0; r < size; ++r) {
        const TpStatPackets* src = slots + (size_t)r * M + m;
        unsigned int lo, hi, mb;
        ok = tp_get(&src->w[0], tag, limit_cycles, lo) && ok;
        ok = tp_get(&src->w[2], tag, limit_cycles, hi) && ok;
        ok = tp_get(&src->w[4], tag, limit_cycles, mb) && ok;
        ss += __longlong_as_double((long long)(((unsigned long long)hi << 32) | lo));
        mx = fmaxf(mx, __uint_as_float(mb));
    }
    return ok;
}

// One thread per CTA, after a CTA barrier: counts the CTA in on a ticket in this GPU's own memory
// and returns true for the last of n_cta, which then speaks for the whole grid to the other ranks
// (this GPU's share of the statistics is added up in its own memory first: atomics of many CTAs on
// one address in another GPU's memory are served one NVLink round trip after the other).
__device__ __forceinline__ bool tp_last_cta(unsigned int* ticket, unsigned int n_cta) {
    __threadfence();
    const unsigned int t = atomicAdd(ticket, 1u);
    if (t + 1 != n_cta) return false;
    atomicExch(ticket, 0u);          // every CTA has drawn: ready for the kernel's next launch
    __threadfence();
    return true;
}

// bf16( float(acc) / a * ws ): the rescale of gpu/bitnet_kernels/bitnet_kernels.h:82
__device__ __forceinline__ float lin_out(int acc, float a, float ws) { return bf16_round(__fdiv_rn((float)acc, a) * ws); }

// ---------------------------------------------------------------------------------------
// Attention for one new token per sequence: RoPE on q and k, append k, v to the cache,
// softmax(q k^T) v over one slice of the cache per CTA (flash-decoding split); the CTA that
// finishes a (sequence, kv head) last combines the slices.  A warp walks keys four at a time,
// a lane owns 4 dims.
// ---------------------------------------------------------------------------------------
template <int GMAX>
struct AttnCfg {
    static constexpr int kWarps = GMAX <= 4 ? 16 : 4;   // bounded by registers (the tensor-core key loop wants 4)
    static constexpr int kThreads = kWarps * 32;
};

// Number of KV slices for a context of P cached keys when at most s_max are available.  The
// split costs a second pass (partials through memory, a ticket, a combine), which only pays
// off once a single CTA would walk the keys for longer than that.
__device__ __forceinline__ int attention_slices(int s_max, int P) { return P <= 384 ? 1 : min(s_max, (P + 64) / 64); }

// Which part of the attention CTA number x of a sequence takes, x in [0, Hkv * s_max).  With a
// single slice every query head gets its own CTA (the scores of one head need a quarter of the
// shuffles); with several slices a CTA takes all query heads of a kv head for one slice.
struct AttnItem {
    int kvh, h0, G, split, S;   // G = 0: nothing to do
};
__device__ __forceinline__ AttnItem attention_item(const AttentionParams& p, int x, int P) {
    const int Gfull = p.H / p.Hkv;
    // Groups of more than four query heads at head_dim 128 always go as whole groups (the
    // tensor-core key loop of the chain's kernel), in slices of 64 keys or more.
    const bool whole_groups = p.D == 128 && Gfull > 4 && p.S > 1;
    const int S = whole_groups ? (P <= 64 ? 1 : min(p.S, (P + 63) / 64)) : attention_slices(p.S, P);
    AttnItem it{0, 0, 0, 0, S};
    if (!whole_groups && S == 1 && p.S >= Gfull) {
        if (x < p.H) { it.kvh = x / Gfull; it.h0 = x - it.kvh * Gfull; it.G = 1; }
    } else {
        it.kvh = x / p.S; it.split = x - it.kvh * p.S;
        if (it.split < S) it.G = Gfull;
    }
    return it;
}

// The key loop of the split-KV body on tensor cores, for head_dim 128 and up to 16 query heads
// per kv head: the heads of the group are the 16 rows of m16n8k16 bf16 MMAs (rows beyond G are
// zero), a warp takes 16 keys per step.  S = Q K^T: the dot product over the 128 dims may be summed
// in any order of the dims, so a lane loads the 16-byte pieces of a key row that it can use as B
// fragments directly - piece i*4 + q of key g for lane 4g+q - and Q's A fragments are arranged to
// match.  O += P V: the B fragment wants two keys' values of one dim in a register; a lane loads
// 32 contiguous bytes of its four keys and pairs them with byte permutes, the dims being assigned
// to the MMA's columns so that those loads are contiguous.  P is rounded to bf16 for the second
// product (as flash attention kernels do), sums and maxima stay in f32.  Leaves each warp's
// (max, sum, unnormalised output) where the scalar body leaves them.
//   q_s [G][128] rotated queries (bf16 values, not yet scaled); knew / vnew: the new token's key and
//   value (bf16 values), attended by warp 0 when with_new; ck / cv: row 0 of this (sequence, kv head).
template <int NW, int GMAX>
__device__ __forceinline__ void attention_keys_mma(const float* q_s, int G, const float* knew, const float* vnew, bool with_new,
                                                   const __nv_bfloat16* ck, const __nv_bfloat16* cv, int64_t key_stride, int lo,
                                                   int hi, int warp, int lane, float* red_m, float* red_l, float* red_o) {
    constexpr int D = 128;
    const int g = lane >> 2, q = lane & 3;
    const float scale = rsqrtf((float)D);
    auto pack = [](float lo_v, float hi_v) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo_v, hi_v);
        return *reinterpret_cast<const uint32_t*>(&h);
    };
    // A fragments of Q: k-step 2i+h covers dims i*32 + q*8 + h*4 .. +3 for this lane
    uint32_t qa[8][4];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const int d = (s >> 1) * 32 + q * 8 + (s & 1) * 4;
        const float* r0 = q_s + g * D + d;
        const float* r1 = q_s + (g + 8) * D + d;
        const bool v0 = g < G, v1 = g + 8 < G;
        qa[s][0] = v0 ? pack(r0[0], r0[1]) : 0u;
        qa[s][2] = v0 ? pack(r0[2], r0[3]) : 0u;
        qa[s][1] = v1 ? pack(r1[0], r1[1]) : 0u;
        qa[s][3] = v1 ? pack(r1[2], r1[3]) : 0u;
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;     // rows g and g+8
    float o[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) { o[nt][0] = 0.f; o[nt][1] = 0.f; o[nt][2] = 0.f; o[nt][3] = 0.f; }

#pragma unroll 1
    for (int j0 = lo + warp * 16; j0 < hi; j0 += NW * 16) {
        uint4 kk[2][4], vv[4][2];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int key = j0 + t * 8 + g;
            const uint4* src = reinterpret_cast<const uint4*>(ck + (int64_t)key * key_stride) + q;
#pragma unroll
            for (int i = 0; i < 4; ++i) kk[t][i] = key < hi ? src[i * 4] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int key = j0 + (x >> 1) * 8 + 2 * q + (x & 1);
            const uint4* src = reinterpret_cast<const uint4*>(cv + (int64_t)key * key_stride) + g;
#pragma unroll
            for (int j = 0; j < 2; ++j) vv[x][j] = key < hi ? src[j * 8] : make_uint4(0, 0, 0, 0);
        }
        float s[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            s[t][0] = 0.f; s[t][1] = 0.f; s[t][2] = 0.f; s[t][3] = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                mma_bf16(s[t], qa[2 * i], kk[t][i].x, kk[t][i].y);
                mma_bf16(s[t], qa[2 * i + 1], kk[t][i].z, kk[t][i].w);
            }
        }
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[t][c] = (j0 + t * 8 + 2 * q + (c & 1) < hi) ? s[t][c] * scale : -INFINITY;
        float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);          // finite: key j0 is inside the slice
        const float c0 = __expf(m0 - mn0), c1 = __expf(m1 - mn1);
        m0 = mn0; m1 = mn1;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            s[t][0] = __expf(s[t][0] - mn0); s[t][1] = __expf(s[t][1] - mn0);
            s[t][2] = __expf(s[t][2] - mn1); s[t][3] = __expf(s[t][3] - mn1);
        }
        l0 = l0 * c0 + (s[0][0] + s[0][1]) + (s[1][0] + s[1][1]);
        l1 = l1 * c1 + (s[0][2] + s[0][3]) + (s[1][2] + s[1][3]);
        const uint32_t pa[4] = {pack(s[0][0], s[0][1]), pack(s[0][2], s[0][3]), pack(s[1][0], s[1][1]), pack(s[1][2], s[1][3])};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t wa[4] = {vv[0][j].x, vv[0][j].y, vv[0][j].z, vv[0][j].w};
            const uint32_t wb[4] = {vv[1][j].x, vv[1][j].y, vv[1][j].z, vv[1][j].w};
            const uint32_t wc[4] = {vv[2][j].x, vv[2][j].y, vv[2][j].z, vv[2][j].w};
            const uint32_t wd[4] = {vv[3][j].x, vv[3][j].y, vv[3][j].z, vv[3][j].w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int nt = j * 8 + e;
                const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(wa[e >> 1], wb[e >> 1], sel);
                const uint32_t b1 = __byte_perm(wc[e >> 1], wd[e >> 1], sel);
                o[nt][0] *= c0; o[nt][1] *= c0; o[nt][2] *= c1; o[nt][3] *= c1;
                mma_bf16(o[nt], pa, b0, b1);
            }
        }
    }
    if (with_new && warp == 0) {     // the new token attends to itself: one more key, from shared memory
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const int d = (s >> 1) * 32 + q * 8 + (s & 1) * 4;
            const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[s][0]));
            const float2 a2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[s][2]));
            const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[s][1]));
            const float2 a3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[s][3]));
            s0 += a0.x * knew[d] + a0.y * knew[d + 1] + a2.x * knew[d + 2] + a2.y * knew[d + 3];
            s1 += a1.x * knew[d] + a1.y * knew[d + 1] + a3.x * knew[d + 2] + a3.y * knew[d + 3];
        }
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
        s0 += __shfl_xor_sync(0xffffffffu, s0, 2); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        s0 *= scale; s1 *= scale;
        const float mn0 = fmaxf(m0, s0), mn1 = fmaxf(m1, s1);
        const float c0 = __expf(m0 - mn0), c1 = __expf(m1 - mn1);
        const float p0 = __expf(s0 - mn0), p1 = __expf(s1 - mn1);
        m0 = mn0; m1 = mn1;
        l0 = l0 * c0 + (q == 0 ? p0 : 0.f);          // the lanes' sums are added up below
        l1 = l1 * c1 + (q == 0 ? p1 : 0.f);
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            const int d = ((nt >> 3) * 8 + 2 * q) * 8 + (nt & 7);
            o[nt][0] = o[nt][0] * c0 + p0 * vnew[d]; o[nt][1] = o[nt][1] * c0 + p0 * vnew[d + 8];
            o[nt][2] = o[nt][2] * c1 + p1 * vnew[d]; o[nt][3] = o[nt][3] * c1 + p1 * vnew[d + 8];
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (q == 0) {
        if (g < G) { red_m[warp * GMAX + g] = m0; red_l[warp * GMAX + g] = l0; }
        if (g + 8 < G) { red_m[warp * GMAX + g + 8] = m1; red_l[warp * GMAX + g + 8] = l1; }
    }
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
        const int d = ((nt >> 3) * 8 + 2 * q) * 8 + (nt & 7);
        if (g < G) { red_o[(warp * G + g) * D + d] = o[nt][0]; red_o[(warp * G + g) * D + d + 8] = o[nt][1]; }
        if (g + 8 < G) { red_o[(warp * G + g + 8) * D + d] = o[nt][2]; red_o[(warp * G + g + 8) * D + d + 8] = o[nt][3]; }
    }
}

// The same loop for groups of at most 8 query heads, within 128 registers per thread (so that it
// can run inside a 512-thread CTA): only rows 0..7 of the MMAs are kept - the other half of every
// accumulator goes to two scratch registers - and the values are requested after the scores have
// been issued instead of together with the keys.
template <int NW, int GMAX, bool kEager>
__device__ __forceinline__ void attention_keys_mma8(const float* q_s, int G, const float* knew, const float* vnew, bool with_new,
                                                    const __nv_bfloat16* ck, const __nv_bfloat16* cv, int64_t key_stride, int lo,
                                                    int hi, int warp, int lane, float* red_m, float* red_l, float* red_o) {
    constexpr int D = 128;
    const int g = lane >> 2, q = lane & 3;
    const float scale = rsqrtf((float)D);
    auto pack = [](float lo_v, float hi_v) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo_v, hi_v);
        return *reinterpret_cast<const uint32_t*>(&h);
    };
    auto mma_half = [](float& d0, float& d1, float& j0, float& j1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};\n"
            : "+f"(d0), "+f"(d1), "+f"(j0), "+f"(j1)
            : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
    };
    uint32_t qa[8][2];                       // rows g (a0, a2); rows g+8 are zero
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const int d = (s >> 1) * 32 + q * 8 + (s & 1) * 4;
        const float* r0 = q_s + g * D + d;
        const bool v0 = g < G;
        qa[s][0] = v0 ? pack(r0[0], r0[1]) : 0u;
        qa[s][1] = v0 ? pack(r0[2], r0[3]) : 0u;
    }
    float m0 = -INFINITY, l0 = 0.f;
    float jk[4][2] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};   // the unused halves; four pairs keep four MMAs independent
    float o[16][2];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) { o[nt][0] = 0.f; o[nt][1] = 0.f; }

#pragma unroll 1
    for (int k0 = lo + warp * 16; k0 < hi; k0 += NW * 16) {
        float s[2][2];
        // kEager (CTAs of their own, 170 registers): every load of the step is issued before the first
        // is used, as in the 16-row loop.  Otherwise halves one after the other: registers.
        uint4 kkE[kEager ? 2 : 1][4], vvE[kEager ? 4 : 1][2];
        if constexpr (kEager) {
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int key = k0 + t * 8 + g;
                const uint4* src = reinterpret_cast<const uint4*>(ck + (int64_t)key * key_stride) + q;
#pragma unroll
                for (int i = 0; i < 4; ++i) kkE[t][i] = key < hi ? src[i * 4] : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int key = k0 + (x >> 1) * 8 + 2 * q + (x & 1);
                const uint4* src = reinterpret_cast<const uint4*>(cv + (int64_t)key * key_stride) + g;
#pragma unroll
                for (int j = 0; j < 2; ++j) vvE[x][j] = key < hi ? src[j * 8] : make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            uint4 kk[4];
            const int key = k0 + t * 8 + g;
            const uint4* src = reinterpret_cast<const uint4*>(ck + (int64_t)key * key_stride) + q;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if constexpr (kEager) kk[i] = kkE[t][i];
                else kk[i] = key < hi ? src[i * 4] : make_uint4(0, 0, 0, 0);
            }
            s[t][0] = 0.f; s[t][1] = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                mma_half(s[t][0], s[t][1], jk[2 * t][0], jk[2 * t][1], qa[2 * i][0], qa[2 * i][1], kk[i].x, kk[i].y);
                mma_half(s[t][0], s[t][1], jk[2 * t][0], jk[2 * t][1], qa[2 * i + 1][0], qa[2 * i + 1][1], kk[i].z, kk[i].w);
            }
        }
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int c = 0; c < 2; ++c) s[t][c] = (k0 + t * 8 + 2 * q + c < hi) ? s[t][c] * scale : -INFINITY;
        float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        const float mn0 = fmaxf(m0, mx0);                               // finite: key k0 is inside the slice
        const float c0 = __expf(m0 - mn0);
        m0 = mn0;
#pragma unroll
        for (int t = 0; t < 2; ++t) { s[t][0] = __expf(s[t][0] - mn0); s[t][1] = __expf(s[t][1] - mn0); }
        l0 = l0 * c0 + (s[0][0] + s[0][1]) + (s[1][0] + s[1][1]);
        const uint32_t pa0 = pack(s[0][0], s[0][1]), pa2 = pack(s[1][0], s[1][1]);
        // the values, in two halves of 64 dims (registers): 16 bytes of each of the lane's four keys
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint4 vv[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int key = k0 + (x >> 1) * 8 + 2 * q + (x & 1);
                const uint4* src = reinterpret_cast<const uint4*>(cv + (int64_t)key * key_stride) + g;
                if constexpr (kEager) vv[x] = vvE[x][j];
                else vv[x] = key < hi ? src[j * 8] : make_uint4(0, 0, 0, 0);
            }
            const uint32_t wa[4] = {vv[0].x, vv[0].y, vv[0].z, vv[0].w};
            const uint32_t wb[4] = {vv[1].x, vv[1].y, vv[1].z, vv[1].w};
            const uint32_t wc[4] = {vv[2].x, vv[2].y, vv[2].z, vv[2].w};
            const uint32_t wd[4] = {vv[3].x, vv[3].y, vv[3].z, vv[3].w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int nt = j * 8 + e;
                const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(wa[e >> 1], wb[e >> 1], sel);
                const uint32_t b1 = __byte_perm(wc[e >> 1], wd[e >> 1], sel);
                o[nt][0] *= c0; o[nt][1] *= c0;
                mma_half(o[nt][0], o[nt][1], jk[nt & 3][0], jk[nt & 3][1], pa0, pa2, b0, b1);
            }
        }
    }
    if (with_new && warp == 0) {     // the new token attends to itself: one more key, from shared memory
        float s0 = 0.f;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const int d = (s >> 1) * 32 + q * 8 + (s & 1) * 4;
            const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[s][0]));
            const float2 a2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[s][1]));
            s0 += a0.x * knew[d] + a0.y * knew[d + 1] + a2.x * knew[d + 2] + a2.y * knew[d + 3];
        }
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
        s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s0 *= scale;
        const float mn0 = fmaxf(m0, s0);
        const float c0 = __expf(m0 - mn0), p0 = __expf(s0 - mn0);
        m0 = mn0;
        l0 = l0 * c0 + (q == 0 ? p0 : 0.f);          // the lanes' sums are added up below
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            const int d = ((nt >> 3) * 8 + 2 * q) * 8 + (nt & 7);
            o[nt][0] = o[nt][0] * c0 + p0 * vnew[d];
            o[nt][1] = o[nt][1] * c0 + p0 * vnew[d + 8];
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    if (q == 0 && g < G) { red_m[warp * GMAX + g] = m0; red_l[warp * GMAX + g] = l0; }
    if (g < G) {
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            const int d = ((nt >> 3) * 8 + 2 * q) * 8 + (nt & 7);
            red_o[(warp * G + g) * D + d] = o[nt][0];
            red_o[(warp * G + g) * D + d + 8] = o[nt][1];
        }
    }
}

// Attention of query heads h0 .. h0+G-1 of kv head kvh of sequence b over KV slice `split` of S,
// by NW warps, with P keys already in the cache (the caller reads p.pos[b]; the body does not).
// A subset of the heads (G < H / Hkv) is only allowed with S = 1.  `smem` needs
// attention_smem() bytes; `sync` is a barrier over the NW * 32 participating threads.
// The first keys of the slice are requested before `wait()`, which returns once the new token's
// q, k, v (xqkv) are visible: the cache rows and the positions must not change meanwhile.
// Returns true when this CTA wrote p.out for its heads (always with S == 1; with several slices
// only the CTA that combined them).
template <int GMAX, int NW, bool kMma = false, bool kEager = false, class Sync, class Wait>
__device__ __forceinline__ bool attention_body(const AttentionParams& p, uint8_t* smem, int* is_last_s, int b, int kvh,
                                               int h0, int G, int split, int S, int P, int tid, Sync sync, Wait wait) {
    constexpr int NT = NW * 32;
    const int warp = tid >> 5, lane = tid & 31;
    const int D = p.D, Gfull = p.H / p.Hkv;
    float* q_s = reinterpret_cast<float*>(smem);          // [G][D]
    float* knew = q_s + G * D;                             // [D]
    float* vnew = knew + D;                                // [D]
    float* red_m = vnew + D;                               // [NW][GMAX]
    float* red_l = red_m + NW * GMAX;                      // [NW][GMAX]
    float* red_o = red_l + NW * GMAX;                      // [NW][G][D]
    // keys per step: their scores are reduced together, then one softmax update
    constexpr int U = 4;
    const int lo = (int)((int64_t)P * split / S), hi = (int)((int64_t)P * (split + 1) / S);
    const int d0 = 4 * lane;
    const bool live = d0 < D;
    const __nv_bfloat16* ck = p.cache_k + ((int64_t)b * p.L * p.Hkv + kvh) * D + d0;
    const __nv_bfloat16* cv = p.cache_v + ((int64_t)b * p.L * p.Hkv + kvh) * D + d0;
    const int64_t key_stride = (int64_t)p.Hkv * D;
    uint2 kr[U], vr[U];
    auto request = [&](int j0) {   // raw rows of keys j0 .. j0+U-1 (zero beyond the slice)
#pragma unroll
        for (int u = 0; u < U; ++u) {
            kr[u] = make_uint2(0, 0); vr[u] = make_uint2(0, 0);
            if (j0 + u < hi && live) {
                kr[u] = *reinterpret_cast<const uint2*>(ck + (j0 + u) * key_stride);
                vr[u] = *reinterpret_cast<const uint2*>(cv + (j0 + u) * key_stride);
            }
        }
    };
    if constexpr (!kMma) request(lo + warp * U);
    wait();
    const __nv_bfloat16* x = p.xqkv + (int64_t)b * p.ld_qkv;
    const float* rope = p.rope + (int64_t)P * D;           // [D/2][2] cos, sin of position P
    const float qscale = rsqrtf((float)D);
    // vectors: G query heads, then k, then v; pairs (2i, 2i+1) rotate together
#pragma unroll 4
    for (int idx = tid; idx < (G + 2) * (D / 2); idx += NT) {
        const int vec = idx / (D / 2), i = idx - vec * (D / 2);
        int col;
        if (vec < G) col = (kvh * Gfull + h0 + vec) * D;
        else if (vec == G) col = p.H * D + kvh * D;
        else col = (p.H + p.Hkv) * D + kvh * D;
        const unsigned int xx = __ldcg(reinterpret_cast<const unsigned int*>(x + col + 2 * i));   // L2: written by other SMs
        float x0 = __uint_as_float(xx << 16), x1 = __uint_as_float(xx & 0xffff0000u);
        if (vec <= G) {
            const float cs = rope[2 * i], sn = rope[2 * i + 1];
            const float r0 = bf16_round(__fmul_rn(x0, cs) - __fmul_rn(x1, sn));
            const float r1 = bf16_round(__fmul_rn(x0, sn) + __fmul_rn(x1, cs));
            x0 = r0; x1 = r1;
        }
        if (vec < G) {     // the tensor-core loop scales the scores instead (its queries must stay bf16 values)
            q_s[vec * D + 2 * i] = kMma ? x0 : x0 * qscale;
            q_s[vec * D + 2 * i + 1] = kMma ? x1 : x1 * qscale;
        }
        else {
            float* dst = vec == G ? knew : vnew;
            dst[2 * i] = x0; dst[2 * i + 1] = x1;
            if (split == 0 && h0 == 0) {
                __nv_bfloat16* c = (vec == G ? p.cache_k : p.cache_v) + (((int64_t)b * p.L + P) * p.Hkv + kvh) * D;
                c[2 * i] = __float2bfloat16_rn(x0);
                c[2 * i + 1] = __float2bfloat16_rn(x1);
            }
        }
    }
    sync();

    if constexpr (kMma && GMAX <= 8) {
        attention_keys_mma8<NW, GMAX, kEager>(q_s, G, knew, vnew, split == S - 1, ck - d0, cv - d0, key_stride, lo, hi, warp, lane, red_m,
                                      red_l, red_o);
    } else if constexpr (kMma) {
        attention_keys_mma<NW, GMAX>(q_s, G, knew, vnew, split == S - 1, ck - d0, cv - d0, key_stride, lo, hi, warp, lane, red_m,
                                     red_l, red_o);
    } else {
    // Online softmax state of the G query heads; a lane owns dims d0..d0+3 of q, k, v and o.
    float m_h[GMAX], l_h[GMAX], o_h[GMAX][4], q_r[GMAX][4];
#pragma unroll
    for (int h = 0; h < GMAX; ++h) {
        m_h[h] = -INFINITY; l_h[h] = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            o_h[h][e] = 0.f;
            q_r[h][e] = (h < G && live) ? q_s[h * D + d0 + e] : 0.f;
        }
    }
    auto visit = [&](const float (&kf)[U][4], const float (&vf)[U][4], int n) {
        float sc[GMAX][U];
#pragma unroll
        for (int h = 0; h < GMAX; ++h)
#pragma unroll
            for (int u = 0; u < U; ++u)
                sc[h][u] = q_r[h][0] * kf[u][0] + q_r[h][1] * kf[u][1] + q_r[h][2] * kf[u][2] + q_r[h][3] * kf[u][3];
        if constexpr (GMAX == 4 && U == 4) {
            // Sixteen partial scores per lane, to be summed over the 32 lanes.  Instead of a
            // butterfly on all of them (80 shuffles) the lanes halve their set in every round
            // (8 + 4 + 2 + 1 + 1 shuffles; the same additions in the same order for each value):
            // lanes 2i and 2i+1 end up with the total of value i = 4 h + u, take the head's
            // maximum with the three other keys' lanes, compute the one weight they own and the
            // head's correction, and shuffles hand the results to everybody.
            const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
            float a8[8], a4[4], a2[2];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float lo_v = sc[i >> 2][i & 3], hi_v = sc[(i + 8) >> 2][i & 3];
                a8[i] = (b4 ? hi_v : lo_v) + __shfl_xor_sync(0xffffffffu, b4 ? lo_v : hi_v, 16);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) a4[i] = (b3 ? a8[i + 4] : a8[i]) + __shfl_xor_sync(0xffffffffu, b3 ? a8[i] : a8[i + 4], 8);
#pragma unroll
            for (int i = 0; i < 2; ++i) a2[i] = (b2 ? a4[i + 2] : a4[i]) + __shfl_xor_sync(0xffffffffu, b2 ? a4[i] : a4[i + 2], 4);
            float s_mine = (b1 ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, b1 ? a2[0] : a2[1], 2);
            s_mine += __shfl_xor_sync(0xffffffffu, s_mine, 1);
            const int h_mine = (lane >> 3) & 3, u_mine = (lane >> 1) & 3;
            const bool valid = h_mine < G && u_mine < n;
            float mx = valid ? s_mine : -INFINITY;
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            const float m_old = h_mine == 0 ? m_h[0] : (h_mine == 1 ? m_h[1] : (h_mine == 2 ? m_h[2] : m_h[3]));
            const float mn_mine = fmaxf(m_old, mx);
            const float p_mine = valid ? __expf(s_mine - mn_mine) : 0.f;
            const float corr_mine = __expf(m_old - mn_mine);
#pragma unroll
            for (int h = 0; h < GMAX; ++h) {
                if (h < G) {
                    const float mn = __shfl_sync(0xffffffffu, mn_mine, h * 8);
                    const float corr = __shfl_sync(0xffffffffu, corr_mine, h * 8);
                    float ps = 0.f, ov[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const float pr = __shfl_sync(0xffffffffu, p_mine, h * 8 + u * 2);
                        ps += pr;
#pragma unroll
                        for (int e = 0; e < 4; ++e) ov[e] += pr * vf[u][e];
                    }
                    l_h[h] = l_h[h] * corr + ps;
#pragma unroll
                    for (int e = 0; e < 4; ++e) o_h[h][e] = o_h[h][e] * corr + ov[e];
                    m_h[h] = mn;
                }
            }
            return;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int h = 0; h < GMAX; ++h)
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (h < G) sc[h][u] += __shfl_xor_sync(0xffffffffu, sc[h][u], o);
        if constexpr (GMAX * U + GMAX <= 32) {
            // Every lane holds all scores.  The exponentials are shared out: lane h*U+u computes the
            // weight of key u for head h, lane GMAX*U+h the correction of head h's running sums (one
            // special-function instruction per warp instead of GMAX*U+GMAX), and shuffles hand them
            // round.  A key beyond n gets exp(-inf) = 0.
            float mn[GMAX];
            float arg = -INFINITY;
#pragma unroll
            for (int h = 0; h < GMAX; ++h) {
                mn[h] = m_h[h];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (u < n) mn[h] = fmaxf(mn[h], sc[h][u]);
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (lane == h * U + u && h < G && u < n) arg = sc[h][u] - mn[h];
                if (lane == GMAX * U + h && h < G) arg = m_h[h] - mn[h];
            }
            const float ex = __expf(arg);
#pragma unroll
            for (int h = 0; h < GMAX; ++h) {
                if (h < G) {
                    const float corr = __shfl_sync(0xffffffffu, ex, GMAX * U + h);
                    float ps = 0.f, ov[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const float pr = __shfl_sync(0xffffffffu, ex, h * U + u);
                        ps += pr;
#pragma unroll
                        for (int e = 0; e < 4; ++e) ov[e] += pr * vf[u][e];
                    }
                    l_h[h] = l_h[h] * corr + ps;
#pragma unroll
                    for (int e = 0; e < 4; ++e) o_h[h][e] = o_h[h][e] * corr + ov[e];
                    m_h[h] = mn[h];
                }
            }
        } else {
#pragma unroll
            for (int h = 0; h < GMAX; ++h) {
                if (h < G) {
                    float mn = m_h[h];
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        if (u < n) mn = fmaxf(mn, sc[h][u]);
                    const float corr = __expf(m_h[h] - mn);
                    float ps = 0.f, ov[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (u < n) {
                            const float pr = __expf(sc[h][u] - mn);
                            ps += pr;
#pragma unroll
                            for (int e = 0; e < 4; ++e) ov[e] += pr * vf[u][e];
                        }
                    }
                    l_h[h] = l_h[h] * corr + ps;
#pragma unroll
                    for (int e = 0; e < 4; ++e) o_h[h][e] = o_h[h][e] * corr + ov[e];
                    m_h[h] = mn;
                }
            }
        }
    };
    auto unpack4 = [](const uint2& r, float (&f)[4]) {
        const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
        const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
        f[0] = __low2float(lo2); f[1] = __high2float(lo2); f[2] = __low2float(hi2); f[3] = __high2float(hi2);
    };
    for (int j0 = lo + warp * U; j0 < hi; j0 += NW * U) {
        float kf[U][4], vf[U][4];
#pragma unroll
        for (int u = 0; u < U; ++u) { unpack4(kr[u], kf[u]); unpack4(vr[u], vf[u]); }
        if (j0 + NW * U < hi) request(j0 + NW * U);   // in flight during this visit
        visit(kf, vf, min(U, hi - j0));
    }
    if (split == S - 1 && warp == 0) {   // the new token attends to itself
        float kf[U][4], vf[U][4];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                kf[u][e] = (u == 0 && live) ? knew[d0 + e] : 0.f;
                vf[u][e] = (u == 0 && live) ? vnew[d0 + e] : 0.f;
            }
        visit(kf, vf, 1);
    }
    // combine the warps
#pragma unroll
    for (int h = 0; h < GMAX; ++h) {
        if (h < G) {
            if (lane == 0) { red_m[warp * GMAX + h] = m_h[h]; red_l[warp * GMAX + h] = l_h[h]; }
            if (live) {
#pragma unroll
                for (int e = 0; e < 4; ++e) red_o[(warp * G + h) * D + d0 + e] = o_h[h][e];
            }
        }
    }
    }
    sync();
    for (int idx = tid; idx < G * D; idx += NT) {
        const int h = idx / D, d = idx - h * D;
        float mx = -INFINITY;
        for (int w = 0; w < NW; ++w) mx = fmaxf(mx, red_m[w * GMAX + h]);
        float l = 0.f, o = 0.f;
        for (int w = 0; w < NW; ++w) {
            const float lw = red_l[w * GMAX + h];
            if (lw > 0.f) {
                const float f = __expf(red_m[w * GMAX + h] - mx);
                l += lw * f;
                o += red_o[(w * G + h) * D + d] * f;
            }
        }
        const float on = l > 0.f ? o / l : 0.f;
        if (S == 1) {                       // a single slice: this is the result
            p.out[(int64_t)b * p.H * D + (kvh * Gfull + h0 + h) * D + d] = __float2bfloat16_rn(on);
            if (p.tap) p.tap[(int64_t)b * p.H * D + (kvh * Gfull + h0 + h) * D + d] = __float2bfloat16_rn(on);
            continue;
        }
        const int64_t slot = ((int64_t)b * p.H + kvh * Gfull + h0 + h) * p.S + split;
        p.part_o[slot * D + d] = on;
        if (d == 0) { p.part_ml[slot * 2] = mx; p.part_ml[slot * 2 + 1] = l; }
    }
    if (S == 1) return true;
    // the last slice of this (sequence, kv head) to finish combines all of them
    __threadfence();
    sync();
    if (tid == 0) {
        int* ctr = &p.counters[b * p.Hkv + kvh];
        const int ticket = atomicAdd(ctr, 1);
        *is_last_s = ticket == S - 1;
        if (*is_last_s) *ctr = 0;
    }
    sync();
    if (!*is_last_s) return false;
    __threadfence();
    // weights of the slices per head, then one pass over the partial outputs
    float* sl_m = red_o;                  // [G][S] weight of slice s for head h
    const int64_t head0 = (int64_t)b * p.H + kvh * Gfull + h0;
    if (S <= 32) {
        // a warp per head, a lane per slice: maximum, weights and their sum by shuffles
        for (int h = warp; h < G; h += NW) {
            float m = -INFINITY, l = 0.f;
            if (lane < S) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((head0 + h) * p.S + lane) * 2));
                m = ml.x; l = ml.y;
            }
            float mx = m;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float w = l > 0.f ? __expf(m - mx) * l : 0.f;
            float den = w;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
            if (lane < S) sl_m[h * p.S + lane] = den > 0.f ? w / den : 0.f;
        }
    } else {
        float* sl_l = red_o + G * p.S;    // [G][S] sum
        for (int idx = tid; idx < G * S; idx += NT) {
            const int h = idx / S, sidx = idx - h * S;
            sl_m[h * p.S + sidx] = __ldcg(&p.part_ml[((head0 + h) * p.S + sidx) * 2]);
            sl_l[h * p.S + sidx] = __ldcg(&p.part_ml[((head0 + h) * p.S + sidx) * 2 + 1]);
        }
        sync();
        if (tid < G) {
            float mx = -INFINITY, den = 0.f;
            for (int sidx = 0; sidx < S; ++sidx) mx = fmaxf(mx, sl_m[tid * p.S + sidx]);
            for (int sidx = 0; sidx < S; ++sidx) {
                const float l = sl_l[tid * p.S + sidx];
                const float w = l > 0.f ? __expf(sl_m[tid * p.S + sidx] - mx) * l : 0.f;
                sl_m[tid * p.S + sidx] = w;
                den += w;
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
            for (int sidx = 0; sidx < S; ++sidx) sl_m[tid * p.S + sidx] *= inv;
        }
    }
    sync();
    // four dims per thread and sixteen slices per batch of loads: the partial outputs come from L2,
    // and one CTA reads all of them, so as many loads as possible are in flight at once
    const int D4 = D >> 2;                   // D is a multiple of 4
    for (int idx = tid; idx < G * D4; idx += NT) {
        const int h = idx / D4, d = (idx - h * D4) * 4;
        const float* po = p.part_o + (head0 + h) * p.S * D + d;
        float num[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s0 = 0; s0 < S; s0 += 16) {
            float4 v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u)
                v[u] = s0 + u < S ? __ldcg(reinterpret_cast<const float4*>(po + (int64_t)(s0 + u) * D)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 16; ++u) {       // slices in their order, as a scalar loop would add them
                const float w = s0 + u < S ? sl_m[h * p.S + s0 + u] : 0.f;
                num[0] += w * v[u].x; num[1] += w * v[u].y; num[2] += w * v[u].z; num[3] += w * v[u].w;
            }
        }
        const int64_t oi = (int64_t)b * p.H * D + (kvh * Gfull + h0 + h) * D + d;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p.out[oi + e] = __float2bfloat16_rn(num[e]);
            if (p.tap) p.tap[oi + e] = __float2bfloat16_rn(num[e]);
        }
    }
    return true;
}

// ---------------------------------------------------------------------------------------
// Output head: final RMSNorm, then logits = x . E^T over a slice of the vocabulary (bf16
// weights, f32 accumulation, bf16-rounded result as gpu/model.py:280-281) and the slice's
// argmax.  One warp per vocabulary row, all loads of a row in flight.
// ---------------------------------------------------------------------------------------
constexpr int kHeadThreads = 512;
constexpr int kHeadMaxLoads = 10;   // 16-byte loads per lane per pass over a row

// The output head over this CTA's slice of the vocabulary by 512 threads; `smem` needs
// head_smem() bytes, `sync` is a barrier over those threads.  Leaves the slice's best
// (value, index) per token in part_val / part_idx[cta].
// kCompact: the normalised activations (bf16 values) are kept as bf16 instead of f32, for batch x
// hidden sizes whose f32 form does not fit shared memory; the products are the same.
// kRing: the weight rows arrive in shared memory by bulk copies - two row slots per warp, the first
// two rows requested by the calling kernel - instead of being loaded by the warps' threads;
// `ring` points at the slots ([warp][2][K] bf16), `bars` at one mbarrier per slot.  Same sums either way.
constexpr int kHeadRingRows = 16;     // rows in flight per slot set: one per warp
// One row of the projection into a warp's slot (one thread).
__device__ __forceinline__ void head_request_row(const HeadParams& p, int row, uint8_t* dst, uint64_t* bar, uint64_t policy) {
    const uint32_t bytes = (uint32_t)((size_t)p.K * sizeof(__nv_bfloat16));
    mbar_expect_tx(bar, bytes);
    bulk_g2s(dst, p.w + (int64_t)row * p.K, bytes, bar, policy);
}
// kOne: one token.  The token loops of the row code are unrolled; with one token their eight-fold
// copy would be straight-line code that is jumped over but still fetched, row after row.
template <bool kCompact, bool kRing, bool kOne, class Sync>
__device__ __forceinline__ void head_body(const HeadParams& p, uint8_t* smem, int cta, int n_cta, int tid, Sync sync,
                                          const uint8_t* ring = nullptr, uint64_t* bars = nullptr) {
    using XT = typename std::conditional<kCompact, __nv_bfloat16, float>::type;
    XT* xs = reinterpret_cast<XT*>(smem);                         // [M][K]
    double* red_d = reinterpret_cast<double*>(xs + (size_t)p.M * p.K);   // [16] (K is a multiple of 8)
    auto put = [&](size_t i, float v) {          // v is a bf16 value: exact either way
        if constexpr (kCompact) xs[i] = __float2bfloat16_rn(v);
        else xs[i] = v;
    };
    auto get = [&](size_t i) -> float {
        if constexpr (kCompact) return __bfloat162float(xs[i]);
        else return xs[i];
    };
    float* best_v = reinterpret_cast<float*>(red_d + 16);       // [16 warps][8]
    int* best_i = reinterpret_cast<int*>(best_v + 16 * 8);      // [16 warps][8]
    const int warp = tid >> 5, lane = tid & 31;

    // final RMSNorm (gpu/model.py:280) of every token into shared memory, as its bf16
    // result; the sum of squares in double precision (see prologue.cuh), taken from the
    // producer's partial statistics when it published them
    for (int m = 0; m < p.M; ++m) {
        double ss = 0.0;
        if (p.stats_in && tid == 0) ss = __ldcg(&p.stats_in[m].ss);
        for (int k = tid; k < p.K; k += kHeadThreads) {
            const float v = __uint_as_float((unsigned int)__ldcg(reinterpret_cast<const unsigned short*>(p.h + (int64_t)m * p.K + k)) << 16);   // L2: written by other SMs
            put((size_t)m * p.K + k, v);
            if (!p.stats_in) ss = fma((double)v, (double)v, ss);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        sync();
        if (lane == 0) red_d[warp] = ss;
        sync();
        double tot = 0.0;
        for (int i = 0; i < kHeadThreads / 32; ++i) tot += red_d[i];
        const float rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn((float)tot, (float)p.K), p.eps)));
        for (int k = tid; k < p.K; k += kHeadThreads)
            put((size_t)m * p.K + k, bf16_round(get((size_t)m * p.K + k) * __bfloat162float(p.gamma[k]) * rinv));
    }
    const int r0 = (int)((int64_t)p.V * cta / n_cta), r1 = (int)((int64_t)p.V * (cta + 1) / n_cta);
    constexpr int MM = kOne ? 1 : 8;     // tokens the row code is unrolled for
    float bv[8];
    int bi[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) { bv[m] = -INFINITY; bi[m] = 0x7fffffff; }
    const int vec_per_row = p.K / 8;     // 16-byte pieces
    const uint64_t w_policy = l2_evict_first_policy();    // the projection is read once per step: first out of L2
    auto do_row = [&](int row, auto fetch) {      // fetch(v): 16-byte piece v of the row's weights
        float dot[MM];
#pragma unroll
        for (int m = 0; m < MM; ++m) dot[m] = 0.f;
        for (int base = 0; base < vec_per_row; base += 32 * kHeadMaxLoads) {
            uint4 wv[kHeadMaxLoads];
#pragma unroll
            for (int u = 0; u < kHeadMaxLoads; ++u) {
                const int v = base + u * 32 + lane;
                if (v < vec_per_row) wv[u] = fetch(v);
            }
#pragma unroll
            for (int u = 0; u < kHeadMaxLoads; ++u) {
                const int v = base + u * 32 + lane;
                if (v < vec_per_row) {
                    const Vec8 wf = unpack_bf16x8(wv[u]);
#pragma unroll
                    for (int m = 0; m < MM; ++m) {
                        if (m < p.M) {
                            Vec8 xf;
                            if constexpr (kCompact) {
                                xf = unpack_bf16x8(*reinterpret_cast<const uint4*>(xs + (size_t)m * p.K + v * 8));
                            } else {
                                const float4 x0 = *reinterpret_cast<const float4*>(xs + (size_t)m * p.K + v * 8);
                                const float4 x1 = *reinterpret_cast<const float4*>(xs + (size_t)m * p.K + v * 8 + 4);
                                xf.v[0] = x0.x; xf.v[1] = x0.y; xf.v[2] = x0.z; xf.v[3] = x0.w;
                                xf.v[4] = x1.x; xf.v[5] = x1.y; xf.v[6] = x1.z; xf.v[7] = x1.w;
                            }
                            dot[m] += wf.v[0] * xf.v[0] + wf.v[1] * xf.v[1] + wf.v[2] * xf.v[2] + wf.v[3] * xf.v[3] +
                                      wf.v[4] * xf.v[4] + wf.v[5] * xf.v[5] + wf.v[6] * xf.v[6] + wf.v[7] * xf.v[7];
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MM; ++m) {
            if (m < p.M) {
                float d = dot[m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                d = bf16_round(d);
                if (lane == 0 && p.logits) p.logits[(int64_t)m * p.V + row] = d;
                if (d > bv[m]) { bv[m] = d; bi[m] = row + p.row_offset; }     // rows ascend: first maximum wins
            }
        }
    };
    if constexpr (kRing) {
        // every warp owns two row slots and refills a slot itself as soon as it has used it up: two
        // rows per warp are in flight or in use at any time, and no warp waits for another
        const size_t row_bytes = (size_t)p.K * sizeof(__nv_bfloat16);
        const uint8_t* slot = ring + (size_t)warp * 2 * row_bytes;
        uint64_t* full = bars + 2 * warp;
        bool ok = true;
        int k = 0;
#pragma unroll 1
        for (int row = r0 + warp; row < r1 && ok; row += kHeadThreads / 32, ++k) {
            ok = mbar_wait(&full[k & 1], (k >> 1) & 1);
            if (ok) {
                const uint4* src = reinterpret_cast<const uint4*>(slot + (k & 1) * row_bytes);
                do_row(row, [&](int v) { return src[v]; });
            }
            __syncwarp();
            const int next = row + 2 * (kHeadThreads / 32);
            if (lane == 0 && ok && next < r1) head_request_row(p, next, const_cast<uint8_t*>(slot) + (k & 1) * row_bytes, &full[k & 1], w_policy);
        }
        if (!ok && lane == 0 && p.error_flag) atomicExch(p.error_flag, kErrConsumerWait);
    } else {
        for (int row = r0 + warp; row < r1; row += kHeadThreads / 32) {
            const uint4* wr = reinterpret_cast<const uint4*>(p.w + (int64_t)row * p.K);
            do_row(row, [&](int v) { return ldg_stream_hint(wr + v, w_policy); });
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < 8; ++m) { best_v[warp * 8 + m] = bv[m]; best_i[warp * 8 + m] = bi[m]; }
    }
    sync();
    if (tid < p.M) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int w = 0; w < kHeadThreads / 32; ++w) {
            const float wv = best_v[w * 8 + tid];
            const int wi = best_i[w * 8 + tid];
            if (wv > v || (wv == v && wi < i)) { v = wv; i = wi; }
        }
        if (p.tp.size > 1) {     // the slice's maxima go to packets [rank][cta] of every rank's area
            const size_t at = ((size_t)p.tp.rank * n_cta + cta) * 8 + tid;
            const unsigned int tag = tp_tag(p.tp_tag_out);
#pragma unroll 1
            for (int pr = 0; pr < p.tp.size; ++pr) {
                tp_put(reinterpret_cast<uint2*>(p.tp.area[pr] + p.tp_val_off) + at, __float_as_uint(v), tag);
                tp_put(reinterpret_cast<uint2*>(p.tp.area[pr] + p.tp_idx_off) + at, (unsigned int)i, tag);
            }
        } else {
            p.part_val[cta * 8 + tid] = v;
            p.part_idx[cta * 8 + tid] = i;
        }
    }
}

}  // namespace

}  // namespace bitnet
