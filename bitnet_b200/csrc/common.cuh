// Shared device helpers for the W2A8 BitLinear kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bitnet {

// ---------------------------------------------------------------------------------------
// Status side channel.  The reference's entry point returns void and prints on an
// unsupported shape (gpu/bitnet_kernels/bitnet_kernels.cu:34-36); here every entry point
// records a code that bitnet_last_status() returns, and never aborts or traps.
// ---------------------------------------------------------------------------------------
enum Status : int {
    kOk = 0,
    kBadArgument = 1,     // null pointer, non-positive size, bad alignment
    kUnsupported = 2,     // shape outside what the kernels cover
    kCudaError = 3,       // a CUDA runtime call failed (see bitnet_last_cuda_error)
    kTooLarge = 4,        // exceeds a fixed-capacity buffer
};

void set_status(int s);
int check_cuda(cudaError_t e);   // records kCudaError on failure, returns the status

// ---------------------------------------------------------------------------------------
// The W2T weight layout: tiles of 16 rows x 128 columns, 512 bytes each, row-group major
// (all K tiles of rows 16i..16i+15 are contiguous).  Inside a tile, lane = 4*g + q of a
// warp owns the 16 bytes at offset 16*lane: four 32-bit words r = 0..3.  Byte b of word
// r carries four 2-bit fields j = 0..3 (bits 2j..2j+1):
//     row = 16*tile_row + g + 8*(r & 1)
//     col = 128*tile_col + 32*q + 8*j + 4*(r >> 1) + b
// A field holds weight + 1 (0, 1, 2; 3 is taken literally as +2).  Padding rows and
// columns hold 1 (a zero weight).  With this order `word_r & (0x03030303 << 2j)` is, with
// no shift, 4^j times the A operand a_r of an m16n8k32 integer MMA over the tile's j-th
// group of 32 columns, and the activations that lane q multiplies are the 32 contiguous
// bytes [128*tile_col + 32*q, +32) of a token.
// ---------------------------------------------------------------------------------------
constexpr int kTileRows = 16;
constexpr int kTileCols = 128;
constexpr int kTileBytes = 512;

__host__ __device__ inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// D(16x8, s32) += A(16x32, u8, row) * B(32x8, s8, col)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The same with an L2 eviction policy (createpolicy) attached.
__device__ __forceinline__ uint4 ldg_stream_hint(const uint4* p, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(policy));
    return v;
}

// d = c + sum_i a.u8[i] * b.s8[i]
__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Streaming 16-byte load that does not allocate in L1 (weights are read exactly once).
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Row segments that share one weight scale: rows [end[i-1], end[i]) use scale i.
struct ScaleSegments {
    int n_seg;
    int end[8];
};

__device__ __forceinline__ int segment_of(const ScaleSegments& s, int row) {
    int seg = 0;
#pragma unroll
    for (int i = 0; i < 7; ++i)
        if (i + 1 < s.n_seg && row >= s.end[i]) seg = i + 1;
    return seg;
}

}  // namespace bitnet
