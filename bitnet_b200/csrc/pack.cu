// Weight format conversion kernels.  They take the three weight forms the reference ships
// (ternary int8 as gpu/convert_checkpoint.py:23-27 produces it, the I2_S bytes of
// src/ggml-bitnet-mad.cpp:51-96, the GPU int2 tiles of gpu/pack_weight.py:76-98) to the
// W2T device layout described in common.cuh, and back to ternary int8.  One thread builds
// one 32-bit word of the destination, so stores are coalesced; these run once per tensor
// at load time.
#include "common.cuh"
#include "kernels.h"

namespace bitnet {

namespace {

struct TernarySource {
    const int8_t* q;
    int N, K;
    __device__ uint32_t code(int row, int col) const {
        return (row < N && col < K) ? (uint32_t)(q[(int64_t)row * K + col] + 1) : 1u;
    }
};

// I2_S: every 128 consecutive elements of the flattened matrix are 32 bytes; byte p holds
// elements p, p+32, p+64, p+96 at shifts 6, 4, 2, 0 (src/ggml-bitnet-mad.cpp:80-88).
struct I2sSource {
    const uint8_t* x;
    int N, K;
    __device__ uint32_t code(int row, int col) const {
        if (row >= N || col >= K) return 1u;
        const int64_t i = (int64_t)row * K + col;
        const int64_t blk = i >> 7;
        const int j = (int)(i & 127);
        return (x[blk * 32 + (j & 31)] >> (6 - 2 * (j >> 5))) & 3u;
    }
};

// The reference's GPU form: 16x32 tiles, element (ii, jj) of a stored tile comes from
// source (row, col) with t = 2*ii + jj/16, row = 8*(t/16) + t%8, col = jj%16 + 16*((t%16)/8)
// (gpu/pack_weight.py:5-14); 16 fields per int32 with field idx at bit
// 8*(idx%4) + 2*(idx/4) (:46-72); a field holds weight + 2.
struct RefGpuSource {
    const uint32_t* words;
    int N, K;
    __device__ uint32_t code(int row, int col) const {
        if (row >= N || col >= K) return 1u;
        const int tn = row >> 4, rr = row & 15, tk = col >> 5, cc = col & 31;
        const int t = (rr >> 3) * 16 + (cc >> 4) * 8 + (rr & 7);
        const int e = (t >> 1) * 32 + (t & 1) * 16 + (cc & 15);
        const int idx = e & 15;
        const uint32_t w = words[((int64_t)tn * (K >> 5) + tk) * 32 + (e >> 4)];
        const uint32_t c = (w >> (8 * (idx & 3) + 2 * (idx >> 2))) & 3u;
        return c - 1u;   // weight + 2 -> weight + 1 (a zero field cannot come from the packer)
    }
};

template <class Source>
__global__ void to_w2t_kernel(Source src, uint32_t* out, int64_t n_words, int k_tiles) {
    const int64_t wi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= n_words) return;
    const int64_t tile = wi >> 7;
    const int in_tile = (int)(wi & 127);
    const int lane = in_tile >> 2, r = in_tile & 3;
    const int g = lane >> 2, q = lane & 3;
    const int row = (int)(tile / k_tiles) * 16 + g + 8 * (r & 1);
    const int col0 = (int)(tile % k_tiles) * 128 + 32 * q + 4 * (r >> 1);
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int b = 0; b < 4; ++b) w |= (src.code(row, col0 + 8 * j + b) & 3u) << (8 * b + 2 * j);
    out[wi] = w;
}

__global__ void from_w2t_kernel(const uint32_t* w2t, int8_t* q, int N, int K, int k_tiles) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)N * K) return;
    const int row = (int)(i / K), col = (int)(i % K);
    const int g = row & 7, rlo = (row >> 3) & 1;
    const int kk = col & 127, qq = kk >> 5, j = (kk >> 3) & 3, h = (kk >> 2) & 1, b = kk & 3;
    const int64_t word = ((int64_t)(row >> 4) * k_tiles + (col >> 7)) * 128 + (g * 4 + qq) * 4 + rlo + 2 * h;
    q[i] = (int8_t)(((w2t[word] >> (8 * b + 2 * j)) & 3u)) - 1;
}

// quantize_i2_s on the device: max|x| over the whole tensor, then codes by sign with the
// reference's |x| < 1e-6 -> zero rule (src/ggml-bitnet-mad.cpp:58-72).
__global__ void absmax_bits_kernel(const float* x, int64_t n, uint32_t* out_bits) {
    float m = 0.f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        m = fmaxf(m, fabsf(x[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));   // non-negative floats order as uints
}

__global__ void i2s_pack_kernel(const float* x, int64_t n, uint8_t* dst, const uint32_t* absmax_bits) {
    const int64_t byte = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (byte < n / 4) {
        const int64_t blk = byte >> 5;
        const int p = (int)(byte & 31);
        uint32_t v = 0;
#pragma unroll
        for (int grp = 0; grp < 4; ++grp) {
            const float f = x[blk * 128 + grp * 32 + p];
            const uint32_t c = fabs((double)f) < 1e-6 ? 1u : (f > 0.f ? 2u : 0u);
            v |= c << (6 - 2 * grp);
        }
        dst[byte] = (uint8_t)v;
    }
    if (byte == 0) {
        // f32 scale after the packed data, then zero padding up to 32 bytes
        uint8_t* tail = dst + n / 4;
        const uint32_t bits = *absmax_bits;
        for (int i = 0; i < 32; ++i) tail[i] = i < 4 ? (uint8_t)(bits >> (8 * i)) : 0;
    }
}

template <class Source>
int launch_to_w2t(Source src, void* w2t, int N, int K, cudaStream_t stream) {
    const int64_t n_pad = round_up(N, 16), k_pad = round_up(K, 128);
    const int64_t n_words = n_pad * k_pad / 16;
    const int threads = 256;
    to_w2t_kernel<<<(unsigned)((n_words + threads - 1) / threads), threads, 0, stream>>>(
        src, reinterpret_cast<uint32_t*>(w2t), n_words, (int)(k_pad / 128));
    return check_cuda(cudaGetLastError());
}

}  // namespace

int pack_ternary_to_w2t(const int8_t* q, void* w2t, int N, int K, cudaStream_t stream) {
    return launch_to_w2t(TernarySource{q, N, K}, w2t, N, K, stream);
}

int pack_i2s_to_w2t(const uint8_t* i2s, void* w2t, int N, int K, cudaStream_t stream) {
    return launch_to_w2t(I2sSource{i2s, N, K}, w2t, N, K, stream);
}

int pack_refgpu_to_w2t(const int8_t* packed, void* w2t, int N, int K, cudaStream_t stream) {
    return launch_to_w2t(RefGpuSource{reinterpret_cast<const uint32_t*>(packed), N, K}, w2t, N, K, stream);
}

int unpack_w2t_to_ternary(const void* w2t, int8_t* q, int N, int K, cudaStream_t stream) {
    const int64_t n = (int64_t)N * K;
    const int threads = 256;
    from_w2t_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, stream>>>(
        reinterpret_cast<const uint32_t*>(w2t), q, N, K, (int)(round_up(K, 128) / 128));
    return check_cuda(cudaGetLastError());
}

int i2s_quantize(const float* src, uint8_t* dst, int64_t n_total, uint32_t* absmax_bits_scratch, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(absmax_bits_scratch, 0, sizeof(uint32_t), stream);
    if (e != cudaSuccess) return check_cuda(e);
    const int threads = 256;
    const int blocks = (int)((n_total / 4 + threads - 1) / threads);
    absmax_bits_kernel<<<blocks < 1184 ? (blocks < 1 ? 1 : blocks) : 1184, threads, 0, stream>>>(src, n_total, absmax_bits_scratch);
    i2s_pack_kernel<<<blocks < 1 ? 1 : blocks, threads, 0, stream>>>(src, n_total, dst, absmax_bits_scratch);
    return check_cuda(cudaGetLastError());
}

}  // namespace bitnet
