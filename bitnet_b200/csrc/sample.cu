// Temperature + top-p (nucleus) sampling of the next token on the device.
//
// What the reference does on the host side of its decode loop (gpu/generate.py:250-257,
// gpu/sample_utils.py:8-30): probs = softmax(logits / temperature); sort descending; drop every
// entry whose exclusive cumulative probability exceeds p; draw one of the rest in proportion to
// its probability.  Here a cluster of eight CTAs per sequence does the same without sorting.  The
// row is read once: every thread keeps its share of e_i = exp((l_i - max) / temperature) in
// registers, and the CTAs exchange a few words per phase through distributed shared memory.
//   1. the row's max, then e_i.  Masses are integers, m_i = floor(e_i * 2^40): sums of them do
//      not depend on the order of addition, so every phase sees the same numbers (S = their total).
//   2. the smallest kept value v*: a radix select (4 passes of 8 bits) over the bit patterns of
//      e_i, guided by the mass above each bin instead of by counts.  With G(v) = mass of all
//      entries greater than v, a value class is kept (at least its first entry) exactly when
//      G(v) <= p S, and of the class v* itself the first c = floor((p S - G(v*)) / m*) + 1
//      entries in index order are kept - the entries a stable descending sort puts before the cut.
//   3. a draw u in [0, 1): the kept entry, in index order, at which the running kept mass first
//      exceeds u * (kept mass).  Any fixed order gives the reference's distribution; index order
//      needs no sort.
// u comes from the caller (one float per sequence) or from a counter hash of (seed, sequence,
// position), so that a captured graph that replays this kernel draws a new number every step.
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace cg = cooperative_groups;

namespace bitnet {

namespace {

constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;
constexpr int kSampleCtas = 8;                    // CTAs of one cluster = of one sequence
typedef unsigned long long u64;

struct SampleParams {
    const float* logits;
    long long ld;
    int V;
    float inv_temp;
    float top_p;
    u64 seed;
    const long long* pos;
    const float* uniforms;
    long long* out;
    long long* tokens;
};

// splitmix64 finaliser over (seed, sequence, position): 24 uniform bits.
__device__ __forceinline__ float counter_uniform(u64 seed, int row, long long pos) {
    u64 x = seed + 0x9E3779B97F4A7C15ull * (u64)(row + 1);
    x ^= (u64)pos * 0xD1B54A32D192ED03ull;
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return (float)(x >> 40) * (1.0f / 16777216.0f);
}

// floor(e * 2^40) for 0 <= e <= 1, from the bits of e (a 64-bit float-to-integer conversion is slow)
__device__ __forceinline__ u64 mass_of(float e) {
    const unsigned int key = __float_as_uint(e);
    const int shift = (int)(key >> 23) - 110;                  // exponent - 127 + 40 - 23
    const u64 mant = (u64)((key & 0x7FFFFFu) | 0x800000u);
    if ((key >> 23) == 0u || shift <= -24) return 0ull;        // zero, denormal, below 2^-40
    return shift >= 0 ? mant << shift : mant >> -shift;
}

__device__ __forceinline__ u64 warp_sum(u64 v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Exclusive scan of a[0..n) in shared memory (n <= 1024, all threads of the CTA call it); returns
// the total.  `tmp` holds one value per warp.
template <class T>
__device__ T block_exclusive_scan(T* a, int n, T* tmp) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    T v = tid < n ? a[tid] : T(0);
    T inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) tmp[warp] = inc;
    __syncthreads();
    T base = T(0), total = T(0);
    for (int w = 0; w < kSampleWarps; ++w) {
        const T t = tmp[w];
        if (w < warp) base += t;
        total += t;
    }
    if (tid < n) a[tid] = base + inc - v;
    __syncthreads();
    return total;
}

// What each CTA shows to the others of its cluster.
struct SampleShared {
    u64 hist_mass[4][256];
    unsigned int hist_cnt[4][256];
    float slot_max;
    u64 slot_gt;            // mass of its entries greater than v*
    unsigned int slot_eq;   // number of its entries equal to v*
};

template <int PER>
__global__ void __cluster_dims__(kSampleCtas, 1, 1) __launch_bounds__(kSampleThreads)
sample_top_p_kernel(const SampleParams p) {
    __shared__ SampleShared sh;
    __shared__ u64 tot_mass[256];
    __shared__ unsigned int tot_cnt[256];
    __shared__ u64 ent_mass[kSampleThreads];
    __shared__ unsigned int ent_eq[kSampleThreads];
    __shared__ u64 tmp64[kSampleWarps];
    __shared__ unsigned int tmp32[kSampleWarps];
    __shared__ float red_f[kSampleWarps];
    __shared__ u64 sh_pS, sh_above, sh_keep, sh_target;
    __shared__ int sh_chosen;

    // one private histogram per warp (dynamic shared memory): a warp's lanes that fall into one
    // bin add up among themselves and one of them updates the warp's own row, so nothing is
    // contended and no atomic is needed
    extern __shared__ __align__(16) unsigned char sample_dyn[];
    u64 (*warp_mass)[256] = reinterpret_cast<u64 (*)[256]>(sample_dyn);
    unsigned int (*warp_cnt)[256] =
        reinterpret_cast<unsigned int (*)[256]>(sample_dyn + sizeof(u64) * 256 * kSampleWarps);

    cg::cluster_group cluster = cg::this_cluster();
    const int crank = (int)cluster.block_rank();
    const int row = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* l = p.logits + (long long)row * p.ld;
    const int V = p.V;
    // thread t of CTA c holds the PER consecutive values from index (c * 1024 + t) * PER on: index
    // order is (CTA, thread, j)
    const int first = (crank * kSampleThreads + tid) * PER;

    // 1. max over the row, then e
    float e[PER];
    float mx = -INFINITY;
    const bool vec = (reinterpret_cast<uintptr_t>(l) & 15u) == 0;
#pragma unroll
    for (int j = 0; j < PER; j += 4) {
        const int i = first + j;
        if (vec && i + 3 < V) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(l + i));
            e[j] = v.x; e[j + 1] = v.y; e[j + 2] = v.z; e[j + 3] = v.w;
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) e[j + k] = i + k < V ? __ldg(l + i + k) : -INFINITY;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) mx = fmaxf(mx, e[j + k]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kSampleWarps; ++w) mx = fmaxf(mx, red_f[w]);
        sh.slot_max = mx;
    }
    cluster.sync();
    mx = -INFINITY;
    for (int r = 0; r < kSampleCtas; ++r) mx = fmaxf(mx, cluster.map_shared_rank(&sh, r)->slot_max);

#pragma unroll
    for (int j = 0; j < PER; ++j)
        e[j] = first + j < V ? expf((e[j] - mx) * p.inv_temp) : -1.0f;     // -1 marks "beyond the row"

    // 2. radix select of v* by mass
    unsigned int prefix = 0;        // the bits of v* found so far (the high 8 * pass bits)
    u64 above = 0;                  // mass of the entries known to be greater than v*'s bin
    unsigned int n_equal = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
#pragma unroll
        for (int k = 0; k < 8; ++k) { warp_mass[warp][lane + 32 * k] = 0ull; warp_cnt[warp][lane + 32 * k] = 0u; }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const unsigned int key = __float_as_uint(e[j]);
            const bool in = e[j] >= 0.0f && (pass == 0 || (key >> (shift + 8)) == prefix);
            const unsigned int bin = in ? ((key >> shift) & 255u) : 256u;
            const u64 m = in ? mass_of(e[j]) : 0ull;
            if (pass == 0) {
                // few distinct bins per warp (the bins are exponents): the lanes of one bin add up
                // among themselves and one of them updates the warp's row
                const unsigned int peers = __match_any_sync(0xffffffffu, bin);
                const unsigned int lo = __reduce_add_sync(peers, (unsigned int)(m & 0xFFFFFu));
                const unsigned int hi = __reduce_add_sync(peers, (unsigned int)(m >> 20));
                if (in && lane == __ffs(peers) - 1) {
                    warp_mass[warp][bin] += ((u64)hi << 20) + (u64)lo;
                    warp_cnt[warp][bin] += (unsigned int)__popc(peers);
                }
                __syncwarp();
            } else if (in) {
                // mantissa digits: spread over the bins, and fewer entries take part each pass
                atomicAdd(&warp_mass[warp][bin], m);
                atomicAdd(&warp_cnt[warp][bin], 1u);
            }
        }
        __syncthreads();
        if (tid < 256) {
            u64 m = 0;
            unsigned int c = 0;
            for (int w = 0; w < kSampleWarps; ++w) { m += warp_mass[w][tid]; c += warp_cnt[w][tid]; }
            sh.hist_mass[pass][tid] = m;
            sh.hist_cnt[pass][tid] = c;
        }
        cluster.sync();
        if (tid < 256) {
            u64 m = 0;
            unsigned int c = 0;
            for (int r = 0; r < kSampleCtas; ++r) {
                const SampleShared* o = cluster.map_shared_rank(&sh, r);
                m += o->hist_mass[pass][tid];
                c += o->hist_cnt[pass][tid];
            }
            tot_mass[tid] = m;
            tot_cnt[tid] = c;
        }
        __syncthreads();
        // the lowest non-empty bin whose mass above is still within p S: warp 0 finds it, lane L
        // looking at the bins 255 - 8L ... 248 - 8L
        if (warp == 0) {
            u64 mine = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) mine += tot_mass[255 - (8 * lane + k)];
            u64 inc = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const u64 t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
            u64 lim = sh_pS;
            if (pass == 0) {    // all bins = the total mass S
                lim = (u64)((double)p.top_p * (double)__shfl_sync(0xffffffffu, inc, 31));
                if (p.top_p >= 1.0f) lim = ~0ull;
            }
            u64 a = above + inc - mine;           // mass above this lane's first bin
            int best = -1, first = 1 << 20;       // as distances d = 255 - bin from the top
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int d = 8 * lane + k;
                if (tot_cnt[255 - d] != 0u) {
                    if (a <= lim) best = d;
                    first = min(first, d);
                }
                a += tot_mass[255 - d];
            }
            best = __reduce_max_sync(0xffffffffu, best);
            first = __reduce_min_sync(0xffffffffu, first);
            if (best < 0) best = first < 256 ? first : 255;
            // mass above the chosen bin = `above` + the masses of the bins over it
            u64 over = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) over += (8 * lane + k < best) ? tot_mass[255 - (8 * lane + k)] : 0ull;
            over = warp_sum(over);
            if (lane == 0) {
                sh_pS = lim;
                sh_above = above + over;
                sh_chosen = 255 - best;
            }
        }
        __syncthreads();
        above = sh_above;
        n_equal = tot_cnt[sh_chosen];
        prefix = (prefix << 8) | (unsigned int)sh_chosen;
        __syncthreads();
    }
    const u64 pS = sh_pS;           // floor(top_p * S): the masses are integers
    const float v_star = __uint_as_float(prefix);
    const u64 m_star = mass_of(v_star);
    if (tid == 0) {     // how many of the values equal to v* are kept, and the draw (64-bit divisions: one thread)
        u64 keep = n_equal;
        if (m_star > 0) {
            const u64 q = (pS > above ? pS - above : 0ull) / m_star + 1ull;
            if (q < keep) keep = q;
        }
        const u64 kept_mass = above + keep * m_star;
        float u = p.uniforms ? p.uniforms[row] : counter_uniform(p.seed, row, p.pos ? p.pos[row] : 0);
        u = fminf(fmaxf(u, 0.0f), 0.99999994f);
        u64 t = (u64)((double)u * (double)kept_mass);
        if (kept_mass > 0 && t >= kept_mass) t = kept_mass - 1;
        sh_keep = keep;
        sh_target = t;
    }

    // 3. per thread: mass of its values over v*, number of its values equal to it
    u64 my_gt = 0;
    unsigned int my_eq = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        if (e[j] > v_star) my_gt += mass_of(e[j]);
        my_eq += e[j] == v_star;
    }
    ent_eq[tid] = my_eq;
    u64 cta_gt = warp_sum(my_gt);
    if (lane == 0) tmp64[warp] = cta_gt;
    __syncthreads();
    const u64 keep_equal = sh_keep, target = sh_target;
    const unsigned int cta_eq = block_exclusive_scan(ent_eq, kSampleThreads, tmp32);
    // (ent_eq[t] now = equals of this CTA before thread t's share)
    if (tid == 0) {
        for (int w = 1; w < kSampleWarps; ++w) cta_gt += tmp64[w];
        sh.slot_gt = cta_gt;
        sh.slot_eq = cta_eq;
    }
    cluster.sync();
    // kept mass and equals of the CTAs before this one
    u64 mass_before = 0, eq_before = 0, my_mass = 0;
    for (int r = 0; r <= crank; ++r) {
        const SampleShared* o = cluster.map_shared_rank(&sh, r);
        const u64 eqs = o->slot_eq;
        const u64 k = keep_equal > eq_before ? min(keep_equal - eq_before, eqs) : 0ull;
        const u64 m = o->slot_gt + k * m_star;
        if (r < crank) { mass_before += m; eq_before += eqs; }
        else my_mass = m;
    }
    cluster.sync();     // no CTA leaves, or reuses what it shows, while another may still read it
    if (!(target >= mass_before && target < mass_before + my_mass)) return;

    // this CTA holds the target: kept mass per thread, its scan, the thread, the entry
    eq_before += ent_eq[tid];
    const u64 k_mine = keep_equal > eq_before ? min(keep_equal - eq_before, (u64)my_eq) : 0ull;
    const u64 own = my_gt + k_mine * m_star;
    ent_mass[tid] = own;
    __syncthreads();
    block_exclusive_scan(ent_mass, kSampleThreads, tmp64);
    const u64 residual = target - mass_before;
    if (!(own > 0 && residual >= ent_mass[tid] && residual < ent_mass[tid] + own)) return;
    u64 run = ent_mass[tid];
    int chosen = -1;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const bool is_eq = e[j] == v_star;
        const bool kept = e[j] > v_star || (is_eq && eq_before < keep_equal);
        eq_before += is_eq;
        if (kept) {
            run += mass_of(e[j]);
            if (chosen < 0 && run > residual) chosen = j;
        }
    }
    const long long token = (long long)first + (chosen < 0 ? 0 : chosen);
    if (p.out) p.out[row] = token;
    if (p.tokens) p.tokens[row] = token;
}

constexpr size_t kSampleDynBytes = (sizeof(u64) + sizeof(unsigned int)) * 256 * kSampleWarps;

// Lets the kernels use their 96 KB of dynamic shared memory: once per device.
cudaError_t prepare_sample_kernels() {
    static std::mutex mutex;
    static bool done[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess || dev < 0 || dev >= 64) return err != cudaSuccess ? err : cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mutex);
    if (done[dev]) return cudaSuccess;
    const int bytes = (int)kSampleDynBytes;
    if ((err = cudaFuncSetAttribute(sample_top_p_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)) ||
        (err = cudaFuncSetAttribute(sample_top_p_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)) ||
        (err = cudaFuncSetAttribute(sample_top_p_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)))
        return err;
    done[dev] = true;
    return cudaSuccess;
}

}  // namespace

int sample_top_p(const float* logits, long long ld, int batch, int vocab, float temperature, float top_p,
                 unsigned long long seed, const long long* pos, const float* uniforms, long long* out,
                 long long* tokens, cudaStream_t stream) {
    if (!logits || (!out && !tokens) || batch <= 0 || vocab <= 0 || ld < vocab) return set_status(kBadArgument), kBadArgument;
    if (!(temperature > 0.0f) || !(top_p >= 0.0f)) return set_status(kBadArgument), kBadArgument;
    if (batch > 65535) return set_status(kTooLarge), kTooLarge;
    SampleParams p;
    p.logits = logits; p.ld = ld; p.V = vocab;
    p.inv_temp = 1.0f / temperature;
    p.top_p = top_p;
    p.seed = seed; p.pos = pos; p.uniforms = uniforms;
    p.out = out; p.tokens = tokens;
    const dim3 grid(kSampleCtas, batch);
    const int per = (vocab + kSampleCtas * kSampleThreads - 1) / (kSampleCtas * kSampleThreads);
    if (check_cuda(prepare_sample_kernels())) return kCudaError;
    if (per <= 4) sample_top_p_kernel<4><<<grid, kSampleThreads, kSampleDynBytes, stream>>>(p);
    else if (per <= 16) sample_top_p_kernel<16><<<grid, kSampleThreads, kSampleDynBytes, stream>>>(p);
    else if (per <= 32) sample_top_p_kernel<32><<<grid, kSampleThreads, kSampleDynBytes, stream>>>(p);
    else return set_status(kUnsupported), kUnsupported;     // more than 262144 entries
    return check_cuda(cudaGetLastError());
}

}  // namespace bitnet
