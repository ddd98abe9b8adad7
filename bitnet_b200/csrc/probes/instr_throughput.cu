// Stand-alone microbenchmark (not part of the library): warp-instructions per clock per SM for the
// integer, logic and MMA instructions the W2A8 tile loops are made of.  One CTA per SM, `clock64`
// around 4096 iterations of 8 independent dependent-chains per thread.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o instr_throughput instr_throughput.cu && ./instr_throughput
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define ITERS 4096
template<int OP> __global__ void k(int* out, int seed, long long* cyc) {
    int a[8]; uint32_t x = threadIdx.x * 2654435761u + seed, y = x ^ 0x9e3779b9u;
    float f[8]; 
    for (int i=0;i<8;++i){a[i]=i+seed; f[i]=i*0.5f+seed;}
    int d[4][4]; for(int i=0;i<4;++i)for(int j=0;j<4;++j)d[i][j]=0;
    __syncthreads();
    long long t0 = clock64();
    #pragma unroll 1
    for (int it=0; it<ITERS; ++it) {
        #pragma unroll
        for (int i=0;i<8;++i) {
            if (OP==0) asm volatile("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(a[i]) : "r"(x), "r"(y));
            if (OP==1) asm volatile("dp4a.s32.s32 %0, %1, %2, %0;" : "+r"(a[i]) : "r"(x), "r"(y));
            if (OP==2) asm volatile("mad.lo.s32 %0, %1, %2, %0;" : "+r"(a[i]) : "r"(x), "r"(y));
            if (OP==3) asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(a[i]) : "r"(x), "r"(y));
            if (OP==4) asm volatile("fma.rn.f32 %0, %1, %2, %0;" : "+f"(f[i]) : "f"(f[(i+1)&7]*0.f+1.0001f), "f"(0.5f));
            if (OP==6) asm volatile("shr.u32 %0, %0, 2;" : "+r"(a[i]));
            if (OP==7) asm volatile("prmt.b32 %0, %0, %1, %2;" : "+r"(a[i]) : "r"(x), "r"(y));
        }
        if (OP==5) {
            #pragma unroll
            for (int i=0;i<4;++i)
            asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
              : "+r"(d[i][0]), "+r"(d[i][1]), "+r"(d[i][2]), "+r"(d[i][3]) : "r"(x), "r"(y), "r"(x+1), "r"(y+1), "r"(x+2), "r"(y+2));
        }
        if (OP==8) {
            #pragma unroll
            for (int i=0;i<4;++i)
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
              : "+f"(f[0+i]), "+f"(f[4+i]), "+f"(f[(1+i)&7]), "+f"(f[(5+i)&7]) : "r"(x), "r"(y), "r"(x+1), "r"(y+1), "r"(x+2), "r"(y+2));
        }
    }
    long long t1 = clock64();
    int s=0; for(int i=0;i<8;++i) s+=a[i]+(int)f[i]; for(int i=0;i<4;++i)for(int j=0;j<4;++j)s+=d[i][j];
    out[blockIdx.x*blockDim.x+threadIdx.x]=s;
    if (threadIdx.x==0 && blockIdx.x==0) *cyc = t1-t0;
}
template<int OP> void run(const char* name, int per_iter_ops, int threads) {
    int* out; long long* cyc; cudaMalloc(&out, 148*1024*4); cudaMalloc(&cyc, 8);
    k<OP><<<148, threads>>>(out, 1, cyc); cudaDeviceSynchronize();
    k<OP><<<148, threads>>>(out, 2, cyc); cudaDeviceSynchronize();
    long long c; cudaMemcpy(&c, cyc, 8, cudaMemcpyDeviceToHost);
    double warp_instr = (double)ITERS * per_iter_ops * (threads/32);
    printf("%-28s threads=%4d cycles=%8lld  warp-instr/clk/SM=%.3f  lane-ops/clk/SM=%.1f\n", name, threads, c, warp_instr/c, warp_instr*32/c);
    cudaFree(out); cudaFree(cyc);
}
int main() {
    for (int th : {128, 512, 1024}) {
        run<0>("dp4a.u32.s32", 8, th); run<1>("dp4a.s32.s32", 8, th); run<2>("mad.lo.s32", 8, th); run<3>("lop3", 8, th);
        run<4>("fma.f32", 8, th); run<6>("shr", 8, th); run<7>("prmt", 8, th);
        run<5>("mma.m16n8k32.u8.s8", 4, th); run<8>("mma.m16n8k16.bf16", 4, th);
    }
    return 0;
}
