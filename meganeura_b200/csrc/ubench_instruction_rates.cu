// Instruction issue-rate microbenchmark behind the GEMV inner-loop design (thread-ops per clock per SM).
// Build and run:  nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o ubench ubench_instruction_rates.cu && ./ubench
#include <cstdio>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#define ITERS 4096
#define NACC 8
template <int OP> __global__ void __launch_bounds__(256) k(unsigned* out, unsigned seed, long long* clk) {
    unsigned a[NACC]; float f[NACC]; float2 g[NACC];
    for (int i = 0; i < NACC; i++) { a[i] = seed + i * 77 + threadIdx.x; f[i] = (float)(seed + i) * 1e-3f; g[i] = make_float2(f[i], f[i] + 1.f); }
    unsigned m1 = seed | 0x0F0F0F0F, m2 = seed * 3 + 1;
    float c1 = __uint_as_float(seed + 0x3f800000), c2 = 0.999f;
    float2 c3 = make_float2(c1, c2);
    long long t0 = clock64();
#pragma unroll 1
    for (int it = 0; it < ITERS; it++) {
#pragma unroll
        for (int i = 0; i < NACC; i++) {
            if (OP == 0) a[i] = (a[i] & m1) ^ m2;                       // LOP3
            if (OP == 1) a[i] = __dp4a((int)a[i], (int)m1, (int)a[i]);  // IDP4A
            if (OP == 2) f[i] = fmaf(f[i], c1, c2);                     // FFMA
            if (OP == 3) g[i] = __ffma2_rn(g[i], c3, c3);               // FFMA2
            if (OP == 4) a[i] = (a[i] >> 3) + m2;                       // SHF+IADD -> lea?
            if (OP == 5) a[i] = a[i] * m1 + m2;                         // IMAD
            if (OP == 6) f[i] = (float)(int)(signed char)(__float_as_uint(f[i]) >> 8) + c2;  // I2F.S8 + FADD
            if (OP == 7) a[i] = __byte_perm(a[i], m1, m2);              // PRMT
            if (OP == 8) f[i] = fmaf(__uint_as_float(__float_as_uint(f[i]) & 0xFF), c1, f[i]); // subnormal FFMA (+LOP)
            if (OP == 9) a[i] = a[i] >> 16;                             // SHF
            if (OP == 10) { __half2 h = *reinterpret_cast<__half2*>(&a[i]); h = __hfma2(h, h, h); a[i] = *reinterpret_cast<unsigned*>(&h); } // HFMA2
            if (OP == 11) { float2 t = __half22float2(*reinterpret_cast<__half2*>(&a[i])); a[i] = __float_as_uint(t.x + t.y); } // cvt f16x2->f32 x2 + FADD
            if (OP == 12) a[i] = a[i] + m2;                             // IADD
            if (OP == 13) f[i] = (float)(int)a[i] , a[i] += __float_as_uint(f[i]); // I2F + IADD
        }
    }
    long long t1 = clock64();
    unsigned r = 0; float fr = 0;
    for (int i = 0; i < NACC; i++) { r ^= a[i]; fr += f[i] + g[i].x + g[i].y; }
    out[blockIdx.x * blockDim.x + threadIdx.x] = r ^ __float_as_uint(fr);
    if (threadIdx.x == 0) clk[blockIdx.x] = t1 - t0;
}
template <int OP> void run(const char* name, int opsPer) {
    unsigned* out; long long* clk; int blocks = 148 * 4, threads = 256;
    cudaMalloc(&out, blocks * threads * 4); cudaMalloc(&clk, blocks * 8);
    k<OP><<<blocks, threads>>>(out, 12345, clk); cudaDeviceSynchronize();
    k<OP><<<blocks, threads>>>(out, 12345, clk); cudaDeviceSynchronize();
    long long h[148 * 4]; cudaMemcpy(h, clk, blocks * 8, cudaMemcpyDeviceToHost);
    double avg = 0; for (int i = 0; i < blocks; i++) avg += h[i]; avg /= blocks;
    // per SM: 4 blocks * 256 threads resident; ops per thread = ITERS*NACC*opsPer
    double ops_per_clk_sm = 4.0 * 256 * ITERS * NACC * opsPer / avg;
    printf("%-28s %8.1f thread-ops/clk/SM  (%.0f cycles)\n", name, ops_per_clk_sm, avg);
    cudaFree(out); cudaFree(clk);
}
int main() {
    run<0>("LOP3", 1); run<1>("IDP4A", 1); run<2>("FFMA", 1); run<3>("FFMA2 (2 fma each)", 2);
    run<4>("SHF+IADD", 2); run<5>("IMAD", 1); run<6>("I2F.S8+FADD (pair)", 1); run<7>("PRMT", 1);
    run<8>("LOP+FFMA subnormal (pair)", 1); run<9>("SHF", 1); run<10>("HFMA2 (2 each)", 2);
    run<11>("cvt f16x2->f32x2 + FADD", 1); run<12>("IADD", 1); run<13>("I2F+IADD (pair)", 1);
    return 0;
}
