// Instruction-throughput probe for sm_100a: thread-ops per clock per SM of the few instructions the fused
// RMSNorm + MXFP8 quantiser and the decode GEMV are built from (each kernel runs 4096 x 8 independent chains per
// thread, 8 blocks of 256 threads per SM; the clock is taken as the device's nominal maximum, so the figures are
// lower bounds).  Build and run: python -m prime_kernels_b200.rmsnorm.pipe_rates
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>

#define ITERS 4096
template <int OP>
__global__ void __launch_bounds__(256) rate_kernel(uint32_t* out, uint32_t seed, float fs) {
    uint32_t a[8];
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = seed * (threadIdx.x + 1) + i * 0x3f803f80u; f[i] = fs * (float)(threadIdx.x + i); }
    const uint32_t w = seed | 0x3f803f80u;
    for (int it = 0; it < ITERS; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (OP == 0) {            // mixed precision fma.rn.f32.bf16
                uint16_t al = (uint16_t)a[i], bl = (uint16_t)w;
                asm volatile("fma.rn.f32.bf16 %0, %1, %2, %0;" : "+f"(f[i]) : "h"(al), "h"(bl));
            } else if (OP == 1) {     // plain FFMA
                asm volatile("fma.rn.f32 %0, %1, %2, %0;" : "+f"(f[i]) : "f"(fs), "f"(fs));
            } else if (OP == 2) {     // unpack by shift + FFMA
                float x = __uint_as_float(a[i] << 16);
                asm volatile("fma.rn.f32 %0, %1, %2, %0;" : "+f"(f[i]) : "f"(x), "f"(fs));
                a[i] += 0x10001u;
            } else if (OP == 3) {     // cvt e4m3x2 from two f32
                uint16_t r;
                asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(f[i]), "f"(fs));
                f[i] = __uint_as_float(0x3f800000u | r);
            } else if (OP == 4) {     // cvt bf16x2 pack from two f32
                uint32_t r;
                asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(f[i]), "f"(fs));
                f[i] = __uint_as_float(0x3f800000u ^ (r >> 9));
            } else if (OP == 5) {     // max.bf16x2
                asm volatile("max.bf16x2 %0, %0, %1;" : "+r"(a[i]) : "r"(w));
            } else if (OP == 6) {     // abs.bf16x2
                asm volatile("abs.bf16x2 %0, %0;" : "+r"(a[i]));
            } else if (OP == 7) {     // e8m0 round-up conversion
                uint16_t r;
                asm volatile("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(r) : "f"(fs), "f"(f[i]));
                f[i] = __uint_as_float(0x3f800000u | r);
            } else if (OP == 8) {     // e4m3x2 from f16x2
                uint16_t r;
                asm volatile("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(a[i]));
                a[i] = 0x3c003c00u | r;
            } else if (OP == 9) {     // fma.rn.bf16x2
                asm volatile("fma.rn.bf16x2 %0, %0, %1, %1;" : "+r"(a[i]) : "r"(w));
            } else if (OP == 10) {    // mul.rn.bf16x2 (scaling)
                asm volatile("mul.rn.bf16x2 %0, %0, %1;" : "+r"(a[i]) : "r"(w));
            } else if (OP == 11) {    // prmt unpack hi + lo (2 ops)
                uint32_t lo, hi;
                asm volatile("prmt.b32 %0, %1, 0, 0x1044;" : "=r"(lo) : "r"(a[i]));
                asm volatile("prmt.b32 %0, %1, 0, 0x3244;" : "=r"(hi) : "r"(a[i]));
                a[i] = lo ^ hi ^ w;
            } else if (OP == 13) {    // abs by mask (LOP3)
                asm volatile("and.b32 %0, %0, %1;" : "+r"(a[i]) : "r"(w));
            } else if (OP == 14) {    // cvt.rn.bf16.f32 single + widen back
                uint16_t r;
                asm volatile("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f[i]));
                f[i] = __uint_as_float(((uint32_t)r << 16) | 0x1234u);
            } else if (OP == 15) {    // MUFU rsqrt
                asm volatile("rsqrt.approx.f32 %0, %0;" : "+f"(f[i]));
            } else if (OP == 16) {    // shfl xor
                asm volatile("shfl.sync.bfly.b32 %0, %0, 1, 0x1f, 0xffffffff;" : "+r"(a[i]));
            } else if (OP == 17) {    // fmul by constant
                asm volatile("mul.rn.f32 %0, %0, %1;" : "+f"(f[i]) : "f"(fs));
            } else if (OP == 18) {    // max.f32
                asm volatile("max.f32 %0, %0, %1;" : "+f"(f[i]) : "f"(fs));
            } else if (OP == 12) {    // mixed fma.rn.f32.f16
                uint16_t al = (uint16_t)a[i], bl = (uint16_t)w;
                asm volatile("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(f[i]) : "h"(al), "h"(bl));
            }
        }
    }
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc ^= a[i] ^ __float_as_uint(f[i]);
    out[blockIdx.x * blockDim.x + threadIdx.x] = acc;
}

template <int OP>
void run(const char* name, int ops_per_iter) {
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0);
    uint32_t* out;
    const int blocks = sms * 8;
    cudaMalloc(&out, (size_t)blocks * 256 * 4);
    rate_kernel<OP><<<blocks, 256>>>(out, 3u, 1.0001f);
    cudaDeviceSynchronize();
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0);
    rate_kernel<OP><<<blocks, 256>>>(out, 3u, 1.0001f);
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    const double ops = (double)blocks * 256 * ITERS * 8 * ops_per_iter;
    // clocks at the nominal max (an upper bound on the real clock, so the figure is a lower bound)
    printf("%-28s %8.3f ms  %7.1f Gops/s  ~%6.1f thread-ops/clk/SM at %d MHz (err %d)\n", name, ms, ops / ms * 1e-6,
           ops / (ms * 1e-3) / ((double)khz * 1e3) / sms, khz / 1000, (int)cudaGetLastError());
    cudaFree(out);
}

int main() {
    run<1>("fma.rn.f32 (FFMA)", 1);
    run<0>("fma.rn.f32.bf16 (mixed)", 1);
    run<12>("fma.rn.f32.f16 (mixed)", 1);
    run<2>("shl + FFMA + IADD", 1);
    run<3>("cvt e4m3x2.f32 (+xor)", 1);
    run<8>("cvt e4m3x2.f16x2 (+xor)", 1);
    run<4>("cvt bf16x2.f32 (+xor)", 1);
    run<7>("cvt ue8m0x2.f32 (+xor)", 1);
    run<5>("max.bf16x2", 1);
    run<6>("abs.bf16x2", 1);
    run<9>("fma.rn.bf16x2", 1);
    run<10>("mul.rn.bf16x2", 1);
    run<11>("2x prmt + 2 xor", 1);
    run<14>("cvt bf16.f32 + shl/or", 1);
    run<15>("rsqrt.approx", 1);
    run<16>("shfl.bfly", 1);
    run<17>("mul.rn.f32", 1);
    run<18>("max.f32", 1);
    return 0;
}
