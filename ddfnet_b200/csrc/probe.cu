// Diagnostic entry points: the launch floor and the issue rates of the instructions the DDF
// kernels are made of.  The roofline statements in the project's documentation rest on
// these measurements; `python bench.py --workload probe` prints them.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ddf_b200.h"

namespace ddf {

__global__ void noop_kernel() {}

// Every thread runs `iters` rounds of 64 independent-chain instructions of one kind.
//   0  float FMA, the same two multiplicands every time (operand-reuse cache hits)
//   1  float FMA, three distinct register operands per instruction
//   2  mixed-precision FMA (bf16 x bf16 + f32), distinct operands, halves selected both ways
//   3  mixed-precision FMA (f16 x f16 + f32), distinct operands
//   4  packed fma.rn.f32x2, distinct operands
//   5  lop3 (integer pipe)
template <int MODE>
__global__ void __launch_bounds__(512) rate_kernel(const uint32_t* in, float* out, int iters) {
    uint32_t x[16], s[16];
    float acc[16], fx[16], fs[16];
    unsigned long long a2[16], p2[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        x[i] = in[threadIdx.x + 512 * i];
        s[i] = in[threadIdx.x + 512 * (16 + i)];
        fx[i] = __uint_as_float(x[i]);
        fs[i] = __uint_as_float(s[i]);
        acc[i] = 0.f;
        a2[i] = 0ull;
        p2[i] = ((unsigned long long)x[i] << 32) | s[i];
    }
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int j = (i + r * 5) & 15;
                if (MODE == 0) {
                    acc[i] = fmaf(acc[i], fx[0], fs[0]);
                } else if (MODE == 1) {
                    acc[i] = fmaf(fx[i], fs[j], acc[i]);
                } else if (MODE == 2) {
                    if (r & 1)
                        asm volatile("{\n\t.reg .b16 a, b, c, d;\n\tmov.b32 {a,b}, %1;\n\tmov.b32 {c,d}, %2;\n\t"
                                     "fma.rn.f32.bf16 %0, b, c, %0;\n\t}" : "+f"(acc[i]) : "r"(x[i]), "r"(s[j]));
                    else
                        asm volatile("{\n\t.reg .b16 a, b, c, d;\n\tmov.b32 {a,b}, %1;\n\tmov.b32 {c,d}, %2;\n\t"
                                     "fma.rn.f32.bf16 %0, a, d, %0;\n\t}" : "+f"(acc[i]) : "r"(x[i]), "r"(s[j]));
                } else if (MODE == 3) {
                    asm volatile("{\n\t.reg .b16 a, b, c, d;\n\tmov.b32 {a,b}, %1;\n\tmov.b32 {c,d}, %2;\n\t"
                                 "fma.rn.f32.f16 %0, a, d, %0;\n\t}" : "+f"(acc[i]) : "r"(x[i]), "r"(s[j]));
                } else if (MODE == 4) {
                    asm volatile("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(a2[i]) : "l"(p2[i]), "l"(p2[j]));
                } else {
                    asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(x[i]) : "r"(s[j]), "r"(s[i]));
                }
            }
        }
    }
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) t += acc[i] + (float)(a2[i] & 0xff) + (float)(x[i] & 0xff);
    out[blockIdx.x * blockDim.x + threadIdx.x] = t;
}

template <int MODE>
static cudaError_t run_rate(const uint32_t* in, float* out, int grid, int iters, cudaStream_t st) {
    rate_kernel<MODE><<<grid, 512, 0, st>>>(in, out, iters);
    return cudaGetLastError();
}

}  // namespace ddf

extern "C" {

int ddf_b200_noop(void* stream) {
    ddf::noop_kernel<<<148, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>();
    return (int)cudaGetLastError();
}

size_t ddf_b200_rate_probe_bytes(void) { return (size_t)512 * 32 * 4 + (size_t)148 * 4 * 512 * 4; }

int ddf_b200_rate_probe(int mode, void* scratch, size_t scratch_bytes, int iters,
                        double* warp_instr_per_ns_per_sm, void* stream) {
    using namespace ddf;
    if (!scratch || !warp_instr_per_ns_per_sm) return DDF_B200_E_NULL;
    if (scratch_bytes < ddf_b200_rate_probe_bytes() || iters < 1 || mode < 0 || mode > 5) return DDF_B200_E_SHAPE;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    if (sms > 148 * 2) return DDF_B200_E_DEVICE;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const uint32_t* in = reinterpret_cast<const uint32_t*>(scratch);
    float* out = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + (size_t)512 * 32 * 4);
    const int grid = sms * 2;
    auto launch = [&](int n) -> cudaError_t {
        switch (mode) {
            case 0: return run_rate<0>(in, out, grid, n, st);
            case 1: return run_rate<1>(in, out, grid, n, st);
            case 2: return run_rate<2>(in, out, grid, n, st);
            case 3: return run_rate<3>(in, out, grid, n, st);
            case 4: return run_rate<4>(in, out, grid, n, st);
            default: return run_rate<5>(in, out, grid, n, st);
        }
    };
    cudaEvent_t e0, e1;
    if ((e = cudaEventCreate(&e0)) != cudaSuccess) return (int)e;
    if ((e = cudaEventCreate(&e1)) != cudaSuccess) { cudaEventDestroy(e0); return (int)e; }
    e = cudaMemsetAsync(scratch, 0x3c, (size_t)512 * 32 * 4, st);
    if (e == cudaSuccess) e = launch(8);
    if (e == cudaSuccess) e = cudaEventRecord(e0, st);
    if (e == cudaSuccess) e = launch(iters);
    if (e == cudaSuccess) e = cudaEventRecord(e1, st);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) return (int)e;
    const double warp_instr = (double)grid * 16.0 * iters * 64.0;
    *warp_instr_per_ns_per_sm = warp_instr / sms / ((double)ms * 1e6);
    return 0;
}

}  // extern "C"
