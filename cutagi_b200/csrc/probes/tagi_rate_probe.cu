// Peak probes for the roofline denominators of the TAGI kernels (not part of the library):
//   1. cycles per tcgen05.mma kind::tf32 (128 x N x 8) for several N, A operand from shared or tensor memory, one or two
//      accumulators, issued by one thread: gives the tensor pipe's tf32 rate (N / 2 cycles = 2048 FMA per clock and SM)
//      and the issue limit of a single thread;
//   2. FP32 FFMA throughput of the whole GPU with eight independent FMA chains per thread.
// Build and run on a B200:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_rate_probe tagi_rate_probe.cu && ./mma_rate_probe
// Every wait is bounded; zero operands.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "../tagi_tc_ptx.cuh"
using namespace tagi::ptx;

template <int TS>
__global__ void __launch_bounds__(128, 1) probe(int n, int nmma, int ndst, long long *out) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar;
    __shared__ uint32_t slot;
    __shared__ int abort_flag;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    // zero operands
    for (int i = threadIdx.x; i < 16384; i += 128) reinterpret_cast<float *>(smem_raw)[i] = 0.f;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag = 0; mbar_init_fence(); }
    if (threadIdx.x < 32) tmem_alloc(&slot, 512);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = slot;
    if (threadIdx.x == 0) {
        const uint32_t idesc = make_idesc_tf32(128, n, 0, 0);
        const uint64_t da = make_smem_desc(base, 16, 512, SWZ_64B);
        const uint64_t db = make_smem_desc(base + 8192, 16, 512, SWZ_64B);
        long long t0 = clock64();
        const uint32_t dstep = (ndst == 1 ? 0 : (n <= 128 ? 128 : 256));
        const uint32_t dA = tmem, dB = tmem + dstep;
        const uint32_t a0 = tmem + 448, a1 = tmem + 456;
#pragma unroll 1
        for (int i = 0; i < nmma; i += 8) {
            if (TS) {
                mma_tf32_ts(dA, a0, db, idesc, 1); mma_tf32_ts(dB, a1, db + 2, idesc, 1);
                mma_tf32_ts(dA, a0, db, idesc, 1); mma_tf32_ts(dB, a1, db + 2, idesc, 1);
                mma_tf32_ts(dA, a0, db, idesc, 1); mma_tf32_ts(dB, a1, db + 2, idesc, 1);
                mma_tf32_ts(dA, a0, db, idesc, 1); mma_tf32_ts(dB, a1, db + 2, idesc, 1);
            } else {
                mma_tf32_ss(dA, da, db, idesc, 1); mma_tf32_ss(dB, da + 2, db + 2, idesc, 1);
                mma_tf32_ss(dA, da, db, idesc, 1); mma_tf32_ss(dB, da + 2, db + 2, idesc, 1);
                mma_tf32_ss(dA, da, db, idesc, 1); mma_tf32_ss(dB, da + 2, db + 2, idesc, 1);
                mma_tf32_ss(dA, da, db, idesc, 1); mma_tf32_ss(dB, da + 2, db + 2, idesc, 1);
            }
        }
        long long t1 = clock64();
        mma_commit(&bar);
        int st = 0;
        mbar_wait(&bar, 0, &abort_flag, &st, 1);
        long long t2 = clock64();
        out[0] = t1 - t0;
        out[1] = t2 - t0;
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

__global__ void __launch_bounds__(256) ffma_probe(float *out, int iters) {
    float a[8], x = 1.0000001f, y = 1e-9f;
#pragma unroll
    for (int i = 0; i < 8; i++) a[i] = threadIdx.x * 1e-6f + i;
    for (int it = 0; it < iters; it++)
#pragma unroll
        for (int i = 0; i < 8; i++) a[i] = fmaf(a[i], x, y);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) s += a[i];
    if (s == 123.456f) out[0] = s;  // never true; keeps the chains alive
}

int main() {
    long long *out;
    cudaMalloc(&out, 16);
    {
        float *fo;
        cudaMalloc(&fo, 4);
        cudaDeviceProp prop;
        cudaGetDeviceProperties(&prop, 0);
        const int blocks = prop.multiProcessorCount * 8, iters = 1 << 16;
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        ffma_probe<<<blocks, 256>>>(fo, iters);
        cudaEventRecord(e0);
        ffma_probe<<<blocks, 256>>>(fo, iters);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        printf("FP32 FFMA: %.1f TFLOP/s (%d SMs, %d threads, %d x 8 FMA each, %.3f ms)\n",
               2.0 * blocks * 256.0 * iters * 8 / (ms * 1e-3) / 1e12, prop.multiProcessorCount, blocks * 256, iters, ms);
    }
    cudaFuncSetAttribute(probe<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100000);
    cudaFuncSetAttribute(probe<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100000);
    const int nmma = 4096;
    for (int ts = 0; ts < 2; ts++)
        for (int ndst = 1; ndst <= 2; ndst++)
            for (int n : {64, 96, 112, 128, 192, 256}) {
                if (ndst == 2 && n > 256) continue;
                if (ndst == 2 && n == 256 && ts) continue;  // no room for A
                long long h[2];
                for (int rep = 0; rep < 2; rep++) {
                    if (ts) probe<1><<<1, 128, 100000>>>(n, nmma, ndst, out);
                    else probe<0><<<1, 128, 100000>>>(n, nmma, ndst, out);
                    cudaError_t e = cudaDeviceSynchronize();
                    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
                    cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost);
                }
                printf("A=%s ndst=%d N=%3d: issue %.1f clk/mma, complete %.1f clk/mma (ideal %.1f at 2048 FMA/clk)\n",
                       ts ? "tmem" : "smem", ndst, n, (double)h[0] / nmma, (double)h[1] / nmma, 128.0 * n * 8 / 2048);
            }
    return 0;
}
