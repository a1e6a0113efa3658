// Instruction-throughput probe: the roofline denominators of bench.py.
//
// Register-only kernels (no memory traffic, every operand loop carried so nothing can be hoisted) time the
// instruction mixes the morphology kernels are made of, in units per second over the whole GPU:
//   a dilation / erosion tap is one add and one max (float: also with the 3-input max and the packed
//   add.f32x2 of sm_100; double: with fmax and with compare + select), a smorph tap is one ex2.
// Every kernel also samples the SM clock while it runs: thread 0 of each block reads the SM cycle counter and the
// device's nanosecond timer at its start and end, and the host averages cycles / nanoseconds over the blocks. The
// per-clock figures below divide by that sampled clock, not by the nominal maximum.
// Prints one JSON object {name: Gunits/s, "per_clk_sm": {name: units per sampled clock per SM}, "sm_mhz": {name: MHz}}.
// Usage: probe_rates  (runs for about 100 ms on the current GPU).
#include <cstdio>
#include <cuda_runtime.h>
#define CHAINS 16
#define ITERS 2048

__device__ __forceinline__ float max3(float a, float b, float c) { float d; asm volatile("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
__device__ __forceinline__ float min3(float a, float b, float c) { float d; asm volatile("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }

__device__ __forceinline__ unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

template <int KIND> __global__ void probe(float* out, float w0, float w1, unsigned long long* stamps)
{
    const long long c0 = clock64();
    const unsigned long long t0 = global_ns();
    float acc[CHAINS], x[CHAINS], x2[CHAINS];
    double dacc[CHAINS], dx[CHAINS];
    int idx[CHAINS];
    for (int i = 0; i < CHAINS; i++) { acc[i] = -1e30f + threadIdx.x; x[i] = threadIdx.x * 0.001f + i; x2[i] = x[i] * 0.5f; dacc[i] = acc[i]; dx[i] = x[i]; idx[i] = 0; }
    #pragma unroll 4
    for (int it = 0; it < ITERS; it++)
    {
        #pragma unroll
        for (int i = 0; i < CHAINS; i++)
        {
            if (KIND == 0) { x[i] += w0; acc[i] = fmaxf(acc[i], x[i]); }                                   // 1 tap: add + max
            if (KIND == 1) { x[i] += w0; x2[i] += w1; acc[i] = max3(acc[i], x[i], x2[i]); }               // 2 taps: 2 add + max3
            if (KIND == 2) { acc[i] = fmaxf(acc[i], x[i]); x[i] = fminf(x[i], acc[(i + 3) % CHAINS]); }   // 2 minmax
            if (KIND == 3) { acc[i] += w0; x[i] += w1; }                                                    // 2 add
            if (KIND == 4) { acc[i] = fmaf(acc[i], w0, w1); x[i] = fmaf(x[i], w1, w0); }                   // 2 fma
            if (KIND == 5) { acc[i] = max3(acc[i], x[i], x2[i]); x[i] = min3(x[i], x2[(i + 1) % CHAINS], acc[(i + 3) % CHAINS]); } // 2 minmax3
            if (KIND == 6) { dx[i] += (double)w0; dacc[i] = fmax(dacc[i], dx[i]); }                        // fp64 tap: add + fmax
            if (KIND == 7) { float e; asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(acc[i])); acc[i] = e; } // 1 ex2
            if (KIND == 9) { dacc[i] += (double)w0; dx[i] += (double)w1; }                                 // 2 dadd
            if (KIND == 10) { dx[i] += (double)w0; dacc[i] = dx[i] > dacc[i] ? dx[i] : dacc[i]; }          // fp64 tap: add + compare/select
            if (KIND == 11) { x[i] += w0; const bool p = x[i] > acc[i]; acc[i] = p ? x[i] : acc[i]; idx[i] = p ? it : idx[i]; } // tracked tap
            if (KIND == 12) { x[i] += w0; acc[i] = fmaxf(acc[i], x[i]); idx[i] = (acc[i] == x[i]) ? it : idx[i]; } // tracked via max + eq
            if (KIND == 13) { x[i] = fmaf(x[i], w0, w1); x2[i] = fmaf(x2[i], w1, w0); acc[i] = fmaf(acc[i], w0, x[i]); } // 3 fma
            if (KIND == 15) { acc[i] = fmaf(acc[i], w0, x[i]); x2[i] = fmaf(x2[i], w1, x[i]); }            // 2 fma, two register sources + one constant each
            if (KIND == 14) { dx[i] += (double)w0; const long long a = __double_as_longlong(dx[i]), b = __double_as_longlong(dacc[i]); dacc[i] = __longlong_as_double(a > b ? a : b); } // fp64 add + int64 max
        }
        if (KIND == 8)  // packed add.f32x2 + max3: 2 taps x 2 pixels
        {
            #pragma unroll
            for (int i = 0; i < CHAINS; i += 2)
            {
                unsigned long long xa, xb, wa, wb;
                asm volatile("mov.b64 %0, {%1, %2};" : "=l"(xa) : "f"(x[i]), "f"(x[i + 1]));
                asm volatile("mov.b64 %0, {%1, %2};" : "=l"(xb) : "f"(x2[i]), "f"(x2[i + 1]));
                asm volatile("mov.b64 %0, {%1, %1};" : "=l"(wa) : "f"(w0));
                asm volatile("mov.b64 %0, {%1, %1};" : "=l"(wb) : "f"(w1));
                asm volatile("add.f32x2 %0, %1, %2;" : "=l"(xa) : "l"(xa), "l"(wa));
                asm volatile("add.f32x2 %0, %1, %2;" : "=l"(xb) : "l"(xb), "l"(wb));
                asm volatile("mov.b64 {%0, %1}, %2;" : "=f"(x[i]), "=f"(x[i + 1]) : "l"(xa));
                asm volatile("mov.b64 {%0, %1}, %2;" : "=f"(x2[i]), "=f"(x2[i + 1]) : "l"(xb));
                acc[i] = max3(acc[i], x[i], x2[i]);
                acc[i + 1] = max3(acc[i + 1], x[i + 1], x2[i + 1]);
            }
        }
    }
    float s = 0; for (int i = 0; i < CHAINS; i++) s += acc[i] + (float)dacc[i] + x[i] + x2[i] + (float)dx[i] + idx[i];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
    if (threadIdx.x == 0)
    {
        stamps[2 * blockIdx.x] = static_cast<unsigned long long>(clock64() - c0);
        stamps[2 * blockIdx.x + 1] = global_ns() - t0;
    }
}

struct Rate { double gunits; double mhz; };


template <int KIND> Rate run(double units)
{
    int blocks = 148 * 8, threads = 256;
    float* out; cudaMalloc(&out, blocks * threads * 4);
    unsigned long long* stamps; cudaMalloc(&stamps, blocks * 2 * sizeof(unsigned long long));
    for (int i = 0; i < 3; i++) probe<KIND><<<blocks, threads>>>(out, 0.5f, 0.25f, stamps);
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0);
    for (int i = 0; i < 5; i++) probe<KIND><<<blocks, threads>>>(out, 0.5f, 0.25f, stamps);
    cudaEventRecord(e1); cudaDeviceSynchronize();
    float ms; cudaEventElapsedTime(&ms, e0, e1); ms /= 5;
    static unsigned long long host[148 * 8 * 2];
    cudaMemcpy(host, stamps, sizeof(host), cudaMemcpyDeviceToHost);   // stamps of the last launch
    double cycles = 0, ns = 0;
    for (int b = 0; b < blocks; b++) { cycles += (double)host[2 * b]; ns += (double)host[2 * b + 1]; }
    cudaFree(out); cudaFree(stamps); cudaEventDestroy(e0); cudaEventDestroy(e1);
    Rate r;
    r.gunits = (double)blocks * threads * ITERS * CHAINS * units / ms / 1e6;
    r.mhz = ns > 0 ? cycles / ns * 1e3 : 0.0;
    return r;
}

int main()
{
    if (cudaFree(0) != cudaSuccess) { printf("{\"error\": \"no CUDA device\"}\n"); return 1; }
    run<3>(2);  // warm up, clocks to their maximum
    const char* names[] = {"add_max_taps", "add_max3_taps", "add2_max3_taps", "minmax_ops", "add_ops", "fma_ops", "fma2_ops", "tracked_argmax_taps",
                           "ex2_ops", "f64_add_fmax_taps", "f64_add_select_taps", "f64_add_ops"};
    const Rate r[] = {run<0>(1), run<1>(2), run<8>(2), run<2>(2), run<3>(2), run<13>(3), run<15>(2), run<11>(1), run<7>(1), run<6>(1), run<10>(1), run<9>(2)};
    const int n = sizeof(r) / sizeof(r[0]);
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    printf("{");
    for (int i = 0; i < n; i++) printf("\"%s\": %.1f, ", names[i], r[i].gunits);
    printf("\"per_clk_sm\": {");
    for (int i = 0; i < n; i++) printf("\"%s\": %.2f%s", names[i], r[i].mhz > 0 ? r[i].gunits * 1e3 / r[i].mhz / sms : 0.0, i + 1 < n ? ", " : "");
    printf("}, \"sm_mhz\": {");
    for (int i = 0; i < n; i++) printf("\"%s\": %.0f%s", names[i], r[i].mhz, i + 1 < n ? ", " : "");
    printf("}}\n");
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
