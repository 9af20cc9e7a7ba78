// hx_probe.cu -- what the tensor pipe can issue for the MMA this library uses: tcgen05.mma kind::mxf4nvf4
// block_scale block16, M = 128, K = 64, N = ncols, both operands resident in shared memory, optionally with the four
// tcgen05.cp scale-factor copies a weight cell needs.  One thread per SM issues `iters` cells of four MMAs through a
// ring of eight commit barriers and the cycles are read from clock64.  The figure is the denominator of the
// tensor-side roofline of the batched GEMM (no vendor figure exists for this MMA shape at small N), and shows why
// the N = 16 decode formulation cannot run ahead of HBM.  Measurement only: no data leaves the kernel.
#include "hx_common.cuh"

namespace {

constexpr int PB_CELL = 18432, PB_NCELL = 8, PB_WAIT = 1 << 22;

__device__ __forceinline__ uint32_t pb_s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t pb_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
           (1ull << 46) | ((uint64_t)layout << 61);
}
__device__ __forceinline__ bool pb_try(uint64_t* b, uint32_t par) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(pb_s32(b)), "r"(par) : "memory");
    return ok != 0;
}

__global__ void __launch_bounds__(128, 1) k_probe_mxf4(int iters, int ncols, int with_sf, long long* out, int* err) {
    extern __shared__ __align__(1024) uint8_t pb_sm[];
    __shared__ uint64_t bar[PB_NCELL];
    __shared__ uint32_t tbase;
    uint8_t* ring = (uint8_t*)(((uintptr_t)pb_sm + 1023) & ~(uintptr_t)1023);
    uint8_t* bop = ring + PB_NCELL * PB_CELL;          // B operand: up to 256 rows x 128 B
    const int tid = threadIdx.x;
    for (int i = tid; i < (PB_NCELL * PB_CELL + 256 * 128) / 4; i += 128) ((uint32_t*)ring)[i] = 0x38383838u;   // scale 1.0 everywhere
    if (tid == 0) for (int i = 0; i < PB_NCELL; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(pb_s32(&bar[i])));
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (tid < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"(pb_s32(&tbase)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tbase;
    if (tid == 0) {
        const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(ncols >> 3) << 17) | (8u << 24);
        const uint64_t a_ring = pb_desc(pb_s32(ring), 16, 1024, 2), sf_ring = pb_desc(pb_s32(ring) + 16384, 16, 128, 0);
        const uint64_t b_base = pb_desc(pb_s32(bop), 16, 1024, 2);
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(tmem + 300), "l"(sf_ring) : "memory");
        const long long t0 = clock64();
        bool ok = true;
        for (int it = 0; it < iters && ok; it++) {
            const int slot = it % PB_NCELL;
            if (it >= PB_NCELL) {                        // the slot's previous MMAs must be complete before its reuse
                const uint32_t par = ((it / PB_NCELL) - 1) & 1;
                int n = 0;
                while (!pb_try(&bar[slot], par)) if (++n > PB_WAIT) { ok = false; *err = 1; break; }
            }
            const uint64_t a_slot = a_ring + (uint64_t)(slot * (PB_CELL >> 4)), sf_slot = sf_ring + (uint64_t)(slot * (PB_CELL >> 4));
            const uint32_t tsf = tmem + 320 + slot * 16;
            if (with_sf)
                for (int e = 0; e < 4; e++)
                    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(tsf + e * 4), "l"(sf_slot + (uint64_t)(e * 32)) : "memory");
            for (int e = 0; e < 4; e++) {
                const uint32_t acc = it > 0 || e > 0;
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                             :: "r"(tmem), "l"(a_slot + (uint64_t)(e * 2)), "l"(b_base + (uint64_t)(e * 2)), "r"(idesc), "r"(acc),
                                "r"(tsf + e * 4), "r"(tmem + 300) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(pb_s32(&bar[slot])) : "memory");
        }
        for (int j = 0; j < PB_NCELL && ok; j++) {        // drain: every commit still in flight
            const int it = iters - PB_NCELL + j;
            if (it < 0) continue;
            const uint32_t par = (it / PB_NCELL) & 1;
            int n = 0;
            while (!pb_try(&bar[it % PB_NCELL], par)) if (++n > PB_WAIT) { *err = 1; break; }
        }
        if (blockIdx.x == 0) out[0] = clock64() - t0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tmem) : "memory");
}

}  // namespace

// clk_per_mma: SM cycles per M128 x N x K64 MMA (a quarter of a cell, scale copies included when asked for);
// tflops: 2*128*N*64 flop per MMA on every SM at the device's current SM clock.
HX_API int hx_probe_mxf4_rate(int ncols, int with_scale_copies, double* clk_per_mma, double* tflops) {
    HX_CHECK_ARG(ncols >= 16 && ncols <= 256 && ncols % 16 == 0 && clk_per_mma && tflops);
    int dev = 0, sms = 0, khz = 0;
    HX_CUDA(cudaGetDevice(&dev));
    HX_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    HX_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
    long long* out = nullptr; int* err = nullptr;
    HX_CUDA(cudaMalloc(&out, 64));
    if (cudaMalloc(&err, 4) != cudaSuccess) { cudaFree(out); return hx_fail(HX_ERR_NOMEM, "probe: allocation failed"); }
    cudaMemset(err, 0, 4);
    const size_t smem = (size_t)PB_NCELL * PB_CELL + 256 * 128 + 2048;
    cudaError_t e = cudaFuncSetAttribute(k_probe_mxf4, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int iters = 4000;
    long long cyc = 0; int herr = 0;
    for (int rep = 0; rep < 2 && e == cudaSuccess; rep++) {
        k_probe_mxf4<<<sms, 128, smem>>>(iters, ncols, with_scale_copies ? 1 : 0, out, err);
        HX_COUNT_LAUNCH(1);
        e = cudaDeviceSynchronize();
    }
    if (e == cudaSuccess) e = cudaMemcpy(&cyc, out, 8, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost);
    cudaFree(out); cudaFree(err);
    if (e != cudaSuccess) return hx_fail(HX_ERR_CUDA, "probe: %s", cudaGetErrorString(e));
    if (herr) return hx_fail(HX_ERR_TIMEOUT, "probe: a bounded wait for an MMA commit ran out");
    *clk_per_mma = (double)cyc / iters / 4.0;
    *tflops = 2.0 * 128.0 * ncols * 64.0 / *clk_per_mma * (double)khz * 1e3 * sms / 1e12;
    return HX_OK;
}
