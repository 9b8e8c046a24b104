// Shared device helpers for the sm_100a flash-GQA kernels: status word, mbarrier, TMA, MMA wrappers.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cllo_flash_gqa.h"

namespace cllo {

// ---------------------------------------------------------------------------------------------
// Device status word.  A wait that runs out of time records where it happened instead of
// trapping; the host reads it through cllo_device_status().
// ---------------------------------------------------------------------------------------------
static __device__ int g_status[4];  // {code, block, site, aux}

enum : int {
    SITE_DECODE_FULL = 1,
    SITE_DECODE_EMPTY = 2,
    SITE_DECODE_DRAIN = 3,
    SITE_DECODE_ISSUE = 4,
    SITE_EXCHANGE_FLAG = 8,
    SITE_PREFILL_BASE = 16,
};

__device__ __forceinline__ void record_timeout(int site, int aux) {
    if (atomicCAS(&g_status[0], 0, CLLO_E_DEVICE_TIMEOUT) == 0) {
        g_status[1] = static_cast<int>(blockIdx.x);
        g_status[2] = site;
        g_status[3] = aux;
    }
}

// Upper bound for any single wait, in SM clock cycles (about one second).
constexpr long long kWaitLimitCycles = 2000000000LL;

// ---------------------------------------------------------------------------------------------
// Shared-memory addresses and mbarriers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  `abort_flag` (shared memory) short-circuits every later wait of the block once
// one wait has given up, so control flow stays intact (all barriers are still reached) and the
// kernel ends quickly with the status word set.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int site,
                                          int aux) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
        if (mbar_try_wait(bar, parity)) return;
    if (*abort_flag) return;
    const long long t0 = clock64();
#pragma unroll 1
    while (true) {
        if (mbar_try_wait(bar, parity)) return;
        if (*abort_flag) return;
        if (clock64() - t0 > kWaitLimitCycles) {
            *abort_flag = 1;
            record_timeout(site, aux);
            return;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// TMA (bulk tensor copy global -> shared, completion on an mbarrier).  One CTA, no cluster forms.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Bulk tensor store shared -> global (rows outside the tensor are clipped), and the group bookkeeping that keeps the
// shared-memory source alive until the copy has been carried out.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* tmap, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
// Waits only until the copy engine has READ the shared-memory source: the block may then retire (or reuse the
// buffer) while the global writes drain like any other store.
__device__ __forceinline__ void tma_store_commit_and_wait() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Warp-level matrix helpers (decode path)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// two fp32 -> packed bf16x2 (lo in the low half), round to nearest even
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Programmatic dependent launch: let the next kernel in the stream get resident early / wait for the
// previous grid's memory to be visible.  Both are no-ops when the launch carries no such dependency.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace cllo
