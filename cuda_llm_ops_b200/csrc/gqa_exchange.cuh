// All-gather of per-GPU decode partials + log-sum-exp combine in ONE kernel, over peer memory.
//
// For a KV cache sharded by position across the GPUs of one NVSwitch domain, every rank holds a packed
// partial (O, m, l) per query head of ITS positions (rows x (D+2) fp32, 33 KB at Hq=64).  This kernel
//   1. stores the local partial into slot [rank] of every peer's gather buffer with plain peer stores
//      (block p serves destination p), fences at system scope and publishes an epoch number in the
//      peer's flag word for this rank;
//   2. waits (bounded) until the flag words of all ranks in its OWN memory show the epoch;
//   3. merges the `world` partials of its share of the rows and writes the bf16 output.
// The exchange is a few tens of KB, so it is latency-bound: compared with a library all-gather followed
// by a combine kernel it removes one collective launch and one kernel boundary from a ~100 us step.
// Gather slots are double-buffered by epoch parity: a rank can be at most one call ahead of a peer,
// because finishing call n needs that peer's flag of call n, which the peer raises only after its own
// call n-1 has completed in stream order.
//
// Every rank must launch this kernel for the same epoch; ranks live on different GPUs, so the kernels
// that wait for one another always run concurrently.  No multicast objects, no TMA: ordinary loads and
// stores to mapped peer memory.
#pragma once

#include "common.cuh"
#include "host_util.cuh"

namespace cllo {
namespace exchange {

constexpr int kD = 128;
constexpr int kPW = kD + 2;
constexpr int kThreads = 512;

struct Params {
    const float* local;             // [rows][D+2]
    float* gather[CLLO_MAX_PEERS];  // gather[p]: rank p's buffer [2][world][rows][D+2], mapped here
    unsigned* flags[CLLO_MAX_PEERS];  // flags[p]: rank p's flag words [world]
    __nv_bfloat16* o;               // [rows][D]
    long long rows;
    int rank, world;
    unsigned epoch;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kThreads) exchange_combine_kernel(Params p) {
    const int dst = blockIdx.x;  // destination rank served by this block; also its share of the rows in step 3
    // epoch 0 = "count the calls on the device": every launch has exactly `world` blocks, each takes one
    // ticket, so all blocks of the n-th launch derive n.  This keeps the call replayable from a CUDA graph.
    __shared__ unsigned s_epoch;
    if (threadIdx.x == 0)
        s_epoch = p.epoch ? p.epoch : atomicAdd(p.flags[p.rank] + p.world, 1u) / static_cast<unsigned>(p.world) + 1u;
    __syncthreads();
    p.epoch = s_epoch;
    const size_t slot_floats = static_cast<size_t>(p.rows) * kPW;
    const size_t parity_off = static_cast<size_t>(p.epoch & 1u) * p.world * slot_floats;

    // 1. push the local partial to peer `dst` (float2 granularity: rows are 520 bytes)
    {
        float2* out = reinterpret_cast<float2*>(p.gather[dst] + parity_off + static_cast<size_t>(p.rank) * slot_floats);
        const float2* in = reinterpret_cast<const float2*>(p.local);
        const size_t n2 = slot_floats / 2;
        for (size_t i = threadIdx.x; i < n2; i += kThreads) out[i] = in[i];
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) st_release_sys(p.flags[dst] + p.rank, p.epoch);
    }

    // 2. wait for everybody's partial to have landed here
    __shared__ int timed_out;
    if (threadIdx.x == 0) timed_out = 0;
    __syncthreads();
    if (threadIdx.x < p.world) {
        const unsigned* f = p.flags[p.rank] + threadIdx.x;
        const long long t0 = clock64();
        // epochs only grow; a later one would mean this call is being replayed out of step
        while (static_cast<int>(ld_acquire_sys(f) - p.epoch) < 0) {
            if (clock64() - t0 > kWaitLimitCycles) {
                timed_out = 1;
                record_timeout(SITE_EXCHANGE_FLAG, threadIdx.x);
                break;
            }
        }
    }
    __syncthreads();
    if (timed_out) return;

    // 3. merge this block's share of the rows; thread = (row, 4 dims); data bypasses L1 (peers wrote it)
    const float* mine = p.gather[p.rank] + parity_off;
    const long long r_lo = p.rows * dst / p.world, r_hi = p.rows * (dst + 1) / p.world;
    for (long long r = r_lo + (threadIdx.x >> 5); r < r_hi; r += kThreads / 32) {
        const int c4 = (threadIdx.x & 31) * 4;
        float mstar = -INFINITY;
#pragma unroll 4
        for (int s = 0; s < p.world; ++s) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(mine + s * slot_floats + r * kPW + kD));
            mstar = fmaxf(mstar, ml.y > 0.f ? ml.x : -INFINITY);
        }
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, lsum = 0.f;
#pragma unroll 4
        for (int s = 0; s < p.world; ++s) {
            const float* row = mine + s * slot_floats + r * kPW;
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(row + kD));
            const float wgt = ml.y > 0.f ? __expf(ml.x - mstar) : 0.f;
            const float2 x = __ldcg(reinterpret_cast<const float2*>(row + c4));
            const float2 y = __ldcg(reinterpret_cast<const float2*>(row + c4 + 2));
            a0 += wgt * x.x;
            a1 += wgt * x.y;
            a2 += wgt * y.x;
            a3 += wgt * y.y;
            lsum += wgt * ml.y;
        }
        const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
        uint2 pk;
        pk.x = pack_bf16x2(a0 * inv, a1 * inv);
        pk.y = pack_bf16x2(a2 * inv, a3 * inv);
        *reinterpret_cast<uint2*>(p.o + r * kD + c4) = pk;
    }
}

static int launch(const float* local, void* const* gather, void* const* flags, int rank, int world, unsigned epoch,
                  void* o, long long rows, int D, cudaStream_t stream) {
    if (!local || !gather || !flags || !o || rows <= 0) return CLLO_E_BAD_ARG;
    if (world < 1 || world > CLLO_MAX_PEERS || rank < 0 || rank >= world) return CLLO_E_BAD_ARG;
    if (D != kD) return CLLO_E_UNSUPPORTED;
    Params p;
    p.local = local;
    for (int i = 0; i < CLLO_MAX_PEERS; ++i) {
        p.gather[i] = i < world ? static_cast<float*>(gather[i]) : nullptr;
        p.flags[i] = i < world ? static_cast<unsigned*>(flags[i]) : nullptr;
        if (i < world && (!p.gather[i] || !p.flags[i] || !aligned_to(p.gather[i], 8))) return CLLO_E_BAD_ARG;
    }
    p.o = static_cast<__nv_bfloat16*>(o);
    p.rows = rows;
    p.rank = rank;
    p.world = world;
    p.epoch = epoch;
    exchange_combine_kernel<<<world, kThreads, 0, stream>>>(p);
    CLLO_CUDA_TRY(cudaGetLastError());
    return CLLO_OK;
}

}  // namespace exchange
}  // namespace cllo
