// All-gather of per-GPU decode partials + log-sum-exp combine in ONE kernel, over peer memory: the exchange
// protocol of gqa_shard.cuh driven from a packed partial that already sits in local memory.
//
// For a KV cache sharded by position across the GPUs of one NVSwitch domain, every rank holds a packed partial
// (O, m, l) per query head of ITS positions (rows x (D+2) fp32, 33 KB at Hq=64).  One block per unit (batch, kv
// head, block of <= 16 query heads) publishes that unit's rows to every peer, waits (bounded) for the peers' rows
// of the same unit and writes the merged bf16 output.  The fused decode kernel (decode_splitkv_kernel<true>) does
// the same from its registers as each unit finishes; this kernel serves ranks whose share of the sequence is empty
// (they publish l = 0), callers that produced the partial some other way, and the protocol's tests.  Both speak
// the same protocol, so ranks may mix them within one step.
//
// Every rank must launch for the same step; ranks live on different GPUs, so the kernels that wait for one another
// always run concurrently.
#pragma once

#include <atomic>

#include "common.cuh"
#include "gqa_shard.cuh"
#include "host_util.cuh"

namespace cllo {
namespace exchange {

// How long a flag wait may take, in SM cycles; settable from the host (cllo_set_exchange_wait_limit).
static std::atomic<long long> g_wait_limit{kWaitLimitCycles};

struct Geometry {
    int B, Hq, Hkv, G, n_gblk;
};

__global__ void __launch_bounds__(shard::kThreads) exchange_combine_kernel(const float* __restrict__ local,
                                                                           __nv_bfloat16* o, Geometry geo,
                                                                           const shard::Params sp) {
    const long long u = blockIdx.x;
    const int gblk = static_cast<int>(u % geo.n_gblk);
    const int kvh = static_cast<int>((u / geo.n_gblk) % geo.Hkv);
    const int b = static_cast<int>(u / (static_cast<long long>(geo.n_gblk) * geo.Hkv));
    const int rows = (geo.G - gblk * shard::kRowsPerUnit) < shard::kRowsPerUnit ? (geo.G - gblk * shard::kRowsPerUnit)
                                                                               : shard::kRowsPerUnit;
    const long long head0 = static_cast<long long>(b) * geo.Hq + static_cast<long long>(kvh) * geo.G +
                            gblk * shard::kRowsPerUnit;
    __shared__ unsigned s_epoch;
    if (threadIdx.x == 0) s_epoch = shard::read_epoch(sp);
    __syncthreads();
    const int tid = threadIdx.x, row = tid >> 4, c8 = (tid & 15) * 8;
    float val[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, m = -INFINITY, l = 0.f;
    if (row < rows) {
        const float* src = local + (head0 + row) * shard::kPW;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 x = *reinterpret_cast<const float2*>(src + c8 + 2 * e);
            val[2 * e] = x.x;
            val[2 * e + 1] = x.y;
        }
        const float2 ml = *reinterpret_cast<const float2*>(src + shard::kD);
        m = ml.x;
        l = ml.y;
    }
    shard::publish_wait_combine(sp, s_epoch, 1, tid, u, head0, rows, val, m, l, o);
}

// Fills the protocol parameters from the caller's pointer tables; shared with the fused decode launcher.
static int fill_shard_params(shard::Params* sp, void* const* gather, void* const* flags, int rank, int world,
                             unsigned epoch, int B, int Hq, int Hkv) {
    if (!gather || !flags) return CLLO_E_BAD_ARG;
    if (world < 1 || world > CLLO_MAX_PEERS || rank < 0 || rank >= world) return CLLO_E_BAD_ARG;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return CLLO_E_BAD_ARG;
    const int G = Hq / Hkv;
    const long long units = static_cast<long long>(B) * Hkv * ((G + shard::kRowsPerUnit - 1) / shard::kRowsPerUnit);
    if (units > shard::kMaxUnits) return CLLO_E_UNSUPPORTED;
    for (int i = 0; i < CLLO_MAX_PEERS; ++i) {
        sp->gather[i] = i < world ? static_cast<float*>(gather[i]) : nullptr;
        sp->flags[i] = i < world ? static_cast<unsigned*>(flags[i]) : nullptr;
        if (i < world && (!sp->gather[i] || !sp->flags[i] || !aligned_to(sp->gather[i], 8) || !aligned_to(sp->flags[i], 4)))
            return CLLO_E_BAD_ARG;
    }
    sp->rows_total = static_cast<long long>(B) * Hq;
    sp->wait_limit = g_wait_limit.load();
    sp->rank = rank;
    sp->world = world;
    sp->units = static_cast<int>(units);
    sp->epoch = epoch;
    return CLLO_OK;
}

static int launch(const float* local, void* const* gather, void* const* flags, int rank, int world, unsigned epoch,
                  void* o, int B, int Hq, int Hkv, int D, cudaStream_t stream) {
    if (!local || !o || !aligned_to(local, 8) || !aligned_to(o, 16)) return CLLO_E_BAD_ARG;
    if (D != shard::kD) return CLLO_E_UNSUPPORTED;
    shard::Params sp;
    int rc = fill_shard_params(&sp, gather, flags, rank, world, epoch, B, Hq, Hkv);
    if (rc != CLLO_OK) return rc;
    Geometry geo;
    geo.B = B;
    geo.Hq = Hq;
    geo.Hkv = Hkv;
    geo.G = Hq / Hkv;
    geo.n_gblk = (geo.G + shard::kRowsPerUnit - 1) / shard::kRowsPerUnit;
    exchange_combine_kernel<<<sp.units, shard::kThreads, 0, stream>>>(local, static_cast<__nv_bfloat16*>(o), geo, sp);
    CLLO_CUDA_TRY(cudaGetLastError());
    return CLLO_OK;
}

}  // namespace exchange
}  // namespace cllo
