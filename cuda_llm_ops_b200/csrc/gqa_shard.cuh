// Exchange protocol of the KV-position-sharded decode, shared by the fused decode kernel and the stand-alone
// exchange kernel, plus the log-sum-exp merge of packed partial rows that both of them (and the split-KV merge
// inside one GPU) use.
//
// Every rank owns, in memory that all ranks of the node can address,
//   gather  [2 parities][world][rows][D+2] fp32   slot [e & 1][r] = rank r's packed (O, m, l) rows of step e
//   flags   [world][CLLO_SHARD_MAX_UNITS] uint32   flag [r][u] = last step whose rows of unit u rank r has delivered
//           followed by one word that counts the units this rank has completed since the buffers were zeroed
// A "unit" is one (batch, kv head, block of <= 16 query heads): the rows that one thread block finishes together.
// The block that holds unit u's merged rows stores them into slot [e & 1][rank] of EVERY rank's gather buffer with
// plain peer stores, fences at system scope, raises flag [rank][u] = e on every rank, then waits (bounded) until the
// flags [0..world)[u] in its OWN memory show e and merges the `world` rows of unit u from its own gather buffer.
// Units are independent: the publish of a unit overlaps whatever the rest of the grid is still computing.
//
// Gather slots are double-buffered by step parity.  A rank can be at most one step ahead of a peer: finishing step
// e needs every peer's flags of step e, which a peer raises only in its own step e, i.e. after its step e-1 has
// completed in stream order; so when slot [e & 1] is overwritten in step e+2, every rank has finished reading it.
// No multicast objects, no TMA, no library collective: ordinary loads and stores to mapped peer memory.
#pragma once

#include "common.cuh"

namespace cllo {
namespace shard {

constexpr int kD = 128;
constexpr int kPW = kD + 2;
constexpr int kMaxUnits = CLLO_SHARD_MAX_UNITS;
constexpr int kRowsPerUnit = 16;
constexpr int kThreads = 256;  // threads that take part: thread = (row = tid / 16, 8 consecutive columns)

struct Params {
    float* gather[CLLO_MAX_PEERS];
    unsigned* flags[CLLO_MAX_PEERS];
    long long rows_total;  // B * Hq
    long long wait_limit;  // SM cycles a flag wait may take
    int rank, world, units;
    unsigned epoch;        // 0: take the step number from the completion counter
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// named barrier that also ORs a predicate over its participants
__device__ __forceinline__ bool named_bar_or(int id, int nthreads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %3, 0;\n\t"
        "barrier.cta.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(id), "r"(nthreads), "r"(pred ? 1u : 0u)
        : "memory");
    return r != 0;
}

// Log-sum-exp merge of n packed rows for one thread's 8 columns.  row_ptr(i) is the i-th row (D+2 floats, 8-byte
// aligned, read through L2 because other blocks or other GPUs wrote it).  Rows are taken kGroup at a time so that
// their loads are in flight together; the running reference is raised between groups, always in the same order, so
// the result does not depend on which block does the merge.  m is in natural-log units, rows with l == 0 are skipped.
template <int kGroup, typename RowPtr>
__device__ __forceinline__ void merge_rows(int n, int c8, RowPtr row_ptr, float (&acc)[8], float& m_out, float& l_out) {
    float mrun = -INFINITY, lrun = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll 1
    for (int i0 = 0; i0 < n; i0 += kGroup) {
        float2 ml[kGroup], d[kGroup][4];
#pragma unroll
        for (int i = 0; i < kGroup; ++i) {
            const int ii = (i0 + i < n) ? i0 + i : n - 1;
            const float* row = row_ptr(ii);
            ml[i] = __ldcg(reinterpret_cast<const float2*>(row + kD));
#pragma unroll
            for (int e = 0; e < 4; ++e) d[i][e] = __ldcg(reinterpret_cast<const float2*>(row + c8 + 2 * e));
            if (i0 + i >= n) ml[i].y = 0.f;
        }
        float mnew = mrun;
#pragma unroll
        for (int i = 0; i < kGroup; ++i) mnew = fmaxf(mnew, ml[i].y > 0.f ? ml[i].x : -INFINITY);
        const float keep = (mrun == -INFINITY) ? 0.f : __expf(mrun - mnew);
        lrun *= keep;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] *= keep;
#pragma unroll
        for (int i = 0; i < kGroup; ++i) {
            const float wgt = ml[i].y > 0.f ? __expf(ml[i].x - mnew) : 0.f;
            lrun += wgt * ml[i].y;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[2 * e] += wgt * d[i][e].x;
                acc[2 * e + 1] += wgt * d[i][e].y;
            }
        }
        mrun = mnew;
    }
    m_out = mrun;
    l_out = lrun;
}

__device__ __forceinline__ void store_packed_row(float* dst, int c8, const float (&acc)[8], float m, float l) {
#pragma unroll
    for (int e = 0; e < 4; ++e) *reinterpret_cast<float2*>(dst + c8 + 2 * e) = make_float2(acc[2 * e], acc[2 * e + 1]);
    if (c8 == 0) *reinterpret_cast<float2*>(dst + kD) = make_float2(m, l);
}

__device__ __forceinline__ void store_bf16_row(__nv_bfloat16* dst, int c8, const float (&acc)[8], float l) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    uint4 pk;
    pk.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
    pk.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
    pk.z = pack_bf16x2(acc[4] * inv, acc[5] * inv);
    pk.w = pack_bf16x2(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(dst + c8) = pk;
}

// The step number of a launch.  With epoch == 0 it comes from the completion counter: every launch completes
// `units` units and raises the counter once for each (count_unit_done, after the unit's output is written), and
// launches on a stream do not overlap, so at the start of the n-th launch the counter reads (n-1) * units.  A call
// sequence that never changes its arguments (a CUDA graph) can therefore pass epoch = 0.  Read it once per block,
// at kernel start, where its latency hides under the set-up.
__device__ __forceinline__ unsigned* done_counter(const Params& sp) {
    return sp.flags[sp.rank] + static_cast<size_t>(sp.world) * kMaxUnits;
}
__device__ __forceinline__ unsigned read_epoch(const Params& sp) {
    if (sp.epoch) return sp.epoch;
    return *reinterpret_cast<volatile unsigned*>(done_counter(sp)) / static_cast<unsigned>(sp.units) + 1u;
}
__device__ __forceinline__ void count_unit_done(const Params& sp) { atomicAdd(done_counter(sp), 1u); }

// Publish this rank's rows of unit u (thread tid holds columns [c8, c8+8) of row head0 + tid / 16), wait for the
// other ranks' rows of the same unit and write the merged bf16 output.  All kThreads threads of the block call it
// (barrier id `bar_id` is theirs); `epoch` is the same in all of them.  On a wait that runs out the unit's output
// rows are filled with NaN and the device status word is set: a late peer gives a visible error, not stale data.
__device__ __forceinline__ void publish_wait_combine(const Params& sp, unsigned epoch, int bar_id, int tid, long long u,
                                                     long long head0, int rows, const float (&val)[8], float m, float l,
                                                     __nv_bfloat16* o) {
    const int row = tid >> 4, c8 = (tid & 15) * 8;
    const size_t slot_floats = static_cast<size_t>(sp.rows_total) * kPW;
    const size_t par = static_cast<size_t>(epoch & 1u) * sp.world * slot_floats;
    if (row < rows) {
        const size_t off = par + static_cast<size_t>(sp.rank) * slot_floats + static_cast<size_t>(head0 + row) * kPW;
        for (int p = 0; p < sp.world; ++p) store_packed_row(sp.gather[p] + off, c8, val, m, l);
    }
    // the barrier orders every thread's row stores before the flag stores below, and a release at system scope is
    // cumulative over that order: a peer that acquires the flag sees the rows
    named_bar_sync(bar_id, kThreads);
    bool late = false;
    if (tid < sp.world) {
        st_release_sys(sp.flags[tid] + static_cast<size_t>(sp.rank) * kMaxUnits + u, epoch);
        const unsigned* f = sp.flags[sp.rank] + static_cast<size_t>(tid) * kMaxUnits + u;
        const long long t0 = clock64();
        // steps only grow; a peer that is already one step ahead has delivered this step as well
        while (static_cast<int>(ld_acquire_sys(f) - epoch) < 0) {
            if (clock64() - t0 > sp.wait_limit) {
                late = true;
                record_timeout(SITE_EXCHANGE_FLAG, tid);
                break;
            }
        }
    }
    late = named_bar_or(bar_id, kThreads, late);
    if (tid == 0) count_unit_done(sp);
    if (row >= rows) return;
    __nv_bfloat16* dst = o + static_cast<size_t>(head0 + row) * kD;
    if (late) {
        const uint32_t nan2 = 0x7fc07fc0u;
        *reinterpret_cast<uint4*>(dst + c8) = make_uint4(nan2, nan2, nan2, nan2);
        return;
    }
    const float* mine = sp.gather[sp.rank] + par + static_cast<size_t>(head0 + row) * kPW;
    float acc[8], mm, ll;
    merge_rows<8>(sp.world, c8, [&](int s) { return mine + static_cast<size_t>(s) * slot_floats; }, acc, mm, ll);
    store_bf16_row(dst, c8, acc, ll);
}

}  // namespace shard
}  // namespace cllo
