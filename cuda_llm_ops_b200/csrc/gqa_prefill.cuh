// Prefill (multi-token) GQA forward for sm_100a: tcgen05 tensor cores, accumulators in tensor memory,
// TMA-fed double-buffered K/V pipeline.
//
// One thread block owns 256 query rows of one query head as two 128-row tiles ("ping" and "pong").
// Per KV tile of 128 tokens it performs, for each of the two query tiles,
//     S = Q K^T          tcgen05.mma  M=128 N=128 K=16 x8, Q and K from shared memory (K-major, 128B swizzle)
//     P = online softmax 128 threads, one query row each, S read from tensor memory with tcgen05.ld
//     O += P V           tcgen05.mma  M=128 N=128 K=16 x8, P from tensor memory (bf16, written with
//                        tcgen05.st), V from shared memory (MN-major, 128B swizzle)
// so that the tensor pipe works on one tile while the other tile's softmax runs on the ALUs.
//
// Tensor memory (512 columns): P0 (64) | C (128) | P1 (64) | O0 (128) | O1 (128).  Every S = Q K^T of either tile
// lands in the one region C; the tile's softmax threads copy it to registers at once (about 80 cycles) and hand
// C back, so the next S -- the other tile's -- can be issued while this tile's softmax is still running, and
// no S ever waits for the P V product of its own tile.  (With S and P sharing columns, the chain
// softmax -> P V -> next S -> softmax of one tile was the critical path and left the tensor pipe idle for a
// quarter of the time.)  The probabilities of tile t live in P_t until P V of that step has retired.
// The running maximum is only raised (and O rescaled in tensor memory) when it grew by more than 2^8, which
// keeps every probability below 256 and makes rescaling rare.
//
// Warp roles (384 threads): warps 0-3 softmax of tile 0, warps 4-7 softmax of tile 1 (a warp may only
// touch the 32 tensor-memory lanes given by its index modulo 4), warp 8 TMA producer, warp 9 MMA issuer,
// warps 10-11 idle (they complete the third warpgroup so that it can hand registers to the softmax warps).
// All hand-offs are mbarriers; every wait is bounded and records a status instead of hanging.
#pragma once

#include "common.cuh"
#include "gqa_decode.cuh"
#include "host_util.cuh"

#include <cstdlib>
#include <type_traits>

namespace cllo {
namespace prefill {

constexpr int kD = 128;
constexpr int kBM = 128;          // query rows per tile
constexpr int kBN = 128;          // kv tokens per tile
constexpr int kTiles = 2;         // query tiles per block
constexpr int kKvStages = 2;
constexpr int kThreads = 384;
// Registers per thread after the warpgroups re-balance themselves (setmaxnreg).  The pool of a block is what it was
// launched with, kLaunchRegs per thread (the cap that __launch_bounds__(384, 1) gives: 65536 / 384 rounded down to
// a multiple of 8); asking for more than that in total would block the second softmax warpgroup for ever.
constexpr int kLaunchRegs = 168;
constexpr int kSoftmaxRegs = 208;
constexpr int kOtherRegs = 88;
static_assert(2 * kSoftmaxRegs + kOtherRegs <= 3 * kLaunchRegs, "setmaxnreg budget exceeds the block's register pool");
static_assert(kSoftmaxRegs % 8 == 0 && kOtherRegs % 8 == 0, "setmaxnreg takes multiples of 8");
// tensor-memory columns
constexpr uint32_t kColP0 = 0, kColC = 64, kColP1 = 192, kColO = 256;
constexpr int kHalfBytes = 128 * 128;        // [128 rows][64 dims] bf16 = 16 KB, one swizzled half tile
constexpr int kTileBytes = 2 * kHalfBytes;   // 32 KB
constexpr int kSmemQ = 0;
constexpr int kSmemK = kTiles * kTileBytes;
constexpr int kSmemV = kSmemK + kKvStages * kTileBytes;
constexpr int kSmemBar = kSmemV + kKvStages * kTileBytes;
constexpr int kNumBars = 1 + 4 * kKvStages + 3 * kTiles + 2;
constexpr int kSmemBytes = kSmemBar + kNumBars * 8 + 32 + 1024;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum : int {
    SITE_Q_FULL = SITE_PREFILL_BASE + 0,
    SITE_K_FULL = SITE_PREFILL_BASE + 1,
    SITE_V_FULL = SITE_PREFILL_BASE + 2,
    SITE_K_EMPTY = SITE_PREFILL_BASE + 3,
    SITE_V_EMPTY = SITE_PREFILL_BASE + 4,
    SITE_S_FULL = SITE_PREFILL_BASE + 5,
    SITE_P_FULL = SITE_PREFILL_BASE + 6,
    SITE_O_FULL = SITE_PREFILL_BASE + 7,
    SITE_DRAIN = SITE_PREFILL_BASE + 8,
    SITE_C_FREE = SITE_PREFILL_BASE + 9,
};

struct Params {
    __nv_bfloat16* o;
    float* lse;  // nullable
    float scale_log2;
    int B, Sq, Skv, Hq, Hkv, G, causal, n_qp;
    int window;         // > 0: sliding window, a query sees kv in [q - (window - 1), q] (implies causal)
    const float* sink;  // nullable, [Hq]: per-head term added to the softmax denominator
    // split-KV mode (n_split > 1): block (.., split) covers one share of the kv tiles and leaves, instead of O and
    // lse, packed fp32 rows {un-normalised O[128], m (natural-log units), l} in part[split][B*Hq*Sq][130]
    float* part;
    int n_split;
};

// ---- tcgen05 wrappers -------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// D(tmem) (+)= A(smem) * B(smem)
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D(tmem) (+)= A(tmem) * B(smem)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same two instructions for the hot loop, taking the LOW words of the shared-memory descriptors (start address
// and leading-dimension offset; the high word -- stride, version, swizzle -- is one constant) and the accumulate flag
// as a compile-time constant, so that the issuing thread spends as few instructions as possible between two MMAs.
template <bool kAccumulate>
__device__ __forceinline__ void tc_mma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                             uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
}
template <bool kAccumulate>
__device__ __forceinline__ void tc_mma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi,
                                             uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
}
// tcgen05.mma / commit issued by the lanes whose `leader` is non-zero while the WHOLE warp runs the surrounding code:
// the operands (descriptor words, tensor-memory addresses) are then warp-uniform values that the compiler keeps in
// uniform registers.  Under an `if (lane == 0)` they live in ordinary registers and every MMA pays several
// register-to-uniform moves in the issuing thread -- measured here: 75-95 cycles per MMA issued, against 48-64 that
// the tensor pipe needs.
template <bool kAccumulate>
__device__ __forceinline__ void tc_mma_ss_lo_if(uint32_t leader, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                uint32_t hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 q, %6, 0;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "n"(kAccumulate ? 1 : 0), "r"(leader)
        : "memory");
}
__device__ __forceinline__ void tc_mma_ts_lo_if(uint32_t leader, uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                                uint32_t hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 q, %6, 0;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}
__device__ __forceinline__ void tc_commit_if(uint32_t leader, uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar), "r"(leader)
        : "memory");
}

// O += P V (eight MMAs, A from tensor memory) by the leader lane, with a look at an mbarrier (one barrier per
// lane) put between the fifth and the sixth MMA and its result read only after the eighth.  Memory-pipe
// instructions of a warp are carried out in order, so a look whose result is needed at once keeps the thread from
// issuing anything behind it for the whole round trip, and the tensor pipe runs dry; this way the round trip is
// covered by the last three MMAs.
__device__ __forceinline__ uint32_t tc_pv_run_with_look(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi,
                                                        uint32_t idesc, uint32_t accumulate_first, uint32_t leader,
                                                        uint32_t look_bar, uint32_t look_parity) {
    uint32_t seen;
    asm volatile(
        "{\n\t"
        ".reg .pred p0, pt, q, w;\n\t"
        ".reg .b64 db;\n\t"
        ".reg .b32 a, b;\n\t"
        "setp.ne.b32 p0, %6, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], db, %5, p0;\n\t"
        "add.u32 a, %2, 8;\n\t  add.u32 b, %3, 128;\n\t  mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a], db, %5, pt;\n\t"
        "add.u32 a, %2, 16;\n\t add.u32 b, %3, 256;\n\t  mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a], db, %5, pt;\n\t"
        "add.u32 a, %2, 24;\n\t add.u32 b, %3, 384;\n\t  mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a], db, %5, pt;\n\t"
        "add.u32 a, %2, 32;\n\t add.u32 b, %3, 512;\n\t  mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a], db, %5, pt;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 w, [%8], %9;\n\t"
        "add.u32 a, %2, 40;\n\t add.u32 b, %3, 640;\n\t  mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a], db, %5, pt;\n\t"
        "add.u32 a, %2, 48;\n\t add.u32 b, %3, 768;\n\t  mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a], db, %5, pt;\n\t"
        "add.u32 a, %2, 56;\n\t add.u32 b, %3, 896;\n\t  mov.b64 db, {b, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a], db, %5, pt;\n\t"
        "selp.u32 %0, 1, 0, w;\n\t"
        "}"
        : "=r"(seen)
        : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate_first), "r"(leader),
          "r"(look_bar), "r"(look_parity)
        : "memory");
    return seen;
}
// 32 columns + wait (see tmem_ld128_wait for why the wait is fused)
__device__ __forceinline__ void tmem_ld32_wait(uint32_t taddr, float (&r)[32]) {
    uint32_t* u = reinterpret_cast<uint32_t*>(r);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
          "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]),
          "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]),
          "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(taddr)
        : "memory");
}
// 16 columns + wait, and the matching store (used by the rare rescale of O, where registers are scarce)
__device__ __forceinline__ void tmem_ld16_wait(uint32_t taddr, uint32_t (&u)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
          "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&u)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
        ::"r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
          "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]),
          "r"(taddr)
        : "memory");
}
// 128 consecutive fp32 columns of this thread's lane.  The wait is part of the same statement so that no
// use of the destination registers can be scheduled ahead of it.
__device__ __forceinline__ void tmem_ld128_wait(uint32_t taddr, float (&r)[128]) {
    uint32_t* u = reinterpret_cast<uint32_t*>(r);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x128.b32 {"
        "%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,"
        "%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63,"
        "%64,%65,%66,%67,%68,%69,%70,%71,%72,%73,%74,%75,%76,%77,%78,%79,"
        "%80,%81,%82,%83,%84,%85,%86,%87,%88,%89,%90,%91,%92,%93,%94,%95,"
        "%96,%97,%98,%99,%100,%101,%102,%103,%104,%105,%106,%107,%108,%109,%110,%111,"
        "%112,%113,%114,%115,%116,%117,%118,%119,%120,%121,%122,%123,%124,%125,%126,%127"
        "}, [%128];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
          "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]),
          "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]),
          "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31]),
          "=r"(u[32]), "=r"(u[33]), "=r"(u[34]), "=r"(u[35]), "=r"(u[36]), "=r"(u[37]), "=r"(u[38]), "=r"(u[39]),
          "=r"(u[40]), "=r"(u[41]), "=r"(u[42]), "=r"(u[43]), "=r"(u[44]), "=r"(u[45]), "=r"(u[46]), "=r"(u[47]),
          "=r"(u[48]), "=r"(u[49]), "=r"(u[50]), "=r"(u[51]), "=r"(u[52]), "=r"(u[53]), "=r"(u[54]), "=r"(u[55]),
          "=r"(u[56]), "=r"(u[57]), "=r"(u[58]), "=r"(u[59]), "=r"(u[60]), "=r"(u[61]), "=r"(u[62]), "=r"(u[63]),
          "=r"(u[64]), "=r"(u[65]), "=r"(u[66]), "=r"(u[67]), "=r"(u[68]), "=r"(u[69]), "=r"(u[70]), "=r"(u[71]),
          "=r"(u[72]), "=r"(u[73]), "=r"(u[74]), "=r"(u[75]), "=r"(u[76]), "=r"(u[77]), "=r"(u[78]), "=r"(u[79]),
          "=r"(u[80]), "=r"(u[81]), "=r"(u[82]), "=r"(u[83]), "=r"(u[84]), "=r"(u[85]), "=r"(u[86]), "=r"(u[87]),
          "=r"(u[88]), "=r"(u[89]), "=r"(u[90]), "=r"(u[91]), "=r"(u[92]), "=r"(u[93]), "=r"(u[94]), "=r"(u[95]),
          "=r"(u[96]), "=r"(u[97]), "=r"(u[98]), "=r"(u[99]), "=r"(u[100]), "=r"(u[101]), "=r"(u[102]), "=r"(u[103]),
          "=r"(u[104]), "=r"(u[105]), "=r"(u[106]), "=r"(u[107]), "=r"(u[108]), "=r"(u[109]), "=r"(u[110]), "=r"(u[111]),
          "=r"(u[112]), "=r"(u[113]), "=r"(u[114]), "=r"(u[115]), "=r"(u[116]), "=r"(u[117]), "=r"(u[118]), "=r"(u[119]),
          "=r"(u[120]), "=r"(u[121]), "=r"(u[122]), "=r"(u[123]), "=r"(u[124]), "=r"(u[125]), "=r"(u[126]), "=r"(u[127])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&u)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
        ::"r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
          "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]),
          "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]),
          "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31]),
          "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }


// ---- packed fp32x2 arithmetic (two floats per 64-bit register pair, one instruction) ------------
__device__ __forceinline__ uint64_t pk2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// three-input maximum / minimum (one instruction on this architecture)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^y for a pair, on the special-function unit
__device__ __forceinline__ void exp2_pair_sfu(uint64_t y, float& p0, float& p1) {
    float a, b;
    upk2(y, a, b);
    p0 = fast_exp2(a);
    p1 = fast_exp2(b);
}

// Shared-memory matrix descriptor, 128-byte swizzle.  Offsets are in bytes.
//   bits [0,14) start >> 4 | [16,30) leading-dim offset >> 4 | [32,46) stride-dim offset >> 4
//   bits [46,48) = 1 (descriptor version of this architecture) | [61,64) = 2 (128-byte swizzle)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return static_cast<uint64_t>((addr >> 4) & 0x3fffu) | (static_cast<uint64_t>((lbo >> 4) & 0x3fffu) << 16) |
           (static_cast<uint64_t>((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}
// The two 32-bit words of that descriptor.
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t addr, uint32_t lbo) {
    return ((addr >> 4) & 0x3fffu) | (((lbo >> 4) & 0x3fffu) << 16);
}
__host__ __device__ constexpr uint32_t smem_desc_hi(uint32_t sbo) { return ((sbo >> 4) & 0x3fffu) | (1u << 14) | (2u << 29); }
// Instruction descriptor for kind::f16: fp32 accumulate (bits 4-5 = 1), bf16 A and B (bits 7-9, 10-12 = 1),
// B major-ness in bit 16 (0 = K-major, 1 = MN-major), N/8 in bits 17-22, M/16 in bits 24-28.
constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24);
constexpr uint32_t kIdescPV = kIdescQK | (1u << 16);

__global__ void __launch_bounds__(kThreads, 1)
prefill_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                   const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar0 = base + kSmemBar;
    // barrier map
    const uint32_t bar_q_full = bar0;
    auto bar_k_full = [&](int s) { return bar0 + 8 * (1 + s); };
    auto bar_k_empty = [&](int s) { return bar0 + 8 * (1 + kKvStages + s); };
    auto bar_v_full = [&](int s) { return bar0 + 8 * (1 + 2 * kKvStages + s); };
    auto bar_v_empty = [&](int s) { return bar0 + 8 * (1 + 3 * kKvStages + s); };
    auto bar_s_full = [&](int t) { return bar0 + 8 * (1 + 4 * kKvStages + t); };               // S_t landed in C
    auto bar_p_full = [&](int t) { return bar0 + 8 * (1 + 4 * kKvStages + kTiles + t); };      // P_t stored
    auto bar_o_full = [&](int t) { return bar0 + 8 * (1 + 4 * kKvStages + 2 * kTiles + t); };  // P_t V retired
    const uint32_t bar_c_free = bar0 + 8 * (kNumBars - 2);
    const uint32_t bar_drain = bar0 + 8 * (kNumBars - 1);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + kSmemBar + kNumBars * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + kSmemBar + kNumBars * 8 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // block -> (batch, kv head, query tile pair, head in group); heads of one group are neighbours so
    // that they stream the same K/V tiles through L2 together; heavy (late) causal pairs go first.
    long long id = blockIdx.x;
    const int g = static_cast<int>(id % p.G);
    id /= p.G;
    const int qp = p.n_qp - 1 - static_cast<int>(id % p.n_qp);
    id /= p.n_qp;
    const int kvh = static_cast<int>(id % p.Hkv);
    id /= p.Hkv;
    const int b = static_cast<int>(id % p.B);
    const int split = static_cast<int>(id / p.B);
    const int h = kvh * p.G + g;
    const int q0 = qp * (kTiles * kBM);

    // KV tiles [j_lo, j_hi) can hold something visible to this block's rows
    int j_hi = (p.Skv + kBN - 1) / kBN;
    if (p.causal) {
        const int last_row = q0 + kTiles * kBM - 1;
        const int lim = last_row / kBN + 1;
        j_hi = lim < j_hi ? lim : j_hi;
    }
    int j_lo = 0;
    if (p.window > 0 && q0 - (p.window - 1) > 0) j_lo = (q0 - (p.window - 1)) / kBN;
    if (j_lo > j_hi - 1) j_lo = j_hi - 1;
    if (p.n_split > 1) {  // this block's share of the tiles (the launcher makes every share non-empty)
        const int len = (j_hi - j_lo + p.n_split - 1) / p.n_split;
        j_lo += split * len;
        j_hi = j_lo + len < j_hi ? j_lo + len : j_hi;
    }
    const int n_kv = j_hi - j_lo;  // >= 1; the loops below count local tiles, tile j is global tile j_lo + j

    if (warp == 8 && lane == 0) {
        mbar_init(bar_q_full, 1);
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(bar_k_full(s), 1);
            mbar_init(bar_k_empty(s), kBM);
            mbar_init(bar_v_full(s), 1);
            mbar_init(bar_v_empty(s), kBM);
        }
        for (int t = 0; t < kTiles; ++t) {
            mbar_init(bar_p_full(t), kBM);
            mbar_init(bar_s_full(t), 1);
            mbar_init(bar_o_full(t), 1);
        }
        mbar_init(bar_c_free, kBM);
        mbar_init(bar_drain, 1);
        *abort_flag = 0;
        fence_mbar_init();
        // The first copies start here, before the block has even met at its first barrier: Q, and K and V of the
        // first kv tile (their stages are fresh, nothing to wait for).  The producer loop below continues at
        // the second K tile.
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        mbar_arrive_expect_tx(bar_q_full, kTiles * kTileBytes);
        for (int t = 0; t < kTiles; ++t) {
            const uint32_t dst = base + kSmemQ + t * kTileBytes;
            tma_load_4d(dst, &tm_q, bar_q_full, 0, q0 + t * kBM, h, b);
            tma_load_4d(dst + kHalfBytes, &tm_q, bar_q_full, 64, q0 + t * kBM, h, b);
        }
        mbar_arrive_expect_tx(bar_k_full(0), kTileBytes);
        tma_load_4d(base + kSmemK, &tm_k, bar_k_full(0), 0, j_lo * kBN, kvh, b);
        tma_load_4d(base + kSmemK + kHalfBytes, &tm_k, bar_k_full(0), 64, j_lo * kBN, kvh, b);
        mbar_arrive_expect_tx(bar_v_full(0), kTileBytes);
        tma_load_4d(base + kSmemV, &tm_v, bar_v_full(0), 0, j_lo * kBN, kvh, b);
        tma_load_4d(base + kSmemV + kHalfBytes, &tm_v, bar_v_full(0), 64, j_lo * kBN, kvh, b);
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Register budget: the softmax warps hold a whole 128-column row per thread, the copy and MMA warps need
    // much less.  Each branch below starts with its own setmaxnreg.
    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
    if (warp == 8) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tm_o);
            for (int j = 1; j < n_kv; ++j) {  // tile 0 was started before the block's first barrier
                const int s = j % kKvStages;
                const uint32_t use = static_cast<uint32_t>(j / kKvStages);
                mbar_wait(bar_k_empty(s), (use & 1u) ^ 1u, abort_flag, SITE_K_EMPTY, j);
                mbar_arrive_expect_tx(bar_k_full(s), kTileBytes);
                const uint32_t kd = base + kSmemK + s * kTileBytes;
                tma_load_4d(kd, &tm_k, bar_k_full(s), 0, (j_lo + j) * kBN, kvh, b);
                tma_load_4d(kd + kHalfBytes, &tm_k, bar_k_full(s), 64, (j_lo + j) * kBN, kvh, b);
                mbar_wait(bar_v_empty(s), (use & 1u) ^ 1u, abort_flag, SITE_V_EMPTY, j);
                mbar_arrive_expect_tx(bar_v_full(s), kTileBytes);
                const uint32_t vd = base + kSmemV + s * kTileBytes;
                tma_load_4d(vd, &tm_v, bar_v_full(s), 0, (j_lo + j) * kBN, kvh, b);
                tma_load_4d(vd + kHalfBytes, &tm_v, bar_v_full(s), 64, (j_lo + j) * kBN, kvh, b);
            }
            if (*abort_flag) {
                // a wait gave up somewhere: let the copies already issued land before the block retires
                for (int j = (n_kv > kKvStages ? n_kv - kKvStages : 0); j < n_kv; ++j) {
                    const int s = j % kKvStages;
                    const uint32_t use = static_cast<uint32_t>(j / kKvStages);
                    const long long t0 = clock64();
                    while (!(mbar_try_wait(bar_k_full(s), use & 1u) && mbar_try_wait(bar_v_full(s), use & 1u)) &&
                           clock64() - t0 < kWaitLimitCycles / 64) {
                    }
                }
            }
        }
    } else if (warp == 9) {
        // -------------------------------- MMA issuer --------------------------------
        // Lane 0 issues every tcgen05.mma.  Measured on this part: a stream of these MMAs runs at 64 cycles each and
        // absorbs a couple of hundred cycles of plain arithmetic in the issuing thread, but NOT its memory-pipe
        // instructions -- those are carried out in order behind the queued MMAs, so a look at an mbarrier whose
        // result is needed at once (about 150-190 cycles round trip while the tensor pipe saturates the
        // shared-memory port), a named barrier or a commit each leave the tensor pipe idle for about that long.
        // So the work is issued in runs of sixteen MMAs -- the next S for region C (the other tile will be waiting for
        // it before anybody waits for P V), then O_t += P_t V of the tile that has just finished its softmax -- and
        // the look at the next run's barriers (the whole warp looks at once, one barrier per lane) is issued inside
        // the P V run with its result read only after the run's last MMA.
        // low descriptor words of the operand tiles (per k step only a constant is added: the tiles are 1024-byte
        // aligned and no sum leaves the 14-bit address field)
        const uint32_t hi = smem_desc_hi(1024);
        const uint32_t q_lo0 = smem_desc_lo(base + kSmemQ, 16), q_lo1 = smem_desc_lo(base + kSmemQ + kTileBytes, 16);
        const uint32_t k_lo0 = smem_desc_lo(base + kSmemK, 16), k_lo1 = smem_desc_lo(base + kSmemK + kTileBytes, 16);
        const uint32_t v_lo0 = smem_desc_lo(base + kSmemV, kHalfBytes);
        const uint32_t v_lo1 = smem_desc_lo(base + kSmemV + kTileBytes, kHalfBytes);
        auto issue_s = [&](int t, int stage) {
            const uint32_t qa = t ? q_lo1 : q_lo0;
            const uint32_t ka = stage ? k_lo1 : k_lo0;
            tc_mma_ss_lo<false>(tmem_base + kColC, qa, ka, hi, kIdescQK);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks) {
                const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
                tc_mma_ss_lo<true>(tmem_base + kColC, qa + off, ka + off, hi, kIdescQK);
            }
        };
        auto issue_pv = [&](int t, int stage, bool first) {
            const uint32_t va = stage ? v_lo1 : v_lo0;
            const uint32_t pa = tmem_base + (t ? kColP1 : kColP0);
            const uint32_t oa = tmem_base + kColO + t * kD;
            if (first)
                tc_mma_ts_lo<false>(oa, pa, va, hi, kIdescPV);
            else
                tc_mma_ts_lo<true>(oa, pa, va, hi, kIdescPV);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks) tc_mma_ts_lo<true>(oa, pa + ks * 8, va + ks * (2048 >> 4), hi, kIdescPV);
        };
        // "Landing" #m is S of tile (m & 1) at kv step (m >> 1), written to region C.  It may be issued once the
        // threads of the other tile have copied landing #m-1 out of C (phase m-1 of c_free) and, for tile 0, once
        // the K tile has arrived.
        const int n_land = 2 * n_kv;
        if (lane == 0) {  // the first three landings, nothing to overlap them with
            mbar_wait(bar_q_full, 0, abort_flag, SITE_Q_FULL, 0);
            for (int m = 0; m < 3 && m < n_land; ++m) {
                const int j = m >> 1, st = j % kKvStages;
                if (m > 0) mbar_wait(bar_c_free, static_cast<uint32_t>(m - 1) & 1u, abort_flag, SITE_C_FREE, m);
                if ((m & 1) == 0)
                    mbar_wait(bar_k_full(st), static_cast<uint32_t>(j / kKvStages) & 1u, abort_flag, SITE_K_FULL, j);
                tc_fence_after();
                issue_s(m & 1, st);
                tc_commit(bar_s_full(m & 1));
            }
        }
        __syncwarp();
        // Main part: the two half-steps of a kv step are written out, so that the tile is a compile-time constant and
        // the choice of barriers needs no branches; the thread that feeds the tensor pipe shares its scheduler with
        // two softmax warps and every instruction it does not have to issue is time the pipe does not idle.
        // the barrier a lane looks at before half-step (t, j): 0 P_t stored, 1 V tile arrived (t = 0), 2 region C free,
        // 3 K tile arrived (t = 1); the other lanes repeat lane 0
        auto my_barrier = [&](auto tc, int j, uint32_t& bar, uint32_t& par) {
            constexpr int t = decltype(tc)::value;
            const int s = j & 1;
            bar = bar_p_full(t);
            par = static_cast<uint32_t>(s);
            if (t == 0 && lane == 1) {
                bar = bar_v_full(s);
                par = static_cast<uint32_t>(j >> 1) & 1u;
            }
            if (lane == 2) {
                bar = bar_c_free;
                par = t;
            }
            if (t == 1 && lane == 3) {
                bar = bar_k_full(s);
                par = static_cast<uint32_t>((j + 2) >> 1) & 1u;
            }
        };
        using I0 = std::integral_constant<int, 0>;
        using I1 = std::integral_constant<int, 1>;
        // `seen`: the look that the previous half-step took at this half-step's barriers came back positive
        auto half_step = [&](auto tc, int j, bool seen) {
            constexpr int t = decltype(tc)::value;   // tile that has finished its softmax
            const int s = j & 1;                      // stage of V(j), parity of P_t(j)
            const int sm = t == 0 ? (s ^ 1) : s;      // stage of the K tile of the landing issued here
            uint32_t my_bar, my_par;
            if (!seen) {
                my_barrier(tc, j, my_bar, my_par);
                if (!__all_sync(0xffffffffu, mbar_try_wait(my_bar, my_par))) {
                    if (lane < 4)
                        mbar_wait(my_bar, my_par, abort_flag,
                                  lane == 0 ? SITE_P_FULL : lane == 2 ? SITE_C_FREE : t == 0 ? SITE_V_FULL : SITE_K_FULL,
                                  2 * j + t);
                    __syncwarp();
                }
            }
            if (lane == 0) {
                tc_fence_after();
                issue_s(t ^ 1, sm);  // first: the other tile is waiting for it sooner than anybody waits for P V
                tc_commit(bar_s_full(t ^ 1));
            }
            __syncwarp();
            // the barriers of the next half-step: (1, j) after (0, j), (0, j + 1) after (1, j)
            if (t == 0)
                my_barrier(I1{}, j, my_bar, my_par);
            else
                my_barrier(I0{}, j + 1, my_bar, my_par);
            const uint32_t mine = tc_pv_run_with_look(
                tmem_base + kColO + t * kD, tmem_base + (t ? kColP1 : kColP0), s ? v_lo1 : v_lo0, hi, kIdescPV,
                j == 0 ? 0u : 1u, lane == 0 ? 1u : 0u, my_bar, my_par);
            if (lane == 0) tc_commit(bar_o_full(t));
            return __all_sync(0xffffffffu, mine != 0);
        };
        int j_main = 0;
        bool seen = false;
#pragma unroll 1
        for (; j_main + 2 < n_kv; ++j_main) {
            seen = half_step(I0{}, j_main, seen);
            seen = half_step(I1{}, j_main, seen);
        }
        // the last few half-steps, where landings run out
#pragma unroll 1
        for (int n = 2 * j_main; n < n_land; ++n) {
            // half-step n: tile t has finished the softmax of kv step j
            const int t = n & 1, j = n >> 1, s = j % kKvStages;
            const int m = n + 3;  // the landing issued in this half-step
            const bool has_land = m < n_land;
            const int jm = m >> 1, sm = jm % kKvStages;
            // one barrier per lane: 0 P_t stored, 1 V tile arrived, 2 region C free, 3 K tile arrived
            uint32_t my_bar = bar_p_full(t), my_par = static_cast<uint32_t>(j) & 1u;
            int my_site = SITE_P_FULL;
            if (lane == 1 && t == 0) {
                my_bar = bar_v_full(s);
                my_par = static_cast<uint32_t>(j / kKvStages) & 1u;
                my_site = SITE_V_FULL;
            } else if (lane == 2 && has_land) {
                my_bar = bar_c_free;
                my_par = static_cast<uint32_t>(m - 1) & 1u;
                my_site = SITE_C_FREE;
            } else if (lane == 3 && has_land && (m & 1) == 0) {
                my_bar = bar_k_full(sm);
                my_par = static_cast<uint32_t>(jm / kKvStages) & 1u;
                my_site = SITE_K_FULL;
            }
            if (!__all_sync(0xffffffffu, mbar_try_wait(my_bar, my_par))) {
                if (lane < 4) mbar_wait(my_bar, my_par, abort_flag, my_site, n);
                __syncwarp();
            }
            if (lane == 0) {
                tc_fence_after();
                if (has_land) {
                    issue_s(m & 1, sm);
                    tc_commit(bar_s_full(m & 1));
                }
                issue_pv(t, s, j == 0);
                tc_commit(bar_o_full(t));
            }
            __syncwarp();
        }
        if (lane == 0) {
            // everything issued must have retired before tensor memory is released
            tc_commit(bar_drain);
            mbar_wait(bar_drain, 0, abort_flag, SITE_DRAIN, 0);
            if (*abort_flag) {
                const long long t0 = clock64();
                while (!mbar_try_wait(bar_drain, 0) && clock64() - t0 < kWaitLimitCycles / 64) {
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
        // ------------------------- softmax + epilogue (one row per thread) -------------------------
        const int t = warp >> 2;
        const int row_in_tile = (warp & 3) * 32 + lane;
        const int qi = q0 + t * kBM + row_in_tile;  // global query row
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t c_addr = tmem_base + lane_base + kColC;
        const uint32_t p_addr = tmem_base + lane_base + (t ? kColP1 : kColP0);
        const uint32_t o_addr = tmem_base + lane_base + kColO + t * kD;
        float m = -INFINITY, l = 0.f;

#pragma unroll 1
        for (int j = 0; j < n_kv; ++j) {
            mbar_wait(bar_s_full(t), static_cast<uint32_t>(j) & 1u, abort_flag, SITE_S_FULL, j);
            __syncwarp();
            tc_fence_after();
            float x[128];
            tmem_ld128_wait(c_addr, x);
            // the scores are in registers: hand region C back for the other tile's next S
            tc_fence_before();
            mbar_arrive(bar_c_free);
            // S of tile 1 was the last user of this K tile
            if (t == kTiles - 1) mbar_arrive(bar_k_empty(j % kKvStages));

            // mask (diagonal / tail tiles only), then the row extreme of the RAW scores: the scale is folded
            // into the exponent argument below, y = s * c - m with m kept in scaled log2 units
            const bool neg = p.scale_log2 < 0.f;
            const int kv0 = (j_lo + j) * kBN;  // first kv position of this tile
            const bool need_mask = (kv0 + kBN > p.Skv) || (p.causal && (kv0 + kBN - 1 > q0 + t * kBM)) ||
                                   (p.window > 0 && (kv0 < q0 + t * kBM + kBM - 1 - (p.window - 1)));
            if (need_mask) {
                int limit = p.Skv - 1 - kv0;  // last valid column of this tile
                if (p.causal) {
                    const int cl = qi - kv0;
                    limit = cl < limit ? cl : limit;
                }
                const int first = p.window > 0 ? qi - (p.window - 1) - kv0 : 0;  // first valid column
                const float masked = neg ? INFINITY : -INFINITY;
#pragma unroll
                for (int c = 0; c < 128; ++c)
                    if (c > limit || c < first) x[c] = masked;
            }
            // (three-input min/max: 64 instructions for the 128 scores instead of 128)
            float e0 = neg ? INFINITY : -INFINITY, e1 = e0, e2 = e0, e3 = e0;
            if (neg) {
#pragma unroll
                for (int c = 0; c < 128; c += 8) {
                    e0 = min3(e0, x[c], x[c + 1]);
                    e1 = min3(e1, x[c + 2], x[c + 3]);
                    e2 = min3(e2, x[c + 4], x[c + 5]);
                    e3 = min3(e3, x[c + 6], x[c + 7]);
                }
            } else {
#pragma unroll
                for (int c = 0; c < 128; c += 8) {
                    e0 = max3(e0, x[c], x[c + 1]);
                    e1 = max3(e1, x[c + 2], x[c + 3]);
                    e2 = max3(e2, x[c + 4], x[c + 5]);
                    e3 = max3(e3, x[c + 6], x[c + 7]);
                }
            }
            e0 = neg ? fminf(e0, e1) : fmaxf(e0, e1);
            e2 = neg ? fminf(e2, e3) : fmaxf(e2, e3);
            const float mx = (neg ? fminf(e0, e2) : fmaxf(e0, e2)) * p.scale_log2;

            // P V of the previous step must have retired before O_t is rescaled or P_t overwritten.  It was issued
            // when this tile's previous softmax ended, so the wait is put as late as possible: inside the (rare)
            // rescale, otherwise after the exponentials, just before the probabilities are stored.
            bool pv_retired = (j == 0);
            auto wait_pv = [&]() {
                if (!pv_retired) {
                    mbar_wait(bar_o_full(t), static_cast<uint32_t>(j - 1) & 1u, abort_flag, SITE_O_FULL, j);
                    __syncwarp();
                    tc_fence_after();
                    pv_retired = true;
                    // P V of tile 1 was the last user of the previous V tile
                    if (t == kTiles - 1) mbar_arrive(bar_v_empty((j - 1) % kKvStages));
                }
            };
            // raise the running maximum only when it pays (always on the first tile)
            float alpha = 1.f;
            const bool grow = (j == 0) || (mx > m + kRescaleThreshold);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = fmaxf(m, mx);
                if (j > 0) {
                    // a lane taken along by the warp vote may still have seen no visible key (sliding window)
                    alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m - m_new);
                    wait_pv();
#pragma unroll 1
                    for (int c = 0; c < 8; ++c) {
                        uint32_t ou[16];
                        tmem_ld16_wait(o_addr + c * 16, ou);
#pragma unroll
                        for (int e = 0; e < 16; ++e) ou[e] = __float_as_uint(__uint_as_float(ou[e]) * alpha);
                        tmem_st16(o_addr + c * 16, ou);
                    }
                }
                m = m_new;
            }

            // probabilities (bf16), row sum from the fp32 values.
            // A row that has not seen a visible key yet (sliding window) still has m = -inf: its scores are all
            // masked, so any finite reference gives the right probabilities (zeros)
            const float m_ref = (m == -INFINITY) ? 0.f : m;
            const uint64_t c2 = pk2(p.scale_log2, p.scale_log2), nm2 = pk2(-m_ref, -m_ref);
            uint64_t sum2 = pk2(0.f, 0.f);
            uint32_t pk[64];
#pragma unroll
            for (int e = 0; e < 64; ++e) {
                const int col = e * 2;
                const uint64_t y = fma2(pk2(x[col], x[col + 1]), c2, nm2);
                float p0, p1;
                exp2_pair_sfu(y, p0, p1);
                sum2 = add2(sum2, pk2(p0, p1));
                pk[e] = pack_bf16x2(p0, p1);
            }
            wait_pv();
            tmem_st32(p_addr, *reinterpret_cast<const uint32_t(*)[32]>(&pk[0]));
            tmem_st32(p_addr + 32, *reinterpret_cast<const uint32_t(*)[32]>(&pk[32]));
            float s_lo, s_hi;
            upk2(sum2, s_lo, s_hi);
            l = l * alpha + (s_lo + s_hi);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar_p_full(t));
        }

        // epilogue: O / l -> bf16, lse = m + log(l)
        mbar_wait(bar_o_full(t), static_cast<uint32_t>(n_kv - 1) & 1u, abort_flag, SITE_O_FULL, n_kv);
        __syncwarp();
        tc_fence_after();
        // optional sink term in the denominator; rows without any visible key give zeros
        const float sink = p.sink ? p.sink[h] : 0.f;
        const bool visible = l > 0.f;
        const float denom = l + ((p.sink && visible) ? sink * fast_exp2(-m) : 0.f);
        const float inv_l = visible ? 1.f / denom : 0.f;
        const bool row_ok = qi < p.Sq;
        if (p.part) {
            // split-KV: the un-normalised accumulator and (m, l) of this share, one packed fp32 row per query row
            // (the share index is worked out again here rather than kept in a register through the kv loop)
            const int share = static_cast<int>(blockIdx.x) / (p.G * p.n_qp * p.Hkv * p.B);
            float* dst = p.part + ((static_cast<size_t>(share) * p.B + b) * p.Hq + h) * static_cast<size_t>(p.Sq) * 130 +
                         static_cast<size_t>(qi) * 130;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float ov[32];
                tmem_ld32_wait(o_addr + c * 32, ov);
                if (row_ok) {
#pragma unroll
                    for (int e = 0; e < 32; e += 2)
                        *reinterpret_cast<float2*>(dst + c * 32 + e) = make_float2(ov[e], ov[e + 1]);
                }
            }
            if (row_ok) *reinterpret_cast<float2*>(dst + 128) = make_float2(m * kLn2, l);
            tc_fence_before();
        } else {
        // O goes out through shared memory and a bulk tensor store: written row by row from the threads, one
        // store instruction touches 32 different lines and the epilogue is bound by those transactions.  The Q
        // tile of this query tile is free (every MMA has retired) and has the layout the store expects: two
        // [128 rows][64 columns] halves, 16-byte chunks of a row XOR-ed with the row index modulo 8.
        const uint32_t stage_o = base + kSmemQ + t * kTileBytes;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            float ov[32];
            tmem_ld32_wait(o_addr + c * 32, ov);
            const uint32_t row_base = stage_o + (c >> 1) * kHalfBytes + row_in_tile * 128;
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
                const uint32_t chunk = static_cast<uint32_t>((c & 1) * 4 + (e >> 3));
                const uint32_t dst = row_base + ((chunk ^ (static_cast<uint32_t>(row_in_tile) & 7u)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                             "r"(pack_bf16x2(ov[e + 0] * inv_l, ov[e + 1] * inv_l)),
                             "r"(pack_bf16x2(ov[e + 2] * inv_l, ov[e + 3] * inv_l)),
                             "r"(pack_bf16x2(ov[e + 4] * inv_l, ov[e + 5] * inv_l)),
                             "r"(pack_bf16x2(ov[e + 6] * inv_l, ov[e + 7] * inv_l))
                             : "memory");
            }
        }
        fence_async_proxy();               // make the rows visible to the copy engine ...
        named_bar_sync(1 + t, kBM);        // ... once all 128 threads of this tile have written theirs
        if (row_in_tile == 0) {
            tma_store_4d(&tm_o, stage_o, 0, q0 + t * kBM, h, b);
            tma_store_4d(&tm_o, stage_o + kHalfBytes, 64, q0 + t * kBM, h, b);
            tma_store_commit_and_wait();
        }
        if (row_ok && p.lse)
            p.lse[(static_cast<long long>(b) * p.Hq + h) * p.Sq + qi] =
                visible ? (m + log2f(denom)) * kLn2 : (p.sink ? logf(fmaxf(sink, 1.0e-9f)) : -INFINITY);
        tc_fence_before();
        }
    }

    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static int encode_bhsd_map(CUtensorMap* map, const void* basep, int B, int H, int S, uint32_t box_rows = 128) {
    const uint64_t row = static_cast<uint64_t>(kD) * 2;
    const uint64_t dims[4] = {static_cast<uint64_t>(kD), static_cast<uint64_t>(S), static_cast<uint64_t>(H),
                              static_cast<uint64_t>(B)};
    const uint64_t strides[3] = {row, row * S, row * S * H};
    const uint32_t box[4] = {64, box_rows, 1, 1};
    return encode_bf16_4d(map, basep, dims, strides, box);
}

// How a forward call is laid out.  Two things can be changed without changing the result, both only for the plain
// (non-causal, no window, no sink) case:
//   * the query heads of a group become extra query ROWS of their kv head (q [B,Hq,Sq,D] read as [B,Hkv,G*Sq,D] is
//     the same memory) when one head alone does not fill a block's two tiles -- the heads of a group read the same
//     K/V, so a block then streams each K/V tile once for 256 rows of several heads;
//   * the kv range is cut into n_split shares handled by different blocks (flash-decoding), when there are fewer
//     blocks than SMs and enough kv tiles; the shares' packed partials go to the workspace and
//     decode::combine_rows_kernel merges them.  Needs a workspace of ws_bytes.
struct Layout {
    int Hq_eff, Sq_eff, n_split;
    size_t ws_bytes;
    bool merged;
};
// Blocks of the launch without any of that: one per (batch, head, 256 rows), or, for chunks of at most 128 rows, the
// one-tile kernel's count (chunks of at most 64 rows share a tile among P heads of a group: rows rounded up to a
// power of two R, P = min(128 / R, largest power of two dividing G)).
static long long plain_block_count(int B, int Sq, int Hq, int Hkv) {
    if (Sq > kBM) return static_cast<long long>(B) * Hq * ((Sq + kTiles * kBM - 1) / (kTiles * kBM));
    const int G = Hq / Hkv;
    int P = 1;
    if (Sq <= 64) {
        int R = 1;
        while (R < Sq) R <<= 1;
        P = kBM / R;
        while (P > 1 && (G % P) != 0) P >>= 1;
    }
    return static_cast<long long>(B) * Hkv * (G / P);
}

static Layout choose_layout(int B, int Sq, int Skv, int Hq, int Hkv, int causal, int window, const float* sink,
                            int sm_count, bool may_split) {
    Layout L;
    L.Hq_eff = Hq;
    L.Sq_eff = Sq;
    L.n_split = 1;
    L.ws_bytes = 0;
    L.merged = false;
    if (causal || window > 0 || sink) return L;
    const int G = Hq / Hkv;
    if (G > 1 && Sq < kTiles * kBM && static_cast<long long>(G) * Sq > kBM) {
        L.merged = true;
        L.Hq_eff = Hkv;
        L.Sq_eff = G * Sq;
    }
    const long long n_qp = (L.Sq_eff + kTiles * kBM - 1) / (kTiles * kBM);
    const long long base = static_cast<long long>(B) * L.Hq_eff * n_qp;
    const int tiles = (Skv + kBN - 1) / kBN;
    // Measured: with the kv range shared out each K/V tile is read by fewer blocks, comes from HBM rather than L2 and
    // the two-stage K/V pipeline stalls on it, and the shares' partials cost a second kernel -- so the cut pays only
    // where the ordinary launch would leave most of the GPU idle.
    if (may_split && base < sm_count && tiles >= 16 && 2 * plain_block_count(B, Sq, Hq, Hkv) < sm_count) {
        long long want = sm_count / base;
        if (want > tiles / 8) want = tiles / 8;  // a share of fewer than eight tiles is mostly start-up and drain
        if (want > 16) want = 16;
        if (want >= 2) {
            const int len = static_cast<int>((tiles + want - 1) / want);
            L.n_split = (tiles + len - 1) / len;  // every share non-empty
            L.ws_bytes = static_cast<size_t>(L.n_split) * B * Hq * Sq * 130 * sizeof(float);
        }
    }
    return L;
}

static int launch(const void* q, const void* k, const void* v, float scale, int causal, int window, const float* sink,
                  void* o, float* lse, int B, int Sq, int Skv, int Hq, int Hkv, int D, cudaStream_t stream,
                  const Layout* layout = nullptr, void* workspace = nullptr) {
    if (window < 0) return CLLO_E_BAD_ARG;
    // masked scores are +-infinity BEFORE the scale is folded into the exponent: a zero (or non-finite) scale would
    // turn them into NaN, so it is refused
    if (!(scale != 0.f) || !isfinite(scale)) return CLLO_E_BAD_ARG;
    if (!q || !k || !v || !o) return CLLO_E_BAD_ARG;
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) return CLLO_E_BAD_ARG;
    if (Hq % Hkv != 0) return CLLO_E_BAD_ARG;
    if (!aligned_to(q, 16) || !aligned_to(k, 16) || !aligned_to(v, 16) || !aligned_to(o, 16)) return CLLO_E_BAD_ARG;
    if (D != kD) return CLLO_E_UNSUPPORTED;
    DeviceInfo* di = nullptr;
    int rc = current_device_info(&di);
    if (rc != CLLO_OK) return rc;
    if (di->cc_major != 10) return CLLO_E_UNSUPPORTED;

    const long long rows_total = static_cast<long long>(B) * Hq * Sq;
    int n_split = 1;
    if (layout) {  // heads as rows and/or kv shares (see choose_layout); the memory is read the same way
        Hq = layout->Hq_eff;
        Sq = layout->Sq_eff;
        n_split = layout->n_split;
        if (n_split > 1 && (!workspace || !aligned_to(workspace, 16))) return CLLO_E_WORKSPACE;
    }
    Params p;
    p.o = static_cast<__nv_bfloat16*>(o);
    p.lse = lse;
    p.scale_log2 = scale * kLog2e;
    p.B = B;
    p.Sq = Sq;
    p.Skv = Skv;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = Hq / Hkv;
    p.causal = (causal || window > 0) ? 1 : 0;
    p.window = window;
    p.sink = sink;
    p.part = n_split > 1 ? static_cast<float*>(workspace) : nullptr;
    p.n_split = n_split;
    p.n_qp = (Sq + kTiles * kBM - 1) / (kTiles * kBM);
    const long long blocks = static_cast<long long>(B) * Hq * p.n_qp * n_split;
    if (blocks > 0x7fffffffLL || rows_total > 0x7fffffffLL) return CLLO_E_UNSUPPORTED;

    CUtensorMap tm_q, tm_k, tm_v, tm_o;
    if ((rc = encode_bhsd_map(&tm_q, q, B, Hq, Sq)) != CLLO_OK) return rc;
    if ((rc = encode_bhsd_map(&tm_k, k, B, Hkv, Skv)) != CLLO_OK) return rc;
    if ((rc = encode_bhsd_map(&tm_v, v, B, Hkv, Skv)) != CLLO_OK) return rc;
    if ((rc = encode_bhsd_map(&tm_o, o, B, Hq, Sq)) != CLLO_OK) return rc;

    if (!di->prefill_attr_set) {
        // the register re-balancing inside the kernel assumes the pool the kernel is launched with: refuse to
        // launch (rather than block inside setmaxnreg) if the compiler gave the kernel fewer registers
        cudaFuncAttributes fa;
        CLLO_CUDA_TRY(cudaFuncGetAttributes(&fa, reinterpret_cast<const void*>(prefill_fwd_kernel)));
        if (fa.numRegs < kLaunchRegs) return CLLO_E_UNSUPPORTED;
        CLLO_CUDA_TRY(cudaFuncSetAttribute(prefill_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        di->prefill_attr_set = true;
    }
    const unsigned grid = static_cast<unsigned>(blocks);
    prefill_fwd_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_o, p);
    CLLO_CUDA_TRY(cudaGetLastError());
    if (n_split > 1) {
        decode::combine_rows_kernel<<<static_cast<unsigned>((rows_total + decode::kCombineRows - 1) / decode::kCombineRows),
                                      decode::kCombineRows * 32, 0, stream>>>(p.part, n_split, rows_total, p.o, lse);
        CLLO_CUDA_TRY(cudaGetLastError());
    }
    return CLLO_OK;
}

}  // namespace prefill
}  // namespace cllo
