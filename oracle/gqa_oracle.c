/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the flash grouped-query attention path.
 *
 * This file restates, in plain C, the CPU reference attention that the upstream
 * project (LiuYiyang-Canton/cuda_llm_ops) uses to check its own GQA kernels.  It is
 * the checker for the CUDA path in this repository; nothing that ships (the package,
 * the C-ABI library) may call it.  Only the tests, the smoke check and the CPU-baseline
 * leg of the benchmark load it.
 *
 * Parity pin: (1) the decode function is bit-identical to the upstream CPU loop when
 * both are run on the upstream test's own inputs (see ref_stubs.cpp + Makefile target
 * `_ref`: the unmodified upstream test program is linked against stubs that hand our
 * result back to it, and it prints "O error = 0"); (2) decode and prefill are checked
 * against vectors produced by importing the upstream torch oracles (tests/golden).
 *
 * bf16 values travel as uint16_t bit patterns.  All index arithmetic is 64-bit.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even, the rounding of __float2bfloat16 / the __nv_bfloat16(float) ctor */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu; /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* element offset of K/V[b, s, h, d] for the two supported cache layouts */
static inline int64_t kv_index(int kv_layout, int64_t b, int64_t s, int64_t h, int64_t d,
                               int64_t S, int64_t Hkv, int64_t D) {
    if (kv_layout == 0) /* [B, S, Hkv, D]: upstream C++ layout, decode_flash_gqa_kernel.cu:144-148 */
        return ((b * S + s) * Hkv + h) * D + d;
    /* [B, Hkv, S, D]: upstream Triton layout, decode_flash_gqa_kernel.py:50-53 */
    return ((b * Hkv + h) * S + s) * D + d;
}

int cllo_oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * Single-token GQA decode over KV positions [s_begin, s_end).
 *
 * Follows examples/cplusplus/test_decode_flash_gqa.cu:184-255 statement by statement:
 * per (batch, query head) a running (rowmax, rowsum, O) over tiles of `tile` tokens
 * (upstream FLASH_BLOCK_SIZE = 128); the score is an fp32 dot product accumulated in
 * d order (:190-196); the tile max is taken over score*scale (:198-204); the tile sum
 * uses fp32 expf (:205-211); P is rounded to bf16 before the PV product (:212-220);
 * O and rowsum are rescaled by expf(rowmax - newrowmax) (:222-244); the result is
 * O / rowsum rounded to bf16 (:247-253).  OpenMP runs over batch exactly as upstream
 * (:183); `par_heads` != 0 moves the pragma to the head loop for B == 1 workloads.
 *
 * A ragged last tile (upstream requires S % 128 == 0) is truncated, which is the masked
 * behaviour of the upstream Triton twin (decode_flash_gqa_kernel.py:87-98).
 *
 * q [B,Hq,D]; k,v per kv_layout; o [B,Hq,D] bf16 (nullable);
 * o_unnorm [B,Hq,D] fp32, m_out/l_out [B,Hq] (all nullable): the un-normalised partial
 * (O, m, l) of the range, with m in units of scaled score and l relative to m.  An empty
 * range yields O = 0, m = -inf, l = 0 and leaves `o` untouched.
 */
int cllo_oracle_gqa_decode_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, float scale,
                                uint16_t* o, float* o_unnorm, float* m_out, float* l_out,
                                int B, int S, int Hq, int Hkv, int D, int kv_layout,
                                int s_begin, int s_end, int tile, int par_heads) {
    if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || tile <= 0) return -1;
    if (Hq % Hkv != 0) return -1;
    if (s_begin < 0) s_begin = 0;
    if (s_end > S) s_end = S;
    const int G = Hq / Hkv;
    const int64_t units = (int64_t)B * Hq;
    int failed = 0;

#pragma omp parallel
    {
        float* sbuf = (float*)malloc(sizeof(float) * (size_t)tile);
        uint16_t* pbuf = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)tile);
        float* oacc = (float*)malloc(sizeof(float) * (size_t)D);
        if (!sbuf || !pbuf || !oacc) {
#pragma omp atomic write
            failed = 1;
        } else {
            /* batch-parallel like upstream, or (batch*head)-parallel when asked */
            const int64_t outer = par_heads ? units : (int64_t)B;
            const int64_t inner = par_heads ? 1 : (int64_t)Hq;
#pragma omp for schedule(static)
            for (int64_t it = 0; it < outer; ++it) {
                for (int64_t jn = 0; jn < inner; ++jn) {
                    const int64_t batch = par_heads ? it / Hq : it;
                    const int64_t head = par_heads ? it % Hq : jn;
                    const int64_t kvh = head / G;
                    const uint16_t* qrow = q + (batch * Hq + head) * D;
                    float rowmax = -INFINITY, newrowmax, rowsum = 0.f, newrowsum;
                    int first = 1;
                    for (int d = 0; d < D; ++d) oacc[d] = 0.f;
                    for (int t0 = s_begin; t0 < s_end; t0 += tile) {
                        const int t1 = (t0 + tile < s_end) ? t0 + tile : s_end;
                        for (int token = t0; token < t1; ++token) {
                            float qk = 0.f;
                            for (int d = 0; d < D; ++d)
                                qk += bf16_to_f32(qrow[d]) *
                                      bf16_to_f32(k[kv_index(kv_layout, batch, token, kvh, d, S, Hkv, D)]);
                            sbuf[token - t0] = qk;
                        }
                        newrowmax = rowmax;
                        for (int token = t0; token < t1; ++token)
                            newrowmax = fmaxf(newrowmax, sbuf[token - t0] * scale);
                        newrowsum = 0.f;
                        for (int token = t0; token < t1; ++token)
                            newrowsum += expf(sbuf[token - t0] * scale - newrowmax);
                        for (int token = t0; token < t1; ++token)
                            pbuf[token - t0] = f32_to_bf16(expf(sbuf[token - t0] * scale - newrowmax));
                        for (int d = 0; d < D; ++d) {
                            float acc = 0.f;
                            for (int token = t0; token < t1; ++token)
                                acc += bf16_to_f32(pbuf[token - t0]) *
                                       bf16_to_f32(v[kv_index(kv_layout, batch, token, kvh, d, S, Hkv, D)]);
                            if (first)
                                oacc[d] = acc;
                            else
                                oacc[d] = oacc[d] * expf(rowmax - newrowmax) + acc;
                        }
                        rowsum = rowsum * expf(rowmax - newrowmax) + newrowsum;
                        rowmax = newrowmax;
                        first = 0;
                    }
                    const int64_t row = batch * Hq + head;
                    if (o && !first)
                        for (int d = 0; d < D; ++d) o[row * D + d] = f32_to_bf16(oacc[d] / rowsum);
                    if (o_unnorm)
                        for (int d = 0; d < D; ++d) o_unnorm[row * D + d] = oacc[d];
                    if (m_out) m_out[row] = rowmax;
                    if (l_out) l_out[row] = rowsum;
                }
            }
        }
        free(sbuf);
        free(pbuf);
        free(oacc);
    }
    return failed ? -2 : 0;
}

/*
 * Log-sum-exp merge of `nsplit` partial results.
 *
 * partials is [nsplit][rows][D+2] fp32: D un-normalised output values, then m, then l.
 * Same monoid as the running update of the decode loop (test_decode_flash_gqa.cu:222-244)
 * and as TileMaxSumReduce (src/cplusplus/Softmax/softmax_kernel.cu:21-34):
 *   m* = max_i m_i;  O = sum_i e^(m_i-m*) O_i / sum_i e^(m_i-m*) l_i.
 * Splits with l == 0 (empty ranges) contribute nothing.  Rows whose every split is empty
 * produce zeros.  o (bf16) and o_f32 are both nullable.
 */
int cllo_oracle_gqa_combine(const float* partials, int nsplit, int64_t rows, int D,
                            uint16_t* o, float* o_f32) {
    if (nsplit <= 0 || rows <= 0 || D <= 0) return -1;
    const int64_t W = (int64_t)D + 2;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float mstar = -INFINITY;
        for (int i = 0; i < nsplit; ++i) {
            const float* p = partials + ((int64_t)i * rows + r) * W;
            if (p[D + 1] > 0.f) mstar = fmaxf(mstar, p[D]);
        }
        float lsum = 0.f;
        for (int i = 0; i < nsplit; ++i) {
            const float* p = partials + ((int64_t)i * rows + r) * W;
            if (p[D + 1] > 0.f) lsum += expf(p[D] - mstar) * p[D + 1];
        }
        for (int d = 0; d < D; ++d) {
            float acc = 0.f;
            for (int i = 0; i < nsplit; ++i) {
                const float* p = partials + ((int64_t)i * rows + r) * W;
                if (p[D + 1] > 0.f) acc += expf(p[D] - mstar) * p[d];
            }
            const float val = lsum > 0.f ? acc / lsum : 0.f;
            if (o) o[r * D + d] = f32_to_bf16(val);
            if (o_f32) o_f32[r * D + d] = val;
        }
    }
    return 0;
}

/*
 * Prefill (multi-token) GQA forward, layout q,o [B,Hq,Sq,D]; k,v [B,Hkv,Skv,D]; lse [B,Hq,Sq].
 *
 * Follows examples/python/Triton/test_flash_gqa_kernel.py:60-94: fp32 scores = (q.k)*scale
 * (:78), masked to -inf above the diagonal (:69-72,79; the mask keeps kv <= q, aligned at the
 * top-left corner like flash_gqa_kernel.py:104,114), row max (:80), exp (:81), probabilities
 * = exp / sum (:82), lse = log(sum) + max (:83), out = probs @ V in fp32 (:85) then rounded to
 * bf16 (:90-92).  Upstream is causal-only; `causal == 0` simply skips the mask.
 *
 * Rows can be restricted to [row_begin, row_end) of every head (sampled checks of big shapes);
 * rows outside the range are not written.  o is nullable, lse is nullable.
 */
int cllo_oracle_gqa_prefill_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, float scale,
                                 int causal, uint16_t* o, float* lse,
                                 int B, int Sq, int Skv, int Hq, int Hkv, int D,
                                 int row_begin, int row_end) {
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) return -1;
    if (Hq % Hkv != 0) return -1;
    if (row_begin < 0) row_begin = 0;
    if (row_end > Sq) row_end = Sq;
    const int G = Hq / Hkv;
    const int64_t nrows = (int64_t)(row_end - row_begin);
    if (nrows <= 0) return 0;
    const int64_t total = (int64_t)B * Hq * nrows;
    int failed = 0;
#pragma omp parallel
    {
        float* sc = (float*)malloc(sizeof(float) * (size_t)Skv);
        float* kf = NULL;
        float* oacc = (float*)malloc(sizeof(float) * (size_t)D);
        float* qf = (float*)malloc(sizeof(float) * (size_t)D);
        if (!sc || !oacc || !qf) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(dynamic, 16)
            for (int64_t idx = 0; idx < total; ++idx) {
                const int64_t b = idx / ((int64_t)Hq * nrows);
                const int64_t h = (idx / nrows) % Hq;
                const int64_t i = row_begin + idx % nrows;
                const int64_t kvh = h / G;
                const uint16_t* qrow = q + ((b * Hq + h) * Sq + i) * D;
                const uint16_t* kb = k + (b * Hkv + kvh) * (int64_t)Skv * D;
                const uint16_t* vb = v + (b * Hkv + kvh) * (int64_t)Skv * D;
                int64_t n = Skv;
                if (causal && i + 1 < n) n = i + 1;
                for (int d = 0; d < D; ++d) qf[d] = bf16_to_f32(qrow[d]);
                float rmax = -INFINITY;
                for (int64_t j = 0; j < n; ++j) {
                    float acc = 0.f;
                    const uint16_t* kr = kb + j * D;
                    for (int d = 0; d < D; ++d) acc += qf[d] * bf16_to_f32(kr[d]);
                    sc[j] = acc * scale;
                    rmax = fmaxf(rmax, sc[j]);
                }
                float sum = 0.f;
                for (int64_t j = 0; j < n; ++j) {
                    sc[j] = expf(sc[j] - rmax);
                    sum += sc[j];
                }
                for (int d = 0; d < D; ++d) oacc[d] = 0.f;
                for (int64_t j = 0; j < n; ++j) {
                    const float p = sc[j] / sum;
                    const uint16_t* vr = vb + j * D;
                    for (int d = 0; d < D; ++d) oacc[d] += p * bf16_to_f32(vr[d]);
                }
                if (o)
                    for (int d = 0; d < D; ++d) o[((b * Hq + h) * Sq + i) * D + d] = f32_to_bf16(oacc[d]);
                if (lse) lse[(b * Hq + h) * Sq + i] = logf(sum) + rmax;
            }
        }
        free(sc);
        free(kf);
        free(oacc);
        free(qf);
    }
    return failed ? -2 : 0;
}

/*
 * MLA-shaped forward: the same attention with head_dim_qk != head_dim_v, layout q [B,Hq,Sq,Dqk]; k [B,Hkv,Skv,Dqk];
 * v [B,Hkv,Skv,Dv]; o [B,Hq,Sq,Dv]; lse [B,Hq,Sq].  Follows flash_mla_forward_reference of
 * examples/python/Triton/test_flash_mla_kernel.py:27-94: fp32 scores = (q.k) * scale (:82), masked to -inf above the
 * diagonal (:70-73,83), row max (:84), exp (:85), probabilities = exp / sum (:86), lse = log(sum) + max (:87),
 * out = probs @ V in fp32 (:89), rounded to bf16 (:93-95).  Upstream's reference is causal-only; `causal == 0` skips
 * the mask.
 */
int cllo_oracle_mla_prefill_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, float scale, int causal,
                                 uint16_t* o, float* lse, int B, int Sq, int Skv, int Hq, int Hkv, int Dqk, int Dv) {
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || Dqk <= 0 || Dv <= 0) return -1;
    if (Hq % Hkv != 0) return -1;
    const int G = Hq / Hkv;
    const int64_t total = (int64_t)B * Hq * Sq;
    int failed = 0;
#pragma omp parallel
    {
        float* sc = (float*)malloc(sizeof(float) * (size_t)Skv);
        float* oacc = (float*)malloc(sizeof(float) * (size_t)Dv);
        float* qf = (float*)malloc(sizeof(float) * (size_t)Dqk);
        if (!sc || !oacc || !qf) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(dynamic, 16)
            for (int64_t idx = 0; idx < total; ++idx) {
                const int64_t b = idx / ((int64_t)Hq * Sq);
                const int64_t h = (idx / Sq) % Hq;
                const int64_t i = idx % Sq;
                const int64_t kvh = h / G;
                const uint16_t* qrow = q + ((b * Hq + h) * Sq + i) * Dqk;
                const uint16_t* kb = k + (b * Hkv + kvh) * (int64_t)Skv * Dqk;
                const uint16_t* vb = v + (b * Hkv + kvh) * (int64_t)Skv * Dv;
                int64_t n = Skv;
                if (causal && i + 1 < n) n = i + 1;
                for (int d = 0; d < Dqk; ++d) qf[d] = bf16_to_f32(qrow[d]);
                float rmax = -INFINITY;
                for (int64_t j = 0; j < n; ++j) {
                    float acc = 0.f;
                    const uint16_t* kr = kb + j * Dqk;
                    for (int d = 0; d < Dqk; ++d) acc += qf[d] * bf16_to_f32(kr[d]);
                    sc[j] = acc * scale;
                    rmax = fmaxf(rmax, sc[j]);
                }
                float sum = 0.f;
                for (int64_t j = 0; j < n; ++j) {
                    sc[j] = expf(sc[j] - rmax);
                    sum += sc[j];
                }
                for (int d = 0; d < Dv; ++d) oacc[d] = 0.f;
                for (int64_t j = 0; j < n; ++j) {
                    const float p = sc[j] / sum;
                    const uint16_t* vr = vb + j * Dv;
                    for (int d = 0; d < Dv; ++d) oacc[d] += p * bf16_to_f32(vr[d]);
                }
                if (o)
                    for (int d = 0; d < Dv; ++d) o[((b * Hq + h) * Sq + i) * Dv + d] = f32_to_bf16(oacc[d]);
                if (lse) lse[(b * Hq + h) * Sq + i] = logf(sum) + rmax;
            }
        }
        free(sc);
        free(oacc);
        free(qf);
    }
    return failed ? -2 : 0;
}

/*
 * Sliding-window attention forward with a sink term, layout as the prefill oracle above.
 *
 * Follows examples/python/Triton/test_flash_swa_kernel.py:28-118: a query at position i sees kv in
 * [i - (window - 1), i] (:84-86); fp32 scores * scale masked to -inf (:93-94); row max (:95);
 * denom = sum exp(s - max) + sink[h] * exp(-max) (:96-98); probs = exp / denom (:99);
 * lse = log(denom) + max (:100); out = probs @ V rounded to bf16 (:101-107).  A row that sees no key at all
 * (possible when Sq > Skv) is defined as in the upstream kernel (src/python/Triton/SWA/flash_swa_kernel.py:
 * has_visible_kv): zeros and lse = log(max(sink, 1e-9)).
 */
int cllo_oracle_swa_prefill_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, float scale,
                                 int window, const float* sink, uint16_t* o, float* lse,
                                 int B, int Sq, int Skv, int Hq, int Hkv, int D) {
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || window <= 0 || !sink) return -1;
    if (Hq % Hkv != 0) return -1;
    const int G = Hq / Hkv;
    const int64_t total = (int64_t)B * Hq * Sq;
    int failed = 0;
#pragma omp parallel
    {
        float* sc = (float*)malloc(sizeof(float) * (size_t)Skv);
        float* oacc = (float*)malloc(sizeof(float) * (size_t)D);
        float* qf = (float*)malloc(sizeof(float) * (size_t)D);
        if (!sc || !oacc || !qf) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(dynamic, 16)
            for (int64_t idx = 0; idx < total; ++idx) {
                const int64_t b = idx / ((int64_t)Hq * Sq);
                const int64_t h = (idx / Sq) % Hq;
                const int64_t i = idx % Sq;
                const int64_t kvh = h / G;
                const uint16_t* qrow = q + ((b * Hq + h) * Sq + i) * D;
                const uint16_t* kb = k + (b * Hkv + kvh) * (int64_t)Skv * D;
                const uint16_t* vb = v + (b * Hkv + kvh) * (int64_t)Skv * D;
                int64_t j0 = i - (window - 1);
                if (j0 < 0) j0 = 0;
                int64_t j1 = i < Skv - 1 ? i : Skv - 1; /* inclusive */
                for (int d = 0; d < D; ++d) oacc[d] = 0.f;
                if (j1 < j0) {
                    if (o)
                        for (int d = 0; d < D; ++d) o[((b * Hq + h) * Sq + i) * D + d] = 0;
                    if (lse) lse[(b * Hq + h) * Sq + i] = logf(fmaxf(sink[h], 1.0e-9f));
                    continue;
                }
                for (int d = 0; d < D; ++d) qf[d] = bf16_to_f32(qrow[d]);
                float rmax = -INFINITY;
                for (int64_t j = j0; j <= j1; ++j) {
                    float acc = 0.f;
                    const uint16_t* kr = kb + j * D;
                    for (int d = 0; d < D; ++d) acc += qf[d] * bf16_to_f32(kr[d]);
                    sc[j - j0] = acc * scale;
                    rmax = fmaxf(rmax, sc[j - j0]);
                }
                float sum = 0.f;
                for (int64_t j = j0; j <= j1; ++j) {
                    sc[j - j0] = expf(sc[j - j0] - rmax);
                    sum += sc[j - j0];
                }
                const float denom = sum + sink[h] * expf(-rmax);
                for (int64_t j = j0; j <= j1; ++j) {
                    const float p = sc[j - j0] / denom;
                    const uint16_t* vr = vb + j * D;
                    for (int d = 0; d < D; ++d) oacc[d] += p * bf16_to_f32(vr[d]);
                }
                if (o)
                    for (int d = 0; d < D; ++d) o[((b * Hq + h) * Sq + i) * D + d] = f32_to_bf16(oacc[d]);
                if (lse) lse[(b * Hq + h) * Sq + i] = logf(denom) + rmax;
            }
        }
        free(sc);
        free(oacc);
        free(qf);
    }
    return failed ? -2 : 0;
}

/*
 * Sparse-index GQA forward: restates flash_sgqa_forward_reference of
 * examples/python/Triton/test_flash_sgqa_kernel.py:102-216.  Per (batch, kv head, query token) a list of kv token
 * indices, shared by the query heads of the group (:185-189); an entry counts when 0 <= index < Skv and, if causal,
 * index <= query position (:191-193); fp32 scores * scale with the other entries at -inf (:199-200); row max,
 * exp, the masked entries forced to 0 (:202-204); probs = exp / denom, zero when denom = 0 (:205-206);
 * out = probs @ V_gathered in fp32, rounded to bf16 (:208,217); lse = log(denom) + max, -inf when denom = 0
 * (:209-213).  Repeated indices count as often as they are listed.
 */
int cllo_oracle_sgqa_prefill_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, const int32_t* sparse_idx,
                                  int num_sparse, float scale, int causal, uint16_t* o, float* lse,
                                  int B, int Sq, int Skv, int Hq, int Hkv, int D) {
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || num_sparse <= 0 || !sparse_idx) return -1;
    if (Hq % Hkv != 0) return -1;
    const int G = Hq / Hkv;
    const int64_t total = (int64_t)B * Hq * Sq;
    int failed = 0;
#pragma omp parallel
    {
        float* sc = (float*)malloc(sizeof(float) * (size_t)num_sparse);
        float* oacc = (float*)malloc(sizeof(float) * (size_t)D);
        float* qf = (float*)malloc(sizeof(float) * (size_t)D);
        if (!sc || !oacc || !qf) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(dynamic, 16)
            for (int64_t idx = 0; idx < total; ++idx) {
                const int64_t b = idx / ((int64_t)Hq * Sq);
                const int64_t h = (idx / Sq) % Hq;
                const int64_t i = idx % Sq;
                const int64_t kvh = h / G;
                const uint16_t* qrow = q + ((b * Hq + h) * Sq + i) * D;
                const uint16_t* kb = k + (b * Hkv + kvh) * (int64_t)Skv * D;
                const uint16_t* vb = v + (b * Hkv + kvh) * (int64_t)Skv * D;
                const int32_t* list = sparse_idx + ((b * Hkv + kvh) * Sq + i) * (int64_t)num_sparse;
                for (int d = 0; d < D; ++d) qf[d] = bf16_to_f32(qrow[d]);
                for (int d = 0; d < D; ++d) oacc[d] = 0.f;
                float rmax = -INFINITY;
                for (int e = 0; e < num_sparse; ++e) {
                    const int64_t j = list[e];
                    const int ok = j >= 0 && j < Skv && (!causal || j <= i);
                    if (!ok) {
                        sc[e] = -INFINITY;
                        continue;
                    }
                    float acc = 0.f;
                    const uint16_t* kr = kb + j * D;
                    for (int d = 0; d < D; ++d) acc += qf[d] * bf16_to_f32(kr[d]);
                    sc[e] = acc * scale;
                    rmax = fmaxf(rmax, sc[e]);
                }
                float denom = 0.f;
                for (int e = 0; e < num_sparse; ++e) {
                    sc[e] = sc[e] == -INFINITY ? 0.f : expf(sc[e] - rmax);
                    denom += sc[e];
                }
                if (denom > 0.f) {
                    for (int e = 0; e < num_sparse; ++e) {
                        if (sc[e] == 0.f) continue;
                        const float p = sc[e] / denom;
                        const uint16_t* vr = vb + (int64_t)list[e] * D;
                        for (int d = 0; d < D; ++d) oacc[d] += p * bf16_to_f32(vr[d]);
                    }
                }
                if (o)
                    for (int d = 0; d < D; ++d) o[((b * Hq + h) * Sq + i) * D + d] = f32_to_bf16(oacc[d]);
                if (lse) lse[(b * Hq + h) * Sq + i] = denom > 0.f ? logf(denom) + rmax : -INFINITY;
            }
        }
        free(sc);
        free(oacc);
        free(qf);
    }
    return failed ? -2 : 0;
}

/*
 * GQA attention backward, layout q,o,grad_o,grad_q [B,Hq,Sq,D]; k,v,grad_k,grad_v [B,Hkv,Skv,D] (bf16).
 *
 * Follows examples/python/Triton/test_flash_gqa_kernel.py:97-173: probabilities are recomputed from
 * fp32 scores with a row-max softmax and the causal mask (:152-156; `causal == 0` skips the mask, upstream
 * is causal-only); grad_p = grad_o V^T (:158); grad_p_dot = rowsum(grad_o o O) (:159);
 * grad_scores = (grad_p - grad_p_dot) o probs (:160); grad_q = grad_scores K * scale (:162);
 * grad_k = grad_scores^T Q * scale summed over the heads of the group (:163,168);
 * grad_v = probs^T grad_o summed over the heads of the group (:164,169); everything fp32, results rounded
 * to bf16 (:171).
 */
static int backward_impl(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* o,
                         const uint16_t* grad_o, float scale, int causal, int window, const float* sink,
                         uint16_t* grad_q, uint16_t* grad_k, uint16_t* grad_v,
                         int B, int Sq, int Skv, int Hq, int Hkv, int D) {
    if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) return -1;
    if (Hq % Hkv != 0) return -1;
    const int G = Hq / Hkv;
    const int64_t units = (int64_t)B * Hkv;
    int failed = 0;
#pragma omp parallel
    {
        float* dk = (float*)malloc(sizeof(float) * (size_t)Skv * D);
        float* dv = (float*)malloc(sizeof(float) * (size_t)Skv * D);
        float* pr = (float*)malloc(sizeof(float) * (size_t)Skv);
        float* dq = (float*)malloc(sizeof(float) * (size_t)D);
        if (!dk || !dv || !pr || !dq) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(dynamic, 1)
            for (int64_t u = 0; u < units; ++u) {
                const int64_t b = u / Hkv, kvh = u % Hkv;
                const uint16_t* kb = k + (b * Hkv + kvh) * (int64_t)Skv * D;
                const uint16_t* vb = v + (b * Hkv + kvh) * (int64_t)Skv * D;
                for (int64_t x = 0; x < (int64_t)Skv * D; ++x) dk[x] = dv[x] = 0.f;
                for (int g = 0; g < G; ++g) {
                    const int64_t h = kvh * G + g;
                    for (int64_t i = 0; i < Sq; ++i) {
                        const int64_t ro = ((b * Hq + h) * Sq + i) * D;
                        int64_t n = Skv;
                        if (causal && i + 1 < n) n = i + 1;
                        int64_t j0 = 0; /* first visible kv position */
                        if (window > 0 && i - (window - 1) > 0) j0 = i - (window - 1);
                        for (int d = 0; d < D; ++d) dq[d] = 0.f;
                        if (j0 >= n) { /* the row sees nothing: no gradient flows through it */
                            for (int d = 0; d < D; ++d) grad_q[ro + d] = 0;
                            continue;
                        }
                        float rmax = -INFINITY;
                        for (int64_t j = j0; j < n; ++j) {
                            float acc = 0.f;
                            for (int d = 0; d < D; ++d) acc += bf16_to_f32(q[ro + d]) * bf16_to_f32(kb[j * D + d]);
                            pr[j] = acc * scale;
                            rmax = fmaxf(rmax, pr[j]);
                        }
                        float sum = 0.f;
                        for (int64_t j = j0; j < n; ++j) {
                            pr[j] = expf(pr[j] - rmax);
                            sum += pr[j];
                        }
                        if (sink) sum += sink[h] * expf(-rmax);
                        float dot = 0.f;
                        for (int d = 0; d < D; ++d) dot += bf16_to_f32(grad_o[ro + d]) * bf16_to_f32(o[ro + d]);
                        for (int64_t j = j0; j < n; ++j) {
                            const float pj = pr[j] / sum;
                            float gp = 0.f;
                            for (int d = 0; d < D; ++d) gp += bf16_to_f32(grad_o[ro + d]) * bf16_to_f32(vb[j * D + d]);
                            const float gs = (gp - dot) * pj;
                            for (int d = 0; d < D; ++d) {
                                dq[d] += gs * bf16_to_f32(kb[j * D + d]);
                                dk[j * D + d] += gs * bf16_to_f32(q[ro + d]);
                                dv[j * D + d] += pj * bf16_to_f32(grad_o[ro + d]);
                            }
                        }
                        for (int d = 0; d < D; ++d) grad_q[ro + d] = f32_to_bf16(dq[d] * scale);
                    }
                }
                for (int64_t x = 0; x < (int64_t)Skv * D; ++x) {
                    grad_k[(b * Hkv + kvh) * (int64_t)Skv * D + x] = f32_to_bf16(dk[x] * scale);
                    grad_v[(b * Hkv + kvh) * (int64_t)Skv * D + x] = f32_to_bf16(dv[x]);
                }
            }
        }
        free(dk);
        free(dv);
        free(pr);
        free(dq);
    }
    return failed ? -2 : 0;
}

int cllo_oracle_gqa_backward_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* o,
                                  const uint16_t* grad_o, float scale, int causal,
                                  uint16_t* grad_q, uint16_t* grad_k, uint16_t* grad_v,
                                  int B, int Sq, int Skv, int Hq, int Hkv, int D) {
    return backward_impl(q, k, v, o, grad_o, scale, causal, 0, NULL, grad_q, grad_k, grad_v, B, Sq, Skv, Hq, Hkv, D);
}

/*
 * Backward of the sliding-window + sink forward.  Follows examples/python/Triton/test_flash_swa_kernel.py:121-220:
 * the same formulas as the plain backward with the window mask (kv in [i - (window - 1), i]) and the sink term
 * sink[h] * exp(-rowmax) added to the softmax denominator; the sink has no value vector, so it only scales the
 * probabilities.
 */
int cllo_oracle_swa_backward_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* o,
                                  const uint16_t* grad_o, float scale, int window, const float* sink,
                                  uint16_t* grad_q, uint16_t* grad_k, uint16_t* grad_v,
                                  int B, int Sq, int Skv, int Hq, int Hkv, int D) {
    if (window <= 0 || !sink) return -1;
    return backward_impl(q, k, v, o, grad_o, scale, 1, window, sink, grad_q, grad_k, grad_v, B, Sq, Skv, Hq, Hkv, D);
}

/*
 * Rotary position embedding over interleaved pairs of the whole hidden dimension.
 *
 * Follows examples/cplusplus/test_rope.cu:69-101: invFreq[i] = powf(base, -2 i / hidden) (:79-82); for each
 * token the fp32 angle token * invFreq[i] (:88), cosf / sinf of that fp32 value (:89-90), and the rotation of
 * the pair (2i, 2i+1) rounded to bf16 (:95-96).  input/output [B, S, hidden] bf16, hidden even.
 */
int cllo_oracle_rope_bf16(const uint16_t* input, uint16_t* output, int B, int S, int hidden, float base) {
    if (B <= 0 || S <= 0 || hidden <= 0 || (hidden & 1)) return -1;
    const int half = hidden / 2;
    float* inv = (float*)malloc(sizeof(float) * (size_t)half);
    if (!inv) return -2;
    const float hidden_inv = 1.0f / (float)hidden;
    for (int i = 0; i < half; ++i) inv[i] = powf(base, -2.0f * (float)i * hidden_inv);
#pragma omp parallel for schedule(static)
    for (int64_t bt = 0; bt < (int64_t)B * S; ++bt) {
        const int token = (int)(bt % S);
        const int64_t row = bt * hidden;
        for (int i = 0; i < half; ++i) {
            const float angle = (float)token * inv[i];
            const float c = cosf(angle), s = sinf(angle);
            const float even = bf16_to_f32(input[row + 2 * i]), odd = bf16_to_f32(input[row + 2 * i + 1]);
            output[row + 2 * i] = f32_to_bf16(even * c - odd * s);
            output[row + 2 * i + 1] = f32_to_bf16(even * s + odd * c);
        }
    }
    free(inv);
    return 0;
}
