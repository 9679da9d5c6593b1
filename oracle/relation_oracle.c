/*
 * CPU oracle for Relation LM's routed selection-and-reduction path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against (and the timed CPU baseline of the benchmark).  Nothing in
 * the shipped library links, loads or falls back to it.
 *
 * It restates, in plain C, the algorithms of the reference project's kernels
 * (paths are relative to the reference project root):
 *   - src/relation_lm/kernels/relation_select.py:50-308   fused anchor + partner selection
 *   - src/relation_lm/kernels/triton_select.py:23-120     anchor half
 *   - src/relation_lm/kernels/triton_select.py:140-252    partner half
 *   - src/relation_lm/kernels/router_cache.py:33-172      router state update
 *   - src/relation_lm/kernels/relation_reduce.py:72-146   factorised first relation layer (cached)
 *   - src/relation_lm/kernels/relation_reduce.py:186-309  same, with current-row cache update
 *   - src/relation_lm/kernels/relation_reduce.py:360-417  per-partner LayerNorm + active-K softmax + sum
 *   - src/relation_lm/inference/packed_cache.py:52-57     packed sparse-cache projection
 *
 * Parity pin: tests/golden/ holds outputs of the reference's own kernels
 * (run on CPU through Triton's interpreter by tests/golden/make_golden.py);
 * tests/test_oracle_golden.py checks every function here against them.
 *
 * Selection arithmetic is "canonical": every floating-point operation that
 * can change an index (dot products, block scores, log-sum-exp over heads,
 * softplus) is evaluated in one documented order with explicit fused
 * multiply-adds and with exp/log implemented in plain fp32 arithmetic, so a
 * GPU kernel following the same order produces bit-identical scores.  Build
 * with -ffp-contract=off so the compiler adds no contractions of its own.
 *
 *   dot64(k, q)   eight segments of eight consecutive elements; a segment is
 *                 acc = 0; acc = fmaf(k[i], q[i], acc) for ascending i; the
 *                 eight segment sums are added as ((s0+s1)+(s2+s3))+((s4+s5)+(s6+s7)).
 *   head dot      (head_dim 16) segment(2h) + segment(2h+1).
 *   head score    ((mdot + softplus(gamma_h) * sdot) * 0.25) + bias[h][bucket],
 *                 each operation rounded separately.
 *   block score   m = max_h s_h; m + log((e_0 + e_1) + (e_2 + e_3)), e_h = exp(s_h - m).
 *
 * All array arguments are fp32 (callers up-cast bf16/fp16 caches exactly, as
 * the kernels do on load) and row-major contiguous.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_D 64        /* exact-score width (gate_dim) */
#define ORC_HEADS 4     /* router heads */
#define ORC_HEAD_D 16   /* router head width */

/* ---------------------------------------------------------------- canonical exp / log */

static inline float as_float(int32_t bits) { float f; memcpy(&f, &bits, 4); return f; }
static inline int32_t as_int(float f) { int32_t b; memcpy(&b, &f, 4); return b; }

/* exp(x): Cody-Waite reduction by ln2 (two-constant split), degree-7 Taylor
 * polynomial on |r| <= 0.347, scaling by an integer add on the exponent field. */
float orc_expf(float x) {
    if (x != x) return x;
    if (x < -86.0f) return 0.0f;
    if (x > 88.0f) return INFINITY;
    const float magic = 12582912.0f; /* 1.5 * 2^23: adding it rounds to nearest-even integer */
    float kf = fmaf(x, 1.44269502f, magic) - magic;
    float r = fmaf(kf, -0.693145752f, x);
    r = fmaf(kf, -1.42860677e-06f, r);
    float p = 1.98412701e-04f;          /* 1/5040 */
    p = fmaf(p, r, 1.38888892e-03f);    /* 1/720 */
    p = fmaf(p, r, 8.33333377e-03f);    /* 1/120 */
    p = fmaf(p, r, 4.16666679e-02f);    /* 1/24 */
    p = fmaf(p, r, 1.66666672e-01f);    /* 1/6 */
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int32_t k = (int32_t)kf;
    return as_float(as_int(p) + k * (1 << 23));
}

/* log(y) for positive normal y: y = m * 2^e with m in [sqrt(1/2), sqrt(2)),
 * log(m) = 2 atanh(z), z = (m-1)/(m+1), odd series through z^11. */
float orc_logf(float y) {
    if (y != y || y < 0.0f) return NAN;
    if (y == 0.0f) return -INFINITY;
    if (y == INFINITY) return INFINITY;
    int32_t bits = as_int(y);
    int32_t e = (bits - 0x3f3504f3) >> 23;
    float m = as_float(bits - e * (1 << 23));
    float f = m - 1.0f;
    float z = f / (2.0f + f);
    float w = z * z;
    float p = 9.09090936e-02f;          /* 1/11 */
    p = fmaf(p, w, 1.11111112e-01f);    /* 1/9 */
    p = fmaf(p, w, 1.42857149e-01f);    /* 1/7 */
    p = fmaf(p, w, 0.2f);               /* 1/5 */
    p = fmaf(p, w, 3.33333343e-01f);    /* 1/3 */
    p = p * w;
    float z2 = z + z;
    float lm = fmaf(z2, p, z2);
    float ef = (float)e;
    float r = fmaf(ef, 1.42860677e-06f, lm);
    return fmaf(ef, 0.693145752f, r);
}

static inline float seg8(const float* a, const float* b) {
    float acc = 0.0f;
    for (int i = 0; i < 8; ++i) acc = fmaf(a[i], b[i], acc);
    return acc;
}

static inline float dot64(const float* k, const float* q) {
    float s[8];
    for (int j = 0; j < 8; ++j) s[j] = seg8(k + 8 * j, q + 8 * j);
    return ((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7]));
}

static inline int bucket_of(int t, int end, int buckets) {
    int d = t - end;
    if (d < 0) d = 0;
    int b = 31 - __builtin_clz((unsigned)(d + 1)); /* floor(log2(d + 1)), relation_select.py:61-65 */
    return b < buckets - 1 ? b : buckets - 1;
}

/* Block scores of one query against one sequence's block statistics
 * (relation_select.py:51-106 / 178-227). */
static void block_scores(const float* mean, const float* std, const float* rq,
                         const float* gamma, const float* bias, int nb, int bs,
                         int buckets, int t, int local, int strict, float* out) {
    float absq[ORC_D], sp[ORC_HEADS];
    for (int i = 0; i < ORC_D; ++i) absq[i] = fabsf(rq[i]);
    for (int h = 0; h < ORC_HEADS; ++h) sp[h] = orc_logf(1.0f + orc_expf(gamma[h]));
    int ls = t - local + 1;
    if (ls < 0) ls = 0;
    for (int n = 0; n < nb; ++n) {
        int end = (n + 1) * bs - 1;
        int eligible = end <= t;
        if (strict) eligible = eligible && end < ls;
        if (!eligible) { out[n] = -INFINITY; continue; }
        int bk = bucket_of(t, end, buckets);
        const float* m = mean + (size_t)n * ORC_D;
        const float* s = std + (size_t)n * ORC_D;
        float sh[ORC_HEADS];
        for (int h = 0; h < ORC_HEADS; ++h) {
            int o = h * ORC_HEAD_D;
            float md = seg8(m + o, rq + o) + seg8(m + o + 8, rq + o + 8);
            float sd = seg8(s + o, absq + o) + seg8(s + o + 8, absq + o + 8);
            float t1 = sp[h] * sd;
            float t2 = md + t1;
            float t3 = t2 * 0.25f;
            sh[h] = t3 + bias[h * buckets + bk];
        }
        /* log-sum-exp over the heads in the max-shifted form of torch.logsumexp
         * (routing/block_router.py:99; the Triton kernels fold the heads pairwise,
         * relation_select.py:97-103, which agrees to rounding). */
        float mx = fmaxf(fmaxf(sh[0], sh[1]), fmaxf(sh[2], sh[3]));
        float e0 = orc_expf(sh[0] - mx), e1 = orc_expf(sh[1] - mx);
        float e2 = orc_expf(sh[2] - mx), e3 = orc_expf(sh[3] - mx);
        float acc = mx + orc_logf((e0 + e1) + (e2 + e3));
        out[n] = acc;
    }
}

/* argmax with lowest-index tie-break (tl.argmax(..., tie_break_left=True)). */
static inline int argmax_left(const float* v, int n, float* best) {
    int bi = 0;
    float bv = v[0];
    for (int i = 1; i < n; ++i)
        if (v[i] > bv) { bv = v[i]; bi = i; }
    *best = bv;
    return bi;
}

/* Anchor selection for one query (relation_select.py:108-163). */
static inline int barred(int p, const int32_t* excl, int n_excl) {
    for (int i = 0; i < n_excl; ++i)
        if (excl[i] == p) return 1;
    return 0;
}

/* excl[0 .. n_excl): positions that may not be chosen (distinct anchors of a multi-anchor
 * layer, src/relation_lm/models/multi_relation_blocks.py:86-95); empty for the reference ops. */
static void anchor_one(const float* aq, const float* ak_seq, const float* bsc_in, int nb, int bs,
                       int t, int local, int top, const int32_t* excl, int n_excl, int* out_idx,
                       float* out_score, int64_t* scored, float* work) {
    int ls = t - local + 1;
    if (ls < 0) ls = 0;
    float best = -INFINITY;
    int best_pos = t - local + 1;
    int first = 1;
    for (int c = 0; c < local; ++c) {
        int p = t - local + 1 + c;
        float sc = -INFINITY;
        if (p >= 0 && p <= t && !barred(p, excl, n_excl)) { sc = dot64(ak_seq + (size_t)p * ORC_D, aq) * 0.125f; ++*scored; }
        if (first || sc > best) { best = sc; best_pos = p; first = 0; }
    }
    memcpy(work, bsc_in, sizeof(float) * (size_t)nb);
    for (int r = 0; r < top; ++r) {
        float bv;
        int bi = argmax_left(work, nb, &bv);
        int usable = bv > -1.0e30f;
        float cs = -INFINITY;
        int cpos = bi * bs;
        int cfirst = 1;
        for (int o = 0; o < bs; ++o) {
            int p = bi * bs + o;
            float sc = -INFINITY;
            if (usable && p <= t && p < ls && !barred(p, excl, n_excl)) { sc = dot64(ak_seq + (size_t)p * ORC_D, aq) * 0.125f; ++*scored; }
            if (cfirst || sc > cs) { cs = sc; cpos = p; cfirst = 0; }
        }
        if (cs > best || (cs == best && cpos < best_pos)) { best = cs; best_pos = cpos; }
        work[bi] = -INFINITY;
    }
    if (!(best > -INFINITY)) best_pos = 0;      /* every candidate was barred */
    *out_idx = best_pos;
    *out_score = best;
}

/* Partner top-K for one query (relation_select.py:229-308). */
static void partner_one(const float* pq, const float* pk_seq, const float* bsc_in, int nb, int bs,
                        int t, int local, int top, int k_out, int anchor, const int32_t* excl,
                        int n_excl, int* out_idx, float* out_score, int64_t* scored, float* work,
                        float* cs, int* cp) {
    int ls = t - local + 1;
    if (ls < 0) ls = 0;
    int cap = local + top * bs;
    memcpy(work, bsc_in, sizeof(float) * (size_t)nb);
    for (int c = 0; c < local; ++c) {
        int p = t - local + 1 + c;
        cp[c] = p;
        int valid = p >= 0 && p <= t && p != anchor && !barred(p, excl, n_excl);
        cs[c] = -INFINITY;
        if (valid) { cs[c] = dot64(pk_seq + (size_t)p * ORC_D, pq) * 0.125f; ++*scored; }
    }
    for (int r = 0; r < top; ++r) {
        float bv;
        int bi = argmax_left(work, nb, &bv);
        int usable = bv > -1.0e30f;
        work[bi] = -INFINITY;
        for (int o = 0; o < bs; ++o) {
            int c = local + r * bs + o;
            int p = bi * bs + o;
            cp[c] = p;
            int valid = usable && p <= t && p < ls && p != anchor && !barred(p, excl, n_excl);
            cs[c] = -INFINITY;
            if (valid) { cs[c] = dot64(pk_seq + (size_t)p * ORC_D, pq) * 0.125f; ++*scored; }
        }
    }
    for (int k = 0; k < k_out; ++k) {
        float bv;
        int bl = argmax_left(cs, cap, &bv);
        out_idx[k] = cp[bl];
        out_score[k] = bv;
        cs[bl] = -INFINITY;
    }
}

/*
 * Fused selection over N query rows.  Row i uses sequence row_batch[i] of the
 * caches at position row_pos[i]; the reference op is the special case
 * row_batch[i] = i, row_pos[i] = position for all i.
 * scored[0] / scored[1] accumulate the number of anchor / partner key rows
 * actually scored (for algorithmic-byte accounting); may be NULL.
 */
int orc_relation_select(int n_rows, int n_seq, int max_t, int nb, int buckets,
                        const int32_t* row_batch, const int32_t* row_pos,
                        const float* aq, const float* ak, const float* arq,
                        const float* amean, const float* astd, const float* agamma,
                        const float* abias, const float* pbase, const float* pac,
                        const float* pk, const float* pmean, const float* pstd,
                        const float* pgamma, const float* pbias, int local, int top,
                        int k_out, int strict, int32_t* out_anchor, float* out_anchor_score,
                        int32_t* out_partner, float* out_partner_score, int64_t* scored) {
    if (nb <= 0 || max_t % nb != 0 || local < 1 || top < 0 || k_out < 1) return -1;
    int bs = max_t / nb;
    int cap = local + top * bs;
    int64_t sa = 0, spn = 0;
    int bad = 0;
#pragma omp parallel reduction(+ : sa, spn) reduction(| : bad)
    {
        float* bsc = (float*)malloc(sizeof(float) * (size_t)nb * 2);
        float* work = bsc + nb;
        float* cs = (float*)malloc(sizeof(float) * (size_t)cap);
        int* cp = (int*)malloc(sizeof(int) * (size_t)cap);
#pragma omp for schedule(static)
        for (int i = 0; i < n_rows; ++i) {
            int b = row_batch[i], t = row_pos[i];
            if (b < 0 || b >= n_seq || t < 0 || t >= max_t) { bad = 1; continue; }
            const float* ak_seq = ak + (size_t)b * max_t * ORC_D;
            const float* pk_seq = pk + (size_t)b * max_t * ORC_D;
            size_t so = (size_t)b * nb * ORC_D;
            block_scores(amean + so, astd + so, arq + (size_t)i * ORC_D, agamma, abias, nb, bs,
                         buckets, t, local, strict, bsc);
            int anchor;
            anchor_one(aq + (size_t)i * ORC_D, ak_seq, bsc, nb, bs, t, local, top, NULL, 0, &anchor,
                       out_anchor_score + i, &sa, work);
            out_anchor[i] = anchor;
            float v[2 * ORC_D];
            const float* base = pbase + (size_t)i * 2 * ORC_D;
            const float* row = pac + ((size_t)b * max_t + anchor) * 2 * ORC_D;
            for (int c = 0; c < 2 * ORC_D; ++c) v[c] = base[c] + row[c];
            block_scores(pmean + so, pstd + so, v + ORC_D, pgamma, pbias, nb, bs, buckets, t,
                         local, strict, bsc);
            partner_one(v, pk_seq, bsc, nb, bs, t, local, top, k_out, anchor, NULL, 0,
                        out_partner + (size_t)i * k_out, out_partner_score + (size_t)i * k_out,
                        &spn, work, cs, cp);
        }
        free(bsc); free(cs); free(cp);
    }
    if (scored) { scored[0] += sa; scored[1] += spn; }
    return bad ? -2 : 0;
}

/* The anchor half alone (triton_select.py:23-120). */
int orc_anchor_select(int n_rows, int n_seq, int max_t, int nb, int buckets,
                      const int32_t* row_batch, const int32_t* row_pos, const float* aq,
                      const float* ak, const float* rq, const float* mean, const float* std,
                      const float* gamma, const float* bias, int local, int top, int strict,
                      const int32_t* exclude, int n_excl, int32_t* out_idx, float* out_score) {
    if (nb <= 0 || max_t % nb != 0 || local < 1 || top < 0) return -1;
    int bs = max_t / nb;
    int bad = 0;
#pragma omp parallel reduction(| : bad)
    {
        float* bsc = (float*)malloc(sizeof(float) * (size_t)nb * 2);
        int64_t dummy = 0;
#pragma omp for schedule(static)
        for (int i = 0; i < n_rows; ++i) {
            int b = row_batch[i], t = row_pos[i];
            if (b < 0 || b >= n_seq || t < 0 || t >= max_t) { bad = 1; continue; }
            size_t so = (size_t)b * nb * ORC_D;
            block_scores(mean + so, std + so, rq + (size_t)i * ORC_D, gamma, bias, nb, bs, buckets,
                         t, local, strict, bsc);
            int anchor;
            anchor_one(aq + (size_t)i * ORC_D, ak + (size_t)b * max_t * ORC_D, bsc, nb, bs, t,
                       local, top, exclude ? exclude + (size_t)i * n_excl : NULL, exclude ? n_excl : 0,
                       &anchor, out_score + i, &dummy, bsc + nb);
            out_idx[i] = anchor;
        }
        free(bsc);
    }
    return bad ? -2 : 0;
}

/* The partner half alone, queries and anchor supplied (triton_select.py:140-252). */
int orc_partner_topk(int n_rows, int n_seq, int max_t, int nb, int buckets,
                     const int32_t* row_batch, const int32_t* row_pos, const float* pq,
                     const float* pk, const float* rq, const float* mean, const float* std,
                     const float* gamma, const float* bias, const int32_t* anchor, int local,
                     int top, int k_out, int strict, const int32_t* exclude, int n_excl,
                     int32_t* out_idx, float* out_score) {
    if (nb <= 0 || max_t % nb != 0 || local < 1 || top < 0 || k_out < 1) return -1;
    int bs = max_t / nb;
    int cap = local + top * bs;
    int bad = 0;
#pragma omp parallel reduction(| : bad)
    {
        float* bsc = (float*)malloc(sizeof(float) * (size_t)nb * 2);
        float* cs = (float*)malloc(sizeof(float) * (size_t)cap);
        int* cp = (int*)malloc(sizeof(int) * (size_t)cap);
        int64_t dummy = 0;
#pragma omp for schedule(static)
        for (int i = 0; i < n_rows; ++i) {
            int b = row_batch[i], t = row_pos[i];
            if (b < 0 || b >= n_seq || t < 0 || t >= max_t) { bad = 1; continue; }
            size_t so = (size_t)b * nb * ORC_D;
            block_scores(mean + so, std + so, rq + (size_t)i * ORC_D, gamma, bias, nb, bs, buckets,
                         t, local, strict, bsc);
            partner_one(pq + (size_t)i * ORC_D, pk + (size_t)b * max_t * ORC_D, bsc, nb, bs, t,
                        local, top, k_out, anchor[i], exclude ? exclude + (size_t)i * n_excl : NULL,
                        exclude ? n_excl : 0, out_idx + (size_t)i * k_out,
                        out_score + (size_t)i * k_out, &dummy, bsc + nb, cs, cp);
        }
        free(bsc); free(cs); free(cp);
    }
    return bad ? -2 : 0;
}

/* Block scores only (for checks against the reference's eager block router,
 * src/relation_lm/routing/block_router.py:70-101, which subtracts log(heads)). */
int orc_block_scores(int max_t, int nb, int buckets, int t, const float* mean, const float* std,
                     const float* rq, const float* gamma, const float* bias, int local,
                     int strict, float* out) {
    if (nb <= 0 || max_t % nb != 0) return -1;
    block_scores(mean, std, rq, gamma, bias, nb, max_t / nb, buckets, t, local, strict, out);
    return 0;
}

/* ---------------------------------------------------------------- value rounding for cache stores */

static inline float round_bf16(float x) {
    if (x != x) return x;
    uint32_t b;
    memcpy(&b, &x, 4);
    b += 0x7fffu + ((b >> 16) & 1u);
    b &= 0xffff0000u;
    memcpy(&x, &b, 4);
    return x;
}

/* dtype codes: 0 fp32, 1 bf16, 2 fp16 */
static inline float round_store(float x, int dtype) {
    if (dtype == 1) return round_bf16(x);
    if (dtype == 2) return (float)(_Float16)x;
    return x;
}

/*
 * router_cache_update (router_cache.py:33-172) for one position shared by the
 * batch.  Caches are [B, T, 64], stats [B, NB, 64], conv weights [64, 3],
 * raw inputs [B, *] with a row stride.  Stores are rounded to cache_dtype /
 * stats_dtype as a GPU store into a bf16/fp16 tensor would be; statistics use
 * the un-rounded fresh row at `t` (router_cache.py:144-146).
 * Canonical order: sum and squared-deviation sum run over rows 0..BS-1 in
 * ascending order; mean = sum / BS; var = fmaf-chain of (x-mean)^2 / BS.
 */
int orc_router_cache_update(int batch, int max_t, int nb, int bs, int t,
                            const float* araw, int64_t araw_stride, const float* praw,
                            int64_t praw_stride, float* araw_cache, float* praw_cache,
                            float* aconv_cache, float* pconv_cache, float* amean, float* astd,
                            float* pmean, float* pstd, const float* aw, const float* pw,
                            int cache_dtype, int stats_dtype, float* out) {
    if (t < 0 || t >= max_t || bs < 1 || t / bs >= nb || (t / bs + 1) * bs > max_t) return -1;
    int p1 = t - 1 > 0 ? t - 1 : 0, p2 = t - 2 > 0 ? t - 2 : 0;
    float v1 = t >= 1 ? 1.0f : 0.0f, v2 = t >= 2 ? 1.0f : 0.0f;
    int blk = t / bs, start = blk * bs;
    for (int b = 0; b < batch; ++b) {
        for (int s = 0; s < 2; ++s) {
            const float* raw = s == 0 ? araw + b * araw_stride : praw + b * praw_stride;
            float* rc = (s == 0 ? araw_cache : praw_cache) + (size_t)b * max_t * ORC_D;
            float* cc = (s == 0 ? aconv_cache : pconv_cache) + (size_t)b * max_t * ORC_D;
            float* mo = (s == 0 ? amean : pmean) + ((size_t)b * nb + blk) * ORC_D;
            float* so = (s == 0 ? astd : pstd) + ((size_t)b * nb + blk) * ORC_D;
            const float* w = s == 0 ? aw : pw;
            for (int c = 0; c < ORC_D; ++c) {
                float conv = raw[c] * w[c * 3 + 2];
                conv = conv + (rc[(size_t)p1 * ORC_D + c] * w[c * 3 + 1]) * v1;
                conv = conv + (rc[(size_t)p2 * ORC_D + c] * w[c * 3 + 0]) * v2;
                float sum = 0.0f;
                for (int r = 0; r < bs; ++r) {
                    float x = (start + r == t) ? conv : cc[(size_t)(start + r) * ORC_D + c];
                    sum = sum + x;
                }
                float mean = sum / (float)bs;
                float acc = 0.0f;
                for (int r = 0; r < bs; ++r) {
                    float x = (start + r == t) ? conv : cc[(size_t)(start + r) * ORC_D + c];
                    float d = x - mean;
                    acc = fmaf(d, d, acc);
                }
                float sd = sqrtf(acc / (float)bs);
                rc[(size_t)t * ORC_D + c] = round_store(raw[c], cache_dtype);
                cc[(size_t)t * ORC_D + c] = round_store(conv, cache_dtype);
                mo[c] = round_store(mean, stats_dtype);
                so[c] = round_store(sd, stats_dtype);
                out[((size_t)b * 2 + s) * ORC_D + c] = conv;
            }
        }
    }
    return 0;
}

/* ---------------------------------------------------------------- relation tail */

static inline double gelu_erf(double x) { return 0.5 * x * (1.0 + erf(x * 0.70710678118654752440)); }

/*
 * relation_hidden_cached / relation_hidden_cache_update
 * (relation_reduce.py:72-146, 186-309).  n_rows query rows; row i gathers
 * from sequence row_batch[i].  If update != 0 the expanded row of position
 * row_pos[i] is first computed from operand_cache and stored (rounded to
 * cache_dtype), and fresh fp32 values replace gathered ones wherever an index
 * equals that position.  Indices outside [0, T) (the sentinel of an empty
 * partner slot) are clamped into range: their result is masked downstream.
 * Accumulation is in double; the comparison with a GPU kernel is by tolerance.
 */
int orc_relation_hidden(int n_rows, int n_seq, int max_t, int rdim, int hdim, int k_out,
                        const int32_t* row_batch, const int32_t* row_pos, float* expanded,
                        const float* operand, const int32_t* anchor_idx,
                        const int32_t* partner_idx, const float* w_anchor,
                        const float* w_partner, const float* w_product, const float* bias,
                        int update, int cache_dtype, float* out) {
    int bad = 0;
    for (int i = 0; i < n_rows; ++i) {
        int b = row_batch[i];
        int t = update ? row_pos[i] : -1;
        if (b < 0 || b >= n_seq || (update && (t < 0 || t >= max_t))) { bad = 1; continue; }
        float* ex = expanded + (size_t)b * max_t * 2 * hdim;
        const float* op = operand + (size_t)b * max_t * rdim;
        float* fresh = NULL;
        if (update) {
            fresh = (float*)malloc(sizeof(float) * 2 * (size_t)hdim);
            const float* o = op + (size_t)t * rdim;
#pragma omp parallel for schedule(static)
            for (int h = 0; h < hdim; ++h) {
                double a = 0.0, p = 0.0;
                for (int r = 0; r < rdim; ++r) {
                    a += (double)w_anchor[(size_t)h * rdim + r] * o[r];
                    p += (double)w_partner[(size_t)h * rdim + r] * o[r];
                }
                fresh[h] = (float)(a + bias[h]);
                fresh[hdim + h] = (float)p;
            }
            for (int h = 0; h < 2 * hdim; ++h) ex[(size_t)t * 2 * hdim + h] = round_store(fresh[h], cache_dtype);
        }
        int a = anchor_idx[i];
        if (a < 0) a = 0;
        if (a >= max_t) a = max_t - 1;
#pragma omp parallel for schedule(static) collapse(2)
        for (int k = 0; k < k_out; ++k) {
            for (int h = 0; h < hdim; ++h) {
                int p = partner_idx[(size_t)i * k_out + k];
                if (p < 0) p = 0;
                if (p >= max_t) p = max_t - 1;
                double acc = 0.0;
                for (int r = 0; r < rdim; ++r)
                    acc += (double)(op[(size_t)p * rdim + r] * op[(size_t)a * rdim + r]) *
                           w_product[(size_t)h * rdim + r];
                double ab = (update && a == t) ? fresh[h] : ex[(size_t)a * 2 * hdim + h];
                double pb = (update && p == t) ? fresh[hdim + h] : ex[(size_t)p * 2 * hdim + hdim + h];
                out[((size_t)i * k_out + k) * hdim + h] = (float)gelu_erf(acc + (ab + pb));
            }
        }
        free(fresh);
    }
    return bad ? -2 : 0;
}

/*
 * relation_norm_reduce (relation_reduce.py:360-417): LayerNorm of each of the
 * K partner rows (biased variance), weights = softmax over active slots,
 * active = k < clamp(ceil(log2(t+2)), 1, K) and score > -1e30, sum.
 */
int orc_relation_norm_reduce(int n_rows, int k_out, int dim, const int32_t* row_pos,
                             const float* raw, const float* scores, const float* gamma,
                             const float* beta, float eps, float* out) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < n_rows; ++i) {
        int t = row_pos[i];
        int k_limit = 32 - __builtin_clz((unsigned)(t + 1)); /* ceil(log2(t + 2)) for t >= 0 */
        if (k_limit < 1) k_limit = 1;
        if (k_limit > k_out) k_limit = k_out;
        double wk[64];
        double mx = -1.0e4;
        int any = 0;
        for (int k = 0; k < k_out; ++k) {
            float s = scores[(size_t)i * k_out + k];
            int active = k < k_limit && s > -1.0e30f;
            wk[k] = active ? (double)s : -1.0e4;
            if (!any || wk[k] > mx) mx = wk[k];
            any = 1;
        }
        double den = 0.0;
        for (int k = 0; k < k_out; ++k) {
            float s = scores[(size_t)i * k_out + k];
            int active = k < k_limit && s > -1.0e30f;
            wk[k] = active ? exp(wk[k] - mx) : 0.0;
            den += wk[k];
        }
        if (den < 1.0e-9) den = 1.0e-9;
        for (int c = 0; c < dim; ++c) out[(size_t)i * dim + c] = 0.0f;
        double* accum = (double*)calloc((size_t)dim, sizeof(double));
        for (int k = 0; k < k_out; ++k) {
            const float* x = raw + ((size_t)i * k_out + k) * dim;
            double mean = 0.0, var = 0.0;
            for (int c = 0; c < dim; ++c) mean += x[c];
            mean /= dim;
            for (int c = 0; c < dim; ++c) var += (x[c] - mean) * (x[c] - mean);
            var /= dim;
            double inv = 1.0 / sqrt(var + (double)eps);
            double w = wk[k] / den;
            for (int c = 0; c < dim; ++c) accum[c] += w * ((x[c] - mean) * inv * gamma[c] + beta[c]);
        }
        for (int c = 0; c < dim; ++c) out[(size_t)i * dim + c] = (float)accum[c];
        free(accum);
    }
    return 0;
}

/* Packed projection: out[rows, n_out] = x[rows, d] . w[n_out, d]^T (packed_cache.py:56). */
int orc_linear(int rows, int d, int n_out, const float* x, const float* w, float* out) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int i = 0; i < rows; ++i)
        for (int o = 0; o < n_out; ++o) {
            double acc = 0.0;
            for (int c = 0; c < d; ++c) acc += (double)x[(size_t)i * d + c] * w[(size_t)o * d + c];
            out[(size_t)i * n_out + o] = (float)acc;
        }
    return 0;
}
