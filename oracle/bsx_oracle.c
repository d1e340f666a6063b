/*
 * CPU oracle for the event-driven synaptic propagation path (plain C + OpenMP).
 *
 * TEST INFRASTRUCTURE ONLY: linked by the tests, the smoke check and the
 * CPU-baseline / reference legs of the benchmark; never by the product.
 *
 * What each function restates (paths are relative to the reference project):
 *  - orc_fixed_num_indices: brainstate/nn/_event_fixedprob.py:165-171, i.e.
 *    numpy.random.RandomState(seed).randint(0, n_post, size=(n_pre, K)) cast to
 *    int32.  NumPy's legacy generator is MT19937 (init_genrand seeding); bounded
 *    integers with a range below 2^32 take one 32-bit draw, mask it with the
 *    smallest all-ones mask covering n_post-1 and reject values above n_post-1.
 *    Checked element for element against NumPy in tests/test_oracle.py.
 *  - orc_random_sample: RandomState.random_sample (two 32-bit draws -> 53-bit
 *    double), the stream behind the afferent_ratio row mask
 *    (_event_fixedprob.py:184).
 *  - orc_event_vecmat / orc_float_vecmat: the scatter-add oracle the reference
 *    test recomputes (_event_fixedprob_test.py:254-259): y[idx[i,k]] += a[i]*w[i,k],
 *    duplicates accumulate, float32, sequential in (i,k).
 *  - orc_float_matvec / orc_event_matvec: y[i] = sum_k w[i,k]*v[idx[i,k]] — the
 *    transposed product pinned by _event_fixedprob_test.py:56-88.
 *  - orc_vecmat_dw: the weight cotangent of the same test.
 *
 * The arithmetic of the reference itself lives in the un-vendored dependency
 * brainevent (pyproject.toml:60, ">=0.0.7", no exact pin) and cannot be built
 * here; parity is anchored on the in-test oracles cited above.
 *
 * Batched entry points parallelise over the batch with OpenMP (each batch row
 * owns its output row, so the per-row accumulation order stays sequential).
 */
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- MT19937 */
#define MT_N 624
#define MT_M 397

typedef struct {
    uint32_t key[MT_N];
    int pos;
} orc_mt_t;

void orc_mt_seed(orc_mt_t* st, uint32_t seed) {
    st->key[0] = seed;
    for (int i = 1; i < MT_N; ++i)
        st->key[i] = 1812433253u * (st->key[i - 1] ^ (st->key[i - 1] >> 30)) + (uint32_t)i;
    st->pos = MT_N;
}

static void mt_refill(orc_mt_t* st) {
    uint32_t* k = st->key;
    int i;
    for (i = 0; i < MT_N - MT_M; ++i) {
        uint32_t y = (k[i] & 0x80000000u) | (k[i + 1] & 0x7fffffffu);
        k[i] = k[i + MT_M] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    }
    for (; i < MT_N - 1; ++i) {
        uint32_t y = (k[i] & 0x80000000u) | (k[i + 1] & 0x7fffffffu);
        k[i] = k[i + (MT_M - MT_N)] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    }
    uint32_t y = (k[MT_N - 1] & 0x80000000u) | (k[0] & 0x7fffffffu);
    k[MT_N - 1] = k[MT_M - 1] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    st->pos = 0;
}

static inline uint32_t mt_next(orc_mt_t* st) {
    if (st->pos == MT_N) mt_refill(st);
    uint32_t y = st->key[st->pos++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9d2c5680u;
    y ^= (y << 15) & 0xefc60000u;
    y ^= y >> 18;
    return y;
}

size_t orc_mt_state_bytes(void) { return sizeof(orc_mt_t); }

/* Draw count integers in [0, n_post) continuing the stream in st. */
void orc_randint_fill(orc_mt_t* st, int64_t n_post, int64_t count, int32_t* out) {
    uint32_t rng = (uint32_t)(n_post - 1);
    if (rng == 0) {               /* NumPy draws nothing for a one-value range */
        memset(out, 0, (size_t)count * sizeof(int32_t));
        return;
    }
    uint32_t mask = rng;
    mask |= mask >> 1; mask |= mask >> 2; mask |= mask >> 4; mask |= mask >> 8; mask |= mask >> 16;
    for (int64_t i = 0; i < count; ++i) {
        uint32_t v;
        do { v = mt_next(st) & mask; } while (v > rng);
        out[i] = (int32_t)v;
    }
}

void orc_fixed_num_indices(uint32_t seed, int64_t n_pre, int64_t n_post, int64_t K, int32_t* out) {
    orc_mt_t st;
    orc_mt_seed(&st, seed);
    orc_randint_fill(&st, n_post, n_pre * K, out);
}

void orc_random_sample(orc_mt_t* st, int64_t count, double* out) {
    for (int64_t i = 0; i < count; ++i) {
        uint32_t a = mt_next(st) >> 5, b = mt_next(st) >> 6;
        out[i] = (a * 67108864.0 + b) / 9007199254740992.0;
    }
}

/* --------------------------------------------------------------- products */
static inline void row_range(const int64_t* indptr, int64_t K, int64_t i, int64_t* s, int64_t* e) {
    if (indptr) { *s = indptr[i]; *e = indptr[i + 1]; }
    else { *s = i * K; *e = *s + K; }
}

/* y[b, idx[i,k]] += a[b,i] * w[i,k]; a = x (event == 0) or [x != 0] (event != 0).
 * x is float32 (batch, n_pre); spikes given as uint8 use orc_event_vecmat_u8. */
void orc_float_vecmat(const float* x, int64_t batch, int64_t n_pre, int64_t n_post, int64_t K,
                      const int64_t* indptr, const int32_t* idx, const float* w, int hetero,
                      int event, float* y) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t b = 0; b < batch; ++b) {
        float* yb = y + b * n_post;
        memset(yb, 0, (size_t)n_post * sizeof(float));
        const float* xb = x + b * n_pre;
        for (int64_t i = 0; i < n_pre; ++i) {
            float a = xb[i];
            if (a == 0.0f) continue;
            if (event) a = 1.0f;
            int64_t s, e;
            row_range(indptr, K, i, &s, &e);
            if (hetero) for (int64_t p = s; p < e; ++p) yb[idx[p]] += a * w[p];
            else { float v = a * w[0]; for (int64_t p = s; p < e; ++p) yb[idx[p]] += v; }
        }
    }
}

void orc_event_vecmat_u8(const uint8_t* spk, int64_t batch, int64_t n_pre, int64_t n_post, int64_t K,
                         const int64_t* indptr, const int32_t* idx, const float* w, int hetero,
                         float* y) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t b = 0; b < batch; ++b) {
        float* yb = y + b * n_post;
        memset(yb, 0, (size_t)n_post * sizeof(float));
        const uint8_t* sb = spk + b * n_pre;
        for (int64_t i = 0; i < n_pre; ++i) {
            if (!sb[i]) continue;
            int64_t s, e;
            row_range(indptr, K, i, &s, &e);
            if (hetero) for (int64_t p = s; p < e; ++p) yb[idx[p]] += w[p];
            else { float v = w[0]; for (int64_t p = s; p < e; ++p) yb[idx[p]] += v; }
        }
    }
}

/* The same product for timing on many cores with FEWER vectors than threads: the active
 * rows of one vector are split over the threads, every thread adding into a private copy of
 * the output that is then summed column-wise in thread order, so that all cores work on a
 * single vector too.  The sums differ from the sequential (row, k) order within float32
 * rounding, so parity tests use orc_event_vecmat_u8. */
void orc_event_vecmat_u8_par(const uint8_t* spk, int64_t batch, int64_t n_pre, int64_t n_post, int64_t K,
                             const int64_t* indptr, const int32_t* idx, const float* w, int hetero,
                             float* y) {
    int nt = 1;
#ifdef _OPENMP
    nt = omp_get_max_threads();
#endif
    if (batch >= nt || nt == 1) {
        orc_event_vecmat_u8(spk, batch, n_pre, n_post, K, indptr, idx, w, hetero, y);
        return;
    }
    float* priv = (float*)malloc((size_t)nt * (size_t)n_post * sizeof(float));
    int32_t* act = (int32_t*)malloc((size_t)(n_pre > 0 ? n_pre : 1) * sizeof(int32_t));
    for (int64_t b = 0; b < batch; ++b) {
        const uint8_t* sb = spk + b * n_pre;
        float* yb = y + b * n_post;
        int64_t na = 0;
        for (int64_t i = 0; i < n_pre; ++i) if (sb[i]) act[na++] = (int32_t)i;
#pragma omp parallel num_threads(nt)
        {
            int t = 0;
#ifdef _OPENMP
            t = omp_get_thread_num();
#endif
            float* mine = priv + (size_t)t * n_post;
            memset(mine, 0, (size_t)n_post * sizeof(float));
#pragma omp for schedule(static)
            for (int64_t q = 0; q < na; ++q) {
                int64_t s, e;
                row_range(indptr, K, act[q], &s, &e);
                if (hetero) for (int64_t p = s; p < e; ++p) mine[idx[p]] += w[p];
                else { float v = w[0]; for (int64_t p = s; p < e; ++p) mine[idx[p]] += v; }
            }
#pragma omp for schedule(static)
            for (int64_t j = 0; j < n_post; ++j) {
                float acc = 0.0f;
                for (int u = 0; u < nt; ++u) acc += priv[(size_t)u * n_post + j];
                yb[j] = acc;
            }
        }
    }
    free(priv);
    free(act);
}

/* Transposed (column-major) copy of a connectivity by counting sort: for every column j
 * the rows that target it in ascending (row, k) order; t_perm[p] = position of the entry in
 * the original arrays.  One-time, like the device's transposed copy; W @ spike is then the
 * event-driven scatter orc_event_vecmat_u8 over (t_indptr, t_rows, w[t_perm]). */
void orc_transpose(int64_t n_pre, int64_t n_post, int64_t K, const int64_t* indptr, const int32_t* idx,
                   int64_t* t_indptr, int32_t* t_rows, int64_t* t_perm) {
    int64_t nnz = indptr ? indptr[n_pre] : n_pre * K;
    memset(t_indptr, 0, (size_t)(n_post + 1) * sizeof(int64_t));
    for (int64_t p = 0; p < nnz; ++p) t_indptr[idx[p] + 1]++;
    for (int64_t j = 0; j < n_post; ++j) t_indptr[j + 1] += t_indptr[j];
    int64_t* fill = (int64_t*)malloc((size_t)(n_post > 0 ? n_post : 1) * sizeof(int64_t));
    memcpy(fill, t_indptr, (size_t)n_post * sizeof(int64_t));
    for (int64_t i = 0; i < n_pre; ++i) {
        int64_t s, e;
        row_range(indptr, K, i, &s, &e);
        for (int64_t p = s; p < e; ++p) {
            int64_t q = fill[idx[p]]++;
            t_rows[q] = (int32_t)i;
            t_perm[q] = p;
        }
    }
    free(fill);
}

/* y[b,i] = sum_k w[i,k] * a[b, idx[i,k]];  a = v or [v != 0]. */
void orc_float_matvec(const float* v, int64_t batch, int64_t n_pre, int64_t n_post, int64_t K,
                      const int64_t* indptr, const int32_t* idx, const float* w, int hetero,
                      int event, float* y) {
    for (int64_t b = 0; b < batch; ++b) {
        const float* vb = v + b * n_post;
        float* yb = y + b * n_pre;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n_pre; ++i) {
            int64_t s, e;
            row_range(indptr, K, i, &s, &e);
            float acc = 0.0f;
            for (int64_t p = s; p < e; ++p) {
                float a = vb[idx[p]];
                if (event) a = (a != 0.0f) ? 1.0f : 0.0f;
                acc += a * (hetero ? w[p] : w[0]);
            }
            yb[i] = acc;
        }
    }
}

void orc_event_matvec_u8(const uint8_t* spk, int64_t batch, int64_t n_pre, int64_t n_post, int64_t K,
                         const int64_t* indptr, const int32_t* idx, const float* w, int hetero,
                         float* y) {
    for (int64_t b = 0; b < batch; ++b) {
        const uint8_t* sb = spk + b * n_post;
        float* yb = y + b * n_pre;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n_pre; ++i) {
            int64_t s, e;
            row_range(indptr, K, i, &s, &e);
            float acc = 0.0f;
            for (int64_t p = s; p < e; ++p)
                if (sb[idx[p]]) acc += hetero ? w[p] : w[0];
            yb[i] = acc;
        }
    }
}

/* heterogeneous weight cotangent: dw[p] = sum_b a[b,row(p)] * ct[b, idx[p]] */
void orc_vecmat_dw(const float* x, const float* ct, int64_t batch, int64_t n_pre, int64_t n_post,
                   int64_t K, const int64_t* indptr, const int32_t* idx, int event, float* dw) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n_pre; ++i) {
        int64_t s, e;
        row_range(indptr, K, i, &s, &e);
        for (int64_t p = s; p < e; ++p) dw[p] = 0.0f;
        for (int64_t b = 0; b < batch; ++b) {
            float a = x[b * n_pre + i];
            if (a == 0.0f) continue;
            if (event) a = 1.0f;
            const float* cb = ct + b * n_post;
            for (int64_t p = s; p < e; ++p) dw[p] += a * cb[idx[p]];
        }
    }
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; a caller that wants all the
 * host cores sets the count explicitly. */
void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
