/*
 * Plain-C restatement of the reference's GGUF Q4_0 / Q4_K / Q8_0 / Q5_0 block decode and
 * of the mat-vec built on it.  TEST INFRASTRUCTURE: used only by tests/, the smoke check
 * and the CPU-baseline legs of bench.py (see oracle/__init__.py).
 *
 * q4_0: adam/loaders/gguf.py:290-299 (GGUFLoader._dq4_0)
 * q4_k: adam/loaders/gguf.py:312-337 (GGUFLoader._dq4k), scale unpack :325-328
 * q8_0: adam/loaders/gguf.py:282-288 (GGUFLoader._dq8)
 * q5_0: adam/loaders/gguf.py:301-310 (GGUFLoader._dq5_0)
 * gemv: y = W x with W decoded to float32 first and a float32 dot product per row,
 *       as the reference's numpy decoder does after pre-decoding the weights
 *       (tests/diagnostics/diag_inference.py:966-969, :985-987).
 *
 * Every product and difference is rounded to float32 separately (no fused
 * multiply-add: compiled with -ffp-contract=off), so results are bit-identical
 * to the numpy restatement in oracle/q4_blocks.py.
 *
 * Rows / blocks are split over POSIX threads (one per online CPU, or
 * Q4REF_THREADS); the split does not change any result.
 *
 * Build: make -C oracle   (gcc -O2 -pthread -ffp-contract=off -shared -fPIC)
 */
#define _GNU_SOURCE
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <stddef.h>
#include <unistd.h>

typedef void (*range_fn)(int64_t lo, int64_t hi, void* ctx);
typedef struct { range_fn fn; void* ctx; int64_t lo, hi; } job_t;
static void* job_main(void* p) { job_t* j = (job_t*)p; j->fn(j->lo, j->hi, j->ctx); return NULL; }

int q4ref_threads(void) {
    const char* e = getenv("Q4REF_THREADS");
    long n = e ? atol(e) : sysconf(_SC_NPROCESSORS_ONLN);
    if (n < 1) n = 1;
    if (n > 256) n = 256;
    return (int)n;
}

static void parallel_for(int64_t n, range_fn fn, void* ctx) {
    int t = q4ref_threads();
    if (n < 2 * t || t == 1) { fn(0, n, ctx); return; }
    pthread_t th[256];
    job_t jobs[256];
    const int64_t step = (n + t - 1) / t;
    int used = 0;
    for (int i = 0; i < t; ++i) {
        const int64_t lo = i * step, hi = lo + step < n ? lo + step : n;
        if (lo >= hi) break;
        jobs[used] = (job_t){fn, ctx, lo, hi};
        if (pthread_create(&th[used], NULL, job_main, &jobs[used]) != 0) { fn(lo, hi, ctx); continue; }
        ++used;
    }
    for (int i = 0; i < used; ++i) pthread_join(th[i], NULL);
}

static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {                                  /* subnormal: renormalise */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static void dq4_0_block(const uint8_t* b, float* out) {
    uint16_t h;
    memcpy(&h, b, 2);
    const float d = half_to_float(h);
    for (int j = 0; j < 16; ++j) {
        out[j]      = ((float)(b[2 + j] & 0x0F) - 8.0f) * d;
        out[j + 16] = ((float)(b[2 + j] >> 4) - 8.0f) * d;
    }
}

static void dq4_k_block(const uint8_t* b, float* out) {
    uint16_t h0, h1;
    memcpy(&h0, b, 2);
    memcpy(&h1, b + 2, 2);
    const float d = half_to_float(h0), dm = half_to_float(h1);
    const uint8_t* rs = b + 4;
    const uint8_t* qs = b + 16;
    float sc[8], mn[8];
    for (int j = 0; j < 8; ++j) {
        int s2, m2;
        if (j < 4) { s2 = rs[j] & 0x3F; m2 = rs[j + 4] & 0x3F; }
        else { s2 = (rs[j + 4] & 0x0F) | ((rs[j - 4] >> 6) << 4); m2 = (rs[j + 4] >> 4) | ((rs[j] >> 6) << 4); }
        sc[j] = d * (float)s2;
        mn[j] = dm * (float)m2;
    }
    for (int g = 0; g < 4; ++g) {
        const uint8_t* q = qs + g * 32;
        float* o = out + g * 64;
        for (int j = 0; j < 32; ++j) {
            const float a = (float)(q[j] & 0x0F) * sc[2 * g];
            const float c = (float)(q[j] >> 4) * sc[2 * g + 1];
            o[j] = a - mn[2 * g];
            o[j + 32] = c - mn[2 * g + 1];
        }
    }
}

/* GGUFLoader._dq8 (adam/loaders/gguf.py:282-288): fp16 d, 32 int8 codes; value = q * d. */
static void dq8_0_block(const uint8_t* b, float* out) {
    uint16_t h;
    memcpy(&h, b, 2);
    const float d = half_to_float(h);
    for (int j = 0; j < 32; ++j) out[j] = (float)(int8_t)b[2 + j] * d;
}

/* GGUFLoader._dq5_0 (adam/loaders/gguf.py:301-310): fp16 d, uint32 qh, 16 nibble bytes;
 * code j = nibble | bit j of qh << 4; value = d * (code - 16). */
static void dq5_0_block(const uint8_t* b, float* out) {
    uint16_t h;
    uint32_t qh;
    memcpy(&h, b, 2);
    memcpy(&qh, b + 2, 4);
    const float d = half_to_float(h);
    for (int j = 0; j < 32; ++j) {
        const int lo = j < 16 ? (b[6 + j] & 0x0F) : (b[6 + j - 16] >> 4);
        const int hi = (int)((qh >> j) & 1u);
        out[j] = d * (float)((lo | (hi << 4)) - 16);
    }
}

/* Block geometry and decoder of a ggml type: 2 Q4_0, 12 Q4_K, 8 Q8_0, 6 Q5_0. */
typedef void (*block_fn)(const uint8_t*, float*);
static int block_kind(int type, int64_t* elems, int64_t* bytes, block_fn* fn) {
    switch (type) {
    case 2:  *elems = 32;  *bytes = 18;  *fn = dq4_0_block; return 0;
    case 12: *elems = 256; *bytes = 144; *fn = dq4_k_block; return 0;
    case 8:  *elems = 32;  *bytes = 34;  *fn = dq8_0_block; return 0;
    case 6:  *elems = 32;  *bytes = 22;  *fn = dq5_0_block; return 0;
    default: return -1;
    }
}

typedef struct { const uint8_t* raw; int64_t be, bb; block_fn fn; float* out; } deq_ctx;
static void deq_range(int64_t lo, int64_t hi, void* p) {
    deq_ctx* c = (deq_ctx*)p;
    for (int64_t i = lo; i < hi; ++i) c->fn(c->raw + i * c->bb, c->out + i * c->be);
}

/* Decode n_blocks blocks of a supported ggml type to float32. */
int q4_dequant(const uint8_t* raw, int ggml_type, int64_t n_blocks, float* out) {
    deq_ctx c = {raw, 0, 0, NULL, out};
    if (block_kind(ggml_type, &c.be, &c.bb, &c.fn)) return -1;
    parallel_for(n_blocks, deq_range, &c);
    return 0;
}

typedef struct { const uint8_t* raw; int64_t be, bb; block_fn fn; int64_t N, K, B; const float* x; float* y; double* y64; } gemv_ctx;
static void gemv_range(int64_t lo, int64_t hi, void* p) {
    gemv_ctx* c = (gemv_ctx*)p;
    const int64_t be = c->be, nb = c->K / be;
    for (int64_t n = lo; n < hi; ++n) {
        float acc[64];
        float w[256];
        for (int64_t b = 0; b < c->B; ++b) acc[b] = 0.0f;
        for (int64_t i = 0; i < nb; ++i) {
            c->fn(c->raw + (n * nb + i) * c->bb, w);
            for (int64_t b = 0; b < c->B; ++b) {
                const float* xb = c->x + b * c->K + i * be;
                float s = acc[b];
                for (int64_t k = 0; k < be; ++k) s += w[k] * xb[k];
                acc[b] = s;
            }
        }
        for (int64_t b = 0; b < c->B; ++b) c->y[b * c->N + n] = acc[b];
    }
}

/* The same product with every term and the sum in double: a reference whose own rounding
 * error is negligible beside the 1e-3 tolerance, for long rows (K of tens of thousands). */
static void gemv64_range(int64_t lo, int64_t hi, void* p) {
    gemv_ctx* c = (gemv_ctx*)p;
    const int64_t be = c->be, nb = c->K / be;
    for (int64_t n = lo; n < hi; ++n) {
        double acc[64];
        float w[256];
        for (int64_t b = 0; b < c->B; ++b) acc[b] = 0.0;
        for (int64_t i = 0; i < nb; ++i) {
            c->fn(c->raw + (n * nb + i) * c->bb, w);
            for (int64_t b = 0; b < c->B; ++b) {
                const float* xb = c->x + b * c->K + i * be;
                double s = acc[b];
                for (int64_t k = 0; k < be; ++k) s += (double)w[k] * (double)xb[k];
                acc[b] = s;
            }
        }
        for (int64_t b = 0; b < c->B; ++b) c->y64[b * c->N + n] = acc[b];
    }
}
int q4_gemv_f64(const uint8_t* raw, int ggml_type, int64_t N, int64_t K, const float* x, int64_t B, double* y) {
    gemv_ctx c = {raw, 0, 0, NULL, N, K, B, x, NULL, y};
    if (block_kind(ggml_type, &c.be, &c.bb, &c.fn) || K % c.be || B < 1 || B > 64) return -1;
    parallel_for(N, gemv64_range, &c);
    return 0;
}

/* y[b][n] = sum_k W[n][k] x[b][k], rows decoded on the fly, float32 accumulation in
 * index order.  x is [B][K], y is [B][N], B <= 64. */
int q4_gemv(const uint8_t* raw, int ggml_type, int64_t N, int64_t K, const float* x, int64_t B, float* y) {
    gemv_ctx c = {raw, 0, 0, NULL, N, K, B, x, y, NULL};
    if (block_kind(ggml_type, &c.be, &c.bb, &c.fn) || K % c.be || B < 1 || B > 64) return -1;
    parallel_for(N, gemv_range, &c);
    return 0;
}
