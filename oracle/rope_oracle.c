/*
 * CPU oracle for the side-aware elementwise path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic that the reference project
 * (ademeure/l2_torch_alloc) defines for its elementwise hot path, so that the
 * CUDA kernels can be checked bit for bit on a machine without the reference.
 * It is never linked into, loaded by, or called from the shipped library; only
 * the test-suite, the smoke check and the CPU-baseline leg of the benchmark
 * may use it.
 *
 * Parity status: PINNED.  The functions below are checked against the
 * reference's own CPU code (example_llmc_rope.cu compiled in place into
 * oracle/_ref/) and against the golden vectors under tests/golden/ that were
 * produced by that compiled reference.
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared rope_oracle.c -o liboracle.so -lm -lpthread
 * (-ffp-contract=off matters: the reference's host code is built without FMA
 * contraction, and the CUDA kernels use explicit round-to-nearest mul/add/sub.)
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifndef M_PI
#define M_PI 3.14159265358979323846
#endif

/* ------------------------------------------------------------------------- */
/* cos/sin table.  Follows example_llmc_rope.cu:19-52 (precompute_freqs_cis):
 * freq_i = 1 / theta^(2i/dim) in fp32, optional llama-3 wavelength rescale
 * (scale 8, low/high factors 1/4, original context 8192), then
 * table[t][i] = (cosf(t*freq_i), sinf(t*freq_i)) laid out [end, dim/2, 2]. */
void oracle_precompute_freqs_cis(float *table, int dim, int end, float theta, int use_scaled)
{
    const int half = dim / 2;
    for (int i = 0; i < half; i++) {
        float freq = 1.0f / powf(theta, (float)(2 * i) / dim);
        if (use_scaled) {
            const int scale_factor = 8, low_factor = 1, high_factor = 4, old_len = 8192;
            const float low_wavelen = (float)old_len / low_factor;
            const float high_wavelen = (float)old_len / high_factor;
            /* 2.0f * M_PI is evaluated in double and the quotient rounded to float,
             * exactly as the reference's expression does. */
            float wavelen = 2.0f * M_PI / freq;
            if (wavelen < high_wavelen) {
                /* high-frequency band: unchanged */
            } else if (wavelen > low_wavelen) {
                freq /= scale_factor;
            } else {
                float smooth = ((float)old_len / wavelen - low_factor) / (high_factor - low_factor);
                freq = (1.0f - smooth) * freq / scale_factor + smooth * freq;
            }
        }
        for (int t = 0; t < end; t++) {
            float angle = (float)t * freq;
            table[(size_t)t * dim + 2 * i] = cosf(angle);
            table[(size_t)t * dim + 2 * i + 1] = sinf(angle);
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Forward rotation over a packed [B, T, Nq + 2*Nkv, HS] fp32 tensor.
 * Follows example_llmc_rope.cu:54-86 (apply_rotary_emb_forward), which is the
 * Nq == Nkv case: heads [0, Nq+Nkv) are rotated pairwise
 *     (x, y) -> (x*c - y*s, x*s + y*c)
 * with (c, s) = table[t][d], heads [Nq+Nkv, Nq+2*Nkv) are copied.  The
 * grouped-query generalisation only changes how many heads are rotated; the
 * arithmetic per pair depends on (t, d) alone (the GPU kernel the reference
 * compares against, example_llmc_rope.cu:89-121, takes Nq and Nkv the same way). */
void oracle_rope_forward_f32(float *out, const float *inp, const float *table,
                             int B, int T, int Nq, int Nkv, int HS)
{
    const int heads = Nq + 2 * Nkv;
    const int rotated = Nq + Nkv;
    for (int b = 0; b < B; b++) {
        for (int t = 0; t < T; t++) {
            const size_t row = ((size_t)b * T + t) * heads * HS;
            const float *trow = table + (size_t)t * HS;
            for (int h = 0; h < heads; h++) {
                const size_t base = row + (size_t)h * HS;
                if (h >= rotated) {
                    memcpy(out + base, inp + base, sizeof(float) * HS);
                    continue;
                }
                for (int d = 0; d < HS / 2; d++) {
                    float x = inp[base + 2 * d], y = inp[base + 2 * d + 1];
                    float c = trow[2 * d], s = trow[2 * d + 1];
                    out[base + 2 * d] = x * c - y * s;
                    out[base + 2 * d + 1] = x * s + y * c;
                }
            }
        }
    }
}

/* Backward pass (gradient w.r.t. the input).  Follows example_llmc_rope.cu:166-195
 * (apply_rotary_emb_backward): the rotation by the opposite angle,
 *     (gx, gy) -> (gx*c + gy*s, -gx*s + gy*c),
 * ACCUMULATED into dinp (the reference adds to a zero-initialised buffer), V heads copied. */
void oracle_rope_backward_f32(float *dinp, const float *dout, const float *table,
                              int B, int T, int Nq, int Nkv, int HS)
{
    const int heads = Nq + 2 * Nkv;
    const int rotated = Nq + Nkv;
    for (int b = 0; b < B; b++) {
        for (int t = 0; t < T; t++) {
            const size_t row = ((size_t)b * T + t) * heads * HS;
            const float *trow = table + (size_t)t * HS;
            for (int h = 0; h < heads; h++) {
                const size_t base = row + (size_t)h * HS;
                if (h >= rotated) {
                    memcpy(dinp + base, dout + base, sizeof(float) * HS);
                    continue;
                }
                for (int d = 0; d < HS / 2; d++) {
                    float gx = dout[base + 2 * d], gy = dout[base + 2 * d + 1];
                    float c = trow[2 * d], s = trow[2 * d + 1];
                    dinp[base + 2 * d] += gx * c + gy * s;
                    dinp[base + 2 * d + 1] += -gx * s + gy * c;
                }
            }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* bfloat16 storage helpers: widening is exact; narrowing is round-to-nearest-
 * even with NaN kept quiet, the conversion CUDA's cvt.rn.bf16.f32 performs. */
static inline float bf16_to_f32(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16_rne(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

void oracle_bf16_to_f32(float *out, const uint16_t *in, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = bf16_to_f32(in[i]);
}

void oracle_f32_to_bf16(uint16_t *out, const float *in, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = f32_to_bf16_rne(in[i]);
}

/* bf16 storage, fp32 math, one rounding at the end: widen, rotate exactly as
 * oracle_rope_forward_f32 does, narrow.  V heads are passed through untouched. */
void oracle_rope_forward_bf16(uint16_t *out, const uint16_t *inp, const float *table,
                              int B, int T, int Nq, int Nkv, int HS)
{
    const int heads = Nq + 2 * Nkv;
    const int rotated = Nq + Nkv;
    for (int b = 0; b < B; b++) {
        for (int t = 0; t < T; t++) {
            const size_t row = ((size_t)b * T + t) * heads * HS;
            const float *trow = table + (size_t)t * HS;
            for (int h = 0; h < heads; h++) {
                const size_t base = row + (size_t)h * HS;
                if (h >= rotated) {
                    memcpy(out + base, inp + base, sizeof(uint16_t) * HS);
                    continue;
                }
                for (int d = 0; d < HS / 2; d++) {
                    float x = bf16_to_f32(inp[base + 2 * d]);
                    float y = bf16_to_f32(inp[base + 2 * d + 1]);
                    float c = trow[2 * d], s = trow[2 * d + 1];
                    out[base + 2 * d] = f32_to_bf16_rne(x * c - y * s);
                    out[base + 2 * d + 1] = f32_to_bf16_rne(x * s + y * c);
                }
            }
        }
    }
}

/* bf16 storage flavour of the backward pass: widen, rotate by the opposite angle with
 * separate fp32 roundings, narrow once (no accumulation: the result replaces the gradient,
 * as the in-place GPU kernel of the reference does, example_llmc_rope.cu:197-228). */
void oracle_rope_backward_bf16(uint16_t *dinp, const uint16_t *dout, const float *table,
                               int B, int T, int Nq, int Nkv, int HS)
{
    const int heads = Nq + 2 * Nkv;
    const int rotated = Nq + Nkv;
    for (int b = 0; b < B; b++) {
        for (int t = 0; t < T; t++) {
            const size_t row = ((size_t)b * T + t) * heads * HS;
            const float *trow = table + (size_t)t * HS;
            for (int h = 0; h < heads; h++) {
                const size_t base = row + (size_t)h * HS;
                if (h >= rotated) {
                    memcpy(dinp + base, dout + base, sizeof(uint16_t) * HS);
                    continue;
                }
                for (int d = 0; d < HS / 2; d++) {
                    float gx = bf16_to_f32(dout[base + 2 * d]);
                    float gy = bf16_to_f32(dout[base + 2 * d + 1]);
                    float c = trow[2 * d], s = trow[2 * d + 1];
                    dinp[base + 2 * d] = f32_to_bf16_rne(gx * c + gy * s);
                    dinp[base + 2 * d + 1] = f32_to_bf16_rne(-gx * s + gy * c);
                }
            }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* User-functor example of the benchmark set: out = bf16(a * sigmoid(a) * b * scale),
 * fp32 math left to right.  The reference ships no implementation of this
 * functor (its functor contract is sideaware.cu:81-109); this is the plain
 * statement of the formula, checked to 1 bf16 ulp because expf differs
 * between libm and the GPU. */
void oracle_silu_mul_bf16(uint16_t *out, const uint16_t *a, const uint16_t *b, float scale, size_t n)
{
    for (size_t i = 0; i < n; i++) {
        float x = bf16_to_f32(a[i]);
        float y = bf16_to_f32(b[i]);
        float sig = 1.0f / (1.0f + expf(-x));
        out[i] = f32_to_bf16_rne(((x * sig) * y) * scale);
    }
}

/* ------------------------------------------------------------------------- */
/* Host-thread helpers for the timed CPU baseline.  The reference has no CPU
 * memcpy of its own (its check is dst == src, test.py:290-294), so libc memcpy
 * split over threads stands in; RoPE shards the batch dimension, which the
 * reference function treats independently. */
typedef struct {
    void *dst;
    const void *src;
    size_t n;
} copy_job_t;

static void *copy_worker(void *arg)
{
    copy_job_t *j = (copy_job_t *)arg;
    memcpy(j->dst, j->src, j->n);
    return NULL;
}

void oracle_memcpy_mt(void *dst, const void *src, size_t n, int threads)
{
    if (threads <= 1 || n < ((size_t)1 << 20)) {
        memcpy(dst, src, n);
        return;
    }
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    copy_job_t job[256];
    size_t per = (((n + threads - 1) / threads) + 63) & ~(size_t)63;
    int used = 0;
    for (int i = 0; i < threads; i++) {
        size_t off = (size_t)i * per;
        if (off >= n) break;
        job[used].dst = (char *)dst + off;
        job[used].src = (const char *)src + off;
        job[used].n = (n - off < per) ? n - off : per;
        pthread_create(&tid[used], NULL, copy_worker, &job[used]);
        used++;
    }
    for (int i = 0; i < used; i++) pthread_join(tid[i], NULL);
}

typedef struct {
    void *out;
    const void *inp;
    const float *table;
    int B, T, Nq, Nkv, HS, bf16;
} rope_job_t;

static void *rope_worker(void *arg)
{
    rope_job_t *j = (rope_job_t *)arg;
    if (j->bf16)
        oracle_rope_forward_bf16((uint16_t *)j->out, (const uint16_t *)j->inp, j->table, j->B, j->T, j->Nq, j->Nkv, j->HS);
    else
        oracle_rope_forward_f32((float *)j->out, (const float *)j->inp, j->table, j->B, j->T, j->Nq, j->Nkv, j->HS);
    return NULL;
}

/* Splits B*T rows over threads (each row depends on its own t only). */
void oracle_rope_forward_mt(void *out, const void *inp, const float *table,
                            int B, int T, int Nq, int Nkv, int HS, int bf16, int threads)
{
    if (threads < 1) threads = 1;
    if (threads > B) threads = B;
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    rope_job_t job[256];
    const size_t esize = bf16 ? 2 : 4;
    const size_t per_batch = (size_t)T * (Nq + 2 * Nkv) * HS * esize;
    int b0 = 0;
    for (int i = 0; i < threads; i++) {
        int nb = (B - b0) / (threads - i);
        job[i].out = (char *)out + (size_t)b0 * per_batch;
        job[i].inp = (const char *)inp + (size_t)b0 * per_batch;
        job[i].table = table;
        job[i].B = nb; job[i].T = T; job[i].Nq = Nq; job[i].Nkv = Nkv; job[i].HS = HS; job[i].bf16 = bf16;
        pthread_create(&tid[i], NULL, rope_worker, &job[i]);
        b0 += nb;
    }
    for (int i = 0; i < threads; i++) pthread_join(tid[i], NULL);
}
