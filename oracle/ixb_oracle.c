/*
 * CPU oracle for the INT8-X (3,5,8) nested-bitmap weight path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the algorithm of
 * the reference implementation (dfytensor/ixrun) so that the CUDA kernels can
 * be checked against it and so that a CPU baseline can be timed.  Nothing in
 * the shipped package may link, import or call it; only the tests, the smoke
 * check and the benchmark's cpu-baseline / reference arm do.
 *
 * Parity status: PINNED.  Every function here is compared, in the CPU test
 * suite, with fixtures produced by running the reference's own Python code
 * (ixrun.quantize.int8x_quantize, ixrun.triton_kernels.decode_weight_scatter,
 * ixrun.triton_kernels.precompute_block_offsets,
 * ixrun.fused.compute_row_prefixes, ixrun.bitpack.*) on seeded inputs; the
 * script that made the fixtures is tests/golden/make_golden.py.
 *
 * Reference citations are paths inside the reference project.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- bf16 --- */

static inline float bf16_to_f32(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even, the rounding torch uses for float32 -> bfloat16 */
static inline uint16_t f32_to_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u)      /* NaN stays NaN */
        return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

int ixo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* the OpenMP runtime reads OMP_NUM_THREADS once, when the first library that uses it is loaded; a launcher that
 * pins it to 1 for its worker processes is overridden here */
void ixo_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------ quantise --- */

/*
 * Per-tensor int8 quantisation of a bf16 weight.
 * ixrun/quantize.py:64-73 -- scale = max|W|.clamp(min=1e-8) / 127.0 evaluated
 * in the weight's dtype (bf16: each step is computed in float and rounded back
 * to bf16), codes = clamp(round_half_even(float(W) / float(scale)), -127, 127).
 * Returns the bf16 bit pattern of the scale.
 */
uint16_t ixo_quantize_bf16(const uint16_t *w, int64_t n, int8_t *codes)
{
    float mx = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        float a = fabsf(bf16_to_f32(w[i]));
        if (a > mx) mx = a;
    }
    /* clamp(min=1e-8) on a bf16 tensor: the bound is applied in float and the
       result is rounded to bf16 */
    float cl = mx < 1e-8f ? 1e-8f : mx;
    uint16_t cl_b = f32_to_bf16(cl);
    uint16_t sc_b = f32_to_bf16(bf16_to_f32(cl_b) / 127.0f);
    float sc = bf16_to_f32(sc_b);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float q = nearbyintf(bf16_to_f32(w[i]) / sc);   /* FE_TONEAREST: half-even */
        if (q > 127.0f) q = 127.0f;
        if (q < -127.0f) q = -127.0f;
        codes[i] = (int8_t)q;
    }
    return sc_b;
}

/* level of a code: 0 -> |c|<=3, 1 -> |c|<=15, 2 -> rest.
 * ixrun/quantize.py:25-37 with thresholds ixrun/config.py:27-36. */
static inline int level_of(int c)
{
    int a = c < 0 ? -c : c;
    return a <= 3 ? 0 : (a <= 15 ? 1 : 2);
}

void ixo_count_levels(const int8_t *codes, int64_t n, int64_t counts[3])
{
    int64_t c0 = 0, c1 = 0, c2 = 0;
#pragma omp parallel for reduction(+ : c0, c1, c2) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int l = level_of(codes[i]);
        c0 += (l == 0);
        c1 += (l == 1);
        c2 += (l == 2);
    }
    counts[0] = c0; counts[1] = c1; counts[2] = c2;
}

/* number of int32 words of each stream for given counts.
 * ixrun/bitpack.py:44 (total_words = ceil(n*bits/32)); B2 is indexed by the
 * rank among non-L1 elements (ixrun/quantize.py:91-96). */
void ixo_stream_words(int64_t n, const int64_t counts[3], int64_t words[4])
{
    words[0] = (n + 31) / 32;                       /* B1 */
    words[1] = (counts[1] + counts[2] + 31) / 32;   /* B2 */
    words[2] = (counts[0] * 3 + 31) / 32;           /* L1 */
    words[3] = (counts[1] * 5 + 31) / 32;           /* L2 */
}

/* storage accounting, ixrun/quantize.py:98-106 */
int64_t ixo_total_bytes(int64_t n, const int64_t counts[3])
{
    int64_t w[4];
    ixo_stream_words(n, counts, w);
    return 2 + 4 * (w[0] + w[1] + w[2] + w[3]) + counts[2];
}

static inline void put_bits(uint32_t *s, int64_t bitpos, uint32_t v, int bits)
{
    int64_t wi = bitpos >> 5;
    int sh = (int)(bitpos & 31);
    s[wi] |= v << sh;
    if (sh + bits > 32) s[wi + 1] |= v >> (32 - sh);
}

/*
 * Pack int8 codes into the five INT8-X streams (buffers sized with
 * ixo_stream_words / counts[2], zero-filled here).
 * ixrun/quantize.py:80-96 and ixrun/bitpack.py:13-61 -- values are laid
 * LSB-first, consecutively, across little-endian int32 words; L1 stores
 * code+3 in 3 bits, L2 code+15 in 5 bits, L3 code+127 as a raw byte; bit e of
 * B1 says "element e is L1", bit r of B2 says "the r-th non-L1 element is L2".
 */
void ixo_pack(const int8_t *codes, int64_t n,
              uint32_t *b1, uint32_t *b2, uint32_t *l1, uint32_t *l2, uint8_t *l3)
{
    int64_t counts[3], words[4];
    ixo_count_levels(codes, n, counts);
    ixo_stream_words(n, counts, words);
    memset(b1, 0, (size_t)words[0] * 4);
    memset(b2, 0, (size_t)words[1] * 4);
    memset(l1, 0, (size_t)words[2] * 4);
    memset(l2, 0, (size_t)words[3] * 4);
    int64_t a = 0, r = 0, c = 0, t = 0;   /* #L1, #nonL1, #L2, #L3 so far */
    for (int64_t e = 0; e < n; ++e) {
        int v = codes[e];
        int lv = level_of(v);
        if (lv == 0) {
            b1[e >> 5] |= 1u << (e & 31);
            put_bits(l1, a * 3, (uint32_t)(v + 3), 3);
            ++a;
        } else {
            if (lv == 1) {
                b2[r >> 5] |= 1u << (r & 31);
                put_bits(l2, c * 5, (uint32_t)(v + 15), 5);
                ++c;
            } else {
                l3[t++] = (uint8_t)(v + 127);
            }
            ++r;
        }
    }
}

/* -------------------------------------------------------------- decode --- */

static inline uint32_t get_bits(const uint32_t *s, int64_t words, int64_t bitpos, int bits)
{
    int64_t wi = bitpos >> 5;
    int sh = (int)(bitpos & 31);
    uint32_t v = s[wi] >> sh;
    if (sh + bits > 32 && wi + 1 < words) v |= s[wi + 1] << (32 - sh);
    return v & ((1u << bits) - 1u);
}

/*
 * Exclusive global counts of L1 and L2 elements before flat positions
 * u*gran, u = 0..n_units-1.  One routine covers the three tables the reference
 * derives at deploy time:
 *   gran = 1024  -> ixrun/triton_kernels.py:180-220 precompute_block_offsets
 *   gran = in_f  -> ixrun/fused.py:60-65   compute_row_prefixes(chunk=None)
 *   gran = chunk -> ixrun/fused.py:67-78   compute_row_prefixes(chunk=C),
 *                   index n*nsplit+c == flat position / chunk
 */
void ixo_prefixes(const uint32_t *b1, const uint32_t *b2, int64_t n,
                  int64_t gran, int64_t n_units, int32_t *q1, int32_t *q2)
{
    int64_t a = 0, r = 0, c = 0, u = 0;
    for (int64_t e = 0; e <= n && u < n_units; ++e) {
        if (e == u * gran) { q1[u] = (int32_t)a; q2[u] = (int32_t)c; ++u; }
        if (e == n) break;
        if ((b1[e >> 5] >> (e & 31)) & 1u) {
            ++a;
        } else {
            c += (b2[r >> 5] >> (r & 31)) & 1u;
            ++r;
        }
    }
}

/*
 * Sequential-walk decode of elements [e0, e1) given the counts before e0.
 * The three running counters advance exactly like the reference's fused
 * kernel (ixrun/fused.py:100-102, 133-165, 175-177): L1 index = a, B2 index =
 * r = e - a, L2 index = c, L3 index = r - c.
 */
static void decode_range(const uint32_t *b1, const uint32_t *b2,
                         const uint32_t *l1, int64_t l1w,
                         const uint32_t *l2, int64_t l2w, const uint8_t *l3,
                         int64_t e0, int64_t e1, int64_t a, int64_t c, int8_t *out)
{
    int64_t r = e0 - a;
    for (int64_t e = e0; e < e1; ++e) {
        int v;
        if ((b1[e >> 5] >> (e & 31)) & 1u) {
            v = (int)get_bits(l1, l1w, a * 3, 3) - 3;
            ++a;
        } else {
            if ((b2[r >> 5] >> (r & 31)) & 1u) {
                v = (int)get_bits(l2, l2w, c * 5, 5) - 15;
                ++c;
            } else {
                v = (int)l3[r - c] - 127;
            }
            ++r;
        }
        out[e] = (int8_t)v;
    }
}

/*
 * Packed streams -> int8 codes (the inverse of ixo_pack).  Same result as
 * ixrun/triton_kernels.py:36-59 decode_weight_scatter before its final scale
 * multiply.  Parallel over 1024-element blocks after one serial prefix pass.
 */
void ixo_decode_codes(const uint32_t *b1, const uint32_t *b2,
                      const uint32_t *l1, int64_t l1w,
                      const uint32_t *l2, int64_t l2w,
                      const uint8_t *l3, int64_t n, int8_t *out,
                      int32_t *scratch_q1, int32_t *scratch_q2)
{
    const int64_t G = 1024;
    int64_t nb = (n + G - 1) / G;
    ixo_prefixes(b1, b2, n, G, nb, scratch_q1, scratch_q2);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        int64_t e0 = b * G, e1 = e0 + G > n ? n : e0 + G;
        decode_range(b1, b2, l1, l1w, l2, l2w, l3, e0, e1,
                     scratch_q1[b], scratch_q2[b], out);
    }
}

/* codes -> bf16 weight, w = bf16(float(code) * float(scale)).
 * ixrun/triton_kernels.py:59 and :175-176, ixrun/fused.py:170. */
void ixo_codes_to_bf16(const int8_t *codes, int64_t n, uint16_t scale_bf16, uint16_t *out)
{
    float sc = bf16_to_f32(scale_bf16);
    uint16_t lut[256];
    for (int c = -128; c < 128; ++c) lut[(uint8_t)c] = f32_to_bf16((float)c * sc);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = lut[(uint8_t)codes[i]];
}

/* --------------------------------------------------------- gemv / gemm --- */

/*
 * y[m][nrow] = sum_k float(x[m][k]) * float(bf16(code[nrow][k] * scale)).
 * Restates the reference result for every M: M==1 ixrun/fused.py:169-172,179;
 * M>1 ixrun/engine.py:171-173 (decode, then F.linear).  Products of two bf16
 * values are exact in float; the sum is carried in double and rounded to
 * float once, so it is at least as accurate as any fp32 accumulation order.
 */
void ixo_gemm_f32(const int8_t *codes, uint16_t scale_bf16,
                  const uint16_t *x, int64_t m_rows,
                  int64_t out_f, int64_t in_f, float *y)
{
    float sc = bf16_to_f32(scale_bf16);
    float lut[256];
    for (int c = -128; c < 128; ++c)
        lut[(uint8_t)c] = bf16_to_f32(f32_to_bf16((float)c * sc));
#pragma omp parallel for schedule(static)
    for (int64_t nrow = 0; nrow < out_f; ++nrow) {
        const int8_t *wr = codes + nrow * in_f;
        for (int64_t m = 0; m < m_rows; ++m) {
            const uint16_t *xr = x + m * in_f;
            double acc = 0.0;
            for (int64_t k = 0; k < in_f; ++k)
                acc += (double)(bf16_to_f32(xr[k]) * lut[(uint8_t)wr[k]]);
            y[m * out_f + nrow] = (float)acc;
        }
    }
}

/*
 * The reference's CPU path for one layer, end to end: packed streams ->
 * weights -> y = W x (decode_weight_scatter + F.linear,
 * ixrun/triton_kernels.py:36-59, ixrun/engine.py:171-173).  The decoded bf16
 * weight is materialised in `w_scratch` (out_f*in_f) like the reference does,
 * then multiplied.  Used as the timed CPU baseline.
 */
void ixo_layer_cpu(const uint32_t *b1, const uint32_t *b2,
                   const uint32_t *l1, int64_t l1w,
                   const uint32_t *l2, int64_t l2w, const uint8_t *l3,
                   uint16_t scale_bf16, const uint16_t *x, int64_t m_rows,
                   int64_t out_f, int64_t in_f,
                   int8_t *codes_scratch, uint16_t *w_scratch,
                   int32_t *q1_scratch, int32_t *q2_scratch, float *y)
{
    int64_t n = out_f * in_f;
    ixo_decode_codes(b1, b2, l1, l1w, l2, l2w, l3, n, codes_scratch, q1_scratch, q2_scratch);
    ixo_codes_to_bf16(codes_scratch, n, scale_bf16, w_scratch);
#pragma omp parallel for schedule(static)
    for (int64_t nrow = 0; nrow < out_f; ++nrow) {
        const uint16_t *wr = w_scratch + nrow * in_f;
        for (int64_t m = 0; m < m_rows; ++m) {
            const uint16_t *xr = x + m * in_f;
            float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
            int64_t k = 0;
            for (; k + 4 <= in_f; k += 4) {
                acc0 += bf16_to_f32(xr[k]) * bf16_to_f32(wr[k]);
                acc1 += bf16_to_f32(xr[k + 1]) * bf16_to_f32(wr[k + 1]);
                acc2 += bf16_to_f32(xr[k + 2]) * bf16_to_f32(wr[k + 2]);
                acc3 += bf16_to_f32(xr[k + 3]) * bf16_to_f32(wr[k + 3]);
            }
            for (; k < in_f; ++k) acc0 += bf16_to_f32(xr[k]) * bf16_to_f32(wr[k]);
            y[m * out_f + nrow] = (acc0 + acc1) + (acc2 + acc3);
        }
    }
}

/* ------------------------------------------------------------ bitpack ---- */

/* ixrun/bitpack.py:13-61 pack_bits_stream for a plain value array */
void ixo_pack_bits(const int32_t *vals, int64_t n, int bits, uint32_t *out)
{
    int64_t words = (n * bits + 31) / 32;
    memset(out, 0, (size_t)words * 4);
    for (int64_t i = 0; i < n; ++i)
        put_bits(out, i * bits, (uint32_t)vals[i] & ((1u << bits) - 1u), bits);
}

/* ixrun/bitpack.py:64-84 unpack_bits_stream */
void ixo_unpack_bits(const uint32_t *packed, int64_t words, int64_t n, int bits, int32_t *out)
{
    for (int64_t i = 0; i < n; ++i)
        out[i] = (int32_t)get_bits(packed, words, i * bits, bits);
}
