// Resident re-layout "P5" of an INT8-X tensor and the kernels that run on it.
//
// The reference's (3,5,8) streams (ixrun/quantize.py:80-96) are kept as the
// on-disk / interchange format.  At deploy time they can be transcoded, on the
// GPU and losslessly on the int8 codes, into a layout with fixed addressing:
//
//   plane   every element owns a 5-bit field, 32 fields = 160 bits per bitmap
//           word, stored as one uint4 + one uint32 per 32 elements.  Levels 1
//           and 2 (|code| <= 15) store code + 15; a level-3 element stores 15
//           (code 0, weight 0) as a placeholder.
//   esc     the level-3 elements as a sparse list per 256-element quarter
//           block: 16-bit entries  (position in quarter : 8) | (code + 127) << 8,
//           in element order, with an int32 offset table per quarter block.
//
// Size: 5 + 16 * P(level 3) + 0.125 bits per weight, i.e. 5.60 bpw for the
// benchmark distribution against 5.44 for the reference streams.  Nothing is
// data dependent any more except the short outlier list, so a warp decodes 1024
// weights with ~4 instructions per weight instead of ~34.
#pragma once
#include "ixb_common.cuh"

namespace ixb {

struct P5 {
    const uint4 *w03;          // [nb * 32] fields 0..24 and the low 3 bits of field 25 of every word
    const uint32_t *w4;        // [nb * 32] the remaining 32 bits
    const int32_t *esc_off;    // [nq + 1] first outlier entry of every 256-element quarter block
    const uint16_t *esc;       // [n3] outlier entries
    const __nv_bfloat16 *scale;
    uint32_t n, out_f, in_f;
};

// ------------------------------------------------------------------ build ---
// codes -> plane words + outlier count per quarter block (one warp per 1024 block, lane = word)
__global__ void __launch_bounds__(256)
k_p5_plane(const int8_t *__restrict__ codes, uint32_t n, uint4 *w03, uint32_t *w4, int32_t *qcnt)
{
    uint32_t nb = (n + kBlk - 1) / kBlk;
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= nb) return;
    uint32_t e0 = (b * 32u + lane) * 32u;
    uint32_t w[5] = {0, 0, 0, 0, 0};
    uint32_t n_esc = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        int c = e0 + i < n ? (int)codes[e0 + i] : 0;
        bool out = c > 15 || c < -15;
        n_esc += out;
        uint32_t f = out ? 15u : (uint32_t)(c + 15);
        const int bit = 5 * i, k = bit >> 5, s = bit & 31;
        w[k] |= f << s;
        if (s > 27) w[k + 1] |= f >> (32 - s);
    }
    w03[b * 32u + lane] = make_uint4(w[0], w[1], w[2], w[3]);
    w4[b * 32u + lane] = w[4];
    // 8 lanes share a quarter block
    n_esc += __shfl_xor_sync(0xffffffffu, n_esc, 1);
    n_esc += __shfl_xor_sync(0xffffffffu, n_esc, 2);
    n_esc += __shfl_xor_sync(0xffffffffu, n_esc, 4);
    uint32_t q = b * 4u + (lane >> 3);
    if ((lane & 7) == 0 && q * 256u < n) qcnt[q] = (int32_t)n_esc;
}

// outlier entries, in element order (one warp per quarter block, lane = 8 elements)
__global__ void __launch_bounds__(256)
k_p5_esc(const int8_t *__restrict__ codes, uint32_t n, const int32_t *__restrict__ esc_off, uint16_t *esc)
{
    uint32_t nq = (n + 255u) / 256u;
    uint32_t q = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (q >= nq) return;
    uint32_t e0 = q * 256u + lane * 8u;
    int c[8];
    uint32_t cnt = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        c[i] = e0 + i < n ? (int)codes[e0 + i] : 0;
        cnt += (c[i] > 15 || c[i] < -15);
    }
    uint32_t at = (uint32_t)esc_off[q] + warp_incl_scan(cnt, lane) - cnt;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (c[i] > 15 || c[i] < -15) esc[at++] = (uint16_t)((lane * 8u + i) | ((uint32_t)(c[i] + 127) << 8));
}

// ---------------------------------------------------------------- decode ----
// field i of a word's 160-bit string, as an integer 0..31
__device__ __forceinline__ uint32_t p5_field(const uint32_t (&w)[5], int i)
{
    const int bit = 5 * i, k = bit >> 5, s = bit & 31;
    uint32_t v = w[k] >> s;
    if (s > 27) v |= w[k + 1] << (32 - s);
    return v & 31u;
}

// P5 -> int8 codes (OUT 0) or bf16 weights (OUT 1); one warp per block
template <int OUT>
__global__ void __launch_bounds__(256) k_p5_decode(P5 p, void *out)
{
    uint32_t nb = (p.n + kBlk - 1) / kBlk;
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= nb) return;
    float sc = __bfloat162float(*p.scale);
    uint4 a = p.w03[b * 32u + lane];
    uint32_t w[5] = {a.x, a.y, a.z, a.w, p.w4[b * 32u + lane]};
    uint32_t e0 = (b * 32u + lane) * 32u;
    uint32_t r[OUT == 0 ? 8 : 16];
#pragma unroll
    for (int i = 0; i < (OUT == 0 ? 8 : 16); ++i) r[i] = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        int c = (int)p5_field(w, i) - 15;
        if (OUT == 0) r[i >> 2] |= (uint32_t)(c & 0xff) << (8 * (i & 3));
        else r[i >> 1] |= (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn((float)c * sc)) << (16 * (i & 1));
    }
    if (e0 + 32u <= p.n) {
        uint4 *o = (uint4 *)((char *)out + (size_t)e0 * (OUT == 0 ? 1 : 2));
#pragma unroll
        for (int j = 0; j < (OUT == 0 ? 2 : 4); ++j) o[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    } else {
        for (uint32_t i = 0; e0 + i < p.n; ++i) {
            if (OUT == 0) ((int8_t *)out)[e0 + i] = (int8_t)((r[i >> 2] >> (8 * (i & 3))) & 0xff);
            else ((uint16_t *)out)[e0 + i] = (uint16_t)((r[i >> 1] >> (16 * (i & 1))) & 0xffff);
        }
    }
    __syncwarp();
    // the block's outliers overwrite their placeholders (all plane stores of this warp are done)
    uint32_t q0 = b * 4u, nq = (p.n + 255u) / 256u;
    int32_t o0 = p.esc_off[q0], o1 = p.esc_off[min(q0 + 1, nq)], o2 = p.esc_off[min(q0 + 2, nq)],
            o3 = p.esc_off[min(q0 + 3, nq)], o4 = p.esc_off[min(q0 + 4, nq)];
    for (int32_t j = o0 + lane; j < o4; j += 32) {
        uint32_t ent = p.esc[j];
        uint32_t quarter = (uint32_t)(j >= o1) + (uint32_t)(j >= o2) + (uint32_t)(j >= o3);
        uint32_t e = b * (uint32_t)kBlk + quarter * 256u + (ent & 255u);
        int c = (int)(ent >> 8) - 127;
        if (OUT == 0) ((int8_t *)out)[e] = (int8_t)c;
        else ((__nv_bfloat16 *)out)[e] = __float2bfloat16_rn((float)c * sc);
    }
}

// ------------------------------------------------------------------ gemv ----
constexpr int kP5Threads = 1024;
constexpr int kP5Warps = kP5Threads / 32;

// One field of a register-resident word, straight to the fp32 bit pattern of bf16(code * scale):
// the field is masked into the mantissa of 2^23 (it sits at bit SH <= 18 of SRC), one FFMA turns that
// into the exact float code, one packed bf16 multiply rounds code * scale like the reference does.
#define IXB_P5_W(SRC, SH, OUT)                                                                              \
    {                                                                                                       \
        uint32_t f_ = ((SRC) & (31u << (SH))) | 0x4B000000u;                                                \
        float c_ = fmaf(__uint_as_float(f_), 1.0f / (float)(1u << (SH)), -(8388608.0f / (float)(1u << (SH)) + 15.0f)); \
        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(OUT) : "r"(__float_as_uint(c_)), "r"(s2));                   \
    }

// XS = 1: activations as swizzled fp32 in shared memory; XS = 0: bf16 straight from global memory (L1/L2)
template <int M, int XS>
__global__ void __launch_bounds__(kP5Threads, 1)
k_p5_gemv(P5 p, const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ bias, void *y, int y_f32,
          float *slots, uint32_t *ticket, uint32_t nb, uint32_t bpw, uint32_t pmax, uint32_t xstride)
{
    extern __shared__ __align__(16) float p5_xs[];     // M rows of x as fp32, swizzled like in k_gemv
    __shared__ uint32_t is_last;
    uint32_t s2;
    {
        uint32_t sb = (uint32_t)__bfloat16_as_ushort(*p.scale);
        s2 = sb | (sb << 16);
        if (XS) {
            for (uint32_t i = threadIdx.x; i < (uint32_t)M * p.in_f; i += blockDim.x) {
                uint32_t m = i / p.in_f, k = i - m * p.in_f;
                uint32_t pos = ((k >> 10) * 8u + ((k & 31u) >> 2)) * 128u + ((k >> 5) & 31u) * 4u + (k & 3u);
                p5_xs[m * xstride + pos] = __bfloat162float(x[i]);
            }
        }
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const uint32_t gw = blockIdx.x * kP5Warps + (threadIdx.x >> 5);
    const uint32_t b_begin = gw * bpw;
    const uint32_t b_end = min(b_begin + bpw, nb);
    const uint32_t nq = (p.n + 255u) / 256u;

    auto emit = [&](uint32_t row, const float (&acc)[M]) {
        uint32_t fb = (uint32_t)(((unsigned long long)row * p.in_f) >> 10);
        uint32_t lb = (uint32_t)((((unsigned long long)(row + 1) * p.in_f) - 1) >> 10);
        bool whole = fb >= b_begin && lb < b_end;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float v = warp_sum(acc[m]);
            if (lane == 0) {
                if (whole) {
                    size_t o = (size_t)m * p.out_f + row;
                    if (y_f32) {
                        ((float *)y)[o] = bias ? v + __bfloat162float(bias[row]) : v;
                    } else {
                        __nv_bfloat16 h = __float2bfloat16_rn(v);
                        if (bias) h = __hadd(h, bias[row]);
                        ((__nv_bfloat16 *)y)[o] = h;
                    }
                } else {
                    slots[((size_t)m * p.out_f + row) * pmax + (gw - fb / bpw)] = v;
                }
            }
        }
    };

    if (b_begin < b_end) {
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        // row and in-row offset of the current block's first element (warp uniform, kept incrementally)
        uint32_t blk_row = (uint32_t)(((unsigned long long)b_begin * kBlk) / p.in_f);
        uint32_t blk_k = (uint32_t)((unsigned long long)b_begin * kBlk - (unsigned long long)blk_row * p.in_f);

        // plane words and outlier offsets of the next two blocks are in flight while one is used
        auto load_w03 = [&](uint32_t b) { return b < b_end ? p.w03[b * 32u + lane] : make_uint4(0, 0, 0, 0); };
        auto load_w4 = [&](uint32_t b) { return b < b_end ? p.w4[b * 32u + lane] : 0u; };
        // lanes 0..4 hold esc_off[4b .. 4b+4]
        auto load_off = [&](uint32_t b) {
            return (b < b_end && lane < 5) ? __ldg(p.esc_off + min(b * 4u + (uint32_t)lane, nq)) : 0;
        };
        uint4 p1_03 = load_w03(b_begin), p2_03 = load_w03(b_begin + 1);
        uint32_t p1_4 = load_w4(b_begin), p2_4 = load_w4(b_begin + 1);
        int32_t p1_off = load_off(b_begin), p2_off = load_off(b_begin + 1);

        for (uint32_t b = b_begin; b < b_end; ++b) {
            const uint4 a = p1_03;
            const uint32_t w4 = p1_4;
            const int32_t off = p1_off;
            p1_03 = p2_03; p1_4 = p2_4; p1_off = p2_off;
            p2_03 = load_w03(b + 2); p2_4 = load_w4(b + 2); p2_off = load_off(b + 2);

            const uint32_t blk_e0 = b * (uint32_t)kBlk;
            const uint32_t blk_cnt = min((uint32_t)kBlk, p.n - blk_e0);          // elements in this block
            const bool one_row = blk_k + blk_cnt <= p.in_f;
            // this lane's word: element offset in the block 32*lane; row / column only needed per path
            const bool valid = 32u * lane < blk_cnt;
            uint32_t k0 = blk_k + 32u * lane, lrow = blk_row;
            if (!one_row) while (k0 >= p.in_f) { k0 -= p.in_f; ++lrow; }

            // five source words plus their halves shifted down by 16 (fields at bit 19..31 are taken from those)
            const uint32_t w0 = a.x, w1 = a.y, w2 = a.z, w3 = a.w;
            const uint32_t h0 = __funnelshift_r(w0, w1, 16), h1 = __funnelshift_r(w1, w2, 16),
                           h2 = __funnelshift_r(w2, w3, 16), h3 = __funnelshift_r(w3, w4, 16), h4 = w4 >> 16;
            const uint32_t xword = (k0 >> 10) * 256u + ((k0 >> 5) & 31u);
            float part[M];
#pragma unroll
            for (int m = 0; m < M; ++m) part[m] = 0.f;
            if (valid) {
#pragma unroll
                for (int g = 0; g < 8; ++g) {       // 4 elements per step: one float4 of x per row
                    float4 xv[M];
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        if (XS) {
                            xv[m] = ((const float4 *)(p5_xs + (size_t)m * xstride))[xword + 32 * g];
                        } else {
                            uint2 r = __ldg((const uint2 *)(x + (size_t)m * p.in_f + k0) + g);
                            xv[m] = make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                                                __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int i = 4 * g + j, bit = 5 * i, k = bit >> 5, s = bit & 31;
                        uint32_t wv;
                        if (s <= 18) {
                            const uint32_t src = k == 0 ? w0 : k == 1 ? w1 : k == 2 ? w2 : k == 3 ? w3 : w4;
                            IXB_P5_W(src, s, wv)
                        } else {
                            const uint32_t src = k == 0 ? h0 : k == 1 ? h1 : k == 2 ? h2 : k == 3 ? h3 : h4;
                            IXB_P5_W(src, s - 16, wv)
                        }
                        const float wt = __uint_as_float(wv);
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            const float xf = j == 0 ? xv[m].x : j == 1 ? xv[m].y : j == 2 ? xv[m].z : xv[m].w;
                            part[m] = fmaf(xf, wt, part[m]);
                        }
                    }
                }
            }

            // ---- level-3 outliers of this block (lane j takes entries j, j+32, ...)
            const int32_t o0 = __shfl_sync(0xffffffffu, off, 0), o1 = __shfl_sync(0xffffffffu, off, 1),
                          o2 = __shfl_sync(0xffffffffu, off, 2), o3 = __shfl_sync(0xffffffffu, off, 3),
                          o4 = __shfl_sync(0xffffffffu, off, 4);
            // contribution of this lane's outlier entries that lie in row r (any row when the block has one row)
            auto outliers = [&](uint32_t r, uint32_t r_k0, bool any_row, float (&dst)[M]) {
                // r_k0: in-row offset of the block's first element if it were in row r (may be "negative")
                for (int32_t j = o0 + lane; j < o4; j += 32) {
                    uint32_t ent = __ldg(p.esc + j);
                    uint32_t quarter = (uint32_t)(j >= o1) + (uint32_t)(j >= o2) + (uint32_t)(j >= o3);
                    uint32_t kk = r_k0 + quarter * 256u + (ent & 255u);          // column if the entry is in row r
                    if (!any_row && kk >= p.in_f) continue;                       // wraps for other rows
                    float cf = (float)((int)(ent >> 8) - 127);
                    uint32_t wv;
                    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(wv) : "r"(__float_as_uint(cf)), "r"(s2));
                    uint32_t pos = ((kk >> 10) * 8u + ((kk & 31u) >> 2)) * 128u + ((kk >> 5) & 31u) * 4u + (kk & 3u);
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        float xf = XS ? p5_xs[(size_t)m * xstride + pos] : __bfloat162float(x[(size_t)m * p.in_f + kk]);
                        dst[m] = fmaf(xf, __uint_as_float(wv), dst[m]);
                    }
                }
            };
            if (one_row) {
                // the usual case: the whole block belongs to blk_row
                if (o4 > o0) outliers(blk_row, blk_k, true, part);
#pragma unroll
                for (int m = 0; m < M; ++m) acc[m] += part[m];
                if (blk_k + blk_cnt == p.in_f || blk_e0 + blk_cnt >= p.n) {      // the row ends with this block
                    emit(blk_row, acc);
#pragma unroll
                    for (int m = 0; m < M; ++m) acc[m] = 0.f;
                }
            } else {
                // the block covers the tail of blk_row and one or more following rows
                uint32_t r = blk_row, r_k0 = blk_k;                               // r_k0 wraps below zero for later rows
                uint32_t covered = 0;
                while (covered < blk_cnt) {
                    if (valid && lrow == r) {
#pragma unroll
                        for (int m = 0; m < M; ++m) acc[m] += part[m];
                    }
                    outliers(r, r_k0, false, acc);
                    uint32_t in_row = min(p.in_f - (r == blk_row ? blk_k : 0u), blk_cnt - covered);
                    covered += in_row;
                    bool row_done = (r == blk_row ? blk_k : 0u) + in_row == p.in_f || blk_e0 + covered >= p.n;
                    if (row_done) {
                        emit(r, acc);
#pragma unroll
                        for (int m = 0; m < M; ++m) acc[m] = 0.f;
                    }
                    ++r;
                    r_k0 -= p.in_f;
                }
            }
            // advance the block position
            blk_k += blk_cnt;
            while (blk_k >= p.in_f) { blk_k -= p.in_f; ++blk_row; }
        }
        // run ended inside a row: hand the partial sum over
        uint32_t end_e = min(b_end * (uint32_t)kBlk, p.n);
        if (end_e < p.n && blk_k != 0) emit(blk_row, acc);
    }

    // ---- last CTA sums the rows that were shared between runs (same scheme as k_gemv)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t t = atomicAdd(ticket, 1u);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    uint32_t n_runs = (nb + bpw - 1) / bpw;
    for (uint32_t g = 1 + threadIdx.x; g < n_runs; g += blockDim.x) {
        unsigned long long e = (unsigned long long)g * bpw * kBlk;
        uint32_t row = (uint32_t)(e / p.in_f);
        unsigned long long row_e0 = (unsigned long long)row * p.in_f;
        if (e == row_e0) continue;
        unsigned long long prev = (unsigned long long)(g - 1) * bpw * kBlk;
        if (prev > row_e0) continue;
        uint32_t fb = (uint32_t)(row_e0 >> 10);
        uint32_t lb = (uint32_t)((row_e0 + p.in_f - 1) >> 10);
        uint32_t np = lb / bpw - fb / bpw + 1;
        for (int m = 0; m < M; ++m) {
            const float *sl = slots + ((size_t)m * p.out_f + row) * pmax;
            float v = 0.f;
            for (uint32_t q = 0; q < np; ++q) v += __ldcg(sl + q);
            size_t o = (size_t)m * p.out_f + row;
            if (y_f32) {
                ((float *)y)[o] = bias ? v + __bfloat162float(bias[row]) : v;
            } else {
                __nv_bfloat16 h = __float2bfloat16_rn(v);
                if (bias) h = __hadd(h, bias[row]);
                ((__nv_bfloat16 *)y)[o] = h;
            }
        }
    }
    if (threadIdx.x == 0) *ticket = 0;
}

}  // namespace ixb
