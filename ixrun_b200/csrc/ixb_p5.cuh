// Resident re-layout "P5" of an INT8-X tensor and the kernels that run on it.
//
// The reference's (3,5,8) streams (ixrun/quantize.py:80-96) are kept as the
// on-disk / interchange format.  At deploy time they can be transcoded, on the
// GPU and losslessly on the int8 codes, into a layout with fixed addressing in
// which nothing but a short outlier list is data dependent:
//
//   plane   every element owns a 5-bit field: code + 15 for |code| <= 15
//           (levels 1 and 2), 15 (code 0, weight 0) as a placeholder for a
//           level-3 element.  The matrix is cut into tiles of 16 rows x 64
//           columns ("blocks", 1024 elements, padded with placeholders at the
//           ragged edges); one warp owns a block, a lane 32 of its fields in
//           five 32-bit words (one uint4 + one uint32), ordered so that after
//           one mask, one subtract and one multiply per PAIR of elements the
//           lane's registers ARE the A fragments of four
//           mma.sync.m16n8k16 (bf16) instructions -- see p5_elem().
//   esc     the level-3 elements of every block as 32-bit entries
//           (slot << 16) | bf16(code * scale): the weight itself, and the
//           byte offset of the 16-bit A-fragment slot it belongs to in a
//           1024-slot image of the block (p5_slot()); blk_off[nb + 1] gives
//           the first entry of every block.
//
// Size: 5 + 32 * P(level 3) bits per weight + 4 bytes per block, i.e. ~6.0 bpw
// for the benchmark distribution against 5.44 for the reference streams.
//
// y = W x is one kernel (k_p5_mma): a warp turns a block's fields into bf16
// weights bf16(code * scale) -- the reference's dequantised weights, bit for
// bit (ixrun/quantize.py:201-204) -- which are the A operand of four mma.sync
// with the activations as B; the block's outliers are scattered into a zeroed
// fragment image in shared memory that feeds four more mma.sync.  Up to 8
// activation rows cost the same as one.  Products are exact, accumulation is
// fp32.
#pragma once
#include "ixb_common.cuh"

namespace ixb {

constexpr int kP5TileRows = 16;
constexpr int kP5TileCols = 64;
constexpr int kP5SlackBlocks = 4;    // readable blocks behind the planes and offsets (the GEMV's prefetch runs past the end)
constexpr int kP5SlackEntries = 64;  // readable entries behind the outlier list

struct P5 {
    const uint4 *w03;          // [(nb + slack) * 32] plane words 0..3 of every lane of every block
    const uint32_t *w4;        // [(nb + slack) * 32] plane word 4
    const int32_t *blk_off;    // [nb + 1 + slack] first outlier entry of every block (the slack repeats the total)
    const uint32_t *esc;       // [n_esc + slack] outlier entries
    const __nv_bfloat16 *scale;
    uint32_t out_f, in_f;
    uint32_t rt, kb;           // row tiles, column blocks per row tile; nb = rt * kb
};

// ----------------------------------------------------------- field layout ---
// Lane l of a block: g = l >> 2, t = l & 3.  Its 16 pairs p = 4 j + q (j = 0..3 the mma, q = 0..3 the A register):
//   row    = 16 R + g + 8 (q & 1)
//   column = 64 kb + 16 t + 4 j + 2 (q >> 1) + h          (h = 0 low half, 1 high half of the register)
// i.e. the k index of mma j is permuted so that a lane needs the 16 consecutive activations 16 t .. 16 t + 15.
// Pair p < 15 lives in word p / 3 at bit 5 (p % 3) (low element) and 16 + 5 (p % 3) (high element);
// pair 15 is spread over the spare bits: bit i of its low / high field is bit 15 / 31 of word i.
__device__ __forceinline__ void p5_elem(int lane, int p, int h, uint32_t &row_in_tile, uint32_t &col_in_tile)
{
    int g = lane >> 2, t = lane & 3, j = p >> 2, q = p & 3;
    row_in_tile = (uint32_t)(g + 8 * (q & 1));
    col_in_tile = (uint32_t)(16 * t + 4 * j + 2 * (q >> 1) + h);
}

__device__ __forceinline__ void p5_put(uint32_t (&w)[5], int p, int h, uint32_t f)
{
    if (p < 15) {
        w[p / 3] |= f << (5 * (p % 3) + 16 * h);
    } else {
#pragma unroll
        for (int i = 0; i < 5; ++i) w[i] |= ((f >> i) & 1u) << (15 + 16 * h);
    }
}

__device__ __forceinline__ uint32_t p5_get(const uint32_t (&w)[5], int p, int h)
{
    if (p < 15) return (w[p / 3] >> (5 * (p % 3) + 16 * h)) & 31u;
    uint32_t f = 0;
#pragma unroll
    for (int i = 0; i < 5; ++i) f |= ((w[i] >> (15 + 16 * h)) & 1u) << i;
    return f;
}

// Byte offset of element (lane, pair p, half h) in the block's fragment image: 64 uint4, uint4 (p >> 2) * 32 + lane
// holds the lane's A registers of mma p >> 2, so that a lane reads its four registers with one conflict-free load.
__device__ __forceinline__ uint32_t p5_slot(int lane, int p, int h)
{
    return (uint32_t)((((p >> 2) * 32 + lane) * 4 + (p & 3)) * 4 + 2 * h);
}

// ------------------------------------------------------------------ build ---
// codes [out_f, in_f] -> plane words and the number of outliers of every block (one warp per block)
__global__ void __launch_bounds__(256)
k_p5_plane(const int8_t *__restrict__ codes, uint32_t out_f, uint32_t in_f, uint32_t rt, uint32_t kb,
           uint4 *w03, uint32_t *w4, int32_t *blk_cnt)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= rt * kb) return;
    uint32_t R = b / kb, kbi = b - R * kb;
    uint32_t w[5] = {0, 0, 0, 0, 0};
    uint32_t n_out = 0;
#pragma unroll
    for (int p = 0; p < 16; ++p) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t r, c;
            p5_elem(lane, p, h, r, c);
            uint32_t row = R * kP5TileRows + r, col = kbi * kP5TileCols + c;
            int code = (row < out_f && col < in_f) ? (int)codes[(size_t)row * in_f + col] : 0;
            bool out = code > 15 || code < -15;
            n_out += out;
            p5_put(w, p, h, out ? 15u : (uint32_t)(code + 15));
        }
    }
    w03[(size_t)b * 32u + lane] = make_uint4(w[0], w[1], w[2], w[3]);
    w4[(size_t)b * 32u + lane] = w[4];
    n_out = warp_incl_scan(n_out, lane);
    if (lane == 31) blk_cnt[b] = (int32_t)n_out;
}

// outlier entries of every block, in (lane, pair, half) order (one warp per block)
__global__ void __launch_bounds__(256)
k_p5_esc(const int8_t *__restrict__ codes, uint32_t out_f, uint32_t in_f, uint32_t rt, uint32_t kb,
         const int32_t *__restrict__ blk_off, const __nv_bfloat16 *__restrict__ scale, uint32_t *esc)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= rt * kb) return;
    uint32_t R = b / kb, kbi = b - R * kb;
    float sc = __bfloat162float(*scale);
    int code[32];
    uint32_t n_out = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        uint32_t r, c;
        p5_elem(lane, i >> 1, i & 1, r, c);
        uint32_t row = R * kP5TileRows + r, col = kbi * kP5TileCols + c;
        code[i] = (row < out_f && col < in_f) ? (int)codes[(size_t)row * in_f + col] : 0;
        n_out += (code[i] > 15 || code[i] < -15);
    }
    uint32_t at = (uint32_t)blk_off[b] + warp_incl_scan(n_out, lane) - n_out;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        if (code[i] > 15 || code[i] < -15) {
            uint32_t wbits = __bfloat16_as_ushort(__float2bfloat16_rn((float)code[i] * sc));
            esc[at++] = (p5_slot(lane, i >> 1, i & 1) << 16) | wbits;
        }
    }
}

// ---------------------------------------------------------------- decode ----
// plane -> int8 codes (OUT 0) or bf16 weights (OUT 1), row major [out_f, in_f]; outliers come out as 0 here.
// A lane holds 16 consecutive columns of two rows: one or two 16-byte stores per row.
template <int OUT>
__global__ void __launch_bounds__(256) k_p5_decode_plane(P5 p, void *out)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= p.rt * p.kb) return;
    uint32_t R = b / p.kb, kbi = b - R * p.kb;
    float sc = __bfloat162float(*p.scale);
    uint4 a = p.w03[(size_t)b * 32u + lane];
    uint32_t w[5] = {a.x, a.y, a.z, a.w, p.w4[(size_t)b * 32u + lane]};
    const bool vec = (OUT == 0 ? (p.in_f & 15u) == 0 : (p.in_f & 7u) == 0) && ((uintptr_t)out & 15u) == 0;
#pragma unroll
    for (int s = 0; s < 2; ++s) {                    // row g, row g + 8
        uint32_t row = R * kP5TileRows + (lane >> 2) + 8 * s, col0 = kbi * kP5TileCols + 16 * (lane & 3);
        if (row >= p.out_f || col0 >= p.in_f) continue;
        uint32_t r[OUT == 0 ? 4 : 8];
#pragma unroll
        for (int i = 0; i < (OUT == 0 ? 4 : 8); ++i) r[i] = 0;
#pragma unroll
        for (int c = 0; c < 16; ++c) {               // column col0 + c = pair 4 (c >> 2) + 2 ((c >> 1) & 1) + s, half c & 1
            int code = (int)p5_get(w, 4 * (c >> 2) + 2 * ((c >> 1) & 1) + s, c & 1) - 15;
            if (OUT == 0) r[c >> 2] |= (uint32_t)(code & 0xff) << (8 * (c & 3));
            else r[c >> 1] |= (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn((float)code * sc)) << (16 * (c & 1));
        }
        size_t o = (size_t)row * p.in_f + col0;
        if (vec && col0 + 16u <= p.in_f) {
            uint4 *dst = (uint4 *)((char *)out + o * (OUT == 0 ? 1 : 2));
            dst[0] = make_uint4(r[0], r[1], r[2], r[3]);
            if (OUT == 1) dst[1] = make_uint4(r[4], r[5], r[6], r[7]);
        } else {
            for (uint32_t c = 0; c < 16u && col0 + c < p.in_f; ++c) {
                if (OUT == 0) ((int8_t *)out)[o + c] = (int8_t)((r[c >> 2] >> (8 * (c & 3))) & 0xff);
                else ((uint16_t *)out)[o + c] = (uint16_t)((r[c >> 1] >> (16 * (c & 1))) & 0xffff);
            }
        }
    }
}

// The outliers overwrite their placeholders (launched after k_p5_decode_plane on the same stream; one warp per
// block).  An entry carries the bf16 weight w = bf16(code * scale).  The code is recovered from it exactly:
// neighbouring codes differ by scale >= |code * scale| / 127, which is more than one bf16 ulp (2^-7 relative),
// so no two codes share a weight, and w / scale is within 0.25 of the code.
template <int OUT>
__global__ void __launch_bounds__(256) k_p5_decode_esc(P5 p, void *out)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= p.rt * p.kb) return;
    uint32_t R = b / p.kb, kbi = b - R * p.kb;
    float sc = __bfloat162float(*p.scale);
    for (int32_t j = p.blk_off[b] + lane; j < p.blk_off[b + 1]; j += 32) {
        uint32_t ent = p.esc[j];
        uint32_t slot = ent >> 16;                       // ((mma * 32 + lane) * 4 + q) * 4 + 2 h
        int h = (slot >> 1) & 1, q = (slot >> 2) & 3, ln = (slot >> 4) & 31, j4 = slot >> 9;
        uint32_t r, c;
        p5_elem(ln, 4 * j4 + q, h, r, c);
        uint32_t row = R * kP5TileRows + r, col = kbi * kP5TileCols + c;
        if (row >= p.out_f || col >= p.in_f) continue;
        size_t o = (size_t)row * p.in_f + col;
        __nv_bfloat16 wv = __ushort_as_bfloat16((unsigned short)(ent & 0xffffu));
        if (OUT == 1) {
            ((__nv_bfloat16 *)out)[o] = wv;
        } else {
            int best = __float2int_rn(__bfloat162float(wv) / sc);
            ((int8_t *)out)[o] = (int8_t)best;
        }
    }
}

// ------------------------------------------------------------- plane pass ---
constexpr int kP5Threads = 768;
constexpr int kP5Warps = kP5Threads / 32;
constexpr int kP5SmemFixed = kP5Warps * (2 * 32 * 16 + 4 * 32 * 16);   // partial sums + outlier fragment images

// (SRC & 0x001F001F) | 0x43004300: the two fields of a pair as the bf16 values 128 + field
__device__ __forceinline__ uint32_t p5_pair_raw(uint32_t src, uint32_t magic)
{
    uint32_t v;
    asm("lop3.b32 %0, %1, 0x001F001F, %2, 0xEA;" : "=r"(v) : "r"(src), "r"(magic));
    return v;
}
// (SRC & MASK) | ACC
__device__ __forceinline__ uint32_t p5_and_or(uint32_t src, uint32_t mask, uint32_t acc)
{
    uint32_t v;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(src), "r"(mask), "r"(acc));
    return v;
}
// two bf16 values 128 + field -> two bf16 weights bf16((field - 15) * scale): the subtraction is exact,
// the multiplication rounds once, like the reference's bf16 product code * scale
__device__ __forceinline__ uint32_t p5_pair_weight(uint32_t v, uint32_t one2, uint32_t neg2, uint32_t s2)
{
    uint32_t d, w;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(v), "r"(one2), "r"(neg2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w) : "r"(d), "r"(s2));
    return w;
}

__device__ __forceinline__ void p5_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// layout -> bf16 weights with the GEMV's own conversion (three instructions per pair of elements) and its outlier
// image, so every weight is stored once, in 16-byte pieces; needs in_f % 8 == 0 and a 16-byte aligned output
__global__ void __launch_bounds__(256) k_p5_decode_bf16(P5 p, __nv_bfloat16 *out)
{
    __shared__ uint4 images[8 * 128];                // one 2 KB fragment image per warp
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= p.rt * p.kb) return;                    // whole warps leave together
    uint4 *img = images + (threadIdx.x >> 5) * 128;
#pragma unroll
    for (int q = 0; q < 4; ++q) img[q * 32 + lane] = make_uint4(0, 0, 0, 0);
    __syncwarp();
    {
        const uint32_t img_s = (uint32_t)__cvta_generic_to_shared(img);
        const int32_t lo = __ldg(p.blk_off + b), hi = __ldg(p.blk_off + b + 1);
        for (int32_t j = lo + lane; j < hi; j += 32) {
            uint32_t e = __ldg(p.esc + j);
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(img_s + (e >> 16)), "h"((unsigned short)e) : "memory");
        }
    }
    __syncwarp();
    uint32_t R = b / p.kb, kbi = b - R * p.kb;
    uint32_t sb = (uint32_t)__bfloat16_as_ushort(*p.scale);
    const uint32_t s2 = sb | (sb << 16), magic = 0x43004300u, one2 = 0x3F803F80u, neg2 = 0xC30FC30Fu;
    uint4 a = p.w03[(size_t)b * 32u + lane];
    const uint32_t w[5] = {a.x, a.y, a.z, a.w, p.w4[(size_t)b * 32u + lane]};
    uint32_t f[16];
#pragma unroll
    for (int k = 0; k < 5; ++k) {
        f[3 * k] = p5_pair_raw(w[k], magic);
        f[3 * k + 1] = p5_pair_raw(w[k] >> 5, magic);
        f[3 * k + 2] = p5_pair_raw(w[k] >> 10, magic);
    }
    {
        uint32_t v = p5_and_or(w[0] >> 15, 0x00010001u, magic);
        v = p5_and_or(w[1] >> 14, 0x00020002u, v);
        v = p5_and_or(w[2] >> 13, 0x00040004u, v);
        v = p5_and_or(w[3] >> 12, 0x00080008u, v);
        f[15] = p5_and_or(w[4] >> 11, 0x00100010u, v);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = p5_pair_weight(f[i], one2, neg2, s2);
#pragma unroll
    for (int q = 0; q < 4; ++q) {                    // placeholders are +0.0, so OR-ing the outlier weights in is exact
        const uint4 v = img[q * 32 + lane];
        f[4 * q] |= v.x;
        f[4 * q + 1] |= v.y;
        f[4 * q + 2] |= v.z;
        f[4 * q + 3] |= v.w;
    }
    // pair 4 j + q: row g + 8 (q & 1), columns 4 j + 2 (q >> 1) + {0, 1} of the lane's 16
    const uint32_t col0 = kbi * kP5TileCols + 16 * (lane & 3);
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        uint32_t row = R * kP5TileRows + (lane >> 2) + 8 * s;
        if (row >= p.out_f || col0 >= p.in_f) continue;
        __nv_bfloat16 *dst = out + (size_t)row * p.in_f + col0;
        const uint32_t r[8] = {f[0 + s], f[2 + s], f[4 + s], f[6 + s], f[8 + s], f[10 + s], f[12 + s], f[14 + s]};
        if (col0 + 16u <= p.in_f) {
            ((uint4 *)dst)[0] = make_uint4(r[0], r[1], r[2], r[3]);
            ((uint4 *)dst)[1] = make_uint4(r[4], r[5], r[6], r[7]);
        } else {
            for (uint32_t c = 0; col0 + c < p.in_f; ++c) ((uint16_t *)dst)[c] = (uint16_t)(r[c >> 1] >> (16 * (c & 1)));
        }
    }
}

// Final value of a row tile's C fragment image: lane (g, t) holds rows g, g + 8 and activation rows 2 t, 2 t + 1.
__device__ __forceinline__ void p5_store_tile(const P5 &p, uint32_t R, int lane, const float (&c)[4], uint32_t m_rows,
                                              const __nv_bfloat16 *__restrict__ bias, void *y, int y_f32)
{
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t m = 2u * t + (i & 1), row = R * kP5TileRows + g + 8 * (i >> 1);
        if (m >= m_rows || row >= p.out_f) continue;
        size_t o = (size_t)m * p.out_f + row;
        float v = c[i];
        if (y_f32) {
            ((float *)y)[o] = bias ? v + __bfloat162float(bias[row]) : v;
        } else {
            __nv_bfloat16 hv = __float2bfloat16_rn(v);
            if (bias) hv = __hadd(hv, bias[row]);
            ((__nv_bfloat16 *)y)[o] = hv;
        }
    }
}

// first element of part i when n elements are cut into `parts` nearly equal contiguous parts, and its inverse
__device__ __forceinline__ uint32_t p5_part_begin(uint32_t i, uint32_t n, uint32_t parts)
{
    return (uint32_t)(((unsigned long long)i * n) / parts);
}
__device__ __forceinline__ uint32_t p5_part_of(uint32_t pos, uint32_t n, uint32_t parts)
{
    return (uint32_t)((((unsigned long long)pos + 1u) * parts - 1u) / n);     // largest i with part_begin(i) <= pos
}

// The nb blocks, in (row tile, column block) order, are cut into gridDim.x nearly equal contiguous CTA ranges
// and every CTA range into 32 warp runs.  Row tiles that a run covers completely are written straight to y.
// Partial tiles go to shared memory and are summed per CTA in warp order; a tile shared between CTAs goes
// through cta_slots, and the CTA that arrives last at the tile's ticket sums the slots in CTA order -- no
// floating-point atomics anywhere, so results are reproducible.  tickets[] (gridDim.x + 1 words) must be zero
// before the first launch and is left zero.  XS = 1: activations staged in shared memory (bf16, padded rows);
// XS = 0: read from global memory.
template <int XS>
__global__ void __launch_bounds__(kP5Threads, 1)
k_p5_mma(P5 p, const __nv_bfloat16 *__restrict__ x, uint32_t m_rows, const __nv_bfloat16 *__restrict__ bias, void *y,
         int y_f32, float4 *cta_slots, uint32_t *tickets, uint32_t nb, uint32_t xstride)
{
    extern __shared__ __align__(16) unsigned char p5_smem[];
    float4 *parts = (float4 *)p5_smem;                                  // [warp][2][32 lanes] partial tile sums
    uint4 *images = (uint4 *)(p5_smem + kP5Warps * 2 * 32 * sizeof(float4));             // [warp][4 mma][32 lanes]
    __nv_bfloat16 *xs = (__nv_bfloat16 *)(p5_smem + kP5SmemFixed);                       // [m_rows][xstride]

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t KB = p.kb, G = gridDim.x;
    uint32_t sb = (uint32_t)__bfloat16_as_ushort(*p.scale);
    const uint32_t s2 = sb | (sb << 16);
    uint32_t magic, one2, neg2;
    // opaque to the optimiser, so that they stay in registers as LOP3 / HFMA2 operands
    asm volatile("mov.b32 %0, 0x43004300;" : "=r"(magic));
    asm volatile("mov.b32 %0, 0x3F803F80;" : "=r"(one2));
    asm volatile("mov.b32 %0, 0xC30FC30F;" : "=r"(neg2));              // -143, -143

    if (XS) {
        // rows of x, zero padded up to kb * 64 columns, row stride xstride elements (16 bytes more than a multiple of 128)
        const uint32_t chunks = KB * (kP5TileCols / 8);
        for (uint32_t i = threadIdx.x; i < m_rows * chunks; i += blockDim.x) {
            uint32_t m = i / chunks, k8 = (i - m * chunks) * 8u;
            uint4 v;
            if ((p.in_f & 7u) == 0 && k8 + 8u <= p.in_f) {
                v = *(const uint4 *)(x + (size_t)m * p.in_f + k8);
            } else {
                unsigned short e[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    e[j] = k8 + j < p.in_f ? __bfloat16_as_ushort(x[(size_t)m * p.in_f + k8 + j]) : (unsigned short)0;
                v = make_uint4(e[0] | ((uint32_t)e[1] << 16), e[2] | ((uint32_t)e[3] << 16), e[4] | ((uint32_t)e[5] << 16),
                               e[6] | ((uint32_t)e[7] << 16));
            }
            *(uint4 *)(xs + (size_t)m * xstride + k8) = v;
        }
    }
    __syncthreads();

    const uint32_t cb0 = p5_part_begin(blockIdx.x, nb, G), cb1 = p5_part_begin(blockIdx.x + 1, nb, G);
    const uint32_t L = cb1 - cb0;
    const uint32_t b_begin = cb0 + p5_part_begin(wid, L, kP5Warps), b_end = cb0 + p5_part_begin(wid + 1, L, kP5Warps);

    if (b_begin < b_end) {
        float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};       // plane / outlier accumulators
        uint32_t R = b_begin / KB;
        const uint32_t R_first = R;
        bool from_start = b_begin == R * KB;          // the current tile's first block belongs to this run
        // this lane's activations: row min(g, m_rows - 1) (rows beyond m_rows only feed unused C columns);
        // xo walks through the row in steps of 64 elements and wraps at the end of a tile
        const uint32_t xrow = min((uint32_t)g, m_rows - 1u);
        const __nv_bfloat16 *xl = XS ? xs + (size_t)xrow * xstride + 16 * t : x + (size_t)xrow * p.in_f + 16 * t;
        const uint32_t xo_end = KB * kP5TileCols;
        uint32_t xo = (b_begin - R * KB) * kP5TileCols;

        auto flush_tile = [&](bool whole) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                c[i] += c2[i];
                c2[i] = 0.f;
            }
            if (whole) p5_store_tile(p, R, lane, c, m_rows, bias, y, y_f32);
            else parts[(wid * 2 + (R == R_first ? 0 : 1)) * 32 + lane] = make_float4(c[0], c[1], c[2], c[3]);
            c[0] = c[1] = c[2] = c[3] = 0.f;
        };
        uint4 *img = images + wid * 4 * 32;                      // this warp's fragment image, all zero between blocks
        const uint32_t img_s = (uint32_t)__cvta_generic_to_shared(img);
#pragma unroll
        for (int q = 0; q < 4; ++q) img[q * 32 + lane] = make_uint4(0, 0, 0, 0);
        __syncwarp();

        // One block.  Everything it consumes was loaded by earlier steps into the register set it is given
        // (plane words two blocks ahead, outlier offsets two blocks ahead, the first 64 entries one block ahead);
        // the step reloads each set right after its last use, so the sets alternate by unrolling with no copies.
        //   a, w4      plane words of this block           -> reloaded with those of block + 2
        //   olo, ohi   blk_off[block], blk_off[block + 1]  -> reloaded with those of block + 2
        //   ent0, ent1 entries olo + lane, olo + 32 + lane of this block
        //   nlo        blk_off[block + 1]; nent0, nent1 receive the next block's first entries
        auto step = [&](uint4 &a, uint32_t &w4, int32_t &olo, int32_t &ohi, const uint32_t ent0, const uint32_t ent1,
                        const int32_t nlo, uint32_t &nent0, uint32_t &nent1, const uint32_t blk) {
            {
                const uint32_t *ne = p.esc + nlo + lane;
                nent0 = __ldg(ne);
                nent1 = __ldg(ne + 32);
            }
            const int32_t lo0 = olo, cnt = ohi - olo;
            olo = __ldg(p.blk_off + blk + 2u);       // a whole step ahead of their first use
            ohi = __ldg(p.blk_off + blk + 3u);
            const uint4 x0 = *(const uint4 *)(xl + xo);
            const uint4 x1 = *(const uint4 *)(xl + xo + 8);
            uint32_t f[16];
            {
                const uint32_t w[5] = {a.x, a.y, a.z, a.w, w4};
#pragma unroll
                for (int k = 0; k < 5; ++k) {
                    f[3 * k] = p5_pair_raw(w[k], magic);
                    f[3 * k + 1] = p5_pair_raw(w[k] >> 5, magic);
                    f[3 * k + 2] = p5_pair_raw(w[k] >> 10, magic);
                }
                uint32_t v = p5_and_or(w[0] >> 15, 0x00010001u, magic);
                v = p5_and_or(w[1] >> 14, 0x00020002u, v);
                v = p5_and_or(w[2] >> 13, 0x00040004u, v);
                v = p5_and_or(w[3] >> 12, 0x00080008u, v);
                f[15] = p5_and_or(w[4] >> 11, 0x00100010u, v);
            }
            {
                const uint32_t i2 = (blk + 2u) * 32u + lane;
                a = p.w03[i2];
                w4 = p.w4[i2];
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) f[i] = p5_pair_weight(f[i], one2, neg2, s2);
            p5_mma(c, f[0], f[1], f[2], f[3], x0.x, x0.y);
            p5_mma(c, f[4], f[5], f[6], f[7], x0.z, x0.w);
            p5_mma(c, f[8], f[9], f[10], f[11], x1.x, x1.y);
            p5_mma(c, f[12], f[13], f[14], f[15], x1.z, x1.w);
            {
                // The block's outliers: entry j goes to lane j % 32 (two were prefetched, more than 64 per block
                // is rare), which drops the weight into its slot of the image.  Then every lane takes its four A
                // registers per mma from the image and clears them.
                const int32_t rel = (int32_t)lane - cnt;                      // < 0: this lane has a first entry
                asm volatile("{\n\t.reg .pred p0, p1;\n\tsetp.lt.s32 p0, %4, 0;\n\tsetp.lt.s32 p1, %4, -32;\n\t"
                             "@p0 st.shared.u16 [%0], %1;\n\t@p1 st.shared.u16 [%2], %3;\n\t}"
                             ::"r"(img_s + (ent0 >> 16)), "h"((unsigned short)ent0), "r"(img_s + (ent1 >> 16)),
                             "h"((unsigned short)ent1), "r"(rel)
                             : "memory");
                if (cnt > 64) {                                               // warp uniform
                    for (int32_t j = 64 + lane; j < cnt; j += 32) {
                        uint32_t e = __ldg(p.esc + lo0 + j);
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(img_s + (e >> 16)), "h"((unsigned short)e) : "memory");
                    }
                }
                __syncwarp();
                const uint4 q0 = img[lane], q1 = img[32 + lane], q2 = img[64 + lane], q3 = img[96 + lane];
#pragma unroll
                for (int q = 0; q < 4; ++q) img[q * 32 + lane] = make_uint4(0, 0, 0, 0);
                __syncwarp();                // the image is clear before any lane writes the next block's entries
                p5_mma(c2, q0.x, q0.y, q0.z, q0.w, x0.x, x0.y);
                p5_mma(c2, q1.x, q1.y, q1.z, q1.w, x0.z, x0.w);
                p5_mma(c2, q2.x, q2.y, q2.z, q2.w, x1.x, x1.y);
                p5_mma(c2, q3.x, q3.y, q3.z, q3.w, x1.z, x1.w);
            }
            xo += kP5TileCols;
            if (xo == xo_end) {                      // the tile is complete, or this was its last part
                flush_tile(from_start);
                xo = 0;
                ++R;
                from_start = true;
            }
        };
        // The loads run up to two blocks past the end of the run: planes, offsets and entries are allocated with
        // that much slack.
        uint4 aA, aB;
        uint32_t eA, eB, nA0, nA1, nB0, nB1;
        int32_t loA, hiA, loB, hiB;
        {
            const uint32_t i0 = b_begin * 32u + lane;
            aA = p.w03[i0];
            eA = p.w4[i0];
            aB = p.w03[i0 + 32u];
            eB = p.w4[i0 + 32u];
            loA = __ldg(p.blk_off + b_begin);
            hiA = __ldg(p.blk_off + b_begin + 1);
            loB = hiA;
            hiB = __ldg(p.blk_off + b_begin + 2);
            nA0 = __ldg(p.esc + loA + lane);
            nA1 = __ldg(p.esc + loA + 32 + lane);
        }
        for (uint32_t b = b_begin;;) {
            step(aA, eA, loA, hiA, nA0, nA1, loB, nB0, nB1, b);
            if (++b == b_end) break;
            step(aB, eB, loB, hiB, nB0, nB1, loA, nA0, nA1, b);
            if (++b == b_end) break;
        }
        __syncwarp();
        if (xo != 0) flush_tile(false);
    }
    __syncthreads();

    // ---- per CTA: sum the parts of every tile that more than one run of this CTA (or another CTA) touched
    if (L) {
        const uint32_t Rc0 = cb0 / KB, Rc1 = (cb1 - 1) / KB;
        for (uint32_t R = Rc0 + wid; R <= Rc1; R += kP5Warps) {
            const uint32_t t0 = R * KB, t1 = t0 + KB;                   // the tile's blocks
            const bool inside = t0 >= cb0 && t1 <= cb1;
            const uint32_t wlo = p5_part_of(max(t0, cb0) - cb0, L, kP5Warps), whi = p5_part_of(min(t1, cb1) - 1 - cb0, L, kP5Warps);
            if (inside && wlo == whi) continue;                          // one run had all of it and wrote y itself
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t w = wlo; w <= whi; ++w) {
                uint32_t wb = p5_part_begin(w, L, kP5Warps);
                if (wb == p5_part_begin(w + 1, L, kP5Warps)) continue;  // a warp without blocks
                uint32_t rf = (cb0 + wb) / KB;
                float4 v = parts[(w * 2 + (R == rf ? 0 : 1)) * 32 + lane];
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            if (inside) {
                const float cc[4] = {s.x, s.y, s.z, s.w};
                p5_store_tile(p, R, lane, cc, m_rows, bias, y, y_f32);
                continue;
            }
            // shared with other CTAs: publish this CTA's sum, take a ticket; the last one finishes the tile
            cta_slots[((size_t)blockIdx.x * 2 + (R == Rc0 ? 0 : 1)) * 32 + lane] = s;
            __threadfence();
            __syncwarp();
            const uint32_t clo = p5_part_of(t0, nb, G), chi = p5_part_of(t1 - 1, nb, G);
            uint32_t prev = 0;
            if (lane == 0) prev = atomicAdd(tickets + clo + 1, 1u);
            prev = __shfl_sync(0xffffffffu, prev, 0);
            if (prev != chi - clo) continue;
            __threadfence();
            float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t cc = clo; cc <= chi; ++cc) {
                uint32_t rf = p5_part_begin(cc, nb, G) / KB;
                const float4 *sl = cta_slots + ((size_t)cc * 2 + (R == rf ? 0 : 1)) * 32 + lane;
                z.x += __ldcg(&sl->x); z.y += __ldcg(&sl->y); z.z += __ldcg(&sl->z); z.w += __ldcg(&sl->w);
            }
            const float cc4[4] = {z.x, z.y, z.z, z.w};
            p5_store_tile(p, R, lane, cc4, m_rows, bias, y, y_f32);
            if (lane == 0) tickets[clo + 1] = 0;
        }
    }
}

}  // namespace ixb
