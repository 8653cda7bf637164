// TPAB tile format (the reference's fixed-width successor format, ixrun/tpab.py:37-203): decode and batch-1 GEMV.
//
// The tensor is cut into tiles of tile_r x 64 (tile_r a power of two <= 64); tile t = row_tile * T_c + col_tile has a
// bit width b in 2..6 (uint8), an fp16 scale and `goff`, its element offset inside the group of tiles of its width;
// element L = r * 64 + c of the tile is the b-bit field at bit  gbase_bit[b] + (goff + L) * b  of one uint32 body,
// q = field - (2^(b-1) - 1),  w = bf16(f32(q) * f32(scale)).  No ranks, no prefix sums: any tile decodes on its own.
// Outliers (tile, element, fp16 value) replace their weights (their body fields decode to 0): the decoder scatters
// them afterwards (ixrun/tpab.py:301-302), the GEMV adds a per-row list  sum bf16(value) * x[column]
// (ixrun/tpab_gemv.py:49-67, 118-123).
//
// Both kernels give a lane one ROW of a tile: its 64 fields are 2 b consecutive words, extracted with compile-time
// shifts (one instantiation per width), so nothing is exchanged between lanes and the row's dot product stays in one
// register.  A row of 64 fields starts on a word boundary (64 b bits), so no field needs more than two words.
#pragma once
#include <cuda_fp16.h>

#include "ixb_common.cuh"

namespace ixb {

struct Tpab {
    const uint32_t *body;        // concatenated bodies of the width groups (+ 2 readable words behind)
    const uint8_t *bits;         // [T] width of every tile
    const __half *scales;        // [T]
    const int32_t *goff;         // [T] element offset of the tile inside its width group
    int32_t gbase[8];            // bit base of every width group (index = width)
    uint32_t out_f, in_f, tile_r, t_c, t_r;
};

__device__ __forceinline__ float bfround_f(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// bit base of the width group (selects instead of a dynamic index into the kernel parameter, which would put the
// whole struct on the stack)
__device__ __forceinline__ uint32_t tpab_gbase(const Tpab &p, uint32_t b)
{
    int32_t v = p.gbase[2];
    v = b == 3u ? p.gbase[3] : v;
    v = b == 4u ? p.gbase[4] : v;
    v = b == 5u ? p.gbase[5] : v;
    v = b == 6u ? p.gbase[6] : v;
    return (uint32_t)v;
}

// the 64 weights of one row of a tile of width B, as fp32 values of the bf16-rounded products
template <int B, class F>
__device__ __forceinline__ void tpab_row(const uint32_t *__restrict__ words, float s, F &&sink)
{
    constexpr int NW = 2 * B;                            // words of one row
    constexpr uint32_t MASK = (1u << B) - 1u;
    constexpr int QMAX = (1 << (B - 1)) - 1;
    uint32_t w[NW + 1];
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] = __ldg(words + i);
    w[NW] = 0u;
#pragma unroll
    for (int c = 0; c < 64; ++c) {
        const int bit = c * B, wi = bit >> 5, sh = bit & 31;
        uint32_t raw = w[wi] >> sh;
        if (sh + B > 32) raw |= w[wi + 1] << (32 - sh);
        const int q = (int)(raw & MASK) - QMAX;
        sink(c, bfround_f((float)q * s));
    }
}

template <class F>
__device__ __forceinline__ void tpab_row_any(uint32_t b, const uint32_t *__restrict__ words, float s, F &&sink)
{
    switch (b) {
    case 2: tpab_row<2>(words, s, sink); break;
    case 3: tpab_row<3>(words, s, sink); break;
    case 4: tpab_row<4>(words, s, sink); break;
    case 5: tpab_row<5>(words, s, sink); break;
    default: tpab_row<6>(words, s, sink); break;
    }
}

// ---------------------------------------------------------------- decode -> bf16 [out_f, in_f]
// One thread per (tile, row of the tile): 64 weights = 128 bytes = eight 16-byte stores.
__global__ void __launch_bounds__(128) k_tpab_decode(Tpab p, __nv_bfloat16 *__restrict__ out)
{
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t n_rows = p.t_r * p.t_c * p.tile_r;
    if (idx >= n_rows) return;
    const uint32_t t = idx / p.tile_r, r = idx - t * p.tile_r;
    const uint32_t rt = t / p.t_c, ct = t - rt * p.t_c;
    const uint32_t b = p.bits[t];
    const float s = __half2float(p.scales[t]);
    const uint32_t bit0 = tpab_gbase(p, b) + ((uint32_t)p.goff[t] + r * 64u) * b;      // (a multiple of 32: rows are word aligned)
    uint32_t o[32] = {0u};
    tpab_row_any(b, p.body + (bit0 >> 5), s, [&](int c, float w) {
        const uint32_t h = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(w));
        if (c & 1) o[c >> 1] |= h << 16;
        else o[c >> 1] = h;
    });
    uint4 *dst = (uint4 *)(out + (size_t)(rt * p.tile_r + r) * p.in_f + ct * 64u);
#pragma unroll
    for (int k = 0; k < 8; ++k) dst[k] = make_uint4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
}

// outliers over their (zero) decoded weights
__global__ void __launch_bounds__(256)
k_tpab_scatter(Tpab p, const int32_t *__restrict__ ol_t, const int32_t *__restrict__ ol_l, const __half *__restrict__ ol_val,
               uint32_t n_ol, __nv_bfloat16 *__restrict__ out)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_ol) return;
    const uint32_t t = (uint32_t)ol_t[i], l = (uint32_t)ol_l[i];
    const uint32_t rt = t / p.t_c, ct = t - rt * p.t_c, r = l >> 6, c = l & 63u;
    out[(size_t)(rt * p.tile_r + r) * p.in_f + ct * 64u + c] = __float2bfloat16_rn(__half2float(ol_val[i]));
}

// ---------------------------------------------------------------- batch-1 GEMV
// grid (row tiles, K splits), 256 threads = 8 warps.  Warp w walks the column tiles ks0 + w, ks0 + w + 8, ... of the
// CTA's K range; lane l owns rows l and l + 32 of the tile (rows >= tile_r idle).  The tile's 64 activations are put
// into the warp's shared-memory slice as fp32 and read back by every lane in the same order (broadcast, no conflicts).
// The warps' sums meet in shared memory; the CTA writes one fp32 partial per row and split, k_tpab_finalize adds the
// splits in order, the row's outlier list and the bias.
constexpr int kTpabWarps = 8;
__global__ void __launch_bounds__(kTpabWarps * 32)
k_tpab_gemv(Tpab p, const __nv_bfloat16 *__restrict__ x, float *__restrict__ part, uint32_t splits)
{
    __shared__ float xs[kTpabWarps][64];
    __shared__ float sums[kTpabWarps][64];
    const uint32_t rt = blockIdx.x, split = blockIdx.y;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint32_t kq = p.t_c / splits, kr = p.t_c - kq * splits;
    const uint32_t k0 = split * kq + min(split, kr), k1 = k0 + kq + (split < kr ? 1u : 0u);
    float acc0 = 0.f, acc1 = 0.f;
    for (uint32_t ct = k0 + (uint32_t)wid; ct < k1; ct += kTpabWarps) {
        const uint32_t t = rt * p.t_c + ct;
        const uint32_t b = p.bits[t];
        const float s = __half2float(p.scales[t]);
        const uint32_t bit_t = tpab_gbase(p, b) + (uint32_t)p.goff[t] * b;
        __syncwarp();                                     // the slice may still be read from the tile before
        const __nv_bfloat162 xv = *(const __nv_bfloat162 *)(x + ct * 64u + 2 * lane);
        xs[wid][2 * lane] = __bfloat162float(xv.x);
        xs[wid][2 * lane + 1] = __bfloat162float(xv.y);
        __syncwarp();
        const float *xw = xs[wid];
        if ((uint32_t)lane < p.tile_r)
            tpab_row_any(b, p.body + ((bit_t + (uint32_t)lane * 64u * b) >> 5), s, [&](int c, float w) { acc0 = fmaf(w, xw[c], acc0); });
        if ((uint32_t)lane + 32u < p.tile_r)
            tpab_row_any(b, p.body + ((bit_t + ((uint32_t)lane + 32u) * 64u * b) >> 5), s, [&](int c, float w) { acc1 = fmaf(w, xw[c], acc1); });
    }
    sums[wid][lane] = acc0;
    sums[wid][lane + 32] = acc1;
    __syncthreads();
    if (threadIdx.x < p.tile_r) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kTpabWarps; ++w) v += sums[w][threadIdx.x];     // in warp order: reproducible
        part[(size_t)split * p.out_f + rt * p.tile_r + threadIdx.x] = v;
    }
}

// y[row] = sum over the splits + the row's outliers (bf16(value) * x[column]) (+ bias), rounded once
__global__ void __launch_bounds__(256)
k_tpab_finalize(const float *__restrict__ part, uint32_t splits, uint32_t out_f, const int32_t *__restrict__ ol_offs,
                const int32_t *__restrict__ ol_k, const __half *__restrict__ ol_v, const __nv_bfloat16 *__restrict__ x,
                const __nv_bfloat16 *__restrict__ bias, void *y, int y_f32)
{
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= out_f) return;
    float v = 0.f;
    for (uint32_t k = 0; k < splits; ++k) v += part[(size_t)k * out_f + row];
    if (ol_offs)
        for (int32_t j = ol_offs[row]; j < ol_offs[row + 1]; ++j)
            v = fmaf(bfround_f(__half2float(ol_v[j])), __bfloat162float(x[ol_k[j]]), v);
    if (y_f32) {
        ((float *)y)[row] = bias ? v + __bfloat162float(bias[row]) : v;
    } else {
        __nv_bfloat16 h = __float2bfloat16_rn(v);
        if (bias) h = __hadd(h, bias[row]);
        ((__nv_bfloat16 *)y)[row] = h;
    }
}

}  // namespace ixb
