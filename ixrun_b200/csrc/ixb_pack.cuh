// Device-side quantiser and packer (deploy time): bf16 weight -> int8 codes ->
// the five (3,5,8) streams, bit for bit what the reference's CPU quantiser
// writes (ixrun/quantize.py:41-122, ixrun/bitpack.py:13-61).
#pragma once
#include "ixb_common.cuh"

namespace ixb {

// max |w| over the tensor as bf16 bits (non-negative floats order like their bit patterns)
__global__ void k_absmax(const uint16_t *__restrict__ w, uint32_t n, uint32_t *out_bits)
{
    uint32_t m = 0;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        uint32_t b = w[i] & 0x7fffu;
        if (b <= 0x7f80u) m = max(m, b);          // NaN payloads are ignored
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0) atomicMax(out_bits, m);
}

// scale = bf16(bf16(max(absmax, 1e-8)) / 127), each step rounded like the reference does in bf16
__device__ __forceinline__ __nv_bfloat16 scale_from_absmax(uint32_t absmax_bits)
{
    float mx = __uint_as_float(absmax_bits << 16);
    float cl = mx < 1e-8f ? 1e-8f : mx;
    __nv_bfloat16 cl_b = __float2bfloat16_rn(cl);
    return __float2bfloat16_rn(__fdiv_rn(__bfloat162float(cl_b), 127.0f));
}

__device__ __forceinline__ int code_level(int c)
{
    int a = c < 0 ? -c : c;
    return a <= 3 ? 0 : (a <= 15 ? 1 : 2);
}

// One warp per 1024-element block, lane = 32-element word.  MODE 0: quantise from bf16 weights and write
// codes; MODE 1: read existing codes.  Both write the B1 word and the block's level-1 / level-2 counts.
template <int MODE>
__global__ void __launch_bounds__(256)
k_codes_and_counts(const uint16_t *__restrict__ w, const uint32_t *absmax_bits, int8_t *codes, uint32_t n,
                   uint32_t *b1, int32_t *cnt1, int32_t *cnt2, __nv_bfloat16 *scale_out)
{
    uint32_t nb = (n + kBlk - 1) / kBlk;
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= nb) return;
    float sc = 1.f;
    if (MODE == 0) {
        __nv_bfloat16 s = scale_from_absmax(*absmax_bits);
        sc = __bfloat162float(s);
        if (b == 0 && lane == 0) *scale_out = s;
    }
    uint32_t e0 = (b * 32u + lane) * 32u;
    uint32_t m1 = 0, e2 = 0;
    for (uint32_t i = 0; i < 32u && e0 + i < n; ++i) {
        int c;
        if (MODE == 0) {
            float q = rintf(__fdiv_rn(__uint_as_float((uint32_t)w[e0 + i] << 16), sc));
            q = fminf(fmaxf(q, -127.f), 127.f);
            c = (int)q;
            codes[e0 + i] = (int8_t)c;
        } else {
            c = codes[e0 + i];
        }
        int lv = code_level(c);
        m1 |= (uint32_t)(lv == 0) << i;
        e2 |= (uint32_t)(lv == 1) << i;
    }
    if (e0 < n) b1[b * 32u + lane] = m1;
    uint32_t n1 = __reduce_add_sync(0xffffffffu, __popc(m1));
    uint32_t n2 = __reduce_add_sync(0xffffffffu, __popc(e2));
    if (lane == 0) { cnt1[b] = (int32_t)n1; cnt2[b] = (int32_t)n2; }
}

__device__ __forceinline__ void or_field(uint32_t *stream, uint32_t bit, uint32_t v, uint32_t width)
{
    uint32_t wi = bit >> 5, sh = bit & 31u;
    atomicOr(stream + wi, v << sh);
    if (sh + width > 32u) atomicOr(stream + wi + 1, v >> (32u - sh));
}

// Streams must be zero on entry.  One warp per block, lane = word; every element ORs its own field in.
__global__ void __launch_bounds__(256)
k_pack(const int8_t *__restrict__ codes, uint32_t n, const int32_t *__restrict__ a_blk, const int32_t *__restrict__ c_blk,
       uint32_t *b2, uint32_t *l1, uint32_t *l2, uint8_t *l3)
{
    uint32_t nb = (n + kBlk - 1) / kBlk;
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= nb) return;
    uint32_t e0 = (b * 32u + lane) * 32u;
    uint32_t valid = e0 >= n ? 0u : min(32u, n - e0);
    int c[32];
    uint32_t m1 = 0, e2 = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        c[i] = (uint32_t)i < valid ? (int)codes[e0 + i] : 0;
        int lv = (uint32_t)i < valid ? code_level(c[i]) : 3;
        m1 |= (uint32_t)(lv == 0) << i;
        e2 |= (uint32_t)(lv == 1) << i;
    }
    uint32_t n1 = __popc(m1), n2 = __popc(e2);
    uint32_t a = (uint32_t)a_blk[b] + warp_incl_scan(n1, lane) - n1;
    uint32_t cc = (uint32_t)c_blk[b] + warp_incl_scan(n2, lane) - n2;
    uint32_t r = e0 - a;          // e0 - (#L1 before e0): rank among non-L1 elements
    // a was computed from block-local scans of whole words, so r is exact for every valid lane
    uint32_t t = r - cc;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        if ((uint32_t)i >= valid) break;
        if ((m1 >> i) & 1u) {
            or_field(l1, a * 3u, (uint32_t)(c[i] + 3), 3u);
            ++a;
        } else {
            if ((e2 >> i) & 1u) {
                atomicOr(b2 + (r >> 5), 1u << (r & 31u));
                or_field(l2, cc * 5u, (uint32_t)(c[i] + 15), 5u);
                ++cc;
            } else {
                l3[t++] = (uint8_t)(c[i] + 127);
            }
            ++r;
        }
    }
}

// ---------------------------------------------------------------- sibling format: per-group scales
// The group-scale variant of the format (ixgs/quantize.py:35-112, decode ixgs/kernels.py:31-102 and
// ixgs/quantize.py:116-151) stores the same five (3,5,8) streams (fields offset by -3 / -15 / -127, so the stream
// decoder above serves it unchanged) and one fp16 scale per `group` consecutive elements of the flat tensor instead of
// one per tensor: w[e] = bf16(f32(code[e]) * f32(scale[e / group])).  Eight weights per thread where the shape allows.
__global__ void __launch_bounds__(256)
k_group_scale(const int8_t *__restrict__ codes, const __half *__restrict__ gscale, uint32_t n, uint32_t group,
              __nv_bfloat16 *__restrict__ out)
{
    const uint32_t e0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8u;
    if (e0 >= n) return;
    if (e0 + 8u <= n && (group & 7u) == 0 && (((uintptr_t)codes | (uintptr_t)out) & 15u) == 0) {
        const float sc = __half2float(gscale[e0 / group]);             // eight consecutive elements share a group
        const uint2 c = *(const uint2 *)(codes + e0);
        const uint32_t cw[2] = {c.x, c.y};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int a = (int)(int8_t)((cw[k >> 1] >> (16 * (k & 1))) & 0xff);
            const int b = (int)(int8_t)((cw[k >> 1] >> (16 * (k & 1) + 8)) & 0xff);
            o[k] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn((float)a * sc)) |
                   ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn((float)b * sc)) << 16);
        }
        *(uint4 *)(out + e0) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
        for (uint32_t e = e0; e < min(e0 + 8u, n); ++e)
            out[e] = __float2bfloat16_rn((float)codes[e] * __half2float(gscale[e / group]));
    }
}

}  // namespace ixb
