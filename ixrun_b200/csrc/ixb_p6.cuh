// Resident re-layout "P6" of an INT8-X tensor and the kernels that run on it.
//
// It is built at deploy time, on the GPU, from the int8 codes that the
// reference's (3,5,8) streams decode to (ixrun/quantize.py:80-96), and keeps
// those codes exactly.  Nothing in it is addressed by rank: every 1024-weight
// block (16 rows x 64 columns, one warp) sits at a fixed address, and turning it
// into tensor-core operands costs three instructions per PAIR of weights:
//
//   plane   every element owns a 6-bit field F that is bits 7..2 of the low
//           byte of the bf16 number a = 1 + code / 32:
//             code in [0, 31]    a in [1, 2)    F = 32 + code
//             code in [-16, -1]  a in [0.5, 1)  F = 32 + 2 code
//           so (F << 2) | 0x3F00 IS a, and one fused multiply-add
//           fma(a, 32 s, -32 s) = bf16(code * s) rounds the exact product once:
//           the reference's dequantised weight bf16(f32(code) * f32(scale))
//           (ixrun/quantize.py:182, ixrun/fused.py:169-170), bit for bit, for any scale s.
//           Other codes ("outliers") leave the placeholder F = 32 (weight 0).
//           Blocks of 16 rows x 64 columns, ragged edges padded with
//           placeholders (p6_elem gives the element of lane / pair / half); a
//           lane owns 32 fields in six 32-bit words,
//           a block is 768 contiguous bytes: 32 x uint4 (words 0..3), then
//           32 x uint2 (words 4, 5).  Word k holds pair 2k at bits 0 / 16 and
//           pair 2k+1 at bits 6 / 22 (low / high element); the 4 + 4 spare
//           bits of words 0..3 hold the low four bits of pairs 12..15, those of
//           words 4, 5 their upper two bits (p6_put).
//   esc     the outliers of every block as 32-bit entries
//             bf16(code * s) << 16 | row_in_tile << 12 | (block & 63) << 6 | column_in_block
//           sorted by block; blk_off[nb + 1] gives the first entry of every block.
//           The low 12 bits are a column offset modulo 4096, so a run of up to
//           64 consecutive blocks of one row tile resolves its columns without
//           knowing which block an entry came from.
//
// Size: 6 + 32 * P(outlier) bits per weight + 4 bytes per block (6.4 bpw for
// the benchmark distribution).
//
// y = W x is one kernel (k_p6_mma): per warp a ring of cp.async-staged blocks,
// twelve shift/mask/fma triples and four five-instruction pairs per lane give
// the A fragments of four mma.sync.m16n8k16 (bf16) with the activations as B;
// the outliers of a warp's run of blocks are staged once in shared memory and
// added on the CUDA cores (weight * x into per-row, per-lane sums) per row-tile
// segment of the run, while the ring keeps fetching.  Products are exact, accumulation is fp32, and no
// floating-point atomics are used: results are reproducible.
#pragma once
#include "ixb_common.cuh"

namespace ixb {

constexpr int kTileRows = 16;      // a block: 16 rows x 64 columns = 1024 weights, one warp
constexpr int kTileCols = 64;

// Lane l of a block: g = l >> 2, t = l & 3.  Its 16 pairs p = 4 j + q (j = 0..3 the mma, q = 0..3 the A register):
//   row    = 16 R + g + 8 (q & 1)
//   column = 64 kb + 16 t + 4 j + 2 (q >> 1) + h          (h = 0 low half, 1 high half of the register)
// i.e. the k index of mma j is permuted so that a lane needs the 16 consecutive activations 16 t .. 16 t + 15.
__device__ __forceinline__ void p6_elem(int lane, int p, int h, uint32_t &row_in_tile, uint32_t &col_in_tile)
{
    int g = lane >> 2, t = lane & 3, j = p >> 2, q = p & 3;
    row_in_tile = (uint32_t)(g + 8 * (q & 1));
    col_in_tile = (uint32_t)(16 * t + 4 * j + 2 * (q >> 1) + h);
}
// (SRC & MASK) | ACC
__device__ __forceinline__ uint32_t p6_and_or(uint32_t src, uint32_t mask, uint32_t acc)
{
    uint32_t v;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(src), "r"(mask), "r"(acc));
    return v;
}
__device__ __forceinline__ void p6_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kP6BlockBytes = 768;
constexpr int kP6Slots = 4;                       // ring slots per warp; blocks are fetched three ahead
constexpr int kP6SlackBlocks = 5;                 // readable blocks behind the plane (the ring fetches past a run end)
constexpr int kP6SlackEntries = 64;               // readable entries behind the outlier list
constexpr int kP6CodeMin = -16, kP6CodeMax = 31;  // codes that the plane holds

struct P6 {
    const unsigned char *plane;  // [(nb + slack) * 768]
    const int32_t *blk_off;      // [nb + 1] first outlier entry of every block
    const uint32_t *esc;         // [n_esc + slack] outlier entries
    const __nv_bfloat16 *scale;  // scale_stride 0: one scale; 1: one per row tile (a tensor fused from several)
    uint32_t out_f, in_f;
    uint32_t rt, kb;             // row tiles, column blocks per row tile; nb = rt * kb
    uint32_t scale_stride;
};

__host__ __device__ __forceinline__ uint32_t p6_field(int code) { return (uint32_t)(code >= 0 ? 32 + code : 32 + 2 * code); }
__host__ __device__ __forceinline__ int p6_code(uint32_t f) { return f >= 32u ? (int)f - 32 : ((int)f - 32) / 2; }

__device__ __forceinline__ void p6_put(uint32_t (&w)[6], int p, int h, uint32_t f)
{
    if (p < 12) {
        w[p >> 1] |= f << (6 * (p & 1) + 16 * h);
    } else {
        const int i = p - 12;
        w[i] |= (f & 15u) << (12 + 16 * h);
        w[4 + (i >> 1)] |= (f >> 4) << (12 + 2 * (i & 1) + 16 * h);
    }
}

__device__ __forceinline__ uint32_t p6_get(const uint32_t (&w)[6], int p, int h)
{
    if (p < 12) return (w[p >> 1] >> (6 * (p & 1) + 16 * h)) & 63u;
    const int i = p - 12;
    return ((w[i] >> (12 + 16 * h)) & 15u) | (((w[4 + (i >> 1)] >> (12 + 2 * (i & 1) + 16 * h)) & 3u) << 4);
}

// ------------------------------------------------------------------ build ---
// codes [out_f, in_f] -> plane blocks and the number of outliers of every block (one warp per block)
__global__ void __launch_bounds__(256)
k_p6_plane(const int8_t *__restrict__ codes, uint32_t out_f, uint32_t in_f, uint32_t rt, uint32_t kb,
           unsigned char *plane, int32_t *blk_cnt)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= rt * kb) return;
    uint32_t R = b / kb, kbi = b - R * kb;
    uint32_t w[6] = {0, 0, 0, 0, 0, 0};
    uint32_t n_out = 0;
#pragma unroll
    for (int p = 0; p < 16; ++p) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t r, c;
            p6_elem(lane, p, h, r, c);
            uint32_t row = R * kTileRows + r, col = kbi * kTileCols + c;
            int code = (row < out_f && col < in_f) ? (int)codes[(size_t)row * in_f + col] : 0;
            bool out = code > kP6CodeMax || code < kP6CodeMin;
            n_out += out;
            p6_put(w, p, h, p6_field(out ? 0 : code));
        }
    }
    unsigned char *blk = plane + (size_t)b * kP6BlockBytes;
    ((uint4 *)blk)[lane] = make_uint4(w[0], w[1], w[2], w[3]);
    ((uint2 *)(blk + 512))[lane] = make_uint2(w[4], w[5]);
    n_out = warp_incl_scan(n_out, lane);
    if (lane == 31) blk_cnt[b] = (int32_t)n_out;
}

// outlier entries of every block, in (lane, pair, half) order (one warp per block)
__global__ void __launch_bounds__(256)
k_p6_esc(const int8_t *__restrict__ codes, uint32_t out_f, uint32_t in_f, uint32_t rt, uint32_t kb,
         const int32_t *__restrict__ blk_off, const __nv_bfloat16 *__restrict__ scale, uint32_t scale_stride, uint32_t *esc,
         uint32_t n_esc)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= rt * kb) return;
    uint32_t R = b / kb, kbi = b - R * kb;
    float sc = __bfloat162float(scale[R * scale_stride]);
    int code[32];
    uint32_t n_out = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        uint32_t r, c;
        p6_elem(lane, i >> 1, i & 1, r, c);
        uint32_t row = R * kTileRows + r, col = kbi * kTileCols + c;
        code[i] = (row < out_f && col < in_f) ? (int)codes[(size_t)row * in_f + col] : 0;
        n_out += (code[i] > kP6CodeMax || code[i] < kP6CodeMin);
    }
    uint32_t at = (uint32_t)blk_off[b] + warp_incl_scan(n_out, lane) - n_out;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        if (code[i] > kP6CodeMax || code[i] < kP6CodeMin) {
            uint32_t r, c;
            p6_elem(lane, i >> 1, i & 1, r, c);
            uint32_t wbits = __bfloat16_as_ushort(__float2bfloat16_rn((float)code[i] * sc));
            if (at < n_esc) esc[at] = (wbits << 16) | (r << 12) | ((b & 63u) << 6) | c;   // never beyond the caller's buffer
            ++at;
        }
    }
}

// ---------------------------------------------------------------- decode ----
// plane -> int8 codes (OUT 0) or bf16 weights (OUT 1), row major [out_f, in_f]; outliers come out as 0 here.
// A lane holds 16 consecutive columns of two rows: one or two 16-byte stores per row.
template <int OUT>
__global__ void __launch_bounds__(256) k_p6_decode_plane(P6 p, void *out)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= p.rt * p.kb) return;
    uint32_t R = b / p.kb, kbi = b - R * p.kb;
    float sc = __bfloat162float(p.scale[R * p.scale_stride]);
    const unsigned char *blk = p.plane + (size_t)b * kP6BlockBytes;
    const uint4 a = ((const uint4 *)blk)[lane];
    const uint2 a2 = ((const uint2 *)(blk + 512))[lane];
    uint32_t w[6] = {a.x, a.y, a.z, a.w, a2.x, a2.y};
    const bool vec = (OUT == 0 ? (p.in_f & 15u) == 0 : (p.in_f & 7u) == 0) && ((uintptr_t)out & 15u) == 0;
#pragma unroll
    for (int s = 0; s < 2; ++s) {                    // row g, row g + 8
        uint32_t row = R * kTileRows + (lane >> 2) + 8 * s, col0 = kbi * kTileCols + 16 * (lane & 3);
        if (row >= p.out_f || col0 >= p.in_f) continue;
        uint32_t r[OUT == 0 ? 4 : 8];
#pragma unroll
        for (int i = 0; i < (OUT == 0 ? 4 : 8); ++i) r[i] = 0;
#pragma unroll
        for (int c = 0; c < 16; ++c) {               // column col0 + c = pair 4 (c >> 2) + 2 ((c >> 1) & 1) + s, half c & 1
            int code = p6_code(p6_get(w, 4 * (c >> 2) + 2 * ((c >> 1) & 1) + s, c & 1));
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

// The outliers overwrite their placeholders (launched after k_p6_decode_plane on the same stream; one warp per
// block).  An entry carries the bf16 weight w = bf16(code * scale); the code is recovered from it exactly:
// neighbouring codes differ by scale >= |code * scale| / 127, more than one bf16 ulp (2^-7 relative), so no two
// codes share a weight and w / scale is within 0.25 of the code.
template <int OUT>
__global__ void __launch_bounds__(256) k_p6_decode_esc(P6 p, void *out)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= p.rt * p.kb) return;
    uint32_t R = b / p.kb, kbi = b - R * p.kb;
    float sc = __bfloat162float(p.scale[R * p.scale_stride]);
    for (int32_t j = p.blk_off[b] + lane; j < p.blk_off[b + 1]; j += 32) {
        uint32_t ent = p.esc[j];
        uint32_t row = R * kTileRows + ((ent >> 12) & 15u), col = kbi * kTileCols + (ent & 63u);
        if (row >= p.out_f || col >= p.in_f) continue;
        size_t o = (size_t)row * p.in_f + col;
        __nv_bfloat16 wv = __ushort_as_bfloat16((unsigned short)(ent >> 16));
        if (OUT == 1) ((__nv_bfloat16 *)out)[o] = wv;
        else ((int8_t *)out)[o] = (int8_t)__float2int_rn(__bfloat162float(wv) / sc);
    }
}

// ------------------------------------------------------------------ GEMV ----
constexpr int kP6Threads = 768;
constexpr int kP6Warps = kP6Threads / 32;
constexpr int kP6StageEntries = 512;                                  // outlier entries a warp stages in shared memory
constexpr int kP6RingBytes = kP6Slots * kP6BlockBytes;                // 3072
// per warp: ring, per-row outlier sums [16][32] fp32, staged entries, two partial tiles [2][32] float4
constexpr int kP6WarpSmem = kP6RingBytes + 16 * 32 * 4 + kP6StageEntries * 4 + 2 * 32 * 16;
constexpr int kP6TailTiles = 32;                                      // row tiles per CTA that the barrier-free tail tracks
constexpr int kP6TailBytes = kP6TailTiles * 12;                       // per tile: arrival counter + two words of plan
constexpr int kP6SmemFixed = kP6Warps * kP6WarpSmem + kP6TailBytes;
static_assert(kP6WarpSmem % 128 == 0, "per-warp shared memory keeps 128-byte alignment");

__device__ __forceinline__ void p6_cp16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// the same copy for the lanes with `on` set (a predicate, not a branch: the warp stays converged)
__device__ __forceinline__ void p6_cp16_if(uint32_t dst, const void *src, bool on)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p cp.async.cg.shared.global [%0], [%1], 16;\n\t}"
                 ::"r"(dst), "l"(src), "r"((uint32_t)on) : "memory");
}
__device__ __forceinline__ uint4 p6_lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint2 p6_lds64(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
    return v;
}
// two fields at bits 7..2 / 23..18 of t -> the two bf16 numbers a = 1 + code / 32 -> the two weights
__device__ __forceinline__ uint32_t p6_pair(uint32_t t, uint32_t e2, uint32_t b2, uint32_t c2)
{
    uint32_t v, w;
    asm("lop3.b32 %0, %1, 0x00FC00FC, %2, 0xEA;" : "=r"(v) : "r"(t), "r"(e2));
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(w) : "r"(v), "r"(b2), "r"(c2));
    return w;
}

// Where the outputs of a row-parallel shard go instead of y: into this rank's slot of EVERY rank's all-reduce buffer
// (see ixb_allreduce.cuh: slots [2 parities][world][n_max] of {fp32 value, call number} words), as plain peer stores
// straight from the GEMV's epilogue.  world == 0: no push, the outputs are written to y.
struct P6Push {
    uint2 *slots[8];              // every rank's slots, as seen from this rank
    const uint2 *mine;            // this rank's own slots (slots[rank])
    uint32_t *epoch;              // this rank's call counters (whoever finishes the exchange advances them)
    uint32_t world, rank, n_max;
    // fin != 0: the GEMV also finishes the exchange itself.  When a warp is done with its blocks it takes its share
    // of the outputs, waits (bounded) for every rank's words of this call in this rank's own buffer, adds them in
    // rank order (+ bias) and writes y; the last warp of the grid to get there advances the call counters.
    uint32_t fin, counters, spin_limit;
    uint32_t *err;                // the buffer's error word
    uint32_t *done;               // scratch word counting finished warps, zero between launches
};

// one output (activation row m, weight row `row`): to y (+ bias), or as a marked word to every rank
__device__ __forceinline__ void p6_put_out(const P6Push &push, uint32_t e, uint32_t out_f, uint32_t m, uint32_t row, float v,
                                           const __nv_bfloat16 *__restrict__ bias, void *y, int y_f32)
{
    const size_t o = (size_t)m * out_f + row;
    if (push.world) {
        const size_t at = ((size_t)((e & 1u) * push.world + push.rank)) * push.n_max + o;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if ((uint32_t)r >= push.world) break;
            asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(push.slots[r] + at), "r"(__float_as_uint(v)), "r"(e) : "memory");
        }
    } else if (y_f32) {
        ((float *)y)[o] = bias ? v + __bfloat162float(bias[row]) : v;
    } else {
        __nv_bfloat16 hv = __float2bfloat16_rn(v);
        if (bias) hv = __hadd(hv, bias[row]);
        ((__nv_bfloat16 *)y)[o] = hv;
    }
}

__device__ __forceinline__ void p6_store_tile(const P6Push &push, uint32_t e, uint32_t out_f, uint32_t R, int lane,
                                              const float (&c)[4], uint32_t m_rows, const __nv_bfloat16 *__restrict__ bias,
                                              void *y, int y_f32)
{
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t m = 2u * t + (i & 1), row = R * kTileRows + g + 8 * (i >> 1);
        if (m >= m_rows || row >= out_f) continue;
        p6_put_out(push, e, out_f, m, row, c[i], bias, y, y_f32);
    }
}

// one half of a lane's C fragment: row g + 8 h of the tile, activation rows 2 t and 2 t + 1
__device__ __forceinline__ void p6_store_pair(const P6Push &push, uint32_t e, uint32_t out_f, uint32_t R, int lane, int h,
                                              const float (&v)[2], uint32_t m_rows, const __nv_bfloat16 *__restrict__ bias,
                                              void *y, int y_f32)
{
    const int g = lane >> 2, t = lane & 3;
    const uint32_t row = R * kTileRows + g + 8 * h;
    if (row >= out_f) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint32_t m = 2u * t + i;
        if (m >= m_rows) continue;
        p6_put_out(push, e, out_f, m, row, v[i], bias, y, y_f32);
    }
}

// n elements cut into `parts` contiguous parts, the first r = n % parts of them one longer than q = n / parts:
// first element of part i, and the part that holds element pos (no 64-bit arithmetic, no division on the way in)
__device__ __forceinline__ uint32_t p6_begin(uint32_t i, uint32_t q, uint32_t r) { return i * q + min(i, r); }
__device__ __forceinline__ uint32_t p6_part_of(uint32_t pos, uint32_t q, uint32_t r)
{
    const uint32_t big = r * (q + 1u);
    return pos < big ? pos / (q + 1u) : r + (pos - big) / q;      // q > 0 whenever pos >= big
}

// layout -> bf16 weights in one pass, with the GEMV's own conversion (shift, mask, one fma per pair of elements): the
// block's outliers are dropped into a zeroed image of the lanes' registers in shared memory first and OR-ed over the
// placeholders (+0.0), so every weight is stored once, in 16-byte pieces; needs in_f % 8 == 0 and a 16-byte aligned
// output.  One warp per block.
__global__ void __launch_bounds__(256) k_p6_decode_bf16(P6 p, __nv_bfloat16 *out)
{
    __shared__ uint4 images[8 * 128];                // per warp: [4 mma][32 lanes] the lane's four A registers
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
            const uint32_t e = __ldg(p.esc + j);
            // element (row r, column c) of the block sits in lane 4 (r & 7) + (c >> 4), pair 4 ((c >> 2) & 3) +
            // 2 ((c >> 1) & 1) + (r >> 3), half c & 1 (the inverse of p6_elem)
            const uint32_t r = (e >> 12) & 15u, c = e & 63u;
            const uint32_t ln = 4u * (r & 7u) + (c >> 4), j4 = (c >> 2) & 3u, q = 2u * ((c >> 1) & 1u) + (r >> 3);
            const uint32_t off = ((j4 * 32u + ln) * 4u + q) * 4u + 2u * (c & 1u);
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(img_s + off), "h"((unsigned short)(e >> 16)) : "memory");
        }
    }
    __syncwarp();
    uint32_t R = b / p.kb, kbi = b - R * p.kb;
    const float s32 = 32.f * __bfloat162float(p.scale[R * p.scale_stride]);
    const uint32_t bb = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(s32));
    const uint32_t b2 = bb | (bb << 16), c2 = b2 ^ 0x80008000u, e2 = 0x3F003F00u;
    const unsigned char *blk = p.plane + (size_t)b * kP6BlockBytes;
    const uint4 a = ((const uint4 *)blk)[lane];
    const uint2 a2 = ((const uint2 *)(blk + 512))[lane];
    const uint32_t w[6] = {a.x, a.y, a.z, a.w, a2.x, a2.y};
    uint32_t f[16];
#pragma unroll
    for (int k = 0; k < 6; ++k) {
        f[2 * k] = p6_pair(w[k] << 2, e2, b2, c2);
        f[2 * k + 1] = p6_pair(w[k] >> 4, e2, b2, c2);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t v = p6_and_or(w[i] >> 10, 0x003C003Cu, e2);
        v = p6_and_or(w[4 + (i >> 1)] >> (6 + 2 * (i & 1)), 0x00C000C0u, v);
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(f[12 + i]) : "r"(v), "r"(b2), "r"(c2));
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {                    // placeholders are +0.0, so OR-ing the outlier weights in is exact
        const uint4 v = img[q * 32 + lane];
        f[4 * q] |= v.x;
        f[4 * q + 1] |= v.y;
        f[4 * q + 2] |= v.z;
        f[4 * q + 3] |= v.w;
    }
    // pair 4 j + q: row g + 8 (q & 1), columns 4 j + 2 (q >> 1) + {0, 1} of the lane's 16
    const uint32_t col0 = kbi * kTileCols + 16 * (lane & 3);
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        uint32_t row = R * kTileRows + (lane >> 2) + 8 * s;
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

// The nb blocks, in (row tile, column block) order, are cut into gridDim.x contiguous CTA ranges and every CTA range
// into kP6Warps runs.  The CTA ranges are counted in units of `unit` blocks (cq, cr = units / and % gridDim.x):
// unit = 1 balances the CTAs to one block, and row tiles at range boundaries are finished across CTAs; unit = blocks
// per row tile gives every CTA whole row tiles, so nothing crosses CTAs (the host picks the cheaper of the two).  A run is walked segment by segment (its part of one row
// tile): the segment's outliers are added first, from the entries staged in shared memory, then its blocks stream
// through the warp's cp.async ring.  Row tiles that a run covers completely are written straight to y; partial
// tiles are summed per CTA in warp order; a tile shared between CTAs goes through cta_slots and a ticket, the
// last arriver sums the slots in CTA order and clears them.  tickets[] (gridDim.x + 1 words) and cta_slots must be
// zero before the first launch and are left zero, so one scratch buffer serves launches of any shape in turn.  XS = 1: activations staged in shared memory (bf16, padded rows); XS = 0: read from
// global memory.

template <int XS>
__global__ void __launch_bounds__(kP6Threads, 1)
k_p6_mma(P6 p, const __nv_bfloat16 *__restrict__ x, uint32_t m_rows, const __nv_bfloat16 *__restrict__ bias, void *y,
         int y_f32, float4 *cta_slots, uint32_t *tickets, uint32_t nb, uint32_t xstride, uint32_t cq, uint32_t cr, uint32_t unit,
         P6Push push)
{
    extern __shared__ __align__(128) unsigned char p6_smem[];
    __nv_bfloat16 *xs = (__nv_bfloat16 *)(p6_smem + kP6SmemFixed);                       // [m_rows][xstride]

    const int lane = threadIdx.x & 31;
    const int wid = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);   // the same in every lane, and known to be
    const int g = lane >> 2, t = lane & 3;
    const uint32_t KB = p.kb;
    unsigned char *wsm = p6_smem + wid * kP6WarpSmem;
    float *oacc = (float *)(wsm + kP6RingBytes);                       // [16 rows][32 lanes] outlier sums, zero between passes
    uint32_t *estage = (uint32_t *)(wsm + kP6RingBytes + 2048);        // the run's first kP6StageEntries outlier entries
    float4 *wparts = (float4 *)(wsm + kP6RingBytes + 4096);            // partial sums of the run's first / last row tile

    const uint32_t cb0 = p6_begin(blockIdx.x, cq, cr) * unit, cb1 = p6_begin(blockIdx.x + 1, cq, cr) * unit;
    const uint32_t L = cb1 - cb0, wq = L / kP6Warps, wr = L - wq * kP6Warps;
    const uint32_t b_begin = cb0 + p6_begin(wid, wq, wr), b_end = cb0 + p6_begin(wid + 1, wq, wr);
    const bool active = b_begin < b_end;
    // ---- plan of the tail, made while nothing else can run yet.  For every row tile R0 + i that this CTA touches
    // (fast path: at most kP6TailTiles): which warps' runs meet it, whether it lies inside the CTA's range, how many
    // partial sums will arrive (0: one run covers it and writes y itself), and the CTAs that share it.
    uint32_t *tcnt = (uint32_t *)(p6_smem + kP6Warps * kP6WarpSmem);   // [kP6TailTiles] arrivals
    uint32_t *tplan = tcnt + kP6TailTiles;                             // [kP6TailTiles][2]
    const uint32_t Rc0 = cb0 / KB, Rc1 = L ? (cb1 - 1u) / KB : Rc0;
    const bool fast_tail = L != 0 && Rc1 - Rc0 < (uint32_t)kP6TailTiles;
    if (fast_tail && lane == 0) {
        for (uint32_t i = wid; i <= Rc1 - Rc0; i += kP6Warps) {
            const uint32_t t0 = (Rc0 + i) * KB, t1 = t0 + KB;
            const uint32_t inside = t0 >= cb0 && t1 <= cb1;
            const uint32_t wlo = p6_part_of(max(t0, cb0) - cb0, wq, wr), whi = p6_part_of(min(t1, cb1) - 1 - cb0, wq, wr);
            const uint32_t need = inside && wlo == whi ? 0u : whi - wlo + 1u;
            uint32_t clo = 0, span = 0;
            if (!inside) {
                clo = p6_part_of(t0, cq, cr);
                span = p6_part_of(t1 - 1u, cq, cr) - clo;
            }
            tcnt[i] = 0;
            tplan[2 * i] = wlo | whi << 8 | need << 16 | inside << 24;
            tplan[2 * i + 1] = clo | span << 16;
        }
    }
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(wsm);
    const uint32_t d16 = ring_s + lane * 16;
    const unsigned char *n16 = p.plane + (size_t)b_begin * kP6BlockBytes + lane * 16;    // this lane's next chunk to fetch
    uint32_t pf_left = b_end - b_begin;                                                  // blocks of the run not yet requested

    // Everything up to griddepcontrol.wait reads only the layer's own (constant) buffers.  When the launch carries
    // the programmatic-stream-serialization attribute this part overlaps the tail of the kernel before it in the
    // stream; without the attribute the two griddepcontrol instructions do nothing.
    asm volatile("griddepcontrol.launch_dependents;");
    // ---- copy group A: the run's first three blocks and the activations
    int32_t j_begin = 0, j_end = 0;
    if (active) {
        j_begin = __ldg(p.blk_off + b_begin);
        j_end = __ldg(p.blk_off + b_end);
#pragma unroll
        for (int s = 0; s < 3; ++s) {
            const bool more = pf_left != 0;               // nothing is fetched past the end of the run
            p6_cp16_if(d16 + s * kP6BlockBytes, n16, more);
            p6_cp16_if(d16 + s * kP6BlockBytes + 512, n16 + 512, more && lane < 16);
            n16 += kP6BlockBytes;
            pf_left -= more ? 1u : 0u;
        }
#pragma unroll
        for (int r = 0; r < 16; ++r) oacc[r * 32 + lane] = 0.f;
    }
    // the scale of the run's first row tile and of the one after it (a fused tensor has one per row tile); the
    // walk below always holds the next tile's scale one segment ahead, so the load is never waited for
    uint32_t e2, b2 = 0, c2 = 0;
    uint32_t sc_cur = 0, sc_next = 0;
    {
        if (p.scale_stride) {                                          // (uniform) a fused tensor: one scale per row tile
            const uint32_t R0 = min(b_begin / KB, p.rt - 1u);
            sc_cur = (uint32_t)__bfloat16_as_ushort(p.scale[R0]);
            sc_next = (uint32_t)__bfloat16_as_ushort(p.scale[min(R0 + 1u, p.rt - 1u)]);
        } else {
            sc_cur = (uint32_t)__bfloat16_as_ushort(p.scale[0]);
        }
        asm volatile("mov.b32 %0, 0x3F003F00;" : "=r"(e2));            // opaque, so that it stays a register operand
    }
    auto set_scale = [&](uint32_t bits) {
        const float s32 = 32.f * __uint_as_float(bits << 16);
        const uint32_t bb = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(s32));    // exact: a power-of-two multiple
        b2 = bb | (bb << 16);
        c2 = b2 ^ 0x80008000u;
    };
    set_scale(sc_cur);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // a pushing launch marks its words with the number of this all-reduce call: one more than the counter that the
    // finishing kernel of the call before left (that kernel is complete: it is ahead of this one in the stream)
    const uint32_t push_e = push.world ? __ldcg(push.epoch) + 1u : 0u;
    if (XS) {
        // whole 16-byte chunks by cp.async; ragged ends are written with plain stores
        const uint32_t chunks = KB * (kTileCols / 8);
        const uint32_t xs_s = (uint32_t)__cvta_generic_to_shared(xs);
        const bool vec = (p.in_f & 7u) == 0;
        for (uint32_t m = 0; m < m_rows; ++m) {
            for (uint32_t k8 = threadIdx.x * 8u; k8 < chunks * 8u; k8 += kP6Threads * 8u) {
                if (vec && k8 + 8u <= p.in_f) {
                    p6_cp16(xs_s + (m * xstride + k8) * 2u, x + (size_t)m * p.in_f + k8);
                } else {
                    unsigned short e[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        e[j] = k8 + j < p.in_f ? __bfloat16_as_ushort(x[(size_t)m * p.in_f + k8 + j]) : (unsigned short)0;
                    *(uint4 *)(xs + (size_t)m * xstride + k8) =
                        make_uint4(e[0] | ((uint32_t)e[1] << 16), e[2] | ((uint32_t)e[3] << 16), e[4] | ((uint32_t)e[5] << 16),
                                   e[6] | ((uint32_t)e[7] << 16));
                }
            }
        }
    }
    cp_async_commit();
    // ---- copy group E: the run's outlier entries, from the 16-byte boundary at or below the first one (their
    // offsets were requested at the top).  From here on every block iteration adds exactly one group, so the
    // entries are complete once three block iterations have waited.
    const int32_t j_base = j_begin & ~3;
    if (active) {
        const uint32_t es = (uint32_t)__cvta_generic_to_shared(estage);
#pragma unroll
        for (int q = 0; q < kP6StageEntries / 128; ++q) {
            const int32_t ch = j_base + (q * 32 + lane) * 4;
            if (ch < j_end) p6_cp16(es + (q * 32 + lane) * 16, p.esc + ch);
        }
    }
    cp_async_commit();
    cp_async_wait<1>();                              // group A has landed for this thread
    __syncthreads();                                 // ... and for the CTA

    // Row tile R is complete in this CTA: sum the partial tiles of warps wlo .. whi in warp order; a tile inside the
    // CTA's range is written to y, a tile shared with other CTAs (clo .. clo + span) is finished across them.
    auto finish_tile = [&](uint32_t R, uint32_t wlo, uint32_t whi, bool inside, uint32_t clo, uint32_t span) {
        const uint32_t t0 = R * KB;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t w = wlo; w <= whi; ++w) {
            const uint32_t wb = p6_begin(w, wq, wr);
            if (wb == p6_begin(w + 1, wq, wr)) continue;                // a warp without blocks
            // the run of warp w meets tile R: R is its first tile unless the run began in the tile before
            const float4 v = ((const float4 *)(p6_smem + w * kP6WarpSmem + kP6RingBytes + 4096))[(cb0 + wb >= t0 ? 0 : 32) + lane];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        if (inside) {
            const float cc[4] = {s.x, s.y, s.z, s.w};
            p6_store_tile(push, push_e, p.out_f, R, lane, cc, m_rows, bias, y, y_f32);
            return;
        }
        const uint32_t chi = clo + span;
        if (span == 1u) {
            // Shared by exactly two CTAs (the usual case): one atomic exchange per 64-bit word carries the
            // partial sums themselves -- no slot store, fence, ticket and slot load, a single round trip to L2.
            // A lane swaps its two words (row g: c[0], c[1]; row g + 8: c[2], c[3]), XOR-ed with a constant so
            // that a deposit is never the all-zero "empty" word, into the tile's area.  Whoever finds the
            // other CTA's deposit adds it to its own values (a + b = b + a bit for bit, so it does not matter
            // which of the two that is, word by word), stores the outputs and empties the word again.
            unsigned long long *w2 = (unsigned long long *)(cta_slots + ((size_t)chi * 2) * 32 + lane);
            const unsigned long long K = 0x7FC0DEAD7FC0DEADull;
            const float mine[4] = {s.x, s.y, s.z, s.w};
            unsigned long long got[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const unsigned long long dep =
                    ((unsigned long long)__float_as_uint(mine[2 * h + 1]) << 32 | __float_as_uint(mine[2 * h])) ^ K;
                got[h] = atomicExch(w2 + h, dep);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (got[h] == 0ull) continue;                            // first to arrive for this word
                const unsigned long long o = got[h] ^ K;
                const float v[2] = {mine[2 * h] + __uint_as_float((uint32_t)o),
                                    mine[2 * h + 1] + __uint_as_float((uint32_t)(o >> 32))};
                p6_store_pair(push, push_e, p.out_f, R, lane, h, v, m_rows, bias, y, y_f32);
                w2[h] = 0ull;
            }
            return;
        }
        // shared by three or more CTAs: publish this CTA's sum, take a ticket; the last one finishes the tile
        cta_slots[((size_t)blockIdx.x * 2 + (R == Rc0 ? 0 : 1)) * 32 + lane] = s;
        __threadfence();
        __syncwarp();
        uint32_t prev = 0;
        if (lane == 0) prev = atomicAdd(tickets + clo + 1, 1u);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev != span) return;
        // the other CTAs' slots were fenced before their tickets; they are read from L2 (ld.global.cg), which
        // every SM shares, so nothing cached on this SM can be stale
        float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t cc = clo; cc <= chi; ++cc) {
            float4 *sl = cta_slots + ((size_t)cc * 2 + (p6_begin(cc, cq, cr) >= t0 ? 0 : 1)) * 32 + lane;
            z.x += __ldcg(&sl->x); z.y += __ldcg(&sl->y); z.z += __ldcg(&sl->z); z.w += __ldcg(&sl->w);
            // the slot goes back to zero: a later launch of another shape uses the same words for its two-CTA
            // hand-over, where any non-zero word counts as a deposit
            __stcg(sl, make_float4(0.f, 0.f, 0.f, 0.f));
        }
        const float cc4[4] = {z.x, z.y, z.z, z.w};
        p6_store_tile(push, push_e, p.out_f, R, lane, cc4, m_rows, bias, y, y_f32);
        if (lane == 0) tickets[clo + 1] = 0;
    };
    // Fast tail: a warp that leaves a partial row tile behind counts itself in; the warp that completes the count
    // finishes the tile at once -- no CTA-wide barrier, nobody waits for an unrelated slow warp.
    auto tile_arrive = [&](uint32_t R) {
        const uint32_t i = R - Rc0;
        __syncwarp();                                                    // all lanes' parts are written
        uint32_t prev = 0;
        if (lane == 0) {
            __threadfence_block();
            prev = atomicAdd(tcnt + i, 1u);
        }
        prev = __shfl_sync(0xffffffffu, prev, 0);
        const uint32_t w0 = tplan[2 * i], w1 = tplan[2 * i + 1];
        if (prev + 1u != ((w0 >> 16) & 0xffu)) return;
        __threadfence_block();
        finish_tile(R, w0 & 0xffu, (w0 >> 8) & 0xffu, (w0 >> 24) & 1u, w1 & 0xffffu, w1 >> 16);
    };

    if (active) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t R = b_begin / KB;
        const uint32_t R_first = R;
        // this lane's activations: row min(g, m_rows - 1) (rows beyond m_rows only feed unused C columns)
        const uint32_t xrow = min((uint32_t)g, m_rows - 1u);
        const __nv_bfloat16 *xg = x + (size_t)xrow * p.in_f + 16 * t;                                  // XS = 0
        const uint32_t xs_l = (uint32_t)__cvta_generic_to_shared(xs) + (xrow * xstride + 16 * t) * 2u;   // XS = 1
        uint32_t cs = 0, is = 3 * kP6BlockBytes;     // byte offsets of the ring slot to consume next / to refill next
        const uint32_t d8 = ring_s + 512 + lane * 8;
        const bool lo16 = lane < 16;
        float c1[4] = {0.f, 0.f, 0.f, 0.f};          // second accumulator set: two independent mma chains per block

        // blocks [b0, b1) of row tile R: fetch block b + 3 into the slot consumed last, take block b from its slot
        auto run = [&](uint32_t b0, uint32_t b1) {
            uint32_t xo = (b0 - R * KB) * (kTileCols * 2u);     // byte offset into the activation row
            for (uint32_t n = b1 - b0; n != 0; --n) {
                const bool more = pf_left != 0;                   // the last three iterations of a run fetch nothing
                p6_cp16_if(d16 + is, n16, more);
                p6_cp16_if(d16 + is + 512, n16 + 512, more && lo16);
                cp_async_commit();
                n16 += kP6BlockBytes;
                pf_left -= more ? 1u : 0u;
                cp_async_wait<3>();                               // this lane's chunks of the block have landed ...
                __syncwarp();                                     // ... and so have the other lanes'
                const uint4 a = p6_lds128(d16 + cs);
                const uint2 a2 = p6_lds64(d8 + cs);
                uint4 x0, x1;
                if (XS) {
                    x0 = p6_lds128(xs_l + xo);
                    x1 = p6_lds128(xs_l + xo + 16u);
                } else {
                    x0 = *(const uint4 *)((const char *)xg + xo);
                    x1 = *(const uint4 *)((const char *)xg + xo + 16);
                }
                uint32_t f[16];
                {
                    const uint32_t w[6] = {a.x, a.y, a.z, a.w, a2.x, a2.y};
#pragma unroll
                    for (int k = 0; k < 6; ++k) {
                        f[2 * k] = p6_pair(w[k] << 2, e2, b2, c2);
                        f[2 * k + 1] = p6_pair(w[k] >> 4, e2, b2, c2);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t v = p6_and_or(w[i] >> 10, 0x003C003Cu, e2);
                        v = p6_and_or(w[4 + (i >> 1)] >> (6 + 2 * (i & 1)), 0x00C000C0u, v);
                        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(f[12 + i]) : "r"(v), "r"(b2), "r"(c2));
                    }
                }
                p6_mma(c, f[0], f[1], f[2], f[3], x0.x, x0.y);
                p6_mma(c1, f[4], f[5], f[6], f[7], x0.z, x0.w);
                p6_mma(c, f[8], f[9], f[10], f[11], x1.x, x1.y);
                p6_mma(c1, f[12], f[13], f[14], f[15], x1.z, x1.w);
                is = cs;
                cs = cs == (uint32_t)(3 * kP6BlockBytes) ? 0u : cs + (uint32_t)kP6BlockBytes;
                xo += kTileCols * 2u;
            }
        };

        // Outliers of blocks [sb, sb + 64) at most, all in row tile R: entries [jlo, jhi).  Every lane multiplies
        // its entries' weights with their activations into oacc[row][lane]; the rows are then summed across the
        // lanes in a fixed order and added to the C fragment (row g -> c[0], c[1]; row g + 8 -> c[2], c[3]).
        auto outlier_pass = [&](uint32_t sb, int32_t jlo, int32_t jhi) {
            if (jlo >= jhi) return;                                       // warp uniform
            const uint32_t s64 = (sb & 63u) << 6, xcol0 = (sb - R * KB) * kTileCols;
            for (uint32_t m = 0; m < m_rows; ++m) {
                const __nv_bfloat16 *xm = (XS ? xs + (size_t)m * xstride : x + (size_t)m * p.in_f) + xcol0;
                for (int32_t j = jlo + lane; j < jhi; j += 32) {
                    const uint32_t rel = (uint32_t)(j - j_base);
                    const uint32_t e = rel < (uint32_t)kP6StageEntries ? estage[rel] : __ldg(p.esc + j);
                    const uint32_t idx = ((e & 0xFFFu) - s64) & 0xFFFu;   // column relative to block sb
                    const float xv = __uint_as_float((uint32_t)__bfloat16_as_ushort(xm[idx]) << 16);
                    const float wv = __uint_as_float(e & 0xFFFF0000u);
                    float *a = oacc + ((e >> 12) & 15u) * 32u + lane;
                    *a = fmaf(wv, xv, *a);
                }
                __syncwarp();
                const uint32_t row = lane & 15, half = lane >> 4;
                float v[16];
#pragma unroll
                for (int jj = 0; jj < 16; ++jj)                           // conflict free: rows rotate through the banks
                    v[jj] = oacc[row * 32u + half * 16u + ((jj + row) & 15u)];
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) oacc[row * 32u + half * 16u + ((jj + row) & 15u)] = 0.f;
                float s = 0.f;
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) s += v[jj];
                s += __shfl_xor_sync(0xffffffffu, s, 16);
                const float v0 = __shfl_sync(0xffffffffu, s, g), v1 = __shfl_sync(0xffffffffu, s, g + 8);
                if ((uint32_t)t == (m >> 1)) {
                    if (m & 1u) { c[1] += v0; c[3] += v1; }
                    else { c[0] += v0; c[2] += v1; }
                }
                __syncwarp();
            }
        };

        uint32_t b = b_begin;
        int32_t seg_j = j_begin;
        bool first = true;
        while (b < b_end) {
            const uint32_t seg_e = min((R + 1u) * KB, b_end);
            const bool whole = b == R * KB && seg_e == (R + 1u) * KB;
            const int32_t seg_je = seg_e == b_end ? j_end : __ldg(p.blk_off + seg_e);
            uint32_t mid = b;
            if (first) {
                // three block iterations complete the copy group of the entries for this lane, the warp barrier
                // for all lanes
                mid = min(b + 3u + 2u * ((uint32_t)wid & 7u), seg_e);      // (the warps' outlier passes do not all fall on the same moment)
                run(b, mid);
                if (mid - b < 3u) cp_async_wait<0>();
                __syncwarp();
                first = false;
            }
            for (uint32_t sb = b; sb < seg_e; sb += 64u) {
                const uint32_t se = min(sb + 64u, seg_e);
                const int32_t jlo = sb == b ? seg_j : __ldg(p.blk_off + sb);
                const int32_t jhi = se == seg_e ? seg_je : __ldg(p.blk_off + se);
                outlier_pass(sb, jlo, jhi);
            }
            run(mid, seg_e);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                c[i] += c1[i];
                c1[i] = 0.f;
            }
            if (whole) p6_store_tile(push, push_e, p.out_f, R, lane, c, m_rows, bias, y, y_f32);
            else {
                wparts[(R == R_first ? 0 : 32) + lane] = make_float4(c[0], c[1], c[2], c[3]);
                if (fast_tail) tile_arrive(R);
            }
            c[0] = c[1] = c[2] = c[3] = 0.f;
            b = seg_e;
            seg_j = seg_je;
            ++R;
#ifndef IXB_P6_UNIFORM_SCALE
            if (p.scale_stride) {                                         // warp uniform
                set_scale(sc_next);
                sc_next = (uint32_t)__bfloat16_as_ushort(p.scale[min(R + 1u, p.rt - 1u) * p.scale_stride]);
            }
#endif
        }
    }
    cp_async_wait<0>();
    if (!fast_tail) __syncthreads();

    // ---- more row tiles per CTA than the fast tail tracks: after a CTA-wide barrier, sum the parts of every tile
    // that more than one run of this CTA (or another CTA) touched
    if (!fast_tail && L) {
        for (uint32_t R = Rc0 + wid; R <= Rc1; R += kP6Warps) {
            const uint32_t t0 = R * KB, t1 = t0 + KB;                   // the tile's blocks
            const bool inside = t0 >= cb0 && t1 <= cb1;
            const uint32_t wlo = p6_part_of(max(t0, cb0) - cb0, wq, wr), whi = p6_part_of(min(t1, cb1) - 1 - cb0, wq, wr);
            if (inside && wlo == whi) continue;                          // one run had all of it and wrote y itself
            uint32_t clo = 0, span = 0;
            if (!inside) {
                clo = p6_part_of(t0, cq, cr);
                span = p6_part_of(t1 - 1u, cq, cr) - clo;
            }
            finish_tile(R, wlo, whi, inside, clo, span);
        }
    }
    if (!push.fin) return;

    // ---- the exchange's second half, by the same kernel: every thread of the grid looks after one pair of outputs
    // (the first n / 2 threads have one).  The words of this rank come from this very launch -- from CTAs that are
    // all resident, one per SM -- and the other ranks' from their launches of the same call.
    {
        const uint32_t n = m_rows * p.out_f, i = (blockIdx.x * kP6Threads + threadIdx.x) * 2u, W = push.world;
        if (i < n) {
            const uint32_t limit = *(volatile uint32_t *)push.err ? 64u : push.spin_limit;
            const uint2 *mine = push.mine;
            float o0 = 0.f, o1 = 0.f;
            for (uint32_t s = 0; s < W; ++s) {
                const uint2 *src = mine + ((size_t)((push_e & 1u) * W + s)) * push.n_max + i;
                uint32_t v0, m0, v1, m1, polls = 0;
                for (;;) {
                    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(m0), "=r"(v1), "=r"(m1) : "l"(src) : "memory");
                    if (m0 == push_e && m1 == push_e) break;
                    __nanosleep(20);
                    if (++polls > limit) {
                        *push.err = 1u + s;                // sender s never arrived: the result is wrong, not a hang
                        break;
                    }
                }
                o0 += __uint_as_float(v0);
                o1 += __uint_as_float(v1);
            }
            const uint32_t r0 = i % p.out_f;               // n is even and so is out_f: both values belong to one activation row
            if (y_f32) {
                float2 r;
                r.x = bias ? o0 + __bfloat162float(bias[r0]) : o0;
                r.y = bias ? o1 + __bfloat162float(bias[r0 + 1]) : o1;
                *(float2 *)((float *)y + i) = r;
            } else {
                __nv_bfloat16 h0 = __float2bfloat16_rn(o0), h1 = __float2bfloat16_rn(o1);
                if (bias) {
                    h0 = __hadd(h0, bias[r0]);
                    h1 = __hadd(h1, bias[r0 + 1]);
                }
                *(__nv_bfloat162 *)((__nv_bfloat16 *)y + i) = __halves2bfloat162(h0, h1);
            }
        }
        // the last warp of the grid to get here advances the call counters: by now every CTA has read them
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            if (atomicAdd(push.done, 1u) == gridDim.x * kP6Warps - 1u) {
                for (uint32_t k = 0; k < push.counters; ++k) push.epoch[k] = push_e;
                *push.done = 0;
            }
        }
    }
}

}  // namespace ixb
