// Shared device helpers for the INT8-X (3,5,8) kernels (sm_100a).
//
// Format recap (reference: ixrun/quantize.py:80-96, ixrun/bitpack.py:13-61):
// for flat element e of the row-major code matrix, with a = #L1 elements
// before e, r = e - a, c = #L2 elements before e:
//   B1 bit e      -> element is level 1; its 3-bit field is L1[3a .. 3a+3)
//   B2 bit r      -> (non-L1) element is level 2; 5-bit field L2[5c .. 5c+5)
//   otherwise     -> level 3; byte L3[r - c]
// Fields are LSB-first across little-endian 32-bit words.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ixb {

constexpr int kBlk = 1024;        // elements per rank block (one warp iteration)
constexpr int kWarp = 32;

// Dequantisation table, indexed by "level slot":
//   level 1 symbol s (0..6)   -> entry 12 + s
//   level 2 symbol s (0..31)  -> entry s        (valid symbols 0..11, 19..30)
//   level 3 byte   b (0..255) -> entry 32 + b
// Every symbol a valid stream can hold for levels 1 and 2 sits in its own
// shared-memory bank (12..18 are never level-2 symbols), so the per-element
// lookup of the two common levels is conflict-free.
constexpr int kLutL1 = 12;
constexpr int kLutL3 = 32;
constexpr int kLutSize = 288;

__host__ __device__ inline int lut_code(int entry)
{
    if (entry >= kLutL3) return entry - kLutL3 - 127;
    if (entry >= kLutL1 && entry < kLutL1 + 7) return entry - kLutL1 - 3;
    return entry - 15;
}

struct Streams {
    const uint32_t *b1, *b2, *l1, *l2;
    const uint8_t *l3;
    uint32_t b1_words, b2_words, l1_words, l2_words, l3_bytes;
    const __nv_bfloat16 *scale;
    uint32_t n;       // out_f * in_f
    uint32_t out_f, in_f;
};

__device__ __forceinline__ uint32_t lowmask(uint32_t nbits)
{
    uint32_t m;
    asm("bmsk.clamp.b32 %0, %1, %2;" : "=r"(m) : "r"(0u), "r"(nbits));
    return m;
}

__device__ __forceinline__ uint32_t warp_incl_scan(uint32_t v, int lane)
{
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t t = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += t;
    }
    return v;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

__device__ __forceinline__ uint32_t ldw(const uint32_t *p, uint32_t i, uint32_t n)
{
    return i < n ? __ldg(p + i) : 0u;
}

// 32 bits of a word stream starting at bit position `bit` (zero beyond the end)
__device__ __forceinline__ uint32_t fetch32(const uint32_t *p, uint32_t words, uint32_t bit)
{
    uint32_t wi = bit >> 5;
    return __funnelshift_r(ldw(p, wi, words), ldw(p, wi + 1, words), bit & 31u);
}

__device__ __forceinline__ uint64_t fetch64(const uint32_t *p, uint32_t words, uint32_t bit)
{
    uint32_t wi = bit >> 5, sh = bit & 31u;
    uint32_t w0 = ldw(p, wi, words), w1 = ldw(p, wi + 1, words), w2 = ldw(p, wi + 2, words);
    return (uint64_t)__funnelshift_r(w0, w1, sh) | ((uint64_t)__funnelshift_r(w1, w2, sh) << 32);
}

// Per-lane rank state of one 32-element bitmap word.
struct WordRanks {
    uint32_t m1;   // B1 word: bit i = element i is level 1
    uint32_t m2;   // B2 bits of this word's non-L1 elements, in order, LSB first
    uint32_t a;    // global L1 rank of the word's first L1 element
    uint32_t c;    // global L2 rank of the word's first L2 element
    uint32_t t;    // global L3 index of the word's first L3 element
};

// Ranks for the 32 words of rank block `blk` (lane = word).  `valid` is the
// number of real elements in this lane's word (32 except at the tensor's end).
__device__ __forceinline__ WordRanks block_ranks(const Streams &s, uint32_t blk, uint32_t a_blk,
                                                 uint32_t c_blk, int lane, uint32_t valid)
{
    WordRanks w;
    uint32_t wi = blk * 32u + lane;
    w.m1 = ldw(s.b1, wi, s.b1_words);
    uint32_t n1 = __popc(w.m1);
    uint32_t ex1 = warp_incl_scan(n1, lane) - n1;
    uint32_t nn = valid - n1;                              // non-L1 elements in this word
    uint32_t nn_before = 32u * lane - ex1;                 // ... in earlier words of the block
    uint32_t r = blk * (uint32_t)kBlk - a_blk + nn_before; // global non-L1 rank
    w.m2 = fetch32(s.b2, s.b2_words, r) & lowmask(nn);
    uint32_t n2 = __popc(w.m2);
    uint32_t ex2 = warp_incl_scan(n2, lane) - n2;
    w.a = a_blk + ex1;
    w.c = c_blk + ex2;
    w.t = r - w.c;
    return w;
}

// Decode the 32 elements of one word in order.  pre(q) runs before each group
// of 8 elements (q = 0..3); sink(i, off) receives the
// element index i (compile-time after unrolling) and the byte offset of the
// element's entry in a 4-byte-per-entry table laid out as described above.
template <class Pre, class Sink>
__device__ __forceinline__ void decode_word(const Streams &s, const WordRanks &w, Pre &&pre, Sink &&sink)
{
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        pre(q);
        // stream cursors at the start of this group of 8 elements
        uint32_t k1 = q ? __popc(w.m1 & ((1u << (8 * q)) - 1u)) : 0u;
        uint32_t nnq = 8u * q - k1;
        uint32_t k2 = q ? __popc(w.m2 & lowmask(nnq)) : 0u;
        uint32_t q1 = fetch32(s.l1, s.l1_words, (w.a + k1) * 3u) << 2;   // <= 24 bits used
        uint64_t q2 = fetch64(s.l2, s.l2_words, (w.c + k2) * 5u) << 2;   // <= 40 bits used
        uint32_t mq = w.m2 >> nnq;
        uint32_t t = w.t + nnq - k2;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = 8 * q + j;
            uint32_t off;
            if ((w.m1 >> i) & 1u) {
                off = (q1 & 28u) + kLutL1 * 4u;
                q1 >>= 3;
            } else {
                if (mq & 1u) {
                    off = (uint32_t)q2 & 124u;
                    q2 >>= 5;
                } else {
                    uint32_t b = t < s.l3_bytes ? (uint32_t)__ldg(s.l3 + t) : 0u;
                    off = kLutL3 * 4u + 4u * b;
                    ++t;
                }
                mq >>= 1;
            }
            sink(i, off);
        }
    }
}

}  // namespace ixb
