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

// ---------------------------------------------------------------- sources ---
// A "source" hands out 32-bit words of the four rank-addressed streams.  Stream
// positions given to it are relative to its own origin (org_*), which is 0 for
// global memory and the staged slice's first word for shared memory.

// Streams read straight from global memory, zero beyond each stream's end.
struct GlobalSrc {
    const Streams &s;
    static constexpr uint32_t org_b2 = 0, org_l1 = 0, org_l2 = 0, org_l3 = 0;   // bits, bits, bits, bytes
    __device__ __forceinline__ uint32_t b2w(uint32_t i) const { return ldw(s.b2, i, s.b2_words); }
    __device__ __forceinline__ uint32_t l1w(uint32_t i) const { return ldw(s.l1, i, s.l1_words); }
    __device__ __forceinline__ uint32_t l2w(uint32_t i) const { return ldw(s.l2, i, s.l2_words); }
    __device__ __forceinline__ uint32_t l3w(uint32_t i) const
    {
        uint32_t byte0 = 4u * i;
        if (byte0 + 4u <= s.l3_bytes) return __ldg((const uint32_t *)s.l3 + i);
        uint32_t v = 0;
        for (uint32_t k = 0; k < 4u; ++k)
            if (byte0 + k < s.l3_bytes) v |= (uint32_t)__ldg(s.l3 + byte0 + k) << (8u * k);
        return v;
    }
};

// Slices of one rank block staged in shared memory (zero-filled past the end
// of a stream, two spare words after every slice).
struct SlotSrc {
    const uint32_t *b2, *l1, *l2, *l3;
    uint32_t org_b2, org_l1, org_l2, org_l3;
    bool too_big;   // a slice did not fit its slot region: the slot is not usable for this block
    __device__ __forceinline__ uint32_t b2w(uint32_t i) const { return b2[i]; }
    __device__ __forceinline__ uint32_t l1w(uint32_t i) const { return l1[i]; }
    __device__ __forceinline__ uint32_t l2w(uint32_t i) const { return l2[i]; }
    __device__ __forceinline__ uint32_t l3w(uint32_t i) const { return l3[i]; }
};

// Per-lane rank state of one 32-element bitmap word.
struct WordRanks {
    uint32_t m1;     // B1 word: bit i = element i is level 1
    uint32_t m2;     // B2 bits of this word's non-L1 elements, in order, LSB first
    uint32_t bit1;   // source-relative bit position of the word's first L1 field
    uint32_t bit2;   // source-relative bit position of the word's first L2 field
    uint32_t byte3;  // source-relative byte position of the word's first L3 byte
};

// Ranks for the 32 words of rank block `blk` (lane = word) from the block's B1
// word of this lane.  `valid` is the number of real elements in this lane's
// word (32 except at the tensor's end); a_blk / c_blk are the block's entries
// of the rank tables.
template <class Src>
__device__ __forceinline__ WordRanks block_ranks(const Src &src, uint32_t m1, uint32_t blk, uint32_t a_blk,
                                                 uint32_t c_blk, int lane, uint32_t valid)
{
    WordRanks w;
    w.m1 = m1;
    uint32_t n1 = __popc(m1);
    uint32_t ex1 = warp_incl_scan(n1, lane) - n1;
    uint32_t nn = valid - n1;                               // non-L1 elements in this word
    uint32_t r = blk * (uint32_t)kBlk - a_blk + 32u * lane - ex1;   // global non-L1 rank
    uint32_t rb = valid ? r - src.org_b2 : 0u;              // words past the tensor's end read slot word 0
    w.m2 = __funnelshift_r(src.b2w(rb >> 5), src.b2w((rb >> 5) + 1), rb & 31u) & lowmask(nn);
    uint32_t n2 = __popc(w.m2);
    uint32_t ex2 = warp_incl_scan(n2, lane) - n2;
    uint32_t a = a_blk + ex1, c = c_blk + ex2;
    w.bit1 = valid ? a * 3u - src.org_l1 : 0u;
    w.bit2 = valid ? c * 5u - src.org_l2 : 0u;
    w.byte3 = valid ? (r - c) - src.org_l3 : 0u;
    return w;
}

// Dequantisation table used by decode_word: 512 four-byte entries, 2 KB
// aligned in shared memory.
//   level 2 symbol s -> byte offset 4 s          (entries 0..31)
//   level 1 symbol s -> byte offset 128 + 4 s    (entries 32..38)
//   level 3 byte b   -> byte offset 1024 + 4 b   (entries 256..511)
// The three levels are looked up by separate predicated loads, so only symbols
// of one level meet in a load: 7 resp. 24 distinct valid symbols, each in its
// own bank.
constexpr uint32_t kOffL1 = 128;
constexpr uint32_t kOffL3 = 1024;
constexpr int kTabEntries = 512;
constexpr int kTabBytes = kTabEntries * 4;

__host__ __device__ inline int tab_code(int entry)
{
    if (entry >= 256) return entry - 256 - 127;
    if (entry >= 32 && entry < 40) return entry - 32 - 3;
    return entry - 15;   // entries 40..255 are never read
}

// Stream cursors of a word at the four 8-element group boundaries.
struct WordCursors {
    uint32_t b1p[4], b2p[4], b3p[4];   // bit positions (source relative) of L1 / L2 / L3 data
    uint32_t nn[4];                    // non-L1 elements before the group
    uint32_t max_l3;                   // largest number of level-3 elements in one group
};

__device__ __forceinline__ WordCursors word_cursors(const WordRanks &w)
{
    WordCursors c;
    uint32_t k1[5], k2[5];
    k1[0] = 0; k2[0] = 0;
#pragma unroll
    for (int q = 1; q < 4; ++q) k1[q] = __popc(w.m1 & ((1u << (8 * q)) - 1u));
    k1[4] = __popc(w.m1);
#pragma unroll
    for (int q = 1; q <= 4; ++q) k2[q] = __popc(w.m2 & lowmask(8u * q - k1[q]));
    c.max_l3 = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        c.nn[q] = 8u * q - k1[q];
        c.b1p[q] = w.bit1 + 3u * k1[q];
        c.b2p[q] = w.bit2 + 5u * k2[q];
        c.b3p[q] = (w.byte3 + c.nn[q] - k2[q]) * 8u;
        uint32_t l3 = (8u - (k1[q + 1] - k1[q])) - (k2[q + 1] - k2[q]);
        c.max_l3 = max(c.max_l3, l3);
    }
    return c;
}

// One element of the branch-free decoder.  Exactly one of the three predicated
// table loads executes; queues hold their fields pre-multiplied by 4.
#define IXB_ELEM(BITMASK)                                                                         \
    asm("{\n\t"                                                                                   \
        ".reg .pred p1, p2, p3;\n\t"                                                              \
        ".reg .b32 t, a1, a2, a3;\n\t"                                                            \
        "and.b32 t, %6, " #BITMASK ";\n\t"                                                        \
        "setp.ne.u32 p1, t, 0;\n\t"                                                               \
        "and.b32 t, %5, 1;\n\t"                                                                   \
        "setp.ne.and.u32 p2, t, 0, !p1;\n\t"                                                      \
        "setp.eq.and.u32 p3, t, 0, !p1;\n\t"                                                      \
        "lop3.b32 a1, %1, 28, %7, 0xEA;\n\t"                                                      \
        "lop3.b32 a2, %2, 124, %8, 0xEA;\n\t"                                                     \
        "lop3.b32 a3, %4, 1020, %9, 0xEA;\n\t"                                                    \
        "@p1 ld.shared.b32 %0, [a1];\n\t"                                                         \
        "@p2 ld.shared.b32 %0, [a2];\n\t"                                                         \
        "@p3 ld.shared.b32 %0, [a3];\n\t"                                                         \
        "@p1 shr.u32 %1, %1, 3;\n\t"                                                              \
        "@p2 shf.r.wrap.b32 %2, %2, %3, 5;\n\t"                                                   \
        "@p2 shr.u32 %3, %3, 5;\n\t"                                                              \
        "@p3 shr.u32 %4, %4, 8;\n\t"                                                              \
        "@!p1 shr.u32 %5, %5, 1;\n\t"                                                             \
        "}"                                                                                       \
        : "=r"(wv), "+r"(q1), "+r"(q2lo), "+r"(q2hi), "+r"(q3), "+r"(mq)                          \
        : "r"(m1), "r"(tL1), "r"(tL2), "r"(tL3))

// Decode the 32 elements of one word in order, without data-dependent
// branches.  `tab` is the shared-window address of the 2 KB-aligned table
// above.  pre(q) runs before each group of 8 elements (q = 0..3); sink(i, v)
// receives the element index i (a compile-time constant after unrolling) and
// the element's 32-bit table entry.  Requires c.max_l3 <= 3 (a group's level-3
// bytes are carried in one register); decode_word_any has no such limit.
template <class Src, class Pre, class Sink>
__device__ __forceinline__ void decode_word_fast(const Src &src, const WordRanks &w, const WordCursors &c,
                                                 uint32_t tab, Pre &&pre, Sink &&sink)
{
    const uint32_t m1 = w.m1;
    const uint32_t tL2 = tab, tL1 = tab + kOffL1, tL3 = tab + kOffL3;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        pre(q);
        uint32_t i1 = c.b1p[q] >> 5, i2 = c.b2p[q] >> 5, i3 = c.b3p[q] >> 5;
        uint32_t q1 = __funnelshift_r(src.l1w(i1), src.l1w(i1 + 1), c.b1p[q] & 31u) << 2;   // 8 x 3 bits
        uint32_t x0 = src.l2w(i2), x1 = src.l2w(i2 + 1), x2 = src.l2w(i2 + 2);
        uint32_t f0 = __funnelshift_r(x0, x1, c.b2p[q] & 31u), f1 = __funnelshift_r(x1, x2, c.b2p[q] & 31u);
        uint32_t q2lo = f0 << 2, q2hi = __funnelshift_l(f0, f1, 2);                          // 8 x 5 bits
        uint32_t q3 = __funnelshift_r(src.l3w(i3), src.l3w(i3 + 1), c.b3p[q] & 31u) << 2;   // 3 bytes
        uint32_t mq = w.m2 >> c.nn[q];
        uint32_t wv;
#define IXB_E(j, mask)                      \
    IXB_ELEM(mask);                         \
    sink(8 * q + j, wv);
        if (q == 0) { IXB_E(0, 0x1) IXB_E(1, 0x2) IXB_E(2, 0x4) IXB_E(3, 0x8) IXB_E(4, 0x10) IXB_E(5, 0x20) IXB_E(6, 0x40) IXB_E(7, 0x80) }
        if (q == 1) { IXB_E(0, 0x100) IXB_E(1, 0x200) IXB_E(2, 0x400) IXB_E(3, 0x800) IXB_E(4, 0x1000) IXB_E(5, 0x2000) IXB_E(6, 0x4000) IXB_E(7, 0x8000) }
        if (q == 2) { IXB_E(0, 0x10000) IXB_E(1, 0x20000) IXB_E(2, 0x40000) IXB_E(3, 0x80000) IXB_E(4, 0x100000) IXB_E(5, 0x200000) IXB_E(6, 0x400000) IXB_E(7, 0x800000) }
        if (q == 3) { IXB_E(0, 0x1000000) IXB_E(1, 0x2000000) IXB_E(2, 0x4000000) IXB_E(3, 0x8000000) IXB_E(4, 0x10000000) IXB_E(5, 0x20000000) IXB_E(6, 0x40000000) IXB_E(7, 0x80000000) }
#undef IXB_E
    }
}

// One element of the table-free decoder used by the fused GEMV: the element's
// code is rebuilt as a float with the 2^23 mantissa trick, and the weight
// bf16(code * scale) comes from one packed bf16 multiply whose upper half is
// the (exactly rounded) product and whose lower half is 0 * scale = 0 -- read
// as fp32 that register is the weight itself.  On sm_100 logic/shift/compare
// instructions issue at half the rate of add/FMA, so the two bitmaps are kept
// bit-reversed and left-aligned: the next B1 / B2 bit is the sign bit (one
// compare each, no mask-and-test) and both queues advance with an add.
#define IXB_ELEM_ARITH()                                                                          \
    asm("{\n\t"                                                                                   \
        ".reg .pred p1, p2, p3;\n\t"                                                              \
        ".reg .b32 f, c;\n\t"                                                                     \
        "setp.lt.s32 p1, %6, 0;\n\t"                                                              \
        "setp.lt.and.s32 p2, %5, 0, !p1;\n\t"                                                     \
        "setp.ge.and.s32 p3, %5, 0, !p1;\n\t"                                                     \
        "add.u32 %6, %6, %6;\n\t"                                                                 \
        "lop3.b32 f, %1, 7, 0x4B000000, 0xEA;\n\t"                                                \
        "sub.f32 c, f, 0f4B000003;\n\t"                                                           \
        "@p2 lop3.b32 f, %2, 31, 0x4B000000, 0xEA;\n\t"                                           \
        "@p2 sub.f32 c, f, 0f4B00000F;\n\t"                                                       \
        "@p3 lop3.b32 f, %4, 255, 0x4B000000, 0xEA;\n\t"                                          \
        "@p3 sub.f32 c, f, 0f4B00007F;\n\t"                                                       \
        "mul.rn.bf16x2 %0, c, %7;\n\t"                                                            \
        "@p1 shr.u32 %1, %1, 3;\n\t"                                                              \
        "@p2 shf.r.wrap.b32 %2, %2, %3, 5;\n\t"                                                   \
        "@p2 shr.u32 %3, %3, 5;\n\t"                                                              \
        "@p3 shr.u32 %4, %4, 8;\n\t"                                                              \
        "@!p1 add.u32 %5, %5, %5;\n\t"                                                            \
        "}"                                                                                       \
        : "=r"(wv), "+r"(q1), "+r"(q2lo), "+r"(q2hi), "+r"(q3), "+r"(mq), "+r"(m1s)               \
        : "r"(s2))

// Table-free variant of decode_word_fast: sink(i, v) receives the fp32 bit
// pattern of the element's weight bf16(code * scale).  `s2` holds the bf16
// scale in both halves.  Requires c.max_l3 <= 4.
template <class Src, class Pre, class Sink>
__device__ __forceinline__ void decode_word_arith(const Src &src, const WordRanks &w, const WordCursors &c,
                                                  uint32_t s2, Pre &&pre, Sink &&sink)
{
    uint32_t m1s = __brev(w.m1);                 // next B1 bit in the sign
    const uint32_t brev_m2 = __brev(w.m2);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        pre(q);
        uint32_t i1 = c.b1p[q] >> 5, i2 = c.b2p[q] >> 5, i3 = c.b3p[q] >> 5;
        uint32_t q1 = __funnelshift_r(src.l1w(i1), src.l1w(i1 + 1), c.b1p[q] & 31u);        // 8 x 3 bits
        uint32_t x0 = src.l2w(i2), x1 = src.l2w(i2 + 1), x2 = src.l2w(i2 + 2);
        uint32_t q2lo = __funnelshift_r(x0, x1, c.b2p[q] & 31u);                            // 8 x 5 bits
        uint32_t q2hi = __funnelshift_r(x1, x2, c.b2p[q] & 31u);
        uint32_t q3 = __funnelshift_r(src.l3w(i3), src.l3w(i3 + 1), c.b3p[q] & 31u);        // 4 bytes
        uint32_t mq = brev_m2 << c.nn[q];                                                   // next B2 bit in the sign
        uint32_t wv;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            IXB_ELEM_ARITH();
            sink(8 * q + j, wv);
        }
    }
}

// Same contract without the limit on level-3 elements per group (plain C++,
// 64-bit level-3 queue); used for the rare words that exceed it.
template <class Src, class Pre, class Sink>
__device__ __noinline__ void decode_word_any(const Src &src, const WordRanks &w, const WordCursors &c,
                                             const uint32_t *tab_ptr, Pre &&pre, Sink &&sink)
{
#pragma unroll 1
    for (int q = 0; q < 4; ++q) {
        pre(q);
        uint32_t i1 = c.b1p[q] >> 5, i2 = c.b2p[q] >> 5, i3 = c.b3p[q] >> 5;
        uint32_t q1 = __funnelshift_r(src.l1w(i1), src.l1w(i1 + 1), c.b1p[q] & 31u);
        uint32_t x0 = src.l2w(i2), x1 = src.l2w(i2 + 1), x2 = src.l2w(i2 + 2);
        uint64_t q2 = (uint64_t)__funnelshift_r(x0, x1, c.b2p[q] & 31u) |
                      ((uint64_t)__funnelshift_r(x1, x2, c.b2p[q] & 31u) << 32);
        uint32_t y0 = src.l3w(i3), y1 = src.l3w(i3 + 1), y2 = src.l3w(i3 + 2);
        uint64_t q3 = (uint64_t)__funnelshift_r(y0, y1, c.b3p[q] & 31u) |
                      ((uint64_t)__funnelshift_r(y1, y2, c.b3p[q] & 31u) << 32);
        uint32_t mq = w.m2 >> c.nn[q];
#pragma unroll 1
        for (int j = 0; j < 8; ++j) {
            const int i = 8 * q + j;
            uint32_t entry;
            if ((w.m1 >> i) & 1u) {
                entry = 32u + (q1 & 7u);
                q1 >>= 3;
            } else {
                if (mq & 1u) {
                    entry = (uint32_t)q2 & 31u;
                    q2 >>= 5;
                } else {
                    entry = 256u + ((uint32_t)q3 & 255u);
                    q3 >>= 8;
                }
                mq >>= 1;
            }
            sink(i, tab_ptr[entry]);
        }
    }
}

// Plain sequential decode of one word: sink(i, code) with the int8 code value.
// No limit on level-3 elements; used by the fused GEMV for the rare words the
// fast decoders cannot take.
template <class Src, class Sink>
__device__ __noinline__ void decode_word_slow(const Src &src, const WordRanks &w, const WordCursors &c, Sink &&sink)
{
    uint32_t b1p = c.b1p[0], b2p = c.b2p[0], b3p = c.b3p[0] >> 3;
    uint32_t mq = w.m2;
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
        int code;
        if ((w.m1 >> i) & 1u) {
            uint32_t v = __funnelshift_r(src.l1w(b1p >> 5), src.l1w((b1p >> 5) + 1), b1p & 31u);
            code = (int)(v & 7u) - 3;
            b1p += 3;
        } else {
            if (mq & 1u) {
                uint32_t v = __funnelshift_r(src.l2w(b2p >> 5), src.l2w((b2p >> 5) + 1), b2p & 31u);
                code = (int)(v & 31u) - 15;
                b2p += 5;
            } else {
                code = (int)((src.l3w(b3p >> 2) >> (8u * (b3p & 3u))) & 255u) - 127;
                b3p += 1;
            }
            mq >>= 1;
        }
        sink(i, code);
    }
}

// ---------------------------------------------------------------- staging ---
// Shared-memory slot of one rank block (32-bit words).  Each slice starts on a
// 16-byte boundary of its stream and is followed by two spare words, so the
// decoder's look-ahead reads never leave the slot.
struct Slot {
    static constexpr int kB1 = 0, kB1Chunks = 8;      //  32 words
    static constexpr int kB2 = 32, kB2Chunks = 10;    //  40 words: 1024 bits + misalignment + spare
    static constexpr int kL1 = 72, kL1Chunks = 26;    // 104 words: 3072 bits ...
    static constexpr int kL2 = 176, kL2Chunks = 42;   // 168 words: 5120 bits ...
    static constexpr int kL3 = 344, kL3Chunks = 10;   //  40 words: up to ~120 level-3 bytes; a block with
                                                      //  more is decoded straight from global memory
    static constexpr int kWords = 384;
};

__device__ __forceinline__ void cp_async_16(uint32_t *dst_smem, const void *src, uint32_t valid_bytes)
{
    uint32_t d = (uint32_t)__cvta_generic_to_shared(dst_smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(valid_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Copy 16-byte chunks [c_lo, c_hi) of a stream of `bytes` bytes into dst
// (zero beyond the stream's end); the whole warp takes part.
__device__ __forceinline__ void stage_chunks(uint32_t *dst, const void *base, uint32_t bytes, uint32_t c_lo,
                                             uint32_t c_hi, int lane)
{
    for (uint32_t c = c_lo + lane; c < c_hi; c += 32) {
        uint32_t off = c * 16u;
        uint32_t valid = bytes > off ? min(16u, bytes - off) : 0u;
        uint32_t *d = dst + (c - c_lo) * 4u;
        if (valid) cp_async_16(d, (const char *)base + off, valid);
        else *(uint4 *)d = make_uint4(0, 0, 0, 0);
    }
}

// Issue the asynchronous copies of rank block `b` into `slot` and describe the
// result.  (a0, c0) are the block's rank-table entries, (a1, c1) those of the
// next block (ignored for the last block, whose slices run to the stream end).
// General version: every slice is copied by a loop over the whole warp.
__device__ __noinline__ SlotSrc stage_block_any(const Streams &s, uint32_t b, bool last, uint32_t a0, uint32_t c0,
                                                uint32_t a1, uint32_t c1, uint32_t *slot, int lane)
{
    SlotSrc src;
    uint32_t e1 = min((b + 1u) * (uint32_t)kBlk, s.n);
    uint32_t r0 = b * (uint32_t)kBlk - a0, r1 = e1 - a1;
    // bit ranges of the four rank-addressed slices
    uint32_t lo[4] = {r0, a0 * 3u, c0 * 5u, (r0 - c0) * 8u};
    uint32_t hi[4] = {r1, a1 * 3u, c1 * 5u, (r1 - c1) * 8u};
    const uint32_t bytes[4] = {s.b2_words * 4u, s.l1_words * 4u, s.l2_words * 4u, s.l3_bytes};
    const void *base[4] = {s.b2, s.l1, s.l2, s.l3};
    const int at[4] = {Slot::kB2, Slot::kL1, Slot::kL2, Slot::kL3};
    const uint32_t cap[4] = {Slot::kB2Chunks, Slot::kL1Chunks, Slot::kL2Chunks, Slot::kL3Chunks};
    uint32_t org[4];
    bool too_big = false;
    stage_chunks(slot + Slot::kB1, s.b1, s.b1_words * 4u, b * 8u, b * 8u + 8u, lane);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint32_t c_lo = lo[k] >> 7;                                   // 128 bits per chunk
        uint32_t w_hi = last ? ((bytes[k] + 3u) >> 2) : ((hi[k] + 31u) >> 5);
        uint32_t c_need = (w_hi + 2u + 3u) >> 2;
        uint32_t c_hi = min(c_need, c_lo + cap[k]);
        too_big = too_big || c_need > c_lo + cap[k];
        stage_chunks(slot + at[k], base[k], bytes[k], c_lo, c_hi, lane);
        org[k] = c_lo * 128u;
    }
    src.too_big = too_big;
    src.b2 = slot + Slot::kB2;
    src.l1 = slot + Slot::kL1;
    src.l2 = slot + Slot::kL2;
    src.l3 = slot + Slot::kL3;
    src.org_b2 = org[0];
    src.org_l1 = org[1];
    src.org_l2 = org[2];
    src.org_l3 = org[3] >> 3;
    return src;
}

// Lane roles for the common case.  The bit range of every slice is a linear
// form  ke * E + ka * a + kc * c  of the block's first element E and its
// rank-table entries, so each lane evaluates only the slice it serves:
//   B1: E            B2: E - a         L1: 3a        L2: 5c       L3: 8(E - a - c)
// Two passes of 32 lanes copy up to 8 / 7 / 20 / 24 / 5 chunks of B1 / B2 /
// L1 / L2 / L3; a block that needs more goes through stage_block_any.
struct StageRole {
    const char *base;     // stream base
    uint32_t bytes;       // stream length
    int32_t ke, ka, kc;   // coefficients of the slice's bit range
    uint32_t idx;         // chunk of the slice this lane copies
    uint32_t allot;       // chunks of the slice served by roles
    uint32_t cap;         // chunks the slot can hold for the slice
    uint32_t at;          // word offset of the slice in the slot
};

__device__ __forceinline__ StageRole make_role(const Streams &s, int slice, uint32_t idx)
{
    StageRole r;
    r.idx = idx;
    switch (slice) {
    case 0: r = {(const char *)s.b1, s.b1_words * 4u, 1, 0, 0, idx, 8u, (uint32_t)Slot::kB1Chunks, (uint32_t)Slot::kB1}; break;
    case 1: r = {(const char *)s.b2, s.b2_words * 4u, 1, -1, 0, idx, 7u, (uint32_t)Slot::kB2Chunks, (uint32_t)Slot::kB2}; break;
    case 2: r = {(const char *)s.l1, s.l1_words * 4u, 0, 3, 0, idx, 20u, (uint32_t)Slot::kL1Chunks, (uint32_t)Slot::kL1}; break;
    case 3: r = {(const char *)s.l2, s.l2_words * 4u, 0, 0, 5, idx, 24u, (uint32_t)Slot::kL2Chunks, (uint32_t)Slot::kL2}; break;
    default: r = {(const char *)s.l3, s.l3_bytes, 8, -8, -8, idx, 5u, (uint32_t)Slot::kL3Chunks, (uint32_t)Slot::kL3}; break;
    }
    return r;
}

// pass A: lanes 0-7 B1, 8-31 L2[0..23];  pass B: lanes 0-19 L1, 20-26 B2, 27-31 L3
__device__ __forceinline__ StageRole role_a(const Streams &s, int lane)
{
    return lane < 8 ? make_role(s, 0, lane) : make_role(s, 3, lane - 8);
}
__device__ __forceinline__ StageRole role_b(const Streams &s, int lane)
{
    return lane < 20 ? make_role(s, 2, lane) : (lane < 27 ? make_role(s, 1, lane - 20) : make_role(s, 4, lane - 27));
}

// One role's copy for a block; returns the slice's first chunk and whether the
// slice needs more chunks than the roles serve.
__device__ __forceinline__ uint32_t stage_role(const StageRole &r, uint32_t E0, uint32_t E1, bool last, uint32_t a0,
                                               uint32_t c0, uint32_t a1, uint32_t c1, uint32_t *slot, bool &overflow)
{
    uint32_t lo = (uint32_t)(r.ke * (int32_t)E0 + r.ka * (int32_t)a0 + r.kc * (int32_t)c0);
    uint32_t hi = (uint32_t)(r.ke * (int32_t)E1 + r.ka * (int32_t)a1 + r.kc * (int32_t)c1);
    uint32_t c_lo = lo >> 7;
    uint32_t w_hi = last ? ((r.bytes + 3u) >> 2) : ((hi + 31u) >> 5);
    uint32_t spare = r.at == (uint32_t)Slot::kB1 ? 0u : 2u;
    uint32_t c_hi = min((w_hi + spare + 3u) >> 2, c_lo + r.cap);
    overflow = c_hi - c_lo > r.allot;
    uint32_t c = c_lo + r.idx;
    if (c < c_hi) {
        uint32_t off = c * 16u;
        uint32_t valid = r.bytes > off ? min(16u, r.bytes - off) : 0u;
        uint32_t *d = slot + r.at + r.idx * 4u;
        if (valid) cp_async_16(d, r.base + off, valid);
        else *(uint4 *)d = make_uint4(0, 0, 0, 0);
    }
    return c_lo;
}

__device__ __forceinline__ SlotSrc stage_block(const Streams &s, const StageRole &ra, const StageRole &rb, uint32_t b,
                                               bool last, uint32_t a0, uint32_t c0, uint32_t a1, uint32_t c1,
                                               uint32_t *slot, int lane)
{
    uint32_t E0 = b * (uint32_t)kBlk, E1 = min(E0 + (uint32_t)kBlk, s.n);
    bool ova, ovb;
    uint32_t lo_a = stage_role(ra, E0, E1, last, a0, c0, a1, c1, slot, ova);
    uint32_t lo_b = stage_role(rb, E0, E1, last, a0, c0, a1, c1, slot, ovb);
    if (__any_sync(0xffffffffu, ova || ovb)) return stage_block_any(s, b, last, a0, c0, a1, c1, slot, lane);
    SlotSrc src;
    src.too_big = false;
    src.b2 = slot + Slot::kB2;
    src.l1 = slot + Slot::kL1;
    src.l2 = slot + Slot::kL2;
    src.l3 = slot + Slot::kL3;
    src.org_l2 = __shfl_sync(0xffffffffu, lo_a, 8) * 128u;
    src.org_l1 = __shfl_sync(0xffffffffu, lo_b, 0) * 128u;
    src.org_b2 = __shfl_sync(0xffffffffu, lo_b, 20) * 128u;
    src.org_l3 = __shfl_sync(0xffffffffu, lo_b, 27) * 16u;
    return src;
}

}  // namespace ixb
