// ixb200: C-ABI entry points and kernels of the B200 INT8-X weight path.
// Built for sm_100a only.  See include/ixb200.h for the contract of each call.
#include "../../include/ixb200.h"
#include <cstdlib>
#include <cuda_fp16.h>
#include "ixb_common.cuh"
#include "ixb_gemm_tc.cuh"
#include "ixb_p6_gemm.cuh"
#include "ixb_pack.cuh"
#include "ixb_p6.cuh"
#include "ixb_allreduce.cuh"
#include "ixb_glue.cuh"
#include "ixb_tpab.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace ixb {

// ----------------------------------------------------------------- errors ---
static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

static int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define IXB_CUDA(call)                                                                        \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess)                                                                \
            return fail(IXB_E_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_));          \
    } while (0)

static int launch_check(const char *what)
{
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(IXB_E_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return IXB_OK;
}

static int num_sms()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// opt-in to more than 48 KB of dynamic shared memory, once per kernel instantiation and device
template <class K>
static cudaError_t opt_in_smem(K kernel, bool (&done)[64], int bytes)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!done[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        done[dev] = true;
    }
    return cudaSuccess;
}

static int to_streams(const ixb_packed *w, Streams *s)
{
    if (!w) return fail(IXB_E_ARG, "packed tensor is NULL");
    if (w->out_f <= 0 || w->in_f <= 0) return fail(IXB_E_ARG, "bad shape %lld x %lld", (long long)w->out_f, (long long)w->in_f);
    long long n = (long long)w->out_f * w->in_f;
    // bit positions (5 bits per element at most) are carried in 32 bits
    if (n > 800000000LL) return fail(IXB_E_UNSUPPORTED, "tensor of %lld elements is too large (max 8e8)", n);
    if (!w->b1 || !w->scale) return fail(IXB_E_ARG, "b1/scale pointer is NULL");
    if (w->b1_words != (n + 31) / 32) return fail(IXB_E_ARG, "b1_words %lld != ceil(N/32)", (long long)w->b1_words);
    if ((w->b2_words && !w->b2) || (w->l1_words && !w->l1) || (w->l2_words && !w->l2) || (w->l3_bytes && !w->l3))
        return fail(IXB_E_ARG, "non-empty stream with NULL pointer");
    const void *ptrs[5] = {w->b1, w->b2, w->l1, w->l2, w->l3};
    for (int i = 0; i < 5; ++i)
        if (ptrs[i] && ((uintptr_t)ptrs[i] & 15u)) return fail(IXB_E_ARG, "stream %d is not 16-byte aligned", i);
    s->b1 = (const uint32_t *)w->b1;
    s->b2 = (const uint32_t *)w->b2;
    s->l1 = (const uint32_t *)w->l1;
    s->l2 = (const uint32_t *)w->l2;
    s->l3 = (const uint8_t *)w->l3;
    s->b1_words = (uint32_t)w->b1_words;
    s->b2_words = (uint32_t)w->b2_words;
    s->l1_words = (uint32_t)w->l1_words;
    s->l2_words = (uint32_t)w->l2_words;
    s->l3_bytes = (uint32_t)w->l3_bytes;
    s->scale = (const __nv_bfloat16 *)w->scale;
    s->n = (uint32_t)n;
    s->out_f = (uint32_t)w->out_f;
    s->in_f = (uint32_t)w->in_f;
    return IXB_OK;
}

// ------------------------------------------------------- prefix tables ------
// cnt1[b] = number of level-1 elements in rank block b (one warp per block)
__global__ void k_count_l1(Streams s, uint32_t nb, int32_t *cnt1)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= nb) return;
    uint32_t c = __popc(ldw(s.b1, b * 32u + lane, s.b1_words));
    c = __reduce_add_sync(0xffffffffu, c);
    if (lane == 0) cnt1[b] = (int32_t)c;
}

// in-place exclusive scan of n int32 values by one CTA of 1024 threads
__global__ void __launch_bounds__(1024) k_excl_scan(const int32_t *in, int32_t *out, uint32_t n)
{
    __shared__ uint32_t warp_tot[32];
    __shared__ uint32_t carry_s;
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (uint32_t base = 0; base < n; base += 1024) {
        uint32_t i = base + threadIdx.x;
        uint32_t v = i < n ? (uint32_t)in[i] : 0u;
        uint32_t inc = warp_incl_scan(v, lane);
        if (lane == 31) warp_tot[wid] = inc;
        __syncthreads();
        if (wid == 0) {
            uint32_t t = warp_tot[lane];
            uint32_t ti = warp_incl_scan(t, lane);
            warp_tot[lane] = ti - t;
        }
        __syncthreads();
        uint32_t carry = carry_s;
        uint32_t excl = carry + warp_tot[wid] + inc - v;
        if (i < n) out[i] = (int32_t)excl;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = excl + v;
        __syncthreads();
    }
}

// number of set B2 bits in bit range [r0, r1), computed by one warp
__device__ __forceinline__ uint32_t b2_range_count(const Streams &s, uint32_t r0, uint32_t r1, int lane)
{
    uint32_t c = 0;
    if (r1 > r0) {
        uint32_t w0 = r0 >> 5, w1 = (r1 - 1) >> 5;
        for (uint32_t w = w0 + lane; w <= w1; w += 32) {
            uint32_t v = ldw(s.b2, w, s.b2_words);
            if (w == w0) v &= ~lowmask(r0 & 31u);
            if (w == w1) v &= lowmask(((r1 - 1) & 31u) + 1u);
            c += __popc(v);
        }
    }
    return __reduce_add_sync(0xffffffffu, c);
}

// cnt2[b] = number of level-2 elements in rank block b, from the B2 bits of
// the block's non-L1 rank range
__global__ void k_count_l2(Streams s, uint32_t nb, const int32_t *a_blk, const int32_t *cnt1, int32_t *cnt2)
{
    uint32_t b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= nb) return;
    uint32_t e0 = b * (uint32_t)kBlk;
    uint32_t e1 = min(e0 + (uint32_t)kBlk, s.n);
    uint32_t r0 = e0 - (uint32_t)a_blk[b];
    uint32_t r1 = r0 + (e1 - e0) - (uint32_t)cnt1[b];
    uint32_t c = b2_range_count(s, r0, r1, lane);
    if (lane == 0) cnt2[b] = (int32_t)c;
}

// q1[u], q2[u] at flat position u*gran from the block tables (one warp per unit)
__global__ void k_unit_prefix(Streams s, uint32_t gran, uint32_t n_units, const int32_t *a_blk,
                              const int32_t *c_blk, int32_t *q1, int32_t *q2)
{
    uint32_t u = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (u >= n_units) return;
    unsigned long long p64 = (unsigned long long)u * gran;
    uint32_t p = p64 > s.n ? s.n : (uint32_t)p64;
    uint32_t nb = (s.n + kBlk - 1) / kBlk;
    uint32_t b = p >> 10;
    uint32_t a, c;
    if (b >= nb) {   // p == n on a block boundary: totals = last block's prefix + its counts
        b = nb - 1;
    }
    uint32_t e0 = b * (uint32_t)kBlk;
    // level-1 elements in [e0, p): whole words plus a masked partial word
    uint32_t wi = (e0 >> 5) + lane;
    uint32_t v = ldw(s.b1, wi, s.b1_words);
    uint32_t nfull = (p - e0) >> 5, rem = (p - e0) & 31u;
    if ((uint32_t)lane > nfull) v = 0;
    else if ((uint32_t)lane == nfull) v &= lowmask(rem);
    uint32_t k1 = __reduce_add_sync(0xffffffffu, __popc(v));
    a = (uint32_t)a_blk[b] + k1;
    uint32_t r0 = e0 - (uint32_t)a_blk[b];
    uint32_t r1 = p - a;
    c = (uint32_t)c_blk[b] + b2_range_count(s, r0, r1, lane);
    if (lane == 0) { q1[u] = (int32_t)a; q2[u] = (int32_t)c; }
}

// ------------------------------------------------------------- decode -------
// One warp per rank block, lane = bitmap word.  OUT = 0: int8 codes, 1: bf16.
template <int OUT>
__global__ void __launch_bounds__(256) k_decode(Streams s, const int32_t *q1, const int32_t *q2, void *out)
{
    __shared__ __align__(2048) uint32_t tab[kTabEntries];
    float sc = __bfloat162float(*s.scale);
    for (int e = threadIdx.x; e < kTabEntries; e += blockDim.x) {
        int code = tab_code(e);
        if (OUT == 0) tab[e] = (uint32_t)(code & 0xff);
        else tab[e] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn((float)code * sc));
    }
    __syncthreads();
    uint32_t nb = (s.n + kBlk - 1) / kBlk;
    uint32_t b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (b >= nb) return;
    uint32_t e0 = (b * 32u + lane) * 32u;
    uint32_t valid = e0 >= s.n ? 0u : min(32u, s.n - e0);
    GlobalSrc src{s};
    WordRanks w = block_ranks(src, ldw(s.b1, b * 32u + lane, s.b1_words), b, (uint32_t)q1[b], (uint32_t)q2[b], lane, valid);
    WordCursors c = word_cursors(w);
    const uint32_t tab_addr = (uint32_t)__cvta_generic_to_shared(tab);
    constexpr int kPer = OUT == 0 ? 4 : 2;          // elements per 32-bit output register
    constexpr int kBits = OUT == 0 ? 8 : 16;
    if (__any_sync(0xffffffffu, c.max_l3 > 3u || valid != 32u)) {
        // rare: a group with more than 3 level-3 elements, or the tensor's ragged end
        if (OUT == 0) {
            int8_t *o = (int8_t *)out + e0;
            decode_word_any(src, w, c, tab, [](int) {}, [&](int i, uint32_t v) { if ((uint32_t)i < valid) o[i] = (int8_t)v; });
        } else {
            uint16_t *o = (uint16_t *)out + e0;
            decode_word_any(src, w, c, tab, [](int) {}, [&](int i, uint32_t v) { if ((uint32_t)i < valid) o[i] = (uint16_t)v; });
        }
        return;
    }
    uint32_t r[32 / kPer];
#pragma unroll
    for (int i = 0; i < 32 / kPer; ++i) r[i] = 0;
    decode_word_fast(src, w, c, tab_addr, [](int) {}, [&](int i, uint32_t v) { r[i / kPer] |= v << (kBits * (i % kPer)); });
    uint4 *o = (uint4 *)((char *)out + (size_t)e0 * (OUT == 0 ? 1 : 2));
#pragma unroll
    for (int j = 0; j < 8 / kPer; ++j) o[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
}

// --------------------------------------------------------------- gemv -------
// Work split: the tensor's rank blocks are dealt to warps in contiguous runs of
// `bpw` blocks.  Each warp streams its run through a private ring of
// shared-memory slots filled with cp.async one block ahead of the decoder.  A
// warp sums, per output row it touches, the products of its run; a row that
// lies entirely inside one run is written straight to y, a row shared between
// runs goes to one fp32 slot per (row, run) and is summed in run order by the
// last CTA to finish (no atomics on data, same bits every run).
constexpr int kGemvThreads = 512;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvCtasPerSm = 1;
constexpr int kStages = 2;
constexpr uint32_t kGemvSmemBudget = 200u * 1024u;

// where the kernel reads activations from
enum XMode { kXF32Smem = 0, kXBf16Smem = 1, kXBf16Global = 2 };

struct GemvPlan {
    uint32_t nb;        // rank blocks
    uint32_t grid;      // CTAs
    uint32_t warps;     // total warps
    uint32_t bpw;       // blocks per warp
    uint32_t pmax;      // slots per row
    uint32_t xmode;     // XMode
    uint32_t smem;      // dynamic shared memory bytes
};

static GemvPlan make_plan(uint32_t out_f, uint32_t in_f, uint32_t m_rows)
{
    GemvPlan p;
    unsigned long long n = (unsigned long long)out_f * in_f;
    p.nb = (uint32_t)((n + kBlk - 1) / kBlk);
    uint32_t max_grid = (uint32_t)num_sms() * kGemvCtasPerSm;
    uint32_t want = (p.nb + kGemvWarps - 1) / kGemvWarps;
    p.grid = want < max_grid ? want : max_grid;
    if (p.grid == 0) p.grid = 1;
    p.warps = p.grid * kGemvWarps;
    p.bpw = (p.nb + p.warps - 1) / p.warps;
    uint32_t row_blocks = (in_f + kBlk - 1) / kBlk + 1;   // blocks one row can touch
    p.pmax = (row_blocks + p.bpw - 1) / p.bpw + 1;
    uint32_t fixed = 2048u + kGemvWarps * kStages * Slot::kWords * 4u;   // alignment slack + rings
    uint32_t x32 = m_rows * ((in_f + 1023u) / 1024u) * 4096u, x16 = m_rows * in_f * 2u;
    if (fixed + x32 <= kGemvSmemBudget) { p.xmode = kXF32Smem; p.smem = fixed + x32; }
    else if (fixed + x16 <= kGemvSmemBudget) { p.xmode = kXBf16Smem; p.smem = fixed + x16; }
    else { p.xmode = kXBf16Global; p.smem = fixed; }
    return p;
}

__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

template <int M, int XM>
__global__ void __launch_bounds__(kGemvThreads, kGemvCtasPerSm)
k_gemv(Streams s, const int32_t *__restrict__ q1, const int32_t *__restrict__ q2,
       const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ bias, void *y, int y_f32,
       float *slots, uint32_t *ticket, GemvPlan plan)
{
    extern __shared__ __align__(16) uint32_t smem[];
    __shared__ uint32_t is_last;
    uint32_t *ring = smem + (threadIdx.x >> 5) * (kStages * Slot::kWords);
    uint32_t *xs_raw = smem + kGemvWarps * kStages * Slot::kWords;
    uint32_t s2;
    {
        uint32_t sb = (uint32_t)__bfloat16_as_ushort(*s.scale);
        s2 = sb | (sb << 16);
        if (XM == kXF32Smem) {
            // fp32 copy of x, laid out so that the 32 lanes of a warp (consecutive 32-element
            // words) read consecutive 16-byte chunks: element k of a row sits at
            //   ((k / 1024) * 8 + (k % 32) / 4) * 128 + ((k / 32) % 32) * 4 + k % 4
            const uint32_t xstride = ((s.in_f + 1023u) / 1024u) * 1024u;
            for (uint32_t i = threadIdx.x; i < (uint32_t)M * s.in_f; i += blockDim.x) {
                uint32_t m = i / s.in_f, k = i - m * s.in_f;
                uint32_t pos = ((k >> 10) * 8u + ((k & 31u) >> 2)) * 128u + ((k >> 5) & 31u) * 4u + (k & 3u);
                ((float *)xs_raw)[m * xstride + pos] = __bfloat162float(x[i]);
            }
        } else if (XM == kXBf16Smem) {
            uint32_t nchunk = (uint32_t)M * s.in_f / 8u;   // in_f % 32 == 0
            for (uint32_t c = threadIdx.x; c < nchunk; c += blockDim.x)
                ((uint4 *)xs_raw)[c] = __ldg((const uint4 *)x + c);
        }
    }
    const float *xs32 = (const float *)xs_raw;
    const __nv_bfloat16 *xs16 = XM == kXBf16Global ? x : (const __nv_bfloat16 *)xs_raw;
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const uint32_t gw = blockIdx.x * kGemvWarps + (threadIdx.x >> 5);
    const uint32_t b_begin = gw * plan.bpw;
    const uint32_t b_end = min(b_begin + plan.bpw, plan.nb);

    auto emit = [&](uint32_t row, const float (&acc)[M]) {
        // all words of `row` inside this warp's run?
        uint32_t fb = (uint32_t)(((unsigned long long)row * s.in_f) >> 10);
        uint32_t lb = (uint32_t)((((unsigned long long)(row + 1) * s.in_f) - 1) >> 10);
        bool whole = fb >= b_begin && lb < b_end;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float v = warp_sum(acc[m]);
            if (lane == 0) {
                if (whole) {
                    size_t o = (size_t)m * s.out_f + row;
                    if (y_f32) {
                        ((float *)y)[o] = bias ? v + __bfloat162float(bias[row]) : v;
                    } else {
                        __nv_bfloat16 h = __float2bfloat16_rn(v);
                        if (bias) h = __hadd(h, bias[row]);
                        ((__nv_bfloat16 *)y)[o] = h;
                    }
                } else {
                    uint32_t piece = gw - fb / plan.bpw;
                    slots[((size_t)m * s.out_f + row) * plan.pmax + piece] = v;
                }
            }
        }
    };

    if (b_begin < b_end) {
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        uint32_t cur_row = (uint32_t)(((unsigned long long)b_begin * kBlk) / s.in_f);

        // rank-table entries of the current block and the two after it
        uint32_t a0 = (uint32_t)__ldg(q1 + b_begin), c0 = (uint32_t)__ldg(q2 + b_begin);
        uint32_t a1 = 0, c1 = 0;
        if (b_begin + 1 < plan.nb) { a1 = (uint32_t)__ldg(q1 + b_begin + 1); c1 = (uint32_t)__ldg(q2 + b_begin + 1); }
        const StageRole ra = role_a(s, lane), rb = role_b(s, lane);
        SlotSrc cur = stage_block(s, ra, rb, b_begin, b_begin + 1 == plan.nb, a0, c0, a1, c1, ring, lane);
        cp_async_commit();

        for (uint32_t b = b_begin; b < b_end; ++b) {
            const uint32_t st = (b - b_begin) % kStages;
            uint32_t *slot = ring + st * Slot::kWords;
            // start fetching the next block of the run while this one is decoded
            SlotSrc nxt = cur;
            uint32_t a2 = 0, c2 = 0;
            if (b + 1 < b_end) {
                if (b + 2 < plan.nb) { a2 = (uint32_t)__ldg(q1 + b + 2); c2 = (uint32_t)__ldg(q2 + b + 2); }
                nxt = stage_block(s, ra, rb, b + 1, b + 2 == plan.nb, a1, c1, a2, c2,
                                  ring + ((st + 1) % kStages) * Slot::kWords, lane);
            }
            cp_async_commit();
            cp_async_wait<1>();
            __syncwarp();

            uint32_t e0 = (b * 32u + lane) * 32u;
            uint32_t valid = e0 < s.n ? 32u : 0u;
            WordRanks w;
            if (cur.too_big) w = block_ranks(GlobalSrc{s}, ldw(s.b1, b * 32u + lane, s.b1_words), b, a0, c0, lane, valid);
            else w = block_ranks(cur, valid ? slot[Slot::kB1 + lane] : 0u, b, a0, c0, lane, valid);
            uint32_t lrow = valid ? e0 / s.in_f : 0xffffffffu;
            uint32_t k0 = valid ? e0 - lrow * s.in_f : 0u;
            // float4 index of this word's first chunk in the swizzled fp32 copy of x
            const uint32_t xstride = ((s.in_f + 1023u) / 1024u) * 1024u;
            const uint32_t xword = (k0 >> 10) * 256u + ((k0 >> 5) & 31u);
            WordCursors c = word_cursors(w);
            float part[M];
#pragma unroll
            for (int m = 0; m < M; ++m) part[m] = 0.f;
            if (cur.too_big || __any_sync(0xffffffffu, c.max_l3 > 4u)) {
                // rare: a group of 8 elements holds more than 4 level-3 values, or the block's
                // slices did not fit the slot (then everything is read from global memory)
                float sc = __uint_as_float(s2 << 16);
                auto slow_sink = [&](int i, int code) {
                    float wt = __bfloat162float(__float2bfloat16_rn((float)code * sc));
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        float xf = XM == kXF32Smem
                                       ? xs32[(size_t)m * xstride + xword * 4u + ((uint32_t)i >> 2) * 128u + ((uint32_t)i & 3u)]
                                       : __bfloat162float(xs16[(size_t)m * s.in_f + k0 + i]);
                        part[m] = fmaf(xf, wt, part[m]);
                    }
                };
                if (cur.too_big) decode_word_slow(GlobalSrc{s}, w, c, slow_sink);
                else decode_word_slow(cur, w, c, slow_sink);
            } else if (XM == kXF32Smem) {
                float4 xa[M], xb[M];
                decode_word_arith(
                    cur, w, c, s2,
                    [&](int q) {
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            const float4 *px = (const float4 *)(xs32 + (size_t)m * xstride) + xword + 64 * q;
                            xa[m] = px[0];
                            xb[m] = px[32];
                        }
                    },
                    [&](int i, uint32_t v) {
                        float wt = __uint_as_float(v);
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            const int j = i & 7;
                            float xf = j == 0 ? xa[m].x : j == 1 ? xa[m].y : j == 2 ? xa[m].z : j == 3 ? xa[m].w
                                     : j == 4 ? xb[m].x : j == 5 ? xb[m].y : j == 6 ? xb[m].z : xb[m].w;
                            part[m] = fmaf(xf, wt, part[m]);
                        }
                    });
            } else {
                uint4 xv[M];
                decode_word_arith(
                    cur, w, c, s2,
                    [&](int q) {
#pragma unroll
                        for (int m = 0; m < M; ++m) xv[m] = *((const uint4 *)(xs16 + (size_t)m * s.in_f + k0) + q);
                    },
                    [&](int i, uint32_t v) {
                        float wt = __uint_as_float(v);
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            const int j = i & 7;
                            uint32_t pr = j < 2 ? xv[m].x : (j < 4 ? xv[m].y : (j < 6 ? xv[m].z : xv[m].w));
                            float xf = (j & 1) ? bf16hi(pr) : bf16lo(pr);
                            part[m] = fmaf(xf, wt, part[m]);
                        }
                    });
            }
            if (!valid) {
#pragma unroll
                for (int m = 0; m < M; ++m) part[m] = 0.f;
            }
            // fold this word's sums into the per-row accumulators
            if (__all_sync(0xffffffffu, !valid || lrow == cur_row)) {
#pragma unroll
                for (int m = 0; m < M; ++m) acc[m] += part[m];
            } else {
                bool used = !valid;
                while (true) {
                    if (!used && lrow == cur_row) {
#pragma unroll
                        for (int m = 0; m < M; ++m) acc[m] += part[m];
                        used = true;
                    }
                    uint32_t pending = __ballot_sync(0xffffffffu, !used);
                    if (!pending) break;
                    emit(cur_row, acc);
#pragma unroll
                    for (int m = 0; m < M; ++m) acc[m] = 0.f;
                    cur_row = __shfl_sync(0xffffffffu, lrow, __ffs(pending) - 1);
                }
            }
            // a row that ends exactly at this block's end is complete
            uint32_t next_e = (b + 1) * (uint32_t)kBlk;
            if (next_e >= s.n || next_e == (cur_row + 1) * s.in_f) {
                emit(cur_row, acc);
#pragma unroll
                for (int m = 0; m < M; ++m) acc[m] = 0.f;
                cur_row += 1;
            }
            __syncwarp();
            cur = nxt;
            a0 = a1; c0 = c1; a1 = a2; c1 = c2;
        }
        cp_async_wait<0>();
        // run ended inside a row
        uint32_t end_e = min(b_end * (uint32_t)kBlk, s.n);
        if (end_e < s.n && end_e != cur_row * s.in_f) emit(cur_row, acc);
    }

    // ---- last CTA sums the rows that were shared between runs
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t t = atomicAdd(ticket, 1u);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    uint32_t n_runs = (plan.nb + plan.bpw - 1) / plan.bpw;
    for (uint32_t g = 1 + threadIdx.x; g < n_runs; g += blockDim.x) {
        unsigned long long e = (unsigned long long)g * plan.bpw * kBlk;   // first element of run g
        uint32_t row = (uint32_t)(e / s.in_f);
        unsigned long long row_e0 = (unsigned long long)row * s.in_f;
        if (e == row_e0) continue;                                   // run starts on a row boundary
        unsigned long long prev = (unsigned long long)(g - 1) * plan.bpw * kBlk;
        if (prev > row_e0) continue;                                 // an earlier run boundary owns this row
        uint32_t fb = (uint32_t)(row_e0 >> 10);
        uint32_t lb = (uint32_t)((row_e0 + s.in_f - 1) >> 10);
        uint32_t np = lb / plan.bpw - fb / plan.bpw + 1;
        for (int m = 0; m < M; ++m) {
            const float *sl = slots + ((size_t)m * s.out_f + row) * plan.pmax;
            float v = 0.f;
            for (uint32_t p = 0; p < np; ++p) v += __ldcg(sl + p);
            size_t o = (size_t)m * s.out_f + row;
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

template <int M, int XM>
static void launch_gemv_x(const Streams &s, const int32_t *q1, const int32_t *q2, const void *x, const void *bias,
                          void *y, int y_f32, float *slots, uint32_t *ticket, const GemvPlan &p, cudaStream_t st)
{
    static bool attr_set[64] = {false};
    (void)opt_in_smem(k_gemv<M, XM>, attr_set, (int)kGemvSmemBudget);   // on failure the launch below fails and is reported
    k_gemv<M, XM><<<p.grid, kGemvThreads, p.smem, st>>>(s, q1, q2, (const __nv_bfloat16 *)x,
                                                        (const __nv_bfloat16 *)bias, y, y_f32, slots, ticket, p);
}

template <int M>
static void launch_gemv(const Streams &s, const int32_t *q1, const int32_t *q2, const void *x, const void *bias,
                        void *y, int y_f32, float *slots, uint32_t *ticket, const GemvPlan &p, cudaStream_t st)
{
    if (p.xmode == kXF32Smem) launch_gemv_x<M, kXF32Smem>(s, q1, q2, x, bias, y, y_f32, slots, ticket, p, st);
    else if (p.xmode == kXBf16Smem) launch_gemv_x<M, kXBf16Smem>(s, q1, q2, x, bias, y, y_f32, slots, ticket, p, st);
    else launch_gemv_x<M, kXBf16Global>(s, q1, q2, x, bias, y, y_f32, slots, ticket, p, st);
}

}  // namespace ixb

// =============================================================== C ABI =======
using namespace ixb;

extern "C" int ixb_version(void) { return 100; }
extern "C" const char *ixb_last_error(void) { return g_err; }
extern "C" int64_t ixb_launch_count(void) { return (int64_t)g_launches.load(); }

extern "C" size_t ixb_prefix_workspace_bytes(int64_t n_elements)
{
    size_t nb = (size_t)((n_elements + kBlk - 1) / kBlk);
    return 4 * nb * sizeof(int32_t) + 256;
}

extern "C" int ixb_prefix_tables(const ixb_packed *w, int64_t gran, int64_t n_units, int32_t *q1, int32_t *q2,
                                 void *ws, size_t ws_bytes, ixb_stream_t stream)
{
    Streams s;
    int rc = to_streams(w, &s);
    if (rc) return rc;
    if (!q1 || !q2 || !ws) return fail(IXB_E_ARG, "q1/q2/workspace is NULL");
    if (gran <= 0 || n_units <= 0) return fail(IXB_E_ARG, "gran and n_units must be positive");
    if ((unsigned long long)(n_units - 1) * (unsigned long long)gran > s.n)
        return fail(IXB_E_ARG, "unit %lld starts beyond the tensor", (long long)(n_units - 1));
    if (gran > 0x7fffffffLL) return fail(IXB_E_ARG, "gran too large");
    if (ws_bytes < ixb_prefix_workspace_bytes(s.n)) return fail(IXB_E_SCRATCH, "prefix workspace too small");
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t nb = (s.n + kBlk - 1) / kBlk;
    int32_t *cnt1 = (int32_t *)ws, *a_blk = cnt1 + nb, *cnt2 = a_blk + nb, *c_blk = cnt2 + nb;
    uint32_t grid = (nb + 7) / 8;
    k_count_l1<<<grid, 256, 0, st>>>(s, nb, cnt1);
    if ((rc = launch_check("k_count_l1"))) return rc;
    k_excl_scan<<<1, 1024, 0, st>>>(cnt1, a_blk, nb);
    if ((rc = launch_check("k_excl_scan"))) return rc;
    k_count_l2<<<grid, 256, 0, st>>>(s, nb, a_blk, cnt1, cnt2);
    if ((rc = launch_check("k_count_l2"))) return rc;
    k_excl_scan<<<1, 1024, 0, st>>>(cnt2, c_blk, nb);
    if ((rc = launch_check("k_excl_scan"))) return rc;
    k_unit_prefix<<<(unsigned)((n_units + 7) / 8), 256, 0, st>>>(s, (uint32_t)gran, (uint32_t)n_units, a_blk, c_blk, q1, q2);
    return launch_check("k_unit_prefix");
}

extern "C" int ixb_decode(const ixb_packed *w, const int32_t *blk_q1, const int32_t *blk_q2, void *out, int out_kind,
                          ixb_stream_t stream)
{
    Streams s;
    int rc = to_streams(w, &s);
    if (rc) return rc;
    if (!blk_q1 || !blk_q2 || !out) return fail(IXB_E_ARG, "table/output pointer is NULL");
    if ((uintptr_t)out & 15u) return fail(IXB_E_ARG, "output is not 16-byte aligned");
    uint32_t nb = (s.n + kBlk - 1) / kBlk;
    cudaStream_t st = (cudaStream_t)stream;
    if (out_kind == 0) k_decode<0><<<(nb + 7) / 8, 256, 0, st>>>(s, blk_q1, blk_q2, out);
    else if (out_kind == 1) k_decode<1><<<(nb + 7) / 8, 256, 0, st>>>(s, blk_q1, blk_q2, out);
    else return fail(IXB_E_ARG, "out_kind must be 0 (int8 codes) or 1 (bf16)");
    return launch_check("k_decode");
}

extern "C" size_t ixb_gemv_scratch_bytes(int64_t out_f, int64_t in_f, int64_t m_rows)
{
    if (out_f <= 0 || in_f <= 0 || m_rows <= 0) return 0;
    GemvPlan p = make_plan((uint32_t)out_f, (uint32_t)in_f, (uint32_t)m_rows);
    return 256 + (size_t)m_rows * (size_t)out_f * p.pmax * sizeof(float);
}

extern "C" int ixb_gemv(const ixb_packed *w, const int32_t *blk_q1, const int32_t *blk_q2, const void *x,
                        int64_t m_rows, const void *bias, void *y, int y_is_f32, void *scratch, size_t scratch_bytes,
                        ixb_stream_t stream)
{
    Streams s;
    int rc = to_streams(w, &s);
    if (rc) return rc;
    if (!blk_q1 || !blk_q2 || !x || !y || !scratch) return fail(IXB_E_ARG, "NULL pointer argument");
    if (m_rows < 1 || m_rows > 8) return fail(IXB_E_UNSUPPORTED, "m_rows=%lld outside 1..8", (long long)m_rows);
    if (s.in_f % 32u) return fail(IXB_E_UNSUPPORTED, "in_f=%u is not a multiple of 32", s.in_f);
    if ((uintptr_t)x & 15u) return fail(IXB_E_ARG, "x is not 16-byte aligned");
    if (scratch_bytes < ixb_gemv_scratch_bytes(s.out_f, s.in_f, m_rows)) return fail(IXB_E_SCRATCH, "gemv scratch too small");
    GemvPlan p = make_plan(s.out_f, s.in_f, (uint32_t)m_rows);
    uint32_t *ticket = (uint32_t *)scratch;
    float *slots = (float *)((char *)scratch + 256);
    cudaStream_t st = (cudaStream_t)stream;
    switch (m_rows) {
    case 1: launch_gemv<1>(s, blk_q1, blk_q2, x, bias, y, y_is_f32, slots, ticket, p, st); break;
    case 2: launch_gemv<2>(s, blk_q1, blk_q2, x, bias, y, y_is_f32, slots, ticket, p, st); break;
    case 3: launch_gemv<3>(s, blk_q1, blk_q2, x, bias, y, y_is_f32, slots, ticket, p, st); break;
    case 4: launch_gemv<4>(s, blk_q1, blk_q2, x, bias, y, y_is_f32, slots, ticket, p, st); break;
    case 5: launch_gemv<5>(s, blk_q1, blk_q2, x, bias, y, y_is_f32, slots, ticket, p, st); break;
    case 6: launch_gemv<6>(s, blk_q1, blk_q2, x, bias, y, y_is_f32, slots, ticket, p, st); break;
    case 7: launch_gemv<7>(s, blk_q1, blk_q2, x, bias, y, y_is_f32, slots, ticket, p, st); break;
    default: launch_gemv<8>(s, blk_q1, blk_q2, x, bias, y, y_is_f32, slots, ticket, p, st); break;
    }
    return launch_check("k_gemv");
}

// ------------------------------------------------------------ quantise + pack
extern "C" size_t ixb_pack_workspace_bytes(int64_t n_elements)
{
    size_t nb = (size_t)((n_elements + kBlk - 1) / kBlk);
    return 256 + 4 * nb * sizeof(int32_t);
}

// workspace layout: [0] absmax bits, [1..2] unused, [64..] cnt1 | a_blk | cnt2 | c_blk (nb int32 each)
static int counts_and_tables(int mode, const void *w, int8_t *codes, uint32_t n, uint32_t *b1, void *scale,
                             int32_t *blk_q1, int32_t *blk_q2, int64_t *counts_host, void *ws, size_t ws_bytes,
                             cudaStream_t st)
{
    if (ws_bytes < ixb_pack_workspace_bytes(n)) return fail(IXB_E_SCRATCH, "pack workspace too small");
    uint32_t nb = (n + kBlk - 1) / kBlk;
    uint32_t *absmax = (uint32_t *)ws;
    int32_t *cnt1 = (int32_t *)((char *)ws + 256), *cnt2 = cnt1 + nb;
    int rc;
    if (mode == 0) {
        IXB_CUDA(cudaMemsetAsync(absmax, 0, 4, st));
        k_absmax<<<(unsigned)min(1024u, (n + 255) / 256), 256, 0, st>>>((const uint16_t *)w, n, absmax);
        if ((rc = launch_check("k_absmax"))) return rc;
        k_codes_and_counts<0><<<(nb + 7) / 8, 256, 0, st>>>((const uint16_t *)w, absmax, codes, n, b1, cnt1, cnt2,
                                                            (__nv_bfloat16 *)scale);
    } else {
        k_codes_and_counts<1><<<(nb + 7) / 8, 256, 0, st>>>(nullptr, absmax, codes, n, b1, cnt1, cnt2, nullptr);
    }
    if ((rc = launch_check("k_codes_and_counts"))) return rc;
    k_excl_scan<<<1, 1024, 0, st>>>(cnt1, blk_q1, nb);
    if ((rc = launch_check("k_excl_scan"))) return rc;
    k_excl_scan<<<1, 1024, 0, st>>>(cnt2, blk_q2, nb);
    if ((rc = launch_check("k_excl_scan"))) return rc;
    // totals = last prefix + last count; the caller sizes the streams from them
    int32_t last[4];
    IXB_CUDA(cudaMemcpyAsync(&last[0], blk_q1 + nb - 1, 4, cudaMemcpyDeviceToHost, st));
    IXB_CUDA(cudaMemcpyAsync(&last[1], cnt1 + nb - 1, 4, cudaMemcpyDeviceToHost, st));
    IXB_CUDA(cudaMemcpyAsync(&last[2], blk_q2 + nb - 1, 4, cudaMemcpyDeviceToHost, st));
    IXB_CUDA(cudaMemcpyAsync(&last[3], cnt2 + nb - 1, 4, cudaMemcpyDeviceToHost, st));
    IXB_CUDA(cudaStreamSynchronize(st));
    counts_host[0] = (int64_t)last[0] + last[1];
    counts_host[1] = (int64_t)last[2] + last[3];
    counts_host[2] = (int64_t)n - counts_host[0] - counts_host[1];
    return IXB_OK;
}

extern "C" int ixb_quantize_codes(const void *w_bf16, int64_t n_elements, void *scale_bf16, int8_t *codes,
                                  void *b1, int32_t *blk_q1, int32_t *blk_q2, int64_t *counts_host, void *ws,
                                  size_t ws_bytes, ixb_stream_t stream)
{
    if (!w_bf16 || !scale_bf16 || !codes || !b1 || !blk_q1 || !blk_q2 || !counts_host || !ws)
        return fail(IXB_E_ARG, "NULL pointer argument");
    if (n_elements <= 0 || n_elements > 800000000LL) return fail(IXB_E_ARG, "bad element count %lld", (long long)n_elements);
    return counts_and_tables(0, w_bf16, codes, (uint32_t)n_elements, (uint32_t *)b1, scale_bf16, blk_q1, blk_q2,
                             counts_host, ws, ws_bytes, (cudaStream_t)stream);
}

extern "C" int ixb_count_codes(const int8_t *codes, int64_t n_elements, void *b1, int32_t *blk_q1, int32_t *blk_q2,
                               int64_t *counts_host, void *ws, size_t ws_bytes, ixb_stream_t stream)
{
    if (!codes || !b1 || !blk_q1 || !blk_q2 || !counts_host || !ws) return fail(IXB_E_ARG, "NULL pointer argument");
    if (n_elements <= 0 || n_elements > 800000000LL) return fail(IXB_E_ARG, "bad element count %lld", (long long)n_elements);
    return counts_and_tables(1, nullptr, (int8_t *)codes, (uint32_t)n_elements, (uint32_t *)b1, nullptr, blk_q1, blk_q2,
                             counts_host, ws, ws_bytes, (cudaStream_t)stream);
}

extern "C" int ixb_pack_codes(const int8_t *codes, const ixb_packed *out, const int32_t *blk_q1, const int32_t *blk_q2,
                              ixb_stream_t stream)
{
    Streams s;
    int rc = to_streams(out, &s);
    if (rc) return rc;
    if (!codes || !blk_q1 || !blk_q2) return fail(IXB_E_ARG, "NULL pointer argument");
    cudaStream_t st = (cudaStream_t)stream;
    if (s.b2_words) IXB_CUDA(cudaMemsetAsync((void *)s.b2, 0, (size_t)s.b2_words * 4, st));
    if (s.l1_words) IXB_CUDA(cudaMemsetAsync((void *)s.l1, 0, (size_t)s.l1_words * 4, st));
    if (s.l2_words) IXB_CUDA(cudaMemsetAsync((void *)s.l2, 0, (size_t)s.l2_words * 4, st));
    uint32_t nb = (s.n + kBlk - 1) / kBlk;
    k_pack<<<(nb + 7) / 8, 256, 0, st>>>(codes, s.n, blk_q1, blk_q2, (uint32_t *)s.b2, (uint32_t *)s.l1,
                                         (uint32_t *)s.l2, (uint8_t *)s.l3);
    return launch_check("k_pack");
}

extern "C" int ixb_group_scale(const int8_t *codes, const void *group_scales_fp16, int64_t n, int64_t group, void *out,
                               ixb_stream_t stream)
{
    if (!codes || !group_scales_fp16 || !out) return fail(IXB_E_ARG, "NULL pointer argument");
    if (n <= 0 || n > 0x7fffffffLL || group <= 0) return fail(IXB_E_ARG, "bad size");
    const uint32_t threads = (uint32_t)((n + 7) / 8);
    k_group_scale<<<(threads + 255) / 256, 256, 0, (cudaStream_t)stream>>>(codes, (const __half *)group_scales_fp16, (uint32_t)n,
                                                                         (uint32_t)group, (__nv_bfloat16 *)out);
    return launch_check("k_group_scale");
}

// ------------------------------------------------------------- TPAB tile format
static int to_tpab(const ixb_tpab *t, Tpab *p)
{
    if (!t) return fail(IXB_E_ARG, "TPAB tensor is NULL");
    if (!t->body || !t->bits || !t->scales || !t->goff) return fail(IXB_E_ARG, "NULL TPAB pointer");
    if (t->out_f <= 0 || t->in_f <= 0 || (t->in_f & 63)) return fail(IXB_E_ARG, "in_f must be a positive multiple of 64");
    if (t->tile_r < 1 || t->tile_r > 64 || (t->tile_r & (t->tile_r - 1)) || t->out_f % t->tile_r)
        return fail(IXB_E_ARG, "tile_r must be a power of two <= 64 that divides out_f");
    if ((long long)t->out_f * t->in_f > 800000000LL) return fail(IXB_E_UNSUPPORTED, "tensor too large");
    p->body = (const uint32_t *)t->body;
    p->bits = (const uint8_t *)t->bits;
    p->scales = (const __half *)t->scales;
    p->goff = (const int32_t *)t->goff;
    for (int b = 0; b < 8; ++b) p->gbase[b] = t->gbase_bit[b];
    p->out_f = (uint32_t)t->out_f;
    p->in_f = (uint32_t)t->in_f;
    p->tile_r = (uint32_t)t->tile_r;
    p->t_c = p->in_f / 64u;
    p->t_r = p->out_f / p->tile_r;
    return IXB_OK;
}

extern "C" int ixb_tpab_decode(const ixb_tpab *t, const int32_t *ol_t, const int32_t *ol_l, const void *ol_val_fp16,
                               int64_t n_ol, void *out, ixb_stream_t stream)
{
    Tpab p;
    int rc = to_tpab(t, &p);
    if (rc) return rc;
    if (!out || ((uintptr_t)out & 15u)) return fail(IXB_E_ARG, "output is NULL or misaligned");
    if (n_ol < 0 || (n_ol && (!ol_t || !ol_l || !ol_val_fp16))) return fail(IXB_E_ARG, "bad outlier arrays");
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t rows = p.t_r * p.t_c * p.tile_r;
    k_tpab_decode<<<(rows + 127) / 128, 128, 0, st>>>(p, (__nv_bfloat16 *)out);
    if ((rc = launch_check("k_tpab_decode"))) return rc;
    if (n_ol) {
        k_tpab_scatter<<<(unsigned)((n_ol + 255) / 256), 256, 0, st>>>(p, ol_t, ol_l, (const __half *)ol_val_fp16, (uint32_t)n_ol,
                                                                     (__nv_bfloat16 *)out);
        rc = launch_check("k_tpab_scatter");
    }
    return rc;
}

static uint32_t tpab_splits(uint32_t t_r, uint32_t t_c)
{
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    uint32_t s = std::max<uint32_t>(1u, (2u * (uint32_t)sms) / t_r);
    s = std::min<uint32_t>(s, std::max<uint32_t>(1u, t_c / (uint32_t)kTpabWarps));
    return std::min<uint32_t>(s, 32u);
}

extern "C" size_t ixb_tpab_gemv_scratch_bytes(int64_t out_f, int64_t in_f, int64_t tile_r)
{
    if (out_f <= 0 || in_f <= 0 || (in_f & 63) || tile_r < 1 || out_f % tile_r) return 0;
    return (size_t)tpab_splits((uint32_t)(out_f / tile_r), (uint32_t)(in_f / 64)) * (size_t)out_f * sizeof(float);
}

extern "C" int ixb_tpab_gemv(const ixb_tpab *t, const void *x, const int32_t *ol_offs, const int32_t *ol_k, const void *ol_v_fp16,
                             const void *bias, void *y, int y_is_f32, void *scratch, size_t scratch_bytes, ixb_stream_t stream)
{
    Tpab p;
    int rc = to_tpab(t, &p);
    if (rc) return rc;
    if (!x || !y || !scratch) return fail(IXB_E_ARG, "NULL pointer argument");
    if ((uintptr_t)x & 3u) return fail(IXB_E_ARG, "x is misaligned");
    if (ol_offs && (!ol_k || !ol_v_fp16)) return fail(IXB_E_ARG, "bad outlier arrays");
    if (scratch_bytes < ixb_tpab_gemv_scratch_bytes(p.out_f, p.in_f, p.tile_r)) return fail(IXB_E_SCRATCH, "TPAB scratch too small");
    const uint32_t splits = tpab_splits(p.t_r, p.t_c);
    cudaStream_t st = (cudaStream_t)stream;
    k_tpab_gemv<<<dim3(p.t_r, splits), kTpabWarps * 32, 0, st>>>(p, (const __nv_bfloat16 *)x, (float *)scratch, splits);
    if ((rc = launch_check("k_tpab_gemv"))) return rc;
    k_tpab_finalize<<<(p.out_f + 255) / 256, 256, 0, st>>>((const float *)scratch, splits, p.out_f, ol_offs, ol_k,
                                                           (const __half *)ol_v_fp16, (const __nv_bfloat16 *)x,
                                                           (const __nv_bfloat16 *)bias, y, y_is_f32);
    return launch_check("k_tpab_finalize");
}

// ------------------------------------------------------------- resident P6 layout
extern "C" int64_t ixb_p6_blocks(int64_t out_f, int64_t in_f)
{
    if (out_f <= 0 || in_f <= 0) return 0;
    return ((out_f + kTileRows - 1) / kTileRows) * ((in_f + kTileCols - 1) / kTileCols);
}

static int to_p6(const ixb_p6 *t, P6 *p)
{
    if (!t) return fail(IXB_E_ARG, "P6 tensor is NULL");
    if (t->out_f <= 0 || t->in_f <= 0) return fail(IXB_E_ARG, "bad shape");
    long long n = (long long)t->out_f * t->in_f;
    if (n > 800000000LL) return fail(IXB_E_UNSUPPORTED, "tensor too large");
    if (!t->plane || !t->blk_off || !t->esc || !t->scale) return fail(IXB_E_ARG, "NULL P6 pointer");
    if (((uintptr_t)t->plane & 15u) || ((uintptr_t)t->esc & 15u)) return fail(IXB_E_ARG, "P6 plane or entries are misaligned");
    p->plane = (const unsigned char *)t->plane;
    p->blk_off = (const int32_t *)t->blk_off;
    p->esc = (const uint32_t *)t->esc;
    p->scale = (const __nv_bfloat16 *)t->scale;
    if (t->scale_stride != 0 && t->scale_stride != 1) return fail(IXB_E_ARG, "scale_stride must be 0 or 1");
    p->scale_stride = (uint32_t)t->scale_stride;
    p->out_f = (uint32_t)t->out_f;
    p->in_f = (uint32_t)t->in_f;
    p->rt = (p->out_f + kTileRows - 1) / kTileRows;
    p->kb = (p->in_f + kTileCols - 1) / kTileCols;
    return IXB_OK;
}

extern "C" int ixb_p6_build(const int8_t *codes, const void *scale, int64_t scale_stride, int64_t out_f, int64_t in_f,
                            void *plane, int32_t *blk_off, void *esc, int64_t n_esc, void *ws, size_t ws_bytes,
                            ixb_stream_t stream)
{
    if (!codes || !scale || !plane || !blk_off || !esc || !ws) return fail(IXB_E_ARG, "NULL pointer argument");
    if (scale_stride != 0 && scale_stride != 1) return fail(IXB_E_ARG, "scale_stride must be 0 or 1");
    if (out_f <= 0 || in_f <= 0 || out_f * in_f > 800000000LL) return fail(IXB_E_ARG, "bad shape");
    if (n_esc < 0) return fail(IXB_E_ARG, "bad outlier count");
    if (((uintptr_t)plane & 15u) || ((uintptr_t)esc & 15u)) return fail(IXB_E_ARG, "P6 plane or entries are misaligned");
    uint32_t rt = (uint32_t)((out_f + kTileRows - 1) / kTileRows), kb = (uint32_t)((in_f + kTileCols - 1) / kTileCols);
    uint32_t nb = rt * kb, n_off = nb + 1;
    if (ws_bytes < (size_t)n_off * 4) return fail(IXB_E_SCRATCH, "P6 workspace too small");
    cudaStream_t st = (cudaStream_t)stream;
    int32_t *blk_cnt = (int32_t *)ws;
    int rc;
    // the slack behind the plane and the entries is zero: it is read, never interpreted
    IXB_CUDA(cudaMemsetAsync(blk_cnt, 0, (size_t)n_off * 4, st));
    IXB_CUDA(cudaMemsetAsync((char *)plane + (size_t)nb * kP6BlockBytes, 0, (size_t)kP6SlackBlocks * kP6BlockBytes, st));
    IXB_CUDA(cudaMemsetAsync((char *)esc + (size_t)n_esc * 4, 0, (size_t)kP6SlackEntries * 4, st));
    k_p6_plane<<<(nb + 7) / 8, 256, 0, st>>>(codes, (uint32_t)out_f, (uint32_t)in_f, rt, kb, (unsigned char *)plane, blk_cnt);
    if ((rc = launch_check("k_p6_plane"))) return rc;
    k_excl_scan<<<1, 1024, 0, st>>>(blk_cnt, blk_off, n_off);      // entry nb = total
    if ((rc = launch_check("k_excl_scan"))) return rc;
    if (n_esc) {
        k_p6_esc<<<(nb + 7) / 8, 256, 0, st>>>(codes, (uint32_t)out_f, (uint32_t)in_f, rt, kb, blk_off,
                                               (const __nv_bfloat16 *)scale, (uint32_t)scale_stride, (uint32_t *)esc,
                                               (uint32_t)n_esc);
        if ((rc = launch_check("k_p6_esc"))) return rc;
    }
    return IXB_OK;
}

extern "C" int ixb_p6_decode(const ixb_p6 *t, void *out, int out_kind, ixb_stream_t stream)
{
    P6 p;
    int rc = to_p6(t, &p);
    if (rc) return rc;
    if (!out) return fail(IXB_E_ARG, "NULL output");
    if (out_kind != 0 && out_kind != 1) return fail(IXB_E_ARG, "out_kind must be 0 (int8 codes) or 1 (bf16 weights)");
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t nb = p.rt * p.kb;
    if (out_kind == 1 && (p.in_f & 7u) == 0 && ((uintptr_t)out & 15u) == 0) {
        k_p6_decode_bf16<<<(nb + 7) / 8, 256, 0, st>>>(p, (__nv_bfloat16 *)out);       // plane and outliers in one pass
        return launch_check("k_p6_decode_bf16");
    }
    if (out_kind == 0) k_p6_decode_plane<0><<<(nb + 7) / 8, 256, 0, st>>>(p, out);
    else k_p6_decode_plane<1><<<(nb + 7) / 8, 256, 0, st>>>(p, out);
    if ((rc = launch_check("k_p6_decode_plane"))) return rc;
    if (t->n_esc) {
        if (out_kind == 0) k_p6_decode_esc<0><<<(nb + 7) / 8, 256, 0, st>>>(p, out);
        else k_p6_decode_esc<1><<<(nb + 7) / 8, 256, 0, st>>>(p, out);
        rc = launch_check("k_p6_decode_esc");
    }
    return rc;
}

struct P6Plan { uint32_t nb, grid, xstride, smem, xs, cq, cr, unit; size_t slot_bytes; };

static P6Plan make_p6_plan(uint32_t out_f, uint32_t in_f, uint32_t m_rows)
{
    P6Plan p;
    uint32_t rt = (out_f + kTileRows - 1) / kTileRows, kb = (in_f + kTileCols - 1) / kTileCols;
    p.nb = rt * kb;
    uint32_t sms = (uint32_t)num_sms();
    uint32_t want = (p.nb + kP6Warps - 1) / kP6Warps;
    p.grid = want < sms ? want : sms;
    if (!p.grid) p.grid = 1;
    p.unit = 1;
    {
        // Balanced to one block, row tiles at CTA boundaries are finished across CTAs: slot store, fence, ticket and
        // slot loads, about 3.4 us at the end of the kernel, worth about 170 blocks of streaming (11.5 us for the 588
        // blocks per CTA of the 5120 x 17408 layer).  Whole row tiles per CTA avoid that at the price of imbalance.
        const uint32_t tgrid = rt < sms ? rt : sms;
        static const uint32_t handover_blocks = []() -> uint32_t {
            const char *e = getenv("IXB200_P6_HANDOVER_BLOCKS");       // tuning knob; default from measurements on B200
            return e && *e ? (uint32_t)atoi(e) : 170u;
        }();
        const uint32_t shared_cost = (p.nb + p.grid - 1) / p.grid + handover_blocks;
        const uint32_t tiles_cost = ((rt + tgrid - 1) / tgrid) * kb;
        if (tiles_cost <= shared_cost) {
            p.grid = tgrid;
            p.unit = kb;
        }
    }
    const uint32_t units = p.nb / p.unit;
    p.cq = units / p.grid;
    p.cr = units % p.grid;
    p.xstride = kb * kTileCols + 8u;
    uint32_t xbytes = m_rows * p.xstride * 2u;
    p.xs = (uint32_t)kP6SmemFixed + xbytes <= 227u * 1024u;
    p.smem = (uint32_t)kP6SmemFixed + (p.xs ? xbytes : 0u);
    p.slot_bytes = (size_t)p.grid * 2u * 32u * sizeof(float4);
    return p;
}

extern "C" size_t ixb_p6_gemv_scratch_bytes(int64_t out_f, int64_t in_f, int64_t m_rows)
{
    if (out_f <= 0 || in_f <= 0 || m_rows <= 0) return 0;
    P6Plan p = make_p6_plan((uint32_t)out_f, (uint32_t)in_f, (uint32_t)m_rows);
    return 1024 + p.slot_bytes;
}

// Programmatic dependent launch for the P6 GEMV (off by default).  When on, a launch may begin before the kernel
// ahead of it in the stream has finished: it fetches its first weight blocks and outlier entries, then waits for that
// kernel to complete before it touches the activations, y or the scratch.
static std::atomic<int> g_p6_pdl{0};

extern "C" int ixb_set_pdl(int on) { return g_p6_pdl.exchange(on ? 1 : 0); }

template <int XS>
static cudaError_t launch_p6(const P6 &p, const void *x, uint32_t m_rows, const void *bias, void *y, int y_f32,
                             float4 *slots, uint32_t *tickets, const P6Plan &pl, const P6Push &push, cudaStream_t st)
{
    static bool attr_set[64] = {false};
    cudaError_t oe = opt_in_smem(k_p6_mma<XS>, attr_set, 227 * 1024);
    if (oe != cudaSuccess) return oe;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.grid);
    cfg.blockDim = dim3(kP6Threads);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_p6_pdl.load() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k_p6_mma<XS>, p, (const __nv_bfloat16 *)x, m_rows, (const __nv_bfloat16 *)bias, y, y_f32,
                              slots, tickets, pl.nb, pl.xstride, pl.cq, pl.cr, pl.unit, push);
}

static int p6_gemv_impl(const ixb_p6 *t, const void *x, int64_t m_rows, const void *bias, void *y, int y_is_f32,
                        void *scratch, size_t scratch_bytes, const P6Push &push, ixb_stream_t stream)
{
    P6 p;
    int rc = to_p6(t, &p);
    if (rc) return rc;
    if (!x || (!y && (!push.world || push.fin)) || !scratch) return fail(IXB_E_ARG, "NULL pointer argument");
    if (m_rows < 1 || m_rows > 8) return fail(IXB_E_UNSUPPORTED, "m_rows=%lld outside 1..8", (long long)m_rows);
    if ((uintptr_t)x & 15u) return fail(IXB_E_ARG, "x is not 16-byte aligned");
    if ((uintptr_t)scratch & 15u) return fail(IXB_E_ARG, "scratch is not 16-byte aligned");
    if (scratch_bytes < ixb_p6_gemv_scratch_bytes(p.out_f, p.in_f, m_rows)) return fail(IXB_E_SCRATCH, "gemv scratch too small");
    if (push.world && (size_t)m_rows * p.out_f > push.n_max)
        return fail(IXB_E_ARG, "m_rows * out_f = %lld exceeds the all-reduce buffer's n_max", (long long)(m_rows * p.out_f));
    P6Plan pl = make_p6_plan(p.out_f, p.in_f, (uint32_t)m_rows);
    if (!pl.xs && (p.in_f % kTileCols))
        return fail(IXB_E_UNSUPPORTED, "in_f=%u: activations too large for shared memory need in_f %% 64 == 0", p.in_f);
    uint32_t *tickets = (uint32_t *)scratch;                  // the first 1024 bytes hold the tile tickets (grid + 1 words) ...
    float4 *slots = (float4 *)((char *)scratch + 1024);
    P6Push pu = push;
    pu.done = tickets + 255;                                   // ... and, in the last word, the count of finished warps
    if (pu.fin && ((p.out_f & 1u) || pl.grid * (uint32_t)kP6Threads * 2u < (uint32_t)m_rows * p.out_f))
        return fail(IXB_E_UNSUPPORTED, "a finishing GEMV needs an even out_f and at most %u outputs", pl.grid * (uint32_t)kP6Threads * 2u);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = pl.xs ? launch_p6<1>(p, x, (uint32_t)m_rows, bias, y, y_is_f32, slots, tickets, pl, pu, st)
                          : launch_p6<0>(p, x, (uint32_t)m_rows, bias, y, y_is_f32, slots, tickets, pl, pu, st);
    if (e != cudaSuccess) return fail(IXB_E_CUDA, "k_p6_mma launch: %s", cudaGetErrorString(e));
    return launch_check("k_p6_mma");
}

extern "C" int ixb_p6_gemv(const ixb_p6 *t, const void *x, int64_t m_rows, const void *bias, void *y, int y_is_f32,
                           void *scratch, size_t scratch_bytes, ixb_stream_t stream)
{
    P6Push push = {};
    return p6_gemv_impl(t, x, m_rows, bias, y, y_is_f32, scratch, scratch_bytes, push, stream);
}

// ------------------------------------------------------- one-shot all-reduce over peer memory
extern "C" size_t ixb_allreduce_bytes(int world, int64_t n_max)
{
    if (world < 1 || world > kArMaxWorld || n_max <= 0 || (n_max & 3)) return 0;
    // slots, call counters, one error word; rounded up to 256 bytes
    size_t b = ar_slots_bytes(world, n_max) + ((size_t)ar_counters(n_max) + 1) * 4;
    return (b + 255) & ~(size_t)255;
}

static std::atomic<uint32_t> g_ar_spin_limit{kArSpinLimit};

extern "C" uint32_t ixb_allreduce_spin_limit(uint32_t polls) { return g_ar_spin_limit.exchange(polls ? polls : kArSpinLimit); }

template <int W>
static cudaError_t launch_ar(const ArPeers &peers, const void *x, int rank, uint32_t n, uint32_t n_max, const void *bias,
                             void *y, int y_f32, uint32_t *epoch, uint32_t *err, cudaStream_t st)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ar_ctas(n_max));
    cfg.blockDim = dim3(kArThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_p6_pdl.load() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k_allreduce_oneshot<W>, peers, (const float *)x, rank, n, n_max,
                              (const __nv_bfloat16 *)bias, y, y_f32, epoch, err, g_ar_spin_limit.load());
}

extern "C" int ixb_allreduce(const void *x, int64_t n, void *const *peer_buffers, int rank, int world, int64_t n_max,
                             const void *bias, void *y, int y_is_f32, ixb_stream_t stream)
{
    if (!x || !y || !peer_buffers) return fail(IXB_E_ARG, "NULL pointer argument");
    if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) return fail(IXB_E_ARG, "bad rank/world");
    if (n <= 0 || n > n_max || (n & 3) || (n_max & 3)) return fail(IXB_E_ARG, "n must be a multiple of 4 and at most n_max");
    if (((uintptr_t)x & 15u) || ((uintptr_t)y & 7u)) return fail(IXB_E_ARG, "x / y are misaligned");
    ArPeers peers;
    const size_t sb = ar_slots_bytes(world, n_max);
    const uint32_t ctas = ar_counters(n_max);
    for (int r = 0; r < world; ++r) {
        if (!peer_buffers[r] || ((uintptr_t)peer_buffers[r] & 15u)) return fail(IXB_E_ARG, "peer buffer %d is NULL or misaligned", r);
        peers.slots[r] = (uint2 *)peer_buffers[r];
    }
    for (int r = world; r < kArMaxWorld; ++r) peers.slots[r] = nullptr;
    uint32_t *epoch = (uint32_t *)((char *)peer_buffers[rank] + sb), *err = epoch + ctas;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    switch (world) {
    case 1: e = launch_ar<1>(peers, x, rank, (uint32_t)n, (uint32_t)n_max, bias, y, y_is_f32, epoch, err, st); break;
    case 2: e = launch_ar<2>(peers, x, rank, (uint32_t)n, (uint32_t)n_max, bias, y, y_is_f32, epoch, err, st); break;
    case 4: e = launch_ar<4>(peers, x, rank, (uint32_t)n, (uint32_t)n_max, bias, y, y_is_f32, epoch, err, st); break;
    case 8: e = launch_ar<8>(peers, x, rank, (uint32_t)n, (uint32_t)n_max, bias, y, y_is_f32, epoch, err, st); break;
    default: return fail(IXB_E_UNSUPPORTED, "world=%d: supported sizes are 1, 2, 4, 8", world);
    }
    if (e != cudaSuccess) return fail(IXB_E_CUDA, "k_allreduce_oneshot launch: %s", cudaGetErrorString(e));
    return launch_check("k_allreduce_oneshot");
}

// ---- the same exchange with the senders' half inside the GEMV: ixb_p6_gemv_push + ixb_allreduce_finish
static int ar_geometry(void *const *peer_buffers, int rank, int world, int64_t n_max, P6Push *push, uint32_t **epoch,
                       uint32_t **err)
{
    if (!peer_buffers) return fail(IXB_E_ARG, "NULL pointer argument");
    if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) return fail(IXB_E_ARG, "bad rank/world");
    if (world != 1 && world != 2 && world != 4 && world != 8) return fail(IXB_E_UNSUPPORTED, "world=%d: supported sizes are 1, 2, 4, 8", world);
    if (n_max <= 0 || (n_max & 3)) return fail(IXB_E_ARG, "n_max must be a positive multiple of 4");
    for (int r = 0; r < world; ++r) {
        if (!peer_buffers[r] || ((uintptr_t)peer_buffers[r] & 15u)) return fail(IXB_E_ARG, "peer buffer %d is NULL or misaligned", r);
        push->slots[r] = (uint2 *)peer_buffers[r];
    }
    for (int r = world; r < 8; ++r) push->slots[r] = nullptr;
    *epoch = (uint32_t *)((char *)peer_buffers[rank] + ar_slots_bytes(world, n_max));
    *err = *epoch + ar_counters(n_max);
    push->epoch = *epoch;
    push->mine = push->slots[rank];
    push->world = (uint32_t)world;
    push->rank = (uint32_t)rank;
    push->n_max = (uint32_t)n_max;
    push->fin = 0;
    push->counters = ar_counters(n_max);
    push->spin_limit = g_ar_spin_limit.load();
    push->err = *err;
    push->done = nullptr;
    return IXB_OK;
}

extern "C" int ixb_p6_gemv_push(const ixb_p6 *t, const void *x, int64_t m_rows, void *const *peer_buffers, int rank,
                                int world, int64_t n_max, void *scratch, size_t scratch_bytes, ixb_stream_t stream)
{
    P6Push push;
    uint32_t *epoch, *err;
    int rc = ar_geometry(peer_buffers, rank, world, n_max, &push, &epoch, &err);
    if (rc) return rc;
    return p6_gemv_impl(t, x, m_rows, nullptr, nullptr, 1, scratch, scratch_bytes, push, stream);
}

extern "C" int ixb_p6_gemv_allreduce(const ixb_p6 *t, const void *x, int64_t m_rows, void *const *peer_buffers, int rank,
                                     int world, int64_t n_max, const void *bias, void *y, int y_is_f32, void *scratch,
                                     size_t scratch_bytes, ixb_stream_t stream)
{
    P6Push push;
    uint32_t *epoch, *err;
    int rc = ar_geometry(peer_buffers, rank, world, n_max, &push, &epoch, &err);
    if (rc) return rc;
    if (((uintptr_t)y & 7u)) return fail(IXB_E_ARG, "y is misaligned");
    push.fin = 1;
    return p6_gemv_impl(t, x, m_rows, bias, y, y_is_f32, scratch, scratch_bytes, push, stream);
}

template <int W>
static cudaError_t launch_ar_finish(const uint2 *mine, uint32_t n, uint32_t n_max, const void *bias, void *y, int y_f32,
                                    uint32_t *epoch, uint32_t *err, cudaStream_t st)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ar_fin_ctas(n_max));
    cfg.blockDim = dim3(kArFinThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_p6_pdl.load() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k_allreduce_finish<W>, mine, n, n_max, (const __nv_bfloat16 *)bias, y, y_f32, epoch, err,
                              g_ar_spin_limit.load());
}

extern "C" int ixb_allreduce_finish(void *const *peer_buffers, int rank, int world, int64_t n, int64_t n_max,
                                    const void *bias, void *y, int y_is_f32, ixb_stream_t stream)
{
    P6Push push;
    uint32_t *epoch, *err;
    int rc = ar_geometry(peer_buffers, rank, world, n_max, &push, &epoch, &err);
    if (rc) return rc;
    if (!y) return fail(IXB_E_ARG, "NULL pointer argument");
    if (n <= 0 || n > n_max || (n & 3)) return fail(IXB_E_ARG, "n must be a multiple of 4 and at most n_max");
    if ((uintptr_t)y & 7u) return fail(IXB_E_ARG, "y is misaligned");
    cudaStream_t st = (cudaStream_t)stream;
    const uint2 *mine = push.mine;
    cudaError_t e;
    switch (world) {
    case 1: e = launch_ar_finish<1>(mine, (uint32_t)n, (uint32_t)n_max, bias, y, y_is_f32, epoch, err, st); break;
    case 2: e = launch_ar_finish<2>(mine, (uint32_t)n, (uint32_t)n_max, bias, y, y_is_f32, epoch, err, st); break;
    case 4: e = launch_ar_finish<4>(mine, (uint32_t)n, (uint32_t)n_max, bias, y, y_is_f32, epoch, err, st); break;
    default: e = launch_ar_finish<8>(mine, (uint32_t)n, (uint32_t)n_max, bias, y, y_is_f32, epoch, err, st); break;
    }
    if (e != cudaSuccess) return fail(IXB_E_CUDA, "k_allreduce_finish launch: %s", cudaGetErrorString(e));
    return launch_check("k_allreduce_finish");
}

// ------------------------------------------------------- per-token glue kernels
// one launch with the programmatic-stream-serialization attribute when ixb_set_pdl is on
template <class... KArgs, class... Args>
static cudaError_t launch_glue(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_p6_pdl.load() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#define IXB_GLUE(what, call)                                                                    \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) return fail(IXB_E_CUDA, "%s launch: %s", what, cudaGetErrorString(e_)); \
        return launch_check(what);                                                            \
    } while (0)

static bool norm_vector_ok(const void *h, const void *delta, const void *w, const void *xn, int64_t hidden, int64_t limit)
{
    return (hidden & 7) == 0 && hidden <= limit &&
           ((((uintptr_t)h | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)xn) & 15u) == 0);
}

extern "C" int ixb_add_rmsnorm(void *h, const void *delta, const void *w, float eps, void *xn, int64_t rows,
                               int64_t hidden, ixb_stream_t stream)
{
    if (!h || !w || !xn) return fail(IXB_E_ARG, "NULL pointer argument");
    if (rows <= 0 || hidden <= 0 || rows > 65535) return fail(IXB_E_ARG, "bad shape");
    if (norm_vector_ok(h, delta, w, xn, hidden, 8192)) {
        const unsigned threads = (unsigned)(((hidden / 8) + 31) / 32 * 32);
        NormExchange none = {};
        IXB_GLUE("k_add_rmsnorm", launch_glue(k_add_rmsnorm<0>, dim3((unsigned)rows), dim3(threads), (cudaStream_t)stream,
                                              (__nv_bfloat16 *)h, (const __nv_bfloat16 *)delta, none, (const __nv_bfloat16 *)w,
                                              eps, (__nv_bfloat16 *)xn, (uint32_t)hidden));
    }
    IXB_GLUE("k_add_rmsnorm_any", launch_glue(k_add_rmsnorm_any, dim3((unsigned)rows), dim3(hidden >= 4096 ? 1024 : 256), (cudaStream_t)stream,
                                              (__nv_bfloat16 *)h, (const __nv_bfloat16 *)delta, (const __nv_bfloat16 *)w, eps,
                                              (__nv_bfloat16 *)xn, (uint32_t)hidden));
}

extern "C" int ixb_allreduce_finish_add_rmsnorm(void *const *peer_buffers, int rank, int world, int64_t n_max, void *h,
                                                const void *w, float eps, void *xn, int64_t rows, int64_t hidden,
                                                ixb_stream_t stream)
{
    P6Push push;
    uint32_t *epoch, *err;
    int rc = ar_geometry(peer_buffers, rank, world, n_max, &push, &epoch, &err);
    if (rc) return rc;
    if (!h || !w || !xn) return fail(IXB_E_ARG, "NULL pointer argument");
    if (rows <= 0 || rows > 8 || hidden <= 0 || rows * hidden > n_max) return fail(IXB_E_ARG, "bad shape");
    if (!norm_vector_ok(h, nullptr, w, xn, hidden, 8 * kNormExchangeThreads))
        return fail(IXB_E_UNSUPPORTED, "hidden=%lld: a multiple of 8, at most %d, 16-byte aligned rows", (long long)hidden,
                    8 * kNormExchangeThreads);
    NormExchange ex;
    ex.mine = push.mine;
    ex.epoch = epoch;
    ex.err = err;
    ex.world = (uint32_t)world;
    ex.n_max = (uint32_t)n_max;
    ex.counters = ar_counters(n_max);
    ex.spin_limit = g_ar_spin_limit.load();
    const unsigned threads = (unsigned)(((hidden / 8) + 31) / 32 * 32);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
#define IXB_NORM_EX(W)                                                                                                  \
    e = launch_glue(k_add_rmsnorm<W>, dim3((unsigned)rows), dim3(threads), st, (__nv_bfloat16 *)h, (const __nv_bfloat16 *)nullptr, \
                    ex, (const __nv_bfloat16 *)w, eps, (__nv_bfloat16 *)xn, (uint32_t)hidden)
    switch (world) {
    case 1: IXB_NORM_EX(1); break;
    case 2: IXB_NORM_EX(2); break;
    case 4: IXB_NORM_EX(4); break;
    default: IXB_NORM_EX(8); break;
    }
#undef IXB_NORM_EX
    if (e != cudaSuccess) return fail(IXB_E_CUDA, "k_add_rmsnorm (exchange) launch: %s", cudaGetErrorString(e));
    return launch_check("k_add_rmsnorm (exchange)");
}

extern "C" int ixb_swiglu(const void *g, const void *u, void *y, int64_t rows, int64_t cols, int64_t in_stride,
                          ixb_stream_t stream)
{
    if (!g || !u || !y) return fail(IXB_E_ARG, "NULL pointer argument");
    if (rows <= 0 || cols <= 0 || in_stride < cols || rows * cols > 0x7fffffffLL) return fail(IXB_E_ARG, "bad shape");
    const int vec = (cols & 7) == 0 && (in_stride & 7) == 0 && ((((uintptr_t)g | (uintptr_t)u | (uintptr_t)y) & 15u) == 0);
    const int64_t threads = vec ? rows * cols / 8 : rows * cols;
    IXB_GLUE("k_swiglu", launch_glue(k_swiglu, dim3((unsigned)((threads + 127) / 128)), dim3(128), (cudaStream_t)stream,
                                     (const __nv_bfloat16 *)g, (const __nv_bfloat16 *)u, (__nv_bfloat16 *)y, (uint32_t)rows,
                                     (uint32_t)cols, (uint32_t)in_stride, vec));
}

extern "C" int ixb_rope_kv(void *q, const void *k, const void *v, const int32_t *pos, void *k_cache, void *v_cache,
                           const void *q_norm, const void *k_norm, const float *cos_tab, const float *sin_tab, int64_t rows,
                           int64_t hq, int64_t hkv, int64_t head_dim, int64_t rot_dim, float eps, int64_t q_stride,
                           int64_t max_seq, int64_t kv_stride, int64_t batch_stride, ixb_stream_t stream)
{
    if (kv_stride < hkv * head_dim || batch_stride < 0 || q_stride < hq * head_dim) return fail(IXB_E_ARG, "bad strides");
    if (!q || !k || !v || !pos || !k_cache || !v_cache || !cos_tab || !sin_tab) return fail(IXB_E_ARG, "NULL pointer argument");
    if (rows <= 0 || hq <= 0 || hkv <= 0 || max_seq <= 0) return fail(IXB_E_ARG, "bad shape");
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return fail(IXB_E_UNSUPPORTED, "head_dim=%lld: 64, 128 or 256", (long long)head_dim);
    if (rot_dim <= 0 || rot_dim > head_dim || (rot_dim & 1)) return fail(IXB_E_ARG, "rot_dim must be even and at most head_dim");
    IXB_GLUE("k_rope_kv", launch_glue(k_rope_kv, dim3((unsigned)rows, (unsigned)(hq + hkv)), dim3((unsigned)(head_dim / 2)), (cudaStream_t)stream,
                                      (__nv_bfloat16 *)q, (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)v, pos,
                                      (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache, (const __nv_bfloat16 *)q_norm,
                                      (const __nv_bfloat16 *)k_norm, cos_tab, sin_tab, (uint32_t)hq, (uint32_t)hkv,
                                      (uint32_t)head_dim, (uint32_t)rot_dim, eps, (uint32_t)q_stride, (uint32_t)max_seq,
                                      (uint32_t)kv_stride, (size_t)batch_stride));
}

extern "C" size_t ixb_attn_scratch_bytes(int64_t hq, int64_t head_dim, int64_t splits)
{
    if (hq <= 0 || head_dim <= 0 || splits <= 0) return 0;
    return (size_t)hq * (size_t)splits * (size_t)(head_dim + 2) * sizeof(float);
}

template <int D>
static cudaError_t launch_attn(int64_t hq, int64_t hkv, int64_t splits, cudaStream_t st, const void *q, const void *k_cache,
                               const void *v_cache, const int32_t *pos, void *scratch, float scale, int64_t batch,
                               int64_t q_stride, int64_t batch_stride)
{
    const int64_t rep = hq / hkv;
#define IXB_ATTN(G)                                                                                                        \
    return launch_glue(k_attn_decode<D, G>, dim3((unsigned)(hq / G), (unsigned)splits, (unsigned)batch), dim3(256), st,   \
                       (const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k_cache, (const __nv_bfloat16 *)v_cache, pos,      \
                       (float *)scratch, (uint32_t)hq, (uint32_t)hkv, scale, (uint32_t)q_stride, (size_t)batch_stride)
    switch (rep) {                      // all query heads of a KV head in one CTA where that is a supported group size
    case 2: IXB_ATTN(2);
    case 3: IXB_ATTN(3);
    case 4: IXB_ATTN(4);
    case 6: IXB_ATTN(6);
    case 8: IXB_ATTN(8);
    default: IXB_ATTN(1);
    }
#undef IXB_ATTN
}

extern "C" int ixb_attn_decode(const void *q, const void *k_cache, const void *v_cache, const int32_t *pos, const void *gate,
                               int64_t gate_stride, void *out, void *scratch, size_t scratch_bytes, int64_t hq, int64_t hkv,
                               int64_t head_dim, int64_t splits, float scale, int64_t batch, int64_t q_stride,
                               int64_t batch_stride, int64_t gate_row_stride, ixb_stream_t stream)
{
    if (!q || !k_cache || !v_cache || !pos || !out || !scratch) return fail(IXB_E_ARG, "NULL pointer argument");
    if (hq <= 0 || hkv <= 0 || hq % hkv || splits <= 0 || splits > kAttnMaxSplits) return fail(IXB_E_ARG, "bad shape");
    if (batch < 1 || batch > 65535 || q_stride < 0 || batch_stride < 0 || (batch > 1 && (q_stride & 7))) return fail(IXB_E_ARG, "bad batch");
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return fail(IXB_E_UNSUPPORTED, "head_dim=%lld: 64, 128 or 256", (long long)head_dim);
    if (scratch_bytes < (size_t)batch * ixb_attn_scratch_bytes(hq, head_dim, splits)) return fail(IXB_E_SCRATCH, "attention scratch too small");
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15u) return fail(IXB_E_ARG, "q / caches are not 16-byte aligned");
    if ((uintptr_t)scratch & 7u) return fail(IXB_E_ARG, "attention scratch is misaligned");
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (head_dim == 64) e = launch_attn<64>(hq, hkv, splits, st, q, k_cache, v_cache, pos, scratch, scale, batch, q_stride, batch_stride);
    else if (head_dim == 128) e = launch_attn<128>(hq, hkv, splits, st, q, k_cache, v_cache, pos, scratch, scale, batch, q_stride, batch_stride);
    else e = launch_attn<256>(hq, hkv, splits, st, q, k_cache, v_cache, pos, scratch, scale, batch, q_stride, batch_stride);
    if (e != cudaSuccess) return fail(IXB_E_CUDA, "k_attn_decode launch: %s", cudaGetErrorString(e));
    int rc = launch_check("k_attn_decode");
    if (rc) return rc;
    const unsigned threads = (unsigned)std::max<int64_t>(head_dim, (splits + 31) / 32 * 32);
    IXB_GLUE("k_attn_combine", launch_glue(k_attn_combine, dim3((unsigned)hq, (unsigned)batch), dim3(threads), st, (const float *)scratch,
                                           (__nv_bfloat16 *)out, (const __nv_bfloat16 *)gate, (uint32_t)splits, (uint32_t)head_dim,
                                           (uint32_t)gate_stride, (uint32_t)gate_row_stride));
}

extern "C" int ixb_conv_update(const void *x, void *state, const void *w, const void *bias, void *y, int64_t channels,
                               int64_t k, ixb_stream_t stream)
{
    if (!x || !state || !w || !y) return fail(IXB_E_ARG, "NULL pointer argument");
    if (channels <= 0 || k < 2 || k > 8) return fail(IXB_E_ARG, "bad shape (kernel size 2..8)");
    if (k == 4 && (channels & 3) == 0 && ((((uintptr_t)x | (uintptr_t)state | (uintptr_t)y | (uintptr_t)bias) & 7u) == 0) &&
        ((uintptr_t)w & 15u) == 0) {
        IXB_GLUE("k_conv_update4", launch_glue(k_conv_update4, dim3((unsigned)((channels / 4 + 63) / 64)), dim3(64), (cudaStream_t)stream,
                                               (const __nv_bfloat16 *)x, (__nv_bfloat16 *)state, (const __nv_bfloat16 *)w,
                                               (const __nv_bfloat16 *)bias, (__nv_bfloat16 *)y, (uint32_t)channels));
    }
    IXB_GLUE("k_conv_update", launch_glue(k_conv_update, dim3((unsigned)((channels + 255) / 256)), dim3(256), (cudaStream_t)stream,
                                          (const __nv_bfloat16 *)x, (__nv_bfloat16 *)state, (const __nv_bfloat16 *)w,
                                          (const __nv_bfloat16 *)bias, (__nv_bfloat16 *)y, (uint32_t)channels, (uint32_t)k));
}

extern "C" int ixb_gdn_step(const void *qkv, const void *z, const void *a, const void *b, const float *A_log,
                            const float *dt_bias, const void *norm_w, float *state, void *out, int64_t hk, int64_t hv,
                            float eps, ixb_stream_t stream)
{
    if (!qkv || !z || !a || !b || !A_log || !dt_bias || !norm_w || !state || !out) return fail(IXB_E_ARG, "NULL pointer argument");
    if (hk <= 0 || hv <= 0 || hv % hk) return fail(IXB_E_ARG, "value heads must be a multiple of key heads");
    IXB_GLUE("k_gdn_step", launch_glue(k_gdn_step<false>, dim3((unsigned)hv), dim3(256), (cudaStream_t)stream, (const __nv_bfloat16 *)qkv,
                                       (const __nv_bfloat16 *)z, (const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, A_log, dt_bias,
                                       (const __nv_bfloat16 *)norm_w, state, (__nv_bfloat16 *)out, (uint32_t)hk, (uint32_t)hv, eps,
                                       (__nv_bfloat16 *)nullptr, (const __nv_bfloat16 *)nullptr, (const int32_t *)nullptr, 0u));
}

extern "C" int ixb_gdn_conv_step(const void *qkv_raw, void *conv_state, const void *conv_w, const int32_t *pos, const void *z,
                                 const void *a, const void *b, const float *A_log, const float *dt_bias, const void *norm_w,
                                 float *state, void *out, int64_t hk, int64_t hv, float eps, ixb_stream_t stream)
{
    if (!qkv_raw || !conv_state || !conv_w || !pos || !z || !a || !b || !A_log || !dt_bias || !norm_w || !state || !out)
        return fail(IXB_E_ARG, "NULL pointer argument");
    if (hk <= 0 || hv <= 0 || hv % hk) return fail(IXB_E_ARG, "value heads must be a multiple of key heads");
    const uint32_t C = (uint32_t)((2 * hk + hv) * 128);
    IXB_GLUE("k_gdn_step (conv)", launch_glue(k_gdn_step<true>, dim3((unsigned)hv), dim3(256), (cudaStream_t)stream,
                                              (const __nv_bfloat16 *)qkv_raw, (const __nv_bfloat16 *)z, (const __nv_bfloat16 *)a,
                                              (const __nv_bfloat16 *)b, A_log, dt_bias, (const __nv_bfloat16 *)norm_w, state,
                                              (__nv_bfloat16 *)out, (uint32_t)hk, (uint32_t)hv, eps, (__nv_bfloat16 *)conv_state,
                                              (const __nv_bfloat16 *)conv_w, pos, C));
}

// ------------------------------------------------------- tensor-core small-M GEMM
static TcPlan make_tc_plan(uint32_t out_f, uint32_t in_f)
{
    TcPlan p;
    p.n_kslab = in_f / (uint32_t)kTcSlab;
    p.n_rowtiles = (out_f + kTcRows - 1) / kTcRows;
    p.n_tiles = p.n_kslab * p.n_rowtiles;
    uint32_t sms = (uint32_t)num_sms();
    p.grid = p.n_tiles < sms ? p.n_tiles : sms;
    if (p.grid == 0) p.grid = 1;
    p.tiles_per_cta = (p.n_tiles + p.grid - 1) / p.grid;
    return p;
}

extern "C" size_t ixb_gemm_scratch_bytes(int64_t out_f, int64_t in_f, int64_t m_rows)
{
    if (out_f <= 0 || in_f <= 0 || m_rows <= 0 || in_f % kTcSlab) return 0;
    return 256 + (size_t)(in_f / kTcSlab) * (size_t)m_rows * (size_t)out_f * sizeof(float);
}

extern "C" int ixb_gemm(const ixb_packed *w, const int32_t *blk_q1, const int32_t *blk_q2, const void *x,
                        int64_t m_rows, const void *bias, void *y, int y_is_f32, void *scratch, size_t scratch_bytes,
                        ixb_stream_t stream)
{
    Streams s;
    int rc = to_streams(w, &s);
    if (rc) return rc;
    if (!blk_q1 || !blk_q2 || !x || !y || !scratch) return fail(IXB_E_ARG, "NULL pointer argument");
    if (m_rows < 1 || m_rows > kTcTok) return fail(IXB_E_UNSUPPORTED, "m_rows=%lld outside 1..%d", (long long)m_rows, kTcTok);
    if (s.in_f % (uint32_t)kTcSlab) return fail(IXB_E_UNSUPPORTED, "in_f=%u is not a multiple of %d", s.in_f, kTcSlab);
    if ((uintptr_t)x & 15u) return fail(IXB_E_ARG, "x is not 16-byte aligned");
    if (scratch_bytes < ixb_gemm_scratch_bytes(s.out_f, s.in_f, m_rows)) return fail(IXB_E_SCRATCH, "gemm scratch too small");
    TcPlan p = make_tc_plan(s.out_f, s.in_f);
    cudaStream_t st = (cudaStream_t)stream;
    static bool attr_set[64] = {false};
    IXB_CUDA(opt_in_smem(k_gemm_tc, attr_set, (int)kTcSmemBytes));
    uint32_t *err = (uint32_t *)scratch;
    float *part = (float *)((char *)scratch + 256);
    IXB_CUDA(cudaMemsetAsync(scratch, 0, 256, st));
    k_gemm_tc<<<p.grid, kTcThreads, kTcSmemBytes, st>>>(s, blk_q1, blk_q2, (const __nv_bfloat16 *)x, (uint32_t)m_rows,
                                                        part, err, p);
    if ((rc = launch_check("k_gemm_tc"))) return rc;
    uint32_t total = (uint32_t)m_rows * s.out_f;
    k_gemm_finalize<<<(total + 255) / 256, 256, 0, st>>>(part, p.n_kslab, (uint32_t)m_rows, s.out_f,
                                                         (const __nv_bfloat16 *)bias, y, y_is_f32, err);
    return launch_check("k_gemm_finalize");
}

// ------------------------------------------------ small-M GEMM on the resident P6 layout
static PgPlan make_pg_plan(uint32_t out_f, uint32_t in_f)
{
    PgPlan p;
    const uint32_t rt = (out_f + kTileRows - 1) / kTileRows, kb = (in_f + kTileCols - 1) / kTileCols;
    p.groups = (rt + kPgConv - 1) / kPgConv;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // K is split only as far as it takes to give about every SM one CTA; a split keeps at least eight column blocks
    uint32_t splits = std::max<uint32_t>(1u, (uint32_t)sms / p.groups);
    splits = std::min<uint32_t>(splits, std::max<uint32_t>(1u, kb / 8u));
    p.splits = std::min<uint32_t>(splits, 16u);
    p.grid = p.groups * p.splits;
    return p;
}

extern "C" size_t ixb_p6_gemm_scratch_bytes(int64_t out_f, int64_t in_f, int64_t m_rows)
{
    if (out_f <= 0 || in_f <= 0 || m_rows < 1 || m_rows > kPgTok || out_f * in_f > 800000000LL) return 0;
    PgPlan p = make_pg_plan((uint32_t)out_f, (uint32_t)in_f);
    return 256 + (size_t)p.splits * (size_t)m_rows * (size_t)out_f * sizeof(float);
}

extern "C" int ixb_p6_gemm(const ixb_p6 *t, const void *x, int64_t m_rows, const void *bias, void *y, int y_is_f32,
                           void *scratch, size_t scratch_bytes, ixb_stream_t stream)
{
    P6 p;
    int rc = to_p6(t, &p);
    if (rc) return rc;
    if (!x || !y || !scratch) return fail(IXB_E_ARG, "NULL pointer argument");
    if (m_rows < 1 || m_rows > kPgTok) return fail(IXB_E_UNSUPPORTED, "m_rows=%lld outside 1..%d", (long long)m_rows, kPgTok);
    if (p.in_f % (uint32_t)kTileCols) return fail(IXB_E_UNSUPPORTED, "in_f=%u is not a multiple of %d", p.in_f, kTileCols);
    if ((uintptr_t)x & 15u) return fail(IXB_E_ARG, "x is not 16-byte aligned");
    if ((uintptr_t)scratch & 255u) return fail(IXB_E_ARG, "scratch is not 256-byte aligned");
    if (scratch_bytes < ixb_p6_gemm_scratch_bytes(p.out_f, p.in_f, m_rows)) return fail(IXB_E_SCRATCH, "gemm scratch too small");
    PgPlan plan = make_pg_plan(p.out_f, p.in_f);
    cudaStream_t st = (cudaStream_t)stream;
    static bool attr_set[64] = {false};
    IXB_CUDA(opt_in_smem(k_p6_gemm, attr_set, (int)kPgSmemBytes));
    uint32_t *err = (uint32_t *)scratch;
    float *part = (float *)((char *)scratch + 256);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(kPgThreads);
    cfg.dynamicSmemBytes = kPgSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_p6_pdl.load() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, k_p6_gemm, p, (const __nv_bfloat16 *)x, (uint32_t)m_rows, part, err, plan);
    if (e != cudaSuccess) return fail(IXB_E_CUDA, "k_p6_gemm launch: %s", cudaGetErrorString(e));
    if ((rc = launch_check("k_p6_gemm"))) return rc;
    uint32_t total = (uint32_t)m_rows * p.out_f;
    IXB_GLUE("k_gemm_finalize", launch_glue(k_gemm_finalize, dim3((total + 255) / 256), dim3(256), st, (const float *)part,
                                            plan.splits, (uint32_t)m_rows, p.out_f, (const __nv_bfloat16 *)bias, y, y_is_f32,
                                            (const uint32_t *)err));
}

// ------------------------------------------------ gemv without caller scratch
// Scratch of ixb_gemv_static: one array per device that loads this library,
// resident until the process exits.  In host code the name below is only a
// handle for cudaGetSymbolAddress; the kernel receives the device address.
static __device__ __align__(256) unsigned char g_static_scratch[IXB_STATIC_SCRATCH_BYTES];

extern "C" int ixb_gemv_static(const ixb_packed *w, const int32_t *blk_q1, const int32_t *blk_q2, const void *x,
                               int64_t m_rows, const void *bias, void *y, int y_is_f32, ixb_stream_t stream)
{
    static void *dev_ptr[64] = {nullptr};   // device address of the array, per device ordinal
    if (!w) return fail(IXB_E_ARG, "packed tensor is NULL");
    size_t need = ixb_gemv_scratch_bytes(w->out_f, w->in_f, m_rows);
    if (need == 0) return fail(IXB_E_ARG, "bad shape or m_rows");
    if (need > (size_t)IXB_STATIC_SCRATCH_BYTES)
        return fail(IXB_E_SCRATCH,
                    "ixb_gemv_static: %lld x %lld with m_rows=%lld needs %zu bytes of scratch, the built-in array holds %d; "
                    "use ixb_gemv with caller scratch",
                    (long long)w->out_f, (long long)w->in_f, (long long)m_rows, need, IXB_STATIC_SCRATCH_BYTES);
    int dev = -1;
    IXB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(IXB_E_UNSUPPORTED, "device ordinal %d outside 0..63", dev);
    if (!dev_ptr[dev]) {
        // first call on this device: resolve the array's device address (the device is current)
        void *p = nullptr;
        IXB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        dev_ptr[dev] = p;
    }
    // the ticket word must start at zero whatever an earlier call left behind
    IXB_CUDA(cudaMemsetAsync(dev_ptr[dev], 0, 256, (cudaStream_t)stream));
    return ixb_gemv(w, blk_q1, blk_q2, x, m_rows, bias, y, y_is_f32, dev_ptr[dev], IXB_STATIC_SCRATCH_BYTES, stream);
}
