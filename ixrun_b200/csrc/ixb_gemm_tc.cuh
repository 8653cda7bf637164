// Fused decode + small-M GEMM on the 5th-generation tensor cores (tcgen05,
// accumulators in TMEM) for 1..64 activation rows; sm_100a only.
//
//   Y[t][n] = sum_k X[t][k] * bf16(code[n][k] * scale)        t < m_tok <= 64
//
// Tiling.  The tensor is cut into tiles of 16 weight rows x one 1024-element
// k-slab (= one rank block per row, so in_f must be a multiple of 1024).  The
// 16 warps of a CTA decode one row block each (same decoder and cp.async slots
// as the GEMV) and write bf16 weights into the shared-memory B operand; the
// activations of the k-slab sit in shared memory as the A operand; one thread
// then issues 64 tcgen05.mma (M = 64 tokens, N = 16 rows, K = 16 each) into a
// 64 x 16 fp32 accumulator in TMEM.  Four warps read the accumulator back
// (tcgen05.ld) and store it as the k-slab's partial result; a second small
// kernel sums the partials over the k-slabs in a fixed order (no atomics).
// CTAs walk tiles in k-slab-major order so the activation slab is reloaded
// only when the k-slab changes.
//
// Both operands use the K-major, no-swizzle canonical layout: 8 rows x 16
// bytes core matrices, LBO = byte distance between the two core matrices of a
// K = 16 step, SBO = byte distance between 8-row groups.
#pragma once
#include "ixb_common.cuh"

namespace ixb {

constexpr int kTcThreads = 512;
constexpr int kTcWarps = 16;
constexpr int kTcRows = 16;          // weight rows per tile (MMA N)
constexpr int kTcTok = 64;           // token rows of the MMA (M)
constexpr int kTcSlab = 1024;        // k elements per tile
constexpr uint32_t kTcABytes = kTcTok * kTcSlab * 2;     // 128 KB
constexpr uint32_t kTcBBytes = kTcRows * kTcSlab * 2;    //  32 KB
constexpr uint32_t kTcRingBytes = kTcWarps * 2 * Slot::kWords * 4;
constexpr uint32_t kTcSmemBytes = kTcABytes + kTcBBytes + kTcRingBytes + 64;
constexpr uint32_t kTcTmemCols = 32;
constexpr uint32_t kTcWaitLimit = 1u << 20;

struct TcPlan {
    uint32_t n_kslab, n_rowtiles, n_tiles, grid, tiles_per_cta;
};

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    // start address [0,14), leading byte offset [16,30), stride byte offset [32,46) (all >> 4),
    // descriptor version 1 at [46,48), no swizzle (layout type 0 at [61,64))
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)(lbo_bytes >> 4) << 16) |
           ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
}

// kind::f16, bf16 x bf16 -> fp32, both operands K-major, M = 64, N = 16
constexpr uint32_t kTcIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTcRows >> 3) << 17) |
                              ((uint32_t)(kTcTok >> 4) << 24);

__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity)
{
    for (uint32_t it = 0; it < kTcWaitLimit; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(mbar), "r"(parity) : "memory");
        if (done) return true;
        __nanosleep(32);
    }
    return false;   // gave up: the caller records an error and carries on
}

__global__ void __launch_bounds__(kTcThreads, 1)
k_gemm_tc(Streams s, const int32_t *__restrict__ q1, const int32_t *__restrict__ q2,
          const __nv_bfloat16 *__restrict__ x, uint32_t m_tok, float *__restrict__ part, uint32_t *err, TcPlan plan)
{
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    unsigned char *a_tile = tc_smem;
    unsigned char *b_tile = tc_smem + kTcABytes;
    uint32_t *ring_all = (uint32_t *)(tc_smem + kTcABytes + kTcBBytes);
    uint64_t *mbar_ptr = (uint64_t *)(tc_smem + kTcABytes + kTcBBytes + kTcRingBytes);
    uint32_t *tmem_slot = (uint32_t *)(mbar_ptr + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t *ring = ring_all + warp * (2 * Slot::kWords);
    const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(a_tile);
    const uint32_t b_addr = (uint32_t)__cvta_generic_to_shared(b_tile);
    const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(mbar_ptr);
    const uint32_t nkb = s.in_f / (uint32_t)kTcSlab;           // rank blocks per row
    const uint32_t nb = (s.n + kBlk - 1) / kBlk;
    uint32_t s2;
    {
        uint32_t sb = (uint32_t)__bfloat16_as_ushort(*s.scale);
        s2 = sb | (sb << 16);
    }

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        uint32_t slot_addr = (uint32_t)__cvta_generic_to_shared(tmem_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(kTcTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // token rows beyond m_tok stay zero for the whole kernel
    for (uint32_t c = tid; c < kTcABytes / 16; c += kTcThreads) ((uint4 *)a_tile)[c] = make_uint4(0, 0, 0, 0);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t t_begin = blockIdx.x * plan.tiles_per_cta;
    const uint32_t t_end = min(t_begin + plan.tiles_per_cta, plan.n_tiles);
    const StageRole ra = role_a(s, lane), rb = role_b(s, lane);
    uint32_t parity = 0, cur_kslab = 0xffffffffu;

    auto tile_block = [&](uint32_t t, uint32_t &row, uint32_t &kslab) {
        kslab = t / plan.n_rowtiles;
        row = (t - kslab * plan.n_rowtiles) * (uint32_t)kTcRows + warp;
        return row * nkb + kslab;
    };
    auto stage_tile = [&](uint32_t t, uint32_t stage, uint32_t &a0, uint32_t &c0) {
        uint32_t row, kslab;
        uint32_t b = tile_block(t, row, kslab);
        SlotSrc src;
        src.too_big = false;
        if (row < s.out_f) {
            a0 = (uint32_t)__ldg(q1 + b);
            c0 = (uint32_t)__ldg(q2 + b);
            uint32_t a1 = 0, c1 = 0;
            if (b + 1 < nb) { a1 = (uint32_t)__ldg(q1 + b + 1); c1 = (uint32_t)__ldg(q2 + b + 1); }
            src = stage_block(s, ra, rb, b, b + 1 == nb, a0, c0, a1, c1, ring + stage * Slot::kWords, lane);
        }
        return src;
    };

    uint32_t a0 = 0, c0 = 0;
    SlotSrc cur;
    cur.too_big = false;
    if (t_begin < t_end) cur = stage_tile(t_begin, 0, a0, c0);
    cp_async_commit();

    for (uint32_t t = t_begin; t < t_end; ++t) {
        const uint32_t st = (t - t_begin) & 1u;
        uint32_t row, kslab;
        const uint32_t b = tile_block(t, row, kslab);
        uint32_t na0 = 0, nc0 = 0;
        SlotSrc nxt = cur;
        if (t + 1 < t_end) nxt = stage_tile(t + 1, st ^ 1u, na0, nc0);
        cp_async_commit();

        if (kslab != cur_kslab) {
            // activations of this k-slab into the A operand (rows = tokens)
            for (uint32_t c = tid; c < m_tok * (kTcSlab / 8); c += kTcThreads) {
                uint32_t tok = c / (kTcSlab / 8), kg = c % (kTcSlab / 8);
                uint4 v = __ldg((const uint4 *)(x + (size_t)tok * s.in_f + (size_t)kslab * kTcSlab) + kg);
                *(uint4 *)(a_tile + kg * 1024u + (tok >> 3) * 128u + (tok & 7u) * 16u) = v;
            }
            cur_kslab = kslab;
        }

        cp_async_wait<1>();
        __syncwarp();
        // ---- decode this warp's row block into the B operand
        unsigned char *brow = b_tile + (uint32_t)(warp >> 3) * 128u + (uint32_t)(warp & 7) * 16u;
        if (row < s.out_f) {
            uint32_t *slot = ring + st * Slot::kWords;
            WordRanks w;
            if (cur.too_big) w = block_ranks(GlobalSrc{s}, ldw(s.b1, b * 32u + lane, s.b1_words), b, a0, c0, lane, 32u);
            else w = block_ranks(cur, slot[Slot::kB1 + lane], b, a0, c0, lane, 32u);
            WordCursors c = word_cursors(w);
            if (cur.too_big || __any_sync(0xffffffffu, c.max_l3 > 4u)) {
                float sc = __uint_as_float(s2 << 16);
                auto slow_sink = [&](int i, int code) {
                    uint32_t k = 32u * lane + (uint32_t)i;
                    *(__nv_bfloat16 *)(brow + (k >> 3) * 256u + (k & 7u) * 2u) = __float2bfloat16_rn((float)code * sc);
                };
                if (cur.too_big) decode_word_slow(GlobalSrc{s}, w, c, slow_sink);
                else decode_word_slow(cur, w, c, slow_sink);
            } else {
                uint32_t pk[16];
                uint32_t prev = 0;
                decode_word_arith(cur, w, c, s2, [](int) {}, [&](int i, uint32_t v) {
                    if (i & 1) pk[i >> 1] = __byte_perm(prev, v, 0x7632);
                    else prev = v;
                });
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *(uint4 *)(brow + (4u * lane + j) * 256u) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) *(uint4 *)(brow + (4u * lane + j) * 256u) = make_uint4(0, 0, 0, 0);
        }
        // make the generic-proxy writes of A and B visible to the tensor core (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();

        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint64_t da = umma_desc(a_addr, 1024u, 128u);
            uint64_t db = umma_desc(b_addr, 256u, 128u);
#pragma unroll 1
            for (uint32_t k = 0; k < kTcSlab / 16; ++k) {
                uint32_t acc = k ? 1u : 0u;
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                             "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                             :: "r"(tmem_base), "l"(da), "l"(db), "r"(kTcIdesc), "r"(acc), "r"(0u) : "memory");
                da += 2048u >> 4;     // two core matrices further along K
                db += 512u >> 4;
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
        }
        if (warp < 4) {
            // accumulator rows 16q..16q+15 live in lanes 32q..32q+15 of TMEM (M = 64 layout)
            bool ok = mbar_wait(mbar, parity);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t r[16];
            uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                           "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                         : "r"(taddr) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (!ok && lane == 0) atomicExch(err, 1u);
            uint32_t tok = (uint32_t)warp * 16u + (uint32_t)lane;
            if (lane < 16 && tok < m_tok) {
                uint32_t row0 = (t - kslab * plan.n_rowtiles) * (uint32_t)kTcRows;
                float *dst = part + ((size_t)kslab * m_tok + tok) * s.out_f + row0;
                if (row0 + 16u <= s.out_f && (s.out_f & 3u) == 0) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        ((float4 *)dst)[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                         __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                } else {
                    for (uint32_t j = 0; j < 16u && row0 + j < s.out_f; ++j) dst[j] = __uint_as_float(r[j]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        parity ^= 1u;
        __syncthreads();          // B operand and accumulator are free again
        cur = nxt;
        a0 = na0;
        c0 = nc0;
    }
    cp_async_wait<0>();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTcTmemCols) : "memory");
}

// y[t][n] = sum over k-slabs of the partial results, in slab order
// (takes part in programmatic dependent launch: nothing of it runs ahead of the dependency wait)
__global__ void k_gemm_finalize(const float *__restrict__ part, uint32_t n_kslab, uint32_t m_tok, uint32_t out_f,
                                const __nv_bfloat16 *__restrict__ bias, void *y, int y_f32, const uint32_t *err)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m_tok * out_f) return;
    float v = 0.f;
    for (uint32_t k = 0; k < n_kslab; ++k) v += part[(size_t)k * m_tok * out_f + i];
    if (*err) v = __int_as_float(0x7fc00000);      // a tensor-core wait gave up: poison the output
    uint32_t row = i % out_f;
    if (y_f32) {
        ((float *)y)[i] = bias ? v + __bfloat162float(bias[row]) : v;
    } else {
        __nv_bfloat16 h = __float2bfloat16_rn(v);
        if (bias) h = __hadd(h, bias[row]);
        ((__nv_bfloat16 *)y)[i] = h;
    }
}

}  // namespace ixb
