// Small-M GEMM on the resident P6 layout: 9..64 activation rows (batched serving, speculative verification) against a
// packed tensor in one pass over its bytes, on the 5th-generation tensor cores (tcgen05, accumulator in TMEM).
//
//   Y[t][n] = sum_k X[t][k] * bf16(code[n][k] * scale)        t < m_tok <= 64
//
// The reference runs this case as decode -> bf16 weight in HBM -> dense matmul (ixrun/engine.py:171-173; structural
// precedent for a fused kernel: ixrun/tpab_gemm.py:34-94).  Here the bf16 weights exist only in shared memory:
//
//   CTA      = 128 weight rows (8 row tiles) x a contiguous range of column blocks (split-K over at most a few CTAs,
//              so that about one CTA per SM is busy); the fp32 partial results of the splits are summed in a fixed
//              order by k_gemm_finalize (no atomics).
//   stage    = one column block (64 k): the MMA's M side = weights [128 rows x 64 k], its N side = activations
//              [tokens rounded up to 16 x 64 k] (rows beyond m_tok stay zero), both bf16, K-major, canonical 8 x 16-byte core matrices without
//              swizzle; the B operand's core-matrix columns are 16 bytes further apart than their size, which makes
//              swizzle; the core-matrix columns of both operands are 16 bytes further apart than their size, which makes
//              the 16-byte stores of the converter warps and of the activation copies conflict free.  Six stages.
//   warps    0,2,3  activation loaders, every third stage each: cp.async of the rows as soon as the slot is free
//            1      one thread issues four tcgen05.mma (M = 128 rows, N = tokens, K = 16) per stage into a
//                   128 x N fp32 accumulator and commits the slot back to its producers
//            4..27  converters, three per row tile, every third block each: P6 blocks through a private cp.async
//                   ring (as in the GEMV), the GEMV's shift / mask / fma conversion, four 16-byte stores into the
//                   B operand, then the block's outliers (requested two blocks ahead) written over their
//                   placeholders.  The chain per block is latency bound, hence many converter warps.
//            0..3   epilogue: tcgen05.ld of the accumulator, partial results to global memory
// Every wait on an mbarrier is bounded; a wait that gives up sets the error word (the finalizing kernel then poisons
// the output) and the kernel carries on to its end, so TMEM is always released.
#pragma once
#include "ixb_gemm_tc.cuh"
#include "ixb_p6.cuh"

namespace ixb {

constexpr int kPgConv = 8;                               // row tiles per CTA
constexpr int kPgPhases = 3;                             // converter warps per row tile: warp (tile, phase) takes every third block
constexpr int kPgConvWarp0 = 4;
constexpr int kPgWarps = kPgConvWarp0 + kPgConv * kPgPhases;   // 28
constexpr int kPgThreads = kPgWarps * 32;                // 896
constexpr int kPgLoaders = 3;                            // warps 0, 2, 3
constexpr int kPgRows = kPgConv * kTileRows;             // 128 weight rows per CTA (MMA N)
constexpr int kPgTok = 64;                               // MMA M
constexpr int kPgStages = 6;                             // deep enough that a slot's round trip through the tensor core is hidden
constexpr uint32_t kPgALbo = kPgTok * 16 + 16;           // 1040: next core matrix along K of the A operand (16 bytes of padding)
constexpr uint32_t kPgBLbo = kPgRows * 16 + 16;          // 2064: ... of the B operand (16 bytes of padding)
constexpr uint32_t kPgABytes = (kTileCols / 8) * kPgALbo;      // 8320
constexpr uint32_t kPgBBytes = (kTileCols / 8) * kPgBLbo;      // 16512
constexpr uint32_t kPgAOff = 0, kPgBOff = kPgStages * kPgABytes;
constexpr uint32_t kPgRingOff = kPgBOff + kPgStages * kPgBBytes;
constexpr uint32_t kPgRingBytes = kPgConv * kPgPhases * kP6RingBytes;
constexpr uint32_t kPgBarOff = kPgRingOff + kPgRingBytes;
constexpr int kPgGroup = 1;                              // stages per hand-shake (2 was measured slower: the ring gets coarser)
constexpr int kPgGroups = kPgStages / kPgGroup;
constexpr int kPgBars = 2 * kPgGroups + 1;
static_assert(kPgStages % kPgGroup == 0, "whole groups of stages");
constexpr uint32_t kPgSmemBytes = kPgBarOff + kPgBars * 8 + 16;
constexpr uint32_t kPgTmemCols = 64;
static_assert(kPgABytes % 16 == 0 && kPgBBytes % 16 == 0 && kPgBarOff % 8 == 0, "operand stages and barriers keep their alignment");
static_assert(kPgSmemBytes <= 227 * 1024, "fits the shared memory of one SM");

// kind::f16, bf16 x bf16 -> fp32, both operands K-major, M = 128 weight rows, N = the token count rounded up to 16
__host__ __device__ __forceinline__ uint32_t pg_idesc(uint32_t n_pad)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n_pad >> 3) << 17) | ((uint32_t)(kPgRows >> 4) << 24);
}

struct PgPlan {
    uint32_t groups, splits, grid;                       // 128-row groups, K splits, CTAs = groups * splits
};

__device__ __forceinline__ void pg_arrive(uint32_t mbar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(mbar) : "memory");
}

__global__ void __launch_bounds__(kPgThreads, 1)
k_p6_gemm(P6 p, const __nv_bfloat16 *__restrict__ x, uint32_t m_tok, float *__restrict__ part, uint32_t *err, PgPlan plan)
{
    extern __shared__ __align__(128) unsigned char pg_smem[];
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(pg_smem);
    const uint32_t bar0 = smem0 + kPgBarOff;             // full[S], empty[S], done
    uint32_t *tmem_slot = (uint32_t *)(pg_smem + kPgBarOff + kPgBars * 8);
    // one pair of barriers per group of kPgGroup consecutive stages (one stage today): `full` collects the activation
    // loaders and the converters of the group's stages, `empty` is the tensor core's commit
    auto grp = [&](uint32_t i) { return (i / kPgGroup) % kPgGroups; };               // barrier index of stage i
    auto grp_par = [&](uint32_t i) { return ((i / kPgGroup) / kPgGroups) & 1u; };    // its phase parity
    auto full_bar = [&](uint32_t gi) { return bar0 + gi * 8u; };
    auto empty_bar = [&](uint32_t gi) { return bar0 + (kPgGroups + gi) * 8u; };
    const uint32_t done_bar = bar0 + 2 * kPgGroups * 8u;
    auto a_stage = [&](uint32_t s) { return smem0 + kPgAOff + s * kPgABytes; };
    auto b_stage = [&](uint32_t s) { return smem0 + kPgBOff + s * kPgBBytes; };

    const uint32_t group = blockIdx.x % plan.groups, split = blockIdx.x / plan.groups;
    const uint32_t KB = p.kb;
    const uint32_t kq = KB / plan.splits, kr = KB - kq * plan.splits;
    const uint32_t kb0 = p6_begin(split, kq, kr), kb1 = p6_begin(split + 1, kq, kr), nk = kb1 - kb0;
    // stages are handed over in groups: the stages nk .. nkp - 1 do not exist, their producers only arrive
    const uint32_t nkp = (nk + kPgGroup - 1) / kPgGroup * kPgGroup;

    if (tid == 0) {
        for (uint32_t gi = 0; gi < (uint32_t)kPgGroups; ++gi) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full_bar(gi)), "r"(kPgGroup * (kPgConv + 1)) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(empty_bar(gi)) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(done_bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        const uint32_t slot_addr = (uint32_t)__cvta_generic_to_shared(tmem_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(kPgTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Only what no producer ever writes is zeroed, and stays zero for the whole kernel: the token rows between m_tok
    // and the MMA's N (the token count rounded up to 16) in every activation stage, and, in the last row group of a
    // tensor whose row count is not a multiple of 128, the weight rows of the row tiles that do not exist.
    {
        const uint32_t n_pad = (m_tok + 15u) & ~15u, zr = n_pad - m_tok;          // zr token rows x 8 core-matrix columns
        for (uint32_t c = tid; c < kPgStages * 8u * zr; c += kPgThreads) {
            const uint32_t st = c / (8u * zr), r = c - st * 8u * zr, kc = r / zr, tok = m_tok + (r - kc * zr);
            *(uint4 *)(pg_smem + kPgAOff + st * kPgABytes + kc * kPgALbo + tok * 16u) = make_uint4(0, 0, 0, 0);
        }
        const uint32_t tiles = min((uint32_t)kPgConv, p.rt - group * kPgConv);      // row tiles of this group that exist
        if (tiles < (uint32_t)kPgConv) {
            const uint32_t row0 = tiles * kTileRows, zrows = kPgRows - row0;
            for (uint32_t c = tid; c < kPgStages * 8u * zrows; c += kPgThreads) {
                const uint32_t st = c / (8u * zrows), r = c - st * 8u * zrows, kc = r / zrows, row = row0 + (r - kc * zrows);
                *(uint4 *)(pg_smem + kPgBOff + st * kPgBBytes + kc * kPgBLbo + row * 16u) = make_uint4(0, 0, 0, 0);
            }
        }
    }
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // everything above touches only this CTA's shared memory and TMEM; from here on the kernel reads the activations
    // and (at its end) writes the partial results, which the kernels ahead of it in the stream may still be using
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // the error word of this call: cleared by the first CTA (all CTAs of the grid are resident at once, one per SM, and
    // a wait gives up only after tens of milliseconds, so no CTA can have reported before this store)
    if (blockIdx.x == 0 && tid == 0) *err = 0u;
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0 || warp == 2 || warp == 3) {
        // ---- activation loaders: loader j takes the stages i = j, j + 3, ...; a stage's rows are requested as soon as
        // its slot is free (up to kPgStages stages ahead of the tensor core) and handed over two of the loader's own
        // iterations later
        const uint32_t j0 = warp == 0 ? 0u : (uint32_t)warp - 1u;
        const uint32_t chunks = m_tok * (kTileCols / 8);            // 16-byte chunks per stage
        const uint32_t mine = nkp > j0 ? (nkp - j0 + kPgLoaders - 1) / kPgLoaders : 0u;
        for (uint32_t n = 0; n < mine + 2; ++n) {
            if (n >= 2) {
                // the rows requested two iterations ago have landed: hand that stage over (before waiting for a free
                // slot, so that the hand-over never waits for the tensor core)
                cp_async_wait<1>();
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) pg_arrive(full_bar(grp(j0 + (n - 2) * kPgLoaders)));
            }
            const uint32_t i = j0 + n * kPgLoaders;
            if (n < mine && i < nk) {
                const uint32_t s = i % kPgStages;
                ok = mbar_wait(empty_bar(grp(i)), grp_par(i) ^ 1u) && ok;
                const __nv_bfloat16 *src = x + (size_t)(kb0 + i) * kTileCols;
                for (uint32_t c = lane; c < chunks; c += 32) {      // eight lanes fetch the 128 contiguous bytes of one row
                    const uint32_t kc = c & 7u, tok = c >> 3;
                    p6_cp16(a_stage(s) + kc * kPgALbo + tok * 16u, src + (size_t)tok * p.in_f + kc * 8u);
                }
            }
            cp_async_commit();
        }
    } else if (warp == 1) {
        // ---- one thread feeds the tensor core
        if (lane == 0) {
            const uint32_t idesc = pg_idesc((m_tok + 15u) & ~15u);
            for (uint32_t i0 = 0; i0 < nk; i0 += kPgGroup) {
                ok = mbar_wait(full_bar(grp(i0)), grp_par(i0)) && ok;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (uint32_t gs = 0; gs < (uint32_t)kPgGroup; ++gs) {
                    const uint32_t i = i0 + gs, st = i % kPgStages;
                    if (i >= nk) break;
                    uint64_t dw = umma_desc(b_stage(st), kPgBLbo, 128u);   // weights: the M side
                    uint64_t dx = umma_desc(a_stage(st), kPgALbo, 128u);   // activations: the N side
#pragma unroll
                    for (uint32_t k = 0; k < kTileCols / 16; ++k) {
                        const uint32_t acc = (i | k) ? 1u : 0u;
                        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                                     :: "r"(tmem_base), "l"(dw), "l"(dx), "r"(idesc), "r"(acc), "r"(0u) : "memory");
                        dw += (2u * kPgBLbo) >> 4;                        // two core matrices further along K
                        dx += (2u * kPgALbo) >> 4;
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(empty_bar(grp(i0))) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(done_bar) : "memory");
        }
        __syncwarp();
    } else if (warp >= kPgConvWarp0) {
        // ---- converters: warp (row tile R, phase ph3) converts the blocks R * KB + kb0 + i for i = ph3, ph3 + 3, ...
        const uint32_t cidx = (uint32_t)(warp - kPgConvWarp0), cw = cidx % kPgConv, ph3 = cidx / kPgConv;
        const uint32_t R = group * kPgConv + cw;
        const bool have = R < p.rt;                                  // (warp uniform) else: zero rows, arrivals only
        const int g = lane >> 2, t = lane & 3;
        const uint32_t ring_s = smem0 + kPgRingOff + cidx * kP6RingBytes;
        const uint32_t d16 = ring_s + lane * 16, d8 = ring_s + 512 + lane * 8;
        const bool lo16 = lane < 16;
        const uint32_t b_first = (have ? R : 0u) * KB + kb0;         // block of i = 0
        constexpr uint32_t kStep = kPgPhases;                        // this warp's blocks are kStep apart
        const unsigned char *n16 = p.plane + (size_t)(b_first + ph3) * kP6BlockBytes + lane * 16;
        uint32_t e2, b2, c2;
        {
            const float s32 = 32.f * __bfloat162float(p.scale[(have ? R : 0u) * p.scale_stride]);
            const uint32_t bb = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(s32));
            b2 = bb | (bb << 16);
            c2 = b2 ^ 0x80008000u;
            asm volatile("mov.b32 %0, 0x3F003F00;" : "=r"(e2));
        }
        // outlier bookkeeping: lane l keeps blk_off[b_first + win + l]; a block's entries are requested two of this
        // warp's blocks ahead
        uint32_t win = 0;
        int32_t off_l = 0;
        auto off_of = [&](uint32_t i) -> int32_t {                   // blk_off[b_first + i], i in [win, win + 32)
            return __shfl_sync(0xffffffffu, off_l, (int)(i - win));
        };
        auto load_window = [&](uint32_t i) {
            win = i;
            off_l = have ? __ldg(p.blk_off + b_first + min(i + (uint32_t)lane, nk)) : 0;
        };
        load_window(ph3);
        struct Ent { int32_t lo, hi; uint32_t e0, e1; };              // a block's entry range and its first 64 entries
        auto fetch_entries = [&](uint32_t i) -> Ent {
            Ent q = {0, 0, 0u, 0u};
            if (!have || i >= nk) return q;                           // warp uniform
            if (i + 1 >= win + 32) load_window(i);
            q.lo = off_of(i);
            q.hi = off_of(i + 1);
            if (q.lo + lane < q.hi) q.e0 = __ldg(p.esc + q.lo + lane);
            if (q.lo + 32 + lane < q.hi) q.e1 = __ldg(p.esc + q.lo + 32 + lane);
            return q;
        };
        if (have) {
#pragma unroll
            for (int s = 0; s < 3; ++s) {
                const bool more = ph3 + (uint32_t)s * kStep < nk;
                p6_cp16_if(d16 + s * kP6BlockBytes, n16, more);
                p6_cp16_if(d16 + s * kP6BlockBytes + 512, n16 + 512, more && lo16);
                n16 += kStep * kP6BlockBytes;
                cp_async_commit();
            }
        }
        Ent en0 = fetch_entries(ph3), en1 = fetch_entries(ph3 + kStep);     // this warp's current and next block
        uint32_t cs = 0, is = 3 * kP6BlockBytes;
        for (uint32_t i = ph3; i < nkp; i += kStep) {
            if (i >= nk) {                                            // a stage that only completes its group
                if (lane == 0) pg_arrive(full_bar(grp(i)));
                continue;
            }
            const uint32_t s = i % kPgStages;
            uint32_t f[16];
            const Ent en2 = fetch_entries(i + 2 * kStep);
            if (have) {
                const bool more = i + 3 * kStep < nk;
                p6_cp16_if(d16 + is, n16, more);
                p6_cp16_if(d16 + is + 512, n16 + 512, more && lo16);
                cp_async_commit();
                n16 += kStep * kP6BlockBytes;
                cp_async_wait<3>();
                __syncwarp();
                const uint4 a = p6_lds128(d16 + cs);
                const uint2 a2 = p6_lds64(d8 + cs);
                const uint32_t w[6] = {a.x, a.y, a.z, a.w, a2.x, a2.y};
#pragma unroll
                for (int k = 0; k < 6; ++k) {
                    f[2 * k] = p6_pair(w[k] << 2, e2, b2, c2);
                    f[2 * k + 1] = p6_pair(w[k] >> 4, e2, b2, c2);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t v = p6_and_or(w[q] >> 10, 0x003C003Cu, e2);
                    v = p6_and_or(w[4 + (q >> 1)] >> (6 + 2 * (q & 1)), 0x00C000C0u, v);
                    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(f[12 + q]) : "r"(v), "r"(b2), "r"(c2));
                }
                is = cs;
                cs = cs == (uint32_t)(3 * kP6BlockBytes) ? 0u : cs + (uint32_t)kP6BlockBytes;
            }
            ok = mbar_wait(empty_bar(grp(i)), grp_par(i) ^ 1u) && ok;   // the slot's last reader (the tensor core) is done
            if (have) {
                // rows g and g + 8 of the tile, columns 16 t .. 16 t + 15: four 16-byte pieces
                const uint32_t bs = b_stage(s) + (2u * cw) * 128u + (uint32_t)g * 16u;
#pragma unroll
                for (int sr = 0; sr < 2; ++sr)
#pragma unroll
                    for (int c = 0; c < 2; ++c)
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(bs + (2u * t + c) * kPgBLbo + sr * 128u),
                                     "r"(f[8 * c + sr]), "r"(f[8 * c + 2 + sr]), "r"(f[8 * c + 4 + sr]), "r"(f[8 * c + 6 + sr]) : "memory");
                __syncwarp();
                // the block's outliers over their placeholders (+0.0)
                const int32_t lo = en0.lo, hi = en0.hi;
                auto patch = [&](uint32_t e) {
                    const uint32_t r = (e >> 12) & 15u, c = e & 63u;
                    const uint32_t at = b_stage(s) + (c >> 3) * kPgBLbo + (2u * cw + (r >> 3)) * 128u + (r & 7u) * 16u + (c & 7u) * 2u;
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(at), "h"((unsigned short)(e >> 16)) : "memory");
                };
                if (lo + lane < hi) patch(en0.e0);
                if (lo + 32 + lane < hi) patch(en0.e1);
                for (int32_t j = lo + 64 + lane; j < hi; j += 32) patch(__ldg(p.esc + j));   // rare: more than 64 in a block
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) pg_arrive(full_bar(grp(i)));
            en0 = en1;
            en1 = en2;
        }
        cp_async_wait<0>();
    }

    if (warp < 4) {
        // ---- epilogue: accumulator row r (a weight row of the CTA's 128) lives in TMEM lane r, column j is token j
        __syncwarp();
        ok = mbar_wait(done_bar, 0u) && ok;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t row = group * (uint32_t)kPgRows + (uint32_t)warp * 32u + (uint32_t)lane;
        float *dst = part + (size_t)split * m_tok * p.out_f + row;
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < m_tok; c0 += 16) {
            uint32_t r[16];
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + c0;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                           "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                         : "r"(taddr) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < p.out_f) {
#pragma unroll
                for (uint32_t j = 0; j < 16u; ++j)                   // the warp's 32 rows of one token: 128 contiguous bytes
                    if (c0 + j < m_tok) dst[(size_t)(c0 + j) * p.out_f] = __uint_as_float(r[j]);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (!ok && lane == 0) atomicExch(err, 1u);
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPgTmemCols) : "memory");
}

}  // namespace ixb
