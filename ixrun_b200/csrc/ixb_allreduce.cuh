// One-shot all-reduce (sum) of a short fp32 vector over peer memory, for the partial outputs of row-parallel
// packed linears (o_proj / down_proj shards): out_f values per token, 20 KB for the 27B hybrid.
//
// The reference is single-GPU; its tensor-parallel form needs one sum of out_f values per row-parallel layer.
// A library all-reduce costs a launch of its own plus its protocol (15 .. 20 us when launched eagerly); at this size
// the transfer itself is a few hundred nanoseconds of
// NVLink time, so the whole exchange is done by one small kernel with plain peer stores and local loads, and the
// data carries its own "arrived" mark, so one crossing of NVLink is all the latency there is:
//
//   every rank owns one buffer that all ranks can address (peer pointers):
//     slots  [2 parities][W ranks][n_max] x {fp32 value, uint32 epoch}      epoch [counters] uint32      error word
//   CTA c of rank r, call number e (epoch[c] + 1), parity e & 1:
//     1. every thread stores its four values as four 8-byte words {value, e} into slot (parity, r) of EVERY
//        rank's buffer (an aligned 8-byte store arrives whole, so value and mark cannot be seen apart),
//     2. then reads the same four words of every sender's slot in ITS OWN buffer until their mark is e -- a
//        bounded wait: after kArSpinLimit polls it records an error word and goes on (later calls stop waiting
//        after 64 polls) --
//     3. adds the values in rank order (every rank gets the same bits), adds the bias, writes y (bf16 or
//        fp32); thread 0 stores e into epoch[c].
// No fences, no separate flags, no barrier after the first.  Two parities are enough: a rank can only reach call
// e + 2 after every other rank has sent call e + 1, which each does after it has finished reading call e.
// Nothing here is a multicast or a TMA load; NVLink carries plain stores only, all loads are local.  The kernel
// takes part in programmatic dependent launch like k_p6_mma, but runs nothing ahead of the dependency wait: the
// epoch is written by the previous all-reduce, which is only known to be complete once the kernel directly ahead
// (which waited for its own predecessor in turn) is complete.
#pragma once
#include "ixb_common.cuh"

namespace ixb {

constexpr int kArMaxWorld = 8;
constexpr int kArThreads = 256;
constexpr int kArPerCta = kArThreads * 4;                 // fp32 values per CTA
constexpr uint32_t kArSpinLimit = 1u << 22;               // polls (>= 32 ns each) before a wait gives up
constexpr int kArFinThreads = 128;
constexpr int kArFinPerCta = kArFinThreads * 2;           // fp32 values per CTA of the finishing kernel

struct ArPeers {
    uint2 *slots[kArMaxWorld];                            // every rank's slots, as seen from this rank
};

__host__ __device__ __forceinline__ size_t ar_slots_bytes(int world, int64_t n_max) { return (size_t)2 * world * n_max * 8; }
__host__ __device__ __forceinline__ uint32_t ar_ctas(int64_t n_max) { return (uint32_t)((n_max + kArPerCta - 1) / kArPerCta); }
__host__ __device__ __forceinline__ uint32_t ar_fin_ctas(int64_t n_max) { return (uint32_t)((n_max + kArFinPerCta - 1) / kArFinPerCta); }
// call counters behind the slots: one per CTA of the kernel with the larger grid; every kernel advances all of them
__host__ __device__ __forceinline__ uint32_t ar_counters(int64_t n_max) { return ar_fin_ctas(n_max); }

template <int W>
__global__ void __launch_bounds__(kArThreads)
k_allreduce_oneshot(ArPeers peers, const float *__restrict__ x, int rank, uint32_t n, uint32_t n_max,
                    const __nv_bfloat16 *__restrict__ bias, void *y, int y_f32, uint32_t *epoch, uint32_t *err, uint32_t spin_limit)
{
    __shared__ uint32_t e_s;
    const uint32_t c = blockIdx.x, tid = threadIdx.x;
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t i = (c * kArThreads + tid) * 4u;
    const bool valid = i < n;                              // n is a multiple of 4
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) e_s = epoch[c] + 1u;
    __syncthreads();
    const uint32_t e = e_s, par = e & 1u;
    if (valid) {
        // 1. this rank's values, marked with the call number, to every rank
        const float4 v = *(const float4 *)(x + i);
        const float in[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int r = 0; r < W; ++r) {
            volatile uint2 *dst = peers.slots[r] + ((size_t)(par * W + rank)) * n_max + i;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint2 wv;
                wv.x = __float_as_uint(in[k]);
                wv.y = e;
                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + k), "r"(wv.x), "r"(wv.y) : "memory");
            }
        }
        // 2. every sender's words in this rank's own buffer, once they carry this call's mark; 3. sum in rank order
        // (once a wait has given up, later calls give up quickly too instead of stalling for the full limit each time)
        const uint32_t limit = *(volatile uint32_t *)err ? 64u : spin_limit;
        float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < W; ++s) {
            const uint2 *src = peers.slots[rank] + ((size_t)(par * W + s)) * n_max + i;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t val, mark, polls = 0;
                for (;;) {
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(val), "=r"(mark) : "l"(src + k) : "memory");
                    if (mark == e) break;
                    __nanosleep(20);
                    if (++polls > limit) {
                        *err = 1u + (uint32_t)s;           // sender s never arrived: the result is wrong, not a hang
                        break;
                    }
                }
                o[k] += __uint_as_float(val);
            }
        }
        if (y_f32) {
#pragma unroll
            for (int k = 0; k < 4; ++k) ((float *)y)[i + k] = bias ? o[k] + __bfloat162float(bias[i + k]) : o[k];
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                __nv_bfloat16 h = __float2bfloat16_rn(o[k]);
                if (bias) h = __hadd(h, bias[i + k]);
                ((__nv_bfloat16 *)y)[i + k] = h;
            }
        }
    }
    if (tid == 0)
        for (uint32_t k = c; k < ar_counters(n_max); k += gridDim.x) epoch[k] = e;     // all counters advance together
}

// Second half of the exchange when the senders' words come straight from the epilogue of the GEMV before it
// (k_p6_mma with a P6Push): wait for every rank's words of this call in this rank's own buffer, add them in rank
// order, add the bias, write y.  Two values per thread, read as one 16-byte load of two marked words; 128 threads per
// CTA, so a 5120-value vector is finished by 20 CTAs.  Every CTA keeps its own call counter (epoch[c]); the grid is
// sized by n_max whatever n is, so all counters advance together, and the pushing GEMV of the next call reads
// epoch[0] + 1 as its mark.  The waits are bounded like k_allreduce_oneshot's.
template <int W>
__global__ void __launch_bounds__(kArFinThreads)
k_allreduce_finish(const uint2 *__restrict__ mine, uint32_t n, uint32_t n_max, const __nv_bfloat16 *__restrict__ bias,
                   void *y, int y_f32, uint32_t *epoch, uint32_t *err, uint32_t spin_limit)
{
    __shared__ uint32_t e_s;
    const uint32_t c = blockIdx.x, tid = threadIdx.x;
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t i = (c * kArFinThreads + tid) * 2u;
    const bool valid = i < n;                              // n is a multiple of 4
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) e_s = epoch[c] + 1u;
    __syncthreads();
    const uint32_t e = e_s, par = e & 1u;
    if (valid) {
        const uint32_t limit = *(volatile uint32_t *)err ? 64u : spin_limit;
        // all senders' words are requested together and looked at once they are all back: one round trip to L2
        // per poll, not one per sender
        uint32_t v0[W], v1[W], m0[W], m1[W];
        for (uint32_t polls = 0;; ++polls) {
            bool all = true;
#pragma unroll
            for (int s = 0; s < W; ++s) {
                const uint2 *src = mine + ((size_t)(par * W + s)) * n_max + i;
                asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v0[s]), "=r"(m0[s]), "=r"(v1[s]), "=r"(m1[s]) : "l"(src) : "memory");
            }
#pragma unroll
            for (int s = 0; s < W; ++s) all = all && m0[s] == e && m1[s] == e;
            if (all) break;
            if (polls > limit) {
#pragma unroll
                for (int s = 0; s < W; ++s)
                    if (m0[s] != e || m1[s] != e) *err = 1u + (uint32_t)s;      // sender s never arrived: the result is wrong, not a hang
                break;
            }
            __nanosleep(20);
        }
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int s = 0; s < W; ++s) {                      // in rank order: the same bits on every rank
            o0 += __uint_as_float(v0[s]);
            o1 += __uint_as_float(v1[s]);
        }
        if (y_f32) {
            float2 r;
            r.x = bias ? o0 + __bfloat162float(bias[i]) : o0;
            r.y = bias ? o1 + __bfloat162float(bias[i + 1]) : o1;
            *(float2 *)((float *)y + i) = r;
        } else {
            __nv_bfloat16 h0 = __float2bfloat16_rn(o0), h1 = __float2bfloat16_rn(o1);
            if (bias) {
                h0 = __hadd(h0, bias[i]);
                h1 = __hadd(h1, bias[i + 1]);
            }
            *(__nv_bfloat162 *)((__nv_bfloat16 *)y + i) = __halves2bfloat162(h0, h1);
        }
    }
    if (tid == 0) epoch[c] = e;
}

}  // namespace ixb
